"""The generic training engine: state init, resume / fine-tune, the step loop, logging, evaluation
scheduling, preemption consensus and checkpoint cadence. Every target goes through this one loop
and is seen only via the `DecomposedModel` protocol.

Parity: param_decomp/core/run.py:1012-1199 (`run_decomposition_training`), :820-871 (Fresh |
Resume | FineTune start), :747-798 (faithfulness warm-up), :1435-1636 (timed loop), :335-379
(SIGTERM consensus), :282-322 (due evaluations), :883-909 (saver, no-checkpoint re-entry marker),
:1202-1353 (targeted loop); core/run_state.py:252-380 (state init).
"""

from __future__ import annotations

import os
import signal
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Protocol

import torch
from torch import nn

from param_decomp_b200.config.run import (
    Cadence,
    KeepLastNCheckpoints,
    NoCheckpointing,
    PDConfig,
    PeriodicCheckpointing,
    ResumeProvenance,
    TargetedPDConfig,
)
from param_decomp_b200.core import checkpoint as ckpt
from param_decomp_b200.core.adversary import PersistentAdversary
from param_decomp_b200.core.components import ComponentStacks
from param_decomp_b200.core.metrics import (
    NO_REENTRY_MARKER,
    MetricsSink,
    PerformanceTracker,
    assert_all_finite,
    get_logger,
    public_record,
)
from param_decomp_b200.core.model import DecomposedModel
from param_decomp_b200.core.objective import NontargetObjective, PDObjective, build_objective
from param_decomp_b200.core.optim import build_group_optimizer
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.core.train import DataCollectives, StepContext, TrainState, faithfulness_warmup


class Evaluation(Protocol):
    """Scheduled evaluation: `run(step, state) -> {key: scalar}` if anything is due at `step`."""

    def is_due(self, step: int) -> bool: ...

    def run(self, step: int, state: TrainState, ctx: StepContext) -> dict[str, Any]: ...


# ---- preemption -------------------------------------------------------------------------------------


class PreemptionFlag:
    """SIGTERM sets a host flag; `consensus()` ORs it over ranks (a host-side all-reduce on the CPU
    group) at a step boundary so every rank stops at the same step."""

    def __init__(self, collectives: DataCollectives) -> None:
        self._flag = threading.Event()
        self._collectives = collectives
        self._installed = False

    def install(self) -> None:
        if threading.current_thread() is threading.main_thread():
            signal.signal(signal.SIGTERM, lambda *_: self._flag.set())
            self._installed = True

    def set(self) -> None:
        self._flag.set()

    def consensus(self) -> bool:
        local = 1.0 if self._flag.is_set() else 0.0
        any_fn = getattr(self._collectives, "host_any", None)
        return bool(any_fn(local)) if any_fn is not None else bool(local)


def _finalized(evaluation: Any, averaged: dict) -> dict:
    """Evaluations may form quantities that are not linear in the batch (ratios) from the averaged metrics."""
    fin = getattr(evaluation, "finalize", None)
    return fin(averaged) if fin is not None else averaged


class StepProfiler:
    """Profiles `n_steps` training steps after `warmup` steps of this entry, then asks the loop to stop.

    `trace`: an in-process `torch.profiler` trace written to `<run_dir>/profile/trace.json`.
    `cuda_profiler_range`: the CUDA profiler start / stop calls around the captured steps, one NVTX range per
    step, for an external profiler attached with a capture range on that API; nothing is written here."""

    def __init__(self, kind: str, warmup: int, n_steps: int, run_dir: Any) -> None:
        assert kind in ("trace", "cuda_profiler_range"), kind
        self.kind, self.warmup, self.n_steps, self.run_dir = kind, warmup, n_steps, run_dir
        self._trace: Any = None
        self._range_open = False
        self._census_cm: Any = None
        self._census: Any = None
        self.captured: list[int] = []

    def before_step(self, entry_step: int) -> None:
        if entry_step < self.warmup:
            return
        cuda = torch.cuda.is_available()
        if entry_step == self.warmup:
            if self.run_dir is not None:  # attribute the first profiled step's memory to its phases
                from param_decomp_b200.core.debug.memory_ledger import Ledger
                from param_decomp_b200.core.train import phase

                phase.ledger = Ledger()
                phase.ledger.mark("step_begin")
                from param_decomp_b200.core.debug.census import census

                self._census_cm = census()  # what the step launches: native entry points and collectives by kind
                self._census = self._census_cm.__enter__()
            if self.kind == "trace":
                from torch.profiler import ProfilerActivity, profile

                acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if cuda else [])
                self._trace = profile(activities=acts)
                self._trace.start()
            elif cuda:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
        if self.kind == "cuda_profiler_range" and cuda:
            torch.cuda.nvtx.range_push(f"train_step_{entry_step}")
            self._range_open = True
        self.captured.append(entry_step)

    def after_step(self, entry_step: int) -> bool:
        """True once the last captured step has run (the loop then leaves)."""
        if entry_step < self.warmup:
            return False
        if self._range_open:
            torch.cuda.nvtx.range_pop()
            self._range_open = False
        if entry_step == self.warmup and self.run_dir is not None:
            from param_decomp_b200.core.train import phase

            if phase.ledger is not None:
                phase.ledger.mark("step_end")
                out = Path(self.run_dir) / "profile"
                out.mkdir(parents=True, exist_ok=True)
                phase.ledger.save(out / "memory_ledger.json")
                phase.ledger = None
                if self._census_cm is not None:
                    import json

                    self._census_cm.__exit__(None, None, None)
                    (out / "census.json").write_text(json.dumps(self._census.summary(), indent=1))
                    self._census_cm = None
        if entry_step < self.warmup + self.n_steps - 1:
            return False
        if self.kind == "trace":
            self._trace.stop()
            out = Path(self.run_dir) / "profile"
            out.mkdir(parents=True, exist_ok=True)
            self._trace.export_chrome_trace(str(out / "trace.json"))
        elif torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        return True


# ---- state ------------------------------------------------------------------------------------------


def init_train_state(model: DecomposedModel, ci_fn: nn.Module, pd: PDConfig | TargetedPDConfig,
                     objective: PDObjective, device: torch.device | str, batch_rows: int,
                     positions: int | None, stack_multiple: int = 1, use_fused_optim: bool = False,
                     init_components: Callable[[ComponentStacks], None] | None = None,
                     shard_group: Any = None, shard_backend: str | None = None,
                     expert_shard: Any = None, data_rank: int = 0, peer_wait_limit_s: float = 30.0) -> TrainState:
    """Seeded init: `init` / `source` / `run` streams are separated like the reference's
    `split(PRNGKey(seed), 3)`."""
    g = torch.Generator().manual_seed(pd.seed)
    from param_decomp_b200.config.run import MuonOptimizerConfig

    muon_sharded = shard_backend is not None and isinstance(pd.components_optimizer, MuonOptimizerConfig)
    if muon_sharded:  # Newton-Schulz work and momentum split along the stack axis: stacks must tile the group
        import torch.distributed as dist

        stack_multiple = max(stack_multiple, dist.get_world_size(shard_group) if shard_group is not None else 1)
    components = ComponentStacks(model.sites, stack_multiple)
    if expert_shard is not None:
        assert shard_backend is None or expert_shard.by_component, \
            "expert-split component stacks use the replicated-optimizer layout"
        expert_shard.init_components(components, g)  # the single-process draw, this rank's expert blocks kept
    else:
        components.init_random(g)
    if init_components is not None:
        init_components(components)
    components.to(device)
    ci_fn.to(device)
    comp_named = [(n, p) for n, p in components.named_parameters()]
    ci_named = [(n, p) for n, p in ci_fn.named_parameters()]
    if muon_sharded:
        from param_decomp_b200.parallel.sharded_muon import StackShardedMuon

        comp_opt = StackShardedMuon(pd.components_optimizer, [n for n, _ in comp_named], [p for _, p in comp_named],
                                    pd.steps, shard_group)
    elif shard_backend is not None:
        from param_decomp_b200.parallel.sharded_optim import ShardedFlatAdamW

        comp_opt = ShardedFlatAdamW(pd.components_optimizer, ["/".join(n.split(".")) for n, _ in comp_named],
                                    [p for _, p in comp_named], pd.steps, shard_group, backend=shard_backend,
                                    keep_lo=True, norm_group=expert_shard.group if expert_shard is not None else None,
                                    wait_limit_s=peer_wait_limit_s)
    else:
        comp_opt = build_group_optimizer(pd.components_optimizer, comp_named, pd.steps, 2, use_fused_optim)
    if expert_shard is not None and (shard_backend is None or muon_sharded):
        comp_opt.norm_fn = expert_shard.grad_norm  # split leaves contribute their group-wide sum of squares
    if expert_shard is not None and hasattr(comp_opt, "column_split"):
        comp_opt.column_split = expert_shard  # Muon: slices of the component axis are gathered for Newton-Schulz
    from param_decomp_b200.config.run import AdamWOptimizerConfig as _AdamW

    if (shard_backend is not None and expert_shard is None and isinstance(pd.ci_fn_optimizer, _AdamW)
            and not muon_sharded and ci_named):
        # the CI function's gradients take the same path as the components': reduce-scatter + AdamW + all-gather in
        # one kernel over its own flat buffers - no separate gradient all-reduce in the step
        from param_decomp_b200.parallel.sharded_optim import ShardedFlatAdamW

        ci_opt = ShardedFlatAdamW(pd.ci_fn_optimizer, [n for n, _ in ci_named], [p for _, p in ci_named], pd.steps,
                                  shard_group, backend=shard_backend, keep_lo=True, wait_limit_s=peer_wait_limit_s,
                                  label="ci_fn")
    else:
        ci_opt = build_group_optimizer(pd.ci_fn_optimizer, ci_named, pd.steps, 2, use_fused_optim)
    state = TrainState(
        components=components,
        ci_fn=ci_fn,
        components_opt=comp_opt,
        ci_fn_opt=ci_opt,
    )
    state.expert_shard = expert_shard  # type: ignore[attr-defined]
    src_key = StepKey(pd.seed ^ 0x5EED, 0)
    for term in objective.persistent_terms():
        cfg = term.cfg
        pool = cfg.pool.size_per_batch_element if hasattr(cfg, "pool") else 1  # type: ignore[attr-defined]
        shape = getattr(cfg, "source_shape", "bc")
        state.adversaries[term.name] = PersistentAdversary.init(
            getattr(model, "global_sites", model.sites), cfg.optimizer, cfg.source_dtype, shape, batch_rows, positions, src_key,  # type: ignore[attr-defined]
            pool_size=pool, device=device, data_rank=data_rank)
    return state


@dataclass
class RunResult:
    final_step: int
    stopped_by_sigterm: bool
    last_metrics: dict[str, float] = field(default_factory=dict)
    run_dir: Path | None = None


def _resolve_start(run_dir: Path | None, state: TrainState, cadence: Cadence,
                   provenance: ResumeProvenance | None, log, data_rank: int = 0, data_world: int = 1,
                   collectives: DataCollectives | None = None) -> str:
    """Fresh | Resume(own newest checkpoint) | FineTune(parent V/U + CI fn, step 0)."""
    if run_dir is not None:
        if isinstance(cadence.checkpointing, NoCheckpointing):
            # one rank owns the marker; every rank learns its verdict (they share the run directory)
            marker = run_dir / NO_REENTRY_MARKER
            refused = False
            if collectives is None or collectives.rank == 0:
                refused = marker.exists()
                if not refused:
                    run_dir.mkdir(parents=True, exist_ok=True)
                    marker.write_text("started\n")
            any_fn = getattr(collectives, "host_any", None)
            if any_fn is not None:
                refused = bool(any_fn(float(refused)))
            assert not refused, f"{run_dir} ran without checkpoints: re-entering it is refused"
        else:
            own = ckpt.latest_readable_step(run_dir, log)
            if own is not None:
                ckpt.restore_state(run_dir, own, state, data_rank, data_world)
                log.info("resumed from %s/ckpts/%d", run_dir, own)
                return "resume"
    if provenance is not None:
        ckpt.restore_decomposition(provenance.parent_run_dir, provenance.parent_step, state.components, state.ci_fn,
                                   getattr(state, "expert_shard", None))
        if hasattr(state.components_opt, "sync_from_parameters"):
            state.components_opt.sync_from_parameters()
        log.info("fine-tune: loaded V/U + CI fn from %s step %d", provenance.parent_run_dir, provenance.parent_step)
        return "finetune"
    return "fresh"


def run_decomposition_training(
    model: DecomposedModel,
    ci_fn: nn.Module,
    pd: PDConfig | TargetedPDConfig,
    cadence: Cadence,
    sample_batch: Callable[[int], Any],
    *,
    device: torch.device | str = "cpu",
    run_dir: Path | None = None,
    sink: MetricsSink | None = None,
    evaluation: Evaluation | None = None,
    collectives: DataCollectives | None = None,
    resume_provenance: ResumeProvenance | None = None,
    nontarget: NontargetObjective | None = None,
    sample_nontarget_batch: Callable[[int], Any] | None = None,
    batch_rows: int | None = None,
    positions: int | None = None,
    units_per_step: int | None = None,
    flops_per_step: float = 0.0,
    peak_flops: float = 0.0,
    lazy_masks: bool = False,
    use_fused_optim: bool = False,
    init_components: Callable[[ComponentStacks], None] | None = None,
    extra_log: Callable[[int, TrainState, StepContext], dict[str, Any]] | None = None,
    max_steps_this_entry: int | None = None,
    profile_steps: int = 0,
    profile_warmup: int | None = None,
    profile_kind: str = "trace",
    state_out: list | None = None,
    shard_group: Any = None,
    shard_backend: str | None = None,
    step_watchdog_s: float | None = None,
    peer_wait_limit_s: float = 30.0,
    record_step: bool = False,
    stack_multiple: int = 1,
    remat_recon_forwards: bool = False,
    remat_ci_fn: bool = False,
) -> RunResult:
    collectives = collectives or DataCollectives()
    log = get_logger(collectives.rank)
    objective = build_objective(pd)
    expert_shard = None
    if getattr(model, "ep", None) is not None or getattr(model, "component_group", None) is not None:
        from param_decomp_b200.parallel.expert_shard import StackSharding

        expert_shard = StackSharding.for_model(model)
    ctx = StepContext.build(model, objective, pd, collectives=collectives, lazy_masks=lazy_masks, nontarget=nontarget,
                            expert_shard=expert_shard, remat_recon_forwards=remat_recon_forwards,
                            remat_ci_fn=remat_ci_fn)
    rows = batch_rows if batch_rows is not None else pd.batch_size // collectives.world_size
    state = init_train_state(model, ci_fn, pd, objective, device, rows, positions, stack_multiple=stack_multiple,
                             use_fused_optim=use_fused_optim, init_components=init_components,
                             shard_group=shard_group, shard_backend=shard_backend, expert_shard=expert_shard,
                             data_rank=getattr(collectives, "data_rank", 0), peer_wait_limit_s=peer_wait_limit_s)
    if state_out is not None:
        state_out.append(state)
    start_kind = _resolve_start(run_dir, state, cadence, resume_provenance, log,
                                getattr(collectives, "data_rank", 0), collectives.world_size, collectives)

    if start_kind != "resume" and isinstance(pd, PDConfig) and pd.faithfulness_warmup_steps > 0:
        last = faithfulness_warmup(ctx, state, pd.faithfulness_warmup_steps, pd.faithfulness_warmup_lr,
                                   pd.faithfulness_warmup_weight_decay,
                                   log=lambda i, v: log.info("faithfulness warm-up %d: %.3e", i, v))
        if hasattr(state.components_opt, "sync_from_parameters"):
            state.components_opt.sync_from_parameters()  # the warm-up stepped the parameters' own storage
        log.info("faithfulness warm-up done (%.3e)", last)

    own_sink = sink is None and run_dir is not None
    if own_sink:
        sink = MetricsSink.for_run(run_dir, collectives.rank)  # type: ignore[arg-type]
    from param_decomp_b200.utils.flops import optimizer_flops

    opt_flops = (optimizer_flops("components", pd.components_optimizer, list(state.components.parameters()))[0]
                 + optimizer_flops("ci_fn", pd.ci_fn_optimizer, list(ci_fn.parameters()))[0])
    perf = PerformanceTracker(pd.steps, units_per_step or pd.batch_size, flops_per_step, peak_flops,
                              optimizer_flops_per_step=opt_flops / max(1, collectives.world_size))
    perf.step_last = state.step
    preempt = PreemptionFlag(collectives)
    preempt.install()

    saving = isinstance(cadence.checkpointing, PeriodicCheckpointing) and run_dir is not None
    keep = None
    if saving and isinstance(cadence.checkpointing.retention, KeepLastNCheckpoints):  # type: ignore[union-attr]
        keep = cadence.checkpointing.retention.n  # type: ignore[union-attr]

    def check_device_status(where: str) -> None:
        """The native kernels report a wait that ran out (a late or dead peer) in a per-device status word and
        then run to completion on whatever data they had, so the parameters can no longer be trusted. Read the
        word at points where the host waits for the device anyway and stop every rank together, before anything
        is logged as healthy or written to a checkpoint."""
        dev = torch.device(device)
        if dev.type != "cuda":
            return
        from param_decomp_b200.ops import native

        if not native.LIB_PATH.exists():
            return
        code = int(native.status_word().item())
        any_fn = getattr(collectives, "host_any", None)
        bad = bool(any_fn(float(code != 0))) if any_fn is not None else code != 0
        if bad:
            native.status_word().zero_()
            raise native.NativeError(
                f"{where} (step {state.step}): a device-side wait timed out on this or another rank "
                f"(local status code {code}); the step's results are not valid, stopping without a checkpoint")

    def sync_masters(for_save: bool) -> None:
        """A sharded optimizer keeps each rank's slice of the masters: before anything reads the parameters
        (evaluation, checkpoint) gather them - and, for a save, the moments - on every rank."""
        for opt in (state.components_opt, state.ci_fn_opt):
            if for_save and hasattr(opt, "gather_state"):
                opt.gather_state()
            elif hasattr(opt, "refresh_full_fp32"):
                opt.refresh_full_fp32()

    def save() -> None:
        check_device_status("before a checkpoint")
        if saving:
            sync_masters(for_save=True)
            for adv in state.adversaries.values():  # per-row sources: every batch shard contributes its rows
                adv.gather_state(collectives.gather_rows)
        if saving and expert_shard is not None:
            # the ranks of one expert group (the first data shard's) assemble the global stacks; rank 0 writes
            if collectives.in_first_tp_group:
                ckpt.save_state(run_dir, state, keep, expert_shard=expert_shard, write=collectives.rank == 0)  # type: ignore[arg-type]
        elif saving and collectives.rank == 0:
            ckpt.save_state(run_dir, state, keep)  # type: ignore[arg-type]
        barrier = getattr(collectives, "barrier", None)
        if barrier is not None:
            barrier()

    from param_decomp_b200.core.recorded_step import RecordedTrainStep

    stepper = RecordedTrainStep(ctx, state, enabled=record_step)
    if record_step:
        log.info("train step: %s", "recorded as a CUDA graph after 3 eager steps" if stepper.eligible
                 else f"eager ({stepper.reason})")
    result = RunResult(final_step=state.step, stopped_by_sigterm=False, run_dir=run_dir)
    entry_steps = 0
    profiler = None
    if profile_steps > 0 and (run_dir is not None or profile_kind == "cuda_profiler_range"):
        # warm-up: past the eager steps that precede the recording of the step, so the trace shows the steady state
        warm = profile_warmup if profile_warmup is not None else (5 if stepper.eligible else 2)
        profiler = StepProfiler(profile_kind, warm, profile_steps, run_dir)

    # A step (or an evaluation / a save between two steps) that takes longer than the limit is treated as a stall:
    # first as a preemption (the loop saves and exits at its next boundary, all ranks together), then - if no
    # boundary is reached within another limit - the process leaves without a checkpoint.
    watchdog = StepWatchdog(step_watchdog_s, on_stall=preempt.set).start() if step_watchdog_s else None
    try:
        while state.step < pd.steps:
            step = state.step
            if watchdog is not None:
                watchdog.beat()
            if evaluation is not None and evaluation.is_due(step):
                check_device_status("before an evaluation")
                sync_masters(for_save=False)
                ev = _finalized(evaluation, collectives.average_scalars(evaluation.run(step, state, ctx)))
                if sink is not None and ev:
                    sink.log(step, ev, prefix="eval/")
            if saving and step > 0 and step % cadence.checkpointing.save_every == 0 and ckpt.latest_step(run_dir) != step:  # type: ignore[union-attr,arg-type]
                save()

            batch = sample_batch(step)
            nt_batch = sample_nontarget_batch(step) if sample_nontarget_batch is not None else None
            if profiler is not None:
                profiler.before_step(entry_steps)
            metrics = stepper(batch, nt_batch)
            if profiler is not None and profiler.after_step(entry_steps):
                break
            entry_steps += 1

            if cadence.should_log_train(step) or state.step == pd.steps:
                check_device_status("at a log step")
                scalars = {k: v for k, v in metrics.items()}
                if "grad_norm/components" in scalars and "grad_norm/ci_fn" in scalars:
                    scalars["grad_norm/total"] = (float(scalars["grad_norm/components"]) ** 2
                                                  + float(scalars["grad_norm/ci_fn"]) ** 2) ** 0.5
                scalars.update(perf.tick(state.step))
                from param_decomp_b200.core.gauge import uv_norm_ratio_metrics

                if hasattr(state.components_opt, "refresh_full_fp32"):
                    state.components_opt.refresh_full_fp32()  # sharded masters: gather the shards before reading
                scalars.update(uv_norm_ratio_metrics(state.components, expert_shard))  # drift of the V/U scale symmetry
                if extra_log is not None:
                    scalars.update(extra_log(step, state, ctx))
                scalars = collectives.average_scalars(scalars)  # per-batch losses: the global-batch mean, as the reference logs
                floats = sink.log(step, scalars) if sink is not None else public_record({("train/" + k): float(v) for k, v in scalars.items()})
                assert_all_finite(step, floats)
                result.last_metrics = floats
                log.info("step %d  total=%.4e  step_time=%.3fs", step, floats.get("train/loss/total", float("nan")),
                         floats.get("train/perf/step_time_s", float("nan")))

            if preempt.consensus():
                log.info("%s at step %d: saving and exiting",
                         "step watchdog fired" if (watchdog is not None and watchdog.fired) else "SIGTERM consensus", state.step)
                save()
                result.stopped_by_sigterm = True
                break
            if max_steps_this_entry is not None and entry_steps >= max_steps_this_entry:
                break

        if state.step >= pd.steps:
            if evaluation is not None and evaluation.is_due(state.step):
                sync_masters(for_save=False)
                ev = _finalized(evaluation, collectives.average_scalars(evaluation.run(state.step, state, ctx)))
                if sink is not None and ev:
                    sink.log(state.step, ev, prefix="eval/")
            save()
    finally:
        if watchdog is not None:
            watchdog.stop()
        stepper.release()  # (also on an exception: a live recording blocks the process group's teardown)
    result.final_step = state.step
    if own_sink and sink is not None:
        sink.close()
    return result


class StepWatchdog:
    """Host thread that turns a stalled step into a clean abort: if `beat()` is not called for `limit_s`,
    `on_stall` runs (default: raise SIGTERM in this process, which the loop treats as a preemption at its next
    boundary); if another `limit_s` passes without a beat - the loop never reached a boundary - `on_dead` runs
    (default: `os._exit(75)`, leaving without a checkpoint). Host-side only: nothing here touches the device."""

    def __init__(self, limit_s: float, on_stall: Callable[[], None] | None = None,
                 on_dead: Callable[[], None] | None = None) -> None:
        self.limit_s = limit_s
        self.on_stall = on_stall or (lambda: signal.raise_signal(signal.SIGTERM))
        self.on_dead = on_dead or (lambda: os._exit(75))
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._watch, daemon=True)

    def start(self) -> "StepWatchdog":
        self._thread.start()
        return self

    def beat(self) -> None:
        self._last = time.monotonic()

    def stop(self) -> None:
        self._stop.set()

    def _watch(self) -> None:
        while not self._stop.wait(min(self.limit_s / 4, 1.0)):
            idle = time.monotonic() - self._last
            if idle > self.limit_s and not self.fired:
                self.fired = True
                self.on_stall()
            elif self.fired and idle > 2 * self.limit_s:
                self.on_dead()
                return
