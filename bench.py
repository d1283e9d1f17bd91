"""Headline benchmark: decomposition tokens/s of the Llama-style 4-layer LM config
(`param_decomp_b200/experiments/configs/lm_llama4l_c4096.yaml`) on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
    python bench.py --impl reference ...                     (the reference arm)

Two measurements, both of full optimizer steps (clean forward, CI function, 2 masked
forward/backward draws with KL over the vocabulary, faithfulness, minimality, clip, AdamW):
  value  device-timed with CUDA events around K steps whose token batches are already on the
         device, max over ranks;
  e2e    the same K steps driven through the public step API with, every step, the host->device
         copy of that step's tokens from pinned memory and a device->host read of the loss.
Global batch is fixed at 64 sequences x 512 tokens for every N (strong scaling).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CONFIG = ROOT / "param_decomp_b200" / "experiments" / "configs" / "lm_llama4l_c4096.yaml"
METRIC = "decomposition tokens/sec/box at 1/2/4/8 B200, device-timed max over ranks"


class ClockSampler:
    """Samples `nvidia-smi` clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.proc = index, [], None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.samples.append([p.strip() for p in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            if len(s) < 7:
                continue
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> None:
    """The reference is a JAX/XLA program (jax, equinox, optax, orbax, tokamax); none of those is
    installed here or present in the offline wheelhouse, so its trainer cannot be imported."""
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import jax  # noqa: F401
        import param_decomp  # noqa: F401
        why = "reference imported but its LM entry point needs a tokenised dataset store and a pretrain cache"
    except Exception as err:  # noqa: BLE001
        why = f"reference not runnable offline: {type(err).__name__}: {str(err)[:120]}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours")
    ap.add_argument("--config", type=Path, default=CONFIG)
    ap.add_argument("--batch", type=int, default=None, help="override the global batch (debugging only)")
    ap.add_argument("--optim", type=str, default=None, choices=["fused_p2p", "collective", "ddp"],
                    help="N>1: override what the config's placement (`runtime.sharding`) selects - fused reduce-scatter + "
                         "AdamW + all-gather kernel, NCCL reduce-scatter / all-gather, or all-reduce + replicated AdamW")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the device-timed steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--tp", type=int, default=1,
                    help="size of the mesh's tp axis (ranks of one tp group see the same tokens and split the experts "
                         "of a mixture-of-experts target or every site's component axis of a dense one)")
    ap.add_argument("--expert-dispatch", type=str, default="allreduce", choices=["allreduce", "all_to_all"],
                    help="with --tp on a mixture-of-experts target: tokens replicated over the tp group and partial "
                         "outputs summed, or the batch sharded over it too and jobs stored into their expert's owner")
    ap.add_argument("--no-record", action="store_true",
                    help="issue every step launch by launch from Python instead of replaying the recorded CUDA graph")
    ap.add_argument("--backend", type=str, default="fused_sm100", choices=["fused_sm100", "eager_torch"],
                    help="eager_torch: the same step on plain PyTorch ops (cuBLAS GEMMs, torch fused attention, torch "
                         "optimizer arithmetic) - a context number for the hand-written path, never the headline")
    ap.add_argument("--trace", action="store_true",
                    help="print a time-stamped line per warm-up step / recording / replay on every rank (diagnostics)")
    ap.add_argument("--no-lanes", action="store_true",
                    help="keep the whole step on one CUDA stream (no side-by-side draws / q,k,v / gate,up)")
    ap.add_argument("--kernel-table", type=Path, default=None,
                    help="after the timed steps, run one more step under the torch profiler and write the kernels "
                         "ranked by device time to this file (never part of a reported number)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.config.run import HsdpMeshShape
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext
    from param_decomp_b200.experiments.lm.build import build_lm_run
    from param_decomp_b200.ops import native
    from param_decomp_b200.parallel import topology

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 under torchrun"
    cfg = LMExperimentConfig.from_file(args.config)
    pd = cfg.pd if args.batch is None else cfg.pd.model_copy(update={"batch_size": args.batch})
    cfg = cfg.model_copy(update={"pd": pd})
    assert world % args.tp == 0, f"--tp {args.tp} does not divide {world} GPUs"
    mesh = HsdpMeshShape(replicate=1, fsdp=world // args.tp, tp=args.tp)  # the config's mesh, sized to this job
    cfg = cfg.model_copy(update={"runtime": cfg.runtime.model_copy(update={"mesh": mesh, "backend": args.backend})})
    fused = args.backend == "fused_sm100"
    topo = topology.initialize(mesh, "cuda", batch_over_tp=args.expert_dispatch == "all_to_all")
    from param_decomp_b200.parallel import layout as layout_mod

    lay = layout_mod.resolve(cfg.runtime, world=world)  # what `runtime.sharding` asks for on this mesh
    if args.optim is None:
        args.optim = ("fused_p2p" if fused else "collective") if lay.optimizer_sharded else "ddp"
    run = build_lm_run(cfg, None, topo.device, topo.data_rank, topo.data_world,
                       expert_group=topo.groups.get("tp") if args.tp > 1 else None, expert_mode=args.expert_dispatch)
    objective = build_objective(cfg.pd)
    expert_shard = None
    if args.tp > 1:
        from param_decomp_b200.parallel.expert_shard import StackSharding

        expert_shard = StackSharding.for_model(run.model)
    ctx = StepContext.build(run.model, objective, cfg.pd, collectives=topo.collectives(), lazy_masks=fused,
                            expert_shard=expert_shard)
    rows = cfg.pd.batch_size // topo.data_world
    shard_backend = args.optim if (topo.data_world > 1 and args.optim != "ddp" and args.tp == 1) else None
    if args.tp > 1 and topo.data_world > 1 and args.optim != "ddp" and run.ep is None:
        shard_backend = "collective"  # component slices: sharded AdamW over the batch axes, clip norm summed over tp
    state = init_train_state(run.model, run.ci_fn, cfg.pd, objective, topo.device, rows, cfg.data.seq_len,
                             use_fused_optim=fused, shard_group=topo.data_group, shard_backend=shard_backend,
                             expert_shard=expert_shard, peer_wait_limit_s=5.0)
    tokens_per_step = cfg.pd.batch_size * cfg.data.seq_len

    def sync() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The public step API: eager for its first steps, then recorded as a CUDA graph and replayed.
    # Warm-up = W eager steps (they allocate gradient buffers and size the allocator's pools) plus, when the
    # step is recorded, the recording call and one replay - all untimed.
    from param_decomp_b200.core.recorded_step import RecordedTrainStep

    step_fn = RecordedTrainStep(ctx, state, enabled=fused and not args.no_record, eager_steps=args.warmup,
                                concurrent=not args.no_lanes)
    t_start = time.perf_counter()

    def trace(what: str) -> None:
        if args.trace:
            torch.cuda.synchronize()
            print(f"[rank {topo.rank} +{time.perf_counter() - t_start:7.2f}s] {what} "
                  f"(status word {int(native.status_word().item())})", file=sys.stderr, flush=True)

    trace(f"start: step issue = {'recorded' if step_fn.eligible else step_fn.reason}")
    for s in range(args.warmup + (2 if step_fn.eligible else 0)):
        step_fn(run.sample_train(s))
        trace(f"warm-up call {s} done, graph {'yes' if step_fn.graph is not None else 'no'}")
    native.check_status()

    # ---- end to end: pinned host tokens -> device, step, loss back to the host, every step ----
    from param_decomp_b200.data.synthetic import ZipfTokenSource

    src = ZipfTokenSource(run.arch.vocab_size, cfg.data.seq_len, 1.1, 0)
    host_batches = [src.batch(1000 + i, cfg.pd.batch_size, topo.data_rank, topo.data_world, pin=True)
                    for i in range(args.steps)]
    h2d = host_batches[0].tokens.numel() * host_batches[0].tokens.element_size()
    trace("before the first barrier")
    sync()
    trace("end-to-end loop starts")
    t0 = time.perf_counter()
    for hb in host_batches:
        m = step_fn(hb.to(topo.device, non_blocking=True))  # pinned host tokens -> device, every step
        loss_host = float(m["loss/total"])  # device -> host read of the step's result
    sync()
    e2e_s = time.perf_counter() - t0
    e2e_t = torch.tensor([e2e_s], device=topo.device)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_tokens_per_s = tokens_per_step * args.steps / float(e2e_t.item())

    # ---- device-timed: batches resident on the device, CUDA events, max over ranks ----
    dev_batches = [hb.to(topo.device) for hb in host_batches]
    sampler = ClockSampler(topo.device.index or 0)
    launches0 = native.launch_count()
    sync()
    if topo.rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.profile_range:
        torch.cuda.profiler.start()
    e0.record()
    host_t0 = time.perf_counter()
    for b in dev_batches:
        step_fn(b)
    host_issue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps  # host time to issue a step (no wait on the device)
    e1.record()
    if args.profile_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    sync()
    clocks = sampler.stop() if topo.rank == 0 else {}
    launches = native.launch_count() - launches0
    native.check_status()
    if args.kernel_table is not None:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            step_fn(dev_batches[0])
            torch.cuda.synchronize()
        if topo.rank == 0:
            args.kernel_table.parent.mkdir(parents=True, exist_ok=True)
            args.kernel_table.write_text(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=40,
                                                                    max_name_column_width=90))
        sync()
    ms = torch.tensor([e0.elapsed_time(e1)], device=topo.device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)

    if topo.rank == 0:
        arch = run.arch
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "impl": "ours" if fused else "ours, eager_torch backend (cuBLAS / torch SDPA): context only",
            "data": "synthetic Zipf(1.1) token ids, seeded random-init target weights",
            "config": {
                "model": (f"{arch.family} {arch.n_layer}L d{arch.d_model} h{arch.n_head} ff{arch.d_ff} vocab{arch.vocab_size}"
                          + (f" experts{arch.n_experts} top{arch.experts_per_token}" if arch.family == "moe" else "")),
                "config_file": str(args.config.relative_to(ROOT)) if args.config.is_relative_to(ROOT) else str(args.config),
                "global_batch": cfg.pd.batch_size, "seq_len": cfg.data.seq_len,
                "parallelism": ((f"fsdp{topo.data_world}" + (f" x tp{args.tp}" + (f" {args.expert_dispatch}" if run.ep is not None else "") if args.tp > 1 else "")
                                 + (f" (placement {lay.rules.name}: masters, moments and gradient reduction sharded over "
                                    f"the batch axes, {args.optim}; bf16 compute copy re-gathered once per step)"
                                    if shard_backend else " (replicated optimizer, gradient all-reduce)"))
                                if world > 1 else "single"),
                "decomposition": (", ".join(f"{k}:{v}" for k, v in cfg.decomposition.sites.cs.items())
                                  + f" components per matrix x {arch.n_layer} layers; CI fn {cfg.decomposition.ci.type}"),
                "losses": ", ".join(type(m).__name__ for m in cfg.pd.loss_metrics),
                "step_issue": ("one CUDA graph per step (recorded after the eager warm-up)" if step_fn.graph is not None
                               else f"launch by launch ({step_fn.reason})"),
                "l2": "per-step working set (>4 GB parameters and optimizer state, >20 GB activations) "
                      "exceeds the 126 MB L2; no explicit flush between steps",
            },
            "clocks": clocks,
            "e2e": {"value": e2e_tokens_per_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "last_loss": loss_host},
            "gpu_launches": launches,
            "host_issue_ms_per_step": round(host_issue_ms, 3),
        }))
    step_fn.release()  # the recorded graph holds NCCL work: it must go before the process group does
    topo.shutdown()


if __name__ == "__main__":
    main()
