"""LM composition root: topology -> target -> CI function -> data -> evaluation -> engine.

Parity: param_decomp/experiments/lm/training.py:197-301 (`_train`), :315-371 (`main`).
"""

from __future__ import annotations

import os
from pathlib import Path


from param_decomp_b200.config.experiments import LMExperimentConfig, LMTargetedExperimentConfig
from param_decomp_b200.core.metrics import MetricsSink, device_peak_flops, get_logger, mint_run_id, pin_launch_config, run_dir_for
from param_decomp_b200.core.run import RunResult, run_decomposition_training
from param_decomp_b200.experiments.lm.build import build_lm_run


def optimizer_sharding(cfg: LMExperimentConfig | LMTargetedExperimentConfig, topo) -> tuple[object, str | None]:
    """The optimizer layout the run's placement table asks for on this topology (`parallel/layout.py`): tables whose
    component optimizer state is sharded over the batch axes (every preset but `ddp`) run the flat-sharded optimizer
    - the fused reduce-scatter + AdamW + all-gather kernel over NVLink peer memory on GPUs, the collective (gloo /
    NCCL) form elsewhere; `ddp` keeps replicated masters and all-reduces gradients."""
    from param_decomp_b200.parallel import layout

    if topo.data_world <= 1:
        return None, None
    if not layout.resolve(cfg.runtime, world=topo.world).optimizer_sharded:
        return None, None
    backend = "fused_p2p" if topo.device.type == "cuda" and getattr(cfg.runtime, "backend", "") == "fused_sm100" else "collective"
    return topo.data_group, backend


def warn_inert_options(cfg, log) -> None:
    """Name every runtime option that parses (the schema is shared with XLA-based configs) and has no effect
    here, once per run, instead of ignoring it silently."""
    rt = cfg.runtime
    if rt.compiler_options != "bare":
        log.warning("runtime.compiler_options=%r has no effect: there is no tracing compiler, the step is hand-written "
                    "kernels recorded as a CUDA graph", rt.compiler_options)
    if "compilation_cache_dir" in rt.model_fields_set:
        log.warning("runtime.compilation_cache_dir has no effect: nothing is compiled at run time")
    name = rt.sharding if isinstance(rt.sharding, str) else "table"
    if name not in ("ddp",) and cfg.runtime.mesh is not None:
        log.info("runtime.sharding=%s: masters, moments and gradient reduction are sharded over the batch axes "
                 "(reduce-scatter + AdamW + all-gather in one kernel per step); the bf16 working copy is re-gathered "
                 "once per step, not per layer", name)


def check_runtime_supported(cfg) -> None:
    """Refuse, rather than silently ignore, runtime options this engine does not act on."""
    if cfg.runtime.sequence_sharding != "replicate":
        family = getattr(getattr(cfg.target.spec, "arch", None), "family", None)
        kind = getattr(cfg.decomposition.sites, "kind", "")
        if family in ("moe", "qwen35_moe") or kind in ("moe", "qwen36_moe"):
            raise NotImplementedError(
                "runtime.sequence_sharding=sequence_parallel (position-sharded residual stream between blocks, "
                "param_decomp/core/placement.py:273-287) is built for dense transformer targets whose component "
                "axis is split over tp; on mixture-of-experts targets the tp axis splits experts and keeps the "
                "residual stream whole on every rank")


def apply_sequence_sharding(cfg, model, topo, log) -> None:
    """`sequence_parallel`: masked passes of a dense target carry the residual position-sharded over the tp group."""
    if cfg.runtime.sequence_sharding == "replicate":
        return
    if getattr(model, "component_group", None) is None:
        log.info("runtime.sequence_sharding=sequence_parallel has no effect without a tp axis (tp = %d)", topo.tp_world)
        return
    assert cfg.data.seq_len % topo.tp_world == 0, \
        f"sequence_parallel: seq_len {cfg.data.seq_len} must be a multiple of the tp axis ({topo.tp_world})"
    model.sequence_parallel = True
    log.info("sequence-parallel residual: masked passes keep [batch, %d / %d, d_model] per rank between blocks",
             cfg.data.seq_len, topo.tp_world)


def expert_mode_of(cfg) -> str:
    """`target.expert_implementation: all_to_all` selects token dispatch to the experts' owners (the batch is then
    sharded over the tp axis as well); every other value keeps the reference's activation slicing."""
    return "all_to_all" if getattr(cfg.target, "expert_implementation", "") == "all_to_all" else "allreduce"


def expert_group_of(topo):
    """The mesh's `tp` axis is the expert-shard axis of a mixture-of-experts target
    (param_decomp/core/placement.py:1040-1048: blocked sites place `expert -> tp`)."""
    return topo.groups.get("tp") if topo.tp_world > 1 else None


def train_lm(cfg: LMExperimentConfig, data_root: Path | None, run_id: str | None = None, device: str | None = None,
             max_steps_this_entry: int | None = None, state_out: list | None = None) -> RunResult:
    from param_decomp_b200.parallel import topology

    check_runtime_supported(cfg)
    mode = expert_mode_of(cfg)
    topo = topology.initialize(cfg.runtime.mesh, device, batch_over_tp=mode == "all_to_all")
    log = get_logger(topo.rank)
    warn_inert_options(cfg, log)
    run = build_lm_run(cfg, data_root, topo.device, topo.data_rank, topo.data_world, expert_group=expert_group_of(topo),
                       expert_mode=mode)
    apply_sequence_sharding(cfg, run.model, topo, log)
    collectives = topo.collectives()
    from param_decomp_b200.parallel import layout as layout_mod

    lay = layout_mod.resolve(cfg.runtime, sites=getattr(run.model, "global_sites", run.model.sites), world=topo.world)
    log.info("placement: %s; stacks padded to multiples of %d", lay.label, lay.stack_multiple)
    shard_group, shard_backend = optimizer_sharding(cfg, topo)
    if run.ep is not None:
        shard_group, shard_backend = None, None  # expert blocks differ per tp rank: replicated-optimizer layout
    elif getattr(run.model, "component_group", None) is not None and shard_backend is not None:
        shard_backend = "collective"  # component slices: sharded over the batch axes, clip norm summed over tp

    run_dir, sink = None, None
    if data_root is not None:
        run_id = topo.broadcast_object(run_id or mint_run_id())
        run_dir = run_dir_for(data_root, run_id)
        if topo.rank == 0:
            pin_launch_config(run_dir, cfg.to_yaml())
        sink = MetricsSink.for_run(run_dir, topo.rank, cfg.wandb, cfg.run_name, cfg.model_dump(mode="json"))
        log.info("run dir %s", run_dir)

    from param_decomp_b200.evals.lm import LMEvaluation
    from param_decomp_b200.utils.flops import decomposition_step_flops

    evaluation = None
    if cfg.eval is not None:
        evaluation = LMEvaluation(cfg.eval, run.sample_eval, run_dir=run_dir,
                                  encode=prompt_encoder_for(cfg, data_root, run.arch.vocab_size, log))
    fused = getattr(run.model, "backend", "") == "fused_sm100"
    flops = decomposition_step_flops(run.model, run.ci_fn, cfg.pd, cfg.data.seq_len)
    try:
        result = run_decomposition_training(
            run.model, run.ci_fn, cfg.pd, cfg.cadence, run.sample_train, device=topo.device, run_dir=run_dir,
            sink=sink, evaluation=evaluation, collectives=collectives, resume_provenance=cfg.resume_provenance,
            batch_rows=cfg.pd.batch_size // topo.data_world, positions=cfg.data.seq_len,
            units_per_step=run.tokens_per_step, flops_per_step=flops / topo.world, peak_flops=device_peak_flops(),
            lazy_masks=fused, use_fused_optim=fused, init_components=run.init_components,
            max_steps_this_entry=max_steps_this_entry, state_out=state_out, stack_multiple=lay.stack_multiple,
            **profiling_arguments(cfg.runtime.profiling),
            shard_group=shard_group, shard_backend=shard_backend, peer_wait_limit_s=cfg.runtime.peer_wait_limit_s,
            record_step=fused and cfg.runtime.step_recording == "cuda_graph",
            remat_recon_forwards=cfg.runtime.remat_recon_forwards, remat_ci_fn=cfg.runtime.remat_ci_fn,
            step_watchdog_s=cfg.runtime.step_watchdog_s)
    except BaseException:
        if sink is not None:
            sink.close()
        topo.shutdown(failed=True)
        raise
    if sink is not None:
        sink.close()
    topo.shutdown()
    return result


def profiling_arguments(profiling) -> dict:
    """`runtime.profiling` as the engine's `profile_*` arguments."""
    if profiling.kind == "ad_hoc":
        return dict(profile_steps=profiling.steps, profile_kind="trace")
    if profiling.kind == "nsight_systems":
        return dict(profile_steps=profiling.capture_steps, profile_warmup=profiling.warmup_steps,
                    profile_kind="cuda_profiler_range")
    return {}


def prompt_encoder_for(cfg, data_root: Path | None, vocab_size: int, log=None):
    """The run's text-to-token encoder, needed only when something builds prompts from text: an
    `ArithmeticCIGrid` metric or a text prompt pool. Otherwise None, and no tokenizer is looked for."""
    from param_decomp_b200.config.evals import ArithmeticCIGridConfig
    from param_decomp_b200.experiments.lm.prompt_encoder import resolve_prompt_encoder

    wants = cfg.eval is not None and any(isinstance(m, ArithmeticCIGridConfig) for m in cfg.eval.metrics)
    pool = getattr(cfg, "prompts", None)
    wants = wants or (pool is not None and (pool.kind != "inline" or pool.prompts is not None))
    if not wants:
        return None
    return resolve_prompt_encoder(cfg.target.spec, cfg.data.train, data_root, vocab_size, log)


def train_lm_targeted(cfg: LMTargetedExperimentConfig, data_root: Path | None, run_id: str | None = None,
                      device: str | None = None, max_steps_this_entry: int | None = None,
                      state_out: list | None = None, encode=None) -> RunResult:
    """Targeted decomposition (tPD): every step sees a TARGET batch drawn from the prompt pool (full
    reconstruction vocabulary, no faithfulness) and a broad NONTARGET batch from the corpus
    (`nontarget:` losses, delta pinned on, no adversaries). Parity:
    param_decomp/experiments/lm/training_targeted.py, targeted_data.py, core/run.py:1202-1353."""
    from param_decomp_b200.core.objective import build_nontarget_objective, build_objective
    from param_decomp_b200.experiments.lm.targeted_data import PromptPool
    from param_decomp_b200.parallel import topology

    check_runtime_supported(cfg)
    mode = expert_mode_of(cfg)
    topo = topology.initialize(cfg.runtime.mesh, device, batch_over_tp=mode == "all_to_all")
    log = get_logger(topo.rank)
    run = build_lm_run(cfg, data_root, topo.device, topo.data_rank, topo.data_world, expert_group=expert_group_of(topo),
                       expert_mode=mode)
    apply_sequence_sharding(cfg, run.model, topo, log)
    if encode is None:
        encode = prompt_encoder_for(cfg, data_root, run.arch.vocab_size, log)
    pool = PromptPool.build(cfg.prompts, run.arch.vocab_size, data_root, cfg.pd.seed, encode=encode)
    n_target_terms = len(build_objective(cfg.pd).recon)
    nontarget = build_nontarget_objective(cfg.nontarget, first_index=n_target_terms)
    nt_rows = cfg.nontarget.batch_size

    def sample_target(step: int):
        return pool.batch(step, cfg.pd.batch_size, topo.data_rank, topo.data_world).to(topo.device)

    def sample_nontarget(step: int):
        full = run.sample_train(step)  # the corpus stream, cut to the non-target batch size
        rows = max(1, nt_rows // topo.data_world)
        cut = lambda t: None if t is None else t[:rows]  # noqa: E731
        return type(full)(tokens=full.tokens[:rows], segment_ids=cut(full.segment_ids), positions=cut(full.positions))

    run_dir, sink = None, None
    if data_root is not None:
        run_id = topo.broadcast_object(run_id or mint_run_id())
        run_dir = run_dir_for(data_root, run_id)
        if topo.rank == 0:
            pin_launch_config(run_dir, cfg.to_yaml())
        sink = MetricsSink.for_run(run_dir, topo.rank, cfg.wandb, cfg.run_name, cfg.model_dump(mode="json"))
        log.info("run dir %s", run_dir)
    from param_decomp_b200.evals.lm import LMEvaluation

    evaluation = None
    if cfg.eval is not None:
        evaluation = LMEvaluation(cfg.eval, run.sample_eval, run_dir=run_dir, encode=encode)
    fused = getattr(run.model, "backend", "") == "fused_sm100"
    try:
        result = run_decomposition_training(
            run.model, run.ci_fn, cfg.pd, cfg.cadence, sample_target, device=topo.device, run_dir=run_dir, sink=sink,
            evaluation=evaluation, collectives=topo.collectives(), nontarget=nontarget,
            step_watchdog_s=cfg.runtime.step_watchdog_s,
            remat_recon_forwards=cfg.runtime.remat_recon_forwards, remat_ci_fn=cfg.runtime.remat_ci_fn,
            # adversary sources exist for the TARGET stream only: its rows per rank and its prompt length
            sample_nontarget_batch=sample_nontarget, batch_rows=cfg.pd.batch_size // topo.data_world,
            positions=pool.seq_len, units_per_step=(cfg.pd.batch_size * pool.seq_len + nt_rows * cfg.data.seq_len),
            lazy_masks=fused, use_fused_optim=fused, init_components=run.init_components,
            max_steps_this_entry=max_steps_this_entry, state_out=state_out)
    except BaseException:
        if sink is not None:
            sink.close()
        topo.shutdown(failed=True)
        raise
    if sink is not None:
        sink.close()
    topo.shutdown()
    return result
