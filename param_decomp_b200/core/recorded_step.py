"""The train step recorded once as a CUDA graph and replayed.

A flagship step is ~1,500 kernel launches; issued one by one from Python they cost more host time
than the GPU needs to run them once the per-rank batch is small (8 GPUs: 4,096 tokens per rank).
The reference removes that cost by compiling the whole step into one executable
(param_decomp/core/run.py:1148-1157). Here the same `train_step` that runs eagerly is recorded into
a CUDA graph after a few eager steps, and every later step is: refresh the step-scalar table
(`ops/step_scalars.py`: seed word, schedules, learning rates, bias corrections, barrier sequence
numbers - one small pinned-memory copy), copy the batch into the recording's input buffers, launch
the graph. Nothing about the step is re-decided on the host, so a replay costs microseconds of CPU.

What may be recorded: steps whose control flow and host-side state do not depend on the step index
beyond what the scalar table carries - stochastic / CI-masked / unmasked reconstruction terms and
fresh PGD, smooth-L0 minimality without the frequency EMA, faithfulness, AdamW (replicated or
sharded). Persistent adversaries, the frequency EMA, L_p annealing, the non-target stream of targeted
runs, Muon and activation recompute keep host state that changes per step; such runs stay eager
(`RecordedTrainStep.eligible` says which, and why).
"""

from __future__ import annotations

from dataclasses import fields, is_dataclass
from typing import Any

import torch
from torch import Tensor

from param_decomp_b200.config import losses as L
from param_decomp_b200.config.run import AdamWOptimizerConfig, TargetedPDConfig
from param_decomp_b200.core.train import StepContext, TrainState, train_step


def _why_not(ctx: StepContext, state: TrainState) -> str | None:
    model = ctx.model
    if getattr(model, "backend", "eager_torch") != "fused_sm100" or not torch.cuda.is_available():
        return "the eager backend is not recorded"
    if isinstance(ctx.pd, TargetedPDConfig) or ctx.nontarget is not None:
        return "targeted runs keep a second stream and CI-scaled weight decay on the host"
    obj = ctx.objective
    if obj.persistent_terms():
        return "persistent adversaries keep optimizer state on the host"
    mini = obj.minimality
    if not isinstance(mini, L.ImportanceMinimalityLossConfig):
        return "L_p annealing is evaluated on the host"
    if mini.frequency is not None and mini.frequency.ema_halflife_steps is not None:
        return "the frequency EMA is updated on the host"
    if obj.nonlinearity is not None:
        return "the nonlinearity-locality threshold is evaluated on the host"
    if any(t.auxiliaries for t in obj.recon):
        return "auxiliary comparisons are evaluated eagerly"
    if ctx.remat_recon_forwards or ctx.remat_ci_fn:
        return "activation recompute re-enters Python during the backward pass"
    if ctx.expert_shard is not None or getattr(model, "ep", None) is not None:
        return "tensor- / expert-split steps are not recorded"
    for opt in (state.components_opt, state.ci_fn_opt):
        if not isinstance(opt.cfg, AdamWOptimizerConfig):
            return "Muon's Newton-Schulz schedule runs on the host"
        if not (getattr(opt, "use_fused", False) or hasattr(opt, "working_view")):
            return "the optimizer runs on torch ops with host-side scalars"
    return None


def _tensors_of(batch: Any) -> list[tuple[Any, str, Tensor]]:
    """`(owner, attribute, tensor)` of every tensor field of a (dataclass or plain tensor) batch."""
    if isinstance(batch, Tensor):
        return [(None, "", batch)]
    assert is_dataclass(batch), f"cannot record a step on a batch of type {type(batch).__name__}"
    return [(batch, f.name, getattr(batch, f.name)) for f in fields(batch) if isinstance(getattr(batch, f.name), Tensor)]


class RecordedTrainStep:
    """`step(batch) -> metrics`, eager for the first `eager_steps` calls (they also size the caching allocator
    and create the gradient buffers), recorded at the next call, replayed afterwards. Metrics are device tensors
    owned by the recording: read them (`float(...)`) before the next call."""

    def __init__(self, ctx: StepContext, state: TrainState, enabled: bool = True, eager_steps: int = 3,
                 concurrent: bool = True) -> None:
        self.ctx, self.state = ctx, state
        self.eager_steps = eager_steps
        self.reason = None if enabled else "recording is switched off"
        if self.reason is None:
            self.reason = _why_not(ctx, state)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._calls = 0
        self._static_batch: Any = None
        self._metrics: dict[str, Tensor] = {}
        self.replays = 0
        if self.eligible:
            from param_decomp_b200.ops.step_scalars import StepScalars

            dev = next(state.components.parameters()).device
            if ctx.scalars is None:
                ctx.scalars = StepScalars(dev)
            for label, opt in (("components", state.components_opt), ("ci_fn", state.ci_fn_opt)):
                opt.scalars, opt.label = ctx.scalars, label
            if concurrent and ctx.lanes is None:
                from param_decomp_b200.ops.lanes import Lanes

                ctx.lanes = Lanes()
                if hasattr(ctx.model, "_block"):
                    ctx.model.lanes = ctx.lanes  # q / k / v and gate / up of a block fork too

    @property
    def eligible(self) -> bool:
        return self.reason is None

    def release(self) -> None:
        """Destroy the recording. Must happen before the process group is torn down: a communicator whose
        collectives are part of a live CUDA graph does not finish its destruction (the process would hang
        at exit)."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph.reset()
            self.graph = None
            self._metrics = {k: v.detach().clone() for k, v in self._metrics.items()}

    def __call__(self, batch: Any, nontarget_batch: Any = None) -> dict[str, Tensor]:
        if not self.eligible:
            return train_step(self.ctx, self.state, batch, nontarget_batch)
        self._calls += 1
        if self._calls <= self.eager_steps:
            return train_step(self.ctx, self.state, batch)
        if self.graph is None:
            return self._record(batch)
        return self._replay(batch)

    # -- recording ---------------------------------------------------------------------------------
    def _record(self, batch: Any) -> dict[str, Tensor]:
        ctx, state = self.ctx, self.state
        dev = ctx.scalars.words.device
        if isinstance(batch, Tensor):
            self._static_batch = batch.to(dev).clone()
        else:
            self._static_batch = type(batch)(**{f.name: (getattr(batch, f.name).to(dev).clone()
                                                        if isinstance(getattr(batch, f.name), Tensor)
                                                        else getattr(batch, f.name)) for f in fields(batch)})
        from param_decomp_b200.ops import native

        torch.cuda.synchronize()
        torch.cuda.empty_cache()  # the eager steps' cached blocks: the recording allocates from its own pool
        ctx.scalars.begin(state.step)
        graph = torch.cuda.CUDAGraph()
        before = native.launch_count()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self._metrics = train_step(ctx, state, self._static_batch)  # advances the host-side counters once
        self.launches_per_step = native.launch_count() - before  # this library's kernels in one step
        ctx.scalars.frozen = True
        self.graph = graph
        graph.replay()  # the recording itself executed nothing: run the step it describes
        self.replays += 1
        return self._metrics

    def _replay(self, batch: Any) -> dict[str, Tensor]:
        from param_decomp_b200.ops import native

        ctx, state = self.ctx, self.state
        for (_, name, dst), (_, _, src) in zip(_tensors_of(self._static_batch), _tensors_of(batch)):
            assert dst.shape == src.shape, f"batch field {name!r} changed shape: {tuple(src.shape)} vs {tuple(dst.shape)}"
            dst.copy_(src, non_blocking=True)
        ctx.scalars.begin(state.step)
        self.graph.replay()  # type: ignore[union-attr]
        self.replays += 1
        native.count_launch(self.launches_per_step)
        state.step += 1
        state.components_opt.advance_replayed()
        state.ci_fn_opt.advance_replayed()
        return self._metrics
