"""The decomposition train step.

One call = one optimizer update of the component stacks and the CI function:

  clean forward (no grad) -> taps, clean output, captures
  compute weights: fp32 masters -> compute dtype, once per step
  CI function -> lower / upper importances
  persistent adversaries: `n_warmup_steps` source ascents on detached weights and CI
  loss = c_f * faithfulness + minimality (+ frequency) (+ nonlinearity locality)
         + sum_terms c_t * mean_draws recon(masked forward under the term's masks)
  backward; per-group clip + AdamW | Muon; final adversary ascent with the main backward's
  source gradients (unscaled by the term coefficient)

Where the reference compiles this into one XLA executable (param_decomp/core/train.py:1113-1349),
here it is an explicit sequence of launches on CUDA streams; the masked forwards dispatch to the
fused sm_100a site kernels when the model was built with `backend="fused_sm100"`.

Parity: core/train.py:578-690 (stream prep, masked recon), :693-811 (adversary ascents),
:814-915 (draw loop), :977-1031 (apply gradients), :1050-1096 (metrics), :1355-1791 (targeted
two-stream step), :1813-1838 (faithfulness warm-up).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch import Tensor, nn

from param_decomp_b200.config import losses as L
from param_decomp_b200.config.run import PDConfig, TargetedPDConfig
from param_decomp_b200.config.schedule import get_scheduled_value, run_fraction, scheduled_or_constant
from param_decomp_b200.core import adversary as adv_mod
from param_decomp_b200.core import losses as loss_fns
from param_decomp_b200.core import masking, rng
from param_decomp_b200.core.adversary import PersistentAdversary
from param_decomp_b200.core.ci_fn.interface import CI, squash
from param_decomp_b200.core.components import ComponentStacks, ComputeWeights, SelectedCI, prepare_compute_weights
from param_decomp_b200.core.model import DecomposedModel, ForwardResult, target_weight_sq_norms, target_weights
from param_decomp_b200.core.objective import NontargetObjective, PDObjective, ReconTerm
from param_decomp_b200.core.optim import GroupOptimizer
from param_decomp_b200.core.rng import StepKey


class phase:
    """NVTX range around one phase of the step (`clean`, `ci_fn`, `adversary`, `losses`, `draws`, `backward`,
    `optimizer`), so that timelines and captures are attributable; free when no CUDA device is in use
    (the reference labels the same phases with `jax.named_scope`, param_decomp/core/train.py:1247)."""

    enabled = torch.cuda.is_available()
    ledger = None
    """A `core/debug/memory_ledger.py::Ledger` while a profiled step is being attributed: every phase leaves a mark
    (allocator counters and the largest live tensors) as it ends."""

    def __init__(self, name: str) -> None:
        self.name = name

    def __enter__(self) -> None:
        if phase.enabled:
            torch.cuda.nvtx.range_push("pd/" + self.name)

    def __exit__(self, *exc) -> None:
        if phase.enabled:
            torch.cuda.nvtx.range_pop()
        if phase.ledger is not None:
            phase.ledger.mark(self.name)


class DataCollectives:
    """What the step needs from the data-parallel group. The default is a single process; the
    `parallel` package supplies the NCCL / gloo implementation."""

    world_size: int = 1
    rank: int = 0

    def mean(self, t: Tensor) -> Tensor:
        """Differentiable mean over data-parallel ranks."""
        return t

    def row_offset(self, local_rows: int) -> int:
        """Global index of this rank's first row (keys the Philox row counter)."""
        return 0

    def reduce_grads(self, params: list[Tensor]) -> None:
        """Average `.grad` over data-parallel ranks (no-op for one process)."""

    def sum_(self, t: Tensor) -> Tensor:
        return t

    def gather_rows(self, t: Tensor) -> Tensor:
        """Concatenation over the batch shards on dim 0 (global-batch layout of a per-row tensor)."""
        return t

    def reduce_grads_everywhere(self, params: list[Tensor]) -> None:
        """Average `.grad` over EVERY rank of the job (leaves replicated over the non-batch axes too)."""
        self.reduce_grads(params)

    def reduce_split_grads(self, params: list[Tensor]) -> None:
        """Average `.grad` of leaves that are split over the tp axis (see the distributed implementation)."""
        self.reduce_grads(params)

    in_first_tp_group: bool = True

    def average_scalars(self, values: dict) -> dict:
        """Mean over ranks of the scalar entries of an evaluation result (every rank evaluated its own rows)."""
        return values
    split_grad_scale: float = 1.0  # see `DistCollectives.split_grad_scale`


@dataclass
class TrainState:
    components: ComponentStacks
    ci_fn: nn.Module
    components_opt: GroupOptimizer
    ci_fn_opt: GroupOptimizer
    adversaries: dict[str, PersistentAdversary] = field(default_factory=dict)
    frequency: dict[str, loss_fns.FrequencyEMA] = field(default_factory=dict)
    step: int = 0


@dataclass
class StepContext:
    """Per-run constants the step closes over."""

    model: DecomposedModel
    objective: PDObjective
    pd: PDConfig | TargetedPDConfig
    weights_W: dict[str, Tensor]
    weights_sq: dict[str, Tensor]
    site_index: dict[str, int]
    collectives: DataCollectives = field(default_factory=DataCollectives)
    lazy_masks: bool = False  # fused backend draws stochastic masks in-kernel
    nontarget: NontargetObjective | None = None
    relative_faithfulness: bool = True
    expert_shard: Any = None  # parallel.expert_shard.StackSharding when expert blocks are split over ranks
    # activation recompute (param_decomp/targets/transformer.py:1910-1918, experiments/lm/runtime.py:340-360):
    # a masked forward / the CI function keeps only its inputs and is run again during the backward pass
    remat_recon_forwards: bool = False
    remat_ci_fn: bool = False
    lanes: Any = None  # `ops.lanes.Lanes`: the mask draws of a term run side by side on CUDA side streams
    # `ops.step_scalars.StepScalars`: when set, everything the host computes per step (Philox seed word,
    # scheduled coefficients, learning rates and bias corrections) is read by the kernels from a device
    # table instead of being passed by value, so the step's launches can be recorded once and replayed
    scalars: Any = None

    def sched(self, name: str, value: Any, step: int):
        """A scheduled quantity at `step`: a python float, or - for a real schedule while the step keeps its
        scalars in device memory - the 0-d device tensor that holds it. Bare floats never change and stay
        python numbers."""
        from param_decomp_b200.config.schedule import ScheduleConfig

        total = self.pd.steps
        if self.scalars is None or not isinstance(value, ScheduleConfig):
            return scheduled_or_constant(value, step, total)
        return self.scalars.f32("sched/" + name, lambda s: get_scheduled_value(min(s, total), total, value))

    def weights_sq_host(self) -> dict[str, float]:
        """`||W_s||^2` as host floats (read back once, then cached)."""
        cached = getattr(self, "_wsq_host", None)
        if cached is None:
            cached = {k: float(v) for k, v in self.weights_sq.items()}
            self._wsq_host = cached
        return cached

    @classmethod
    def build(cls, model: DecomposedModel, objective: PDObjective, pd, **kw: Any) -> "StepContext":
        wsq = target_weight_sq_norms(model)
        shard = kw.get("expert_shard")
        if shard is not None:  # a split expert bank is normalised by the norm of the WHOLE bank
            for s in model.sites:
                if s.blocked:
                    wsq[s.name] = shard.sum_over_group(wsq[s.name].clone())
        return cls(model=model, objective=objective, pd=pd, weights_W=target_weights(model), weights_sq=wsq,
                   site_index={s.name: i for i, s in enumerate(model.sites)}, **kw)


# ---- recon evaluation -----------------------------------------------------------------------------


def _aux_loss(term: ReconTerm, clean: ForwardResult, masked: ForwardResult, step: int, total: int,
              metrics: dict[str, Tensor] | None) -> Tensor | None:
    total_aux = None
    for aux in term.auxiliaries:
        vals = []
        for cmp_ in aux.comparisons:
            a, b = clean.captures[cmp_.capture], masked.captures[cmp_.capture]
            if cmp_.distance == "relative_squared_error":
                vals.append(loss_fns.relative_squared_error(b, a))
            elif cmp_.distance == "categorical_kl_from_logits":
                vals.append(loss_fns.kl_from_logits(a, b))
            else:
                from param_decomp_b200.ops.attention_kl import attention_pattern_kl

                vals.append(attention_pattern_kl(a, b))
        mean = torch.stack(vals).mean()
        if metrics is not None:
            metrics[f"loss/{term.name}/{aux.name}"] = mean.detach()
        c = scheduled_or_constant(aux.coeff, step, total)  # (terms with auxiliaries are not recorded)
        total_aux = c * mean if total_aux is None else total_aux + c * mean
    return total_aux


def masked_recon(ctx: StepContext, weights: ComputeWeights, batch: Any, clean: ForwardResult,
                 masks: masking.Masks, term: ReconTerm, step: int, with_aux: bool,
                 metrics: dict[str, Tensor] | None = None) -> tuple[Tensor, Tensor]:
    """Returns `(e2e output loss, full term loss incl. auxiliaries)`."""
    keys = term.capture_keys() if with_aux else ()
    out = ctx.model.masked_forward(weights, batch, masks, capture=keys, clean=clean)
    e2e = ctx.model.recon_loss(clean, out)
    full = e2e
    if with_aux and term.auxiliaries:
        aux = _aux_loss(term, clean, out, step, ctx.pd.steps, metrics)
        if aux is not None:
            full = e2e + aux
    return e2e, full


def _routing_for(ctx: StepContext, term: ReconTerm, lead: tuple[int, ...], key: StepKey, draw: int,
                 row_offset: int, device) -> dict[str, Tensor | None] | None:
    if term.routing_kind == "all":
        return None
    return masking.sample_routing(term.routing_kind, term.routing_p, [s.name for s in ctx.model.sites],
                                  lead, key, term.index, draw, row_offset, device)


def _lead_of(ci_lower: dict[str, Tensor]) -> tuple[int, ...]:
    first = next(iter(ci_lower.values()))
    return tuple(first.shape[:-1])


def _rows(lead: tuple[int, ...]) -> int:
    n = 1
    for d in lead:
        n *= d
    return n


def build_masks(ctx: StepContext, term: ReconTerm, ci_lower: dict[str, Tensor], key: StepKey, draw: int,
                leaves: dict[str, Tensor] | None, state: TrainState | None, step: int) -> masking.Masks:
    lead = _lead_of(ci_lower)
    device = next(iter(ci_lower.values())).device
    row_offset = ctx.collectives.row_offset(_rows(lead))
    s = term.strategy
    if s == "ci_masked":
        masks = masking.ci_masks(ci_lower)
        routes = _routing_for(ctx, term, lead, key, draw, row_offset, device)
        if term.delta_pinned is not None:
            masks = {n: masking.SiteMask(mask=m.mask, delta=torch.full((*lead, 1), term.delta_pinned, device=device,
                                                                       dtype=m.mask.dtype)) for n, m in masks.items()}
        if routes is not None:
            masks = {n: masking.SiteMask(mask=m.mask, delta=m.delta, route=routes[n]) for n, m in masks.items()}
        return masks
    if s == "unmasked":
        return masking.unmasked(ci_lower)
    if s == "unmasked_no_delta":
        return masking.unmasked_no_delta(ci_lower)
    if s == "stochastic":
        routes = _routing_for(ctx, term, lead, key, draw, row_offset, device)
        return masking.stochastic_masks(ci_lower, key, term.index, draw, site_index=ctx.site_index,
                                        row_offset=row_offset, delta_pinned=term.delta_pinned, routing=routes,
                                        lazy=ctx.lazy_masks)
    assert leaves is not None, f"{term.name}: adversarial strategy needs source leaves"
    src, dlt = PersistentAdversary.split(leaves)
    if s in ("fresh_pgd", "persistent"):
        routes = _routing_for(ctx, term, lead, key, draw, row_offset, device)
        return masking.source_masks(ci_lower, src, dlt, routes)
    # merged (plain or pooled)
    frac = get_scheduled_value(step, ctx.pd.steps, term.cfg.adv_fraction)  # type: ignore[attr-defined]
    return masking.merged_masks(ci_lower, src, dlt, frac, key, term.index, draw, site_index=ctx.site_index,
                                routing_kind=term.routing_kind, routing_p=term.routing_p, row_offset=row_offset)


def _pool_pick(ctx: StepContext, term: ReconTerm, adv: PersistentAdversary, batch_rows: int, key: StepKey,
               device) -> Tensor | None:
    if adv.pool_size == 1:
        return None
    off = ctx.collectives.row_offset(batch_rows)
    u = rng.uniform(key, StepKey.stream(rng.PURPOSE_POOL, term.index), batch_rows, 1, off, device)[:, 0]
    return torch.clamp((u * adv.pool_size).long(), max=adv.pool_size - 1)


# ---- minimality -----------------------------------------------------------------------------------


def evaluate_minimality(ctx: StepContext, state: TrainState, ci: CI, step: int, metrics: dict[str, Tensor],
                        coeff_override: float | None = None, update_ema: bool = True) -> Tensor:
    cfg = ctx.objective.minimality
    total = ctx.pd.steps
    coeff = coeff_override if coeff_override is not None else ctx.sched("minimality", cfg.coeff, step)
    if isinstance(cfg, L.LpImportanceMinimalityLossConfig):
        p = loss_fns.anneal_linear(cfg.p_start, cfg.p_end, run_fraction(step, total))
        val = loss_fns.lp_importance_minimality(ci.dense_upper(), p, cfg.eps, cfg.beta, ctx.collectives.world_size,
                                                mean_over_ranks=ctx.collectives.mean)
        metrics["loss/" + cfg.instance_key] = val.detach()
        metrics["schedules/p"] = torch.tensor(p)
        return coeff * val
    gamma = ctx.sched("gamma", cfg.gamma, step)
    metrics["schedules/gamma"] = gamma if isinstance(gamma, Tensor) else torch.tensor(gamma)
    activity = None
    freq_total = None
    names = list(ci.lower)
    f_locals = [ci.activity[n] if ci.activity is not None
                else loss_fns.component_activity(ci.upper[n], gamma, cfg.normalize_at_one) for n in names]
    if ctx.collectives.world_size > 1:
        # global-batch mean BEFORE the log, all sites' `[C]` vectors packed into ONE (differentiable) all-reduce
        flat = ctx.collectives.mean(torch.cat([f.reshape(-1).float() for f in f_locals]))
        f_globals = [t.view_as(f) for t, f in zip(flat.split([f.numel() for f in f_locals]), f_locals)]
    else:
        f_globals = f_locals
    for name, f in zip(names, f_globals):
        act = f.sum()
        activity = act if activity is None else activity + act
        if cfg.frequency is not None:
            fr = cfg.frequency
            if fr.ema_halflife_steps is not None:
                ema = state.frequency.get(name)
                if ema is None:
                    ema = loss_fns.FrequencyEMA(fr.ema_halflife_steps, torch.zeros_like(f.detach()))
                    state.frequency[name] = ema
                if update_ema:
                    pen = ema.surrogate(f, fr.reference_datapoint_count)
                else:
                    pen = loss_fns.frequency_penalty(f, fr.reference_datapoint_count)
                metrics.setdefault("loss/FrequencyMinimalityLoss_batch", torch.zeros((), device=f.device))
                metrics["loss/FrequencyMinimalityLoss_batch"] = (
                    metrics["loss/FrequencyMinimalityLoss_batch"]
                    + loss_fns.frequency_penalty(f.detach(), fr.reference_datapoint_count))
            else:
                pen = loss_fns.frequency_penalty(f, fr.reference_datapoint_count)
            freq_total = pen if freq_total is None else freq_total + pen
    assert activity is not None
    metrics["loss/" + cfg.instance_key] = activity.detach()
    out = coeff * activity
    if freq_total is not None:
        fc = ctx.sched("frequency", cfg.frequency.coeff, step)  # type: ignore[union-attr]
        metrics["loss/FrequencyMinimalityLoss"] = freq_total.detach()
        out = out + fc * freq_total
    return out


# ---- the step -------------------------------------------------------------------------------------


def _lr_metric(ctx: StepContext, opt, lr: float) -> Tensor:
    """The applied learning rate for the log: read from the device table when the step keeps its scalars there
    (a replayed recording then still reports the current value)."""
    if ctx.scalars is not None:
        name = f"opt/{getattr(opt, 'label', '')}/hyper"
        if name in ctx.scalars._entries:
            e = ctx.scalars._entries[name]
            return ctx.scalars.words[e.slot:e.slot + 1].view(torch.float32).reshape(())
    return torch.tensor(lr)


def _detach_weights(w: ComputeWeights) -> ComputeWeights:
    return w.detached()


def _detach_ci(ci_lower: dict[str, Tensor]) -> dict[str, Tensor]:
    if hasattr(ci_lower, "map"):  # keeps the block selections of narrow sites
        return ci_lower.map(lambda v: v.detach())  # type: ignore[attr-defined]
    return {k: v.detach() for k, v in ci_lower.items()}


def _fusable_pre(v) -> bool:
    if isinstance(v, SelectedCI):
        t = v.values
        return t.is_cuda and t.dtype == torch.bfloat16 and v.C_block % 8 == 0
    return isinstance(v, torch.Tensor) and v.is_cuda and v.dtype == torch.bfloat16 and v.shape[-1] % 8 == 0


def run_ci_fn(ctx: StepContext, state: TrainState, clean: ForwardResult, step: int | None = None) -> CI:
    def ci_forward():
        return state.ci_fn(clean.taps, aux=clean.aux, components=state.components,
                           segment_ids=clean.aux.get("segment_ids"), positions=clean.aux.get("positions"))

    if ctx.remat_ci_fn and torch.is_grad_enabled():
        from torch.utils.checkpoint import checkpoint

        pre = checkpoint(ci_forward, use_reentrant=False)
    else:
        pre = ci_forward()
    cfg = ctx.objective.minimality
    needs_upper = isinstance(ctx.pd, TargetedPDConfig) and ctx.pd.ci_scaled_weight_decay is not None
    fusable = (step is not None and ctx.lazy_masks and isinstance(cfg, L.ImportanceMinimalityLossConfig)
               and not needs_upper  # (the fused pass emits lower importances + activity, no upper tensor)
               and all(_fusable_pre(v) for v in pre.values()))
    if fusable:
        from param_decomp_b200.core.ci_fn.interface import squash_fused

        return squash_fused(pre, ctx.sched("gamma", cfg.gamma, step), cfg.normalize_at_one)
    return squash(pre)


def reduce_source_grads(ctx: StepContext, grads: dict[str, Tensor], batch_shared: bool) -> dict[str, Tensor]:
    """Gradients of adversary sources under data parallelism, as the global-batch loss defines them
    (param_decomp/core/init_placed.py:197-235, core/train.py:790-807, core/recon_eval.py:142-257). A source
    shared over the batch (shape `c`, the evaluation probes) takes the MEAN over the batch shards of the
    ranks' gradients - one packed all-reduce for all leaves - so every rank ascends the same source. A per-row
    source (`bc` / `bsc`, every training adversary) belongs to one rank, whose local-mean loss over-weights
    it by the number of shards."""
    W = ctx.collectives.world_size
    if W == 1:
        return grads
    if not batch_shared:
        return {k: g / W for k, g in grads.items()}
    names = list(grads)
    flat = ctx.collectives.sum_(torch.cat([grads[k].reshape(-1).float() for k in names])) / W
    out, off = {}, 0
    for k in names:
        n = grads[k].numel()
        out[k] = flat[off:off + n].view_as(grads[k]).to(grads[k].dtype)
        off += n
    return out


def ascend_persistent(ctx: StepContext, state: TrainState, term: ReconTerm, weights: ComputeWeights, batch: Any,
                      clean: ForwardResult, ci_lower: dict[str, Tensor], key: StepKey, step: int) -> None:
    adv = state.adversaries[term.name]
    cfg = term.cfg
    n = cfg.n_warmup_steps  # type: ignore[attr-defined]
    if n == 0:
        return
    lr = get_scheduled_value(step, ctx.pd.steps, cfg.optimizer.lr_schedule)  # type: ignore[attr-defined]
    w_d, ci_d = _detach_weights(weights), _detach_ci(ci_lower)
    B = ctx.model.batch_size(batch)
    pick = _pool_pick(ctx, term, adv, B, key, next(iter(ci_d.values())).device)
    use_aux = cfg.adversary_objective == "term"  # type: ignore[attr-defined]
    for _ in range(n):
        all_leaves = adv.leaves()
        leaves = adv.select_particles(all_leaves, pick) if pick is not None else all_leaves
        masks = build_masks(ctx, term, ci_d, key, 0, leaves, state, step)
        e2e, full = masked_recon(ctx, w_d, batch, clean, masks, term, step, with_aux=use_aux)
        target = full if use_aux else e2e
        names = list(all_leaves)
        grads = torch.autograd.grad(target, [all_leaves[k] for k in names], allow_unused=True)
        gdict = {k: (g if g is not None else torch.zeros_like(all_leaves[k])) for k, g in zip(names, grads)}
        adv.ascend(reduce_source_grads(ctx, gdict, adv.batch_shared), lr, key)


def train_step(ctx: StepContext, state: TrainState, batch: Any, nontarget_batch: Any | None = None) -> dict[str, float]:
    """One update. Returns scalar metrics (python floats are produced by the caller on log steps;
    here they stay 0-d tensors to avoid host syncs)."""
    step, total = state.step, ctx.pd.steps
    key = StepKey(ctx.pd.seed, step)
    obj = ctx.objective
    metrics: dict[str, Tensor] = {}
    if ctx.scalars is not None:
        from param_decomp_b200.ops import native

        if ctx.scalars.step != step:  # (a recorded step's table is refreshed by whoever replays it)
            ctx.scalars.begin(step)
        seed_word = ctx.scalars.u64("philox_seed", lambda s: StepKey(ctx.pd.seed, s).seed64)
        native.set_step_seed(key.seed64, seed_word.data_ptr())

    with torch.no_grad(), phase("clean"):
        clean = ctx.model.clean_forward(batch, capture=obj.capture_keys())
    direct = getattr(ctx.model, "backend", "eager_torch") == "fused_sm100"
    sharded = hasattr(state.components_opt, "working_view")  # ZeRO-style optimizer owns grads + working copy
    ci_sharded = hasattr(state.ci_fn_opt, "working_view")  # the CI function's gradients ride the same fused path
    if sharded:
        state.components_opt.zero_grad()
    if ci_sharded:
        state.ci_fn_opt.zero_grad()
        state.ci_fn_opt.refresh_compute_fp32()  # this step's values into the modules' own fp32 storage (local)
    for p in ([] if sharded else state.components_opt.params) + ([] if ci_sharded else state.ci_fn_opt.params):
        if direct and p.grad is not None:
            p.grad.zero_()
        else:
            p.grad = None
    working = None
    if sharded and direct:
        opt = state.components_opt
        working = {n: opt.working_view(i) for i, n in enumerate(opt.names)}
    elif sharded:
        # eager backend: weight gradients come from autograd, so the forward reads the (gathered) fp32 masters
        # themselves; their `.grad` are views of the optimizer's flat gradient buffer and accumulate in place
        state.components_opt.refresh_full_fp32()
    weights = prepare_compute_weights(state.components, ctx.model.compute_dtype, direct_grads=direct,
                                      working=working)
    with phase("ci_fn"):
        ci = run_ci_fn(ctx, state, clean, step)
        ci_lower = ci.mask_inputs()

    with phase("adversary"):
        for term in obj.persistent_terms():
            ascend_persistent(ctx, state, term, weights, batch, clean, ci_lower, key, step)

    total_loss = None

    def add(x: Tensor) -> None:
        nonlocal total_loss
        total_loss = x if total_loss is None else total_loss + x

    losses_range = phase("losses")
    losses_range.__enter__()
    if obj.faith is not None:
        c_f = ctx.sched("faithfulness", obj.faith.coeff, step)
        from param_decomp_b200.ops import faithfulness as fused_faith

        shard = ctx.expert_shard
        if shard is not None:
            # each rank holds some experts' blocks: its loss (and gradients) cover those, the logged value is
            # the sum over the expert group of the split sites' terms plus the replicated sites' terms
            assert ctx.relative_faithfulness, "expert-split runs use the target-relative faithfulness"
            by_c = shard.by_component
            if sharded and direct:
                state.components_opt.refresh_full_fp32()  # the terms below read the fp32 masters
            terms = loss_fns.faithfulness_terms(state.components, ctx.weights_W, ctx.weights_sq,
                                                component_group=shard.group if by_c else None)
            split = torch.tensor([s.blocked and not by_c for s in state.components.sites], device=terms.device)
            faith = terms.mean()
            whole = (terms.detach() * ~split).sum() + shard.sum_over_group((terms.detach() * split).sum())
            metrics["loss/" + obj.faith.instance_key] = whole / len(state.components.sites)
            unseen = c_f * (whole / len(state.components.sites) - faith.detach())  # other ranks' experts
            k = ctx.collectives.split_grad_scale
            if k != 1.0:  # batch-independent term on split leaves: cancel the batch-shard division of their gradients
                faith_g = (terms * torch.where(split, k, 1.0)).mean()
                faith = faith.detach() + (faith_g - faith_g.detach())
            add(c_f * faith)
        elif direct and ctx.relative_faithfulness and fused_faith.blocked_supported(state.components):
            fused_faithfulness = fused_faith.fused_faithfulness

            hi_lo = None
            if sharded and state.components_opt.work_lo_flat is not None:
                opt = state.components_opt
                hi_lo = {n: (opt.working_view(i), opt.working_lo_view(i)) for i, n in enumerate(opt.names)}
            faith = fused_faithfulness(state.components, ctx.weights_W, ctx.weights_sq_host(), c_f, hi_lo=hi_lo,
                                       rank=getattr(ctx.collectives, "data_rank", 0) if sharded else 0,
                                       world=ctx.collectives.world_size if sharded else 1)
            if sharded:
                faith = ctx.collectives.sum_(faith)
        else:
            faith = loss_fns.faithfulness_loss(state.components, ctx.weights_W, ctx.weights_sq,
                                               relative=ctx.relative_faithfulness)
        if shard is None:
            metrics["loss/" + obj.faith.instance_key] = faith.detach()
            add(c_f * faith)
    add(evaluate_minimality(ctx, state, ci, step, metrics))
    if obj.nonlinearity is not None:
        nl = obj.nonlinearity
        thr = get_scheduled_value(step, total, nl.relative_threshold)
        metrics["schedules/nonlinearity_relative_threshold"] = torch.tensor(thr)
        val = loss_fns.nonlinearity_locality(state.components, thr, dict(nl.unit_kind_coefficients), nl.normalize_at_one,
                                             expert_shard=ctx.expert_shard,
                                             split_grad_scale=ctx.collectives.split_grad_scale)
        metrics["loss/" + nl.instance_key] = val.detach()
        add(scheduled_or_constant(nl.coeff, step, total) * val)

    losses_range.__exit__()
    draws_range = phase("draws")
    draws_range.__enter__()
    source_grad_requests: list[tuple[ReconTerm, dict[str, Tensor], Tensor]] = []
    B = ctx.model.batch_size(batch)
    for term in obj.recon:
        leaves = None
        all_leaves = None
        if term.is_persistent:
            adv = state.adversaries[term.name]
            all_leaves = adv.leaves()
            pick = _pool_pick(ctx, term, adv, B, key, next(iter(ci_lower.values())).device)
            leaves = adv.select_particles(all_leaves, pick) if pick is not None else all_leaves
        elif term.strategy == "fresh_pgd":
            leaves = fresh_pgd_sources(ctx, term, weights, batch, clean, ci_lower, key, step)
        vals_e2e, vals_full = [], []

        def one_draw(draw: int, term=term, leaves=leaves):
            masks = build_masks(ctx, term, ci_lower, key, draw, leaves, state, step)
            if ctx.remat_recon_forwards and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint

                # masks are counter-based (same draw on the second run); the closure's tensors are tracked by
                # the checkpoint's saved-tensor hooks, so nothing of the forward stays alive until backward
                aux_metrics: dict[str, Tensor] = {}
                pair = checkpoint(lambda m=masks, am=aux_metrics: masked_recon(
                    ctx, weights, batch, clean, m, term, step, with_aux=True, metrics=am), use_reentrant=False)
                metrics.update({k: v.detach() for k, v in aux_metrics.items()})
                return pair
            return masked_recon(ctx, weights, batch, clean, masks, term, step, with_aux=True, metrics=metrics)

        if ctx.lanes is not None and term.n_samples > 1:  # the draws are independent: side by side on the device
            pairs = ctx.lanes.run([lambda d=d: one_draw(d) for d in range(term.n_samples)])
        else:
            pairs = [one_draw(d) for d in range(term.n_samples)]
        for e2e, full in pairs:
            vals_e2e.append(e2e)
            vals_full.append(full)
        e2e_mean = torch.stack(vals_e2e).mean()
        full_mean = torch.stack(vals_full).mean()
        metrics["loss/" + term.name] = e2e_mean.detach()
        add(ctx.sched("term/" + term.name, term.cfg.coeff, step) * full_mean)
        if term.is_persistent:
            tgt = full_mean if term.cfg.adversary_objective == "term" else e2e_mean  # type: ignore[attr-defined]
            source_grad_requests.append((term, all_leaves, tgt))  # type: ignore[arg-type]

    draws_range.__exit__()
    if ctx.nontarget is not None:
        assert nontarget_batch is not None
        add(_nontarget_pass(ctx, state, weights, nontarget_batch, key, step, metrics))

    assert total_loss is not None
    metrics["loss/total"] = total_loss.detach() + (unseen if ctx.expert_shard is not None and obj.faith is not None else 0)

    # source gradients first (they need the graph), then the parameter backward
    final_grads = []
    for term, all_leaves, tgt in source_grad_requests:
        names = list(all_leaves)
        gs = torch.autograd.grad(tgt, [all_leaves[k] for k in names], retain_graph=True, allow_unused=True)
        final_grads.append((term, reduce_source_grads(
            ctx, {k: (g if g is not None else torch.zeros_like(all_leaves[k])) for k, g in zip(names, gs)},
            state.adversaries[term.name].batch_shared)))

    with phase("backward"):
        total_loss.backward()
        if ctx.lanes is not None:
            ctx.lanes.join_all()  # direct weight-gradient kernels on side streams precede the optimizer
    if ctx.expert_shard is not None and sharded:
        assert ctx.expert_shard.by_component, "expert-split component stacks use the replicated-optimizer layout"
        ctx.collectives.reduce_grads_everywhere(state.ci_fn_opt.params)  # component grads: inside the optimizer step
    elif ctx.expert_shard is not None:
        opt = state.components_opt
        split = [p for n, p in zip(opt.names, opt.params) if ctx.expert_shard.is_split(n)]
        whole = [p for n, p in zip(opt.names, opt.params) if not ctx.expert_shard.is_split(n)]
        ctx.collectives.reduce_split_grads(split)
        ctx.collectives.reduce_grads_everywhere(whole + state.ci_fn_opt.params)
    else:
        ctx.collectives.reduce_grads(([] if sharded else state.components_opt.params)
                                     + ([] if ci_sharded else state.ci_fn_opt.params))

    with phase("optimizer"):
        info_c = state.components_opt.step(step)
        info_f = state.ci_fn_opt.step(step)
    metrics["grad_norm/components"] = state.components_opt.last_grad_norm_t.detach()
    metrics["grad_norm/ci_fn"] = state.ci_fn_opt.last_grad_norm_t.detach()
    metrics["schedules/lr_components"] = _lr_metric(ctx, state.components_opt, info_c["lr"])
    metrics["schedules/lr_ci_fn"] = _lr_metric(ctx, state.ci_fn_opt, info_f["lr"])

    if isinstance(ctx.pd, TargetedPDConfig) and ctx.pd.ci_scaled_weight_decay is not None:
        opt = state.components_opt
        if hasattr(opt, "refresh_full_fp32"):  # sharded masters: edit the gathered values, then re-adopt them
            opt.refresh_full_fp32()
        _ci_scaled_weight_decay(ctx, state, ci, info_c["lr"], ctx.pd.ci_scaled_weight_decay)
        if hasattr(opt, "sync_from_parameters"):
            opt.sync_from_parameters()

    final_key = StepKey(ctx.pd.seed ^ 0x51C, step)
    for term, grads in final_grads:
        lr = get_scheduled_value(step, total, term.cfg.optimizer.lr_schedule)  # type: ignore[attr-defined]
        state.adversaries[term.name].ascend(grads, lr, final_key)
        metrics["schedules/lr_src"] = torch.tensor(lr)  # written as `train/schedules/lr/src`

    if ctx.scalars is not None:
        native.set_step_seed(None)
    state.step += 1
    return metrics  # type: ignore[return-value]


def fresh_pgd_sources(ctx: StepContext, term: ReconTerm, weights: ComputeWeights, batch: Any, clean: ForwardResult,
                      ci_lower: dict[str, Tensor], key: StepKey, step: int) -> dict[str, Tensor]:
    """Initialise sources and run `n_steps` sign-gradient ascents on detached weights and CI."""
    cfg = term.cfg
    lead = _lead_of(ci_lower)
    positions = lead[1] if ctx.model.has_position_axis and len(lead) > 1 else None
    device = next(iter(ci_lower.values())).device
    off = ctx.collectives.row_offset(adv_mod.fresh_source_rows(cfg.source_shape, lead[0], positions))  # type: ignore[attr-defined]
    leaves = adv_mod.fresh_sources(getattr(ctx.model, "global_sites", ctx.model.sites), cfg.init, cfg.source_shape, lead[0], positions, key,  # type: ignore[attr-defined]
                                   term.index, device, row_offset=off)
    w_d, ci_d = _detach_weights(weights), _detach_ci(ci_lower)
    for _ in range(cfg.n_steps):  # type: ignore[attr-defined]
        masks = build_masks(ctx, term, ci_d, key, 0, leaves, None, step)
        e2e, _ = masked_recon(ctx, w_d, batch, clean, masks, term, step, with_aux=False)
        names = list(leaves)
        gs = torch.autograd.grad(e2e, [leaves[k] for k in names], allow_unused=True)
        adv_mod.sign_ascent_(leaves, reduce_source_grads(
            ctx, {k: (g if g is not None else torch.zeros_like(leaves[k])) for k, g in zip(names, gs)},
            cfg.source_shape == "c"), cfg.step_size)  # type: ignore[attr-defined]
    return {k: v.detach() for k, v in leaves.items()}


def _nontarget_pass(ctx: StepContext, state: TrainState, weights: ComputeWeights, batch: Any, key: StepKey,
                    step: int, metrics: dict[str, Tensor]) -> Tensor:
    """The broad-stream half of a targeted (tPD) step: its own clean forward and CI, recon terms with
    the delta pinned on (or the delta-free full sum), its own minimality coefficient, no adversaries."""
    nt = ctx.nontarget
    assert nt is not None
    with torch.no_grad():
        clean = ctx.model.clean_forward(batch)
    ci = run_ci_fn(ctx, state, clean)
    ci_lower = ci.mask_inputs()
    m2: dict[str, Tensor] = {}
    coeff = scheduled_or_constant(nt.impmin_coeff, step, ctx.pd.steps)
    total = evaluate_minimality(ctx, state, ci, step, m2, coeff_override=coeff, update_ema=False)
    for term in nt.recon:
        vals = []
        for draw in range(term.n_samples):
            masks = build_masks(ctx, term, ci_lower, key, draw, None, state, step)
            e2e, _ = masked_recon(ctx, weights, batch, clean, masks, term, step, with_aux=False)
            vals.append(e2e)
        mean = torch.stack(vals).mean()
        m2["loss/" + term.name] = mean.detach()
        total = total + term.coeff(step, ctx.pd.steps) * mean
    metrics.update({"nontarget/" + k: v for k, v in m2.items()})
    state._nontarget_ci_upper = ci.upper  # type: ignore[attr-defined]
    return total


@torch.no_grad()
def _ci_scaled_weight_decay(ctx: StepContext, state: TrainState, ci: CI, lr: float, wd: float) -> None:
    """`V[:, c], U[c, :] *= 1 - lr * wd * (1 - max CI_c)`, max over both streams' batches."""
    other = getattr(state, "_nontarget_ci_upper", None)
    for s in ctx.model.sites:
        def cmax(v):
            if isinstance(v, SelectedCI):
                return v.max_per_component()
            return v.reshape(-1, v.shape[-1]).amax(0)
        m = cmax(ci.upper[s.name]).clamp(0, 1)
        if other is not None:
            m = torch.maximum(m, cmax(other[s.name]).clamp(0, 1))
        scale = 1 - lr * wd * (1 - m)
        V, U = state.components.site(s.name)
        if V.dim() == 2:
            V.mul_(scale[None, :])
            U.mul_(scale[:, None])
        else:
            sc = scale.reshape(V.shape[0], -1)
            V.mul_(sc[:, None, :])
            U.mul_(sc[:, :, None])


def faithfulness_warmup(ctx: StepContext, state: TrainState, steps: int, lr: float, weight_decay: float,
                        log: Callable[[int, float], None] | None = None) -> float:
    """Plain AdamW on the faithfulness loss alone, before step 0."""
    if steps == 0:
        return float("nan")
    params = list(state.components.parameters())
    # A sharded optimizer (and the fused backend's direct weight gradients) keep every `.grad` as a view of
    # their own flat buffer. The warm-up must not replace those views: park them, run on private gradients,
    # and put the (zeroed) views back afterwards.
    parked = [p.grad for p in params]
    for p in params:
        p.grad = None
    opt = torch.optim.AdamW(params, lr=lr, weight_decay=weight_decay, betas=(0.9, 0.999), eps=1e-8)
    last = float("nan")
    try:
        last = _faithfulness_warmup_loop(ctx, state, opt, steps, log)
    finally:
        for p, g in zip(params, parked):
            p.grad = g
            if g is not None:
                g.zero_()
    return last


def _faithfulness_warmup_loop(ctx: StepContext, state: TrainState, opt: torch.optim.Optimizer, steps: int,
                              log: Callable[[int, float], None] | None) -> float:
    last = float("nan")
    for i in range(steps):
        opt.zero_grad(set_to_none=True)
        shard = ctx.expert_shard
        if shard is not None:  # split stacks: per-site terms with this rank's experts / the group-wide product
            loss = loss_fns.faithfulness_terms(state.components, ctx.weights_W, ctx.weights_sq,
                                               component_group=shard.group if shard.by_component else None).mean()
        else:
            loss = loss_fns.faithfulness_loss(state.components, ctx.weights_W, ctx.weights_sq,
                                              relative=ctx.relative_faithfulness)
        loss.backward()
        opt.step()
        if log is not None and (i % 50 == 0 or i == steps - 1):
            last = float(loss.detach())
            log(i, last)
    return last
