"""A single-file, plain-PyTorch statement of the decomposition method, for readers.

Nothing here imports the rest of the package; nothing in the package imports this file. It wraps
every `nn.Linear` of a target you name in a `ComponentLinear`, learns rank-one components
`W ~ sum_c U[:, c] V[c, :]` and a causal-importance (CI) network, and trains them with

  * faithfulness        sum ||W - U V||^2 / n_params
  * stochastic recon    KL(target logits || logits with masks m = ci + (1 - ci) u, u ~ U(0,1))
  * adversarial recon   the same with persistent sources ascended by sign steps (persistent PGD)
  * minimality          sum_c |ci_upper + eps|^p  (+ a frequency term), p annealed towards sparsity

It runs on CPU or one GPU, slowly; the optimised engine lives in `core/` and `ops/`. The role in the
reference: nano_param_decomp/run.py (a readable oracle of the algorithm, not of any file layout).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Iterator

import torch
import torch.nn.functional as F
from torch import Tensor, nn


# ---------------------------------------------------------------------------------------------------
# configuration
# ---------------------------------------------------------------------------------------------------
@dataclass
class NanoConfig:
    n_components: int = 64
    ci_hidden: int = 64
    steps: int = 200
    lr: float = 1e-3
    warmup_frac: float = 0.05
    faithfulness_warmup_steps: int = 20
    coeff_faithfulness: float = 1e3
    coeff_stochastic: float = 1.0
    coeff_pgd: float = 0.5
    coeff_minimality: float = 1e-3
    p_start: float = 2.0
    p_end: float = 0.5
    eps: float = 1e-12
    beta: float = 0.5           # weight of the frequency term inside the minimality loss
    pgd_step: float = 0.05
    leaky_alpha: float = 0.01
    grad_clip: float = 1.0
    seed: int = 0
    log_every: int = 50
    history: list = field(default_factory=list)


# ---------------------------------------------------------------------------------------------------
# leaky-hard sigmoids
# ---------------------------------------------------------------------------------------------------
class _LowerLeaky(torch.autograd.Function):
    """clamp(x, 0, 1) forward. Backward: identity inside (0, 1]; zero above 1; below 0 a small leak,
    and only for gradients that would push x UP (so dead components can come back, live ones cannot
    be dragged further below zero)."""

    @staticmethod
    def forward(ctx, x: Tensor, alpha: float) -> Tensor:  # type: ignore[override]
        ctx.save_for_backward(x)
        ctx.alpha = alpha
        return x.clamp(0, 1)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        (x,) = ctx.saved_tensors
        inside = (x > 0) & (x <= 1)
        leak = (x <= 0) & (g < 0)
        return g * inside + ctx.alpha * g * leak, None


def lower_leaky(x: Tensor, alpha: float) -> Tensor:
    return _LowerLeaky.apply(x, alpha)


def upper_leaky(x: Tensor, alpha: float) -> Tensor:
    return torch.where(x > 1, 1 + alpha * (x - 1), x.clamp(0, 1))


# ---------------------------------------------------------------------------------------------------
# the decomposed layer
# ---------------------------------------------------------------------------------------------------
class ComponentLinear(nn.Module):
    """Stands in for one frozen `nn.Linear`. With `mask [.., C]` (and `delta_mask [.., 1]`) set it
    computes `((x V) * mask) U + delta_mask * x (W - V U)^T + b`; with no mask it is the target layer."""

    def __init__(self, target: nn.Linear, n_components: int, gen: torch.Generator) -> None:
        super().__init__()
        self.weight = nn.Parameter(target.weight.detach().clone(), requires_grad=False)  # [out, in]
        self.bias = None if target.bias is None else nn.Parameter(target.bias.detach().clone(), requires_grad=False)
        d_out, d_in = self.weight.shape
        self.V = nn.Parameter(torch.randn(d_in, n_components, generator=gen) / math.sqrt(d_in))
        self.U = nn.Parameter(torch.randn(n_components, d_out, generator=gen) / math.sqrt(n_components))
        self.mask: Tensor | None = None
        self.delta_mask: Tensor | None = None
        self.last_input: Tensor | None = None

    def delta(self) -> Tensor:
        return self.weight - (self.V @ self.U).T

    def forward(self, x: Tensor) -> Tensor:
        self.last_input = x
        if self.mask is None:
            return F.linear(x, self.weight, self.bias)
        y = ((x @ self.V) * self.mask) @ self.U
        if self.delta_mask is not None:
            y = y + self.delta_mask * F.linear(x, self.delta())
        return y if self.bias is None else y + self.bias


def wrap_linears(model: nn.Module, names: list[str], n_components: int, seed: int) -> dict[str, ComponentLinear]:
    gen = torch.Generator().manual_seed(seed)
    out: dict[str, ComponentLinear] = {}
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        lin = getattr(parent, leaf)
        assert isinstance(lin, nn.Linear), f"{name} is not an nn.Linear"
        comp = ComponentLinear(lin, n_components, gen).to(lin.weight.device)
        setattr(parent, leaf, comp)
        out[name] = comp
    return out


class CINet(nn.Module):
    """One small MLP per decomposed layer, reading that layer's clean input: pre-activations `[.., C]`."""

    def __init__(self, comps: dict[str, ComponentLinear], hidden: int, n_components: int) -> None:
        super().__init__()
        self.nets = nn.ModuleDict({
            k.replace(".", "_"): nn.Sequential(nn.Linear(c.weight.shape[1], hidden), nn.GELU(), nn.Linear(hidden, n_components))
            for k, c in comps.items()})

    def forward(self, inputs: dict[str, Tensor]) -> dict[str, Tensor]:
        return {k: self.nets[k.replace(".", "_")](x) for k, x in inputs.items()}


# ---------------------------------------------------------------------------------------------------
# losses
# ---------------------------------------------------------------------------------------------------
def kl_from_logits(target: Tensor, pred: Tensor) -> Tensor:
    lt, lp = F.log_softmax(target.float(), -1), F.log_softmax(pred.float(), -1)
    return (lt.exp() * (lt - lp)).sum(-1).mean()


def minimality(ci_upper: dict[str, Tensor], p: float, eps: float, beta: float) -> Tensor:
    total = ci_upper[next(iter(ci_upper))].new_zeros(())
    for v in ci_upper.values():
        per_pos = (v + eps).pow(p)                      # [.., C]
        flat = per_pos.reshape(-1, per_pos.shape[-1])
        freq = flat.mean(0)                             # how often / how strongly each component fires
        total = total + flat.sum(-1).mean() + beta * (freq * torch.log2(1 + freq * flat.shape[0])).sum()
    return total


def set_masks(comps: dict[str, ComponentLinear], masks: dict[str, Tensor] | None, deltas: dict[str, Tensor] | None) -> None:
    for k, c in comps.items():
        c.mask = None if masks is None else masks[k]
        c.delta_mask = None if deltas is None else deltas[k]


def lr_at(cfg: NanoConfig, step: int) -> float:
    warm = max(1, int(cfg.warmup_frac * cfg.steps))
    if step < warm:
        return cfg.lr * (step + 1) / warm
    t = (step - warm) / max(1, cfg.steps - warm)
    return cfg.lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * t)))


# ---------------------------------------------------------------------------------------------------
# training
# ---------------------------------------------------------------------------------------------------
def decompose(model: nn.Module, layer_names: list[str], batches: Iterator[Tensor], cfg: NanoConfig,
              forward: Callable[[nn.Module, Tensor], Tensor] | None = None) -> tuple[dict[str, ComponentLinear], CINet]:
    """`batches` yields token tensors `[B, S]`; `forward(model, tokens)` returns logits (default: call)."""
    forward = forward or (lambda m, t: m(t))
    torch.manual_seed(cfg.seed)
    for p in model.parameters():
        p.requires_grad_(False)
    comps = wrap_linears(model, layer_names, cfg.n_components, cfg.seed)
    ci_net = CINet(comps, cfg.ci_hidden, cfg.n_components).to(next(model.parameters()).device)
    params = [p for c in comps.values() for p in (c.V, c.U)] + list(ci_net.parameters())
    opt = torch.optim.AdamW(params, lr=cfg.lr, weight_decay=0.0)
    n_weights = sum(c.weight.numel() for c in comps.values())

    def faithfulness() -> Tensor:
        return sum(c.delta().pow(2).sum() for c in comps.values()) / n_weights

    # faithfulness warm-up: fit U V to W before anything else moves
    warm = torch.optim.AdamW([p for c in comps.values() for p in (c.V, c.U)], lr=cfg.lr)
    for _ in range(cfg.faithfulness_warmup_steps):
        warm.zero_grad()
        faithfulness().backward()
        warm.step()

    sources: dict[str, Tensor] = {}  # persistent adversarial sources, one [1, 1, C] row per layer
    for step in range(cfg.steps):
        tokens = next(batches)
        for g in opt.param_groups:
            g["lr"] = lr_at(cfg, step)
        p_now = cfg.p_start + (cfg.p_end - cfg.p_start) * step / max(1, cfg.steps - 1)

        set_masks(comps, None, None)
        with torch.no_grad():
            target_logits = forward(model, tokens)
        inputs = {k: c.last_input.detach() for k, c in comps.items()}  # type: ignore[union-attr]
        pre = ci_net(inputs)
        lower = {k: lower_leaky(v, cfg.leaky_alpha) for k, v in pre.items()}
        upper = {k: upper_leaky(v, cfg.leaky_alpha) for k, v in pre.items()}

        # stochastic reconstruction: every component kept at least as much as its importance says
        masks = {k: v + (1 - v) * torch.rand_like(v) for k, v in lower.items()}
        deltas = {k: torch.rand_like(v[..., :1]) for k, v in lower.items()}
        set_masks(comps, masks, deltas)
        loss_stoch = kl_from_logits(target_logits, forward(model, tokens))

        # persistent PGD: sources ascend the reconstruction loss across steps, the model descends it
        if not sources:
            sources = {k: torch.rand(1, 1, v.shape[-1], device=v.device, requires_grad=True) for k, v in lower.items()}
        adv_masks = {k: v + (1 - v) * sources[k] for k, v in lower.items()}
        set_masks(comps, adv_masks, {k: torch.ones_like(v[..., :1]) for k, v in lower.items()})
        loss_pgd = kl_from_logits(target_logits, forward(model, tokens))
        src_grads = torch.autograd.grad(loss_pgd, list(sources.values()), retain_graph=True)

        loss_min = minimality(upper, p_now, cfg.eps, cfg.beta)
        loss_faith = faithfulness()
        loss = (cfg.coeff_faithfulness * loss_faith + cfg.coeff_stochastic * loss_stoch + cfg.coeff_pgd * loss_pgd
                + cfg.coeff_minimality * loss_min)
        opt.zero_grad()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, cfg.grad_clip)
        opt.step()
        with torch.no_grad():  # the adversary moves after the model's gradients have been taken
            for s, g in zip(sources.values(), src_grads):
                s.add_(cfg.pgd_step * g.sign()).clamp_(0, 1)
        if step % cfg.log_every == 0 or step == cfg.steps - 1:
            l0 = sum(float((v > 0).float().sum(-1).mean()) for v in lower.values()) / len(lower)
            cfg.history.append({"step": step, "loss": float(loss), "faith": float(loss_faith), "stoch": float(loss_stoch),
                                "pgd": float(loss_pgd), "min": float(loss_min), "l0": l0, "p": p_now})
    set_masks(comps, None, None)
    return comps, ci_net


@torch.no_grad()
def evaluate(model: nn.Module, comps: dict[str, ComponentLinear], ci_net: CINet, tokens: Tensor,
             forward: Callable[[nn.Module, Tensor], Tensor] | None = None, alpha: float = 0.01) -> dict[str, float]:
    """KL and next-token CE under the usual mask variants: CI-masked, rounded, stochastic, unmasked, zero."""
    forward = forward or (lambda m, t: m(t))
    set_masks(comps, None, None)
    target = forward(model, tokens)
    inputs = {k: c.last_input for k, c in comps.items()}
    lower = {k: v.clamp(0, 1) for k, v in ci_net(inputs).items()}
    ones = {k: torch.ones_like(v[..., :1]) for k, v in lower.items()}
    variants = {
        "ci_masked": lower, "rounded_masked": {k: (v > 0).float() for k, v in lower.items()},
        "stoch_masked": {k: v + (1 - v) * torch.rand_like(v) for k, v in lower.items()},
        "unmasked": {k: torch.ones_like(v) for k, v in lower.items()}, "zero_masked": {k: torch.zeros_like(v) for k, v in lower.items()},
    }
    out: dict[str, float] = {}
    for name, m in variants.items():
        set_masks(comps, m, ones if name != "zero_masked" else {k: torch.zeros_like(v) for k, v in ones.items()})
        logits = forward(model, tokens)
        out[f"kl/{name}"] = float(kl_from_logits(target, logits))
        out[f"ce/{name}"] = float(F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1)))
    set_masks(comps, None, None)
    out["l0"] = sum(float((v > 0).float().sum(-1).mean()) for v in lower.values()) / len(lower)
    return out
