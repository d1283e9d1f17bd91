"""Optimizers for the two trainable groups (component stacks, CI function).

AdamW follows optax's `adamw(lr, b1, b2, eps=1e-8, weight_decay)` update with a torch-style
global-norm clip `g * min(max_norm / (norm + 1e-6), 1)` applied per group, and the learning rate
evaluated once per update from the knot schedule (logged as `applied_learning_rate`).
Muon: Nesterov momentum, Newton-Schulz orthogonalisation batched over each stack (every matrix of a
`[g, m, n]` leaf in one batched iteration), `sqrt(max(fan_in, fan_out)) * consistent_rms` scaling,
Adam(0.9, 0.999) for non-matrix leaves.

Parity: param_decomp/core/run_state.py:69-88,133-231; core/muon_stacked.py:74-110 (NS),
:259-396 (update rule); core/configs.py:581-645; torch parity tests
param_decomp/tests/core/test_optim_torch_parity.py.

On CUDA the AdamW update of all leaves of a group is one multi-tensor kernel (`ops/optim.py`).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor

from param_decomp_b200.config.run import AdamWOptimizerConfig, MuonOptimizerConfig
from param_decomp_b200.config.schedule import get_scheduled_value

# optax / Keller-Jordan quintic coefficients
NS_COEFFS = (3.4445, -4.7750, 2.0315)


def global_norm(grads: list[Tensor]) -> Tensor:
    if not grads:
        return torch.zeros(())
    return torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float()) for g in grads]))


def clip_scale(norm: Tensor, max_norm: float | None) -> Tensor:
    if max_norm is None:
        return torch.ones_like(norm)
    return torch.clamp(max_norm / (norm + 1e-6), max=1.0)


def newton_schulz(G: Tensor, steps: int = 5, dtype: torch.dtype = torch.bfloat16, eps: float = 1e-8) -> Tensor:
    """Approximate `U V^T` of each matrix in `G [..., m, n]` (batched over leading axes)."""
    a, b, c = NS_COEFFS
    X = G.to(dtype)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) + eps).to(dtype)
    if _native_ns_ok(X):
        X = _newton_schulz_native(X, steps)
    else:
        for _ in range(steps):
            A = X @ X.transpose(-1, -2)
            B = b * A + c * (A @ A)
            X = a * X + B @ X
    if transposed:
        X = X.transpose(-1, -2)
    return X.to(G.dtype)


def newton_schulz_of_slice(name: str, mix: Tensor, split, steps: int, dtype: torch.dtype) -> tuple[Tensor, int, int]:
    """Orthogonalise the matrix a leaf is a slice of. `split` (`parallel/expert_shard.py::StackSharding` in
    component mode) says that every rank of its group holds a slice of the component axis of `name` (the last axis
    of a `V`, the one before last of a `U`): the slices are gathered, the WHOLE matrix is orthogonalised - the
    orthogonal factor of a slice is not the slice of the orthogonal factor - and this rank's slice of the result
    is returned with the whole matrix's `(fan_in, fan_out)`. Without a split this is plain `newton_schulz`.
    Parity: the reference's Newton-Schulz row names no component axis, i.e. it sees whole matrices
    (param_decomp/core/placement.py:1011-1116, `components/ns_compute`)."""
    if split is None or not getattr(split, "by_component", False) or not split.is_split(name) or split.world == 1:
        return newton_schulz(mix, steps, dtype), mix.shape[-2], mix.shape[-1]
    import torch.distributed as dist

    axis = split._axis(name) % mix.dim()
    parts = [torch.empty_like(mix) for _ in range(split.world)]
    dist.all_gather(parts, mix.contiguous(), group=split.group)
    whole = torch.cat(parts, dim=axis)
    O = newton_schulz(whole, steps, dtype)
    n = mix.shape[axis]
    return O.narrow(axis, split.rank * n, n), whole.shape[-2], whole.shape[-1]


def _native_ns_ok(X: Tensor) -> bool:
    if not (X.is_cuda and X.dtype == torch.bfloat16 and X.dim() in (2, 3)):
        return False
    from param_decomp_b200.ops import native as nv

    return nv.available() and X.shape[-1] % 8 == 0 and X.shape[-2] % 8 == 0


def _newton_schulz_native(X: Tensor, steps: int) -> Tensor:
    """The quintic iteration on the batched tcgen05 GEMM: `A = X X^T` and `A A` are K-major products
    (A is symmetric, so it is its own transposed operand), `B X` reads X as the MN-major operand; the
    polynomial's scalings ride in the epilogue's alpha, the two axpys are single elementwise passes."""
    from param_decomp_b200.ops import native as nv

    a, b, c = NS_COEFFS
    squeeze = X.dim() == 2
    X = (X.unsqueeze(0) if squeeze else X).contiguous()
    g, m, n = X.shape
    A = torch.empty(g, m, m, device=X.device, dtype=torch.bfloat16)
    AA = torch.empty_like(A)
    BX = torch.empty_like(X)
    for _ in range(steps):
        nv.gemm(X, X, A)                        # A = X X^T
        nv.gemm(A, A, AA, alpha=c)              # c A A   (A^T = A)
        Bm = torch.add(AA, A, alpha=b)          # B = b A + c A A
        nv.gemm(Bm, X, BX, b_mn=True)           # B X
        X = torch.add(BX, X, alpha=a)           # a X + B X
    return X[0] if squeeze else X


@dataclass
class GroupOptimizer:
    """One optimizer over a list of named fp32 leaves. State is plain tensors (checkpointable)."""

    cfg: AdamWOptimizerConfig | MuonOptimizerConfig
    names: list[str]
    params: list[Tensor]
    total_steps: int
    matrix_ndim_min: int = 2  # leaves with ndim >= this are "matrices" for Muon
    state: dict[str, Tensor] = field(default_factory=dict)
    count: int = 0
    applied_learning_rate: float = 0.0
    last_grad_norm: float = 0.0
    use_fused: bool = False
    norm_fn: Any = None  # (names, grads) -> global L2 norm, for leaves that are split over a process group
    column_split: Any = None  # `StackSharding` in component mode: Muon orthogonalises the gathered whole matrices
    scalars: Any = None  # ops.step_scalars.StepScalars: learning rate and bias corrections live in device memory
    label: str = "group"

    def lr_at(self, step: int) -> float:
        return get_scheduled_value(min(step, self.total_steps), self.total_steps, self.cfg.lr_schedule)

    def _get(self, key: str, like: Tensor) -> Tensor:
        if key not in self.state:
            self.state[key] = torch.zeros_like(like, dtype=torch.float32)
        return self.state[key]

    @torch.no_grad()
    def step(self, step_idx: int, grads: list[Tensor | None] | None = None) -> dict[str, float]:
        if grads is None:
            grads = [p.grad for p in self.params]
        live = [(n, p, g) for n, p, g in zip(self.names, self.params, grads) if g is not None]
        if self.norm_fn is not None and live:
            norm = self.norm_fn([n for n, _, _ in live], [g for _, _, g in live])
            scale = clip_scale(norm, self.cfg.grad_clip_norm)
        elif self.use_fused and live and live[0][1].is_cuda:
            from param_decomp_b200.ops import optim as fused

            norm, scale = fused.grad_norm_and_scale_multi([p for _, p, _ in live], [g for _, _, g in live],
                                                          self.cfg.grad_clip_norm)
        else:
            norm = global_norm([g for _, _, g in live])
            scale = clip_scale(norm, self.cfg.grad_clip_norm)
        lr = self.lr_at(step_idx)
        self.count += 1
        self._step_idx = step_idx
        self.applied_learning_rate = lr
        self.last_grad_norm_t = norm
        if isinstance(self.cfg, AdamWOptimizerConfig):
            self._adamw(live, scale, lr, self.cfg.betas[0], self.cfg.betas[1], self.cfg.weight_decay)
        else:
            self._muon(live, scale, lr)
        return {"lr": lr}

    def grad_norm(self) -> float:
        return float(self.last_grad_norm_t)

    def advance_replayed(self) -> None:
        """Host bookkeeping of a step whose launches ran from a recording (no Python ran for it)."""
        self.count += 1
        self._step_idx = getattr(self, "_step_idx", -1) + 1
        self.applied_learning_rate = self.lr_at(self._step_idx)

    def _adamw(self, live, scale: Tensor, lr: float, b1: float, b2: float, wd: float) -> None:
        t = self.count
        bc1, bc2 = 1 - b1**t, 1 - b2**t
        if self.use_fused and live and live[0][1].is_cuda:
            from param_decomp_b200.ops import optim as fused

            hyper = None
            if self.scalars is not None:
                off = t - self._step_idx  # updates so far minus steps so far (constant within a run entry)
                hyper = self.scalars.f32_block(f"opt/{self.label}/hyper", 3, lambda s: (
                    self.lr_at(s), 1.0 / (1 - b1 ** (s + off)), 1.0 / (1 - b2 ** (s + off))))
            fused.adamw_step_multi([p for _, p, _ in live], [g for _, _, g in live],
                                   [self._get(n + "/mu", p) for n, p, _ in live],
                                   [self._get(n + "/nu", p) for n, p, _ in live],
                                   lr=lr, b1=b1, b2=b2, eps=1e-8, wd=wd, bc1=bc1, bc2=bc2, grad_scale=scale, hyper=hyper)
            return
        for n, p, g in live:
            g = g.float() * scale.to(g.device)
            mu, nu = self._get(n + "/mu", p), self._get(n + "/nu", p)
            mu.mul_(b1).add_(g, alpha=1 - b1)
            nu.mul_(b2).addcmul_(g, g, value=1 - b2)
            upd = (mu / bc1) / ((nu / bc2).sqrt() + 1e-8)
            if wd:
                upd = upd + wd * p
            p.add_(upd, alpha=-lr)

    def _muon(self, live, scale: Tensor, lr: float) -> None:
        cfg = self.cfg
        assert isinstance(cfg, MuonOptimizerConfig)
        ns_dtype = torch.bfloat16 if cfg.ns_dtype == "bfloat16" else torch.float32
        fallback = []
        for n, p, g in live:
            if p.dim() < self.matrix_ndim_min or min(p.shape[-2:]) == 1:
                fallback.append((n, p, g))
                continue
            g = g.float() * scale.to(g.device)
            # optax `scale_by_muon(nesterov=True)`: an EMA momentum and a bias-corrected Nesterov mix of it
            # with the current gradient (param_decomp/core/muon_stacked.py scale_by_stacked_muon)
            t, b = self.count, cfg.beta
            mom = self._get(n + "/mom", p)
            mom.mul_(b).add_(g, alpha=1 - b)
            nesterov = (b / (1 - b ** (t + 1))) * mom + ((1 - b) / (1 - b**t)) * g
            O, fan_in, fan_out = newton_schulz_of_slice(n, nesterov, self.column_split, cfg.ns_steps, ns_dtype)
            if cfg.consistent_rms is not None:
                s = math.sqrt(max(fan_in, fan_out)) * cfg.consistent_rms
            else:
                s = math.sqrt(max(1.0, fan_out / fan_in))
            if cfg.weight_decay:
                p.mul_(1 - lr * cfg.weight_decay)
            p.add_(O.float(), alpha=-lr * s)
        if fallback:
            self._nadam(fallback, scale, lr, 0.9, 0.999)

    def _nadam(self, live, scale: Tensor, lr: float, b1: float, b2: float) -> None:
        """Muon's rule for leaves that are not matrices: `optax.adamw(b1=0.9, b2=0.999, eps=1e-8,
        weight_decay=0, nesterov=True)` at the Muon learning rate (param_decomp/core/muon_stacked.py
        `stacked_muon`, the "adam" partition)."""
        t = self.count
        for n, p, g in live:
            g = g.float() * scale.to(g.device)
            mu, nu = self._get(n + "/mu", p), self._get(n + "/nu", p)
            mu.mul_(b1).add_(g, alpha=1 - b1)
            nu.mul_(b2).addcmul_(g, g, value=1 - b2)
            mu_hat = (b1 / (1 - b1 ** (t + 1))) * mu + ((1 - b1) / (1 - b1**t)) * g
            p.add_(mu_hat / ((nu / (1 - b2**t)).sqrt() + 1e-8), alpha=-lr)

    # -- checkpoint ----------------------------------------------------------------------------
    def state_dict(self) -> dict[str, Tensor]:
        out = dict(self.state)
        out["count"] = torch.tensor(self.count, dtype=torch.int64)
        return out

    def load_state_dict(self, sd: dict[str, Tensor]) -> None:
        for k, v in sd.items():
            if k == "count":
                self.count = int(v.item())
            else:
                self.state[k] = v


def build_group_optimizer(cfg, named_params: list[tuple[str, Tensor]], total_steps: int,
                          matrix_ndim_min: int = 2, use_fused: bool = False) -> GroupOptimizer:
    names = [n for n, _ in named_params]
    params = [p for _, p in named_params]
    return GroupOptimizer(cfg=cfg, names=names, params=params, total_steps=total_steps,
                          matrix_ndim_min=matrix_ndim_min, use_fused=use_fused)
