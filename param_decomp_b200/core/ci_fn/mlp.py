"""MLP causal-importance functions: per-site (`layerwise_mlp`) and joint (`global_mlp`).

Both are pointwise over all leading axes, so the same module serves positionless toys `[B, d]` and
per-token LM activations `[B, T, d]`.

Parity: param_decomp/core/ci_fn/implementations/mlp.py:57-92 (`SiteMLP`: Linear + exact-erf GELU
... Linear, Kaiming-normal weights, zero biases), layerwise_mlp.py:30-164, global_mlp.py:30-170.

Sites of one group share their shapes, so `LayerwiseMLPCIFn` stores each group's MLPs stacked
(`W1 [g, d_in, h]`, ...) and evaluates the whole group as one batched GEMM chain; on the fused
backend that chain is one launch of the batched tcgen05 kernel per layer.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from param_decomp_b200.core.ci_fn.interface import census


def _kaiming_(w: Tensor, fan_in: int, generator: torch.Generator | None) -> None:
    std = math.sqrt(2.0 / fan_in)
    with torch.no_grad():
        w.copy_(torch.randn(w.shape, generator=generator, dtype=torch.float32).to(w.device) * std)


class SiteMLP(nn.Module):
    """`d_in -> hidden... -> d_out` for `n_stack` independent copies evaluated together."""

    def __init__(self, n_stack: int, d_in: int, hidden_dims: tuple[int, ...], d_out: int,
                 generator: torch.Generator | None = None) -> None:
        super().__init__()
        dims = (d_in, *hidden_dims, d_out)
        self.dims = dims
        self.n_stack = n_stack
        self.fused = False  # set by the builder on the fused sm_100a backend
        self.weights = nn.ParameterList()
        self.biases = nn.ParameterList()
        for a, b in zip(dims[:-1], dims[1:]):
            w = nn.Parameter(torch.empty(n_stack, a, b))
            _kaiming_(w, a, generator)
            self.weights.append(w)
            self.biases.append(nn.Parameter(torch.zeros(n_stack, 1, b)))

    def forward(self, x: Tensor) -> Tensor:
        """`x [n_stack, N, d_in] -> [n_stack, N, d_out]`."""
        h = x
        last = len(self.weights) - 1
        fused = self.fused and x.is_cuda and all(d % 8 == 0 for d in self.dims)
        if fused:
            from param_decomp_b200.ops.linear import bmm_bias

            h = h.to(torch.bfloat16)
        for i, (w, b) in enumerate(zip(self.weights, self.biases)):
            h = bmm_bias(h, w, b) if fused else torch.baddbmm(b.to(h.dtype), h, w.to(h.dtype))
            if i != last:
                h = F.gelu(h)  # exact erf form
        return h

    def flops_per_row(self) -> int:
        return sum(2 * a * b for a, b in zip(self.dims[:-1], self.dims[1:])) * self.n_stack


class BlockedSiteMLP(nn.Module):
    """CI for an expert-blocked site, emitted only for each token's selected experts:
    `hidden = gelu(x W1 + b1)` shared by all experts, then one head per expert
    `[E, hidden, C_block]` applied to the tokens routed to it -> `SelectedCI [.., k * C_block]`."""

    def __init__(self, d_in: int, hidden: int, n_blocks: int, c_block: int, generator: torch.Generator | None) -> None:
        super().__init__()
        self.n_blocks, self.c_block = n_blocks, c_block
        self.w1 = nn.Parameter(torch.empty(d_in, hidden))
        _kaiming_(self.w1, d_in, generator)
        self.b1 = nn.Parameter(torch.zeros(hidden))
        self.heads = nn.Parameter(torch.empty(n_blocks, hidden, c_block))
        _kaiming_(self.heads, hidden, generator)
        self.head_bias = nn.Parameter(torch.zeros(n_blocks, c_block))

    fused = False  # set by the builder on the fused sm_100a backend

    def forward(self, x: Tensor, sel) -> "SelectedCI":
        from param_decomp_b200.core.components import SelectedCI

        lead = x.shape[:-1]
        idx = sel.indices.reshape(-1, sel.indices.shape[-1])  # [N, k]
        N, k = idx.shape
        flat_e = idx.reshape(-1)
        x2 = x.reshape(-1, x.shape[-1])
        hidden = self.w1.shape[1]
        if (self.fused and x.is_cuda and x2.shape[1] % 8 == 0 and hidden % 64 == 0 and self.c_block % 8 == 0):
            # one batched GEMM for the shared trunk, then the per-expert heads as a grouped GEMM over
            # (token, slot) jobs sorted by expert: no Python loop over experts, no host sync
            from param_decomp_b200.ops.grouped import JobLayout, grouped_linear_trainable
            from param_decomp_b200.ops.linear import bmm_bias

            h = F.gelu(bmm_bias(x2.to(torch.bfloat16).unsqueeze(0), self.w1.unsqueeze(0), self.b1.view(1, 1, -1))[0])
            layout = JobLayout.cached(sel.indices, self.n_blocks)
            hj = layout.expand_tokens(h, k)
            out = layout.gather_rows(grouped_linear_trainable(hj, self.heads, self.head_bias, layout))
            return SelectedCI(out.reshape(*lead, k * self.c_block), sel, self.n_blocks)
        h = F.gelu(x2.float() @ self.w1 + self.b1)  # [N, hidden]
        order = flat_e.argsort(stable=True)
        counts = torch.bincount(flat_e, minlength=self.n_blocks).tolist()
        pieces, start = [], 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            jobs = order[start:start + n]
            pieces.append(h[jobs // k] @ self.heads[e] + self.head_bias[e])
            start += n
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        out = torch.cat(pieces)[inv]  # back to job order without in-place slice writes
        return SelectedCI(out.reshape(*lead, k * self.c_block), sel, self.n_blocks)


class LayerwiseMLPCIFn(nn.Module):
    """One MLP per site, reading that site's own tap. `site_taps[site] = tap key`.
    `blocked[site] = (layer, n_blocks, C_block)` marks expert-blocked sites (narrow emission)."""

    def __init__(self, site_shapes: dict[str, tuple[int, int]], site_taps: dict[str, str],
                 hidden_dims: tuple[int, ...], generator: torch.Generator | None = None,
                 blocked: dict[str, tuple[int, int, int]] | None = None) -> None:
        super().__init__()
        self.site_taps = dict(site_taps)
        self.input_taps = tuple(dict.fromkeys(site_taps.values()))
        self.blocked = dict(blocked or {})
        self.blocked_mlps = nn.ModuleDict({
            s.replace(".", "_"): BlockedSiteMLP(site_shapes[s][0], hidden_dims[0], nb, cb, generator)
            for s, (_, nb, cb) in self.blocked.items()})
        site_shapes = {s: v for s, v in site_shapes.items() if s not in self.blocked}
        # group sites by (d_in, C) so each group is one stacked MLP
        self.group_members: dict[str, list[str]] = {}
        for site, (d_in, C) in site_shapes.items():
            self.group_members.setdefault(f"{d_in}_{C}", []).append(site)
        self.mlps = nn.ModuleDict()
        for key, members in self.group_members.items():
            d_in, C = site_shapes[members[0]]
            self.mlps[key] = SiteMLP(len(members), d_in, tuple(hidden_dims), C, generator)

    def forward(self, taps: dict[str, Tensor], **context: Any) -> dict[str, Tensor]:
        out: dict[str, Tensor] = {}
        for key, members in self.group_members.items():
            xs = [taps[self.site_taps[s]] for s in members]
            lead = xs[0].shape[:-1]
            x = torch.stack([t.reshape(-1, t.shape[-1]) for t in xs])
            mlp = self.mlps[key]
            y = mlp(x if mlp.fused else x.float())
            for s, yi in zip(members, y.unbind(0)):  # one stacked gradient per group in backward
                out[s] = yi.reshape(*lead, -1)
        if self.blocked:
            routing = (context.get("aux") or {}).get("routing", {})
            for s, (layer, _, _) in self.blocked.items():
                out[s] = self.blocked_mlps[s.replace(".", "_")](taps[self.site_taps[s]], routing[layer])
        return out

    def parameter_census(self) -> dict[str, int]:
        return census(self)

    def useful_flops_per_position(self) -> int:
        return sum(m.flops_per_row() for m in self.mlps.values())  # type: ignore[union-attr]


class GlobalMLPCIFn(nn.Module):
    """One MLP over the concatenation of all taps; its output splits into per-site CI."""

    def __init__(self, taps: tuple[tuple[str, int], ...], site_cs: dict[str, int],
                 hidden_dims: tuple[int, ...], generator: torch.Generator | None = None) -> None:
        super().__init__()
        self.input_taps = tuple(k for k, _ in taps)
        self.site_cs = dict(site_cs)
        d_in = sum(w for _, w in taps)
        self.mlp = SiteMLP(1, d_in, tuple(hidden_dims), sum(site_cs.values()), generator)

    def forward(self, taps: dict[str, Tensor], **context: Any) -> dict[str, Tensor]:
        xs = [taps[k] for k in self.input_taps]
        lead = xs[0].shape[:-1]
        x = torch.cat([t.reshape(-1, t.shape[-1]) for t in xs], dim=-1)
        y = self.mlp((x if self.mlp.fused else x.float())[None])[0]
        parts = torch.split(y, list(self.site_cs.values()), dim=-1)
        return {s: p.reshape(*lead, -1) for s, p in zip(self.site_cs, parts)}

    def parameter_census(self) -> dict[str, int]:
        return census(self)

    def useful_flops_per_position(self) -> int:
        return self.mlp.flops_per_row()
