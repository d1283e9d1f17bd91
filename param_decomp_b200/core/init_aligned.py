"""Nonlinearity-aligned initialisation of components.

Each component starts aligned with ONE unit on the nonlinearity-facing side of its matrix (a
neuron of an MLP matrix, or a coordinate inside one attention head block): the aligned side is a
one-hot on that coordinate, the other side is the corresponding row/column of the frozen weight
(normalised), so `V[:, c] U[c, :]` is a rank-one slice of `W`. Units are dealt round-robin so the C
components cover the units evenly.

Parity: param_decomp/targets/transformer.py:2188-2306; targets/qwen36_moe.py:1069-1138.
"""

from __future__ import annotations

import torch

from param_decomp_b200.core.components import ComponentStacks


@torch.no_grad()
def nonlinearity_aligned_init(stacks: ComponentStacks, model, seed: int) -> None:
    g = torch.Generator().manual_seed(seed + 23)
    for s in stacks.sites:
        al = s.alignment
        if al is None or s.blocked:
            continue
        W = model.target_weight(s.name).float().cpu()  # [d_out, d_in]
        V, U = stacks.site(s.name)
        width = s.d_out if al.side == "output" else s.d_in
        units = torch.randperm(width, generator=g).repeat((s.C + width - 1) // width)[: s.C]
        if al.side == "output":  # component c writes only to output coordinate u: U[c] = e_u, V[:, c] ~ W[u, :]
            rows = W[units]  # [C, d_in]
            scale = rows.norm(dim=-1, keepdim=True).clamp_min(1e-12)
            Vn = (rows / scale).T  # unit-norm read directions
            Un = torch.zeros(s.C, s.d_out)
            Un[torch.arange(s.C), units] = scale[:, 0]
        else:  # component c reads only input coordinate u: V[:, c] = e_u, U[c] ~ W[:, u]
            cols = W[:, units].T  # [C, d_out]
            scale = cols.norm(dim=-1, keepdim=True).clamp_min(1e-12)
            Un = cols / scale
            Vn = torch.zeros(s.d_in, s.C)
            Vn[units, torch.arange(s.C)] = scale[:, 0]
        V.copy_(Vn.to(V.device))
        U.copy_(Un.to(U.device))
