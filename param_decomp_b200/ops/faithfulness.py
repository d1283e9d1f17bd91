"""Faithfulness loss and its gradients on the tcgen05 engine, never materialising fp32 `V U`.

Per site:  D = W - (V U)^T  comes out of ONE GEMM whose epilogue subtracts the accumulator from `W`
and reduces `sum D^2` on the fly; the product uses split-precision operands
(`V = V_hi + V_lo`, `U = U_hi + U_lo` in bf16, three K-phases `U_hi V_hi + U_lo V_hi + U_hi V_lo`
laid side by side along K), which restores ~16 mantissa bits so the loss keeps falling below the
bf16 rounding floor. Gradients `dV = -2s (U D)^T`, `dU = -2s V^T D^T` are two more GEMMs that
accumulate straight into the fp32 master gradients (`s = coeff / (n_sites ||W||^2)`).

Parity: param_decomp/core/faithfulness.py:16-104 (target-relative mean over sites, pads contribute
nothing), targets/transformer.py:2134-2185 (weight deltas).
"""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.core.components import ComponentStacks
from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.elementwise import split3_bf16, split_bf16


_WSQ: dict[tuple, Tensor] = {}


def _wsq_tensor(sites, w_sq_host: dict[str, float], dev) -> Tensor:
    """`||W_s||^2` per site on the device, uploaded once (the target is frozen)."""
    key = (str(dev), tuple((s.name, w_sq_host[s.name]) for s in sites))
    t = _WSQ.get(key)
    if t is None:
        if len(_WSQ) > 16:
            _WSQ.clear()
        t = _WSQ[key] = torch.tensor([w_sq_host[s.name] for s in sites], device=dev, dtype=torch.float32)
    return t


def fused_faithfulness(stacks: ComponentStacks, W: dict[str, Tensor], w_sq_host: dict[str, float], coeff,
                       accumulate_grads: bool = True, hi_lo: dict[str, tuple[Tensor, Tensor]] | None = None,
                       rank: int = 0, world: int = 1) -> Tensor:
    """Returns the (detached) loss `mean_s ||D_s||^2 / ||W_s||^2`; adds `coeff * dLoss` to `.grad`.
    `coeff` is a float, or a 0-d fp32 device tensor (a scheduled coefficient kept in device memory), which
    the gradient GEMMs then read at run time.

    `hi_lo["V/<group>"] = (hi, lo)`: split-precision working copies published by the sharded
    optimizer (then no fp32 master is read). With `world > 1` the sites are dealt round-robin to the
    ranks: each rank does the GEMMs of its own sites only, writes their gradients scaled by `world`
    (the gradient reduction averages over ranks), and returns its partial loss; the caller sums it."""
    sites = list(stacks.sites)
    dev = next(stacks.parameters()).device
    coeff_dev = coeff if isinstance(coeff, Tensor) else None
    coeff = 1.0 if coeff_dev is not None else coeff
    sumsq = torch.zeros(len(sites), 8, device=dev, dtype=torch.float32)
    n_sites = len(sites)
    row_of = {s.name: i for i, s in enumerate(sites)}  # sumsq rows follow `sites`, not the group walk
    k = 0
    for gname, members in stacks.groups.items():
        key = stacks.param_key(gname)
        pV, pU = stacks.V[key], stacks.U[key]
        V3 = U3 = None
        if hi_lo is not None:
            (Vh, Vl), (Uh, Ul) = hi_lo["V/" + key], hi_lo["U/" + key]
        elif pV.dim() == 3 and pV.shape[-1] % 8 == 0 and pU.shape[-1] % 8 == 0:
            # dense stacks: one pass writes the three K-phases side by side; hi parts are views of them
            C_ = pV.shape[-1]
            V3, U3 = split3_bf16(pV.detach(), along_cols=True), split3_bf16(pU.detach(), along_cols=False)
            Vh, Vl, Uh, Ul = V3[..., :C_], V3[..., 2 * C_:], U3[:, :C_], U3[:, C_:2 * C_]
        else:
            Vh, Vl = split_bf16(pV.detach())
            Uh, Ul = split_bf16(pU.detach())
        if accumulate_grads:
            if pV.grad is None:
                pV.grad = torch.zeros_like(pV)
            if pU.grad is None:
                pU.grad = torch.zeros_like(pU)
        for i, s in enumerate(members):
            if k % world != rank:
                k += 1
                continue
            Wb = W[s.name]
            assert Wb.dtype == torch.bfloat16, "the fused faithfulness path expects a bf16 target"
            if s.blocked:
                _blocked_site(s, Vh[i], Vl[i], Uh[i], Ul[i], Wb, sumsq[row_of[s.name]:row_of[s.name] + 1],
                              pV.grad[i] if accumulate_grads else None, pU.grad[i] if accumulate_grads else None,
                              -2.0 * coeff * world / (n_sites * w_sq_host[s.name]), coeff_dev)
                k += 1
                continue
            if V3 is not None:
                U_cat, V_cat = U3[i], V3[i]
            else:
                U_cat = torch.cat([Uh[i], Ul[i], Uh[i]], dim=0)  # [3C, d_out]
                V_cat = torch.cat([Vh[i], Vh[i], Vl[i]], dim=1)  # [d_in, 3C]
            D = torch.empty(s.d_out, s.d_in, device=dev, dtype=torch.bfloat16)
            r = row_of[s.name]
            nv.gemm(U_cat, V_cat, D, a_mn=True, epi=nv.EPI_FAITH, ci=Wb, dci=sumsq[r:r + 1])
            if accumulate_grads:
                alpha = -2.0 * coeff * world / (n_sites * w_sq_host[s.name])
                nv.gemm(D, Uh[i], pV.grad[i], a_mn=True, accumulate=True, alpha=alpha, alpha_dev=coeff_dev)
                nv.gemm(Vh[i], D, pU.grad[i], a_mn=True, accumulate=True, alpha=alpha, alpha_dev=coeff_dev)
            k += 1
    return (sumsq[:, 0] / _wsq_tensor(sites, w_sq_host, dev)).sum() / n_sites


def blocked_supported(stacks: ComponentStacks) -> bool:
    """Blocked sites run as one grouped product over the `[E * d_out, d_in]` view of the expert bank:
    a 128-row tile must not straddle two experts."""
    return all(not s.blocked or (s.d_out % 128 == 0 and s.d_in % 8 == 0 and s.C_block % 8 == 0) for s in stacks.sites)


def _blocked_site(s, Vh: Tensor, Vl: Tensor, Uh: Tensor, Ul: Tensor, Wb: Tensor, sumsq: Tensor, gV: Tensor | None,
                  gU: Tensor | None, alpha: float, alpha_dev: Tensor | None = None) -> None:
    """`V [E, d_in, c]`, `U [E, c, d_out]`, `W [E, d_out, d_in]`: the residual of all experts in one
    launch (each 128-row tile of the stacked rows picks its expert's `V`), then two batched products
    for the gradients."""
    E, d_out, d_in = Wb.shape
    A = torch.cat([Uh, Ul, Uh], dim=1).transpose(1, 2).reshape(E * d_out, -1)  # rows (e, o), K = 3c
    V_cat = torch.cat([Vh, Vh, Vl], dim=2)  # [E, d_in, 3c]
    D = torch.empty(E, d_out, d_in, device=Wb.device, dtype=torch.bfloat16)
    owner = torch.arange(E, device=Wb.device, dtype=torch.int32).repeat_interleave(d_out // 128)
    nv.gemm(A, V_cat, D.view(E * d_out, d_in), epi=nv.EPI_FAITH, ci=Wb.reshape(E * d_out, d_in), dci=sumsq,
            bgroup_of_mblock=owner)
    if gV is not None:
        nv.gemm(D, Uh, gV, a_mn=True, accumulate=True, alpha=alpha, alpha_dev=alpha_dev)  # dV[e] = alpha D_e^T U_e^T
        nv.gemm(Vh, D, gU, a_mn=True, accumulate=True, alpha=alpha, alpha_dev=alpha_dev)  # dU[e] = alpha V_e^T D_e^T
