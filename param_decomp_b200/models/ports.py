"""Model math shared by the LM targets and the CI transformers.

Each op has an eager torch definition (the oracle, runs anywhere) and, on CUDA with the native
library loaded, dispatches to the hand-written sm_100a kernel in `ops/`.

Parity: param_decomp/target_ports/llama.py:34-129 (`rms_norm`, `rope_cos_sin`, `rotate_half`,
`apply_rope`, `repeat_kv`, llama3 rope scaling); param_decomp/attention.py:248-279 (materialised
causal / document-segmented attention oracle); target_ports/qwen3_5_moe.py:33-74 (zero-centred
RMSNorm `(1 + w)`, gated RMSNorm `norm(x) * silu(z)`, causal depthwise conv1d + SiLU, partial RoPE).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor


def rms_norm(x: Tensor, weight: Tensor | None, eps: float, zero_centered: bool = False) -> Tensor:
    """fp32 statistics, output in `x.dtype`. `zero_centered` scales by `1 + w` (Qwen3.5)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1 + w if zero_centered else w)
    return y.to(x.dtype)


def gated_rms_norm(x: Tensor, z: Tensor, weight: Tensor, eps: float) -> Tensor:
    return (rms_norm(x, weight, eps).float() * F.silu(z.float())).to(x.dtype)


def llama3_scale_inv_freq(inv_freq: Tensor, factor: float = 8.0, low: float = 1.0, high: float = 4.0,
                          original_len: int = 8192) -> Tensor:
    """Llama-3.1 long-context rescaling of the RoPE frequencies."""
    wavelen = 2 * math.pi / inv_freq
    low_wl, high_wl = original_len / low, original_len / high
    smooth = ((original_len / wavelen) - low) / (high - low)
    scaled = torch.where(wavelen > low_wl, inv_freq / factor, inv_freq)
    mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    return torch.where((wavelen <= low_wl) & (wavelen >= high_wl), mid, scaled)


def rope_cos_sin(positions: Tensor, rotary_dim: int, theta: float, scaling=None) -> tuple[Tensor, Tensor]:
    """`positions [..., T]` -> `cos, sin [..., T, rotary_dim]` (halves duplicated, rotate-half form). `scaling`:
    an object with the Llama-3.1 fields `factor`, `low_freq_factor`, `high_freq_factor`,
    `original_max_position_embeddings`, or None."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, device=positions.device, dtype=torch.float32) / rotary_dim))
    if scaling is not None:
        inv = llama3_scale_inv_freq(inv, scaling.factor, scaling.low_freq_factor, scaling.high_freq_factor,
                                    scaling.original_max_position_embeddings)
    ang = positions.float().unsqueeze(-1) * inv
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def rotate_half(x: Tensor) -> Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """`x [B, T, H, hd]`, `cos/sin [B|1, T, rd]`; rotates the first `rd` channels (partial RoPE)."""
    rd = cos.shape[-1]
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    xr = x[..., :rd].float()
    out = xr * c + rotate_half(xr) * s
    if rd == x.shape[-1]:
        return out.to(x.dtype)
    return torch.cat([out.to(x.dtype), x[..., rd:]], dim=-1)


def repeat_kv(x: Tensor, n_rep: int) -> Tensor:
    """`[B, T, Hkv, hd] -> [B, T, Hkv * n_rep, hd]` (query head h reads kv head h // n_rep)."""
    if n_rep == 1:
        return x
    B, T, H, D = x.shape
    return x[:, :, :, None, :].expand(B, T, H, n_rep, D).reshape(B, T, H * n_rep, D)


def attention_mask(T: int, causal: bool, segment_ids: Tensor | None, device) -> Tensor | None:
    """Boolean `[B|1, 1, T, T]` mask (True = attend) or None when everything attends."""
    m = None
    if causal:
        m = torch.ones(T, T, dtype=torch.bool, device=device).tril()[None, None]
    if segment_ids is not None:
        same = (segment_ids[:, :, None] == segment_ids[:, None, :])[:, None]
        m = same if m is None else (m & same)
    return m


def attention_scores(q: Tensor, k: Tensor, scale: float | None = None) -> Tensor:
    """Pre-softmax logits `[B, H, T, T]` (fp32) from `[B, T, H, hd]` operands, GQA-expanded."""
    n_rep = q.shape[2] // k.shape[2]
    kk = repeat_kv(k, n_rep)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return torch.einsum("bthd,bshd->bhts", q.float(), kk.float()) * scale


def sdpa_reference(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, segment_ids: Tensor | None = None,
                   softcap: float | None = None, sink: Tensor | None = None) -> Tensor:
    """Materialised attention (the oracle). `q [B,T,H,hd]`, `k/v [B,T,Hkv,hd]` -> `[B,T,H,hd]`.
    `sink [H]`: one learned logit per head joins the softmax as a slot whose value is zero."""
    s = attention_scores(q, k)
    if softcap is not None:
        s = softcap * torch.tanh(s / softcap)
    m = attention_mask(q.shape[1], causal, segment_ids, q.device)
    if m is not None:
        s = s.masked_fill(~m, float("-inf"))
    if sink is not None:
        B, H, T, _ = s.shape
        s = torch.cat([s, sink.float().view(1, H, 1, 1).expand(B, H, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    if sink is not None:
        p = p[..., :-1]
    vv = repeat_kv(v, q.shape[2] // v.shape[2])
    return torch.einsum("bhts,bshd->bthd", p, vv.float()).to(q.dtype)


def sdpa(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, segment_ids: Tensor | None = None,
         implementation: str = "flash") -> Tensor:
    """Attention dispatcher. `flash`: the hand-written sm_100a kernel (shapes outside its native range are padded
    to it, see `ops/attention.py`; nothing is handed to a library kernel behind the caller's back); `sdpa`: torch's
    fused attention, the eager backend's explicit choice on a GPU; `xla`: the materialised oracle (and every CPU
    call)."""
    if implementation == "xla" or not q.is_cuda:
        return sdpa_reference(q, k, v, causal, segment_ids)
    if implementation != "sdpa":
        from param_decomp_b200.ops import attention as attn_ops

        return attn_ops.flash_attention(q, k, v, causal, segment_ids)
    mask = attention_mask(q.shape[1], False, segment_ids, q.device) if segment_ids is not None else None
    if mask is not None and causal:
        mask = mask & torch.ones(q.shape[1], q.shape[1], dtype=torch.bool, device=q.device).tril()
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                         is_causal=causal and mask is None, enable_gqa=q.shape[2] != k.shape[2])
    return out.transpose(1, 2)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def gelu_tanh(x: Tensor) -> Tensor:
    return F.gelu(x, approximate="tanh")


def causal_depthwise_conv1d_silu(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """`x [B, T, D]`, `weight [D, K]`: each channel convolved with its own length-K causal filter,
    then SiLU."""
    B, T, D = x.shape
    K = weight.shape[-1]
    xp = F.pad(x.transpose(1, 2).float(), (K - 1, 0))
    y = F.conv1d(xp, weight.float().unsqueeze(1), bias.float() if bias is not None else None, groups=D)
    return F.silu(y).transpose(1, 2).to(x.dtype)


# ---- Qwen3.5 (gated DeltaNet) pieces ------------------------------------------------------------
# Parity: param_decomp/target_ports/qwen3_5_moe.py:33-74 (norms, l2norm, conv), :89-158 (sequential
# rule), :187-293 (chunkwise WY form), :296-312 (partial RoPE).

GATED_DELTA_CHUNK = 64


def l2norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """Unit-normalise the last axis; eps joins the SUM of squares inside the rsqrt."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def apply_partial_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """RoPE on the first `cos.shape[-1]` dims of each head, pass-through on the rest.
    `x [B, T, H, hd]`, `cos/sin [B|1, T, r]`."""
    r = cos.shape[-1]
    rot, rest = x[..., :r], x[..., r:]
    c, s = cos.unsqueeze(2), sin.unsqueeze(2)
    out = (rot.float() * c + rotate_half(rot.float()) * s).to(x.dtype)
    return torch.cat([out, rest], dim=-1)


def _delta_rule_sequential(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor) -> Tensor:
    """Per-token recurrence (the oracle). fp32 `[B, T, H, *]` inputs, q already scaled."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    S = q.new_zeros(B, H, dk, dv)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        mem = torch.einsum("bhkv,bhk->bhv", S, k[:, t])
        delta = (v[:, t] - mem) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]))
    return torch.stack(outs, dim=1)


def _solve_unit_lower(a_strict: Tensor, rhs: Tensor, block: int = 8) -> Tensor:
    """`(I + A) x = rhs`, `A` strictly lower triangular: block forward substitution with small
    diagonal blocks inverted by the (exact, nilpotent) Neumann series. Substitution keeps every
    partial result a prefix of the bounded solution, unlike a full log-depth inverse."""
    c = a_strict.shape[-1]
    block = min(block, c)
    assert c % block == 0
    eye = torch.eye(block, dtype=a_strict.dtype, device=a_strict.device)
    xs: list[Tensor] = []
    for i in range(c // block):
        sl = slice(i * block, (i + 1) * block)
        acc = rhs[..., sl, :]
        for j, xj in enumerate(xs):
            acc = acc - a_strict[..., sl, j * block:(j + 1) * block] @ xj
        d = a_strict[..., sl, sl]
        inv, term = eye - d, -d
        for _ in range(block - 2):  # (I + D)^-1 = sum_j (-D)^j, D^block = 0
            term = term @ (-d)
            inv = inv + term
        xs.append(inv @ acc)
    return torch.cat(xs, dim=-2)


def _delta_rule_chunkwise(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, chunk: int) -> Tensor:
    """The same recurrence in WY form: one sequential step per `chunk` tokens."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    n = -(-T // chunk)
    pad = n * chunk - T
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        g, beta = (F.pad(x, (0, 0, 0, pad)) for x in (g, beta))

    def ch(x: Tensor) -> Tensor:  # [B, n*c, H, ...] -> [n, B, H, c, ...]
        p = x.reshape(B, n, chunk, H, *x.shape[3:])
        return p.permute(1, 0, 3, 2, *range(4, p.dim()))

    q, k, v, g, beta = map(ch, (q, k, v, g, beta))
    gc = g.cumsum(-1)
    idx = torch.arange(chunk, device=q.device)
    lower = idx[:, None] >= idx[None, :]
    diff = gc[..., :, None] - gc[..., None, :]
    decay = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    kb = k * beta[..., None]
    a = (kb @ k.transpose(-1, -2) * decay).tril(-1)
    rhs = torch.cat([v * beta[..., None], kb * torch.exp(gc)[..., None]], dim=-1)
    solved = _solve_unit_lower(a, rhs)
    w, u = solved[..., :dv], solved[..., dv:]
    q_dec = q * torch.exp(gc)[..., None]
    local = q @ k.transpose(-1, -2) * decay
    g_last = gc[..., -1]
    k_dec = k * torch.exp(g_last[..., None] - gc)[..., None]
    S = q.new_zeros(B, H, dk, dv)
    outs = []
    for i in range(n):
        delta = w[i] - u[i] @ S
        outs.append(q_dec[i] @ S + local[i] @ delta)
        S = S * torch.exp(g_last[i])[..., None, None] + k_dec[i].transpose(-1, -2) @ delta
    out = torch.stack(outs, dim=0)  # [n, B, H, c, dv]
    return out.permute(1, 0, 3, 2, 4).reshape(B, n * chunk, H, dv)[:, :T]


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, kernel: str = "chunkwise") -> Tensor:
    """`S_t = exp(g_t) S_{t-1};  S_t += k_t (x) beta_t (v_t - S_t^T k_t);  o_t = S_t^T q_t / sqrt(dk)`.
    `q, k [B, T, H, dk]` (already repeated to the value-head count), `v [B, T, H, dv]`, `g, beta [B, T, H]`.
    q and k are l2-normalised in the input dtype, the recurrence runs in fp32. `kernel`:
    `sequential` (oracle), `chunkwise` (WY form), `cuda` (the sm_100a kernel; falls back off-GPU)."""
    in_dtype = q.dtype
    q, k = l2norm(q), l2norm(k)
    q = q.float() * q.shape[-1] ** -0.5
    k, v, g, beta = k.float(), v.float(), g.float(), beta.float()
    if kernel == "cuda" and q.is_cuda:
        from param_decomp_b200.ops import delta_rule

        if delta_rule.supported(q, v):
            return delta_rule.gated_delta_rule(q, k, v, g, beta).to(in_dtype)
        kernel = "chunkwise"
    if kernel == "sequential":
        out = _delta_rule_sequential(q, k, v, g, beta)
    else:
        out = _delta_rule_chunkwise(q, k, v, g, beta, GATED_DELTA_CHUNK)
    return out.to(in_dtype)
