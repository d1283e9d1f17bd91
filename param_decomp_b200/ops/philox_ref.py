"""Pure-torch restatement of the device Philox4x32-7 stream (`csrc/common.cuh`).

Used by tests and by the eager fallback of the mask sampler so that a mask element is the same
function of `(seed, stream, row, column)` on CPU and in the fused GEMM epilogues.
"""

from __future__ import annotations

import torch

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF
ROUNDS = 7


def _mulhilo(a: int, b: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    # b holds uint32 values in int64. a * b < 2^64 wraps in int64, but two's-complement wrapping keeps all 64 bits
    # of the product: the low word is `p & MASK`, the high word the (sign-extending) shift masked back to 32 bits.
    p = b * a
    return (p >> 32) & _MASK, p & _MASK


def philox4x32(c0, c1, c2, c3, k0: int, k1: int):
    """`ROUNDS` rounds on int64 tensors holding uint32 values. Returns four such tensors."""
    for _ in range(ROUNDS):
        hi0, lo0 = _mulhilo(_M0, c0)
        hi1, lo1 = _mulhilo(_M1, c2)
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _MASK, lo1, (hi0 ^ c3 ^ k1) & _MASK, lo0
        k0 = (k0 + _W0) & _MASK
        k1 = (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def uniform(seed: int, stream: int, rows: int, cols: int, row_offset: int = 0,
            device: torch.device | str = "cpu") -> torch.Tensor:
    """`[rows, cols]` fp32 uniforms in (0,1) with 16 random bits, matching `philox_uniform8`."""
    assert cols % 8 == 0
    groups = cols // 8
    r = torch.arange(row_offset, row_offset + rows, dtype=torch.int64, device=device)[:, None]
    g = torch.arange(groups, dtype=torch.int64, device=device)[None, :]
    c0 = g.expand(rows, groups).clone()
    c1 = r.expand(rows, groups).clone()
    c2 = torch.full_like(c0, stream & _MASK)
    c3 = torch.full_like(c0, 0x5044)
    w = philox4x32(c0, c1, c2, c3, seed & _MASK, (seed >> 32) & _MASK)
    parts = []
    for word in w:
        parts.append(word & 0xFFFF)
        parts.append(word >> 16)
    bits = torch.stack(parts, dim=-1).reshape(rows, cols)
    return (bits.to(torch.float32) + 0.5) * (1.0 / 65536.0)
