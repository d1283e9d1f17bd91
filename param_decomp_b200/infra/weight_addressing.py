"""Canonical addresses of target weights, for comparing decompositions across runs and families:
`(layer, role)` with `role` in `{attn.q, attn.k, attn.v, attn.o, mlp.in, mlp.gate, mlp.out, experts.*}`.

Parity: param_decomp/topology/ (canonical weight addressing).
"""

from __future__ import annotations

import re
from dataclasses import dataclass

_ROLE = {"q": "attn.q", "k": "attn.k", "v": "attn.v", "o": "attn.o", "q_proj": "attn.q", "k_proj": "attn.k",
         "v_proj": "attn.v", "o_proj": "attn.o", "gate": "mlp.gate", "up": "mlp.in", "c_fc": "mlp.in",
         "down": "mlp.out", "down_proj": "mlp.out", "experts_gate": "experts.gate", "experts_up": "experts.in",
         "experts_down": "experts.out"}
_PATTERNS = (re.compile(r"^layers\.(\d+)\.(?:self_attn|mlp)\.(\w+?)(?:_proj)?$"), re.compile(r"^h\.(\d+)\.(?:attn|mlp)\.(\w+)$"))


@dataclass(frozen=True, order=True)
class WeightAddress:
    layer: int
    role: str


def address_of(site: str) -> WeightAddress:
    for pat in _PATTERNS:
        m = pat.match(site)
        if m and m.group(2) in _ROLE:
            return WeightAddress(int(m.group(1)), _ROLE[m.group(2)])
    raise ValueError(f"no canonical address for site {site!r}")
