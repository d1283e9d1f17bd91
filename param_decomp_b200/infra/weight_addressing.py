"""Canonical addresses of decomposed weights, for comparing decompositions across runs and model families:
every site name of either grammar resolves to `(layer, role)`, and back to a short display label.

  GLU family      layers.{i}.self_attn.{q,k,v,o}_proj, layers.{i}.mlp.{gate,up,down}_proj,
                  layers.{i}.mlp.{experts,shared}_{gate,up,down}
  simple-MLP      h.{i}.attn.{q,k,v,o}_proj, h.{i}.mlp.{c_fc,down_proj}
  toys            linear1 / linear2 / hidden_layers.{i} (TMS), layers.{i}.mlp_in / mlp_out (ResidualMLP)

Roles: `attn.q|k|v|o`, `mlp.gate|in|out`, `experts.gate|in|out`, `shared.gate|in|out`. `c_fc` and `up` are both
the MLP's input projection (`mlp.in`), so a plain-MLP and a gated-MLP decomposition line up.

Parity: param_decomp/topology/canonical.py, path_schemas.py (canonical weight addressing, per-family path
schemas).
"""

from __future__ import annotations

import re
from dataclasses import dataclass

_ROLE = {"q": "attn.q", "k": "attn.k", "v": "attn.v", "o": "attn.o", "q_proj": "attn.q", "k_proj": "attn.k",
         "v_proj": "attn.v", "o_proj": "attn.o", "gate": "mlp.gate", "up": "mlp.in", "c_fc": "mlp.in",
         "down": "mlp.out", "down_proj": "mlp.out", "experts_gate": "experts.gate", "experts_up": "experts.in",
         "experts_down": "experts.out", "shared_gate": "shared.gate", "shared_up": "shared.in",
         "shared_down": "shared.out", "mlp_in": "mlp.in", "mlp_out": "mlp.out"}
_PATTERNS = (
    re.compile(r"^(?:model\.)?layers\.(\d+)\.(?:self_attn|mlp)\.((?:experts_|shared_)?\w+?)(?:_proj)?$"),
    re.compile(r"^h\.(\d+)\.(?:attn|mlp)\.(\w+)$"),
    re.compile(r"^layers\.(\d+)\.(mlp_in|mlp_out)$"),
)
_TOY = {"linear1": (0, "mlp.in"), "linear2": (0, "mlp.out")}
ROLE_ORDER = ("attn.q", "attn.k", "attn.v", "attn.o", "mlp.gate", "mlp.in", "mlp.out", "experts.gate", "experts.in",
              "experts.out", "shared.gate", "shared.in", "shared.out")


@dataclass(frozen=True)
class WeightAddress:
    layer: int
    role: str

    @property
    def label(self) -> str:
        """`layer-03-02-attn-k`: sortable by depth, then by the role's place in a block."""
        return f"layer-{self.layer:02d}-{ROLE_ORDER.index(self.role) + 1:02d}-{self.role.replace('.', '-')}"

    def sort_key(self) -> tuple[int, int]:
        return self.layer, ROLE_ORDER.index(self.role)


def address_of(site: str) -> WeightAddress:
    if site in _TOY:
        return WeightAddress(*_TOY[site])
    m = re.match(r"^hidden_layers\.(\d+)$", site)
    if m:
        return WeightAddress(int(m.group(1)) + 1, "mlp.in")
    for pat in _PATTERNS:
        m = pat.match(site)
        if m and m.group(2) in _ROLE:
            return WeightAddress(int(m.group(1)), _ROLE[m.group(2)])
    raise ValueError(f"no canonical address for site {site!r}")


def try_address(site: str) -> WeightAddress | None:
    try:
        return address_of(site)
    except ValueError:
        return None


def align_sites(a: list[str], b: list[str]) -> list[tuple[str, str]]:
    """Pairs of site names from two runs (possibly of different families) that address the same weight, in
    canonical order."""
    by_addr = {address_of(s): s for s in b}
    pairs = [(s, by_addr[address_of(s)]) for s in a if address_of(s) in by_addr]
    return sorted(pairs, key=lambda p: address_of(p[0]).sort_key())
