"""From a run's placement table to what the runtime does with it.

`runtime.sharding` (a preset name or an explicit table, `parallel/placement.py`) is resolved against the run's
mesh; the engine then reads these facts from the resolved rules:

  * are the components' masters / optimizer state sharded over the batch axes (every preset but `ddp`)? Then the
    component group runs the flat-sharded AdamW (reduce-scatter + update + all-gather in one kernel over NVLink
    peer memory on GPUs, the collective form elsewhere) or, for Muon, the stack-split Newton-Schulz optimizer;
    otherwise gradients are all-reduced and every rank keeps whole state;
  * does the component axis `C` split over `tp` (every preset on a mesh with `tp > 1`)?
  * the multiple every stack is padded to, so the `stack` axis tiles each role that shards it
    (`placement.stack_multiple`) and the Newton-Schulz split;
  * whether the site set can be placed at all (`placement.validate_sites`, fails before any GPU work).

What the presets do NOT change here: the bf16 compute copy of the components is re-gathered whole once per step
(the reference's resident family) rather than per layer inside the forward, whatever the preset says about
`compute_weights`; the run log states this.

Parity: param_decomp/core/placement.py:1011-1116 (presets), :1688-1728 (`from_config`), :183-220 (stack
padding), experiments/lm/training.py:197-301 (where the reference hands the rules to the engine).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from param_decomp_b200.parallel import placement as pl
from param_decomp_b200.parallel.topology import mesh_axes


@dataclass(frozen=True)
class RuntimeLayout:
    rules: pl.PlacementRules
    mesh: dict[str, int]
    optimizer_sharded: bool
    components_split_over_tp: bool
    stack_multiple: int

    @property
    def label(self) -> str:
        axes = " x ".join(f"{k}{v}" for k, v in self.mesh.items() if v > 1) or "single"
        opt = "sharded masters / moments / gradient reduction" if self.optimizer_sharded else "replicated, all-reduce"
        return f"{axes} ({self.rules.name}: {opt}{', C split over tp' if self.components_split_over_tp else ''})"


def resolve(runtime_cfg: Any, sites: tuple | None = None, world: int | None = None) -> RuntimeLayout:
    """`world`: the job's real size; a single process runs any mesh as its own 1-rank slice (every axis 1)."""
    mesh = dict(mesh_axes(runtime_cfg.mesh))
    rules = pl.from_config(runtime_cfg.sharding, mesh)
    if world == 1:
        mesh = {k: 1 for k in mesh}
    batch = [a for a in rules.batch_axes() if a in mesh]
    batch_mesh = {a: (mesh[a] if a in batch else 1) for a in mesh}
    opt = rules.components.optimizer_state
    sharded = any(rules.shard_factor(opt, axis, batch_mesh) > 1 for axis in ("d_in", "d_out", "C", "stack"))
    tp_mesh = {a: (mesh[a] if a == "tp" else 1) for a in mesh}
    c_split = rules.shard_factor(rules.components.compute_weights, "C", tp_mesh) > 1 or \
        rules.shard_factor(rules.components.operands, "C", tp_mesh) > 1
    if sites is not None:
        pl.validate_sites(rules, mesh, sites)
    # this runtime's sharded optimizers split a group's stack (Muon: whole matrices for Newton-Schulz) or its flat
    # buffer over EVERY batch rank, so stacks tile the batch axes' product whenever the state is sharded
    batch_world = 1
    for a in batch:
        batch_world *= mesh[a]
    splits_ns = bool(rules.components.ns_compute.get("stack"))  # a table with replicated Newton-Schulz needs no tiling
    multiple = max(pl.stack_multiple(rules, mesh), batch_world if (sharded and splits_ns) else 1)
    return RuntimeLayout(rules, mesh, sharded, c_split, multiple)
