"""Placement: which mesh axes each tensor role's dimensions are sharded over.

A *rule* maps semantic axis names (`stack`, `d_in`, `d_out`, `C`, `expert`, `batch`, `position`,
`vocab`, ...) to ordered tuples of mesh axes; unlisted axes replicate. A *placement table* names one
rule per tensor role (component masters / compute weights / operands / Newton-Schulz staging,
activations, frozen-target weight roles). Presets are spelled exactly as in the run YAML
(`runtime.sharding`): `ddp`, `owner`, `zero1`, and the `*-replicated-resident*` family for the
two-axis `(data, tp)` mesh; an explicit `PlacementTableConfig` is folded to the same structure.

How the runtime uses a table:
  * `optimizer_state` decides which slice of each stacked master (and of its Adam/Muon state) a
    rank owns -> the fused reduce-scatter + AdamW + all-gather kernel works on exactly that slice;
  * `compute_weights` says whether the bf16 working copy is resident whole (÷tp only) or gathered
    per use;
  * `C -> tp` on operands makes the site's second GEMM a partial sum over the tp group
    (GEMM -> reduce-scatter / all-reduce), `expert -> tp` places expert blocks for expert parallelism;
  * stacks whose length does not tile their mesh axes are padded with inert zero matrices
    (`stack_multiple`), stripped again in checkpoints.

Parity: param_decomp/core/placement.py:96-101 (batch axes), :183-220,733-751 (stack padding),
:1011-1188 (preset tables), :1688-1728 (`from_config`); core/configs.py:738-836 (table schema);
core/PLACEMENT_DESIGN.md.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from param_decomp_b200.config.run import PlacementTableConfig

Rule = dict[str, tuple[str, ...]]

HSDP_AXES = ("replicate", "fsdp", "tp")
RESIDENT_AXES = ("data", "tp")


def _rule(**kw: str | tuple[str, ...] | list[str] | None) -> Rule:
    out: Rule = {}
    for k, v in kw.items():
        if v is None:
            out[k] = ()
        elif isinstance(v, str):
            out[k] = (v,)
        else:
            out[k] = tuple(v)
    return out


@dataclass(frozen=True)
class ComponentsPlacement:
    optimizer_state: Rule
    compute_weights: Rule
    faithfulness_weights: Rule
    faithfulness_deltas: Rule
    operands: Rule
    ns_compute: Rule


@dataclass(frozen=True)
class TargetPlacement:
    embedding_persist: Rule
    column_persist: Rule  # weight [d_out, d_in] of a column-parallel linear
    row_persist: Rule
    column_operand: Rule
    row_operand: Rule
    output_persist: Rule
    intermediate: Rule


@dataclass(frozen=True)
class PlacementRules:
    name: str
    mesh_axes: tuple[str, ...]
    components: ComponentsPlacement
    activations_external: Rule
    activations_component: Rule
    target: TargetPlacement
    ci_fn_preset: str
    resident: bool = False  # the bf16 working copy is held whole (÷tp) between steps
    expert_blocked: bool = False

    def batch_axes(self) -> tuple[str, ...]:
        return tuple(a for a in self.mesh_axes if a != "tp")

    def shard_factor(self, rule: Rule, axis: str, mesh: dict[str, int]) -> int:
        n = 1
        for m in rule.get(axis, ()):
            n *= mesh.get(m, 1)
        return n


def _target(batch: tuple[str, ...], fsdp: tuple[str, ...], tensor_parallel: bool = True) -> TargetPlacement:
    """The frozen target's rows: column / row parallel linears over `tp` (persisted further over `fsdp` where the
    mesh has that axis), embedding and output head persisted over `fsdp` along `d_model` and used whole. `ddp`
    keeps the target whole on every rank (`tensor_parallel=False`)."""
    tp = ("tp",) if tensor_parallel else ()
    return TargetPlacement(
        embedding_persist=_rule(d_model=fsdp),
        column_persist=_rule(d_in=fsdp, d_out=tp),
        row_persist=_rule(d_in=tp, d_out=fsdp),
        column_operand=_rule(d_out=tp),
        row_operand=_rule(d_in=tp),
        output_persist=_rule(d_model=fsdp),
        intermediate=_rule(batch=batch, feature=tp, q_head=tp, kv_head=tp),
    )


def _preset(name: str) -> PlacementRules:
    hs_batch, rs_batch = ("replicate", "fsdp"), ("data",)
    ext_h = _rule(batch=hs_batch)
    ext_r = _rule(batch=rs_batch)
    comp_h, comp_r = _rule(batch=hs_batch, C="tp"), _rule(batch=rs_batch, C="tp")
    # The rows below restate the reference's preset tables (param_decomp/core/placement.py:1011-1116); the resolved
    # rules of the dense presets are compared with its recorded tables in tests/test_reference_goldens.py.
    if name == "ddp":
        rep = _rule()
        c = ComponentsPlacement(rep, rep, rep, rep, rep, ns_compute=_rule(stack="replicate"))
        return PlacementRules(name, HSDP_AXES, c, ext_h, comp_h, _target(hs_batch, (), tensor_parallel=False), "ddp")
    if name == "owner":
        c = ComponentsPlacement(
            optimizer_state=_rule(stack="replicate", d_in="fsdp", d_out="fsdp", C="tp"),
            compute_weights=_rule(d_in="fsdp", d_out="fsdp", C="tp"),
            faithfulness_weights=_rule(stack="replicate", d_in="fsdp", d_out="fsdp", C="tp"),
            faithfulness_deltas=_rule(stack="replicate", d_out="fsdp"),
            operands=_rule(C="tp"),
            ns_compute=_rule(stack="replicate"),
        )
        return PlacementRules(name, HSDP_AXES, c, ext_h, comp_h, _target(hs_batch, ("fsdp",)), "owner")
    if name == "zero1":
        c = ComponentsPlacement(
            optimizer_state=_rule(d_in="fsdp", d_out="fsdp", C=("tp", "replicate")),
            compute_weights=_rule(d_in="fsdp", d_out="fsdp", C="tp"),
            faithfulness_weights=_rule(d_in="fsdp", d_out="fsdp", C=("tp", "replicate")),
            faithfulness_deltas=_rule(d_out="fsdp", d_in=("tp", "replicate")),
            operands=_rule(C="tp"),
            ns_compute=_rule(stack="replicate"),
        )
        return PlacementRules(name, HSDP_AXES, c, ext_h, comp_h, _target(hs_batch, ("fsdp",)), "zero1")
    resident = {
        "zero1-replicated-resident": ("zero1", False, False),
        "owner-replicated-resident": ("owner", False, False),
        "zero1-replicated-resident-moe": ("zero1", True, False),
        "owner-replicated-resident-moe": ("owner", True, False),
        "zero1-replicated-resident-moe-replicated-ns": ("zero1", True, True),
    }
    if name in resident:
        kind, moe, rep_ns = resident[name]
        if kind == "zero1" and moe:
            opt = _rule(d_in="data", d_out="data", C="tp", C_block="data", expert="tp")
        elif kind == "zero1":
            opt = _rule(C=("tp", "data"))  # intra-matrix: the component axis carries both splits
        else:
            opt = _rule(stack="data", C="tp", expert="tp" if moe else None)
        working = _rule(C="tp", expert="tp" if moe else None)
        if kind == "owner":
            deltas = _rule(stack="data")
        else:
            deltas = _rule(d_out="data", d_in="tp") if moe else _rule(d_in=("tp", "data"))
        c = ComponentsPlacement(
            optimizer_state=opt, compute_weights=working, faithfulness_weights=opt, faithfulness_deltas=deltas,
            operands=working, ns_compute=_rule() if rep_ns else _rule(stack="data"),
        )
        return PlacementRules(name, RESIDENT_AXES, c, ext_r, comp_r, _target(rs_batch, ()), name,
                              resident=True, expert_blocked=moe)
    raise ValueError(f"unknown placement preset {name!r}")


PRESET_NAMES = ("owner", "zero1", "zero1-replicated-resident", "owner-replicated-resident",
                "zero1-replicated-resident-moe", "owner-replicated-resident-moe",
                "zero1-replicated-resident-moe-replicated-ns", "ddp")
PRESETS = {n: _preset(n) for n in PRESET_NAMES}


def _fold(rule_cfg: dict) -> Rule:
    return _rule(**{k: v for k, v in rule_cfg.items()})


def from_config(spec: str | PlacementTableConfig, mesh: dict[str, int]) -> PlacementRules:
    """Resolve `runtime.sharding` against the run's mesh; fails closed on axes the mesh lacks."""
    if isinstance(spec, str):
        rules = PRESETS[spec]
    else:
        c, t = spec.components, spec.target
        rules = PlacementRules(
            name="explicit", mesh_axes=tuple(mesh),
            components=ComponentsPlacement(*(_fold(getattr(c, f)) for f in (
                "optimizer_state", "compute_weights", "faithfulness_weights", "faithfulness_deltas", "operands",
                "ns_compute"))),
            activations_external=_fold(spec.activations.external),
            activations_component=_fold(spec.activations.component),
            target=TargetPlacement(_fold(t.embedding.persist), _fold(t.column.persist), _fold(t.row.persist),
                                   _fold(t.column.operand), _fold(t.row.operand), _fold(t.output.persist),
                                   _fold(t.intermediate)),
            ci_fn_preset=spec.ci_fn,
            resident=set(mesh) == set(RESIDENT_AXES),
        )
    assert set(rules.mesh_axes) == set(mesh), (
        f"placement {rules.name!r} is written for mesh axes {rules.mesh_axes}, the run declares {tuple(mesh)}"
    )
    for role in (rules.components.optimizer_state, rules.components.compute_weights, rules.components.operands,
                 rules.components.ns_compute, rules.activations_external, rules.activations_component):
        for axis, axes in role.items():
            for m in axes:
                assert m in mesh, f"rule maps {axis!r} to mesh axis {m!r}, which the mesh does not declare"
    return rules


def stack_multiple(rules: PlacementRules, mesh: dict[str, int]) -> int:
    """The multiple the placement itself asks stacks to be padded to: the factor by which the persisted state
    splits the `stack` axis (param_decomp/core/placement.py:183-220). What this runtime adds on top (its sharded
    optimizers deal whole matrices or flat ranges to every batch rank) is `layout.resolve`'s business."""
    return rules.shard_factor(rules.components.optimizer_state, "stack", mesh)


@dataclass
class ShardSpec:
    """Slice of a tensor a rank owns: per-dimension `(start, length)`; full length = replicated."""

    slices: list[tuple[int, int]] = field(default_factory=list)

    def apply(self, t):
        for dim, (start, length) in enumerate(self.slices):
            t = t.narrow(dim, start, length)
        return t


def shard_of(shape: tuple[int, ...], dim_names: tuple[str, ...], rule: Rule, mesh: dict[str, int],
             coords: dict[str, int]) -> ShardSpec:
    """The slice of a tensor with semantic dims `dim_names` that the rank at `coords` holds.
    A dim sharded over several mesh axes is linearised in the rule's order (first axis slowest)."""
    out = []
    for size, name in zip(shape, dim_names):
        axes = rule.get(name, ())
        parts, index = 1, 0
        for a in axes:
            parts, index = parts * mesh[a], index * mesh[a] + coords[a]
        assert size % parts == 0, f"dim {name!r} of size {size} does not tile {axes} = {parts} parts"
        out.append((index * (size // parts), size // parts))
    return ShardSpec(out)


def validate_sites(rules: PlacementRules, mesh: dict[str, int], sites) -> None:
    """Refuse, before any GPU work, a site set the table cannot place."""
    for s in sites:
        for role_name in ("optimizer_state", "compute_weights", "operands"):
            role = getattr(rules.components, role_name)
            for axis, size in (("d_in", s.d_in), ("d_out", s.d_out), ("C", s.C_block if s.blocked else s.C)):
                f = rules.shard_factor(role, axis, mesh)
                assert size % f == 0, f"{s.name}: {axis}={size} does not tile {role_name} factor {f}"
            if s.blocked:
                f = rules.shard_factor(role, "expert", mesh)
                assert s.n_blocks % f == 0, f"{s.name}: {s.n_blocks} expert blocks do not tile {f}"
