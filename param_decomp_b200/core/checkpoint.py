"""safetensors checkpoints of a decomposition run.

Layout under `<run_dir>/ckpts/<step>/`:
  decomposition.safetensors   components/<group>/V  [g, d_in, C]   (stack pads stripped)
                              components/<group>/U  [g, C, d_out]
                              ci_fn/<parameter path>
                              metadata: JSON `site_stack_indices` {site: [group, index]} so a
                              component key "<site>:<idx>" addresses column idx of that slice
  training.safetensors        opt/components/<leaf>/{mu,nu,mom}, opt/ci_fn/...,
                              adversaries/<term>/{sources,delta,opt}/..., frequency/<site>, step
Multi-rank runs write `<name>-rank<r>-of-<n>.safetensors` holding each rank's shard plus an
`index.json` of `{key: {axis, world}}`; `load_*` re-assembles (or re-shards) them, so a checkpoint
written on one mesh restores on another.

The reference stores the same two items (`decomposition`, `training`) with Orbax
(param_decomp/core/checkpoint.py:63-239); the key paths here mirror its tree paths. Retention
(`keep_last n | keep_all`) follows core/configs.py:1048-1089.
"""

from __future__ import annotations

import json
import shutil
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file
from torch import Tensor, nn

from param_decomp_b200.core.components import ComponentStacks
from param_decomp_b200.core.losses import FrequencyEMA

DECOMPOSITION_FILE = "decomposition.safetensors"
TRAINING_FILE = "training.safetensors"


def ckpt_root(run_dir: Path) -> Path:
    return Path(run_dir) / "ckpts"


def list_steps(run_dir: Path) -> list[int]:
    root = ckpt_root(run_dir)
    if not root.exists():
        return []
    return sorted(int(p.name) for p in root.iterdir() if p.is_dir() and p.name.isdigit()
                  and (p / DECOMPOSITION_FILE).exists())


def latest_step(run_dir: Path) -> int | None:
    steps = list_steps(run_dir)
    return steps[-1] if steps else None


def is_readable(run_dir: Path, step: int) -> bool:
    """Both files of a step open and their headers agree with their sizes (a truncated or half-copied file fails
    here, before anything is restored from it)."""
    from safetensors import safe_open

    try:
        for name in (DECOMPOSITION_FILE, TRAINING_FILE):
            with safe_open(str(ckpt_root(run_dir) / str(step) / name), framework="pt") as f:
                for k in f.keys():
                    f.get_slice(k).get_shape()
        return True
    except Exception:  # noqa: BLE001  (any failure to open / parse means: not a usable checkpoint)
        return False


def latest_readable_step(run_dir: Path, log=None) -> int | None:
    """The newest step whose files can be read; damaged newer ones are named in the log and skipped. Every rank
    reads the same files, so every rank lands on the same step."""
    for step in reversed(list_steps(run_dir)):
        if is_readable(run_dir, step):
            return step
        if log is not None:
            log.warning("checkpoint %s/ckpts/%d is damaged (truncated or unreadable): falling back to an older one",
                        run_dir, step)
    return None


def _storable(t: Tensor) -> Tensor:
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16) if t.dtype == torch.uint16 else t


def decomposition_tensors(components: ComponentStacks, ci_fn: nn.Module,
                          expert_shard=None) -> tuple[dict[str, Tensor], dict[str, str]]:
    """`expert_shard` (`parallel.expert_shard.StackSharding`): blocked groups hold this rank's experts
    only; they are gathered over the expert group (a collective every rank of it must enter) so the
    file always has the global `[sites, E, ...]` stacks."""
    out: dict[str, Tensor] = {}
    for gname, members in components.groups.items():
        key = components.param_key(gname)
        n = len(members)
        V, U = components.V[key][:n].detach(), components.U[key][:n].detach()
        if expert_shard is not None and key in expert_shard.blocked_keys:
            V, U = expert_shard.gather(V, "V"), expert_shard.gather(U, "U")
        out[f"components/{gname}/V"] = _storable(V)
        out[f"components/{gname}/U"] = _storable(U)
    for name, p in ci_fn.state_dict().items():
        out[f"ci_fn/{name}"] = _storable(p)
    meta = {
        "site_stack_indices": json.dumps({s: list(v) for s, v in components.site_stack_indices.items()}),
        "format": "param_decomp_b200/decomposition/v1",
    }
    return out, meta


def _stack_extents(components: ComponentStacks) -> dict[str, tuple[int, int]]:
    """`"V.<key>" / "U.<key>" -> (real entries, padded entries)` of every component stack. Stacks are padded to the
    multiple the run's layout needs (`ComponentStacks(stack_multiple)`); files hold the real entries only, so a
    checkpoint written under one padding resumes under another."""
    out = {}
    for gname, members in components.groups.items():
        key = components.param_key(gname)
        out["V." + key] = out["U." + key] = (len(members), len(members) + components.stack_pads[gname])
    return out


def _strip_stack_pads(extents: dict[str, tuple[int, int]], k: str, v: Tensor) -> Tensor:
    real, padded = extents.get(k.rsplit("/", 1)[0], (0, 0))
    return v[:real] if padded > real and v.dim() >= 1 and v.shape[0] == padded else v


def _restore_stack_pads(extents: dict[str, tuple[int, int]], k: str, v: Tensor) -> Tensor:
    real, padded = extents.get(k.rsplit("/", 1)[0], (0, 0))
    if padded > real and v.dim() >= 1 and v.shape[0] == real:
        return torch.cat([v, v.new_zeros(padded - real, *v.shape[1:])])
    return v


def training_tensors(state, expert_shard=None) -> tuple[dict[str, Tensor], dict[str, str]]:
    out: dict[str, Tensor] = {"step": torch.tensor(state.step, dtype=torch.int64)}
    uint16_keys = []
    extents = _stack_extents(state.components)
    for group, opt in (("components", state.components_opt), ("ci_fn", state.ci_fn_opt)):
        for k, v in sorted(opt.state_dict().items()):  # sorted: the gathers below must line up across ranks
            if expert_shard is not None and group == "components" and v.dim() >= 2 and expert_shard.is_split(k):
                v = expert_shard.gather(v, k)
            if group == "components":
                v = _strip_stack_pads(extents, k, v)  # moments of the inert padding matrices never reach the file
            out[f"opt/{group}/{k}"] = _storable(v)
    for term, adv in state.adversaries.items():
        for k, v in adv.state_dict().items():
            if v.dtype == torch.uint16:
                uint16_keys.append(f"adversaries/{term}/{k}")
            out[f"adversaries/{term}/{k}"] = _storable(v)
    for site, ema in state.frequency.items():
        out[f"frequency/{site}/value"] = _storable(ema.value)
        out[f"frequency/{site}/weight"] = torch.tensor(ema.weight, dtype=torch.float64)
        out[f"frequency/{site}/halflife"] = torch.tensor(ema.halflife_steps, dtype=torch.float64)
    meta = {"uint16_keys": json.dumps(uint16_keys), "format": "param_decomp_b200/training/v1"}
    return out, meta


def save_state(run_dir: Path, state, retention_keep_last: int | None = None, expert_shard=None,
               write: bool = True) -> Path:
    """Synchronous save of both items at `state.step`, then prune per the retention policy. With
    `expert_shard` every rank of the expert group calls this (the tensors are gathered collectively)
    and only the one with `write=True` touches the file system."""
    step_dir = ckpt_root(run_dir) / str(state.step)
    if expert_shard is not None:
        d, dm = decomposition_tensors(state.components, state.ci_fn, expert_shard)
        t, tm = training_tensors(state, expert_shard)
        if not write:
            return step_dir
        return _write_step(run_dir, step_dir, d, dm, t, tm, retention_keep_last)
    d, dm = decomposition_tensors(state.components, state.ci_fn)
    t, tm = training_tensors(state)
    return _write_step(run_dir, step_dir, d, dm, t, tm, retention_keep_last)


def _write_step(run_dir: Path, step_dir: Path, d, dm, t, tm, retention_keep_last: int | None) -> Path:
    tmp = step_dir.with_name(step_dir.name + ".tmp")
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    save_file(d, str(tmp / DECOMPOSITION_FILE), metadata=dm)
    save_file(t, str(tmp / TRAINING_FILE), metadata=tm)
    if step_dir.exists():
        shutil.rmtree(step_dir)
    tmp.rename(step_dir)  # a step directory is visible only once complete
    if retention_keep_last is not None:
        for old in list_steps(run_dir)[:-retention_keep_last]:
            shutil.rmtree(ckpt_root(run_dir) / str(old))
    return step_dir


def _read(path: Path) -> tuple[dict[str, Tensor], dict[str, str]]:
    tensors = {}
    with safe_open(str(path), framework="pt") as f:
        meta = f.metadata() or {}
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return tensors, meta


def restore_components(run_dir: Path, step: int, components: ComponentStacks, expert_shard=None) -> None:
    """V/U only (analysis-time partial restore). Pads of the destination are re-derived (zero). With
    `expert_shard` the file's global blocked stacks are cut to this rank's experts."""
    tensors, _ = _read(ckpt_root(run_dir) / str(step) / DECOMPOSITION_FILE)
    with torch.no_grad():
        for gname, members in components.groups.items():
            key, n = components.param_key(gname), len(members)
            V, U = tensors[f"components/{gname}/V"], tensors[f"components/{gname}/U"]
            if expert_shard is not None and key in expert_shard.blocked_keys:
                V, U = expert_shard.local_slice(V, "V"), expert_shard.local_slice(U, "U")
            assert V.shape[0] == n, f"group {gname}: checkpoint has {V.shape[0]} sites, run has {n}"
            components.V[key].zero_()
            components.U[key].zero_()
            components.V[key][:n].copy_(V)
            components.U[key][:n].copy_(U)


def restore_decomposition(run_dir: Path, step: int, components: ComponentStacks, ci_fn: nn.Module,
                          expert_shard=None) -> None:
    restore_components(run_dir, step, components, expert_shard)
    tensors, _ = _read(ckpt_root(run_dir) / str(step) / DECOMPOSITION_FILE)
    sd = {k[len("ci_fn/"):]: v for k, v in tensors.items() if k.startswith("ci_fn/")}
    ci_fn.load_state_dict(sd)


def restore_state(run_dir: Path, step: int, state, data_rank: int = 0, data_world: int = 1) -> None:
    """Full resume: decomposition + optimizer states + adversaries + frequency EMA + step. Per-row adversary
    sources are stored for the global batch; each of `data_world` batch shards keeps its own rows."""
    expert_shard = getattr(state, "expert_shard", None)
    restore_decomposition(run_dir, step, state.components, state.ci_fn, expert_shard)
    tensors, meta = _read(ckpt_root(run_dir) / str(step) / TRAINING_FILE)
    uint16_keys = set(json.loads(meta.get("uint16_keys", "[]")))
    dev = next(state.components.parameters()).device

    def get(k: str) -> Tensor:
        v = tensors[k]
        if (expert_shard is not None and k.startswith("opt/components/") and v.dim() >= 2
                and expert_shard.is_split(k[len("opt/components/"):])):
            v = expert_shard.local_slice(v, k[len("opt/components/"):])
        return (v.view(torch.uint16) if k in uint16_keys else v).to(dev)

    state.step = int(tensors["step"].item())
    extents = _stack_extents(state.components)
    for group, opt in (("components", state.components_opt), ("ci_fn", state.ci_fn_opt)):
        prefix = f"opt/{group}/"
        sd = {k[len(prefix):]: get(k) for k in tensors if k.startswith(prefix)}
        if group == "components":  # this run's stacks may be padded differently from the writer's
            sd = {k: _restore_stack_pads(extents, k, v) for k, v in sd.items()}
        opt.load_state_dict(sd)
    for term, adv in state.adversaries.items():
        prefix = f"adversaries/{term}/"
        adv.load_state_dict({k[len(prefix):]: get(k) for k in tensors if k.startswith(prefix)}, data_rank, data_world)
    sites = {k.split("/")[1] for k in tensors if k.startswith("frequency/")}
    for site in sites:
        state.frequency[site] = FrequencyEMA(
            halflife_steps=float(tensors[f"frequency/{site}/halflife"].item()),
            value=get(f"frequency/{site}/value"),
            weight=float(tensors[f"frequency/{site}/weight"].item()),
        )


# ---- sharded files ----------------------------------------------------------------------------------


def save_sharded(path: Path, tensors: dict[str, Tensor], shard_axes: dict[str, int], rank: int, world: int) -> None:
    """Each rank writes its shard; rank 0 also writes the index naming every key's shard axis."""
    path = Path(path)
    save_file({k: _storable(v) for k, v in tensors.items()},
              str(path.with_name(f"{path.stem}-rank{rank}-of-{world}.safetensors")))
    if rank == 0:
        path.with_name(path.stem + ".index.json").write_text(json.dumps({"world": world, "axes": shard_axes}))


def load_sharded(path: Path, rank: int = 0, world: int = 1) -> dict[str, Tensor]:
    """Re-assemble every key along its shard axis, then cut the `rank`-of-`world` slice of the NEW
    mesh (world=1 returns whole tensors), so checkpoints move between topologies."""
    path = Path(path)
    index = json.loads(path.with_name(path.stem + ".index.json").read_text())
    old_world, axes = index["world"], index["axes"]
    parts = [_read(path.with_name(f"{path.stem}-rank{r}-of-{old_world}.safetensors"))[0] for r in range(old_world)]
    out = {}
    for k in parts[0]:
        ax = axes.get(k)
        if ax is None:
            out[k] = parts[0][k]
            continue
        full = torch.cat([p[k] for p in parts], dim=ax)
        if world > 1:
            n = full.shape[ax]
            assert n % world == 0, f"{k}: axis {ax} of size {n} does not tile {world} ranks"
            full = full.narrow(ax, rank * (n // world), n // world).contiguous()
        out[k] = full
    return out
