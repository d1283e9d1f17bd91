"""Adversarial mask sources: persistent (PPGD) and fresh (PGD).

A *source* `s in [0,1]` replaces the uniform noise of a stochastic mask: `m = ci + (1 - ci) s`;
a *delta source* does the same for the delta mask. Persistent sources live across steps and are
ascended on the reconstruction loss; fresh sources are initialised per use and ascended with
sign-gradient steps.

Parity: param_decomp/core/adversary.py:96-150 (`SourceStacks`), :153-209 (fp32 / bf16 / uint16
fixed-point storage with stochastic rounding), :283-358 (shapes `c`/`bc`/`bsc`, pools),
:392-496 (adam / sgd / momentum ascent + clip to [0,1]), :499-567 (warm-up and final ascents);
core/train.py:790-807 and core/recon_eval.py:142-257 (fresh sign-PGD).
"""

from __future__ import annotations

import zlib
from dataclasses import dataclass, field

import torch
from torch import Tensor

from param_decomp_b200.config.losses import AdamPGDConfig, MomentumSgdPGDConfig, SgdPGDConfig
from param_decomp_b200.core import rng
from param_decomp_b200.core.components import SiteSpec
from param_decomp_b200.core.rng import StepKey

UINT16_UNIT_SCALE = 65535.0


def source_lead_shape(shape: str, batch: int, positions: int | None) -> tuple[int, ...]:
    """Leading shape of a source for a target with (`positions` not None) or without a position
    axis. Omitted axes are size-1 broadcast axes."""
    if positions is None:
        return {"c": (1,), "bc": (batch,)}[shape]
    return {"c": (1, 1), "bc": (batch, 1), "bsc": (batch, positions)}[shape]


# ---- storage ---------------------------------------------------------------------------------


def encode_sources(values: Tensor, dtype: str, key: StepKey | None = None, stream: int = 0) -> Tensor:
    """fp32 values in [0,1] -> storage. uint16 uses stochastic rounding so sub-half-step updates
    are kept in expectation (round-to-nearest would stall them)."""
    if dtype == "float32":
        return values.float()
    if dtype == "bfloat16":
        return values.to(torch.bfloat16)
    assert dtype == "uint16", dtype
    scaled = values.float().clamp(0, 1) * UINT16_UNIT_SCALE
    floor = scaled.floor()
    if key is None:
        noise = torch.rand_like(scaled)
    else:
        flat = scaled.reshape(-1, scaled.shape[-1])
        noise = rng.uniform(key, stream, flat.shape[0], flat.shape[1], 0, scaled.device).reshape(scaled.shape)
    up = (scaled - floor) > noise
    return (floor + up.float()).clamp(0, UINT16_UNIT_SCALE).to(torch.int32).to(torch.uint16)


def decode_sources(stored: Tensor) -> Tensor:
    if stored.dtype == torch.uint16:
        return stored.to(torch.int32).float() / UINT16_UNIT_SCALE
    return stored.float()


def velocity_dtype(source_dtype: str) -> torch.dtype:
    return torch.float32 if source_dtype == "float32" else torch.bfloat16


# ---- persistent adversary ----------------------------------------------------------------------


@dataclass
class PersistentAdversary:
    """Sources for every site plus the optimizer state of their ascent.

    `sources[site] [*lead, C]`, `delta[site] [*lead, 1]` (stored in `source_dtype`);
    with a pool, `lead = (batch * pool_size,)` (+ a size-1 position axis) and each step picks one
    particle per batch row.
    """

    optimizer: AdamPGDConfig | SgdPGDConfig | MomentumSgdPGDConfig
    source_dtype: str
    sources: dict[str, Tensor] = field(default_factory=dict)
    delta: dict[str, Tensor] = field(default_factory=dict)
    state: dict[str, Tensor] = field(default_factory=dict)  # "<site>/mu", "<site>/nu", "<site>/vel", + "d:<site>/..."
    n_updates: int = 0
    pool_size: int = 1
    batch_shared: bool = False  # shape `c`: one source for the whole batch, identical on every batch shard

    @classmethod
    def init(cls, sites: tuple[SiteSpec, ...], optimizer, source_dtype: str, shape: str, batch: int,
             positions: int | None, key: StepKey, pool_size: int = 1,
             device: torch.device | str = "cpu", data_rank: int = 0) -> "PersistentAdversary":
        """`batch` is this rank's share of the global batch and `data_rank` its place among the batch shards:
        per-row sources are drawn at their GLOBAL row, so ranks start from different rows of one stream and
        the job's sources do not depend on the device count; batch-shared (`c`) sources are the same draw
        on every rank."""
        adv = cls(optimizer=optimizer, source_dtype=source_dtype, pool_size=pool_size, batch_shared=shape == "c")
        lead = source_lead_shape(shape, batch * pool_size, positions)
        for i, s in enumerate(sites):
            rows = 1
            for n in lead:
                rows *= n
            off = 0 if adv.batch_shared else data_rank * rows
            u = rng.uniform(key, StepKey.stream(rng.PURPOSE_SOURCE_INIT, 0, 0, i), rows, s.C, off, device)
            ud = rng.uniform(key, StepKey.stream(rng.PURPOSE_SOURCE_INIT, 1, 0, i), rows, 1, off, device)
            adv.sources[s.name] = encode_sources(u.reshape(*lead, s.C), source_dtype)
            adv.delta[s.name] = encode_sources(ud.reshape(*lead, 1), source_dtype)
        return adv

    # -- views ---------------------------------------------------------------------------------
    def leaves(self) -> dict[str, Tensor]:
        """fp32 leaf tensors (requires_grad) for one ascent/forward: `{site, 'd:'+site}`."""
        out = {}
        for name, s in self.sources.items():
            out[name] = decode_sources(s).requires_grad_(True)
            out["d:" + name] = decode_sources(self.delta[name]).requires_grad_(True)
        return out

    @staticmethod
    def split(leaves: dict[str, Tensor]) -> tuple[dict[str, Tensor], dict[str, Tensor]]:
        src = {k: v for k, v in leaves.items() if not k.startswith("d:")}
        dlt = {k[2:]: v for k, v in leaves.items() if k.startswith("d:")}
        return src, dlt

    def select_particles(self, leaves: dict[str, Tensor], particle: Tensor) -> dict[str, Tensor]:
        """With a pool: gather one particle per batch row (`particle [B]` in `[0, pool_size)`)."""
        if self.pool_size == 1:
            return leaves
        B = particle.shape[0]
        idx = torch.arange(B, device=particle.device) * self.pool_size + particle
        return {k: v[idx] for k, v in leaves.items()}

    # -- ascent --------------------------------------------------------------------------------
    @torch.no_grad()
    def ascend(self, grads: dict[str, Tensor], lr: float, key: StepKey | None = None) -> None:
        """One projected ascent step on every leaf given `d loss / d leaf` (unscaled by the term's
        coefficient). Updates storage in place and advances the optimizer state."""
        self.n_updates += 1
        t = self.n_updates
        opt = self.optimizer
        for k, g in grads.items():
            is_delta = k.startswith("d:")
            store = self.delta if is_delta else self.sources
            name = k[2:] if is_delta else k
            cur = decode_sources(store[name])
            g = g.float()
            if isinstance(opt, AdamPGDConfig):
                sd = torch.float32 if self.source_dtype == "float32" else torch.bfloat16
                mu = self.state.get(k + "/mu", torch.zeros_like(cur)).float()
                nu = self.state.get(k + "/nu", torch.zeros_like(cur)).float()
                mu = opt.beta1 * mu + (1 - opt.beta1) * g
                nu = opt.beta2 * nu + (1 - opt.beta2) * g * g
                mhat = mu / (1 - opt.beta1**t)
                vhat = nu / (1 - opt.beta2**t)
                new = cur + lr * mhat / (vhat.sqrt() + opt.eps)
                self.state[k + "/mu"], self.state[k + "/nu"] = mu.to(sd), nu.to(sd)
            elif isinstance(opt, MomentumSgdPGDConfig):
                vel = self.state.get(k + "/vel", torch.zeros_like(cur)).float()
                vel = opt.momentum * vel + g
                new = cur + lr * vel
                self.state[k + "/vel"] = vel.to(velocity_dtype(self.source_dtype))
            else:
                new = cur + lr * g
            stream = StepKey.stream(rng.PURPOSE_ROUND, 0, 0, zlib.crc32(k.encode()) % (1 << 20))
            store[name] = encode_sources(new.clamp_(0, 1), self.source_dtype, key, stream)

    def _local_state(self) -> dict[str, Tensor]:
        out = {f"sources/{k}": v for k, v in self.sources.items()}
        out.update({f"delta/{k}": v for k, v in self.delta.items()})
        out.update({f"opt/{k}": v for k, v in self.state.items()})
        return out

    def gather_state(self, gather_rows) -> None:
        """Collective over the batch shards (every rank calls it before a save): per-row sources and their
        optimizer state are assembled into the global-batch layout with `gather_rows(t) -> cat over ranks on
        dim 0`; batch-shared sources are identical on every rank and stay as they are."""
        if self.batch_shared:
            return
        self._gathered = {k: gather_rows(v) for k, v in sorted(self._local_state().items())}

    def state_dict(self) -> dict[str, Tensor]:
        out = getattr(self, "_gathered", None) or self._local_state()
        self._gathered = None
        out = dict(out)
        out["n_updates"] = torch.tensor(self.n_updates, dtype=torch.int64)
        return out

    def load_state_dict(self, sd: dict[str, Tensor], data_rank: int = 0, data_world: int = 1) -> None:
        """Entries written in the global-batch layout are cut to this rank's rows (`data_rank` of
        `data_world` batch shards); a checkpoint of a different device count restores the same way."""
        def local(leaf: str, v: Tensor) -> Tensor:
            base = leaf.split("/")[0]
            ref = self.delta.get(base[2:]) if base.startswith("d:") else self.sources.get(base)
            if ref is None or v.dim() == 0 or ref.shape[0] == v.shape[0]:
                return v
            assert v.shape[0] == ref.shape[0] * data_world, \
                f"{leaf}: checkpoint has {v.shape[0]} rows, this run {ref.shape[0]} x {data_world} batch shards"
            return v[data_rank * ref.shape[0]:(data_rank + 1) * ref.shape[0]].contiguous()

        for k, v in sd.items():
            if k.startswith("sources/"):
                self.sources[k[8:]] = local(k[8:], v)
            elif k.startswith("delta/"):
                self.delta[k[6:]] = local("d:" + k[6:], v)
            elif k.startswith("opt/"):
                self.state[k[4:]] = local(k[4:], v)
            elif k == "n_updates":
                self.n_updates = int(v.item())


# ---- fresh PGD -----------------------------------------------------------------------------------


def fresh_source_rows(shape: str, batch: int, positions: int | None) -> int:
    """Rows of one rank's fresh sources once the leading axes are flattened (what `row_offset` counts in)."""
    rows = 1
    for n in source_lead_shape(shape, batch, positions):
        rows *= n
    return rows


def fresh_sources(sites: tuple[SiteSpec, ...], init: str, shape: str, batch: int, positions: int | None,
                  key: StepKey, term: int, device: torch.device | str, row_offset: int = 0) -> dict[str, Tensor]:
    """`batch` is this rank's share of the global batch. Per-row shapes draw their random initial values at the
    GLOBAL row (`row_offset` = this rank's first flattened row), so the sources of a job do not depend on how
    many ranks split its batch; batch-shared (`c`) sources are the same draw on every rank."""
    lead = source_lead_shape(shape, batch, positions)
    rows = fresh_source_rows(shape, batch, positions)
    off = 0 if shape == "c" else row_offset
    out = {}
    for i, s in enumerate(sites):
        for prefix, width, sub in (("", s.C, 0), ("d:", 1, 1)):
            if init == "random":
                v = rng.uniform(key, StepKey.stream(rng.PURPOSE_SOURCE_INIT, term, 2 + sub, i), rows, width, off, device)
            elif init == "ones":
                v = torch.ones(rows, width, device=device)
            else:
                v = torch.zeros(rows, width, device=device)
            out[prefix + s.name] = v.reshape(*lead, width).requires_grad_(True)
    return out


@torch.no_grad()
def sign_ascent_(leaves: dict[str, Tensor], grads: dict[str, Tensor], step_size: float) -> None:
    for k, v in leaves.items():
        v.add_(step_size * grads[k].sign()).clamp_(0, 1)
