"""Toy Model of Superposition target.

`x [B, F] -> h = x W1^T (W1 [H, F], no bias) -> optional frozen hidden layers h <- h W_i^T
-> out = relu(h W2^T + b2)`, with the target's `W2 = W1^T` tied. The decomposition is untied: two
independent sites `linear1 [F -> H]` and `linear2 [H -> F]` (+ `hidden_layers.{i} [H -> H]`);
`b2` stays frozen.

Parity: param_decomp/targets/tms.py:137-143 (model), :214-234 (sites), :311-388 (forwards and
`tms_mse`), :584-609 (sparse-feature sampler), :629-682 (in-process pretraining with
`mean((|x| - out)^2)`), :688-751 (identity-CI ground truth).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.config.experiments import TMSTargetConfig
from param_decomp_b200.core.components import ComputeWeights, SiteSpec
from param_decomp_b200.core.decomposed_linear import site_forward
from param_decomp_b200.core.masking import Masks
from param_decomp_b200.core.model import ForwardResult

_N_ACTIVE = {"exactly_one_active": 1, "exactly_two_active": 2, "exactly_three_active": 3,
             "exactly_four_active": 4, "exactly_five_active": 5}


def sample_sparse_features(batch: int, n_features: int, p: float, kind: str, generator: torch.Generator,
                           device: torch.device | str = "cpu", low: float = 0.0) -> Tensor:
    """`at_least_zero_active`: each feature on w.p. `p`, value U(low, 1). `exactly_n_active`: a
    uniformly random n-subset is on. `low=-1` gives the ResidualMLP value range."""
    vals = torch.rand(batch, n_features, generator=generator) * (1 - low) + low
    if kind == "at_least_zero_active":
        on = torch.rand(batch, n_features, generator=generator) < p
    else:
        n = _N_ACTIVE[kind]
        order = torch.rand(batch, n_features, generator=generator).argsort(dim=-1)
        on = order < n
    return (vals * on).to(device)


@dataclass
class TMSParams:
    W1: Tensor  # [H, F]
    b2: Tensor  # [F]
    hidden: list[Tensor]  # each [H, H]


def init_tms(cfg: TMSTargetConfig, generator: torch.Generator) -> TMSParams:
    F_, H = cfg.n_features, cfg.n_hidden
    W1 = torch.empty(H, F_)
    bound = 1.0 / F_**0.5
    W1.copy_((torch.rand(H, F_, generator=generator) * 2 - 1) * bound)
    if cfg.init_bias_to_zero:
        b2 = torch.zeros(F_)
    else:
        b2 = (torch.rand(F_, generator=generator) * 2 - 1) / H**0.5
    hidden = []
    for _ in range(cfg.n_hidden_layers):
        if cfg.hidden_layer_init == "identity":
            hidden.append(torch.eye(H))
        else:
            hidden.append((torch.rand(H, H, generator=generator) * 2 - 1) / H**0.5)
    return TMSParams(W1, b2, hidden)


def tms_forward(p: TMSParams, x: Tensor) -> Tensor:
    h = x @ p.W1.T
    for Wh in p.hidden:
        h = h @ Wh.T
    return F.relu(h @ p.W1 + p.b2)


def pretrain_tms(cfg: TMSTargetConfig, feature_probability: float, kind: str,
                 device: torch.device | str = "cpu") -> TMSParams:
    """AdamW (wd 0) on `(W1, b2)` only; hidden layers stay frozen; loss `mean((|x| - out)^2)`."""
    g = torch.Generator().manual_seed(cfg.pretrain.seed)
    p = init_tms(cfg, g)
    W1 = p.W1.to(device).requires_grad_(True)
    b2 = p.b2.to(device).requires_grad_(True)
    hidden = [h.to(device) for h in p.hidden]
    opt = torch.optim.AdamW([W1, b2], lr=cfg.pretrain.lr, weight_decay=0.0)
    data_g = torch.Generator().manual_seed(cfg.pretrain.seed + 17)
    for _ in range(cfg.pretrain.steps):
        x = sample_sparse_features(cfg.pretrain.batch_size, cfg.n_features, feature_probability, kind, data_g, device)
        out = tms_forward(TMSParams(W1, b2, hidden), x)
        loss = (x.abs() - out).pow(2).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
    return TMSParams(W1.detach(), b2.detach(), hidden)


class TMSDecomposedModel:
    has_position_axis = False
    compute_dtype = torch.float32

    def __init__(self, params: TMSParams, site_cs: dict[str, int]) -> None:
        self.params = params
        H, F_ = params.W1.shape
        specs = []
        self._W: dict[str, Tensor] = {}
        order = ["linear1", *[f"hidden_layers.{i}" for i in range(len(params.hidden))], "linear2"]
        for name in order:
            if name not in site_cs:
                continue
            if name == "linear1":
                d_in, d_out, W = F_, H, params.W1
            elif name == "linear2":
                d_in, d_out, W = H, F_, params.W1.T.contiguous()
            else:
                d_in, d_out, W = H, H, params.hidden[int(name.split(".")[1])]
            specs.append(SiteSpec(name, d_in, d_out, site_cs[name], group=name))
            self._W[name] = W
        unknown = set(site_cs) - set(order)
        assert not unknown, f"unknown TMS sites {unknown}"
        self.sites = tuple(specs)
        self.n_features, self.n_hidden = F_, H

    # -- protocol ---------------------------------------------------------------------------------
    def batch_size(self, batch: Tensor) -> int:
        return batch.shape[0]

    def tap_for_site(self, site: str) -> str:
        return site

    def target_weight(self, site: str) -> Tensor:
        return self._W[site]

    def _layers(self) -> list[tuple[str, Tensor]]:
        p = self.params
        return [("linear1", p.W1), *[(f"hidden_layers.{i}", w) for i, w in enumerate(p.hidden)],
                ("linear2", p.W1.T)]

    def clean_forward(self, batch: Tensor, capture: tuple[str, ...] = ()) -> ForwardResult:
        h = batch
        taps = {}
        for name, W in self._layers():
            taps[name] = h
            h = F.linear(h, W)
        out = F.relu(h + self.params.b2)
        return ForwardResult(output=out, taps=taps)

    def masked_forward(self, weights: ComputeWeights, batch: Tensor, masks: Masks,
                       capture: tuple[str, ...] = (), clean: ForwardResult | None = None) -> ForwardResult:
        h = batch
        for name, W in self._layers():
            if name in masks and name in weights.V:
                V, U = weights.site(name)
                h = site_forward(h, V, U, W, masks[name])
            else:
                h = F.linear(h, W)
        return ForwardResult(output=F.relu(h + self.params.b2))

    def recon_loss(self, clean: ForwardResult, masked: ForwardResult) -> Tensor:
        """`tms_mse`: squared error summed over features, mean over the batch."""
        return (masked.output - clean.output).pow(2).sum(-1).mean()

    def to(self, device) -> "TMSDecomposedModel":
        p = self.params
        self.params = TMSParams(p.W1.to(device), p.b2.to(device), [h.to(device) for h in p.hidden])
        self._W = {k: v.to(device) for k, v in self._W.items()}
        return self
