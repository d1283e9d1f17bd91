"""Residual-MLP toy target.

`resid = x W_E;  for each layer: hidden = act(resid W_in^T (+ b_in)); resid += hidden W_out^T
(+ b_out);  out = resid W_U`. `W_E [F, d_embed]` is a fixed random matrix with unit-norm rows (or
the identity), `W_U = W_E^T`. Decomposed sites per layer: `layers.{i}.mlp_in [d_embed -> d_mlp]`
(its CI reads the clean residual) and `layers.{i}.mlp_out [d_mlp -> d_embed]` (reads the clean
hidden activations).

Parity: param_decomp/targets/resid_mlp.py:102-156 (config), :228-288 (forward), :411-419 (recon
MSE), :421-560 (pretraining on `act(c*x) + x` read-off or `|c*x|` labels), :643-662 (data:
features on w.p. p, values U(-1, 1)), :733-803 (decomposed model).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.config.experiments import ResidMLPTargetConfig
from param_decomp_b200.core.components import ComputeWeights, SiteSpec
from param_decomp_b200.core.decomposed_linear import site_forward
from param_decomp_b200.core.masking import Masks
from param_decomp_b200.core.model import ForwardResult
from param_decomp_b200.models.tms import sample_sparse_features


@dataclass
class ResidMLPParams:
    W_E: Tensor  # [F, d_embed]
    W_in: list[Tensor]  # [d_mlp, d_embed]
    W_out: list[Tensor]  # [d_embed, d_mlp]
    b_in: list[Tensor | None]
    b_out: list[Tensor | None]
    act: str

    @property
    def W_U(self) -> Tensor:
        return self.W_E.T


def _act(name: str):
    return F.gelu if name == "gelu" else F.relu


def init_resid_mlp(cfg: ResidMLPTargetConfig, generator: torch.Generator) -> ResidMLPParams:
    if cfg.fixed_identity_embedding:
        W_E = torch.eye(cfg.n_features)
    else:
        W_E = torch.randn(cfg.n_features, cfg.d_embed, generator=generator)
        W_E = W_E / W_E.norm(dim=-1, keepdim=True)
    W_in, W_out, b_in, b_out = [], [], [], []
    for _ in range(cfg.n_layers):
        W_in.append(torch.randn(cfg.d_mlp, cfg.d_embed, generator=generator) / cfg.d_embed**0.5)
        W_out.append(torch.randn(cfg.d_embed, cfg.d_mlp, generator=generator) / cfg.d_mlp**0.5)
        b_in.append(torch.zeros(cfg.d_mlp) if cfg.in_bias else None)
        b_out.append(torch.zeros(cfg.d_embed) if cfg.out_bias else None)
    return ResidMLPParams(W_E, W_in, W_out, b_in, b_out, cfg.act_fn_name)


def resid_mlp_forward(p: ResidMLPParams, x: Tensor, return_resid: bool = False) -> Tensor:
    act = _act(p.act)
    resid = x @ p.W_E
    for Wi, Wo, bi, bo in zip(p.W_in, p.W_out, p.b_in, p.b_out):
        hidden = act(F.linear(resid, Wi, bi))
        resid = resid + F.linear(hidden, Wo, bo)
    return resid if return_resid else resid @ p.W_U


def pretrain_resid_mlp(cfg: ResidMLPTargetConfig, feature_probability: float, kind: str,
                       device: torch.device | str = "cpu") -> ResidMLPParams:
    pc = cfg.pretrain
    g = torch.Generator().manual_seed(pc.seed)
    p = init_resid_mlp(cfg, g)
    act = _act(cfg.act_fn_name)
    coeffs = torch.ones(cfg.n_features) if pc.use_trivial_label_coeffs else torch.rand(cfg.n_features, generator=g) + 1
    coeffs = coeffs.to(device)
    importance = (pc.importance_val ** torch.arange(cfg.n_features, dtype=torch.float32)).to(device)
    W_E = p.W_E.to(device)
    train = []
    for lst in (p.W_in, p.W_out):
        for i, w in enumerate(lst):
            lst[i] = w.to(device).requires_grad_(True)
            train.append(lst[i])
    for lst in (p.b_in, p.b_out):
        for i, b in enumerate(lst):
            if b is not None:
                lst[i] = b.to(device).requires_grad_(True)
                train.append(lst[i])
    cur = ResidMLPParams(W_E, p.W_in, p.W_out, p.b_in, p.b_out, p.act)
    opt = torch.optim.AdamW(train, lr=pc.lr, weight_decay=0.0)
    data_g = torch.Generator().manual_seed(pc.seed + 17)
    for _ in range(pc.steps):
        x = sample_sparse_features(pc.batch_size, cfg.n_features, feature_probability, kind, data_g, device, low=-1.0)
        labels = act(coeffs * x) + x if pc.label_type == "act_plus_resid" else (coeffs * x).abs()
        if pc.loss_type == "readoff":
            pred = resid_mlp_forward(cur, x)
            loss = ((pred - labels).pow(2) * importance).mean()
        else:
            pred = resid_mlp_forward(cur, x, return_resid=True)
            loss = (pred - labels @ W_E).pow(2).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
    return ResidMLPParams(W_E, [w.detach() for w in p.W_in], [w.detach() for w in p.W_out],
                          [None if b is None else b.detach() for b in p.b_in],
                          [None if b is None else b.detach() for b in p.b_out], p.act)


class ResidMLPDecomposedModel:
    has_position_axis = False
    compute_dtype = torch.float32

    def __init__(self, params: ResidMLPParams, site_cs: dict[str, int]) -> None:
        self.params = params
        specs = []
        self._W: dict[str, Tensor] = {}
        for i, (Wi, Wo) in enumerate(zip(params.W_in, params.W_out)):
            for suffix, W in (("mlp_in", Wi), ("mlp_out", Wo)):
                name = f"layers.{i}.{suffix}"
                if name in site_cs:
                    specs.append(SiteSpec(name, W.shape[1], W.shape[0], site_cs[name], group=suffix))
                    self._W[name] = W
        unknown = set(site_cs) - set(self._W)
        assert not unknown, f"unknown ResidMLP sites {unknown}"
        self.sites = tuple(specs)

    def batch_size(self, batch: Tensor) -> int:
        return batch.shape[0]

    def tap_for_site(self, site: str) -> str:
        return site

    def target_weight(self, site: str) -> Tensor:
        return self._W[site]

    def clean_forward(self, batch: Tensor, capture: tuple[str, ...] = ()) -> ForwardResult:
        p, act = self.params, _act(self.params.act)
        resid = batch @ p.W_E
        taps = {}
        for i, (Wi, Wo, bi, bo) in enumerate(zip(p.W_in, p.W_out, p.b_in, p.b_out)):
            taps[f"layers.{i}.mlp_in"] = resid
            hidden = act(F.linear(resid, Wi, bi))
            taps[f"layers.{i}.mlp_out"] = hidden
            resid = resid + F.linear(hidden, Wo, bo)
        return ForwardResult(output=resid @ p.W_U, taps=taps)

    def masked_forward(self, weights: ComputeWeights, batch: Tensor, masks: Masks,
                       capture: tuple[str, ...] = (), clean: ForwardResult | None = None) -> ForwardResult:
        p, act = self.params, _act(self.params.act)
        resid = batch @ p.W_E

        def lin(name: str, x: Tensor, W: Tensor, b: Tensor | None) -> Tensor:
            if name in masks and name in weights.V:
                V, U = weights.site(name)
                return site_forward(x, V, U, W, masks[name], bias=b)
            return F.linear(x, W, b)

        for i, (Wi, Wo, bi, bo) in enumerate(zip(p.W_in, p.W_out, p.b_in, p.b_out)):
            hidden = act(lin(f"layers.{i}.mlp_in", resid, Wi, bi))
            resid = resid + lin(f"layers.{i}.mlp_out", hidden, Wo, bo)
        return ForwardResult(output=resid @ p.W_U)

    def recon_loss(self, clean: ForwardResult, masked: ForwardResult) -> Tensor:
        return (masked.output - clean.output).pow(2).sum(-1).mean()

    def to(self, device) -> "ResidMLPDecomposedModel":
        p = self.params
        mv = lambda lst: [None if t is None else t.to(device) for t in lst]  # noqa: E731
        self.params = ResidMLPParams(p.W_E.to(device), mv(p.W_in), mv(p.W_out), mv(p.b_in), mv(p.b_out), p.act)
        self._W = {k: v.to(device) for k, v in self._W.items()}
        return self
