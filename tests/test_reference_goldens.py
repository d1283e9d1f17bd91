"""Golden values frozen from the reference's earlier torch implementation, read as data from a checkout of the
reference beside this repository (skipped where there is none): a three-layer gated-MLP suffix with zeroed
attention, fixed component matrices, fixed causal importances and fixed adversary sources, so every loss is a
deterministic function of the file. This package's own model, masks and losses must reproduce the recorded numbers.

Also the tiny `LlamaSimpleMLP` logits recorded from the reference's torch model.
"""
import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from param_decomp_b200.config.experiments import TransformerArchConfig
from param_decomp_b200.core import losses, masking
from param_decomp_b200.core.components import ComponentStacks, prepare_compute_weights
from param_decomp_b200.models import transformer as tf

_root = Path(os.environ.get("PARAM_DECOMP_REFERENCE", Path(__file__).resolve().parents[2] / "reference"))
TARGETS = _root / "param_decomp" / "param_decomp" / "tests" / "targets"
pytestmark = pytest.mark.skipif(not (TARGETS / "equivalence" / "fixtures.npz").exists(),
                                reason="no checkout of the reference beside this repository")


def test_fixed_source_reconstruction_and_faithfulness_match_the_recorded_values():
    f = dict(np.load(TARGETS / "equivalence" / "fixtures.npz"))
    gold = json.loads((TARGETS / "equivalence" / "torch_reference.json").read_text())
    t = lambda k: torch.from_numpy(np.asarray(f[k])).float()  # noqa: E731
    L, n_tail, d, di = (int(f[f"_scalar_{k}"]) for k in ("N_DECOMP_LAYERS", "N_TAIL", "N_EMBD", "N_INTERMEDIATE"))
    B, T, C = int(f["_scalar_B"]), int(f["_scalar_T"]), int(f["_scalar_C"])
    resid = t("resid")

    # the residual stream enters as an embedding table with one row per position
    arch = TransformerArchConfig(family="glu_transformer", n_layer=L + n_tail, d_model=d, n_head=2, n_kv_head=1,
                                 d_ff=di, vocab_size=B * T, rms_eps=float(f["_scalar_EPS"]))
    w = tf.random_init_weights(arch, 0, torch.float32)
    w["embed.weight"] = resid.reshape(B * T, d)
    for i in range(L + n_tail):
        tail = i >= L
        pre = "tail_" if tail else ""
        j = i - L if tail else i
        w[f"layers.{i}.attn_norm.weight"] = t(f"{pre}ln1_{j}")
        w[f"layers.{i}.mlp_norm.weight"] = t(f"{pre}ln2_{j}")
        for p in ("q", "k", "v", "o"):  # zeroed attention: the block is `resid + mlp(norm(resid))`
            w[f"layers.{i}.self_attn.{p}_proj.weight"].zero_()
        for kind, key in (("gate", "Wg"), ("up", "Wu"), ("down", "Wd")):
            w[f"layers.{i}.mlp.{kind}_proj.weight"] = t(f"{pre}{key}_{j}")
    w["final_norm.weight"] = t("norm")
    w["lm_head.weight"] = t("lm_head")
    # (the embedding table has B*T rows, the head keeps the fixture's own 48-entry vocabulary)
    names = {(i, k): tf.site_name("glu_transformer", i, k) for i in range(L) for k in ("gate", "up", "down")}
    model = tf.TransformerDecomposedModel(arch, w, {n: C for n in names.values()}, backend="eager_torch", attention="xla")
    stacks = ComponentStacks(model.sites)
    for (i, k), n in names.items():
        stacks.set_site(n, t(f"V{k[0]}_{i}"), t(f"U{k[0]}_{i}"))

    batch = tf.LMBatch(torch.arange(B * T).reshape(B, T))
    with torch.no_grad():
        clean = model.clean_forward(batch)
        weights = prepare_compute_weights(stacks, torch.float32)
        ci = {n: t(f"ci_lower_{k}")[:, :, i] for (i, k), n in names.items()}
        src = {n: t(f"ppgd_source_{k}")[:, :, i, :-1] for (i, k), n in names.items()}   # [1, T, C]
        dlt = {n: t(f"ppgd_source_{k}")[:, :, i, -1:] for (i, k), n in names.items()}   # [1, T, 1]
        masked = model.masked_forward(weights, batch, masking.source_masks(ci, src, dlt), clean=clean)
        ppgd = float(model.recon_loss(clean, masked))
    assert ppgd == pytest.approx(gold["ppgd"], rel=2e-4, abs=1e-5)

    targets = {n: w[n + ".weight"] for n in names.values()}
    paper = float(losses.faithfulness_loss(stacks, targets, relative=False).detach())
    assert paper == pytest.approx(gold["faith"], rel=2e-4), (paper, gold["faith"])


def test_llama_simple_mlp_logits_match_the_recorded_torch_model(tmp_path):
    f = np.load(TARGETS / "simple_mlp_equivalence" / "tiny_fixture.npz")
    cfg = json.loads(str(f["config_json"]))
    from safetensors.torch import save_file

    from param_decomp_b200.models import loaders

    entry = tmp_path / "pretrain_cache" / "spd-t-00000000"
    entry.mkdir(parents=True)
    import yaml

    (entry / "model_config.yaml").write_text(yaml.safe_dump(cfg))
    save_file({k[len("weights."):]: torch.from_numpy(np.asarray(f[k])).contiguous() for k in f.files if k.startswith("weights.")},
              str(entry / "model_step_1.safetensors"))
    arch, weights = loaders.load_simple_mlp_cache(entry, torch.float32, "cpu")
    model = tf.TransformerDecomposedModel(arch, weights, {}, backend="eager_torch", attention="xla")
    idx = torch.from_numpy(np.asarray(f["idx"]))
    with torch.no_grad():
        out = model.clean_forward(tf.LMBatch(idx))
        logits = model.logits(out.output)
    want = torch.from_numpy(np.asarray(f["logits"]))
    assert torch.allclose(logits, want, atol=2e-4, rtol=1e-4), float((logits - want).abs().max())


def _snapshot_from_fixture(npz, tmp_path, extra_config: dict) -> Path:
    from safetensors.torch import save_file

    snap = tmp_path / "snap"
    snap.mkdir()
    cfg = json.loads(str(npz["config_json"]))
    cfg.update(extra_config)
    (snap / "config.json").write_text(json.dumps(cfg))
    save_file({k[4:]: torch.from_numpy(np.asarray(npz[k])).contiguous() for k in npz.files if k.startswith("sd::")},
              str(snap / "model.safetensors"))
    return snap


@pytest.mark.parametrize("fixture, extra, model_kind", [
    ("qwen3_hf_parity/qwen3_tiny_hf_fixtures.npz", {"model_type": "qwen3"}, "dense"),
    ("qwen36_moe_hf_parity/qwen36_moe_tiny_hf_fixtures.npz", {}, "hybrid"),
])
def test_recorded_huggingface_logits_and_residual_streams(tmp_path, fixture, extra, model_kind):
    """Weights, tokens, every block's residual stream and the logits recorded from the HuggingFace implementations
    (tiny Qwen3; tiny Qwen3.6-style hybrid with gated DeltaNet, gated attention and routed + shared experts): the
    snapshot loader and the target models reproduce them."""
    from param_decomp_b200.models import loaders

    f = np.load(TARGETS / fixture)
    arch, weights = loaders.load_hf_snapshot(_snapshot_from_fixture(f, tmp_path, extra), torch.float32, "cpu")
    if model_kind == "hybrid":
        from param_decomp_b200.models.qwen35 import Qwen35DecomposedModel as Model
    else:
        Model = tf.TransformerDecomposedModel
    model = Model(arch, weights, {}, backend="eager_torch", attention="xla")
    tokens = torch.from_numpy(np.asarray(f["tokens"]))
    keys = tuple(f"resid.{i}" for i in range(arch.n_layer + 1))
    with torch.no_grad():
        out = model.clean_forward(tf.LMBatch(tokens), capture=keys)
        logits = model.logits(out.output)
    for i in range(arch.n_layer + 1):
        want = torch.from_numpy(np.asarray(f[f"resid::{i}"]))
        got = out.captures[f"resid.{i}"]
        assert torch.allclose(got, want, atol=5e-4, rtol=1e-3), (i, float((got - want).abs().max()))
    want = torch.from_numpy(np.asarray(f["logits"]))
    assert torch.allclose(logits, want, atol=5e-4, rtol=1e-3), float((logits - want).abs().max())


def test_gqa_suffix_with_scaled_rope_matches_recorded_clean_and_masked_logits():
    """Five Llama blocks (grouped-query attention, Llama-3.1 rescaled RoPE) fed a recorded residual stream, gated-MLP
    sites of the first three decomposed with recorded `V`, `U`, component masks and delta masks: recorded clean
    logits, every site's input, every weight delta and the all-sites masked logits."""
    from param_decomp_b200.config.experiments import Llama3RopeScalingConfig
    from param_decomp_b200.core.masking import SiteMask

    f = dict(np.load(TARGETS / "stacked_parity" / "stacked_fixtures.npz"))
    t = lambda k: torch.from_numpy(np.asarray(f[k])).float()  # noqa: E731
    first, last, C = int(f["_scalar_FIRST_LAYER"]), int(f["_scalar_LAST_LAYER"]), int(f["_scalar_C"])
    B, T, n_layer_total = int(f["_scalar_B"]), int(f["_scalar_T"]), 8
    resid = t("resid")
    d = resid.shape[-1]
    arch = TransformerArchConfig(
        family="glu_transformer", n_layer=n_layer_total - first, d_model=d, n_head=4, n_kv_head=2, d_ff=64,
        vocab_size=B * T, rms_eps=1e-5, rope_theta=500000.0, max_seq_len=512,
        rope_scaling=Llama3RopeScalingConfig(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                             original_max_position_embeddings=128))
    w = tf.random_init_weights(arch, 0, torch.float32)
    w["embed.weight"] = resid.reshape(B * T, d)
    for i in range(arch.n_layer):
        src = f"tgt::layers.{i + first}."
        w[f"layers.{i}.attn_norm.weight"], w[f"layers.{i}.mlp_norm.weight"] = t(src + "ln1"), t(src + "ln2")
        for ours, theirs in (("q", "wq"), ("k", "wk"), ("v", "wv"), ("o", "wo")):
            w[f"layers.{i}.self_attn.{ours}_proj.weight"] = t(src + theirs)
        for ours, theirs in (("gate", "Wg"), ("up", "Wu"), ("down", "Wd")):
            w[f"layers.{i}.mlp.{ours}_proj.weight"] = t(src + theirs)
    w["final_norm.weight"], w["lm_head.weight"] = t("tgt::norm"), t("tgt::lm_head")

    theirs_of = {tf.site_name("glu_transformer", i - first, k): f"layers.{i}.mlp.{k}_proj"
                 for i in range(first, last + 1) for k in ("gate", "up", "down")}
    model = tf.TransformerDecomposedModel(arch, w, {n: C for n in theirs_of}, backend="eager_torch", attention="xla")
    stacks = ComponentStacks(model.sites)
    for ours, theirs in theirs_of.items():
        stacks.set_site(ours, t(f"vu::V::{theirs}"), t(f"vu::U::{theirs}"))
    batch = tf.LMBatch(torch.arange(B * T).reshape(B, T))
    close = lambda a, b: torch.allclose(a, b, rtol=1e-4, atol=2e-5)  # noqa: E731
    with torch.no_grad():
        clean = model.clean_forward(batch)
        assert close(model.logits(clean.output), t("out::clean"))
        for ours, theirs in theirs_of.items():
            layer = int(ours.split(".")[1])
            tap = clean.taps[f"mlp_hidden.{layer}" if ours.endswith("down_proj") else f"mlp_in.{layer}"]
            assert close(tap, t(f"out::site_input::{theirs}")), ours
            V, U = stacks.site(ours)
            assert close(losses.weight_delta(w[ours + ".weight"], V, U), t(f"out::wd::{theirs}")), ours
        masks = {ours: SiteMask(mask=t(f"mask::{theirs}"), delta=t(f"delta_mask::{theirs}").unsqueeze(-1))
                 for ours, theirs in theirs_of.items()}
        weights = prepare_compute_weights(stacks, torch.float32)
        masked = model.masked_forward(weights, batch, masks, clean=clean)
        assert close(model.logits(masked.output), t("out::masked_all"))


def test_dense_placement_presets_match_the_recorded_tables():
    """Every dense preset on every recorded mesh: the resolved rules of the component roles, the activations and the
    target rows, the stack padding of the recorded site groups, and a refusal wherever the preset's axis vocabulary
    is not the mesh's."""
    from param_decomp_b200.parallel import placement as pl

    gold = json.loads((TARGETS.parent / "core" / "placement_goldens.json").read_text())
    presets = {"ddp": "ddp", "owner": "owner", "zero1": "zero1", "owner_replicated_resident": "owner-replicated-resident",
               "zero1_replicated_resident": "zero1-replicated-resident"}

    def norm(rule) -> dict:
        return {k: tuple(v) for k, v in rule.items() if tuple(v)}

    checked = 0
    for key, entry in gold.items():
        head, mesh_name, _sites = (key.split("|") + ["", ""])[:3]
        if not head.startswith("preset_") or head[7:] not in presets:
            continue
        mesh = {m.rstrip("0123456789"): int(m[len(m.rstrip("0123456789")):]) for m in mesh_name.split("_")}
        name = presets[head[7:]]
        if "refused" in entry:
            with pytest.raises(AssertionError):
                pl.from_config(name, mesh)
            checked += 1
            continue
        rules = pl.from_config(name, mesh)
        want = entry["rules"]
        for role in ("optimizer_state", "compute_weights", "faithfulness_weights", "faithfulness_deltas", "operands",
                     "ns_compute"):
            assert norm(getattr(rules.components, role)) == norm(want["components"][role]["rule"]), (key, role)
        assert norm(rules.activations_external) == norm(want["activations"]["external"]["rule"]), key
        assert norm(rules.activations_component) == norm(want["activations"]["component"]["rule"]), key
        t = want["target"]
        for ours, theirs in (("embedding_persist", t["embedding"]["persist"]), ("column_persist", t["column"]["persist"]),
                             ("row_persist", t["row"]["persist"]), ("column_operand", t["column"]["operand"]),
                             ("row_operand", t["row"]["operand"]), ("output_persist", t["output"]["persist"]),
                             ("intermediate", t["intermediate"])):
            assert norm(getattr(rules.target, ours)) == norm(theirs["rule"]), (key, ours)
        assert rules.ci_fn_preset == want["ci_fn"]
        multiple = pl.stack_multiple(rules, mesh)
        for group, census in want["components"]["group_census"].items():
            assert (-census["stack_len"]) % multiple == census["stack_pad"], (key, group)
        checked += 1
    assert checked >= 25
