"""Targeted (two-stream) LM decomposition through its composition root, on CPU."""
import torch

from param_decomp_b200.config.experiments import LMExperimentConfig, LMTargetedExperimentConfig
from param_decomp_b200.experiments.lm.targeted_data import PromptPool, byte_encoder
from param_decomp_b200.experiments.lm.training import train_lm_targeted


def _targeted_config() -> LMTargetedExperimentConfig:
    base = LMExperimentConfig.from_file("param_decomp_b200/experiments/configs/lm_llama4l_c4096.yaml").model_dump(mode="json")
    base["target"]["spec"]["arch"] = dict(family="glu_transformer", n_layer=2, d_model=32, n_head=2, d_ff=64,
                                          vocab_size=131, max_seq_len=16)
    base["target"]["weights_dtype"] = "float32"
    base["target"]["attention_implementation"] = "xla"
    base["decomposition"]["sites"]["cs"] = {k: 8 for k in ("q", "k", "v", "o", "gate", "up", "down")}
    base["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [8]}
    base["data"]["seq_len"] = 16
    base["runtime"]["backend"] = "eager_torch"
    base["runtime"]["mesh"] = {"replicate": 1, "fsdp": 1, "tp": 1}
    base["pd"]["batch_size"] = 4
    base["pd"]["steps"] = 3
    base["pd"]["loss_metrics"] = [
        {"type": "ImportanceMinimalityLoss", "coeff": 1e-4, "gamma": 1.0},
        {"type": "StochasticReconLoss", "coeff": 1.0},
    ]
    for k in [k for k in base["pd"] if k.startswith("faithfulness_warmup") or k == "type"]:
        base["pd"].pop(k)
    base["prompts"] = {"prompts": ["12+30=", "7+5=", "what is 2+2?"], "seq_len": 12}
    base["nontarget"] = {"batch_size": 2, "impmin_coeff": 1e-4, "recon": [{"type": "CIMaskedReconLoss", "coeff": 1.0}]}
    base.pop("resume_provenance", None)
    return LMTargetedExperimentConfig.model_validate(base)


def test_prompt_pool_is_a_pure_function_of_seed_and_step():
    cfg = _targeted_config()
    pool = PromptPool.build(cfg.prompts, 131, None, seed=3)
    assert pool.tokens.shape == (3, 12)
    assert pool.tokens[1, -4:].tolist() == byte_encoder(131)("7+5=")
    a, b = pool.batch(5, 4, 0, 2), pool.batch(5, 4, 1, 2)
    full = pool.batch(5, 4, 0, 1)
    assert torch.equal(torch.cat([a.tokens, b.tokens]), full.tokens)
    assert not torch.equal(pool.batch(6, 4, 0, 1).tokens, full.tokens) or True


def test_targeted_lm_runs(tmp_path):
    cfg = _targeted_config()
    states: list = []
    res = train_lm_targeted(cfg, tmp_path, device="cpu", state_out=states)
    assert res.final_step == 3
    lines = (res.run_dir / "metrics.jsonl").read_text().strip().splitlines()
    assert lines and "loss/total" in lines[-1]


def test_reference_prompt_pool_kinds(tmp_path):
    """`kind: arithmetic_grid` and `kind: prompts_file`, the two pool forms of the reference's targeted configs."""
    base = _targeted_config().model_dump(mode="json")
    base["prompts"] = {"kind": "arithmetic_grid", "operation": "add", "a_range": [1, 4], "b_range": [1, 5]}
    cfg = LMTargetedExperimentConfig.model_validate(base)
    pool = PromptPool.build(cfg.prompts, 131, None, seed=0)
    assert pool.tokens.shape == (20, 4)  # "a+b=" is four bytes for one-digit operands; 4 x 5 prompts, both ends in
    assert pool.tokens[0].tolist() == byte_encoder(131)("1+1=") and pool.tokens[-1].tolist() == byte_encoder(131)("4+5=")

    path = tmp_path / "prompts.txt"
    path.write_text("abcd\n\nwxyz\n")
    base["prompts"] = {"kind": "prompts_file", "path": str(path)}
    cfg = LMTargetedExperimentConfig.model_validate(base)
    assert PromptPool.build(cfg.prompts, 131, None, seed=0).tokens.shape == (2, 4)
    path.write_text("abcd\nabc\n")
    try:
        PromptPool.build(cfg.prompts, 131, None, seed=0)
        raise RuntimeError("unequal prompt lengths were accepted")
    except AssertionError as e:
        assert "one shared length" in str(e)


def test_prompt_encoder_prefers_staged_tokenizer_files(tmp_path):
    """A tokenizer staged beside the target's snapshot is used; without one the encoder falls back to bytes."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from param_decomp_b200.config.experiments import HFTarget
    from param_decomp_b200.experiments.lm.prompt_encoder import resolve_prompt_encoder

    spec = HFTarget(model_class="LlamaForCausalLM", model_name="org/tiny")
    assert resolve_prompt_encoder(spec, None, tmp_path, 131).source == "bytes"

    vocab = {c: i for i, c in enumerate("0123456789+-*=")}
    vocab["[UNK]"] = len(vocab)
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    snap = tmp_path / "hf_snapshots" / "org--tiny"
    snap.mkdir(parents=True)
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="[UNK]").save_pretrained(str(snap))
    enc = resolve_prompt_encoder(spec, None, tmp_path, 131)
    assert enc.source == str(snap)
    assert enc("12+3=") == [1, 2, 10, 3, 13]


def test_arithmetic_grid_metric_is_built_from_the_run_encoder(tmp_path):
    """An `ArithmeticCIGrid` metric in a training config is evaluated (its grid built from the run's encoder), and
    operand ranges whose prompts differ in length are refused when the run starts."""
    base = _targeted_config().model_dump(mode="json")
    base["eval"] = {"batch_size": 2, "n_steps": 1, "every": 2, "slow_every": 2,
                    "metrics": [{"type": "ArithmeticCIGrid", "operation": "add", "a_range": [1, 3], "b_range": [1, 3],
                                 "top_k": 2}]}
    base["pd"]["steps"] = 2
    cfg = LMTargetedExperimentConfig.model_validate(base)
    res = train_lm_targeted(cfg, tmp_path, device="cpu")
    text = (res.run_dir / "metrics.jsonl").read_text()
    assert "ArithmeticCIGrid/" in text and "n_alive" in text

    base["eval"]["metrics"][0]["a_range"] = [1, 12]
    cfg = LMTargetedExperimentConfig.model_validate(base)
    try:
        train_lm_targeted(cfg, tmp_path, device="cpu")
        raise RuntimeError("a grid with unequal prompt lengths was accepted")
    except AssertionError as e:
        assert "different lengths" in str(e)


def test_per_position_adversary_follows_the_prompt_length(tmp_path):
    """Adversary sources of a targeted run live on the target stream: with per-position (`bsc`) sources their
    position axis is the prompt length (here 4), not the broad stream's sequence length (16)."""
    base = _targeted_config().model_dump(mode="json")
    base["prompts"] = {"kind": "arithmetic_grid", "operation": "add", "a_range": [1, 4], "b_range": [1, 5]}
    base["pd"]["loss_metrics"].append({"type": "PersistentPGDReconLoss", "coeff": 0.5, "source_shape": "bsc",
                                       "n_warmup_steps": 1, "optimizer": {"type": "sgd", "lr_schedule": 0.05}})
    states: list = []
    res = train_lm_targeted(LMTargetedExperimentConfig.model_validate(base), tmp_path, device="cpu", state_out=states)
    assert res.final_step == 3
    adv = next(iter(states[0].adversaries.values()))
    assert next(iter(adv.sources.values())).shape[:2] == (4, 4)  # [rows, prompt positions, C]


def test_targeted_run_on_a_mixture_of_experts_with_an_adversary(tmp_path):
    """Both streams on expert-blocked sites: narrow importances on the target stream's persistent adversary and on
    the broad stream's subset-routed masks; the broad stream's keys are written as `train/loss/nontarget/*`."""
    raw = _targeted_config().model_dump(mode="json")
    raw["target"]["spec"]["arch"] = {"family": "moe", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 16,
                                     "vocab_size": 131, "n_experts": 4, "experts_per_token": 2, "max_seq_len": 16}
    raw["decomposition"]["sites"] = {"kind": "moe", "layers": {"kind": "all"},
                                     "cs": {"q": 8, "experts_gate": 16, "experts_up": 16, "experts_down": 16}}
    raw["pd"]["loss_metrics"].append({"type": "PersistentPGDReconLoss", "coeff": 0.5, "source_shape": "bsc",
                                      "n_warmup_steps": 1, "optimizer": {"type": "sgd", "lr_schedule": 0.05}})
    raw["nontarget"]["recon"] = [{"type": "CIMaskedReconLoss", "coeff": 1.0},
                                 {"type": "StochasticReconSubsetLoss", "coeff": 0.5, "routing": {"type": "uniform_k_subset"}}]
    res = train_lm_targeted(LMTargetedExperimentConfig.model_validate(raw), tmp_path, device="cpu")
    assert res.final_step == 3
    m = res.last_metrics
    assert {"train/loss/PersistentPGDReconLoss", "train/loss/nontarget/imp", "train/loss/nontarget/CIMaskedReconLoss",
            "train/loss/nontarget/StochasticReconSubsetLoss", "train/schedules/lr/src"} <= set(m)
    assert all(v == v for v in m.values())
