"""Text-to-token encoder for prompts built at startup (targeted prompt pools, the arithmetic probe).

Every rank builds the same prompts from the same encoder, so the result needs no coordination. The encoder is
found OFFLINE, in this order:

1. tokenizer files beside the target's weights (a staged HuggingFace snapshot, or a pretrain cache entry),
2. `<data_root>/tokenizers/<name>` for the tokenizer the training dataset's metadata names,
3. a byte-level encoder (UTF-8 bytes folded into the vocabulary), with a warning: random-init and synthetic
   targets have no tokenizer, and a byte per digit is the per-digit behaviour of the Qwen number tokenizers.

Parity: param_decomp/experiments/lm/arithmetic_probe.py:44-47 (`PromptEncoder`, the slice of a HuggingFace
tokenizer the probe needs); the reference always loads the target's tokenizer from the hub.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

TOKENIZER_FILES = ("tokenizer.json", "tokenizer.model", "vocab.json", "tokenizer_config.json")


@dataclass(frozen=True)
class PromptEncoder:
    """`encode(text, add_special_tokens)` -> token ids; `source` says where the vocabulary came from."""

    fn: Callable[[str, bool], list[int]]
    source: str

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        return [int(t) for t in self.fn(text, add_special_tokens)]

    def __call__(self, text: str) -> list[int]:
        return self.encode(text, True)


def byte_level(vocab_size: int) -> PromptEncoder:
    return PromptEncoder(lambda s, _special: [b % vocab_size for b in s.encode("utf-8")], "bytes")


def has_tokenizer_files(path: Path) -> bool:
    return path.is_dir() and any((path / f).exists() for f in TOKENIZER_FILES)


def from_directory(path: Path) -> PromptEncoder:
    """A HuggingFace tokenizer read from local files only."""
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(str(path), local_files_only=True)
    return PromptEncoder(lambda s, special: list(tok.encode(s, add_special_tokens=special)), str(path))


def candidate_directories(target_spec: Any, train_ref: Any, data_root: Path | None) -> list[Path]:
    """Where tokenizer files may be staged for this run, most specific first."""
    if data_root is None:
        return []
    root = Path(data_root)
    out: list[Path] = []
    model_name = getattr(target_spec, "model_name", None)
    if model_name:
        out.append(root / "hf_snapshots" / model_name.replace("/", "--"))
    run_path = getattr(target_spec, "run_path", None)
    if run_path:
        from param_decomp_b200.models.loaders import pretrain_cache_dir

        out.append(pretrain_cache_dir(root, run_path))
    if train_ref is not None:
        from param_decomp_b200.formats import dataset_store as ds

        try:
            name = ds.read_dataset_identity(ds.resolve_dataset_ref(train_ref, root)).tokenizer_name
            out.append(root / "tokenizers" / name.replace("/", "--"))
        except (FileNotFoundError, AttributeError, TypeError, KeyError):
            pass  # synthetic streams carry no dataset directory
    return out


def resolve_prompt_encoder(target_spec: Any, train_ref: Any, data_root: Path | None, vocab_size: int,
                           log: Any = None) -> PromptEncoder:
    for path in candidate_directories(target_spec, train_ref, data_root):
        if has_tokenizer_files(path):
            enc = from_directory(path)
            if log is not None:
                log.info("prompt encoder: tokenizer files in %s", path)
            return enc
    if log is not None:
        log.warning("prompt encoder: no tokenizer files staged for this target; prompts are encoded as UTF-8 bytes")
    return byte_level(vocab_size)
