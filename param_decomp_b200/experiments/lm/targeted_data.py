"""The target stream of a targeted (tPD) run: a fixed pool of prompts, sampled by a pure function of
(seed, step) so every rank and every resume sees the same batches.

Pool sources: an arithmetic operand grid (`kind: arithmetic_grid`, the construction of
`evals/lm_ops.build_arithmetic_prompt_grid`), a text file with one prompt per line (`kind: prompts_file`), and
two additions under `kind: inline`: literal prompts and rows of a tokenised dataset. Text is tokenised by the
encoder `experiments/lm/prompt_encoder.py` finds (the target's tokenizer files, else bytes). All rows share
one length.
Parity: param_decomp/experiments/lm/targeted_data.py:1-92, arithmetic_probe.py.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch
from torch import Tensor

from param_decomp_b200.models.transformer import LMBatch


def byte_encoder(vocab_size: int) -> Callable[[str], list[int]]:
    """UTF-8 bytes folded into the vocabulary: deterministic and tokenizer-free."""
    return lambda s: [b % vocab_size for b in s.encode("utf-8")]


@dataclass
class PromptPool:
    tokens: Tensor  # [n_prompts, L] int64
    seed: int

    @property
    def seq_len(self) -> int:
        return self.tokens.shape[1]

    @classmethod
    def build(cls, cfg: Any, vocab_size: int, data_root: Path | None, seed: int,
              encode: Callable[[str], list[int]] | None = None) -> "PromptPool":
        kind = getattr(cfg, "kind", "inline")
        enc = encode or byte_encoder(vocab_size)
        if kind == "arithmetic_grid":
            from param_decomp_b200.evals.lm_ops import build_arithmetic_prompt_grid, inclusive_range

            grid = build_arithmetic_prompt_grid(enc, inclusive_range(cfg.a_range), inclusive_range(cfg.b_range),
                                                cfg.operation)
            return cls(grid.tokens, seed)
        if kind == "prompts_file":
            lines = [ln for ln in Path(cfg.path).read_text().splitlines() if ln.strip()]
            assert lines, f"no prompts in {cfg.path}"
            rows = [enc(ln) for ln in lines]
            lengths = sorted({len(r) for r in rows})
            assert len(lengths) == 1, f"prompts must tokenise to one shared length, got {lengths}"
            return cls(torch.tensor(rows, dtype=torch.int64), seed)
        if cfg.prompts is not None:
            rows = [enc(p) for p in cfg.prompts]
            L = cfg.seq_len or max(len(r) for r in rows)
            assert all(len(r) <= L for r in rows), "a prompt is longer than prompts.seq_len"
            # left-pad by repeating the first token so the last position is always the prompt's end
            rows = [[r[0]] * (L - len(r)) + r for r in rows]
            return cls(torch.tensor(rows, dtype=torch.int64), seed)
        assert cfg.dataset is not None, "prompts: needs `prompts` or `dataset`"
        from param_decomp_b200.config.experiments import SyntheticZipfDataset

        L = cfg.seq_len or 64
        if isinstance(cfg.dataset, SyntheticZipfDataset):
            from param_decomp_b200.data.synthetic import ZipfTokenSource

            src = ZipfTokenSource(vocab_size, L, cfg.dataset.exponent, cfg.dataset.seed)
            return cls(src.batch(0, 256, 0, 1).tokens.long(), seed)
        from param_decomp_b200.data.shards import ShardServer

        assert data_root is not None
        server = ShardServer.open(cfg.dataset, data_root, L, "unsegmented_tokens", seed=seed)
        return cls(server.batch(0, 256, 0, 1).tokens.long(), seed)

    def batch(self, step: int, global_batch: int, rank: int, world: int) -> LMBatch:
        """Rows of the global batch are drawn with replacement by a generator keyed on (seed, step);
        rank `r` takes its contiguous share."""
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + step) & 0x7FFFFFFFFFFFFFFF)
        idx = torch.randint(self.tokens.shape[0], (global_batch,), generator=g)
        rows = global_batch // world
        return LMBatch(self.tokens[idx[rank * rows:(rank + 1) * rows]])
