"""`BaseConfig`: the frozen, extra-forbidding pydantic base of every config, with YAML/JSON I/O.

Parity: param_decomp_formats/config.py:14-70 (same `extra="forbid"`, `frozen=True` contract and
`from_file` / `to_file` helpers, so reference YAMLs and ours round-trip the same way).
"""

from __future__ import annotations

import json
from functools import cached_property
from pathlib import Path
from typing import Annotated, Any, ClassVar, Self

import yaml
from annotated_types import Ge, Le
from pydantic import BaseModel, ConfigDict

Probability = Annotated[float, Ge(0), Le(1)]

_LOADERS = {".json": json.loads, ".yaml": yaml.safe_load, ".yml": yaml.safe_load}


class BaseConfig(BaseModel):
    model_config: ClassVar[ConfigDict] = ConfigDict(
        extra="forbid", frozen=True, ignored_types=(cached_property,)
    )

    @classmethod
    def from_file(cls, path: Path | str) -> Self:
        path = Path(path)
        if path.suffix not in _LOADERS:
            raise ValueError(f"config files are .json/.yaml/.yml, got {path}")
        raw: Any = _LOADERS[path.suffix](path.read_text())
        try:
            return cls.model_validate(raw)
        except Exception as err:  # attach the source so a bad sweep cell is findable
            err.add_note(f"while validating {cls.__name__} from {path.as_posix()}")
            raise

    def to_file(self, path: Path | str) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        if path.suffix == ".json":
            path.write_text(self.model_dump_json(indent=2))
        elif path.suffix in (".yaml", ".yml"):
            path.write_text(yaml.dump(self.model_dump(mode="json")))
        else:
            raise ValueError(f"config files are .json/.yaml/.yml, got {path}")

    def to_yaml(self) -> str:
        return yaml.dump(self.model_dump(mode="json"), sort_keys=False)
