"""Component identity: `(site, index)` persisted as `"<site>:<index>"`.

Parity: param_decomp_formats/component_key.py:23-43.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Annotated

from pydantic import AfterValidator

_SITE_RE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,127}$")


def check_site_id(value: str) -> str:
    if not isinstance(value, str) or not _SITE_RE.fullmatch(value) or value in (".", ".."):
        raise ValueError(f"invalid site ID: {value!r}")
    return value


SiteId = Annotated[str, AfterValidator(check_site_id)]


@dataclass(frozen=True, order=True)
class ComponentKey:
    site: str
    component_idx: int

    def __post_init__(self) -> None:
        check_site_id(self.site)
        if not isinstance(self.component_idx, int) or isinstance(self.component_idx, bool):
            raise ValueError(f"component index must be an int: {self.component_idx!r}")
        if self.component_idx < 0:
            raise ValueError(f"component index must be non-negative: {self.component_idx}")

    def encoded(self) -> str:
        return f"{self.site}:{self.component_idx}"

    @classmethod
    def decode(cls, text: str) -> "ComponentKey":
        site, sep, idx = text.rpartition(":")
        if not sep or not site or not (idx.isascii() and idx.isdecimal()):
            raise ValueError(f"invalid encoded component key: {text!r}")
        key = cls(site, int(idx))
        if key.encoded() != text:
            raise ValueError(f"non-canonical encoded component key: {text!r}")
        return key
