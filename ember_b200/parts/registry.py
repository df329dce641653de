"""Registry from (family, kind) to the class that implements a part.

Families: "norm", "position", "mixer", "feed_forward", "arrangement".  A layer names its
parts by spec; ``build_part`` looks the class up by the spec's ``kind``.  Registering a new
class here is all that adding a part takes (no framework file changes).
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from ..config.spec import ConfigError, PartSpec

_PARTS: Dict[Tuple[str, str], Callable] = {}
FAMILIES = ("norm", "position", "mixer", "feed_forward", "arrangement")


def register_part(family: str, kind: str, cls: Callable) -> None:
    if family not in FAMILIES:
        raise ConfigError(f"unknown part family {family!r} (families: {', '.join(FAMILIES)})")
    _PARTS[(family, kind)] = cls


def registered_parts(family: str):
    return sorted(k for f, k in _PARTS if f == family)


def part_class(family: str, kind: str) -> Callable:
    try:
        return _PARTS[(family, kind)]
    except KeyError:
        raise ConfigError(f"no {family} of kind {kind!r} is registered "
                          f"(registered: {', '.join(registered_parts(family)) or 'none'})") from None


def build_part(family: str, spec: PartSpec, prefix: str = ""):
    return part_class(family, spec.kind)(spec, prefix)
