"""The registry of parts: role ("mixer", "ffn", "norm", "position", "embedding",
"head", "block") and kind -> class.  A new kind of part is added by registering a
class; the framework's files need no change for it."""
from __future__ import annotations

from .spec import PartSpec

ROLES = ("mixer", "ffn", "norm", "position", "embedding", "head", "block")
_PARTS: dict[tuple[str, str], type] = {}


def register_part(role: str, kind: str, cls: type | None = None):
    """`register_part("mixer", "attention", Attention)` or as a class decorator."""
    if role not in ROLES:
        raise ValueError(f"unknown role {role!r} (roles: {', '.join(ROLES)})")

    def _do(c):
        _PARTS[(role, kind)] = c
        return c
    return _do(cls) if cls is not None else _do


def registered_parts(role: str) -> list[str]:
    return sorted(k for r, k in _PARTS if r == role)


def make_part(role: str, spec: PartSpec, runtime, **extra):
    """Build the part `spec` names.  Its class is called as cls(runtime, **params)."""
    try:
        cls = _PARTS[(role, spec.kind)]
    except KeyError:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered "
                         f"(registered: {', '.join(registered_parts(role)) or 'none'})") from None
    return cls(runtime, **spec.params, **extra)
