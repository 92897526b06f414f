"""Registry from (role, kind) to the class that runs a spec of that kind.

Roles: ``"norm"``, ``"position"``, ``"mixer"``, ``"feed_forward"`` and ``"block"``
(the arrangement of one layer's parts).  A new kind
of part is added by registering its class here; nothing else in the package
names the kinds.
"""
from __future__ import annotations

from typing import Any, Dict

ROLES = ("norm", "position", "mixer", "feed_forward", "block")
_PARTS: Dict[str, Dict[str, type]] = {r: {} for r in ROLES}


def register_part(role: str, kind: str, cls: type, replace: bool = False) -> None:
    if role not in _PARTS:
        raise KeyError(f"unknown part role {role!r}; roles are {ROLES}")
    if kind in _PARTS[role] and not replace and _PARTS[role][kind] is not cls:
        raise KeyError(f"{role} kind {kind!r} is already registered")
    _PARTS[role][kind] = cls


def unregister_part(role: str, kind: str) -> None:
    _PARTS[role].pop(kind, None)


def build_part(role: str, spec: Any, ctx, prefix: str):
    if spec is None:
        return None
    kind = getattr(spec, "kind", None)
    table = _PARTS[role]
    if kind not in table:
        raise KeyError(f"no {role} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind](spec, ctx, prefix)


def known(role: str):
    return sorted(_PARTS[role])
