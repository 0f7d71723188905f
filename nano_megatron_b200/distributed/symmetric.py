"""Registry of symmetric-memory workspaces per process group (filled in by
:mod:`nano_megatron_b200.distributed.symm_mem`)."""
from __future__ import annotations

from typing import Any, Optional

_WORKSPACES: dict[int, Any] = {}


def register_workspace(group: Any, ws: Any) -> None:
    _WORKSPACES[id(group)] = ws


def unregister_workspace(group: Any) -> None:
    _WORKSPACES.pop(id(group), None)


def workspace_for(group: Any) -> Optional[Any]:
    return _WORKSPACES.get(id(group))


def clear() -> None:
    _WORKSPACES.clear()


def close_all() -> None:
    """Release every registered workspace (collective over each one's group, in
    registration order, which is the same on all ranks) and forget them."""
    seen = set()
    for ws in list(_WORKSPACES.values()):
        if id(ws) in seen:
            continue
        seen.add(id(ws))
        ws.close()
    _WORKSPACES.clear()


def cp_flash_attention_peer(q, k, v, scale, ws, cp_rank, cp_size):
    from .symm_ops import cp_flash_attention_peer as impl
    return impl(q, k, v, scale, ws, cp_rank, cp_size)
