"""Host runtime (control plane): nodes, messages, customers, the executor DAG
engine, membership and the socket/in-process van -- implemented in C++
(``csrc/core``) and exposed through the ``_core`` extension module."""
from __future__ import annotations

from .. import _build


def _load():
    try:
        from .. import _core  # type: ignore
    except ImportError:
        _build.build_core()
        from .. import _core  # type: ignore
    return _core


core = _load()

from .cluster import LocalCluster  # noqa: E402,F401
