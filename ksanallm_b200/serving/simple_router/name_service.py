"""Where the router finds a prefill / decode pair.

The reference's router delegates pair selection to a pluggable "name service" (simple_router/name_service/
name_service.py: an abstract provider loaded from a dotted module path, ``auto_provider.py`` reading the router's own
database, ``polaris_provider.py`` asking an external discovery service) and reports the outcome of every forwarded
call back to it. The same three pieces here:

* ``NameServiceProvider`` - ``get_available_nodes`` returns (prefill, decode) descriptions, ``update_call_result``
  hears whether the forwarded calls succeeded;
* ``RegistryProvider`` - the built-in provider: the pair with the fewest requests in flight among the nodes that
  registered with this router and still send heartbeats;
* ``StaticProvider`` - a fixed list of pairs (no registration), for deployments where another system owns discovery;
* ``load_provider("pkg.module")`` imports a module exposing ``create_provider()``.
"""
from __future__ import annotations

import importlib
import itertools
import threading
from typing import Any, Dict, List, Optional, Tuple

Node = Dict[str, Any]  # node_id, group_name, addr (host:port of /generate)


class NameServiceProvider:
    name = "abstract"

    def get_available_nodes(self, **kwargs) -> Optional[Tuple[Node, Node]]:
        raise NotImplementedError

    def update_call_result(self, prefill: Node, decode: Node, prefill_ok: bool, decode_ok: bool) -> None:
        """Called after both forwarded requests ended."""


class RegistryProvider(NameServiceProvider):
    name = "registry"

    def __init__(self, registry):
        self.registry = registry

    def get_available_nodes(self, **kwargs) -> Optional[Tuple[Node, Node]]:
        pair = self.registry.pick_pair()
        if pair is None:
            return None
        (p_id, p_group, p_addr, _), (d_id, d_group, d_addr, _) = pair
        return ({"node_id": p_id, "group_name": p_group, "addr": p_addr},
                {"node_id": d_id, "group_name": d_group, "addr": d_addr})


class StaticProvider(NameServiceProvider):
    """Round-robin over configured pairs; a pair whose last call failed is skipped ``penalty`` times."""
    name = "static"

    def __init__(self, pairs: List[Tuple[str, str]], penalty: int = 3):
        if not pairs:
            raise ValueError("StaticProvider needs at least one (prefill_addr, decode_addr) pair")
        self.pairs = [({"node_id": f"p{i}", "group_name": f"prefill_{i}", "addr": p},
                       {"node_id": f"d{i}", "group_name": f"decode_{i}", "addr": d}) for i, (p, d) in enumerate(pairs)]
        self.penalty = penalty
        self._skip = [0] * len(self.pairs)
        self._rr = itertools.count()
        self._lock = threading.Lock()

    def get_available_nodes(self, **kwargs) -> Optional[Tuple[Node, Node]]:
        with self._lock:
            for _ in range(len(self.pairs)):
                i = next(self._rr) % len(self.pairs)
                if self._skip[i] > 0:
                    self._skip[i] -= 1
                    continue
                return self.pairs[i]
            return self.pairs[next(self._rr) % len(self.pairs)]  # everything penalised: try anyway

    def update_call_result(self, prefill: Node, decode: Node, prefill_ok: bool, decode_ok: bool) -> None:
        if prefill_ok and decode_ok:
            return
        with self._lock:
            for i, (p, d) in enumerate(self.pairs):
                if p["addr"] == prefill["addr"] and d["addr"] == decode["addr"]:
                    self._skip[i] = self.penalty


def load_provider(module_path: str) -> NameServiceProvider:
    mod = importlib.import_module(module_path)
    factory = getattr(mod, "create_provider", None)
    if factory is None:
        raise ImportError(f"{module_path} does not expose create_provider()")
    provider = factory()
    if not isinstance(provider, NameServiceProvider):
        raise TypeError(f"{module_path}.create_provider() did not return a NameServiceProvider")
    return provider
