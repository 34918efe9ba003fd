"""Loader of the native host runtime (``_lib/_ksana_host.so``): scheduler, KV block manager, draft trie.

The module is built in-tree on first use when the shared object is missing or older than its sources.
"""
from __future__ import annotations

import importlib.util
import sys

from . import _build

_so = _build.build_host()
_spec = importlib.util.spec_from_file_location("_ksana_host", str(_so))
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
sys.modules.setdefault("ksanallm_b200._ksana_host", _mod)

globals().update({k: getattr(_mod, k) for k in dir(_mod) if not k.startswith("__")})
