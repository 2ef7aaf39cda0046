"""Loads the host C++ module (built on first use) and re-exports its classes."""

from __future__ import annotations

import importlib.util
import sys

from ..build import ensure_core

_NAME = "prefixserve_b200.cache._core"


def _load():
    if _NAME in sys.modules:
        return sys.modules[_NAME]
    path = ensure_core()
    spec = importlib.util.spec_from_file_location(_NAME, str(path))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load the host core from {path}")
    module = importlib.util.module_from_spec(spec)
    sys.modules[_NAME] = module
    spec.loader.exec_module(module)
    return module


_core = _load()

BLOCK_SIZE: int = _core.BLOCK_SIZE
CoreError = _core.CoreError
BlockManager = _core.BlockManager
RadixTree = _core.RadixTree
SlotPool = _core.SlotPool
SeqTables = _core.SeqTables
SlotRecords = _core.SlotRecords

__all__ = ["BLOCK_SIZE", "BlockManager", "CoreError", "RadixTree", "SeqTables", "SlotPool", "SlotRecords"]
