from .core import BLOCK_SIZE, BlockManager, CoreError, RadixTree, SeqTables, SlotPool
from .manager import CacheError, CacheManager, pages_for

__all__ = ["BLOCK_SIZE", "BlockManager", "CacheError", "CacheManager", "CoreError", "RadixTree", "SeqTables",
           "SlotPool", "pages_for"]
