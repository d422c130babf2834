"""The cache: host bookkeeping (pages, block tables, state slots) and the device storage behind it."""
from .manager import CacheManager, GroupSpec, OutOfPages, chain_hash

__all__ = ["CacheManager", "GroupSpec", "OutOfPages", "chain_hash"]
