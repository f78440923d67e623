"""KV-cache bookkeeping: block pool, radix prefix cache, recurrent-state slots."""
from .block_manager import BlockPool, OutOfBlocks, SlotPool  # noqa: F401
from .radix_cache import PrefixMatch, RadixCache  # noqa: F401
