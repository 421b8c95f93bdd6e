"""Drop-in for kv_cache_manager/py_connector/kernel: same operator names and arguments."""
from .batch_gather_scatter_helper import (batch_gather_kv_caches, batch_gather_kv_pages,  # noqa: F401
                                          batch_scatter_kv_caches, batch_scatter_kv_pages)
from .gather_scatter_helper import CopyBufferAllocator, gather_kv_caches, scatter_kv_caches  # noqa: F401
from .block_table import generate_blocks_idx, generate_block_page_table  # noqa: F401
