"""Batched twins of the CacheManager / MetaSearcher operators on the hash + match path."""
from .block_index import BlockIndex, encode_locations, status_task  # noqa: F401
from .cache_manager import GpuCacheManager, IsBlockMaskValid, IsIndexInMaskRange  # noqa: F401
from .hash_util import ApplyPrefixHashBatch, GenKeyVectorBatch, key_offsets, length_order  # noqa: F401
from .meta_searcher import BatchMetaSearcher, QueryType  # noqa: F401
from .sharded_searcher import CudaShardBackend, ShardedMetaSearcher, shard_of_keys  # noqa: F401
