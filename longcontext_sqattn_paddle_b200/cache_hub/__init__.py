"""Key clustering and the KV cache (mirror of the reference's ``cache_hub``)."""
from .flash_attn_cache import HybridKVCache, flash_attn_cache, kv_memory_model, split_blocks  # noqa: F401
from .kmeans import segment_k_means  # noqa: F401
from .retrieval import ClusteredKV, RaggedClusteredDecoder, num_clusters_for  # noqa: F401
