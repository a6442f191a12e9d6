"""Key clustering and the KV cache (mirror of the reference's ``cache_hub``)."""
from .kmeans import segment_k_means  # noqa: F401
