"""Host-side mirror of the reference's ``sqattn`` operator surface."""
from .kernels import (attn_causal, attn_hierarchical_relative_window, attn_hierarchical_window,  # noqa: F401
                      attn_unified)
from .attn_replacer import HostPrefillPipeline, mp_triton_wrapper, process_model  # noqa: F401
