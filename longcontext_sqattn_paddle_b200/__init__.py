"""B200 (sm_100a) implementation of the SQAttn long-context attention path.

Layout:
  csrc/               CUDA kernels and the C ABI (built into libsqattn_b200.so)
  _lib.py, ops.py     ctypes binding and tensor-level wrappers
  sqattn/             host-side mirror of the reference operator surface
                      (attention_fn adapter, kernel launchers)
  cache_hub/          kmeans clustering and the KV cache
  dist.py             sequence-parallel prefill and cross-GPU split-KV decode

Importing the package never falls back to a CPU or PyTorch path: without the
built shared library the import fails.
"""
from . import _lib  # noqa: F401  (fails loudly when the library is missing)
from . import ops  # noqa: F401

__all__ = ["ops"]
