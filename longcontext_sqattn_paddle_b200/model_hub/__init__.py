"""The caller of the attention operator: a random-weight decoder with the reference runtime's layer loops."""
from .decoder import (DecoderConfig, DecoderLayer, RandomInitDecoder, install_sequence_parallel,  # noqa: F401
                      yarn_cos_sin_cache)
