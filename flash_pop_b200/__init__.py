"""flash_pop_b200 — B200 (sm_100a) kernels behind the flash-pop operator API.

Exports the names of the reference package (flash_pop/__init__.py:1-7)."""
from flash_pop_b200._lib import build  # noqa: F401
from flash_pop_b200.fused_retention import fused_chunk_retention, retention_step  # noqa: F401
from flash_pop_b200.pop_retention import flash_pop_retention, pop_suffix_retention  # noqa: F401
from flash_pop_b200.retnet import RetNetDecoderLayer, RetNetDecoder  # noqa: F401
from flash_pop_b200.pop_retnet import POPRetNetDecoder, POPDecoderLayer  # noqa: F401
from flash_pop_b200.diffusion_retnet import (DiffusionRetNetDecoder, DiffusionRetNetDecoderLayer,  # noqa: F401
                                             DiffusionRetNetFinalLayer)
from flash_pop_b200.recurrent_state import RecurrentState  # noqa: F401
