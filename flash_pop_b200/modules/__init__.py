from flash_pop_b200.modules.adaln import AdaLayerNorm, AdaLayerNormZero  # noqa: F401
from flash_pop_b200.modules.timestep import TimestepEmbedder  # noqa: F401
