"""moeflow_b200: a Blackwell-native expert-parallel MoE serving backend.

PyTorch framework layer + hand-written sm_100a CUDA kernels (tcgen05 / TMEM / TMA) + peer-memory
all-to-all over NVLink.  See ``fixed.FixedEPLayer`` for the product path.
"""

from .config import GLM53_FLASH, GLM53_FLASH_I1536, MoEConfig

__all__ = ["GLM53_FLASH", "GLM53_FLASH_I1536", "MoEConfig"]
__version__ = "0.1.0"
