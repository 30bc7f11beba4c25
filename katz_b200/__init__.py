"""katz_b200: the SDXL UNet denoising step with adapters (LoRA merge/restore, ControlNet residual intake, one UNet
step, latent-row parallelism) on hand-written sm_100a kernels behind a C ABI (include/katz_b200.h)."""
from ._lib import KatzError, LIB_PATH, load as load_library  # noqa: F401

__version__ = "0.1.0"
