"""Configuration and MFU accounting."""

from .config import ConfigValidationError, MoEConfig, load_config  # noqa: F401
from .mfu import MFUAccountant, MFUResult, compute_mfu, compute_mfu_detailed, compute_moe_flops  # noqa: F401
