"""flash-attn-3 style API (`flash_attn_npu_3` of the reference) on NVIDIA B200."""
__version__ = "0.3.0"

from .flash_attn_npu_interface import (  # noqa: F401
    flash_attn_combine,
    flash_attn_func,
    flash_attn_mla_with_kvcache,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_with_kvcache,
    get_scheduler_metadata,
)
