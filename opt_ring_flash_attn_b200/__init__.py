"""B200-native ring flash attention behind the reference's ``ring_flash_attn`` operator."""
from .api import balanced, check, deterministic, ring_flash_attn, ring_flash_attn_with_lse  # noqa: F401
from .compat import (  # noqa: F401
    ring_flash_attn_func,
    ring_flash_attn_kvpacked_func,
    ring_flash_attn_qkvpacked_func,
)
from .schedule import shutdown  # noqa: F401

__all__ = [
    "ring_flash_attn",
    "ring_flash_attn_with_lse",
    "ring_flash_attn_func",
    "ring_flash_attn_kvpacked_func",
    "ring_flash_attn_qkvpacked_func",
    "deterministic",
    "balanced",
    "check",
    "shutdown",
]
