"""B200-native ring flash attention behind the reference's ``ring_flash_attn`` operator."""
from .api import ring_flash_attn, ring_flash_attn_with_lse  # noqa: F401

__all__ = ["ring_flash_attn", "ring_flash_attn_with_lse"]
