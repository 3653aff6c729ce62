"""Drop-in for the reference package ``flash_attn_v100`` (flash_attn_v100/__init__.py:1-5):
``from flash_attn_v100 import flash_attn_func`` keeps working, now on B200 (sm_100a)."""
__version__ = "0.2.0"

from flash_attn_v100.flash_attn_interface import (  # noqa: F401
    flash_attn_func,
    flash_attn_padded_func,
)
