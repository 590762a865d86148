"""Blackwell-native flash-attention forward behind a C ABI (include/fa_b200.h)."""
from .api import (cast_output, dropout_mask, flash_attn_forward, flash_attn_forward_host, merge_partial,  # noqa: F401
                  num_splits_heuristic)
