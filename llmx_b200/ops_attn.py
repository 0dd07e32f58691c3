"""Python face of the tiled bfloat16 attention kernels (csrc/attention_decode.cu, csrc/attention_prefill.cu)."""
from __future__ import annotations


def supported(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    return False
