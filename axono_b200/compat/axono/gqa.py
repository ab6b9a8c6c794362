"""axono.gqa (axono/python/axono/gqa.py:13-33)."""
from axono_b200 import native as _native

_l = _native.load()


def gqa_decode_attention(q, k, v):
    """q (1, n_q_heads, head_dim), k / v (seq_len, n_kv_heads, head_dim) on a CUDA device, FLOAT32 or
    FLOAT16; scale 1/sqrt(head_dim); equals scaled_dot_product_attention(q, k, v, is_causal=False)."""
    return _l.gqa_decode_attention(q, k, v)
