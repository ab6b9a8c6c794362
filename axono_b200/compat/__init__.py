"""The reference's Python surface for the decode path, `import axono`, over this library's native
module (no PyTorch).

    import axono_b200.compat as compat
    compat.install()          # puts this directory's `axono` package at the front of sys.path
    import axono
    axono.set_default_device("cuda")
    out = axono.gqa_decode_attention(q, k, v)

Covered: Tensor / DataType / Status, set_default_device / set_backend, gqa_decode_attention,
axono.fused.{silu_mul, add_rms_norm}, rope / rope_thd / rope_with_cos_sin / mrope_cos_sin,
scaled_dot_product_attention, concat, embedding, argmax, rms_norm, nn.{KVCache, DynamicKVCache},
compile, CUDAGraph, cuda_graph - the names a user of the reference calls on this path
(axono/python/axono/__init__.py, gqa.py, fused.py, core/ops/{sequence,llm}.py, nn/kv_cache.py).
Everything else of the reference's package (Linear, Module, elementwise operators, the CPU backend)
is outside this library: the missing names raise AttributeError, CPU tensors are refused by the
operators."""
import os
import sys


def path() -> str:
    return os.path.dirname(os.path.abspath(__file__))


def install() -> None:
    """Makes `import axono` resolve to this package's shim (idempotent)."""
    p = path()
    if p not in sys.path:
        sys.path.insert(0, p)
