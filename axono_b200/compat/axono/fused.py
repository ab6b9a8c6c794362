"""axono.fused (axono/python/axono/fused.py:19-44)."""
from axono_b200 import native as _native

_l = _native.load()


def silu_mul(gate, up):
    """silu(gate) * up, elementwise; gate and up of one shape."""
    return _l.silu_mul(gate, up)


def add_rms_norm(x, residual, weight, eps: float = 1e-6):
    """y = x + residual; out = y * rsqrt(mean(y^2) + eps) * weight.  Returns (y, out)."""
    return _l.add_rms_norm(x, residual, weight, eps)
