"""Shape of the text tower whose decode step is the caller of the path (hidden 2048, 28 layers, 16 query /
8 KV heads of 128, vocabulary 151936: the reference's Qwen3-VL-2B text config,
axono/python/examples/vlm/qwen3vl/model.py:440-486).  Kept free of PyTorch so the native tower can use it."""
from dataclasses import dataclass
from typing import Tuple


@dataclass
class TextTowerConfig:
    hidden: int = 2048
    intermediate: int = 6144
    n_q_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 151936
    n_layers: int = 28
    eps: float = 1e-6
    rope_theta: float = 1e6
    mrope_section: Tuple[int, int, int] = (24, 20, 20)
    use_mrope: bool = True
    qk_norm: bool = True
