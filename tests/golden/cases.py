"""Seeded inputs for the golden vectors of the decode hot path.

Each case names the reference test or configuration whose inputs it reproduces
(paths relative to the reference project).  `make_golden.py` feeds these inputs
to the reference's own CPU library and stores the outputs in
`decode_path_golden.npz`; the tests feed the same inputs to the C restatement
and to the CUDA kernels.  numpy only.
"""
from __future__ import annotations

import numpy as np

HQ, HKV, D = 16, 8, 128


def gqa_reference_test_cases():
    """axono/python/tests/core/test_gqa.py:33-42 - one RandomState(3) stream, skv in
    (1, 7, 256, 512, 1024), q (1,16,128), k/v (skv,8,128)."""
    rng = np.random.RandomState(3)
    out = {}
    for skv in (1, 7, 256, 512, 1024):
        q = rng.randn(1, HQ, D).astype(np.float32)
        k = rng.randn(skv, HKV, D).astype(np.float32)
        v = rng.randn(skv, HKV, D).astype(np.float32)
        out[f"gqa_rs3_skv{skv}"] = (q, k, v)
    return out


def gqa_sdpa_op_case():
    """axono/python/tests/core/test_gqa.py:45-55 - RandomState(4), skv=300."""
    rng = np.random.RandomState(4)
    q = rng.randn(1, HQ, D).astype(np.float32)
    k = rng.randn(300, HKV, D).astype(np.float32)
    v = rng.randn(300, HKV, D).astype(np.float32)
    return {"gqa_rs4_skv300": (q, k, v)}


def gqa_config_cases():
    """The CPU-runnable configuration (batch 1, 16 q / 8 kv heads, head_dim 128, KV length
    4096, N(0,1) from a seed) and the lengths either side of the reference's split-K
    threshold (src/ops/cuda/gqa.cu:150)."""
    out = {}
    for name, seed, skv in (("gqa_c1_skv4096", 1000, 4096), ("gqa_skv2047", 1001, 2047),
                            ("gqa_skv2048", 1002, 2048), ("gqa_skv2049", 1003, 2049)):
        rng = np.random.default_rng(seed)
        q = rng.standard_normal((1, HQ, D)).astype(np.float32)
        k = rng.standard_normal((skv, HKV, D)).astype(np.float32)
        v = rng.standard_normal((skv, HKV, D)).astype(np.float32)
        out[name] = (q, k, v)
    return out


def all_gqa_cases():
    out = {}
    out.update(gqa_reference_test_cases())
    out.update(gqa_sdpa_op_case())
    out.update(gqa_config_cases())
    return out


def sdpa_causal_case():
    """axono/python/tests/core/test_sequence_ops.py:85-111 shapes (sq 4, skv 6, 4q/2kv, d 8)."""
    rng = np.random.default_rng(1010)
    q = rng.standard_normal((4, 4, 8)).astype(np.float32)
    k = rng.standard_normal((6, 2, 8)).astype(np.float32)
    v = rng.standard_normal((6, 2, 8)).astype(np.float32)
    return q, k, v


def rope_cases():
    """(x, pos, theta): the reference test's shape (test_sequence_ops.py:62-79: seq 4, 2 heads,
    dim 8, theta 1e4, pos 0..3) and the fused-decode-block shapes (q [8,16,128], k [8,8,128],
    theta 1e6, position = cache length 8192) plus ragged long positions."""
    out = {}
    rng = np.random.default_rng(1020)
    out["rope_small"] = (rng.standard_normal((4, 2, 8)).astype(np.float32),
                         np.arange(4, dtype=np.int64), 10000.0)
    out["rope_c2_q"] = (rng.standard_normal((8, HQ, D)).astype(np.float32),
                        np.full(8, 8192, np.int64), 1e6)
    out["rope_c2_k"] = (rng.standard_normal((8, HKV, D)).astype(np.float32),
                        np.full(8, 8192, np.int64), 1e6)
    out["rope_ragged"] = (rng.standard_normal((8, HKV, D)).astype(np.float32),
                          rng.integers(16384, 32769, 8).astype(np.int64), 1e6)
    return out


def inv_freq(theta: float, d: int = D) -> np.ndarray:
    """examples/vlm/qwen3vl/model.py:474-481 and test_sequence_ops.py:260:
    1 / theta ** (arange(0, d, 2, float32) / d), float32."""
    return (1.0 / (theta ** (np.arange(0, d, 2, dtype=np.float32) / d))).astype(np.float32)


def build_mrope_pos3(n, img_start, want, llm_h, llm_w):
    """Position rule of examples/vlm/qwen3vl/model.py:49-61, written from its description:
    text before the image counts up on all axes, image token j sits at
    (T, H, W) = (s, s + j // w, s + j % w), text after resumes at s + max(h, w)."""
    pos3 = np.zeros((3, n), np.int64)
    for i in range(n):
        if i < img_start:
            pos3[:, i] = i
        elif i < img_start + want:
            j = i - img_start
            pos3[:, i] = (img_start, img_start + j // llm_w, img_start + j % llm_w)
        else:
            pos3[:, i] = img_start + max(llm_h, llm_w) + (i - img_start - want)
    return pos3


def mrope_cases():
    """mrope_cos_sin: test_sequence_ops.py:252-290 (default_rng(7): seq 33; default_rng(8):
    seq 17; theta 5e6, sections (20,20)).  rope_thd: the multimodal configuration - sections
    24/20/20, 1024 image tokens on a 32x32 grid then 512 text tokens; a sample of prefix rows
    and the 16 decode rows (T=H=W=prev_len+rope_delta, rope_delta = 32-1024)."""
    out = {}
    for seed, seq in ((7, 33), (8, 17)):
        rng = np.random.default_rng(seed)
        pos3 = rng.integers(0, 50, size=(3, seq)).astype(np.int64)
        out[f"mrope_cs_seed{seed}"] = (pos3, inv_freq(5e6), 20, 20)
    rng = np.random.default_rng(1030)
    full = build_mrope_pos3(1536, 0, 1024, 32, 32)
    rows = np.concatenate([np.arange(0, 1024, 67), np.arange(1020, 1536, 43)])
    out["rope_thd_prefix"] = (rng.standard_normal((len(rows), HKV, D)).astype(np.float32),
                              np.ascontiguousarray(full[:, rows]), inv_freq(1e6), (24, 20, 20))
    dec = np.full((3, 16), 1536 + (32 - 1024), np.int64) + np.arange(16)[None, :]
    out["rope_thd_decode"] = (rng.standard_normal((16, HQ, D)).astype(np.float32),
                              dec, inv_freq(1e6), (24, 20, 20))
    return out


def fused_cases():
    """silu_mul: tests/core/test_fused.py:18-25 (RandomState(0), 37x53) and :34-39 edge values;
    add_rms_norm: :42-53 (RandomState(1), 4x128, eps 1e-6) and the fused-decode-block shape
    ([8,2048], weights N(1,0.02)); rms_norm: tests/core/test_llm_ops.py:141-146 shape (8x16, eps 1e-5)
    and the per-head q-norm shape (rows x 128)."""
    out = {}
    rng = np.random.RandomState(0)
    out["silu_rs0"] = (rng.randn(37, 53).astype(np.float32), rng.randn(37, 53).astype(np.float32))
    out["silu_edge"] = (np.array([-10.0, -1.0, 0.0, 1.0, 10.0, -88.0, 88.0, -100.0], np.float32),
                        np.ones(8, np.float32))
    rng = np.random.RandomState(1)
    out["addrms_rs1"] = (rng.randn(4, 128).astype(np.float32), rng.randn(4, 128).astype(np.float32),
                         rng.randn(128).astype(np.float32), 1e-6)
    rng = np.random.default_rng(1040)
    out["addrms_c2"] = (rng.standard_normal((8, 2048)).astype(np.float32),
                        rng.standard_normal((8, 2048)).astype(np.float32),
                        (1.0 + 0.02 * rng.standard_normal(2048)).astype(np.float32), 1e-6)
    out["rms_8x16"] = (rng.standard_normal((8, 16)).astype(np.float32),
                       rng.standard_normal(16).astype(np.float32), 1e-5)
    out["rms_qnorm"] = (rng.standard_normal((8 * HQ, D)).astype(np.float32),
                        (1.0 + 0.02 * rng.standard_normal(D)).astype(np.float32), 1e-6)
    return out


def concat_case():
    """tests/nn/test_kv_cache.py:27-45 pattern: a cache of 5 tokens gets one more (fp16 bits)."""
    rng = np.random.default_rng(1050)
    a = rng.standard_normal((5, HKV, D)).astype(np.float16)
    b = rng.standard_normal((1, HKV, D)).astype(np.float16)
    return a, b
