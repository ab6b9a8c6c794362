"""ctypes binding of the C ABI declared in include/axono_b200.h.

Loading fails loudly when the library is missing: there is no CPU or PyTorch fallback for any
operator of this package.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_vp, _i, _i64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); mirrors include/axono_b200.h one to one.
SIGNATURES = {
    "axb200_version": (C.c_char_p, []),
    "axb200_last_error": (C.c_uint, []),
    "axb200_set_wait_limit_ns": (_i, [C.c_uint64]),
    "axb200_set_fused_merge": (_i, [_i]),
    "axb200_set_device_plan": (_i, [_i]),
    "axb200_set_chunk_tiles": (_i, [_i]),
    "axb200_set_dependent_launch": (_i, [_i]),
    "axb200_gqa_chunk_plan": (_i, [_vp, _i, _i, _i, _i, _i64, _vp, _vp, _vp, _vp]),
    "axb200_profile_enable": (_i, [_i]),
    "axb200_profile_collect": (_i, [C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "axb200_gqa_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i]),
    "axb200_gqa_decode": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _vp, _sz, _vp]),
    "axb200_static_scratch_bytes": (_sz, []),
    "axb200_gqa_decode_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _vp]),
    "axb200_gqa_decode_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i,
                                     _vp, _sz, _vp]),
    "axb200_sdpa_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i]),
    "axb200_sdpa": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _i, _vp, _sz, _vp]),
    "axb200_gqa_decode_paged_window": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _i,
                                            _vp, _sz, _vp]),
    "axb200_gqa_decode_paged_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _vp, _sz,
                                            _vp, _vp, _vp, _i, _i, _i, _vp]),
    "axb200_gqa_decode_paged_cp": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _vp, _sz,
                                        _vp, _vp, _vp, _i, _i, _vp]),
    "axb200_nccl_unique_id": (_i, [_vp]),
    "axb200_nccl_init": (_i, [_vp, _i, _i, C.POINTER(_vp)]),
    "axb200_nccl_all_gather": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "axb200_nccl_destroy": (_i, [_vp]),
    "axb200_swap_leading_dims": (_i, [_vp, _vp, _i, _i, _sz, _vp]),
    "axb200_p2p_alloc": (_i, [_sz, C.POINTER(_vp), _vp]),
    "axb200_p2p_open": (_i, [_vp, C.POINTER(_vp)]),
    "axb200_p2p_close": (_i, [_vp]),
    "axb200_p2p_free": (_i, [_vp]),
    "axb200_kv_append_rope": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i,
                                   _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "axb200_kv_prefill_write": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i64, _i, _i, _i,
                                     _i, _i, _i, _i64, _i, _vp]),
    "axb200_qkv_norm_rope_append": (_i, [_vp, _i64, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i,
                                         _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "axb200_silu_mul_rows": (_i, [_vp, _i64, _i, _i64, _vp, _i, _vp]),
    "axb200_decode_step_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i]),
    "axb200_decode_step_launches": (_i, [_i, _i, _i, _i, _i64, _i]),
    "axb200_set_step_fused": (_i, [_i]),
    # q, k_new, v_new, out, k_pages, v_pages, block_table, seq_lens, pos, inv_freq | theta | rotate, mrope, h_sec,
    # w_sec, batch, hq, hkv, d, page_tokens, max_blocks, num_pages | max_seq_len | dtype | workspace, bytes, stream
    "axb200_decode_step_paged": (_i, [_vp] * 10 + [_f] + [_i] * 11 + [_i64, _i, _vp, _sz, _vp]),
    # qkv, ld, q_norm_w, k_norm_w, eps, out, k_pages, v_pages, block_table, seq_lens, pos, inv_freq, theta, rotate,
    # mrope, h_sec, w_sec, batch, hq, hkv, d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, slot_delta,
    # advance, workspace, bytes, peer_out, peer_flags, local_state, world, rank, hq_total, stream
    "axb200_qkv_decode_step_paged": (_i, [_vp, _i64, _vp, _vp, _f] + [_vp] * 7 + [_f] + [_i] * 11 + [_i64] + [_i] * 3 +
                                     [_vp, _sz, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "axb200_decode_step_host": (_i, [_vp] * 12 + [_vp, _vp, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i64, _i,
                                          _vp, _sz, _vp]),
    "axb200_kv_arena_create": (_i, [_i, _i, _i, _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "axb200_kv_arena_destroy": (_i, [_vp]),
    "axb200_kv_arena_alloc_seq": (_i, [_vp, _i64, C.POINTER(_i)]),
    "axb200_kv_arena_reserve": (_i, [_vp, _i, _i64]),
    "axb200_kv_arena_shuffle_free": (_i, [_vp, C.c_uint64]),
    "axb200_kv_arena_free_seq": (_i, [_vp, _i, _vp]),
    "axb200_kv_arena_sync": (_i, [_vp, _vp]),
    "axb200_kv_arena_stats": (_i, [_vp, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "axb200_kv_arena_seq_pages": (_i, [_vp, _i, _vp, _i]),
    "axb200_kv_arena_geometry": (_i, [_vp] + [C.POINTER(_i)] * 8),
    "axb200_kv_arena_k_pages": (_vp, [_vp, _i]),
    "axb200_kv_arena_v_pages": (_vp, [_vp, _i]),
    "axb200_kv_arena_block_table": (_vp, [_vp]),
    "axb200_kv_arena_seq_lens": (_vp, [_vp]),
    "axb200_rope": (_i, [_vp, _vp, _f, _vp, _i64, _i, _i, _i, _vp]),
    "axb200_rope_thd": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i64, _i, _i, _i, _vp]),
    "axb200_rope_with_cos_sin": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "axb200_mrope_cos_sin": (_i, [_vp, _vp, _i, _i, _vp, _vp, _i64, _i, _vp]),
    "axb200_add_rms_norm": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _i64, _i, _i, _vp]),
    "axb200_silu_mul": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "axb200_rms_norm": (_i, [_vp, _vp, _f, _vp, _i64, _i, _i, _vp]),
    "axb200_embedding": (_i, [_vp, _i, _vp, _vp, _i64, _i64, _i, _i, _vp]),
    "axb200_argmax_last_dim": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "axb200_linear_nobias": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]),
    "axb200_randn": (_i, [_vp, _i64, _i, _f, _f, C.c_uint64, _vp]),
    "axb200_cast": (_i, [_vp, _i, _vp, _i, _i64, _vp]),
    "axb200_concat": (_i, [_vp, _vp, _vp, _i64, _sz, _sz, _vp]),
}

STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "OUT_OF_MEMORY", "UNSUPPORTED_TYPE", "SHAPE_MISMATCH",
                "INTERNAL_ERROR", "DEVICE_ERROR", "INVALID_PTR", "DEVICE_MISMATCH"]

# axono::core::DataType values (include/axono/core/types.h:18-27 of the reference)
INT8, INT16, INT32, INT64, FLOAT16, FLOAT32, FLOAT64, BOOLEAN = range(8)

_lib = None


def library_path() -> str:
    return _build.LIB


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises when it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m axono_b200.build` (needs nvcc). "
                "axono_b200 has no fallback path.")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, op: str) -> None:
    """Status != OK becomes RuntimeError, as the reference's binding does
    (axono/python/src/nanobind_module.cpp:1022-1024)."""
    if status != 0:
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else "?"
        raise RuntimeError(f"{op} failed, status {status} ({name})")
