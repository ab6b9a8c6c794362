"""Host-side mirror of the reference's operator API for the decode path.

Function names, argument order and meaning, and error behaviour (RuntimeError on a non-OK
status) follow the reference's Python surface:

    gqa_decode_attention(q, k, v)              axono/python/axono/gqa.py:13-33
    silu_mul(gate, up)                         axono/python/axono/fused.py:19-36
    add_rms_norm(x, residual, weight, eps)     axono/python/axono/fused.py:39-44
    rope / rope_thd / rope_with_cos_sin / mrope_cos_sin / concat
                                               axono/python/axono/core/ops/sequence.py
    rms_norm(x, weight, eps=1e-5)              axono/python/axono/core/ops/llm.py:99-109

Tensors are CUDA `torch.Tensor`s: PyTorch supplies device memory and the current stream and
nothing else - every operator is one call into the C ABI (include/axono_b200.h), and there is
no fallback when the library is missing.  Outputs are allocated here, as the reference's
binding allocates them (nanobind_module.cpp:1019).
"""
from __future__ import annotations

import torch

from . import _capi

_DTYPES = {torch.float16: _capi.FLOAT16, torch.float32: _capi.FLOAT32}
_workspaces: dict = {}
_retired: list = []  # outgrown workspaces, never freed (graphs captured earlier may still write to them)
_launches = 0  # operator calls that reached the C ABI (used to tell an empty graph capture)


def launch_count() -> int:
    return _launches


def _call(status: int, op: str) -> None:
    global _launches
    _capi.check(status, op)
    _launches += 1


def _dt(t: torch.Tensor, op: str) -> int:
    if not t.is_cuda:
        raise RuntimeError(f"{op}: expected a CUDA tensor (this package has no CPU path)")
    code = _DTYPES.get(t.dtype)
    if code is None:
        _capi.check(3, op)  # UNSUPPORTED_TYPE
    return code


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def last_error() -> int:
    return int(_capi.lib().axb200_last_error())


def workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch for the decode-attention partials, cached per device and grown on demand.
    Call once with the largest size before capturing a CUDA graph."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            # a captured graph may have the old buffer's address baked in: keep it alive for good
            _retired.append(buf)
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=key)
        _workspaces[key] = buf
    return buf


def gqa_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype=torch.float16) -> int:
    return int(_capi.lib().axb200_gqa_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), _DTYPES[dtype]))


def decode_step_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype=torch.float16) -> int:
    """Scratch of `decode_step_paged` (the attention partials plus room for a rotated q)."""
    return int(_capi.lib().axb200_decode_step_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), _DTYPES[dtype]))


def gqa_decode_attention(q, k, v):
    """q (1, n_q_heads, head_dim); k/v (seq_len, n_kv_heads, head_dim) -> (1, n_q_heads, head_dim).
    Equals scaled_dot_product_attention(q, k, v, is_causal=False); scale 1/sqrt(head_dim)."""
    op = "gqa_decode_attention"
    dt = _dt(q, op)
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        _capi.check(3, op)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        _capi.check(3, op)
    sq, hq, d = q.shape
    skv, hkv, dk = k.shape
    if sq != 1:
        _capi.check(1, op)
    if dk != d or tuple(v.shape) != (skv, hkv, d) or hkv == 0 or hq % hkv != 0:
        _capi.check(4, op)
    q, k, v = _c(q), _c(k), _c(v)
    out = torch.empty_like(q)
    lib = _capi.lib()
    ws_bytes = lib.axb200_gqa_workspace_bytes(1, hq, hkv, d, skv, dt)
    ws = workspace(q.device, ws_bytes)
    _call(lib.axb200_gqa_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), hq, hkv, d,
                                      skv, dt, ws.data_ptr(), ws.numel(), _stream(q)), op)
    return out


def gqa_decode_attention_paged(q, k_pages, v_pages, block_table, seq_lens, max_seq_len, out=None, gather=None,
                               window: int = 0, context_parallel=None):
    """Batched decode over a paged cache (extension of the reference op to a batch).
    q (batch, hq, d); k_pages/v_pages (num_pages, hkv, page_tokens, d); block_table int32
    (batch, max_blocks); seq_lens int32 (batch) on the device; max_seq_len a host upper bound.
    gather=(PeerGather, slot): heads are sharded across ranks; the kernel writes this rank's heads into
    every rank's gathered buffer and the full (batch, hq_total, d) tensor of this rank is returned.
    window > 0: each sequence attends only its last `window` tokens.
    context_parallel=(PeerGather(kind="records"), slot): every rank caches a share of each sequence's
    tokens; the ranks exchange un-normalised partials over peer memory and all return the full result."""
    op = "gqa_decode_attention_paged"
    dt = _dt(q, op)
    batch, hq, d = q.shape
    num_pages, hkv, page_tokens, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape:
        _capi.check(4, op)
    if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        _capi.check(3, op)
    q = _c(q)
    lib = _capi.lib()
    ws_bytes = lib.axb200_gqa_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), dt)
    ws = workspace(q.device, ws_bytes)
    if gather is not None:
        pg, slot = gather
        if pg.batch != batch or pg.d != d or pg.hq_total != hq * pg.world or pg.dtype != q.dtype:
            _capi.check(4, op)
        _call(lib.axb200_gqa_decode_paged_gather(
            q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(),
            batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages, int(max_seq_len), dt,
            ws.data_ptr(), ws.numel(), pg.out_ptrs(slot), pg.flag_ptrs, pg.state_ptr, pg.world, pg.rank,
            pg.hq_total, _stream(q)), op)
        return pg.tensor(slot)
    if out is None:
        out = torch.empty_like(q)
    if context_parallel is not None:
        pg, slot = context_parallel
        if pg.kind != "records" or pg.batch != batch or pg.d != d or pg.hq_total != hq:
            _capi.check(4, op)
        _call(lib.axb200_gqa_decode_paged_cp(
            q.data_ptr(), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
            seq_lens.data_ptr(), batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages,
            int(max_seq_len), dt, ws.data_ptr(), ws.numel(), pg.out_ptrs(slot), pg.flag_ptrs, pg.state_ptr,
            pg.world, pg.rank, _stream(q)), op)
        return out
    if window:
        _call(lib.axb200_gqa_decode_paged_window(
            q.data_ptr(), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
            seq_lens.data_ptr(), batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages,
            int(max_seq_len), int(window), dt, ws.data_ptr(), ws.numel(), _stream(q)), op)
        return out
    _call(lib.axb200_gqa_decode_paged(
        q.data_ptr(), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        seq_lens.data_ptr(), batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages,
        int(max_seq_len), dt, ws.data_ptr(), ws.numel(), _stream(q)), op)
    return out


def kv_append_rope(q, k_new, v_new, k_pages, v_pages, block_table, seq_lens, pos=None, inv_freq=None,
                   theta=10000.0, mrope_section=None, rotate=True, advance=True, slot_delta=0):
    """One decode step's rope(q), rope(k) and cache append in one launch.  q (batch,hq,d) is rotated
    in place; k_new/v_new (batch,hkv,d) land in slot seq_lens[b] + slot_delta; seq_lens advances when
    asked (first layer of a step: slot_delta 0, advance; later layers: slot_delta -1, no advance).
    pos: int64 (batch), or (3,batch) with mrope_section=(t,h,w); None = the cache length."""
    op = "kv_append_rope"
    dt = _dt(k_new, op)
    batch, hkv, d = k_new.shape
    hq = q.shape[1] if q is not None else 0
    num_pages, _, page_tokens, _ = k_pages.shape
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    for t in (q, k_new, v_new):
        if t is not None and not t.is_contiguous():
            raise RuntimeError(f"{op}: tensors must be contiguous (q is updated in place)")
    _call(_capi.lib().axb200_kv_append_rope(
        _ptr(q), k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), seq_lens.data_ptr(), _ptr(pos), _ptr(inv_freq), float(theta),
        int(rotate), int(mrope), h_sec, w_sec, batch, hq, hkv, d, page_tokens, block_table.shape[1],
        num_pages, dt, int(slot_delta), int(advance), _stream(k_new)), op)
    return q


def decode_step_paged(q, k_new, v_new, k_pages, v_pages, block_table, seq_lens, max_seq_len, out=None, pos=None,
                      inv_freq=None, theta=10000.0, mrope_section=None, rotate=True):
    """One decode step as one operator: rope(q), rope(k_new), append of (k_new, v_new), attention of q over
    the cache including the new token.  q is read, not rotated in place; seq_lens grows by one.  One launch
    where the library's one-launch step applies (fp16, head_dim 64 or 128), else the two kernels.
    max_seq_len bounds the lengths after the append."""
    op = "decode_step_paged"
    dt = _dt(q, op)
    batch, hq, d = q.shape
    hkv = k_new.shape[1]
    num_pages, _, page_tokens, _ = k_pages.shape
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    for t in (q, k_new, v_new):
        if not t.is_contiguous():
            raise RuntimeError(f"{op}: tensors must be contiguous")
    if out is None:
        out = torch.empty_like(q)
    lib = _capi.lib()
    ws = workspace(q.device, lib.axb200_decode_step_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), dt))
    _call(lib.axb200_decode_step_paged(
        q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), seq_lens.data_ptr(), _ptr(pos), _ptr(inv_freq), float(theta), int(rotate), int(mrope),
        h_sec, w_sec, batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages, int(max_seq_len), dt,
        ws.data_ptr(), ws.numel(), _stream(q)), op)
    return out


def kv_prefill_write(q, k, v, k_pages, v_pages, block_row, start=0, pos=None, inv_freq=None, theta=10000.0,
                     mrope_section=None, rotate=True):
    """Writes the n tokens k, v (n,hkv,d) of one sequence into its pages at slots start.., rotating k (and
    q (n,hq,d) in place when given) with each token's position: pos int64 (n) / (3,n) / None = start+i."""
    op = "kv_prefill_write"
    dt = _dt(k, op)
    n, hkv, d = k.shape
    num_pages, _, page_tokens, _ = k_pages.shape
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    for t in (q, k, v):
        if t is not None and not t.is_contiguous():
            raise RuntimeError(f"{op}: tensors must be contiguous")
    _call(_capi.lib().axb200_kv_prefill_write(
        _ptr(q), k.data_ptr(), v.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_row.data_ptr(),
        _ptr(pos), _ptr(inv_freq), float(theta), int(rotate), int(mrope), h_sec, w_sec, n,
        q.shape[1] if q is not None else 0, hkv, d, page_tokens, block_row.numel(), num_pages, int(start), dt,
        _stream(k)), op)
    return q


def qkv_norm_rope_append(qkv, n_q_heads, q_norm_weight, k_norm_weight, eps, k_pages, v_pages, block_table, seq_lens,
                         pos=None, inv_freq=None, theta=10000.0, mrope_section=None, rotate=True, advance=True,
                         slot_delta=0):
    """Per-head rms_norm(q), rms_norm(k), rope on both and the cache append, straight from the QKV
    projection output qkv (batch, (hq + 2*hkv) * d) (rows may be strided).  Returns the normed, rotated
    q as a new (batch, hq, d) tensor."""
    op = "qkv_norm_rope_append"
    dt = _dt(qkv, op)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        _capi.check(4, op)
    num_pages, hkv, page_tokens, d = k_pages.shape
    batch = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * hkv) * d:
        _capi.check(4, op)
    for w in (q_norm_weight, k_norm_weight):
        if w is not None and (w.dtype != qkv.dtype or tuple(w.shape) != (d,) or not w.is_contiguous()):
            _capi.check(4, op)
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    q_out = torch.empty((batch, n_q_heads, d), dtype=qkv.dtype, device=qkv.device)
    _call(_capi.lib().axb200_qkv_norm_rope_append(
        qkv.data_ptr(), qkv.stride(0), _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), q_out.data_ptr(),
        k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(), _ptr(pos),
        _ptr(inv_freq), float(theta), int(rotate), int(mrope), h_sec, w_sec, batch, n_q_heads, hkv, d,
        page_tokens, block_table.shape[1], num_pages, dt, int(slot_delta), int(advance), _stream(qkv)), op)
    return q_out


def qkv_decode_step_paged(qkv, n_q_heads, q_norm_weight, k_norm_weight, eps, k_pages, v_pages, block_table, seq_lens,
                          max_seq_len, out=None, pos=None, inv_freq=None, theta=10000.0, mrope_section=None, rotate=True,
                          advance=True, slot_delta=0, gather=None):
    """`qkv_norm_rope_append` followed by `gqa_decode_attention_paged` as one operator (one launch for fp16
    with head_dim 64 / 128): the tower layer's step straight from the QKV projection output qkv
    (batch, (hq + 2*hkv) * d), rows may be strided.  Returns the attention output (batch, hq, d), or with
    gather=(PeerGather, slot) this rank's gathered (batch, hq_total, d)."""
    op = "qkv_decode_step_paged"
    dt = _dt(qkv, op)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        _capi.check(4, op)
    num_pages, hkv, page_tokens, d = k_pages.shape
    batch = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * hkv) * d:
        _capi.check(4, op)
    for w in (q_norm_weight, k_norm_weight):
        if w is not None and (w.dtype != qkv.dtype or tuple(w.shape) != (d,) or not w.is_contiguous()):
            _capi.check(4, op)
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    lib = _capi.lib()
    ws = workspace(qkv.device, lib.axb200_decode_step_workspace_bytes(batch, n_q_heads, hkv, d, int(max_seq_len), dt))
    if gather is not None:
        pg, slot = gather
        if pg.batch != batch or pg.d != d or pg.hq_total != n_q_heads * pg.world or pg.dtype != qkv.dtype:
            _capi.check(4, op)
        peers, out_ptr = (pg.out_ptrs(slot), pg.flag_ptrs, pg.state_ptr, pg.world, pg.rank, pg.hq_total), None
    else:
        if out is None:
            out = torch.empty((batch, n_q_heads, d), dtype=qkv.dtype, device=qkv.device)
        peers, out_ptr = (None, None, None, 0, 0, n_q_heads), out.data_ptr()
    _call(lib.axb200_qkv_decode_step_paged(
        qkv.data_ptr(), qkv.stride(0), _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), out_ptr, k_pages.data_ptr(),
        v_pages.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(), _ptr(pos), _ptr(inv_freq), float(theta),
        int(rotate), int(mrope), h_sec, w_sec, batch, n_q_heads, hkv, d, page_tokens, block_table.shape[1], num_pages,
        int(max_seq_len), dt, int(slot_delta), int(advance), ws.data_ptr(), ws.numel(), *peers, _stream(qkv)), op)
    return pg.tensor(slot) if gather is not None else out


def silu_mul_rows(gate_up, n: int):
    """silu(gate) * up for gate = gate_up[:, :n], up = gate_up[:, n:2n] (one fused gate|up projection
    output, rows may be strided) -> (rows, n)."""
    op = "silu_mul_rows"
    dt = _dt(gate_up, op)
    if gate_up.dim() != 2 or gate_up.stride(1) != 1 or gate_up.shape[1] != 2 * n:
        _capi.check(4, op)
    out = torch.empty((gate_up.shape[0], n), dtype=gate_up.dtype, device=gate_up.device)
    _call(_capi.lib().axb200_silu_mul_rows(gate_up.data_ptr(), gate_up.stride(0), n, gate_up.shape[0],
                                           out.data_ptr(), dt, _stream(gate_up)), op)
    return out


def decode_step_host(q_host, k_new_host, v_new_host, out_host, staging, k_pages, v_pages, block_table, seq_lens,
                     max_seq_len, theta=10000.0, pos=None, inv_freq=None, mrope_section=None, rotate=True):
    """One decode step whose activations live on the host: q/k_new/v_new/out are CPU tensors (pinned for
    asynchronous copies), `staging` = (q_dev, k_dev, v_dev, out_dev) device buffers of the same shapes.
    Copies in, rope + append, paged decode attention, copies out and waits; a single C-ABI call."""
    op = "decode_step_host"
    q_dev, k_dev, v_dev, out_dev = staging
    dt = _dt(q_dev, op)
    for t in (q_host, k_new_host, v_new_host, out_host):
        if t.is_cuda or not t.is_contiguous() or t.dtype != q_dev.dtype:
            _capi.check(1, op)
    batch, hq, d = q_dev.shape
    num_pages, hkv, page_tokens, _ = k_pages.shape
    mrope = mrope_section is not None
    h_sec, w_sec = (mrope_section[1], mrope_section[2]) if mrope else (0, 0)
    lib = _capi.lib()
    ws_bytes = lib.axb200_gqa_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), dt)
    ws = workspace(q_dev.device, ws_bytes)
    _call(lib.axb200_decode_step_host(
        q_host.data_ptr(), k_new_host.data_ptr(), v_new_host.data_ptr(), out_host.data_ptr(), q_dev.data_ptr(),
        k_dev.data_ptr(), v_dev.data_ptr(), out_dev.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), seq_lens.data_ptr(), _ptr(pos), _ptr(inv_freq), float(theta), int(rotate),
        int(mrope), h_sec, w_sec, batch, hq, hkv, d, page_tokens, block_table.shape[1], num_pages,
        int(max_seq_len), dt, ws.data_ptr(), ws.numel(), _stream(q_dev)), op)
    return out_host


def rope(x, pos_ids, theta: float = 10000.0):
    op = "rope"
    dt = _dt(x, op)
    if x.dim() != 3:
        _capi.check(3, op)
    rows, heads, dim = x.shape
    if pos_ids.dtype != torch.int64 or pos_ids.numel() != rows:
        _capi.check(3, op)
    x = _c(x)
    out = torch.empty_like(x)
    _call(_capi.lib().axb200_rope(x.data_ptr(), _c(pos_ids).data_ptr(), float(theta), out.data_ptr(),
                                        rows, heads, dim, dt, _stream(x)), op)
    return out


def rope_thd(x, pos, inv_freq, mrope_section):
    op = "rope_thd"
    dt = _dt(x, op)
    if x.dim() != 3:
        _capi.check(3, op)
    rows, heads, dim = x.shape
    if pos.dtype != torch.int64 or tuple(pos.shape) != (3, rows):
        _capi.check(4, op)
    if inv_freq.dtype != torch.float32 or tuple(inv_freq.shape) != (dim // 2,):
        _capi.check(4, op)
    x = _c(x)
    out = torch.empty_like(x)
    t, h, w = mrope_section
    _call(_capi.lib().axb200_rope_thd(x.data_ptr(), _c(pos).data_ptr(), _c(inv_freq).data_ptr(), t, h, w,
                                            out.data_ptr(), rows, heads, dim, dt, _stream(x)), op)
    return out


def rope_with_cos_sin(x, cos, sin):
    op = "rope_with_cos_sin"
    dt = _dt(x, op)
    rows, heads, dim = x.shape
    if tuple(cos.shape) != (rows, dim) or tuple(sin.shape) != (rows, dim) or cos.dtype != torch.float32:
        _capi.check(4, op)
    x = _c(x)
    out = torch.empty_like(x)
    _call(_capi.lib().axb200_rope_with_cos_sin(x.data_ptr(), _c(cos).data_ptr(), _c(sin).data_ptr(),
                                                     out.data_ptr(), rows, heads, dim, dt, _stream(x)), op)
    return out


def mrope_cos_sin(pos, inv_freq, h_sec: int, w_sec: int):
    op = "mrope_cos_sin"
    if pos.dim() != 2 or pos.shape[0] != 3 or pos.dtype != torch.int64:
        _capi.check(4, op)
    rows, half = pos.shape[1], inv_freq.shape[0]
    cos = torch.empty((rows, 2 * half), dtype=torch.float32, device=pos.device)
    sin = torch.empty_like(cos)
    _call(_capi.lib().axb200_mrope_cos_sin(_c(pos).data_ptr(), _c(inv_freq).data_ptr(), h_sec, w_sec,
                                                 cos.data_ptr(), sin.data_ptr(), rows, half, _stream(pos)), op)
    return cos, sin


def add_rms_norm(x, residual, weight, eps: float = 1e-6):
    """y = x + residual; out = y * rsqrt(mean(y^2) + eps) * weight.  Returns (y, out)."""
    op = "add_rms_norm"
    dt = _dt(x, op)
    if x.shape != residual.shape or x.dtype != residual.dtype:
        _capi.check(4, op)
    hidden = x.shape[-1]
    if weight.dim() != 1 or weight.shape[0] != hidden or weight.dtype != x.dtype:
        _capi.check(4, op)
    x, residual, weight = _c(x), _c(residual), _c(weight)
    y = torch.empty_like(x)
    out = torch.empty_like(x)
    _call(_capi.lib().axb200_add_rms_norm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), float(eps),
                                                y.data_ptr(), out.data_ptr(), x.numel() // hidden, hidden, dt,
                                                _stream(x)), op)
    return y, out


def silu_mul(gate, up):
    op = "silu_mul"
    dt = _dt(gate, op)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        _capi.check(4, op)
    gate, up = _c(gate), _c(up)
    out = torch.empty_like(gate)
    _call(_capi.lib().axb200_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), dt,
                                            _stream(gate)), op)
    return out


def rms_norm(x, weight, eps: float = 1e-5):
    op = "rms_norm"
    dt = _dt(x, op)
    cols = x.shape[-1]
    has_w = weight is not None and weight.numel() != 0
    if has_w and (weight.dim() != 1 or weight.shape[0] != cols or weight.dtype != x.dtype):
        _capi.check(4, op)
    x = _c(x)
    out = torch.empty_like(x)
    _call(_capi.lib().axb200_rms_norm(x.data_ptr(), _c(weight).data_ptr() if has_w else None, float(eps),
                                            out.data_ptr(), x.numel() // cols, cols, dt, _stream(x)), op)
    return out


def linear_nobias(x, weight):
    """x (rows, in) . weight (out, in)^T -> (rows, out): one cuBLASLt call whose algorithm is timed and
    chosen on the first use of a shape (so call it once eagerly before capturing it)."""
    op = "linear_nobias"
    dt = _dt(x, op)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or weight.dtype != x.dtype:
        _capi.check(4, op)  # SHAPE_MISMATCH
    x, weight = _c(x), _c(weight)
    out = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
    _call(_capi.lib().axb200_linear_nobias(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.shape[0], weight.shape[0],
                                           x.shape[1], dt, _stream(x)), op)
    return out


def cast(x, dtype):
    """Tensor.cast_to on the device (src/core/cuda/tensor/kernel.cu:175-193): float16 <-> float32."""
    op = "cast"
    src = _dt(x, op)
    if dtype == x.dtype:
        return x
    if {x.dtype, dtype} != {torch.float16, torch.float32}:
        raise RuntimeError(f"{op}: only float16 <-> float32")
    if not x.is_contiguous():
        raise RuntimeError(f"{op}: tensor must be contiguous")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    dst = _DTYPES[dtype]
    _call(_capi.lib().axb200_cast(x.data_ptr(), src, out.data_ptr(), dst, x.numel(), _stream(x)), op)
    return out


def concat(a, b, axis: int):
    op = "concat"
    if a.dim() < 1 or a.dim() != b.dim() or a.dtype != b.dtype:
        _capi.check(1, op)
    nd = a.dim()
    ax = axis + nd if axis < 0 else axis
    if ax < 0 or ax >= nd:
        _capi.check(1, op)
    for i in range(nd):
        if i != ax and a.shape[i] != b.shape[i]:
            _capi.check(4, op)
    a, b = _c(a), _c(b)
    shape = list(a.shape)
    shape[ax] += b.shape[ax]
    out = torch.empty(shape, dtype=a.dtype, device=a.device)
    outer = 1
    for i in range(ax):
        outer *= a.shape[i]
    es = a.element_size()
    a_bytes = (a.numel() // max(outer, 1)) * es
    b_bytes = (b.numel() // max(outer, 1)) * es
    _call(_capi.lib().axb200_concat(a.data_ptr(), b.data_ptr(), out.data_ptr(), outer, a_bytes, b_bytes,
                                          _stream(a)), op)
    return out


def embedding(ids, table):
    """table[ids]: ids int32/int64 of any shape, table (vocab, hidden) -> ids.shape + (hidden,)."""
    op = "embedding"
    dt = _dt(table, op)
    if table.dim() != 2 or ids.dim() < 1:
        _capi.check(1, op)
    code = {torch.int64: _capi.INT64, torch.int32: _capi.INT32}.get(ids.dtype)
    if code is None:
        _capi.check(3, op)
    ids, table = _c(ids), _c(table)
    out = torch.empty(tuple(ids.shape) + (table.shape[1],), dtype=table.dtype, device=table.device)
    _call(_capi.lib().axb200_embedding(ids.data_ptr(), code, table.data_ptr(), out.data_ptr(), ids.numel(),
                                       table.shape[0], table.shape[1], dt, _stream(table)), op)
    return out


def argmax_last_dim(x):
    """Index of the first maximum along the last dim -> int64 tensor of shape x.shape[:-1]."""
    op = "argmax_last_dim"
    dt = _dt(x, op)
    if x.dim() < 1:
        _capi.check(1, op)
    x = _c(x)
    cols = x.shape[-1]
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    _call(_capi.lib().axb200_argmax_last_dim(x.data_ptr(), out.data_ptr(), x.numel() // cols, cols, dt, _stream(x)), op)
    return out


def scaled_dot_product_attention(q, k, v, is_causal: bool = False):
    """q (sq, hq, d), k/v (skv, hkv, d) -> (sq, hq, d); with is_causal row t sees keys [0, t]
    (axono/python/axono/core/ops/sequence.py scaled_dot_product_attention of the reference)."""
    op = "scaled_dot_product_attention"
    dt = _dt(q, op)
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        _capi.check(1, op)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        _capi.check(3, op)
    sq, hq, d = q.shape
    skv, hkv, dk = k.shape
    if dk != d or tuple(v.shape) != (skv, hkv, d) or hkv == 0 or hq % hkv != 0:
        _capi.check(4, op)
    q, k, v = _c(q), _c(k), _c(v)
    out = torch.empty_like(q)
    lib = _capi.lib()
    ws = workspace(q.device, lib.axb200_sdpa_workspace_bytes(sq, hq, hkv, d, skv, dt))
    _call(lib.axb200_sdpa(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), sq, hq, hkv, d, skv,
                          int(bool(is_causal)), dt, ws.data_ptr(), ws.numel(), _stream(q)), op)
    return out
