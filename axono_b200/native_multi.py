"""Multi-GPU plumbing of the decode path on the native runtime (no PyTorch): peer-mapped buffers
exchanged through `axono_b200.rendezvous`, and the two decode calls that store into them.

One process per GPU.  The only things that cross a process boundary on the host are the 64-byte CUDA
IPC handles at set-up and barriers; everything per step happens inside the kernels (plain stores to
peer-mapped pointers over NVLink, generation flags with bounded waits).

    rdv = Rendezvous.from_env()
    bufs = PeerBuffers(rdv, batch, hq_total, d, lx.DataType.FLOAT16, slots=28, device="cuda:3")
    attn = attend_gather(q_local, arena, layer, max_len, bufs, slot)      # (batch, hq_total, d), this rank's copy

Tensors are `libaxono.Tensor`s; C-ABI calls go through ctypes with their device pointers.
"""
from __future__ import annotations

import ctypes as C

from . import _capi, native
from .rendezvous import Rendezvous

_ALIGN = 256


def _dtype_code(lx, dtype) -> int:
    return {lx.DataType.FLOAT16: _capi.FLOAT16, lx.DataType.FLOAT32: _capi.FLOAT32}[dtype]


class PeerBuffers:
    """On every rank: `slots` buffers, a flag array and two state words in one CUDA-IPC allocation,
    mapped into every other rank.  kind "heads": a slot is a gathered head output (batch, hq_total, d)
    of `dtype`; kind "records": a slot holds context-parallel records (batch, hq_total, world, d + 2)
    fp32.  Successive calls must use different slots (one per layer)."""

    def __init__(self, rdv: Rendezvous, batch: int, hq_total: int, d: int, dtype, slots: int = 2,
                 kind: str = "heads", device: str = "cuda"):
        if kind not in ("heads", "records"):
            raise ValueError(kind)
        if slots < 2:
            raise RuntimeError("PeerBuffers needs at least two slots (successive calls must alternate)")
        if rdv.world > 8:
            raise RuntimeError("PeerBuffers supports up to 8 ranks (one NVSwitch node)")
        lx = native.load()
        self.lx, self.rdv, self.kind, self.device = lx, rdv, kind, device
        self.world, self.rank = rdv.world, rdv.rank
        self.batch, self.hq_total, self.d, self.dtype, self.slots = batch, hq_total, d, dtype, slots
        es = 2 if dtype == lx.DataType.FLOAT16 else 4
        raw = batch * hq_total * d * es if kind == "heads" else batch * hq_total * self.world * (d + 2) * 4
        self.slot_bytes = (raw + _ALIGN - 1) // _ALIGN * _ALIGN
        self.flags_off = self.slot_bytes * slots
        self.state_off = self.flags_off + _ALIGN
        total = self.state_off + _ALIGN
        lib = _capi.lib()
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        _capi.check(lib.axb200_p2p_alloc(total, C.byref(ptr), handle), "p2p_alloc")
        self.local_ptr = ptr.value
        handles = rdv.all_gather(bytes(handle.raw))
        self.peer_ptrs, self._opened = [], []
        for r in range(self.world):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            p = C.c_void_p()
            _capi.check(lib.axb200_p2p_open(C.create_string_buffer(handles[r], 64), C.byref(p)), "p2p_open")
            self.peer_ptrs.append(p.value)
            self._opened.append(p.value)
        rdv.barrier()  # every rank has mapped every peer before the first kernel
        arr = C.c_void_p * self.world
        self._flags = arr(*[p + self.flags_off for p in self.peer_ptrs])
        self._outs = [arr(*[p + s * self.slot_bytes for p in self.peer_ptrs]) for s in range(slots)]
        shape = [batch, hq_total, d] if kind == "heads" else [batch, hq_total, self.world, d + 2]
        vdt = dtype if kind == "heads" else lx.DataType.FLOAT32
        self._views = [lx.Tensor.from_device_ptr(self.local_ptr + s * self.slot_bytes, vdt, shape, device)
                       for s in range(slots)]

    def out_ptrs(self, slot: int):
        return self._outs[slot]

    @property
    def flag_ptrs(self):
        return self._flags

    @property
    def state_ptr(self) -> int:
        return self.local_ptr + self.state_off

    def tensor(self, slot: int):
        """This rank's buffer `slot` as a tensor that aliases the IPC allocation."""
        return self._views[slot]

    def close(self) -> None:
        lib = _capi.lib()
        self.lx.synchronize()
        self.rdv.barrier()  # nobody unmaps while a peer may still write
        for p in self._opened:
            lib.axb200_p2p_close(p)
        self._opened = []
        if self.local_ptr:
            self._views = []
            lib.axb200_p2p_free(self.local_ptr)
            self.local_ptr = 0


class NcclGather:
    """All-gather of per-head attention outputs through NCCL - the library form of what `attend_gather`
    fuses into the attention kernel.  The communicator is created here (every rank constructs one,
    before any stream capture); `gather(local)` enqueues ncclAllGather and a re-layout on the current
    stream and returns (batch, hq_total, d), so it can be recorded into a CUDA graph."""

    def __init__(self, rdv: Rendezvous, batch: int, hq_local: int, d: int, dtype, device: str = "cuda"):
        lx = native.load()
        lib = _capi.lib()
        self.lx, self.rdv, self.world, self.device = lx, rdv, rdv.world, device
        self.batch, self.hq_local, self.d, self.dtype = batch, hq_local, d, dtype
        uid = C.create_string_buffer(128)
        if rdv.rank == 0:
            _capi.check(lib.axb200_nccl_unique_id(uid), "nccl_unique_id")
        uid = C.create_string_buffer(rdv.all_gather(bytes(uid.raw))[0], 128)
        comm = C.c_void_p()
        _capi.check(lib.axb200_nccl_init(uid, rdv.world, rdv.rank, C.byref(comm)), "nccl_init")
        self._comm = comm
        self._tmp = lx.Tensor(dtype, [self.world, batch, hq_local, d], device)
        self._out = lx.Tensor(dtype, [batch, self.world * hq_local, d], device)
        rdv.barrier()

    def gather(self, local):
        """local (batch, hq_local, d) of this rank -> this rank's copy of (batch, hq_total, d)."""
        lx, lib = self.lx, _capi.lib()
        if tuple(local.shape) != (self.batch, self.hq_local, self.d) or local.dtype != self.dtype:
            raise RuntimeError("NcclGather.gather: tensor does not match the communicator's buffers")
        st = lx.current_stream()
        _capi.check(lib.axb200_nccl_all_gather(self._comm, local.data_ptr, self._tmp.data_ptr, local.num_bytes, st),
                    "nccl_all_gather")
        _capi.check(lib.axb200_swap_leading_dims(self._tmp.data_ptr, self._out.data_ptr, self.world, self.batch,
                                                 local.num_bytes // self.batch, st), "swap_leading_dims")
        return self._out

    def close(self) -> None:
        """Destroys the communicator.  Reset every graph that recorded `gather` first: NCCL's destroy waits
        for graphs that hold the communicator's work, for good if one is still alive."""
        if self._comm:
            self.lx.synchronize()
            self.rdv.barrier()
            _capi.lib().axb200_nccl_destroy(self._comm)
            self._comm = None


class Scratch:
    """The decode calls' workspace as one tensor that lives as long as its user (a graph that was
    captured with it keeps its address)."""

    def __init__(self, batch, hq, hkv, d, max_seq_len, dtype, device: str = "cuda", step: bool = False):
        lx = native.load()
        if step:  # the one-operator step: the partials plus room for a rotated q
            n = int(_capi.lib().axb200_decode_step_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), _dtype_code(lx, dtype)))
        else:
            n = int(lx.gqa_workspace_bytes(batch, hq, hkv, d, int(max_seq_len), dtype))
        self.tensor = lx.Tensor(lx.DataType.INT8, [max(n, 256)], device)

    @property
    def ptr(self) -> int:
        return self.tensor.data_ptr

    @property
    def nbytes(self) -> int:
        return self.tensor.num_bytes


def _arena_args(lx, arena, layer):
    g = arena.geometry()
    return g, (arena.k_pages_ptr(layer), arena.v_pages_ptr(layer), arena.block_table_ptr, arena.seq_lens_ptr)


def attend_gather(q, arena, layer: int, max_seq_len: int, bufs: PeerBuffers, slot: int, scratch: Scratch):
    """Decode attention of this rank's heads q (batch, hq_local, d) over its share of the KV heads; the
    kernel stores the rows into every rank's buffer `slot` and exchanges flags, so the returned tensor
    - this rank's buffer, (batch, hq_total, d) - holds all heads when the call's kernel completes."""
    lx = native.load()
    g, (kp, vp, bt, sl) = _arena_args(lx, arena, layer)
    batch, hq, d = q.shape
    if bufs.kind != "heads" or bufs.batch != batch or bufs.d != d or bufs.hq_total != hq * bufs.world:
        raise RuntimeError("attend_gather: buffers do not match the call")
    _capi.check(_capi.lib().axb200_gqa_decode_paged_gather(
        q.data_ptr, kp, vp, bt, sl, batch, hq, g["hkv"], d, g["page_tokens"], g["max_blocks"], g["num_pages"],
        int(max_seq_len), _dtype_code(lx, q.dtype), scratch.ptr, scratch.nbytes, bufs.out_ptrs(slot), bufs.flag_ptrs,
        bufs.state_ptr, bufs.world, bufs.rank, bufs.hq_total, lx.current_stream()), "gqa_decode_paged_gather")
    return bufs.tensor(slot)


def qkv_decode_step(qkv, hq: int, arena, layer: int, max_seq_len: int, scratch: Scratch, q_norm_w=None, k_norm_w=None,
                    eps: float = 1e-6, inv_freq=None, theta: float = 1e6, rotate: bool = True, mrope_section=None,
                    slot_delta: int = 0, advance: bool = True, out=None, bufs: PeerBuffers = None, slot: int = 0):
    """The tower layer's decode step as one operator, straight from the QKV projection's output qkv (batch, ld):
    per-head RMS norm of q and k, rotation, append, attention - one launch where the library can
    (`axb200_qkv_decode_step_paged`).  Without `bufs` the result goes to `out` (batch, hq, d), which is
    returned; with `bufs` (heads sharded over the ranks) the rows go into every rank's gathered buffer `slot`
    and this rank's buffer (batch, hq_total, d) is returned.  `scratch` must be a `Scratch(..., step=True)`."""
    lx = native.load()
    g, (kp, vp, bt, sl) = _arena_args(lx, arena, layer)
    batch, ld = qkv.shape
    d = g["d"]
    mrope = mrope_section is not None
    h_sec, w_sec = (int(mrope_section[1]), int(mrope_section[2])) if mrope else (0, 0)
    if bufs is not None:
        if bufs.kind != "heads" or bufs.batch != batch or bufs.d != d or bufs.hq_total != hq * bufs.world:
            raise RuntimeError("qkv_decode_step: buffers do not match the call")
        peers = (bufs.out_ptrs(slot), bufs.flag_ptrs, bufs.state_ptr, bufs.world, bufs.rank, bufs.hq_total)
        out_ptr = None
    else:
        if out is None:
            out = lx.Tensor(qkv.dtype, [batch, hq, d], qkv.device)
        peers = (None, None, None, 0, 0, hq)
        out_ptr = out.data_ptr
    _capi.check(_capi.lib().axb200_qkv_decode_step_paged(
        qkv.data_ptr, int(ld), q_norm_w.data_ptr if q_norm_w is not None else None,
        k_norm_w.data_ptr if k_norm_w is not None else None, float(eps), out_ptr, kp, vp, bt, sl, None,
        inv_freq.data_ptr if inv_freq is not None else None, float(theta), int(rotate), int(mrope), h_sec, w_sec, batch, hq,
        g["hkv"], d, g["page_tokens"], g["max_blocks"], g["num_pages"], int(max_seq_len), _dtype_code(lx, qkv.dtype),
        int(slot_delta), int(advance), scratch.ptr, scratch.nbytes, *peers, lx.current_stream()), "qkv_decode_step_paged")
    return bufs.tensor(slot) if bufs is not None else out


def attend_context_parallel(q, out, arena, layer: int, max_seq_len: int, bufs: PeerBuffers, slot: int, scratch: Scratch):
    """Context-parallel decode: every rank caches a share of each sequence's tokens; the ranks exchange
    un-normalised partials over peer memory and each writes the full result into `out`."""
    lx = native.load()
    g, (kp, vp, bt, sl) = _arena_args(lx, arena, layer)
    batch, hq, d = q.shape
    if bufs.kind != "records" or bufs.batch != batch or bufs.d != d or bufs.hq_total != hq:
        raise RuntimeError("attend_context_parallel: buffers do not match the call")
    _capi.check(_capi.lib().axb200_gqa_decode_paged_cp(
        q.data_ptr, out.data_ptr, kp, vp, bt, sl, batch, hq, g["hkv"], d, g["page_tokens"], g["max_blocks"],
        g["num_pages"], int(max_seq_len), _dtype_code(lx, q.dtype), scratch.ptr, scratch.nbytes, bufs.out_ptrs(slot),
        bufs.flag_ptrs, bufs.state_ptr, bufs.world, bufs.rank, lx.current_stream()), "gqa_decode_paged_cp")
    return out


def write_tokens(arena, layer: int, seq: int, k, v, start: int = 0) -> None:
    """Stores k, v - host arrays (n, hkv, d) of the arena's dtype - as tokens start .. start+n-1 of
    sequence `seq`, as they are (no rotation).  The block table must be on the device (arena.sync())
    and the sequence must hold the pages.  The caller sets the lengths."""
    import numpy as np

    lx = native.load()
    g = arena.geometry()
    n, hkv, d = k.shape
    if hkv != g["hkv"] or d != g["d"] or v.shape != k.shape:
        raise RuntimeError("write_tokens: k / v do not match the arena")
    if n == 0:
        return
    dev = "cuda:%d" % lx.current_device()
    kd = lx.Tensor.from_numpy(np.ascontiguousarray(k), dev)
    vd = lx.Tensor.from_numpy(np.ascontiguousarray(v), dev)
    if kd.dtype != g["dtype"]:
        raise RuntimeError("write_tokens: dtype differs from the arena's")
    row = arena.block_table_ptr + seq * g["max_blocks"] * 4
    _capi.check(_capi.lib().axb200_kv_prefill_write(
        None, kd.data_ptr, vd.data_ptr, arena.k_pages_ptr(layer), arena.v_pages_ptr(layer), row, None, None, 1.0, 0, 0,
        0, 0, n, 0, hkv, d, g["page_tokens"], g["max_blocks"], g["num_pages"], int(start), _dtype_code(lx, kd.dtype),
        lx.current_stream()), "kv_prefill_write")
    lx.synchronize()  # kd / vd may go back to the pool now


def multi_gpu_parity(rdv: Rendezvous, device: str, iterations: int = 6) -> dict:
    """The two cross-GPU forms of decode attention against the same attention computed locally, on small
    seeded inputs: (gather) KV heads sharded, rows stored into every rank's buffer - against attention
    over all heads of an unsharded copy of the cache; (cp) every sequence's pages dealt round-robin to
    the ranks, partials exchanged and merged - against the unsharded cache.  Returns the largest
    normalised errors over all ranks.  Every rank of the job must call it."""
    import numpy as np

    from . import partition

    lx = native.load()
    f16 = lx.DataType.FLOAT16
    world, rank = rdv.world, rdv.rank
    rng = np.random.default_rng(7000)
    hq, hkv, d, page = 16, 8, 128, 64
    lens = [3000, 2999, 64, 1000, 2049]
    B, L = len(lens), max(lens)
    q = rng.standard_normal((B, hq, d)).astype(np.float16)
    k = (0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float16)
    v = (0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float16)

    def arena_of(n_heads, rows_k, rows_v, lengths):
        blocks = (L + page - 1) // page
        a = lx.KVArena(1, B * blocks, n_heads, page, d, f16, B, blocks)
        for _ in range(B):
            a.alloc_seq(L)
        a.sync()
        for b in range(B):
            write_tokens(a, 0, b, rows_k[b], rows_v[b])
        a.set_seq_lens(np.asarray(lengths, np.int32))
        return a

    def rel(got, want):
        got, want = got.astype(np.float32), want.astype(np.float32)
        return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))

    full = arena_of(hkv, [k[b, : lens[b]] for b in range(B)], [v[b, : lens[b]] for b in range(B)], lens)
    to_dev = lambda a: lx.Tensor.from_numpy(np.ascontiguousarray(a), device)  # noqa: E731

    # ---- KV heads sharded, attention fused with the all-gather ----
    kvh, qh = partition.shard_kv_heads(hq, hkv, world, rank)
    local = arena_of(len(kvh), [k[b, : lens[b], kvh.start:kvh.stop] for b in range(B)],
                     [v[b, : lens[b], kvh.start:kvh.stop] for b in range(B)], lens)
    bufs = PeerBuffers(rdv, B, hq, d, f16, slots=2, device=device)
    scratch = Scratch(B, len(qh), len(kvh), d, L, f16, device)
    err_gather = 0.0
    for it in range(iterations):  # several generations, alternating buffers, another q every time
        qi = (q.astype(np.float32) * (1.0 + 0.01 * it)).astype(np.float16)
        want = lx.gqa_decode_attention_paged(to_dev(qi), full, 0, L).numpy()
        got = attend_gather(to_dev(qi[:, qh.start:qh.stop]), local, 0, L, bufs, it % 2, scratch)
        lx.synchronize()
        err_gather = max(err_gather, rel(got.numpy(), want))
    bufs.close()

    # ---- context parallel: pages dealt round-robin, one sequence of which some ranks hold nothing ----
    lens_cp = [3000, 2999, 40, 1000, 2049]
    full_cp = arena_of(hkv, [k[b, : lens_cp[b]] for b in range(B)], [v[b, : lens_cp[b]] for b in range(B)], lens_cp)
    mine = [partition.shard_tokens_by_page(lens_cp[b], page, world, rank) for b in range(B)]
    part = arena_of(hkv, [k[b, mine[b]] for b in range(B)], [v[b, mine[b]] for b in range(B)], [len(m) for m in mine])
    recs = PeerBuffers(rdv, B, hq, d, f16, slots=2, kind="records", device=device)
    scratch_cp = Scratch(B, hq, hkv, d, L, f16, device)
    out = lx.Tensor(f16, [B, hq, d], device)
    err_cp = 0.0
    for it in range(iterations):
        qi = (q.astype(np.float32) * (1.0 + 0.01 * it)).astype(np.float16)
        want = lx.gqa_decode_attention_paged(to_dev(qi), full_cp, 0, L).numpy()
        attend_context_parallel(to_dev(qi), out, part, 0, L, recs, it % 2, scratch_cp)
        lx.synchronize()
        err_cp = max(err_cp, rel(out.numpy(), want))
    recs.close()
    bits = int(lx.device_error_bits())
    return {"gather": rdv.max(err_gather), "cp": rdv.max(err_cp), "ranks": world, "device_error_bits": int(rdv.max(bits)),
            "tolerance": 1e-3}
