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


class Scratch:
    """The decode calls' workspace as one tensor that lives as long as its user (a graph that was
    captured with it keeps its address)."""

    def __init__(self, batch, hq, hkv, d, max_seq_len, dtype, device: str = "cuda"):
        lx = native.load()
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
