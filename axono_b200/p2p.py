"""Peer-mapped buffers for the fused attention + all-gather kernel (KV heads sharded across the GPUs
of one node, one process per GPU).

`PeerGather` owns, on each rank, `slots` gathered buffers (batch, hq_total, d), a flag array and two
state words, all in one CUDA-IPC allocation; the constructor exchanges the IPC handles through the
process group (any backend - only Python objects travel) and maps every peer's allocation.  After
that no library collective is involved: `ops.gqa_decode_attention_paged(..., gather=(pg, slot))`
makes every rank's kernel store its heads into every rank's buffer `slot` and returns this rank's
buffer, complete, as a tensor.  Successive calls must use different slots (one per layer).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _capi
from .kv_cache import _DeviceView

_ALIGN = 256


class PeerGather:
    def __init__(self, batch: int, hq_total: int, d: int, dtype=torch.float16, slots: int = 2, group=None,
                 kind: str = "heads"):
        """kind "heads": slots hold gathered head outputs (batch, hq_total, d) of `dtype`;
        kind "records": slots hold context-parallel records (batch, hq_total, world, d + 2) fp32."""
        if kind not in ("heads", "records"):
            raise ValueError(kind)
        self.kind = kind
        if slots < 2:
            raise RuntimeError("PeerGather needs at least two slots (successive calls must alternate)")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise RuntimeError("PeerGather supports up to 8 ranks (one NVSwitch node)")
        self.batch, self.hq_total, self.d, self.dtype, self.slots = batch, hq_total, d, dtype, slots
        es = torch.tensor([], dtype=dtype).element_size()
        raw = batch * hq_total * d * es if kind == "heads" else batch * hq_total * self.world * (d + 2) * 4
        self.slot_bytes = (raw + _ALIGN - 1) // _ALIGN * _ALIGN
        self.flags_off = self.slot_bytes * slots
        self.state_off = self.flags_off + _ALIGN
        total = self.state_off + _ALIGN
        lib = _capi.lib()
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        _capi.check(lib.axb200_p2p_alloc(total, C.byref(ptr), handle), "p2p_alloc")
        self.local_ptr = ptr.value
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
        else:
            handles[0] = bytes(handle.raw)
        self.peer_ptrs, self._opened = [], []
        for r in range(self.world):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            p = C.c_void_p()
            _capi.check(lib.axb200_p2p_open(C.create_string_buffer(handles[r], 64), C.byref(p)), "p2p_open")
            self.peer_ptrs.append(p.value)
            self._opened.append(p.value)
        if self.world > 1:
            dist.barrier(group=group)  # every rank has mapped every peer before the first kernel
        arr = C.c_void_p * self.world
        self._flags = arr(*[p + self.flags_off for p in self.peer_ptrs])
        self._outs = [arr(*[p + s * self.slot_bytes for p in self.peer_ptrs]) for s in range(slots)]
        typestr = {torch.float16: "<f2", torch.float32: "<f4"}[dtype]
        shape, ts = ((batch, hq_total, d), typestr) if kind == "heads" else ((batch, hq_total, self.world, d + 2), "<f4")
        self._views = [torch.as_tensor(_DeviceView(self.local_ptr + s * self.slot_bytes, shape, ts),
                                       device=torch.device("cuda", torch.cuda.current_device()))
                       for s in range(slots)]

    def out_ptrs(self, slot: int):
        return self._outs[slot]

    @property
    def flag_ptrs(self):
        return self._flags

    @property
    def state_ptr(self) -> int:
        return self.local_ptr + self.state_off

    def tensor(self, slot: int) -> torch.Tensor:
        """This rank's gathered buffer `slot`, (batch, hq_total, d), aliasing the IPC allocation."""
        return self._views[slot]

    def close(self):
        lib = _capi.lib()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody unmaps while a peer may still write
        for p in self._opened:
            lib.axb200_p2p_close(p)
        self._opened = []
        if self.local_ptr:
            self._views = []
            lib.axb200_p2p_free(self.local_ptr)
            self.local_ptr = 0
