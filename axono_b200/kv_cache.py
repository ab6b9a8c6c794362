"""KV-cache components behind the reference's `KVCache` interface
(axono/python/axono/nn/kv_cache.py:41-68: update / get / reset / __len__).

`PagedKVCache` replaces `DynamicKVCache` (kv_cache.py:71-117), whose `update` re-copies the whole
cache with `concat` every step: here pages have fixed addresses, an append writes one token per
sequence, and the sequence lengths live in device memory so a captured CUDA graph follows the
growing cache.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _capi, ops


class KVCache:
    """Abstract cache: subclasses implement update / get / reset / __len__."""

    def update(self, layer_idx: int, k_new, v_new):  # pragma: no cover
        raise NotImplementedError

    def append_qkv(self, layer_idx: int, qkv, n_q_heads, q_norm_weight=None, k_norm_weight=None, eps=1e-6,
                   pos=None, inv_freq=None, theta=10000.0, mrope_section=None):
        """Per-head norm + rope + append straight from the QKV projection output; returns q (batch,hq,d)."""
        first = layer_idx == 0
        q = ops.qkv_norm_rope_append(qkv, n_q_heads, q_norm_weight, k_norm_weight, eps, self.k_pages[layer_idx],
                                     self.v_pages[layer_idx], self.block_table, self.seq_lens, pos=pos,
                                     inv_freq=inv_freq, theta=theta, mrope_section=mrope_section, rotate=True,
                                     advance=first, slot_delta=0 if first else -1)
        if first:
            self._host_len_bound += 1
        return q

    def step_host(self, q_host, k_new_host, v_new_host, out_host, theta=10000.0, pos=None, inv_freq=None,
                  mrope_section=None, layer_idx: int = 0):
        """One decode step with host activations (pinned CPU tensors): stage in, rope + append, attend,
        copy the output back and wait - a single C-ABI call.  Returns out_host."""
        st = getattr(self, "_staging", None)
        if st is None or st[0].dtype != q_host.dtype or st[0].shape != q_host.shape:
            mk = lambda t: torch.empty(t.shape, dtype=t.dtype, device=self.device)  # noqa: E731
            st = (mk(q_host), mk(k_new_host), mk(v_new_host), mk(q_host))
            self._staging = st
        self._host_len_bound = min(self.max_seq_len, self._host_len_bound + 1)
        ops.decode_step_host(q_host, k_new_host, v_new_host, out_host, st, self.k_pages[layer_idx],
                             self.v_pages[layer_idx], self.block_table, self.seq_lens, self._host_len_bound,
                             theta=theta, pos=pos, inv_freq=inv_freq, mrope_section=mrope_section)
        return out_host

    def prefill(self, layer_idx: int, b: int, q, k, v, pos=None, inv_freq=None, theta=10000.0, mrope_section=None,
                rotate=True, set_length=True):
        """Stores a prompt: k, v (n,hkv,d) of sequence `b` go to slots 0..n-1 with k rotated (q (n,hq,d)
        too, in place, when given).  With set_length the sequence's length becomes n."""
        ops.kv_prefill_write(q, k, v, self.k_pages[layer_idx], self.v_pages[layer_idx], self.block_table[b], 0,
                             pos=pos, inv_freq=inv_freq, theta=theta, mrope_section=mrope_section, rotate=rotate)
        if set_length:
            self.seq_lens[b : b + 1].fill_(k.shape[0])
            self._host_len_bound = max(self._host_len_bound, int(k.shape[0]))
        return q

    def get(self, layer_idx: int):  # pragma: no cover
        raise NotImplementedError

    def reset(self):  # pragma: no cover
        raise NotImplementedError

    def __len__(self) -> int:  # pragma: no cover
        raise NotImplementedError


class PagedKVCache(KVCache):
    """Per-layer page pools (num_pages, n_kv_heads, page_tokens, head_dim) shared by `batch`
    sequences, one block table and one device-resident length vector per cache.

    All layers share the block table and `seq_lens`, which advances once per decode step: layer 0's
    append writes slot `len` and advances, so that every layer's attention sees the new token; the
    other layers write slot `len - 1` and leave the lengths alone.
    """

    def __init__(self, n_layers, batch, n_kv_heads, head_dim, max_seq_len, dtype=torch.float16,
                 device="cuda", page_tokens=64, page_order=None):
        if page_tokens % 64 != 0:
            raise RuntimeError("PagedKVCache: page_tokens must be a multiple of 64")
        self.n_layers, self.batch = n_layers, batch
        self.n_kv_heads, self.head_dim = n_kv_heads, head_dim
        self.page_tokens = page_tokens
        self.max_blocks = (max_seq_len + page_tokens - 1) // page_tokens
        self.max_seq_len = self.max_blocks * page_tokens
        self.num_pages = batch * self.max_blocks
        self.dtype, self.device = dtype, torch.device(device)
        shape = (self.num_pages, n_kv_heads, page_tokens, head_dim)
        # zero-filled like every new reference tensor (src/core/cuda/detail.cu:217-247)
        self.k_pages = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.v_pages = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        if page_order is None:
            page_order = torch.arange(self.num_pages, dtype=torch.int32)
        self.block_table = page_order.to(torch.int32).reshape(batch, self.max_blocks).contiguous().to(device)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=device)
        self._host_len_bound = 0  # host-side upper bound of seq_lens (sizes grids, no sync)

    # -- reference interface ------------------------------------------------------------------
    def update(self, layer_idx: int, k_new, v_new):
        """Appends one token per sequence: k_new/v_new (batch, n_kv_heads, head_dim), no rotation."""
        first = layer_idx == 0
        ops.kv_append_rope(None, k_new, v_new, self.k_pages[layer_idx], self.v_pages[layer_idx],
                           self.block_table, self.seq_lens, rotate=False, advance=first,
                           slot_delta=0 if first else -1)
        if first:
            self._host_len_bound += 1

    def append_rope(self, layer_idx: int, q, k_new, v_new, pos=None, inv_freq=None, theta=10000.0,
                    mrope_section=None):
        """rope(q) in place + rope(k_new) + append of (k_new, v_new) in one launch."""
        first = layer_idx == 0
        ops.kv_append_rope(q, k_new, v_new, self.k_pages[layer_idx], self.v_pages[layer_idx],
                           self.block_table, self.seq_lens, pos=pos, inv_freq=inv_freq, theta=theta,
                           mrope_section=mrope_section, rotate=True, advance=first,
                           slot_delta=0 if first else -1)
        if first:
            self._host_len_bound += 1
        return q

    def step(self, layer_idx: int, q, k_new, v_new, out=None, pos=None, inv_freq=None, theta=10000.0,
             mrope_section=None):
        """append_rope + attend as one operator (one launch where the library can); q is not modified."""
        bound = self.max_seq_len if torch.cuda.is_current_stream_capturing() else min(self.max_seq_len,
                                                                                      self._host_len_bound + 1)
        out = ops.decode_step_paged(q, k_new, v_new, self.k_pages[layer_idx], self.v_pages[layer_idx], self.block_table,
                                    self.seq_lens, max(bound, 1), out=out, pos=pos, inv_freq=inv_freq, theta=theta,
                                    mrope_section=mrope_section)
        self._host_len_bound += 1
        return out

    def get(self, layer_idx: int):
        """(k_pages, v_pages, block_table, seq_lens) of the layer - the paged equivalent of the
        reference's (k_full, v_full)."""
        return self.k_pages[layer_idx], self.v_pages[layer_idx], self.block_table, self.seq_lens

    def attend(self, layer_idx: int, q, out=None, gather=None, window: int = 0, context_parallel=None):
        """Decode attention of q (batch, hq, d) over the layer's cache.  The grid is sized from a
        host-side upper bound of the lengths; while a CUDA graph is being captured that bound is the
        capacity, so replays stay correct as the cache grows."""
        bound = self._host_len_bound
        if torch.cuda.is_current_stream_capturing():
            bound = self.max_seq_len
        bound = min(self.max_seq_len, bound)
        return ops.gqa_decode_attention_paged(q, self.k_pages[layer_idx], self.v_pages[layer_idx],
                                              self.block_table, self.seq_lens, max(bound, 1), out=out,
                                              gather=gather, window=window or getattr(self, "window", 0),
                                              context_parallel=context_parallel)

    def note_replayed(self, steps: int = 1):
        """Tells the host-side bound that `steps` captured decode steps have been replayed."""
        self._host_len_bound = min(self.max_seq_len, self._host_len_bound + steps)

    def reset(self):
        self.seq_lens.zero_()
        self._host_len_bound = 0

    def __len__(self) -> int:
        return int(self.seq_lens.max().item()) if self.batch else 0

    # -- bulk fill (prefill stand-in for tests and benchmarks) -----------------------------------
    def fill(self, layer_idx: int, k, v, lens):
        """Writes k/v (batch, L, n_kv_heads, head_dim) token-major into the pages and sets the
        lengths (host list or tensor).  Data movement only; not a hot-path operator."""
        lens_t = torch.as_tensor(lens, dtype=torch.int32)
        L = k.shape[1]
        nb = (L + self.page_tokens - 1) // self.page_tokens
        pad = nb * self.page_tokens - L
        for src, pool in ((k, self.k_pages[layer_idx]), (v, self.v_pages[layer_idx])):
            if pad:
                src = torch.nn.functional.pad(src, (0, 0, 0, 0, 0, pad))
            blk = src.reshape(self.batch, nb, self.page_tokens, self.n_kv_heads, self.head_dim)
            blk = blk.permute(0, 1, 3, 2, 4).reshape(self.batch * nb, self.n_kv_heads, self.page_tokens,
                                                     self.head_dim)
            idx = self.block_table[:, :nb].reshape(-1).long()
            pool[idx] = blk.to(pool.dtype)
        self.seq_lens.copy_(lens_t)
        self._host_len_bound = int(lens_t.max().item())

    def gather(self, layer_idx: int, b: int):
        """Sequence b's cache as token-major (len, n_kv_heads, head_dim) tensors (for checks)."""
        n = int(self.seq_lens[b].item())
        nb = (n + self.page_tokens - 1) // self.page_tokens
        idx = self.block_table[b, :nb].long()
        outs = []
        for pool in (self.k_pages[layer_idx], self.v_pages[layer_idx]):
            t = pool[idx].permute(0, 2, 1, 3).reshape(nb * self.page_tokens, self.n_kv_heads, self.head_dim)
            outs.append(t[:n].contiguous())
        return outs[0], outs[1]


class SlidingWindowKVCache(PagedKVCache):
    """A KVCache whose attention sees only the last `window` tokens of each sequence - the custom
    component the reference's interface is designed for (axono/python/axono/nn/kv_cache.py:27-34 and
    the sliding-window subclass in axono/python/tests/nn/test_kv_cache.py:75-114).  Appends go to the
    paged pools as usual; `attend` passes the window to the kernel, which never reads the pages that
    lie wholly before it."""

    def __init__(self, window: int, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if window <= 0:
            raise RuntimeError("SlidingWindowKVCache: window must be positive")
        self.window = int(window)

    def __len__(self) -> int:
        return min(super().__len__(), self.window)


class _DeviceView:
    """__cuda_array_interface__ carrier: lets torch alias device memory the library allocated."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}


class KVArena:
    """Page allocator of the paged cache (C ABI axb200_kv_arena_*): fixed per-layer pools, a free list
    of pages, sequence slots that own pages through one shared block table.  `cache()` gives the
    `PagedKVCache` view the operators run on; `alloc_seq` / `reserve` / `free_seq` manage sequences
    between steps and `sync()` uploads the changed block-table rows.

    With `device_memory=False` only the host-side bookkeeping exists (usable without a GPU)."""

    def __init__(self, n_layers, num_pages, n_kv_heads, head_dim, max_seqs, max_seq_len, dtype=torch.float16,
                 page_tokens=64, device_memory=True):
        self.n_layers, self.num_pages, self.n_kv_heads, self.head_dim = n_layers, num_pages, n_kv_heads, head_dim
        self.max_seqs, self.page_tokens, self.dtype = max_seqs, page_tokens, dtype
        self.max_blocks = (max_seq_len + page_tokens - 1) // page_tokens
        self.device_memory = device_memory
        code = {torch.float16: _capi.FLOAT16, torch.float32: _capi.FLOAT32}[dtype]
        h = C.c_void_p()
        _capi.check(_capi.lib().axb200_kv_arena_create(n_layers, num_pages, n_kv_heads, page_tokens, head_dim, code,
                                                       max_seqs, self.max_blocks, int(device_memory), C.byref(h)),
                    "kv_arena_create")
        self._h = h
        self._cache = None

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream if self.device_memory else None

    def alloc_seq(self, reserve_tokens: int = 0) -> int:
        sid = C.c_int(-1)
        _capi.check(_capi.lib().axb200_kv_arena_alloc_seq(self._h, int(reserve_tokens), C.byref(sid)), "kv_arena_alloc_seq")
        return sid.value

    def reserve(self, seq_id: int, tokens: int) -> None:
        _capi.check(_capi.lib().axb200_kv_arena_reserve(self._h, seq_id, int(tokens)), "kv_arena_reserve")

    def free_seq(self, seq_id: int) -> None:
        _capi.check(_capi.lib().axb200_kv_arena_free_seq(self._h, seq_id, self._stream()), "kv_arena_free_seq")

    def sync(self) -> None:
        _capi.check(_capi.lib().axb200_kv_arena_sync(self._h, self._stream()), "kv_arena_sync")

    def stats(self) -> dict:
        vals = [C.c_int64(0) for _ in range(4)]
        _capi.check(_capi.lib().axb200_kv_arena_stats(self._h, *[C.byref(v) for v in vals]), "kv_arena_stats")
        return dict(zip(("pages_total", "pages_free", "seqs_live", "device_bytes"), (v.value for v in vals)))

    def seq_pages(self, seq_id: int):
        buf = (C.c_int32 * self.max_blocks)()
        n = _capi.lib().axb200_kv_arena_seq_pages(self._h, seq_id, buf, self.max_blocks)
        if n < 0:
            raise RuntimeError("kv_arena_seq_pages: no such live sequence")
        return list(buf[:n])

    def cache(self) -> "PagedKVCache":
        """The operator-facing view: a PagedKVCache whose pools, block table and lengths alias the
        arena's device memory (batch = max_seqs rows)."""
        if not self.device_memory:
            raise RuntimeError("KVArena was created without device memory")
        if self._cache is None:
            lib = _capi.lib()
            dev = torch.device("cuda", torch.cuda.current_device())
            ts = {torch.float16: "<f2", torch.float32: "<f4"}[self.dtype]
            shape = (self.num_pages, self.n_kv_heads, self.page_tokens, self.head_dim)
            c = PagedKVCache.__new__(PagedKVCache)
            c.n_layers, c.batch = self.n_layers, self.max_seqs
            c.n_kv_heads, c.head_dim, c.page_tokens = self.n_kv_heads, self.head_dim, self.page_tokens
            c.max_blocks, c.max_seq_len, c.num_pages = self.max_blocks, self.max_blocks * self.page_tokens, self.num_pages
            c.dtype, c.device = self.dtype, dev
            c.k_pages = [torch.as_tensor(_DeviceView(lib.axb200_kv_arena_k_pages(self._h, l), shape, ts), device=dev)
                         for l in range(self.n_layers)]
            c.v_pages = [torch.as_tensor(_DeviceView(lib.axb200_kv_arena_v_pages(self._h, l), shape, ts), device=dev)
                         for l in range(self.n_layers)]
            c.block_table = torch.as_tensor(_DeviceView(lib.axb200_kv_arena_block_table(self._h),
                                                        (self.max_seqs, self.max_blocks), "<i4"), device=dev)
            c.seq_lens = torch.as_tensor(_DeviceView(lib.axb200_kv_arena_seq_lens(self._h), (self.max_seqs,), "<i4"),
                                         device=dev)
            c._host_len_bound = 0
            self._cache = c
        return self._cache

    def close(self) -> None:
        if self._h:
            self._cache = None
            _capi.lib().axb200_kv_arena_destroy(self._h)
            self._h = None
