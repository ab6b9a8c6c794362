"""KV caches over libaxono tensors.

`KVCache` and `DynamicKVCache` keep the reference's contract (axono/python/axono/nn/kv_cache.py:41-117):
k / v are (seq, n_kv_head, d_head); the first update stores the tensors themselves, later ones
concatenate along axis 0; `get` before any update raises; `len` is the cached length.
`PagedKVCache` is this library's cache for batched decode: pages in a KV arena, append with RoPE in
one launch, attention straight from the pages (no O(S) copy per step)."""
from __future__ import annotations

from axono_b200 import native as _native

_l = _native.load()


class KVCache:
    """Interface: update(layer_idx, k_new, v_new), get(layer_idx) -> (k, v), reset(), len()."""

    def update(self, layer_idx: int, k_new, v_new):  # pragma: no cover
        raise NotImplementedError

    def get(self, layer_idx: int):  # pragma: no cover
        raise NotImplementedError

    def reset(self):  # pragma: no cover
        raise NotImplementedError

    def __len__(self) -> int:  # pragma: no cover
        raise NotImplementedError


class DynamicKVCache(KVCache):
    def __init__(self, n_layers: int, device: str | None = None):
        self.n_layers, self.device = n_layers, device
        self._k = [None] * n_layers
        self._v = [None] * n_layers

    def update(self, layer_idx: int, k_new, v_new) -> None:
        if self._k[layer_idx] is None:
            self._k[layer_idx], self._v[layer_idx] = k_new, v_new
            return
        self._k[layer_idx] = _l.concat(self._k[layer_idx], k_new, 0)
        self._v[layer_idx] = _l.concat(self._v[layer_idx], v_new, 0)

    def get(self, layer_idx: int):
        if self._k[layer_idx] is None:
            raise RuntimeError("DynamicKVCache: no update yet (prefill not run?)")
        return self._k[layer_idx], self._v[layer_idx]

    def reset(self) -> None:
        self._k = [None] * self.n_layers
        self._v = [None] * self.n_layers

    def __len__(self) -> int:
        for k in self._k:
            if k is not None:
                return int(k.shape[0])
        return 0


class PagedKVCache(KVCache):
    """`batch` sequences decoded in lock step, their K/V in pages of a KV arena.

    update(layer, k_new, v_new, q=None, ...) appends one token per sequence - rotating q (in place) and
    k with RoPE / M-RoPE on the way when `rotate` - and attend(layer, q) runs the split-K decode
    attention over the pages.  The first layer of a step advances the shared lengths; later layers
    write to the same slot."""

    def __init__(self, n_layers: int, batch: int, n_kv_heads: int, head_dim: int, max_seq_len: int,
                 dtype=None, page_tokens: int = 64):
        dtype = dtype if dtype is not None else _l.DataType.FLOAT16
        blocks = (max_seq_len + page_tokens - 1) // page_tokens
        self.n_layers, self.batch, self.max_seq_len = n_layers, batch, max_seq_len
        self.arena = _l.KVArena(n_layers, batch * blocks, n_kv_heads, page_tokens, head_dim, dtype, batch, blocks)
        for _ in range(batch):
            self.arena.alloc_seq(max_seq_len)
        self.arena.sync()
        self._len = 0

    def update(self, layer_idx: int, k_new, v_new, q=None, pos=None, inv_freq=None, theta: float = 1e6,
               rotate: bool = True, mrope_section=None) -> None:
        first = layer_idx == 0
        _l.kv_append_rope(self.arena, layer_idx, q, k_new, v_new, pos=pos, inv_freq=inv_freq, theta=theta,
                          rotate=rotate, mrope_section=mrope_section, slot_delta=0 if first else -1, advance=first)
        if first:
            self._len += 1

    def attend(self, layer_idx: int, q):
        return _l.gqa_decode_attention_paged(q, self.arena, layer_idx, max(self._len, 1))

    def get(self, layer_idx: int):
        raise RuntimeError("PagedKVCache keeps K/V in pages: use attend(layer_idx, q)")

    def reset(self) -> None:
        for b in range(self.batch):
            self.arena.free_seq(b)
        for _ in range(self.batch):
            self.arena.alloc_seq(self.max_seq_len)
        self.arena.sync()
        self._len = 0

    def __len__(self) -> int:
        return self._len
