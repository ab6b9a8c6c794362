"""Callers of the decode path: the fused decode block and the text-tower decode step.

`decode_block` is the composition the fused-decode-block configuration names: add_rms_norm ->
RoPE on q/k -> KV-cache append -> gqa_decode_attention -> silu_mul.

`TextTower` is the decode step of the reference's only consumer of the path, the Qwen3-VL text
tower (axono/python/examples/vlm/qwen3vl/model.py:330-373 attention, :408-436 layer, :483-486 final
norm + tied lm_head, :729-761 decode_step), extended from one sequence to a batch of rows.  Its
projections are library GEMMs (one cuBLASLt call each through `ops.linear_nobias`, whose algorithm is
timed per shape on first use; `lt_gemm=False` takes torch.matmul), which stay outside the rewritten path;
everything between them is this package's kernels.  Two fusions the reference's layer does not have:
the residual add that ends a layer is folded into the next layer's input norm (one add_rms_norm),
and rope + append is one launch.  KV heads shard across ranks (`world`, `rank`): each rank projects
and attends its own heads and the per-head outputs are all-gathered before o_proj - the only
collective of the step.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops, sharding
from .kv_cache import PagedKVCache
from .tower_config import TextTowerConfig  # noqa: F401 - re-exported


_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=key)
    return _side_streams[key]


def decode_block(x, residual, norm_weight, q, k_new, v_new, cache: PagedKVCache, layer: int, gate, up,
                 eps: float = 1e-6, theta: float = 1e6, pos=None, inv_freq=None, mrope_section=None,
                 parallel: bool = False, one_op: bool = True):
    """One fused decode block.  Returns (y, xn, attn, act): the residual sum and its norm, the attention
    output of the rotated q over the cache including the appended token, and silu(gate)*up.  With
    `one_op` (default) rope, append and attention are the one operator `cache.step` (one launch for fp16
    with head_dim 64 or 128; q is left as it is); without it, `append_rope` (q rotated in place) followed
    by `attend`.

    In this block the three parts do not depend on one another (the norm's and the activation's inputs
    are given), so with `parallel` the two launch-latency kernels go to a second stream while
    append -> attention runs on the current one; under CUDA-graph capture that makes them parallel
    branches of the graph and the block's time that of its attention chain."""
    if not parallel:
        y, xn = ops.add_rms_norm(x, residual, norm_weight, eps)
        attn = _rope_append_attend(cache, layer, q, k_new, v_new, pos, inv_freq, theta, mrope_section, one_op)
        act = ops.silu_mul(gate, up)
        return y, xn, attn, act
    cur = torch.cuda.current_stream(x.device)
    side = _side_stream(x.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        y, xn = ops.add_rms_norm(x, residual, norm_weight, eps)
        act = ops.silu_mul(gate, up)
    attn = _rope_append_attend(cache, layer, q, k_new, v_new, pos, inv_freq, theta, mrope_section, one_op)
    cur.wait_stream(side)
    return y, xn, attn, act


def _rope_append_attend(cache, layer, q, k_new, v_new, pos, inv_freq, theta, mrope_section, one_op):
    if one_op:
        return cache.step(layer, q, k_new, v_new, pos=pos, inv_freq=inv_freq, theta=theta, mrope_section=mrope_section)
    cache.append_rope(layer, q, k_new, v_new, pos=pos, inv_freq=inv_freq, theta=theta, mrope_section=mrope_section)
    return cache.attend(layer, q)


class TextTower:
    """Random-init text tower with a paged KV cache; `decode_step` is capturable in one CUDA graph."""

    def __init__(self, cfg: TextTowerConfig, batch: int, max_seq_len: int, device="cuda",
                 dtype=torch.float16, world: int = 1, rank: int = 0, seed: int = 0, page_tokens: int = 64,
                 fused_gather: bool = True, fused_qkv: bool = True, lt_gemm: bool = True):
        self.cfg, self.batch, self.device, self.dtype = cfg, batch, torch.device(device), dtype
        self.fused_qkv = fused_qkv
        self._linear = ops.linear_nobias if lt_gemm else (lambda x, w: torch.matmul(x, w.t()))
        self.world, self.rank = world, rank
        self.peer_gather = None
        if world > 1 and fused_gather:
            from .p2p import PeerGather

            # one gathered buffer per layer (at least two): successive calls never share a buffer
            self.peer_gather = PeerGather(batch, cfg.n_q_heads, cfg.head_dim, dtype, slots=max(2, cfg.n_layers))
        kv_heads, q_heads = sharding.shard_kv_heads(cfg.n_q_heads, cfg.n_kv_heads, world, rank)
        self.local_kv, self.local_q = len(kv_heads), len(q_heads)
        g = torch.Generator(device=self.device).manual_seed(seed)  # same seed on every rank: replicas agree

        def w(rows, cols):
            return (0.02 * torch.randn((rows, cols), generator=g, device=self.device)).to(dtype)

        def ones(n):
            return (1.0 + 0.02 * torch.randn((n,), generator=g, device=self.device)).to(dtype)

        d = cfg.head_dim
        self.embed = w(cfg.vocab, cfg.hidden)  # tied with the lm_head (model.py:483-486)
        self.layers = []
        for _ in range(cfg.n_layers):
            full_q, full_k, full_v = w(cfg.n_q_heads * d, cfg.hidden), w(cfg.n_kv_heads * d, cfg.hidden), \
                w(cfg.n_kv_heads * d, cfg.hidden)
            lw = {
                "input_ln": ones(cfg.hidden), "post_ln": ones(cfg.hidden),
                # column-parallel: only this rank's heads
                "qkv": torch.cat([full_q[q_heads.start * d:q_heads.stop * d],
                                  full_k[kv_heads.start * d:kv_heads.stop * d],
                                  full_v[kv_heads.start * d:kv_heads.stop * d]]).contiguous(),
                "q_norm": ones(d), "k_norm": ones(d),
                "o": w(cfg.hidden, cfg.n_q_heads * d),
                "gate_up": torch.cat([w(cfg.intermediate, cfg.hidden), w(cfg.intermediate, cfg.hidden)]).contiguous(),
                "down": w(cfg.hidden, cfg.intermediate),
            }
            del full_q, full_k, full_v
            self.layers.append(lw)
        self.final_ln = ones(cfg.hidden)
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(self.device)
        self.cache = PagedKVCache(cfg.n_layers, batch, self.local_kv, d, max_seq_len, dtype=dtype,
                                  device=self.device, page_tokens=page_tokens)
        # static step state (graph inputs/outputs)
        self.token_ids = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.pos3 = torch.zeros((3, batch), dtype=torch.int64, device=self.device)
        self.rope_delta = 0

    # ---------------------------------------------------------------------------------------------
    def _attention(self, li: int, xn: torch.Tensor) -> torch.Tensor:
        cfg, lw, d = self.cfg, self.layers[li], self.cfg.head_dim
        qkv = self._linear(xn, lw["qkv"])  # library GEMM
        if self.fused_qkv:  # per-head norms + rope + append in one launch, straight from the GEMM output
            q = self.cache.append_qkv(li, qkv, self.local_q, lw["q_norm"] if cfg.qk_norm else None,
                                      lw["k_norm"] if cfg.qk_norm else None, cfg.eps,
                                      pos=self.pos3 if cfg.use_mrope else self.pos3[0],
                                      inv_freq=self.inv_freq if cfg.use_mrope else None, theta=cfg.rope_theta,
                                      mrope_section=cfg.mrope_section if cfg.use_mrope else None)
        else:  # the reference's operator sequence (model.py:353-362)
            nq, nk = self.local_q * d, self.local_kv * d
            q = qkv[:, :nq].reshape(self.batch, self.local_q, d)
            k = qkv[:, nq:nq + nk].reshape(self.batch, self.local_kv, d)
            v = qkv[:, nq + nk:].reshape(self.batch, self.local_kv, d).contiguous()
            if cfg.qk_norm:  # per-head norm over head_dim (model.py:356-357)
                q = ops.rms_norm(q, lw["q_norm"], cfg.eps)
                k = ops.rms_norm(k, lw["k_norm"], cfg.eps)
            else:
                q, k = q.contiguous(), k.contiguous()
            if cfg.use_mrope:
                self.cache.append_rope(li, q, k, v, pos=self.pos3, inv_freq=self.inv_freq,
                                       mrope_section=cfg.mrope_section)
            else:
                self.cache.append_rope(li, q, k, v, pos=self.pos3[0], theta=cfg.rope_theta)
        if self.peer_gather is not None:  # attention fused with the all-gather over peer memory
            attn = self.cache.attend(li, q, gather=(self.peer_gather, li % self.peer_gather.slots))
        else:
            attn = self.cache.attend(li, q)  # (batch, local_q, d)
            if self.world > 1:
                attn = sharding.all_gather_heads(attn)  # library collective (NCCL): the baseline
        return self._linear(attn.reshape(self.batch, cfg.n_q_heads * d), lw["o"])

    def decode_step(self) -> torch.Tensor:
        """One token for every row: reads `token_ids` / `pos3`, appends to every layer's cache, writes
        the greedy next token back into `token_ids`, advances `pos3`, and returns the next ids."""
        cfg = self.cfg
        h = ops.embedding(self.token_ids, self.embed)
        mlp_out: Optional[torch.Tensor] = None
        for li, lw in enumerate(self.layers):
            if mlp_out is None:
                xn = ops.rms_norm(h, lw["input_ln"], cfg.eps)
            else:  # previous layer's h + mlp folded into this layer's input norm
                h, xn = ops.add_rms_norm(mlp_out, h, lw["input_ln"], cfg.eps)
            attn_out = self._attention(li, xn)
            h, xn2 = ops.add_rms_norm(attn_out, h, lw["post_ln"], cfg.eps)
            gu = self._linear(xn2, lw["gate_up"])
            if self.fused_qkv:
                act = ops.silu_mul_rows(gu, cfg.intermediate)
            else:
                act = ops.silu_mul(gu[:, :cfg.intermediate].contiguous(), gu[:, cfg.intermediate:].contiguous())
            mlp_out = self._linear(act, lw["down"])
        _, xf = ops.add_rms_norm(mlp_out, h, self.final_ln, cfg.eps)
        logits = self._linear(xf, self.embed)
        self.last_logits = logits
        nxt = ops.argmax_last_dim(logits)
        self.token_ids.copy_(nxt)
        self.pos3.add_(1)
        return nxt

    def set_state(self, token_ids, lens, rope_delta: int = 0):
        """Starts decoding at cache lengths `lens` (host list): positions are length + rope_delta on all
        three axes (model.py:746-748)."""
        self.token_ids.copy_(torch.as_tensor(token_ids, dtype=torch.int64))
        lens_t = torch.as_tensor(lens, dtype=torch.int64)
        self.pos3.copy_((lens_t + rope_delta).unsqueeze(0).expand(3, -1))
        self.cache.seq_lens.copy_(lens_t.to(torch.int32))
        self.cache._host_len_bound = int(lens_t.max().item())
        self.rope_delta = rope_delta

    def kv_bytes_per_step(self, lens) -> float:
        """Algorithmic KV bytes this rank's attention reads in one step at cache lengths `lens`."""
        e = torch.tensor([], dtype=self.dtype).element_size()
        return float(2 * sum(int(n) + 1 for n in lens) * self.local_kv * self.cfg.head_dim * e * self.cfg.n_layers)

    def weight_bytes(self) -> float:
        n = self.embed.numel() + self.final_ln.numel()
        for lw in self.layers:
            n += sum(t.numel() for t in lw.values())
        return float(n * self.embed.element_size())
