"""The text tower's decode step on the native runtime (no PyTorch): the caller of the path that the
full-step configuration names, written over `libaxono` tensors exactly as the reference's model is
written over its own (axono/python/examples/vlm/qwen3vl/model.py:330-373 attention, :408-436 layer,
:483-486 final norm + tied lm_head, :729-761 decode_step), batched, with the two fusions of this
library (per-head norm + rope + append in one launch after the QKV projection; the residual add that
ends a layer folded into the next add_rms_norm).  Projections are cuBLASLt calls (`linear_nobias`).

On several GPUs (one process each, `rdv` = their host rendezvous) the KV heads are sharded: rank r
projects and caches heads [r * hkv / world, ...) and attends them; the attention kernel stores its
rows into every rank's gathered buffer over peer memory (axono_b200.native_multi), so the output
projection that follows reads local memory only.  Everything else is replicated, as the
configuration states."""
from __future__ import annotations

import numpy as np

from . import native
from .tower_config import TextTowerConfig


class NativeTextTower:
    """Random-init weights (numpy, fp16; the same on every rank), KV pages in an arena, one token per
    row and step.  `decode_step()` is capturable: positions are the cache lengths on the device, the
    next token ids are written back into `token_ids` on the device."""

    def __init__(self, cfg: TextTowerConfig, batch: int, max_seq_len: int, seed: int = 0, page_tokens: int = 64,
                 weights=None, device: str = "cuda", rdv=None, gather: str = "fused", fused_step: bool = True):
        lx = native.load()
        self.lx, self.cfg, self.batch, self.max_seq_len, self.device = lx, cfg, batch, max_seq_len, device
        self.world = rdv.world if rdv is not None else 1
        self.rank = rdv.rank if rdv is not None else 0
        if cfg.n_kv_heads % self.world:
            raise ValueError(f"cannot shard {cfg.n_kv_heads} KV heads over {self.world} ranks")
        self.local_kv = cfg.n_kv_heads // self.world
        self.local_q = cfg.n_q_heads // self.world
        d = cfg.head_dim
        rng = np.random.default_rng(seed)
        pool = (0.02 * rng.standard_normal(1 << 24, dtype=np.float32)).astype(np.float16)

        def w(rows, cols):  # N(0, 0.02) drawn from a pool at a random offset: cheap for 1.7 G parameters
            n = rows * cols
            off = int(rng.integers(0, pool.size))
            return np.resize(np.roll(pool, -off), n).reshape(rows, cols)

        def ones(n):
            return (1.0 + 0.02 * rng.standard_normal(n, dtype=np.float32)).astype(np.float16)

        if weights is None:
            weights = {"embed": w(cfg.vocab, cfg.hidden), "final_ln": ones(cfg.hidden), "layers": []}
            for _ in range(cfg.n_layers):
                weights["layers"].append({
                    "input_ln": ones(cfg.hidden), "post_ln": ones(cfg.hidden),
                    "qkv": w((cfg.n_q_heads + 2 * cfg.n_kv_heads) * d, cfg.hidden),
                    "q_norm": ones(d), "k_norm": ones(d),
                    "o": w(cfg.hidden, cfg.n_q_heads * d),
                    "gate_up": w(2 * cfg.intermediate, cfg.hidden),
                    "down": w(cfg.hidden, cfg.intermediate),
                })
        self.host_weights = weights

        def dev(a):
            return lx.Tensor.from_numpy(np.ascontiguousarray(a), device)

        def local_qkv(full):  # column-parallel: the rows of this rank's query, key and value heads
            nq, nk = cfg.n_q_heads * d, cfg.n_kv_heads * d
            q0, k0 = self.rank * self.local_q * d, self.rank * self.local_kv * d
            return np.concatenate([full[q0:q0 + self.local_q * d], full[nq + k0:nq + k0 + self.local_kv * d],
                                   full[nq + nk + k0:nq + nk + k0 + self.local_kv * d]])

        self.embed, self.final_ln = dev(weights["embed"]), dev(weights["final_ln"])
        self.layers = []
        self._weight_elems = weights["embed"].size + weights["final_ln"].size
        for lw in weights["layers"]:
            dl = {k: dev(local_qkv(v) if k == "qkv" and self.world > 1 else v) for k, v in lw.items()}
            self._weight_elems += sum(int(t.num_elements) for t in dl.values())
            self.layers.append(dl)
        self.inv_freq = dev((1.0 / (cfg.rope_theta ** (np.arange(0, d, 2, dtype=np.float32) / d))).astype(np.float32))
        blocks = (max_seq_len + page_tokens - 1) // page_tokens
        self.arena = lx.KVArena(cfg.n_layers, batch * blocks, self.local_kv, page_tokens, d, lx.DataType.FLOAT16,
                                batch, blocks)
        for _ in range(batch):
            self.arena.alloc_seq(max_seq_len)
        self.arena.sync()
        self.token_ids = dev(np.zeros(batch, np.int64))
        self.last_logits = None
        self.bufs = self.scratch = self.nccl = None
        if gather not in ("fused", "nccl"):
            raise ValueError(gather)
        if self.world > 1 and gather == "nccl":  # the library collective: attention, ncclAllGather, projection
            from .native_multi import NcclGather

            self.nccl = NcclGather(rdv, batch, self.local_q, d, lx.DataType.FLOAT16, device)
        elif self.world > 1:
            from .native_multi import PeerBuffers, Scratch

            # one gathered buffer per layer (at least two): successive calls never share a buffer
            self.bufs = PeerBuffers(rdv, batch, cfg.n_q_heads, d, lx.DataType.FLOAT16, slots=max(2, cfg.n_layers),
                                    device=device)
            self.scratch = Scratch(batch, self.local_q, self.local_kv, d, max_seq_len, lx.DataType.FLOAT16, device,
                                   step=True)
        # fused_step: a layer's norm + rope + append + attention (+ gather) is the one operator qkv_decode_step
        # (one launch); without it, qkv_norm_rope_append followed by the attention call.  The NCCL form keeps
        # the two calls: its gather is a library call after the attention kernel either way.
        self.fused_step = fused_step and self.nccl is None
        if self.fused_step and self.scratch is None:
            from .native_multi import Scratch

            self.scratch = Scratch(batch, self.local_q, self.local_kv, d, max_seq_len, lx.DataType.FLOAT16, device,
                                   step=True)
        # the step operator's output when it is not a gathered buffer: one buffer for all layers (a layer's
        # projection has read it before the next layer's attention writes it)
        self.attn_out = lx.Tensor(lx.DataType.FLOAT16, [batch, self.local_q, d], device) if self.fused_step and \
            self.bufs is None else None

    def set_state(self, token_ids, lens) -> None:
        """Starts decoding at cache lengths `lens` (one per row); positions are the lengths."""
        self.token_ids.copy_from_numpy(np.asarray(token_ids, dtype=np.int64))
        self.arena.set_seq_lens(np.asarray(lens, dtype=np.int32))

    def decode_step(self):
        lx, cfg = self.lx, self.cfg
        h = lx.embedding(self.token_ids, self.embed)
        mlp_out = None
        for li, lw in enumerate(self.layers):
            if mlp_out is None:
                xn = lx.rms_norm(h, lw["input_ln"], cfg.eps)
            else:  # previous layer's h + mlp folded into this layer's input norm
                h, xn = lx.add_rms_norm(mlp_out, h, lw["input_ln"], cfg.eps)
            qkv = lx.linear_nobias(xn, lw["qkv"])
            if self.fused_step:
                from .native_multi import qkv_decode_step

                attn = qkv_decode_step(
                    qkv, self.local_q, self.arena, li, self.max_seq_len, self.scratch,
                    lw["q_norm"] if cfg.qk_norm else None, lw["k_norm"] if cfg.qk_norm else None, cfg.eps,
                    inv_freq=self.inv_freq, theta=cfg.rope_theta,
                    mrope_section=list(cfg.mrope_section) if cfg.use_mrope else None,
                    slot_delta=0 if li == 0 else -1, advance=li == 0, out=self.attn_out, bufs=self.bufs,
                    slot=li % self.bufs.slots if self.bufs is not None else 0)
                attn = lx.Tensor.from_device_ptr(attn.data_ptr, attn.dtype, [self.batch, cfg.n_q_heads * cfg.head_dim],
                                                 self.device)
                h, xn2 = lx.add_rms_norm(lx.linear_nobias(attn, lw["o"]), h, lw["post_ln"], cfg.eps)
                act = lx.silu_mul_rows(lx.linear_nobias(xn2, lw["gate_up"]), cfg.intermediate)
                mlp_out = lx.linear_nobias(act, lw["down"])
                continue
            q = lx.qkv_norm_rope_append(
                self.arena, li, qkv, self.local_q, lw["q_norm"] if cfg.qk_norm else None,
                lw["k_norm"] if cfg.qk_norm else None, cfg.eps, inv_freq=self.inv_freq, theta=cfg.rope_theta,
                mrope_section=list(cfg.mrope_section) if cfg.use_mrope else None,
                slot_delta=0 if li == 0 else -1, advance=li == 0)
            if self.bufs is not None:  # attention fused with the all-gather of head outputs over peer memory
                from .native_multi import attend_gather

                attn = attend_gather(q, self.arena, li, self.max_seq_len, self.bufs, li % self.bufs.slots, self.scratch)
                attn = lx.Tensor.from_device_ptr(attn.data_ptr, attn.dtype, [self.batch, cfg.n_q_heads * cfg.head_dim],
                                                 self.device)
            else:
                attn = lx.gqa_decode_attention_paged(q, self.arena, li, self.max_seq_len)
                if self.nccl is not None:
                    attn = self.nccl.gather(attn)
                    attn = lx.Tensor.from_device_ptr(attn.data_ptr, attn.dtype, [self.batch, cfg.n_q_heads * cfg.head_dim],
                                                     self.device)
                else:
                    attn.reshape([self.batch, cfg.n_q_heads * cfg.head_dim])
            h, xn2 = lx.add_rms_norm(lx.linear_nobias(attn, lw["o"]), h, lw["post_ln"], cfg.eps)
            act = lx.silu_mul_rows(lx.linear_nobias(xn2, lw["gate_up"]), cfg.intermediate)
            mlp_out = lx.linear_nobias(act, lw["down"])
        _, xf = lx.add_rms_norm(mlp_out, h, self.final_ln, cfg.eps)
        self.last_logits = lx.linear_nobias(xf, self.embed)  # tied lm_head
        nxt = lx.argmax(self.last_logits)
        self.token_ids.copy_from(nxt)
        return nxt

    def kv_bytes_per_step(self, lens) -> float:
        """Algorithmic KV bytes this rank's attention reads in one step at cache lengths `lens`."""
        return float(2 * sum(int(n) + 1 for n in lens) * self.local_kv * self.cfg.head_dim * 2 * self.cfg.n_layers)

    def weight_bytes(self) -> float:
        """Bytes of weights this rank holds and reads once per step."""
        return float(2 * self._weight_elems)

    def close(self) -> None:
        if self.bufs is not None:
            self.bufs.close()
            self.bufs = None
        if self.nccl is not None:
            self.nccl.close()
            self.nccl = None
