"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default `c3_ragged`): long-context split-K decode attention in fp16 with fp32
accumulation - one batch of 64 sequences, 16 query / 8 KV heads, head_dim 128, per-sequence KV lengths
uniform in [16384, 32768], K/V = 0.5 * N(0,1), q = N(0,1), all seeded and synthetic.  On N GPUs that
batch is sharded over the ranks by KV bytes (`--scaling strong`, the default; `weak` gives every GPU
its own batch of 64).  `b64_l32k` is the same with every sequence at 32768 tokens.  A step is one
decode step of the path for the whole batch - RoPE of q and of the new key, KV-cache append of the new
token, split-K decode attention over the paged cache, merge of the partials by the CTA that finishes a
sequence's last chunk - as the one operator `decode_step_paged`, which is ONE kernel launch;
`--two-kernel-step` runs it as `kv_append_rope` + `gqa_decode_attention_paged` (two launches).

The default arm runs on the native runtime - libaxono tensors, the KV arena, the C ABI - with no
PyTorch in the process at any N; ranks meet over a local socket (axono_b200.rendezvous).

One JSON line on rank 0.  `value` = KV-cache GB/s of the whole job with inputs resident in HBM:
algorithmic bytes (K and V read once, q read, out written) of all ranks / device time of the timed
steps (CUDA events, max over ranks).  `e2e` = the same metric through the host-buffer entry point:
each step copies q, k_new, v_new from pinned host memory and reads the attention output back.
`roofline` = the dominant kernel alone - with the one-launch step that is the step kernel itself (event
pairs recorded around its launches by the library) - against the measured HBM peak.  `cpu_baseline` = the reference's CPU SDPA-GQA on the host cores, on a bounded
sample of the same sequences.  `extra` carries, for the record: a check of the timed output against the
CPU checker, the batch-64 x 32 K case, the 28-layer text-tower step (`c5_tower`, KV heads sharded over
the GPUs with the attention kernel storing into every rank's gathered buffer) and, on several GPUs,
the weak-scaling figure with identical lengths on every rank; `parity` (N > 1) = the two cross-GPU
forms of attention against the same attention computed locally.

`--impl reference` times only the CPU path (oracle/_ref when built, else the C restatement), the whole
batch of 64 sequences per step.

Other workloads, each with its own JSON line: `c2_block` (the fused decode block, batch 8, KV 8192, one
CUDA graph), `c5_tower` (the text-tower step by itself; `--runtime torch` runs it on the torch-tensor
mirror), `prefill` (causal prefill attention; `--dtype f32` for the reference's own type), `ops` (the
standalone operators at the multimodal prompt's shapes); `--impl reference-cuda` times the reference's
own CUDA kernels compiled for sm_100; `--runtime torch` runs the attention workload on the torch mirror.
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import statistics
import sys
import threading
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, D = 16, 8, 128
PAGE_TOKENS = 64
METRIC = "gqa_decode_kv_cache_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes moved per algorithmic byte by the split kernel: (dram read + write) / algorithmic bytes of one
# launch of this workload's full batch of 64 under ncu (a one-pass capture of the two DRAM byte counters).
TRAFFIC_PER_ALGO_BYTE = 1.003

WORKLOADS = {
    "c3_ragged": dict(batch=64, lo=16384, hi=32768),
    "b64_l32k": dict(batch=64, lo=32768, hi=32768),
    "c2_b8_l8k": dict(batch=8, lo=8192, hi=8192),
}


def seq_lengths(workload: str, rank: int = 0) -> np.ndarray:
    """The workload's batch of lengths (seeded).  Every rank draws the same batch: under strong scaling
    it is sharded, under weak scaling every GPU runs a copy, so that nothing but the hardware can make
    the ranks differ."""
    w = WORKLOADS[workload]
    rng = np.random.default_rng(3000)
    return rng.integers(w["lo"], w["hi"] + 1, w["batch"]).astype(np.int64)


def common_config(workload: str, world: int, scaling: str) -> dict:
    """The workload as both arms describe it."""
    w = WORKLOADS[workload]
    return {"workload": workload, "global_batch": w["batch"] * (world if scaling == "weak" else 1), "hq": HQ, "hkv": HKV,
            "head_dim": D, "kv_len": [int(w["lo"]), int(w["hi"])], "page_tokens": PAGE_TOKENS,
            "sharding": f"batch x{world}, no collective on the attention path",
            "l2": "inputs larger than L2 (several GB of KV per step)",
            "step": "kv_append_rope + gqa_decode_paged, one CUDA graph per step"}


def algo_bytes(lens: np.ndarray, elem: int = 2) -> float:
    """K and V read once + q read + out written."""
    return float(2 * lens.sum() * HKV * D * elem + 2 * len(lens) * HQ * D * elem)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) on a thread."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_index: int, use_torch: bool = True, pci_bus_id: str = ""):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._active = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                if pci_bus_id:  # the CUDA runtime's name for the GPU: the same device whatever NVML's order
                    self.h = pynvml.nvmlDeviceGetHandleByPciBusId(pci_bus_id.encode())
                    raise StopIteration
                if not use_torch:  # a process without PyTorch: NVML's own index (no CUDA_VISIBLE_DEVICES remapping)
                    raise LookupError
                import torch

                uuid = str(torch.cuda.get_device_properties(torch_index).uuid)
                if not uuid.startswith("GPU-"):
                    uuid = "GPU-" + uuid
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except StopIteration:
                pass
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(0.01)

    def start(self):
        self._active.set()

    def pause(self):
        self._active.clear()

    def summary(self):
        self._stop.set()
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU reference arm ---------------------------------------------------------------------------
def use_all_host_threads() -> int:
    """The CPU legs use every host core this process may run on, also under torchrun, which exports
    OMP_NUM_THREADS=1 for its children."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(n))
    except OSError:
        pass
    return int(n)


def cpu_attention_sample(workload: str, budget_s: float, max_seqs: int):
    """Times the reference's CPU SDPA-GQA (fp32, the only type it supports) on the first sequences
    of rank 0's batch, one call per sequence as the reference evaluates a batch, until the time
    budget is spent.  Returns (GB/s in the workload's fp16 byte accounting, tokens/s, info)."""
    import oracle

    orc = oracle.best()
    threads = use_all_host_threads()
    lens = seq_lengths(workload, 0)
    rng = np.random.default_rng(4000)
    done_bytes, done_seqs, spent, reps = 0.0, 0, 0.0, 4
    for b in range(min(max_seqs, len(lens))):
        L = int(lens[b])
        q = rng.standard_normal((1, HQ, D)).astype(np.float32)
        k = (0.5 * rng.standard_normal((L, HKV, D))).astype(np.float32)
        v = (0.5 * rng.standard_normal((L, HKV, D))).astype(np.float32)
        run, _, release = orc.prepare_sdpa(q, k, v)
        run()
        best = float("inf")
        for _ in range(reps):
            t0 = time.perf_counter()
            run()
            best = min(best, time.perf_counter() - t0)
        release()
        dt = best
        spent += dt
        done_bytes += algo_bytes(np.asarray([L]))
        done_seqs += 1
        if spent >= budget_s:
            break
    info = {"kind": orc.kind, "cores": threads,
            "sample": f"{done_seqs} sequences of workload {workload} (lengths {int(lens[:done_seqs].min())}.."
                      f"{int(lens[:done_seqs].max())}), one fp32 SDPA call per sequence on exactly-widened inputs; "
                      f"bytes counted as the workload's fp16 KV bytes; best of {reps} calls per sequence, buffers wrapped once outside the timed region; "
                      f"the reference parallelises over its 16 query heads only"}
    return done_bytes / spent / 1e9, done_seqs / spent, spent, info


def run_reference_arm(args):
    """The reference's CPU SDPA-GQA over the whole batch: a step = one fp32 SDPA call per sequence of the
    workload's batch (the reference's op takes one sequence), all host threads, tensors wrapped once
    outside the timed region.  Rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    orc = oracle.best()
    cores = use_all_host_threads()
    lens = seq_lengths(args.workload)
    rng = np.random.default_rng(4000)
    pool_k = (0.5 * rng.standard_normal((int(lens.max()) + 4096, HKV, D))).astype(np.float32)
    pool_v = (0.5 * rng.standard_normal((int(lens.max()) + 4096, HKV, D))).astype(np.float32)
    calls = []
    for b, L in enumerate(lens):  # every sequence its own memory; contents = the pools at a per-sequence offset
        off = int(rng.integers(0, 4096))
        k = np.ascontiguousarray(pool_k[off : off + int(L)])
        v = np.ascontiguousarray(pool_v[off : off + int(L)])
        calls.append(orc.prepare_sdpa(rng.standard_normal((1, HQ, D)).astype(np.float32), k, v))
    step_bytes = algo_bytes(lens)
    for _ in range(min(args.warmup, 2)):  # a CPU pass needs no more warming than that
        for run, _, _ in calls:
            run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for run, _, _ in calls:
            run()
    dt = time.perf_counter() - t0
    for _, _, release in calls:
        release()
    value = step_bytes * args.steps / dt / 1e9
    world = int(os.environ.get("WORLD_SIZE", "1"))
    scaling = args.scaling or "strong"
    sample = (f"all {len(lens)} sequences of workload {args.workload} per step (lengths {int(lens.min())}..{int(lens.max())}), "
              f"one fp32 SDPA call each; bytes counted as the workload's fp16 KV bytes; the reference parallelises over "
              f"its 16 query heads only; warm-up passes capped at 2")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": common_config(args.workload, world, scaling),
        "arithmetic": "fp32 on the CPU (the only type the reference's op takes)",
        "bytes_actually_read_gbs": 2.0 * value,  # the CPU code streams fp32 K/V: twice the workload's fp16 bytes
        "tokens_per_s": len(lens) * args.steps / dt,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": orc.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- our arm on the native runtime (no PyTorch in the process) ---------------------------------------
class NativeStep:
    """One rank's decode step of the attention workload on the native runtime: a KV arena with `lens`
    cached tokens per sequence on scattered pages (contents 0.5 * N(0,1), seeded), q / k_new / v_new
    resident on the device, and `step()` = kv_append_rope + gqa_decode_attention_paged."""

    def __init__(self, lx, device, lens, capacity, dtype_name, seed, one_op=True):
        self.lx, self.device = lx, device
        self.one_op = one_op  # the step as the one operator decode_step_paged; False: append, then attention
        self.lens = np.asarray(lens, np.int64)
        self.B = len(self.lens)
        self.dtype = lx.DataType.FLOAT16 if dtype_name == "f16" else lx.DataType.FLOAT32
        self.np_dtype = np.float16 if dtype_name == "f16" else np.float32
        self.elem = 2 if dtype_name == "f16" else 4
        blocks = (capacity + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.capacity = blocks * PAGE_TOKENS
        self.arena = lx.KVArena(1, self.B * blocks, HKV, PAGE_TOKENS, D, self.dtype, self.B, blocks)
        self.arena.shuffle_free(99 + seed)  # sequences do not own contiguous runs of pages
        for _ in range(self.B):
            self.arena.alloc_seq(self.capacity)
        self.arena.sync()
        self.arena.fill_normal(1234 + seed, 0.5)  # K, V = 0.5 * N(0,1), generated on the device
        rng = np.random.default_rng(4321 + seed)
        mk = lambda h, s: lx.Tensor.from_numpy((s * rng.standard_normal((self.B, h, D))).astype(self.np_dtype), device)  # noqa: E731
        self.q, self.k_new, self.v_new = mk(HQ, 1.0), mk(HKV, 0.5), mk(HKV, 0.5)
        self.out = lx.Tensor(self.dtype, [self.B, HQ, D], device)
        self.bound = 0
        self.set_lengths(self.lens)

    def set_lengths(self, lens):
        self.cur = np.asarray(lens, np.int64).copy()
        self.arena.set_seq_lens(self.cur.astype(np.int32))
        self.bound = int(self.cur.max())

    def step(self):
        self.cur += 1
        self.bound = min(self.capacity, self.bound + 1)
        if self.one_op:
            self.lx.decode_step_paged(self.q, self.k_new, self.v_new, self.arena, 0, self.bound, out=self.out, theta=1e6)
        else:
            self.lx.kv_append_rope(self.arena, 0, self.q, self.k_new, self.v_new, theta=1e6)
            self.lx.gqa_decode_attention_paged(self.q, self.arena, 0, self.bound, out=self.out)

    def launches_per_step(self):
        if not self.one_op:
            return 2
        return int(self.lx.decode_step_launches(self.B, HQ, HKV, D, max(self.bound, 1), self.dtype))

    def attend(self):
        self.lx.gqa_decode_attention_paged(self.q, self.arena, 0, max(self.bound, 1), out=self.out)

    def bytes_of_steps(self, count):
        """Algorithmic bytes of the next `count` steps from the current lengths."""
        return sum(algo_bytes(self.cur + s + 1, self.elem) for s in range(count))

    def timed_steps(self, rdv, steps, sampler=None):
        """K steps between two CUDA events, a barrier and a device synchronisation on both sides;
        returns (max over ranks of the device milliseconds, this rank's algorithmic bytes)."""
        lx = self.lx
        my_bytes = self.bytes_of_steps(steps)
        timer = lx.EventTimer()
        lx.synchronize()
        rdv.barrier()
        if sampler:
            sampler.start()
        timer.start()
        for _ in range(steps):
            self.step()
        timer.stop()
        ms = timer.elapsed_ms()
        lx.synchronize()
        rdv.barrier()
        if sampler:
            sampler.pause()
        return rdv.max(ms), my_bytes

    def capture_step(self, total_steps, per_graph=1):
        """`per_graph` consecutive steps as one CUDA graph (each the step operator, or append + attention; the
        grid is sized for the lengths the sequences can reach within `total_steps` steps, so the graph follows
        the growing cache that far).  Consecutive step kernels in one graph are joined by programmatic edges:
        the next step's CTAs are scheduled while the last ones of this step finish.  Capturing runs the
        steps once for real."""
        from axono_b200 import native

        def body():
            for _ in range(per_graph):
                if self.one_op:
                    self.lx.decode_step_paged(self.q, self.k_new, self.v_new, self.arena, 0, bound, out=self.out, theta=1e6)
                else:
                    self.lx.kv_append_rope(self.arena, 0, self.q, self.k_new, self.v_new, theta=1e6)
                    self.lx.gqa_decode_attention_paged(self.q, self.arena, 0, bound, out=self.out)
            return self.out

        bound = min(self.capacity, int(self.bound) + int(total_steps) + per_graph)  # what the lengths can reach under this graph
        g = native.CUDAGraph().capture(body)
        self.per_graph = per_graph
        self.cur += per_graph
        self.bound = min(self.capacity, self.bound + per_graph)
        return g

    def timed_replays(self, rdv, g, steps):
        """K replays of the captured step, launched back to back from native code between two CUDA events
        on the graph's stream, a barrier and a device synchronisation on both sides.  Returns (max over
        ranks of the device milliseconds, this rank's algorithmic bytes, every rank's milliseconds)."""
        lx = self.lx
        my_bytes = self.bytes_of_steps(steps)
        lx.synchronize()
        rdv.barrier()
        replays = steps // self.per_graph
        ms = g.replay_timed(replays) * replays
        self.cur += steps
        self.bound = min(self.capacity, self.bound + steps)
        lx.synchronize()
        rdv.barrier()
        per_rank = [float(x) for x in rdv.all_gather_object(ms)]
        return max(per_rank), my_bytes, per_rank

    def kernel_alone(self, steps):
        """The dominant kernel by itself: event pairs the library records around its launches.  With the
        one-operator step that kernel IS the step (the same launches the timed region replays, lengths growing
        by one a launch); with the two-kernel step it is the attention call.  Returns (average milliseconds,
        launches, average algorithmic bytes per launch)."""
        lx = self.lx
        total_bytes = self.bytes_of_steps(steps) if self.one_op else steps * algo_bytes(self.cur, self.elem)
        lx.profile_enable(True)
        for _ in range(steps):
            if self.one_op:
                self.step()
            else:
                self.attend()
        ms_total, launches = lx.profile_collect()
        lx.profile_enable(False)
        return ms_total / max(launches, 1), launches, total_bytes / max(steps, 1)

    def host_steps(self, rdv, steps, warmup):
        """The same step through the host-buffer entry point: q, k_new, v_new come from pinned host
        memory and the attention output goes back to it, every step, inside the timed region."""
        lx = self.lx
        shape_q, shape_k = [self.B, HQ, D], [self.B, HKV, D]
        q_h, out_h = lx.pinned_empty(shape_q, self.dtype), lx.pinned_empty(shape_q, self.dtype)
        k_h, v_h = lx.pinned_empty(shape_k, self.dtype), lx.pinned_empty(shape_k, self.dtype)
        q_h[...] = self.q.numpy()
        k_h[...] = self.k_new.numpy()
        v_h[...] = self.v_new.numpy()
        q_d, o_d = lx.Tensor(self.dtype, shape_q, self.device), lx.Tensor(self.dtype, shape_q, self.device)
        k_d, v_d = lx.Tensor(self.dtype, shape_k, self.device), lx.Tensor(self.dtype, shape_k, self.device)
        ws = lx.Tensor(lx.DataType.INT8, [max(256, lx.gqa_workspace_bytes(self.B, HQ, HKV, D, self.capacity, self.dtype))],
                       self.device)

        def one():
            self.cur += 1
            self.bound = min(self.capacity, self.bound + 1)
            lx.decode_step_host(self.arena, 0, q_h, k_h, v_h, out_h, q_d, k_d, v_d, o_d, ws, self.bound, 1e6)

        for _ in range(warmup):
            one()
        my_bytes = self.bytes_of_steps(steps)
        lx.synchronize()
        rdv.barrier()
        gc.disable()  # a collection in the middle of a few-millisecond region would be most of it
        t0 = time.perf_counter()
        for _ in range(steps):
            one()
        dt = time.perf_counter() - t0
        gc.enable()
        rdv.barrier()
        return rdv.max(dt), my_bytes, (q_h.nbytes + k_h.nbytes + v_h.nbytes), out_h.nbytes

    def check_output(self, rows):
        """The attention output of the last step against the CPU checker on `rows` of this batch."""
        import oracle

        orc = oracle.best()
        q = self.q.numpy().astype(np.float32)
        out = self.out.numpy().astype(np.float32)
        worst = 0.0
        for b in rows:
            k, v = self.arena.gather(0, int(b), int(self.cur[b]))
            qb = q[b : b + 1]
            if self.one_op:  # the operator leaves q as it was: the checker rotates it (position = tokens cached before)
                qb = orc.rope(qb, [int(self.cur[b]) - 1], 1e6)
                if self.elem == 2:
                    qb = qb.astype(np.float16).astype(np.float32)
            ref = orc.gqa_decode(qb, k.astype(np.float32), v.astype(np.float32))
            worst = max(worst, float(oracle.rel_err(out[b : b + 1], ref)))
        return {"rows": [int(b) for b in rows], "lengths": [int(self.cur[b]) for b in rows], "rel_err": worst,
                "checker": orc.kind, "tolerance": 2e-3 if self.elem == 2 else 1e-5}

    def close(self):
        self.arena = None


def tower_figures(args, lx, rdv, device, sampler=None, gather="fused"):
    """The 28-layer text-tower decode step (batch 32, context 16384, random fp16 weights) as one captured
    graph on the native runtime, KV heads sharded over the ranks with the attention kernel storing into
    every rank's gathered buffer.  Returns the figures for `extra.c5_tower`."""
    from axono_b200 import native
    from axono_b200.native_tower import NativeTextTower
    from axono_b200.tower_config import TextTowerConfig

    B, L = args.tower_batch, args.tower_len
    cfg = TextTowerConfig()
    steps = max(3, min(args.steps, 20))
    warm = max(3, min(args.warmup, 5))
    tower = NativeTextTower(cfg, B, L + 2 * (steps + warm) + 72, seed=5, device=device, rdv=rdv, gather=gather,
                            fused_step=not args.two_kernel_step)
    tower.arena.fill_normal(77 + rdv.rank, 0.5)
    lens = [L] * B
    tower.set_state(np.arange(B) % cfg.vocab, lens)
    g = native.CUDAGraph().capture(tower.decode_step)
    lx.synchronize()
    # After the capture's warm-up run - one real step from identical inputs on every rank - the gathered
    # attention output of layer 0 must be the same bytes on every rank (each rank's rows were stored
    # into every rank's buffer), and the next tokens agree except where the replicated projections, tuned
    # per rank, round a near-tie differently.
    first_tokens = g.output.numpy().tolist()
    gathered_crc = zlib.crc32(tower.bufs.tensor(0).numpy().tobytes()) if tower.bufs is not None else 0
    seen = rdv.all_gather_object((gathered_crc, first_tokens))
    gathered_same = all(c == seen[0][0] for c, _ in seen)
    token_agreement = float(np.mean([np.mean(np.asarray(t) == np.asarray(seen[0][1])) for _, t in seen]))
    tower.set_state(np.arange(B) % cfg.vocab, lens)  # the warm-up run was a real step: start again
    for _ in range(warm):
        g.replay()
    lx.synchronize()
    rdv.barrier()
    step_ms = rdv.max(g.replay_timed(steps))  # CUDA events on the capture stream around the replays
    rdv.barrier()
    bits = int(rdv.max(lx.device_error_bits()))
    kv_bytes, w_bytes = tower.kv_bytes_per_step(lens), tower.weight_bytes()
    peak, kind = measured_peak()
    out = {"tokens_per_s": B / (step_ms / 1e3), "ms_per_step": step_ms, "batch": B, "kv_len": L, "steps": steps,
           "hbm_floor_ms": (kv_bytes + w_bytes) / (peak * 1e9) * 1e3, "peak_source": f"of {kind}",
           "graph_nodes": int(g.num_nodes), "nodes_per_layer": round((int(g.num_nodes) - 5) / cfg.n_layers, 2),
           "kv_gb_per_gpu": kv_bytes / 1e9, "weights_gb_per_gpu": w_bytes / 1e9,
           "sharding": f"KV heads x{rdv.world}" + ("" if rdv.world == 1 else
                                                   ", attention kernel stores into every rank's buffer over NVLink"
                                                   if gather == "fused" else
                                                   ", NCCL all-gather of attention outputs inside the captured graph"),
           "gathered_layer0_identical_on_all_ranks": gathered_same, "first_step_token_agreement": token_agreement,
           "device_error_bits": bits}
    if not gathered_same or bits:
        raise SystemExit(f"text tower: the ranks' gathered attention outputs differ or a device error was raised: {out}")
    g.reset()
    tower.close()
    return out


def run_native(args):
    """The attention workload on the native runtime; no PyTorch is imported at any N."""
    from axono_b200 import native, partition
    from axono_b200.rendezvous import Rendezvous

    lx = native.load()
    if not lx.cuda_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    if args.no_dependent_launch:
        from axono_b200 import _capi

        _capi.lib().axb200_set_dependent_launch(0)
    rdv = Rendezvous.from_env(timeout=600.0)  # set-up of a rank (weights, tens of GB of cache) may take minutes
    world, rank = rdv.world, rdv.rank
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    lx.set_device(local_rank)
    device = f"cuda:{local_rank}"
    scaling = args.scaling or "strong"
    w = WORKLOADS[args.workload]
    elem = 2 if args.dtype == "f16" else 4
    all_lens = seq_lengths(args.workload)
    if args.shard_of > 1:  # one rank's share of the batch sharded over `shard_of` GPUs, run alone
        lens = all_lens[partition.shard_sequences(all_lens.tolist(), args.shard_of)[0]]
    elif scaling == "strong":  # one global batch, sequences assigned to ranks by KV bytes (longest first)
        lens = all_lens[partition.shard_sequences(all_lens.tolist(), world)[rank]]
    else:
        lens = all_lens
    total_steps = 2 * (args.warmup + args.steps) + 2100
    capacity = int(w["hi"]) + total_steps + 64
    sampler = ClockSampler(local_rank, use_torch=False, pci_bus_id=lx.device_pci_bus_id(local_rank))
    peak, peak_kind = measured_peak()

    parity = None
    if world > 1:  # the cross-GPU forms of attention against the same attention computed locally
        from axono_b200.native_multi import multi_gpu_parity

        parity = multi_gpu_parity(rdv, device)
        if max(parity["gather"], parity["cp"]) > parity["tolerance"] or parity["device_error_bits"]:
            raise SystemExit(f"multi-GPU parity failed: {parity}")

    run = NativeStep(lx, device, lens, capacity, args.dtype, seed=rank, one_op=not args.two_kernel_step)
    B = run.B
    launches_per_step = run.launches_per_step()
    # ---- value: inputs resident, CUDA events around K steps ----
    sampler.start()  # sampled from here to the end of the host-buffer phase: the GPU is under this load throughout
    # The steps are captured as a CUDA graph (`per_graph` consecutive steps, the way a serving loop submits
    # several decode steps at once) and the K timed steps are K / per_graph replays launched from native
    # code: at several GPUs a step lasts 0.1-0.2 ms and the whole timed region a few milliseconds, which a
    # single scheduling hiccup of the Python thread on any one rank would otherwise double (max over ranks).
    per_graph = args.steps_per_graph if args.steps_per_graph > 0 and args.steps % args.steps_per_graph == 0 else 1
    graph = run.capture_step(args.warmup + args.steps + per_graph, per_graph)  # its warm-up run: per_graph real steps
    more_warm = max(0, -(-(args.warmup - per_graph) // per_graph))  # replays that complete the W warm-up steps
    if more_warm:
        graph.replay_timed(more_warm)
        run.cur += more_warm * per_graph
        run.bound = min(run.capacity, run.bound + more_warm * per_graph)
    dev_ms, my_bytes, ms_by_rank = run.timed_replays(rdv, graph, args.steps)
    all_bytes = rdv.sum(my_bytes)
    value = all_bytes / (dev_ms / 1e3) / 1e9
    total_seqs = rdv.sum(B)
    tokens_per_s = total_seqs * args.steps / (dev_ms / 1e3)
    err = lx.device_error_bits()
    if err:
        raise SystemExit(f"device error word {err:#x} after the timed steps")
    check = run.check_output([0, B - 1] if B > 1 else [0]) if rank == 0 and not args.no_check else None
    if check and check["rel_err"] > check["tolerance"]:
        raise SystemExit(f"the timed output differs from the CPU checker: {check}")

    # the same K steps launched one by one from Python (two operator calls a step), for the record
    run.set_lengths(lens)
    for _ in range(min(args.warmup, 3)):
        run.step()
    eager_ms, eager_bytes = run.timed_steps(rdv, args.steps)
    eager = {"value": rdv.sum(eager_bytes) / (eager_ms / 1e3) / 1e9, "unit": UNIT, "ms_per_step": eager_ms / args.steps,
             "launch": "one operator call per step from Python" if run.one_op else "two operator calls per step from Python"}
    graph.reset()

    # ---- roofline: the dominant kernel's launches ----
    # Two-kernel step: the attention kernel between event pairs the library records around its launches.
    # One-launch step: the timed region above IS K launches of that kernel, so its CUDA-event time / K is the
    # kernel's average launch duration; the event-pair figure of separately issued launches goes beside it.
    run.set_lengths(lens)
    kern_ms, launches, launch_bytes = run.kernel_alone(min(args.steps, 2000))
    pairs = {"kernel_ms": kern_ms, "launches": launches, "algorithmic_bytes_per_launch": launch_bytes}
    if launches_per_step == 1:
        kern_ms, launches, launch_bytes = ms_by_rank[rank] / args.steps, args.steps, my_bytes / args.steps
    achieved = launch_bytes / (kern_ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "kernel": f"gqa_split_{args.dtype}_kernel<paged" + (", step>" if launches_per_step == 1 else ">"),
                "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "kernel_ms": kern_ms,
                "launches_timed": launches, "algorithmic_bytes_per_launch": launch_bytes,
                "traffic": None if TRAFFIC_PER_ALGO_BYTE is None else TRAFFIC_PER_ALGO_BYTE * launch_bytes,
                "timed_as": "the K launches of the timed region (one kernel per step)" if launches_per_step == 1
                            else "event pairs around separately issued launches",
                "event_pairs": pairs}

    # ---- e2e: the host-buffer entry point, copies inside the timed region ----
    run.set_lengths(lens)
    e2e_s, e2e_my_bytes, h2d, d2h = run.host_steps(rdv, args.steps, max(3, args.warmup // 2))
    e2e_bytes = rdv.sum(e2e_my_bytes)
    e2e = {"value": e2e_bytes / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_s / args.steps * 1e3, "tokens_per_s": total_seqs * args.steps / e2e_s,
           "transfer": "q, k_new, v_new and the output live in page-locked host memory; the kernels read the inputs "
                       "from it and the attention kernel stores the output into it (the bytes cross the bus every "
                       "step, no copy-engine operation), then the host waits for the stream"}
    sampler.pause()
    clocks = sampler.summary()

    extra = {"eager_steps": eager, "timed_ms_by_rank": [round(x, 4) for x in ms_by_rank]}
    if check:
        extra["output_check"] = check
    full = args.workload == "c3_ragged" and not args.no_extra and args.dtype == "f16" and args.shard_of == 1
    def for_the_record(name, fn):
        """An entry of `extra`: measured after everything the line's own figures need; a failure in it is
        reported in place and does not take the line with it."""
        try:
            extra[name] = fn()
        except (Exception, SystemExit) as e:  # noqa: BLE001
            extra[name] = {"error": f"{type(e).__name__}: {e}"[:400]}

    def target_case():
        # batch 64 x 32 K: the kernel alone, the step, and the step with host buffers
        lens32 = np.full(B, 32768, np.int64)
        run.set_lengths(lens32)
        for _ in range(3):
            run.step()
        run.set_lengths(lens32)
        ms32, b32 = run.timed_steps(rdv, 20)
        run.set_lengths(lens32)
        k32, _, kb32 = run.kernel_alone(100)
        run.set_lengths(lens32)
        s32, eb32, _, _ = run.host_steps(rdv, 20, 3)
        pairs32 = k32
        if launches_per_step == 1:  # the step is one launch of the kernel: its time in the timed steps is the kernel's
            k32, kb32 = ms32 / 20, b32 / 20
        gbs = kb32 / (k32 / 1e3) / 1e9
        return {"split_kernel_ms": k32, "kernel_ms_between_event_pairs": pairs32, "kv_gbs": gbs, "frac_of_measured": gbs / peak,
                "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS,
                "step_ms": ms32 / 20, "step_kv_gbs": b32 / (ms32 / 1e3) / 1e9,
                "step_frac_of_nominal_8TBs": b32 / (ms32 / 1e3) / 1e9 / NOMINAL_HBM_GBS,
                "tokens_per_s": B * 20 / (ms32 / 1e3),
                "e2e_ms_per_step": s32 / 20 * 1e3, "e2e_kv_gbs": eb32 / s32 / 1e9}

    if full and world == 1:
        for_the_record("b64_l32k", target_case)
    run.close()
    del run

    def weak_scaling():
        # every GPU runs the same batch of 64 with the same lengths, so the figure can only fall below N times
        # one GPU's if the hardware makes it
        wk = NativeStep(lx, device, all_lens, capacity, args.dtype, seed=0, one_op=not args.two_kernel_step)
        for _ in range(args.warmup):
            wk.step()
        wms, wbytes = wk.timed_steps(rdv, args.steps)
        res = {"value": rdv.sum(wbytes) / (wms / 1e3) / 1e9, "unit": UNIT, "ms_per_step": wms / args.steps,
               "batch_per_gpu": int(wk.B), "lengths": "identical on every rank"}
        wk.close()
        return res

    if full and world > 1:
        for_the_record("weak", weak_scaling)
    if full and not args.no_tower:
        for_the_record("c5_tower", lambda: tower_figures(args, lx, rdv, device))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, tps, spent, info = cpu_attention_sample(args.workload, args.cpu_budget, 64)
        cpu = {"value": gbs, "unit": UNIT, "tokens_per_s": tps, "seconds": spent, **info}

    assert "torch" not in sys.modules, "the native arm must not pull PyTorch into the process"
    seqs_per_gpu = [int(x) for x in rdv.all_gather_object(B)]
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": common_config(args.workload, world, scaling),
            "runtime": "native (libaxono tensors, KV arena, C ABI; no PyTorch in the process)",
            "sequences_per_gpu": seqs_per_gpu,
            "tokens_per_s": tokens_per_s,
            "frac_of_nominal_8TBs": value / (NOMINAL_HBM_GBS * world),
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "launches_per_step": launches_per_step,
            "steps_per_graph": per_graph,
            "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu, "parity": parity, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    rdv.close()


# ---- the same workload on the torch-tensor mirror (--runtime torch) ------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from axono_b200 import _capi, ops
    from axono_b200.kv_cache import PagedKVCache

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from axono_b200 import sharding

    max_over_ranks, sum_over_ranks = sharding.max_over_ranks, sharding.sum_over_ranks

    lib = _capi.lib()
    tdtype = torch.float16 if args.dtype == "f16" else torch.float32
    elem = 2 if args.dtype == "f16" else 4
    w = WORKLOADS[args.workload]
    if args.shard_of > 1:
        # one rank's share of a batch sharded over `shard_of` GPUs, run alone (the ranks are independent)
        all_lens = seq_lengths(args.workload, 0)
        lens = all_lens[sharding.shard_sequences(all_lens.tolist(), args.shard_of)[0]]
    elif args.scaling == "strong":
        # one global batch, sequences assigned to ranks by KV bytes (longest first)
        all_lens = seq_lengths(args.workload, 0)
        lens = all_lens[sharding.shard_sequences(all_lens.tolist(), world)[rank]]
    else:
        lens = seq_lengths(args.workload, rank)
    B = len(lens)
    total_steps = args.warmup + args.steps
    capacity = int(w["hi"]) + 2 * total_steps + 64
    gen = torch.Generator(device=device).manual_seed(1234 + rank)

    cache = PagedKVCache(1, B, HKV, D, capacity, dtype=tdtype, device=device, page_tokens=PAGE_TOKENS)
    for pool in (cache.k_pages[0], cache.v_pages[0]):  # K, V = 0.5 * N(0,1), generated in slabs
        step_pages = 512
        for p0 in range(0, pool.shape[0], step_pages):
            n = min(step_pages, pool.shape[0] - p0)
            pool[p0 : p0 + n] = (0.5 * torch.randn((n,) + tuple(pool.shape[1:]), generator=gen, device=device)).to(tdtype)
    # a scattered page table: sequences do not own contiguous runs of pages
    perm = torch.randperm(cache.num_pages, generator=torch.Generator().manual_seed(99 + rank)).to(torch.int32)
    cache.block_table = perm.reshape(B, cache.max_blocks).contiguous().to(device)

    def set_lengths():
        cache.seq_lens.copy_(torch.from_numpy(lens.astype(np.int32)))
        cache._host_len_bound = int(lens.max())

    q = torch.randn((B, HQ, D), generator=gen, device=device).to(tdtype)
    k_new = (0.5 * torch.randn((B, HKV, D), generator=gen, device=device)).to(tdtype)
    v_new = (0.5 * torch.randn((B, HKV, D), generator=gen, device=device)).to(tdtype)
    out = torch.empty_like(q)
    ops.workspace(device, ops.gqa_workspace_bytes(B, HQ, HKV, D, capacity, tdtype))

    def step(qt):
        cache.append_rope(0, qt, k_new, v_new, theta=1e6)
        cache.attend(0, qt, out=out)

    def bytes_of_steps(first: int, count: int) -> float:
        return sum(algo_bytes(lens + first + s + 1, elem) for s in range(count))

    sampler = ClockSampler(local_rank)

    # ---- value: inputs resident, CUDA events around K steps ----
    set_lengths()
    for _ in range(args.warmup):
        step(q)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see only the timed steps
    ev0.record()
    for _ in range(args.steps):
        step(q)
    ev1.record()
    barrier()
    torch.cuda.profiler.stop()
    sampler.pause()
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1))
    my_bytes = bytes_of_steps(args.warmup, args.steps)
    all_bytes = sum_over_ranks(my_bytes)
    value = all_bytes / (dev_ms / 1e3) / 1e9
    total_seqs = sum_over_ranks(B)
    tokens_per_s = total_seqs * args.steps / (dev_ms / 1e3)
    err = ops.last_error()
    if err:
        raise SystemExit(f"device error word {err:#x} after the timed steps")

    # ---- roofline: the split kernel alone, event pairs around its launches ----
    set_lengths()
    prof_steps = min(args.steps, 2000)
    lib.axb200_profile_enable(1)
    barrier()
    for _ in range(prof_steps):
        cache.attend(0, q, out=out)
    ms_total, launches = ctypes.c_double(0), ctypes.c_int(0)
    lib.axb200_profile_collect(ctypes.byref(ms_total), ctypes.byref(launches))
    lib.axb200_profile_enable(0)
    kern_ms = ms_total.value / max(launches.value, 1)
    launch_bytes = algo_bytes(lens, elem)
    achieved = launch_bytes / (kern_ms / 1e3) / 1e9
    peak, peak_kind = measured_peak()
    roofline = {"bound": "hbm", "kernel": f"gqa_split_{args.dtype}_kernel<paged>", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "kernel_ms": kern_ms,
                "launches_timed": launches.value, "algorithmic_bytes_per_launch": launch_bytes,
                "traffic": None if TRAFFIC_PER_ALGO_BYTE is None else TRAFFIC_PER_ALGO_BYTE * launch_bytes}

    # ---- e2e: public API with host buffers, copies inside the timed region ----
    set_lengths()
    pin = lambda t: t.cpu().pin_memory()  # noqa: E731
    q_h, k_h, v_h = pin(q), pin(k_new), pin(v_new)
    out_h = torch.empty_like(q_h).pin_memory()
    h2d = (q_h.numel() + k_h.numel() + v_h.numel()) * elem
    d2h = out_h.numel() * elem

    def e2e_step():
        # host buffers in, host buffer out, one call: H2D copies, rope + append, attention, D2H, wait
        cache.step_host(q_h, k_h, v_h, out_h, theta=1e6)

    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    base = int(cache._host_len_bound - int(lens.max()))
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_bytes = sum_over_ranks(sum(algo_bytes(lens + base + s + 1, elem) for s in range(args.steps)))
    e2e = {"value": e2e_bytes / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_s / args.steps * 1e3, "tokens_per_s": total_seqs * args.steps / e2e_s}

    clocks = sampler.summary()

    # ---- the other single-GPU case of the same kernel, for the record ----
    extra = {}
    if world == 1 and args.workload == "c3_ragged" and not args.no_extra and args.dtype == "f16":
        lens32 = np.full(B, 32768, np.int64)
        cache.seq_lens.copy_(torch.from_numpy(lens32.astype(np.int32)))
        cache._host_len_bound = 32768
        lib.axb200_profile_enable(1)
        for _ in range(20):
            cache.attend(0, q, out=out)
        lib.axb200_profile_collect(ctypes.byref(ms_total), ctypes.byref(launches))
        for _ in range(100):
            cache.attend(0, q, out=out)
        lib.axb200_profile_collect(ctypes.byref(ms_total), ctypes.byref(launches))
        lib.axb200_profile_enable(0)
        ms32 = ms_total.value / max(launches.value, 1)
        gbs32 = algo_bytes(lens32) / (ms32 / 1e3) / 1e9
        extra["b64_l32k"] = {"split_kernel_ms": ms32, "kv_gbs": gbs32, "frac_of_measured": gbs32 / peak,
                             "frac_of_nominal_8TBs": gbs32 / NOMINAL_HBM_GBS, "tokens_per_s": B / (ms32 / 1e3)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, tps, spent, info = cpu_attention_sample(args.workload, args.cpu_budget, 64)
        cpu = {"value": gbs, "unit": UNIT, "tokens_per_s": tps, "seconds": spent, **info}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": w["batch"] if args.scaling == "weak" else None,
                       "global_batch": int(total_seqs), "hq": HQ, "hkv": HKV, "head_dim": D,
                       "kv_len": [int(w["lo"]), int(w["hi"])], "page_tokens": PAGE_TOKENS,
                       "sharding": f"batch x{world}, no collective on the attention path",
                       "l2": "inputs larger than L2 (several GB of KV per step)",
                       "step": "kv_append_rope + gqa_decode_paged (split + combine)"},
            "tokens_per_s": tokens_per_s,
            "frac_of_nominal_8TBs": value / (NOMINAL_HBM_GBS * world),
            "e2e": e2e, "gpu_launches": 3 * args.steps, "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---- the callers of the path: fused decode block and text-tower step under CUDA-graph replay ----------
def run_tower(args):
    """`c5_tower`: full 28-layer text-tower decode step (hidden 2048, intermediate 6144, 16 q / 8 KV
    heads, head_dim 128, vocab 151936, random fp16 weights), batch 32, context 16384, one CUDA graph per
    step; KV heads sharded over the GPUs with an all-gather of attention outputs per layer.
    `c2_block`: the fused decode block (add_rms_norm -> RoPE -> append -> attention -> silu_mul) at batch 8,
    KV length 8192, one CUDA graph.  Reports decode tokens/s and the KV-cache GB/s inside the step."""
    import torch
    import torch.distributed as dist

    from axono_b200 import ops, sharding
    from axono_b200.cuda_graph import CUDAGraph
    from axono_b200.decode import TextTower, TextTowerConfig, decode_block
    from axono_b200.kv_cache import PagedKVCache

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fill_random(pool, gen):
        for p0 in range(0, pool.shape[0], 512):
            n = min(512, pool.shape[0] - p0)
            pool[p0 : p0 + n] = (0.5 * torch.randn((n,) + tuple(pool.shape[1:]), generator=gen, device=device)).half()

    gen = torch.Generator(device=device).manual_seed(77 + rank)
    total_steps = args.warmup + args.steps + 2
    if args.workload == "c5_tower":
        B, L = args.tower_batch, args.tower_len
        cfg = TextTowerConfig()
        tower = TextTower(cfg, B, L + total_steps + 64, device=device, world=world, rank=rank, seed=5,
                          fused_gather=args.gather == "fused")
        for li in range(cfg.n_layers):
            fill_random(tower.cache.k_pages[li], gen)
            fill_random(tower.cache.v_pages[li], gen)
        lens = [L] * B
        tower.set_state(np.arange(B) % cfg.vocab, lens)
        ops.workspace(device, ops.gqa_workspace_bytes(B, tower.local_q, tower.local_kv, cfg.head_dim, tower.cache.max_seq_len))
        body = tower.decode_step
        cache = tower.cache
        kv_bytes = tower.kv_bytes_per_step(lens)
        launches_note = "28 x (rms/add_rms_norm x2, rms_norm x2, kv_append_rope, split, combine, silu_mul) + library GEMMs"
        other_bytes = tower.weight_bytes()
    else:
        B, L = 8, 8192
        cache = PagedKVCache(1, B, HKV, D, L + total_steps + 64, dtype=torch.float16, device=device)
        fill_random(cache.k_pages[0], gen)
        fill_random(cache.v_pages[0], gen)
        lens = [L] * B
        cache.seq_lens.fill_(L)
        cache._host_len_bound = L
        rn = lambda *s: torch.randn(s, generator=gen, device=device).half()  # noqa: E731
        x, res, w = rn(B, 2048), rn(B, 2048), (1 + 0.02 * torch.randn(2048, generator=gen, device=device)).half()
        q0, kn, vn, gate, up = rn(B, HQ, D), rn(B, HKV, D), rn(B, HKV, D), rn(B, 6144), rn(B, 6144)
        ops.workspace(device, ops.decode_step_workspace_bytes(B, HQ, HKV, D, cache.max_seq_len))

        def body():
            return decode_block(x, res, w, q0, kn, vn, cache, 0, gate, up, theta=1e6, parallel=not args.no_fork,
                                one_op=not args.two_kernel_step)

        kv_bytes = algo_bytes(np.asarray(lens) + 1)
        launches_note = (("rope + append + attention + merge in one kernel" if not args.two_kernel_step
                          else "kv_append_rope -> attention (split + merge in one kernel)") + ", with add_rms_norm and silu_mul "
                         + ("on a second stream: parallel branches of the graph" if not args.no_fork else "in line"))
        other_bytes = 0.0

    use_graph = not (world > 1 and args.workload == "c5_tower" and args.gather == "nccl")
    if use_graph:
        g = CUDAGraph().capture(body)
        cache.note_replayed()
    else:
        # baseline with the library collective: eager launches (a torch.distributed collective is not
        # put inside a captured graph here)
        class _Eager:
            num_nodes = 0
            output = None

            def replay_async(self):
                self.output = body()

            def replay(self):
                self.output = body()
                torch.cuda.current_stream().synchronize()

        g = _Eager()
        before = ops.launch_count()
        g.replay()
        g.num_nodes = ops.launch_count() - before
    for _ in range(args.warmup):
        g.replay_async()
    sampler = ClockSampler(local_rank)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see only the timed steps
    ev0.record()
    for _ in range(args.steps):
        g.replay_async()
    ev1.record()
    barrier()
    torch.cuda.profiler.stop()
    sampler.pause()
    ms = sharding.max_over_ranks(ev0.elapsed_time(ev1))
    err = ops.last_error()
    if err:
        raise SystemExit(f"device error word {err:#x}")
    # e2e: the host reads the step's result (next tokens / attention output) after every replay
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        g.replay()
        _ = g.output.cpu()
    barrier()
    e2e_s = sharding.max_over_ranks(time.perf_counter() - t0)
    all_kv = sharding.sum_over_ranks(kv_bytes)
    if rank == 0:
        step_ms = ms / args.steps
        peak, kind = measured_peak()
        line = {
            "metric": "decode_tokens_per_s", "value": B * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "batch": B, "kv_len": L, "cuda_graph": use_graph, "graph_nodes": g.num_nodes,
                       "sharding": f"KV heads x{world}" + ((", attention fused with the all-gather over peer memory"
                                                            if args.gather == "fused" else
                                                            ", NCCL all-gather of attention outputs per layer")
                                                           if world > 1 and args.workload == "c5_tower" else ""),
                       "kernels": launches_note, "l2": "KV per step larger than L2"},
            "kv_cache_gbs": all_kv / (step_ms / 1e3) / 1e9,
            "kv_frac_of_measured_peak": all_kv / (step_ms / 1e3) / 1e9 / (peak * world),
            "hbm_bytes_per_step": {"kv": all_kv, "weights_per_gpu": other_bytes},
            "hbm_floor_ms": (kv_bytes + other_bytes) / (peak * 1e9) * 1e3,
            "e2e": {"value": B * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": int(g.output.numel() * g.output.element_size()), "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": g.num_nodes * args.steps, "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_tower_native(args):
    """`c5_tower`: the 28-layer decode step on the native runtime - libaxono tensors, cuBLASLt projections,
    one captured graph, KV heads sharded over the ranks - with no PyTorch in the process."""
    from axono_b200 import native
    from axono_b200.rendezvous import Rendezvous

    lx = native.load()
    rdv = Rendezvous.from_env(timeout=600.0)  # set-up of a rank (weights, tens of GB of cache) may take minutes
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    lx.set_device(local_rank)
    sampler = ClockSampler(local_rank, use_torch=False, pci_bus_id=lx.device_pci_bus_id(local_rank))
    sampler.start()
    fig = tower_figures(args, lx, rdv, f"cuda:{local_rank}", gather=args.gather)
    sampler.pause()
    assert "torch" not in sys.modules
    if rdv.rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": fig["tokens_per_s"], "unit": "tokens/s", "n_gpus": rdv.world,
            "steps": fig["steps"], "warmup": max(3, min(args.warmup, 5)), "ms_per_step": fig["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "runtime": "native (libaxono tensors, cuBLASLt projections, no PyTorch)",
                       "batch": fig["batch"], "kv_len": fig["kv_len"], "cuda_graph": True, "graph_nodes": fig["graph_nodes"],
                       "sharding": fig["sharding"], "l2": "KV per step larger than L2"},
            "hbm_floor_ms": fig["hbm_floor_ms"], "details": fig,
            "gpu_launches": fig["graph_nodes"] * fig["steps"], "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    rdv.close()


def run_reference_cuda(args):
    """`--impl reference-cuda`: the reference's own CUDA kernels, compiled for sm_100, timed on this GPU
    next to this package's kernel on the same inputs - the reference's op is fp32 and takes one
    sequence, so the comparison is single-sequence fp32 in the reference's layout."""
    import torch

    import oracle
    from axono_b200 import _capi

    if not oracle.have_reference_cuda():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref/libaxono_ref_cuda.so is not built"}))
        return
    ref = oracle.reference_cuda()
    lib = _capi.lib()
    rows = []
    for skv in (4096, 8192, 32768):
        rng = np.random.default_rng(5000 + skv)
        q = rng.standard_normal((1, HQ, D)).astype(np.float32)
        k = (0.5 * rng.standard_normal((skv, HKV, D))).astype(np.float32)
        v = (0.5 * rng.standard_normal((skv, HKV, D))).astype(np.float32)
        want, ref_ms = ref.gqa_decode(q, k, v, iters=args.steps)
        qd, kd, vd = (torch.from_numpy(a).cuda() for a in (q, k, v))
        out = torch.empty_like(qd)
        ws = torch.empty(max(lib.axb200_gqa_workspace_bytes(1, HQ, HKV, D, skv, _capi.FLOAT32), 256), dtype=torch.uint8,
                         device="cuda")
        st = torch.cuda.current_stream().cuda_stream

        def call():
            return lib.axb200_gqa_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), HQ, HKV, D, skv,
                                         _capi.FLOAT32, ws.data_ptr(), ws.numel(), st)

        for _ in range(max(3, args.warmup)):
            call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ours_ms = e0.elapsed_time(e1) / args.steps
        nbytes = algo_bytes(np.asarray([skv]), 4)
        err = oracle.rel_err(out.cpu().numpy(), want)
        rows.append({"skv": skv, "reference_ms": ref_ms, "ours_ms": ours_ms, "reference_gbs": nbytes / ref_ms / 1e6,
                     "ours_gbs": nbytes / ours_ms / 1e6, "speedup": ref_ms / ours_ms, "rel_err": err})
    print(json.dumps({"impl": "reference-cuda", "metric": METRIC, "unit": UNIT, "dtype": "f32",
                      "config": {"workload": "single sequence, 16 q / 8 kv heads, head_dim 128, reference layout",
                                 "note": "KV of one short sequence fits in L2 after the first call"},
                      "steps": args.steps, "cases": rows}), flush=True)


def run_prefill(args):
    """`prefill`: causal prefill attention (sq = skv = --prefill-len, 16 q / 8 kv heads, head_dim 128).
    fp16 runs on the tcgen05 kernel: tensor-bound, the roofline is the measured dense GEMM peak.
    `--dtype f32` (the reference's own type) runs on the tiled FMA kernel: the bound is the fp32 FMA
    pipe, 148 SMs x 128 lanes x 2 flop x the maximum SM clock (nominal; no measured figure exists)."""
    import torch

    from axono_b200 import ops

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    S = args.prefill_len
    gen = torch.Generator(device="cuda").manual_seed(11)
    f32 = args.dtype == "f32"
    cast = (lambda t: t) if f32 else (lambda t: t.half())
    q = cast(torch.randn((S, HQ, D), generator=gen, device="cuda"))
    k = cast(torch.randn((S, HKV, D), generator=gen, device="cuda"))
    v = cast(torch.randn((S, HKV, D), generator=gen, device="cuda"))
    for _ in range(max(3, args.warmup)):
        ops.scaled_dot_product_attention(q, k, v, True)
    sampler = ClockSampler(torch.cuda.current_device())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.steps):
        ops.scaled_dot_product_attention(q, k, v, True)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    sampler.pause()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * HQ * D * (S * (S + 1) / 2)  # causal: QK^T and PV on the lower triangle
    tflops = flops / (ms / 1e3) / 1e12
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, kind = float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        peak, kind = 1590.0, "fallback"
    kernel = "prefill_attn_f16_pair_kernel" if S >= 256 else "prefill_attn_f16_kernel"
    bound = "tensor"
    if f32:
        peak, kind, kernel, bound = 148 * 128 * 2 * 1.965e9 / 1e12, "nominal fp32 FMA", "sdpa_tiled_kernel<float>", "fma"
    err = ops.last_error()
    print(json.dumps({
        "metric": "prefill_attention_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": "prefill", "sq": S, "skv": S, "hq": HQ, "hkv": HKV, "head_dim": D, "causal": True},
        "tokens_per_s": S / (ms / 1e3), "gpu_launches": args.steps, "error_word": err, "clocks": sampler.summary(),
        "roofline": {"bound": bound, "kernel": kernel, "achieved": tflops, "peak": peak,
                     "unit": "TFLOP/s", "frac": tflops / peak, "peak_source": f"of {kind}", "traffic": None},
    }), flush=True)


def run_small_ops(args):
    """`ops`: the standalone operators of the path at the multimodal configuration's shapes (1536-token
    prompt = 1024 image + 512 text tokens, batch 16 decode, 16 q / 8 kv heads, head_dim 128, sections
    24/20/20) plus the byte-copy and fallback kernels, each timed alone with CUDA events.  Most are
    launch-latency kernels (a few hundred KB): the line reports microseconds per call, and GB/s where
    the operator moves enough bytes for that to mean something."""
    import torch

    from axono_b200 import ops
    from axono_b200.kv_cache import PagedKVCache

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    gen = torch.Generator(device="cuda").manual_seed(21)
    rn = lambda *sh, dt=torch.float16: torch.randn(sh, generator=gen, device="cuda").to(dt)  # noqa: E731
    n_prompt, B = 1536, 16
    sec = (24, 20, 20)
    inv = (1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).cuda()
    pos1 = torch.arange(n_prompt, dtype=torch.int64, device="cuda")
    pos3 = torch.stack([pos1, pos1 // 32, pos1 % 32])
    xq, xk, xv = rn(n_prompt, HQ, D), rn(n_prompt, HKV, D), rn(n_prompt, HKV, D)
    cos, sin = ops.mrope_cos_sin(pos3, inv, sec[1], sec[2])
    cache = PagedKVCache(1, 2, HKV, D, 2048, dtype=torch.float16, device="cuda")
    big_a, big_b = rn(16384, HKV, D), rn(1, HKV, D)            # the reference's cache.update at 16 K tokens
    half_src, wn = rn(B, 2048), torch.ones(D, dtype=torch.float16, device="cuda")
    q80, k80, v80 = rn(1, 16, 80), rn(8192, 8, 80), rn(8192, 8, 80)  # rides in the 128-wide TMA tile, zero-filled
    q84, k84, v84 = rn(1, 16, 84), rn(8192, 8, 84), rn(8192, 8, 84)  # not a multiple of 8: the generic kernel
    q64, k64, v64 = rn(1, 16, 64), rn(32768, 8, 64), rn(32768, 8, 64)  # head_dim 64: the TMA kernel's second shape
    qf, kf, vf = rn(1, HQ, D, dt=torch.float32), rn(8192, HKV, D, dt=torch.float32), rn(8192, HKV, D, dt=torch.float32)
    elem = 2
    cases = [
        ("rope q [1536,16,128]", lambda: ops.rope(xq, pos1, 1e6), 2 * xq.numel() * elem),
        ("rope_thd q [1536,16,128]", lambda: ops.rope_thd(xq, pos3, inv, sec), 2 * xq.numel() * elem),
        ("mrope_cos_sin [1536]", lambda: ops.mrope_cos_sin(pos3, inv, sec[1], sec[2]), 2 * n_prompt * D * 4),
        ("rope_with_cos_sin k [1536,8,128]", lambda: ops.rope_with_cos_sin(xk, cos, sin), 2 * xk.numel() * elem),
        ("kv_prefill_write 1536 tokens (+ rope of q, k)", lambda: cache.prefill(0, 0, xq, xk, xv, pos=pos3, inv_freq=inv,
                                                                                 mrope_section=sec),
         2 * (xq.numel() + 2 * xk.numel()) * elem),
        ("concat axis 0: [16384,8,128] ++ [1,8,128]", lambda: ops.concat(big_a, big_b, 0), 2 * big_a.numel() * elem),
        ("rms_norm q heads [16,16,128]", lambda: ops.rms_norm(xq[:B], wn, 1e-6), 2 * B * HQ * D * elem),
        ("gqa_decode TMA kernel, head_dim 80 (zero-filled to 128), 8192 keys", lambda: ops.gqa_decode_attention(q80, k80, v80),
         2 * k80.numel() * elem),
        ("gqa_decode generic kernel, head_dim 84, 8192 keys", lambda: ops.gqa_decode_attention(q84, k84, v84),
         2 * k84.numel() * elem),
        ("gqa_decode TMA kernel, head_dim 64, 32768 keys", lambda: ops.gqa_decode_attention(q64, k64, v64),
         2 * k64.numel() * elem),
        ("gqa_decode fp32, one sequence of 8192 keys", lambda: ops.gqa_decode_attention(qf, kf, vf), 2 * kf.numel() * 4),
    ]
    cases.append(("cast f16 -> f32 [16,2048]", lambda: ops.cast(half_src, torch.float32), half_src.numel() * 6))
    from axono_b200.cuda_graph import CUDAGraph

    rows, launches, per_graph = [], 0, 20
    if args.ops_once:  # one launch of every operator inside the profiler range, for a per-kernel ncu capture
        for _, fn, _ in cases:
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _, fn, _ in cases:
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"workload": "ops", "ops_once": [c[0] for c in cases]}), flush=True)
        return
    torch.cuda.profiler.start()
    for name, fn, nbytes in cases:
        for _ in range(max(3, args.warmup)):
            fn()
        before = ops.launch_count()
        fn()
        per_call = ops.launch_count() - before

        def body(fn=fn):  # twenty calls per graph: replay shows the kernels' cadence without the host's per-call cost
            out = None
            for _ in range(per_graph):
                out = fn()
            return out

        g = CUDAGraph().capture(body)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            g.replay_async()
        e1.record()
        torch.cuda.synchronize()
        launches += per_call * per_graph * args.steps
        us = e0.elapsed_time(e1) / (args.steps * per_graph) * 1e3
        rows.append({"op": name, "us_per_call": round(us, 2), "abi_calls_per_call": per_call,
                     "algorithmic_bytes": int(nbytes), "gbs": round(nbytes / (us * 1e-6) / 1e9, 1)})
        g.reset()
    torch.cuda.profiler.stop()
    err = ops.last_error()
    if err:
        raise SystemExit(f"device error word {err:#x}")
    print(json.dumps({
        "metric": "operator_latency_us", "value": sum(r["us_per_call"] for r in rows), "unit": "us (sum over the operators)",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "ops", "timing": "CUDA-graph replays of 20 calls each between two CUDA events: the "
                                                 "kernels' cadence inside a graph; small inputs stay in L2"},
        "operators": rows, "gpu_launches": launches,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--workload", default="c3_ragged", choices=sorted(WORKLOADS) + ["c2_block", "c5_tower", "prefill", "ops"])
    ap.add_argument("--prefill-len", type=int, default=8192)
    ap.add_argument("--ops-once", action="store_true",
                    help="ops: launch every operator once inside the profiler range and exit (for ncu)")
    ap.add_argument("--runtime", default="native", choices=["native", "torch"],
                    help="native = libaxono runtime, no PyTorch in the process (default); torch = the torch-tensor mirror")
    ap.add_argument("--tower-batch", type=int, default=32, help="c5_tower: batch (default: the configuration's 32)")
    ap.add_argument("--tower-len", type=int, default=16384, help="c5_tower: context length (default 16384)")
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="strong (default): one batch of 64 sharded over the GPUs; weak: every GPU gets its own batch")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="run, on one GPU, rank 0's share of the batch sharded over this many GPUs")
    ap.add_argument("--dtype", default="f16", choices=["f16", "f32"], help="storage type of q/K/V (fp32 accumulation either way)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="c5_tower on >1 GPU: fused = attention kernel writes into peers' buffers; nccl = library all-gather")
    ap.add_argument("--cpu-budget", type=float, default=10.0, help="seconds of CPU work for cpu_baseline")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the check of the timed output against the CPU checker")
    ap.add_argument("--no-fork", action="store_true", help="c2_block: all kernels on one stream (no parallel graph branches)")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="launch the attention kernel in plain stream order (A/B of the programmatic dependent launch)")
    ap.add_argument("--no-tower", action="store_true", help="skip the text-tower figures in `extra`")
    ap.add_argument("--steps-per-graph", type=int, default=5,
                    help="consecutive steps captured into one CUDA graph, joined by programmatic edges "
                         "(used when it divides --steps, else 1)")
    ap.add_argument("--two-kernel-step", action="store_true",
                    help="the step as kv_append_rope + gqa_decode_attention_paged instead of the one operator (A/B)")
    args = ap.parse_args()
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if args.impl == "reference-cuda":
        if rank0:
            run_reference_cuda(args)
    elif args.impl == "reference":
        if args.workload in ("c2_block", "c5_tower", "prefill", "ops"):
            args.workload = "c2_b8_l8k" if args.workload == "c2_block" else "c3_ragged"
        run_reference_arm(args)
    elif args.workload == "prefill":
        if rank0:
            run_prefill(args)
    elif args.workload == "ops":
        if rank0:
            run_small_ops(args)
    elif args.workload == "c5_tower" and args.runtime == "native":
        run_tower_native(args)
    elif args.workload in ("c2_block", "c5_tower"):
        args.scaling = args.scaling or "strong"
        run_tower(args)
    elif args.runtime == "torch":
        args.scaling = args.scaling or "strong"
        run_ours(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
