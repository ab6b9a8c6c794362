"""Regenerates tests/golden/decode_path_golden.npz from the reference's own CPU library.

Run where the reference sources are present:  make -C oracle ref && python tests/golden/make_golden.py
The outputs (not the inputs, which `cases.py` rebuilds from seeds) are stored as float32.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import cases  # noqa: E402
import oracle  # noqa: E402


def main():
    ref = oracle.reference()
    g = {}
    for name, (q, k, v) in cases.all_gqa_cases().items():
        g[name] = ref.gqa_decode(q, k, v)
    q, k, v = cases.sdpa_causal_case()
    g["sdpa_causal"] = ref.sdpa(q, k, v, True)
    g["sdpa_noncausal"] = ref.sdpa(q, k, v, False)
    for name, (x, pos, theta) in cases.rope_cases().items():
        g[name] = ref.rope(x, pos, theta)
    for name, case in cases.mrope_cases().items():
        if name.startswith("mrope_cs"):
            pos3, inv, h, w = case
            c, s = ref.mrope_cos_sin(pos3, inv, h, w)
            g[name + "_cos"], g[name + "_sin"] = c, s
        else:
            x, pos3, inv, sec = case
            g[name] = ref.rope_thd(x, pos3, inv, sec)
    f = cases.fused_cases()
    g["silu_rs0"] = ref.silu_mul(*f["silu_rs0"])
    g["silu_edge"] = ref.silu_mul(*f["silu_edge"])
    for name in ("addrms_rs1", "addrms_c2"):
        y, o = ref.add_rms_norm(*f[name])
        g[name + "_y"], g[name + "_out"] = y, o
    for name in ("rms_8x16", "rms_qnorm"):
        g[name] = ref.rms_norm(*f[name])
    a, b = cases.concat_case()
    g["concat_fp16_bits"] = ref.concat_axis0(a, b).view(np.uint16)
    bits = np.arange(65536, dtype=np.uint16)
    g["half_to_float_all_bits"] = ref.half_to_float(bits).view(np.uint32)
    path = os.path.join(HERE, "decode_path_golden.npz")
    np.savez_compressed(path, **g)
    print(f"wrote {path}: {len(g)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
