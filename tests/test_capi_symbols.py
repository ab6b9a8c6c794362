"""The C-ABI library loads and exports every entry point the header declares (no compute here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "axono_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(axb200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    for must in ("axb200_gqa_decode", "axb200_gqa_decode_paged", "axb200_kv_append_rope", "axb200_rope",
                 "axb200_rope_thd", "axb200_add_rms_norm", "axb200_silu_mul", "axb200_rms_norm"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from axono_b200 import _capi, build

    if not os.path.exists(build.LIB):
        build.build()
    handle = ctypes.CDLL(build.LIB)
    for name in _declared():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert set(_capi.SIGNATURES) == set(_declared())
    assert b"sm_100a" in _capi.lib().axb200_version()


def test_workspace_plan_is_host_only_and_monotone():
    from axono_b200 import _capi

    lib = _capi.lib()
    small = lib.axb200_gqa_workspace_bytes(1, 16, 8, 128, 4096, _capi.FLOAT32)
    big = lib.axb200_gqa_workspace_bytes(64, 16, 8, 128, 32768, _capi.FLOAT16)
    assert 0 < small < big < 64 << 20
    assert lib.axb200_gqa_workspace_bytes(0, 16, 8, 128, 4096, _capi.FLOAT32) == 0


def test_status_to_runtime_error():
    from axono_b200 import _capi

    _capi.check(0, "op")
    with pytest.raises(RuntimeError):
        _capi.check(4, "op")


def test_bench_cli_parses_without_a_gpu():
    """bench.py's command line loads on a CPU-only host (no CUDA call before a workload starts)."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0, out.stderr
    for word in ("--gpus", "--steps", "--warmup", "--impl", "--workload", "c5_tower", "prefill", "ops"):
        assert word in out.stdout
