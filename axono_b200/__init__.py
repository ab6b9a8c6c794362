"""axono_b200 - the B200 (sm_100a) decode hot path behind Axono's operator API.

`axono_b200.ops` mirrors the reference's Python operators for this path, `axono_b200.kv_cache`
its KV-cache component; both call the C ABI of include/axono_b200.h through `axono_b200._capi`.
"""
__all__ = ["ops", "kv_cache", "build"]
