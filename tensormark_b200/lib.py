"""ctypes binding of libtm_cuda.so — the C ABI declared in include/cuda_shim.h.

The library is the product; this module only declares argument types so Python
callers (tests, the benchmark) can reach the same entry points a C++ caller links
against. There is no fallback: when the shared library is missing, load() raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtm_cuda.so")

_vp, _u, _sz, _u64 = C.c_void_p, C.c_uint, C.c_size_t, C.c_uint64
_f32p = C.POINTER(C.c_float)

# name -> (restype, argtypes); one line per entry of include/cuda_shim.h
SIGNATURES = {
    "tm_cuda_init": (C.c_bool, [C.c_int]),
    "tm_cuda_last_error": (C.c_char_p, []),
    "tm_cuda_fallback_count": (C.c_ulonglong, []),
    "tm_cuda_launch_count": (C.c_ulonglong, []),
    "tm_cuda_sm_count": (C.c_int, []),
    "tm_cuda_set_wait_limit_ms": (C.c_uint, [C.c_uint]),
    "tm_cuda_peer_open_loopback": (C.c_bool, [C.c_int, C.c_int]),
    "tm_cuda_peer_bump": (C.c_bool, [C.c_int, C.c_int, _u]),
    "tm_cuda_q4_gemv": (C.c_bool, [_vp, _vp, _vp, _u, _u]),
    "tm_cuda_sgemm_q4": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u]),
    "tm_cuda_q4_prefill": (C.c_bool, [_vp, C.POINTER(_vp), C.POINTER(_u), _u, _vp, _u, _u]),
    "tm_cuda_gemv_q": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u]),
    "tm_cuda_sgemm_q": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u, _u]),
    "tm_cuda_dequant": (C.c_bool, [_vp, _vp, _u, _u, _u]),
    "tm_cuda_release_weights": (None, []),
    "tm_cuda_weight_bytes": (_sz, [_u, _sz, _sz]),
    "tm_cuda_gemv_q_dev": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u, _vp]),
    "tm_cuda_gemv_seg_dev": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u, C.POINTER(_u64), C.POINTER(_u), _u, _vp]),
    "tm_cuda_dequant_dev": (C.c_bool, [_vp, _vp, _u, _u, _u, _vp]),
    "tm_cuda_sgemm_q_workspace": (_sz, [_u, _u, _u, _u]),
    "tm_cuda_sgemm_q_dev": (C.c_bool, [_vp, _vp, _vp, _u, _u, _u, _u, _vp, _sz, _vp]),
    "tm_cuda_rmsnorm_dev": (C.c_bool, [_vp, _vp, _vp, _u, C.c_float, _vp]),
    "tm_cuda_add_dev": (C.c_bool, [_vp, _vp, _u, _vp]),
    "tm_cuda_silu_mul_dev": (C.c_bool, [_vp, _vp, _u, _vp]),
    "tm_cuda_argmax_dev": (C.c_bool, [_vp, _vp, _u, _vp]),
    "tm_cuda_attn_decode_scratch": (_sz, [_u, _u, _u, _u, _u]),
    "tm_cuda_attn_decode_dev": (C.c_bool, [_vp, _vp, _vp, _vp, _sz, _vp, _u, _u, _u, _u, _u, C.c_float, C.c_int, _vp]),
    "tm_cuda_attn_decode_static_dev": (C.c_bool, [_vp, _vp, _vp, _vp, _u, _u, _u, _u, _u, C.c_float, C.c_int, _vp]),
    "tm_cuda_tok_begin": (C.c_bool, []),
    "tm_cuda_tok_flush": (C.c_bool, []),
    "tm_cuda_tok_end": (C.c_bool, [C.c_int, _vp, _u]),
    "tm_cuda_tok_end_async": (C.c_bool, []),
    "tm_cuda_tok_wait_pending": (C.c_bool, []),
    "tm_cuda_tok_reserve": (C.c_bool, [C.c_int, _sz]),
    "tm_cuda_tok_upload": (C.c_bool, [C.c_int, _sz, _vp, _sz]),
    "tm_cuda_tok_download": (C.c_bool, [C.c_int, _sz, _vp, _sz]),
    "tm_cuda_tok_kv_reserve": (C.c_bool, [C.c_int, _sz]),
    "tm_cuda_tok_kv_upload": (C.c_bool, [C.c_int, _sz, _vp, _sz]),
    "tm_cuda_tok_kv_download": (C.c_bool, [C.c_int, _sz, _vp, _sz]),
    "tm_cuda_tok_wbuf": (C.c_int, [_vp, _sz, _vp, _sz, C.c_int, C.POINTER(_u64)]),
    "tm_cuda_tok_wbuf_pack": (C.c_int, [C.POINTER(_vp), C.POINTER(_sz), _u, C.POINTER(_u64)]),
    "tm_cuda_tok_probe_copy": (C.c_bool, [C.c_int, _sz, C.c_int, _u]),
    "tm_cuda_tok_gemv": (None, [C.c_int, C.c_int, _u64, C.c_int, _sz, _u, _u]),
    "tm_cuda_tok_gemv_seg_supported": (C.c_bool, [_u]),
    "tm_cuda_tok_gemv_seg": (None, [C.c_int, C.c_int, C.c_int, _sz, _u, _u, C.POINTER(_u64), C.POINTER(_u), _u]),
    "tm_cuda_tok_gemv_seg_dt": (None, [C.c_int, C.c_int, C.c_int, _sz, _u, _u, _u, C.POINTER(_u64), C.POINTER(_u), _u]),
    "tm_cuda_tok_gemv_kq": (None, [C.c_int, C.c_int, _u64, C.c_int, _sz, _u, _u, _u]),
    "tm_cuda_tok_embed_q4": (None, [C.c_int, _u, C.c_int, _u64, C.c_int, _u]),
    "tm_cuda_tok_embed_kq": (None, [C.c_int, _u, C.c_int, _u64, C.c_int, _u, _u]),
    "tm_cuda_tok_gemv_h": (None, [C.c_int, C.c_int, _u64, C.c_int, _sz, _u, _u]),
    "tm_cuda_tok_embed_h": (None, [C.c_int, _u, C.c_int, _u64, C.c_int, _u]),
    "tm_cuda_tok_wbuf_q4_from_gguf": (C.c_bool, [C.c_int, _u64, _sz]),
    "tm_cuda_q4_0_from_gguf_dev": (C.c_bool, [_vp, _sz, _vp]),
    "tm_cuda_tok_bias_qkv": (None, [C.c_int, C.c_int, _sz, _u]),
    "tm_cuda_tok_rmsnorm": (None, [C.c_int, _vp, C.c_int, _u, C.c_float]),
    "tm_cuda_tok_add": (None, [C.c_int, C.c_int, _u]),
    "tm_cuda_tok_silu_mul": (None, [C.c_int, _sz, C.c_int, _sz, _u]),
    "tm_cuda_tok_rope_q": (None, [C.c_int, _u, _u, C.c_int, C.c_float]),
    "tm_cuda_tok_rope_k_cache": (None, [C.c_int, _sz, C.c_int, _u, _u, _u, C.c_int, C.c_float]),
    "tm_cuda_tok_v_cache": (None, [C.c_int, _sz, C.c_int, _u, _u, _u, C.c_int]),
    "tm_cuda_tok_attn": (None, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u, _u, _u, _u, _u, C.c_int, C.c_float, _u]),
    "tm_cuda_tok_argmax": (None, [C.c_int, C.c_int, _u, _u]),
    "tm_cuda_tok_sample": (None, [C.c_int, C.c_int, _u, _u, C.c_float, _u]),
    "tm_cuda_tok_peek": (_u, [C.c_int, _u]),
    "tm_cuda_tok_gemv_fused": (None, [C.c_int, _sz, C.c_int, C.c_int, _sz, _vp, C.c_float, C.c_int, C.c_int, _sz, _u, _u, _u,
                                      C.POINTER(_u64), C.POINTER(_u), _u, C.c_int]),
    "tm_cuda_llama_create": (_vp, [_vp]),
    "tm_cuda_llama_create_dt": (_vp, [_vp, _u]),
    "tm_cuda_llama_prefill": (C.c_int, [_vp, _vp, C.c_int, C.c_int]),
    "tm_cuda_llama_prefill_begin": (C.c_int, [_vp, _vp, C.c_int, C.c_int]),
    "tm_cuda_llama_prefill_wait_layer": (C.c_int, [C.c_int]),
    "tm_cuda_llama_prefill_end": (C.c_int, []),
    "tm_cuda_llama_prefill_gpu_ms": (C.c_double, []),
    "tm_cuda_llama_reserve": (C.c_int, [_vp, C.c_int]),
    "tm_cuda_llama_prefill_begin_tokens": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_int, _u]),
    "tm_cuda_llama_destroy": (None, [_vp]),
    "tm_cuda_llama_kv_to_slots": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tm_cuda_tok_qkv_post_at": (None, [C.c_int, C.c_int, C.c_int, _u, _u, _u, _u, C.c_float, C.c_int]),
    "tm_cuda_tok_attn_at": (None, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u, _u, _u, _u, _u, C.c_float, _u, C.c_int]),
    "tm_cuda_tok_attn_fused_at": (None, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u, _u, _u, _u, C.c_float, C.c_float, C.c_int]),
    "tm_cuda_tok_sample_at": (None, [C.c_int, C.c_int, _u, _u, C.c_float, _u, C.c_int, C.c_int]),
    "tm_cuda_tok_argmax_at": (None, [C.c_int, C.c_int, _u, _u, C.c_int]),
    "tm_cuda_tok_embed_at": (None, [C.c_int, C.c_int, _u64, C.c_int, _u, _u, _u, C.c_int]),
    "tm_cuda_tok_advance": (None, [C.c_int]),
    "tm_cuda_tok_graph_begin": (C.c_bool, []),
    "tm_cuda_tok_graph_end": (C.c_int, []),
    "tm_cuda_tok_graph_launch": (C.c_bool, [C.c_int, _u]),
    "tm_cuda_tok_graph_destroy": (None, [C.c_int]),
    "tm_cuda_comm_id_bytes": (C.c_size_t, []),
    "tm_cuda_comm_unique_id": (C.c_bool, [_vp]),
    "tm_cuda_comm_init": (C.c_bool, [C.c_int, C.c_int, _vp]),
    "tm_cuda_comm_rank": (C.c_int, []),
    "tm_cuda_comm_world": (C.c_int, []),
    "tm_cuda_comm_destroy": (C.c_bool, []),
    "tm_cuda_tok_all_gather": (None, [C.c_int, C.c_size_t, C.c_int, C.c_size_t, C.c_uint]),
    "tm_cuda_peer_handle_bytes": (C.c_size_t, []),
    "tm_cuda_peer_arena": (C.c_bool, [C.c_size_t, _vp]),
    "tm_cuda_peer_open": (C.c_bool, [C.c_int, C.c_int, _vp]),
    "tm_cuda_peer_world": (C.c_int, []),
    "tm_cuda_peer_rank": (C.c_int, []),
    "tm_cuda_peer_unmap": (C.c_bool, []),
    "tm_cuda_peer_close": (C.c_bool, []),
    "tm_cuda_tok_reserve_shared": (C.c_bool, [C.c_int, C.c_size_t]),
    "tm_cuda_tok_gemv_xchg": (None, [C.c_int, _sz, C.c_int, C.c_int, _sz, _vp, C.c_float, C.c_int, C.c_int, C.POINTER(_sz), _u, _u, _u,
                                     C.POINTER(_u64), C.POINTER(_u), _u, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tm_cuda_tok_argmax_xchg": (None, [C.c_int, C.c_int, _u, _u, C.c_int, C.c_int]),
    "tm_cuda_tok_choose_shard": (None, [C.c_int, _u, _u, _u, C.c_int, _u, C.c_float, _u, C.c_int, C.c_int, C.c_int]),
    "tm_cuda_trace_read": (C.c_size_t, [_vp, C.c_size_t]),
    "tm_cuda_tok_slot_ptr": (_vp, [C.c_int]),
    "tm_cuda_tok_stream": (_vp, []),
}

_lib = None


def load() -> C.CDLL:
    """Load libtm_cuda.so and type its entry points. Raises when it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tensormark_b200.build` "
                "(this package has no CPU implementation to fall back to)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError here = the ABI lost a symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().tm_cuda_last_error().decode()


def check(ok: bool, what: str) -> None:
    if not ok:
        raise RuntimeError(f"{what} failed: {last_error()}")
