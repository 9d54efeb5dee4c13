"""ctypes view of the CPU checker libraries (TEST INFRASTRUCTURE).

Only tests, the smoke check and the benchmark's CPU-baseline legs import this
module. `oracle()` is the plain-C restatement (tm_oracle.c); `reference()` is the
reference's own quant.h behind C entry points (ref_wrap.cpp), present only when
it was built where the reference tree exists.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_c_f32p = C.POINTER(C.c_float)
_c_f64p = C.POINTER(C.c_double)


def build() -> None:
    """Compile the checker libraries (make; also builds _ref when the reference tree is present)."""
    subprocess.run(["make", "-s", "-C", _HERE, "-f", os.path.join(_HERE, "Makefile"), "all"], check=True)


def _ptr(a: np.ndarray, ty=C.c_void_p):
    return a.ctypes.data_as(ty)


class Oracle:
    def __init__(self, path: str):
        self.lib = lib = C.CDLL(path)
        lib.tmo_fp16_to_fp32.restype = C.c_float
        lib.tmo_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.tmo_fp32_to_fp16.restype = C.c_uint16
        lib.tmo_fp32_to_fp16.argtypes = [C.c_float]
        lib.tmo_dequant.argtypes = [C.c_int, C.c_void_p, _c_f32p, C.c_size_t]
        lib.tmo_q4_split_to_interleaved.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        lib.tmo_gemv.argtypes = [C.c_int, C.c_void_p, _c_f32p, _c_f32p, C.c_int, C.c_int]
        lib.tmo_gemv_mt.argtypes = [C.c_int, C.c_void_p, _c_f32p, _c_f32p, C.c_int, C.c_int, C.c_int]
        lib.tmo_gemv_f64.argtypes = [C.c_int, C.c_void_p, _c_f32p, _c_f64p, _c_f64p, C.c_int, C.c_int]
        lib.tmo_gemm.argtypes = [C.c_int, C.c_void_p, _c_f32p, _c_f32p, C.c_int, C.c_int, C.c_int, C.c_int]
        lib.tmo_gemm_f64_samples.argtypes = [C.c_int, C.c_void_p, _c_f32p, C.c_int, C.c_int,
                                             C.POINTER(C.c_int), C.c_int, _c_f64p, _c_f64p]
        lib.tmo_rmsnorm.argtypes = [_c_f32p, _c_f32p, _c_f32p, C.c_int, C.c_float]
        lib.tmo_rope_head.argtypes = [_c_f32p, C.c_int, C.c_int, C.c_float]
        lib.tmo_rope_table.argtypes = [_c_f32p, C.c_int, C.c_int, C.c_float]
        lib.tmo_attn_group.argtypes = [_c_f32p, _c_f32p, _c_f32p, _c_f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        lib.tmo_silu_mul.argtypes = [_c_f32p, _c_f32p, C.c_int]
        lib.tmo_argmax.restype = C.c_uint
        lib.tmo_argmax.argtypes = [_c_f32p, C.c_uint]
        lib.tmo_chain_step.argtypes = [C.c_void_p, C.c_uint, C.c_int, _c_f32p, C.c_int, _c_f32p]

    # -- block formats
    def dequant(self, dtype: int, blocks: np.ndarray, n: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        if not self.lib.tmo_dequant(dtype, _ptr(blocks), _ptr(out, _c_f32p), n):
            raise ValueError("tmo_dequant rejected its arguments")
        return out

    def q4_split_to_interleaved(self, blocks: np.ndarray) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty_like(blocks)
        self.lib.tmo_q4_split_to_interleaved(_ptr(blocks), _ptr(out), blocks.size // 18)
        return out

    def fp16_to_fp32(self, h: int) -> float:
        return self.lib.tmo_fp16_to_fp32(h)

    def fp32_to_fp16(self, f: float) -> int:
        return self.lib.tmo_fp32_to_fp16(f)

    # -- matmul
    def gemv(self, dtype: int, W: np.ndarray, x: np.ndarray, n_out: int, n_in: int, threads: int = 1) -> np.ndarray:
        W = np.ascontiguousarray(W, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(n_out, dtype=np.float32)
        if threads > 1:
            ok = self.lib.tmo_gemv_mt(dtype, _ptr(W), _ptr(x, _c_f32p), _ptr(y, _c_f32p), n_out, n_in, threads)
        else:
            ok = self.lib.tmo_gemv(dtype, _ptr(W), _ptr(x, _c_f32p), _ptr(y, _c_f32p), n_out, n_in)
        if not ok:
            raise ValueError("tmo_gemv rejected its arguments")
        return y

    def gemv_f64(self, dtype: int, W: np.ndarray, x: np.ndarray, n_out: int, n_in: int):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(n_out, dtype=np.float64)
        ya = np.empty(n_out, dtype=np.float64)
        if not self.lib.tmo_gemv_f64(dtype, _ptr(W), _ptr(x, _c_f32p), _ptr(y, _c_f64p), _ptr(ya, _c_f64p), n_out, n_in):
            raise ValueError("tmo_gemv_f64 rejected its arguments")
        return y, ya

    def gemm(self, dtype: int, W: np.ndarray, A: np.ndarray, M: int, N: int, K: int, threads: int = 1) -> np.ndarray:
        W = np.ascontiguousarray(W, dtype=np.uint8)
        A = np.ascontiguousarray(A, dtype=np.float32)
        Cm = np.empty((M, N), dtype=np.float32)
        if not self.lib.tmo_gemm(dtype, _ptr(W), _ptr(A, _c_f32p), _ptr(Cm, _c_f32p), M, N, K, threads):
            raise ValueError("tmo_gemm rejected its arguments")
        return Cm

    def gemm_f64_samples(self, dtype: int, W: np.ndarray, A: np.ndarray, N: int, K: int, idx: np.ndarray):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        A = np.ascontiguousarray(A, dtype=np.float32)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        ns = idx.shape[0]
        y = np.empty(ns, dtype=np.float64)
        ya = np.empty(ns, dtype=np.float64)
        if not self.lib.tmo_gemm_f64_samples(dtype, _ptr(W), _ptr(A, _c_f32p), N, K,
                                             _ptr(idx, C.POINTER(C.c_int)), ns, _ptr(y, _c_f64p), _ptr(ya, _c_f64p)):
            raise ValueError("tmo_gemm_f64_samples rejected its arguments")
        return y, ya

    # -- glue
    def rmsnorm(self, x, w, eps):
        x = np.ascontiguousarray(x, dtype=np.float32); w = np.ascontiguousarray(w, dtype=np.float32)
        out = np.empty_like(x)
        self.lib.tmo_rmsnorm(_ptr(x, _c_f32p), _ptr(w, _c_f32p), _ptr(out, _c_f32p), x.size, eps)
        return out

    def rope_head(self, r, pos, theta):
        r = np.array(r, dtype=np.float32, copy=True)
        self.lib.tmo_rope_head(_ptr(r, _c_f32p), r.size, pos, theta)
        return r

    def rope_table(self, dh, npos, theta):
        cs = np.empty((npos, dh // 2, 2), dtype=np.float32)
        self.lib.tmo_rope_table(_ptr(cs, _c_f32p), dh, npos, theta)
        return cs

    def attn_group(self, q, K, V, scale):
        q = np.ascontiguousarray(q, dtype=np.float32); K = np.ascontiguousarray(K, dtype=np.float32)
        V = np.ascontiguousarray(V, dtype=np.float32)
        rep, dh = q.shape
        out = np.empty_like(q)
        self.lib.tmo_attn_group(_ptr(q, _c_f32p), _ptr(K, _c_f32p), _ptr(V, _c_f32p), _ptr(out, _c_f32p),
                                rep, dh, K.shape[0], scale)
        return out

    def silu_mul(self, g, u):
        g = np.array(g, dtype=np.float32, copy=True); u = np.ascontiguousarray(u, dtype=np.float32)
        self.lib.tmo_silu_mul(_ptr(g, _c_f32p), _ptr(u, _c_f32p), g.size)
        return g

    def argmax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return int(self.lib.tmo_argmax(_ptr(x, _c_f32p), x.size))


class _ModelStruct(C.Structure):
    _fields_ = [
        ("L", C.c_int), ("D", C.c_int), ("H", C.c_int), ("KVH", C.c_int), ("dh", C.c_int),
        ("F", C.c_int), ("V", C.c_int), ("ctx", C.c_int),
        ("theta", C.c_float), ("eps", C.c_float),
        ("dt_proj", C.c_int), ("dt_head", C.c_int), ("dt_embed", C.c_int),
        ("embed", C.c_void_p), ("head", C.c_void_p),
        ("wq", C.POINTER(C.c_void_p)), ("wk", C.POINTER(C.c_void_p)), ("wv", C.POINTER(C.c_void_p)),
        ("wo", C.POINTER(C.c_void_p)), ("wgate", C.POINTER(C.c_void_p)), ("wup", C.POINTER(C.c_void_p)),
        ("wdown", C.POINTER(C.c_void_p)),
        ("rms1", C.POINTER(C.c_void_p)), ("rms2", C.POINTER(C.c_void_p)), ("rmsf", C.c_void_p),
        ("kc", C.c_void_p), ("vc", C.c_void_p),
        ("kv_half", C.c_int), ("threads", C.c_int),
        ("qb", C.POINTER(C.c_void_p)), ("kb", C.POINTER(C.c_void_p)), ("vb", C.POINTER(C.c_void_p)),
    ]


class ChainModel:
    """CPU decode chain over a dict of numpy weights (see tmo_chain_step)."""

    def __init__(self, orc: Oracle, cfg: dict, weights: dict, kv_half: bool = False, threads: int = 1, biases: dict | None = None):
        self.orc, self.cfg, self.weights = orc, cfg, weights
        L = cfg["L"]
        self.kc = np.zeros((L, cfg["KVH"], cfg["ctx"], cfg["dh"]), dtype=np.float32)
        self.vc = np.zeros_like(self.kc)
        self._keep = []

        def arr(names):
            a = (C.c_void_p * L)(*[weights[n].ctypes.data for n in names])
            self._keep.append(a)
            return C.cast(a, C.POINTER(C.c_void_p))

        def per(fmt):
            return [fmt.format(l) for l in range(L)]

        s = _ModelStruct()
        for k in ("L", "D", "H", "KVH", "dh", "F", "V", "ctx"):
            setattr(s, k, cfg[k])
        s.theta, s.eps = cfg["theta"], cfg["eps"]
        s.dt_proj, s.dt_head, s.dt_embed = cfg["dt_proj"], cfg["dt_head"], cfg["dt_embed"]
        s.embed = weights["embed"].ctypes.data
        s.head = weights["head"].ctypes.data
        s.wq, s.wk, s.wv, s.wo = arr(per("l{}.q")), arr(per("l{}.k")), arr(per("l{}.v")), arr(per("l{}.o"))
        s.wgate, s.wup, s.wdown = arr(per("l{}.gate")), arr(per("l{}.up")), arr(per("l{}.down"))
        s.rms1, s.rms2 = arr(per("l{}.rms1")), arr(per("l{}.rms2"))
        s.rmsf = weights["rmsf"].ctypes.data
        s.kc, s.vc = self.kc.ctypes.data, self.vc.ctypes.data
        s.kv_half, s.threads = int(kv_half), threads
        if biases:
            for field, name in (("qb", "q_bias"), ("kb", "k_bias"), ("vb", "v_bias")):
                arrs = [np.ascontiguousarray(biases[f"l{l}.{name}"], np.float32) for l in range(L)]
                self._keep.append(arrs)
                a = (C.c_void_p * L)(*[x.ctypes.data for x in arrs])
                self._keep.append(a)
                setattr(s, field, C.cast(a, C.POINTER(C.c_void_p)))
        self.s = s

    def tap_size(self):
        c = self.cfg
        QD, KVD = c["H"] * c["dh"], c["KVH"] * c["dh"]
        return c["D"] + QD + 2 * KVD + QD + c["D"] + c["D"] + c["F"] + c["D"]

    def step(self, tok: int, pos: int, tap_layer: int = -1):
        logits = np.empty(self.cfg["V"], dtype=np.float32)
        taps = np.zeros(self.tap_size(), dtype=np.float32) if tap_layer >= 0 else None
        ok = self.orc.lib.tmo_chain_step(C.byref(self.s), int(tok), pos, _ptr(logits, _c_f32p), tap_layer,
                                         _ptr(taps, _c_f32p) if taps is not None else None)
        if not ok:
            raise ValueError("tmo_chain_step rejected its arguments")
        return (logits, taps) if taps is not None else logits


class Reference:
    def __init__(self, path: str):
        self.lib = lib = C.CDLL(path)
        lib.tmref_dequant.argtypes = [C.c_int, C.c_void_p, _c_f32p, C.c_size_t]
        lib.tmref_fp16_to_fp32.restype = C.c_float
        lib.tmref_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.tmref_fp32_to_fp16.restype = C.c_uint16
        lib.tmref_fp32_to_fp16.argtypes = [C.c_float]
        lib.tmref_quantize_q4_0.argtypes = [_c_f32p, C.c_void_p, C.c_size_t]
        lib.tmref_quantize_q8_0.argtypes = [_c_f32p, C.c_void_p, C.c_size_t]
        lib.tmref_quantize_tq2.argtypes = [_c_f32p, C.c_void_p, C.c_size_t]

    def dequant(self, dtype: int, blocks: np.ndarray, n: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        if not self.lib.tmref_dequant(dtype, _ptr(blocks), _ptr(out, _c_f32p), n):
            raise ValueError("reference dequantizer rejected its arguments")
        return out

    def quantize(self, dtype: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        bb, be = {0: (34, 32), 1: (18, 32), 7: (34, 128)}[dtype]
        out = np.empty(x.size // be * bb, dtype=np.uint8)
        fn = {0: self.lib.tmref_quantize_q8_0, 1: self.lib.tmref_quantize_q4_0, 7: self.lib.tmref_quantize_tq2}[dtype]
        fn(_ptr(x, _c_f32p), _ptr(out), x.size)
        return out


_oracle = None
_fast = None
_ref = None


def oracle() -> Oracle:
    global _oracle
    if _oracle is None:
        path = os.path.join(_HERE, "libtm_oracle.so")
        if not os.path.exists(path):
            build()
        _oracle = Oracle(path)
    return _oracle


def oracle_fast() -> Oracle:
    """-O3 -march=native build of the same source, for timing the CPU baseline."""
    global _fast
    if _fast is None:
        # -march=native must be compiled on the host that runs it, so this build
        # goes to the temp directory of the current machine, never into the tree.
        import tempfile
        path = os.path.join(tempfile.mkdtemp(prefix="tmo_fast_"), "libtm_oracle_fast.so")
        subprocess.run(["gcc", "-O3", "-march=native", "-ffp-contract=off", "-fPIC", "-shared",
                        "-fvisibility=hidden", "-pthread", "-o", path,
                        os.path.join(_HERE, "tm_oracle.c"), "-lm"], check=True)
        _fast = Oracle(path)
    return _fast


def reference():
    """The reference's own quant.h, or None when it was never built for this checkout."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libtm_ref.so")
        if not os.path.exists(path):
            return None
        _ref = Reference(path)
    return _ref
