"""ctypes view of the prefill layer stack (include/llama_gpu_api.h) for tests and benchmarks."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib

_f32p = C.POINTER(C.c_float)


class GpuLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q", "k", "v", "o", "gate", "up", "down")] + \
               [("rms1", _f32p), ("rms2", _f32p), ("q_bias", _f32p), ("k_bias", _f32p), ("v_bias", _f32p),
                ("kc", _f32p), ("vc", _f32p)]


class GpuDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("L", "D", "H", "KVH", "dh", "F", "ctx")] + \
               [("theta", C.c_float), ("eps", C.c_float), ("map_base", C.c_void_p), ("map_size", C.c_size_t),
                ("layers", C.POINTER(GpuLayer))]


class Stack:
    """The layer stack of a model made by synth.make_llama. Owns the host K/V arrays the contract asks the caller for:
    kc[l], vc[l] are float32 [KVH, ctx, dh]."""

    def __init__(self, cfg: dict, weights: dict, shared_mapping: bool = True, biases: dict | None = None, device_only: bool = False):
        self.L = lib.load()
        self.cfg, self.weights = cfg, weights
        n = cfg["L"]
        self.kc = [np.zeros((cfg["KVH"], cfg["ctx"], cfg["dh"]), np.float32) for _ in range(n)]
        self.vc = [np.zeros((cfg["KVH"], cfg["ctx"], cfg["dh"]), np.float32) for _ in range(n)]
        self._layers = (GpuLayer * n)()
        self._keep = []
        for l in range(n):
            s = self._layers[l]
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                setattr(s, name, weights[f"l{l}.{name}"].ctypes.data)
            s.rms1 = weights[f"l{l}.rms1"].ctypes.data_as(_f32p)
            s.rms2 = weights[f"l{l}.rms2"].ctypes.data_as(_f32p)
            if biases:
                for name in ("q_bias", "k_bias", "v_bias"):
                    a = np.ascontiguousarray(biases[f"l{l}.{name}"], np.float32)
                    self._keep.append(a)
                    setattr(s, name, a.ctypes.data_as(_f32p))
            if not device_only:                         # else: NULL, the K/V rows stay on the device
                s.kc = self.kc[l].ctypes.data_as(_f32p)
                s.vc = self.vc[l].ctypes.data_as(_f32p)
        d = GpuDesc()
        for k in ("L", "D", "H", "KVH", "dh", "F", "ctx"):
            setattr(d, k, cfg[k])
        d.theta, d.eps = cfg["theta"], cfg["eps"]
        blob = weights["blob"]
        d.map_base = blob.ctypes.data if shared_mapping else None
        d.map_size = blob.nbytes if shared_mapping else 0
        d.layers = self._layers
        self._desc = d
        if cfg["dt_proj"] == 1:
            self.h = self.L.tm_cuda_llama_create(C.byref(d))
        else:
            self.h = self.L.tm_cuda_llama_create_dt(C.byref(d), cfg["dt_proj"])
        if not self.h:
            raise RuntimeError(lib.last_error())

    def prefill(self, x: np.ndarray, pos0: int) -> np.ndarray:
        """x: [T, D] float32; returns the residual stream after every layer (x is not modified)."""
        x = np.array(x, dtype=np.float32, copy=True, order="C")
        if not self.L.tm_cuda_llama_prefill(self.h, x.ctypes.data, x.shape[0], pos0):
            raise RuntimeError(lib.last_error())
        return x

    def begin_tokens(self, toks: np.ndarray, pos0: int) -> None:
        """prefill_begin whose residual stream is gathered on the device from the model's embedding table."""
        w = self.weights["embed"]
        woff = C.c_uint64(0)
        blob = self.weights["blob"]
        wid = self.L.tm_cuda_tok_wbuf(w.ctypes.data, w.nbytes, blob.ctypes.data, blob.nbytes, 1, C.byref(woff))
        if wid < 0:
            raise RuntimeError(lib.last_error())
        self._toks = np.ascontiguousarray(toks, np.int32)
        if not self.L.tm_cuda_llama_prefill_begin_tokens(self.h, self._toks.ctypes.data, self._toks.size, pos0, wid, woff.value,
                                                         self.cfg["V"], self.cfg["dt_embed"]):
            raise RuntimeError(lib.last_error())

    def begin(self, x: np.ndarray, pos0: int) -> None:
        self._x_in = np.ascontiguousarray(x, np.float32)
        if not self.L.tm_cuda_llama_prefill_begin(self.h, self._x_in.ctypes.data, self._x_in.shape[0], pos0):
            raise RuntimeError(lib.last_error())

    def wait_layer(self, l: int) -> bool:
        return bool(self.L.tm_cuda_llama_prefill_wait_layer(l))

    def end(self) -> bool:
        return bool(self.L.tm_cuda_llama_prefill_end())

    def gpu_ms(self) -> float:
        return float(self.L.tm_cuda_llama_prefill_gpu_ms())

    def close(self) -> None:
        if self.h:
            self.L.tm_cuda_llama_destroy(self.h)
            self.h = None
