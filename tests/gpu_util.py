"""Helpers for the gpu-marked tests: torch owns the device memory, the C ABI does the work."""
from __future__ import annotations

import ctypes as C

import numpy as np


def dev_bytes(torch, arr: np.ndarray, pad: int = 32):
    """uint8 array -> device tensor with `pad` spare bytes after the payload (16-byte aligned base)."""
    flat = np.ascontiguousarray(arr, dtype=np.uint8).reshape(-1)
    t = torch.zeros(flat.size + pad, dtype=torch.uint8, device="cuda")
    t[: flat.size] = torch.from_numpy(flat).cuda()
    return t


def dev_f32(torch, arr: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).cuda()


def stream_ptr(torch):
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr())


def gemv_dev(cuda, torch, dt, W_dev, x_dev, n, k):
    from tensormark_b200 import lib
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    ok = cuda.tm_cuda_gemv_q_dev(ptr(x_dev), ptr(W_dev), ptr(y), n, k, dt, stream_ptr(torch))
    lib.check(ok, "tm_cuda_gemv_q_dev")
    torch.cuda.synchronize()
    return y.cpu().numpy()
