"""ctypes view of libtm_chain.so: the C++ decode-chain driver (include/llama_chain.h)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtm_chain.so")
_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m tensormark_b200.build`")
        L = C.CDLL(LIB_PATH)
        L.tmchain_error.restype = C.c_char_p
        L.tmchain_create.restype = C.c_void_p
        L.tmchain_create.argtypes = [C.POINTER(C.c_int), C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.POINTER(C.c_void_p), C.c_void_p, C.c_size_t]
        L.tmchain_destroy.argtypes = [C.c_void_p]
        L.tmchain_seen.argtypes = [C.c_void_p]
        L.tmchain_set_seen.argtypes = [C.c_void_p, C.c_int]
        L.tmchain_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.tmchain_greedy.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.tmchain_feed.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.tmchain_chain_begin.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.tmchain_chain_begin_sampled.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_uint, C.c_int]
        L.tmchain_chain_poll.argtypes = [C.c_void_p, C.c_int]
        L.tmq_upload.argtypes = [C.c_char_p, C.POINTER(C.c_char_p), C.c_int, C.POINTER(C.c_ulonglong), C.POINTER(C.c_uint),
                                 C.POINTER(C.c_ulonglong)]
        L.tmchain_chain_end.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.tmchain_logits.argtypes = [C.c_void_p, C.c_void_p]
        L.tmchain_logit_rows.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.tmchain_logit_rows.restype = None
        L.tmchain_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.tmchain_prefill_prepare.argtypes = [C.c_void_p, C.c_int]
        L.tmchain_prefill_gpu_ms.argtypes = [C.c_void_p]
        L.tmchain_prefill_gpu_ms.restype = C.c_double
        _lib = L
    return _lib


def init_comm(cuda_lib, rank: int, world: int) -> None:
    """Create the lane's communicator on every rank of an initialised torch.distributed group:
    rank 0 makes the id, the group's broadcast carries it (any backend; gloo is enough)."""
    import torch
    import torch.distributed as dist

    n = int(cuda_lib.tm_cuda_comm_id_bytes())
    buf = (C.c_ubyte * n)()
    if rank == 0 and not cuda_lib.tm_cuda_comm_unique_id(buf):
        raise RuntimeError(cuda_lib.tm_cuda_last_error().decode())
    t = torch.tensor(list(bytes(buf)), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.broadcast(t, src=0)
    raw = bytes(t.cpu().tolist())
    if not cuda_lib.tm_cuda_comm_init(rank, world, (C.c_ubyte * n).from_buffer_copy(raw)):
        raise RuntimeError(cuda_lib.tm_cuda_last_error().decode())


def peer_arena_bytes(cfg: dict) -> int:
    """Bytes of shared slots a sharded model gathers into: the residual, gate|up and the logits."""
    return 4 * (cfg["D"] + 2 * cfg["F"] + cfg["V"]) + 4096


def init_peer(cuda_lib, rank: int, world: int, arena_bytes: int) -> None:
    """Create this rank's peer arena, exchange the IPC handles over the torch.distributed group and
    map the other ranks' arenas."""
    import torch
    import torch.distributed as dist

    n = int(cuda_lib.tm_cuda_peer_handle_bytes())
    buf = (C.c_ubyte * n)()
    if not cuda_lib.tm_cuda_peer_arena(arena_bytes, buf):
        raise RuntimeError(cuda_lib.tm_cuda_last_error().decode())
    mine = torch.tensor(list(bytes(buf)), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        mine = mine.cuda()
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    raw = b"".join(bytes(t.cpu().tolist()) for t in every)
    if not cuda_lib.tm_cuda_peer_open(rank, world, (C.c_ubyte * len(raw)).from_buffer_copy(raw)):
        raise RuntimeError(cuda_lib.tm_cuda_last_error().decode())


def tmq_upload(path: str, names: list[str]):
    """Tensors of a .tmq container onto the GPU under one weight handle (include/tmq_reader.h). Returns
    (handle, {name: (byte offset, dtype, nblocks)})."""
    L = load()
    n = len(names)
    arr = (C.c_char_p * n)(*[s.encode() for s in names])
    woff, dt, nb = (C.c_ulonglong * n)(), (C.c_uint * n)(), (C.c_ulonglong * n)()
    wid = L.tmq_upload(path.encode(), arr, n, woff, dt, nb)
    if wid < 0:
        raise RuntimeError(L.tmchain_error().decode())
    return wid, {names[i]: (int(woff[i]), int(dt[i]), int(nb[i])) for i in range(n)}


class Chain:
    """A model on the GPU decode lane. `weights` is the dict synth.make_llama returns (kept alive here:
    registrations are keyed by host address)."""

    def __init__(self, cfg: dict, weights: dict, shared_mapping: bool = True, rank: int = 0, world: int = 1,
                 peer_gather: bool = False):
        self.L, self.cfg, self.weights = load(), cfg, weights
        icfg = (C.c_int * 14)(cfg["L"], cfg["D"], cfg["H"], cfg["KVH"], cfg["dh"], cfg["F"], cfg["V"], cfg["ctx"],
                              cfg["dt_proj"], cfg["dt_head"], cfg["dt_embed"], rank, world, int(peer_gather))
        ptrs = []
        for l in range(cfg["L"]):
            for n in ("q", "k", "v", "o", "gate", "up", "down", "rms1", "rms2"):
                ptrs.append(weights[f"l{l}.{n}"].ctypes.data)
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        blob = weights["blob"]
        self.h = self.L.tmchain_create(icfg, cfg["theta"], cfg["eps"], weights["embed"].ctypes.data, weights["head"].ctypes.data,
                                       weights["rmsf"].ctypes.data, arr,
                                       blob.ctypes.data if shared_mapping else None, blob.nbytes if shared_mapping else 0)
        if not self.h:
            raise RuntimeError(self.L.tmchain_error().decode())

    def _check(self, ok):
        if not ok:
            raise RuntimeError(self.L.tmchain_error().decode())

    @property
    def seen(self) -> int:
        return self.L.tmchain_seen(self.h)

    @seen.setter
    def seen(self, v: int):
        self.L.tmchain_set_seen(self.h, v)

    def forward(self, tok: int) -> np.ndarray:
        logits = np.empty(self.cfg["V"], np.float32)
        self._check(self.L.tmchain_forward(self.h, int(tok), logits.ctypes.data))
        return logits

    def greedy(self, first: int, n: int, graph: bool = True):
        out = np.empty(n, np.int32)
        logits = np.empty(self.cfg["V"], np.float32)
        self._check(self.L.tmchain_greedy(self.h, int(first), n, out.ctypes.data, logits.ctypes.data, int(graph)))
        return out, logits

    def feed(self, tokens) -> int:
        """Run known tokens (a prompt) through the graph lane; returns the token chosen after the last one."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = self.L.tmchain_feed(self.h, t.ctypes.data, t.size)
        self._check(nxt >= 0)
        return nxt

    def prefill(self, tokens) -> int:
        """Run a prompt (three or more tokens) through the batched layer stack, its last token through the decode lane;
        returns the token chosen after it."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = self.L.tmchain_prefill(self.h, t.ctypes.data, t.size)
        self._check(nxt >= 0)
        return nxt

    def prefill_prepare(self, max_tokens: int = 0) -> None:
        """Create the layer stack ahead of the first prefill (device K/V caches, page-locked host arrays)."""
        self._check(self.L.tmchain_prefill_prepare(self.h, int(max_tokens)))

    def prefill_gpu_ms(self) -> float:
        return float(self.L.tmchain_prefill_gpu_ms(self.h))

    def chain_begin(self, first: int, n: int, graph: bool = True):
        self._check(self.L.tmchain_chain_begin(self.h, int(first), n, int(graph)))

    def chain_begin_sampled(self, first: int, n: int, inv_temp: float, seed: int, graph: bool = True):
        """Gumbel-max sampling on the GPU instead of the greedy choice (inv_temp = 1 / temperature)."""
        self._check(self.L.tmchain_chain_begin_sampled(self.h, int(first), n, float(inv_temp), int(seed), int(graph)))

    def chain_poll(self, i: int) -> int:
        return self.L.tmchain_chain_poll(self.h, i)

    def chain_end(self, n: int, keep: int = -1) -> np.ndarray:
        out = np.empty(n, np.int32)
        got = self.L.tmchain_chain_end(self.h, keep, out.ctypes.data, n)
        self._check(got >= 0)
        return out[:got]

    def logits(self) -> np.ndarray:
        """Logits of the most recent forward or finished chain."""
        out = np.empty(self.cfg["V"], np.float32)
        self.L.tmchain_logits(self.h, out.ctypes.data)
        return out

    def logit_rows(self) -> tuple[int, int]:
        """Rows of logits() that a finished chain left valid on this rank: all of them, or this rank's rows of the head
        when the ranks of a row-sharded model exchange only their choices."""
        lo, hi = C.c_int(0), C.c_int(0)
        self.L.tmchain_logit_rows(self.h, C.byref(lo), C.byref(hi))
        return lo.value, hi.value

    def close(self):
        if self.h:
            self.L.tmchain_destroy(self.h)
            self.h = None
