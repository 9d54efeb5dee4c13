"""CPU: the host-side headers under include/, the GEMV lane maps, and the C ABI's symbol table."""
from __future__ import annotations

import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from tensormark_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [synth.Q8_0, synth.Q4_0, synth.Q4_1, synth.Q5_K, synth.Q6_K, synth.Q4_K, synth.TQ2]
_f32p = C.POINTER(C.c_float)


def _build(tmp, src, out, extra=()):
    path = os.path.join(tmp, out)
    subprocess.run(["g++", "-std=c++23", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
                    "-I" + os.path.join(ROOT, "include"), *extra, "-o", path, os.path.join(ROOT, "tests", "host", src)],
                   check=True)
    return C.CDLL(path)


@pytest.fixture(scope="module")
def hc(tmp_path_factory):
    lib = _build(str(tmp_path_factory.mktemp("hc")), "host_contracts.cpp", "libhc.so")
    lib.hc_dequant.argtypes = [C.c_uint, C.c_void_p, _f32p, C.c_size_t]
    lib.hc_fp16_to_fp32.restype = C.c_float
    lib.hc_fp16_to_fp32.argtypes = [C.c_uint16]
    lib.hc_fp32_to_fp16.restype = C.c_uint16
    lib.hc_fp32_to_fp16.argtypes = [C.c_float]
    lib.hc_weight_bytes.restype = C.c_size_t
    lib.hc_weight_bytes.argtypes = [C.c_uint, C.c_size_t, C.c_size_t]
    lib.hc_pool_gemv.argtypes = [C.c_uint, C.c_void_p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
    return lib


@pytest.fixture(scope="module")
def lanes(tmp_path_factory):
    lib = _build(str(tmp_path_factory.mktemp("lanes")), "lane_emul.cpp", "liblanes.so")
    lib.lane_emul_gemv.argtypes = [C.c_int, C.c_void_p, _f32p, _f32p, C.c_uint, C.c_uint]
    return lib


@pytest.mark.parametrize("dt", DTYPES)
def test_header_dequant_matches_golden(hc, golden, dt):
    name = synth.DTYPE_NAMES[dt]
    blocks = np.ascontiguousarray(golden[f"{name}_blocks"])
    n = blocks.shape[0] * synth.BLOCK_ELEMS[dt]
    out = np.empty(n, np.float32)
    assert hc.hc_dequant(dt, blocks.ctypes.data, out.ctypes.data_as(_f32p), n)
    assert np.array_equal(out.view(np.uint32), golden[f"{name}_dequant_bits"])


def test_header_fp16_and_geometry(hc, golden):
    fin = golden["fp32_to_fp16_in_bits"].view(np.float32)
    got = np.array([hc.hc_fp32_to_fp16(float(v)) for v in fin], dtype=np.uint16)
    assert np.array_equal(got, golden["fp32_to_fp16_out"])
    want = golden["fp16_to_fp32_bits"]
    for h in list(range(0, 2048)) + list(range(0x7bf0, 0x7c00)) + list(range(0x8000, 0x8400)):
        assert np.float32(hc.hc_fp16_to_fp32(h)).view(np.uint32) == want[h]
    for dt in DTYPES:
        assert hc.hc_weight_bytes(dt, 7, 512) == synth.weight_bytes(dt, 7, 512)
    assert hc.hc_weight_bytes(synth.Q6_K, 7, 96) == 0          # not whole super-blocks
    out = np.empty(96, np.float32)
    assert hc.hc_dequant(synth.Q6_K, out.ctypes.data, out.ctypes.data_as(_f32p), 96) == 0


def test_projection_strategy_contract(hc):
    assert hc.hc_strategy_selftest() == 0


@pytest.mark.parametrize("dt", [synth.Q4_0, synth.Q5_K])
def test_gemv_pool_rows(hc, orc, dt):
    n, k = 200, 512                         # 200 rows: three full 64-row chunks and a ragged one
    W = synth.make_weights(dt, n, k, seed=8)
    x = synth.make_activations(k, seed=9)
    y = np.zeros(n, np.float32)
    used = hc.hc_pool_gemv(dt, W.ctypes.data, x.ctypes.data_as(_f32p), y.ctypes.data_as(_f32p), n, k, 3)
    assert used == 3
    y64, yabs = orc.gemv_f64(dt, W, x, n, k)
    assert np.all(np.abs(y - y64) <= 1e-5 * yabs)


@pytest.mark.parametrize("dt,shapes", [
    (synth.Q4_0, [(5, 2048), (3, 5632), (3, 96), (2, 32)]),
    (synth.Q8_0, [(5, 2048), (3, 5632), (2, 32)]),
    (synth.Q4_1, [(5, 2048), (3, 5632), (2, 160)]),
    (synth.Q5_K, [(4, 4096), (2, 14336), (3, 256), (2, 768)]),
    (synth.Q6_K, [(4, 4096), (2, 14336), (3, 2048), (2, 256), (2, 5632)]),
    (synth.Q4_K, [(4, 4096), (2, 14336), (3, 256), (2, 768)]),
    (synth.GGUF_Q4_0, [(5, 2048), (3, 5632), (3, 96), (2, 32)]),
])
def test_gemv_lane_maps_on_cpu(lanes, orc, dt, shapes):
    """The kernel's lane decomposition, replayed on the CPU, against the fp64 reference.
    Tolerance: 1e-3 * sum|w x| is the path's bar; the lane arithmetic must also stay inside the bound derived
    from its activation format (tests/bounds.py) plus fp32 accumulation noise."""
    from tests.bounds import activation_rounding_bound
    for n, k in shapes:
        W = synth.make_weights(dt, n, k, seed=11)
        x = synth.make_activations(k, seed=12)
        y = np.zeros(n, np.float32)
        assert lanes.lane_emul_gemv(dt, W.ctypes.data, x.ctypes.data_as(_f32p), y.ctypes.data_as(_f32p), n, k)
        y64, yabs = orc.gemv_f64(dt, W, x, n, k)
        err = np.abs(y - y64)
        assert np.all(err <= 1e-3 * yabs), (synth.DTYPE_NAMES[dt], n, k)
        assert np.all(err <= activation_rounding_bound(orc, dt, W, x, n, k) + 2e-6 * yabs), (synth.DTYPE_NAMES[dt], n, k)


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            names.update(re.findall(r"\b(tm_cuda_\w+)\s*\(", text))
    return names


def test_c_abi_exports_every_declared_symbol():
    """Loads the library (no device needed for dlopen) and resolves every entry point the headers declare,
    plus the reference's tm_metal_* names for the same entries."""
    from tensormark_b200 import lib
    if not os.path.exists(lib.LIB_PATH):
        from tensormark_b200 import build
        build.build()
    L = lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 50
    for name in declared:
        assert hasattr(L, name), name
    assert declared == set(lib.SIGNATURES), declared ^ set(lib.SIGNATURES)
    metal = ["tm_metal_q4_gemv", "tm_metal_sgemm_q4", "tm_metal_q4_prefill", "tm_metal_tok_begin", "tm_metal_tok_end",
             "tm_metal_tok_gemv", "tm_metal_tok_gemv_seg", "tm_metal_tok_gemv_seg_dt", "tm_metal_tok_gemv_kq",
             "tm_metal_tok_wbuf", "tm_metal_tok_attn", "tm_metal_tok_argmax", "tm_metal_tok_rmsnorm", "tm_metal_tok_peek"]
    for name in metal:
        assert hasattr(L, name), name
    # pure host arithmetic works without a device
    assert L.tm_cuda_weight_bytes(1, 2048, 2048) == 2048 * 64 * 18
    assert L.tm_cuda_weight_bytes(6, 4, 100) == 0


# ---- .tmq container reader (include/tmq_reader.h) ---------------------------------------------------------
def _tmq_bytes(tensors) -> bytes:
    """Serialize [(name, dtype, shape, payload bytes)] as the format tensormark/tmq.h:4-6 describes."""
    import struct
    out = [b"TMQ1", struct.pack("<I", len(tensors))]
    for name, dt, shape, payload in tensors:
        nb = name.encode()
        n = int(np.prod(shape))
        be = {0: 32, 1: 32, 2: 1, 3: 1, 4: 32, 5: 256, 6: 256, 7: 128, 8: 256}[dt]
        out += [struct.pack("<I", len(nb)), nb, struct.pack("<II", dt, len(shape)),
                struct.pack("<%dI" % len(shape), *shape), struct.pack("<Q", n // be), payload]
    return b"".join(out)


def test_tmq_reader_accepts_and_rejects(hc, tmp_path):
    hc.hc_tmq_count.argtypes = [C.c_char_p]
    hc.hc_tmq_tensor.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong),
                                 C.POINTER(C.c_uint), C.POINTER(C.c_uint)]
    w1 = synth.make_weights(synth.Q4_0, 6, 64, seed=1).tobytes()
    w2 = synth.make_weights(synth.Q6_K, 3, 512, seed=2).tobytes()
    f16 = np.arange(10, dtype=np.float16).tobytes()
    good = _tmq_bytes([("layers.0.q", 1, (6, 64), w1), ("head", 6, (3, 512), w2), ("norm", 3, (10,), f16)])

    def count(data: bytes) -> int:
        p = tmp_path / "t.tmq"
        p.write_bytes(data)
        return hc.hc_tmq_count(str(p).encode())

    assert count(good) == 3
    dt, nb, off, rank = C.c_uint(), C.c_ulonglong(), C.c_ulonglong(), C.c_uint()
    dims = (C.c_uint * 4)()
    assert hc.hc_tmq_tensor(str(tmp_path / "t.tmq").encode(), b"head", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims)
    assert (dt.value, nb.value, rank.value, dims[0], dims[1]) == (6, 6, 2, 3, 512)
    assert good[off.value: off.value + len(w2)] == w2                 # the view points at the tensor's blocks
    assert not hc.hc_tmq_tensor(str(tmp_path / "t.tmq").encode(), b"absent", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims)
    # the reference parser's rejections (tensormark/tmq.h:157-161): trailing bytes, truncation, bad magic, unknown
    # dtype, zero dimension, block count that does not match the shape, a count larger than the file can hold
    assert count(good + b"\0") == -1
    assert count(good[:-1]) == -1
    assert count(b"TMQ2" + good[4:]) == -1
    assert count(_tmq_bytes([("x", 8, (256,), b"\0" * 144)])) == -1   # Q4_K only comes from the GGUF-native reader
    import struct
    bad_dim = b"TMQ1" + struct.pack("<I", 1) + struct.pack("<I", 1) + b"x" + struct.pack("<II", 1, 2) + struct.pack("<II", 0, 32) + struct.pack("<Q", 0)
    assert count(bad_dim) == -1
    wrong_blocks = bytearray(_tmq_bytes([("x", 1, (2, 32), w1[:36])]))
    i = wrong_blocks.index(struct.pack("<Q", 2))
    wrong_blocks[i: i + 8] = struct.pack("<Q", 1)
    assert count(bytes(wrong_blocks)) == -1
    assert count(b"TMQ1" + struct.pack("<I", 1000)) == -1
    assert count(b"TMQ1" + struct.pack("<I", 0)) == 0                 # an empty container is a valid one


# ---- GGUF files read natively (include/gguf_reader.h through tmmq::Mapped) ------------------------------------
def _gguf_bytes(tensors, arch="llama", alignment=None, extra_kv=(), version=3, dup_key=False) -> bytes:
    """Serialize [(gguf name, gguf type, dims innermost first, payload)] as a GGUF v3 file."""
    import struct

    def s(t: str) -> bytes:
        b = t.encode()
        return struct.pack("<Q", len(b)) + b

    kv = [s("general.architecture") + struct.pack("<I", 8) + s(arch)]
    if alignment is not None:
        kv.append(s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", alignment))
    kv.append(s("general.name") + struct.pack("<I", 8) + s("synthetic"))
    kv.append(s("llama.block_count") + struct.pack("<I", 4) + struct.pack("<I", 1))
    kv.append(s("tokenizer.scores") + struct.pack("<I", 9) + struct.pack("<IQ", 6, 3) + struct.pack("<3f", 1, 2, 3))     # array of f32
    kv.append(s("tokenizer.tokens") + struct.pack("<I", 9) + struct.pack("<IQ", 8, 2) + s("a") + s("bc"))                # array of strings
    kv += list(extra_kv)
    if dup_key:
        kv.append(kv[2])
    align = alignment or 32
    infos, blobs, rel = [], [], 0
    for name, typ, dims, payload in tensors:
        infos.append(s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, rel))
        pad = (-len(payload)) % align
        blobs.append(payload + b"\0" * pad)
        rel += len(payload) + pad
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    head += b"\0" * ((-len(head)) % align)
    return head + b"".join(blobs)


def test_gguf_index_is_read_natively(hc, tmp_path):
    hc.hc_tmq_count.argtypes = [C.c_char_p]
    hc.hc_tmq_tensor.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong),
                                 C.POINTER(C.c_uint), C.POINTER(C.c_uint)]
    q4 = synth.make_weights(synth.GGUF_Q4_0, 6, 64, seed=1).tobytes()      # 6 x 64, GGUF type 2
    q6 = synth.make_weights(synth.Q6_K, 3, 512, seed=2).tobytes()           # GGUF type 14
    q8 = synth.make_weights(synth.Q8_0, 4, 64, seed=3).tobytes()            # GGUF type 8
    nrm = np.arange(64, dtype=np.float32).tobytes()                         # GGUF type 0
    bf = np.arange(128, dtype=np.uint16).tobytes()                          # GGUF type 30
    tensors = [("blk.0.attn_q.weight", 2, (64, 6), q4), ("output.weight", 14, (512, 3), q6), ("token_embd.weight", 8, (64, 4), q8),
               ("output_norm.weight", 0, (64,), nrm), ("blk.0.ffn_down.weight", 30, (64, 2), bf),
               ("v.patch_embd.weight", 0, (64,), nrm)]                      # a vision tensor: indexed, not kept
    good = _gguf_bytes(tensors)

    def count(data: bytes) -> int:
        p = tmp_path / "m.gguf"
        p.write_bytes(data)
        return hc.hc_tmq_count(str(p).encode())

    assert count(good) == 5
    dt, nb, off, rank = C.c_uint(), C.c_ulonglong(), C.c_ulonglong(), C.c_uint()
    dims = (C.c_uint * 4)()
    path = str(tmp_path / "m.gguf").encode()
    # names are the engine's; shapes outermost first; GGUF's Q4_0 is container dtype 9, not 1 (tmq.h:446-457)
    assert hc.hc_tmq_tensor(path, b"model.layers.0.self_attn.q_proj.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims)
    assert (dt.value, nb.value, rank.value, dims[0], dims[1]) == (9, 12, 2, 6, 64)
    assert good[off.value: off.value + len(q4)] == q4
    assert hc.hc_tmq_tensor(path, b"lm_head.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims)
    assert (dt.value, nb.value, dims[0], dims[1]) == (6, 6, 3, 512) and good[off.value: off.value + len(q6)] == q6
    assert hc.hc_tmq_tensor(path, b"model.embed_tokens.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims) and dt.value == 0
    assert hc.hc_tmq_tensor(path, b"model.norm.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims) and dt.value == 2
    assert hc.hc_tmq_tensor(path, b"model.layers.0.mlp.down_proj.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims) and dt.value == 10
    assert not hc.hc_tmq_tensor(path, b"v.patch_embd.weight", C.byref(dt), C.byref(nb), C.byref(off), C.byref(rank), dims)
    assert count(_gguf_bytes(tensors, alignment=64)) == 5
    # refusals (tensormark/gguf_native.h:142-222): other versions, truncated payload, duplicate metadata key, duplicate
    # tensor name, an alignment that is not a power of two, a type outside the engine's set, rows that are not whole
    # blocks, a zero dimension, five dimensions, overlapping payloads
    import struct
    assert count(_gguf_bytes(tensors, version=2)) == -1
    assert count(good[:-40]) == -1
    assert count(_gguf_bytes(tensors, dup_key=True)) == -1
    assert count(_gguf_bytes(tensors + [("output.weight", 0, (64,), nrm)])) == -1
    assert count(_gguf_bytes(tensors, alignment=48)) == -1
    assert count(_gguf_bytes([("blk.0.attn_q.weight", 6, (64, 6), q4)])) == -1          # Q5_0 is not carried
    assert count(_gguf_bytes([("blk.0.attn_q.weight", 2, (48, 8), q4)])) == -1
    assert count(_gguf_bytes([("blk.0.attn_q.weight", 0, (0,), b"")])) == -1
    assert count(_gguf_bytes([("blk.0.attn_q.weight", 0, (2, 2, 2, 2, 4), nrm)])) == -1
    over = bytearray(_gguf_bytes([("a.weight", 0, (64,), nrm), ("b.weight", 0, (64,), nrm)]))
    i = over.rindex(struct.pack("<IQ", 0, 256))                                         # second tensor's (type, offset)
    over[i: i + 12] = struct.pack("<IQ", 0, 128)
    assert count(bytes(over)) == -1
