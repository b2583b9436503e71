"""CPU-side checks of the shipped library: the C-ABI loads and exports what include/nwc_ops.h declares, its host
entry points (nwc_info, nwc_layout, nwc_build_tab) agree with the oracle, and the encoder rules the GPU encoder runs
per thread reproduce the oracle's (= the reference's) output when driven from a host loop."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

import oracle as O
from helpers import golden_cases, packed_from_fixture, same_compressed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "nwc_b200", "lib", "nwc_ops.so")
P = lambda a: ctypes.c_void_p(a.ctypes.data)


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        subprocess.run(["python", os.path.join(ROOT, "nwc_b200", "build.py")], check=True)
    return ctypes.CDLL(LIB)


def test_abi_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "nwc_ops.h")).read()
    declared = set(re.findall(r"\b(nwc_[a-z0-9_]+)\s*\(", header))
    assert {"nwc_info", "nwc_layout", "nwc_encode", "nwc_build_tab", "nwc_linear_bf16", "nwc_matvec", "nwc_dequant",
            "nwc_gather", "nwc_ref_fp8", "nwc_setup"} <= declared
    for name in declared: assert hasattr(lib, name), name


@pytest.mark.parametrize("H", [8, 1024, 2560, 8192, 16384])
def test_exchange_buffer_size_follows_the_documented_layout(lib, H):
    """A tensor-parallel exchange buffer = a 512-byte header, two pull slots of H bf16 values and, for each of two push
    slots, one partial per possible rank (8) of H / 2 eight-byte words {two bf16 rows, push number}; every slot rounded up
    to 256 bytes.  Pure host arithmetic: the hosts that allocate the buffer themselves rely on it."""
    lib.nwc_comm_bytes.restype, lib.nwc_comm_bytes.argtypes = ctypes.c_uint64, [ctypes.c_uint32]
    up = lambda n: (n + 255) // 256 * 256
    assert lib.nwc_comm_bytes(H) == 512 + 2 * up(2 * H) + 2 * 8 * up(4 * H)


def test_info_and_layout_match_reference_contract(lib):
    lib.nwc_info.restype = ctypes.c_int
    assert [lib.nwc_info(i) for i in range(9)] == [11, 1, 4096, 32, 4096, 1, 1, 1, -1]
    lib.nwc_layout.restype = ctypes.c_int; lib.nwc_layout.argtypes = [ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p]
    out = np.zeros(4, np.uint64)
    for M, K in [(1, 1), (8, 512), (13, 40), (3, 4097), (17, 520), (1001, 1000), (4096, 4096), (151936, 1024), (57344, 8192)]:
        for elem in (0, 1):
            for layout in (0, 1, 2):
                code = O.code_of(elem, layout)
                assert lib.nwc_layout(M, K, code, P(out)) == 0
                assert [int(v) for v in out] == O.layout(M, K, code)
                if O.ref_available(): assert [int(v) for v in out] == O.ref_layout(M, K, code)[1]
    assert lib.nwc_layout(0, 5, 0, P(out)) == -1 and lib.nwc_layout(5, 0, 0, P(out)) == -1


def test_build_tab_matches_oracle(lib):
    lib.nwc_build_tab.restype = None; lib.nwc_build_tab.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_int, ctypes.c_void_p]
    w, _ = O.synth_weights(64, 2048, 5)
    q, _ = O.quantize_fp8(w)
    for elem, src in ((0, w), (1, q)):
        for layout in (0, 1, 2):
            p = O.encode(src, O.code_of(elem, layout))
            lut = np.zeros(4096, np.uint32)
            lib.nwc_build_tab(None, P(p.psym), p.code, P(lut))
            assert np.array_equal(lut, p.lut)


def test_decode_entry_points_reject_bad_arguments_without_a_device(lib):
    """Shape and alignment errors are reported as -1 before anything touches the GPU."""
    lib.nwc_dequant.restype = ctypes.c_int
    lib.nwc_dequant.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int]
    assert lib.nwc_dequant(None, None, None, None, None, None, None, 4096, 2048, 512, 0) == -1      # block != 4096
    assert lib.nwc_dequant(None, None, None, None, None, None, None, 1000, 4096, 512, 0) == -1      # n % K
    assert lib.nwc_dequant(None, 8, None, None, 16, 16, 16, 4096, 4096, 512, 0) == -1              # data not 16-byte aligned
    assert lib.nwc_dequant(None, None, None, None, None, None, None, 4096, 4096, 512, 3 << 4) == -1  # unknown layout


@pytest.fixture(scope="module")
def harness():
    so = os.path.join(ROOT, "tests", "_build", "encode_core_harness.so")
    src = os.path.join(ROOT, "tests", "encode_core_harness.cpp")
    os.makedirs(os.path.dirname(so), exist_ok=True)
    deps = [src] + [os.path.join(ROOT, "nwc_b200", "csrc", f) for f in ("nwc_encode_core.h", "nwc_geometry.h")]
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", so, src], check=True)
    h = ctypes.CDLL(so)
    h.harness_encode.restype = ctypes.c_int64
    h.harness_encode.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    return h


def harness_encode(h, w, code):
    M, K = w.shape
    nb, n_low, n_scratch, K16 = O.layout(M, K, code)
    psym = np.zeros(1024, np.uint16); bases = np.zeros(nb, np.uint32); hdr = np.zeros(nb * 32, np.uint8)
    cap = 3 * w.size + nb * 64 + 4096
    data = np.zeros(cap, np.uint8); low = np.zeros(n_low + 512, np.uint8); lut = np.zeros(4096, np.uint32)
    w = np.ascontiguousarray(w)
    dl = h.harness_encode(P(w), w.size, K, code, P(psym), P(bases), P(hdr), P(data), cap, P(low), P(lut))
    if dl < 0: return dl
    return O.Packed(M, K, code, data[: dl + 64].copy(), bases, hdr, lut, low, psym, int(dl), K16, n_low, n_scratch)


@pytest.mark.parametrize("name,elem,layout,M,K,path", golden_cases(), ids=[c[0] for c in golden_cases()])
def test_encoder_rules_reproduce_golden_streams(harness, name, elem, layout, M, K, path):
    z = np.load(path)
    ref = packed_from_fixture(path, elem, layout, M, K)
    mine = harness_encode(harness, z["w"] if elem == 0 else z["q"], O.code_of(elem, layout))
    assert mine.data_len == ref.data_len and same_compressed(mine, ref)


@pytest.mark.parametrize("M,K", [(1, 1), (16, 512), (33, 1040), (5, 2049), (200, 513), (512, 4096)])
def test_encoder_rules_match_oracle(harness, M, K):
    w, _ = O.synth_weights(M, K, 7 * M + K)
    w = w.copy(); w.reshape(-1)[:: max(1, M * K // 41)] = 0x7149
    q, _ = O.quantize_fp8(np.where((w & 0x7F80) == 0x7100, 0x3C00, w).astype(np.uint16))
    for elem, src in ((0, w), (1, q)):
        for layout in (0, 1, 2):
            code = O.code_of(elem, layout)
            a, b = harness_encode(harness, src, code), O.encode(src, code)
            assert a.data_len == b.data_len and same_compressed(a, b) and np.array_equal(a.psym, b.psym)


def test_encoder_rules_error_codes(harness):
    assert harness_encode(harness, np.full((8, 512), 0x7F, np.uint8), O.code_of(1, 0)) == -2
    rng = np.random.default_rng(0)
    w = np.empty((16, 1024), np.uint16)
    w[:, :512] = rng.integers(10, 110, size=(16, 512)).astype(np.uint16) << 8
    w[:, 512:] = rng.integers(1, 8, size=(16, 512)).astype(np.uint16) << 8
    assert harness_encode(harness, w, O.code_of(0, 2)) == -3
