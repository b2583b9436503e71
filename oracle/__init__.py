"""ctypes front end of the CPU oracle (``oracle/nwc_oracle.cpp``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the benchmark may import this package;
the shipped library never does.  It also wraps the *host* entry points of the reference's own kernel library when
that library was compiled from the reference sources into ``oracle/_ref/nwc_ops.so`` (see ``oracle/Makefile``), so the
oracle's encoder can be compared with it byte for byte.

All arrays are numpy: bf16 values travel as ``uint16`` bit patterns, fp8 values as ``uint8``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libnwc_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "nwc_ops.so")

ELEM_BF16, ELEM_FP8 = 0, 1
LANES, SYM_TABLE_LEN, LUT_WORDS, RAW_SLACK = 32, 1024, 4096, 512

_P, _U64, _U32, _I = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int


def reference_root() -> str:
    """Where the reference checkout lies: the NWC_REFERENCE_ROOT variable, else a directory `reference` next to this
    repository.  Empty when there is none (the GPU box: only the prebuilt files travel there)."""
    cand = os.environ.get("NWC_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.exists(os.path.join(cand, "csrc", "nwc_ops.cu")) else ""


def build(ref: bool = True) -> None:
    """Compile the oracle (and the reference library when its sources are reachable)."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)
    root = reference_root()
    if ref and root:
        subprocess.run(["make", "-s", "-C", HERE, "ref", "REF=" + root], check=True)


def code_of(elem: int, layout: int) -> int:
    """The library's ``elem`` parameter: element type in bits 0..3, layout in bits 4..7."""
    return int(elem) | (int(layout) << 4)


def _ptr(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        L = ctypes.CDLL(ORACLE_SO)
        L.nwo_layout.restype = _I; L.nwo_layout.argtypes = [_U64, _U32, _I, _P]
        L.nwo_encode.restype = ctypes.c_int64; L.nwo_encode.argtypes = [_P, _U64, _U32, _I, _P, _P, _P, _P, _P, _U64, _P]
        L.nwo_build_tab.restype = None; L.nwo_build_tab.argtypes = [_P, _I, _P]
        L.nwo_decode.restype = _I; L.nwo_decode.argtypes = [_P, _P, _P, _P, _P, _U64, _U32, _I, _P, _I]
        L.nwo_matvec_f32.restype = _I; L.nwo_matvec_f32.argtypes = [_P, _P, _P, _P, _P, _P, _U64, _U32, _I, _P, _I]
        L.nwo_finalize.restype = None; L.nwo_finalize.argtypes = [_P, _P, _P, _U64, _P]
        L.nwo_gather.restype = _I; L.nwo_gather.argtypes = [_P, _P, _P, _P, _P, _P, _U32, _U64, _U32, _I, _P]
        L.nwo_fp8_to_bf16.restype = None; L.nwo_fp8_to_bf16.argtypes = [_P, _U64, _P]
        L.nwo_ref_fp8.restype = None; L.nwo_ref_fp8.argtypes = [_P, _P, _P, _U64, _U32, _P]
        _lib = L
    return _lib


@dataclass
class Packed:
    """One compressed matrix: the five format tensors plus sizes."""
    M: int
    K: int
    code: int
    data: np.ndarray          # uint8, length data_len (payload incl. 64 bytes of slack) + 64
    bases: np.ndarray         # uint32[nb]
    hdr: np.ndarray           # uint8[nb * 32]
    lut: np.ndarray           # uint32[4096]
    low: np.ndarray           # uint8[n_low + 512]
    psym: np.ndarray          # uint16[1024]
    data_len: int
    K16: int
    n_low: int
    n_scratch: int
    scale: np.ndarray | None = None
    extra: dict = field(default_factory=dict)

    @property
    def elem(self): return self.code & 15
    @property
    def layout(self): return (self.code >> 4) & 15
    @property
    def nb(self): return int(self.bases.size)

    @property
    def bytes(self) -> int:
        """Algorithmic bytes one matvec has to read: the reference's own size accounting."""
        return (self.data_len + 4 * self.bases.size + self.hdr.size + 4 * self.lut.size + self.n_low
                + (4 * self.scale.size if self.scale is not None else 0))

    def payloads(self) -> bytes:
        """Concatenated per-block payloads (bytes between blocks and after the last one are undefined)."""
        unit = 4 if self.layout != 2 else (2 if self.elem == ELEM_FP8 else 3)
        per_block = self.hdr.reshape(-1, LANES).astype(np.int64).sum(1) * unit
        raw = self.data.tobytes()
        return b"".join(raw[int(b): int(b) + int(n)] for b, n in zip(self.bases, per_block))


def layout(M: int, K: int, code: int):
    out = np.zeros(4, np.uint64)
    if lib().nwo_layout(M, K, code, _ptr(out)):
        raise ValueError("bad shape")
    return [int(v) for v in out]          # nb, raw-plane bytes, scratch floats, K16


def _encode_with(fn_encode, fn_tab, w: np.ndarray, code: int, tab_takes_freq: bool) -> Packed:
    assert w.ndim == 2 and w.dtype == (np.uint8 if code & 15 else np.uint16)
    M, K = w.shape
    n = M * K
    nb, n_low, n_scratch, K16 = layout(M, K, code)
    w = np.ascontiguousarray(w)
    freq = np.zeros(SYM_TABLE_LEN, np.uint16); psym = np.zeros(SYM_TABLE_LEN, np.uint16)
    bases = np.zeros(nb, np.uint32); hdr = np.zeros(nb * LANES, np.uint8)
    low = np.zeros(n_low + RAW_SLACK, np.uint8)
    dl = -1
    for cap in (n + n // 2 + nb * 64 + 4096, 3 * n + nb * 64 + 4096):
        data = np.zeros(cap, np.uint8)
        dl = fn_encode(_ptr(w), n, K, code, _ptr(freq), _ptr(psym), _ptr(bases), _ptr(hdr), _ptr(data), cap, _ptr(low))
        if dl >= 0 or dl in (-2, -3):
            break
    if dl < 0:
        raise EncodeError(int(dl))
    lut = np.zeros(LUT_WORDS, np.uint32)
    if tab_takes_freq: fn_tab(_ptr(freq), _ptr(psym), code, _ptr(lut))
    else: fn_tab(_ptr(psym), code, _ptr(lut))
    return Packed(M, K, code, data[: dl + 64].copy(), bases, hdr, lut, low, psym, int(dl), K16, n_low, n_scratch)


class EncodeError(ValueError):
    def __init__(self, rc):
        super().__init__({-1: "shape, capacity or over-long lane stream", -2: "fp8 weights contain NaN",
                          -3: "more than 255 exceptions in one lane (layout 2)"}.get(rc, f"rc {rc}"))
        self.rc = rc


def encode(w: np.ndarray, code: int) -> Packed:
    """Encode with the oracle's restatement of the host encoder."""
    L = lib()
    return _encode_with(L.nwo_encode, L.nwo_build_tab, w, code, tab_takes_freq=False)


def decode(p: Packed, threads: int = 1) -> np.ndarray:
    """uint16[M, K16] bf16 bits (fp8: the unscaled values); columns K..K16-1 are zero."""
    out = np.zeros((p.M, p.K16), np.uint16)
    rc = lib().nwo_decode(_ptr(p.data), _ptr(p.bases), _ptr(p.hdr), _ptr(p.lut), _ptr(p.low), p.M, p.K, p.code, _ptr(out), threads)
    if rc: raise ValueError(f"format violation {rc}")
    return out


def matvec_f32(p: Packed, x: np.ndarray, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32); assert x.size >= p.K
    y = np.zeros(p.M, np.float32)
    rc = lib().nwo_matvec_f32(_ptr(p.data), _ptr(p.bases), _ptr(p.hdr), _ptr(p.lut), _ptr(p.low), _ptr(x), p.M, p.K, p.code, _ptr(y), threads)
    if rc: raise ValueError(f"format violation {rc}")
    return y


def finalize(y32: np.ndarray, bias: np.ndarray | None = None, scale: np.ndarray | None = None) -> np.ndarray:
    y32 = np.ascontiguousarray(y32, np.float32); y = np.zeros(y32.size, np.uint16)
    if bias is not None: bias = np.ascontiguousarray(bias, np.uint16)
    if scale is not None: scale = np.ascontiguousarray(scale, np.float32)
    lib().nwo_finalize(_ptr(y32), _ptr(bias), _ptr(scale), y32.size, _ptr(y))
    return y


def linear_bf16(p: Packed, x: np.ndarray, bias=None, threads: int = 1) -> np.ndarray:
    """bf16 bits of scale * (W x) + bias with fp32 accumulation: what the fused token kernel must reproduce."""
    return finalize(matvec_f32(p, x, threads), bias, p.scale)


def gather(p: Packed, ids: np.ndarray) -> np.ndarray:
    ids = np.ascontiguousarray(ids, np.int64).reshape(-1)
    out = np.zeros((ids.size, p.K16), np.uint16)
    rc = lib().nwo_gather(_ptr(p.data), _ptr(p.bases), _ptr(p.hdr), _ptr(p.lut), _ptr(p.low), _ptr(ids), ids.size, p.M, p.K, p.code, _ptr(out))
    if rc: raise ValueError(f"format violation {rc}")
    return out


def fp8_to_bf16(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8); out = np.zeros(q.shape, np.uint16)
    lib().nwo_fp8_to_bf16(_ptr(q), q.size, _ptr(out))
    return out


def ref_fp8(q: np.ndarray, scale: np.ndarray, x: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8); M, K = q.shape
    y = np.zeros(M, np.uint16)
    lib().nwo_ref_fp8(_ptr(q), _ptr(np.ascontiguousarray(scale, np.float32)), _ptr(np.ascontiguousarray(x, np.float32)), M, K, _ptr(y))
    return y


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(v: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(v, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


# ------------------------------------------------------------------------------------------------------------------
# the reference's own library (host half), when compiled from its sources
_ref = None


def ref_available() -> bool:
    return os.path.exists(REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        R = ctypes.CDLL(REF_SO)
        R.nwc_info.restype = _I; R.nwc_info.argtypes = [_I]
        R.nwc_layout.restype = _I; R.nwc_layout.argtypes = [_U64, _U32, _I, _P]
        R.nwc_encode.restype = ctypes.c_int64; R.nwc_encode.argtypes = [_P, _U64, _U32, _I, _P, _P, _P, _P, _P, _U64, _P]
        R.nwc_build_tab.restype = None; R.nwc_build_tab.argtypes = [_P, _P, _I, _P]
        _ref = R
    return _ref


def ref_encode(w: np.ndarray, code: int) -> Packed:
    """Encode with the reference's compiled host encoder (bit-exact ground truth for the format)."""
    R = ref_lib()
    return _encode_with(R.nwc_encode, R.nwc_build_tab, w, code, tab_takes_freq=True)


def ref_layout(M, K, code):
    out = np.zeros(4, np.uint64)
    rc = ref_lib().nwc_layout(M, K, code, _ptr(out))
    return rc, [int(v) for v in out]


# ------------------------------------------------------------------------------------------------------------------
# synthetic inputs shared by tests and the benchmark

def synth_weights(M: int, K: int, seed: int = 0):
    """Rows scaled log-normally: W[i, j] = r_i * 0.02 * z_ij, r_i = exp(0.3 n_i); returns (W bf16 bits, x bf16 bits).
    Drawn with torch's CPU generator in the order r, z, x so the values match the known-answer hashes."""
    import torch
    g = torch.Generator().manual_seed(seed)
    r = torch.exp(0.3 * torch.randn(M, generator=g))
    z = torch.randn(M, K, generator=g)
    w = (r[:, None] * 0.02 * z).to(torch.bfloat16)
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    return w.view(torch.int16).numpy().view(np.uint16), x.view(torch.int16).numpy().view(np.uint16)


def quantize_fp8(w_bits: np.ndarray):
    """bf16 bits [M, K] -> (fp8 e4m3 bytes, fp32 scale[M]) with per-row absmax / 448 scaling."""
    import torch
    wf = torch.from_numpy(w_bits.view(np.int16)).view(torch.bfloat16).float()
    scale = wf.abs().amax(dim=1).clamp_min(1e-12) / 448.0
    q = (wf / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).numpy(), scale.numpy()
