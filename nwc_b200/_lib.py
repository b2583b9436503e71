"""ctypes bridge to nwc_ops.so (the C-ABI declared in include/nwc_ops.h).

Search order: the NWC_DLL environment variable (A/B tests against another build), then nwc_b200/lib/nwc_ops.so.  There
is no fallback: without the CUDA library the package does not import.  Mirrors the binding block of the reference's
bridge (reference: nwc/nwc_torch.py:14-82).
"""
import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "nwc_ops.so"


def find_library() -> str:
    tried = []
    for cand in (os.environ.get("NWC_DLL"), os.path.join(HERE, "lib", LIB_NAME)):
        if not cand: continue
        tried.append(cand)
        if os.path.exists(cand): return cand
    raise ImportError("nwc_b200: kernel library not found (run `python nwc_b200/build.py`, needs nvcc); looked for " + ", ".join(tried))


LIB_PATH = find_library()
lib = ctypes.CDLL(LIB_PATH)

P, U64, U32, I = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
_SIGNATURES = {
    "nwc_info": (I, [I]),
    "nwc_layout": (I, [U64, U32, I, P]),
    "nwc_encode": (ctypes.c_int64, [P, U64, U32, I, P, P, P, P, P, U64, P]),
    "nwc_encode_device": (ctypes.c_int64, [P, P, U64, U32, I, P, P, P, P, U64, P]),
    "nwc_build_tab": (None, [P, P, I, P]),
    "nwc_linear_bf16": (I, [P, P, P, P, P, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_linear_bf16_splits": (I, [P, P, P, P, P, P, P, P, P, P, P, U64, U32, U32, I, U32]),
    "nwc_linear_x16": (I, [P, P, P, P, P, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_add_rmsnorm": (I, [P, P, P, P, P, ctypes.c_float, U32, P, P]),
    "nwc_linear_fused": (I, [P, P, P, P, P, P, I, P, P, P, P, P, ctypes.c_float, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_set_dependent_launch": (None, [I]),
    "nwc_linear_launches": (I, [U64, U32, I, I]),
    "nwc_linear_prefill": (I, [P, P, P, P, P, P, P, U32, U32, P, P, P, U32, U64, U32, U32, I]),
    "nwc_attention_decode": (I, [P, P, P, P, P, P, P, P, P, U32, U32, U32, U32, ctypes.c_float, P, P]),
    "nwc_set_plain_attention": (None, [I]),
    "nwc_swiglu": (I, [P, P, U32, P, P]),
    "nwc_argmax": (I, [P, P, U32, P, P, P, P, U32, U32]),
    "nwc_argmax_tp": (I, [P, P, U32, P, P, P, P, U32, U32, P, I, I]),
    "nwc_linear_fused_opt": (I, [P, P, P, P, P, P, I, P, P, P, P, P, ctypes.c_float, P, P, P, P, P, P, U64, U32, U32, I, P]),
    "nwc_comm_set_timeout_ms": (None, [U32]),
    "nwc_side_table_bytes": (U64, [U64, U32]),
    "nwc_build_side_table": (I, [P, P, P, P, P, U64, U32, U32, I]),
    "nwc_linear_bf16_static": (I, [P, P, P, P, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_matvec": (I, [P, P, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_dequant": (I, [P, P, P, P, P, P, P, U64, U32, U32, I]),
    "nwc_gather": (I, [P, P, P, P, P, P, P, U32, P, U64, U32, U32, I]),
    "nwc_gather_side": (I, [P, P, P, P, P, P, P, U32, P, U64, U32, U32, I, P]),
    "nwc_ref_fp8": (I, [P, P, P, P, P, U64, U32]),
    "nwc_setup": (I, []),
    "nwc_kernel_status": (I, [I]),
    "nwc_set_ring_kernels": (None, [I]),
    "nwc_set_prefill_halves": (None, [I]),
    "nwc_set_fixup_plans": (None, [I]),
    "nwc_set_pool_kernels": (None, [I]),
    "nwc_set_peer_sharing": (None, [I]),
    "nwc_comm_bytes": (U64, [U32]),
    "nwc_comm_alloc": (I, [P, U32]),
    "nwc_comm_free": (I, [P]),
    "nwc_comm_export": (I, [P, P]),
    "nwc_comm_import": (I, [P, P]),
    "nwc_comm_release": (I, [P]),
    "nwc_comm_slot": (P, [P, U32, I]),
    "nwc_allreduce_add_rmsnorm": (I, [P, P, I, I, I, P, P, P, ctypes.c_float, U32, P]),
}
for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)            # AttributeError here = a library that does not implement the C-ABI
    _fn.restype, _fn.argtypes = _res, _args



class FusedOptions(ctypes.Structure):
    """nwc_fused_options of include/nwc_ops.h: the exchange buffers of a tensor-parallel group with the push slots one
    nwc_linear_fused_opt call reads (in_slot) and writes (out_slot), -1 = unused; a layout-0 matrix's side table; and the hint that names the matrix the next call on the stream reads."""
    _fields_ = [("buffers", ctypes.c_void_p), ("rank", ctypes.c_int), ("world", ctypes.c_int), ("in_slot", ctypes.c_int),
                ("out_slot", ctypes.c_int), ("H", ctypes.c_uint32), ("side", ctypes.c_void_p),
                ("next_low", ctypes.c_void_p), ("next_n", ctypes.c_uint64), ("next_K", ctypes.c_uint32), ("next_elem", ctypes.c_int),
                ("next_mode", ctypes.c_int)]


VERSION = lib.nwc_info(0)
TAB_WORDS = lib.nwc_info(2)
HDR_BLOCK = lib.nwc_info(3)
FIXED_BLOCK = lib.nwc_info(4)
NPAIR = 1024                      # length of the freq / psym arrays of the encoder interface
RAW_SLACK = 512                   # bytes after the raw plane: the plane is read one super-chunk slot ahead
LANES = 32

SM_COUNT = lib.nwc_setup() if torch.cuda.is_available() else 0


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("nwc_b200 runs on CUDA devices only (no CPU path)")
