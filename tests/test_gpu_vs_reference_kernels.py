"""A/B against the reference's own GPU kernels on the same compressed tensors.

The reference's library compiles unchanged for sm_100a (oracle/_ref/nwc_ops.so, checker only, made by `make -C oracle ref`
where the reference is mounted).  Both libraries are driven through the same ten-symbol C-ABI on the same device tensors
(matrices of a Qwen3-0.6B decoder layer and a slice of its lm_head, all layouts and element types): dequantised matrices and
gathered rows must be bit-identical, token matvecs must agree to bf16 output rounding (both accumulate in fp32, in
different orders).  Skipped where the reference library is absent."""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "nwc_ops.so")

P, U64, U32, I = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO): pytest.skip("reference library not built (oracle/_ref/nwc_ops.so)")
    R = ctypes.CDLL(REF_SO)
    R.nwc_setup.restype = I
    assert R.nwc_setup() > 0
    R.nwc_linear_bf16.restype, R.nwc_linear_bf16.argtypes = I, [P] * 11 + [U64, U32, U32, I]
    R.nwc_dequant.restype, R.nwc_dequant.argtypes = I, [P] * 7 + [U64, U32, U32, I]
    R.nwc_gather.restype, R.nwc_gather.argtypes = I, [P] * 7 + [U32, P, U64, U32, U32, I]
    return R


SHAPES = [("qkv", 4096, 1024), ("o", 1024, 2048), ("gate_up", 6144, 1024), ("down", 1024, 3072), ("lm_head slice", 16384, 1024), ("ragged", 1001, 1000)]


@pytest.mark.parametrize("elem", ["bf16", "fp8"])
@pytest.mark.parametrize("layout", [0, 1, 2])
@pytest.mark.parametrize("name,M,K", SHAPES)
def test_same_results_as_the_reference_kernels(ref, name, M, K, layout, elem):
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    w = NWCWeight(synthetic_matrix(M, K, M + K + layout), layout=layout, elem=elem)
    ops = (L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low))
    shape = (w.n, w.block, K, w.code)
    # dequant: bit-identical
    mine = w.dequant().contiguous()
    theirs = torch.zeros(M, w.K16, dtype=torch.bfloat16, device="cuda")
    assert ref.nwc_dequant(L.stream(), *ops, L.ptr(theirs), *shape) == 0
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs[:, :K].contiguous())
    # gather: bit-identical, incl. the first and last row
    ids = torch.tensor([0, M - 1, M // 2, 7 % M, M - 1], dtype=torch.int64, device="cuda")
    rows = torch.zeros(ids.numel(), w.K16, dtype=torch.bfloat16, device="cuda")
    assert ref.nwc_gather(L.stream(), *ops, L.ptr(ids), ids.numel(), L.ptr(rows), *shape) == 0
    torch.cuda.synchronize()
    assert torch.equal(w.gather(ids), rows[:, :K])
    # token matvec: x fp32 for layout 0, bf16 otherwise (the reference ABI), same bias and scale
    g = torch.Generator().manual_seed(K)
    x = torch.randn(K, generator=g).to(torch.bfloat16).cuda()
    bias = (0.1 * torch.randn(M, generator=g)).to(torch.bfloat16).cuda()
    xin = w._padded_x((x.float() if layout == 0 else x).contiguous())
    y_ref = torch.zeros(M, dtype=torch.bfloat16, device="cuda")
    assert ref.nwc_linear_bf16(L.stream(), *ops, L.ptr(xin), L.ptr(bias), L.ptr(w.scale), L.ptr(w.scratch), L.ptr(y_ref), *shape) == 0
    torch.cuda.synchronize()
    y = w.linear_bf16(x, bias).float()
    yr = y_ref.float()
    assert torch.isfinite(y).all()
    assert ((y - yr).norm() / yr.norm()).item() <= 2e-3
    assert (y - yr).abs().max().item() <= 2.0 ** -7 * yr.abs().max().item() + 1e-6
    assert L.lib.nwc_kernel_status(1) == 0
