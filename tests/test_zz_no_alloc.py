"""nwc_linear_bf16_static: the token matvec for hosts that cannot allocate device memory for the library (their
runtime owns all of HBM, or the allocator is off limits to plugins).  Its partial sums live in a fixed area inside the
library instead of a caller buffer.  Called through the C-ABI twice in a row per matrix - the second call meets the
first call's leftovers in the shared area - and compared with nwc_linear_bf16 on the same inputs, with the tolerance
the other matvec tests use (relative L2 2e-3; both run the same deterministic kernels, so they normally agree bit for
bit).  The file name keeps it last in collection order, and it runs the same alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from helpers import rel_l2

pytestmark = pytest.mark.gpu

CASES = [(1001, 1000, 0, 0), (64, 2048, 0, 1), (130, 1536, 0, 2), (512, 4096, 0, 0), (100, 1000, 1, 1), (2048, 1024, 0, 2)]


def run(entry, nw, x, bias, with_scratch):
    from nwc_b200 import _lib as L
    y = torch.full((nw.out_features + 32,), 9.0, dtype=torch.bfloat16, device="cuda")       # canary tail
    head = [L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), L.ptr(x), L.ptr(bias), L.ptr(nw.scale)]
    tail = [L.ptr(y), nw.n, nw.block, nw.in_features, nw.code]
    err = entry(*(head + ([L.ptr(nw.scratch)] if with_scratch else []) + tail))
    assert err == 0, err
    torch.cuda.synchronize()
    assert (y[nw.out_features:] == 9.0).all()
    return y[: nw.out_features].clone()


@pytest.mark.parametrize("M,K,elem,layout", CASES)
def test_static_scratch_matches_caller_scratch(M, K, elem, layout):
    from gpu_helpers import bits, bf16_tensor, make_case, to_weight
    from nwc_b200 import _lib as L
    p, values, x_bits = make_case(M, K, elem, layout, seed=7 * M + K)
    nw = to_weight(p)
    bias = bf16_tensor(O.f32_to_bf16(np.linspace(-0.25, 0.25, M).astype(np.float32))).cuda()
    g = torch.Generator().manual_seed(M)
    for call in range(2):                                              # two calls in a row share the built-in area
        xb = torch.randn(K, generator=g).to(torch.bfloat16).cuda()
        xin = nw._padded_x((xb if layout else xb.float()).contiguous())
        want = run(L.lib.nwc_linear_bf16, nw, xin, bias, True)
        got = run(L.lib.nwc_linear_bf16_static, nw, xin, bias, False)
        a, b = O.bf16_to_f32(bits(got)), O.bf16_to_f32(bits(want))
        assert np.isfinite(a).all()
        assert rel_l2(a, b) <= 2e-3, (call, rel_l2(a, b))
        ref = O.bf16_to_f32(O.linear_bf16(p, O.bf16_to_f32(bits(xb)), bits(bias)))
        assert rel_l2(a, ref) <= 2e-3
    assert L.lib.nwc_kernel_status(1) == 0


def test_static_scratch_rejects_oversized_matrices():
    from nwc_b200 import _lib as L
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rows, K = 2_200_000, 512                                            # 2.2 M padded rows x 1 column block > 1 Mi floats
    err = L.lib.nwc_linear_bf16_static(L.stream(), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), None, None,
                                       L.ptr(dummy), rows * K, 4096, K, 0)
    assert err == -4
    assert L.lib.nwc_linear_bf16_static(L.stream(), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), L.ptr(dummy), None, None,
                                        L.ptr(dummy), 1000, 4096, 512, 0) == -1      # n % K != 0: the usual shape error
