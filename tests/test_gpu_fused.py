"""nwc_linear_fused (activation prologue fused into the token matvec) against the separate kernels and the oracle."""
import numpy as np
import pytest
import torch

import oracle as O
from helpers import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,layout,elem", [(4096, 1024, 0, 0), (1024, 2048, 0, 0), (1024, 3072, 0, 0), (6144, 1024, 0, 0), (100, 1000, 0, 0), (13, 40, 0, 0),
                                             (1024, 5120, 0, 0), (256, 1024, 0, 1), (512, 1024, 2, 0), (512, 1024, 1, 0),
                                             (6144, 2560, 2, 0), (2560, 9728, 2, 0), (100, 1000, 2, 0), (13, 40, 2, 0), (48, 1004, 2, 0),
                                             # layout 2 shapes whose row groups do not divide over the SMs: equal runs per CTA, cut row groups completed
                                             # inside the kernel by the last CTA to arrive (no finalize launch)
                                             (1280, 8192, 2, 0), (2000, 4096, 2, 0), (4100, 3000, 2, 0), (16, 28672, 2, 0), (7168, 1536, 2, 0)])
def test_fused_modes_match_separate_kernels(M, K, layout, elem):
    from gpu_helpers import bits, bf16_tensor, make_case, to_weight
    from nwc_b200 import _lib as L
    p, values, _ = make_case(M, K, elem, layout, seed=M + 3 * K, escapes=False)
    nw = to_weight(p)
    g = torch.Generator().manual_seed(K)
    pad = (K + 31) // 32 * 32
    def vec(n, scale=1.0): return (torch.randn(n, generator=g) * scale).to(torch.bfloat16).cuda()
    h_in, delta, norm_w, gate_up = vec(pad), vec(pad, 0.5), (1.0 + 0.1 * torch.randn(pad, generator=g)).to(torch.bfloat16).cuda(), vec(2 * K)
    xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")

    def fused(mode, x=None, h_out=None):
        y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
        err = L.lib.nwc_linear_fused(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), mode, L.ptr(x), L.ptr(h_in),
                                     L.ptr(delta), L.ptr(h_out), L.ptr(norm_w), 1e-6, L.ptr(gate_up), L.ptr(xtmp), None, L.ptr(nw.scale), L.ptr(nw.scratch),
                                     L.ptr(y), nw.n, nw.block, K, nw.code)
        assert err == 0, err
        return y

    def separate(x):
        y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
        err = L.lib.nwc_linear_x16(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), L.ptr(x), None, L.ptr(nw.scale),
                                   L.ptr(nw.scratch), L.ptr(y), nw.n, nw.block, K, nw.code)
        assert err == 0, err
        return y

    def close(a, b):
        a, b = O.bf16_to_f32(bits(a)), O.bf16_to_f32(bits(b))
        assert np.isfinite(a).all() and rel_l2(a, b) <= 2e-3, rel_l2(a, b)

    # mode 0 (twice: the fix-up counters of the first call must be back at zero for the second)
    x0 = vec(pad); x0[K:] = 0
    close(fused(0, x=x0), separate(x0))
    assert torch.equal(fused(0, x=x0), fused(0, x=x0))
    # mode 1: residual add + RMSNorm
    h_ref, xn = h_in.clone(), torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    assert L.lib.nwc_add_rmsnorm(L.stream(), L.ptr(h_in), L.ptr(delta), L.ptr(h_ref), L.ptr(norm_w), 1e-6, K, L.ptr(xn), None) == 0
    h_out = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    close(fused(1, h_out=h_out), separate(xn))
    assert torch.equal(h_out[:K], h_ref[:K])
    want = (h_in[:K].float() + delta[:K].float()).to(torch.bfloat16)
    assert torch.equal(h_out[:K], want)
    # mode 2: SwiGLU
    act = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    assert L.lib.nwc_swiglu(L.stream(), L.ptr(gate_up), K, L.ptr(act), None) == 0
    close(fused(2), separate(act))
    # and against the oracle on the plain mode
    want0 = O.bf16_to_f32(O.linear_bf16(p, O.bf16_to_f32(bits(x0[:K]))))
    assert rel_l2(O.bf16_to_f32(bits(fused(0, x=x0))), want0) <= 2e-3
    assert L.lib.nwc_kernel_status(1) == 0
