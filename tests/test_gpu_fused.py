"""nwc_linear_fused (activation prologue fused into the token matvec) against the separate kernels and the oracle."""
import numpy as np
import pytest
import torch

import oracle as O
from helpers import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,layout,elem", [(4096, 1024, 0, 0), (1024, 2048, 0, 0), (1024, 3072, 0, 0), (6144, 1024, 0, 0), (100, 1000, 0, 0), (13, 40, 0, 0),
                                             (1024, 5120, 0, 0), (256, 1024, 0, 1), (512, 1024, 2, 0), (512, 1024, 1, 0),
                                             # layout 0 with many column blocks and more row groups than one round of the small kernel holds:
                                             # the entry point takes prologue + ring kernel + finalize instead
                                             (2560, 9728, 0, 0),
                                             (6144, 2560, 2, 0), (2560, 9728, 2, 0), (100, 1000, 2, 0), (13, 40, 2, 0), (48, 1004, 2, 0),
                                             # layout 2 shapes whose row groups do not divide over the SMs: equal runs per CTA, cut row groups completed
                                             # inside the kernel by the last CTA to arrive (no finalize launch)
                                             (1280, 8192, 2, 0), (2000, 4096, 2, 0), (4100, 3000, 2, 0), (16, 28672, 2, 0), (32, 28672, 2, 0), (7168, 1536, 2, 0),
                                             (512, 1024, 2, 1), (2560, 4096, 2, 1), (100, 1024, 2, 1)])
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


# ---- layout 0 with a side table: four warps per block ----

def _python_side_table(p):
    """Bit positions after 32, 64 and 96 symbols of every lane stream, walked with the code's length rule on the CPU."""
    M, K = p.M, p.K
    groups, CB = -(-M // 8), -(-K // 512)
    max_rank = 10 if p.elem else 15
    out = np.zeros((groups * CB, 3, 32), np.uint16)
    hdr = p.hdr.reshape(-1, 32).astype(np.int64)
    for b in range(groups * CB):
        words = np.frombuffer(p.data.tobytes()[int(p.bases[b]): int(p.bases[b]) + 4 * int(hdr[b].sum()) + 16], dtype="<u4")
        start = 0
        for lane in range(32):
            bits = "".join(format(int(w), "032b") for w in words[start: start + int(hdr[b, lane]) + 2])
            pos = 0
            for part in range(3):
                for _ in range(32):
                    zeros = 0
                    while zeros < 15 and bits[pos + zeros] == "0": zeros += 1
                    pos += zeros + 2 if (p.elem or zeros < max_rank) else 24
                out[b, part, lane] = pos
            start += int(hdr[b, lane])
    return out


@pytest.mark.parametrize("M,K,elem", [(13, 40, 0), (100, 1000, 0), (64, 2048, 0), (100, 1000, 1), (1024, 3072, 0)])
def test_side_table_matches_a_python_walk_of_the_streams(M, K, elem):
    from gpu_helpers import make_case, to_weight
    p, _, _ = make_case(M, K, elem, 0, seed=M + K, escapes=True)
    nw = to_weight(p)
    side = nw.build_side_table().cpu().numpy().view(np.uint16).reshape(-1, 3, 32)
    if M * K <= 200000: assert np.array_equal(side, _python_side_table(p))
    assert (np.diff(side.astype(np.int64), axis=1) >= 64).all() and (side[:, 0] >= 64).all()      # 32 symbols of at least two bits each
    assert nw.side_bytes == side.size * 2


@pytest.mark.parametrize("M,K,elem", [(4096, 1024, 0), (1024, 2048, 0), (6144, 1024, 0), (1024, 3072, 0), (100, 1000, 0), (13, 40, 0), (8, 512, 0), (1024, 5120, 0),
                                      (256, 1024, 1), (1001, 1000, 1)])
def test_split_kernel_matches_the_single_warp_kernel_and_the_oracle(M, K, elem):
    """nwc_linear_fused_opt with a side table (four warps per block) against the same call without one and the oracle, in
    all three input modes; escapes planted so that lanes leave the fast path in the middle of a row pair."""
    import ctypes
    from gpu_helpers import bits, make_case, to_weight
    from nwc_b200 import _lib as L
    p, values, _ = make_case(M, K, elem, 0, seed=3 * M + K, escapes=True)
    nw = to_weight(p)
    nw.build_side_table()
    g = torch.Generator().manual_seed(K)
    pad = (K + 31) // 32 * 32
    def vec(n, scale=1.0): return (torch.randn(n, generator=g) * scale).to(torch.bfloat16).cuda()
    x0, h_in, delta, norm_w, gate_up = vec(pad), vec(pad), vec(pad, 0.5), (1.0 + 0.1 * torch.randn(pad, generator=g)).to(torch.bfloat16).cuda(), vec(2 * K)
    x0[K:] = 0
    xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    opt = L.FusedOptions(None, 0, 0, -1, -1, 0, nw.side.data_ptr())

    def run(mode, with_side):
        y, h_out = torch.empty(M, dtype=torch.bfloat16, device="cuda"), torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
        err = L.lib.nwc_linear_fused_opt(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), mode, L.ptr(x0), L.ptr(h_in),
                                         L.ptr(delta), L.ptr(h_out), L.ptr(norm_w), 1e-6, L.ptr(gate_up), L.ptr(xtmp), None, L.ptr(nw.scale), L.ptr(nw.scratch),
                                         L.ptr(y), nw.n, nw.block, K, nw.code, ctypes.byref(opt) if with_side else None)
        assert err == 0, err
        torch.cuda.synchronize()
        return O.bf16_to_f32(bits(y)), h_out

    for mode in (0, 1, 2):
        a, ha = run(mode, True)
        b, hb = run(mode, False)
        assert np.isfinite(a).all() and rel_l2(a, b) <= 2e-3, (mode, rel_l2(a, b))
        assert np.abs(a - b).max() <= 2.0 ** -7 * np.abs(b).max() + 1e-6, mode
        assert torch.equal(ha, hb)
    want = O.bf16_to_f32(O.linear_bf16(p, O.bf16_to_f32(bits(x0[:K]))))
    assert rel_l2(run(0, True)[0], want) <= 2e-3
    assert L.lib.nwc_kernel_status(1) == 0


@pytest.mark.parametrize("M,K", [(4100, 3000), (2368, 3008), (4736, 1504)])
def test_row_groups_that_end_on_warp_boundaries(M, K):
    """Shapes on which a CTA of the layout-2 ring kernel owns exactly two row groups and the boundary between them falls
    between two of its warps: every warp then contributes only partial row sums, added up in shared memory.  Several weight
    and activation draws, both entry points, each result against the oracle."""
    from gpu_helpers import bits, make_case, to_weight
    from nwc_b200 import _lib as L
    pad = (K + 31) // 32 * 32
    xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    for seed in range(4):
        p, _, _ = make_case(M, K, 0, 2, seed=M + 3 * K + seed, escapes=bool(seed & 1))
        nw = to_weight(p)
        g = torch.Generator().manual_seed(K + seed)
        x0 = torch.randn(pad, generator=g).to(torch.bfloat16).cuda(); x0[K:] = 0
        want = O.bf16_to_f32(O.linear_bf16(p, O.bf16_to_f32(bits(x0[:K]))))
        for fused in (True, False):
            y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
            if fused:
                err = L.lib.nwc_linear_fused(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), 0, L.ptr(x0), None, None, None, None, 1e-6,
                                             None, L.ptr(xtmp), None, None, L.ptr(nw.scratch), L.ptr(y), nw.n, nw.block, K, nw.code)
            else:
                err = L.lib.nwc_linear_x16(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), L.ptr(x0), None, None, L.ptr(nw.scratch), L.ptr(y),
                                           nw.n, nw.block, K, nw.code)
            assert err == 0
            torch.cuda.synchronize()
            assert rel_l2(O.bf16_to_f32(bits(y)), want) <= 2e-3, (seed, fused)
    assert L.lib.nwc_kernel_status(1) == 0


@pytest.mark.parametrize("elem", [0, 1])
def test_next_matrix_hint_changes_no_result(elem):
    """The hint that names the next call's matrix (its first bytes are asked into L2 at this call's end) leaves y bit for bit
    as without it, whatever matrix it names: a larger one, a smaller one, the other element type, one of a layout the ring
    kernel does not take (ignored), or the matrix itself."""
    import ctypes
    from gpu_helpers import bits, make_case, to_weight
    from nwc_b200 import _lib as L
    shapes = [(512, 1024), (2560, 4096), (100, 1024), (48, 1024), (4100, 3008)]
    cases = [to_weight(make_case(M, K, elem, 2, seed=M + K, escapes=True)[0]) for M, K in shapes]
    cases.append(to_weight(make_case(256, 1024, 1 - elem, 2, seed=5, escapes=False)[0]))
    cases.append(to_weight(make_case(256, 1024, 0, 0, seed=6, escapes=False)[0]))
    g = torch.Generator().manual_seed(9)
    for nw in cases[:len(shapes)]:
        K, M = nw.in_features, nw.out_features
        pad = (K + 31) // 32 * 32
        x0 = torch.randn(pad, generator=g).to(torch.bfloat16).cuda(); x0[K:] = 0
        xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
        def run(opt):
            y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
            err = L.lib.nwc_linear_fused_opt(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), 0, L.ptr(x0), None, None, None, None,
                                             1e-6, None, L.ptr(xtmp), None, L.ptr(nw.scale), L.ptr(nw.scratch), L.ptr(y), nw.n, nw.block, K, nw.code, opt)
            assert err == 0, err
            torch.cuda.synchronize()
            return y
        plain = run(None)
        for nxt in cases:
            for mode in (0, 1, 2):
                o = L.FusedOptions(None, 0, 0, -1, -1, 0, None)
                o.next_low, o.next_n, o.next_K, o.next_elem, o.next_mode = nxt.low.data_ptr(), nxt.n, nxt.in_features, nxt.code, mode
                assert torch.equal(run(ctypes.byref(o)), plain), (M, K, nxt.out_features, nxt.in_features, mode)
    assert L.lib.nwc_kernel_status(1) == 0


@pytest.mark.parametrize("M,K,elem", [(10240, 8192, 0), (4100, 3000, 0), (7168, 1536, 0), (16, 28672, 0), (1280, 8192, 0), (2560, 4096, 1), (100, 1024, 0), (2368, 3008, 0)])
def test_pool_kernel_repeats_bit_for_bit_and_agrees_with_the_ring_kernel(M, K, elem):
    """Layout 2 on the kernel whose warps draw their stages from a per-CTA pool: which warp takes which stage changes from
    run to run, the result must not (stage partials are added in stage order, the parts of a cut row group in CTA order) -
    30 runs, bit for bit; and it agrees with the oracle and with the kernel of fixed per-warp runs, through both entry
    points (equal runs with cut row groups; whole row groups)."""
    from gpu_helpers import bits, make_case, to_weight
    from nwc_b200 import _lib as L
    p, _, _ = make_case(M, K, elem, 2, seed=7 * M + K, escapes=True)
    nw = to_weight(p)
    pad = (K + 31) // 32 * 32
    g = torch.Generator().manual_seed(M + K)
    x0 = torch.randn(pad, generator=g).to(torch.bfloat16).cuda(); x0[K:] = 0
    xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    want = O.bf16_to_f32(O.linear_bf16(p, O.bf16_to_f32(bits(x0[:K]))))
    def run(fused):
        y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
        if fused:
            err = L.lib.nwc_linear_fused(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), 0, L.ptr(x0), None, None, None, None, 1e-6,
                                         None, L.ptr(xtmp), None, L.ptr(nw.scale), L.ptr(nw.scratch), L.ptr(y), nw.n, nw.block, K, nw.code)
        else:
            err = L.lib.nwc_linear_x16(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), L.ptr(x0), None, L.ptr(nw.scale), L.ptr(nw.scratch),
                                       L.ptr(y), nw.n, nw.block, K, nw.code)
        assert err == 0, err
        torch.cuda.synchronize()
        return y
    try:
        for fused in (True, False):
            L.lib.nwc_set_pool_kernels(1)
            first = run(fused)
            assert rel_l2(O.bf16_to_f32(bits(first)), want) <= 2e-3, fused
            for _ in range(30): assert torch.equal(run(fused), first), fused
            L.lib.nwc_set_pool_kernels(0)
            fixed_runs = run(fused)
            assert rel_l2(O.bf16_to_f32(bits(fixed_runs)), O.bf16_to_f32(bits(first))) <= 2e-3, fused
    finally:
        L.lib.nwc_set_pool_kernels(0)
    assert L.lib.nwc_kernel_status(1) == 0


@pytest.mark.parametrize("M,K,elem", [(100, 1000, 0), (64, 2048, 0), (100, 1000, 1), (4096, 1024, 0), (13, 40, 0)])
def test_gather_with_side_table_is_bit_identical(M, K, elem):
    """Layout 0: with the side table the walk of a lane's stream starts at the row pair that holds the requested row; the
    rows must come back bit for bit as without it (every row of the matrix, so every position inside a block), and both
    equal the oracle's dequantised rows."""
    from gpu_helpers import bits, make_case, to_weight
    from nwc_b200 import _lib as L
    p, _, _ = make_case(M, K, elem, 0, seed=M + K, escapes=True)
    nw = to_weight(p)
    ids = torch.randperm(M, generator=torch.Generator().manual_seed(3)).cuda()
    plain = nw.gather(ids)
    assert nw.side is None
    nw.build_side_table()
    with_side = nw.gather(ids)
    assert torch.equal(plain, with_side)
    want = O.gather(p, ids.cpu().numpy())[:, :K]
    assert np.array_equal(bits(with_side)[:, :K], want)
    out = torch.empty(M, plain.shape[1], dtype=torch.bfloat16, device="cuda")
    other = to_weight(make_case(64, 1024, 0, 2, seed=1, escapes=False)[0])
    err = L.lib.nwc_gather_side(L.stream(), L.ptr(other.data), L.ptr(other.bases), L.ptr(other.hdr), L.ptr(other.lut), L.ptr(other.low), L.ptr(ids), 1, L.ptr(out),
                                other.n, other.block, 1024, other.code, L.ptr(nw.side))
    assert err == -1                                                  # a side table goes with layout 0 only
