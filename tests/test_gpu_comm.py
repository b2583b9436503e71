"""The tensor-parallel reduction kernel on one GPU: with a single rank it must equal the plain add + RMSNorm kernel (the
residual bit for bit, the normalised vector to one bf16 step), with two "ranks" that are two local buffers it must add both partials, and a peer that never announces itself
must end in status 3 after the bounded wait - no hang, the context stays usable."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(L, H, n):
    out = []
    for _ in range(n):
        p = ctypes.c_void_p()
        assert L.lib.nwc_comm_alloc(ctypes.byref(p), H) == 0
        out.append(p.value)
    return out


def _slot_tensor(L, buf, H, slot):
    """Device address of a partial slot of an exchange buffer."""
    return L.lib.nwc_comm_slot(ctypes.c_void_p(buf), H, slot)


def _write(addr, t):
    """Copy a tensor into library-owned device memory (the slot a matvec would write)."""
    from cuda.bindings import runtime as rt
    torch.cuda.synchronize()
    (rc,) = rt.cudaMemcpy(addr, t.data_ptr(), t.numel() * t.element_size(), rt.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
    assert int(rc) == 0, rc
    torch.cuda.synchronize()


@pytest.mark.parametrize("H", [256, 1024, 8192])
def test_single_rank_equals_add_rmsnorm(H):
    from nwc_b200 import _lib as L
    g = torch.Generator().manual_seed(H)
    h = torch.randn(H, generator=g).to(torch.bfloat16).cuda()
    part = (0.5 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    (buf,) = _buffers(L, H, 1)
    try:
        for slot in (0, 1, 0):                                        # three calls: the call counter advances, both slots work
            _write(_slot_tensor(L, buf, H, slot), part)
            h_out, xn = torch.zeros_like(h), torch.zeros_like(h)
            table = (ctypes.c_void_p * 1)(buf)
            assert L.lib.nwc_allreduce_add_rmsnorm(L.stream(), table, 0, 1, slot, L.ptr(h), L.ptr(h_out), L.ptr(w), 1e-6, H, L.ptr(xn)) == 0
            want_h, want_x = torch.zeros_like(h), torch.zeros_like(h)
            assert L.lib.nwc_add_rmsnorm(L.stream(), L.ptr(h), L.ptr(part), L.ptr(want_h), L.ptr(w), 1e-6, H, L.ptr(want_x), None) == 0
            torch.cuda.synchronize()
            assert torch.equal(h_out, want_h)
            # the sum of squares is added in a different order (eight CTAs): the normalised vector may differ by one bf16 step
            assert ((xn.float() - want_x.float()).abs() <= 2.0 ** -7 * want_x.float().abs() + 1e-30).all()
            assert (xn != want_x).float().mean().item() < 0.02
        assert L.lib.nwc_kernel_status(1) == 0
    finally:
        L.lib.nwc_comm_free(ctypes.c_void_p(buf))


def test_two_local_ranks_add_in_rank_order_and_missing_peer_times_out():
    from nwc_b200 import _lib as L
    H = 1024
    g = torch.Generator().manual_seed(7)
    h = torch.randn(H, generator=g).to(torch.bfloat16).cuda()
    parts = [(0.5 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda() for _ in range(2)]
    w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    a, b = _buffers(L, H, 2)
    try:
        _write(_slot_tensor(L, a, H, 0), parts[0]); _write(_slot_tensor(L, b, H, 0), parts[1])
        table = (ctypes.c_void_p * 2)(a, b)
        outs = []
        # both "ranks" run on this GPU one after the other: rank 0 waits for rank 1's announcement, which only comes with
        # rank 1's own launch afterwards, so rank 0's bounded wait runs out first (status 3) and it carries on
        for rank in (0, 1):
            h_out, xn = torch.zeros_like(h), torch.zeros_like(h)
            assert L.lib.nwc_allreduce_add_rmsnorm(L.stream(), table, rank, 2, 0, L.ptr(h), L.ptr(h_out), L.ptr(w), 1e-6, H, L.ptr(xn)) == 0
            torch.cuda.synchronize()
            outs.append(h_out)
            if rank == 0: assert L.lib.nwc_kernel_status(1) == 3          # gave up waiting, reported, context still usable
            else: assert L.lib.nwc_kernel_status(1) == 0                  # rank 0 had announced itself: no wait
        total = (parts[0].float() + parts[1].float()).to(torch.bfloat16)
        want = (h.float() + total.float()).to(torch.bfloat16)
        assert torch.equal(outs[0], want) and torch.equal(outs[1], want)  # the data was there all along: same sums on both
        y = torch.ones(4, device="cuda") * 2                              # the context still works
        assert float(y.sum()) == 8.0
    finally:
        L.lib.nwc_comm_free(ctypes.c_void_p(a)); L.lib.nwc_comm_free(ctypes.c_void_p(b))
