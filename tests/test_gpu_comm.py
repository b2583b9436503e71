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


# ---- the push protocol: partial sums stored into every rank's buffer by the row-parallel matvec, added by the next
# matvec's prologue.  Two "ranks" = two exchange buffers on this GPU; their kernels run one after the other in stream
# order (pushers first), so nothing ever waits for a kernel that has not been launched yet. ----

def _tp_linear(L, nw, mode, tp, x=None, h_in=None, h_out=None, norm_w=None, gate_up=None, y=None, K=None):
    pad = (nw.in_features + 31) // 32 * 32
    xtmp = torch.zeros(pad, dtype=torch.bfloat16, device="cuda")
    return L.lib.nwc_linear_fused_opt(L.stream(), L.ptr(nw.data), L.ptr(nw.bases), L.ptr(nw.hdr), L.ptr(nw.lut), L.ptr(nw.low), mode, L.ptr(x), L.ptr(h_in), None,
                                     L.ptr(h_out), L.ptr(norm_w), 1e-6, L.ptr(gate_up), L.ptr(xtmp), None, None, L.ptr(nw.scratch), L.ptr(y), nw.n, nw.block,
                                     nw.in_features, nw.code, tp)


def _io(L, table, rank, world, in_slot, out_slot, H):
    io = L.FusedOptions(ctypes.cast(table, ctypes.c_void_p), rank, world, in_slot, out_slot, H)
    return io, ctypes.byref(io)


@pytest.mark.parametrize("sharing", [0, 2])
@pytest.mark.parametrize("H,Kshard,world,rows", [(1024, 512, 2, 768), (2048, 1536, 2, 768), (8192, 1024, 2, 768), (1024, 512, 4, 768), (8192, 1024, 4, 768),
                                                 (8192, 1024, 8, 768), (2048, 512, 8, 768), (8192, 512, 8, 7168), (4096, 512, 4, 2576)])
def test_push_protocol_local_ranks(H, Kshard, world, rows, sharing):
    """o-projection shards of `world` ranks (all on this GPU, one exchange buffer each) push into every buffer; the consumer
    (a column-parallel matrix with the fused peer prologue) must see h + (the partials added in rank order) and the RMSNorm
    of it, for every rank alike, twice in a row - whether every CTA of the consumer adds up all partials (sharing 0) or the
    CTAs of a cluster share that work (from 2 ranks on)."""
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    g = torch.Generator().manual_seed(H + Kshard)
    o_shards = [NWCWeight(synthetic_matrix(H, Kshard, 10 + r), layout=2) for r in range(world)]   # row-parallel: [H, K / world] each
    consumer = NWCWeight(synthetic_matrix(rows, H, 20), layout=2)                                 # the matrix after the sum
    L.lib.nwc_set_peer_sharing(sharing)
    xs = [torch.randn(Kshard, generator=g).to(torch.bfloat16).cuda() for _ in range(world)]
    h = torch.randn(H, generator=g).to(torch.bfloat16).cuda()
    norm_w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    bufs = _buffers(L, H, world)
    table = (ctypes.c_void_p * world)(*bufs)
    try:
        for round_no in range(2):
            slot = round_no & 1
            parts = []
            for r in range(world):                                        # all pushers first
                keep, io = _io(L, table, r, world, -1, slot, H)
                assert _tp_linear(L, o_shards[r], 0, io, x=xs[r]) == 0
                parts.append(o_shards[r].linear_bf16(xs[r], None))           # the same product through the plain entry point
            total = parts[0].float()
            for part in parts[1:]: total = total + part.float()           # fp32, in rank order
            total = total.to(torch.bfloat16)
            want_h = (h.float() + total.float()).to(torch.bfloat16)
            want_x = torch.zeros(H, dtype=torch.bfloat16, device="cuda")
            assert L.lib.nwc_add_rmsnorm(L.stream(), L.ptr(h), L.ptr(total), L.ptr(torch.zeros_like(h)), L.ptr(norm_w), 1e-6, H, L.ptr(want_x), None) == 0
            want_y = consumer.linear_bf16(want_x, None)
            for r in range(world):                                        # then the consumers: every word is already there
                keep, io = _io(L, table, r, world, slot, -1, H)
                h_out, y = torch.zeros_like(h), torch.zeros(rows, dtype=torch.bfloat16, device="cuda")
                assert _tp_linear(L, consumer, 1, io, h_in=h, h_out=h_out, norm_w=norm_w, y=y) == 0
                torch.cuda.synchronize()
                assert torch.equal(h_out, want_h), (round_no, r)
                assert (y.float() - want_y.float()).abs().max().item() <= 2.0 ** -6 * want_y.float().abs().max().item() + 1e-6
            assert L.lib.nwc_kernel_status(1) == 0
    finally:
        L.lib.nwc_set_peer_sharing(0)
        for buf in bufs: L.lib.nwc_comm_free(ctypes.c_void_p(buf))


@pytest.mark.parametrize("world,sharing", [(2, 0), (4, 0), (4, 2)])
def test_push_consumer_gives_up_when_a_rank_never_pushes(world, sharing):
    """The last rank never pushes: rank 0's consumer waits the (shortened) limit, reports status 3 and poisons its output with
    NaN instead of publishing a sum that misses a partial; the context stays usable.  (sharing 2: the CTAs of a cluster
    share the sum, and all of them learn that a word is missing.)"""
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    H = 1024
    o0 = NWCWeight(synthetic_matrix(H, 512, 1), layout=2)
    consumer = NWCWeight(synthetic_matrix(256, H, 2), layout=2)
    x = torch.ones(512, dtype=torch.bfloat16, device="cuda")
    h = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    bufs = _buffers(L, H, world)
    table = (ctypes.c_void_p * world)(*bufs)
    L.lib.nwc_comm_set_timeout_ms(40)
    L.lib.nwc_set_peer_sharing(sharing)
    try:
        for r in range(world - 1):                                        # everybody but the last rank pushes
            keep, io = _io(L, table, r, world, -1, 0, H)
            assert _tp_linear(L, o0, 0, io, x=x) == 0
        keep2, io2 = _io(L, table, 0, world, 0, -1, H)
        h_out, y = torch.zeros_like(h), torch.zeros(256, dtype=torch.bfloat16, device="cuda")
        assert _tp_linear(L, consumer, 1, io2, h_in=h, h_out=h_out, norm_w=h, y=y) == 0
        torch.cuda.synchronize()
        assert L.lib.nwc_kernel_status(1) == 3
        assert torch.isnan(y.float()).all()
        assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    finally:
        L.lib.nwc_set_peer_sharing(0)
        L.lib.nwc_comm_set_timeout_ms(2000)
        for buf in bufs: L.lib.nwc_comm_free(ctypes.c_void_p(buf))


def test_sharded_argmax_exchanges_one_word_per_rank():
    """Two local ranks with half the vocabulary each.  Rank 0 runs first and cannot hear from rank 1 (its kernel is not
    launched yet): bounded wait, status 3, local best.  Rank 1 then finds rank 0's word and must return the global
    winner with its global index; log / pos / step obey their limits."""
    from nwc_b200 import _lib as L
    V = 4096
    g = torch.Generator().manual_seed(3)
    logits = [torch.randn(V, generator=g).to(torch.bfloat16).cuda() for _ in range(2)]
    logits[0][1234] = 9.0; logits[1][77] = 8.0                          # the winner lives on rank 0
    a, b = _buffers(L, 256, 2)
    table = (ctypes.c_void_p * 2)(a, b)
    L.lib.nwc_comm_set_timeout_ms(40)
    try:
        outs = []
        for r in range(2):
            cur = torch.zeros(1, dtype=torch.int64, device="cuda"); log = torch.full((4,), -1, dtype=torch.int64, device="cuda")
            pos = torch.zeros(1, dtype=torch.int32, device="cuda"); step = torch.zeros(1, dtype=torch.int32, device="cuda")
            assert L.lib.nwc_argmax_tp(L.stream(), L.ptr(logits[r]), V, L.ptr(cur), L.ptr(log), L.ptr(pos), L.ptr(step), 4, 16, table, r, 2) == 0
            torch.cuda.synchronize()
            outs.append((int(cur), int(log[0]), int(pos), int(step), L.lib.nwc_kernel_status(1)))
        assert outs[0] == (1234, 1234, 1, 1, 3)                          # alone: its own best, and it says so
        assert outs[1] == (1234, 1234, 1, 1, 0)                          # global winner (rank 0, index 1234)
        # limits: a full log or a position at the end of the cache stops the increments, nothing is written past them
        cur = torch.zeros(1, dtype=torch.int64, device="cuda"); log = torch.full((4,), -1, dtype=torch.int64, device="cuda")
        pos = torch.full((1,), 16, dtype=torch.int32, device="cuda"); step = torch.full((1,), 2, dtype=torch.int32, device="cuda")
        assert L.lib.nwc_argmax(L.stream(), L.ptr(logits[1]), V, L.ptr(cur), L.ptr(log), L.ptr(pos), L.ptr(step), 4, 16) == 0
        torch.cuda.synchronize()
        assert int(cur) == 77 and int(pos) == 16 and int(step) == 2 and log.tolist() == [-1, -1, -1, -1]
        step.fill_(4); pos.fill_(3)
        assert L.lib.nwc_argmax(L.stream(), L.ptr(logits[1]), V, L.ptr(cur), L.ptr(log), L.ptr(pos), L.ptr(step), 4, 16) == 0
        torch.cuda.synchronize()
        assert int(pos) == 3 and int(step) == 4 and log.tolist() == [-1, -1, -1, -1]
    finally:
        L.lib.nwc_comm_set_timeout_ms(2000)
        L.lib.nwc_comm_free(ctypes.c_void_p(a)); L.lib.nwc_comm_free(ctypes.c_void_p(b))
