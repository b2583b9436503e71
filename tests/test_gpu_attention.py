"""One token of grouped-query attention (nwc_attention_decode): the lane-per-dimension kernel that head sizes 64, 128 and
256 take, against the general kernel and against a plain fp32 PyTorch reference of the same operation (per-head RMSNorm,
rotary embedding with bf16 rounding per step, cache append, softmax over the cached positions, fp32 accumulation)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(qkv, q_norm, k_norm, cos, sin, k_cache, v_cache, pos, n_q, n_kv, hd, eps):
    """fp32 PyTorch restatement; returns (out [n_q * hd] fp32, new key rows [n_kv, hd] bf16)."""
    bf = lambda t: t.to(torch.bfloat16).float()
    q = qkv[: n_q * hd].float().view(n_q, hd); k = qkv[n_q * hd: (n_q + n_kv) * hd].float().view(n_kv, hd)
    v = qkv[(n_q + n_kv) * hd:].float().view(n_kv, hd)
    def norm(x, w): return bf(w.float() * bf(x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)))
    if q_norm is not None: q, k = norm(q, q_norm), norm(k, k_norm)
    c, s = cos[pos].float(), sin[pos].float()
    def rope(x):
        half = hd // 2
        rot = torch.cat([-x[:, half:], x[:, :half]], -1)
        return bf(bf(x * c) + bf(rot * s))
    q, k = rope(q), rope(k)
    out = torch.zeros(n_q, hd)
    rep = n_q // n_kv
    for h in range(n_q):
        g = h // rep
        keys = torch.cat([k_cache[g, :pos].float(), k[g:g + 1]], 0); vals = torch.cat([v_cache[g, :pos].float(), v[g:g + 1]], 0)
        p = torch.softmax((keys @ q[h]) / hd ** 0.5, 0)
        out[h] = p @ vals
    return out.reshape(-1), k.to(torch.bfloat16)


@pytest.mark.parametrize("hd,n_q,n_kv,norm", [(128, 16, 8, True), (128, 8, 1, False), (64, 4, 2, True), (256, 4, 4, False), (96, 4, 2, True)])
@pytest.mark.parametrize("pos,max_len", [(0, 768), (1, 768), (7, 768), (8, 768), (9, 768), (100, 768), (700, 768), (100, 256), (5, 2304), (1000, 2304), (2300, 2304)])
def test_attention_decode_matches_reference_and_the_general_kernel(hd, n_q, n_kv, norm, pos, max_len):
    """max_len decides over how many CTAs a head's cached positions are split (1, 2, 4 or 8); each split count is covered."""
    from nwc_b200 import _lib as L
    g = torch.Generator().manual_seed(hd + pos)
    rnd = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)
    qkv, kc, vc = rnd((n_q + 2 * n_kv) * hd), rnd(n_kv, max_len, hd), rnd(n_kv, max_len, hd)
    ang = torch.rand(max_len, hd, generator=g) * 6.28
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16) if norm else None
    kn = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16) if norm else None
    want, new_k = reference(qkv, qn, kn, cos, sin, kc, vc, pos, n_q, n_kv, hd, 1e-6)
    outs = []
    for plain in (0, 1):
        L.lib.nwc_set_plain_attention(plain)
        try:
            d = lambda t: None if t is None else t.cuda()
            q_d, kc_d, vc_d, cos_d, sin_d, qn_d, kn_d = d(qkv), d(kc), d(vc), d(cos), d(sin), d(qn), d(kn)
            p_d = torch.full((1,), pos, dtype=torch.int32, device="cuda"); st = torch.zeros(1, dtype=torch.int32, device="cuda")
            out = torch.zeros(n_q * hd, dtype=torch.bfloat16, device="cuda")
            err = L.lib.nwc_attention_decode(L.stream(), L.ptr(q_d), L.ptr(qn_d), L.ptr(kn_d), L.ptr(cos_d), L.ptr(sin_d), L.ptr(kc_d), L.ptr(vc_d), L.ptr(p_d), n_q, n_kv, hd,
                                             max_len, 1e-6, L.ptr(out), L.ptr(st))
            assert err == 0 and int(st) == 0
            torch.cuda.synchronize()
        finally:
            L.lib.nwc_set_plain_attention(0)
        got = out.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= 2.0 ** -6 * want.abs().max().item() + 1e-3, (plain, (got - want).abs().max().item())
        assert torch.equal(kc_d[:, pos].cpu(), new_k)                                   # appended key: bit-exact
        assert torch.equal(vc_d[:, pos].cpu(), qkv[(n_q + n_kv) * hd:].view(n_kv, hd))   # appended value: the projection's bits
        assert torch.equal(kc_d[:, :pos].cpu(), kc[:, :pos]) and torch.equal(vc_d[:, pos + 1:].cpu(), vc[:, pos + 1:])
        outs.append(got)
    assert (outs[0] - outs[1]).abs().max().item() <= 2.0 ** -7 * want.abs().max().item() + 1e-3   # the two kernels agree to bf16 rounding


def test_position_outside_the_cache_is_refused():
    from nwc_b200 import _lib as L
    hd, n_q, n_kv, max_len = 128, 4, 2, 16
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda")
    qkv, kc, vc, cos, sin, out = z((n_q + 2 * n_kv) * hd), z(n_kv, max_len, hd), z(n_kv, max_len, hd), z(max_len, hd), z(max_len, hd), z(n_q * hd) + 5
    for pos in (max_len, -1):
        p = torch.full((1,), pos, dtype=torch.int32, device="cuda"); st = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert L.lib.nwc_attention_decode(L.stream(), L.ptr(qkv), None, None, L.ptr(cos), L.ptr(sin), L.ptr(kc), L.ptr(vc), L.ptr(p), n_q, n_kv, hd, max_len, 1e-6, L.ptr(out), L.ptr(st)) == 0
        torch.cuda.synchronize()
        assert int(st) == 1 and (out == 5).all()
