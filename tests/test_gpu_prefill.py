"""Prefill GEMM with tile-wise decoding (tcgen05 / tensor memory) against dequantise + fp32 matmul."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,T", [(128, 64, 16), (128, 512, 32), (300, 1000, 33), (1024, 1024, 256), (130, 1536, 300), (2048, 2560, 512), (16, 40, 1), (256, 1024, 1100), (384, 200, 257)])
@pytest.mark.parametrize("halves", [1, 2])
def test_prefill_matches_dequant_matmul(M, K, T, halves):
    """halves: a CTA multiplies its 128 rows with one or two halves of 256 tokens (the launcher's own choice depends on how
    many CTAs the shape gives; both kernels must agree with the reference product on every shape)."""
    from gpu_helpers import make_case, to_weight, bf16_tensor
    from nwc_b200 import _lib as L
    L.lib.nwc_set_prefill_halves(halves)
    try:
        _prefill_case(M, K, T, L)
    finally:
        L.lib.nwc_set_prefill_halves(0)


def _prefill_case(M, K, T, L):
    from gpu_helpers import make_case, to_weight, bf16_tensor
    values, _ = O.synth_weights(M, K, M + K + T)
    values = values.copy(); values.reshape(-1)[:: max(1, M * K // 50)] = 0x4F00       # 2^31: a rare exponent -> exception entries
    p = O.encode(values, O.code_of(0, 2))
    assert M * K < 4096 or p.hdr.astype(int).sum() > 0
    nw = to_weight(p)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    bias = (torch.randn(M, generator=g) * 0.1).to(torch.bfloat16).cuda()
    w = bf16_tensor(values).cuda().float()
    finite = True
    y = nw.linear_prefill(x, bias)
    assert y is not None and y.shape == (T, M)
    assert L.lib.nwc_kernel_status(1) == 0
    ref = (x.double() @ w.double().t() + bias.double()).float()
    # identity rows of X read the decoded matrix back through the GEMM: bit-exact incl. exception entries
    eye = torch.zeros(min(T, K), K, dtype=torch.bfloat16, device="cuda"); eye[torch.arange(min(T, K)), torch.arange(min(T, K))] = 1
    back = nw.linear_prefill(eye, None)
    assert torch.equal(back.t().contiguous().view(torch.int16).cpu(), torch.from_numpy(values[:, : min(T, K)].view(np.int16).copy()))
    if finite:
        err = ((y.float() - ref).norm() / ref.norm()).item()
        assert err <= (2e-3 if M * T >= 1024 else 2.0 ** -8), err      # a handful of outputs: one bf16 rounding (half an ulp, up to 2^-8) can dominate the norm
        assert (y.float() - ref).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item() + 1e-3
    # the same through the module: tokens batched -> prefill path, one token -> fused matvec; both agree with each other
    one = nw.linear_bf16(x[0], bias).float()
    assert ((one - y[0].float()).norm() / one.norm()).item() <= 4e-3 or not finite


def test_prefill_declines_uncovered_layouts():
    from gpu_helpers import make_case, to_weight
    p, _, _ = make_case(64, 512, 0, 0, seed=1)
    assert to_weight(p).linear_prefill(torch.zeros(4, 512, dtype=torch.bfloat16, device="cuda")) is None
