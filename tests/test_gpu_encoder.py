"""The GPU encoder against the oracle (= the reference's host encoder): byte-identical streams, headers, offsets,
tables and planes, and the reference's error codes."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from helpers import golden_cases, packed_from_fixture, same_compressed

pytestmark = pytest.mark.gpu


def packed_from_weight(nw, M, K):
    c = lambda t, dt: t.detach().cpu().numpy().view(dt).copy()
    code = nw.code
    nb, n_low, n_scratch, K16 = O.layout(M, K, code)
    data = c(nw.data, np.uint8)
    return O.Packed(M, K, code, data, c(nw.bases, np.uint32), c(nw.hdr, np.uint8), c(nw.lut, np.uint32), c(nw.low, np.uint8),
                    np.zeros(1024, np.uint16), data.size - 64, K16, n_low, n_scratch)


def encode_gpu(src_bits, elem, layout, scale=None):
    from nwc_b200 import NWCWeight
    if elem:
        t = torch.from_numpy(src_bits.copy()).view(torch.float8_e4m3fn)
        return NWCWeight(t, elem="fp8", scale=torch.ones(src_bits.shape[0]) if scale is None else torch.from_numpy(scale), layout=layout)
    return NWCWeight(torch.from_numpy(src_bits.view(np.int16).copy()).view(torch.bfloat16), layout=layout)


@pytest.mark.parametrize("name,elem,layout,M,K,path", golden_cases(), ids=[c[0] for c in golden_cases()])
def test_gpu_encoder_reproduces_reference_streams(name, elem, layout, M, K, path):
    z = np.load(path)
    ref = packed_from_fixture(path, elem, layout, M, K)
    nw = encode_gpu(z["w"] if elem == 0 else z["q"], elem, layout)
    mine = packed_from_weight(nw, M, K)
    assert mine.data_len == ref.data_len and same_compressed(mine, ref)
    assert nw.bytes == ref.data_len + 4 * ref.nb + 32 * ref.nb + 16384 + ref.n_low + (4 * M if elem else 0)


@pytest.mark.parametrize("M,K", [(1, 1), (16, 512), (33, 1040), (5, 2049), (200, 513), (1001, 1000), (4096, 4096), (2048, 6144)])
def test_gpu_encoder_matches_oracle(M, K):
    w, _ = O.synth_weights(M, K, 11 * M + K)
    w = w.copy(); w.reshape(-1)[:: max(1, M * K // 41)] = 0x7149
    q, _ = O.quantize_fp8(np.where((w & 0x7F80) == 0x7100, 0x3C00, w).astype(np.uint16))
    for elem, src in ((0, w), (1, q)):
        for layout in (0, 1, 2):
            ref = O.encode(src, O.code_of(elem, layout))
            mine = packed_from_weight(encode_gpu(src, elem, layout), M, K)
            assert mine.data_len == ref.data_len and same_compressed(mine, ref), (elem, layout)


def test_gpu_encoder_error_codes_and_host_pointer_entry():
    from nwc_b200 import NWCWeight, _lib as L
    nan = torch.full((8, 512), float("nan")).to(torch.float8_e4m3fn)
    for layout in (0, 1, 2):
        with pytest.raises(ValueError, match="NaN"): NWCWeight(nan, elem="fp8", scale=torch.ones(8), layout=layout)
    rng = np.random.default_rng(0)
    w = np.empty((16, 1024), np.uint16)
    w[:, :512] = rng.integers(10, 110, size=(16, 512)).astype(np.uint16) << 8
    w[:, 512:] = rng.integers(1, 8, size=(16, 512)).astype(np.uint16) << 8
    with pytest.raises(ValueError, match="255 exceptions"): encode_gpu(w, 0, 2)
    for layout in (0, 1):
        assert same_compressed(packed_from_weight(encode_gpu(w, 0, layout), 16, 1024), O.encode(w, O.code_of(0, layout)))
    # the reference's host-pointer nwc_encode contract, including "buffer too small -> -1"
    P = lambda a: ctypes.c_void_p(a.ctypes.data)
    w2, _ = O.synth_weights(100, 1000, 4)
    for code in (0, 16, 32, 1 | 16):
        src = w2 if not (code & 15) else O.quantize_fp8(w2)[0]
        ref = O.encode(src, code)
        nb, n_low, _, _ = O.layout(100, 1000, code)
        freq = np.ones(1024, np.uint16); psym = np.zeros(1024, np.uint16); bases = np.zeros(nb, np.uint32); hdr = np.zeros(nb * 32, np.uint8)
        cap = 3 * src.size + nb * 64 + 4096
        data = np.zeros(cap, np.uint8); low = np.zeros(n_low + 512, np.uint8)
        src = np.ascontiguousarray(src)
        dl = L.lib.nwc_encode(P(src), src.size, 1000, code, P(freq), P(psym), P(bases), P(hdr), P(data), cap, P(low))
        assert dl == ref.data_len and not freq.any() and np.array_equal(psym, ref.psym)
        lut = np.zeros(4096, np.uint32); L.lib.nwc_build_tab(P(freq), P(psym), code, P(lut))
        mine = O.Packed(100, 1000, code, data[: dl + 64].copy(), bases, hdr, lut, low, psym, int(dl), ref.K16, n_low, 0)
        assert same_compressed(mine, ref)
        assert L.lib.nwc_encode(P(src), src.size, 1000, code, P(freq), P(psym), P(bases), P(hdr), P(data), 128, P(low)) == -1
    assert L.lib.nwc_encode(P(src), src.size, 999, 0, P(freq), P(psym), P(bases), P(hdr), P(data), cap, P(low)) == -1
