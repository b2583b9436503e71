"""The CPU oracle against the reference: committed golden vectors, known-answer hashes, and (when the reference's
library was compiled into oracle/_ref) the reference host encoder itself on further shapes and error cases."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle as O
from helpers import GOLDEN, golden_cases, packed_from_fixture, same_compressed


def sha(b): return hashlib.sha256(b).hexdigest()[:16]


@pytest.mark.parametrize("name,elem,layout,M,K,path", golden_cases(), ids=[c[0] for c in golden_cases()])
def test_decoder_matches_reference_decoder(name, elem, layout, M, K, path):
    z = np.load(path)
    p = packed_from_fixture(path, elem, layout, M, K)
    got = O.decode(p)
    want = z["decoded"] if elem == 0 else O.fp8_to_bf16(z["q"])      # bf16: reference Python decoder; fp8: lossless input
    assert np.array_equal(got[:, :K], want)
    assert not got[:, K:].any()


@pytest.mark.parametrize("name,elem,layout,M,K,path", golden_cases(), ids=[c[0] for c in golden_cases()])
def test_encoder_matches_reference_encoder(name, elem, layout, M, K, path):
    z = np.load(path)
    ref = packed_from_fixture(path, elem, layout, M, K)
    mine = O.encode(z["w"] if elem == 0 else z["q"], O.code_of(elem, layout))
    assert mine.data_len == ref.data_len
    assert same_compressed(mine, ref)


def test_known_answers_benchmark_matrix():
    """4096 x 4096 seeded matrix: hashes of what the reference encoder produced for it."""
    with open(os.path.join(GOLDEN, "known_answers.json")) as f: known = json.load(f)
    w, x = O.synth_weights(4096, 4096, 0)
    if sha(w.tobytes()) != known["w"]: pytest.skip("torch RNG differs from the one the hashes were made with")
    assert sha(x.tobytes()) == known["x"]
    q, scale = O.quantize_fp8(w)
    assert sha(q.tobytes()) == known["q"] and sha(scale.tobytes()) == known["scale"]
    for el, src in (("bf16", w), ("fp8", q)):
        for layout in (0, 1, 2):
            p = O.encode(src, O.code_of(0 if el == "bf16" else 1, layout))
            k = known[f"{el}_L{layout}"]
            if el == "fp8": p.scale = scale
            pay = p.payloads()
            assert (len(pay), sha(pay)) == (k["payload_bytes"], k["payload"])
            assert sha(p.hdr.tobytes()) == k["hdr"] and sha(p.bases.tobytes()) == k["bases"]
            assert sha(p.lut.tobytes()) == k["lut"] and sha(p.low[:p.n_low].tobytes()) == k["low"]
            assert p.bytes == k["bytes"]
            want = src if el == "bf16" else O.fp8_to_bf16(src)
            assert np.array_equal(O.decode(p, threads=8), want)


def test_matvec_and_finalize():
    w, x = O.synth_weights(257, 1100, 3)
    p = O.encode(w, O.code_of(0, 1))
    xf = O.bf16_to_f32(x)
    y = O.matvec_f32(p, xf)
    ref = O.bf16_to_f32(w).astype(np.float64) @ xf.astype(np.float64)
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    bias = O.f32_to_bf16(np.linspace(-1, 1, 257).astype(np.float32))
    yb = O.finalize(y, bias)
    want = O.f32_to_bf16(y + O.bf16_to_f32(bias))
    assert np.array_equal(yb, want)
    ids = np.array([0, 256, 5, 256, -1, 9999])
    g = O.gather(p, ids)
    assert np.array_equal(g[0, :1100], w[0]) and np.array_equal(g[1, :1100], w[256]) and not g[4].any() and not g[5].any()


needs_ref = pytest.mark.skipif(not O.ref_available(), reason="reference library not compiled (oracle/_ref)")


@needs_ref
@pytest.mark.parametrize("M,K", [(1, 1), (8, 16), (16, 512), (33, 1040), (5, 2049), (200, 513), (1001, 1000), (64, 6144)])
def test_encoder_vs_compiled_reference(M, K):
    w, _ = O.synth_weights(M, K, M + K)
    w = w.copy(); w.reshape(-1)[:: max(1, M * K // 37)] = 0x7149
    q, _ = O.quantize_fp8(np.where((w & 0x7F80) == 0x7100, 0x3C00, w).astype(np.uint16))
    for elem, src in ((0, w), (1, q)):
        for layout in (0, 1, 2):
            code = O.code_of(elem, layout)
            assert O.layout(M, K, code) == O.ref_layout(M, K, code)[1]
            a, b = O.encode(src, code), O.ref_encode(src, code)
            assert a.data_len == b.data_len and same_compressed(a, b) and np.array_equal(a.psym, b.psym)
            want = src if elem == 0 else O.fp8_to_bf16(src)
            assert np.array_equal(O.decode(a)[:, :K], want)


@needs_ref
def test_error_codes_match_reference():
    nan = np.full((8, 512), 0x7F, np.uint8)
    for layout in (0, 1, 2):
        for enc in (O.encode, O.ref_encode):
            with pytest.raises(O.EncodeError) as e: enc(nan, O.code_of(1, layout))
            assert e.value.rc == -2
    # layout 2: one block whose weights all carry rare exponents (the 7 frequent ones live in the other block):
    # every lane of it holds 256 exceptions, one more than a header byte can count
    rng = np.random.default_rng(0)
    w = np.empty((16, 1024), np.uint16)
    w[:, :512] = rng.integers(10, 110, size=(16, 512)).astype(np.uint16) << 8
    w[:, 512:] = rng.integers(1, 8, size=(16, 512)).astype(np.uint16) << 8
    for enc in (O.encode, O.ref_encode):
        with pytest.raises(O.EncodeError) as e: enc(w, O.code_of(0, 2))
        assert e.value.rc == -3
    # the prefix layouts code the same matrix (escapes), and both encoders agree on it
    for layout in (0, 1):
        a, b = O.encode(w, O.code_of(0, layout)), O.ref_encode(w, O.code_of(0, layout))
        assert same_compressed(a, b) and np.array_equal(O.decode(a), w)
    # too small a buffer -> -1 from both
    import ctypes
    for fn in (O.lib().nwo_encode, O.ref_lib().nwc_encode):
        freq = np.zeros(1024, np.uint16); psym = np.zeros(1024, np.uint16); bases = np.zeros(2, np.uint32)
        hdr = np.zeros(64, np.uint8); data = np.zeros(256, np.uint8); low = np.zeros(16 * 1024 + 512, np.uint8)
        P = lambda a: ctypes.c_void_p(a.ctypes.data)
        assert fn(P(w), w.size, 1024, 0, P(freq), P(psym), P(bases), P(hdr), P(data), 256, P(low)) == -1
        assert fn(P(w), w.size, 1000, 0, P(freq), P(psym), P(bases), P(hdr), P(data), 256, P(low)) == -1     # n % K != 0
    assert O.ref_layout(0, 5, 0)[0] == -1
    with pytest.raises(ValueError): O.layout(0, 5, 0)
