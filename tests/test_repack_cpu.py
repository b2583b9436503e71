"""Tensor-parallel shards cut out of a compressed matrix by re-packing its blocks (nwc_b200/repack.py), checked on the
CPU: the oracle's decoder applied to a shard must return exactly the rows / columns of the original matrix, for every
layout and element type, with ragged edges, several row ranges (a fused q/k/v projection) and escapes / exceptions."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_repack():
    # by path: the package import needs the CUDA library, this module is plain torch
    spec = importlib.util.spec_from_file_location("nwc_repack", os.path.join(ROOT, "nwc_b200", "repack.py"))
    import sys
    m = importlib.util.module_from_spec(spec); sys.modules["nwc_repack"] = m; spec.loader.exec_module(m)
    return m


def make(M, K, elem, layout, seed=0):
    w, _ = O.synth_weights(M, K, seed)
    w = w.copy()
    if elem == 0:
        w.reshape(-1)[:: max(1, M * K // 60)] = 0x7149                    # rare exponents: escapes (layouts 0, 1) / exceptions (layout 2)
        return O.encode(w, O.code_of(0, layout)), w
    q, scale = O.quantize_fp8(w)
    p = O.encode(q, O.code_of(1, layout)); p.scale = scale
    return p, O.fp8_to_bf16(q)


def to_compressed(R, p):
    t = lambda a, dt: torch.from_numpy(a.view(dt).copy())
    return R.Compressed(p.M, p.K, p.layout, "fp8" if p.elem else "bf16", t(p.data, np.uint8), t(p.bases, np.int32), t(p.hdr, np.uint8), t(p.lut, np.int32),
                        t(p.low, np.uint8), None if p.scale is None else torch.from_numpy(p.scale.copy()))


def to_packed(c, code):
    nb, n_low, n_scratch, K16 = O.layout(c.M, c.K, code)
    assert c.bases.numel() == nb and c.hdr.numel() == nb * 32 and c.low.numel() == n_low + 512
    return O.Packed(c.M, c.K, code, c.data.numpy().copy(), c.bases.numpy().view(np.uint32).copy(), c.hdr.numpy().copy(), c.lut.numpy().view(np.uint32).copy(),
                    c.low.numpy().copy(), None, c.data.numel() - 64, K16, n_low, n_scratch, None if c.scale is None else c.scale.numpy().copy())


COMBOS = [(e, l) for e in (0, 1) for l in (0, 1, 2)]


@pytest.mark.parametrize("elem,layout", COMBOS)
@pytest.mark.parametrize("M,K,ranges", [(96, 1536, [(0, 32)]), (96, 1536, [(32, 96)]), (100, 1000, [(16, 48), (80, 100)]), (160, 520, [(0, 16), (64, 96), (128, 160)]),
                                        (48, 40, [(16, 48)])])
def test_row_shards_decode_to_the_rows(elem, layout, M, K, ranges):
    R = load_repack()
    p, values = make(M, K, elem, layout, seed=M + K)
    shard = R.take_rows(to_compressed(R, p), ranges)
    want = np.concatenate([values[a:b] for a, b in ranges])
    got = O.decode(to_packed(shard, p.code))
    assert np.array_equal(got[:, :K], want)
    if elem: assert np.array_equal(shard.scale.numpy(), np.concatenate([p.scale[a:b] for a, b in ranges]))
    # every block payload of the shard is a block payload of the full matrix, in the order of the ranges
    g = shard.geometry
    full_blocks = [b for a, e in ranges for b in range(a // g.rows * g.CB, -(-e // g.rows) * g.CB)]
    unit = g.unit
    per = p.hdr.reshape(-1, 32).astype(np.int64).sum(1) * unit
    for i, b in enumerate(full_blocks):
        n = int(per[b]); s0, s1 = int(p.bases[b]), int(shard.bases[i]) & 0xFFFFFFFF
        assert bytes(p.data[s0:s0 + n]) == bytes(shard.data.numpy()[s1:s1 + n])


@pytest.mark.parametrize("elem,layout", COMBOS)
@pytest.mark.parametrize("M,K,c0,c1", [(40, 1536, 0, 512), (40, 1536, 512, 1536), (33, 2000, 1024, 2000), (33, 2000, 0, 1024), (16, 4097, 3584, 4097), (24, 1100, 512, 1100)])
def test_column_shards_decode_to_the_columns(elem, layout, M, K, c0, c1):
    R = load_repack()
    p, values = make(M, K, elem, layout, seed=M * 3 + K)
    shard = R.take_cols(to_compressed(R, p), c0, c1)
    got = O.decode(to_packed(shard, p.code))
    assert np.array_equal(got[:, :c1 - c0], values[:, c0:c1])


def test_shards_of_all_ranks_tile_the_matrix_and_bad_cuts_are_refused():
    R = load_repack()
    p, values = make(128, 2048, 0, 2)
    c = to_compressed(R, p)
    x = np.random.default_rng(0).standard_normal(2048).astype(np.float32)
    full = O.matvec_f32(p, x)
    # column-parallel over 4 ranks: the outputs concatenate; row-parallel: the outputs add up
    rows = np.concatenate([O.matvec_f32(to_packed(R.take_rows(c, [(32 * r, 32 * r + 32)]), p.code), x) for r in range(4)])
    assert np.allclose(rows, full, rtol=1e-6, atol=1e-6)
    cols = sum(O.matvec_f32(to_packed(R.take_cols(c, 512 * r, 512 * r + 512), p.code), x[512 * r:512 * r + 512]) for r in range(4))
    assert np.allclose(cols, full, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError): R.take_rows(c, [(8, 32)])              # layout 2 blocks are 16 rows high
    with pytest.raises(ValueError): R.take_rows(c, [(0, 24), (32, 64)])    # only the last range may end off a block boundary (with the matrix)
    with pytest.raises(ValueError): R.take_cols(c, 256, 1024)
    with pytest.raises(ValueError): R.take_cols(c, 0, 700)
    assert R.rows_divisible(2, 1024, 128) and not R.rows_divisible(2, 24) and R.rows_divisible(0, 24)
