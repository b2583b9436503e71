"""Shared helpers of the test-suite (CPU side)."""
import glob
import os

import numpy as np

import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_cases(kind=None):
    """[(name, elem, layout, M, K, path)] of the committed fixtures."""
    out = []
    for path in sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))):
        name = os.path.basename(path)[:-4]
        el, lay, shape = name.split("_")
        if kind and el != kind: continue
        M, K = (int(v) for v in shape.split("x"))
        out.append((name, 0 if el == "bf16" else 1, int(lay[1]), M, K, path))
    return out


def packed_from_fixture(path, elem, layout, M, K) -> O.Packed:
    z = np.load(path)
    code = O.code_of(elem, layout)
    nb, n_low, n_scratch, K16 = O.layout(M, K, code)
    low = np.zeros(n_low + O.RAW_SLACK, np.uint8); low[:n_low] = z["low"]
    p = O.Packed(M, K, code, z["data"].copy(), z["bases"].copy(), z["hdr"].copy(), z["lut"].copy(), low,
                 np.zeros(O.SYM_TABLE_LEN, np.uint16), int(z["data"].size) - 64, K16, n_low, n_scratch)
    if elem: p.scale = z["scale"].copy()
    return p


def same_compressed(a: O.Packed, b: O.Packed) -> bool:
    return (a.payloads() == b.payloads() and np.array_equal(a.hdr, b.hdr) and np.array_equal(a.bases, b.bases)
            and np.array_equal(a.lut, b.lut) and np.array_equal(a.low[:a.n_low], b.low[:b.n_low]))


def rel_l2(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
