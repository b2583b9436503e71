"""Regenerates the golden fixtures in this directory from the REFERENCE implementation.

Run where the reference checkout is mounted (its path: the NWC_REFERENCE_ROOT variable) and its kernel library is compiled from
source by `make -C oracle ref`:

    python tests/golden/make_golden.py

For every case it stores, in one compressed .npz: the input weights, the five format tensors written by the
reference's host encoder (called through the reference's own Python bridge, nwc/nwc_torch.py), and - for bf16 - the
matrix returned by the reference's pure-Python format decoder (tests/test_format_cpu.py: decode / decode2).
The reference has no CPU decoder for fp8, so fp8 cases store encoder outputs only; their decode target is the input.
known_answers.json holds SHA-256 prefixes of the encoder outputs for the 4096 x 4096 benchmark matrix, which is too
large to commit.
"""
import hashlib, importlib.util, json, os, sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import oracle                                                # noqa: E402
REF = oracle.reference_root()
if not REF: raise SystemExit("reference checkout not found: set NWC_REFERENCE_ROOT")
os.environ["NWC_DLL"] = os.path.join(ROOT, "oracle", "_ref", "nwc_ops.so")
sys.path.insert(0, REF)
from nwc.nwc_torch import NWCWeight, quantize_fp8          # the reference's bridge   # noqa: E402

spec = importlib.util.spec_from_file_location("ref_format_test", os.path.join(REF, "tests", "test_format_cpu.py"))
ref_test = importlib.util.module_from_spec(spec); spec.loader.exec_module(ref_test)
from oracle import synth_weights                             # noqa: E402


def sha(b): return hashlib.sha256(b).hexdigest()[:16]


def tensors(c):
    n_low = c.low.numel() - 512
    return dict(data=c.data.numpy(), bases=c.bases.numpy().view(np.uint32), hdr=c.hdr.numpy(),
                lut=c.lut.numpy().view(np.uint32), low=c.low.numpy()[:n_low])


def weights(M, K, seed, escapes):
    w_bits, x_bits = synth_weights(M, K, seed)
    w = torch.from_numpy(w_bits.view(np.int16).copy()).view(torch.bfloat16)
    if escapes: w.view(-1)[:: max(1, M * K // 50)] = torch.tensor(1e30, dtype=torch.bfloat16)   # rare exponents
    return w, x_bits


CASES = [(8, 512, 0), (13, 40, 1), (3, 4097, 2), (17, 520, 3), (100, 1000, 4)]
for M, K, seed in CASES:
    w, x_bits = weights(M, K, seed, escapes=True)
    for layout in (0, 1, 2):
        c = NWCWeight(w, device="cpu", layout=layout)
        back = ref_test.decode2(c) if layout == 2 else ref_test.decode(c)
        assert torch.equal(back, w)
        np.savez_compressed(os.path.join(HERE, f"bf16_L{layout}_{M}x{K}.npz"), w=w.view(torch.int16).numpy().view(np.uint16),
                            x=x_bits, decoded=back.view(torch.int16).numpy().view(np.uint16), **tensors(c))
    if (M, K) in ((13, 40), (17, 520), (100, 1000)):
        wq = w.clone(); wq.view(-1)[::97] *= 40                 # outliers -> many fp8 subnormals
        wq[wq.abs() > 1e20] = 0.5
        q, scale = quantize_fp8(wq)
        for layout in (0, 1, 2):
            c = NWCWeight(q, device="cpu", elem="fp8", scale=scale, layout=layout)
            np.savez_compressed(os.path.join(HERE, f"fp8_L{layout}_{M}x{K}.npz"), q=q.view(torch.uint8).numpy(), scale=scale.numpy(),
                                x=x_bits, **tensors(c))

known = {}
w_bits, x_bits = synth_weights(4096, 4096, 0)
w = torch.from_numpy(w_bits.view(np.int16).copy()).view(torch.bfloat16)
known["w"] = sha(w_bits.tobytes()); known["x"] = sha(x_bits.tobytes())
q, scale = quantize_fp8(w)
known["q"] = sha(q.view(torch.uint8).numpy().tobytes()); known["scale"] = sha(scale.numpy().tobytes())
for elem, src, kw in (("bf16", w, {}), ("fp8", q, {"scale": scale})):
    for layout in (0, 1, 2):
        c = NWCWeight(src, device="cpu", elem=elem, layout=layout, **kw)
        t = tensors(c)
        unit = 4 if layout != 2 else (2 if elem == "fp8" else 3)
        per_block = t["hdr"].reshape(-1, 32).astype(np.int64).sum(1) * unit
        raw = t["data"].tobytes()
        payload = b"".join(raw[int(b): int(b) + int(n)] for b, n in zip(t["bases"], per_block))
        known[f"{elem}_L{layout}"] = {"payload_bytes": len(payload), "payload": sha(payload), "hdr": sha(t["hdr"].tobytes()),
                                     "bases": sha(t["bases"].tobytes()), "lut": sha(t["lut"].tobytes()), "low": sha(t["low"].tobytes()),
                                     "bytes": int(c.bytes)}
with open(os.path.join(HERE, "known_answers.json"), "w") as f: json.dump({"case": "4096x4096 seed 0", "torch": torch.__version__, **known}, f, indent=1)
print("golden fixtures written to", HERE)
