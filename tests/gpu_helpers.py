"""Helpers of the GPU tests: oracle-packed matrices as NWCWeight objects, canary-padded buffers."""
import numpy as np
import torch

import oracle as O
from nwc_b200 import NWCWeight


def to_weight(p: O.Packed) -> NWCWeight:
    """An oracle-encoded matrix loaded through the checkpoint path (no GPU encoder involved)."""
    t = lambda a, dt: torch.from_numpy(a.view(dt).copy())
    return NWCWeight.from_tensors(p.M, p.K, 4096, t(p.data, np.uint8), t(p.bases, np.int32), t(p.hdr, np.uint8), t(p.lut, np.int32),
                                  t(p.low, np.uint8), "cuda", elem="fp8" if p.elem else "bf16",
                                  scale=None if p.scale is None else torch.from_numpy(p.scale.copy()), layout=p.layout)


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy bit patterns"""
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def bf16_tensor(b: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16)


def make_case(M, K, elem, layout, seed=0, escapes=True):
    """(Packed, original values as bf16 bits [M, K], x bf16 bits [K])"""
    w, x = O.synth_weights(M, K, seed)
    w = w.copy()
    if escapes and elem == 0: w.reshape(-1)[:: max(1, M * K // 50)] = 0x7149       # ~1e30: rare exponents -> escapes / exceptions
    if elem == 0:
        return O.encode(w, O.code_of(0, layout)), w, x
    wf = O.bf16_to_f32(w).copy(); wf.reshape(-1)[::97] *= 40                      # outliers -> many subnormals after scaling
    q, scale = O.quantize_fp8(O.f32_to_bf16(wf).reshape(M, K))
    p = O.encode(q, O.code_of(1, layout)); p.scale = scale
    return p, O.fp8_to_bf16(q), x
