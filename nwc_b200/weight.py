"""NWCWeight: one [out, in] matrix kept entropy-coded in HBM, plus the calls that use it without decompressing it
to memory.  Python-side mirror of the reference's compressed-tensor object (reference: nwc/nwc_torch.py:126-269): same
constructor, attributes and methods, so checkpoint code and modules written against the reference work on it.
"""
import os

import torch
import torch.nn.functional as F

from . import _lib as L

ELEM_BF16, ELEM_FP8 = 0, 1
ELEMS = {"bf16": ELEM_BF16, "fp8": ELEM_FP8}
LAYOUTS = (0, 1, 2)
FP8_MAX = 448.0
# default layout per element type; NWC_LAYOUT=0|1|2 overrides (same switch as the reference)
LAYOUT_DEFAULT = {ELEM_BF16: 0, ELEM_FP8: 0}
if "NWC_LAYOUT" in os.environ:
    LAYOUT_DEFAULT = {k: int(os.environ["NWC_LAYOUT"]) for k in LAYOUT_DEFAULT}


def quantize_fp8(w: torch.Tensor):
    """bf16 / float [out, in] -> (float8_e4m3fn tensor, fp32 scale[out]): symmetric absmax scaling per output channel
    (reference: nwc/nwc_torch.py:88-94)."""
    wf = w.detach().float()
    scale = wf.abs().amax(dim=1).clamp_min(1e-12) / FP8_MAX
    q = (wf / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def fits(out_features, in_features):
    """Every non-empty shape is supported: blocks are padded to 8 or 16 rows x 512 columns."""
    return in_features >= 1 and out_features >= 1


def choose_block(n):
    return L.FIXED_BLOCK


def _layout_query(out_f, in_f, code):
    lay = torch.empty(4, dtype=torch.int64)
    if L.lib.nwc_layout(out_f, in_f, code, L.ptr(lay)): raise RuntimeError("nwc_layout: bad shape")
    return lay.tolist()          # blocks, raw-plane bytes, scratch floats, K16


class NWCWeight:
    """Compressed [out, in] matrix on the GPU.  elem "bf16": lossless.  elem "fp8": weight-only fp8 e4m3 with an fp32
    scale per output channel (from a bf16 matrix through quantize_fp8, or a float8 tensor plus `scale`), the fp8 bytes
    stored lossless.  The encoder runs on the GPU; `w` may live on either side."""

    def __init__(self, w: torch.Tensor, device="cuda", block=None, elem="bf16", scale=None, layout=None):
        L.require_cuda()
        if w.dim() != 2: raise ValueError("a 2-d weight matrix is expected")
        device = torch.device(device)
        if device.type != "cuda": raise RuntimeError("nwc_b200 encodes and decodes on CUDA devices only")
        out_f, in_f = w.shape
        if not fits(out_f, in_f): raise ValueError(f"shape {tuple(w.shape)} not supported")
        self.elem = ELEMS[elem]
        self.layout = LAYOUT_DEFAULT[self.elem] if layout is None else int(layout)
        if self.layout not in LAYOUTS: raise ValueError(f"unknown layout {self.layout}")
        with torch.cuda.device(device):
            if self.elem == ELEM_FP8:
                if w.dtype == torch.float8_e4m3fn:
                    if scale is None: raise ValueError("fp8 weights need their per-row scale")
                    q = w
                else:
                    q, scale = quantize_fp8(w.to(device))
                src = q.detach().to(device).contiguous().view(torch.uint8)
                self.scale = scale.detach().float().contiguous().to(device)
            else:
                if w.dtype != torch.bfloat16: raise ValueError("bf16 weights expected (elem='fp8' for fp8 weights)")
                src = w.detach().to(device).contiguous().view(torch.int16)
                self.scale = None
            n = out_f * in_f
            nb, n_low, n_scratch, self.K16 = _layout_query(out_f, in_f, self.code)
            psym = torch.zeros(L.NPAIR, dtype=torch.int16)
            bases = torch.empty(nb, dtype=torch.int32, device=device)
            hdr = torch.empty(nb * L.HDR_BLOCK, dtype=torch.uint8, device=device)
            low = torch.zeros(n_low + L.RAW_SLACK, dtype=torch.uint8, device=device)
            dl = -1
            for cap in (n + n // 2 + nb * 64 + 4096, 3 * n + nb * 64 + 4096):     # ~12 bits per weight nearly always suffice
                data = torch.empty(cap, dtype=torch.uint8, device=device)
                dl = L.lib.nwc_encode_device(L.stream(), L.ptr(src), n, in_f, self.code, L.ptr(psym), L.ptr(bases), L.ptr(hdr), L.ptr(data), cap, L.ptr(low))
                if dl >= 0 or dl in (-2, -3): break
            if dl == -2: raise ValueError("fp8 weights contain NaN")
            if dl == -3: raise ValueError("layout 2 cannot code this matrix (a lane stream has more than 255 exceptions); use layout 0 or 1")
            if dl < 0: raise RuntimeError(f"nwc_encode failed ({dl})")
            lut = torch.empty(L.TAB_WORDS, dtype=torch.int32)
            L.lib.nwc_build_tab(None, L.ptr(psym), self.code, L.ptr(lut))
            self.out_features, self.in_features, self.n, self.block = out_f, in_f, n, block or L.FIXED_BLOCK
            self.data = torch.zeros(dl + 64, dtype=torch.uint8, device=device)
            self.data[: min(dl, cap)].copy_(data[: min(dl, cap)])
            del data
            self.bases, self.hdr, self.low, self.lut = bases, hdr, low, lut.to(device)
            self._finish(dl, n_low, n_scratch, device)

    @property
    def code(self):
        """The library's elem parameter: element type in bits 0..3, layout in bits 4..7."""
        return self.elem | (self.layout << 4)

    def _finish(self, dl, n_low, n_scratch, device):
        n = self.n
        self.bytes = dl + self.bases.numel() * 4 + self.hdr.numel() + self.lut.numel() * 4 + n_low + (self.scale.numel() * 4 if self.scale is not None else 0)
        self.bytes_bf16 = 2 * n
        self.bytes_native = n + self.out_features * 4 if self.elem == ELEM_FP8 else 2 * n
        self.scratch = torch.empty(n_scratch, dtype=torch.float32, device=device)

    @classmethod
    def from_tensors(cls, out_f, in_f, block, data, bases, hdr, lut, low, device="cuda", elem="bf16", scale=None, layout=0):
        """Compressed matrix from stored tensors (checkpoints), without the original weights."""
        L.require_cuda()
        self = cls.__new__(cls)
        self.elem = ELEMS[elem]; self.layout = int(layout)
        if self.layout not in LAYOUTS: raise ValueError(f"unknown layout {self.layout}")
        n = out_f * in_f
        nb, n_low, n_scratch, self.K16 = _layout_query(out_f, in_f, self.code)
        if bases.numel() != nb or hdr.numel() != nb * L.HDR_BLOCK or low.numel() not in (n_low, n_low + L.RAW_SLACK) or lut.numel() != L.TAB_WORDS:
            raise ValueError("checkpoint does not match this library version")
        self.out_features, self.in_features, self.n, self.block = out_f, in_f, n, block
        if low.numel() == n_low: low = F.pad(low, (0, L.RAW_SLACK))      # the planes are read one slot ahead
        self.data, self.bases, self.hdr, self.lut, self.low = (t.contiguous().to(device) for t in (data, bases, hdr, lut, low))
        self.scale = None if scale is None else scale.float().contiguous().to(device)
        self._finish(self.data.numel(), n_low, n_scratch, device)
        return self

    def tensors(self):
        """The tensors that fully describe the compressed state."""
        t = {"data": self.data, "bases": self.bases, "hdr": self.hdr, "lut": self.lut, "low": self.low}
        if self.scale is not None: t["scale"] = self.scale
        return t

    def _padded_x(self, x):
        """x zero-extended to the length the kernels read: K16 for layout 0, K rounded up to 32 otherwise."""
        want = (self.in_features + 31) // 32 * 32 if self.layout else self.K16
        return x if want == self.in_features else F.pad(x, (0, want - self.in_features))

    _x16 = _padded_x

    def matvec(self, x_f32: torch.Tensor) -> torch.Tensor:
        """fp32 test path: y = W x, fp32 in and out."""
        y = torch.empty(self.out_features, dtype=torch.float32, device=x_f32.device)
        xin = self._padded_x(x_f32.float().contiguous())
        err = L.lib.nwc_matvec(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low),
                               L.ptr(xin), L.ptr(y), self.n, self.block, self.in_features, self.code)
        if err: raise RuntimeError(f"nwc_matvec error {err}")
        return y if self.scale is None else y * self.scale

    def linear_bf16(self, x: torch.Tensor, bias, splits: int = 0) -> torch.Tensor:
        """Token path: y = scale * (W x) + bias; x bf16 or fp32 [in], y bf16 [out]."""
        y = torch.empty(self.out_features, dtype=torch.bfloat16, device=x.device)
        if self.layout: xin = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        else: xin = x if x.dtype == torch.float32 else x.float()
        xin = self._padded_x(xin.contiguous())
        err = L.lib.nwc_linear_bf16_splits(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low),
                                           L.ptr(xin), L.ptr(bias), L.ptr(self.scale), L.ptr(self.scratch), L.ptr(y),
                                           self.n, self.block, self.in_features, self.code, splits)
        if err: raise RuntimeError(f"nwc_linear_bf16 error {err}")
        return y

    def linear_prefill(self, x: torch.Tensor, bias=None):
        """Many tokens at once: x bf16 [T, in] -> bf16 [T, out] on the tcgen05 GEMM with tile-wise decoding, or None when
        this matrix's layout / element type is not covered by that path (the caller then dequantises)."""
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.in_features: return None
        T, K = x.shape
        if K % 8: x = F.pad(x, (0, 8 - K % 8))
        x = x.contiguous()
        y = torch.empty(T, self.out_features, dtype=torch.bfloat16, device=x.device)
        err = L.lib.nwc_linear_prefill(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low), L.ptr(x), T,
                                       x.shape[1], L.ptr(bias), L.ptr(self.scale), L.ptr(y), self.out_features, self.n, self.block, self.in_features, self.code)
        if err == -2: return None
        if err: raise RuntimeError(f"nwc_linear_prefill error {err}")
        return y

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        """Rows ids -> bf16[..., in] (embedding lookup straight from the compressed matrix)."""
        flat = ids.reshape(-1).to(device=self.data.device, dtype=torch.int64).contiguous()
        out = torch.empty(flat.numel(), self.K16, dtype=torch.bfloat16, device=self.data.device)
        err = L.lib.nwc_gather(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low),
                               L.ptr(flat), flat.numel(), L.ptr(out), self.n, self.block, self.in_features, self.code)
        if err: raise RuntimeError(f"nwc_gather error {err}")
        if self.K16 != self.in_features: out = out[:, : self.in_features].contiguous()
        return out.view(*ids.shape, self.in_features)

    def dequant(self) -> torch.Tensor:
        """The whole matrix as bf16 (a view with row stride K16 when K is not a multiple of 16).  fp8: the unscaled
        fp8 values, exact in bf16; multiply rows by `scale` for the weights."""
        w = torch.empty((self.out_features, self.K16), dtype=torch.bfloat16, device=self.data.device)
        err = L.lib.nwc_dequant(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low),
                                L.ptr(w), self.n, self.block, self.in_features, self.code)
        if err: raise RuntimeError(f"nwc_dequant error {err}")
        return w if self.K16 == self.in_features else w[:, : self.in_features]

    def dequant_fp8(self):
        """fp8 matrices: (float8_e4m3fn [out, in], fp32 scale[out]), bit-exact with what was encoded."""
        if self.elem != ELEM_FP8: raise ValueError("not an fp8 matrix")
        return self.dequant().to(torch.float8_e4m3fn), self.scale


def ref_fp8_matvec(w8: torch.Tensor, scale: torch.Tensor, x_f32: torch.Tensor) -> torch.Tensor:
    """Uncompressed fp8 weight-only matvec of the library (bandwidth baseline): y = bf16(scale * (W8 x))."""
    M, K = w8.shape
    y = torch.empty(M, dtype=torch.bfloat16, device=w8.device)
    xin = x_f32 if x_f32.numel() % 16 == 0 else F.pad(x_f32, (0, 16 - x_f32.numel() % 16))
    err = L.lib.nwc_ref_fp8(L.stream(), L.ptr(w8.view(torch.uint8)), L.ptr(scale), L.ptr(xin.contiguous()), L.ptr(y), M, K)
    if err: raise RuntimeError(f"nwc_ref_fp8 error {err}")
    return y
