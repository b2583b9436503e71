"""NWCWeight: one [out, in] matrix kept entropy-coded in HBM and the kernels that consume it without ever writing a
decompressed copy.

The attribute and method names are the reference's compressed-tensor contract (reference: nwc/nwc_torch.py:126-269:
data, bases, hdr, lut, low, scale, scratch, K16, bytes, bytes_bf16, bytes_native, elem, layout, code, block;
linear_bf16 / matvec / gather / dequant / tensors / from_tensors), because checkpoints and model code are written
against them.  Behind them this class is a thin owner of device tensors around three things of this library: the GPU
encoder (construction), `repack.Compressed` (the stored form, also what tensor-parallel shards are cut from) and the
C-ABI calls.
"""
import os

import torch
import torch.nn.functional as F

from . import _lib as L
from .repack import Compressed

ELEM_BF16, ELEM_FP8 = 0, 1
ELEMS = {"bf16": ELEM_BF16, "fp8": ELEM_FP8}
ELEM_NAMES = {v: k for k, v in ELEMS.items()}
LAYOUTS = (0, 1, 2)
FP8_MAX = 448.0
# default layout per element type; NWC_LAYOUT=0|1|2 overrides (same switch as the reference)
LAYOUT_DEFAULT = {ELEM_BF16: 0, ELEM_FP8: 0}
if "NWC_LAYOUT" in os.environ:
    LAYOUT_DEFAULT = {k: int(os.environ["NWC_LAYOUT"]) for k in LAYOUT_DEFAULT}


def quantize_fp8(w: torch.Tensor):
    """[out, in] weights -> (float8_e4m3fn codes, fp32 scale[out]) with scale = row absmax / 448, the weight-only fp8
    scheme of the reference (nwc/nwc_torch.py:88-94)."""
    full = w.detach().to(torch.float32)
    scale = torch.clamp_min(full.abs().amax(dim=1), 1e-12) / FP8_MAX
    codes = torch.clamp(full / scale.unsqueeze(1), -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes, scale


def fits(out_features, in_features):
    """Every non-empty shape is supported: blocks are padded to 8 or 16 rows x 512 columns."""
    return in_features >= 1 and out_features >= 1


def choose_block(n):
    return L.FIXED_BLOCK


class _Sizes:
    """What nwc_layout reports for a shape: block count, raw-plane bytes, scratch floats, padded row length."""

    def __init__(self, out_f, in_f, code):
        answer = torch.empty(4, dtype=torch.int64)
        if L.lib.nwc_layout(out_f, in_f, code, L.ptr(answer)): raise RuntimeError("nwc_layout: bad shape")
        self.blocks, self.raw_bytes, self.scratch_floats, self.K16 = answer.tolist()


def _encode_on_device(src, out_f, in_f, code, sizes, device):
    """Run the GPU encoder over `src` (int16 bf16 bits or uint8 fp8 codes, on `device`).  The stream buffer is sized for
    ~12 bits per weight first and for the worst case if that does not suffice.  Returns (data, bases, hdr, low, lut)."""
    n = out_f * in_f
    psym = torch.zeros(L.NPAIR, dtype=torch.int16)
    bases = torch.empty(sizes.blocks, dtype=torch.int32, device=device)
    hdr = torch.empty(sizes.blocks * L.HDR_BLOCK, dtype=torch.uint8, device=device)
    low = torch.zeros(sizes.raw_bytes + L.RAW_SLACK, dtype=torch.uint8, device=device)
    overhead = sizes.blocks * 64 + 4096
    for capacity in (n + n // 2 + overhead, 3 * n + overhead):
        stream = torch.empty(capacity, dtype=torch.uint8, device=device)
        length = L.lib.nwc_encode_device(L.stream(), L.ptr(src), n, in_f, code, L.ptr(psym), L.ptr(bases), L.ptr(hdr), L.ptr(stream), capacity, L.ptr(low))
        if length != -1: break
    if length == -2: raise ValueError("fp8 weights contain NaN")
    if length == -3: raise ValueError("layout 2 cannot code this matrix (a lane stream has more than 255 exceptions); use layout 0 or 1")
    if length < 0: raise RuntimeError(f"nwc_encode failed ({length})")
    data = torch.zeros(length + 64, dtype=torch.uint8, device=device)         # exact size + the slack the kernels may read
    data[:length].copy_(stream[:length])
    lut = torch.empty(L.TAB_WORDS, dtype=torch.int32)
    L.lib.nwc_build_tab(None, L.ptr(psym), code, L.ptr(lut))
    return data, bases, hdr, low, lut.to(device)


class NWCWeight:
    """Compressed [out, in] matrix on the GPU.  elem "bf16": lossless.  elem "fp8": weight-only fp8 e4m3 with an fp32
    scale per output channel (from a bf16 matrix through quantize_fp8, or a float8 tensor plus `scale`), the fp8 bytes
    stored lossless.  The encoder runs on the GPU; `w` may live on either side."""

    def __init__(self, w: torch.Tensor, device="cuda", block=None, elem="bf16", scale=None, layout=None):
        L.require_cuda()
        device = torch.device(device)
        if device.type != "cuda": raise RuntimeError("nwc_b200 encodes and decodes on CUDA devices only")
        if w.dim() != 2: raise ValueError("a 2-d weight matrix is expected")
        if not fits(*w.shape): raise ValueError(f"shape {tuple(w.shape)} not supported")
        self._describe(w.shape[0], w.shape[1], ELEMS[elem], LAYOUT_DEFAULT[ELEMS[elem]] if layout is None else int(layout), block or L.FIXED_BLOCK)
        with torch.cuda.device(device):
            if self.elem == ELEM_FP8:
                if w.dtype != torch.float8_e4m3fn: w, scale = quantize_fp8(w.to(device))
                elif scale is None: raise ValueError("fp8 weights need their per-row scale")
                src = w.detach().to(device).contiguous().view(torch.uint8)
                scale = scale.detach().to(device=device, dtype=torch.float32).contiguous()
            else:
                if w.dtype != torch.bfloat16: raise ValueError("bf16 weights expected (elem='fp8' for fp8 weights)")
                src, scale = w.detach().to(device).contiguous().view(torch.int16), None
            sizes = _Sizes(self.out_features, self.in_features, self.code)
            data, bases, hdr, low, lut = _encode_on_device(src, self.out_features, self.in_features, self.code, sizes, device)
            self._adopt(data, bases, hdr, lut, low, scale, sizes, data.numel() - 64, device)

    # ---- construction helpers ----
    def _describe(self, out_f, in_f, elem, layout, block):
        if layout not in LAYOUTS: raise ValueError(f"unknown layout {layout}")
        self.out_features, self.in_features, self.n = int(out_f), int(in_f), int(out_f) * int(in_f)
        self.elem, self.layout, self.block = elem, layout, block

    def _adopt(self, data, bases, hdr, lut, low, scale, sizes, stream_bytes, device):
        """Take ownership of the device tensors and do the byte accounting (the roofline numerator of every matvec: stream +
        offsets + headers + table + raw planes + scales, as the reference counts them, nwc/nwc_torch.py:185-190)."""
        self.data, self.bases, self.hdr, self.lut, self.low, self.scale, self.K16 = data, bases, hdr, lut, low, scale, sizes.K16
        self.bytes = stream_bytes + 4 * bases.numel() + hdr.numel() + 4 * lut.numel() + sizes.raw_bytes + (4 * scale.numel() if scale is not None else 0)
        self.bytes_bf16 = 2 * self.n
        self.bytes_native = self.n + 4 * self.out_features if self.elem == ELEM_FP8 else 2 * self.n
        self.scratch = torch.empty(sizes.scratch_floats, dtype=torch.float32, device=device)
        self.side, self.side_bytes = None, 0

    def build_side_table(self):
        """Layout 0: the engine-private table of per-lane bit positions at which rows 2, 4 and 6 of every block begin
        (nwc_build_side_table), so that four warps can decode a block in parallel.  Never stored in checkpoints; its bytes
        are read by every token matvec that uses it and are counted in `side_bytes`."""
        if self.layout != 0: raise ValueError("side tables exist for layout 0 only")
        if getattr(self, "side", None) is None:
            nbytes = L.lib.nwc_side_table_bytes(self.out_features, self.in_features)
            side = torch.empty(nbytes // 2, dtype=torch.int16, device=self.data.device)
            err = L.lib.nwc_build_side_table(L.stream(), L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(side), *self._shape_args())
            if err: raise RuntimeError(f"nwc_build_side_table error {err}")
            self.side, self.side_bytes = side, nbytes
        return self.side

    @property
    def code(self):
        """The library's elem parameter: element type in bits 0..3, layout in bits 4..7."""
        return self.elem | (self.layout << 4)

    @classmethod
    def from_compressed(cls, c: Compressed, device="cuda", block=None):
        """A matrix in its stored form (a checkpoint record or a tensor-parallel shard cut from one) onto `device`."""
        L.require_cuda()
        self = cls.__new__(cls)
        self._describe(c.M, c.K, ELEMS[c.elem], int(c.layout), block or L.FIXED_BLOCK)
        sizes = _Sizes(c.M, c.K, self.code)
        low = c.low
        if (c.bases.numel(), c.hdr.numel(), c.lut.numel()) != (sizes.blocks, sizes.blocks * L.HDR_BLOCK, L.TAB_WORDS) or low.numel() not in (sizes.raw_bytes, sizes.raw_bytes + L.RAW_SLACK):
            raise ValueError("checkpoint does not match this library version")
        if low.numel() == sizes.raw_bytes: low = F.pad(low, (0, L.RAW_SLACK))          # the planes are read one slot ahead
        put = lambda t: t.contiguous().to(device)
        scale = None if c.scale is None else put(c.scale.float())
        self._adopt(put(c.data), put(c.bases), put(c.hdr), put(c.lut), put(low), scale, sizes, c.data.numel(), device)
        return self

    @classmethod
    def from_tensors(cls, out_f, in_f, block, data, bases, hdr, lut, low, device="cuda", elem="bf16", scale=None, layout=0):
        """Compressed matrix from stored tensors (checkpoints), without the original weights."""
        return cls.from_compressed(Compressed(out_f, in_f, int(layout), elem, data, bases, hdr, lut, low, scale), device, block)

    def compressed(self) -> Compressed:
        return Compressed(self.out_features, self.in_features, self.layout, ELEM_NAMES[self.elem], self.data, self.bases, self.hdr, self.lut, self.low, self.scale)

    def tensors(self):
        """The tensors that fully describe the compressed state."""
        named = {"data": self.data, "bases": self.bases, "hdr": self.hdr, "lut": self.lut, "low": self.low}
        if self.scale is not None: named["scale"] = self.scale
        return named

    # ---- calls ----
    def _operands(self):
        return (L.ptr(self.data), L.ptr(self.bases), L.ptr(self.hdr), L.ptr(self.lut), L.ptr(self.low))

    def _shape_args(self):
        return (self.n, self.block, self.in_features, self.code)

    def _padded_x(self, x):
        """x zero-extended to the length the kernels read: K16 for layout 0, K rounded up to 32 otherwise."""
        want = (self.in_features + 31) // 32 * 32 if self.layout else self.K16
        return x if want == self.in_features else F.pad(x, (0, want - self.in_features))

    _x16 = _padded_x

    def matvec(self, x_f32: torch.Tensor) -> torch.Tensor:
        """fp32 test path: y = W x, fp32 in and out."""
        y = torch.empty(self.out_features, dtype=torch.float32, device=x_f32.device)
        xin = self._padded_x(x_f32.float().contiguous())
        err = L.lib.nwc_matvec(L.stream(), *self._operands(), L.ptr(xin), L.ptr(y), *self._shape_args())
        if err: raise RuntimeError(f"nwc_matvec error {err}")
        return y if self.scale is None else y * self.scale

    def linear_bf16(self, x: torch.Tensor, bias, splits: int = 0) -> torch.Tensor:
        """Token path: y = scale * (W x) + bias; x bf16 or fp32 [in], y bf16 [out].  The ABI takes fp32 x for layout 0 and
        bf16 x for layouts 1 and 2."""
        y = torch.empty(self.out_features, dtype=torch.bfloat16, device=x.device)
        xin = self._padded_x(x.to(torch.bfloat16 if self.layout else torch.float32).contiguous())
        err = L.lib.nwc_linear_bf16_splits(L.stream(), *self._operands(), L.ptr(xin), L.ptr(bias), L.ptr(self.scale), L.ptr(self.scratch), L.ptr(y),
                                           *self._shape_args(), splits)
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
        err = L.lib.nwc_linear_prefill(L.stream(), *self._operands(), L.ptr(x), T, x.shape[1], L.ptr(bias), L.ptr(self.scale), L.ptr(y), self.out_features,
                                       *self._shape_args())
        if err == -2: return None
        if err: raise RuntimeError(f"nwc_linear_prefill error {err}")
        return y

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        """Rows ids -> bf16[..., in] (embedding lookup straight from the compressed matrix)."""
        flat = ids.reshape(-1).to(device=self.data.device, dtype=torch.int64).contiguous()
        out = torch.empty(flat.numel(), self.K16, dtype=torch.bfloat16, device=self.data.device)
        err = L.lib.nwc_gather_side(L.stream(), *self._operands(), L.ptr(flat), flat.numel(), L.ptr(out), *self._shape_args(), L.ptr(self.side))
        if err: raise RuntimeError(f"nwc_gather error {err}")
        if self.K16 != self.in_features: out = out[:, : self.in_features].contiguous()
        return out.view(*ids.shape, self.in_features)

    def dequant(self) -> torch.Tensor:
        """The whole matrix as bf16 (a view with row stride K16 when K is not a multiple of 16).  fp8: the unscaled
        fp8 values, exact in bf16; multiply rows by `scale` for the weights."""
        w = torch.empty((self.out_features, self.K16), dtype=torch.bfloat16, device=self.data.device)
        err = L.lib.nwc_dequant(L.stream(), *self._operands(), L.ptr(w), *self._shape_args())
        if err: raise RuntimeError(f"nwc_dequant error {err}")
        return w if self.K16 == self.in_features else w[:, : self.in_features]

    def dequant_fp8(self):
        """fp8 matrices: (float8_e4m3fn [out, in], fp32 scale[out]), bit-exact with what was encoded."""
        if self.elem != ELEM_FP8: raise ValueError("not an fp8 matrix")
        return self.dequant().to(torch.float8_e4m3fn), self.scale

    def dense(self) -> torch.Tensor:
        """The weights as a plain bf16 matrix (fp8: codes times scale, rounded to bf16)."""
        full = self.dequant()
        return full if self.scale is None else (full.float() * self.scale[:, None]).to(torch.bfloat16)


def ref_fp8_matvec(w8: torch.Tensor, scale: torch.Tensor, x_f32: torch.Tensor) -> torch.Tensor:
    """Uncompressed fp8 weight-only matvec of the library (bandwidth baseline): y = bf16(scale * (W8 x))."""
    M, K = w8.shape
    y = torch.empty(M, dtype=torch.bfloat16, device=w8.device)
    xin = x_f32 if x_f32.numel() % 16 == 0 else F.pad(x_f32, (0, 16 - x_f32.numel() % 16))
    err = L.lib.nwc_ref_fp8(L.stream(), L.ptr(w8.view(torch.uint8)), L.ptr(scale), L.ptr(xin.contiguous()), L.ptr(y), M, K)
    if err: raise RuntimeError(f"nwc_ref_fp8 error {err}")
    return y
