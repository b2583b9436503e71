"""nn.Module drop-ins on compressed matrices and the model-wide conversion helpers.

Same public names and behaviour as the reference's integration layer (reference: nwc/nwc_torch.py:272-445):
NWCLinear / NWCEmbedding replace nn.Linear / nn.Embedding, `fuse` concatenates sibling projections into one matrix,
`convert` walks a model and swaps every supported layer.  One token (x.numel() == in_features, bf16) takes the fused
decode-matvec; anything else dequantises and calls a dense matmul.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .weight import NWCWeight, fits, quantize_fp8, ref_fp8_matvec


class NWCLinear(nn.Module):
    """nn.Linear on a compressed matrix (elem "bf16" lossless, or "fp8" weight-only)."""

    def __init__(self, linear: nn.Linear = None, device="cuda", block=None, w: NWCWeight = None, bias=None, elem="bf16", layout=None):
        super().__init__()
        self.w = w if w is not None else NWCWeight(linear.weight.data, device, block, elem=elem, layout=layout)
        self.in_features, self.out_features = self.w.in_features, self.w.out_features
        if linear is not None and linear.bias is not None: bias = linear.bias.data
        self.bias = None if bias is None else nn.Parameter(bias.to(device=device, dtype=torch.bfloat16), requires_grad=False)

    def forward(self, x):
        if x.numel() == self.in_features and x.dtype == torch.bfloat16:            # one token: fused kernel
            y = self.w.linear_bf16(x.contiguous().view(-1), None if self.bias is None else self.bias.data)
            return y.view(*x.shape[:-1], self.out_features)
        if x.dtype == torch.bfloat16:                                                # prefill: decode tile-wise into the tensor-core GEMM where covered
            y = self.w.linear_prefill(x.reshape(-1, self.in_features), None if self.bias is None else self.bias.data)
            if y is not None: return y.view(*x.shape[:-1], self.out_features)
        if self.w.scale is None: return F.linear(x, self.w.dequant(), self.bias)    # otherwise: temporary dequantisation
        y = F.linear(x, self.w.dequant()).float() * self.w.scale                     # fp8: unscaled matmul, then the row scale
        if self.bias is not None: y = y + self.bias.float()
        return y.to(x.dtype)

    def extra_repr(self):
        return (f"in={self.in_features}, out={self.out_features}, elem={'fp8' if self.w.elem else 'bf16'}, layout={self.w.layout}, "
                f"{self.w.bytes / 1e6:.1f} MB (BF16: {self.w.bytes_bf16 / 1e6:.1f} MB)")


class NWCEmbedding(nn.Module):
    """nn.Embedding on a compressed matrix (may share it with a tied lm_head)."""

    def __init__(self, emb: nn.Embedding = None, w: NWCWeight = None, padding_idx=None):
        super().__init__()
        self.w = w
        self.num_embeddings, self.embedding_dim = w.out_features, w.in_features
        self.padding_idx = emb.padding_idx if emb is not None else padding_idx

    def forward(self, ids):
        rows = self.w.gather(ids)
        if self.w.scale is None: return rows
        return (rows.float() * self.w.scale[ids.to(self.w.scale.device)][..., None]).to(torch.bfloat16)

    def extra_repr(self):
        return f"{self.num_embeddings}, {self.embedding_dim}, {self.w.bytes / 1e6:.1f} MB (BF16: {self.w.bytes_bf16 / 1e6:.1f} MB)"


class _FusedHead(nn.Module):
    """One output slice of a fused projection: head 0 runs the fused matvec, the others pick their slice of its result."""

    def __init__(self, shared, index, start, end):
        super().__init__()
        self.g, self.index, self.start, self.end = shared, index, start, end
        self.in_features, self.out_features = shared["lin"].in_features, end - start

    def forward(self, x):
        g = self.g
        if self.index == 0 or g["x_id"] != id(x) or g["y"] is None:
            g["y"] = g["lin"](x); g["x_id"] = id(x)
        return g["y"][..., self.start:self.end]


def fuse(model: nn.Module, groups=(("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj")), device="cuda", elem="bf16", layout=None, verbose=True):
    """Concatenate sibling nn.Linear layers that read the same input into one compressed matrix (fewer, larger
    launches).  Call before `convert`.  Returns the number of fused groups."""
    count = 0
    for mod in list(model.modules()):
        for names in groups:
            lins = [getattr(mod, nm, None) for nm in names]
            if not all(isinstance(l, nn.Linear) for l in lins): continue
            if len({l.in_features for l in lins}) != 1 or any(l.weight.dtype != torch.bfloat16 for l in lins): continue
            W = torch.cat([l.weight.data for l in lins], 0)
            if not fits(*W.shape): continue
            bias = None
            if any(l.bias is not None for l in lins):
                bias = torch.cat([l.bias.data if l.bias is not None else torch.zeros(l.out_features, dtype=W.dtype, device=W.device) for l in lins], 0)
            lin = NWCLinear(w=NWCWeight(W, device, elem=elem, layout=layout), bias=bias, device=device)
            shared = {"lin": lin, "y": None, "x_id": None, "names": list(names), "sizes": [l.out_features for l in lins]}
            start = 0
            for i, (nm, l) in enumerate(zip(names, lins)):
                setattr(mod, nm, _FusedHead(shared, i, start, start + l.out_features)); start += l.out_features
                l.weight.data = torch.empty(0)
            count += 1
    if verbose: print(f"NWC: {count} projection groups fused")
    return count


def _children(model):
    for name, mod in list(model.named_modules()):
        for child, cm in list(mod.named_children()):
            yield name, mod, child, cm


def convert(model: nn.Module, device="cuda", verbose=True, tied=True, elem="bf16", embeddings=True, layout=None):
    """Replace every supported nn.Linear (and embeddings) by NWC modules and move the rest to `device`.
    Returns (bytes_nwc, bytes_bf16) of the compressed matrices."""
    total_nwc = total_bf16 = replaced = 0
    skipped = []

    def account(w):
        nonlocal total_nwc, total_bf16, replaced
        total_nwc += w.bytes; total_bf16 += w.bytes_bf16; replaced += 1

    shared_ptrs = {m.weight.data_ptr() for m in model.modules() if isinstance(m, nn.Embedding)}
    if tied:       # tied embedding + lm_head: one compressed matrix serves the lookup (gather) and the logits (matvec)
        embs = {m.weight.data_ptr(): m for m in model.modules()
                if isinstance(m, nn.Embedding) and m.weight.dtype == torch.bfloat16 and m.weight.numel() and fits(m.num_embeddings, m.embedding_dim)}
        for name, mod, child, cm in list(_children(model)):
            if not (isinstance(cm, nn.Linear) and cm.weight.numel() and cm.weight.data_ptr() in embs): continue
            emb = embs[cm.weight.data_ptr()]
            w = NWCWeight(emb.weight.data, device, elem=elem, layout=layout)
            setattr(mod, child, NWCLinear(cm, device, w=w))
            for _, emod, echild, ecm in list(_children(model)):
                if ecm is emb: setattr(emod, echild, NWCEmbedding(emb, w))
            account(w)
            shared_ptrs.discard(cm.weight.data_ptr())
            emb.weight.data = torch.empty(0); cm.weight.data = torch.empty(0)
    if embeddings:  # untied tables: always lossless bf16, looked up with the gather kernel
        for name, mod, child, cm in list(_children(model)):
            if isinstance(cm, nn.Embedding) and cm.weight.dtype == torch.bfloat16 and cm.weight.numel() and fits(cm.num_embeddings, cm.embedding_dim):
                w = NWCWeight(cm.weight.data, device, elem="bf16", layout=layout)
                setattr(mod, child, NWCEmbedding(cm, w))
                account(w); cm.weight.data = torch.empty(0)
    for m in model.modules():
        if isinstance(m, _FusedHead) and m.index == 0: account(m.g["lin"].w)
    for name, mod, child, cm in list(_children(model)):
        if not isinstance(cm, nn.Linear): continue
        if cm.weight.dtype == torch.bfloat16 and cm.weight.numel() and fits(cm.out_features, cm.in_features) and cm.weight.data_ptr() not in shared_ptrs:
            new = NWCLinear(cm, device, elem=elem, layout=layout)
            setattr(mod, child, new); account(new.w)
            cm.weight.data = torch.empty(0)
        else:
            skipped.append(f"{name}.{child} {tuple(cm.weight.shape)} [{'tied' if cm.weight.data_ptr() in shared_ptrs else 'shape'}]")
    model.to(device)
    if verbose:
        print(f"NWC ({elem}): {replaced} linear layers replaced, {total_bf16 / 1e9:.2f} GB BF16 -> {total_nwc / 1e9:.2f} GB "
              f"(ratio {total_nwc / max(total_bf16, 1):.4f})")
        if skipped: print("  skipped:", ", ".join(skipped[:6]), "..." if len(skipped) > 6 else "")
    return total_nwc, total_bf16


class RefFP8Linear(nn.Module):
    """Comparison only: uncompressed weight-only fp8 served by the library's plain fp8 matvec at batch 1."""

    def __init__(self, linear: nn.Linear, device="cuda"):
        super().__init__()
        q, scale = quantize_fp8(linear.weight.data)
        self.w8 = q.contiguous().to(device); self.scale = scale.to(device)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.bias = None if linear.bias is None else nn.Parameter(linear.bias.data.to(device=device, dtype=torch.bfloat16), requires_grad=False)

    def forward(self, x):
        if x.numel() == self.in_features and x.dtype == torch.bfloat16:
            y = ref_fp8_matvec(self.w8, self.scale, x.reshape(-1).float())
            if self.bias is not None: y = y + self.bias
            return y.view(*x.shape[:-1], self.out_features)
        y = F.linear(x, self.w8.to(torch.bfloat16)).float() * self.scale
        if self.bias is not None: y = y + self.bias.float()
        return y.to(x.dtype)


def convert_ref_fp8(model: nn.Module, device="cuda", verbose=True):
    """Replace every untied nn.Linear by RefFP8Linear (the uncompressed fp8 baseline)."""
    shared = {m.weight.data_ptr() for m in model.modules() if isinstance(m, nn.Embedding)}
    n = 0
    for name, mod, child, cm in list(_children(model)):
        if isinstance(cm, nn.Linear) and cm.weight.dtype == torch.bfloat16 and cm.weight.data_ptr() not in shared:
            setattr(mod, child, RefFP8Linear(cm, device)); cm.weight.data = torch.empty(0); n += 1
    model.to(device)
    if verbose: print(f"reference fp8: {n} linear layers replaced")
    return n
