"""nn.Module drop-ins on compressed matrices, and the model-wide conversion.

Public names and call signatures follow the reference's integration layer (reference: nwc/nwc_torch.py:272-445):
NWCLinear / NWCEmbedding stand in for nn.Linear / nn.Embedding, `fuse` merges sibling projections that read the same
input into one compressed matrix, `convert` swaps every supported layer of a model.  How they work here:

  * one token (x.numel() == in_features, bf16) runs the fused decode-matvec; more tokens run `NWCLinear.prefill_backend`:
    "dense" (default: dequantise into a temporary, then the vendor matmul - what the reference does, and the faster of
    the two on B200 today) or "tcgen05" (this library's tile-wise decode into a tensor-memory GEMM, layout 2 bf16);
  * a fused projection is ONE module-level object (`FusedProjection`) that owns the matrix and remembers its latest
    result together with the identity of the input storage it was computed from; its heads are views into that result;
  * `convert` first makes a plan (which layer becomes what, which table is shared with the lm_head) from one scan of the
    model and then carries it out, so nothing depends on module iteration order.
"""
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from .weight import NWCWeight, fits, quantize_fp8, ref_fp8_matvec


def _bias_param(bias, device):
    return None if bias is None else nn.Parameter(bias.detach().to(device=device, dtype=torch.bfloat16), requires_grad=False)


def _drop_storage(param):
    """Free a replaced layer's original weights (the module object may still be referenced elsewhere)."""
    param.data = torch.empty(0)


class NWCLinear(nn.Module):
    """nn.Linear on a compressed matrix (elem "bf16" lossless, or "fp8" weight-only)."""

    prefill_backend = os.environ.get("NWC_PREFILL", "dense")      # "dense" | "tcgen05"

    def __init__(self, linear: nn.Linear = None, device="cuda", block=None, w: NWCWeight = None, bias=None, elem="bf16", layout=None):
        super().__init__()
        if w is None:
            if linear is None: raise ValueError("NWCLinear needs an nn.Linear or a compressed matrix")
            w = NWCWeight(linear.weight.data, device, block, elem=elem, layout=layout)
        if linear is not None and linear.bias is not None: bias = linear.bias.data
        self.w, self.bias = w, _bias_param(bias, device)
        self.in_features, self.out_features = w.in_features, w.out_features

    def _bias_data(self):
        return None if self.bias is None else self.bias.data

    def _many_tokens(self, x):
        """x [..., in] with more than one token."""
        if self.prefill_backend == "tcgen05" and x.dtype == torch.bfloat16:
            y = self.w.linear_prefill(x.reshape(-1, self.in_features), self._bias_data())
            if y is not None: return y.view(*x.shape[:-1], self.out_features)
        dense = self.w.dequant()                                   # temporary bf16 copy, freed after the matmul
        if self.w.scale is None: return F.linear(x, dense, self.bias)
        y = F.linear(x, dense).float() * self.w.scale              # fp8: matmul over the unscaled codes, then the row scale
        if self.bias is not None: y = y + self.bias.float()
        return y.to(x.dtype)

    def forward(self, x):
        if x.dtype == torch.bfloat16 and x.numel() == self.in_features:
            y = self.w.linear_bf16(x.reshape(-1), self._bias_data())
            return y.view(*x.shape[:-1], self.out_features)
        return self._many_tokens(x)

    def extra_repr(self):
        w = self.w
        return (f"in={self.in_features}, out={self.out_features}, elem={'fp8' if w.elem else 'bf16'}, layout={w.layout}, "
                f"{w.bytes / 1e6:.1f} MB (BF16: {w.bytes_bf16 / 1e6:.1f} MB)")


class NWCEmbedding(nn.Module):
    """nn.Embedding on a compressed matrix (may share it with a tied lm_head)."""

    def __init__(self, emb: nn.Embedding = None, w: NWCWeight = None, padding_idx=None):
        super().__init__()
        if w is None: raise ValueError("NWCEmbedding needs the compressed table")
        self.w = w
        self.num_embeddings, self.embedding_dim = w.out_features, w.in_features
        self.padding_idx = padding_idx if emb is None else emb.padding_idx

    def forward(self, ids):
        # many ids at once (a prompt) from a layout-0 table: the side table lets every row's walk start at its row pair
        if self.w.layout == 0 and self.w.side is None and ids.numel() >= 64: self.w.build_side_table()
        rows = self.w.gather(ids)
        if self.w.scale is None: return rows
        row_scale = self.w.scale[ids.to(self.w.scale.device)]     # fp8 table: codes come back unscaled
        return (rows.float() * row_scale.unsqueeze(-1)).to(torch.bfloat16)

    def extra_repr(self):
        return f"{self.num_embeddings}, {self.embedding_dim}, {self.w.bytes / 1e6:.1f} MB (BF16: {self.w.bytes_bf16 / 1e6:.1f} MB)"


class FusedProjection:
    """Several projections of the same input stored as one compressed matrix (q/k/v, gate/up).  Not a module itself: its
    heads are the modules the model calls.  The first head called with a new input runs the matrix once; the others slice
    the stored result.  "Same input" = same storage address, shape and version counter, so a recycled Python object id or
    an in-place update of x can never return a stale result."""

    def __init__(self, lin: NWCLinear, names, sizes):
        self.lin, self.names, self.sizes = lin, list(names), [int(s) for s in sizes]
        self.offsets = [sum(self.sizes[:i]) for i in range(len(self.sizes))]
        self._key, self._out = None, None

    def result(self, x):
        key = (x.data_ptr(), tuple(x.shape), x._version, x.dtype)
        if key != self._key or self._out is None:
            self._out, self._key = self.lin(x), key
        return self._out

    def heads(self):
        return [_FusedHead(self, i) for i in range(len(self.names))]


class _FusedHead(nn.Module):
    """One output slice of a FusedProjection."""

    def __init__(self, group: FusedProjection, index: int):
        super().__init__()
        self.g, self.index = group, index
        self.start = group.offsets[index]
        self.end = self.start + group.sizes[index]
        self.in_features, self.out_features = group.lin.in_features, group.sizes[index]

    def forward(self, x):
        return self.g.result(x)[..., self.start:self.end]


def install_fused(parent: nn.Module, group: FusedProjection):
    """Put the heads of `group` in place of the attributes it names on `parent`."""
    for name, head in zip(group.names, group.heads()): setattr(parent, name, head)


def fused_groups(model: nn.Module):
    """(parent path, FusedProjection) for every fused projection of the model, each once."""
    seen, found = set(), []
    for path, mod in model.named_modules():
        if isinstance(mod, _FusedHead) and id(mod.g) not in seen:
            seen.add(id(mod.g)); found.append((path.rpartition(".")[0], mod.g))
    return found


def fuse(model: nn.Module, groups=(("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj")), device="cuda", elem="bf16", layout=None, verbose=True):
    """Concatenate sibling nn.Linear layers that read the same input into one compressed matrix (fewer, larger
    launches).  Call before `convert`.  Returns the number of fused groups."""
    made = 0
    for parent in list(model.modules()):
        for names in groups:
            members = [getattr(parent, n, None) for n in names]
            if not all(isinstance(m, nn.Linear) for m in members): continue
            if any(m.in_features != members[0].in_features or m.weight.dtype != torch.bfloat16 for m in members): continue
            stacked = torch.cat([m.weight.data for m in members], dim=0)
            if not fits(*stacked.shape): continue
            bias = None
            if any(m.bias is not None for m in members):            # members without a bias contribute zeros
                bias = torch.cat([m.bias.data if m.bias is not None else stacked.new_zeros(m.out_features) for m in members])
            lin = NWCLinear(w=NWCWeight(stacked, device, elem=elem, layout=layout), bias=bias, device=device)
            install_fused(parent, FusedProjection(lin, names, [m.out_features for m in members]))
            for m in members: _drop_storage(m.weight)
            made += 1
    if verbose: print(f"NWC: {made} projection groups fused")
    return made


class _ConversionPlan:
    """What `convert` will do, decided from one scan: `tables` = embeddings to compress (with the lm_head modules that
    share their storage), `linears` = plain layers, `skipped` = layers left alone and why."""

    def __init__(self, model, tied, embeddings):
        self.tables, self.linears, self.skipped = [], [], []
        sites = [(path, parent, attr, child) for path, parent in model.named_modules() for attr, child in parent.named_children()]
        table_sites = [(s, s[3].weight.data_ptr()) for s in sites if isinstance(s[3], nn.Embedding)]
        table_ptrs = {ptr for _, ptr in table_sites}
        usable = lambda t: t.dtype == torch.bfloat16 and t.numel() > 0
        claimed = set()
        for site, ptr in table_sites:
            emb = site[3]
            if not (usable(emb.weight) and fits(emb.num_embeddings, emb.embedding_dim)): continue
            sharers = [s for s in sites if isinstance(s[3], nn.Linear) and s[3].weight.numel() and s[3].weight.data_ptr() == ptr] if tied else []
            if sharers or embeddings:
                self.tables.append((site, sharers))
                claimed.update(id(s[3]) for s in sharers)
        for s in sites:
            lin = s[3]
            if not isinstance(lin, nn.Linear) or id(lin) in claimed: continue
            name = f"{s[0]}.{s[2]}" if s[0] else s[2]
            if lin.weight.data_ptr() in table_ptrs and lin.weight.numel(): self.skipped.append(f"{name} {tuple(lin.weight.shape)} [tied]")
            elif usable(lin.weight) and fits(lin.out_features, lin.in_features): self.linears.append(s)
            else: self.skipped.append(f"{name} {tuple(lin.weight.shape)} [shape]")


def convert(model: nn.Module, device="cuda", verbose=True, tied=True, elem="bf16", embeddings=True, layout=None):
    """Replace every supported nn.Linear (and embeddings) by NWC modules and move the rest to `device`.
    Returns (bytes_nwc, bytes_bf16) of the compressed matrices.  A tied embedding + lm_head pair becomes ONE compressed
    matrix serving the lookup (gather kernel) and the logits (matvec); untied tables are always stored lossless."""
    plan = _ConversionPlan(model, tied, embeddings)
    done = [g.lin.w for _, g in fused_groups(model)]                # matrices `fuse` already made count towards the totals
    for (path, parent, attr, emb), sharers in plan.tables:
        w = NWCWeight(emb.weight.data, device, elem=elem if sharers else "bf16", layout=layout)
        setattr(parent, attr, NWCEmbedding(emb, w))
        for _, head_parent, head_attr, head in sharers:
            setattr(head_parent, head_attr, NWCLinear(head, device, w=w))
            _drop_storage(head.weight)
        _drop_storage(emb.weight)
        done.append(w)
    for path, parent, attr, lin in plan.linears:
        new = NWCLinear(lin, device, elem=elem, layout=layout)
        setattr(parent, attr, new)
        _drop_storage(lin.weight)
        done.append(new.w)
    model.to(device)
    total_nwc, total_bf16 = sum(w.bytes for w in done), sum(w.bytes_bf16 for w in done)
    if verbose:
        print(f"NWC ({elem}): {len(done)} linear layers replaced, {total_bf16 / 1e9:.2f} GB BF16 -> {total_nwc / 1e9:.2f} GB "
              f"(ratio {total_nwc / max(total_bf16, 1):.4f})")
        if plan.skipped: print("  skipped:", ", ".join(plan.skipped[:6]), "..." if len(plan.skipped) > 6 else "")
    return total_nwc, total_bf16


class RefFP8Linear(nn.Module):
    """Comparison only: uncompressed weight-only fp8 served by the library's plain fp8 matvec at batch 1 (the baseline the
    fp8 configuration is measured against; reference: nwc/nwc_torch.py:272-292)."""

    def __init__(self, linear: nn.Linear, device="cuda"):
        super().__init__()
        codes, scale = quantize_fp8(linear.weight.data)
        self.w8, self.scale = codes.contiguous().to(device), scale.to(device)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.bias = _bias_param(None if linear.bias is None else linear.bias.data, device)

    def forward(self, x):
        if x.dtype == torch.bfloat16 and x.numel() == self.in_features:
            y = ref_fp8_matvec(self.w8, self.scale, x.reshape(-1).float())
            return (y if self.bias is None else y + self.bias).view(*x.shape[:-1], self.out_features)
        y = F.linear(x, self.w8.to(torch.bfloat16)).float() * self.scale
        if self.bias is not None: y = y + self.bias.float()
        return y.to(x.dtype)


def convert_ref_fp8(model: nn.Module, device="cuda", verbose=True):
    """Replace every untied nn.Linear by RefFP8Linear (the uncompressed fp8 baseline)."""
    tables = {m.weight.data_ptr() for m in model.modules() if isinstance(m, nn.Embedding)}
    swapped = 0
    for parent in list(model.modules()):
        for attr, lin in list(parent.named_children()):
            if isinstance(lin, nn.Linear) and lin.weight.dtype == torch.bfloat16 and lin.weight.data_ptr() not in tables:
                setattr(parent, attr, RefFP8Linear(lin, device)); _drop_storage(lin.weight); swapped += 1
    model.to(device)
    if verbose: print(f"reference fp8: {swapped} linear layers replaced")
    return swapped
