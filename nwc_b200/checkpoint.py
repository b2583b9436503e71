"""save_pretrained / load_pretrained / export_bf16 for converted Hugging Face models.

The on-disk schema is the reference's (nwc/checkpoint.py; restated in nwc_b200/store.py), so checkpoints written by
either implementation load in the other.  The code around it is this library's:

  * saving walks the model once and turns every NWC module into a schema record (`_describe_model`);
  * loading builds the model skeleton on the meta device with plain torch, then installs one module per record, each
    matrix streamed from the tensor file directly onto the GPU (`store.CheckpointReader`): neither bf16 originals nor a
    host copy of the whole checkpoint ever exist;
  * exporting decodes matrix by matrix back to the plain bf16 tensor names of the original model.
The decode loop reads the same checkpoints without Transformers: `nwc_b200.decode.DecodeEngine.from_pretrained`.
"""
import os
import shutil

import torch
import torch.nn as nn

from ._lib import VERSION
from .modules import FusedProjection, NWCEmbedding, NWCLinear, fused_groups, install_fused
from .store import CheckpointReader, resolve, write_checkpoint  # noqa: F401  (resolve is part of this module's interface)
from .weight import ELEM_NAMES, NWCWeight


def _describe_model(model):
    """(matrix records, module records, extra tensors) of a converted model.  A matrix shared by several modules (tied
    embedding + lm_head) is stored once; fused groups contribute one record for all their heads."""
    matrices, modules, extra, ids = [], [], {}, {}

    def matrix_id(w: NWCWeight):
        if id(w) not in ids:
            ids[id(w)] = len(matrices)
            matrices.append({"id": len(matrices), "out": w.out_features, "in": w.in_features, "block": w.block, "bytes": w.bytes,
                             "elem": ELEM_NAMES[w.elem], "layout": w.layout, "tensors": w.tensors()})
        return ids[id(w)]

    fused_lins = {id(g.lin) for _, g in fused_groups(model)}
    for path, mod in model.named_modules():
        if isinstance(mod, NWCLinear) and id(mod) not in fused_lins:
            modules.append({"path": path, "kind": "linear", "weight": matrix_id(mod.w), "bias": f"{path}.bias" if mod.bias is not None else None})
        elif isinstance(mod, NWCEmbedding):
            modules.append({"path": path, "kind": "embedding", "weight": matrix_id(mod.w), "padding_idx": mod.padding_idx})
    for parent, g in fused_groups(model):                           # their bias is not a registered parameter of the model
        key = f"nwc/fused/{parent}.bias" if g.lin.bias is not None else None
        if key: extra[key] = g.lin.bias.data
        modules.append({"path": parent, "kind": "fused", "weight": matrix_id(g.lin.w), "names": g.names, "sizes": g.sizes, "bias": key})
    return matrices, modules, extra


def save_pretrained(model: nn.Module, path: str, tokenizer=None, base_model: str = None):
    """Write a converted model as an NWC checkpoint.  Returns the nwc_config dict."""
    matrices, modules, extra = _describe_model(model)
    plain = dict(model.state_dict()); plain.update(extra)
    config = write_checkpoint(path, plain, matrices, modules, VERSION, base_model)
    model.config.save_pretrained(path)
    for part in (getattr(model, "generation_config", None), tokenizer):
        if part is not None: part.save_pretrained(path)
    return config


def _attach(model, path, module):
    parent, _, name = path.rpartition(".")
    setattr(model.get_submodule(parent) if parent else model, name, module)


def _skeleton(hf_config):
    """The model without any storage (meta device), built with plain torch."""
    from transformers import AutoModelForCausalLM
    with torch.device("meta"):
        try: return AutoModelForCausalLM.from_config(hf_config, dtype=torch.bfloat16)
        except TypeError: return AutoModelForCausalLM.from_config(hf_config, torch_dtype=torch.bfloat16)


def _fill(model, name, value):
    """Give the meta parameter / buffer `name` its stored value."""
    owner_path, _, leaf = name.rpartition(".")
    owner = model.get_submodule(owner_path) if owner_path else model
    if leaf in owner._parameters: owner._parameters[leaf] = nn.Parameter(value, requires_grad=False)
    elif leaf in owner._buffers: owner._buffers[leaf] = value
    else: raise KeyError(f"{name} is not a parameter or buffer of the model")


def _recompute_buffers(model, hf_config, device):
    """Buffers that checkpoints do not store (rotary inv_freq and the like) are still on the meta device after loading:
    re-create the modules that own them from the config and take their freshly computed buffers."""
    for path, mod in list(model.named_modules()):
        missing = [n for n, b in mod.named_buffers(recurse=False) if b.device.type == "meta"]
        if not missing: continue
        fresh = None
        for make in (lambda: type(mod)(config=hf_config, device="cpu"), lambda: type(mod)(config=hf_config), lambda: type(mod)(hf_config)):
            try: fresh = make(); break
            except TypeError: continue
        if fresh is None: raise RuntimeError(f"buffer {path}.{missing[0]} is not in the checkpoint and its module cannot be rebuilt from the config")
        computed = dict(fresh.named_buffers(recurse=False))
        for n in missing: mod._buffers[n] = computed[n].detach().clone().to(device)
        for attr, value in vars(fresh).items():                    # plain tensor attributes computed next to the buffers (e.g. original_inv_freq)
            mine = getattr(mod, attr, None)
            if isinstance(value, torch.Tensor) and isinstance(mine, torch.Tensor) and mine.device.type == "meta": setattr(mod, attr, value.to(device))


def load_pretrained(path: str, device="cuda", verbose=True):
    """Load an NWC checkpoint: the model on `device` with NWC modules in place; no bf16 originals are ever created."""
    from transformers import AutoConfig
    reader = CheckpointReader(path)
    hf_config = AutoConfig.from_pretrained(reader.path)
    model = _skeleton(hf_config)
    cache = {}

    def matrix(wid):                                                # a matrix shared by two modules is loaded once
        if wid not in cache: cache[wid] = NWCWeight.from_compressed(reader.matrix(wid, device), device, reader.records[wid]["block"])
        return cache[wid]

    taken = set()
    def bias_of(record):
        if not record.get("bias"): return None
        taken.add(record["bias"])
        return reader.tensor(record["bias"], device)

    for rec in reader.modules:
        if rec["kind"] == "embedding": _attach(model, rec["path"], NWCEmbedding(w=matrix(rec["weight"]), padding_idx=rec["padding_idx"]))
        elif rec["kind"] == "linear": _attach(model, rec["path"], NWCLinear(w=matrix(rec["weight"]), bias=bias_of(rec), device=device))
        elif rec["kind"] == "fused":
            lin = NWCLinear(w=matrix(rec["weight"]), bias=bias_of(rec), device=device)
            install_fused(model.get_submodule(rec["path"]) if rec["path"] else model, FusedProjection(lin, rec["names"], rec["sizes"]))
        else: raise RuntimeError(f"unknown module kind '{rec['kind']}' in the checkpoint")
    for name in reader.plain_names():
        if name not in taken: _fill(model, name, reader.tensor(name, device))
    _recompute_buffers(model, hf_config, device)
    for n, p in model.named_parameters():
        if p.device.type == "meta": raise RuntimeError(f"parameter {n} missing in the checkpoint")
    model.to(device).eval()
    if verbose:
        c = reader.config
        print(f"NWC: checkpoint loaded, {c['bytes_bf16'] / 1e9:.2f} GB BF16 -> {c['bytes_nwc'] / 1e9:.2f} GB (ratio {c['bytes_nwc'] / max(c['bytes_bf16'], 1):.4f})")
    return model


def export_bf16(path: str, out: str, device="cuda", verbose=True):
    """NWC checkpoint -> plain bf16 Transformers checkpoint at `out` (bit-identical weights).  Returns the bf16 bytes."""
    from safetensors.torch import save_file
    reader = CheckpointReader(path)
    tied = bool(reader.hf_config().get("tie_word_embeddings", False))
    users = {}
    for rec in reader.modules: users.setdefault(rec["weight"], []).append(rec)
    result, total, consumed = {}, 0, set()

    def take(name):
        consumed.add(name)
        return reader.tensor(name, "cpu")

    for wid, records in users.items():
        full = NWCWeight.from_compressed(reader.matrix(wid, device), device).dense().contiguous().cpu()
        total += 2 * full.numel()
        is_table = any(r["kind"] == "embedding" for r in records)
        for rec in records:
            if rec["kind"] == "embedding": result[f"{rec['path']}.weight"] = full
            elif rec["kind"] == "linear":
                if not (tied and is_table): result[f"{rec['path']}.weight"] = full          # a tied lm_head has no tensor of its own
                if rec.get("bias"): result[f"{rec['path']}.bias"] = take(rec["bias"])
            else:
                bias, at = (take(rec["bias"]) if rec.get("bias") else None), 0
                for name, size in zip(rec["names"], rec["sizes"]):
                    prefix = f"{rec['path']}.{name}" if rec["path"] else name
                    result[f"{prefix}.weight"] = full[at:at + size].clone()
                    if bias is not None: result[f"{prefix}.bias"] = bias[at:at + size].clone()
                    at += size
    for name in reader.plain_names():
        if name not in consumed: result[name] = reader.tensor(name, "cpu")
    os.makedirs(out, exist_ok=True)
    save_file(result, os.path.join(out, "model.safetensors"), metadata={"format": "pt"})
    for name in os.listdir(reader.path):
        src = os.path.join(reader.path, name)
        if name not in ("model.safetensors", "nwc_config.json") and os.path.isfile(src): shutil.copyfile(src, os.path.join(out, name))
    if verbose: print(f"NWC: exported {total / 1e9:.2f} GB of BF16 weights to {out}")
    return total
