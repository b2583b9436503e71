"""Compressed checkpoints: the reference's on-disk format, read and written (reference: nwc/checkpoint.py).

A checkpoint is a directory:
  config.json, generation_config.json, tokenizer files    Hugging Face files, untouched
  nwc_config.json    {nwc_checkpoint: 1, library_version: 9|10|11, base_model, weights: [{id, out, in, block, bytes,
                     elem?, layout?}], modules: [{path, kind: linear|embedding|fused, weight, bias | padding_idx |
                     names, sizes}], bytes_nwc, bytes_bf16}; missing elem / layout mean bf16 / 0
  model.safetensors  the remaining parameters plus, per matrix, "nwc/<id>/{data,bases,hdr,lut,low[,scale]}"
Versions 9, 10 and 11 (layouts 0, 1, 2) all load.  The model skeleton is built on the meta device with plain torch,
so no weights other than the compressed ones ever exist in host or device memory.
"""
import json
import os
import shutil

import torch
import torch.nn as nn
from safetensors.torch import load_file, save_file

from ._lib import VERSION
from .modules import NWCEmbedding, NWCLinear, _FusedHead
from .weight import NWCWeight

FORMAT = 1
COMPATIBLE = {9, 10, 11}
TENSOR_NAMES = ("data", "bases", "hdr", "lut", "low")


def _parent(path): return path.rsplit(".", 1)[0] if "." in path else ""


def _collect(model):
    """Unique NWCWeight objects and the modules that use them."""
    index, weights, modules, groups = {}, [], [], set()

    def key(w):
        if id(w) not in index:
            index[id(w)] = len(weights)
            weights.append({"id": len(weights), "out": w.out_features, "in": w.in_features, "block": w.block, "bytes": w.bytes,
                            "elem": "fp8" if w.elem else "bf16", "layout": w.layout, "w": w})
        return index[id(w)]

    for path, m in model.named_modules():
        if isinstance(m, NWCLinear):
            modules.append({"path": path, "kind": "linear", "weight": key(m.w), "bias": f"{path}.bias" if m.bias is not None else None})
        elif isinstance(m, NWCEmbedding):
            modules.append({"path": path, "kind": "embedding", "weight": key(m.w), "padding_idx": m.padding_idx})
        elif isinstance(m, _FusedHead) and id(m.g) not in groups:
            groups.add(id(m.g))
            lin, parent = m.g["lin"], _parent(path)
            modules.append({"path": parent, "kind": "fused", "weight": key(lin.w), "names": m.g["names"], "sizes": m.g["sizes"],
                            "bias": f"nwc/fused/{parent}.bias" if lin.bias is not None else None})
    return weights, modules


def save_pretrained(model: nn.Module, path: str, tokenizer=None, base_model: str = None):
    """Write a converted model as an NWC checkpoint.  Returns the nwc_config dict."""
    os.makedirs(path, exist_ok=True)
    weights, modules = _collect(model)
    tensors = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
    for e in weights:
        for name, t in e["w"].tensors().items(): tensors[f"nwc/{e['id']}/{name}"] = t.detach().cpu().contiguous()
    for m in modules:                   # biases of fused groups are not registered parameters of the model
        if m["kind"] != "fused" or not m["bias"]: continue
        for p, mod in model.named_modules():
            if isinstance(mod, _FusedHead) and _parent(p) == m["path"]:
                tensors[m["bias"]] = mod.g["lin"].bias.detach().cpu().contiguous(); break
    save_file(tensors, os.path.join(path, "model.safetensors"), metadata={"format": "pt", "nwc": str(FORMAT)})
    config = {"nwc_checkpoint": FORMAT, "library_version": VERSION,
              "base_model": base_model, "weights": [{k: v for k, v in e.items() if k != "w"} for e in weights], "modules": modules,
              "bytes_nwc": sum(e["bytes"] for e in weights), "bytes_bf16": sum(2 * e["out"] * e["in"] for e in weights)}
    with open(os.path.join(path, "nwc_config.json"), "w", encoding="utf-8") as f: json.dump(config, f, indent=1)
    model.config.save_pretrained(path)
    gc = getattr(model, "generation_config", None)
    if gc is not None: gc.save_pretrained(path)
    if tokenizer is not None: tokenizer.save_pretrained(path)
    return config


def _set(model, path, module):
    parent, _, name = path.rpartition(".")
    setattr(model.get_submodule(parent) if parent else model, name, module)


def resolve(path: str) -> str:
    """A local directory as is; anything else is treated as a Hugging Face repo id and fetched into the HF cache."""
    if os.path.isdir(path): return path
    if os.path.exists(path): raise FileNotFoundError(f"{path} is a file, an NWC checkpoint is a directory")
    try:
        from huggingface_hub import snapshot_download
    except ImportError:
        raise FileNotFoundError(f"{path} is not a directory, and huggingface_hub is not installed")
    return snapshot_download(path)


def _read_config(path):
    cfg_path = os.path.join(path, "nwc_config.json")
    if not os.path.exists(cfg_path):
        raise FileNotFoundError(f"{path} is not an NWC checkpoint (no nwc_config.json)")
    with open(cfg_path, encoding="utf-8") as f: config = json.load(f)
    if config.get("library_version") not in COMPATIBLE:
        raise RuntimeError(f"checkpoint is format version {config.get('library_version')}, this library reads {sorted(COMPATIBLE)}")
    return config


def _weight_from(tensors, e, device):
    t = {n: tensors.pop(f"nwc/{e['id']}/{n}") for n in TENSOR_NAMES}
    return NWCWeight.from_tensors(e["out"], e["in"], e["block"], t["data"], t["bases"], t["hdr"], t["lut"], t["low"], device,
                                  elem=e.get("elem", "bf16"), scale=tensors.pop(f"nwc/{e['id']}/scale", None), layout=e.get("layout", 0))


def _materialize(model, name, value, device):
    """Replace the meta parameter / buffer `name` by `value` on `device`."""
    parent, _, leaf = name.rpartition(".")
    mod = model.get_submodule(parent) if parent else model
    value = value.to(device)
    if leaf in mod._parameters: mod._parameters[leaf] = nn.Parameter(value, requires_grad=False)
    elif leaf in mod._buffers: mod._buffers[leaf] = value
    else: raise KeyError(f"{name} is not a parameter or buffer of the model")


def _rebuild_meta_buffers(model, hf_config, device):
    """Buffers that checkpoints do not store (rotary inv_freq and the like) are still on the meta device after loading:
    re-create the modules that own them from the config and take their freshly computed buffers."""
    for path, mod in list(model.named_modules()):
        names = [n for n, b in mod.named_buffers(recurse=False) if b.device.type == "meta"]
        if not names: continue
        fresh = None
        for build in (lambda: type(mod)(config=hf_config, device="cpu"), lambda: type(mod)(config=hf_config), lambda: type(mod)(hf_config)):
            try:
                fresh = build(); break
            except TypeError:
                continue
        if fresh is None: raise RuntimeError(f"buffer {path}.{names[0]} is not in the checkpoint and its module cannot be rebuilt from the config")
        for n in names: mod._buffers[n] = dict(fresh.named_buffers(recurse=False))[n].detach().clone().to(device)
        for k, v in vars(fresh).items():             # plain attributes computed next to the buffers (e.g. original_inv_freq)
            if isinstance(v, torch.Tensor) and isinstance(getattr(mod, k, None), torch.Tensor) and getattr(mod, k).device.type == "meta": setattr(mod, k, v.to(device))


def load_pretrained(path: str, device="cuda", verbose=True):
    """Load an NWC checkpoint: the model on `device` with NWC modules in place; no bf16 originals are ever created."""
    from transformers import AutoConfig, AutoModelForCausalLM
    path = resolve(path)
    config = _read_config(path)
    hf_config = AutoConfig.from_pretrained(path)
    with torch.device("meta"):
        try: model = AutoModelForCausalLM.from_config(hf_config, dtype=torch.bfloat16)
        except TypeError: model = AutoModelForCausalLM.from_config(hf_config, torch_dtype=torch.bfloat16)
    tensors = load_file(os.path.join(path, "model.safetensors"))
    weights = {e["id"]: _weight_from(tensors, e, device) for e in config["weights"]}
    for m in config["modules"]:
        w = weights[m["weight"]]
        if m["kind"] == "linear":
            _set(model, m["path"], NWCLinear(w=w, bias=tensors.pop(m["bias"], None) if m["bias"] else None, device=device))
        elif m["kind"] == "embedding":
            _set(model, m["path"], NWCEmbedding(w=w, padding_idx=m["padding_idx"]))
        else:
            lin = NWCLinear(w=w, bias=tensors.pop(m["bias"], None) if m["bias"] else None, device=device)
            shared = {"lin": lin, "y": None, "x_id": None, "names": m["names"], "sizes": m["sizes"]}
            start = 0
            for i, (name, size) in enumerate(zip(m["names"], m["sizes"])):
                _set(model, f"{m['path']}.{name}" if m["path"] else name, _FusedHead(shared, i, start, start + size)); start += size
    for k, v in tensors.items(): _materialize(model, k, v, device)
    _rebuild_meta_buffers(model, hf_config, device)
    for n, p in model.named_parameters():
        if p.device.type == "meta": raise RuntimeError(f"parameter {n} missing in the checkpoint")
    model.to(device).eval()
    if verbose:
        print(f"NWC: checkpoint loaded, {config['bytes_bf16'] / 1e9:.2f} GB BF16 -> {config['bytes_nwc'] / 1e9:.2f} GB "
              f"(ratio {config['bytes_nwc'] / max(config['bytes_bf16'], 1):.4f})")
    return model


def export_bf16(path: str, out: str, device="cuda", verbose=True):
    """NWC checkpoint -> plain bf16 Transformers checkpoint at `out` (bit-identical weights).  Returns the bf16 bytes."""
    path = resolve(path)
    config = _read_config(path)
    with open(os.path.join(path, "config.json"), encoding="utf-8") as f: tied = json.load(f).get("tie_word_embeddings", False)
    tensors = load_file(os.path.join(path, "model.safetensors"))
    embedding_ids = {m["weight"] for m in config["modules"] if m["kind"] == "embedding"}
    result, total = {}, 0
    for e in config["weights"]:
        w = _weight_from(tensors, e, device)
        full = w.dequant()
        if w.scale is not None: full = (full.float() * w.scale[:, None]).to(torch.bfloat16)
        full = full.contiguous().cpu(); del w
        total += full.numel() * 2
        for m in config["modules"]:
            if m["weight"] != e["id"]: continue
            if m["kind"] == "embedding": result[f"{m['path']}.weight"] = full
            elif m["kind"] == "linear":
                if not (tied and e["id"] in embedding_ids): result[f"{m['path']}.weight"] = full
                if m["bias"]: result[f"{m['path']}.bias"] = tensors.pop(m["bias"])
            else:
                bias = tensors.pop(m["bias"]) if m["bias"] else None
                start = 0
                for name, size in zip(m["names"], m["sizes"]):
                    key = f"{m['path']}.{name}" if m["path"] else name
                    result[f"{key}.weight"] = full[start:start + size].clone()
                    if bias is not None: result[f"{key}.bias"] = bias[start:start + size].clone()
                    start += size
    result.update(tensors)
    os.makedirs(out, exist_ok=True)
    save_file(result, os.path.join(out, "model.safetensors"), metadata={"format": "pt"})
    for name in os.listdir(path):
        if name not in ("model.safetensors", "nwc_config.json") and os.path.isfile(os.path.join(path, name)):
            shutil.copyfile(os.path.join(path, name), os.path.join(out, name))
    if verbose: print(f"NWC: exported {total / 1e9:.2f} GB of BF16 weights to {out}")
    return total
