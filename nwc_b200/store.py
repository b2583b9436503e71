"""The on-disk schema of compressed checkpoints, read and written one tensor at a time.

A checkpoint is a directory (reference: nwc/checkpoint.py:14-16, 43-64 for the schema):
  config.json, generation_config.json, tokenizer files    Hugging Face files, untouched
  nwc_config.json    {nwc_checkpoint: 1, library_version: 9|10|11, base_model, weights: [{id, out, in, block, bytes,
                     elem?, layout?}], modules: [{path, kind: linear|embedding|fused, weight, bias | padding_idx |
                     names, sizes}], bytes_nwc, bytes_bf16}; missing elem / layout mean bf16 / 0
  model.safetensors  the remaining parameters plus, per matrix, "nwc/<id>/{data,bases,hdr,lut,low[,scale]}"
Versions 9, 10 and 11 (layouts 0, 1, 2) all load.  `CheckpointReader` opens the tensor file lazily (safetensors'
`safe_open`) and hands out one matrix at a time straight onto the target device, so loading a 100 GB checkpoint never
stages it in host memory; `write_checkpoint` is the writer `save_pretrained` uses.
"""
import json
import os

import torch

from .repack import Compressed

FORMAT = 1
COMPATIBLE = {9, 10, 11}
MATRIX_TENSORS = ("data", "bases", "hdr", "lut", "low")


def resolve(path: str) -> str:
    """A local directory as is; anything else is treated as a Hugging Face repo id and fetched into the HF cache."""
    if os.path.isdir(path): return path
    if os.path.exists(path): raise FileNotFoundError(f"{path} is a file, an NWC checkpoint is a directory")
    try:
        from huggingface_hub import snapshot_download
    except ImportError:
        raise FileNotFoundError(f"{path} is not a directory, and huggingface_hub is not installed")
    return snapshot_download(path)


class CheckpointReader:
    """nwc_config.json plus lazy access to the tensors of model.safetensors."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self.path = resolve(path)
        cfg_path = os.path.join(self.path, "nwc_config.json")
        if not os.path.exists(cfg_path): raise FileNotFoundError(f"{self.path} is not an NWC checkpoint (no nwc_config.json)")
        with open(cfg_path, encoding="utf-8") as f: self.config = json.load(f)
        version = self.config.get("library_version")
        if version not in COMPATIBLE: raise RuntimeError(f"checkpoint is format version {version}, this library reads {sorted(COMPATIBLE)}")
        self._open = lambda device: safe_open(os.path.join(self.path, "model.safetensors"), framework="pt", device=device)
        self._files = {}
        self.records = {e["id"]: e for e in self.config["weights"]}
        self.modules = self.config["modules"]

    def _file(self, device):
        key = str(device)
        if key not in self._files: self._files[key] = self._open(key)
        return self._files[key]

    def names(self):
        return list(self._file("cpu").keys())

    def plain_names(self):
        """Tensors that are not part of a compressed matrix (norms, biases, buffers)."""
        return [k for k in self.names() if not k.startswith("nwc/") or k.startswith("nwc/fused/")]

    def has(self, name): return name in self._file("cpu").keys()

    def tensor(self, name, device="cpu"):
        return self._file(device).get_tensor(name)

    def hf_config(self) -> dict:
        with open(os.path.join(self.path, "config.json"), encoding="utf-8") as f: return json.load(f)

    def matrix(self, wid: int, device="cpu") -> Compressed:
        """The stored tensors of compressed matrix `wid`, read directly onto `device`."""
        e = self.records[wid]
        f = self._file(device)
        t = {n: f.get_tensor(f"nwc/{wid}/{n}") for n in MATRIX_TENSORS}
        scale = f.get_tensor(f"nwc/{wid}/scale") if f"nwc/{wid}/scale" in f.keys() else None
        return Compressed(e["out"], e["in"], int(e.get("layout", 0)), e.get("elem", "bf16"), t["data"], t["bases"], t["hdr"], t["lut"], t["low"], scale)


def write_checkpoint(path: str, plain: dict, matrices: list, modules: list, library_version: int, base_model=None) -> dict:
    """matrices: [{"id", "out", "in", "block", "bytes", "elem", "layout", "tensors": {name: tensor}}]; plain: the other
    tensors by name.  Returns the nwc_config dict it wrote."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    tensors = {k: v.detach().cpu().contiguous() for k, v in plain.items()}
    for m in matrices:
        for name, t in m["tensors"].items(): tensors[f"nwc/{m['id']}/{name}"] = t.detach().cpu().contiguous()
    save_file(tensors, os.path.join(path, "model.safetensors"), metadata={"format": "pt", "nwc": str(FORMAT)})
    config = {"nwc_checkpoint": FORMAT, "library_version": library_version, "base_model": base_model,
              "weights": [{k: v for k, v in m.items() if k != "tensors"} for m in matrices], "modules": modules,
              "bytes_nwc": sum(m["bytes"] for m in matrices), "bytes_bf16": sum(2 * m["out"] * m["in"] for m in matrices)}
    with open(os.path.join(path, "nwc_config.json"), "w", encoding="utf-8") as f: json.dump(config, f, indent=1)
    return config
