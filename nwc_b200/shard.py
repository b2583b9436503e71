"""Per-rank shard files of an NWC checkpoint, so that a tensor-parallel engine loads its part without re-packing.

    python -m nwc_b200.shard CHECKPOINT OUT_DIR --world 8 [--device cuda]

writes OUT_DIR/rank_<r>/ for r = 0 .. world-1, each holding
  shard.json          {nwc_shard: 1, tp_rank, tp_world, config: the FULL decoder configuration, lm_head_is_embed,
                       matrices: {name: {out, in, layout, elem}}}
  model.safetensors   per matrix "m/<name>/{data,bases,hdr,lut,low[,scale]}" - this rank's blocks in the library's own
                      format (v9 / v10 / v11 by layout), cut by the block re-pack of nwc_b200/repack.py exactly as
                      DecoderWeights.from_checkpoint cuts them at load time - and the norm vectors "v/<name>".
Matrix names: embed, lm_head, L<i>.qkv, L<i>.o, L<i>.gate_up, L<i>.down; vectors: final_norm, L<i>.in_norm, L<i>.post_norm,
L<i>.q_norm, L<i>.k_norm.  `DecodeEngine.from_pretrained(OUT_DIR, tp_group=...)` recognises the directory (shards.json at its
top) and every rank reads only its own folder.

The reference keeps whole matrices per module and has no tensor-parallel loader (nwc/checkpoint.py:83-128 loads every
module onto one device); this file format exists only on this side of the drop-in boundary.
"""
import argparse
import dataclasses
import json
import os
import sys

import torch

FORMAT = 1
MATRIX_KINDS = ("qkv", "o", "gate_up", "down")
VECTOR_KINDS = ("in_norm", "post_norm", "q_norm", "k_norm")


def _named_matrices(w):
    out = {"embed": w.embed}
    if w.lm_head is not w.embed: out["lm_head"] = w.lm_head
    for i, l in enumerate(w.layers):
        for k in MATRIX_KINDS: out[f"L{i}.{k}"] = l[k]
    return out


def save_shard(weights, path):
    """Write one rank's matrices and vectors (a DecoderWeights) to `path`."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    tensors, described = {}, {}
    for name, m in _named_matrices(weights).items():
        for tname, t in m.tensors().items(): tensors[f"m/{name}/{tname}"] = t.detach().cpu().contiguous()
        c = m.compressed()
        described[name] = {"out": c.M, "in": c.K, "layout": c.layout, "elem": c.elem}
    tensors["v/final_norm"] = weights.final_norm.detach().cpu().contiguous()
    for i, l in enumerate(weights.layers):
        for k in VECTOR_KINDS:
            if l.get(k) is not None: tensors[f"v/L{i}.{k}"] = l[k].detach().cpu().contiguous()
    save_file(tensors, os.path.join(path, "model.safetensors"), metadata={"format": "pt", "nwc_shard": str(FORMAT)})
    meta = {"nwc_shard": FORMAT, "tp_rank": weights.tp_rank, "tp_world": weights.tp_world, "config": dataclasses.asdict(weights.full_cfg),
            "lm_head_is_embed": weights.lm_head is weights.embed, "matrices": described}
    with open(os.path.join(path, "shard.json"), "w", encoding="utf-8") as f: json.dump(meta, f, indent=1)
    return meta


def load_shard(path, device="cuda"):
    """The DecoderWeights that save_shard wrote to `path`, tensors read straight onto `device`."""
    from safetensors import safe_open
    from . import tp as TP
    from .decode import DecoderConfig, DecoderWeights
    from .repack import Compressed
    from .weight import NWCWeight
    with open(os.path.join(path, "shard.json"), encoding="utf-8") as f: meta = json.load(f)
    if meta.get("nwc_shard") != FORMAT: raise RuntimeError(f"{path}: shard format {meta.get('nwc_shard')}, this library reads {FORMAT}")
    full = DecoderConfig(**meta["config"])
    self = DecoderWeights.__new__(DecoderWeights)
    self.full_cfg, self.tp_rank, self.tp_world = full, int(meta["tp_rank"]), int(meta["tp_world"])
    self.cfg = TP.local_config(full, self.tp_world) if self.tp_world > 1 else full
    f = safe_open(os.path.join(path, "model.safetensors"), framework="pt", device=str(device))
    keys = set(f.keys())

    def matrix(name):
        d = meta["matrices"][name]
        t = {n: f.get_tensor(f"m/{name}/{n}") for n in ("data", "bases", "hdr", "lut", "low")}
        scale = f.get_tensor(f"m/{name}/scale") if f"m/{name}/scale" in keys else None
        return NWCWeight.from_compressed(Compressed(d["out"], d["in"], int(d["layout"]), d["elem"], t["data"], t["bases"], t["hdr"], t["lut"], t["low"], scale), device)

    vec = lambda name: f.get_tensor(f"v/{name}").to(torch.bfloat16).contiguous() if f"v/{name}" in keys else None
    self.embed = matrix("embed")
    self.lm_head = self.embed if meta["lm_head_is_embed"] else matrix("lm_head")
    self.layers = []
    for i in range(full.layers):
        layer = {k: matrix(f"L{i}.{k}") for k in MATRIX_KINDS}
        layer.update({k: vec(f"L{i}.{k}") for k in VECTOR_KINDS})
        self.layers.append(layer)
    self.final_norm = vec("final_norm")
    return self


def is_sharded(path):
    return os.path.isdir(path) and os.path.exists(os.path.join(path, "shards.json"))


def rank_dir(path, rank, world):
    """The folder of rank `rank`; the directory must have been written for exactly `world` ranks."""
    with open(os.path.join(path, "shards.json"), encoding="utf-8") as f: top = json.load(f)
    if int(top["tp_world"]) != int(world): raise ValueError(f"{path} holds shards for {top['tp_world']} ranks, the group has {world}")
    return os.path.join(path, f"rank_{rank}")


def shard_checkpoint(src, out, world, device="cuda", log=print):
    """Cut checkpoint `src` into `world` per-rank folders under `out` (one rank in device memory at a time)."""
    from .decode import DecoderWeights
    os.makedirs(out, exist_ok=True)
    total = 0
    for r in range(world):
        w = DecoderWeights.from_checkpoint(src, device, r, world)
        meta = save_shard(w, os.path.join(out, f"rank_{r}"))
        size = os.path.getsize(os.path.join(out, f"rank_{r}", "model.safetensors"))
        total += size
        log(f"rank {r}/{world}: {len(meta['matrices'])} matrices, {size / 1e6:.1f} MB")
        del w
        if torch.cuda.is_available(): torch.cuda.empty_cache()
    with open(os.path.join(out, "shards.json"), "w", encoding="utf-8") as f:
        json.dump({"nwc_shards": FORMAT, "tp_world": world, "source": str(src), "bytes": total}, f, indent=1)
    return total


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m nwc_b200.shard", description="cut an NWC checkpoint into per-rank tensor-parallel shards")
    ap.add_argument("checkpoint", help="NWC checkpoint: a local directory or a Hugging Face repo id")
    ap.add_argument("out", help="output directory (rank_<r>/ folders and shards.json)")
    ap.add_argument("--world", type=int, required=True, help="number of tensor-parallel ranks (2, 4 or 8)")
    ap.add_argument("--device", default="cuda", help="GPU that re-packs (default cuda)")
    a = ap.parse_args(argv)
    shard_checkpoint(a.checkpoint, a.out, a.world, a.device)
    return 0


if __name__ == "__main__":
    sys.exit(main())
