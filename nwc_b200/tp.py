"""Tensor-parallel sharding of a decoder's matrices (the reference is single-GPU; this is the layout the decode loop
uses on 2, 4 and 8 GPUs).

Column-parallel (output rows split): the fused q/k/v projection by attention heads, the fused gate/up projection by
intermediate channels, the lm_head by vocabulary rows.  Row-parallel (input columns split): o_proj by heads, down_proj
by intermediate channels; their partial outputs are summed over the ranks with one all-reduce each per layer.
Norm vectors, the embedding table and the residual stream are replicated.  Everything here is plain index arithmetic
on torch tensors, so it runs (and is tested) on the CPU.
"""
from dataclasses import replace

import torch


def check_divisible(cfg, world):
    for what, n in (("query heads", cfg.n_q), ("kv heads", cfg.n_kv), ("intermediate size", cfg.intermediate), ("vocabulary", cfg.vocab)):
        if n % world: raise ValueError(f"{what} ({n}) is not divisible by the tensor-parallel degree {world}")


def local_config(cfg, world):
    """The per-rank view: heads, intermediate channels and vocabulary rows divided by `world`; hidden size unchanged."""
    check_divisible(cfg, world)
    return replace(cfg, n_q=cfg.n_q // world, n_kv=cfg.n_kv // world, intermediate=cfg.intermediate // world, vocab=cfg.vocab // world)


def shard(kind, full, cfg, rank, world):
    """Rank `rank`'s part of the full matrix `full` of kind qkv | o | gate_up | down | lm_head (cfg = full config)."""
    hd, nq, nkv, I = cfg.head_dim, cfg.n_q // world, cfg.n_kv // world, cfg.intermediate // world
    if kind == "qkv":
        q0, k0, v0 = 0, cfg.n_q * hd, (cfg.n_q + cfg.n_kv) * hd
        return torch.cat([full[q0 + rank * nq * hd: q0 + (rank + 1) * nq * hd], full[k0 + rank * nkv * hd: k0 + (rank + 1) * nkv * hd],
                          full[v0 + rank * nkv * hd: v0 + (rank + 1) * nkv * hd]], 0).contiguous()
    if kind == "o": return full[:, rank * nq * hd: (rank + 1) * nq * hd].contiguous()
    if kind == "gate_up": return torch.cat([full[rank * I: (rank + 1) * I], full[cfg.intermediate + rank * I: cfg.intermediate + (rank + 1) * I]], 0).contiguous()
    if kind == "down": return full[:, rank * I: (rank + 1) * I].contiguous()
    if kind == "lm_head":
        V = cfg.vocab // world
        return full[rank * V: (rank + 1) * V].contiguous()
    raise ValueError(kind)


def full_shape(kind, cfg):
    return {"qkv": (cfg.qkv_rows, cfg.hidden), "o": (cfg.hidden, cfg.n_q * cfg.head_dim), "gate_up": (2 * cfg.intermediate, cfg.hidden),
            "down": (cfg.hidden, cfg.intermediate), "lm_head": (cfg.vocab, cfg.hidden), "embed": (cfg.vocab, cfg.hidden)}[kind]
