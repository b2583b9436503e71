"""Tensor-parallel sharding on the CPU: two gloo ranks shard a small random decoder layer with nwc_b200.tp, run the
layer's linear algebra on their shards with the same collectives the GPU loop uses (all-reduce after the row-parallel
matrices, all-gather of the vocabulary-sharded logits) and must reproduce the unsharded result."""
import importlib.util
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_tp():
    # by path: the package import needs the CUDA library, this module is plain torch
    spec = importlib.util.spec_from_file_location("nwc_tp", os.path.join(ROOT, "nwc_b200", "tp.py"))
    m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
    return m


class Cfg:
    def __init__(self, **kw): self.__dict__.update(kw)
    @property
    def qkv_rows(self): return (self.n_q + 2 * self.n_kv) * self.head_dim


def make_cfg():
    import dataclasses
    @dataclasses.dataclass
    class C:
        name: str = "t"; layers: int = 1; hidden: int = 64; intermediate: int = 96; n_q: int = 4; n_kv: int = 2; head_dim: int = 16; vocab: int = 128
        tied: bool = False; qk_norm: bool = False
        @property
        def qkv_rows(self): return (self.n_q + 2 * self.n_kv) * self.head_dim
    return C()


def layer_math(cfg, mats, x, attn_fn):
    """One layer without norms/attention details: qkv -> (attention replaced by a per-head mixing) -> o -> gate_up -> down."""
    qkv = mats["qkv"] @ x
    a = attn_fn(qkv, cfg)
    o = mats["o"] @ a
    gu = mats["gate_up"] @ (x + o)
    I = gu.numel() // 2
    act = torch.nn.functional.silu(gu[:I]) * gu[I:]
    return x + o, mats["down"] @ act


def attn_like(qkv, cfg):
    # every query head takes the value vector of its kv head, scaled by <q, k>: enough to catch head mis-assignment
    hd = cfg.head_dim
    q = qkv[: cfg.n_q * hd].view(cfg.n_q, hd); k = qkv[cfg.n_q * hd: (cfg.n_q + cfg.n_kv) * hd].view(cfg.n_kv, hd)
    v = qkv[(cfg.n_q + cfg.n_kv) * hd:].view(cfg.n_kv, hd)
    rep = cfg.n_q // cfg.n_kv
    return torch.cat([(q[h] * k[h // rep]).sum() * v[h // rep] for h in range(cfg.n_q)])


def worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = load_tp()
    cfg = make_cfg()
    g = torch.Generator().manual_seed(0)
    full = {k: torch.randn(*tp.full_shape(k, cfg), generator=g, dtype=torch.float64) * 0.1 for k in ("qkv", "o", "gate_up", "down", "lm_head")}
    x = torch.randn(cfg.hidden, generator=g, dtype=torch.float64)
    lc = tp.local_config(cfg, world)
    mine = {k: tp.shard(k, full[k], cfg, rank, world) for k in full}
    assert mine["qkv"].shape == (lc.qkv_rows, cfg.hidden) and mine["o"].shape == (cfg.hidden, lc.n_q * cfg.head_dim)
    assert mine["gate_up"].shape == (2 * lc.intermediate, cfg.hidden) and mine["down"].shape == (cfg.hidden, lc.intermediate)
    qkv = mine["qkv"] @ x
    a = attn_like(qkv, lc)
    o = mine["o"] @ a; dist.all_reduce(o)
    gu = mine["gate_up"] @ (x + o)
    act = torch.nn.functional.silu(gu[: lc.intermediate]) * gu[lc.intermediate:]
    d = mine["down"] @ act; dist.all_reduce(d)
    logits_local = mine["lm_head"] @ (x + o + d)
    logits = torch.empty(cfg.vocab, dtype=torch.float64); dist.all_gather_into_tensor(logits, logits_local)
    h_ref, d_ref = layer_math(cfg, full, x, attn_like)
    ok = torch.allclose(x + o, h_ref, atol=1e-12) and torch.allclose(d, d_ref, atol=1e-12) and torch.allclose(logits, full["lm_head"] @ (h_ref + d_ref), atol=1e-12)
    out[rank] = bool(ok) and int(logits.argmax()) == int((full["lm_head"] @ (h_ref + d_ref)).argmax())
    dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_unsharded_layer():
    mgr = mp.Manager(); out = mgr.dict()
    mp.spawn(worker, args=(2, 29541, out), nprocs=2, join=True)
    assert out[0] and out[1]


def test_shards_tile_the_full_matrices_and_bad_degrees_are_rejected():
    tp = load_tp(); cfg = make_cfg()
    full = {k: torch.arange(tp.full_shape(k, cfg)[0] * tp.full_shape(k, cfg)[1], dtype=torch.float32).view(*tp.full_shape(k, cfg)) for k in ("qkv", "o", "gate_up", "down", "lm_head")}
    for world in (1, 2):
        for k, f in full.items():
            parts = [tp.shard(k, f, cfg, r, world) for r in range(world)]
            assert sum(p.numel() for p in parts) == f.numel()
            assert torch.equal(torch.cat([p.flatten() for p in parts]).sort().values, f.flatten().sort().values)
    with pytest.raises(ValueError): tp.local_config(cfg, 3)
    with pytest.raises(ValueError): tp.local_config(cfg, 4)          # 2 kv heads cannot be split four ways
