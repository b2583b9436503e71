"""Batch-1 greedy decode loop over compressed weights, replayed as one CUDA graph per token.

Replaces the reference's graph-captured Hugging Face forward (reference: scripts/graph_decode.py:37-70,
nwc/demo.py:71-89) with a fixed chain of this library's kernels: compressed embedding gather, then per layer
add+RMSNorm -> fused qkv matvec -> q/k-norm + rotary + cache append + attention -> o matvec -> add+RMSNorm ->
fused gate/up matvec -> SwiGLU -> down matvec, then final norm -> lm_head matvec -> argmax.  Token, position and step
counter live in device memory, so the captured graph is replayed unchanged for every token.

Architectures: Qwen3 (per-head q/k RMSNorm, tied or untied embeddings) and Llama-3 style (no q/k norm) decoders.
"""
import ctypes

import torch

from . import _lib as L
from . import tp as TP
from .presets import PRESETS, DecoderConfig
from .weight import NWCWeight


def synthetic_matrix(rows, cols, seed, device="cuda"):
    """W[i, j] = r_i * 0.02 * z_ij with r_i log-normal(0, 0.3), z standard normal, seeded per tensor; bf16."""
    g = torch.Generator(device=device).manual_seed(seed)
    r = torch.exp(0.3 * torch.randn(rows, 1, generator=g, device=device))
    return (r * 0.02 * torch.randn(rows, cols, generator=g, device=device)).to(torch.bfloat16)


class DecoderWeights:
    """Compressed matrices and norm vectors of a decoder.  `source(name, rows, cols)` returns the bf16 matrix to
    compress; `vector(name, n)` a bf16 norm weight."""

    def __init__(self, cfg: DecoderConfig, source, vector, layout=0, elem="bf16", device="cuda", tp_rank=0, tp_world=1):
        """cfg is the FULL model; with tp_world > 1 `source` still returns full matrices and this rank keeps its shard."""
        self.full_cfg, self.tp_rank, self.tp_world = cfg, tp_rank, tp_world
        self.cfg = lc = TP.local_config(cfg, tp_world) if tp_world > 1 else cfg

        def mk(name, kind, e=elem):
            full = source(name, *TP.full_shape(kind, cfg))
            part = TP.shard(kind, full, cfg, tp_rank, tp_world) if tp_world > 1 and kind != "embed" else full
            return NWCWeight(part, device, elem=e, layout=layout)

        if tp_world == 1:
            self.embed = mk("embed", "embed", "bf16" if not cfg.tied else elem)
            self.lm_head = self.embed if cfg.tied else mk("lm_head", "lm_head")
        else:                       # the lookup needs every row, the logits only this rank's rows
            self.embed = mk("embed", "embed", "bf16")
            self.lm_head = mk("embed" if cfg.tied else "lm_head", "lm_head")
        self.layers = []
        for i in range(cfg.layers):
            self.layers.append({
                "in_norm": vector(f"l{i}.in_norm", cfg.hidden), "post_norm": vector(f"l{i}.post_norm", cfg.hidden),
                "q_norm": vector(f"l{i}.q_norm", cfg.head_dim) if cfg.qk_norm else None,
                "k_norm": vector(f"l{i}.k_norm", cfg.head_dim) if cfg.qk_norm else None,
                "qkv": mk(f"l{i}.qkv", "qkv"), "o": mk(f"l{i}.o", "o"), "gate_up": mk(f"l{i}.gate_up", "gate_up"), "down": mk(f"l{i}.down", "down")})
        self.final_norm = vector("final_norm", cfg.hidden)
        assert lc.qkv_rows == self.layers[0]["qkv"].out_features

    @classmethod
    def synthetic(cls, cfg, layout=0, elem="bf16", device="cuda", seed=0, tp_rank=0, tp_world=1):
        """Seeded random-init model; every tensor has its own seed (derived from its name), so all ranks of a
        tensor-parallel group generate the same full matrices and keep different shards."""
        names = {}
        def source(name, r, c):
            if name not in names: names[name] = len(names) + 1
            return synthetic_matrix(r, c, seed * 100003 + names[name], device)
        return cls(cfg, source, lambda name, n: torch.ones(n, dtype=torch.bfloat16, device=device), layout, elem, device, tp_rank, tp_world)

    @classmethod
    def from_checkpoint(cls, path, device="cuda", tp_rank=0, tp_world=1, relayout=None):
        """The compressed matrices of an NWC checkpoint (formats v9 / v10 / v11, as written by save_pretrained of this
        library or of the reference) mapped onto the decode loop, without ever creating bf16 weights: the `fused` records
        of q/k/v and gate/up, the `linear` records of o, down and lm_head and the `embedding` record are taken as stored.
        With tp_world > 1 every matrix is cut into this rank's shard by re-packing its blocks (nwc_b200/repack.py).  Only
        checkpoints whose projections were not fused, or whose head sizes do not fall on block boundaries, are
        dequantised and re-encoded instead.  relayout = 0 | 1 | 2 re-encodes every matrix stored in another layout into
        that one while loading (lossless: the decoded weights stay bit-identical; the GPU encoder does a 4B model in a
        fraction of a second) - layout 2 is the fastest layout on B200, so a v9 / v10 checkpoint can be served at
        layout-2 speed for about 10 % more memory.  Architectures: Qwen3 and Llama style decoders without biases."""
        from . import repack as R
        from .store import CheckpointReader
        rd = CheckpointReader(path)
        hf = rd.hf_config()
        kind = hf.get("model_type", "")
        if kind not in ("qwen3", "llama"): raise ValueError(f"the decode loop knows qwen3 and llama decoders, not '{kind}'")
        heads = hf["num_attention_heads"]
        cfg = DecoderConfig(hf.get("_name_or_path") or kind, hf["num_hidden_layers"], hf["hidden_size"], hf["intermediate_size"], heads,
                            hf.get("num_key_value_heads", heads), hf.get("head_dim") or hf["hidden_size"] // heads, hf["vocab_size"],
                            bool(hf.get("tie_word_embeddings", False)), kind == "qwen3",
                            rope_theta=float((hf.get("rope_parameters") or {}).get("rope_theta", hf.get("rope_theta", 1e4))), eps=float(hf.get("rms_norm_eps", 1e-6)))
        self = cls.__new__(cls)
        self.full_cfg, self.tp_rank, self.tp_world = cfg, tp_rank, tp_world
        self.cfg = TP.local_config(cfg, tp_world) if tp_world > 1 else cfg
        by_path = {m["path"]: m for m in rd.modules}
        for m in rd.modules:
            if m.get("bias"): raise ValueError(f"{m['path']} has a bias; the decode loop runs bias-free decoders")
        cache = {}

        def stored(wid):
            if wid not in cache: cache.clear(); cache[wid] = rd.matrix(wid, device)      # one matrix in flight at a time
            return cache[wid]

        def weight_of(c):
            return NWCWeight.from_tensors(c.M, c.K, L.FIXED_BLOCK, c.data, c.bases, c.hdr, c.lut, c.low, device, elem=c.elem, scale=c.scale, layout=c.layout)

        def reencoded(full_bf16, shard_kind, like):
            part = TP.shard(shard_kind, full_bf16, cfg, tp_rank, tp_world) if tp_world > 1 and shard_kind else full_bf16
            return NWCWeight(part.contiguous(), device, elem="bf16" if like.elem == "bf16" else "fp8", layout=like.layout if relayout is None else relayout)

        def other_layout(c):
            """The matrix is stored in another layout than the one asked for (fp8 matrices are re-laid only unsharded: their
            codes and scales are taken as stored, never re-quantised)."""
            return relayout is not None and c.layout != relayout and (c.elem == "bf16" or tp_world == 1)

        def relaid(c, shard_kind):
            if c.elem == "fp8":
                codes, row_scale = weight_of(c).dequant_fp8()
                return NWCWeight(codes.contiguous(), device, elem="fp8", scale=row_scale, layout=relayout)
            return reencoded(dense(c), shard_kind, c)

        def dense(c):
            w = weight_of(c); full = w.dequant()
            return full if w.scale is None else (full.float() * w.scale[:, None]).to(torch.bfloat16)

        def projection(parent, names, shard_kind):
            """A fused group stored under `parent`, or separate linears parent.<name> (then concatenated and re-encoded)."""
            rec = by_path.get(parent)
            if rec is not None and rec["kind"] == "fused" and list(rec["names"]) == list(names):
                c = stored(rec["weight"])
                if other_layout(c): return relaid(c, shard_kind)
                if tp_world == 1: return weight_of(c)
                sizes, starts, ranges = rec["sizes"], [0], []
                for n in sizes: starts.append(starts[-1] + n)
                per = [n // tp_world for n in sizes]
                if all(n % tp_world == 0 for n in sizes) and R.rows_divisible(c.layout, *per):
                    for s0, n in zip(starts, per): ranges.append((s0 + tp_rank * n, s0 + (tp_rank + 1) * n))
                    return weight_of(R.take_rows(c, ranges))
                return reencoded(dense(c), shard_kind, c)
            parts = [stored(by_path[f"{parent}.{n}"]["weight"]) for n in names]
            like = parts[0]
            return reencoded(torch.cat([dense(p) for p in parts], 0), shard_kind, like)

        def row_parallel(path_, shard_kind):
            c = stored(by_path[path_]["weight"])
            if other_layout(c): return relaid(c, shard_kind)
            if tp_world == 1: return weight_of(c)
            n = c.K // tp_world
            if c.K % tp_world == 0 and n % R.BLOCK_COLS == 0: return weight_of(R.take_cols(c, tp_rank * n, (tp_rank + 1) * n))
            return reencoded(dense(c), shard_kind, c)

        emb_rec = next(m for m in rd.modules if m["kind"] == "embedding")
        emb_c = stored(emb_rec["weight"])
        self.embed = relaid(emb_c, None) if other_layout(emb_c) else weight_of(emb_c)
        head_rec = by_path.get("lm_head")
        if head_rec is None: raise ValueError("checkpoint has no compressed lm_head")
        if tp_world == 1:
            if head_rec["weight"] == emb_rec["weight"]: self.lm_head = self.embed
            else:
                c = stored(head_rec["weight"])
                self.lm_head = relaid(c, None) if other_layout(c) else weight_of(c)
        else:
            c = stored(head_rec["weight"]); V = cfg.vocab // tp_world
            self.lm_head = (weight_of(R.take_rows(c, [(tp_rank * V, (tp_rank + 1) * V)])) if R.rows_divisible(c.layout, V) and not other_layout(c)
                            else reencoded(dense(c), "lm_head", c))
        vec = lambda name: rd.tensor(name, device).to(torch.bfloat16).contiguous()
        self.layers = []
        for i in range(cfg.layers):
            pre = f"model.layers.{i}"
            self.layers.append({
                "in_norm": vec(f"{pre}.input_layernorm.weight"), "post_norm": vec(f"{pre}.post_attention_layernorm.weight"),
                "q_norm": vec(f"{pre}.self_attn.q_norm.weight") if cfg.qk_norm else None,
                "k_norm": vec(f"{pre}.self_attn.k_norm.weight") if cfg.qk_norm else None,
                "qkv": projection(f"{pre}.self_attn", ("q_proj", "k_proj", "v_proj"), "qkv"), "o": row_parallel(f"{pre}.self_attn.o_proj", "o"),
                "gate_up": projection(f"{pre}.mlp", ("gate_proj", "up_proj"), "gate_up"), "down": row_parallel(f"{pre}.mlp.down_proj", "down")})
        self.final_norm = vec("model.norm.weight")
        cache.clear()
        assert self.cfg.qkv_rows == self.layers[0]["qkv"].out_features
        return self

    def matrices(self):
        seen, out = set(), []
        for w in [self.embed, self.lm_head] + [l[k] for l in self.layers for k in ("qkv", "o", "gate_up", "down")]:
            if id(w) not in seen: seen.add(id(w)); out.append(w)
        return out

    def bytes_per_token(self):
        """Compressed bytes one decode step streams: every matvec matrix once (the embedding lookup reads one row)."""
        ws = [self.lm_head] + [l[k] for l in self.layers for k in ("qkv", "o", "gate_up", "down")]
        return sum(w.bytes + w.side_bytes for w in ws)


def rope_tables(cfg, max_len, device):
    """cos / sin as the Transformers rotary module computes them: fp32 angles, rounded to bf16; [max_len, head_dim]."""
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.int64).float() / cfg.head_dim))
    freqs = torch.arange(max_len, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16).to(device).contiguous(), emb.sin().to(torch.bfloat16).to(device).contiguous()


class DecodeEngine:
    def __init__(self, weights: DecoderWeights, max_len=1024, device="cuda", dependent_launch=False, tp_group=None, tp_reduce="push", side_tables=False, prefetch_next=True):
        """tp_group: torch.distributed process group of the tensor-parallel ranks (weights.tp_world > 1), else None.
        tp_reduce, how the ranks' partial o / down outputs are summed:
          "push"  the row-parallel matvec stores its partial into every rank's exchange buffer over NVLink and the next
                  matvec's prologue adds them (no kernel of its own; layout 2 bf16 matrices, else "pull" is used);
          "pull"  one kernel of this library per sum reads the peers' partials over NVLink (also called "peer");
          "nccl"  one NCCL all-reduce per sum.
        prefetch_next: every matvec names the matrix of the matvec after it, whose first bytes then travel to L2 across the
        kernel boundary (layout-2 matrices)."""
        L.require_cuda()
        self.prefetch_next = bool(prefetch_next)
        self.dependent_launch = bool(dependent_launch)
        self.tp_group, self.tp_world = tp_group, weights.tp_world
        if self.tp_world > 1 and tp_group is None: raise ValueError("sharded weights need the process group of their ranks")
        if tp_reduce == "peer": tp_reduce = "pull"
        if tp_reduce not in ("push", "pull", "nccl"): raise ValueError("tp_reduce is 'push', 'pull' or 'nccl'")
        if tp_reduce == "push" and not all(w.layout == 2 and w.elem == 0 for w in weights.matrices()): tp_reduce = "pull"
        self.tp_reduce = tp_reduce if self.tp_world > 1 else None
        self.peers = None
        if self.tp_world > 1 and tp_reduce in ("push", "pull"):
            from .comm import PeerBuffers
            self.peers = PeerBuffers(tp_group, weights.cfg.hidden)
        self.w, self.cfg, self.max_len, self.device = weights, weights.cfg, max_len, torch.device(device)
        self._opts = {}
        # Optional: layout-0 matrices small enough for the single-launch kernel decoded by four warps per block along a side
        # table.  Off by default: measured on B200 (Qwen3-0.6B shapes) the launch is bound by its prologue (offsets -> bulk
        # copy -> stream, table staging) and by kernel-to-kernel release, not by the serial walk of a block, and the fourfold
        # warp count leaves no room for the next kernel's blocks to start early: 761 tokens/s with, 826 without.
        if side_tables:
            for m in weights.matrices():
                blocks = -(-m.out_features // 8) * -(-m.in_features // 512)
                if m.layout == 0 and blocks <= 2 * L.SM_COUNT * 32 and m.K16 <= 40960: m.build_side_table()
        c = self.cfg
        bf = lambda n: torch.zeros(n, dtype=torch.bfloat16, device=device)
        pad32 = lambda n: (n + 31) // 32 * 32
        self.h, self.h2 = bf(pad32(c.hidden)), bf(pad32(c.hidden))
        self.xtmp = bf(pad32(max(c.hidden, c.intermediate)))
        self.xn = bf(pad32(c.hidden))                               # normalised activations (peer-reduce path)
        self.qkv, self.attn, self.proj, self.proj2 = bf(c.qkv_rows), bf(pad32(c.n_q * c.head_dim)), bf(pad32(c.hidden)), bf(pad32(c.hidden))
        self.gu = bf(2 * c.intermediate)
        self.logits = bf(c.vocab)                                   # this rank's vocabulary rows
        self.logits_all = bf(c.vocab * self.tp_world) if self.tp_world > 1 else self.logits
        self.k_cache = torch.zeros(c.layers, c.n_kv, max_len, c.head_dim, dtype=torch.bfloat16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(c, max_len, device)
        self.cur = torch.zeros(1, dtype=torch.int64, device=device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.step_no = torch.zeros(1, dtype=torch.int32, device=device)
        self.log = torch.zeros(max_len + 8, dtype=torch.int64, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.pinned_in = torch.zeros(1, dtype=torch.int64).pin_memory()
        self.pinned_out = torch.zeros(1, dtype=torch.int64).pin_memory()
        self.graph = None
        self.launches_per_step = 0
        self._count = 0
        if weights.embed.scale is not None: raise NotImplementedError("fp8 embedding tables are not supported by the decode loop")

    @classmethod
    def from_pretrained(cls, path, max_len=1024, device="cuda", tp_group=None, relayout=None, **kw):
        """Decode engine on an NWC checkpoint directory (see DecoderWeights.from_checkpoint); with a process group the
        matrices are cut into this rank's tensor-parallel shards while loading, or - a directory of per-rank shards
        written by `python -m nwc_b200.shard` - read as they are."""
        rank, world = 0, 1
        if tp_group is not None:
            import torch.distributed as dist
            rank, world = dist.get_rank(tp_group), dist.get_world_size(tp_group)
        from . import shard as S
        if S.is_sharded(path):                                       # per-rank folders written by `python -m nwc_b200.shard`: nothing to re-pack
            weights = S.load_shard(S.rank_dir(path, rank, world), device)
        else:
            weights = DecoderWeights.from_checkpoint(path, device, rank, world, relayout=relayout)
        return cls(weights, max_len=max_len, device=device, tp_group=tp_group, **kw)

    # ---- one token, eager: every call below is one or two kernels of this library on the current stream ----
    def _linear(self, w: NWCWeight, x, y, mode=0, h_in=None, delta=None, h_out=None, norm_w=None, gate_up=None, tp_in=-1, tp_out=-1, then=None):
        """y = W x with the activation prologue the mode names (0: x given; 1: x = RMSNorm(h_in + delta), h_out updated;
        2: x = SwiGLU(gate_up)), through nwc_linear_fused.  tp_in / tp_out: push slots of the tensor-parallel exchange
        (delta = the ranks' summed partials of slot tp_in; y pushed to every rank's slot tp_out instead of written).
        then = (weight, mode) of the matvec that follows on the stream: its first bytes are asked into L2 at this one's end."""
        out = y if isinstance(y, ctypes.c_void_p) else L.ptr(y)      # a raw device pointer: this rank's slot of the exchange buffer
        tp = self._options(w, tp_in, tp_out, then if self.prefetch_next else None)
        err = L.lib.nwc_linear_fused_opt(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), mode, L.ptr(x), L.ptr(h_in),
                                        L.ptr(delta), L.ptr(h_out), L.ptr(norm_w), self.cfg.eps, L.ptr(gate_up), L.ptr(self.xtmp), None, L.ptr(w.scale),
                                        L.ptr(w.scratch), out, w.n, w.block, w.in_features, w.code, tp)
        if err: raise RuntimeError(f"nwc_linear_fused error {err}")
        self._count += L.lib.nwc_linear_launches(w.n, w.in_features, w.code, mode)

    def _options(self, w, tp_in, tp_out, then=None):
        """nwc_fused_options of one call (kept alive by the engine: the library reads them at launch time), or None."""
        if then is not None and ((then[0].code >> 4) & 15) != 2: then = None      # the hint serves layout-2 matrices only
        if w.side is None and tp_in < 0 and tp_out < 0 and then is None: return None
        key = (id(w), tp_in, tp_out, 0 if then is None else id(then[0]), 0 if then is None else then[1])
        if key not in self._opts:
            side = None if w.side is None else w.side.data_ptr()
            if tp_in >= 0 or tp_out >= 0:
                p = self.peers
                o = L.FusedOptions(ctypes.cast(p.table, ctypes.c_void_p), p.rank, p.world, tp_in, tp_out, p.hidden, side)
            else:
                o = L.FusedOptions(None, 0, 0, -1, -1, 0, side)
            if then is not None:
                nw, nmode = then
                o.next_low, o.next_n, o.next_K, o.next_elem, o.next_mode = nw.low.data_ptr(), nw.n, nw.in_features, nw.code, nmode
            self._opts[key] = o
        return ctypes.byref(self._opts[key])

    def _argmax(self, c, st):
        """Greedy token from this rank's logits; with exchange buffers the ranks swap one (value, index) word each."""
        if self.peers is not None:
            self._check(L.lib.nwc_argmax_tp(st(), L.ptr(self.logits), c.vocab, L.ptr(self.cur), L.ptr(self.log), L.ptr(self.pos), L.ptr(self.step_no),
                                            self.log.numel(), self.max_len, self.peers.table, self.peers.rank, self.peers.world), "nwc_argmax_tp")
            return
        if self.tp_world > 1:                                        # NCCL path: gather the vocabulary-sharded logits, every rank picks the same token
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.logits_all, self.logits, group=self.tp_group)
            self._count += 1
        self._check(L.lib.nwc_argmax(st(), L.ptr(self.logits_all), c.vocab * self.tp_world, L.ptr(self.cur), L.ptr(self.log), L.ptr(self.pos), L.ptr(self.step_no),
                                     self.log.numel(), self.max_len), "nwc_argmax")

    def _all_reduce(self, t):
        """Sum the row-parallel partial outputs over the tensor-parallel ranks (one NCCL all-reduce over NVLink)."""
        if self.tp_world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.tp_group)
            self._count += 1

    def _check(self, err, what):
        if err: raise RuntimeError(f"{what} error {err}")
        self._count += 1

    def forward_token(self):
        """Kernels of one decode step: reads self.cur / self.pos, leaves the greedy token in self.cur, advances pos.
        The residual stream alternates between two buffers because the fused kernels read h while one CTA writes h + delta."""
        c, w, st = self.cfg, self.w, L.stream
        self._count = 0
        e = w.embed
        h, h_next = self.h, self.h2
        L.lib.nwc_set_dependent_launch(1 if self.dependent_launch else 0)
        try:
            self._forward(c, w, st, e, h, h_next)
        finally:
            L.lib.nwc_set_dependent_launch(0)
        self.launches_per_step = self._count

    def _forward_peer(self, c, w, st, e, h, h_next):
        """Tensor-parallel step with the partial sums exchanged through peer memory: every linear takes a ready x, the
        kernel after o / down adds the ranks' partials, the residual and applies the next RMSNorm."""
        self._check(L.lib.nwc_gather(st(), L.ptr(e.data), L.ptr(e.bases), L.ptr(e.hdr), L.ptr(e.lut), L.ptr(e.low), L.ptr(self.cur), 1, L.ptr(h),
                                     e.n, e.block, e.in_features, e.code), "nwc_gather")
        self._check(L.lib.nwc_add_rmsnorm(st(), L.ptr(h), None, L.ptr(h), L.ptr(w.layers[0]["in_norm"]), c.eps, c.hidden, L.ptr(self.xn), None), "nwc_add_rmsnorm")
        for i, l in enumerate(w.layers):
            self._linear(l["qkv"], self.xn, self.qkv)
            self._check(L.lib.nwc_attention_decode(st(), L.ptr(self.qkv), L.ptr(l["q_norm"]), L.ptr(l["k_norm"]), L.ptr(self.cos), L.ptr(self.sin),
                                                   L.ptr(self.k_cache[i]), L.ptr(self.v_cache[i]), L.ptr(self.pos), c.n_q, c.n_kv, c.head_dim, self.max_len,
                                                   c.eps, L.ptr(self.attn), L.ptr(self.status)), "nwc_attention_decode")
            self._linear(l["o"], self.attn, self.peers.slot(0))
            self.peers.allreduce_add_rmsnorm(0, h, h_next, l["post_norm"], c.eps, self.xn); self._count += 1
            h, h_next = h_next, h
            self._linear(l["gate_up"], self.xn, self.gu)
            self._linear(l["down"], None, self.peers.slot(1), mode=2, gate_up=self.gu)
            nxt = w.layers[i + 1]["in_norm"] if i + 1 < len(w.layers) else w.final_norm
            self.peers.allreduce_add_rmsnorm(1, h, h_next, nxt, c.eps, self.xn); self._count += 1
            h, h_next = h_next, h
        self._linear(w.lm_head, self.xn, self.logits)
        self._argmax(c, st)

    def _forward_push(self, c, w, st, e, h, h_next):
        """Tensor-parallel step with the sums over the ranks fused into the matvecs: o and down push their partial to every
        rank, the matvec after them (gate/up, the next layer's q/k/v, the lm_head) adds the partials, the residual and
        applies its RMSNorm while it builds x.  Five launches per layer, as on one GPU."""
        self._check(L.lib.nwc_gather(st(), L.ptr(e.data), L.ptr(e.bases), L.ptr(e.hdr), L.ptr(e.lut), L.ptr(e.low), L.ptr(self.cur), 1, L.ptr(h),
                                     e.n, e.block, e.in_features, e.code), "nwc_gather")
        for i, l in enumerate(w.layers):
            after = (w.layers[i + 1]["qkv"], 1) if i + 1 < len(w.layers) else (w.lm_head, 1)
            self._linear(l["qkv"], None, self.qkv, mode=1, h_in=h, h_out=h_next, norm_w=l["in_norm"], tp_in=1 if i else -1, then=(l["o"], 0))
            h, h_next = h_next, h
            self._check(L.lib.nwc_attention_decode(st(), L.ptr(self.qkv), L.ptr(l["q_norm"]), L.ptr(l["k_norm"]), L.ptr(self.cos), L.ptr(self.sin),
                                                   L.ptr(self.k_cache[i]), L.ptr(self.v_cache[i]), L.ptr(self.pos), c.n_q, c.n_kv, c.head_dim, self.max_len,
                                                   c.eps, L.ptr(self.attn), L.ptr(self.status)), "nwc_attention_decode")
            self._linear(l["o"], self.attn, None, tp_out=0, then=(l["gate_up"], 1))
            self._linear(l["gate_up"], None, self.gu, mode=1, h_in=h, h_out=h_next, norm_w=l["post_norm"], tp_in=0, then=(l["down"], 2))
            h, h_next = h_next, h
            self._linear(l["down"], None, None, mode=2, gate_up=self.gu, tp_out=1, then=after)
        self._linear(w.lm_head, None, self.logits, mode=1, h_in=h, h_out=h_next, norm_w=w.final_norm, tp_in=1, then=(w.layers[0]["qkv"], 1))
        self._argmax(c, st)

    def close(self):
        """Release the exchange buffers (all ranks: after synchronising and a barrier)."""
        if self.peers is not None: self.peers.close(); self.peers = None

    def _forward(self, c, w, st, e, h, h_next):
        if self.tp_reduce == "push": return self._forward_push(c, w, st, e, h, h_next)
        if self.peers is not None: return self._forward_peer(c, w, st, e, h, h_next)
        self._check(L.lib.nwc_gather(st(), L.ptr(e.data), L.ptr(e.bases), L.ptr(e.hdr), L.ptr(e.lut), L.ptr(e.low), L.ptr(self.cur), 1, L.ptr(h),
                                     e.n, e.block, e.in_features, e.code), "nwc_gather")
        delta = None
        for i, l in enumerate(w.layers):
            after = (w.layers[i + 1]["qkv"], 1) if i + 1 < len(w.layers) else (w.lm_head, 1)
            self._linear(l["qkv"], None, self.qkv, mode=1, h_in=h, delta=delta, h_out=h_next, norm_w=l["in_norm"], then=(l["o"], 0))
            h, h_next = h_next, h
            self._check(L.lib.nwc_attention_decode(st(), L.ptr(self.qkv), L.ptr(l["q_norm"]), L.ptr(l["k_norm"]), L.ptr(self.cos), L.ptr(self.sin),
                                                   L.ptr(self.k_cache[i]), L.ptr(self.v_cache[i]), L.ptr(self.pos), c.n_q, c.n_kv, c.head_dim, self.max_len,
                                                   c.eps, L.ptr(self.attn), L.ptr(self.status)), "nwc_attention_decode")
            self._linear(l["o"], self.attn, self.proj, then=(l["gate_up"], 1))
            self._all_reduce(self.proj)
            self._linear(l["gate_up"], None, self.gu, mode=1, h_in=h, delta=self.proj, h_out=h_next, norm_w=l["post_norm"], then=(l["down"], 2))
            h, h_next = h_next, h
            self._linear(l["down"], None, self.proj2, mode=2, gate_up=self.gu, then=after)
            self._all_reduce(self.proj2)
            delta = self.proj2
        self._linear(w.lm_head, None, self.logits, mode=1, h_in=h, delta=delta, h_out=h_next, norm_w=w.final_norm, then=(w.layers[0]["qkv"], 1))
        self._argmax(c, st)

    # ---- graph ----
    def capture(self, warmup=3):
        """Capture one decode step as a CUDA graph (state is saved and restored around the warm-up runs)."""
        saved = (self.cur.clone(), self.pos.clone(), self.step_no.clone())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.pos.zero_(); self.forward_token()
        torch.cuda.current_stream().wait_stream(side)
        self.pos.zero_()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.forward_token()
        for t, s in zip((self.cur, self.pos, self.step_no), saved): t.copy_(s)
        self.log.zero_()
        torch.cuda.synchronize()

    def reset(self):
        self.pos.zero_(); self.step_no.zero_(); self.log.zero_(); self.status.zero_()

    def _run(self):
        if self.graph is not None: self.graph.replay()
        else: self.forward_token()

    def _check_status(self):
        """After a synchronise: the position must have stayed inside the KV cache and no bounded wait inside a kernel
        (bulk copy, peer rank) may have run out - a step that did is not a valid token."""
        if int(self.status.item()): raise RuntimeError("decode position left the KV cache")
        st = L.lib.nwc_kernel_status(1)
        if st: raise RuntimeError(f"a bounded wait inside a kernel gave up (status {st}: 2 = bulk copy, 3 = a tensor-parallel rank did not answer)")

    def prefill(self, prompt_ids):
        """Feed the prompt token by token through the decode step (teacher forcing); returns the first generated token
        id as a device tensor.  Positions restart at 0."""
        self.reset()
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64, device=self.device).reshape(-1)
        if prompt.numel() > self.max_len: raise ValueError(f"prompt of {prompt.numel()} tokens does not fit the KV cache ({self.max_len})")
        for i in range(prompt.numel()):
            self.cur.copy_(prompt[i:i + 1])
            self._run()
        self.step_no.zero_()
        torch.cuda.synchronize()
        self._check_status()
        return self.cur

    def generate(self, n_tokens):
        """n_tokens greedy steps from the current state; returns the generated ids (the token in self.cur is consumed
        first, its successors are returned)."""
        start, pos = int(self.step_no.item()), int(self.pos.item())
        if pos + n_tokens > self.max_len or start + n_tokens > self.log.numel():
            raise ValueError(f"{n_tokens} more tokens from position {pos} do not fit the KV cache ({self.max_len})")
        for _ in range(n_tokens): self._run()
        torch.cuda.synchronize()
        self._check_status()
        return self.log[start:start + n_tokens].clone()

    def step(self, token_id: int) -> int:
        """Serving-style call with host values: token in from pinned host memory, next token back to the host."""
        self.pinned_in[0] = token_id
        self.cur.copy_(self.pinned_in, non_blocking=True)
        self._run()
        self.pinned_out.copy_(self.cur, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self.tp_world > 1: self._check_status()                  # rank skew must never turn into a silently wrong token
        return int(self.pinned_out[0])
