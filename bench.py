"""Benchmark of the NWC batch-1 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--model llama3-70b] [--layout 2] [--elem bf16]

Default workload: a Llama-3-70B-architecture decoder (80 layers, hidden 8192, MLP 28672, 64 q / 8 kv heads, vocabulary
128256) with random-init weights of the reference's distribution (W = r_i * 0.02 * z, r_i log-normal(0, 0.3), norms 1),
compressed bf16 layout 2 (about 105 GB), batch 1, 32 random prompt ids, greedy decode replayed as one CUDA graph per
token.  A step is one decoded token.  `--model qwen3-0.6b --layout 0` and `--model qwen3-4b` select the smaller
configurations.
  N = 1   the whole model on one GPU.
  N > 1   (torchrun, one rank per GPU) the SAME model sharded tensor-parallel over the N ranks: q/k/v, gate/up and lm_head
          by rows, o and down by columns, the partial sums of o and down exchanged over NVLink inside the matvec kernels
          (`--tp-reduce push`; `pull` = one reduction kernel per sum, `nccl` = NCCL all-reduce).  Strong scaling: value =
          K / max-over-ranks time.  `--parallel replicas` runs N independent copies instead (weak scaling, small models).
  value     tokens/s of K graph replays, device-timed, nothing copied to or from the host inside the region
  e2e       the same through DecodeEngine.step(): token id from pinned host memory in, next token id back, every step
  tokens_sha16   hash of the ids generated in the timed region (equal across N when no near-tie flips a token)
  roofline  the token-matvec kernel with the largest share of the step (each of the five matrix kinds is timed alone, back
            to back over the layers' own matrices so that no launch finds its matrix in L2): algorithmic bytes (the
            reference's per-matrix byte count) / CUDA-event time, against the measured HBM peak
  cpu_baseline  (N = 1) the CPU oracle's fused decode+matvec on all host cores over a bounded sample, extrapolated to a token
--impl reference runs the CPU path alone (rank 0), each step one pass over the bounded sample.
"""
import argparse
import hashlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path: sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--layout", type=int, default=None, help="default: 2 (0 for qwen3-0.6b, the layout its configuration names)")
    ap.add_argument("--elem", default="bf16")
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default="", help="time one token matvec alone: lm_head | qkv | o | gate_up | down | MxK (small case for ncu)")
    ap.add_argument("--op", default="", help="time one of the other kernels alone (small cases for ncu): gather:N | attention:POS | encode:MxK | prefill:MxKxT | native_fp8:MxK | exchange:WORLD")
    ap.add_argument("--vs-ref", action="store_true", help="--kernel: also time the reference's own kernel (oracle/_ref/nwc_ops.so) on the same matrices")
    ap.add_argument("--parallel", default="auto", choices=["auto", "replicas", "tp"], help="N > 1: tensor parallel (auto, tp) or independent replicas")
    ap.add_argument("--tp-reduce", default="push", choices=["push", "pull", "nccl"], help="how the partial outputs of o and down are summed over the ranks")
    ap.add_argument("--peer-sharing", type=int, default=0, help="tensor parallel: from this many ranks on, clusters of CTAs share the sum of the pushed partials (0 = every CTA adds up all of them; A/B)")
    ap.add_argument("--pool", type=int, default=0, help="1: layout-2 matvecs on the kernel whose warps draw stages from a per-CTA pool instead of one fixed run per warp (A/B)")
    ap.add_argument("--prefetch-next", type=int, default=1, help="0: matvecs do not ask L2 for the next matrix's first bytes at their end (A/B)")
    ap.add_argument("--side-tables", type=int, default=0, help="1: layout 0 decoder-layer matrices on four warps per block along a side table instead of one (A/B)")
    ap.add_argument("--fixup", type=int, default=1, help="0: work splits of whole row groups instead of equal runs with in-kernel fix-up (A/B)")
    ap.add_argument("--dependent-launch", type=int, default=1, help="programmatic dependent launch between the decode-step kernels")
    a = ap.parse_args()
    if a.layout is None: a.layout = 0 if a.model == "qwen3-0.6b" else 2
    return a


def load_presets():
    """The architecture table, by path: the reference arm must not load the CUDA library."""
    spec = importlib.util.spec_from_file_location("nwc_presets", os.path.join(ROOT, "nwc_b200", "presets.py"))
    m = importlib.util.module_from_spec(spec); sys.modules["nwc_presets"] = m; spec.loader.exec_module(m)
    return m.PRESETS


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f: return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True); self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout: self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None: return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25); self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
# CPU path (oracle port of the reference's format; the reference ships no compiled CPU decoder for formats v9+)

class CpuSample:
    """A bounded sample of one token's matvec work for the CPU arm: the first 1 / `cut` of the rows of each of a decoder
    layer's four matrices and 1 / (8 cut) of the lm_head rows, encoded once; a pass multiplies all five and the token time
    is extrapolated as layers * cut * (layer part) + 8 cut * (lm_head part)."""

    def __init__(self, cfg, layout, elem_code):
        import oracle as O
        self.O, self.cfg = O, cfg
        weights = sum(r * c for k, (r, c) in cfg.matrix_shapes().items() if k != "lm_head")
        self.cut = 1 if weights <= 120e6 else (4 if weights <= 500e6 else 8)     # keeps encoding + a pass within seconds
        code = O.code_of(elem_code, layout)
        self.packed = []
        for i, (name, (M, K)) in enumerate(cfg.matrix_shapes().items()):
            rows = max(16, M // (self.cut * (8 if name == "lm_head" else 1)) // 16 * 16)
            w, x = O.synth_weights(rows, K, 1000 + i)
            src = O.quantize_fp8(w)[0] if elem_code else w
            self.packed.append((O.encode(src, code), O.bf16_to_f32(x), M / rows))
        self.what = ("rows [0, M/%d) of one decoder layer's qkv, o, gate_up and down plus 1/%d of the lm_head rows per pass; token time = layers x layer part + lm_head part, each "
                     "scaled by its row fraction" % (self.cut, 8 * self.cut))

    def seconds_per_token(self, threads):
        per = []
        for p, x, scale in self.packed:
            t = time.perf_counter(); self.O.matvec_f32(p, x, threads=threads); per.append((time.perf_counter() - t) * scale)
        return self.cfg.layers * sum(per[:4]) + per[4]


def run_reference(a, cfg):
    threads = os.cpu_count() or 1
    sample = CpuSample(cfg, a.layout, 1 if a.elem == "fp8" else 0)
    for _ in range(a.warmup): sample.seconds_per_token(threads)
    times = [sample.seconds_per_token(threads) for _ in range(max(1, a.steps))]
    sec = statistics.mean(times)
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": 1.0 / sec, "unit": "tokens/s", "n_gpus": a.gpus, "steps": max(1, a.steps), "warmup": a.warmup,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": scaling_of(a, a.gpus), "vs_baseline": None, "dtype": a.elem, "data": "synthetic",
            "config": workload(a, cfg, a.gpus), "cpu_baseline": {"value": 1.0 / sec, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample.what},
            "e2e": {"value": 1.0 / sec, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def is_tp(a, world): return world > 1 and a.parallel in ("auto", "tp")
def scaling_of(a, world): return "strong" if is_tp(a, world) else "weak"


def workload(a, cfg, world=1):
    """The `config` object; identical in both arms so that their lines can be compared key by key."""
    par = "1 GPU"
    if world > 1:
        how = {"push": "pushed over NVLink inside the matvec kernels", "pull": "NVLink peer-memory reduction kernel", "nccl": "NCCL all-reduce"}[a.tp_reduce]
        par = ("tp%d: q/k/v, gate/up, lm_head split by rows, o/down by columns, partial sums added after o and down (%s)" % (world, how) if is_tp(a, world)
               else "replicas x%d (no data-path collective)" % world)
    return {"workload": f"{cfg.name}-architecture decoder, random init, NWC {a.elem} layout {a.layout}, batch 1, {a.prompt} random prompt ids, greedy decode as a CUDA graph",
            "layers": cfg.layers, "hidden": cfg.hidden, "vocab": cfg.vocab,
            "l2_policy": "no flush: the compressed weights streamed per token are larger than the 126 MB L2, and the roofline leg walks the layers' own matrices (more than L2 in total) back to back",
            "parallelism": par}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch over its algorithmic bytes, from the ncu captures summarised
# under profiles/ (a smaller matrix of the same kernel and K where the full one is too large to capture; the kernel reads
# every plane byte once, so traffic grows in proportion to the bytes); kinds without a capture report null
NCU_TRAFFIC_RATIO = {("ring_kernel_layout2", 8192): 1.008,      # 57344 x 8192 itself: 713.1 MB of DRAM traffic for 707.5 MB (profiles/ring_kernel_layout2_llama3_70b_shapes.md)
                     ("ring_kernel_layout2", 1024): 1.02, ("prefix_ring_kernel_layout0", 1024): 1.018, ("prefix_ring_kernel_layout1", 1024): 1.023}


def token_kernel_name(layout, elem, small=False):
    if layout == 0: return "small_kernel_layout0" if small else "prefix_ring_kernel_layout0"
    if layout == 1: return "prefix_ring_kernel_layout1"
    if layout == 2 and elem == "bf16": return "ring_kernel_layout2"
    return "segment_kernel<layout %d, %s>" % (layout, elem)


# ---------------------------------------------------------------------------------------------------------------------

def trace(msg):
    """Phase markers on stderr (NWC_BENCH_TRACE=1) for diagnosing a multi-rank run that stops."""
    if os.environ.get("NWC_BENCH_TRACE"): print(f"[bench rank {os.environ.get('RANK', 0)}] {msg}", file=sys.stderr, flush=True)


def kernel_only(a, cfg):
    """The token matvec on synthetic matrices of one shape, back to back inside a CUDA graph over enough rotating copies
    that no launch finds its matrix in L2.  Prints one JSON line with the roofline of one call."""
    import ctypes
    import torch
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    shapes = cfg.matrix_shapes()
    M, K = shapes[a.kernel] if a.kernel in shapes else tuple(int(v) for v in a.kernel.lower().split("x"))
    torch.cuda.set_device(0)
    L.lib.nwc_set_fixup_plans(int(a.fixup))
    L.lib.nwc_set_pool_kernels(int(a.pool))
    L.lib.nwc_set_peer_sharing(int(a.peer_sharing))
    L.lib.nwc_set_dependent_launch(int(a.dependent_launch))
    first = NWCWeight(synthetic_matrix(M, K, 1), layout=a.layout, elem=a.elem)
    copies = max(1, min(64, -(-(320 << 20) // first.bytes)))          # rotate over > 320 MB so that no launch finds its matrix in L2
    mats = [first] + [NWCWeight(synthetic_matrix(M, K, 1 + i), layout=a.layout, elem=a.elem) for i in range(1, copies)]
    nw = first
    x = torch.randn((K + 31) // 32 * 32, device="cuda").to(torch.bfloat16); x[K:] = 0
    y = torch.empty(M, dtype=torch.bfloat16, device="cuda")
    xtmp = torch.zeros_like(x)
    def launch(w):                           # the decode loop's entry point with a ready x (mode 0): same kernels as inside a decode step
        err = L.lib.nwc_linear_fused(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), 0, L.ptr(x), None, None, None, None,
                                     1e-6, None, L.ptr(xtmp), None, L.ptr(w.scale), L.ptr(w.scratch), L.ptr(y), w.n, w.block, K, w.code)
        if err: raise RuntimeError(f"nwc_linear_fused error {err}")
    reps = max(copies, 8)
    def timed(call, n_copies):
        side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side): call(0)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps): call(i % n_copies)
        times = []
        for i in range(a.warmup + a.steps):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(); graph.replay(); t1.record(); torch.cuda.synchronize()
            if i >= a.warmup: times.append(t0.elapsed_time(t1) / reps)
        return statistics.median(times)
    ms = timed(lambda i: launch(mats[i]), copies)
    if L.lib.nwc_kernel_status(1): raise RuntimeError("a bounded wait inside a kernel gave up")
    peak, kind = measured_peak()
    # the same product as a dense bf16 GEMV from the vendor library, same timing method (a reported comparison only)
    dense_ms = None
    if a.elem == "bf16" and a.steps > 1:
        dense_copies = max(1, min(16, -(-(320 << 20) // (2 * M * K))))
        dense = [synthetic_matrix(M, K, 1 + i).cuda() for i in range(dense_copies)]
        dense_ms = timed(lambda i: torch.nn.functional.linear(x[:K], dense[i]), dense_copies)
        del dense
    # fp8: the library's uncompressed fp8 weight-only matvec (one byte per weight) on the same quantised matrix
    native_fp8_ms = None
    if a.elem == "fp8" and a.steps > 1:
        from nwc_b200.weight import quantize_fp8
        n8 = max(1, min(16, -(-(320 << 20) // (M * K))))
        q8 = [quantize_fp8(synthetic_matrix(M, K, 1 + i)) for i in range(n8)]
        xf, y8 = x.float().contiguous(), torch.empty(M, dtype=torch.bfloat16, device="cuda")
        def native(i):
            err = L.lib.nwc_ref_fp8(L.stream(), L.ptr(q8[i][0].view(torch.uint8)), L.ptr(q8[i][1]), L.ptr(xf), L.ptr(y8), M, K)
            if err: raise RuntimeError(f"nwc_ref_fp8 error {err}")
        native_fp8_ms = timed(native, n8)
        del q8
    # the reference's own kernel for the same call (its library compiled unchanged for sm_100a; a comparison arm of this
    # benchmark only): the reference ABI's nwc_linear_bf16 takes fp32 x for layout 0 and bf16 x otherwise
    ref_ms = None
    if a.vs_ref and a.steps > 1:
        path = os.path.join(ROOT, "oracle", "_ref", "nwc_ops.so")
        if os.path.exists(path):
            ref = ctypes.CDLL(path)
            ref.nwc_setup.restype = ctypes.c_int; ref.nwc_setup()
            P, U64, U32, I = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
            ref.nwc_linear_bf16.restype, ref.nwc_linear_bf16.argtypes = I, [P] * 11 + [U64, U32, U32, I]
            xr = (x.float() if a.layout == 0 else x).contiguous()
            def ref_call(i):
                w = mats[i]
                err = ref.nwc_linear_bf16(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), L.ptr(xr), None, L.ptr(w.scale),
                                          L.ptr(w.scratch), L.ptr(y), w.n, w.block, K, w.code)
                if err: raise RuntimeError(f"reference nwc_linear_bf16 error {err}")
            ref_ms = timed(ref_call, copies)
    print(json.dumps({"kernel": f"token matvec {M}x{K} {a.elem} layout {a.layout}", "launches_per_call": L.lib.nwc_linear_launches(nw.n, K, nw.code, 0), "us_per_call": ms * 1e3,
                      "bytes_per_call": nw.bytes, "bits_per_weight": 8 * nw.bytes / nw.n, "dense_bf16_gemv_us": None if dense_ms is None else dense_ms * 1e3,
                      "native_fp8_matvec_us": None if native_fp8_ms is None else native_fp8_ms * 1e3,
                      "reference_kernel_us": None if ref_ms is None else ref_ms * 1e3,
                      "roofline": {"bound": "hbm", "achieved": nw.bytes / ms / 1e6, "peak": peak, "peak_kind": kind, "unit": "GB/s", "frac": nw.bytes / ms / 1e6 / peak},
                      "note": "%d calls on %d rotating copies replayed as one CUDA graph, CUDA events around the replay (a call includes its finalize launch when it needs one)" % (reps, copies)}))


def op_only(a, cfg):
    """One of the kernels around the token matvec, timed alone with CUDA events (median of --steps runs after --warmup);
    prints one JSON line.  Small cases, so that the same command can be captured under ncu."""
    import torch
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    torch.cuda.set_device(0)
    what, _, arg = a.op.partition(":")
    peak, kind = measured_peak()

    def timed(call, reps=1, graph=True):
        """Median microseconds per call; `reps` calls per measurement, replayed as one CUDA graph so that short kernels are
        not timed by the host's launch rate."""
        runner = None
        if graph:
            side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side): call()
            torch.cuda.current_stream().wait_stream(side)
            runner = torch.cuda.CUDAGraph()
            with torch.cuda.graph(runner):
                for _ in range(reps): call()
        times = []
        for i in range(a.warmup + a.steps):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            if runner is not None: runner.replay()
            else:
                for _ in range(reps): call()
            t1.record(); torch.cuda.synchronize()
            if i >= a.warmup: times.append(t0.elapsed_time(t1) / reps)
        return statistics.median(times) * 1e3                      # microseconds

    out = {"op": a.op, "elem": a.elem, "layout": a.layout}
    if what == "gather":            # compressed embedding lookup: N random rows of the model's table
        n = int(arg or 512)
        w = NWCWeight(synthetic_matrix(cfg.vocab, cfg.hidden, 1), layout=a.layout, elem="bf16")
        ids = torch.randint(0, cfg.vocab, (n,), device="cuda")
        out_rows = torch.empty(n, w.K16, dtype=torch.bfloat16, device="cuda")
        def lookup():
            err = L.lib.nwc_gather(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), L.ptr(ids), n, L.ptr(out_rows), w.n, w.block, w.in_features, w.code)
            if err: raise RuntimeError(f"nwc_gather error {err}")
        us = timed(lookup, reps=4)
        out.update({"rows": n, "us": us, "kernel": "gather_kernel", "output_GBs": n * w.K16 * 2 / us / 1e3, "table_bits_per_weight": 8 * w.bytes / w.n})
        if a.layout == 0:           # the same lookup with the side table: every row's walk starts at its row pair
            w.build_side_table()
            def lookup_side():
                err = L.lib.nwc_gather_side(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), L.ptr(ids), n, L.ptr(out_rows), w.n, w.block,
                                            w.in_features, w.code, L.ptr(w.side))
                if err: raise RuntimeError(f"nwc_gather_side error {err}")
            out["us_with_side_table"] = timed(lookup_side, reps=4)
    elif what == "attention":       # one token of grouped-query attention over POS cached positions
        pos = int(arg or 256)
        c = cfg
        bf = lambda *shape: torch.randn(*shape, device="cuda").to(torch.bfloat16)
        qkv, k_cache, v_cache = bf(c.qkv_rows), bf(c.n_kv, pos + 8, c.head_dim), bf(c.n_kv, pos + 8, c.head_dim)
        from nwc_b200.decode import rope_tables
        cos, sin = rope_tables(c, pos + 8, "cuda")
        norm = torch.ones(c.head_dim, dtype=torch.bfloat16, device="cuda") if c.qk_norm else None
        p = torch.full((1,), pos, dtype=torch.int32, device="cuda"); status = torch.zeros(1, dtype=torch.int32, device="cuda")
        o = torch.empty(c.n_q * c.head_dim, dtype=torch.bfloat16, device="cuda")
        def call():
            err = L.lib.nwc_attention_decode(L.stream(), L.ptr(qkv), L.ptr(norm), L.ptr(norm), L.ptr(cos), L.ptr(sin), L.ptr(k_cache), L.ptr(v_cache), L.ptr(p), c.n_q, c.n_kv,
                                             c.head_dim, pos + 8, c.eps, L.ptr(o), L.ptr(status))
            if err: raise RuntimeError(f"nwc_attention_decode error {err}")
        us = timed(call, reps=8)
        cache_bytes = 2 * c.n_kv * pos * c.head_dim * 2
        out.update({"positions": pos, "heads": [c.n_q, c.n_kv], "us": us, "kernel": "attention_decode_lanes_kernel", "cache_GBs": cache_bytes / us / 1e3})
    elif what == "encode":          # GPU encoder on a matrix that already lives in HBM
        M, K = (int(v) for v in (arg or "4096x4096").lower().split("x"))
        w = synthetic_matrix(M, K, 1)
        us = timed(lambda: NWCWeight(w, layout=a.layout, elem=a.elem), graph=False)        # the encoder synchronises: not capturable
        out.update({"shape": [M, K], "us": us, "Mweights_per_s": M * K / us, "kernel": "measure_kernel / pack_kernel (whole NWCWeight construction, host table build and allocation included)"})
        if a.vs_ref:                # the reference's own host encoder (one thread, as written) on the same matrix; bounded to 16 M weights
            import numpy as np
            import oracle as O
            if O.ref_available():
                rows = max(16, min(M, (16 << 20) // K) // 16 * 16)
                bits = w[:rows].cpu().view(torch.int16).numpy().view(np.uint16)
                src = O.quantize_fp8(bits)[0] if a.elem == "fp8" else bits
                t = time.perf_counter(); O.ref_encode(src, O.code_of(1 if a.elem == "fp8" else 0, a.layout)); dt = time.perf_counter() - t
                out["reference_host_encoder_Mweights_per_s"] = rows * K / dt / 1e6
                out["reference_sample"] = f"first {rows} rows, 1 thread"
    elif what == "prefill":         # T tokens at once: tile-wise decode into the tcgen05 GEMM against dequantise + dense matmul
        M, K, T = (int(v) for v in (arg or "6144x2560x512").lower().split("x"))
        w = NWCWeight(synthetic_matrix(M, K, 1), layout=a.layout, elem=a.elem)
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        dense_us = timed(lambda: torch.nn.functional.linear(x, w.dequant()), reps=4)
        out.update({"shape": [M, K, T], "dequant_plus_dense_matmul_us": dense_us, "dense_TFLOPs": 2 * M * K * T / dense_us / 1e6})
        if w.linear_prefill(x) is not None:
            us = timed(lambda: w.linear_prefill(x), reps=4)
            out.update({"us": us, "TFLOPs": 2 * M * K * T / us / 1e6, "kernel": "prefill_kernel_layout2"})
    elif what == "native_fp8":      # the uncompressed fp8 weight-only matvec (bandwidth baseline of the fp8 configuration)
        from nwc_b200.weight import quantize_fp8
        M, K = (int(v) for v in (arg or "19456x2560").lower().split("x"))
        n8 = max(1, min(16, -(-(320 << 20) // (M * K))))
        q8 = [quantize_fp8(synthetic_matrix(M, K, 1 + i)) for i in range(n8)]
        xf, y8 = torch.randn(K, device="cuda"), torch.empty(M, dtype=torch.bfloat16, device="cuda")
        it = [0]
        def call():
            q, sc = q8[it[0] % n8]; it[0] += 1
            err = L.lib.nwc_ref_fp8(L.stream(), L.ptr(q.view(torch.uint8)), L.ptr(sc), L.ptr(xf), L.ptr(y8), M, K)
            if err: raise RuntimeError(f"nwc_ref_fp8 error {err}")
        us = timed(call, reps=n8)
        out.update({"shape": [M, K], "us": us, "kernel": "native_fp8_kernel", "roofline": {"bound": "hbm", "achieved": (M * K + 4 * M) / us / 1e3, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                                                                                               "frac": (M * K + 4 * M) / us / 1e3 / peak}})
    elif what == "exchange":        # tensor-parallel consumer on ONE GPU: WORLD local exchange buffers stand in for the ranks' buffers
        import ctypes
        world = int(arg or 8)
        H, rows = cfg.hidden, 2 * cfg.intermediate // world
        bufs = []
        for _ in range(world):
            p = ctypes.c_void_p()
            if L.lib.nwc_comm_alloc(ctypes.byref(p), H): raise RuntimeError("nwc_comm_alloc failed")
            bufs.append(p.value)
        table = (ctypes.c_void_p * world)(*bufs)
        o_shard = NWCWeight(synthetic_matrix(H, cfg.n_q * cfg.head_dim // world, 1), layout=2)                 # row-parallel producer: [H, K / world]
        copies = max(2, min(8, -(-(400 << 20) // (rows * H * 3 // 2))))
        gate_up = [NWCWeight(synthetic_matrix(rows, H, 10 + i), layout=2) for i in range(copies)]              # the consumer's shard, rotating copies
        bf = lambda n, v=0.0: torch.full((n,), v, dtype=torch.bfloat16, device="cuda")
        attn, h, h2, nw, y, delta = bf(o_shard.in_features, 0.1), bf(H, 1.0), bf(H), bf(H, 1.0), bf(rows), bf(H, 0.01)
        xtmp = bf(H + 32)
        L.lib.nwc_set_dependent_launch(1)
        L.lib.nwc_set_peer_sharing(int(a.peer_sharing))
        def fused(w, mode, opt, **kw):
            g_ = lambda k: L.ptr(kw.get(k))
            err = L.lib.nwc_linear_fused_opt(L.stream(), L.ptr(w.data), L.ptr(w.bases), L.ptr(w.hdr), L.ptr(w.lut), L.ptr(w.low), mode, g_("x"), g_("h_in"), g_("delta"), g_("h_out"),
                                             g_("norm_w"), cfg.eps, None, L.ptr(xtmp), None, None, L.ptr(w.scratch), g_("y"), w.n, w.block, w.in_features, w.code, opt)
            if err: raise RuntimeError(f"nwc_linear_fused_opt error {err}")
        for r in range(world):          # every "rank" pushes its partial of slot 0 into every buffer, once: the words stay valid for all timed calls
            fused(o_shard, 0, ctypes.byref(L.FusedOptions(ctypes.cast(table, ctypes.c_void_p), r, world, -1, 0, H, None)), x=attn)
        torch.cuda.synchronize()
        peer_opt = L.FusedOptions(ctypes.cast(table, ctypes.c_void_p), 0, world, 0, -1, H, None)
        it = [0]
        def consumer(peer):
            w = gate_up[it[0] % copies]; it[0] += 1
            if peer: fused(w, 1, ctypes.byref(peer_opt), h_in=h, h_out=h2, norm_w=nw, y=y)
            else: fused(w, 1, None, h_in=h, delta=delta, h_out=h2, norm_w=nw, y=y)
        local_us = timed(lambda: consumer(False), reps=2 * copies)
        peer_us = timed(lambda: consumer(True), reps=2 * copies)
        if L.lib.nwc_kernel_status(1): raise RuntimeError("a bounded wait inside a kernel gave up")
        out.update({"world": world, "consumer": [rows, H], "kernel": "ring_kernel_layout2 (RMSNorm prologue over the ranks' pushed partials)", "us_local_delta": local_us,
                    "us_peer_partials": peer_us, "us_sum_over_ranks": peer_us - local_us, "partial_bytes_read_per_cta": world * H * 4,
                    "peer_sharing_from_ranks": int(a.peer_sharing)})
        for b in bufs: L.lib.nwc_comm_free(ctypes.c_void_p(b))
    else:
        raise SystemExit(f"unknown --op {a.op}")
    if L.lib.nwc_kernel_status(1): raise RuntimeError("a bounded wait inside a kernel gave up")
    print(json.dumps(out))


def matvec_shares(eng, weights, cfg, reps_target=24):
    """Each of the five kinds of token matvec timed alone: the layers' own matrices of that kind back to back (plain x,
    mode 0) inside one CUDA graph, CUDA events around the replay.  Returns {kind: (us per launch, bytes per launch, launches
    per token)}."""
    import torch
    from nwc_b200 import _lib as L
    out = {}
    L.lib.nwc_set_dependent_launch(1 if eng.dependent_launch else 0)       # launched as inside the decode step
    for kind in ("qkv", "o", "gate_up", "down", "lm_head"):
        mats = [weights.lm_head] if kind == "lm_head" else [l[kind] for l in weights.layers]
        total = sum(m.bytes for m in mats)
        reps = max(8, min(reps_target, len(mats))) if len(mats) > 1 else 12
        x = eng.xtmp if mats[0].in_features <= eng.xtmp.numel() else torch.zeros(mats[0].in_features + 32, dtype=torch.bfloat16, device="cuda")
        y = torch.empty(max(m.out_features for m in mats), dtype=torch.bfloat16, device="cuda")
        side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side): eng._linear(mats[0], x, y)
        torch.cuda.current_stream().wait_stream(side)
        kg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kg):
            for i in range(reps): eng._linear(mats[i % len(mats)], x, y, then=(mats[(i + 1) % len(mats)], 0))
        for _ in range(3): kg.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(); kg.replay(); k1.record(); torch.cuda.synchronize()
        out[kind] = (k0.elapsed_time(k1) / reps * 1e3, total / len(mats), 1 if kind == "lm_head" else len(weights.layers), min(reps, len(mats)) * (total / len(mats)))
        del kg
    L.lib.nwc_set_dependent_launch(0)
    return out


def finish(eng, dist):
    """Orderly multi-rank exit: CUDA graphs that hold NCCL kernels are released before the communicator goes away."""
    if dist is None: return
    import gc
    import torch
    eng.graph = None
    gc.collect(); torch.cuda.synchronize()
    dist.barrier(); torch.cuda.synchronize()
    eng.close()
    dist.destroy_process_group()


def main():
    a = parse()
    cfg = load_presets()[a.model]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if a.impl == "reference":                # the CPU arm: rank 0 alone, no CUDA library, no CUDA context
        if rank == 0: run_reference(a, cfg)
        return
    if a.kernel:
        if rank == 0: kernel_only(a, cfg)
        return
    if a.op:
        if rank == 0: op_only(a, cfg)
        return
    import torch
    from nwc_b200.decode import DecodeEngine, DecoderWeights  # the package import fails loudly when the CUDA library is missing
    from nwc_b200 import _lib as L
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    tp = is_tp(a, world)
    L.lib.nwc_set_pool_kernels(int(a.pool))
    L.lib.nwc_set_peer_sharing(int(a.peer_sharing))
    if tp and a.tp_reduce == "nccl": a.dependent_launch = 0         # NCCL kernels sit in the chain: keep plain stream order around them
    max_len = a.prompt + 2 * (a.warmup + a.steps) + 16
    if tp:      # one model sharded over all ranks: same seed everywhere, every rank keeps its shard and decodes the same sequence
        weights = DecoderWeights.synthetic(cfg, layout=a.layout, elem=a.elem, seed=0, tp_rank=rank, tp_world=world)
        eng = DecodeEngine(weights, max_len=max_len, dependent_launch=bool(a.dependent_launch), tp_group=dist.group.WORLD, tp_reduce=a.tp_reduce, prefetch_next=bool(a.prefetch_next))
        a.tp_reduce = eng.tp_reduce                                  # what actually runs (push needs layout 2 bf16)
    else:
        weights = DecoderWeights.synthetic(cfg, layout=a.layout, elem=a.elem, seed=rank if world > 1 else 0)
        eng = DecodeEngine(weights, max_len=max_len, dependent_launch=bool(a.dependent_launch), side_tables=bool(a.side_tables), prefetch_next=bool(a.prefetch_next))
    trace("weights built")
    if dist is not None: torch.cuda.synchronize(); dist.barrier()    # ranks start their first kernels together (bounded waits inside)
    eng.capture()
    trace("graph captured")
    g = torch.Generator().manual_seed(1234 + (0 if tp or world == 1 else rank))
    prompt = torch.randint(0, cfg.vocab, (a.prompt,), generator=g)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None: dist.barrier()
        torch.cuda.synchronize()

    # ---- value: K graph replays, device-timed ----
    barrier()
    eng.prefill(prompt)
    trace("prefill done")
    for _ in range(a.warmup): eng._run()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps): eng._run()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    trace("timed region done")
    clocks = sampler.stop() if sampler else None
    eng._check_status()                                               # position inside the cache, no bounded wait gave up
    ids = eng.log[a.warmup: a.warmup + a.steps].cpu().tolist()
    sha = hashlib.sha256(",".join(str(int(t)) for t in ids).encode()).hexdigest()[:16]
    # ---- e2e: host token in, host token out, every step ----
    barrier()
    eng.prefill(prompt)
    tok = int(eng.cur.item())
    for _ in range(a.warmup): tok = eng.step(tok)
    barrier()
    w0 = time.perf_counter()
    for _ in range(a.steps): tok = eng.step(tok)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - w0) * 1e3
    trace("e2e done")
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank != 0:                          # rank 0 alone measures the kernel roofline and the CPU baseline; the others wait for it
        finish(eng, dist)
        return
    trace("reduced over ranks")
    # ---- roofline of the dominant kernel: the matrix kind with the largest share of the step's matvec time ----
    peak, peak_kind = measured_peak()
    shares = matvec_shares(eng, weights, cfg)
    per_token = {k: us * n for k, (us, _, n, _) in shares.items()}
    top = max(per_token, key=per_token.get)
    us, nbytes, count, walked = shares[top]
    w = weights.lm_head if top == "lm_head" else weights.layers[0][top]
    small = a.layout == 0 and -(-w.out_features // 8) * -(-w.in_features // 512) <= 2 * L.SM_COUNT * 32      # the single-launch small-matrix kernel
    name = token_kernel_name(w.layout, a.elem, small)
    achieved = nbytes / (us * 1e-6) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get((name, w.in_features))
    roofline = {"bound": "hbm", "kernel": "%s (fused decode-matvec), %s %dx%d layout %d%s" % (name, top, w.out_features, w.in_features, w.layout, " (this rank's shard)" if tp else ""),
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None if ratio is None else ratio * nbytes,
                "bytes_per_launch": nbytes, "us_per_launch": us, "share_of_matvec_time": per_token[top] / sum(per_token.values()),
                "bytes_walked_per_replay": walked,
                "matvec_us": {k: round(v[0], 2) for k, v in shares.items()}, "matvec_frac": {k: round(v[1] / (v[0] * 1e-6) / 1e9 / peak, 3) for k, v in shares.items()},
                "matvec_ms_per_token": sum(per_token.values()) / 1e3,
                "model_bytes_per_token": weights.bytes_per_token(), "model_frac_of_roofline": weights.bytes_per_token() / (ms / a.steps * 1e-3) / 1e9 / peak}
    cpu = None
    if not a.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        sample = CpuSample(cfg, a.layout, 1 if a.elem == "fp8" else 0)
        cpu = {"value": 1.0 / min(sample.seconds_per_token(threads) for _ in range(2)), "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample.what}
    streams = 1 if (tp or world == 1) else world          # sequences decoded at once
    line = {"metric": "decode_tokens_per_s", "value": streams * a.steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": scaling_of(a, world), "vs_baseline": None, "dtype": a.elem, "data": "synthetic",
            "config": workload(a, cfg, world),
            "e2e": {"value": streams * a.steps / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": a.steps * eng.launches_per_step, "launches_per_step": eng.launches_per_step,
            "tokens_sha16": sha, "tokens_head": [int(t) for t in ids[:8]],
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu}
    print(json.dumps(line), flush=True)
    finish(eng, dist)


if __name__ == "__main__":
    main()
