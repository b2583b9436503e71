"""Benchmark of the NWC batch-1 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--model qwen3-0.6b] [--layout 0] [--elem bf16]

Workload (N = 1): a Qwen3-0.6B-architecture decoder with random-init weights of the reference's distribution
(W = r_i * 0.02 * z, r_i log-normal(0, 0.3), norms 1), compressed bf16 layout 0, batch 1, 32 random prompt ids, greedy
decode replayed as one CUDA graph per token.  A step is one decoded token.
  value     tokens/s of K graph replays, device-timed, nothing copied to or from the host inside the region
  e2e       the same through DecodeEngine.step(): token id from pinned host memory in, next token id back, every step
  roofline  the dominant kernel (the fused decode-matvec on the lm_head matrix, larger than L2) launched back to back:
            algorithmic bytes (the reference's own per-matrix byte count) / CUDA-event time, against the measured HBM peak
  cpu_baseline  the CPU oracle's fused decode+matvec on all host cores over a bounded sample (one decoder layer plus
            1/8 of the lm_head rows), extrapolated to a whole token
With N > 1 (torchrun, one rank per GPU) every rank decodes its own sequence on its own replica of the model: no
data-path collective, weak scaling; value = N * K / max-over-ranks time.
--impl reference runs the CPU path alone (rank 0), each step one pass over the bounded sample.
"""
import argparse
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
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--layout", type=int, default=0)
    ap.add_argument("--elem", default="bf16")
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default="", help="time one token matvec alone: lm_head | qkv | o | gate_up | down | MxK (small case for ncu)")
    ap.add_argument("--parallel", default="replicas", choices=["replicas", "tp"], help="N > 1: independent replicas (weak scaling) or tensor parallel with NCCL all-reduce (strong scaling)")
    ap.add_argument("--tp-reduce", default="peer", choices=["peer", "nccl"], help="--parallel tp: sum partial outputs with this library's NVLink peer-memory kernel or with NCCL")
    ap.add_argument("--dependent-launch", type=int, default=1, help="programmatic dependent launch between the decode-step kernels")
    return ap.parse_args()


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

def cpu_sample(cfg, layout, elem_code, threads, repeats=1):
    """Seconds per token of the CPU fused decode+matvec, extrapolated from one layer + 1/8 of the lm_head rows."""
    import numpy as np
    import oracle as O
    code = O.code_of(elem_code, layout)
    shapes = [("qkv", cfg.qkv_rows, cfg.hidden), ("o", cfg.hidden, cfg.n_q * cfg.head_dim), ("gate_up", 2 * cfg.intermediate, cfg.hidden),
              ("down", cfg.hidden, cfg.intermediate), ("lm_head/8", cfg.vocab // 8, cfg.hidden)]
    packed = []
    for i, (name, M, K) in enumerate(shapes):
        w, x = O.synth_weights(M, K, 1000 + i)
        src = w
        if elem_code: src, _ = O.quantize_fp8(w)
        packed.append((O.encode(src, code), O.bf16_to_f32(x)))
    times = []
    for _ in range(repeats):
        per = []
        for p, x in packed:
            t = time.perf_counter(); O.matvec_f32(p, x, threads=threads); per.append(time.perf_counter() - t)
        times.append(cfg.layers * sum(per[:4]) + 8.0 * per[4])
    return times, "1 decoder layer (qkv, o, gate_up, down) + 1/8 of the lm_head rows per pass, extrapolated to layers x layer + 8 x slice"


def run_reference(a, cfg):
    threads = os.cpu_count() or 1
    elem_code = 1 if a.elem == "fp8" else 0
    for _ in range(max(0, min(a.warmup, 1))): cpu_sample(cfg, a.layout, elem_code, threads)
    steps = max(1, min(a.steps, 8))
    times, what = cpu_sample(cfg, a.layout, elem_code, threads, repeats=steps)
    sec = statistics.mean(times)
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": 1.0 / sec, "unit": "tokens/s", "n_gpus": a.gpus, "steps": steps, "warmup": min(a.warmup, 1),
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": a.elem, "data": "synthetic",
            "config": workload(a, cfg, a.gpus, a.parallel == "tp"), "cpu_baseline": {"value": 1.0 / sec, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": what},
            "e2e": {"value": 1.0 / sec, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload(a, cfg, world=1, tp=False):
    """The `config` object; identical in both arms so that their lines can be compared key by key."""
    par = "1 GPU"
    if world > 1:
        par = ("tp%d: q/k/v, gate/up, lm_head split by rows, o/down by columns, partial sums added after o and down (%s)" % (world, "NVLink peer-memory kernel" if a.tp_reduce == "peer" else "NCCL all-reduce") if tp
               else "replicas x%d (no data-path collective)" % world)
    return {"workload": f"{cfg.name}-architecture decoder, random init, NWC {a.elem} layout {a.layout}, batch 1, {a.prompt} random prompt ids, greedy decode as a CUDA graph",
            "layers": cfg.layers, "hidden": cfg.hidden, "vocab": cfg.vocab,
            "l2_policy": "no flush: the compressed weights streamed per token and the lm_head matrix of the roofline leg are each larger than the 126 MB L2",
            "parallelism": par}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the lm_head kernel, from the ncu captures summarised
# under profiles/ (same command line as `--kernel lm_head`); other workloads report null
NCU_TRAFFIC = {("qwen3-0.6b", 0, "bf16"): 217.5e6, ("qwen3-0.6b", 2, "bf16"): 239.1e6}


def token_kernel_name(layout, elem):
    if layout == 0: return "prefix_ring_kernel_layout0"
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
    import torch
    from nwc_b200 import NWCWeight, _lib as L
    from nwc_b200.decode import synthetic_matrix
    shapes = {"lm_head": (cfg.vocab, cfg.hidden), "qkv": (cfg.qkv_rows, cfg.hidden), "o": (cfg.hidden, cfg.n_q * cfg.head_dim),
              "gate_up": (2 * cfg.intermediate, cfg.hidden), "down": (cfg.hidden, cfg.intermediate)}
    M, K = shapes[a.kernel] if a.kernel in shapes else tuple(int(v) for v in a.kernel.lower().split("x"))
    torch.cuda.set_device(0)
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
    print(json.dumps({"kernel": f"token matvec {M}x{K} {a.elem} layout {a.layout}", "launches_per_call": L.lib.nwc_linear_launches(nw.n, K, nw.code, 0), "us_per_call": ms * 1e3,
                      "bytes_per_call": nw.bytes, "bits_per_weight": 8 * nw.bytes / nw.n, "dense_bf16_gemv_us": None if dense_ms is None else dense_ms * 1e3,
                      "native_fp8_matvec_us": None if native_fp8_ms is None else native_fp8_ms * 1e3,
                      "roofline": {"bound": "hbm", "achieved": nw.bytes / ms / 1e6, "peak": peak, "peak_kind": kind, "unit": "GB/s", "frac": nw.bytes / ms / 1e6 / peak},
                      "note": "%d calls on %d rotating copies replayed as one CUDA graph, CUDA events around the replay (a call includes its finalize launch when it needs one)" % (reps, copies)}))


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
    from nwc_b200.decode import PRESETS  # the package import fails loudly when the CUDA library is missing
    cfg = PRESETS[a.model]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if a.impl == "reference":
        if rank == 0: run_reference(a, cfg)
        return
    if a.kernel:
        if rank == 0: kernel_only(a, cfg)
        return
    import torch
    from nwc_b200.decode import DecodeEngine, DecoderWeights
    from nwc_b200 import _lib as L
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    tp = a.parallel == "tp" and world > 1
    if tp and a.tp_reduce == "nccl": a.dependent_launch = 0         # NCCL kernels sit in the chain: keep plain stream order around them
    if tp:      # one model sharded over all ranks: same seed everywhere, every rank keeps its shard and decodes the same sequence
        weights = DecoderWeights.synthetic(cfg, layout=a.layout, elem=a.elem, seed=0, tp_rank=rank, tp_world=world)
        eng = DecodeEngine(weights, max_len=a.prompt + a.warmup + 2 * a.steps + 16, dependent_launch=bool(a.dependent_launch), tp_group=dist.group.WORLD, tp_reduce=a.tp_reduce)
    else:
        weights = DecoderWeights.synthetic(cfg, layout=a.layout, elem=a.elem, seed=rank)
        eng = DecodeEngine(weights, max_len=a.prompt + a.warmup + 2 * a.steps + 16, dependent_launch=bool(a.dependent_launch))
    trace("weights built")
    eng.capture()
    trace("graph captured")
    g = torch.Generator().manual_seed(1234 + (0 if tp else rank))
    prompt = torch.randint(0, cfg.vocab, (a.prompt,), generator=g)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None: dist.barrier()
        torch.cuda.synchronize()

    # ---- value: K graph replays, device-timed ----
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
    if int(eng.status.item()): raise RuntimeError("decode position left the KV cache")
    # ---- e2e: host token in, host token out, every step ----
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
    # ---- roofline of the dominant kernel: lm_head matvec back to back inside one graph ----
    peak, peak_kind = measured_peak()
    w = weights.lm_head
    reps = 20
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side): eng._linear(w, eng.xtmp, eng.logits)
    torch.cuda.current_stream().wait_stream(side)
    kg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(kg):
        for _ in range(reps): eng._linear(w, eng.xtmp, eng.logits)
    for _ in range(3): kg.replay()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record(); kg.replay(); k1.record(); torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / reps
    achieved = w.bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "%s (fused decode-matvec), lm_head %dx%d layout %d" % (token_kernel_name(w.layout, a.elem), w.out_features, w.in_features, w.layout),
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC.get((a.model, a.layout, a.elem)) if not tp else None,
                "bytes_per_launch": w.bytes, "us_per_launch": kernel_ms * 1e3,
                "model_bytes_per_token": weights.bytes_per_token(), "model_frac_of_roofline": weights.bytes_per_token() / (ms / a.steps * 1e-3) / 1e9 / peak}
    cpu = None
    if not a.no_cpu_baseline:
        threads = os.cpu_count() or 1
        times, what = cpu_sample(cfg, a.layout, 1 if a.elem == "fp8" else 0, threads, repeats=2)
        cpu = {"value": 1.0 / min(times), "unit": "tokens/s", "cores": threads, "kind": "port", "sample": what}
    streams = 1 if tp else world          # sequences decoded at once
    line = {"metric": "decode_tokens_per_s", "value": streams * a.steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": a.elem, "data": "synthetic",
            "config": workload(a, cfg, world, tp),
            "e2e": {"value": streams * a.steps / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": a.steps * eng.launches_per_step, "launches_per_step": eng.launches_per_step,
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu}
    print(json.dumps(line), flush=True)
    finish(eng, dist)


if __name__ == "__main__":
    main()
