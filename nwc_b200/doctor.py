"""Command line self-check: is this machine able to run the library, and does a round trip come out right?

    python -m nwc_b200.doctor [--shape 1000x2048]

Counterpart of the reference's `python -m nwc.doctor` (reference: nwc/doctor.py:18-110) for this library: it reports
the GPU and the kernel library, then encodes one random matrix on the GPU in every layout and element type and checks
the three things a user relies on - decoded weights bit-identical, gathered rows bit-identical, token matvec equal to a
float64 product within one bf16 rounding - and that no bounded wait inside a kernel gave up.  Exit code 0 = ready."""
import argparse
import sys


def checks(M, K):
    """Yields (ok, what, detail) rows."""
    try:
        import torch
    except ImportError:
        yield False, "torch", "not installed"; return
    yield True, "torch", f"{torch.__version__}, CUDA build {torch.version.cuda}"
    if not torch.cuda.is_available():
        yield False, "cuda device", "torch.cuda.is_available() is False: no usable GPU or a driver older than torch's CUDA build"; return
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    free, total = torch.cuda.mem_get_info()
    yield (props.major, props.minor) == (10, 0), "cuda device", f"{props.name}, sm_{props.major}{props.minor}, {props.multi_processor_count} SMs, {free / 1e9:.1f} of {total / 1e9:.1f} GB free (the library is built for sm_100a only)"
    try:
        from . import _lib as L
        from .weight import NWCWeight
    except (ImportError, OSError) as e:
        yield False, "kernel library", f"{e}"; return
    yield True, "kernel library", f"{L.LIB_PATH} (format v{L.VERSION}, {L.SM_COUNT} SMs prepared)"
    g = torch.Generator().manual_seed(0)
    w = (torch.exp(0.3 * torch.randn(M, 1, generator=g)) * 0.02 * torch.randn(M, K, generator=g)).to(torch.bfloat16)
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    ids = torch.tensor([0, M - 1, M // 2])
    for elem in ("bf16", "fp8"):
        for layout in (0, 1, 2):
            try:
                c = NWCWeight(w, elem=elem, layout=layout)
                want = w if elem == "bf16" else c.dequant_fp8()[0].to(torch.bfloat16).cpu()          # fp8: the stored codes
                full = want.double() if c.scale is None else want.double() * c.scale.cpu().double()[:, None]
                ref = full @ x.double()
                y = c.linear_bf16(x.cuda(), None).cpu().double()
                problems = []
                if elem == "bf16" and not torch.equal(c.dequant().cpu(), w): problems.append("decoded weights differ")
                if not torch.equal(c.gather(ids.cuda()).cpu(), c.dequant().cpu()[ids]): problems.append("gathered rows differ")
                if (y - ref).abs().max().item() > 2.0 ** -7 * ref.abs().max().item() + 1e-6: problems.append("token matvec off")
                if L.lib.nwc_kernel_status(1): problems.append("a bounded wait inside a kernel gave up")
                yield not problems, f"round trip {elem} layout {layout}", ("; ".join(problems) if problems else
                                                                          f"{M} x {K}: decode and gather bit-exact, matvec within bf16 rounding, {8 * c.bytes / c.n:.2f} bits per weight")
            except (RuntimeError, ValueError) as e:
                yield False, f"round trip {elem} layout {layout}", str(e)
    for mod, why in (("transformers", "convert / load_pretrained on Hugging Face models"), ("safetensors", "reading and writing checkpoints")):
        try:
            __import__(mod); yield True, mod, "installed"
        except ImportError:
            yield None, mod, f"not installed (needed for {why})"


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m nwc_b200.doctor", description="environment and round-trip self-check")
    ap.add_argument("--shape", default="1000x2048", help="rows x columns of the test matrix")
    a = ap.parse_args(argv)
    M, K = (int(v) for v in a.shape.lower().split("x"))
    rows = list(checks(M, K))
    width = max(len(r[1]) for r in rows)
    for ok, what, detail in rows:
        print(f"[{'ok' if ok else ('warn' if ok is None else 'FAIL')}] {what.ljust(width)}  {detail}")
    failed = [r for r in rows if r[0] is False]
    print(f"\n{len(failed)} problem(s)." if failed else "\nReady.")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
