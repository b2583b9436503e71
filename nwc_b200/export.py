"""Command line: NWC checkpoint -> plain bf16 Transformers checkpoint with bit-identical weights.

    python -m nwc_b200.export CHECKPOINT OUT_DIR [--device cuda]

Same role and arguments as the reference's `python -m nwc.export` (reference: nwc/export.py)."""
import argparse
import sys


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m nwc_b200.export", description="decode an NWC checkpoint back to bf16")
    ap.add_argument("checkpoint", help="NWC checkpoint: a local directory or a Hugging Face repo id")
    ap.add_argument("out", help="output directory (model.safetensors, config and tokenizer files)")
    ap.add_argument("--device", default="cuda", help="GPU that decodes (default cuda)")
    a = ap.parse_args(argv)
    from .checkpoint import export_bf16
    export_bf16(a.checkpoint, a.out, device=a.device)
    return 0


if __name__ == "__main__":
    sys.exit(main())
