"""nwc_b200 -- B200-native NWC (Neural Weight Compression) decode engine.

Transformer weights stay losslessly entropy-coded in HBM (bf16, or weight-only fp8 e4m3 with a per-channel scale;
on-disk formats v9 / v10 / v11) and are decoded in registers inside hand-written sm_100a kernels.  Same public API
as the reference package:

    from nwc_b200 import fuse, convert, save_pretrained, load_pretrained, export_bf16
    fuse(model); convert(model)                 # nn.Linear -> NWCLinear on the GPU
    save_pretrained(model, "dir"); model = load_pretrained("dir"); export_bf16("dir", "plain")
"""
__version__ = "0.1.0"

from .weight import NWCWeight, fits, choose_block, quantize_fp8, ref_fp8_matvec                    # noqa: F401
from .modules import NWCLinear, NWCEmbedding, convert, fuse, RefFP8Linear, convert_ref_fp8          # noqa: F401
from .checkpoint import save_pretrained, load_pretrained, export_bf16                                # noqa: F401

__all__ = ["NWCWeight", "NWCLinear", "NWCEmbedding", "convert", "fuse", "fits", "choose_block", "quantize_fp8",
           "save_pretrained", "load_pretrained", "export_bf16", "__version__"]
