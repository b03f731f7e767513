"""B200-native Metis NVFP4 linear-layer path.

    fp4_post_b200.cabi     ctypes binding of include/metis_nvfp4.h
    fp4_post_b200.ops      tensor-level wrappers (quantize, RMSNorm->quantize, GEMM, ...)
    fp4_post_b200.Metis    host-side mirror of the reference's Metis package
    fp4_post_b200.grpo     MetisArgs / replace_linear_with_metis

`install_reference_aliases()` makes the reference's own import paths (`Metis.Metis.bitlinear`,
`Metis.Metis.quant`, `Metis.models.llama`, `grpo.grpo`) resolve to this package, so the
reference's scripts and tests run unchanged on top of it.
"""
import importlib
import sys

__version__ = "0.1.0"


def install_reference_aliases() -> None:
    names = {
        "Metis": "fp4_post_b200.Metis",
        "Metis.Metis": "fp4_post_b200.Metis.Metis",
        "Metis.Metis.quant": "fp4_post_b200.Metis.Metis.quant",
        "Metis.Metis.bitlinear": "fp4_post_b200.Metis.Metis.bitlinear",
        "Metis.models": "fp4_post_b200.Metis.models",
        "Metis.models.llama": "fp4_post_b200.Metis.models.llama",
        "grpo": "fp4_post_b200.grpo",
        "grpo.grpo": "fp4_post_b200.grpo.grpo",
    }
    for alias, real in names.items():
        sys.modules.setdefault(alias, importlib.import_module(real))
