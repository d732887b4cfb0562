"""Launch options accepted by the kernel launchers.

The reference passes compiler flags as extra keyword arguments on ``kernel[grid](...)``; they are
the field names of its HexagonOptions dataclass (qcom_hexagon_backend/backend/hexagon_options.py:16-107).
None of them changes what a hand-written CUDA kernel computes, so the launchers accept every one of
these names and ignore the value; a keyword that merely looks like an option (``enable*``,
``scratch``, ``*_scratch``) but is not a known field is ignored with a warning, as the reference
does (qcom_hexagon_backend/backend/triton_hexagon_launcher.py:606-622).
"""
from __future__ import annotations

import warnings

HEXAGON_OPTION_FIELDS = frozenset({
    "allow_fp8e4nv", "allowed_dot_input_precisions", "arch_triple", "arch_features", "device_type",
    "vectorize", "vector_length", "num_threads", "data_layout", "num_warps", "num_stages", "num_ctas",
    "shared", "cluster_dims", "supported_fp8_dtypes", "sanitize_overflow", "debug", "name",
    "instrumentation_mode", "htp_kernel_gen", "target_artifact", "iterations", "fusion",
    "fusionAllowRecompute", "fusionDoMultiUse", "enableBufferization", "enableCollapseAddressSpace",
    "enableConvTiling", "enableDoubleBuffering", "convTileSizes", "enableConvertToHexagonmem",
    "enableHexagonmemCopyToDMA", "enableHexKL", "hexKLMode", "enableMultiThreading",
    "enableThreadedDispatch", "enableSCFThreading", "enableSplitReduction", "enableSplitReduceGeneric",
    "enableVectorization", "enableVTCMTiling", "scratch", "enableHVXInlining", "enableSCFLoopUnroll",
    "enableConversionToFp16", "enableSeedLayoutConversions", "tileSizes",
    "lowerConstantsInSeparateSharedObjects", "enableLWP", "disableLWPLoop", "LWPloopDepth",
    "deviceCleanup",
})

_VALID_ARTIFACTS = {"ttir", "ttsharedir", "llir", "o", "so"}


def split_options(kwargs: dict, known_params) -> tuple[dict, dict]:
    """Splits call kwargs into (kernel arguments, launch options).

    Raises ValueError for an invalid ``target_artifact`` (hexagon_options.py:109-116) and TypeError
    for a keyword that is neither a kernel parameter nor option-like.
    """
    args, opts, suspicious = {}, {}, []
    for k, v in kwargs.items():
        if k in known_params:
            args[k] = v
        elif k in HEXAGON_OPTION_FIELDS:
            opts[k] = v
        elif k == "scratch" or k.startswith("enable") or k.endswith("_scratch"):
            suspicious.append(k)
        else:
            raise TypeError(f"unexpected keyword argument '{k}'")
    if "target_artifact" in opts and opts["target_artifact"] not in _VALID_ARTIFACTS:
        raise ValueError(
            f"Invalid target_artifact '{opts['target_artifact']}'. Must be one of: "
            + ", ".join(sorted(_VALID_ARTIFACTS))
        )
    if suspicious:
        warnings.warn("Unsupported runtime options ignored: " + ", ".join(sorted(suspicious)), stacklevel=3)
    return args, opts
