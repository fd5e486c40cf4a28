"""vLLM general plugin: puts the libstrix_b200 kernels (sm_100a, B200) behind vLLM's
own kernel-selection points.

The counterpart of the reference's python/strix_vllm package
(python/strix_vllm/__init__.py:137-199), with its gate moved from ROCm / gfx1151
to CUDA compute capability 10.x and its hook points those of vLLM 0.22:

    int8    compressed-tensors W8A8 int8 linears    -> _POSSIBLE_INT8_KERNELS[CUDA]
    fp8     block-scaled / per-channel FP8 linears   -> _POSSIBLE_FP8_BLOCK_KERNELS,
                                                        _POSSIBLE_FP8_KERNELS
    moe     FP8 block-scaled experts                 -> fused_moe.oracle.fp8 selector
    attn    int8_per_token_head / bf16 paged attention, KV-cache write
                                                     -> a registered attention backend
    dense_w8  int8 decode copies of bf16 linears (opt-in: STRIX_ENABLE=dense_w8)

`register()` is the `vllm.general_plugins` entry point: it runs in every vLLM
process, possibly more than once, and does nothing off a B200. STRIX_DISABLE=all
(or a comma list of the names above, or of single swaps such as attn_prefill)
keeps vLLM's own kernels.
"""

from __future__ import annotations

import os

_registered = False


def _env_names(var: str) -> set[str]:
    return {s.strip() for s in os.environ.get(var, "").split(",") if s.strip()}


def disabled(op: str) -> bool:
    names = _env_names("STRIX_DISABLE")
    return "all" in names or op in names


def on_b200() -> bool:
    """CUDA platform with a compute-capability 10.x device (the build target)."""
    try:
        from vllm.platforms import current_platform
    except Exception:  # noqa: BLE001
        return False
    if not current_platform.is_cuda():
        return False
    cap = current_platform.get_device_capability()
    return cap is not None and cap.major == 10


def register() -> None:
    global _registered
    if _registered:
        return
    _registered = True
    from vllm.logger import init_logger

    logger = init_logger(f"vllm.{__name__}")
    if not on_b200():
        logger.info("libstrix_b200: no sm_100 device, plugin inactive")
        return
    if disabled("all"):
        logger.info("libstrix_b200: disabled by STRIX_DISABLE=all")
        return
    import libstrix_b200  # noqa: F401  (loads torch.ops.strix in this process)

    from strix_vllm import attn, dense_w8, fp8, int8, moe

    int8.register()
    fp8.register()
    moe.register()
    attn.register()
    dense_w8.register()          # opt-in: STRIX_ENABLE=dense_w8
    logger.info("libstrix_b200: plugin registered")
