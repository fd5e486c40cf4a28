"""dense_w8: int8 decode copies of unquantised bf16 linear weights.

A bf16 model streams every dense weight once per decode step. This keeps the
bf16 weight for large batches and adds a symmetric int8 copy (excess-128 bytes,
one scale per 128-element group, or per channel when K is not a multiple of 128)
that batches of up to 8 rows read through strix::w8a16_skinny_gemm: half the
bytes per step for +50 % of the dense weight memory. The counterpart of the
reference's python/strix_vllm/dense_w8.py; like there it changes numerics and
memory, so it is off unless STRIX_ENABLE names it, every copy is checked once
against the bf16 product, and the copies stop at STRIX_DENSE_W8_MAX_GB.
"""

from __future__ import annotations

import os

import torch

from strix_vllm import _env_names, disabled

MAX_ROWS = 8                     # rows strix::w8a16_skinny_gemm takes
_GROUP = 128
_MAX_BYTES = float(os.environ.get("STRIX_DENSE_W8_MAX_GB", "12")) * 2 ** 30
_BY_WEIGHT: dict[int, tuple] = {}    # weight.data_ptr() -> (w_q, w_s, group)
_used_bytes = 0


def enabled() -> bool:
    return "dense_w8" in _env_names("STRIX_ENABLE") and not disabled("dense_w8")


def quantize(w: torch.Tensor):
    """bf16 [N, K] -> (excess-128 bytes uint8 [N, K], 16-bit scales [N, K / 128] or [N],
    group): symmetric, s = amax / 127 per group, q = round(w / s) + 128."""
    n, k = w.shape
    group = _GROUP if k % _GROUP == 0 else 0
    wf = w.float()
    g = wf.view(n, k // group, group) if group else wf.view(n, 1, k)
    # the scale is rounded to the 16-bit type it is stored in BEFORE the weights are
    # divided by it, so that the kernel multiplies by exactly the divisor used here
    s = (g.abs().amax(-1) / 127.0).clamp_min(1e-12).to(w.dtype).contiguous()
    q = torch.round(g / s.float()[..., None]).clamp(-127, 127).view(n, k) + 128
    return q.to(torch.uint8).contiguous(), (s if group else s.reshape(n)), group


def lookup(weight: torch.Tensor):
    """The int8 decode copy of a converted layer's bf16 weight, if any."""
    return _BY_WEIGHT.get(weight.data_ptr())


def add_copy(weight: torch.Tensor) -> bool:
    """Builds and registers the int8 copy of `weight` (bf16 [N, K] on the GPU) if the
    kernel takes the shape, the budget allows it and a random row agrees with bf16."""
    global _used_bytes
    n, k = weight.shape
    if weight.dtype != torch.bfloat16 or k % 128 or n % 16 or not weight.is_cuda:
        return False
    if _used_bytes + weight.numel() > _MAX_BYTES:
        return False
    w_q, w_s, group = quantize(weight)
    x = torch.randn(1, k, device=weight.device, dtype=torch.bfloat16)
    got = torch.ops.strix.w8a16_skinny_gemm(w_q, x, w_s, None, 0, group).float()
    ref = torch.nn.functional.linear(x, weight).float()
    if not torch.isfinite(got).all() or (got - ref).abs().max() > 3e-2 * ref.abs().max().clamp_min(1e-6):
        return False
    _BY_WEIGHT[weight.data_ptr()] = (w_q, w_s, group)
    _used_bytes += weight.numel()
    return True


def apply(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x @ weight^T (+ bias): up to MAX_ROWS rows read the int8 copy, larger batches bf16."""
    x_2d = x.reshape(-1, x.shape[-1])
    copy = lookup(weight) if x_2d.size(0) <= MAX_ROWS and x.dtype == torch.bfloat16 else None
    if copy is None:
        return torch.nn.functional.linear(x, weight, bias)
    w_q, w_s, group = copy
    out = torch.ops.strix.w8a16_skinny_gemm(w_q, x_2d.contiguous(), w_s,
                                            None if bias is None else bias.contiguous(), 0, group)
    return out.reshape(*x.shape[:-1], weight.size(0))


def register() -> None:
    """Wraps vLLM's UnquantizedLinearMethod: copies are made after the weights are
    loaded, and apply() consults them. Off unless STRIX_ENABLE=dense_w8."""
    if not enabled():
        return
    from vllm.model_executor.layers.linear import UnquantizedLinearMethod

    if getattr(UnquantizedLinearMethod.apply, "strix_orig", None) is not None:
        return
    orig_apply = UnquantizedLinearMethod.apply
    orig_load = UnquantizedLinearMethod.process_weights_after_loading

    def process_weights_after_loading(self, layer):
        orig_load(self, layer)
        add_copy(layer.weight.data)

    def apply_with_copy(self, layer, x, bias=None):
        if lookup(layer.weight) is not None and x.reshape(-1, x.shape[-1]).size(0) <= MAX_ROWS:
            return apply(x, layer.weight, bias)
        return orig_apply(self, layer, x, bias)

    apply_with_copy.strix_orig = orig_apply
    UnquantizedLinearMethod.process_weights_after_loading = process_weights_after_loading
    UnquantizedLinearMethod.apply = apply_with_copy
