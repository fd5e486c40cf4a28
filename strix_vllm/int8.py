"""W8A8 int8 linears (compressed-tensors int-quantized checkpoints) on B200.

vLLM's contract for these layers: per-channel int8 weights [N, K] and dynamic
symmetric per-token int8 activations. Here the activations are quantised by
strix::act_quant_token_i8 and the product runs on tcgen05 (kind::i8, exact int32
sums in tensor memory) through strix::w8a8_int8_gemm. The reference's kernel for
the same layers (python/strix_vllm/int8.py:41-83) re-quantises per 128-element
group inside its GEMM and needs the weights as excess-128 bytes; this one keeps
the checkpoint's signed bytes and vLLM's per-token rule.
"""

from __future__ import annotations

import torch

from strix_vllm import disabled

_registered = False


def apply_w8a8(x_2d: torch.Tensor, w_q: torch.Tensor, w_s: torch.Tensor,
               bias: torch.Tensor | None) -> torch.Tensor:
    x_q, x_s = torch.ops.strix.act_quant_token_i8(x_2d.contiguous())
    out = torch.ops.strix.w8a8_int8_gemm(x_q, x_s, w_q, w_s)
    out = out if x_2d.dtype == torch.bfloat16 else out.to(x_2d.dtype)
    return out if bias is None else out + bias


def _apply_fake(x_2d, w_q, w_s, bias):
    return x_2d.new_empty((x_2d.size(0), w_q.size(0)))


def kernel_class():
    """The linear-kernel class (built lazily: vLLM must be importable)."""
    from vllm.model_executor.kernels.linear.scaled_mm.triton import TritonInt8ScaledMMLinearKernel

    class StrixW8A8LinearKernel(TritonInt8ScaledMMLinearKernel):
        """vLLM's int8 scaled-MM contract with the GEMM on tcgen05."""

        @classmethod
        def can_implement(cls, c) -> tuple[bool, str | None]:
            if c.is_static_input_scheme:
                return False, "strix W8A8 takes dynamic per-token activations"
            if not c.is_channelwise:
                return False, "strix W8A8 takes per-channel weight scales"
            if not c.input_symmetric:
                return False, "strix W8A8 takes symmetric activations"
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            w_name, s_name = self.layer_param_names[0], self.layer_param_names[1]
            w, s = getattr(layer, w_name), getattr(layer, s_name)
            if w.dtype != torch.int8 or w.dim() != 2:
                raise RuntimeError(f"strix W8A8 takes int8 [N, K] weights, got {w.dtype} {tuple(w.shape)}")
            if w.size(1) % 128:
                raise RuntimeError(f"strix W8A8 needs K % 128 == 0, got K = {w.size(1)}")
            setattr(layer, w_name, torch.nn.Parameter(w.data.contiguous(), requires_grad=False))
            setattr(layer, s_name, torch.nn.Parameter(s.data.float().reshape(-1).contiguous(),
                                                      requires_grad=False))

        def apply_weights(self, layer: torch.nn.Module, x: torch.Tensor,
                          bias: torch.Tensor | None = None) -> torch.Tensor:
            w_q = getattr(layer, self.layer_param_names[0])
            w_s = getattr(layer, self.layer_param_names[1])
            x_2d = x.reshape(-1, x.shape[-1])
            fn = getattr(torch.ops.vllm, "strix_w8a8_apply", None) if _registered else None
            out = (fn or apply_w8a8)(x_2d, w_q, w_s, bias if bias is None else bias.contiguous())
            return out.reshape(*x.shape[:-1], w_q.size(0))

    return StrixW8A8LinearKernel


def register() -> None:
    """Puts the kernel at the front of CUDA's int8 candidates (idempotent)."""
    global _registered
    if _registered or disabled("int8"):
        return
    from vllm.model_executor.kernels.linear import _POSSIBLE_INT8_KERNELS
    from vllm.platforms import PlatformEnum
    from vllm.utils.torch_utils import direct_register_custom_op

    direct_register_custom_op(op_name="strix_w8a8_apply", op_func=apply_w8a8, mutates_args=[],
                              fake_impl=_apply_fake)
    _registered = True
    kernels = _POSSIBLE_INT8_KERNELS.setdefault(PlatformEnum.CUDA, [])
    if not any(k.__name__ == "StrixW8A8LinearKernel" for k in kernels):
        kernels.insert(0, kernel_class())
