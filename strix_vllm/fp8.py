"""FP8 (e4m3) linears on B200: block-scaled (128 x 128 fp32 scales) and
per-channel checkpoints as W8A16 - the activations stay bf16, the weights are
widened exactly inside the kernel (strix::fp8_skinny_gemm up to 8 rows,
strix::fp8_wmma_gemm beyond). Follows the reference's kernels for the same
layers (python/strix_vllm/fp8.py:121-262); its row padding and compute-unit
hints are gfx1151 tuning and are not carried over.
"""

from __future__ import annotations

import torch

from strix_vllm import disabled

_BLOCK = 128
_registered = False


def apply_fp8(x_2d: torch.Tensor, w: torch.Tensor, scales: torch.Tensor,
              bias: torch.Tensor | None) -> torch.Tensor:
    """x bf16 [M, K] x e4m3 [N, K] with fp32 scales [ceil(N/128), K/128] or [N]."""
    x_2d = x_2d.contiguous()
    if x_2d.size(0) <= 8:
        return torch.ops.strix.fp8_skinny_gemm(w, x_2d, scales, bias, 0)
    out = torch.ops.strix.fp8_wmma_gemm(w, x_2d, scales)
    return out if bias is None else out + bias


def _apply_fake(x_2d, w, scales, bias):
    return x_2d.new_empty((x_2d.size(0), w.size(0)))


def _apply(x_2d, w, scales, bias):
    fn = getattr(torch.ops.vllm, "strix_fp8_apply", None) if _registered else None
    return (fn or apply_fp8)(x_2d, w, scales, bias)


def block_kernel_class():
    from vllm.model_executor.kernels.linear.scaled_mm.BlockScaledMMLinearKernel import (
        Fp8BlockScaledMMLinearKernel,
    )
    from vllm.model_executor.utils import replace_parameter

    class StrixFp8BlockScaledMMKernel(Fp8BlockScaledMMLinearKernel):
        # W8A16: no dynamic activation quantisation in front of the GEMM
        apply_input_quant = False

        @classmethod
        def is_supported(cls, compute_capability=None):
            from strix_vllm import on_b200

            return (True, None) if on_b200() else (False, "strix FP8 W8A16 is built for sm_100")

        @classmethod
        def can_implement(cls, config):
            ok, why = super().can_implement(config)
            if not ok:
                return ok, why
            if tuple(config.weight_quant_key.scale.group_shape) != (_BLOCK, _BLOCK):
                return False, "needs 128x128 weight blocks"
            if config.out_dtype != torch.bfloat16:
                return False, f"needs bf16 activations, got {config.out_dtype}"
            if config.weight_shape[-1] % _BLOCK:
                return False, f"K={config.weight_shape[-1]} must be a multiple of 128"
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            super().process_weights_after_loading(layer)
            params = self._get_layer_params(layer)
            w, bs = params.weight, params.block_scale
            if w.dtype != torch.float8_e4m3fn:
                raise RuntimeError(f"strix FP8 takes float8_e4m3fn, got {w.dtype}")
            replace_parameter(layer, params.WEIGHT, w.contiguous())
            replace_parameter(layer, params.block_scale_attr, bs.float().contiguous())

        def apply_weights(self, layer, x, bias=None, **kwargs):
            params = self._get_layer_params(layer)
            x_2d = x.reshape(-1, x.shape[-1])
            out = _apply(x_2d, params.weight, params.block_scale, bias)
            return out.reshape(*x.shape[:-1], params.weight.size(0))

        def apply_block_scaled_mm(self, A, B, As, Bs):
            raise NotImplementedError("strix FP8 overrides apply_weights")

    return StrixFp8BlockScaledMMKernel


def channel_kernel_class():
    from vllm.model_executor.kernels.linear.scaled_mm.ScaledMMLinearKernel import (
        FP8ScaledMMLinearKernel,
    )
    from vllm.model_executor.layers.quantization.utils.quant_utils import GroupShape
    from vllm.model_executor.utils import replace_parameter

    class StrixFp8ChannelMMKernel(FP8ScaledMMLinearKernel):
        """W8A16 for per-channel FP8 weights (bf16 activations in)."""

        @classmethod
        def is_supported(cls, compute_capability=None):
            from strix_vllm import on_b200

            return (True, None) if on_b200() else (False, "strix FP8 W8A16 is built for sm_100")

        @classmethod
        def can_implement(cls, config):
            wkey = config.weight_quant_key
            if wkey.dtype != torch.float8_e4m3fn:
                return False, f"needs float8_e4m3fn weights, got {wkey.dtype}"
            if tuple(wkey.scale.group_shape) != tuple(GroupShape.PER_CHANNEL):
                return False, "needs per-channel weight scales"
            if config.out_dtype not in (None, torch.bfloat16):
                return False, f"needs bf16 activations, got {config.out_dtype}"
            if config.weight_shape[-1] % 64:
                return False, f"K={config.weight_shape[-1]} must be a multiple of 64"
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            w_name, s_name = self.layer_param_names[0], self.layer_param_names[1]
            w, s = getattr(layer, w_name), getattr(layer, s_name)
            if w.dtype != torch.float8_e4m3fn:
                raise RuntimeError(f"strix FP8 takes float8_e4m3fn, got {w.dtype}")
            if w.size(0) != self.config.weight_shape[0]:     # handed over as a (K, N) view
                w = w.t()
            n = w.size(0)
            s = s.float().reshape(-1).contiguous()
            if s.numel() != n:
                raise RuntimeError(f"per-channel scale has {s.numel()} values for N={n}")
            replace_parameter(layer, w_name, w.contiguous())
            replace_parameter(layer, s_name, s)

        def apply_weights(self, layer, x, bias=None, **kwargs):
            w = getattr(layer, self.layer_param_names[0])
            s = getattr(layer, self.layer_param_names[1])
            x_2d = x.reshape(-1, x.shape[-1])
            return _apply(x_2d, w, s, bias).reshape(*x.shape[:-1], w.size(0))

        def apply_scaled_mm(self, **kwargs):
            raise NotImplementedError("strix FP8 overrides apply_weights")

    return StrixFp8ChannelMMKernel


def register() -> None:
    global _registered
    if _registered or disabled("fp8"):
        return
    import vllm.model_executor.kernels.linear as linear_kernels
    from vllm.platforms import PlatformEnum
    from vllm.utils.torch_utils import direct_register_custom_op

    direct_register_custom_op(op_name="strix_fp8_apply", op_func=apply_fp8, mutates_args=[],
                              fake_impl=_apply_fake)
    _registered = True
    block = linear_kernels._POSSIBLE_FP8_BLOCK_KERNELS.setdefault(PlatformEnum.CUDA, [])
    if not any(k.__name__ == "StrixFp8BlockScaledMMKernel" for k in block):
        block.insert(0, block_kernel_class())
    if disabled("fp8_channel"):
        return
    chan = linear_kernels._POSSIBLE_FP8_KERNELS.setdefault(PlatformEnum.CUDA, [])
    if not any(k.__name__ == "StrixFp8ChannelMMKernel" for k in chan):
        chan.insert(0, channel_kernel_class())
