"""FP8 block-scaled experts of vLLM's fused MoE layers on B200.

vLLM decides the routing (its router, shared-expert and parallel-config logic
stay untouched) and hands hidden states, top-k ids and weights to an "experts"
object; this one runs permute -> e4m3 activation quantisation per (token, 128)
-> gate-up GEMM with the fused gate -> quantisation -> down GEMM x routing weight
-> sum on the tcgen05 kernels of libstrix_b200 (libstrix_b200.moe.experts_fp8_w8a8).
It takes the place of the reference's StrixFp8Experts
(python/strix_vllm/moe.py:827-1014), hooked the same way: the FP8 oracle's
backend_to_kernel_cls answers with this class for the Triton backend. Anything it
does not cover (expert maps, biases, LoRA, other activations or scale layouts)
goes to the parent class, i.e. to vLLM's own Triton experts.
"""

from __future__ import annotations

import torch

from strix_vllm import disabled

_FUSED = {"silu": "silu", "gelu_tanh": "gelu_tanh"}


def block_scales(w: torch.Tensor, s: torch.Tensor | None) -> torch.Tensor | None:
    """fp32 [E, N/128, K/128] or [E, N] scales for e4m3 experts w [E, N, K], or None
    when the layout is not one the kernels take."""
    if s is None:
        return None
    e, n, k = w.shape
    if s.dim() == 3 and s.size(1) != n:
        if tuple(s.shape) != (e, n // 128, k // 128):
            return None
        return s.to(torch.float32).contiguous()
    if s.numel() != e * n:
        return None
    return s.reshape(e, n).to(torch.float32).contiguous()


def covered(hidden_states, w1, w2, s1, s2, activation: str, expert_map, a1q_scale,
            has_bias: bool, has_lora: bool) -> list[str]:
    """Names of the checks that fail (empty: the strix path runs)."""
    checks = {
        "2d": hidden_states.dim() == 2,
        "act": hidden_states.dtype == torch.bfloat16 and a1q_scale is None,
        "w_fp8": w1.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn,
        "scales": s1 is not None and s2 is not None,
        "bias": not has_bias,
        "lora": not has_lora,
        "expert_map": expert_map is None,
        "activation": activation in _FUSED,
        "k128": w1.size(2) % 128 == 0 and w2.size(2) % 128 == 0,
        "n128": w1.size(1) % 256 == 0 and w2.size(1) % 128 == 0,
        "aligned": w1.stride(1) % 16 == 0 and w2.stride(1) % 16 == 0,
    }
    return [name for name, ok in checks.items() if not ok]


def experts_class():
    from vllm.model_executor.layers.fused_moe.experts.triton_moe import TritonExperts

    class StrixFp8Experts(TritonExperts):
        """FP8 W8A8 block-scaled experts on tcgen05; falls back to the parent."""

        @property
        def expects_unquantized_inputs(self) -> bool:
            # the permute-and-quantise kernel of the strix path wants the bf16 rows
            return True

        def apply(self, output, hidden_states, w1, w2, topk_weights, topk_ids, activation,
                  global_num_experts, expert_map, a1q_scale, a2_scale, workspace13, workspace2,
                  expert_tokens_meta, apply_router_weight_on_input):
            from libstrix_b200 import moe as smoe

            act = getattr(activation, "value", activation)
            s1, s2 = block_scales(w1, self.w1_scale), block_scales(w2, self.w2_scale)
            bad = covered(hidden_states, w1, w2, s1, s2, act, expert_map, a1q_scale,
                          self.w1_bias is not None or self.w2_bias is not None,
                          getattr(self, "_lora_context", None) is not None)
            if bad or apply_router_weight_on_input:
                from vllm.logger import init_logger

                init_logger("vllm.strix").warning_once(
                    "moe_fp8 falls back to vLLM's experts: " + ", ".join(bad or ["router weight on input"]))
                if a1q_scale is None and hidden_states.dtype == torch.bfloat16 \
                        and self.quant_config.use_fp8_w8a8:
                    # the parent expects quantised input when it does the FP8 product
                    from vllm.model_executor.layers.fused_moe.utils import moe_kernel_quantize_input

                    hidden_states, a1q_scale = moe_kernel_quantize_input(
                        hidden_states, None, self.quant_config.quant_dtype,
                        self.quant_config.per_act_token_quant, self.quant_config.block_shape)
                return super().apply(output, hidden_states, w1, w2, topk_weights, topk_ids, activation,
                                     global_num_experts, expert_map, a1q_scale, a2_scale, workspace13,
                                     workspace2, expert_tokens_meta, apply_router_weight_on_input)
            smoe.experts_fp8_w8a8(hidden_states, topk_weights, topk_ids, w1, s1, w2, s2, out=output,
                                  activation=_FUSED[act])
            return None

    return StrixFp8Experts


def register() -> None:
    if disabled("moe") or disabled("moe_fp8"):
        return
    from vllm.model_executor.layers.fused_moe.oracle import fp8 as fp8_oracle

    if getattr(fp8_oracle.backend_to_kernel_cls, "strix_orig", None) is not None:
        return                                           # already hooked in this process
    cls = experts_class()
    orig = fp8_oracle.backend_to_kernel_cls

    def backend_to_kernel_cls(backend, _orig=orig, _cls=cls):
        if backend == fp8_oracle.Fp8MoeBackend.TRITON:
            return [_cls]
        return _orig(backend)

    backend_to_kernel_cls.strix_orig = orig
    # the selector imports the experts class inside its body, so the name to rebind
    # is the selector itself
    fp8_oracle.backend_to_kernel_cls = backend_to_kernel_cls
