"""Paged attention and the KV-cache write of vLLM's Triton attention backend on
B200, for bf16 and int8_per_token_head caches.

A subclass of vLLM 0.22's TritonAttentionImpl, as the reference's
StrixTritonAttentionImpl is (python/strix_vllm/attn.py:205-334): `forward` sends
single-token batches to strix.attn_decode and batches with queries of
PREFILL_MIN_QUERY tokens or more to strix.attn_prefill, `do_kv_cache_update`
writes int8 caches with strix.kv_write_int8, everything else (and every geometry
strix.select() does not cover) runs the parent's kernels. Which (head_dim, GQA)
pairs are covered comes from the kernel table, so the gate cannot drift from the
kernels that exist. vLLM 0.22 stores an int8_per_token_head cache as
[blocks, 2, block_size, Hkv, D + 4] with each head's fp32 scale after its bytes:
libstrix_b200.packed_int8_kv_views carves the four views the kernels take.
"""

from __future__ import annotations

import torch

from strix_vllm import disabled

# batches whose longest query has at least this many tokens run the prefill kernel;
# shorter multi-token batches (speculative verify) stay on vLLM's kernel
PREFILL_MIN_QUERY = 16


def covers(kind: str, head_dim: int, gqa: int, kv_dtype: str, window: bool, sinks: bool) -> bool:
    """Whether the kernel table has a row for this attention geometry."""
    import libstrix_b200 as strix

    if kind == "decode":
        return strix.select("attn_decode", head_dim=head_dim, gqa=gqa, queries=1, dtype="bf16",
                            kv_dtype=kv_dtype, window=window, sinks=sinks) is not None
    return strix.select("attn_prefill", head_dim=head_dim, gqa=gqa, dtype="bf16", kv_dtype=kv_dtype,
                        split_kv=False, window=window, causal=True, sinks=sinks) is not None


def kv_views(kv_cache: torch.Tensor, head_size: int):
    """(key_cache, value_cache, k_scale, v_scale) views of vLLM's cache tensor."""
    import libstrix_b200 as strix

    if kv_cache.dtype == torch.int8:
        return strix.packed_int8_kv_views(kv_cache)
    key_cache, value_cache = kv_cache.unbind(1)
    return key_cache[..., :head_size], value_cache[..., :head_size], None, None


def impl_class():
    from vllm.v1.attention.backends.triton_attn import TritonAttentionImpl

    class StrixTritonAttentionImpl(TritonAttentionImpl):
        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            window = tuple(self.sliding_window) if self.sliding_window is not None else (-1, -1)
            plain = (self.alibi_slopes is None and not self.logits_soft_cap
                     and (window == (-1, -1) or (window[0] >= 0 and window[1] == 0)))
            gqa = self.num_heads // self.num_kv_heads
            has_window, has_sinks = window[0] >= 0, self.sinks is not None
            self._strix = {
                (kind, dt): plain and not disabled(f"attn_{kind}")
                and covers(kind, self.head_size, gqa, dt, has_window, has_sinks)
                for kind in ("decode", "prefill") for dt in ("bf16", "int8")
            }
            self._window_left = window[0]

        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            if kv_cache.dtype != torch.int8 or disabled("kv_write") or key is None:
                return super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
            import libstrix_b200 as strix

            kc, vc, ks, vs = strix.packed_int8_kv_views(kv_cache)
            n = slot_mapping.numel()
            strix.kv_write_int8(key[:n], value[:n], kc, vc, ks, vs, slot_mapping, rule="vllm")

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output,
                    output_scale=None, output_block_scale=None):
            md = attn_metadata
            dt = {torch.int8: "int8", torch.bfloat16: "bf16"}.get(kv_cache.dtype)
            max_q = md.max_query_len if md is not None else 0
            kind = "decode" if max_q == 1 else "prefill" if max_q >= PREFILL_MIN_QUERY else None
            if (md is None or dt is None or kind is None or not self._strix[(kind, dt)]
                    or output_scale is not None or output_block_scale is not None
                    or query.dtype != torch.bfloat16 or getattr(md, "use_cascade", False)
                    or getattr(md, "mm_prefix_range_tensor", None) is not None):
                return super().forward(layer, query, key, value, kv_cache, attn_metadata, output,
                                       output_scale, output_block_scale)
            import libstrix_b200 as strix

            n = md.num_actual_tokens
            kc, vc, ks, vs = kv_views(kv_cache, self.head_size)
            out = output[:n].view(n, self.num_heads, self.head_size)
            q = query[:n].view(n, self.num_heads, self.head_size)
            if kind == "decode":
                strix.attn_decode(out, q, kc, vc, md.seq_lens[:n], md.block_table[:n], self.scale, 0,
                                  self._window_left, ks, vs, self.sinks)
            else:
                strix.attn_prefill(out, q, kc, vc, md.query_start_loc, md.seq_lens, md.block_table,
                                   self.scale, 1, self._window_left, ks, vs, self.sinks)
            return output

    return StrixTritonAttentionImpl


def backend_class():
    from vllm.v1.attention.backends.triton_attn import TritonAttentionBackend

    impl = impl_class()

    class StrixTritonAttentionBackend(TritonAttentionBackend):
        @staticmethod
        def get_impl_cls():
            return impl

    return StrixTritonAttentionBackend


def __getattr__(name: str):
    # the backend registry imports the class by dotted path, lazily
    if name == "StrixTritonAttentionBackend":
        globals()[name] = backend_class()
        return globals()[name]
    raise AttributeError(name)


def register() -> None:
    if disabled("attn"):
        return
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.TRITON_ATTN, "strix_vllm.attn.StrixTritonAttentionBackend")
