"""Kernel table of libstrix_b200: which entry point serves which op at which geometry.

Same contract as the reference's python/strix/registry.py (Kernel :87, select
:930, explain :918, geometries :895, kernels, ops, selections, Range :65):

  * `select(op, **geometry)` returns the NAME of the first row of `op` whose
    every constraint key was passed and is satisfied, else `None` - the caller
    then keeps its default path. Every query is recorded for `selections()`.
  * a constraint is a single required value (also a *geometry point*), a tuple
    of allowed values, or a `Range` bound;
  * `geometries(op, *keys, **where)` collects the points of the rows that accept
    `where`, so a plugin can derive its shape gate from the table.

The rows below describe the sm_100a kernels actually built in csrc/; shapes the
reference built for gfx1151 but that have no kernel here are absent, so
`select` answers `None` for them.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

_SHORT = {
    torch.bfloat16: "bf16",
    torch.float16: "fp16",
    torch.float32: "fp32",
    torch.float8_e4m3fn: "fp8_e4m3",
    torch.int8: "int8",
}


def _norm(value: Any) -> Any:
    """torch dtypes (or their 'torch.xxx' spelling) become the table's short names."""
    if isinstance(value, torch.dtype):
        return _SHORT.get(value, str(value))
    if isinstance(value, str) and value.startswith("torch."):
        return _SHORT.get(getattr(torch, value[len("torch."):], None), value)
    return value


@dataclass(frozen=True)
class Range:
    """Inclusive integer bound; `Range(lo=6)` reads "6 or more"."""

    lo: int | None = None
    hi: int | None = None

    def covers(self, got: Any) -> bool:
        if isinstance(got, bool) or not isinstance(got, int):
            return False
        return (self.lo is None or got >= self.lo) and (self.hi is None or got <= self.hi)

    def __str__(self) -> str:
        if self.lo is not None and self.hi is not None:
            return f"in {self.lo}..{self.hi}"
        return f">= {self.lo}" if self.lo is not None else f"<= {self.hi}"


def _satisfies(want: Any, got: Any) -> bool:
    if isinstance(want, Range):
        return want.covers(got)
    if isinstance(want, tuple):
        return got in want
    return got == want


def _describe(want: Any) -> str:
    if isinstance(want, Range):
        return str(want)
    return f"in {want}" if isinstance(want, tuple) else f"== {want}"


@dataclass(frozen=True)
class Kernel:
    name: str
    op: str
    doc: str
    constraints: dict[str, Any] = field(default_factory=dict)
    spec: dict[str, Any] = field(default_factory=dict)  # informational only

    def check(self, geometry: dict[str, Any]) -> str | None:
        """None when the row takes the geometry, else the first failed key."""
        for key, want in self.constraints.items():
            if key not in geometry:
                return f"{key} not given"
            got = _norm(geometry[key])
            if not _satisfies(want, got):
                return f"{key}={got}, needs {_describe(want)}"
        return None

    def accepts(self, partial: dict[str, Any]) -> bool:
        """Whether a partial geometry lies inside this row."""
        for key, value in partial.items():
            if key not in self.constraints:
                return False
            if not _satisfies(self.constraints[key], _norm(value)):
                return False
        return True


def _decode_row(head_dim: int, gqa: int, doc: str) -> Kernel:
    return Kernel(
        "attn_decode_bf16",
        "attn_decode",
        doc,
        {
            "head_dim": head_dim,
            "gqa": gqa,
            "queries": 1,
            "dtype": "bf16",
            "kv_dtype": ("int8",),
            "window": (True, False),
            "sinks": (True, False),
        },
        {"tile_keys": 16, "mma": "m16n8k16 f16, keys as M", "bound": "hbm"},
    )


_GATES = ("silu", "gelu_tanh")
_STREAM_SPEC = {
    "tile": "16 weight rows per warp x 8-token tiles, K blocks of 128",
    "staging": "cp.async ring, 4 stages",
    "bound": "hbm (weight stream) at small token counts",
}


def _moe_row(name: str, op: str, doc: str, **constraints: Any) -> Kernel:
    base = {"silu_mul": (True, False), "activation": _GATES}
    return Kernel(name, op, doc, {**base, **constraints}, dict(_STREAM_SPEC))


_MOE_ROWS = [
    Kernel(
        "moe_gemm_fp8_sorted", "moe_gemm_fp8",
        "e4m3 experts x e4m3 activations laid out by sorted position, on tcgen05 "
        "(kind::f8f6f4, fp32 partial sums in TMEM folded per 128-wide K block with "
        "the block scale x the token's scale): 128 weight rows are the MMA's M, the "
        "m-block's tokens its N; both operands arrive by TMA",
        {"dtype": "bf16", "activation_dtype": "fp8_e4m3", "weight_dtype": "fp8_e4m3",
         "weight_bits": 8, "quant": "fp8", "group_size": (0, 128), "layout": "sorted",
         "block_m": (16, 32, 64, 128), "silu_mul": (True, False), "activation": _GATES},
        {"tile": "128 weight rows x block_m tokens (block_m <= 64); 128 tokens x 256 weight rows "
                 "(block_m 128); K blocks of 128",
         "pipeline": "TMA producer thread, issuing thread, metadata warp, 8-16 folding warps; "
                     "one commit per K block, persistent grid",
         "bound": "hbm (weight stream) at small token counts, L2 -> shared memory at 4k tokens"},
    ),
    Kernel("moe_act_quant_fp8_sorted", "moe_act_quant_fp8",
           "e4m3 activations per (row, 128 group) written in sorted order (row p = token "
           "sorted_ids[p] / top_k, zeros for padding), the input layout of moe_gemm_fp8_sorted",
           {"dtype": ("bf16", "fp16"), "activation_dtype": "fp8_e4m3", "group_size": 128,
            "layout": "sorted"}),
    Kernel("moe_act_quant_fp8_scatter", "moe_act_quant_fp8",
           "the sorted-layout e4m3 quantiser by scatter: a token is quantised once and stored "
           "at the sorted positions of its top_k slots (inverse permutation from the align kernel)",
           {"dtype": ("bf16", "fp16"), "activation_dtype": "fp8_e4m3", "group_size": 128,
            "layout": "sorted", "scatter": True}),
    Kernel("moe_align_block_size_pos", "moe_align",
           "moe_align_block_size that also writes the inverse permutation (slot -> sorted position)",
           {"experts": Range(1, 8192), "block_m": Range(1, 1024), "positions": True}),
    _moe_row(
        "moe_gemm_fp8_w8a8", "moe_gemm_fp8",
        "e4m3 experts x e4m3 activations (one fp32 scale per token and 128-wide K "
        "group): the MMA runs on the raw bytes, block or channel weight scales and "
        "the activation scale fold into the fp32 partial sums per K block",
        dtype="bf16", activation_dtype="fp8_e4m3", weight_dtype="fp8_e4m3", weight_bits=8,
        quant="fp8", group_size=(0, 128),
    ),
    _moe_row(
        "moe_gemm_fp8", "moe_gemm_fp8",
        "e4m3 experts x bf16 activations; weights widened exactly in registers, "
        "scales applied to fp32 sums",
        dtype="bf16", weight_dtype="fp8_e4m3", weight_bits=8, quant="fp8", group_size=(0, 128),
    ),
    _moe_row(
        "moe_gemm_fp8_raw", "moe_gemm_fp8",
        "e4m3 experts x fp16 activations (fp16 out under the fused gate, bf16 otherwise)",
        dtype="fp16", weight_dtype="fp8_e4m3", weight_bits=8, quant="fp8", group_size=(0, 128),
    ),
    _moe_row(
        "moe_gemm_w8a16", "moe_gemm_w8a16",
        "int8 experts with one scale per output channel x bf16 activations",
        dtype="bf16", weight_dtype="int8", weight_bits=8, quant="int8", group_size=(0,),
    ),
    _moe_row(
        "moe_gemm_bf16", "moe_gemm",
        "bf16 experts x bf16 activations, fused gate epilogue",
        dtype="bf16", weight_dtype="bf16", quant=None,
    ),
    Kernel("moe_act_quant_i8", "moe_act_quant_i8",
           "int8 activations per (row, 128 group): s = amax / 127, q = rint(x / s)",
           {"dtype": ("bf16", "fp16"), "activation_dtype": "int8", "group_size": 128}),
    Kernel("moe_act_quant_fp8", "moe_act_quant_fp8",
           "e4m3 activations per (row, 128 group): s = amax / 448",
           {"dtype": ("bf16", "fp16"), "activation_dtype": "fp8_e4m3", "group_size": 128}),
    Kernel("moe_topk_softmax", "moe_router",
           "fp32 softmax -> top-k (ties to the lower index) -> renormalise, one warp per token",
           {"experts": Range(1, 1024), "top_k": Range(1, 32), "dtype": "fp32"}),
    Kernel("moe_align_block_size", "moe_align",
           "stable per-expert permutation padded to block_m; one CTA per expert, single launch",
           {"experts": Range(1, 8192), "block_m": Range(1, 1024)}),
    Kernel("moe_sum", "moe_sum", "fp32 sum of the top-k expert rows, one bf16 rounding",
           {"dtype": "bf16"}),
]

KERNELS: list[Kernel] = [
    Kernel("_umma_tile", "umma_tile",
           "one-CTA tcgen05 tile product, the layout probe of the sm_100a kernels",
           {"weight_dtype": ("int8", "fp8_e4m3"), "m": 128}),
    *_MOE_ROWS,
    # ------------------------------------------------- 4-bit experts, dense 4-/8-bit
    Kernel("moe_gemm_w4a16", "moe_gemm_w4a16",
           "int4 experts (nibble - 8, low nibble = even k) with 16-bit scales per 32/64/128 "
           "elements x bf16 activations; weights widened in registers to scaled bf16",
           {"silu_mul": (True, False), "dtype": "bf16", "weight_dtype": "uint8", "weight_bits": 4,
            "quant": "wna16", "group_size": (32, 64, 128), "activation": _GATES},
           dict(_STREAM_SPEC)),
    Kernel("moe_gemm_mxfp4", "moe_gemm_mxfp4",
           "MXFP4 experts (e2m1 nibbles, e8m0 scale per 32 elements, byte 0 = zero block) x bf16 "
           "activations; the decode is exact in bf16. K % 32 == 0 (hidden 2880 is covered)",
           {"silu_mul": (True, False), "dtype": "bf16", "weight_dtype": "uint8", "weight_bits": 4,
            "quant": "mxfp4", "group_size": 32, "scale_dtype": "e8m0", "activation": _GATES},
           dict(_STREAM_SPEC)),
    Kernel("moe_gemm_mxfp4_sorted", "moe_gemm_mxfp4",
           "MXFP4 experts on tcgen05 for m-blocks of 128 tokens in sorted order: weights decoded "
           "to bf16 operand tiles on the way (byte-permute table, exact), bf16 x bf16 -> f32 MMAs "
           "of 128 x 256 x 16, the whole K accumulated in TMEM",
           {"silu_mul": (True, False), "dtype": "bf16", "weight_dtype": "uint8", "weight_bits": 4,
            "quant": "mxfp4", "group_size": 32, "scale_dtype": "e8m0", "activation": _GATES,
            "layout": "sorted", "block_m": 128},
           {"tile": "128 tokens x 256 weight rows, K blocks of 64",
            "pipeline": "TMA producer, 8 transform warps, issuing thread, 4 epilogue warps",
            "bound": "tensor"}),
    Kernel("moe_permute_bf16", "moe_permute",
           "bf16 rows into sorted order by scatter (inverse permutation from the align kernel)",
           {"dtype": "bf16", "layout": "sorted"}),
    Kernel("moe_permute_rows", "moe_permute",
           "rows of any element type (whole 16-byte chunks, e.g. e4m3 bytes followed by their "
           "fp32 group scales) into sorted order by scatter; rows without a position are skipped",
           {"dtype": ("uint8", "bf16", "fp8_e4m3"), "layout": "sorted", "bytes": True}),
    Kernel("mxfp4_gemv", "mxfp4_gemv", "MXFP4 W4A16 at 1-8 rows (the dense form of moe_gemm_mxfp4)",
           {"weight_bits": 4, "group_size": 32, "dtype": "bf16", "m_max": 8}, dict(_STREAM_SPEC)),
    Kernel("mxfp4_wmma_gemm", "mxfp4", "MXFP4 W4A16 dense GEMM, optional bias [N] or [M, N]",
           {"weight_bits": 4, "group_size": 32, "dtype": "bf16", "scale_dtype": "e8m0"},
           dict(_STREAM_SPEC)),
    Kernel("w4a8_wmma_gemm", "w4a16",
           "int4 weights (ExLlama word order) x activations quantised to int8 per (row, 128 "
           "group) inside the op: s8 MMAs, int32-exact per group, fp32 fold; the dense twin of "
           "moe_gemm_w4a8 on the weight-streaming kernel. Scales per 32 elements ([K/32, N]) "
           "run with bf16 activations on the w4a16 kernel instead",
           {"weight_bits": 4, "group_size": (0, 32, 128), "dtype": "bf16", "rows": Range(hi=128),
            "act_quant": "int8"}, dict(_STREAM_SPEC)),
    Kernel("w4a16_wmma_gemm", "w4a16",
           "int4 W4A16 dense GEMM (ExLlama word order), optional bias; the dense form of "
           "moe_gemm_w4a16 on the weight-streaming kernel",
           {"weight_bits": 4, "group_size": (32, 64, 128), "dtype": "bf16",
            "scale_dtype": ("bf16", "fp16")}, dict(_STREAM_SPEC)),
    Kernel("mxfp4_dequant", "mxfp4_dequant", "MXFP4 -> bf16 [N, K], byte-exact",
           {"weight_bits": 4, "group_size": 32, "dtype": "bf16"}),
    Kernel("w4a16_dequant", "w4a16_dequant", "int4 (ExLlama word order) -> bf16 [N, K]",
           {"weight_bits": 4, "group_size": (32, 64, 128), "dtype": "bf16"}),
    Kernel("fp8_dequant", "fp8_dequant", "e4m3 x fp32 block or channel scales -> bf16 [N, K]",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128), "dtype": "bf16"}),
    Kernel("w8a16_skinny_gemm", "w8a16",
           "excess-128 byte weights x bf16 activations at 1-8 rows, scales per channel or per "
           "(row, 32 / 64 / 128 group); the dense form of the grouped weight-streaming kernel",
           {"weight_bits": 8, "group_size": (0, 32, 64, 128), "rows": Range(hi=8), "dtype": "bf16"},
           dict(_STREAM_SPEC)),
    Kernel("fp8_skinny_gemm", "fp8", "e4m3 weights x bf16 activations at 1-8 rows",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128),
            "rows": Range(hi=8), "dtype": "bf16"}, dict(_STREAM_SPEC)),
    Kernel("fp8_wmma_gemm", "fp8", "e4m3 weights x bf16 activations, any row count",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128),
            "rows": Range(lo=9), "dtype": "bf16"}, dict(_STREAM_SPEC)),
    Kernel("fp8_wmma_gemm_raw", "fp8", "e4m3 weights (exact) x fp16 activations, scales on the sums",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128),
            "rows": Range(lo=1), "dtype": "fp16"}, dict(_STREAM_SPEC)),
    Kernel("moe_gemm_w4a8", "moe_gemm_w4a8",
           "int4 experts x int8 activations (one fp32 scale per row and 128 group): s8 x s8 "
           "MMAs, int32-exact per group, fp32 fold with the two scales",
           {"silu_mul": (True, False), "dtype": "bf16", "activation_dtype": "int8",
            "weight_dtype": "uint8", "weight_bits": 4, "quant": "wna16", "group_size": (128,),
            "activation": _GATES}, dict(_STREAM_SPEC)),
    Kernel("w8a8_wmma_gemm", "w8a16",
           "excess-128 byte weights x activations quantised to int8 per (row, 128 group) inside "
           "the op, int32-exact per group, fp32 group-scale fold. K % 128 == 0",
           {"weight_bits": 8, "group_size": (0, 128), "rows": Range(lo=9), "dtype": "bf16"},
           dict(_STREAM_SPEC)),
    *[Kernel(name, op, f"bench-only: {name[:-4]} pinned to one token tile (cfg 0 / 1 / 2 = 16 / 32 / "
             "64 tokens x 128 weight rows) instead of the choice by row count",
             cons, {"cfg": "0..2"})
      for name, op, cons in (
          ("fp8_wmma_gemm_cfg", "fp8_tile_sweep",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128), "dtype": "bf16"}),
          ("fp8_wmma_gemm_raw_cfg", "fp8_tile_sweep",
           {"weight_bits": 8, "weight_dtype": "fp8_e4m3", "group_size": (0, 128), "dtype": "fp16"}),
          ("mxfp4_wmma_gemm_cfg", "mxfp4_tile_sweep",
           {"weight_bits": 4, "group_size": 32, "dtype": "bf16"}),
          ("w8a8_wmma_gemm_cfg", "w8a8_tile_sweep",
           {"weight_bits": 8, "group_size": (0, 128), "rows": Range(lo=1), "dtype": "bf16"}),
      )],
    # ---------------------------------------------------------- dense GEMMs
    Kernel("w8a8_int8_gemm", "w8a8",
           "dense W8A8 INT8 GEMM on tcgen05 kind::i8 (int32 sums in TMEM, exact): int8 "
           "activations with one fp32 scale per token, int8 weights with one per output "
           "channel. K % 128 == 0. Up to 64 rows the weights are the MMA's M dimension "
           "and the kernel is a weight stream; beyond that 128 x 256 tiles",
           {"weight_bits": 8, "weight_dtype": "int8", "act_dtype": "int8", "group_size": 0,
            "dtype": "bf16"},
           {"tile": "128 weights x 16/32/64 tokens (rows <= 64), 128 tokens x 256 weights",
            "pipeline": "4 producer warps (cp.async ring, 128B swizzle), 1 issuing thread, "
                        "4 epilogue warps, 2 TMEM accumulators, persistent grid"}),
    Kernel("act_quant_token_i8", "act_quant_token",
           "dynamic symmetric per-token int8 activations (scale = absmax / 127), the input "
           "form of w8a8_int8_gemm",
           {"dtype": ("bf16", "fp16"), "activation_dtype": "int8", "group_size": 0}),
    # ------------------------------------------------------------ attention
    Kernel("kv_write_i8", "kv_write",
           "new K/V rows quantised per (token, KV head) into the int8 paged cache with their "
           "fp32 scales; separate scale tensors or the packed layout with the scale inline "
           "after each head's bytes (through strides)",
           {"dtype": ("bf16", "fp16"), "kv_dtype": "int8", "head_dim": Range(8, 512),
            "rule": ("reference", "vllm")},
           {"unit": "one warp per (token, head, K or V)", "bound": "hbm"}),
    _decode_row(
        128, 8,
        "one query per sequence over an int8_per_token_head paged cache: 16-key "
        "tiles streamed global->registers, exact int8->fp16 widening by byte "
        "permutes, K scale on the score, V scale on P, split-KV partials merged "
        "by a reduce kernel, sinks after the merge",
    ),
    _decode_row(128, 4, "as (128, 8); the unused query-head columns of the MMA are zero"),
    _decode_row(128, 2, "as (128, 8); the unused query-head columns of the MMA are zero"),
    _decode_row(128, 1, "as (128, 8); the unused query-head columns of the MMA are zero"),
    _decode_row(256, 8, "head 256 GQA 8, four warps per CTA (255 registers)"),
    _decode_row(256, 6, "head 256 GQA 6 (two MMA columns idle)"),
    _decode_row(256, 2, "head 256 GQA 2 (sliding layers)"),
    Kernel("attn_decode_bf16", "attn_decode",
           "every other int8 geometry: GQA ratios 3, 5, 7 on the split-KV kernel; head 64 or 512 "
           "and ratios above 8 have no split-KV kernel - the prefill kernel in its decode form (the "
           "query heads of a KV head as the rows of one sequence, all at the last position: a KV "
           "head is read once, in one pass)",
           {"head_dim": (64, 128, 256, 512), "gqa": Range(1, 64), "queries": 1, "dtype": "bf16",
            "kv_dtype": ("int8",), "window": (True, False), "sinks": (True, False)},
           {"tile": "64 queries x 64 / 32 keys", "bound": "hbm"}),
    *[Kernel("attn_decode_bf16", "attn_decode",
             "bf16 KV cache, split-KV: one warp per KV head, per-warp cp.async ring of 16-key "
             "tiles, K and V^T fragments by ldmatrix, bf16 m16n8k16 MMAs (rows on 16-byte "
             "boundaries, GQA 1-8; other layouts go through the prefill kernel with one query "
             "per sequence)",
             {"head_dim": hd, "gqa": Range(1, 64), "queries": 1, "dtype": "bf16",
              "kv_dtype": ("bf16",), "window": (True, False), "sinks": (True, False)},
             {"tile_keys": 16, "mma": "m16n8k16 bf16, keys as M", "bound": "hbm"})
      for hd in (128, 64)],
    Kernel("attn_decode_bf16", "attn_decode",
           "bf16 KV cache at head 256, two KV heads per CTA so that two 96 KB rings share an SM "
           "(GQA above 8: the prefill kernel's decode form)",
           {"head_dim": 256, "gqa": Range(1, 64), "queries": 1, "dtype": "bf16",
            "kv_dtype": ("bf16",), "window": (True, False), "sinks": (True, False)},
           {"tile_keys": 16, "mma": "m16n8k16 bf16, keys as M", "bound": "hbm"}),
    Kernel("attn_decode_bf16", "attn_decode",
           "bf16 KV cache at head 512 (the reference's GQA 8 row; GQA 1-8): the head's dims split "
           "over a pair of warps, each with its half of every K and V row in its own ring; the pair "
           "adds its score partials through shared memory once per 16-key tile (GQA above 8: the "
           "prefill kernel's decode form)",
           {"head_dim": 512, "gqa": Range(1, 64), "queries": 1, "dtype": "bf16",
            "kv_dtype": ("bf16",), "window": (True, False), "sinks": (True, False)},
           {"tile_keys": 16, "mma": "m16n8k16 bf16, keys as M", "bound": "hbm"}),
    *[Kernel(
        "attn_prefill_bf16", "attn_prefill",
        "causal paged flash attention over ragged sequences: 64 queries x one head per CTA, "
        "64-key tiles double-buffered with cp.async, int8 caches widened once per tile to fp16 "
        "(K scale on the score, V scale on P), mma.sync m16n8k16 through ldmatrix",
        {"head_dim": hd, "gqa": Range(1, 64), "dtype": "bf16", "kv_dtype": ("bf16", "int8"),
         "split_kv": (True, False), "window": (True, False), "causal": True,
         "sinks": (True, False)},
        {"tile": "64 queries x 64 keys", "mma": "m16n8k16 f16 (int8 KV) / bf16", "bound": "tensor"},
    ) for hd in (128, 64)],
    Kernel(
        "attn_prefill_bf16", "attn_prefill",
        "head 256 (the reference's GQA 6 / 8 / 2 rows and any other ratio): the same mma.sync "
        "kernel over 64 x 32 tiles, two CTAs per SM, with the query tile in shared memory (its "
        "fragments re-read by ldmatrix per key tile) because 128 accumulator registers leave no "
        "room for it",
        {"head_dim": 256, "gqa": Range(1, 64), "dtype": "bf16", "kv_dtype": ("bf16", "int8"),
         "split_kv": (True, False), "window": (True, False), "causal": True,
         "sinks": (True, False)},
        {"tile": "64 queries x 32 keys", "mma": "m16n8k16 f16 (int8 KV) / bf16", "bound": "tensor"},
    ),
    Kernel(
        "attn_prefill_bf16", "attn_prefill",
        "head 512 (the reference's GQA 8 row and any other ratio): 64 queries x 32 keys, eight "
        "warps - each group of 16 queries belongs to a pair of warps that own 256 of the head's "
        "dims each (their part of Q, K, V and O) and add their score partials through shared memory",
        {"head_dim": 512, "gqa": Range(1, 64), "dtype": "bf16", "kv_dtype": ("bf16", "int8"),
         "split_kv": (True, False), "window": (True, False), "causal": True,
         "sinks": (True, False)},
        {"tile": "64 queries x 32 keys", "mma": "m16n8k16 f16 (int8 KV) / bf16", "bound": "tensor"},
    ),
]

_POINT_TYPES = (int, bool, str)
_selections: dict[tuple, dict[str, Any]] = {}


def ops() -> dict[str, list[str]]:
    """op -> kernel names implementing it, in priority order, without repeats."""
    table: dict[str, list[str]] = {}
    for row in KERNELS:
        names = table.setdefault(row.op, [])
        if row.name not in names:
            names.append(row.name)
    return table


def geometries(op: str, *keys: str, **where: Any) -> set[tuple]:
    """Shape points `op` covers as tuples of `keys`; `where` narrows the rows first.

    A row whose value for one of `keys` is a set or a Range is not a point and
    contributes nothing.
    """
    points: set[tuple] = set()
    for row in KERNELS:
        if row.op != op or not row.accepts(where):
            continue
        values = [row.constraints.get(k) for k in keys]
        if all(isinstance(v, _POINT_TYPES) for v in values):
            points.add(tuple(_norm(v) for v in values))
    return points


def explain(op: str, **geometry: Any) -> list[dict[str, Any]]:
    """One entry per row of `op`: its name, whether it matches, and why not."""
    report = []
    for row in KERNELS:
        if row.op != op:
            continue
        reason = row.check(geometry)
        report.append({"name": row.name, "ok": reason is None, "reason": reason})
    return report


def select(op: str, **geometry: Any) -> str | None:
    report = explain(op, **geometry)
    hit = next((r["name"] for r in report if r["ok"]), None)
    query = tuple(sorted((k, _norm(v)) for k, v in geometry.items()))
    record = _selections.get((op, query))
    if record is None:
        why = None if hit else ("; ".join(r["reason"] for r in report) or "no kernel")
        record = {"op": op, "query": dict(query), "kernel": hit, "reason": why, "count": 0}
        _selections[(op, query)] = record
    record["count"] += 1
    return hit


def selections() -> list[dict[str, Any]]:
    """Every distinct `select` query so far with its answer and hit count."""
    return list(_selections.values())


def kernels() -> list[dict[str, Any]]:
    return [
        {
            "name": row.name,
            "op": row.op,
            "doc": row.doc,
            "constraints": dict(row.constraints),
            "spec": dict(row.spec),
        }
        for row in KERNELS
    ]
