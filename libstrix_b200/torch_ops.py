"""Registers the `torch.ops.strix.*` ops and binds each to its C-ABI entry point.

Schema strings are the reference's (csrc/torch_ops.cpp:179-304), implementation
key CUDA (csrc/torch_ops.cpp:306). An op body only validates what the C side
cannot see (dtypes, ranks), hands raw pointers, sizes and element strides to
libstrix_b200.so on the current CUDA stream, and allocates scratch with torch's
caching allocator. A failed check raises RuntimeError like TORCH_CHECK does.
There is no CPU implementation: calling an op with CPU tensors raises
NotImplementedError from the dispatcher.
"""

from __future__ import annotations

import os

import torch

from . import _lib

# Which prefill-attention kernel attn_prefill_bf16 runs: "auto" = the tcgen05 kernel
# where it covers the geometry, else the mma.sync kernel; "umma" / "mma" force one.
PREFILL_IMPL = os.environ.get("STRIX_PREFILL_IMPL", "auto")

_LIBRARY = torch.library.Library("strix", "DEF")
_registered: list[str] = []


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _define(schema: str, fake=None):
    """Decorator: define `schema` in namespace strix and use the function as its CUDA impl."""
    name = schema.split("(", 1)[0]

    def wrap(fn):
        _LIBRARY.define(schema)
        _LIBRARY.impl(name, fn, "CUDA")
        torch.library.register_fake(f"strix::{name}")(fake or (lambda *a, **k: None))
        _registered.append(name)
        return fn

    return wrap


def registered_ops() -> list[str]:
    return list(_registered)


# ----------------------------------------------------------------- attention

def group_queries(q: torch.Tensor, hkv: int) -> torch.Tensor:
    """[nseq, hq, d] -> contiguous [nseq * G, hkv, d]: row n * G + j, head h holds query
    head h * G + j (the layout strix_attn_decode_grouped_bf16 reads)."""
    nseq, hq, d = q.shape
    g = hq // hkv
    return q.reshape(nseq, hkv, g, d).transpose(1, 2).reshape(nseq * g, hkv, d).contiguous()


def ungroup_queries(og: torch.Tensor, nseq: int) -> torch.Tensor:
    """Inverse of group_queries: [nseq * G, hkv, d] -> [nseq, hkv * G, d]."""
    rows, hkv, d = og.shape
    g = rows // max(nseq, 1)
    return og.reshape(nseq, g, hkv, d).transpose(1, 2).reshape(nseq, hkv * g, d)



@_define(
    "attn_decode_bf16(Tensor(a!) out, Tensor q, Tensor key_cache, "
    "Tensor value_cache, Tensor seq_lens, Tensor block_table, float scale, "
    "int num_splits, int window_left=-1, Tensor? k_scale=None, "
    "Tensor? v_scale=None, Tensor? sinks=None) -> ()"
)
def attn_decode_bf16(
    out, q, key_cache, value_cache, seq_lens, block_table, scale, num_splits,
    window_left=-1, k_scale=None, v_scale=None, sinks=None,
):
    """Host side of strix_attn_decode_bf16; checks follow
    csrc/attn/attn_decode_bf16.hip:317-364 of the reference. num_splits = 0
    (an extension) selects fixed-length key segments."""
    _check(q.dim() == 3 and key_cache.dim() == 4 and value_cache.dim() == 4,
           "q [N, H, D], caches [blocks, block_size, Hkv, D]")
    d = q.size(-1)
    _check(q.dtype == torch.bfloat16 and q.stride(-1) == 1,
           "q must be bf16 with a contiguous head_dim")
    q8 = key_cache.dtype != torch.bfloat16
    _check(key_cache.dtype == (torch.int8 if q8 else torch.bfloat16)
           and value_cache.dtype == key_cache.dtype,
           "caches must both be bf16 or both int8")
    for t in (key_cache, value_cache):
        _check(t.size(-1) >= d and t.stride(-1) == 1,
               "cache head_dim must be at least q's, contiguous")
    if q8:
        _check(k_scale is not None and v_scale is not None, "int8 KV needs k_scale and v_scale")
        for t in (k_scale, v_scale):
            _check(t.dtype == torch.float32 and t.dim() == 3
                   and tuple(t.shape) == tuple(key_cache.shape[:3]),
                   "scales must be fp32 [blocks, block_size, Hkv]")
    _check(out.dtype == torch.bfloat16 and out.shape == q.shape and out.stride(-1) == 1,
           "out must match q")
    _check(seq_lens.dtype == torch.int32 and block_table.dtype == torch.int32
           and block_table.stride(1) == 1 and seq_lens.numel() >= q.size(0)
           and seq_lens.is_contiguous(),
           "int32 metadata")
    if sinks is not None:
        _check(sinks.dtype == torch.float32 and sinks.dim() == 1 and sinks.size(0) == q.size(1)
               and sinks.is_contiguous(), "sinks must be contiguous fp32 [Hq]")
    _check(0 <= num_splits <= 64, "num_splits in [1, 64]")
    bf16_rows_ok = not q8 and d in (64, 128, 256, 512) and q.size(1) // key_cache.size(2) <= 8 and all(
        st % 8 == 0 for t in (key_cache, value_cache) for st in t.stride()[:3]) and \
        key_cache.data_ptr() % 16 == 0 and value_cache.data_ptr() % 16 == 0
    gqa = q.size(1) // max(key_cache.size(2), 1)
    if (not q8 and not bf16_rows_ok) or (q8 and (d not in (128, 256) or gqa > 8)):
        # caches the split-KV decode kernels do not take (a GQA ratio above 8, int8 caches
        # at head 64 or 512, bf16 rows off 16-byte boundaries): the prefill kernel in its decode
        # form - the query heads of a KV head become the rows of one sequence, all at the
        # last position, so a KV head is read once
        nseq, hq, hkv = q.size(0), q.size(1), key_cache.size(2)
        _check(hkv > 0 and hq % hkv == 0, "Hq % Hkv")
        g = hq // hkv
        if nseq == 0:
            return
        qg = group_queries(q, hkv)
        og = torch.empty_like(qg)
        cu = torch.arange(0, (nseq + 1) * g, g, dtype=torch.int32, device=q.device)
        ks, vs = (k_scale, v_scale) if q8 else (None, None)
        with torch.cuda.device(q.device):
            _lib.call(
                "strix_attn_decode_grouped_bf16",
                og.data_ptr(), qg.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), _ptr(ks),
                _ptr(vs), cu.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(), _ptr(sinks),
                nseq * g, nseq, hkv, hkv, d, key_cache.size(1), block_table.stride(0), qg.stride(0),
                qg.stride(1), og.stride(0), og.stride(1), key_cache.stride(0), key_cache.stride(1),
                key_cache.stride(2), value_cache.stride(0), value_cache.stride(1),
                value_cache.stride(2), *(ks.stride() if q8 else (0, 0, 0)),
                *(vs.stride() if q8 else (0, 0, 0)), float(scale), 1, window_left, int(q8), _stream(),
            )
        out.copy_(ungroup_queries(og, nseq))
        return
    nseq, hq = q.size(0), q.size(1)
    bs, hkv = key_cache.size(1), key_cache.size(2)
    max_blocks = block_table.size(1)
    lib = _lib.load()
    ws_bytes = lib.strix_attn_decode_workspace(nseq, hq, d, num_splits, max_blocks, bs)
    _check(ws_bytes >= 0, "num_splits in [1, 64]")
    with torch.cuda.device(q.device):
        ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=q.device) if ws_bytes else None
        ks = k_scale if q8 else None
        vs = v_scale if q8 else None
        _lib.call(
            "strix_attn_decode_bf16",
            out.data_ptr(), q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
            _ptr(ks), _ptr(vs), seq_lens.data_ptr(), block_table.data_ptr(), _ptr(sinks),
            _ptr(ws), nseq, hq, hkv, d, bs, max_blocks, block_table.stride(0),
            q.stride(0), q.stride(1), out.stride(0), out.stride(1),
            key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
            value_cache.stride(0), value_cache.stride(1), value_cache.stride(2),
            *(ks.stride() if q8 else (0, 0, 0)), *(vs.stride() if q8 else (0, 0, 0)),
            float(scale), num_splits, window_left, int(q8), _stream(),
        )


# Not in the reference (vLLM's reshape_and_cache does it there): quantise new K/V
# rows per (token, head) into the int8 paged cache; rule "reference" is quantize()
# of tests/test_attn_prefill.py:202-206, "vllm" the rule of vLLM 0.22's writer.
@_define("kv_write_i8(Tensor key, Tensor value, Tensor(a!) key_cache, Tensor(b!) value_cache, "
         "Tensor(c!) k_scale, Tensor(d!) v_scale, Tensor slot_mapping, str rule='reference') -> ()")
def kv_write_i8(key, value, key_cache, value_cache, k_scale, v_scale, slot_mapping,
                rule="reference"):
    _check(key.dim() == 3 and value.dim() == 3 and key.shape == value.shape,
           "key / value must be [tokens, Hkv, D]")
    _check(key.dtype in (torch.bfloat16, torch.float16) and value.dtype == key.dtype
           and key.stride(-1) == 1 and value.stride(-1) == 1, "key / value bf16 or fp16, contiguous D")
    t, hkv, d = key.shape
    for c in (key_cache, value_cache):
        _check(c.dim() == 4 and c.dtype == torch.int8 and c.size(2) == hkv and c.size(3) >= d
               and c.stride(3) == 1, "caches must be int8 [blocks, block_size, Hkv, >= D]")
    for sc in (k_scale, v_scale):
        _check(sc.dtype == torch.float32 and tuple(sc.shape) == tuple(key_cache.shape[:3]),
               "scales must be fp32 [blocks, block_size, Hkv]")
    _check(slot_mapping.dtype == torch.int64 and slot_mapping.is_contiguous()
           and slot_mapping.numel() >= t, "slot_mapping must be contiguous int64 [tokens]")
    _check(rule in ("reference", "vllm"), "rule must be 'reference' or 'vllm'")
    with torch.cuda.device(key.device):
        _lib.call("strix_kv_write_i8", key.data_ptr(), value.data_ptr(), key_cache.data_ptr(),
                  value_cache.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(),
                  slot_mapping.data_ptr(), t, hkv, d, key_cache.size(1), key.stride(0),
                  key.stride(1), value.stride(0), value.stride(1), *key_cache.stride()[:3],
                  *value_cache.stride()[:3], *k_scale.stride(), *v_scale.stride(),
                  int(key.dtype == torch.float16), 0 if rule == "reference" else 1, _stream())


@_define(
    "attn_prefill_bf16(Tensor(a!) out, Tensor q, Tensor key_cache, "
    "Tensor value_cache, Tensor? k_scale, Tensor? v_scale, "
    "Tensor cu_seqlens_q, Tensor seq_lens, "
    "Tensor block_table, Tensor tile_offsets, int max_tiles, float scale, "
    "int num_splits, int window_left=-1, Tensor? sinks=None) -> ()"
)
def attn_prefill_bf16(out, q, key_cache, value_cache, k_scale, v_scale, cu_seqlens_q, seq_lens,
                      block_table, tile_offsets, max_tiles, scale, num_splits, window_left=-1,
                      sinks=None):
    """Host side of strix_attn_prefill_bf16; checks follow
    csrc/attn/attn_prefill_bf16.hip:516-580 of the reference. tile_offsets and
    max_tiles (the reference's 16-query tiling) are accepted and not used."""
    _check(q.dim() == 3 and key_cache.dim() == 4 and value_cache.dim() == 4,
           "q [T, H, D], caches [blocks, block_size, Hkv, D]")
    d = q.size(-1)
    _check(q.dtype == torch.bfloat16 and q.stride(-1) == 1,
           "q must be bf16 with a contiguous head_dim")
    q8 = key_cache.dtype != torch.bfloat16
    _check(key_cache.dtype == (torch.int8 if q8 else torch.bfloat16)
           and value_cache.dtype == key_cache.dtype, "caches must both be bf16 or both int8")
    for t in (key_cache, value_cache):
        _check(t.size(-1) >= d and t.stride(-1) == 1, "cache head_dim must be at least q's, contiguous")
    if q8:
        _check(k_scale is not None and v_scale is not None, "int8 KV needs k_scale and v_scale")
        for t in (k_scale, v_scale):
            _check(t.dtype == torch.float32 and t.dim() == 3
                   and tuple(t.shape) == tuple(key_cache.shape[:3]),
                   "scales must be fp32 [blocks, block_size, Hkv]")
    _check(out.dtype == torch.bfloat16 and out.shape == q.shape and out.stride(-1) == 1,
           "out must match q")
    _check(cu_seqlens_q.dtype == torch.int32 and seq_lens.dtype == torch.int32
           and block_table.dtype == torch.int32 and block_table.stride(1) == 1
           and cu_seqlens_q.is_contiguous() and seq_lens.is_contiguous()
           and seq_lens.numel() >= cu_seqlens_q.numel() - 1, "int32 metadata")
    if sinks is not None:
        _check(num_splits == 1, "sinks need num_splits == 1")
        _check(sinks.dtype == torch.float32 and sinks.dim() == 1 and sinks.size(0) == q.size(1)
               and sinks.is_contiguous(), "sinks must be contiguous fp32 [Hq]")
    ks = k_scale if q8 else None
    vs = v_scale if q8 else None
    nseq, hkv, bs, max_blocks = cu_seqlens_q.numel() - 1, key_cache.size(2), key_cache.size(1), \
        block_table.size(1)
    lib = _lib.load()
    umma = PREFILL_IMPL != "mma" and bool(lib.strix_attn_prefill_umma_covers(
        d, q.stride(0), q.stride(1), out.stride(0), out.stride(1), int(q8))) \
        and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
    _check(umma or PREFILL_IMPL != "umma", "the tcgen05 prefill kernel does not cover this geometry")
    if umma and nseq > 0 and q.size(0) > 0:
        # tensor-core path: the batch's keys and values are gathered (int8: dequantised) once
        # into a contiguous 16-bit workspace, which the attention kernel reads by TMA
        ws_bytes = lib.strix_attn_prefill_workspace(nseq, max_blocks, bs, hkv, d)
        with torch.cuda.device(q.device):
            ws = torch.empty(ws_bytes + 1024, dtype=torch.uint8, device=q.device)
            ws_ptr = (ws.data_ptr() + 1023) // 1024 * 1024
            _lib.call(
                "strix_attn_prefill_umma",
                out.data_ptr(), q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), _ptr(ks),
                _ptr(vs), cu_seqlens_q.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(),
                _ptr(sinks), ws_ptr, ws_bytes, q.size(0), nseq, q.size(1), hkv, d, bs, max_blocks,
                block_table.stride(0), q.stride(0), q.stride(1), out.stride(0), out.stride(1),
                key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
                value_cache.stride(0), value_cache.stride(1), value_cache.stride(2),
                *(ks.stride() if q8 else (0, 0, 0)), *(vs.stride() if q8 else (0, 0, 0)),
                float(scale), window_left, int(q8), _stream(),
            )
            _lib.after_tcgen05("attn_prefill_bf16")
        return
    with torch.cuda.device(q.device):
        _lib.call(
            "strix_attn_prefill_bf16",
            out.data_ptr(), q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), _ptr(ks),
            _ptr(vs), cu_seqlens_q.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(),
            _ptr(sinks), q.size(0), cu_seqlens_q.numel() - 1, q.size(1), key_cache.size(2), d,
            key_cache.size(1), block_table.stride(0), q.stride(0), q.stride(1), out.stride(0),
            out.stride(1), key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
            value_cache.stride(0), value_cache.stride(1), value_cache.stride(2),
            *(ks.stride() if q8 else (0, 0, 0)), *(vs.stride() if q8 else (0, 0, 0)),
            float(scale), num_splits, window_left, int(q8), _stream(),
        )


# ----------------------------------------------------------------------- MoE

_W_E4M3, _W_INT8, _W_BF16 = 0, 1, 2
_W_INT4X = 6       # int4, 32-bit words in ExLlama nibble order (the dense int4 ops)
_A_BF16, _A_F16, _A_E4M3 = 0, 1, 2
_S_NONE, _S_CHANNEL, _S_BLOCK = 0, 1, 2
_SCALE_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_ACTS = {"silu": 1, "gelu_tanh": 2}


def _moe_gemm(c, a, w, scales, act_scales, sorted_ids, expert_ids, num_post_padded, topk_weights,
              top_k, block_m, block_n, silu_mul, activation, *, wfmt, afmt, name):
    """Shared host side of the moe_gemm_* ops; the checks (and their messages)
    follow moe_gemm_impl, csrc/moe/moe_gemm_w8a16.hip:444-514 of the reference.
    block_n is the caller's tile hint and is only validated."""
    a_dtype = {_A_BF16: torch.bfloat16, _A_F16: torch.float16, _A_E4M3: torch.float8_e4m3fn}[afmt]
    w_dtype = {_W_E4M3: torch.float8_e4m3fn, _W_INT8: torch.int8, _W_BF16: torch.bfloat16}[wfmt]
    c_f16 = afmt == _A_F16 and silu_mul and c.dtype != torch.bfloat16
    c_dtype = torch.float16 if c_f16 else torch.bfloat16
    _check(a.dtype == a_dtype and w.dtype == w_dtype and c.dtype == c_dtype
           and (scales is None or scales.dtype in _SCALE_DTYPES),
           f"{name}: a {a_dtype}, c {c_dtype}; scales bf16, fp16 or fp32; w {w_dtype}")
    _check(a.dim() == 2 and w.dim() == 3 and c.dim() == 2, "bad ranks")
    e, n, k = w.shape
    _check(a.size(1) == k and c.size(1) == (n // 2 if silu_mul else n), "shape mismatch")
    scale_kind, s_se, s_sn, s_dtype = _S_NONE, 0, 0, 0
    if wfmt != _W_BF16:
        _check(scales is not None and scales.dim() in (2, 3), "scales must be [E, N]")
        block = wfmt == _W_E4M3 and scales.dim() == 3 and scales.size(1) != n
        if block:
            _check(scales.dtype == torch.float32 and n % 128 == 0 and k % 128 == 0
                   and tuple(scales.shape) == (e, n // 128, k // 128),
                   "block scales must be fp32 [E, N/128, K/128]")
            scale_kind, s_sn = _S_BLOCK, scales.stride(1)
        else:
            _check(scales.size(0) == e and scales.size(1) == n
                   and (scales.dim() == 2 or scales.size(2) == 1),
                   "scales must be [E, N] or [E, N, 1]")
            scale_kind = _S_CHANNEL
            _check(scales.stride(1) == 1 or scales.dim() == 3, "last dims must be contiguous")
        _check(scales.stride(-1) == 1, "last dims must be contiguous")
        s_se, s_dtype = scales.stride(0), _SCALE_DTYPES[scales.dtype]
    _check(a.stride(1) == 1 and w.stride(2) == 1 and c.stride(1) == 1,
           "last dims must be contiguous")
    _check(not silu_mul or (n % 2 == 0 and topk_weights is None),
           "silu_mul needs even N and no topk weights")
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    _check(k % 64 == 0 and n % block_n == 0, "K % 64 and N % block_n")
    _check(sorted_ids.dtype == torch.int32 and expert_ids.dtype == torch.int32
           and num_post_padded.dtype == torch.int32, "routing tensors must be int32")
    _check(expert_ids.numel() * block_m >= sorted_ids.numel(),
           f"expert_ids too short for block_m {block_m}")
    if topk_weights is not None:
        _check(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
               and topk_weights.numel() == c.size(0),
               "topk_weights must be contiguous fp32 [num_valid]")
    sa_stride = 0
    if afmt == _A_E4M3:
        _check(act_scales is not None and act_scales.dtype == torch.float32
               and act_scales.dim() == 2 and act_scales.size(0) == a.size(0)
               and act_scales.size(1) == k // 128 and act_scales.stride(1) == 1,
               "activation scales must be fp32 [rows, K/128]")
        sa_stride = act_scales.stride(0)
    with torch.cuda.device(c.device):
        _lib.call(
            "strix_moe_gemm",
            c.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(scales), _ptr(act_scales),
            sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post_padded.data_ptr(),
            _ptr(topk_weights), c.size(0), a.size(0), e, n, k, a.stride(0), c.stride(0),
            w.stride(0), w.stride(1), s_se, s_sn, sa_stride, sorted_ids.numel(),
            expert_ids.numel(), top_k, block_m, wfmt, afmt, scale_kind, s_dtype,
            _ACTS[activation] if silu_mul else 0, int(c_f16), _stream(),
        )


_MOE_TAIL = ("Tensor sorted_ids, Tensor expert_ids, Tensor num_post_padded, "
             "Tensor? topk_weights, int top_k, int block_m, int block_n, "
             "bool silu_mul=False, str activation='silu') -> ()")


@_define("moe_gemm_bf16(Tensor(a!) c, Tensor a, Tensor b, " + _MOE_TAIL)
def moe_gemm_bf16(c, a, b, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
                  block_m, block_n, silu_mul=False, activation="silu"):
    _moe_gemm(c, a, b, None, None, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
              block_m, block_n, silu_mul, activation, wfmt=_W_BF16, afmt=_A_BF16,
              name="moe_gemm_bf16")


@_define("moe_gemm_w8a16(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, " + _MOE_TAIL)
def moe_gemm_w8a16(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
                   block_m, block_n, silu_mul=False, activation="silu"):
    _moe_gemm(c, a, b, scales, None, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
              block_m, block_n, silu_mul, activation, wfmt=_W_INT8, afmt=_A_BF16,
              name="moe_gemm_w8a16/fp8")


@_define("moe_gemm_fp8(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, " + _MOE_TAIL)
def moe_gemm_fp8(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
                 block_m, block_n, silu_mul=False, activation="silu"):
    _moe_gemm(c, a, b, scales, None, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
              block_m, block_n, silu_mul, activation, wfmt=_W_E4M3, afmt=_A_BF16,
              name="moe_gemm_w8a16/fp8")


@_define("moe_gemm_fp8_raw(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, " + _MOE_TAIL)
def moe_gemm_fp8_raw(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights,
                     top_k, block_m, block_n, silu_mul=False, activation="silu"):
    _moe_gemm(c, a, b, scales, None, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
              block_m, block_n, silu_mul, activation, wfmt=_W_E4M3, afmt=_A_F16,
              name="moe_gemm_w8a16/fp8")


# Not in the reference: the W8A8 form of the FP8 experts (e4m3 activations with
# one fp32 scale per token and 128-wide K group), modelled on moe_gemm_w4a8's
# argument order (csrc/torch_ops.cpp:214-217).
@_define("moe_gemm_fp8_w8a8(Tensor(a!) c, Tensor qa, Tensor sa, Tensor b, Tensor scales, "
         + _MOE_TAIL)
def moe_gemm_fp8_w8a8(c, qa, sa, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights,
                      top_k, block_m, block_n, silu_mul=False, activation="silu"):
    _moe_gemm(c, qa, b, scales, sa, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
              block_m, block_n, silu_mul, activation, wfmt=_W_E4M3, afmt=_A_E4M3,
              name="moe_gemm_fp8_w8a8")


def _act_quant(entry, x, q, sa, q_dtype):
    _check(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and x.stride(1) == 1,
           "x must be bf16 or fp16 [rows, K]")
    _check(q.dtype == q_dtype and q.shape == x.shape and q.stride(1) == 1,
           f"q must be {q_dtype} [rows, K]")
    _check(x.size(1) % 128 == 0, "K must be a multiple of 128")
    _check(sa.dtype == torch.float32 and tuple(sa.shape) == (x.size(0), x.size(1) // 128)
           and sa.stride(1) == 1, "sa must be fp32 [rows, K / 128]")
    with torch.cuda.device(x.device):
        _lib.call(entry, x.data_ptr(), q.data_ptr(), sa.data_ptr(), x.size(0), x.size(1),
                  x.stride(0), q.stride(0), sa.stride(0), int(x.dtype == torch.float16), _stream())


@_define("moe_act_quant_i8(Tensor x, Tensor(a!) q, Tensor(b!) sa) -> ()")
def moe_act_quant_i8(x, q, sa):
    _act_quant("strix_moe_act_quant_i8", x, q, sa, torch.int8)


@_define("moe_act_quant_fp8(Tensor x, Tensor(a!) q, Tensor(b!) sa) -> ()")
def moe_act_quant_fp8(x, q, sa):
    _act_quant("strix_moe_act_quant_fp8", x, q, sa, torch.float8_e4m3fn)


# ---- sorted-layout forms (not in the reference): the activations are laid out
# by sorted position, so an m-block's tokens are consecutive rows and the
# tcgen05 grouped GEMM fetches them with one TMA box.

@_define("moe_act_quant_fp8_sorted(Tensor x, Tensor(a!) q, Tensor(b!) sa, Tensor? sorted_ids, "
         "Tensor num_post_padded, int top_k, int num_valid) -> ()")
def moe_act_quant_fp8_sorted(x, q, sa, sorted_ids, num_post_padded, top_k, num_valid):
    """q[p], sa[p] = quantised x[sorted_ids[p] // top_k] for p < num_post_padded
    (zeros for padding slots); with sorted_ids None, row p from row p."""
    _check(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and x.stride(1) == 1,
           "x must be bf16 or fp16 [rows, K]")
    k = x.size(1)
    _check(k % 128 == 0, "K must be a multiple of 128")
    rows = q.size(0)
    _check(q.dtype == torch.float8_e4m3fn and q.dim() == 2 and q.size(1) == k and q.stride(1) == 1,
           "q must be float8_e4m3fn [sorted rows, K]")
    _check(sa.dtype == torch.float32 and tuple(sa.shape) == (rows, k // 128) and sa.stride(1) == 1,
           "sa must be fp32 [sorted rows, K / 128]")
    _check(num_post_padded.dtype == torch.int32, "num_post_padded must be int32")
    if sorted_ids is None:
        _check(x.size(0) >= rows, "x has fewer rows than q")
    else:
        _check(sorted_ids.dtype == torch.int32 and sorted_ids.numel() >= rows
               and sorted_ids.is_contiguous(), "sorted_ids must be int32 with an entry per row of q")
        _check(num_valid <= x.size(0) * top_k, "num_valid exceeds rows(x) * top_k")
    with torch.cuda.device(x.device):
        _lib.call("strix_moe_act_quant_fp8_sorted", x.data_ptr(), q.data_ptr(), sa.data_ptr(),
                  _ptr(sorted_ids), num_post_padded.data_ptr(), rows, k, top_k, num_valid,
                  x.stride(0), q.stride(0), sa.stride(0), int(x.dtype == torch.float16), _stream())


@_define("moe_align_block_size_pos(Tensor topk_ids, int num_experts, int block_size, "
         "Tensor(a!) sorted_token_ids, Tensor(b!) experts_ids, Tensor(c!) num_tokens_post_pad, "
         "Tensor(d!) slot_pos) -> ()")
def moe_align_block_size_pos(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids,
                             num_tokens_post_pad, slot_pos):
    """moe_align_block_size plus the inverse permutation slot_pos [numel] int32."""
    _check(all(t.dtype == torch.int32 and t.is_contiguous()
               for t in (topk_ids, sorted_token_ids, experts_ids, num_tokens_post_pad, slot_pos)),
           "routing tensors must be contiguous int32")
    _check(slot_pos.numel() >= topk_ids.numel(), "slot_pos must have an entry per slot")
    _align(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, slot_pos)


def _align(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, slot_pos):
    """The permutation, through the two-level kernels (and a scratch from torch's
    caching allocator) where the batch is large enough for them to pay."""
    n = topk_ids.numel()
    nbytes = _lib.load().strix_moe_align_scratch_bytes(n, num_experts) if n > 4096 else 0
    scratch = torch.empty(nbytes // 4, dtype=torch.int32, device=topk_ids.device) if nbytes > 0 else None
    with torch.cuda.device(topk_ids.device):
        _lib.call("strix_moe_align_scratch", topk_ids.data_ptr(), sorted_token_ids.data_ptr(),
                  experts_ids.data_ptr(), num_tokens_post_pad.data_ptr(),
                  None if slot_pos is None else slot_pos.data_ptr(), None,
                  None if scratch is None else scratch.data_ptr(), nbytes, n, num_experts, block_size,
                  sorted_token_ids.numel(), experts_ids.numel(), _stream())


@_define("moe_act_quant_fp8_scatter(Tensor x, Tensor(a!) q, Tensor(b!) sa, Tensor slot_pos, "
         "Tensor sorted_ids, Tensor num_post_padded, int top_k) -> ()")
def moe_act_quant_fp8_scatter(x, q, sa, slot_pos, sorted_ids, num_post_padded, top_k):
    """Sorted-layout quantiser by scatter: x[t] is quantised once and stored at
    the sorted positions slot_pos[t * top_k + j]; padding rows become zeros."""
    _check(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and x.stride(1) == 1,
           "x must be bf16 or fp16 [tokens, K]")
    k = x.size(1)
    _check(k % 128 == 0, "K must be a multiple of 128")
    rows = q.size(0)
    _check(q.dtype == torch.float8_e4m3fn and q.dim() == 2 and q.size(1) == k and q.stride(1) == 1,
           "q must be float8_e4m3fn [sorted rows, K]")
    _check(sa.dtype == torch.float32 and tuple(sa.shape) == (rows, k // 128) and sa.stride(1) == 1,
           "sa must be fp32 [sorted rows, K / 128]")
    _check(all(t.dtype == torch.int32 and t.is_contiguous()
               for t in (slot_pos, sorted_ids, num_post_padded)), "routing tensors must be int32")
    _check(slot_pos.numel() >= x.size(0) * top_k and sorted_ids.numel() >= rows,
           "slot_pos / sorted_ids too short")
    with torch.cuda.device(x.device):
        _lib.call("strix_moe_act_quant_fp8_scatter", x.data_ptr(), q.data_ptr(), sa.data_ptr(),
                  slot_pos.data_ptr(), sorted_ids.data_ptr(), num_post_padded.data_ptr(), x.size(0),
                  rows, k, top_k, x.stride(0), q.stride(0), sa.stride(0),
                  int(x.dtype == torch.float16), _stream())


@_define("moe_gemm_fp8_sorted(Tensor(a!) c, Tensor qa, Tensor sa, Tensor b, Tensor scales, "
         "Tensor sorted_ids, Tensor expert_ids, Tensor num_post_padded, Tensor? topk_weights, "
         "int num_valid, int block_m, bool silu_mul=False, str activation='silu', "
         "bool c_sorted=False) -> ()")
def moe_gemm_fp8_sorted(c, qa, sa, b, scales, sorted_ids, expert_ids, num_post_padded,
                        topk_weights, num_valid, block_m, silu_mul=False, activation="silu",
                        c_sorted=False):
    f8 = torch.float8_e4m3fn
    _check(qa.dtype == f8 and b.dtype == f8 and c.dtype == torch.bfloat16
           and scales.dtype == torch.float32, "qa, b float8_e4m3fn; c bf16; scales fp32")
    _check(qa.dim() == 2 and b.dim() == 3 and c.dim() == 2, "bad ranks")
    e, n, k = b.shape
    _check(qa.size(1) == k and c.size(1) == (n // 2 if silu_mul else n), "shape mismatch")
    _check(qa.stride(1) == 1 and b.stride(2) == 1 and c.stride(1) == 1 and scales.stride(-1) == 1,
           "last dims must be contiguous")
    if scales.dim() == 3 and scales.size(1) != n:
        _check(tuple(scales.shape) == (e, n // 128, k // 128),
               "block scales must be fp32 [E, N/128, K/128]")
        scale_kind, s_sn = _S_BLOCK, scales.stride(1)
    else:
        _check(scales.size(0) == e and scales.size(1) == n, "scales must be [E, N] or [E, N, 1]")
        scale_kind, s_sn = _S_CHANNEL, 0
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    _check(sorted_ids.dtype == torch.int32 and expert_ids.dtype == torch.int32
           and num_post_padded.dtype == torch.int32, "routing tensors must be int32")
    sorted_len = sorted_ids.numel() // block_m * block_m
    _check(qa.size(0) >= sorted_len and sa.size(0) >= sorted_len
           and tuple(sa.shape[1:]) == (k // 128,) and sa.stride(1) == 1 and sa.dtype == torch.float32,
           "qa / sa must cover every sorted position: [sorted_len, K] and fp32 [sorted_len, K/128]")
    _check(expert_ids.numel() * block_m >= sorted_len, f"expert_ids too short for block_m {block_m}")
    _check(c.size(0) >= (sorted_len if c_sorted else num_valid), "c has too few rows")
    if topk_weights is not None:
        _check(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
               and topk_weights.numel() >= num_valid, "topk_weights must be contiguous fp32 [num_valid]")
    with torch.cuda.device(c.device):
        _lib.call("strix_moe_gemm_fp8_sorted", c.data_ptr(), qa.data_ptr(), sa.data_ptr(),
                  b.data_ptr(), scales.data_ptr(), sorted_ids.data_ptr(), expert_ids.data_ptr(),
                  num_post_padded.data_ptr(), _ptr(topk_weights), num_valid, e, n, k, qa.stride(0),
                  c.stride(0), b.stride(0), b.stride(1), scales.stride(0), s_sn, sa.stride(0),
                  sorted_len, block_m, scale_kind, _ACTS[activation] if silu_mul else 0,
                  int(c_sorted), _stream())
        _lib.after_tcgen05("moe_gemm_fp8_sorted")


@_define("moe_topk_softmax(Tensor(a!) topk_weights, Tensor(b!) topk_ids, Tensor gating_output, "
         "bool renormalize=True) -> ()")
def moe_topk_softmax(topk_weights, topk_ids, gating_output, renormalize=True):
    _check(gating_output.dim() == 2 and gating_output.dtype == torch.float32
           and gating_output.stride(1) == 1, "gating_output must be fp32 [tokens, experts]")
    t, k = topk_ids.shape
    _check(topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
           and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
           and topk_weights.shape == topk_ids.shape and t == gating_output.size(0),
           "topk_ids int32 and topk_weights fp32, contiguous [tokens, top_k]")
    with torch.cuda.device(gating_output.device):
        _lib.call("strix_moe_topk_softmax", gating_output.data_ptr(), topk_ids.data_ptr(),
                  topk_weights.data_ptr(), t, gating_output.size(1), k, gating_output.stride(0),
                  int(renormalize), _stream())


@_define("moe_align_block_size(Tensor topk_ids, int num_experts, int block_size, "
         "Tensor(a!) sorted_token_ids, Tensor(b!) experts_ids, Tensor(c!) num_tokens_post_pad) -> ()")
def moe_align_block_size(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids,
                         num_tokens_post_pad):
    _check(topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
           and sorted_token_ids.dtype == torch.int32 and sorted_token_ids.is_contiguous()
           and experts_ids.dtype == torch.int32 and experts_ids.is_contiguous()
           and num_tokens_post_pad.dtype == torch.int32, "routing tensors must be int32")
    _align(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, None)


@_define("moe_sum(Tensor input, Tensor(a!) output) -> ()")
def moe_sum(input, output):
    _check(input.dim() == 3 and input.dtype == torch.bfloat16 and input.stride(2) == 1
           and output.dtype == torch.bfloat16 and output.stride(1) == 1
           and tuple(output.shape) == (input.size(0), input.size(2)),
           "input bf16 [tokens, top_k, hidden], output bf16 [tokens, hidden]")
    with torch.cuda.device(input.device):
        _lib.call("strix_moe_sum", input.data_ptr(), output.data_ptr(), input.size(0),
                  input.size(1), input.size(2), input.stride(0), input.stride(1),
                  output.stride(0), _stream())


# ------------------------------------------------- 4-bit experts and dense 4-/8-bit GEMMs
_W_MXFP4, _W_INT4, _W_U8B128 = 3, 4, 5
_S_GROUP = 3


def _dense_block_m(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64


# Token-tile sizes of the weight-streaming GEMMs that the bench-only *_cfg ops pin
# (the reference's *_cfg ops pin one of its own tile shapes the same way).
TILE_CFGS = (16, 32, 64)


def _cfg_block_m(cfg: int) -> int:
    _check(0 <= cfg < len(TILE_CFGS), f"cfg must be in [0, {len(TILE_CFGS)})")
    return TILE_CFGS[cfg]


def _gemm_w4(c, a, w, scales, bias, routing, topk_weights, top_k, block_m, wfmt, group, gate):
    """Host side of strix_gemm_w4a16; routing = (sorted_ids, expert_ids, num_post) or None."""
    dense = routing is None
    if dense:
        e, (n, kh) = 1, w.shape
        w_se, w_sn, s_se, s_sn = 0, w.stride(0), 0, scales.stride(0)
    else:
        e, n, kh = w.shape
        w_se, w_sn, s_se, s_sn = w.stride(0), w.stride(1), scales.stride(0), scales.stride(1)
    k = kh * 2
    _check(a.dtype == torch.bfloat16 and c.dtype == torch.bfloat16 and w.dtype == torch.uint8,
           "a, c bf16; w uint8 (two 4-bit values per byte)")
    _check(a.dim() == 2 and a.size(1) == k and a.stride(1) == 1 and w.stride(-1) == 1
           and c.stride(1) == 1 and scales.stride(-1) == 1, "shape mismatch / last dims must be contiguous")
    if wfmt == _W_MXFP4:
        _check(scales.dtype == torch.uint8, "scale must be uint8 (e8m0)")
        sdt = 0
    else:
        _check(scales.dtype in (torch.bfloat16, torch.float16), "scales must be bf16 or fp16")
        sdt = _SCALE_DTYPES[scales.dtype]
    _check(k % group == 0 and tuple(scales.shape[-2:]) == (n, k // group),
           f"scales must be [..., N, K / {group}]")
    bias_stride = 0
    if bias is not None:
        _check(bias.dtype == torch.bfloat16 and bias.stride(-1) == 1
               and (tuple(bias.shape) == (n,) or tuple(bias.shape) == (c.size(0), n)),
               "bias must be bf16 [N] or [M, N]")
        bias_stride = bias.stride(0) if bias.dim() == 2 else 0
    if dense:
        m = a.size(0)
        sid = eid = npp = None
        sorted_len, expert_len, num_valid = (m + block_m - 1) // block_m * block_m, 0, m
    else:
        sid, eid, npp = routing
        _check(sid.dtype == torch.int32 and eid.dtype == torch.int32 and npp.dtype == torch.int32,
               "routing tensors must be int32")
        _check(eid.numel() * block_m >= sid.numel(), f"expert_ids too short for block_m {block_m}")
        sorted_len, expert_len, num_valid = sid.numel(), eid.numel(), c.size(0)
    with torch.cuda.device(c.device):
        _lib.call("strix_gemm_w4a16", c.data_ptr(), a.data_ptr(), w.data_ptr(), scales.data_ptr(),
                  _ptr(bias), _ptr(sid), _ptr(eid), _ptr(npp), _ptr(topk_weights), num_valid,
                  a.size(0), e, n, k, a.stride(0), c.stride(0), w_se, w_sn, s_se, s_sn, bias_stride,
                  sorted_len, expert_len, top_k, block_m, wfmt, group, sdt, gate, _stream())


@_define("moe_gemm_w4a16(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, Tensor sorted_ids, "
         "Tensor expert_ids, Tensor num_post_padded, Tensor? topk_weights, int top_k, int block_m, "
         "int block_n, bool silu_mul=False, str activation='silu', int group_size=32) -> ()")
def moe_gemm_w4a16(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
                   block_m, block_n, silu_mul=False, activation="silu", group_size=32):
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    _check(group_size in (32, 64, 128), "group_size must be 32, 64 or 128")
    _check(c.size(1) == (b.size(1) // 2 if silu_mul else b.size(1)), "shape mismatch")
    _check(not silu_mul or topk_weights is None, "silu_mul needs even N and no topk weights")
    _gemm_w4(c, a, b, scales, None, (sorted_ids, expert_ids, num_post_padded), topk_weights, top_k,
             block_m, _W_INT4, group_size, _ACTS[activation] if silu_mul else 0)


# Not in the reference: MXFP4 experts (e2m1 + e8m0 per 32), the grouped form of
# mxfp4_wmma_gemm with moe_gemm_w4a16's argument order.
@_define("moe_gemm_mxfp4(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, Tensor sorted_ids, "
         "Tensor expert_ids, Tensor num_post_padded, Tensor? topk_weights, int top_k, int block_m, "
         "int block_n, bool silu_mul=False, str activation='silu') -> ()")
def moe_gemm_mxfp4(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights, top_k,
                   block_m, block_n, silu_mul=False, activation="silu"):
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    _check(c.size(1) == (b.size(1) // 2 if silu_mul else b.size(1)), "shape mismatch")
    _check(not silu_mul or topk_weights is None, "silu_mul needs even N and no topk weights")
    _gemm_w4(c, a, b, scales, None, (sorted_ids, expert_ids, num_post_padded), topk_weights, top_k,
             block_m, _W_MXFP4, 32, _ACTS[activation] if silu_mul else 0)


@_define("moe_permute_bf16(Tensor x, Tensor(a!) y, Tensor slot_pos, Tensor sorted_ids, "
         "Tensor num_post_padded, int top_k) -> ()")
def moe_permute_bf16(x, y, slot_pos, sorted_ids, num_post_padded, top_k):
    """y[slot_pos[t * top_k + j]] = x[t]; padding rows below num_post_padded = 0."""
    _check(x.dtype == torch.bfloat16 and y.dtype == torch.bfloat16 and x.dim() == 2 and y.dim() == 2
           and x.size(1) == y.size(1) and x.stride(1) == 1 and y.stride(1) == 1,
           "x, y bf16 [rows, K] with contiguous rows")
    _check(all(t.dtype == torch.int32 and t.is_contiguous()
               for t in (slot_pos, sorted_ids, num_post_padded)), "routing tensors must be int32")
    _check(slot_pos.numel() >= x.size(0) * top_k and sorted_ids.numel() >= y.size(0),
           "slot_pos / sorted_ids too short")
    with torch.cuda.device(x.device):
        _lib.call("strix_moe_permute_bf16", x.data_ptr(), y.data_ptr(), slot_pos.data_ptr(),
                  sorted_ids.data_ptr(), num_post_padded.data_ptr(), x.size(0), y.size(0), x.size(1),
                  top_k, x.stride(0), y.stride(0), _stream())


@_define("moe_permute_rows(Tensor x, Tensor(a!) y, Tensor slot_pos, Tensor sorted_ids, "
         "Tensor num_post_padded, int top_k) -> ()")
def moe_permute_rows(x, y, slot_pos, sorted_ids, num_post_padded, top_k):
    """moe_permute_bf16 for rows of any element type (whole 16-byte chunks), e.g.
    e4m3 activations followed by their fp32 group scales: y[slot_pos[r * top_k + j]]
    = x[r]; rows none of whose slots has a position are not read."""
    _check(x.dim() == 2 and y.dim() == 2 and x.dtype == y.dtype and x.size(1) == y.size(1)
           and x.stride(1) == 1 and y.stride(1) == 1, "x, y [rows, K] of one dtype, contiguous rows")
    _check(all(t.dtype == torch.int32 and t.is_contiguous()
               for t in (slot_pos, sorted_ids, num_post_padded)), "routing tensors must be int32")
    _check(slot_pos.numel() >= x.size(0) * top_k and sorted_ids.numel() >= y.size(0),
           "slot_pos / sorted_ids too short")
    eb = x.element_size()
    with torch.cuda.device(x.device):
        _lib.call("strix_moe_permute_rows", x.data_ptr(), y.data_ptr(), slot_pos.data_ptr(),
                  sorted_ids.data_ptr(), num_post_padded.data_ptr(), x.size(0), y.size(0),
                  x.size(1) * eb, top_k, x.stride(0) * eb, y.stride(0) * eb, _stream())


@_define("moe_gemm_mxfp4_sorted(Tensor(a!) c, Tensor a, Tensor b, Tensor scales, Tensor sorted_ids, "
         "Tensor expert_ids, Tensor num_post_padded, Tensor? topk_weights, int num_valid, "
         "int block_m, bool silu_mul=False, str activation='silu', bool c_sorted=False) -> ()")
def moe_gemm_mxfp4_sorted(c, a, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights,
                          num_valid, block_m, silu_mul=False, activation="silu", c_sorted=False):
    _check(a.dtype == torch.bfloat16 and c.dtype == torch.bfloat16 and b.dtype == torch.uint8
           and scales.dtype == torch.uint8, "a, c bf16; b uint8; scale must be uint8 (e8m0)")
    _check(a.dim() == 2 and b.dim() == 3 and c.dim() == 2, "bad ranks")
    e, n, kh = b.shape
    k = kh * 2
    _check(a.size(1) == k and c.size(1) == (n // 2 if silu_mul else n)
           and tuple(scales.shape) == (e, n, k // 32), "shape mismatch")
    _check(a.stride(1) == 1 and b.stride(2) == 1 and c.stride(1) == 1 and scales.stride(2) == 1,
           "last dims must be contiguous")
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    sorted_len = sorted_ids.numel() // block_m * block_m
    _check(a.size(0) >= sorted_len and c.size(0) >= (sorted_len if c_sorted else num_valid),
           "a / c have too few rows")
    _check(expert_ids.numel() * block_m >= sorted_len, f"expert_ids too short for block_m {block_m}")
    if topk_weights is not None:
        _check(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
               and topk_weights.numel() >= num_valid, "topk_weights must be contiguous fp32 [num_valid]")
    with torch.cuda.device(c.device):
        _lib.call("strix_moe_gemm_mxfp4_sorted", c.data_ptr(), a.data_ptr(), b.data_ptr(),
                  scales.data_ptr(), sorted_ids.data_ptr(), expert_ids.data_ptr(),
                  num_post_padded.data_ptr(), _ptr(topk_weights), num_valid, e, n, k, a.stride(0),
                  c.stride(0), b.stride(0), b.stride(1), scales.stride(0), scales.stride(1),
                  sorted_len, block_m, _ACTS[activation] if silu_mul else 0, int(c_sorted), _stream())
        _lib.after_tcgen05("moe_gemm_mxfp4_sorted")


def _dense_fake(rows_from, w_from):
    def fake(*args, **kw):
        x, w = args[rows_from], args[w_from]
        return x.new_empty((x.size(0), w.size(0)), dtype=torch.bfloat16)
    return fake


@_define("mxfp4_wmma_gemm(Tensor w, Tensor x, Tensor scales, Tensor? bias) -> Tensor",
         fake=_dense_fake(1, 0))
def mxfp4_wmma_gemm(w, x, scales, bias=None, block_m=None):
    _check(w.dim() == 2 and x.dim() == 2, "bad ranks")
    _check(x.size(1) % 128 == 0, "K must be a multiple of 128")
    out = torch.empty(x.size(0), w.size(0), dtype=torch.bfloat16, device=x.device)
    if x.size(0):
        _gemm_w4(out, x, w, scales, bias, None, None, 1, block_m or _dense_block_m(x.size(0)),
                 _W_MXFP4, 32, 0)
    return out


def _dense_cfg_fake(w, x, *a):
    return x.new_empty((x.size(0), w.size(0)), dtype=torch.bfloat16)


@_define("mxfp4_wmma_gemm_cfg(Tensor w, Tensor x, Tensor scales, Tensor? bias, int cfg) -> Tensor",
         fake=_dense_cfg_fake)
def mxfp4_wmma_gemm_cfg(w, x, scales, bias, cfg):
    """mxfp4_wmma_gemm pinned to the token tile TILE_CFGS[cfg] instead of the choice
    by row count (bench-only, as csrc/torch_ops.cpp:288-292 of the reference)."""
    return mxfp4_wmma_gemm(w, x, scales, bias, _cfg_block_m(cfg))


@_define("mxfp4_gemv(Tensor x, Tensor w, Tensor scales) -> Tensor", fake=_dense_fake(0, 1))
def mxfp4_gemv(x, w, scales):
    _check(1 <= x.size(0) <= 8, "mxfp4_gemv takes 1-8 rows")
    return mxfp4_wmma_gemm(w, x, scales, None)


@_define("w4a16_wmma_gemm(Tensor x, Tensor w, Tensor scales, Tensor? bias, int group_size) -> Tensor",
         fake=_dense_fake(0, 1))
def w4a16_wmma_gemm(x, w, scales, bias, group_size):
    """int4 weights in vLLM's ExLlama word order (each 32-bit word holds k = 0 2 4 6 1
    3 5 7 in its nibbles; uint8 or int8 view [N, K / 2]), as the reference's dense op
    (csrc/gemm/w8a8_wmma_gemm.hip:128-132); the MoE ops keep the sequential order."""
    _check(group_size in (32, 64, 128), "group_size must be 32, 64 or 128")
    out = torch.empty(x.size(0), w.size(0), dtype=torch.bfloat16, device=x.device)
    if x.size(0):
        _gemm_w4(out, x, _as_u8(w), scales, bias, None, None, 1, _dense_block_m(x.size(0)),
                 _W_INT4X, group_size, 0)
    return out


def _as_u8(w):
    return w.view(torch.uint8) if w.dtype == torch.int8 else w


def _dequant(w, scales, fmt, group, scale_kind, k):
    n = w.size(0)
    out = torch.empty(n, k, dtype=torch.bfloat16, device=w.device)
    _check(w.dim() == 2 and w.stride(1) == 1, "w must be [N, bytes] with a contiguous last dim")
    s_n = scales.stride(0)
    s_g = scales.stride(1) if scales.dim() == 2 else 0
    sdt = _SCALE_DTYPES.get(scales.dtype, 0)
    with torch.cuda.device(w.device):
        _lib.call("strix_dequant_bf16", out.data_ptr(), w.data_ptr(), scales.data_ptr(), n, k,
                  w.stride(0), out.stride(0), s_n, s_g, fmt, group, scale_kind, sdt, _stream())
    return out


def _dq_fake(w, scales, *a):
    return w.new_empty((w.size(0), w.size(1) * (1 if w.dtype == torch.float8_e4m3fn else 2)),
                       dtype=torch.bfloat16)


@_define("mxfp4_dequant(Tensor w, Tensor scales) -> Tensor", fake=_dq_fake)
def mxfp4_dequant(w, scales):
    k = w.size(1) * 2
    _check(w.dtype == torch.uint8 and scales.dtype == torch.uint8, "scale must be uint8 (e8m0)")
    _check(k % 32 == 0 and tuple(scales.shape) == (w.size(0), k // 32), "scales must be [N, K / 32]")
    return _dequant(w, scales, 0, 32, 0, k)


@_define("w4a16_dequant(Tensor w, Tensor scales, int group_size) -> Tensor", fake=_dq_fake)
def w4a16_dequant(w, scales, group_size):
    w = _as_u8(w)
    k = w.size(1) * 2
    _check(w.dtype == torch.uint8 and scales.dtype in (torch.bfloat16, torch.float16),
           "w uint8, scales bf16 or fp16")
    _check(group_size in (32, 64, 128) and tuple(scales.shape) == (w.size(0), k // group_size),
           "scales must be [N, K / group_size]")
    return _dequant(w, scales, 3, group_size, 0, k)     # 3: int4 in ExLlama word order


@_define("fp8_dequant(Tensor w, Tensor scales) -> Tensor", fake=_dq_fake)
def fp8_dequant(w, scales):
    n, k = w.shape
    _check(w.dtype == torch.float8_e4m3fn and scales.dtype == torch.float32, "w e4m3, scales fp32")
    if scales.dim() == 2 and scales.size(1) != 1:
        _check(k % 128 == 0 and tuple(scales.shape) == ((n + 127) // 128, k // 128),
               "block scales must be [ceil(N/128), K/128]")
        return _dequant(w, scales, 2, 128, 2, k)
    _check(scales.numel() == n, "channel scales must be [N]")
    return _dequant(w, scales.reshape(n), 2, 128, 1, k)


def _dense_w8(x, w, scales, bias, wfmt, afmt, scale_kind, group=0, block_m=None):
    m, k = x.shape
    n = w.size(0)
    _check(w.dim() == 2 and w.size(1) == k and x.stride(1) == 1 and w.stride(1) == 1,
           "shape mismatch / last dims must be contiguous")
    _check(k % 128 == 0, "K must be a multiple of 128")
    out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    bias_stride = 0
    if bias is not None:
        _check(bias.dtype == torch.bfloat16 and bias.stride(-1) == 1
               and (tuple(bias.shape) == (n,) or tuple(bias.shape) == (m, n)),
               "bias must be bf16 [N] or [M, N]")
        bias_stride = bias.stride(0) if bias.dim() == 2 else 0
    if m:
        with torch.cuda.device(x.device):
            _lib.call("strix_dense_gemm_w8a16", out.data_ptr(), x.data_ptr(), w.data_ptr(),
                      scales.data_ptr(), _ptr(bias), m, n, k, x.stride(0), out.stride(0), w.stride(0),
                      scales.stride(0) if scale_kind != _S_CHANNEL else 0, bias_stride,
                      block_m or _dense_block_m(m), wfmt, afmt, scale_kind,
                      _SCALE_DTYPES[scales.dtype], group, _stream())
    return out


@_define("w8a16_skinny_gemm(Tensor in_a, Tensor in_b, Tensor in_scale, Tensor? in_bias, int CuCount, "
         "int group_size) -> Tensor", fake=_dense_fake(1, 0))
def w8a16_skinny_gemm(in_a, in_b, in_scale, in_bias, CuCount, group_size):
    """in_a: excess-128 weights uint8 [N, K]; in_b: activations bf16 [M <= 8, K];
    in_scale: 16-bit [N] (group_size 0) or [N, K / group_size] (32, 64 or 128)."""
    _check(1 <= in_b.size(0) <= 8, "w8a16_skinny_gemm takes 1-8 rows")
    _check(in_a.dtype == torch.uint8 and in_b.dtype == torch.bfloat16
           and in_scale.dtype in _SCALE_DTYPES, "in_a uint8, in_b bf16")
    _check(group_size in (0, 32, 64, 128), "group_size must be 0, 32, 64 or 128")
    n, k = in_a.shape
    if group_size:
        _check(tuple(in_scale.shape) == (n, k // group_size) and in_scale.stride(1) == 1,
               f"scales must be [N, K / {group_size}]")
        return _dense_w8(in_b, in_a, in_scale, in_bias, _W_U8B128, _A_BF16, _S_GROUP, group_size)
    _check(in_scale.numel() == n, "scales must be [N]")
    return _dense_w8(in_b, in_a, in_scale.reshape(n), in_bias, _W_U8B128, _A_BF16, _S_CHANNEL)


def _fp8_dense(w, x, scales, bias, afmt, block_m=None):
    _check(w.dtype == torch.float8_e4m3fn and scales.dtype == torch.float32, "w e4m3, scales fp32")
    n, k = w.shape
    if scales.dim() == 2 and scales.size(1) != 1:
        _check(tuple(scales.shape) == ((n + 127) // 128, k // 128) and scales.stride(1) == 1,
               "block scales must be [ceil(N/128), K/128]")
        return _dense_w8(x, w, scales, bias, _W_E4M3, afmt, _S_BLOCK, block_m=block_m)
    _check(scales.numel() == n, "channel scales must be [N]")
    return _dense_w8(x, w, scales.reshape(n), bias, _W_E4M3, afmt, _S_CHANNEL, block_m=block_m)


@_define("fp8_skinny_gemm(Tensor in_a, Tensor in_b, Tensor in_scale, Tensor? in_bias, int CuCount) "
         "-> Tensor", fake=_dense_fake(1, 0))
def fp8_skinny_gemm(in_a, in_b, in_scale, in_bias, CuCount):
    _check(1 <= in_b.size(0) <= 8, "fp8_skinny_gemm takes 1-8 rows")
    _check(in_b.dtype == torch.bfloat16, "in_b must be bf16")
    return _fp8_dense(in_a, in_b, in_scale, in_bias, _A_BF16)


@_define("fp8_wmma_gemm(Tensor w, Tensor x, Tensor scales) -> Tensor", fake=_dense_fake(1, 0))
def fp8_wmma_gemm(w, x, scales):
    _check(x.dtype == torch.bfloat16, "x must be bf16")
    return _fp8_dense(w, x, scales, None, _A_BF16)


@_define("fp8_wmma_gemm_raw(Tensor w, Tensor x, Tensor scales) -> Tensor", fake=_dense_fake(1, 0))
def fp8_wmma_gemm_raw(w, x, scales):
    _check(x.dtype == torch.float16, "x must be fp16")
    return _fp8_dense(w, x, scales, None, _A_F16)


@_define("fp8_wmma_gemm_cfg(Tensor w, Tensor x, Tensor scales, int cfg) -> Tensor",
         fake=_dense_cfg_fake)
def fp8_wmma_gemm_cfg(w, x, scales, cfg):
    """fp8_wmma_gemm pinned to the token tile TILE_CFGS[cfg] (bench-only, as
    csrc/torch_ops.cpp:258 of the reference)."""
    _check(x.dtype == torch.bfloat16, "x must be bf16")
    return _fp8_dense(w, x, scales, None, _A_BF16, _cfg_block_m(cfg))


@_define("fp8_wmma_gemm_raw_cfg(Tensor w, Tensor x, Tensor scales, int cfg) -> Tensor",
         fake=_dense_cfg_fake)
def fp8_wmma_gemm_raw_cfg(w, x, scales, cfg):
    """fp8_wmma_gemm_raw pinned to the token tile TILE_CFGS[cfg] (bench-only, as
    csrc/torch_ops.cpp:260 of the reference)."""
    _check(x.dtype == torch.float16, "x must be fp16")
    return _fp8_dense(w, x, scales, None, _A_F16, _cfg_block_m(cfg))


def _gemm_a8(c, qa, sa, w, scales, routing, topk_weights, top_k, block_m, wfmt, gate,
             s_sn, s_sg, scale_kind):
    """Host side of strix_gemm_w8a8_group (int8 activations, per-128-group fold)."""
    dense = routing is None
    n = w.size(-2)
    k = qa.size(1)
    _check(qa.dtype == torch.int8 and qa.stride(1) == 1 and sa.dtype == torch.float32
           and tuple(sa.shape) == (qa.size(0), k // 128) and sa.stride(1) == 1,
           "qa int8 [rows, K], sa fp32 [rows, K / 128]")
    _check(k % 128 == 0, "K must be a multiple of 128")
    if dense:
        sid = eid = npp = None
        m = qa.size(0)
        e, w_se, w_sn, s_se = 1, 0, w.stride(0), 0
        sorted_len, expert_len, num_valid = (m + block_m - 1) // block_m * block_m, 0, m
    else:
        sid, eid, npp = routing
        _check(sid.dtype == torch.int32 and eid.dtype == torch.int32 and npp.dtype == torch.int32,
               "routing tensors must be int32")
        _check(eid.numel() * block_m >= sid.numel(), f"expert_ids too short for block_m {block_m}")
        e, w_se, w_sn, s_se = w.size(0), w.stride(0), w.stride(1), scales.stride(0)
        sorted_len, expert_len, num_valid = sid.numel(), eid.numel(), c.size(0)
    with torch.cuda.device(c.device):
        _lib.call("strix_gemm_w8a8_group", c.data_ptr(), qa.data_ptr(), sa.data_ptr(), w.data_ptr(),
                  scales.data_ptr(), _ptr(sid), _ptr(eid), _ptr(npp), _ptr(topk_weights), num_valid,
                  qa.size(0), e, n, k, qa.stride(0), c.stride(0), w_se, w_sn, s_se, s_sn, s_sg,
                  sa.stride(0), sorted_len, expert_len, top_k, block_m, wfmt, scale_kind,
                  _SCALE_DTYPES[scales.dtype], gate, _stream())


@_define("moe_gemm_w4a8(Tensor(a!) c, Tensor qa, Tensor sa, Tensor b, Tensor scales, "
         "Tensor sorted_ids, Tensor expert_ids, Tensor num_post_padded, Tensor? topk_weights, "
         "int top_k, int block_m, int block_n, bool silu_mul=False, str activation='silu') -> ()")
def moe_gemm_w4a8(c, qa, sa, b, scales, sorted_ids, expert_ids, num_post_padded, topk_weights,
                  top_k, block_m, block_n, silu_mul=False, activation="silu"):
    _check(activation in _ACTS, f"activation must be silu or gelu_tanh, got {activation}")
    _check(b.dtype == torch.uint8 and b.dim() == 3 and b.size(2) * 2 == qa.size(1)
           and b.stride(2) == 1 and c.dtype == torch.bfloat16, "b uint8 [E, N, K / 2], c bf16")
    e, n, _ = b.shape
    _check(scales.dtype in (torch.bfloat16, torch.float16)
           and tuple(scales.shape) == (e, n, qa.size(1) // 128) and scales.stride(2) == 1,
           "scales must be bf16 or fp16 [E, N, K / 128]")
    _check(c.size(1) == (n // 2 if silu_mul else n), "shape mismatch")
    _check(not silu_mul or topk_weights is None, "silu_mul needs even N and no topk weights")
    _gemm_a8(c, qa, sa, b, scales, (sorted_ids, expert_ids, num_post_padded), topk_weights, top_k,
             block_m, _W_INT4, _ACTS[activation] if silu_mul else 0, scales.stride(1), 1, _S_GROUP)


@_define("w8a8_wmma_gemm(Tensor in_w8, Tensor in_act, Tensor in_scale) -> Tensor",
         fake=_dense_fake(1, 0))
def w8a8_wmma_gemm(in_w8, in_act, in_scale, block_m=None):
    """Excess-128 byte weights [N, K] x bf16 activations quantised to int8 per (row,
    128 group) inside the op; int32-exact sums per group, fp32 fold. in_scale fp32
    [N], [K/128, N] (group-major) or [N, K/128]."""
    n, k = in_w8.shape
    m = in_act.size(0)
    _check(in_w8.dtype == torch.uint8 and in_w8.stride(1) == 1, "in_w8 must be uint8 [N, K]")
    _check(in_act.dtype == torch.bfloat16 and in_act.dim() == 2 and in_act.size(1) == k,
           "in_act must be bf16 [M, K]")
    _check(k % 128 == 0, "K must be a multiple of 128")
    _check(in_scale.dtype == torch.float32, "in_scale must be fp32")
    g = k // 128
    if in_scale.dim() == 1 or in_scale.numel() == n:
        _check(in_scale.numel() == n, "in_scale must be [N], [K/128, N] or [N, K/128]")
        kind, s_sn, s_sg, sc = _S_CHANNEL, 0, 1, in_scale.reshape(n)
    elif tuple(in_scale.shape) == (g, n):
        kind, s_sn, s_sg, sc = _S_GROUP, in_scale.stride(1), in_scale.stride(0), in_scale
    else:
        _check(tuple(in_scale.shape) == (n, g), "in_scale must be [N], [K/128, N] or [N, K/128]")
        kind, s_sn, s_sg, sc = _S_GROUP, in_scale.stride(0), in_scale.stride(1), in_scale
    out = torch.empty(m, n, dtype=torch.bfloat16, device=in_act.device)
    if m == 0:
        return out
    qa = torch.empty(m, k, dtype=torch.int8, device=in_act.device)
    sa = torch.empty(m, g, dtype=torch.float32, device=in_act.device)
    moe_act_quant_i8(in_act, qa, sa)
    _gemm_a8(out, qa, sa, in_w8, sc, None, None, 1, block_m or _dense_block_m(m), _W_U8B128, 0,
             s_sn, s_sg, kind)
    return out


@_define("w8a8_wmma_gemm_cfg(Tensor in_w8, Tensor in_act, Tensor in_scale, int cfg) -> Tensor",
         fake=_dense_cfg_fake)
def w8a8_wmma_gemm_cfg(in_w8, in_act, in_scale, cfg):
    """w8a8_wmma_gemm pinned to the token tile TILE_CFGS[cfg]: same arithmetic and the
    same activation quantiser (bench-only, as csrc/torch_ops.cpp:280-282 of the
    reference; any row count, where the reference wants a multiple of 128)."""
    return w8a8_wmma_gemm(in_w8, in_act, in_scale, _cfg_block_m(cfg))


@_define("w4a8_wmma_gemm(Tensor in_w4, Tensor in_act, Tensor in_scale) -> Tensor",
         fake=_dense_fake(1, 0))
def w4a8_wmma_gemm(in_w4, in_act, in_scale):
    """int4 weights (nibble - 8, ExLlama word order, uint8 or int8 view [N, K / 2]) x
    bf16 activations quantised to int8 per (row, 128 group) inside the op; int32-exact
    sums per group, fp32 fold (csrc/torch_ops.cpp:283,
    csrc/gemm/w8a8_wmma_gemm.hip:128-132,278-291 of the reference). in_scale fp32 [N]
    or [K/128, N] (group-major). The [K/32, N] form (a weight scale per 32 elements
    cannot ride a 128-wide integer sum) runs on the bf16-activation kernel instead:
    the activations are not quantised there, the scales are rounded to bf16."""
    w = _as_u8(in_w4)
    n, k = w.size(0), w.size(1) * 2
    m = in_act.size(0)
    _check(w.dtype == torch.uint8 and w.dim() == 2 and w.stride(1) == 1, "in_w4 must be 8-bit [N, K / 2]")
    _check(in_act.dtype == torch.bfloat16 and in_act.dim() == 2 and in_act.size(1) == k,
           "in_act must be bf16 [M, K]")
    _check(k % 128 == 0, "K must be a multiple of 128")
    _check(in_scale.dtype == torch.float32, "in_scale must be fp32")
    g = k // 128
    if in_scale.numel() != n and tuple(in_scale.shape) == (k // 32, n):
        return w4a16_wmma_gemm(in_act, w, in_scale.t().to(torch.bfloat16).contiguous(), None, 32)
    if in_scale.numel() == n:
        kind, s_sn, s_sg, sc = _S_CHANNEL, 0, 1, in_scale.reshape(n)
    else:
        _check(tuple(in_scale.shape) == (g, n), "in_scale must be [N], [K/128, N] or [K/32, N]")
        kind, s_sn, s_sg, sc = _S_GROUP, in_scale.stride(1), in_scale.stride(0), in_scale
    out = torch.empty(m, n, dtype=torch.bfloat16, device=in_act.device)
    if m == 0:
        return out
    qa = torch.empty(m, k, dtype=torch.int8, device=in_act.device)
    sa = torch.empty(m, g, dtype=torch.float32, device=in_act.device)
    moe_act_quant_i8(in_act, qa, sa)
    _gemm_a8(out, qa, sa, w, sc, None, None, 1, _dense_block_m(m), _W_INT4X, 0, s_sn, s_sg, kind)
    return out


# ------------------------------------------------------------ dense quantized GEMMs

def _w8a8_int8_fake(a_q, a_scale, w, w_scale, acc_out=None):
    return a_q.new_empty((a_q.size(0), w.size(0)), dtype=torch.bfloat16)


# Not in the reference: the per-token form of its w8a8_wmma_gemm
# (csrc/torch_ops.cpp:277, which takes bf16 activations and quantises per
# 128-group inside). acc_out, if given, receives the exact int32 sums.
@_define("w8a8_int8_gemm(Tensor a_q, Tensor a_scale, Tensor w, Tensor w_scale, "
         "Tensor(a!)? acc_out=None) -> Tensor", fake=_w8a8_int8_fake)
def w8a8_int8_gemm(a_q, a_scale, w, w_scale, acc_out=None):
    _check(a_q.dim() == 2 and w.dim() == 2 and a_q.dtype == torch.int8 and w.dtype == torch.int8
           and a_q.size(1) == w.size(1) and a_q.stride(1) == 1 and w.stride(1) == 1,
           "a_q int8 [M, K], w int8 [N, K]")
    m, k = a_q.shape
    n = w.size(0)
    _check(k % 128 == 0, "K must be a multiple of 128")
    _check(a_scale.dtype == torch.float32 and a_scale.numel() == m and a_scale.is_contiguous()
           and w_scale.dtype == torch.float32 and w_scale.numel() == n and w_scale.is_contiguous(),
           "scales must be contiguous fp32 [M] and [N]")
    out = torch.empty(m, n, dtype=torch.bfloat16, device=a_q.device)
    if acc_out is not None:
        _check(acc_out.dtype == torch.int32 and tuple(acc_out.shape) == (m, n)
               and acc_out.is_contiguous(), "acc_out must be contiguous int32 [M, N]")
    with torch.cuda.device(a_q.device):
        _lib.call("strix_w8a8_int8_gemm", out.data_ptr(), _ptr(acc_out), a_q.data_ptr(),
                  a_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(), m, n, k, a_q.stride(0),
                  w.stride(0), out.stride(0), _stream())
        _lib.after_tcgen05("w8a8_int8_gemm")
    return out


def _act_quant_token_fake(x):
    return (x.new_empty(x.shape, dtype=torch.int8),
            x.new_empty((x.size(0),), dtype=torch.float32))


@_define("act_quant_token_i8(Tensor x) -> (Tensor, Tensor)", fake=_act_quant_token_fake)
def act_quant_token_i8(x):
    """(q int8 [M, K], scale fp32 [M]): dynamic symmetric per-token quantisation, the
    activation form w8a8_int8_gemm takes."""
    _check(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and x.stride(1) == 1
           and x.size(1) % 8 == 0, "x must be bf16 or fp16 [M, K], K a multiple of 8")
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x.size(0), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call("strix_act_quant_token_i8", x.data_ptr(), q.data_ptr(), s.data_ptr(), x.size(0),
                  x.size(1), x.stride(0), q.stride(0), int(x.dtype == torch.float16), _stream())
    return q, s


# ----------------------------------------------------------- tcgen05 layout probe

def _umma_tile_fake(a, b):
    return a.new_empty((128, b.size(0)), dtype=torch.int32 if a.dtype == torch.int8 else torch.float32)


@_define("_umma_tile(Tensor a, Tensor b) -> Tensor", fake=_umma_tile_fake)
def _umma_tile(a, b):
    """D[128, N] = A[128, K] @ B[N, K]^T on one CTA through tcgen05 / TMEM: int8
    operands give an exact int32 result, float8_e4m3fn operands an fp32 one."""
    _check(a.dim() == 2 and b.dim() == 2 and a.size(0) == 128 and a.size(1) == b.size(1)
           and a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype
           and a.dtype in (torch.int8, torch.float8_e4m3fn),
           "a [128, K], b [N, K]: contiguous int8 or float8_e4m3fn")
    kind = 0 if a.dtype == torch.int8 else 1
    d = torch.empty(128, b.size(0), dtype=torch.int32 if kind == 0 else torch.float32,
                    device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        _lib.call("strix_umma_tile", d.data_ptr(), a.data_ptr(), b.data_ptr(), status.data_ptr(),
                  b.size(0), a.size(1), kind, _stream())
    _check(int(status.item()) == 0, "_umma_tile: a bounded wait ran out inside the kernel")
    return d
