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

import torch

from . import _lib

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
