"""The allocation-free decode entry point against the ordinary one.

strix_attn_decode_bf16_static is for hosts that cannot give the library scratch
memory (they own only the input and output buffers, or their device memory was
budgeted at start-up): it keeps the split-KV partials in an array built into
the library. This file is named to be collected last, so a run that stops at
the first failure has already run every other test. It calls both entry points
through the C-ABI with raw pointers and must pass alone in a fresh process as
well as after the other tests.
"""

import pytest
import torch

pytest.importorskip("libstrix_b200", reason="libstrix_b200.so is not built")   # noqa: E402
from libstrix_b200 import _lib  # noqa: E402
from libstrix_b200.workloads import decode_batch  # noqa: E402
from oracle import attention as A  # noqa: E402

DEV = "cuda"


def oracle_ok(out, b):
    """The output against the CPU oracle, at the bound the decode tests use."""
    c = b.to("cpu")
    ref = A.decode_reference(c.q, c.key_cache, c.value_cache, c.k_scale, c.v_scale, c.seq_lens,
                             c.block_table, c.scale)
    err = (out.float().cpu() - ref).abs()
    rms = ref.pow(2).mean().sqrt().item()
    return bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all())


def _args(b, out, workspace, num_splits):
    """Argument list of strix_attn_decode_bf16; drop `workspace` for the static form."""
    head = [out.data_ptr(), b.q.data_ptr(), b.key_cache.data_ptr(), b.value_cache.data_ptr(),
            b.k_scale.data_ptr(), b.v_scale.data_ptr(), b.seq_lens.data_ptr(),
            b.block_table.data_ptr(), None]
    tail = [b.q.size(0), b.q.size(1), b.key_cache.size(2), b.q.size(2), b.key_cache.size(1),
            b.block_table.size(1), b.block_table.stride(0),
            b.q.stride(0), b.q.stride(1), out.stride(0), out.stride(1),
            *b.key_cache.stride()[:3], *b.value_cache.stride()[:3],
            *b.k_scale.stride(), *b.v_scale.stride(),
            float(b.scale), num_splits, -1, 1, torch.cuda.current_stream().cuda_stream]
    return head + ([] if workspace is False else [workspace]) + tail


@pytest.mark.gpu
def test_static_scratch_matches_the_workspace_entry_point_twice_in_a_row():
    lib = _lib.load()
    b = decode_batch(ctx_lens=[3000, 77, 1500, 9], seed=11).to(DEV)
    for call, num_splits in enumerate((4, 13)):   # two calls in a row, different partitions
        nbytes = lib.strix_attn_decode_workspace(b.q.size(0), b.q.size(1), b.q.size(2), num_splits,
                                                 b.block_table.size(1), 16)
        assert 0 < nbytes <= 16 * 1024 * 1024
        ws = torch.empty(nbytes // 4, dtype=torch.float32, device=DEV)
        want = torch.full_like(b.q, float("nan"))
        got = torch.full_like(b.q, float("nan"))
        _lib.call("strix_attn_decode_bf16", *_args(b, want, ws.data_ptr(), num_splits))
        _lib.call("strix_attn_decode_bf16_static", *_args(b, got, False, num_splits))
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), f"call {call}"
        # same kernels, same partition: the tests' tolerance (2e-2) is far from tight here
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want), f"call {call}"
        assert oracle_ok(got, b), f"call {call}: the static entry point against the oracle"
    # a shorter batch afterwards sees the previous call's leftovers in the array
    b2 = decode_batch(ctx_lens=[40, 700], seed=12).to(DEV)
    ws = torch.empty(lib.strix_attn_decode_workspace(2, 32, 128, 4, b2.block_table.size(1), 16) // 4,
                     dtype=torch.float32, device=DEV)
    want, got = torch.empty_like(b2.q), torch.empty_like(b2.q)
    _lib.call("strix_attn_decode_bf16", *_args(b2, want, ws.data_ptr(), 4))
    _lib.call("strix_attn_decode_bf16_static", *_args(b2, got, False, 4))
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert oracle_ok(got, b2)


@pytest.mark.gpu
def test_static_scratch_single_segment_and_exact_capacity():
    """num_splits = 1 needs no scratch at all (no partials, no array lookup); a launch
    whose partials fill the 16 MiB array exactly is still accepted."""
    lib = _lib.load()
    b = decode_batch(ctx_lens=[500, 31], seed=13).to(DEV)
    assert lib.strix_attn_decode_workspace(2, 32, 128, 1, b.block_table.size(1), 16) == 0
    got = torch.full_like(b.q, float("nan"))
    _lib.call("strix_attn_decode_bf16_static", *_args(b, got, False, 1))
    torch.cuda.synchronize()
    assert oracle_ok(got, b)
    # 16 sequences x 32 heads x 63 segments x 130 floats x 4 bytes = 16,773,120 <= 16 MiB;
    # one more segment would not fit
    big = decode_batch(ctx_lens=[300 + 64 * i for i in range(16)], seed=14).to(DEV)
    need = lib.strix_attn_decode_workspace(16, 32, 128, 63, big.block_table.size(1), 16)
    assert need == 16 * 32 * 63 * 130 * 4 <= 16 * 1024 * 1024
    assert lib.strix_attn_decode_workspace(16, 32, 128, 64, big.block_table.size(1), 16) > 16 * 1024 * 1024
    got = torch.full_like(big.q, float("nan"))
    _lib.call("strix_attn_decode_bf16_static", *_args(big, got, False, 63))
    torch.cuda.synchronize()
    assert oracle_ok(got, big)


def test_static_scratch_rejects_oversized_launches():
    """Needs no GPU: the size check comes before any CUDA call."""
    # 64 sequences x 32 heads x 64 segments x 130 floats = 68 MB > 16 MiB
    args = [8, 8, 16, 16, 4, 4, 4, 4, None,
            64, 32, 4, 128, 16, 4096, 4096, 4096, 128, 4096, 128,
            8192, 512, 128, 8192, 512, 128, 64, 4, 1, 64, 4, 1,
            0.1, 64, -1, 1, None]
    with pytest.raises(_lib.StrixError, match="built-in array holds 16777216"):
        _lib.call("strix_attn_decode_bf16_static", *args)
