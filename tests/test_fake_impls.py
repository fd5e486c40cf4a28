"""Shape inference of the tensor-returning ops under FakeTensorMode (what
torch.compile / vLLM's profiling trace sees), as the reference registers fakes for
the same ops (python/strix/__init__.py:380-460). Needs no GPU."""

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import libstrix_b200  # noqa: F401  (registers torch.ops.strix)

ops = torch.ops.strix
M, N, K = 7, 256, 1024


def _t(*shape, dtype):
    return torch.empty(*shape, dtype=dtype, device="cuda")


CASES = {
    "fp8_wmma_gemm": lambda: ops.fp8_wmma_gemm(
        _t(N, K, dtype=torch.float8_e4m3fn), _t(M, K, dtype=torch.bfloat16), _t(2, 8, dtype=torch.float32)),
    "fp8_wmma_gemm_cfg": lambda: ops.fp8_wmma_gemm_cfg(
        _t(N, K, dtype=torch.float8_e4m3fn), _t(M, K, dtype=torch.bfloat16), _t(2, 8, dtype=torch.float32), 1),
    "fp8_wmma_gemm_raw_cfg": lambda: ops.fp8_wmma_gemm_raw_cfg(
        _t(N, K, dtype=torch.float8_e4m3fn), _t(M, K, dtype=torch.float16), _t(N, dtype=torch.float32), 2),
    "mxfp4_wmma_gemm": lambda: ops.mxfp4_wmma_gemm(
        _t(N, K // 2, dtype=torch.uint8), _t(M, K, dtype=torch.bfloat16), _t(N, K // 32, dtype=torch.uint8), None),
    "mxfp4_wmma_gemm_cfg": lambda: ops.mxfp4_wmma_gemm_cfg(
        _t(N, K // 2, dtype=torch.uint8), _t(M, K, dtype=torch.bfloat16), _t(N, K // 32, dtype=torch.uint8), None, 0),
    "w8a8_wmma_gemm": lambda: ops.w8a8_wmma_gemm(
        _t(N, K, dtype=torch.uint8), _t(M, K, dtype=torch.bfloat16), _t(N, dtype=torch.float32)),
    "w8a8_wmma_gemm_cfg": lambda: ops.w8a8_wmma_gemm_cfg(
        _t(N, K, dtype=torch.uint8), _t(M, K, dtype=torch.bfloat16), _t(N, dtype=torch.float32), 0),
    "w4a8_wmma_gemm": lambda: ops.w4a8_wmma_gemm(
        _t(N, K // 2, dtype=torch.uint8), _t(M, K, dtype=torch.bfloat16), _t(K // 32, N, dtype=torch.float32)),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_fake_output_is_bf16_rows_by_channels(name):
    with FakeTensorMode():
        out = CASES[name]()
    assert tuple(out.shape) == (M, N) and out.dtype == torch.bfloat16


def test_query_regrouping_of_the_grouped_decode_form():
    """group_queries puts query head h * G + j of sequence n at row n * G + j, head h -
    also for a q that is a strided slice of a fused qkv tensor - and ungroup_queries is
    its inverse."""
    from libstrix_b200 import torch_ops

    nseq, hkv, g, d = 3, 2, 4, 8
    qkv = torch.randn(nseq, (hkv * g + 2 * hkv) * d)
    q = qkv[:, :hkv * g * d].view(nseq, hkv * g, d)
    qg = torch_ops.group_queries(q, hkv)
    assert qg.is_contiguous() and tuple(qg.shape) == (nseq * g, hkv, d)
    for n in range(nseq):
        for h in range(hkv):
            for j in range(g):
                assert torch.equal(qg[n * g + j, h], q[n, h * g + j])
    assert torch.equal(torch_ops.ungroup_queries(qg, nseq), q)
