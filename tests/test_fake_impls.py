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
