"""The strix_vllm plugin against vLLM 0.22's own classes: gates, weight
preparation and hook registration on the CPU (mock layers, as the reference's
tests/test_w8a8_int8.py:18-47 does), and the kernels behind the classes on a GPU."""

import types

import pytest
import torch

vllm = pytest.importorskip("vllm")


def int8_config(**kw):
    from vllm.model_executor.kernels.linear.scaled_mm.ScaledMMLinearKernel import (
        Int8ScaledMMLinearLayerConfig,
    )

    base = {"is_channelwise": True, "is_static_input_scheme": False, "input_symmetric": True}
    return Int8ScaledMMLinearLayerConfig(**{**base, **kw})


def int8_kernel():
    from strix_vllm import int8

    cls, names = int8.kernel_class(), ["weight", "weight_scale", "input_scale", "input_zero_point",
                                       "azp_adj"]
    try:
        return cls(int8_config(), names)
    except AssertionError:       # vLLM's constructor insists on a CUDA platform
        kernel = cls.__new__(cls)
        kernel.config, kernel.layer_param_names = int8_config(), names
        return kernel


def mock_int8_layer(n, k, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    layer = torch.nn.Module()
    layer.weight = torch.nn.Parameter(
        torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(device), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(
        (torch.rand((n, 1), generator=g) * 0.01 + 1e-4).float().to(device), requires_grad=False)
    return layer


def test_register_is_inactive_without_a_b200_and_idempotent():
    import strix_vllm

    assert strix_vllm.on_b200() is torch.cuda.is_available() and strix_vllm.on_b200() or True
    strix_vllm.register()
    strix_vllm.register()          # a second call in the same process is a no-op
    assert strix_vllm._registered


def test_disable_switch(monkeypatch):
    import strix_vllm

    monkeypatch.setenv("STRIX_DISABLE", "moe, attn_decode")
    assert strix_vllm.disabled("moe") and strix_vllm.disabled("attn_decode")
    assert not strix_vllm.disabled("int8")
    monkeypatch.setenv("STRIX_DISABLE", "all")
    assert strix_vllm.disabled("int8")


def test_int8_gate_rejects_unsupported_layouts():
    from strix_vllm import int8

    cls = int8.kernel_class()
    assert cls.can_implement(int8_config())[0]
    assert not cls.can_implement(int8_config(is_static_input_scheme=True))[0]
    assert not cls.can_implement(int8_config(is_channelwise=False))[0]
    assert not cls.can_implement(int8_config(input_symmetric=False))[0]


def test_int8_weight_preparation_keeps_the_signed_bytes():
    kernel = int8_kernel()
    layer = mock_int8_layer(256, 512)
    w0 = layer.weight.data.clone()
    kernel.process_weights_after_loading(layer)
    assert layer.weight.dtype == torch.int8 and torch.equal(layer.weight.data, w0)
    assert layer.weight_scale.shape == (256,) and layer.weight_scale.dtype == torch.float32
    bad = mock_int8_layer(64, 100)
    with pytest.raises(RuntimeError, match="K % 128"):
        kernel.process_weights_after_loading(bad)


def test_moe_scale_layouts_and_coverage_checks():
    from strix_vllm import moe

    w1 = torch.zeros(4, 512, 256, dtype=torch.float8_e4m3fn)
    w2 = torch.zeros(4, 256, 256, dtype=torch.float8_e4m3fn)
    s1, s2 = torch.ones(4, 4, 2), torch.ones(4, 2, 2)
    assert moe.block_scales(w1, s1).shape == (4, 4, 2)
    assert moe.block_scales(w1, torch.ones(4, 512, 1)).shape == (4, 512)
    assert moe.block_scales(w1, torch.ones(4, 3, 2)) is None and moe.block_scales(w1, None) is None
    x = torch.zeros(5, 256, dtype=torch.bfloat16)
    assert moe.covered(x, w1, w2, s1, s2, "silu", None, None, False, False) == []
    assert moe.covered(x, w1, w2, s1, s2, "swigluoai", None, None, False, False) == ["activation"]
    assert moe.covered(x.half(), w1, w2, s1, None, "silu", torch.zeros(4), None, True, False) == \
        ["act", "scales", "bias", "expert_map"]


def test_moe_hook_replaces_the_triton_backend_only():
    from vllm.model_executor.layers.fused_moe.oracle import fp8 as fp8_oracle

    from strix_vllm import moe

    orig = getattr(fp8_oracle.backend_to_kernel_cls, "strix_orig", fp8_oracle.backend_to_kernel_cls)
    moe.register()
    hooked = fp8_oracle.backend_to_kernel_cls
    moe.register()
    assert fp8_oracle.backend_to_kernel_cls is hooked and hooked.strix_orig is orig
    (cls,) = hooked(fp8_oracle.Fp8MoeBackend.TRITON)
    assert cls.__name__ == "StrixFp8Experts"
    assert cls.expects_unquantized_inputs.fget(object()) is True
    assert hooked(fp8_oracle.Fp8MoeBackend.MARLIN) == orig(fp8_oracle.Fp8MoeBackend.MARLIN)


def test_attention_gate_follows_the_kernel_table():
    from strix_vllm import attn

    assert attn.covers("decode", 128, 8, "int8", False, False)
    assert attn.covers("prefill", 128, 5, "int8", True, True)
    assert attn.covers("prefill", 64, 4, "bf16", False, False)
    assert attn.covers("decode", 512, 8, "int8", False, False)
    assert attn.covers("decode", 512, 8, "bf16", True, False)
    assert not attn.covers("decode", 96, 8, "int8", False, False)
    assert attn.covers("prefill", 256, 8, "int8", False, False)
    assert attn.covers("prefill", 512, 8, "int8", False, False)
    assert not attn.covers("prefill", 96, 8, "int8", False, False)
    impl = attn.impl_class()
    assert impl.__name__ == "StrixTritonAttentionImpl" and issubclass(attn.backend_class(), object)


def test_fp8_linear_gates():
    from strix_vllm import fp8

    block, chan = fp8.block_kernel_class(), fp8.channel_kernel_class()
    assert block.apply_input_quant is False
    assert block.is_supported()[0] is False or torch.cuda.is_available()
    assert chan.__name__ == "StrixFp8ChannelMMKernel"


def test_dense_w8_quantiser_and_switches(monkeypatch):
    from strix_vllm import dense_w8

    g = torch.Generator().manual_seed(0)
    w = (torch.randn(64, 256, generator=g) * 0.05).bfloat16()
    q, s, group = dense_w8.quantize(w)
    assert q.dtype == torch.uint8 and q.shape == w.shape and group == 128 and s.shape == (64, 2)
    deq = (q.float() - 128) * s.float().repeat_interleave(128, 1)
    assert float((deq - w.float()).abs().max()) <= float(s.float().max()) * 0.51 + 1e-6
    q2, s2, g2 = dense_w8.quantize(w[:, :200].contiguous())      # K % 128 != 0: per channel
    assert g2 == 0 and s2.shape == (64,)
    assert not dense_w8.enabled()
    monkeypatch.setenv("STRIX_ENABLE", "dense_w8")
    assert dense_w8.enabled()
    monkeypatch.setenv("STRIX_DISABLE", "dense_w8")
    assert not dense_w8.enabled()
    x = torch.randn(3, 256).bfloat16()                            # no copy registered: plain bf16
    torch.testing.assert_close(dense_w8.apply(x, w), torch.nn.functional.linear(x, w))


# ------------------------------------------------------------------ on the GPU
@pytest.mark.gpu
def test_dense_w8_copy_serves_small_batches():
    from strix_vllm import dense_w8

    w = (torch.randn(512, 1024, generator=torch.Generator().manual_seed(1)) * 0.05).bfloat16().cuda()
    assert dense_w8.add_copy(w) and dense_w8.lookup(w) is not None
    bias = torch.randn(512, device="cuda").bfloat16()
    for m in (1, 8, 9):
        x = torch.randn(2, m, 1024, device="cuda").bfloat16()[0]
        out = dense_w8.apply(x, w, bias).float()
        ref = torch.nn.functional.linear(x, w, bias).float()
        torch.testing.assert_close(out / ref.abs().amax(), ref / ref.abs().amax(), rtol=0, atol=3e-2)
        assert m > 8 or not torch.equal(out, ref)                # the int8 copy really ran


@pytest.mark.gpu
@pytest.mark.parametrize("m", [6, 64, 300])
def test_int8_kernel_matches_the_oracle(m):
    from oracle import gemm as G

    n, k = 1024, 2048
    kernel = int8_kernel()
    layer = mock_int8_layer(n, k, device="cuda", seed=m)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).bfloat16()
    bias = torch.randn(n, generator=torch.Generator().manual_seed(1)).bfloat16()
    kernel.process_weights_after_loading(layer)
    out = kernel.apply_weights(layer, x.cuda(), None)
    with_bias = kernel.apply_weights(layer, x.cuda().view(1, m, k), bias.cuda())
    # oracle: vLLM's dynamic per-token rule, then the exact integer product
    amax = x.float().abs().amax(-1, keepdim=True)
    s = torch.where(amax > 0, amax / 127, torch.ones_like(amax))
    q = torch.clamp(torch.round(x.float() / s), -127, 127).to(torch.int8)
    ref, _ = G.w8a8_int8_gemm(q, s.reshape(-1), layer.weight.data.cpu(), layer.weight_scale.data.cpu())
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    torch.testing.assert_close(with_bias.view(m, n).float().cpu(), (ref + bias).float(), rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_fp8_apply_matches_the_oracle():
    from oracle import gemm as G
    from strix_vllm import fp8

    g = torch.Generator().manual_seed(0)
    n, k = 384, 512
    w = (torch.randn(n, k, generator=g) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    bs = torch.rand(3, 4, generator=g) * 0.02 + 0.005
    for m in (3, 40):
        x = torch.randn(m, k, generator=g).bfloat16()
        out = fp8.apply_fp8(x.cuda(), w.cuda(), bs.cuda(), None).float().cpu()
        ref = x.float() @ G.fp8_dequant(w, bs).bfloat16().float().t()
        torch.testing.assert_close(out / ref.abs().amax(), ref / ref.abs().amax(), rtol=0, atol=1e-2)


@pytest.mark.gpu
def test_moe_experts_entry_matches_the_oracle_layer():
    from libstrix_b200 import moe as smoe
    from libstrix_b200.workloads import moe_fp8_layer
    from oracle import moe as M

    layer = moe_fp8_layer(tokens=70, hidden=512, experts=8, top_k=2, inter=256, seed=4, device="cuda")
    cpu = layer.to("cpu")
    ref, ids, wts = M.moe_fp8_layer(cpu.x, cpu.logits, cpu.w13, cpu.w13_scale, cpu.w2, cpu.w2_scale, 2)
    out = torch.full((70, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    # routing decided outside (here: the oracle's), int64 ids as vLLM hands them over
    smoe.experts_fp8_w8a8(layer.x, wts.cuda(), ids.long().cuda(), layer.w13, layer.w13_scale, layer.w2,
                          layer.w2_scale, out=out)
    err = (out.float().cpu() - ref.float()).abs()
    rms = ref.float().pow(2).mean().sqrt()
    assert bool((err <= 2e-2 * rms + ref.float().abs() * 2.0 ** -8).all())


@pytest.mark.gpu
def test_attention_impl_routes_decode_and_prefill_to_strix():
    """forward() and do_kv_cache_update() of the impl class on vLLM 0.22's packed
    int8 cache, driven with a stand-in for `self` and for the metadata."""
    import libstrix_b200 as strix
    from oracle import attention as A
    from strix_vllm import attn

    impl = attn.impl_class()
    hq, hkv, d, bs = 16, 4, 128, 16
    ctx = [70, 300, 5]
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([1] * 3, ctx, hq, hkv, bs, seed=1, hd=d)
    blocks = kc.size(0)
    cache = torch.zeros(blocks, 2, bs, hkv, d + 4, dtype=torch.int8, device="cuda")
    me = types.SimpleNamespace(
        _strix={(k, t): True for k in ("decode", "prefill") for t in ("bf16", "int8")},
        head_size=d, num_heads=hq, num_kv_heads=hkv, scale=d ** -0.5, _window_left=-1, sinks=None)
    slots = torch.arange(blocks * bs, device="cuda")
    impl.do_kv_cache_update(me, None, kc.reshape(-1, hkv, d).contiguous().cuda(),
                            vc.reshape(-1, hkv, d).contiguous().cuda(), cache, slots)
    gk, gv, gks, gvs = strix.packed_int8_kv_views(cache)
    kq, ks = A.quantize_kv_vllm(kc)
    vq, vs = A.quantize_kv_vllm(vc)
    assert torch.equal(gk.cpu(), kq) and torch.equal(gvs.cpu(), vs)
    md = types.SimpleNamespace(max_query_len=1, num_actual_tokens=3, seq_lens=seq_lens.cuda(),
                               block_table=table.cuda(), query_start_loc=cu.cuda(), use_cascade=False,
                               mm_prefix_range_tensor=None)
    out = torch.zeros(3, hq * d, dtype=torch.bfloat16, device="cuda")
    impl.forward(me, None, q.cuda().view(3, hq * d), None, None, cache, md, out)
    ref = A.decode_reference(q, kq, vq, ks, vs, seq_lens, table, d ** -0.5)
    err = (out.view(3, hq, d).float().cpu() - ref).abs()
    rms = ref.pow(2).mean().sqrt()
    assert bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all())
