"""Pins oracle/ against golden vectors produced by the reference's own in-test
reference functions (tests/golden/make_golden.py)."""

from pathlib import Path

import torch

from oracle import attention as A

GOLDEN = Path(__file__).parent / "golden"


def test_attention_oracle_matches_reference_outputs():
    cases = torch.load(GOLDEN / "attn_decode.pt")
    assert len(cases) >= 4
    for c in cases:
        out = A.decode_reference(
            c["q"], c["key_cache"], c["value_cache"], c["k_scale"], c["v_scale"],
            c["seq_lens"], c["block_table"], c["scale"], c["window_left"], c["sinks"])
        torch.testing.assert_close(out, c["out"], rtol=0, atol=0)


def test_quantize_kv_properties():
    torch.manual_seed(1)
    x = torch.randn(3, 16, 2, 64).bfloat16()
    x[0, 0, 0] = 0  # all-zero row: scale clamps to 1e-8 / 127, bytes are 0
    q, s = A.quantize_kv(x)
    assert q.dtype == torch.int8 and s.shape == (3, 16, 2)
    assert int(q.abs().max()) == 127 and int(q[0, 0, 0].abs().max()) == 0
    err = (q.float() * s[..., None] - x.float()).abs()
    assert bool((err <= s[..., None] * 0.5 + 1e-6).all())


def test_build_paged_kv_tables_are_a_permutation():
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([1, 1], [40, 5], 8, 2, 16, hd=64)
    used = torch.cat([table[0, :3], table[1, :1]]).tolist()
    assert len(set(used)) == len(used) and max(used) < kc.size(0)
    assert kc.shape == (kc.size(0), 16, 2, 64) and kc.stride(-1) == 1


def test_moe_oracle_matches_reference_outputs():
    from oracle import moe as M

    gold = torch.load(GOLDEN / "moe.pt")
    for c in gold["align"]:
        s, x, n = M.align(c["topk_ids"], c["block_m"], c["experts"])
        assert torch.equal(s, c["sorted_ids"]) and torch.equal(x, c["expert_ids"])
        assert torch.equal(n, c["num_post"])
    for c in gold["grouped"]:
        out = M.grouped_reference(c["a"], c["b"], c["topk_ids"], c["top_k"], c["weights"])
        torch.testing.assert_close(out, c["out"], rtol=0, atol=0)
        out = M.grouped_reference(c["a"], c["b"], c["topk_ids"], c["top_k"])
        torch.testing.assert_close(out, c["out_unweighted"], rtol=0, atol=0)
    for c in gold["fp8"]:
        w, scales, deq = M.make_fp8_weights(2, 256, 128, c["scheme"], keep_fp32=c["kind"] == "raw")
        assert torch.equal(w.view(torch.uint8), c["w"]) and torch.equal(scales, c["scales"])
        assert torch.equal(deq, c["deq"])
        h = M.grouped_reference(c["a"], deq, c["topk_ids"], 2)
        torch.testing.assert_close(h, c["h"], rtol=0, atol=0)
        torch.testing.assert_close(M.gate_mul(h, "silu"), c["silu"], rtol=0, atol=0)
        torch.testing.assert_close(M.gate_mul(h, "gelu_tanh"), c["gelu"], rtol=0, atol=0)


def test_act_quant_oracles():
    from oracle import moe as M

    torch.manual_seed(0)
    x = (torch.randn(37, 640) * 3).bfloat16()
    x[5, 128:256] = 0
    q, s = M.act_quant_i8(x)
    assert float(s[5, 1]) == 1.0 and int(q[5, 128:256].abs().max()) == 0
    assert int(q.abs().max()) == 127
    assert bool(((M.dequant_act(q, s) - x.float()).abs() <= s.repeat_interleave(128, -1) * 0.5 + 1e-6).all())
    q8, s8 = M.act_quant_fp8(x)
    assert q8.dtype == torch.float8_e4m3fn and float(s8[5, 1]) == 1.0
    assert float(q8.float().abs().max()) == 448.0
    rel = (M.dequant_act(q8, s8) - x.float()).abs() / x.float().abs().clamp_min(1e-3)
    assert float(rel.max()) <= 2 ** -4 + 1e-6      # e4m3: 3 mantissa bits


def test_router_oracle_properties():
    from oracle import moe as M

    torch.manual_seed(0)
    logits = torch.randn(64, 128)
    ids, w = M.router(logits, 8)
    assert ids.dtype == torch.int32 and ids.shape == (64, 8)
    torch.testing.assert_close(w.sum(-1), torch.ones(64))
    # the chosen experts are the 8 largest logits of each row, in descending order
    want = torch.sort(logits, dim=-1, descending=True).indices[:, :8]
    assert torch.equal(ids.long(), want)


def test_gemm_oracle_matches_reference_outputs():
    """oracle/gemm.py and the activation quantiser against vectors produced by the
    reference's own in-test functions (tests/golden/make_golden.py::golden_gemm)."""
    from oracle import gemm as G
    from oracle import moe as M

    gold = torch.load(GOLDEN / "gemm.pt")
    c = gold["mxfp4"]
    assert tuple(c["lut"].tolist()) == G.MX_VALUES
    assert torch.equal(G.mxfp4_dequant(c["w"], c["s"]), c["deq"])
    for c in gold["int4"]:
        assert torch.equal(G.int4_pack(c["q"]), c["packed"])
        # groups that are a multiple of 64 are judged against the exact fp32 weights
        # (tests/test_moe_wna16.py:52-62), the others against their bf16 rounding
        deq = G.int4_dequant(c["packed"], c["scales"], c["group"], exact=c["group"] % 64 == 0)
        assert deq.dtype == c["deq"].dtype and torch.equal(deq, c["deq"])
    for c in gold["w8a16"]:
        out = G.w8a16_reference(c["x"], c["w"], c["scales"], c["group"])
        torch.testing.assert_close(out, c["out"], rtol=0, atol=0)
    c = gold["w8a8_group"]
    torch.testing.assert_close(G.w8a8_group_reference(c["x"], c["w"], c["scale"]), c["out"],
                               rtol=0, atol=0)
    c = gold["fp8_block"]
    w = c["w"].view(torch.float8_e4m3fn)
    assert torch.equal(G.fp8_dequant(w, c["scales"]), c["deq"])
    c = gold["act_quant_i8"]
    q, s = M.act_quant_i8(c["x"])
    assert torch.equal(q, c["q"]) and torch.equal(s, c["sa"])
    # the dense op's in-kernel quantiser follows the same rule
    q2, s2 = G.act_quant_group_i8(c["x"])
    assert torch.equal(s2, c["sa"]) and int((q2.int() - c["q"].int()).abs().max()) <= 1
