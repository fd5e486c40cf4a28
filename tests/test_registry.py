"""Kernel table behaviour: same contract as the reference's tests/test_registry.py
(first-match priority, reason strings, geometry sets, table <-> registered ops)."""

import torch

import libstrix_b200 as strix
from libstrix_b200 import registry, torch_ops

DECODE = dict(head_dim=128, gqa=8, queries=1, dtype=torch.bfloat16, kv_dtype=torch.int8,
              window=False, sinks=False)


def test_every_registered_op_has_a_row_and_back():
    table = {k["name"] for k in strix.kernels()}
    assert table == set(torch_ops.registered_ops())


def test_select_hits_and_misses():
    assert strix.select("attn_decode", **DECODE) == "attn_decode_bf16"
    assert strix.select("attn_decode", **{**DECODE, "head_dim": 512}) == "attn_decode_bf16"
    assert strix.select("attn_decode", **{**DECODE, "head_dim": 96}) is None
    assert strix.select("attn_decode", **{**DECODE, "kv_dtype": "fp8_e4m3"}) is None
    assert strix.select("no_such_op", x=1) is None


def test_missing_key_is_a_miss_with_a_reason():
    geo = {k: v for k, v in DECODE.items() if k != "gqa"}
    assert strix.select("attn_decode", **geo) is None
    reasons = [r["reason"] for r in strix.explain("attn_decode", **geo)]
    assert reasons[0] == "gqa not given" and "gqa not given" not in reasons[-1]


def test_reason_strings():
    rows = strix.explain("attn_decode", **{**DECODE, "kv_dtype": torch.bfloat16})
    assert rows[0]["reason"] == "kv_dtype=bf16, needs in ('int8',)"
    rows = strix.explain("attn_decode", **{**DECODE, "head_dim": 64})
    assert rows[0]["reason"] == "head_dim=64, needs == 128"


def test_dtype_spellings_normalise():
    assert strix.select("attn_decode", **{**DECODE, "dtype": "torch.bfloat16"}) == "attn_decode_bf16"
    assert strix.select("attn_decode", **{**DECODE, "dtype": "bf16"}) == "attn_decode_bf16"


def test_geometries_are_the_scalar_points():
    pts = strix.geometries("attn_decode", "head_dim", "gqa")
    assert (128, 8) in pts and (256, 2) in pts and (512, 8) not in pts
    assert strix.geometries("attn_decode", "head_dim", "gqa", kv_dtype="bf16") == set()
    assert strix.geometries("attn_decode", "kv_dtype") == set()  # a set, not a point


def test_range_semantics():
    r = registry.Range(lo=6)
    assert r.covers(6) and not r.covers(5) and not r.covers(True) and not r.covers(6.0)
    assert str(registry.Range(2, 5)) == "in 2..5" and str(registry.Range(hi=5)) == "<= 5"
    k = registry.Kernel("k", "o", "", {"rows": registry.Range(hi=5)})
    assert k.check({"rows": 5}) is None and k.check({"rows": 6}) == "rows=6, needs <= 5"


def test_selections_are_recorded():
    before = {(s["op"], tuple(sorted(s["query"].items()))): s["count"] for s in strix.selections()}
    strix.select("attn_decode", **DECODE)
    strix.select("attn_decode", **DECODE)
    recs = [s for s in strix.selections() if s["op"] == "attn_decode" and s["kernel"]
            and s["query"].get("head_dim") == 128 and s["query"].get("gqa") == 8
            and s["query"].get("dtype") == "bf16" and s["query"].get("sinks") is False]
    assert recs and recs[0]["count"] >= 2
    miss = strix.select("attn_decode", **{**DECODE, "head_dim": 96})
    assert miss is None
    rec = [s for s in strix.selections() if s["query"].get("head_dim") == 96][0]
    assert rec["kernel"] is None and "head_dim=96" in rec["reason"]


def test_every_head_size_of_the_reference_table_is_covered():
    """(head_dim, gqa, kv_dtype) of the reference's attention rows
    (python/strix/registry.py:368-560): each selects a kernel here."""
    prefill = [(256, 6), (256, 8), (256, 2), (512, 8), (64, 4), (128, 8)]
    decode = [(256, 2), (512, 8), (256, 8), (128, 8)]
    for hd, gqa in prefill:
        for kv in ("bf16", "int8"):
            assert strix.select("attn_prefill", head_dim=hd, gqa=gqa, dtype="bf16", kv_dtype=kv,
                                split_kv=False, window=True, causal=True, sinks=False) \
                == "attn_prefill_bf16", (hd, gqa, kv)
    for hd, gqa in decode:
        for kv in ("bf16", "int8"):
            assert strix.select("attn_decode", head_dim=hd, gqa=gqa, queries=1, dtype="bf16",
                                kv_dtype=kv, window=False, sinks=False) == "attn_decode_bf16", (hd, gqa, kv)


def test_tile_sweep_ops_take_a_bounded_cfg():
    import pytest

    assert [torch_ops._cfg_block_m(i) for i in range(len(torch_ops.TILE_CFGS))] == list(torch_ops.TILE_CFGS)
    for bad in (-1, len(torch_ops.TILE_CFGS)):
        with pytest.raises(RuntimeError, match="cfg must be in"):
            torch_ops._cfg_block_m(bad)
    sweeps = {"fp8_wmma_gemm_cfg": "fp8_tile_sweep", "fp8_wmma_gemm_raw_cfg": "fp8_tile_sweep",
              "w8a8_wmma_gemm_cfg": "w8a8_tile_sweep", "mxfp4_wmma_gemm_cfg": "mxfp4_tile_sweep"}
    rows = {k["name"]: k["op"] for k in strix.kernels()}
    for name, op in sweeps.items():
        assert name in torch_ops.registered_ops() and rows[name] == op
