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
