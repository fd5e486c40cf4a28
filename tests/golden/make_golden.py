"""Generates the golden vectors under tests/golden/ from the reference's own tests.

Run once, in a container that has the asf0/libstrix tree, with its location in
$STRIX_REFERENCE:

    STRIX_REFERENCE=<path to the asf0/libstrix checkout> python tests/golden/make_golden.py

The reference's kernel tests carry their torch reference implementations
in-file (tests/test_attn_prefill.py: build/quantize/reference, ...). Those test
modules `import strix` (the HIP extension, which cannot load here) and create
tensors on "cuda"; this script loads each module's source with a stub `strix`
module and the device string replaced by "cpu", calls the reference's OWN
helper functions on small seeded inputs, and stores inputs and outputs. No
reference source is copied into this repository: only tensors are written.
tests/test_oracle_golden.py then pins oracle/ against these files.
"""

from __future__ import annotations

import os
import sys
import types
from pathlib import Path

import torch

if "STRIX_REFERENCE" not in os.environ:
    raise SystemExit("set STRIX_REFERENCE to the asf0/libstrix checkout")
REF = Path(os.environ["STRIX_REFERENCE"])
OUT = Path(__file__).resolve().parent


def load_reference_test(name: str) -> types.ModuleType:
    """Executes tests/<name>.py of the reference on the CPU with a stub `strix`."""
    stub = types.ModuleType("strix")
    stub.is_supported_device = lambda: False
    sys.modules.setdefault("strix", stub)
    src = (REF / "tests" / f"{name}.py").read_text()
    src = src.replace('"cuda"', '"cpu"').replace("'cuda'", "'cpu'")
    mod = types.ModuleType(f"ref_{name}")
    mod.__file__ = str(REF / "tests" / f"{name}.py")
    exec(compile(src, mod.__file__, "exec"), mod.__dict__)
    return mod


def golden_attn_decode() -> None:
    """Decode cases of test_h128_g8_decode_sinks / test_decode_int8_matches_reference
    (tests/test_attn_prefill.py:167-195, 283-312) evaluated by the reference's
    build(), quantize() and reference()."""
    ref = load_reference_test("test_attn_prefill")
    cases = []
    specs = [
        # hq, hkv, hd, ctx_lens, block_size, window_left, sinks
        (32, 4, 128, [70, 200, 3], 16, -1, False),
        (32, 4, 128, [300, 31, 450, 64], 16, 40, True),
        (32, 4, 128, [0], 16, -1, True),
        (8, 1, 128, [70, 290, 3], 272, 31, False),
        (4, 2, 256, [33, 90], 16, -1, False),
    ]
    for hq, hkv, hd, ctx, bs, win, use_sinks in specs:
        q_lens = [1] * len(ctx)
        q, kc, vc, cu, seq_lens, table = ref.build(q_lens, ctx, hq, hkv, bs, hd=hd)
        kq, ks = ref.quantize(kc, bs, hkv)
        vq, vs = ref.quantize(vc, bs, hkv)
        sinks = (torch.randn(hq) * 2).float() if use_sinks else None
        scale = hd ** -0.5
        out = ref.reference(q, kq.float() * ks[..., None], vq.float() * vs[..., None],
                            cu, seq_lens, table, scale, win, sinks)
        cases.append({
            "hq": hq, "hkv": hkv, "hd": hd, "block_size": bs, "window_left": win,
            "scale": scale, "q": q, "key_cache": kq.contiguous(), "value_cache": vq.contiguous(),
            "k_scale": ks, "v_scale": vs, "cu": cu.int(), "seq_lens": seq_lens.int(),
            "block_table": table, "sinks": sinks, "out": out,
        })
    torch.save(cases, OUT / "attn_decode.pt")


def golden_moe() -> None:
    """align() and reference() of tests/test_moe_gemm.py:9-42, make_weights() of
    tests/test_moe_fp8.py:17-29 and tests/test_moe_fp8_raw.py:17-28 (with the
    module constant E shrunk so the fixture stays small), and a full
    w13 -> gate -> w2 chain evaluated by the reference's functions."""
    import torch.nn.functional as F

    ref = load_reference_test("test_moe_gemm")
    sys.modules["test_moe_w8a16"] = load_reference_test("test_moe_w8a16")
    fp8 = load_reference_test("test_moe_fp8")
    raw = load_reference_test("test_moe_fp8_raw")
    out = {"align": [], "grouped": [], "fp8": []}
    g = torch.Generator().manual_seed(0)
    for tokens, top_k, e, block_m in [(1, 2, 4, 16), (5, 3, 8, 4), (37, 4, 16, 16), (64, 8, 128, 64)]:
        ids = torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(tokens)])
        s, x, n = ref.align(ids, block_m, e)
        out["align"].append({"topk_ids": ids, "block_m": block_m, "experts": e,
                             "sorted_ids": s, "expert_ids": x, "num_post": n})
    for tokens, top_k, e, n, k in [(5, 2, 4, 64, 128), (9, 1, 3, 32, 64)]:
        ids = torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(tokens)])
        a = torch.randn(tokens * (1 if top_k > 1 else 1), k, generator=g).bfloat16()
        b = (torch.randn(e, n, k, generator=g) / k ** 0.5).bfloat16()
        wts = torch.rand(tokens, top_k, generator=g)
        a_in = a if top_k > 1 else torch.randn(tokens, k, generator=g).bfloat16()
        out["grouped"].append({"a": a_in, "b": b, "topk_ids": ids, "top_k": top_k, "weights": wts,
                               "out": ref.reference(a_in, b, ids, top_k, wts),
                               "out_unweighted": ref.reference(a_in, b, ids, top_k, None)})
    for mod, name in ((fp8, "plain"), (raw, "raw")):
        mod.E = 2
        for scheme in ("block", "channel"):
            w, scales, deq = mod.make_weights(256, 128, scheme)
            ids = torch.stack([torch.randperm(2, generator=g)[:2] for _ in range(6)])
            a = torch.randn(6, 128, generator=g).to(torch.bfloat16 if name == "plain" else torch.float16)
            h = (fp8 if name == "plain" else raw).reference(a, deq, ids, 2, None) \
                if name == "raw" else ref.reference(a, deq, ids, 2, None)
            gate, up = h[:, :128], h[:, 128:]
            out["fp8"].append({"kind": name, "scheme": scheme, "w": w.view(torch.uint8),
                               "scales": scales, "deq": deq, "a": a, "topk_ids": ids,
                               "h": h, "silu": F.silu(gate) * up,
                               "gelu": F.gelu(gate, approximate="tanh") * up})
    torch.save(out, OUT / "moe.pt")


def golden_gemm() -> None:
    """The in-test reference functions of the dense and 4-bit ops evaluated on
    seeded inputs: torch_dequant() of tests/test_mxfp4.py:28-45, pack() and
    dequant() of tests/test_moe_wna16.py:44-62, reference() of
    tests/test_w8a16.py:9-17 and of tests/test_w8a8_int8.py:50-57, ref_weight()
    of tests/test_fp8.py:17-20. The activation quantiser of
    tests/test_moe_w4a8.py:24-36 has its expectation inline in a test function;
    that function is run here with torch.ops.strix.moe_act_quant_i8 served by the
    oracle, so the stored vector is one the reference's own test accepted."""
    root = Path(__file__).resolve().parents[2]
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    from oracle import moe as M

    mx = load_reference_test("test_mxfp4")
    wna = load_reference_test("test_moe_wna16")
    sys.modules["test_moe_wna16"] = wna
    w8a16 = load_reference_test("test_w8a16")
    w8a8 = load_reference_test("test_w8a8_int8")
    fp8 = load_reference_test("test_fp8")
    w4a8 = load_reference_test("test_moe_w4a8")
    g = torch.Generator().manual_seed(0)
    out = {}

    w = torch.randint(0, 256, (48, 80), generator=g, dtype=torch.uint8)        # K = 160
    s = torch.randint(118, 134, (48, 5), generator=g, dtype=torch.uint8)
    out["mxfp4"] = {"w": w, "s": s, "deq": mx.torch_dequant(w, s),
                    "lut": torch.tensor(mx.MX_VALUES)}

    out["int4"] = []
    for group, sdt in ((32, torch.bfloat16), (64, torch.float16), (128, torch.bfloat16)):
        q = torch.randint(0, 16, (3, 24, 256), generator=g, dtype=torch.uint8)
        sc = (torch.rand(3, 24, 256 // group, generator=g) * 0.05 + 0.01).to(sdt)
        packed = wna.pack(q)
        out["int4"].append({"q": q, "packed": packed, "scales": sc, "group": group,
                            "deq": wna.dequant(packed, sc, group)})

    out["w8a16"] = []
    for group in (0, 128):
        x = torch.randn(5, 384, generator=g).bfloat16()
        wu = torch.randint(0, 256, (40, 384), generator=g, dtype=torch.uint8)
        sc = (torch.rand(40, 384 // group if group else 1, generator=g) * 0.01).bfloat16()
        if group == 0:
            sc = sc.reshape(40)
        out["w8a16"].append({"x": x, "w": wu, "scales": sc, "group": group,
                             "out": w8a16.reference(x, wu, sc, group)})

    x = torch.randn(7, 512, generator=g).bfloat16()
    x[2, 128:256] = 0
    wi = torch.randint(-127, 128, (24, 512), generator=g, dtype=torch.int8)
    sw = (torch.rand(24, 1, generator=g) * 0.01 + 1e-4).float()
    out["w8a8_group"] = {"x": x, "w": wi, "scale": sw, "out": w8a8.reference(x, wi, sw)}

    wq = (torch.randn(200, 256, generator=g) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    bs = torch.rand(2, 2, generator=g) * 0.02 + 0.005
    out["fp8_block"] = {"w": wq.view(torch.uint8), "scales": bs, "deq": fp8.ref_weight(wq, bs)}

    # the reference's own acceptance test of the activation quantiser, over the oracle
    seen = {}
    lib = torch.library.Library("strix", "DEF")
    lib.define("moe_act_quant_i8(Tensor x, Tensor(a!) q, Tensor(b!) sa) -> ()")

    def impl(x, q, sa):
        qq, ss = M.act_quant_i8(x)
        q.copy_(qq), sa.copy_(ss)
        seen.update(x=x.clone(), q=qq.clone(), sa=ss.clone())

    lib.impl("moe_act_quant_i8", impl, "CPU")
    w4a8.test_act_quant_matches_reference()          # raises if the oracle breaks the reference's rule
    out["act_quant_i8"] = dict(seen, accepted_by="tests/test_moe_w4a8.py:24-36")
    torch.save(out, OUT / "gemm.pt")


GENERATORS = {"attn_decode": golden_attn_decode, "moe": golden_moe, "gemm": golden_gemm}

if __name__ == "__main__":
    wanted = sys.argv[1:] or list(GENERATORS)
    for name in wanted:
        GENERATORS[name]()
        f = OUT / f"{name}.pt"
        print(f"{name}: {f.stat().st_size / 1024:.0f} KiB")
