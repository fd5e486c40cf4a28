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


GENERATORS = {"attn_decode": golden_attn_decode, "moe": golden_moe}

if __name__ == "__main__":
    wanted = sys.argv[1:] or list(GENERATORS)
    for name in wanted:
        GENERATORS[name]()
        f = OUT / f"{name}.pt"
        print(f"{name}: {f.stat().st_size / 1024:.0f} KiB")
