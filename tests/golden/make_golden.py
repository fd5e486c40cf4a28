"""Generates the golden vectors under tests/golden/ from the reference's own tests.

Run once, in a container that has the asf0/libstrix tree (default
/root/reference, or $STRIX_REFERENCE):

    python tests/golden/make_golden.py

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

REF = Path(os.environ.get("STRIX_REFERENCE", "/root/reference"))
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


GENERATORS = {"attn_decode": golden_attn_decode}

if __name__ == "__main__":
    wanted = sys.argv[1:] or list(GENERATORS)
    for name in wanted:
        GENERATORS[name]()
        f = OUT / f"{name}.pt"
        print(f"{name}: {f.stat().st_size / 1024:.0f} KiB")
