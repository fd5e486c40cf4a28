"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad geometry before touching the device."""

import ctypes

import pytest

from libstrix_b200 import _lib


def test_library_exports_every_declared_symbol():
    protos = _lib.parse_header()
    assert "strix_attn_decode_bf16" in protos and len(protos) >= 5
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in protos:
        assert hasattr(lib, name), name


def test_version_and_error_string():
    lib = _lib.load()
    assert lib.strix_version() >= 1000
    assert isinstance(lib.strix_last_error(), bytes)


def test_decode_segments_and_workspace():
    lib = _lib.load()
    assert lib.strix_attn_decode_segments(4, 10, 16) == 4
    assert lib.strix_attn_decode_segments(0, 4096, 16) == 64
    assert lib.strix_attn_decode_segments(0, 0, 16) == 1
    assert lib.strix_attn_decode_segments(65, 1, 16) == -1
    # a batch below one wave of 1024-key segments gets 512-key segments
    assert lib.strix_attn_decode_segments_n(64, 0, 4096, 16) == 64
    assert lib.strix_attn_decode_segments_n(16, 0, 4096, 16) == 64
    assert lib.strix_attn_decode_segments_n(8, 0, 4096, 16) == 128
    assert lib.strix_attn_decode_segments_n(8, 4, 4096, 16) == 4
    assert lib.strix_attn_decode_workspace(8, 32, 128, 0, 4096, 16) == 8 * 32 * 128 * 130 * 4
    assert lib.strix_attn_decode_workspace(3, 32, 128, 1, 10, 16) == 0
    assert lib.strix_attn_decode_workspace(3, 32, 128, 4, 10, 16) == 3 * 32 * 4 * 130 * 4


def _decode_args(**over):
    a = dict(out=8, q=8, kc=16, vc=16, ks=4, vs=4, sl=4, bt=4, sinks=None, ws=None,
             nseq=1, hq=32, hkv=4, d=128, bs=16, max_blocks=4, bt_stride=4,
             q_st=4096, q_sh=128, o_st=4096, o_sh=128,
             k_sb=8192, k_ss=512, k_sh=128, v_sb=8192, v_ss=512, v_sh=128,
             ks_sb=64, ks_ss=4, ks_sh=1, vs_sb=64, vs_ss=4, vs_sh=1,
             scale=0.1, splits=1, win=-1, q8=1, stream=None)
    a.update(over)
    return list(a.values())


@pytest.mark.parametrize(
    "over,fragment",
    [
        (dict(d=64), "not built"),
        (dict(hq=30), "Hq % Hkv"),
        (dict(bs=24), "multiple of 16"),
        (dict(splits=65), "num_splits in [1, 64]"),
        (dict(q8=0, d=96), "bf16 KV: head_dim 96 GQA 8 not built"),
        (dict(q8=0, k_ss=516), "bf16 cache rows must be 16-byte aligned"),
        (dict(ks=None), "int8 KV needs k_scale and v_scale"),
        (dict(splits=4), "workspace"),
        (dict(k_ss=510), "aligned cache rows"),
    ],
)
def test_decode_rejects_bad_arguments_without_a_gpu(over, fragment):
    with pytest.raises(_lib.StrixError, match=fragment.replace("[", r"\[").replace("]", r"\]")):
        _lib.call("strix_attn_decode_bf16", *_decode_args(**over))


def test_sorted_layout_gives_way_to_gather_above_the_m_block_limit():
    """Needs no GPU: the padded list's capacity is host arithmetic. 2048 m-blocks of
    128 rows hold the benchmark layer's 4096 x 8 slots with room to spare; a batch
    whose padded list needs more blocks than one launch walks takes the gather
    layout instead of failing."""
    from libstrix_b200 import moe

    lib = _lib.load()
    assert moe.fits_sorted_grid(4096 * 8, 128, 128)
    assert moe.fits_sorted_grid(1, 128, 16)
    # capacity = slots + experts * (block_m - 1) rounded up to whole blocks
    cap = lib.strix_moe_align_capacity(4096 * 8, 128, 128)
    assert cap % 128 == 0 and cap >= 4096 * 8 + 128 * 127
    limit = moe.MAX_SORTED_M_BLOCKS * 128
    slots_at_limit = limit - 128 * 127
    assert moe.fits_sorted_grid(slots_at_limit, 128, 128)
    assert not moe.fits_sorted_grid(slots_at_limit + 1, 128, 128)
    assert not moe.fits_sorted_grid(1 << 20, 128, 16)
