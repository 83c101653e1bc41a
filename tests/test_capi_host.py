"""CPU-side checks of libsfq.so: it loads, exports every symbol include/sfq.h declares, its host
packers produce the reference's bytes (NVFP4) or bytes the reference's decode rules accept
(W4A8 / W6A8 / INT8), and device entry points fail loudly without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "sfq.h")).read()
    declared = set(re.findall(r"SFQ_API\s+[\w\s\*]+?\b(sfq_\w+)\s*\(", header))
    assert len(declared) >= 36
    assert declared == set(sfq.EXPORTS)
    raw = C.CDLL(sfq.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert sfq.lib.sfq_version() == 100


def test_weight_descriptor_defaults_match_reference():
    # include/slopfab/cuda/linear.cuh:80-152 defaults
    w = sfq.new_weight()
    assert (w.format, w.packed_group_size, w.global_scale, w.convrot, w.convrot_group) == (sfq.BF16, 16, 1.0, 0, 256)
    assert (w.nf4_block_size, w.nf4_nested_block_size, w.bias_format, w.input_scale) == (64, 256, sfq.F32, 0.0)


def test_pack_nvfp4_is_byte_identical_to_reference_fixture(golden):
    rng = np.random.default_rng(0)
    w = (0.02 * rng.standard_normal((256, 192))).astype(np.float32)
    w[3, 16:32] = 0.0  # a zero block
    g = float(np.abs(w).max() / (6 * 448))
    data = np.zeros((256, 96), np.uint8)
    scale = np.zeros(256 * 12, np.uint8)
    sfq.check(sfq.lib.sfq_pack_nvfp4(P(w), 256, 192, g, P(data), P(scale)))
    od, os_, _ = oracle.nvfp4_pack(w, g)
    assert np.array_equal(data, od) and np.array_equal(scale, os_)
    # and against the bytes the reference's own packer wrote for the golden weight
    gw = golden["pack_w"]
    gg = float(golden["pack_global"])
    sfq.check(sfq.lib.sfq_pack_nvfp4(P(gw), 256, 192, gg, P(data), P(scale)))
    assert np.array_equal(data.ravel(), golden["pack_data_11"]) and np.array_equal(scale, golden["pack_scale_11"])
    # shapes the tile map cannot address are refused (launch_dequant_nvfp4 refuses 200x128 and 256x96)
    for n, k in ((200, 128), (256, 96)):
        assert sfq.lib.sfq_pack_nvfp4(P(w), n, k, g, P(data), P(scale)) == sfq.ERR_INVALID_ARGUMENT
    assert b"128" in sfq.lib.sfq_last_error()


def _rotate(w):
    return oracle.convrot_dense(w.astype(np.float32))


@pytest.mark.parametrize("bits,group", [(4, 16), (6, 16), (6, 32), (6, 64)])
def test_packed_int8_encoders_obey_the_decode_contract(bits, group):
    rng = np.random.default_rng(bits * 100 + group)
    n, k = 48, 512
    w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    w[5] = 0.0  # a zero row
    packed = np.zeros((n, k * bits // 8), np.int8)
    s_rel = np.zeros(n * k // group, np.uint8)
    s_ch = np.zeros(n, np.float32)
    book = np.zeros(16, np.float32)
    if bits == 4:
        sfq.check(sfq.lib.sfq_pack_w4a8(P(w), n, k, P(packed), P(s_rel), P(s_ch), P(book)))
        assert np.array_equal(book, np.arange(16, dtype=np.float32) - 8)
        w8 = oracle.w4a8_decode(packed.view(np.uint8), s_rel, book, n, k)
    else:
        sfq.check(sfq.lib.sfq_pack_w6a8(P(w), n, k, group, P(packed), P(s_rel), P(s_ch)))
        w8 = oracle.w6a8_decode(packed.view(np.uint8), s_rel, n, k, group)
    # validate_packed_int8_weight (src/core/w4a8.cpp:127-162): scale bytes non-negative and not 0x7F,
    # channel scales finite and positive
    assert not (s_rel & 0x80).any() and not ((s_rel & 0x7F) == 0x7F).any()
    assert np.isfinite(s_ch).all() and (s_ch > 0).all()
    # decode(encode(W)) reproduces the rotated weight to quantization accuracy
    approx = w8.astype(np.float32) * s_ch[:, None]
    target = _rotate(w)
    err = np.sqrt(((approx - target) ** 2).sum() / (target ** 2).sum())
    assert err < (0.12 if bits == 4 else 0.03), err
    assert not w8[5].any()
    # deterministic
    packed2 = np.zeros_like(packed)
    s2 = np.zeros_like(s_rel)
    c2 = np.zeros_like(s_ch)
    if bits == 4:
        sfq.check(sfq.lib.sfq_pack_w4a8(P(w), n, k, P(packed2), P(s2), P(c2), P(book)))
    else:
        sfq.check(sfq.lib.sfq_pack_w6a8(P(w), n, k, group, P(packed2), P(s2), P(c2)))
    assert np.array_equal(packed, packed2) and np.array_equal(s_rel, s2) and np.array_equal(s_ch, c2)


def test_pack_int8_round_trips_through_the_reference_unpack():
    rng = np.random.default_rng(9)
    for g in (0, 4, 16, 64, 256):
        cols = 512
        w = (0.05 * rng.standard_normal((6, cols))).astype(np.float32)
        codes = np.zeros((6, cols), np.int8)
        scale = np.zeros(6, np.float32)
        sfq.check(sfq.lib.sfq_pack_int8(P(w), 6, cols, g, P(codes), P(scale)))
        out = np.empty((6, cols), np.uint16)
        oracle.lib.orc_int8_unpack_f16(P(codes), P(scale), 6, cols, max(g, 1), 0, P(out))
        back = out.view(np.float16).astype(np.float32)
        assert np.abs(back - w).max() < 2.5 * scale.max(), g  # one int8 step per element, spread by the rotation
    assert sfq.lib.sfq_pack_int8(P(w), 6, cols, 8, P(codes), P(scale)) == sfq.ERR_INVALID_ARGUMENT
    # ragged rows skip the rotation, as the third-party quantizer does (src/core/int8_weight.cpp:47-49)
    w = (0.05 * rng.standard_normal((2, 267))).astype(np.float32)
    codes = np.zeros((2, 267), np.int8)
    scale = np.zeros(2, np.float32)
    sfq.check(sfq.lib.sfq_pack_int8(P(w), 2, 267, 256, P(codes), P(scale)))
    assert np.abs(codes.astype(np.float32) * scale[:, None] - w).max() <= 0.51 * scale.max()


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful without a GPU")
def test_device_entry_points_fail_loudly_without_a_gpu():
    handle = C.c_void_p()
    assert sfq.lib.sfq_runner_create(None, C.byref(handle)) == sfq.ERR_RUNTIME
    assert b"CUDA" in sfq.lib.sfq_last_error() or b"device" in sfq.lib.sfq_last_error()
    ep = sfq.Epilogue()
    assert sfq.lib.sfq_gemm_int8(1, 1, C.byref(ep), 1, 128, 128, 256, None) != sfq.OK


def _adaln(L, C_, Ca, explicit, Sa, V, vt, at):
    total = L + C_ + Ca + Sa + V
    tags, idx, ada = (np.zeros(total, np.int32) for _ in range(3))
    uniq = np.zeros(2, np.float32)
    n = C.c_int(0)
    sfq.check(sfq.lib.sfq_build_adaln_index(L, C_, Ca, explicit, Sa, V, vt, at, P(tags), P(idx), P(ada), P(uniq), C.byref(n)))
    return tags, idx, ada, uniq[:n.value]


def test_adaln_index_known_answers():
    # packing_row_timesteps (tests/test_packing.cpp:416-466) on the reference t2va layout: 4 text rows,
    # no conditioning, audio rows then video rows
    L, Sa, V = 4, 500, 2000
    audio_start, video_start = L, L + Sa
    tags, idx, ada, uniq = _adaln(L, 0, 0, 0, Sa, V, 0.25, 0.75)
    assert list(uniq) == [0.25, 0.75]
    assert (idx[0], idx[audio_start], idx[video_start]) == (0, 1, 0)
    assert (ada[0], ada[audio_start], ada[video_start]) == (0 * 3 + 1, 1 * 3 + 2, 0 * 3 + 0)
    tags, idx, ada, uniq = _adaln(L, 0, 0, 0, Sa, V, 0.75, 0.25)   # schedules crossed: index 0 flips
    assert uniq[0] == np.float32(0.25) and idx[0] == 1 and idx[audio_start] == 0
    assert (ada[0], ada[audio_start]) == (1 * 3 + 1, 0 * 3 + 2)
    tags, idx, ada, uniq = _adaln(L, 0, 0, 0, Sa, V, 0.5, 0.5)     # equal timesteps collapse
    assert len(uniq) == 1 and (ada[0], ada[audio_start], ada[video_start]) == (1, 2, 0)
    tags, idx, ada, uniq = _adaln(L, 0, 0, 0, Sa, V, 0.9, 0.1)
    assert ada.min() >= 0 and ada.max() < 6
    # against numpy's unique over the per-row timestep vector, several layouts incl. conditioning prefixes
    rng = np.random.default_rng(3)
    for L, C_, Ca, explicit, Sa, V in ((3, 0, 0, 0, 10, 7), (5, 6, 0, 0, 12, 9), (2, 4, 3, 1, 8, 5), (0, 0, 0, 0, 0, 11),
                                       (1, 0, 0, 0, 6, 0), (2, 9, 0, 0, 4, 3)):
        for vt, at in ((0.3, 0.6), (0.6, 0.3), (0.4, 0.4)):
            tags, idx, ada, uniq = _adaln(L, C_, Ca, explicit, Sa, V, vt, at)
            a0 = L + C_ + Ca
            row_t = np.full(a0 + Sa + V, vt, np.float32)
            prefix = min(Ca if explicit else C_, Sa)
            row_t[a0 + prefix:a0 + Sa] = at
            want_u, want_i = np.unique(row_t, return_inverse=True)
            want_tag = np.ones_like(idx)
            want_tag[L:a0] = 0
            want_tag[a0:a0 + Sa] = 2
            want_tag[a0 + Sa:] = 0
            assert np.array_equal(uniq, want_u) and np.array_equal(idx, want_i) and np.array_equal(tags, want_tag)
            assert np.array_equal(ada, want_i * 3 + want_tag)


def test_token_packing_matches_the_reference_packing_code(golden):
    """build_indices and both forms of build_row_timesteps against vectors written by the reference's own
    src/dit/packing.cpp (tests/golden/make_golden.py), padding tags (-1) and the four-timestep form included."""
    layouts, times = golden["packing_layouts"], golden["packing_times"]
    for li, lay in enumerate(layouts):
        L, Cv, Ca, ex, Sa, V = (int(v) for v in lay)
        total = L + Cv + Ca + Sa + V
        layout = sfq.SequenceLayout(L, Cv, Ca, ex, Sa, V)
        text, audio, video, tags = (np.full(n, -7, np.int32) for n in (L, Sa, Cv + Ca + V, total))
        sfq.check(sfq.lib.sfq_build_indices(C.byref(layout), P(text), P(audio), P(video), P(tags)))
        for name, got in (("text", text), ("audio", audio), ("video", video), ("tags", tags)):
            assert np.array_equal(got, golden[f"packing_{li}_{name}"]), (li, name)
        padded = np.ascontiguousarray(golden[f"packing_{li}_padded_tags"])
        for ti, tt in enumerate(times):
            for count in (2, 4):
                for pad, use in (("own", None), ("pad", padded)):
                    idx, ada = np.full(total, -7, np.int32), np.full(total, -7, np.int32)
                    uniq = np.zeros(4, np.float32)
                    n = C.c_int(0)
                    tp = None if use is None else P(use)
                    if count == 2:
                        sfq.check(sfq.lib.sfq_build_row_timesteps(C.byref(layout), tp, tt[0], tt[1], P(idx), P(ada), P(uniq), 4,
                                                                  C.byref(n)))
                    else:
                        sfq.check(sfq.lib.sfq_build_row_timesteps4(C.byref(layout), tp, tt[0], tt[1], tt[2], tt[3], P(idx), P(ada),
                                                                   P(uniq), 4, C.byref(n)))
                    key = f"packing_{li}_{ti}_{count}_{pad}"
                    assert np.array_equal(idx, golden[key + "_indices"]), key
                    assert np.array_equal(ada, golden[key + "_adaln"]), key
                    assert np.array_equal(uniq[:n.value], golden[key + "_unique"]), key
                    assert ada.min(initial=0) >= 0  # padding rows never index backwards into the table
    bad = sfq.SequenceLayout(-1, 0, 0, 0, 0, 0)
    assert sfq.lib.sfq_build_indices(C.byref(bad), None, None, None, None) == sfq.ERR_INVALID_ARGUMENT


def test_weight_row_block_views_follow_build_block():
    # build_block (src/dit/transformer_load.cpp:660-737): q/k/v are views over one [3 * inner, hidden] upload, and every
    # row-indexed array moves with the view. Pointers are opaque here: use small integers as "addresses".
    inner, hidden = 256, 512
    third = inner * hidden

    def block(w, i):
        out = sfq.QuantWeight()
        rc = sfq.lib.sfq_weight_row_block(C.byref(w), 3, i, C.byref(out))
        return rc, out

    base = dict(data=1 << 20, out_features=3 * inner, in_features=hidden)
    # NVFP4: data by K/2 bytes per row, block scales by K/16 bytes per row (both arrays sliced)
    w = sfq.new_weight(format=sfq.NVFP4, block_scale=2 << 20, global_scale=0.5, **base)
    for i in range(3):
        rc, v = block(w, i)
        assert rc == 0 and v.out_features == inner and v.in_features == hidden and v.global_scale == 0.5
        assert v.data == (1 << 20) + i * third // 2 and v.block_scale == (2 << 20) + i * third // 16
    # ... and refused when a third does not fall on a 128-row scale tile boundary
    bad = sfq.new_weight(format=sfq.NVFP4, block_scale=2 << 20, data=1 << 20, out_features=3 * 192, in_features=hidden)
    assert block(bad, 1)[0] == sfq.ERR_INVALID_ARGUMENT
    # W4A8 / W6A8: packed bytes, group scales [N, K/g], channel scales [N]
    for fmt, bits, group in ((sfq.W4A8, 4, 16), (sfq.W6A8, 6, 64)):
        w = sfq.new_weight(format=fmt, block_scale=2 << 20, weight_scale=3 << 20, w4_codebook=4 << 20 if bits == 4 else None,
                           packed_group_size=group, convrot=1, convrot_group=256, **base)
        rc, v = block(w, 2)
        assert rc == 0
        assert v.data == (1 << 20) + 2 * third * bits // 8
        assert v.block_scale == (2 << 20) + 2 * third // group
        assert v.weight_scale == (3 << 20) + 2 * inner * 4
        assert v.w4_codebook == w.w4_codebook and v.packed_group_size == group
    # NF4: data, absmax and nested absmax; refused when a third is not a whole number of nested blocks
    w = sfq.new_weight(format=sfq.NF4, nf4_absmax=2 << 20, nf4_nested_absmax=3 << 20, nf4_block_size=64,
                       nf4_nested_block_size=256, **base)
    rc, v = block(w, 1)
    assert rc == 0 and v.data == (1 << 20) + third // 2 and v.nf4_absmax == (2 << 20) + third // 64
    assert v.nf4_nested_absmax == (3 << 20) + (third // 64 // 256) * 4
    w.nf4_nested_block_size = 1024 * 1024
    assert block(w, 1)[0] == sfq.ERR_INVALID_ARGUMENT
    # dense formats: element width; the scale moves only when it is per channel
    for fmt, width in ((sfq.BF16, 2), (sfq.F32, 4), (sfq.F8E4M3, 1), (sfq.I8, 1)):
        w = sfq.new_weight(format=fmt, weight_scale=3 << 20, per_channel_scale=1 if fmt == sfq.I8 else 0, bias=5 << 20,
                           bias_format=sfq.F32, **base)
        rc, v = block(w, 1)
        assert rc == 0 and v.data == (1 << 20) + third * width
        assert v.weight_scale == (3 << 20) + (inner * 4 if fmt == sfq.I8 else 0)
        assert v.bias == (5 << 20) + inner * 4
    # argument checks
    assert block(sfq.new_weight(format=sfq.BF16, data=1, out_features=10, in_features=4), 0)[0] == sfq.ERR_INVALID_ARGUMENT  # 10 % 3
    assert sfq.lib.sfq_weight_row_block(C.byref(w), 3, 3, C.byref(sfq.QuantWeight())) == sfq.ERR_INVALID_ARGUMENT
