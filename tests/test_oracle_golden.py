"""Pins the CPU oracle (oracle/oracle.cpp) to the reference.

Two sources of truth: tests/golden/golden.npz, written by the reference's own
host fixtures (tests/golden/make_golden.py), and the known-answer cases spelled
out in the reference's tests, restated here with their file:line. When the
compiled reference (oracle/_ref) is present it is compared directly as well.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from oracle import lib


def test_generators(golden):
    assert np.array_equal(oracle.make_data(1280, 131, 1.0), golden["make_data_131"])
    assert np.array_equal(oracle.make_gaussian(7 * 64, 4242, 0.7), golden["make_gaussian_4242"])


def test_scalar_tables(golden):
    # include/slopfab/dtype.h:123-161 -- every e4m3 byte and every e2m1 nibble
    got8 = np.array([lib.orc_e4m3_to_f32(i) for i in range(256)], np.float32)
    assert np.array_equal(got8.view(np.uint32), golden["e4m3_table"].view(np.uint32))
    got4 = np.array([lib.orc_e2m1_to_f32(i) for i in range(16)], np.float32)
    assert np.array_equal(got4.view(np.uint32), golden["e2m1_table"].view(np.uint32))
    got16 = np.array([lib.orc_f16_to_f32(i) for i in range(65536)], np.float32).view(np.uint32)
    assert np.array_equal(got16, golden["f16_table"])


def test_narrowing_conversions(golden):
    v = golden["conv_vals"]
    assert np.array_equal(np.array([lib.orc_f32_to_bf16(float(x)) for x in v], np.uint16), golden["conv_bf16"])
    assert np.array_equal(np.array([lib.orc_f32_to_f16(float(x)) for x in v], np.uint16), golden["conv_f16"])
    # every finite e4m3 pattern survives decode -> encode (tests/detail/nn_kernels_fixture.h:390-392)
    for b in range(256):
        if (b & 0x7F) == 0x7F:
            continue
        assert lib.orc_f32_to_e4m3(lib.orc_e4m3_to_f32(b)) == b


def test_fp4_fp8_rounding_known_answers(golden):
    # tests/test_nn_kernels_nvfp4_synthetic.cu:346-378: ties 0.25/0.75/1.25/1.75/2.5/3.5/5.0,
    # saturation at +-1e4, and 512 uniform values in (-8, 8).
    vals = golden["round_vals"]
    assert np.array_equal(np.array([lib.orc_f32_to_e2m1(float(x)) for x in vals], np.uint8), golden["round_e2m1"])
    nonneg = vals >= 0
    search = np.array([lib.orc_e4m3_nearest_nonneg(float(x)) for x in vals], np.uint8)
    direct = np.array([lib.orc_f32_to_e4m3(float(x)) for x in vals], np.uint8)
    assert np.array_equal(search[nonneg], golden["round_e4m3"][nonneg])
    assert np.array_equal(direct[nonneg], golden["round_e4m3"][nonneg])
    # spelled-out ties: round half to the even code
    expect = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6, 6.0: 7, 1e4: 7, -1e4: 15, -0.1: 8}
    for v, code in expect.items():
        assert lib.orc_f32_to_e2m1(v) == code, v
    assert lib.orc_f32_to_e4m3(1e4) == 0x7E and lib.orc_f32_to_e4m3(float("nan")) == 0x7F
    # the direct encoder equals the exhaustive search on a dense sweep
    sweep = np.concatenate([np.linspace(0, 500, 20001), np.logspace(-12, 3, 4000)]).astype(np.float32)
    for x in sweep:
        assert lib.orc_f32_to_e4m3(float(x)) == lib.orc_e4m3_nearest_nonneg(float(x)), x


def test_nvfp4_scale_tile_map():
    # src/cuda/linear_weights.cu:111-115 evaluated by hand for a 256x128 weight (8 blocks per row)
    assert lib.orc_nvfp4_scale_slot(0, 0, 8) == 0
    assert lib.orc_nvfp4_scale_slot(1, 0, 8) == 16
    assert lib.orc_nvfp4_scale_slot(32, 0, 8) == 4
    assert lib.orc_nvfp4_scale_slot(0, 3, 8) == 3
    assert lib.orc_nvfp4_scale_slot(0, 4, 8) == 512
    assert lib.orc_nvfp4_scale_slot(128, 0, 8) == 1024
    assert lib.orc_nvfp4_scale_slot(255, 7, 8) == 1024 + 512 + 31 * 16 + 3 * 4 + 3
    slots = {lib.orc_nvfp4_scale_slot(o, k, 8) for o in range(256) for k in range(8)}
    assert slots == set(range(256 * 8))


def test_nvfp4_dequant_matches_reference_bits(golden):
    # tests/test_nn_kernels_nvfp4_synthetic.cu:4-76 and :78-128 (bit-exact, tolerance 0)
    g = np.float32(1.3580322e-3)
    got = oracle.nvfp4_dequant_bf16(golden["nvfp4_256x128_packed"], golden["nvfp4_256x128_stored"], g, 256, 128)
    assert np.array_equal(got.ravel(), golden["nvfp4_256x128_ref"])
    # the wrong forms must NOT match: row-major scales, swapped nibbles
    flat = oracle.nvfp4_dequant_bf16(golden["nvfp4_256x128_packed"], golden["nvfp4_256x128_plain"], g, 256, 128)
    assert np.abs(oracle.from_bf16(flat).ravel() - oracle.from_bf16(golden["nvfp4_256x128_ref"])).max() > 1e-4
    sw = golden["nvfp4_256x128_packed"]
    swapped = ((sw << 4) | (sw >> 4)).astype(np.uint8)
    bad = oracle.nvfp4_dequant_bf16(swapped, golden["nvfp4_256x128_stored"], g, 256, 128)
    assert np.abs(oracle.from_bf16(bad).ravel() - oracle.from_bf16(golden["nvfp4_256x128_ref"])).max() > 1e-4
    for i, (n, k) in enumerate([(128, 64), (128, 512), (384, 128), (256, 320), (512, 64)]):
        got = oracle.nvfp4_dequant_bf16(golden[f"nvfp4_tile{i}_packed"], golden[f"nvfp4_tile{i}_stored"],
                                        np.float32(0.0021), n, k)
        assert np.array_equal(got.ravel(), golden[f"nvfp4_tile{i}_ref"]), (n, k)


def test_nvfp4_fixture_packer(golden):
    # tests/detail/nn_weight_fixture.h:333-360, all four (nibble, tiling) conventions
    w = golden["pack_w"]
    g = float(golden["pack_global"])
    for he in (1, 0):
        for sw in (1, 0):
            data, scale, dense = oracle.nvfp4_pack(w, g, bool(he), bool(sw))
            assert np.array_equal(data.ravel(), golden[f"pack_data_{he}{sw}"])
            assert np.array_equal(scale, golden[f"pack_scale_{he}{sw}"])
    _, _, dense = oracle.nvfp4_pack(w, g)
    assert np.array_equal(dense.ravel().view(np.uint32), golden["pack_dense_11"].view(np.uint32))


def test_nvfp4_activation_quantizer(golden):
    # tests/test_nn_kernels_nvfp4_synthetic.cu:380-453
    x = golden["act_x_bf16"]
    packed, scales, dense = oracle.nvfp4_quantize_act(x)
    assert np.array_equal(dense.ravel().view(np.uint32), golden["act_dense"].ravel().view(np.uint32))
    assert scales[0, 0] == 0 and not packed[0, :8].any()        # all-zero block: scale 0, nibbles 0
    assert scales[1, 1] == 0                                      # underflow flushes the block
    assert lib.orc_e4m3_to_f32(int(scales[2, 2])) == 448.0        # overflow saturates the scale ...
    assert (packed[2, 16:24] == 0x77).all()                       # ... and the elements clip at +6
    assert np.isfinite(dense).all()
    # low nibble is the even element
    xf = oracle.from_bf16(x)
    r, b = 3, 1
    sd = lib.orc_e4m3_to_f32(int(scales[r, b]))
    assert lib.orc_f32_to_e2m1(float(np.float32(xf[r, 16]) * np.float32(1.0 / sd))) == packed[r, 8] & 15


def test_int8_weight_unpack(golden):
    # tests/test_int8_weight.cu:95-141 -- groups {1,4,16,64,256} x widths {2g, 267}, bit-exact fp16
    for g in (1, 4, 16, 64, 256):
        for cols in (2 * g, 267):
            grp = g if cols % g == 0 else 1
            codes, scales = golden[f"i8_{g}_{cols}_codes"], golden[f"i8_{g}_{cols}_scales"]
            for canon in (0, 1):
                out = np.empty((5, cols), np.uint16)
                lib.orc_int8_unpack_f16(codes.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p),
                                        5, cols, grp, canon, out.ctypes.data_as(C.c_void_p))
                assert np.array_equal(out, golden[f"i8_{g}_{cols}_{canon}"]), (g, cols, canon)


def test_convrot_is_the_regular_hadamard(golden):
    # tests/test_nn_kernels_linear_synthetic.cu:251-383: kron^4(h4)/16, not Sylvester
    H = golden["kron_h4_256"].astype(np.float64) / 16.0
    x = oracle.from_bf16(oracle.to_bf16(golden["make_data_131"].reshape(5, 256)))
    want = x.astype(np.float64) @ H.T
    dense = oracle.convrot_dense(x)
    assert np.abs(dense - want).max() < 1e-5
    fly = oracle.from_bf16(oracle.convrot_bf16(oracle.to_bf16(x)))
    assert np.abs(fly - want).max() < 1e-2 * np.abs(want).max()          # bf16 store
    assert np.array_equal(oracle.to_bf16(dense.astype(np.float32)) != oracle.convrot_bf16(oracle.to_bf16(x)),
                          np.zeros((5, 256), bool)) or np.abs(fly - want).max() < 4e-3
    # H is symmetric, orthogonal and involutory
    assert np.array_equal(H, H.T) and np.allclose(H @ H, np.eye(256))
    # Sylvester's construction differs grossly
    s2 = np.array([[1, 1], [1, -1]], np.float64)
    S = s2
    for _ in range(7):
        S = np.kron(S, s2)
    assert np.abs(x @ (S / 16.0).T - want).max() > 0.1
    # three groups per row (seed 132) and group 16 (seed 133)
    x3 = oracle.from_bf16(oracle.to_bf16(oracle.make_data(2 * 768, 132, 1.0).reshape(2, 768)))
    want3 = np.concatenate([x3[:, i * 256:(i + 1) * 256].astype(np.float64) @ H.T for i in range(3)], axis=1)
    assert np.abs(oracle.convrot_dense(x3) - want3).max() < 1e-5
    h4 = np.array([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], np.float64)
    H16 = np.kron(h4, h4) / 4.0
    x16 = oracle.make_data(3 * 64, 133, 1.0).reshape(3, 64)
    want16 = np.concatenate([x16[:, i * 16:(i + 1) * 16].astype(np.float64) @ H16.T for i in range(4)], axis=1)
    assert np.abs(oracle.convrot_dense(x16, 16) - want16).max() < 1e-6


def _packed_case(bits, group, rows=3, out=4, k=256):
    """Builds the bytes of tests/test_nn_kernels_linear_synthetic.cu:820-834."""
    packed = np.zeros((out, k * bits // 8), np.uint8)
    levels = np.zeros((out, k), np.int32)
    for o in range(out):
        for i in range(k):
            code = (i * 7 + o * 13) % (1 << bits)
            levels[o, i] = code - (1 << (bits - 1))
            packed[o, i // 2] |= (code & 15) << ((i & 1) * 4)
            if bits == 6:
                packed[o, k // 2 + i // 4] |= (code >> 4) << ((i & 3) * 2)
    sv = [0, 0x30, 0x38, 0x48, 0x78]
    scales = np.array([sv[i % 5] for i in range(out * k // group)], np.uint8)
    book = np.arange(16, dtype=np.float32) - 8.0
    channel = np.array([.25, .5, 1., 2.], np.float32)
    x = np.zeros((rows, k), np.float32)
    x[1, 0] = 1.0
    x[2, :] = 1.0
    return packed, levels, scales, book, channel, x


@pytest.mark.parametrize("bits,group", [(4, 16), (6, 16), (6, 32), (6, 64)])
def test_packed_int8_linear_known_answer(golden, bits, group):
    # tests/test_nn_kernels_linear_synthetic.cu:820-890: the test's own integer reference, restated in
    # numpy (dense Kronecker rotation, bf16 scale/quotient rounding, e4m3 group scales), must equal the
    # oracle's butterfly pipeline bit for bit.
    packed, levels, scales, book, channel, x = _packed_case(bits, group)
    rows, out, k = 3, 4, 256
    H = golden["kron_h4_256"].astype(np.float32)
    y = oracle.packed_int8_linear(oracle.to_bf16(x), packed, scales, channel, book if bits == 4 else None,
                                  bits, group, out, k)
    rb = lambda v: oracle.from_bf16(oracle.to_bf16(np.float32(v)))  # noqa: E731
    for r in range(rows):
        rot = np.zeros(k, np.float32)
        for i in range(k):
            acc = np.float32(0)
            for j in range(k):
                acc = np.float32(acc + np.float32(H[i, j] / np.float32(16)) * x[r, j])
            rot[i] = acc
        scale = max(np.float32(np.abs(rot).max() / np.float32(127)), np.float32(1e-30))
        rounded = rb(scale)
        quo = rb(rot / rounded)
        q = np.clip(np.rint(quo), -128, 127).astype(np.int32)
        for o in range(out):
            sdec = np.array([lib.orc_e4m3_to_f32(int(scales[(o * k + i) // group])) for i in range(k)], np.float32)
            w = np.clip(np.rint(levels[o].astype(np.float32) * sdec), -127, 127).astype(np.int32)
            s = int((q * w).sum())
            want = oracle.to_bf16(np.float32(np.float32(np.float32(s) * scale) * channel[o]))
            assert y[r, o] == want, (r, o)


def test_w4a8_weight_decode_known_answer():
    # tests/test_nn_kernels_linear_synthetic.cu:152-186: unit scales + codebook i-8 decode to code-8
    out_f, in_f = 3, 256
    packed = np.zeros((out_f, in_f // 2), np.uint8)
    want = np.zeros((out_f, in_f), np.int8)
    for o in range(out_f):
        for i in range(0, in_f, 2):
            lo, hi = (o * 5 + i) & 15, (o * 7 + i + 1) & 15
            packed[o, i // 2] = lo | (hi << 4)
            want[o, i], want[o, i + 1] = lo - 8, hi - 8
    gs = np.full(out_f * in_f // 16, 0x38, np.uint8)
    book = np.arange(16, dtype=np.float32) - 8.0
    assert np.array_equal(oracle.w4a8_decode(packed, gs, book, out_f, in_f), want)


def test_vulkan_suite_cpu_reference_w4_w6():
    # tests/test_vulkan_linear_synthetic.cpp:1046-1083: rows=5, N=34, K=512, non-integer codebook
    # (i-7)*0.5, scale bytes {0,0x38,0x48,0x78}, channel 2^(i%4-3); checked here through an independent
    # numpy evaluation of the same equations.
    rows, n, k = 5, 34, 512
    for bits, group in ((4, 16), (6, 32)):
        packed = np.zeros((n, k * bits // 8), np.uint8)
        code = np.zeros((n, k), np.int32)
        for o in range(n):
            for i in range(k):
                c = (i * 7 + o * 13) % (1 << bits)
                code[o, i] = c
                packed[o, i // 2] |= (c & 15) << ((i & 1) * 4)
                if bits == 6:
                    packed[o, k // 2 + i // 4] |= (c >> 4) << ((i & 3) * 2)
        sv = [0, 0x38, 0x48, 0x78]
        scales = np.array([sv[i % 4] for i in range(n * k // group)], np.uint8)
        book = ((np.arange(16) - 7) * 0.5).astype(np.float32)
        channel = np.array([2.0 ** (i % 4 - 3) for i in range(n)], np.float32)
        x = np.zeros((rows, k), np.float32)
        x[1, 3] = 1.0
        x[2] = ((np.arange(k) * 37) % 53 - 26) / 8.0
        x[3] = -0.5
        x[4] = oracle.make_data(k, 7, 2.0)
        xb = oracle.to_bf16(x)
        y, inter = oracle.packed_int8_linear(xb, packed, scales, channel, book if bits == 4 else None, bits,
                                             group, n, k, want_intermediates=True)
        sdec = np.array([lib.orc_e4m3_to_f32(int(s)) for s in scales], np.float32).reshape(n, k // group)
        lev = book[code] if bits == 4 else (code - 32).astype(np.float32)
        w8 = np.clip(np.rint(lev * np.repeat(sdec, group, axis=1)), -127, 127).astype(np.int8)
        assert np.array_equal(inter["w8"], w8)
        acc = inter["q"].astype(np.int64) @ w8.astype(np.int64).T
        assert np.array_equal(acc, inter["acc"])
        want = oracle.to_bf16((inter["acc"].astype(np.float32) * inter["row_scale"][:, None]) * channel[None, :])
        assert np.array_equal(want, y)
        assert not y[0].any()  # zero row stays zero


def test_int8_token_quantizer_rules():
    # src/cuda/w4a8.cu:193-216: division by 127, bf16-rounded divisor and quotient, clamp to [-128, 127]
    x = oracle.to_bf16(np.array([[0.0] * 256, [1.0] + [0.0] * 255, [3.0, -3.0, 1.5, 0.011] + [0.0] * 252], np.float32))
    q, s = oracle.quantize_int8_token(x)
    assert s[0] == np.float32(1e-30) and not q[0].any()
    assert s[1] == np.float32(1.0) / np.float32(127.0) and q[1, 0] == 127
    # 3/127 rounds UP to bf16 0.02368, 3/0.02368 = 126.68 rounds to bf16 126.5, which ties to even 126:
    # the bf16 round trips are part of the rule, and the top code is not always 127.
    assert q[2, 0] == 126 and q[2, 1] == -126 and q[2, 2] in (63, 64)


def test_rmsnorm_bit_level_vs_spec():
    # tests/test_nn_kernels.cu:3-100 tolerance 1e-3 abs / 1e-2 rel against the double-precision form
    rng = np.random.default_rng(5)
    rows, dim = 9, 5120
    x = oracle.to_bf16(rng.standard_normal((rows, dim), dtype=np.float32))
    w = oracle.to_bf16(1.0 + 0.1 * rng.standard_normal(dim, dtype=np.float32))
    scale = (0.1 * rng.standard_normal((3, dim))).astype(np.float32)
    shift = (0.1 * rng.standard_normal((3, dim))).astype(np.float32)
    a = (np.arange(rows) % 3).astype(np.int32)
    for mod in (False, True):
        got = oracle.from_bf16(oracle.rmsnorm_bf16(x, w, 1e-5, *( (scale, shift, a) if mod else ())))
        want = np.empty((rows, dim), np.float32)
        xf, wf = oracle.from_bf16(x), oracle.from_bf16(w)
        V = C.c_void_p
        P = lambda arr: arr.ctypes.data_as(V) if arr is not None else None  # noqa: E731
        lib.orc_rmsnorm_spec_f32(P(xf), P(wf), P(scale if mod else None), P(shift if mod else None),
                                 P(a if mod else None), rows, dim, 1e-5, P(want))
        assert np.all(np.abs(got - want) <= 1e-3 + 1e-2 * np.abs(want))
    # the missing-"1+" hazard form must not match
    bad = oracle.from_bf16(oracle.rmsnorm_bf16(x, w, 1e-5)) * scale[a] + shift[a]
    good = oracle.from_bf16(oracle.rmsnorm_bf16(x, w, 1e-5, scale, shift, a))
    assert np.abs(bad - good).max() > 0.5


def test_integer_rsqrt_is_within_one_ulp_of_double():
    rng = np.random.default_rng(11)
    for v in np.concatenate([rng.random(2000) * 10 + 1e-6, 10.0 ** rng.uniform(-30, 30, 2000)]).astype(np.float32):
        got = lib.orc_rsqrt_q30(float(v))
        want = np.float32(1.0 / np.sqrt(np.float64(v)))
        assert abs(np.float32(got).view(np.int32) - want.view(np.int32)) <= 1, v


@pytest.mark.skipif(oracle.ref is None, reason="compiled reference not present")
def test_oracle_against_compiled_reference_host_code():
    ref = oracle.ref
    P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    ref.ref_pack_nvfp4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int] + [C.c_void_p] * 3
    ref.ref_host_quantise_act.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    ref.ref_cpu_matmul_nt.argtypes = [C.c_void_p] * 2 + [C.c_int] * 3 + [C.c_void_p]
    rng = np.random.default_rng(0)
    # config 1 of the benchmark set: N=K=1024 Gaussian(0, 0.02) weights
    w = (0.02 * rng.standard_normal((1024, 1024))).astype(np.float32)
    g = float(np.abs(w).max() / (6 * 448))
    d = np.empty(w.size // 2, np.uint8)
    s = np.empty(w.size // 16, np.uint8)
    dn = np.empty(w.size, np.float32)
    ref.ref_pack_nvfp4(P(w), 1024, 1024, g, 1, 1, P(d), P(s), P(dn))
    od, os_, odn = oracle.nvfp4_pack(w, g)
    assert np.array_equal(od.ravel(), d) and np.array_equal(os_, s)
    assert np.array_equal(odn.ravel().view(np.uint32), dn.view(np.uint32))
    x = oracle.from_bf16(oracle.to_bf16(rng.standard_normal((64, 1024)).astype(np.float32)))
    q = np.empty_like(x)
    ref.ref_host_quantise_act(P(x), 64, 1024, P(q))
    _, _, dense = oracle.nvfp4_quantize_act(oracle.to_bf16(x))
    assert np.array_equal(dense.view(np.uint32), q.view(np.uint32))
    c_ref = np.empty((64, 1024), np.float32)
    ref.ref_cpu_matmul_nt(P(q), P(dn), 64, 1024, 1024, P(c_ref))
    c_orc = np.empty((64, 1024), np.float32)
    lib.orc_matmul_nt(P(dense), P(odn), 64, 1024, 1024, P(c_orc))
    assert np.array_equal(c_ref.view(np.uint32), c_orc.view(np.uint32))


def test_lora_statement_known_answer():
    """tests/test_lora_backends.cu:84-101 on numbers small enough to do by hand (all exact in bf16)."""
    x = oracle.to_bf16(np.array([[1.0, 2.0, 0.0, -1.0], [0.5, 0.0, 0.0, 0.0]], np.float32))
    a = np.array([[1.0, 0.5, 0.0, 1.0], [0.0, 0.0, 2.0, 0.0]], np.float32)           # rank 2, in 4
    b = np.array([[9.0, 9.0], [1.0, 0.0], [2.0, 1.0], [0.0, 3.0]], np.float32)       # out_total 4, rank 2
    y0 = oracle.to_bf16(np.array([[1.0, 1.0], [0.25, 0.0]], np.float32))
    # hidden = x A^T = [[1, 0], [0.5, 0]]; rows 1..2 of b -> [[1, 0], [2, 1]]; delta = [[1, 2], [0.5, 1]]
    got = oracle.from_bf16(oracle.lora_apply(x, a, b, 1, 2, y0))
    assert np.array_equal(got, np.array([[2.0, 3.0], [0.75, 1.0]], np.float32))
    # rounding points: hidden is rounded to bf16 before the second product
    x = oracle.to_bf16(np.array([[1.0, 2.0 ** -9]], np.float32))
    a = np.array([[1.0, 1.0]], np.float32)                                              # 1 + 2^-9 rounds to 1 in bf16
    b = np.array([[256.0]], np.float32)
    got = oracle.from_bf16(oracle.lora_apply(x, a, b, 0, 1, oracle.to_bf16(np.zeros((1, 1), np.float32))))
    assert got[0, 0] == 256.0


def test_head_norm_rope_statement_against_plain_formulas():
    """QK-norm then MM-RoPE: x / rms(x) * w per head, then channel j rotated with j + 48 over the first 96 channels and
    96..127 passed through (include/slopfab/cuda/nn_kernels.cuh:95-134), here against float64 numpy."""
    rng = np.random.default_rng(4)
    rows, heads = 5, 3
    x = oracle.to_bf16(rng.standard_normal((rows, heads * 128)).astype(np.float32))
    w = oracle.to_bf16((1 + 0.1 * rng.standard_normal(128)).astype(np.float32))
    ang = rng.uniform(-3, 3, (rows, 96))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    got = oracle.from_bf16(oracle.head_norm_rope(x, heads, w, cos, sin, 1e-6)).reshape(rows, heads, 128).astype(np.float64)
    xf = oracle.from_bf16(x).reshape(rows, heads, 128).astype(np.float64)
    n = xf / np.sqrt((xf ** 2).mean(axis=2, keepdims=True) + 1e-6) * oracle.from_bf16(w).astype(np.float64)
    c, s = cos[:, None, :48].astype(np.float64), sin[:, None, :48].astype(np.float64)
    want = n.copy()
    want[:, :, :48] = n[:, :, :48] * c - n[:, :, 48:96] * s
    want[:, :, 48:96] = n[:, :, 48:96] * c + n[:, :, :48] * s
    assert np.abs(got - want).max() <= 3e-2  # two bf16 roundings of O(1..4) values
    assert np.array_equal(got[:, :, 96:], oracle.from_bf16(oracle.head_norm_rope(x, heads, w, None, None, 1e-6)).reshape(rows, heads, 128)[:, :, 96:])
    # rotation alone by 90 degrees swaps the halves with a sign
    x1 = oracle.to_bf16(np.arange(128, dtype=np.float32)[None, :] / 16)
    quarter = oracle.from_bf16(oracle.head_norm_rope(x1, 1, None, np.zeros((1, 96), np.float32), np.ones((1, 96), np.float32)))
    v = oracle.from_bf16(x1)
    assert np.array_equal(quarter[0, :48], -v[0, 48:96]) and np.array_equal(quarter[0, 48:96], v[0, :48])
    assert np.array_equal(quarter[0, 96:], v[0, 96:])
