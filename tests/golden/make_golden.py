"""Writes tests/golden/golden.npz from the REFERENCE's own host code.

Run in a container that has the reference tree:  make -C oracle ref  &&
python tests/golden/make_golden.py.  Every array is produced by a function of
oracle/_ref/libslopfab_ref.so, i.e. by the reference's unmodified fixtures
(tests/detail/nn_weight_fixture.h, tests/detail/nn_kernels_fixture.h,
tests/harness.cpp, include/slopfab/dtype.h, src/core/int8_weight.cpp, src/dit/packing.cpp); nothing
here comes from the oracle or from the product. The oracle is then pinned to
these vectors by tests/test_oracle_golden.py wherever the reference tree is
not available.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

ref = oracle.ref
assert ref is not None, "build oracle/_ref first (make -C oracle ref)"
P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
ref.ref_make_data.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_float]
ref.ref_make_gaussian.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_float]
ref.ref_make_nvfp4.argtypes = [C.c_int, C.c_int, C.c_float, C.c_uint32] + [C.c_void_p] * 4
ref.ref_pack_nvfp4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int] + [C.c_void_p] * 3
ref.ref_host_quantise_act.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
ref.ref_unpack_int8_weight.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
ref.ref_kron_h4_256.argtypes = [C.c_void_p]
for name, res, arg in [("ref_f32_to_bf16", C.c_uint16, C.c_float), ("ref_f32_to_f16", C.c_uint16, C.c_float),
                       ("ref_f16_to_f32", C.c_float, C.c_uint16), ("ref_e4m3_to_f32", C.c_float, C.c_uint8),
                       ("ref_e2m1_to_f32", C.c_float, C.c_uint8), ("ref_host_e4m3", C.c_uint8, C.c_float),
                       ("ref_host_e2m1", C.c_uint8, C.c_float)]:
    getattr(ref, name).restype = res
    getattr(ref, name).argtypes = [arg]

out = {}


def data(n, seed, scale):
    a = np.empty(n, np.float32)
    ref.ref_make_data(P(a), n, seed, scale)
    return a


def gauss(n, seed, sigma):
    a = np.empty(n, np.float32)
    ref.ref_make_gaussian(P(a), n, seed, sigma)
    return a


# generators
out["make_data_131"] = data(1280, 131, 1.0)
out["make_gaussian_4242"] = gauss(7 * 64, 4242, 0.7)

# scalar tables
out["e4m3_table"] = np.array([ref.ref_e4m3_to_f32(i) for i in range(256)], np.float32)
out["e2m1_table"] = np.array([ref.ref_e2m1_to_f32(i) for i in range(16)], np.float32)
vals = np.concatenate([np.array([0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 1e4, -1e4, 0.0], np.float32),
                       data(512, 909, 8.0)])
out["round_vals"] = vals
out["round_e2m1"] = np.array([ref.ref_host_e2m1(float(v)) for v in vals], np.uint8)
out["round_e4m3"] = np.array([ref.ref_host_e4m3(float(v)) for v in vals], np.uint8)
cv = np.concatenate([data(4000, 77, 70000.0), data(2000, 78, 1e-4), data(2000, 79, 2.0)]).astype(np.float32)
out["conv_vals"] = cv
out["conv_bf16"] = np.array([ref.ref_f32_to_bf16(float(v)) for v in cv], np.uint16)
out["conv_f16"] = np.array([ref.ref_f32_to_f16(float(v)) for v in cv], np.uint16)
out["f16_table"] = np.array([ref.ref_f16_to_f32(i) for i in range(65536)], np.float32).view(np.uint32)

# nn_dequant_nvfp4: make_nvfp4(256, 128, 1.3580322e-3, 20260804) and the tile-shape sweep
def nvfp4_case(n, k, g, seed):
    packed = np.empty(n * k // 2, np.uint8)
    stored = np.empty(n * k // 16, np.uint8)
    plain = np.empty(n * k // 16, np.uint8)
    refv = np.empty(n * k, np.float32)
    ref.ref_make_nvfp4(n, k, g, seed, P(packed), P(stored), P(plain), P(refv))
    return packed, stored, plain, oracle.to_bf16(refv)  # values are bf16-exact by construction


pk, st, pl, rv = nvfp4_case(256, 128, 1.3580322e-3, 20260804)
out["nvfp4_256x128_packed"], out["nvfp4_256x128_stored"], out["nvfp4_256x128_plain"], out["nvfp4_256x128_ref"] = pk, st, pl, rv
for i, (n, k) in enumerate([(128, 64), (128, 512), (384, 128), (256, 320), (512, 64)]):
    pk, st, pl, rv = nvfp4_case(n, k, 0.0021, 90210 + 7 * i)
    out[f"nvfp4_tile{i}_packed"], out[f"nvfp4_tile{i}_stored"], out[f"nvfp4_tile{i}_ref"] = pk, st, rv

# pack_nvfp4 on Gaussian weights (the GEMM tests' weights), right form and the three wrong forms
w = gauss(256 * 192, 5151, 0.02).reshape(256, 192)
gs = float(np.abs(w).max() / (6.0 * 448.0))
out["pack_w"] = w
out["pack_global"] = np.float32(gs)
for he in (1, 0):
    for sw in (1, 0):
        d = np.empty(256 * 192 // 2, np.uint8)
        s = np.empty(256 * 192 // 16, np.uint8)
        dn = np.empty(256 * 192, np.float32)
        ref.ref_pack_nvfp4(P(w), 256, 192, gs, he, sw, P(d), P(s), P(dn))
        out[f"pack_data_{he}{sw}"], out[f"pack_scale_{he}{sw}"] = d, s
        if he and sw:
            out["pack_dense_11"] = dn

# host_quantise_act on the activation-quantisation test's input (special blocks included)
x = out["make_gaussian_4242"].copy().reshape(7, 64)
x[0, :16] = 0.0
x[1, 16:32] = 1e-6 * np.arange(1, 17, dtype=np.float32)
x[2, 32:48] = 5000.0
xr = oracle.from_bf16(oracle.to_bf16(x))
q = np.empty_like(xr)
ref.ref_host_quantise_act(P(xr), 7, 64, P(q))
out["act_x_bf16"] = oracle.to_bf16(x)
out["act_dense"] = q

# unpack_int8_weight for every group and both widths of test_int8_weight.cu
rng = np.random.default_rng(20260805)
for g in (1, 4, 16, 64, 256):
    for cols in (2 * g, 267):
        if cols % g:
            grp = 1  # rotation skipped when the row does not hold whole groups
        else:
            grp = g
        codes = rng.integers(-127, 128, size=(5, cols), dtype=np.int8)
        scales = (rng.random(5, dtype=np.float32) * 0.02 + 1e-4).astype(np.float32)
        for canon in (0, 1):
            o = np.empty((5, cols), np.uint16)
            ref.ref_unpack_int8_weight(P(codes), P(scales), 5, cols, grp, canon, P(o))
            out[f"i8_{g}_{cols}_{canon}"] = o
        out[f"i8_{g}_{cols}_codes"], out[f"i8_{g}_{cols}_scales"] = codes, scales

h = np.empty(256 * 256, np.float32)
ref.ref_kron_h4_256(P(h))
out["kron_h4_256"] = h.reshape(256, 256).astype(np.int8)

# token packing: build_indices and both forms of build_row_timesteps (src/dit/packing.cpp) on a set of layouts, with
# the layout's own tags and with padding rows (-1) written over some of them
ref.ref_build_indices.argtypes = [C.c_void_p] * 5
ref.ref_build_row_timesteps.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.POINTER(C.c_int)]
PACK_LAYOUTS = [(4, 0, 0, 0, 500, 2000), (3, 0, 0, 0, 10, 7), (5, 6, 0, 0, 12, 9), (2, 4, 3, 1, 8, 5), (0, 0, 0, 0, 0, 11),
                (1, 0, 0, 0, 6, 0), (2, 9, 0, 0, 4, 3), (7, 5, 4, 1, 3, 20), (6, 2, 0, 1, 9, 4)]
PACK_TIMES = [(0.25, 0.75, 0.0, 1.0), (0.75, 0.25, 1.0, 0.0), (0.5, 0.5, 0.5, 0.5), (0.9, 0.1, 0.9, 0.3), (0.3, 0.6, 0.6, 0.3)]
out["packing_layouts"] = np.array(PACK_LAYOUTS, np.int32)
out["packing_times"] = np.array(PACK_TIMES, np.float32)
prng = np.random.default_rng(416)
for li, lay in enumerate(PACK_LAYOUTS):
    L, Cv, Ca, ex, Sa, V = lay
    total = L + Cv + Ca + Sa + V
    l6 = np.array(lay, np.int32)
    text, audio, video, tags = (np.zeros(n, np.int32) for n in (L, Sa, Cv + Ca + V, total))
    assert ref.ref_build_indices(P(l6), P(text), P(audio), P(video), P(tags)) == 0
    out[f"packing_{li}_text"], out[f"packing_{li}_audio"], out[f"packing_{li}_video"], out[f"packing_{li}_tags"] = text, audio, video, tags
    padded = tags.copy()
    padded[prng.random(total) < 0.2] = -1
    out[f"packing_{li}_padded_tags"] = padded
    for ti, tt in enumerate(PACK_TIMES):
        for count in (2, 4):
            for pad, use in (("own", None), ("pad", padded)):
                idx, ada = np.zeros(total, np.int32), np.zeros(total, np.int32)
                uniq = np.zeros(4, np.float32)
                n = C.c_int(0)
                t4 = np.array(tt, np.float32)
                assert ref.ref_build_row_timesteps(P(l6), None if use is None else P(use), P(t4), count, P(idx), P(ada), P(uniq),
                                                   C.byref(n)) == 0
                key = f"packing_{li}_{ti}_{count}_{pad}"
                out[key + "_indices"], out[key + "_adaln"], out[key + "_unique"] = idx, ada, uniq[:n.value].copy()

np.savez_compressed(os.path.join(ROOT, "tests", "golden", "golden.npz"), **out)
print("wrote", len(out), "arrays")
