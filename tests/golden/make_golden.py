"""Generates tests/golden/ref_vectors.npz from the reference's own portable C++.

Run in a container that has the reference checkout (``make -C oracle ref`` first).  Inputs are
drawn with the reference's seeded generators (test/common/data_generator.h: mt19937, seed 42 for
A and C, 123 for B, 7 for bias) on the shape lists of its gtest suites
(test/gemm/test_gemm_i8_i8_rvv.cpp:31-41, test/gemm/test_gemm_f16_i4_rvv.cpp:19-49); outputs
come from the reference functions behind oracle/ref_shim.cpp.  The file is small (< 1 MB) and
committed, so the pins also run where the reference checkout does not exist.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.tqo import TD_BF16, TD_F16, TD_F32, ConvGeometry, Reference  # noqa: E402

I8_SHAPES = [(32, 32, 32, False), (3, 8, 11, False), (5, 11, 10, False), (9, 19, 23, False),
             (15, 32, 25, False), (60, 63, 127, False), (32, 32, 32, True), (60, 63, 127, True)]
# (m, n, k, bl, bias, c, clamp)
W4A16_CASES = [(8, 8, 4, 2, 0, 0, None), (16, 16, 8, 2, 0, 0, None), (32, 32, 32, 2, 0, 0, None),
               (32, 32, 32, 4, 0, 0, None), (32, 32, 32, 32, 0, 0, None), (5, 11, 10, 2, 0, 0, None),
               (7, 3, 10, 2, 0, 0, None), (17, 19, 24, 4, 0, 0, None), (31, 35, 64, 32, 0, 0, None),
               (60, 61, 128, 32, 0, 0, None), (32, 32, 32, 2, 1, 0, None), (17, 19, 24, 4, 1, 0, None),
               (32, 32, 32, 4, 0, 0, (-0.5, 0.5)), (32, 32, 32, 4, 0, 1, None),
               (32, 32, 32, 4, 1, 1, (-0.5, 0.5))]
# test/gemm/test_gemm_i8_i4_rvv.cpp:164-179: (m, n, k, bias, c, clamp)
W4A8_CASES = [(8, 8, 8, 0, 0, None), (16, 16, 16, 0, 0, None), (32, 32, 32, 0, 0, None), (5, 11, 16, 0, 0, None),
              (7, 3, 8, 0, 0, None), (17, 19, 24, 0, 0, None), (31, 35, 64, 0, 0, None), (60, 61, 128, 0, 0, None),
              (32, 32, 32, 1, 0, None), (17, 19, 24, 1, 0, None), (32, 32, 32, 0, 0, (-0.5, 0.5)),
              (32, 32, 32, 0, 1, None), (32, 32, 32, 1, 1, (-0.5, 0.5))]
# test/conv/test_conv_i8_i8_rvv.cpp:21-41 (ic, oc, groups, ih, iw, kh, kw + stride / pad / dilation setters), then
# cases the reference's list lacks: depth, groups (group index 1), channel counts that are multiples of 16, 1x1 stride 2
def _conv2d(ic, oc, g, ih, iw, kh, kw, stride=(1, 1), pad=(0, 0), dil=(1, 1), group_idx=0):
    return (ConvGeometry(ic, oc, g, (1, ih, iw), (1, kh, kw), (1,) + stride, (1,) + dil, (0,) + pad), group_idx)


CONV_CASES = [_conv2d(3, 16, 1, 8, 8, 3, 3), _conv2d(16, 32, 1, 8, 8, 3, 3), _conv2d(16, 32, 1, 8, 8, 1, 1),
              _conv2d(3, 16, 1, 8, 8, 3, 3, pad=(1, 1)), _conv2d(3, 16, 1, 8, 8, 3, 3, stride=(2, 2)),
              _conv2d(3, 16, 1, 8, 8, 3, 3, dil=(2, 2), pad=(2, 2)),
              _conv2d(3, 16, 1, 8, 8, 3, 3, pad=(1, 1), stride=(2, 2)), _conv2d(8, 16, 1, 7, 11, 3, 5),
              _conv2d(64, 128, 1, 4, 4, 1, 1), _conv2d(3, 32, 1, 16, 16, 3, 3, pad=(1, 1)), _conv2d(3, 8, 1, 6, 6, 3, 3),
              _conv2d(64, 32, 1, 4, 4, 3, 3, pad=(1, 1)),
              (ConvGeometry(4, 8, 1, (3, 5, 6), (2, 3, 2), (1, 2, 1), (1, 1, 2), (1, 0, 1)), 0),
              _conv2d(8, 16, 2, 9, 7, 3, 3, pad=(1, 1), group_idx=1),
              _conv2d(32, 32, 2, 12, 13, 3, 3, pad=(1, 1), group_idx=1),
              _conv2d(16, 8, 1, 9, 9, 1, 1, stride=(2, 2))]
MULTIPLIERS = [0.0025, 0.0, 1.0, 0.5, 0.75, 1e-12, 1e-9, 2.0 ** -31, 2.0 ** -32, 2.0 ** -33, 123.456,
               0.05 * 0.001 / 0.1, 0.05 * 0.01 / 0.1, 0.9999999999, 0.99999999999999989,
               1.0 - 2.0 ** -31, 1.0 - 2.0 ** -32, 0.5 + 2.0 ** -32, 0.5 + 3 * 2.0 ** -33,
               0.5 + 2.0 ** -33, -0.0025, -1.5, 3.0e-5, 7.7e-3, 1.0 / 3.0, 2.0 / 3.0]


def main():
    ref = Reference()
    assert ref.available(), "build oracle/_ref first: make -C oracle ref"
    out = {}
    # ---- gemm_clamp_i32_i8_i8: int8 in U[-50,50], C in U[-1000,1000], clamp +-100000 ----------
    for idx, (m, n, k, has_c) in enumerate(I8_SHAPES):
        A = ref.fill_uniform((m, k), np.int8, -50, 50, 42)
        Bt = ref.fill_uniform((n, k), np.int8, -50, 50, 123)   # [n, k]
        Bn = ref.fill_uniform((k, n), np.int8, -50, 50, 123)   # [k, n]
        Cm = ref.fill_uniform((m, n), np.int32, -1000, 1000, 42) if has_c else None
        out[f"i8_{idx}_A"], out[f"i8_{idx}_Bt"], out[f"i8_{idx}_Bn"] = A, Bt, Bn
        if has_c:
            out[f"i8_{idx}_C"] = Cm
        out[f"i8_{idx}_Dt"] = ref.gemm_i32_i8(A, Bt, True, Cm, (-100000, 100000))
        out[f"i8_{idx}_Dn"] = ref.gemm_i32_i8(A, Bn, False, Cm, (-100000, 100000))
        # a narrow clamp so that both clamp edges are exercised
        out[f"i8_{idx}_Dn_narrow"] = ref.gemm_i32_i8(A, Bn, False, Cm, (-3000, 2500))
    out["i8_shapes"] = np.array([(m, n, k, int(c)) for m, n, k, c in I8_SHAPES], np.int64)
    # ---- requantisation multiplier ---------------------------------------------------------
    ms = [ref.quantize_multiplier(v) for v in MULTIPLIERS]
    rng = np.random.default_rng(5)
    rnd = np.concatenate([rng.uniform(1e-6, 1.0, 200), np.exp(rng.uniform(-30, 5, 200))])
    out["mult_in"] = np.concatenate([np.array(MULTIPLIERS, np.float64), rnd])
    out["mult_out"] = np.array([ref.quantize_multiplier(float(v)) for v in out["mult_in"]], np.int64)
    assert ms[0] == (1374389535, -8)
    # ---- scalar quantiser ----------------------------------------------------------------
    vals = rng.normal(0, 2, 4000).astype(np.float32)
    scales = rng.uniform(1e-3, 0.1, 4000).astype(np.float32)
    zps = rng.integers(-128, 128, 4000).astype(np.int32)
    vals[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, 1e9, -1e9, 0.0]
    scales[:8] = 1.0
    zps[:8] = 0
    out["qi8_val"], out["qi8_scale"], out["qi8_zp"] = vals, scales, zps
    out["qi8_out"] = np.array([ref.lib.ref_quantize_i8(float(v), float(s), int(z))
                               for v, s, z in zip(vals, scales, zps)], np.int8)
    # ---- zero-point fusion ------------------------------------------------------------------
    data = ref.fill_uniform((19, 23), np.int8, -128, 127, 123)
    bias = ref.fill_uniform((1, 19), np.int32, -1000, 1000, 7).reshape(19)
    out["fuse_data"], out["fuse_bias"] = data, bias
    out["fuse_out"] = ref.fuse_zp_to_bias(bias, data, 3)
    # ---- 16-bit float conversions ----------------------------------------------------------
    bits = rng.integers(0, 2 ** 32, 6000, dtype=np.uint64).astype(np.uint32)
    f = bits.view(np.float32)
    f = f[np.isfinite(f)]
    special = np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                        6.1e-5, 6.0975552e-5, 1.0009765625, 1.00048828125, 1.00146484375, 3.0e38,
                        -3.0e38, 1e-40], np.float32)
    f = np.concatenate([special, f, rng.normal(0, 1, 3000).astype(np.float32)])
    out["cvt_in"] = f
    out["cvt_f16"] = np.array([ref.lib.ref_f32_to_f16(float(x)) for x in f], np.uint16)
    out["cvt_bf16"] = np.array([ref.lib.ref_f32_to_bf16(float(x)) for x in f], np.uint16)
    # ---- W4A16 ------------------------------------------------------------------------------
    for idx, (m, n, k, bl, has_bias, has_c, clamp) in enumerate(W4A16_CASES):
        A = ref.fill_uniform((m, k), np.float16, -1.0, 1.0, 42)
        W = ref.fill_uniform((n, k), np.float16, -1.0, 1.0, 123)
        nib, sc = ref.quantize_fp16_to_int4(W.view(np.uint16), bl)
        out[f"w4a16_{idx}_A"], out[f"w4a16_{idx}_W"] = A, W
        out[f"w4a16_{idx}_nib"], out[f"w4a16_{idx}_scale"] = nib, sc
        cl = clamp if clamp else (-65504.0, 65504.0)
        for td, tag, dt in ((TD_F16, "f16", np.float16), (TD_F32, "f32", np.float32)):
            Cm = ref.fill_uniform((m, n), dt, -5.0, 5.0, 42) if has_c else None
            bias = ref.fill_uniform((1, n), dt, -0.5, 0.5, 7).reshape(n) if has_bias else None
            if has_c:
                out[f"w4a16_{idx}_C_{tag}"] = Cm
            if has_bias:
                out[f"w4a16_{idx}_bias_{tag}"] = bias
            cv = None if Cm is None else (Cm.view(np.uint16) if td == TD_F16 else Cm)
            bv = None if bias is None else (bias.view(np.uint16) if td == TD_F16 else bias)
            cl_td = cl if clamp else ((-65504.0, 65504.0) if td == TD_F16 else (-3.4028234663852886e38, 3.4028234663852886e38))
            out[f"w4a16_{idx}_D_{tag}"] = ref.gemm_w4a16(A.view(np.uint16), nib, sc, bl, td, cv, bv, cl_td)
    out["w4a16_cases"] = np.array([(m, n, k, bl, b, c, 0 if cl is None else 1)
                                   for m, n, k, bl, b, c, cl in W4A16_CASES], np.int64)
    # ---- W4A8: the helpers of test/gemm/test_gemm_i8_i4_rvv.cpp:36-158, compiled from the reference -----
    # Inputs as run_w4a8_packed_gemm_test draws them (:337-367): one generator U(-1,1) seed 42 fills A then B;
    # C in TD U(-2,2) seed 42; bias in TD U(-0.5,0.5) seed 7.
    assert ref.has_w4a8(), "oracle/_ref was built without the W4A8 helpers: make -C oracle ref REF=..."
    FMAX = 3.4028234663852886e38
    for idx, (m, n, k, has_bias, has_c, clamp) in enumerate(W4A8_CASES):
        AB = ref.fill_uniform((1, m * k + n * k), np.float32, -1.0, 1.0, 42).reshape(-1)
        A, W = AB[:m * k].reshape(m, k).copy(), AB[m * k:].reshape(n, k).copy()
        q, sa, zp = ref.w4a8_quantize_a_per_row_asym(A)
        nib, sb = ref.w4a8_quantize_b_per_channel_sym_int4(W)
        out[f"w4a8_{idx}_A"], out[f"w4a8_{idx}_W"] = A, W
        out[f"w4a8_{idx}_q"], out[f"w4a8_{idx}_sa"], out[f"w4a8_{idx}_zp"] = q, sa, zp
        out[f"w4a8_{idx}_nib"], out[f"w4a8_{idx}_sb"] = nib, sb
        cl = clamp if clamp else (-FMAX, FMAX)
        for td, tag, dt in ((TD_F32, "f32", np.float32), (TD_F16, "f16", np.float16), (TD_BF16, "bf16", "bf16")):
            Cm = ref.fill_uniform((m, n), dt, -2.0, 2.0, 42) if has_c else None
            bias = ref.fill_uniform((1, n), dt, -0.5, 0.5, 7).reshape(n) if has_bias else None
            if Cm is not None and Cm.dtype == np.float16:
                Cm = Cm.view(np.uint16)
            if bias is not None and bias.dtype == np.float16:
                bias = bias.view(np.uint16)
            if has_c:
                out[f"w4a8_{idx}_C_{tag}"] = Cm
            if has_bias:
                out[f"w4a8_{idx}_bias_{tag}"] = bias
            out[f"w4a8_{idx}_D_{tag}"] = ref.w4a8_gemm(q, nib, sa, zp, sb, td, Cm, bias, cl)
    out["w4a8_cases"] = np.array([(m, n, k, b, c, 0 if cl is None else 1) for m, n, k, b, c, cl in W4A8_CASES],
                                 np.int64)
    # rows that exercise the quantiser's branches: all-zero, all-positive, all-negative, tiny range, huge range,
    # values on rounding boundaries of x / s
    rng2 = np.random.default_rng(17)
    Aq = rng2.normal(0, 1, (24, 40)).astype(np.float32)
    Aq[0] = 0.0
    Aq[1] = np.abs(Aq[1])
    Aq[2] = -np.abs(Aq[2])
    Aq[3] *= np.float32(1e-30)
    Aq[4] *= np.float32(1e30)
    Aq[5] = np.float32(0.25)
    Aq[6, :] = np.linspace(-1.0, 1.0, 40, dtype=np.float32) * np.float32(127.5)
    Aq[7] = np.round(Aq[7] * 8) / 8
    Aq[8] *= np.float32(1e-41)          # subnormal row
    out["w4a8_edge_A"] = Aq
    q, sa, zp = ref.w4a8_quantize_a_per_row_asym(Aq)
    out["w4a8_edge_q"], out["w4a8_edge_sa"], out["w4a8_edge_zp"] = q, sa, zp
    Wq = rng2.normal(0, 0.02, (12, 40)).astype(np.float32)
    Wq[0] = 0.0
    Wq[1] = np.float32(0.5)
    Wq[2, ::2] = np.float32(-1.0)
    Wq[3] = np.round(Wq[3] * 400) / 400
    out["w4a8_edge_W"] = Wq
    nib, sb = ref.w4a8_quantize_b_per_channel_sym_int4(Wq)
    out["w4a8_edge_nib"], out["w4a8_edge_sb"] = nib, sb
    # ---- im2col of the int8 convolution wrappers: the same flat input read as [C,D,H,W] and as [D,H,W,C] ----
    for idx, (geom, group_idx) in enumerate(CONV_CASES):
        act = ref.fill_uniform((int(np.prod(geom.input_shape)), geom.input_channel), np.int8, -128, 127, 42)
        out[f"conv_{idx}_geom"] = np.concatenate([geom.as_array().astype(np.int64), [group_idx]])
        out[f"conv_{idx}_cl"] = ref.im2col_i8(act, geom, False, group_idx)
        out[f"conv_{idx}_cf"] = ref.im2col_i8(act, geom, True, group_idx)
    out["conv_cases"] = np.array([len(CONV_CASES)], np.int64)
    # ---- unquantised GEMM families: reference_gemm<TA, TD> on the suite's shapes and options
    # (test/gemm/test_gemm_f32_f32_rvv.cpp:30-49; inputs U(-1,1) seed 42 for A then B, seed 43 for C then bias,
    # test/common/gemm_test_runner.h:326-365), both B layouts, column and row bias ----
    tname = {TD_F32: "f32", TD_F16: "f16", TD_BF16: "bf16"}
    npdt = {TD_F32: np.float32, TD_F16: np.float16, TD_BF16: "bf16"}
    # (m, n, k, bias, c, clamp)
    fl_cases = [(32, 32, 32, 0, 0, None), (5, 11, 10, 0, 0, None), (17, 19, 23, 0, 0, None), (60, 61, 127, 0, 0, None),
                (31, 35, 63, 1, 0, None), (32, 32, 32, 0, 0, (-100.0, 150.0)), (31, 35, 63, 0, 1, None),
                (60, 61, 127, 1, 1, (-100.0, 150.0)), (31, 35, 63, 1, 1, (-1.5, 2.0))]
    for ta, td in ((TD_F32, TD_F32), (TD_F16, TD_F16), (TD_BF16, TD_BF16), (TD_BF16, TD_F32), (TD_BF16, TD_F16)):
        for idx, (m, n, k, has_bias, has_c, clamp) in enumerate(fl_cases):
            tag = f"fl_{tname[ta]}_{tname[td]}_{idx}"
            AB = ref.fill_uniform((1, m * k + n * k), npdt[ta], -1.0, 1.0, 42).reshape(-1)
            A, B = AB[:m * k].reshape(m, k).copy(), AB[m * k:].reshape(n, k).copy()
            CB = ref.fill_uniform((1, m * n + max(m, n)), npdt[td], -1.0, 1.0, 43).reshape(-1)
            Cm = CB[:m * n].reshape(m, n).copy() if has_c else None
            bias_n = CB[m * n:m * n + n].copy() if has_bias else None
            bias_m = CB[m * n:m * n + m].copy() if has_bias else None
            bits = lambda x: None if x is None else (x.view(np.uint16) if x.dtype == np.float16 else x)
            A_, B_ = bits(A), bits(B)
            Bn_ = np.ascontiguousarray(B_.T)
            cl = clamp if clamp else (-FMAX, FMAX)
            out[tag + "_A"], out[tag + "_B"] = A_, B_
            if has_c:
                out[tag + "_C"] = bits(Cm)
            if has_bias:
                out[tag + "_bias"] = bits(CB[m * n:].copy())
            out[tag + "_Dt"] = ref.gemm_float(ta, td, A_, B_, True, bits(Cm), bits(bias_n), False, cl)
            out[tag + "_Dn"] = ref.gemm_float(ta, td, A_, Bn_, False, bits(Cm), bits(bias_n), False, cl)
            out[tag + "_Dr"] = ref.gemm_float(ta, td, A_, B_, True, bits(Cm), bits(bias_m), True, cl)
    out["fl_cases"] = np.array([(m, n, k, b, c, 0 if cl is None else 1, 0.0 if cl is None else cl[0], 0.0 if cl is None else cl[1])
                                for m, n, k, b, c, cl in fl_cases], np.float64)
    path = os.path.join(HERE, "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
