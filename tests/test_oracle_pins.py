"""Pins the restated CPU oracle (oracle/tqt_oracle.c) against the reference.

Two sources: the committed golden vectors generated from the reference's own portable C++
(tests/golden/make_golden.py) and, where oracle/_ref has been built, the same functions live.
"""
import numpy as np
import pytest

from oracle.tqo import TD_BF16, TD_F16, TD_F32, Reference

FMAX = 3.4028234663852886e38
# first draws of std::mt19937(42) through libstdc++'s uniform_int_distribution<int8_t>(-128, 127) and
# normal_distribution<float>(0, 1)
KNOWN_I8_SEED42 = [-33, 75, 115, -82]
KNOWN_NORMAL_SEED42 = np.array([1.2219213247299194, -0.5169641375541687, 0.8696359395980835], np.float32)


def test_known_answer_quantize_multiplier(oracle):
    # produced by the reference's tqt_quantize_multiplier (src/gemm/gemm_i8_i8/tqt_utils_i8_i8.h:98-132)
    assert oracle.quantize_multiplier(0.0025) == (1374389535, -8)
    assert oracle.quantize_multiplier(0.0) == (0, 0)


def test_quantize_multiplier_golden(oracle, golden):
    for v, (m, s) in zip(golden["mult_in"], golden["mult_out"]):
        assert oracle.quantize_multiplier(float(v)) == (int(m), int(s)), v


def test_gemm_i32_golden(oracle, golden):
    for idx, (m, n, k, has_c) in enumerate(golden["i8_shapes"]):
        A, Bt, Bn = golden[f"i8_{idx}_A"], golden[f"i8_{idx}_Bt"], golden[f"i8_{idx}_Bn"]
        Cm = golden[f"i8_{idx}_C"] if has_c else None
        assert np.array_equal(oracle.gemm_clamp_i32_i8_i8(A, Bt, True, Cm, (-100000, 100000)), golden[f"i8_{idx}_Dt"])
        assert np.array_equal(oracle.gemm_clamp_i32_i8_i8(A, Bn, False, Cm, (-100000, 100000)), golden[f"i8_{idx}_Dn"])
        assert np.array_equal(oracle.gemm_clamp_i32_i8_i8(A, Bn, False, Cm, (-3000, 2500)), golden[f"i8_{idx}_Dn_narrow"])


def test_quantize_i8_golden(oracle, golden):
    got = np.array([oracle.lib.tqo_quantize_i8(float(v), float(s), int(z))
                    for v, s, z in zip(golden["qi8_val"], golden["qi8_scale"], golden["qi8_zp"])], np.int8)
    assert np.array_equal(got, golden["qi8_out"])


def test_fuse_zp_golden(oracle, golden):
    assert np.array_equal(oracle.fuse_zp_to_bias(golden["fuse_bias"], golden["fuse_data"], 3), golden["fuse_out"])


def test_half_conversions_golden(oracle, golden):
    f = golden["cvt_in"]
    f16 = np.array([oracle.lib.tqo_f32_to_f16(float(x)) for x in f], np.uint16)
    bf16 = np.array([oracle.lib.tqo_f32_to_bf16(float(x)) for x in f], np.uint16)
    assert np.array_equal(f16, golden["cvt_f16"])
    assert np.array_equal(bf16, golden["cvt_bf16"])
    # widening is exact: compare with numpy's for every f16 pattern
    allh = np.arange(65536, dtype=np.uint16)
    want = allh.view(np.float16).astype(np.float32)
    got = np.array([oracle.lib.tqo_f16_to_f32(int(h)) for h in allh], np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


def test_w4a16_golden(oracle, golden):
    for idx, (m, n, k, bl, has_bias, has_c, has_clamp) in enumerate(golden["w4a16_cases"]):
        A, W = golden[f"w4a16_{idx}_A"], golden[f"w4a16_{idx}_W"]
        nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), int(bl))
        assert np.array_equal(nib, golden[f"w4a16_{idx}_nib"])
        assert np.array_equal(sc, golden[f"w4a16_{idx}_scale"])
        for td, tag in ((TD_F16, "f16"), (TD_F32, "f32")):
            Cm = golden[f"w4a16_{idx}_C_{tag}"] if has_c else None
            bias = golden[f"w4a16_{idx}_bias_{tag}"] if has_bias else None
            if td == TD_F16:
                Cm = None if Cm is None else Cm.view(np.uint16)
                bias = None if bias is None else bias.view(np.uint16)
            clamp = (-0.5, 0.5) if has_clamp else ((-65504.0, 65504.0) if td == TD_F16 else (-FMAX, FMAX))
            D = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, int(bl), td, Cm, bias, clamp)
            want = golden[f"w4a16_{idx}_D_{tag}"]
            assert np.array_equal(D.view(np.uint8), want.view(np.uint8)), (idx, tag)


def _w4a8_bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a


def test_w4a8_golden(oracle, golden):
    """The W4A8 quantisers and GEMM restatement against outputs of the reference's own helpers
    (test/gemm/test_gemm_i8_i4_rvv.cpp:36-158, compiled by oracle/Makefile ref), on the suite's shape
    list with its bias / C / clamp options and all three output types, bit for bit."""
    for idx, (m, n, k, has_bias, has_c, has_clamp) in enumerate(golden["w4a8_cases"]):
        A, W = golden[f"w4a8_{idx}_A"], golden[f"w4a8_{idx}_W"]
        q, sa, zp = oracle.quantize_a_per_row_asym(A)
        assert np.array_equal(q, golden[f"w4a8_{idx}_q"])
        assert np.array_equal(sa.view(np.uint32), golden[f"w4a8_{idx}_sa"].view(np.uint32))
        assert np.array_equal(zp, golden[f"w4a8_{idx}_zp"])
        nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
        assert np.array_equal(nib, golden[f"w4a8_{idx}_nib"])
        assert np.array_equal(sb.view(np.uint32), golden[f"w4a8_{idx}_sb"].view(np.uint32))
        clamp = (-0.5, 0.5) if has_clamp else (-FMAX, FMAX)
        for td, tag in ((TD_F32, "f32"), (TD_F16, "f16"), (TD_BF16, "bf16")):
            Cm = golden[f"w4a8_{idx}_C_{tag}"] if has_c else None
            bias = golden[f"w4a8_{idx}_bias_{tag}"] if has_bias else None
            D = oracle.gemm_w4a8(q, nib, sa, zp, sb, td, Cm, bias, clamp)
            assert np.array_equal(_w4a8_bits(D), _w4a8_bits(golden[f"w4a8_{idx}_D_{tag}"])), (idx, tag)


def test_w4a8_quantiser_edge_rows_golden(oracle, golden):
    """All-zero, one-signed, tiny, huge, subnormal and boundary rows through both quantisers."""
    q, sa, zp = oracle.quantize_a_per_row_asym(golden["w4a8_edge_A"])
    assert np.array_equal(q, golden["w4a8_edge_q"])
    assert np.array_equal(sa.view(np.uint32), golden["w4a8_edge_sa"].view(np.uint32))
    assert np.array_equal(zp, golden["w4a8_edge_zp"])
    nib, sb = oracle.quantize_b_per_channel_sym_int4(golden["w4a8_edge_W"])
    assert np.array_equal(nib, golden["w4a8_edge_nib"])
    assert np.array_equal(sb.view(np.uint32), golden["w4a8_edge_sb"].view(np.uint32))


def test_w4a8_live_reference_when_built(oracle):
    """Larger random cases and 16-bit activations against the reference's helpers where oracle/_ref exists."""
    ref = Reference()
    if not ref.has_w4a8():
        pytest.skip("oracle/_ref (with the W4A8 helpers) not built on this machine")
    rng = np.random.default_rng(23)
    for (m, n, k) in [(33, 70, 96), (128, 130, 256), (3, 257, 1024)]:
        A = rng.normal(0, 1, (m, k)).astype(np.float32)
        W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
        q, sa, zp = oracle.quantize_a_per_row_asym(A)
        rq, rsa, rzp = ref.w4a8_quantize_a_per_row_asym(A)
        assert np.array_equal(q, rq) and np.array_equal(sa, rsa) and np.array_equal(zp, rzp)
        nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
        rnib, rsb = ref.w4a8_quantize_b_per_channel_sym_int4(W)
        assert np.array_equal(nib, rnib) and np.array_equal(sb, rsb)
        bias = rng.normal(0, 0.1, n).astype(np.float32)
        Cm = rng.uniform(-2, 2, (m, n)).astype(np.float32)
        for td in (TD_F32, TD_F16, TD_BF16):
            if td == TD_F32:
                b, c = bias, Cm
            elif td == TD_F16:
                b, c = bias.astype(np.float16).view(np.uint16), Cm.astype(np.float16).view(np.uint16)
            else:
                b = np.array([oracle.lib.tqo_f32_to_bf16(float(x)) for x in bias], np.uint16)
                c = np.array([oracle.lib.tqo_f32_to_bf16(float(x)) for x in Cm.ravel()], np.uint16).reshape(m, n)
            for cl in ((-FMAX, FMAX), (-0.25, 0.3)):
                D = oracle.gemm_w4a8(q, nib, sa, zp, sb, td, c, b, cl)
                R = ref.w4a8_gemm(q, nib, sa, zp, sb, td, c, b, cl)
                assert np.array_equal(_w4a8_bits(D), _w4a8_bits(R)), (m, n, k, td, cl)
        # 16-bit activation rows: the oracle widens them (exactly) before the same arithmetic
        a16 = A.astype(np.float16)
        q16, s16, z16 = oracle.quantize_a_per_row_asym(a16.view(np.uint16), TD_F16)
        rq, rsa, rzp = ref.w4a8_quantize_a_per_row_asym(a16.astype(np.float32))
        assert np.array_equal(q16, rq) and np.array_equal(s16, rsa) and np.array_equal(z16, rzp)
        ab = np.array([oracle.lib.tqo_f32_to_bf16(float(x)) for x in A.ravel()[:m * 64]], np.uint16).reshape(m, 64)
        qb, sbb, zb = oracle.quantize_a_per_row_asym(ab, TD_BF16)
        abf = (ab.astype(np.uint32) << 16).view(np.float32)
        rq, rsa, rzp = ref.w4a8_quantize_a_per_row_asym(abf)
        assert np.array_equal(qb, rq) and np.array_equal(sbb, rsa) and np.array_equal(zb, rzp)


def test_seeded_generators_match_the_reference(oracle):
    """tqo_fill_uniform_* reproduce test/common/data_generator.cpp's streams (same engine, seed, distribution)."""
    ref = Reference()
    if not ref.available():
        pytest.skip("oracle/_ref not built on this machine")
    assert np.array_equal(oracle.fill_uniform((7, 33), np.int8, -128, 127, 42), ref.fill_uniform((7, 33), np.int8, -128, 127, 42))
    assert np.array_equal(oracle.fill_uniform((5, 19), np.int8, -50, 50, 123), ref.fill_uniform((5, 19), np.int8, -50, 50, 123))
    assert np.array_equal(oracle.fill_uniform((3, 41), np.int32, -1000, 1000, 7), ref.fill_uniform((3, 41), np.int32, -1000, 1000, 7))
    assert np.array_equal(oracle.fill_uniform((9, 21), np.float32, -1.0, 1.0, 42), ref.fill_uniform((9, 21), np.float32, -1.0, 1.0, 42))


def test_seeded_generators_known_stream(oracle):
    """First draws of the seeded streams, so that a box with another standard library is noticed
    (mt19937 is specified exactly; the distributions' algorithms are the library's)."""
    a = oracle.fill_uniform((1, 4), np.int8, -128, 127, 42).ravel().tolist()
    b = oracle.fill_normal((1, 3), 0.0, 1.0, 42).ravel()
    assert a == KNOWN_I8_SEED42, a
    assert np.allclose(b, KNOWN_NORMAL_SEED42, rtol=0, atol=0), b.tolist()


def test_w4a8_integer_core_against_i32_golden(oracle, golden):
    """The W4A8 restatement has no compilable counterpart; its integer core is pinned by
    unpacking nibbles to int8 and comparing with the pinned int32 GEMM: with scale 1, zero point 0
    the f32 output equals float(acc) exactly while |acc| < 2^24."""
    rng = np.random.default_rng(11)
    for (m, n, k) in [(8, 8, 8), (5, 11, 16), (7, 3, 8), (17, 19, 24), (31, 35, 64), (60, 61, 128)]:
        A = rng.integers(-128, 128, (m, k), dtype=np.int8)
        q = rng.integers(-8, 8, (n, k), dtype=np.int8)
        nib = ((q[:, 0::2] + 8).astype(np.uint8) | ((q[:, 1::2] + 8).astype(np.uint8) << 4)).astype(np.uint8)
        sa = np.ones(m, np.float32)
        zp = np.zeros(m, np.int32)
        sb = np.ones(n, np.float32)
        D = oracle.gemm_w4a8(A, np.ascontiguousarray(nib), sa, zp, sb, TD_F32)
        want = oracle.gemm_clamp_i32_i8_i8(A, np.ascontiguousarray(q), True)
        assert np.array_equal(D, want.astype(np.float32))
        # zero-point correction: acc - zp * rowsum(q)
        zp2 = rng.integers(-128, 128, m).astype(np.int32)
        D2 = oracle.gemm_w4a8(A, np.ascontiguousarray(nib), sa, zp2, sb, TD_F32)
        want2 = want.astype(np.int64) - zp2[:, None].astype(np.int64) * q.sum(1, dtype=np.int64)[None, :]
        assert np.array_equal(D2, want2.astype(np.float32))


def test_w4a8_quantisers_and_epilogue_numpy(oracle):
    """Cross-check of the restated quantisers and float epilogue against an independent numpy
    statement of the formulas in test/gemm/test_gemm_i8_i4_rvv.cpp:40-156."""
    rng = np.random.default_rng(3)
    m, n, k = 17, 19, 24
    A = rng.normal(0, 1, (m, k)).astype(np.float32)
    A[3] = 0.0                 # all-zero row: scale 1, zp 0
    A[4] = np.abs(A[4])        # all-positive row: fmin forced to 0
    W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    W[2] = 0.0
    q, s, z = oracle.quantize_a_per_row_asym(A)
    fmin = np.minimum(A.min(1), 0).astype(np.float32)
    fmax = np.maximum(A.max(1), 0).astype(np.float32)
    s_np = ((fmax - fmin) / np.float32(255.0)).astype(np.float32)
    for r in range(m):
        if s_np[r] == 0:
            assert s[r] == 1.0 and z[r] == 0 and not q[r].any()
            continue
        assert s[r] == s_np[r]
        zp = int(np.clip(np.rint(np.float32(-128.0) - fmin[r] / s_np[r]), -128, 127))
        assert z[r] == zp
        want = np.clip(np.rint(A[r] / s_np[r]) + np.float32(zp), -128, 127).astype(np.int8)
        assert np.array_equal(q[r], want)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    amax = np.abs(W).max(1)
    sb_np = np.where(amax == 0, np.float32(1.0), amax / np.float32(8.0)).astype(np.float32)
    assert np.array_equal(sb, sb_np)
    qw = np.clip(np.rint(W / sb_np[:, None]), -8, 7).astype(np.int32)
    assert np.array_equal(nib & 0xF, (qw[:, 0::2] + 8))
    assert np.array_equal(nib >> 4, (qw[:, 1::2] + 8))
    bias = rng.normal(0, 0.1, n).astype(np.float32)
    Cm = rng.uniform(-2, 2, (m, n)).astype(np.float32)
    D = oracle.gemm_w4a8(q, nib, s, z, sb, TD_F32, Cm, bias, (-0.5, 0.5))
    acc = q.astype(np.int64) @ qw.T.astype(np.int64) - z[:, None].astype(np.int64) * qw.sum(1)[None, :]
    r = (acc.astype(np.float32) * s[:, None]).astype(np.float32) * sb[None, :]
    r = (r + Cm).astype(np.float32)
    r = (r + bias[None, :]).astype(np.float32)
    r = np.clip(r, np.float32(-0.5), np.float32(0.5))
    assert np.array_equal(D, r)
    # bf16 / f16 outputs are the f32 result rounded to nearest even
    Dh = oracle.gemm_w4a8(q, nib, s, z, sb, TD_F16, None, None, (-65504.0, 65504.0))
    Df = oracle.gemm_w4a8(q, nib, s, z, sb, TD_F32)
    assert np.array_equal(Dh, Df.astype(np.float16).view(np.uint16))
    Db = oracle.gemm_w4a8(q, nib, s, z, sb, TD_BF16, None, None, (-65504.0, 65504.0))
    u = Df.view(np.uint32).astype(np.uint64)
    want_b = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(Db, want_b)


def test_requant_tail_semantics(oracle):
    """The integer tail follows the RVV sequence (vmulh, vsra with the low five shift bits, wrapping
    add, two saturating narrows): spot values worked out by hand."""
    f = oracle.lib.tqo_requantize_one
    assert f(400, 1 << 30, 0, 0) == 100           # mulh(400, 2^30) = 100
    assert f(-1, 1 << 30, 0, 0) == -1             # floor, not round-to-zero
    assert f(-400, 1 << 30, 3, 0) == -13          # -100 >> 3 = floor(-12.5)
    assert f(1 << 30, 0x7FFFFFFF, 0, 5) == 127    # saturates
    assert f(-(1 << 30), 0x7FFFFFFF, 0, 5) == -128
    assert f(400, 1 << 30, 32 + 1, 0) == 50       # shift operand uses only its low five bits
    rng = np.random.default_rng(0)
    m, n, k = 9, 19, 23
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    Bt = rng.integers(-127, 128, (n, k), dtype=np.int8)
    bias = rng.integers(-1000, 1000, n).astype(np.int32)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    D = oracle.gemm_reqi32toi8(A, Bt, True, 0.05, sb, 3.0, -5, bias)
    acc = A.astype(np.int64) @ Bt.T.astype(np.int64) + bias[None, :]
    for j in range(n):
        real = float(np.float32(0.05)) * float(sb[j]) / float(np.float32(3.0))
        mult, s = oracle.quantize_multiplier(real)
        sh = (-s - 1) & 31
        t = ((acc[:, j] * mult) >> 32) >> sh
        t = np.clip(t - 5, -128, 127)
        assert np.array_equal(D[:, j], t.astype(np.int8))
    # per-tensor mode shares column 0's multiplier
    D1 = oracle.gemm_reqi32toi8(A, Bt, True, 0.05, sb, 3.0, -5, bias, quant_channel_b=1)
    sb0 = np.full(n, sb[0], np.float32)
    assert np.array_equal(D1, oracle.gemm_reqi32toi8(A, Bt, True, 0.05, sb0, 3.0, -5, bias))


@pytest.mark.parametrize("m,n,k", [(32, 32, 32), (3, 8, 11), (5, 11, 10), (9, 19, 23), (15, 32, 25), (60, 63, 127)])
def test_requant_restatement_passes_the_reference_acceptance_test(oracle, m, n, k):
    """The integer tail of the requantising kernels exists only as RVV instructions in the reference, so its
    restatement cannot be pinned bit for bit ("parity unpinned" for the int8 bit pattern).  What the reference's
    own suite checks of these kernels is checked here of the restatement: same inputs, same criterion, on the
    suite's shape list (test_gemm_i8_i8_rvv.cpp:31-41)."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from tqt_testlib import requant_acceptance_case, requant_acceptance_check
    c = requant_acceptance_case(oracle, m, n, k)
    D = oracle.gemm_reqi32toi8(c["A"], c["B"], True, c["scale_a"], c["scale_b"], c["scale_d"], c["zp_d"], c["bias_fused"])
    requant_acceptance_check(D, c)


def test_live_reference_when_built(oracle):
    ref = Reference()
    if not ref.available():
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(2)
    for v in np.exp(rng.uniform(-40, 10, 3000)):
        assert oracle.quantize_multiplier(float(v)) == ref.quantize_multiplier(float(v))
    A = rng.integers(-128, 128, (33, 70), dtype=np.int8)
    B = rng.integers(-128, 128, (70, 41), dtype=np.int8)
    assert np.array_equal(oracle.gemm_clamp_i32_i8_i8(A, B, False), ref.gemm_i32_i8(A, B, False))
    # every f16 bit pattern round-trips, and a dense sweep of f32 inputs narrows identically
    f = rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    f = f[np.isfinite(f)]
    f = np.concatenate([f, rng.normal(0, 1, 50000).astype(np.float32) * np.float32(1e-6),
                        rng.normal(0, 300, 50000).astype(np.float32) * np.float32(200.0)])
    for x in f[::7]:
        assert oracle.lib.tqo_f32_to_f16(float(x)) == ref.lib.ref_f32_to_f16(float(x)), x
        assert oracle.lib.tqo_f32_to_bf16(float(x)) == ref.lib.ref_f32_to_bf16(float(x)), x


def _conv_cases(golden):
    from tqt_conv_cases import conv_geometry_from_golden
    for idx in range(int(golden["conv_cases"][0])):
        geom, group_idx = conv_geometry_from_golden(golden[f"conv_{idx}_geom"])
        yield idx, geom, group_idx


def test_im2col_golden(oracle, golden):
    """The im2col restatement against outputs of the reference's tqt_im2col_cf / tqt_im2col_cl (src/common/tqt_conv.h:
    52-196, compiled by oracle/Makefile ref) on the shapes of its int8 convolution suite
    (test/conv/test_conv_i8_i8_rvv.cpp:21-41) plus depth, groups and 16-multiple channel counts, both layouts."""
    from tqt_conv_cases import im2col_index
    n = 0
    for idx, geom, group_idx in _conv_cases(golden):
        act = oracle.fill_uniform((int(np.prod(geom.input_shape)) * geom.input_channel,), np.int8, -128, 127, 42)
        for cf, tag in ((False, "cl"), (True, "cf")):
            want = golden[f"conv_{idx}_{tag}"]
            got = oracle.im2col_i8(act, geom, cf, group_idx)
            assert got.shape == want.shape and np.array_equal(got, want), (idx, tag)
            # the vectorised index map the GPU tests build real-valued convolutions with
            ix = im2col_index(geom, cf, group_idx)
            via = np.where(ix >= 0, act[np.maximum(ix, 0)], 0).astype(np.int8)
            assert np.array_equal(via.T if cf else via, want), (idx, tag)
        n += 1
    assert n >= 16


def test_im2col_live_reference_when_built(oracle):
    """Where oracle/_ref carries the reference's im2col, random geometries (depth, groups, stride, dilation, padding)
    through both implementations."""
    from oracle.tqo import ConvGeometry, Reference
    ref = Reference()
    if not (ref.available() and ref.has_conv()):
        pytest.skip("oracle/_ref without the im2col shim on this machine")
    rng = np.random.default_rng(11)
    for _ in range(40):
        groups = int(rng.choice([1, 1, 2, 3]))
        ic = groups * int(rng.integers(1, 7))
        ker = [int(rng.integers(1, 4)) for _ in range(3)]
        dil = [int(rng.integers(1, 3)) for _ in range(3)]
        pad = [int(rng.integers(0, 3)) for _ in range(3)]
        stride = [int(rng.integers(1, 3)) for _ in range(3)]
        shape = [int(rng.integers(dil[i] * (ker[i] - 1) + 1, dil[i] * (ker[i] - 1) + 6)) for i in range(3)]
        geom = ConvGeometry(ic, groups * 2, groups, shape, ker, stride, dil, pad)
        act = rng.integers(-128, 128, int(np.prod(shape)) * ic).astype(np.int8)
        g = int(rng.integers(0, groups))
        for cf in (False, True):
            assert np.array_equal(oracle.im2col_i8(act, geom, cf, g), ref.im2col_i8(act, geom, cf, g))


_FL_TYPES = (("f32", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("bf16", "f32"), ("bf16", "f16"))
_FL_TD = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}


def test_float_gemm_golden(oracle, golden):
    """The unquantised GEMM restatement against the reference's reference_gemm<TA, TD> (test/common/reference_gemm.cpp:
    11-88, compiled by oracle/Makefile ref) for the five type combinations it instantiates, on the float suites' shapes
    with their bias / C / clamp options, B as [n, k] and [k, n], bias per column and per row: bit for bit."""
    checked = 0
    for ta, td in _FL_TYPES:
        for idx, (m, n, k, has_bias, has_c, has_clamp, lo, hi) in enumerate(golden["fl_cases"]):
            m, n, k = int(m), int(n), int(k)
            tag = f"fl_{ta}_{td}_{idx}"
            A, B = golden[tag + "_A"], golden[tag + "_B"]
            Cm = golden[tag + "_C"] if has_c else None
            bias = golden[tag + "_bias"] if has_bias else None
            clamp = (lo, hi) if has_clamp else (-FMAX, FMAX)
            bits = lambda x: x.view(np.uint32) if x.dtype == np.float32 else x
            got = oracle.gemm_float(_FL_TD[ta], _FL_TD[td], A, B, True, Cm, None if bias is None else bias[:n].copy(), False, clamp)
            assert np.array_equal(bits(got), bits(golden[tag + "_Dt"])), tag
            got = oracle.gemm_float(_FL_TD[ta], _FL_TD[td], A, np.ascontiguousarray(B.T), False, Cm,
                                    None if bias is None else bias[:n].copy(), False, clamp)
            assert np.array_equal(bits(got), bits(golden[tag + "_Dn"])), tag
            got = oracle.gemm_float(_FL_TD[ta], _FL_TD[td], A, B, True, Cm, None if bias is None else bias[:m].copy(), True, clamp)
            assert np.array_equal(bits(got), bits(golden[tag + "_Dr"])), tag
            checked += 3
    assert checked == 5 * 9 * 3
