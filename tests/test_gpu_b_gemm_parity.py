"""GPU parity tests of the GEMM kernel types against the CPU oracle, through the C ABI.

Integer outputs (int32, requantised int8) are compared bit for bit.  The W4A8 float epilogue is a
fixed sequence of IEEE f32 operations on an exact int32 accumulator, so it is compared bit for bit
as well (the stated bars, rel 1e-3 for f32 and 2e-2 for f16/bf16, are implied).  W4A16 accumulates
f16 products in f32 in a different order than the oracle: tolerance rel 2e-2 with an RMS floor,
plus the reference's own thresholds (abs 1.0, cosine 0.9999; test/common/test_common.h:47-66).

Each packed kernel type is run on the path run_gemm picks by itself and, through the library's path switch
(tqt_cuda_debug_set_path), on the generic CUDA-core path, so that the tensor-core, GEMV and CUDA-core kernels
check each other.
"""
import numpy as np
import pytest

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import (FMAX, bf16_bits_to_f32, cosine, f16_bits_to_f32, f32_to_bf16_bits, rel_err, requant_acceptance_case,
                         requant_acceptance_check, run_i32_packed, run_i32_unpacked, run_requant, run_w4a16, run_w4a8)

pytestmark = pytest.mark.gpu

TD_CODE = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}
# shape lists of the reference's suites (test_gemm_i8_i8_rvv.cpp:31-41, test_gemm_i8_i4_rvv.cpp:164-179)
I8_SHAPES = [(32, 32, 32), (3, 8, 11), (5, 11, 10), (9, 19, 23), (15, 32, 25), (60, 63, 127)]
W4A8_SHAPES = [(8, 8, 8), (16, 16, 16), (32, 32, 32), (5, 11, 16), (7, 3, 8), (17, 19, 24), (31, 35, 64), (60, 61, 128)]
BIG_SHAPES = [(129, 257, 130), (200, 300, 1000), (256, 512, 512), (300, 130, 384)]
PATHS = ["auto", "simt"]


@pytest.fixture(params=PATHS)
def path(request, force_path):
    force_path(request.param)
    return request.param


# ---- gemm_clamp_i32_i8_i8 (configuration 1) and its packed sibling ---------------------------------
def test_i32_unpacked_golden(golden):
    for idx, (m, n, k, has_c) in enumerate(golden["i8_shapes"]):
        A, Bn = golden[f"i8_{idx}_A"], golden[f"i8_{idx}_Bn"]
        Cm = golden[f"i8_{idx}_C"] if has_c else None
        assert np.array_equal(run_i32_unpacked(A, Bn, Cm, (-100000, 100000)), golden[f"i8_{idx}_Dn"])
        assert np.array_equal(run_i32_unpacked(A, Bn, Cm, (-3000, 2500)), golden[f"i8_{idx}_Dn_narrow"])


def test_i32_unpacked_config1(oracle):
    """M=64, K=512, N=256, int8 uniform in [-128,127], clamp to int32 min/max."""
    rng = np.random.default_rng(42)
    A = rng.integers(-128, 128, (64, 512), dtype=np.int8)
    B = rng.integers(-128, 128, (512, 256), dtype=np.int8)
    assert np.array_equal(run_i32_unpacked(A, B), oracle.gemm_clamp_i32_i8_i8(A, B, False))


def test_i32_packed_golden(golden, path):
    for idx, (m, n, k, has_c) in enumerate(golden["i8_shapes"]):
        A, Bt, Bn = golden[f"i8_{idx}_A"], golden[f"i8_{idx}_Bt"], golden[f"i8_{idx}_Bn"]
        Cm = golden[f"i8_{idx}_C"] if has_c else None
        assert np.array_equal(run_i32_packed(A, Bt, True, Cm, (-100000, 100000)), golden[f"i8_{idx}_Dt"])
        assert np.array_equal(run_i32_packed(A, Bn, False, Cm, (-100000, 100000)), golden[f"i8_{idx}_Dn"])


@pytest.mark.parametrize("m,n,k", BIG_SHAPES + [(64, 256, 512)])
def test_i32_packed_big(oracle, path, m, n, k):
    rng = np.random.default_rng(m + n + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    Bt = rng.integers(-128, 128, (n, k), dtype=np.int8)
    Cm = rng.integers(-100000, 100000, (m, n)).astype(np.int32)
    assert np.array_equal(run_i32_packed(A, Bt, True, Cm, (-900000, 800000)),
                          oracle.gemm_clamp_i32_i8_i8(A, Bt, True, Cm, (-900000, 800000)))


# ---- static W8A8 with int8 requantisation (configuration 4) -------------------------------------------
@pytest.mark.parametrize("m,n,k", I8_SHAPES + BIG_SHAPES)
@pytest.mark.parametrize("scale_d", [0.1, 30.0])
def test_requant_bit_exact(oracle, path, m, n, k, scale_d):
    """scale_d = 0.1 is the configuration's value (most outputs saturate at K = 4096); 30.0 keeps the
    outputs inside the int8 range so that the multiply / shift path is what is compared."""
    rng = np.random.default_rng(m * 3 + n * 5 + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    fused = oracle.fuse_zp_to_bias(bias, W, 3)       # callers fold zero_point_a into the bias
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, scale_d, -5, fused)
    got = run_requant(A, W, 0.05, sb, scale_d, -5, fused)
    assert np.array_equal(got, want)
    if scale_d == 30.0:
        assert (np.abs(want.astype(np.int32)) < 127).mean() > 0.5


@pytest.mark.parametrize("m,n,k", I8_SHAPES + [(200, 300, 1000)])
def test_requant_reference_acceptance(oracle, path, m, n, k):
    """The reference's own test of this kernel type, inputs and criterion (quantized_gemm_test_runner.h:193-306),
    beside the bit-exact comparison with the oracle."""
    c = requant_acceptance_case(oracle, m, n, k)
    got = run_requant(c["A"], c["B"], c["scale_a"], c["scale_b"], c["scale_d"], c["zp_d"], c["bias_fused"])
    requant_acceptance_check(got, c)
    want = oracle.gemm_reqi32toi8(c["A"], c["B"], True, c["scale_a"], c["scale_b"], c["scale_d"], c["zp_d"], c["bias_fused"])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [(2560, 2176, 256), (4096, 4096, 128), (2560, 2304, 130), (300, 1100, 384)])
def test_requant_split_tail_wave(oracle, m, n, k):
    """Launches whose last wave of pair tiles is at most half full run its tiles as two one-block halves each
    (90 tiles with an odd block count, so one half does not exist; 256 tiles; 90 whole; 10 tiles on a grid enlarged to 20
    pairs): every output cell against the oracle."""
    rng = np.random.default_rng(m + n + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 0.02 * np.sqrt(k), -5, bias)
    got = run_requant(A, W, 0.05, sb, 0.02 * np.sqrt(k), -5, bias)
    assert np.array_equal(got, want)


def test_requant_options(oracle, path):
    rng = np.random.default_rng(8)
    m, n, k = 130, 260, 200
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    Cm = rng.integers(-5000, 5000, (m, n)).astype(np.int32)
    # C without bias, narrow clamp, per-tensor scale (quant_channel_b == 1 uses column 0 for all)
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 8.0, 4, None, Cm, (-50, 60), 1)
    got = run_requant(A, W, 0.05, sb, 8.0, 4, None, Cm, (-50, 60), 1)
    assert np.array_equal(got, want)
    # caller-side tile loop with offset helpers: scale_b is indexed from each call's first column
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 8.0, 4, bias)
    got = run_requant(A, W, 0.05, sb, 8.0, 4, bias, tile=(128, 128))
    assert np.array_equal(got, want)


# ---- W4A8 (configurations 2 and 3) ---------------------------------------------------------------------
def _w4a8_case(oracle, rng, m, n, k, td, has_c, has_bias, clamp):
    A = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    W = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    q, sa, zp = oracle.quantize_a_per_row_asym(A)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    Cm = bias = None
    if has_c:
        Cm = rng.uniform(-2, 2, (m, n)).astype(np.float32)
    if has_bias:
        bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    if td == "f16":
        Cm = None if Cm is None else Cm.astype(np.float16).view(np.uint16)
        bias = None if bias is None else bias.astype(np.float16).view(np.uint16)
    elif td == "bf16":
        Cm = None if Cm is None else f32_to_bf16_bits(Cm)
        bias = None if bias is None else f32_to_bf16_bits(bias)
    if clamp is None:
        clamp = (-FMAX, FMAX) if td == "f32" else (-65504.0, 65504.0)
    want = oracle.gemm_w4a8(q, nib, sa, zp, sb, TD_CODE[td], Cm, bias, clamp)
    return q, sa, zp, nib, sb, Cm, bias, clamp, want


@pytest.mark.parametrize("td", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,n,k", W4A8_SHAPES + BIG_SHAPES)
def test_w4a8_shapes(oracle, path, td, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 11 + k)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, m, n, k, td, False, False, None)
    got = run_w4a8(td, q, sa, zp, nib, sb, Cm, bias, clamp)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("td", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("has_c,has_bias,clamp", [(False, True, None), (False, False, (-0.5, 0.5)), (True, False, None),
                                                  (True, True, (-0.5, 0.5))])
@pytest.mark.parametrize("m,n,k", [(32, 32, 32), (17, 19, 24), (140, 270, 256)])
def test_w4a8_options(oracle, path, td, has_c, has_bias, clamp, m, n, k):
    rng = np.random.default_rng(m + n + k + 3 * has_c + 5 * has_bias)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, m, n, k, td, has_c, has_bias, clamp)
    got = run_w4a8(td, q, sa, zp, nib, sb, Cm, bias, clamp)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 11, 16, 17])
@pytest.mark.parametrize("n,k", [(128, 128), (130, 258), (512, 1024), (1000, 384), (4096, 4096), (8, 128), (24, 256), (5000, 640)])
def test_w4a8_decode_gemv(oracle, m, n, k):
    """m <= 16 takes the HBM-streaming GEMV (17 is the first tensor-core size); the integer combine makes it
    bit-exact like the GEMM.  Column counts that are not multiples of 16 leave the last CTA half a set."""
    rng = np.random.default_rng(m * 100 + n + k)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, m, n, k, "f32", m % 2 == 0, True, None)
    got = run_w4a8("f32", q, sa, zp, nib, sb, Cm, bias, clamp)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("td", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (7, 520, 384), (16, 1000, 512), (12, 14336, 256)])
def test_w4a8_decode_gemv_forced(oracle, force_path, td, m, n, k):
    """The GEMV forced through the path switch (so that nothing falls through to the GEMM), 16-bit outputs,
    a column count whose 8-column groups need more than one round of CTAs."""
    force_path("gemv")
    rng = np.random.default_rng(m + n + k)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, m, n, k, td, m % 2 == 1, True, (-0.75, 0.5))
    got = run_w4a8(td, q, sa, zp, nib, sb, Cm, bias, clamp)
    assert np.array_equal(got, want)


def test_w4a8_decode_on_the_tensor_core_path(oracle, force_path):
    force_path("umma")
    rng = np.random.default_rng(77)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, 3, 300, 512, "bf16", False, True, None)
    assert np.array_equal(run_w4a8("bf16", q, sa, zp, nib, sb, Cm, bias, clamp), want)


def test_w4a8_tile_portions(oracle, path):
    """A caller may compute any sub-rectangle whose origin is a multiple of (m_step, n_step); the params
    arrays are indexed from the call's origin, so it passes offset pointers."""
    rng = np.random.default_rng(5)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, 300, 520, 256, "bf16", True, True, None)
    for tile in ((128, 128), (256, 384), (128, 512)):
        got = run_w4a8("bf16", q, sa, zp, nib, sb, Cm, bias, clamp, tile=tile)
        assert np.array_equal(got, want), tile


# ---- W4A16 (configuration 5) -----------------------------------------------------------------------------
def _check_w4a16(got, want, td):
    g = f16_bits_to_f32(got) if td == "f16" else got
    w = f16_bits_to_f32(want) if td == "f16" else want
    assert rel_err(g, w) <= 2e-2                     # the stated bar, RMS floor against 0/0
    assert np.max(np.abs(g - w)) <= 1.0 and cosine(g, w) >= 0.9999   # the reference's own thresholds


def test_w4a16_golden(golden, path):
    for idx, (m, n, k, bl, has_bias, has_c, has_clamp) in enumerate(golden["w4a16_cases"]):
        A = golden[f"w4a16_{idx}_A"].view(np.uint16)
        nib, sc = golden[f"w4a16_{idx}_nib"], golden[f"w4a16_{idx}_scale"]
        for td in ("f16", "f32"):
            Cm = golden[f"w4a16_{idx}_C_{td}"] if has_c else None
            bias = golden[f"w4a16_{idx}_bias_{td}"] if has_bias else None
            if td == "f16":
                Cm = None if Cm is None else Cm.view(np.uint16)
                bias = None if bias is None else bias.view(np.uint16)
            clamp = (-0.5, 0.5) if has_clamp else None
            got = run_w4a16(td, A, nib, sc, int(bl), Cm, bias, clamp)
            want = golden[f"w4a16_{idx}_D_{td}"]
            _check_w4a16(got, want.view(np.uint16) if td == "f16" else want, td)


@pytest.mark.parametrize("m,n,k,bl", [(129, 257, 192, 32), (256, 512, 512, 32), (200, 300, 448, 64), (130, 140, 256, 128),
                                      (70, 260, 320, 8)])
def test_w4a16_big(oracle, path, m, n, k, bl):
    rng = np.random.default_rng(m + n + k + bl)
    A = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    bias = rng.normal(0, 0.1, n).astype(np.float16).view(np.uint16)
    want = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_F16, None, bias)
    got = run_w4a16("f16", A.view(np.uint16), nib, sc, bl, None, bias)
    _check_w4a16(got, want, "f16")


# ---- the two tensor-core kernels against each other and the oracle ---------------------------------------
@pytest.fixture(params=["single", "pair"])
def umma_variant(request, force_path):
    """Forces the single-CTA or the CTA-pair (cta_group::2) kernel whatever the shape."""
    force_path("umma", request.param)
    return request.param


@pytest.mark.parametrize("m,n,k", I8_SHAPES + BIG_SHAPES + [(512, 384, 640), (1000, 1000, 264)])
def test_i8_kernels_forced(oracle, umma_variant, m, n, k):
    rng = np.random.default_rng(m + 2 * n + 3 * k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-128, 128, (n, k), dtype=np.int8)
    Cm = rng.integers(-100000, 100000, (m, n)).astype(np.int32)
    assert np.array_equal(run_i32_packed(A, W, True, Cm, (-2**31, 2**31 - 1)), oracle.gemm_clamp_i32_i8_i8(A, W, True, Cm))
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 20.0, -5, bias)
    assert np.array_equal(run_requant(A, W, 0.05, sb, 20.0, -5, bias), want)


@pytest.fixture(params=["single", "pair", "ts"])
def w4a8_variant(request, force_path):
    """single: weights expanded in shared memory; pair / ts: weights expanded into tensor memory, on a
    CTA pair or on one CTA."""
    force_path("umma", request.param)
    return request.param


@pytest.mark.parametrize("td", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,n,k", W4A8_SHAPES[3:] + BIG_SHAPES + [(192, 256, 128), (193, 257, 384), (500, 640, 1152), (97, 128, 256)])
def test_w4a8_kernels_forced(oracle, w4a8_variant, td, m, n, k):
    rng = np.random.default_rng(m * 5 + n * 3 + k)
    q, sa, zp, nib, sb, Cm, bias, clamp, want = _w4a8_case(oracle, rng, m, n, k, td, m % 2 == 1, True, None)
    got = run_w4a8(td, q, sa, zp, nib, sb, Cm, bias, clamp)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k,bl", [(129, 257, 192, 32), (256, 512, 512, 32), (200, 300, 448, 64), (130, 140, 256, 128),
                                      (70, 260, 320, 8), (192, 128, 64, 2), (400, 384, 1088, 32), (33, 19, 24, 4)])
def test_w4a16_kernels_forced(oracle, w4a8_variant, m, n, k, bl):
    """W4A16 on the three tensor-core kernels (weights expanded in shared memory / in tensor memory on a
    CTA pair / in tensor memory on one CTA); odd numbers of 64-element K steps included."""
    rng = np.random.default_rng(m + n + k + bl)
    A = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    bias = rng.normal(0, 0.1, n).astype(np.float16).view(np.uint16)
    Cm = rng.normal(0, 1, (m, n)).astype(np.float16).view(np.uint16) if m % 2 else None
    want = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_F16, Cm, bias)
    got = run_w4a16("f16", A.view(np.uint16), nib, sc, bl, Cm, bias)
    _check_w4a16(got, want, "f16")
    want32 = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_F32, None, None, (-FMAX, FMAX))
    got32 = run_w4a16("f32", A.view(np.uint16), nib, sc, bl, None, None)
    _check_w4a16(got32, want32, "f32")


@pytest.mark.parametrize("m,n", [(2048, 1792), (1500, 2600), (400, 7700)])
def test_w4a8_wide_tile_single_wave(oracle, m, n):
    """Shapes for which 192-row activation tiles need a second wave on 74 CTA pairs and 256-row tiles do
    not (the per-GPU shape of the prefill config sharded 8 ways among them): the CTA-pair kernel then runs
    one 256 x 256 tile per pair on a single accumulator.  Ragged last tiles included."""
    k = 256
    rng = np.random.default_rng(m + n)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    bias = f32_to_bf16_bits(rng.normal(0, 0.1, n).astype(np.float32))
    want = oracle.gemm_w4a8(A, nib, sa, zp, sb, TD_BF16, None, bias, (-65504.0, 65504.0))
    got = run_w4a8("bf16", A, sa, zp, nib, sb, None, bias)
    assert np.array_equal(got, want)


def test_w4a16_wide_tile_single_wave(oracle):
    m, n, k, bl = 2048, 1792, 128, 32
    rng = np.random.default_rng(77)
    A = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    want = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_F16, None, None)
    got = run_w4a16("f16", A.view(np.uint16), nib, sc, bl, None, None)
    assert rel_err(f16_bits_to_f32(got), f16_bits_to_f32(want)) < 2e-2
