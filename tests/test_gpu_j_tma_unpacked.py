"""int8 x int8 kernel types whose operands stay in the caller's row-major layouts: with base addresses and row
strides that are multiples of 16 bytes they run on the tcgen05 CTA-pair kernel, each stage fetched by tiled TMA loads
through tensor maps (K-major boxes for A [m, lda] and B^T [n, ldb], MN-major boxes for B [k, ldb]); anything a tensor map
cannot describe runs on the generic CUDA-core kernel.  Both are bit-exact against the oracle, and the test checks
which kernel family ran."""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import DEV, FMAX, bits16, cosine, f16_bits_to_f32, pkg, rel_err, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

SIMT, PAIR_BLOCKS, PAIR_TMA, TS_TMA = 1, 2, 3, 4
# (m, n, k, lda - k, ldb - rows): ragged in every dimension, odd block counts (a whole box beyond the matrix),
# several K blocks, padding columns behind k / n that hold other data
SHAPES = [(64, 256, 512, 0, 0), (5, 7, 16, 0, 9), (130, 257, 194, 14, 15), (33, 140, 1026, 6, 4), (300, 520, 640, 0, 8),
          (700, 390, 1100, 20, 10), (129, 128, 128, 16, 16)]


def _padded(rng, rows, cols, pad):
    """A [rows, cols + pad] int8 matrix; the operand is its first ``cols`` columns."""
    full = rng.integers(-128, 128, (rows, cols + pad), dtype=np.int8)
    return full, np.ascontiguousarray(full[:, :cols])


def _aligned(ld):
    return ld % 16 == 0


@pytest.mark.parametrize("m,n,k,pa,pb", SHAPES)
def test_i32_unpacked(oracle, m, n, k, pa, pb):
    """gemm_clamp_i32_i8_i8: A [m, lda], B [k, ldb] (n contiguous: an MN-major operand)."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    A_full, A = _padded(rng, m, k, pa)
    B_full, B = _padded(rng, k, n, pb)
    Cm = rng.integers(-1000, 1000, (m, n), dtype=np.int32) if m % 2 else None
    uk = p.GemmClampI32I8I8()
    d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    uk.run_gemm(m, n, k, to_dev(A_full), k + pa, 0, to_dev(B_full), n + pb, 0, None if Cm is None else to_dev(Cm), n, d, n,
                -3000000, 2500000)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), oracle.gemm_clamp_i32_i8_i8(A, B, False, Cm, (-3000000, 2500000)))
    assert p.debug_last_kernel() == (PAIR_TMA if _aligned(k + pa) and _aligned(n + pb) else SIMT)


def _requant_inputs(rng, n):
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1000, n, dtype=np.int32)
    return sb, bias


@pytest.mark.parametrize("b_packed", [False, True])
@pytest.mark.parametrize("m,n,k,pa,pb", SHAPES)
def test_requant_unpacked(oracle, m, n, k, pa, pb, b_packed):
    """1xN-bias requantising GEMM with A [m, lda] and B^T [n, ldb] (K-major both), or B packed."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + 5 * n + 11 * k)
    A_full, A = _padded(rng, m, k, pa)
    W_full, W = _padded(rng, n, k, pb)
    sb, bias = _requant_inputs(rng, n)
    Cm = rng.integers(-500, 500, (m, n), dtype=np.int32) if n % 2 else None
    scale_d = 0.02 * np.sqrt(k)
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, scale_d, -5, bias, Cm)
    uk = p.SiblingGemm("gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cx" + ("p" if b_packed else "t"))
    sb_d = to_dev(sb)
    params = p.QaI8QaI8QsI8CxParams(0.05, 0, sb_d.data_ptr(), n, scale_d, -5)
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    if b_packed:
        b_dev = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_bt_pack(n, k, k + pb, k, 0, to_dev(W_full), b_dev)
        ldb = k
    else:
        b_dev, ldb = to_dev(W_full), k + pb
    uk.run_gemm(m, n, k, to_dev(A_full), k + pa, 0, b_dev, ldb, 0, None if Cm is None else to_dev(Cm), n, d, n, to_dev(bias),
                -128, 127, params)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), want)
    tma = _aligned(k + pa) and (b_packed or _aligned(k + pb))
    assert p.debug_last_kernel() == (PAIR_TMA if tma else SIMT)


@pytest.mark.parametrize("m,n,k,pa,pb", SHAPES)
def test_requant_rows_unpacked(oracle, m, n, k, pa, pb):
    """Mx1-bias requantising GEMM: A [m, lda] with per-row scales, B [k, ldb] (MN-major)."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + 13 * n + 17 * k)
    A_full, A = _padded(rng, m, k, pa)
    B_full, B = _padded(rng, k, n, pb)
    sa = rng.uniform(0.001, 0.01, m).astype(np.float32)
    bias = rng.integers(-1000, 1000, m, dtype=np.int32)
    scale_d = 0.02 * np.sqrt(k)
    want = oracle.gemm_mx1bias_reqi32toi8(A, B, sa, 0.05, scale_d, 3, bias)
    uk = p.SiblingGemm("gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8")
    sa_d = to_dev(sa)
    params = p.QaI8QsI8DxQaI8Params(sa_d.data_ptr(), m, 0.05, 0, scale_d, 3)
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    uk.run_gemm(m, n, k, to_dev(A_full), k + pa, 0, to_dev(B_full), n + pb, 0, None, n, d, n, to_dev(bias), -128, 127, params)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), want)
    assert p.debug_last_kernel() == (PAIR_TMA if _aligned(k + pa) and _aligned(n + pb) else SIMT)


@pytest.mark.parametrize("td", ["f32", "f16"])
@pytest.mark.parametrize("m,n,k,pa,pb", SHAPES)
def test_dynamic_activation_float_out_unpacked(oracle, td, m, n, k, pa, pb):
    """gemm_1xnbias_clamp_{f32,f16}_qai8dx_qsi8cxt: A [m, lda], B^T [n, ldb]; the zero-point correction needs the row
    sums of B, which the epilogue adds up from the row-major matrix."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + 19 * n + 23 * k)
    A_full, A = _padded(rng, m, k, pa)
    W_full, W = _padded(rng, n, k, pb)
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    tdt = torch.float32 if td == "f32" else torch.float16
    bias_d = to_dev(rng.normal(0, 0.5, n).astype(np.float32)).to(tdt)
    bias_o = bias_d.cpu().numpy() if td == "f32" else bits16(bias_d)
    want = oracle.gemm_qai8dx_qsi8cx(A, W, True, sa, zp, sb, TD_F32 if td == "f32" else TD_F16, bias_o, (-3.0, 2.5))
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_qai8dx_qsi8cxt")
    sa_d, zp_d, sb_d = to_dev(sa), to_dev(zp), to_dev(sb)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)
    params = p.QaI8DxpQsI8CxpParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    uk.run_gemm(m, n, k, to_dev(A_full), k + pa, 0, to_dev(W_full), k + pb, 0, None, n, d, n, bias_d, -3.0, 2.5, params)
    sync_and_check()
    got = d.cpu().numpy() if td == "f32" else bits16(d)
    assert np.array_equal(got, want)
    assert p.debug_last_kernel() == (PAIR_TMA if _aligned(k + pa) and _aligned(k + pb) else SIMT)


# (m, n, k, lda - k, ldb - k): k even; the nibble matrix has ldb / 2 bytes per row
W4_SHAPES = [(5, 7, 16, 0, 16), (64, 96, 128, 0, 0), (130, 257, 194, 14, 30), (33, 140, 1026, 6, 4), (300, 520, 640, 16, 32),
             (200, 260, 96, 0, 0), (450, 390, 1100, 20, 20)]


@pytest.mark.parametrize("td", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,n,k,pa,pb", W4_SHAPES)
def test_w4a8_unpacked(oracle, td, m, n, k, pa, pb):
    """gemm_1xnbias_clamp_{f32,f16,bf16}_qai8dx_qsi4cxt: A int8 [m, lda], B nibbles [n, ldb / 2 bytes] in the reference's
    unpacked encoding; tiled TMA loads feed the tensor-memory kernel, whose converters decode that nibble order and add
    up the row sums.  Bit-exact like the packed types."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m * 31 + n + k)
    A_full, A = _padded(rng, m, k, pa)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    nib_full = rng.integers(0, 256, (n, (k + pb) // 2), dtype=np.uint8)
    nib_full[:, :k // 2] = nib
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[td]
    tdi = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}[td]
    bias_d = to_dev(rng.normal(0, 0.1, n).astype(np.float32)).to(tdt)
    bias_o = bias_d.cpu().numpy() if td == "f32" else bits16(bias_d)
    c_d = to_dev(rng.normal(0, 1, (m, n)).astype(np.float32)).to(tdt) if m % 2 else None
    c_o = None if c_d is None else (c_d.cpu().numpy() if td == "f32" else bits16(c_d))
    clamp = (-FMAX, FMAX) if td == "f32" else (-65504.0, 65504.0)
    want = oracle.gemm_w4a8(A, nib, sa, zp, sb, tdi, c_o, bias_o, clamp)
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_qai8dx_qsi4cxt")
    sa_d, zp_d, sb_d = to_dev(sa), to_dev(zp), to_dev(sb)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)
    params = p.QaI8DxQsI4CxParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    uk.run_gemm(m, n, k, to_dev(A_full), k + pa, 0, to_dev(nib_full), k + pb, 0, c_d, n, d, n, bias_d, clamp[0], clamp[1], params)
    sync_and_check()
    got = d.cpu().numpy() if td == "f32" else bits16(d)
    assert np.array_equal(got, want)
    tma = _aligned(k + pa) and _aligned((k + pb) // 2)
    assert p.debug_last_kernel() == (TS_TMA if tma else SIMT)


@pytest.mark.parametrize("td", ["f16", "f32"])
@pytest.mark.parametrize("m,n,k,bl,pa,pb", [(5, 7, 16, 2, 0, 16), (64, 96, 128, 32, 0, 0), (130, 257, 192, 64, 8, 64),
                                            (33, 140, 1024, 128, 0, 0), (300, 390, 640, 32, 24, 32), (200, 130, 200, 8, 0, 24)])
def test_w4a16_unpacked(oracle, td, m, n, k, bl, pa, pb):
    """gemm_1xnbias_clamp_{f16,f32}_f16_qsi4c2t: A f16 [m, lda], B nibbles [n, ldb / 2 bytes], scale_b f16 [n, k / bl]."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n + k + bl)
    A_full = rng.normal(0, 1, (m, k + pa)).astype(np.float16)
    A = np.ascontiguousarray(A_full[:, :k])
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    nib_full = rng.integers(0, 256, (n, (k + pb) // 2), dtype=np.uint8)
    nib_full[:, :k // 2] = nib
    bias = rng.normal(0, 0.1, n).astype(np.float16 if td == "f16" else np.float32)
    bias_o = bias.view(np.uint16) if td == "f16" else bias
    clamp = (-65504.0, 65504.0) if td == "f16" else (-FMAX, FMAX)
    want = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_F16 if td == "f16" else TD_F32, None, bias_o, clamp)
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_f16_qsi4c2t")
    d = torch.full((m, n), 7.0, dtype=torch.float16 if td == "f16" else torch.float32, device=DEV)
    uk.run_gemm(m, n, k, to_dev(A_full.view(np.uint16)), k + pa, 0, to_dev(nib_full), k + pb, 0, None, n, d, n, to_dev(bias_o),
                clamp[0], clamp[1], bl=bl, scale_b=to_dev(sc), ldsb=k // bl)
    sync_and_check()
    got = d.float().cpu().numpy()
    ref = f16_bits_to_f32(want) if td == "f16" else want
    assert rel_err(got, ref) < 2e-2
    assert np.max(np.abs(got - ref)) <= 1.0 and cosine(got, ref) >= 0.9999
    tma = _aligned(2 * (k + pa)) and _aligned((k + pb) // 2)
    assert p.debug_last_kernel() == (TS_TMA if tma else SIMT)


def test_unaligned_base_falls_back(oracle):
    """A base address off the 16-byte grid cannot be a tensor map: the generic kernel takes the call."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(5)
    m, n, k = 70, 64, 160
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    B = rng.integers(-128, 128, (k, n), dtype=np.int8)
    buf = torch.zeros(m * k + 16, dtype=torch.int8, device=DEV)
    buf[3:3 + m * k] = to_dev(A).reshape(-1)
    d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    p.GemmClampI32I8I8().run_gemm(m, n, k, buf.data_ptr() + 3, k, 0, to_dev(B), n, 0, None, n, d, n, -2**31, 2**31 - 1)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), oracle.gemm_clamp_i32_i8_i8(A, B, False))
    assert p.debug_last_kernel() == SIMT


def test_forced_generic_kernel_agrees(oracle, force_path):
    """TQT_B200_PATH=simt keeps the generic kernel for an aligned call: same bits from both kernels."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(6)
    m, n, k = 200, 272, 384
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    B = rng.integers(-128, 128, (k, n), dtype=np.int8)
    outs = []
    for path, fam in (("simt", SIMT), (None, PAIR_TMA)):
        force_path(path, None)
        d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
        p.GemmClampI32I8I8().run_gemm(m, n, k, to_dev(A), k, 0, to_dev(B), n, 0, None, n, d, n, -2**31, 2**31 - 1)
        sync_and_check()
        assert p.debug_last_kernel() == fam
        outs.append(d.cpu().numpy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], oracle.gemm_clamp_i32_i8_i8(A, B, False))
