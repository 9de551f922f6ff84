"""Parity of the sibling kernel types (include/tqt_b200_gemm_siblings.h) against the oracle: the
unpacked ("t" layout) W4A8 / W4A16 / W8A8 types, the packed dynamic-activation W8A8 types with float
output and the Mx1-bias requantising types.  Integer and W4A8 outputs bit-exact; W4A16 within 2e-2.
Shapes are ragged on purpose; one case per family is driven as a tile-portion call through the offset
helpers, with the params arrays offset to the call's origin as the reference's callers do."""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import DEV, FMAX, bits16, f16_bits_to_f32, from_bits16, pkg, rel_err, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

TD_ID = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}
TD_TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
SHAPES = [(5, 7, 16), (64, 96, 128), (130, 257, 194), (33, 140, 1026), (300, 520, 640)]


def _as_td(x, td):
    """numpy float32 -> (device tensor of type td, its bit/np representation for the oracle)."""
    t = torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(TD_TORCH[td])
    return t, (t.cpu().numpy() if td == "f32" else bits16(t))


def _out(d, td):
    return d.cpu().numpy() if td == "f32" else bits16(d)


@pytest.mark.parametrize("td", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_w4a8_unpacked(oracle, td, m, n, k):
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m * 31 + n + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    bias_d, bias_o = _as_td(rng.normal(0, 0.1, n).astype(np.float32), td)
    c_d, c_o = _as_td(rng.normal(0, 1, (m, n)).astype(np.float32), td) if m % 2 else (None, None)
    clamp = (-FMAX, FMAX) if td == "f32" else (-65504.0, 65504.0)
    want = oracle.gemm_w4a8(A, nib, sa, zp, sb, TD_ID[td], c_o, bias_o, clamp)
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_qai8dx_qsi4cxt")
    a_d, b_d, sa_d, zp_d, sb_d = to_dev(A), to_dev(nib), to_dev(sa), to_dev(zp), to_dev(sb)
    d = torch.full((m, n), 7.0, dtype=TD_TORCH[td], device=DEV)
    params = p.QaI8DxQsI4CxParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    uk.run_gemm(m, n, k, a_d, k, 0, b_d, k, 0, c_d, n, d, n, bias_d, clamp[0], clamp[1], params)
    sync_and_check()
    assert np.array_equal(_out(d, td), want)


def test_w4a8_unpacked_tile_portion(oracle):
    """Rows [128, m) x columns [128, n) of a larger problem through the offset helpers (lda > k)."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(8)
    m, n, k, lda = 200, 300, 130, 160
    A_full = rng.integers(-128, 128, (m, lda), dtype=np.int8)
    A = np.ascontiguousarray(A_full[:, :k])
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    bias = rng.normal(0, 0.1, n).astype(np.float32)
    want = oracle.gemm_w4a8(A, nib, sa, zp, sb, TD_F32, None, bias, (-FMAX, FMAX))
    uk = p.SiblingGemm("gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt")
    a_d, b_d, sa_d, zp_d, sb_d, bias_d = to_dev(A_full), to_dev(nib), to_dev(sa), to_dev(zp), to_dev(sb), to_dev(bias)
    d = torch.full((m, n), 7.0, dtype=torch.float32, device=DEV)
    m0, n0 = 128, 128
    params = p.QaI8DxQsI4CxParams(sa_d.data_ptr() + 4 * m0, zp_d.data_ptr() + 4 * m0, sb_d.data_ptr() + 4 * n0)
    uk.run_gemm(m - m0, n - n0, k, a_d.data_ptr() + uk.get_a_offset(m0, 0, lda), lda, 0,
                b_d.data_ptr() + uk.get_b_offset(n0, 0, k), k, 0, None, n,
                d.data_ptr() + uk.get_d_offset(m0, n0, n), n, bias_d.data_ptr() + uk.get_bias_offset(n0),
                -FMAX, FMAX, params)
    sync_and_check()
    got = d.cpu().numpy()
    assert np.array_equal(got[m0:, n0:], want[m0:, n0:])
    assert np.all(got[:m0] == 7.0) and np.all(got[:, :n0] == 7.0)


@pytest.mark.parametrize("b_packed", [False, True])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_requant_1xn_unpacked_a(oracle, b_packed, m, n, k):
    """gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cx{t,p}: A [m,k]; B [n,k] as is, or packed."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n * 3 + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1000, n).astype(np.int32)
    Cm = rng.integers(-5000, 5000, (m, n)).astype(np.int32) if n % 2 else None
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 0.1 * np.sqrt(k / 64.0), -5, bias, Cm)
    uk = p.SiblingGemm("gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cx" + ("p" if b_packed else "t"))
    a_d, w_d, sb_d, bias_d = to_dev(A), to_dev(W), to_dev(sb), to_dev(bias)
    c_d = None if Cm is None else to_dev(Cm)
    if b_packed:
        b_arg = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_bt_pack(n, k, k, k, 0, w_d, b_arg)
    else:
        b_arg = w_d
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    params = p.QaI8QaI8QsI8CxParams(0.05, 3, sb_d.data_ptr(), 0, float(np.float32(0.1 * np.sqrt(k / 64.0))), -5)
    uk.run_gemm(m, n, k, a_d, k, 0, b_arg, k, 0, c_d, n, d, n, bias_d, -128, 127, params)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), want)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("per_tensor", [False, True])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_requant_mx1(oracle, packed, per_tensor, m, n, k):
    """gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx[p]_qai8[p]: per-row scale of A, bias per row."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m * 7 + n + k + packed)
    A = rng.integers(-127, 128, (m, k), dtype=np.int8)
    B = rng.integers(-128, 128, (k, n), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, m).astype(np.float32)
    bias = rng.integers(-1000, 1000, m).astype(np.int32)
    sd = float(np.float32(0.05 * np.sqrt(k / 64.0)))
    want = oracle.gemm_mx1bias_reqi32toi8(A, B, sa, 0.04, sd, 7, bias, None, (-100, 110), 1 if per_tensor else m)
    uk = p.SiblingGemm("gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx" + ("p_qai8p" if packed else "_qai8"))
    a_d, b_d, sa_d, bias_d = to_dev(A), to_dev(B), to_dev(sa), to_dev(bias)
    if packed:
        a_arg = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
        b_arg = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_a_pack(m, k, k, k, 0, a_d, a_arg)
        uk.run_b_pack(n, k, n, k, 0, b_d, b_arg)
        lda, ldb = k, k
    else:
        a_arg, b_arg, lda, ldb = a_d, b_d, k, n
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    params = p.QaI8QsI8DxQaI8Params(sa_d.data_ptr(), 1 if per_tensor else m, 0.04, 2, sd, 7)
    uk.run_gemm(m, n, k, a_arg, lda, 0, b_arg, ldb, 0, None, n, d, n, bias_d, -100, 110, params)
    sync_and_check()
    assert np.array_equal(d.cpu().numpy(), want)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("td", ["f32", "f16"])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_qai8dx_qsi8cx_float_out(oracle, packed, td, m, n, k):
    """gemm_1xnbias_clamp_{f32,f16}_qai8dx[p]_qsi8cx{t,p}: C is ignored, f16 adds the bias in f16."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n + k * 5)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias_d, bias_o = _as_td(rng.normal(0, 0.5, n).astype(np.float32), td)
    clamp = (-3.0, 2.5)
    want = oracle.gemm_qai8dx_qsi8cx(A, W, True, sa, zp, sb, TD_ID[td], bias_o, clamp)
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_qai8dx" + ("p_qsi8cxp" if packed else "_qsi8cxt"))
    a_d, w_d, sa_d, zp_d, sb_d = to_dev(A), to_dev(W), to_dev(sa), to_dev(zp), to_dev(sb)
    if packed:
        a_arg = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
        b_arg = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_a_pack(m, k, k, k, 0, a_d, a_arg)
        uk.run_bt_pack(n, k, k, k, 0, w_d, b_arg)
    else:
        a_arg, b_arg = a_d, w_d
    junk_c = torch.full((m, n), 1000.0, dtype=TD_TORCH[td], device=DEV)   # must not be added
    d = torch.full((m, n), 7.0, dtype=TD_TORCH[td], device=DEV)
    params = p.QaI8DxpQsI8CxpParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    uk.run_gemm(m, n, k, a_arg, k, 0, b_arg, k, 0, junk_c, n, d, n, bias_d, clamp[0], clamp[1], params)
    sync_and_check()
    assert np.array_equal(_out(d, td), want)


@pytest.mark.parametrize("td", ["f16", "f32"])
@pytest.mark.parametrize("m,n,k,bl", [(5, 7, 16, 2), (64, 96, 128, 32), (130, 257, 192, 64), (33, 140, 1024, 128)])
def test_w4a16_unpacked(oracle, td, m, n, k, bl):
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n + k + bl)
    A = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    bias = rng.normal(0, 0.1, n).astype(np.float16 if td == "f16" else np.float32)
    bias_o = bias.view(np.uint16) if td == "f16" else bias
    clamp = (-65504.0, 65504.0) if td == "f16" else (-FMAX, FMAX)
    want = oracle.gemm_w4a16(A.view(np.uint16), nib, sc, bl, TD_ID[td], None, bias_o, clamp)
    uk = p.SiblingGemm(f"gemm_1xnbias_clamp_{td}_f16_qsi4c2t")
    a_d, b_d, sc_d = to_dev(A.view(np.uint16)), to_dev(nib), to_dev(sc)
    bias_d = to_dev(bias_o)
    d = torch.full((m, n), 7.0, dtype=TD_TORCH[td], device=DEV)
    uk.run_gemm(m, n, k, a_d, k, 0, b_d, k, 0, None, n, d, n, bias_d, clamp[0], clamp[1], bl=bl, scale_b=sc_d,
                ldsb=k // bl)
    sync_and_check()
    got = d.float().cpu().numpy()
    ref = f16_bits_to_f32(want) if td == "f16" else want
    assert rel_err(got, ref) < 2e-2


def test_sibling_null_params_is_silent():
    p = pkg()
    uk = p.SiblingGemm("gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8")
    d = torch.full((4, 4), 9, dtype=torch.int8, device=DEV)
    a = torch.zeros((4, 8), dtype=torch.int8, device=DEV)
    uk.run_gemm(4, 4, 8, a, 8, 0, a, 4, 0, None, 4, d, 4, None, -128, 127, None)
    sync_and_check()
    assert torch.all(d == 9)
