"""The int8 convolution wrappers (include/tqt_b200_conv_i8_i8.h): im2col kernels against the golden outputs of the
reference's tqt_im2col_cf / tqt_im2col_cl, and whole convolutions driven the way the reference's runners drive them
(test/common/quantized_conv_test_runner.h), bit-exact against the oracle's requantising GEMMs on the oracle's im2col
matrix and within the reference's own acceptance thresholds of the real-valued convolution."""
import numpy as np
import pytest
import torch

from tqt_conv_cases import conv_acceptance_case, conv_geometry_from_golden
from tqt_testlib import DEV, cosine, pkg, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

N_CASES = 16
CL_PACKED, CL_PLAIN, CF_PLAIN, CF_PACKED = range(4)


def _params(p, geom):
    return p.ConvParams.make(geom.input_channel, geom.output_channel, geom.groups, geom.input_shape, geom.kernel_shape,
                             geom.stride, geom.dilation, geom.pad, geom.output_shape)


def _activation(oracle, geom):
    return oracle.fill_uniform((int(np.prod(geom.input_shape)) * geom.input_channel,), np.int8, -128, 127, 42)


@pytest.mark.parametrize("idx", range(N_CASES))
def test_im2col_plain_against_the_reference(oracle, golden, idx):
    p = pkg()
    p.use_current_torch_stream()
    geom, group_idx = conv_geometry_from_golden(golden[f"conv_{idx}_geom"])
    act = to_dev(_activation(oracle, geom))
    cp = _params(p, geom)
    for type_idx, tag in ((CL_PLAIN, "cl"), (CF_PLAIN, "cf")):
        uk = p.ConvI8(p.CONV_TYPES[type_idx])
        want = golden[f"conv_{idx}_{tag}"]
        size = uk.get_b_im2col_size(geom.k, geom.rows) if uk.channel_first else uk.get_a_im2col_size(geom.rows, geom.k)
        assert size == want.size
        buf = torch.full((size,), 77, dtype=torch.int8, device=DEV)
        uk.run_im2col(group_idx, act, buf, cp)
        sync_and_check()
        assert np.array_equal(buf.cpu().numpy().reshape(want.shape), want)


@pytest.mark.parametrize("idx", range(N_CASES))
def test_im2colpack_against_the_reference(oracle, golden, idx):
    """The fused im2col + pack: unpacked again it is the reference's im2col matrix, and every padding row and column of
    the last blocks is zero (the buffer starts as 0x55)."""
    p = pkg()
    p.use_current_torch_stream()
    geom, group_idx = conv_geometry_from_golden(golden[f"conv_{idx}_geom"])
    act = to_dev(_activation(oracle, geom))
    cp = _params(p, geom)
    rows, k = geom.rows, geom.k
    rows_pad, k_pad = -(-rows // 128) * 128, -(-k // 128) * 128
    for type_idx, tag in ((CL_PACKED, "cl"), (CF_PACKED, "cf")):
        uk = p.ConvI8(p.CONV_TYPES[type_idx])
        want = golden[f"conv_{idx}_{tag}"]
        want = want.T if uk.channel_first else want          # [positions, K]
        size = uk.get_b_im2colpack_size(rows, k) if uk.channel_first else uk.get_a_im2colpack_size(rows, k)
        assert size == rows_pad * k_pad
        packed = torch.full((size,), 0x55, dtype=torch.uint8, device=DEV)
        uk.run_im2colpack(group_idx, act, k, 0, packed, cp)
        back = torch.full((rows_pad, k_pad), 33, dtype=torch.int8, device=DEV)
        p.a_unpack_i8(rows_pad, k_pad, packed, k_pad, back, k_pad)
        sync_and_check()
        back = back.cpu().numpy()
        assert np.array_equal(back[:rows, :k], want)
        assert not back[rows:].any() and not back[:, k:].any()


def _run_conv(p, type_idx, geom, group_idx, case):
    """Drives one wrapper the way the reference's runner does; returns the int8 output [m, n] of its GEMM view."""
    uk = p.ConvI8(p.CONV_TYPES[type_idx])
    cp = _params(p, geom)
    rows, k, oc = geom.rows, geom.k, geom.output_channel // geom.groups
    act, W, fused = to_dev(case["act"]), to_dev(case["W"]), to_dev(case["bias_fused"])
    s_w = to_dev(case["scale_w"])
    if uk.channel_first:
        m, n = oc, rows
        params = p.QaI8QsI8DxQaI8Params(s_w.data_ptr(), oc, case["scale_act"], case["zp_act"], case["scale_d"], case["zp_d"])
    else:
        m, n = rows, oc
        params = p.QaI8QaI8QsI8CxParams(case["scale_act"], case["zp_act"], s_w.data_ptr(), oc, case["scale_d"], case["zp_d"])
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    if type_idx == CL_PACKED:
        a = torch.zeros(uk.get_a_im2colpack_size(m, k), dtype=torch.uint8, device=DEV)
        b = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_im2colpack(group_idx, act, k, 0, a, cp)
        uk.run_bt_pack(n, k, k, k, 0, W, b)
        uk.run_conv(m, n, k, a, k, 0, b, k, 0, None, n, d, n, fused, -128, 127, params)
    elif type_idx == CL_PLAIN:
        a = torch.zeros(uk.get_a_im2col_size(m, k), dtype=torch.int8, device=DEV)
        uk.run_im2col(group_idx, act, a, cp)
        uk.run_conv(m, n, k, a, k, 0, W, k, 0, None, n, d, n, fused, -128, 127, params)
    elif type_idx == CF_PLAIN:
        b = torch.zeros(uk.get_b_im2col_size(k, n), dtype=torch.int8, device=DEV)
        uk.run_im2col(group_idx, act, b, cp)
        uk.run_conv(m, n, k, W, k, 0, b, n, 0, None, n, d, n, fused, -128, 127, params)
    else:
        a = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
        b = torch.zeros(uk.get_b_im2colpack_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_a_pack(m, k, k, k, 0, W, a)
        uk.run_im2colpack(group_idx, act, k, 0, b, cp)
        uk.run_conv(m, n, k, a, k, 0, b, k, 0, None, n, d, n, fused, -128, 127, params)
    sync_and_check()
    return d.cpu().numpy()


@pytest.mark.parametrize("type_idx", range(4))
@pytest.mark.parametrize("idx", range(N_CASES))
def test_conv_requant(oracle, golden, idx, type_idx):
    p = pkg()
    p.use_current_torch_stream()
    geom, group_idx = conv_geometry_from_golden(golden[f"conv_{idx}_geom"])
    cf = type_idx in (CF_PLAIN, CF_PACKED)
    case = conv_acceptance_case(oracle, geom, cf, group_idx)
    got = _run_conv(p, type_idx, geom, group_idx, case)
    col = oracle.im2col_i8(case["act"], geom, cf, group_idx)
    if cf:
        want = oracle.gemm_mx1bias_reqi32toi8(case["W"], col, case["scale_w"], case["scale_act"], case["scale_d"], case["zp_d"],
                                              case["bias_fused"])
    else:
        want = oracle.gemm_reqi32toi8(col, case["W"], True, case["scale_act"], case["scale_w"], case["scale_d"], case["zp_d"],
                                      case["bias_fused"])
    assert np.array_equal(got, want)
    # the reference's pass criterion (quantized_conv_test_runner.h:252-262, 620-630)
    deq = (got.astype(np.float32) - np.float32(case["zp_d"])) * np.float32(case["scale_d"])
    assert np.max(np.abs(deq - case["real"])) <= 1.0
    assert cosine(deq, case["real"]) >= 0.999


@pytest.mark.parametrize("type_idx", range(4))
@pytest.mark.parametrize("idx", range(N_CASES))
def test_igemm_requant(oracle, golden, idx, type_idx):
    """The implicit-GEMM types: no im2col matrix; the whole output in one call and, for larger cases, as two calls that
    split the output positions (the reference's m_idx / n_idx tile portions: D stays the base of the whole output)."""
    p = pkg()
    p.use_current_torch_stream()
    geom, group_idx = conv_geometry_from_golden(golden[f"conv_{idx}_geom"])
    uk = p.IgemmI8(p.IGEMM_TYPES[type_idx])
    cf = uk.channel_first
    case = conv_acceptance_case(oracle, geom, cf, group_idx)
    col = oracle.im2col_i8(case["act"], geom, cf, group_idx)
    rows, k, oc = geom.rows, geom.k, geom.output_channel // geom.groups
    cp = _params(p, geom)
    act, W, fused, s_w = to_dev(case["act"]), to_dev(case["W"]), to_dev(case["bias_fused"]), to_dev(case["scale_w"])
    if uk.packed:
        size = uk.get_a_packed_size(oc, k) if cf else uk.get_b_packed_size(oc, k)
        wbuf = torch.zeros(size, dtype=torch.uint8, device=DEV)
        (uk.run_a_pack if cf else uk.run_bt_pack)(oc, k, k, k, 0, W, wbuf)
    else:
        wbuf = W
    if cf:
        want = oracle.gemm_mx1bias_reqi32toi8(case["W"], col, case["scale_w"], case["scale_act"], case["scale_d"], case["zp_d"],
                                              case["bias_fused"])
        params = p.QaI8QsI8DxQaI8Params(s_w.data_ptr(), oc, case["scale_act"], case["zp_act"], case["scale_d"], case["zp_d"])
        d = torch.full((oc, rows), 99, dtype=torch.int8, device=DEV)
        splits = [(0, rows)] if rows < 8 else [(0, rows // 2), (rows // 2, rows - rows // 2)]
        for p0, cnt in splits:
            uk.run_igemm(oc, cnt, k, act, group_idx, p0, wbuf, k, d, rows, fused, -128, 127, cp, params)
    else:
        want = oracle.gemm_reqi32toi8(col, case["W"], True, case["scale_act"], case["scale_w"], case["scale_d"], case["zp_d"],
                                      case["bias_fused"])
        params = p.QaI8QaI8QsI8CxParams(case["scale_act"], case["zp_act"], s_w.data_ptr(), oc, case["scale_d"], case["zp_d"])
        d = torch.full((rows, oc), 99, dtype=torch.int8, device=DEV)
        splits = [(0, rows)] if rows < 8 else [(0, rows // 2), (rows // 2, rows - rows // 2)]
        for p0, cnt in splits:
            uk.run_igemm(cnt, oc, k, act, group_idx, p0, wbuf, k, d, oc, fused, -128, 127, cp, params)
    sync_and_check()
    got = d.cpu().numpy()
    assert np.array_equal(got, want)
    deq = (got.astype(np.float32) - np.float32(case["zp_d"])) * np.float32(case["scale_d"])
    assert np.max(np.abs(deq - case["real"])) <= 1.0 and cosine(deq, case["real"]) >= 0.999


def test_igemm_argument_checks():
    p = pkg()
    p.use_current_torch_stream()
    uk = p.IgemmI8(p.IGEMM_TYPES[1])
    cp = p.ConvParams.make(4, 8, 1, (1, 4, 4), (1, 3, 3))          # 2 x 2 = 4 output positions, K = 36
    buf = torch.zeros(256, dtype=torch.int8, device=DEV)
    qp = p.QaI8QaI8QsI8CxParams(0.1, 0, buf.data_ptr(), 8, 0.1, 0)
    with pytest.raises(p.TqtError):
        uk.run_igemm(4, 8, 36, buf, 0, 2, buf, 36, buf, 8, None, -128, 127, cp, qp)    # positions 2 .. 6 of 4
    uk.run_igemm(4, 8, 36, buf, 0, 0, buf, 36, buf, 8, None, -128, 127, None, qp)       # null geometry: silent
    uk.run_igemm(4, 8, 36, buf, 0, 0, buf, 36, buf, 8, None, -128, 127, cp, None)


def test_conv_layer_sized(oracle):
    """A layer-sized channel-last convolution (56 x 56 x 64 -> 128 channels, 3 x 3, pad 1: M = 3136, K = 576) through the
    packed wrapper: 128-bit gather path and the CTA-pair GEMM, whole output against the oracle."""
    from oracle.tqo import ConvGeometry
    p = pkg()
    p.use_current_torch_stream()
    geom = ConvGeometry(64, 128, 1, (1, 56, 56), (1, 3, 3), pad=(0, 1, 1))
    case = conv_acceptance_case(oracle, geom, False)
    got = _run_conv(p, CL_PACKED, geom, 0, case)
    col = oracle.im2col_i8(case["act"], geom, False)
    want = oracle.gemm_reqi32toi8(col, case["W"], True, case["scale_act"], case["scale_w"], case["scale_d"], case["zp_d"],
                                  case["bias_fused"])
    assert np.array_equal(got, want)
    got_cf = _run_conv(p, CF_PACKED, geom, 0, conv_acceptance_case(oracle, geom, True))
    assert got_cf.shape == (128, 3136)


def test_conv_argument_checks():
    p = pkg()
    p.use_current_torch_stream()
    uk = p.ConvI8(p.CONV_TYPES[CL_PACKED])
    cp = p.ConvParams.make(8, 8, 2, (1, 4, 4), (1, 3, 3))
    buf = torch.zeros(uk.get_a_im2colpack_size(4, 36), dtype=torch.uint8, device=DEV)
    act = torch.zeros(128, dtype=torch.int8, device=DEV)
    with pytest.raises(p.TqtError):
        uk.run_im2colpack(2, act, 36, 0, buf, cp)          # group index out of range
    with pytest.raises(p.TqtError):
        uk.run_im2colpack(0, act, 36, 64, buf, cp)         # k_idx not a multiple of the K step
    uk.run_im2colpack(0, act, 36, 0, buf, None)            # null geometry: silently nothing, like null GEMM params
    uk.run_im2colpack(1, act, 36, 0, buf, cp)
    sync_and_check()
