"""K-split accumulation through the micro-kernel API, as the reference's tiled runner drives it
(test/common/gemm_test_runner.h:380-419): the K extent is walked in slabs, every call after the first
receives the previous output as C (the same buffer: C == D), bias and the caller's clamp go to the last
slab only, earlier slabs run with a neutral clamp.  Operands of a slab are found with the kernel type's
own offset helpers inside buffers packed once for the full K (lda / ldb = full K).

The expected values come from the CPU oracle driven through the same chain of calls, so integer outputs and
the W4A8 float outputs are compared bit for bit; W4A16 (tensor-core accumulation order) to its tolerance.
"""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import (DEV, cosine, f16_bits_to_f32, f32_to_bf16_bits, from_bits16, bits16, pkg, rel_err, sync_and_check,
                         to_dev)

pytestmark = pytest.mark.gpu

INF = float("inf")
TD_CODE = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}
TD_TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _slabs(k, first):
    return [(0, first), (first, k)]


@pytest.mark.parametrize("m,n,k,first", [(64, 256, 512, 256), (9, 19, 23, 7), (60, 63, 127, 64)])
def test_ksplit_i32_unpacked(oracle, m, n, k, first):
    """gemm_clamp_i32_i8_i8: slabs addressed with get_a_offset / get_b_offset, C == D from the second call on."""
    p = pkg()
    uk = p.GemmClampI32I8I8()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    B = rng.integers(-128, 128, (k, n), dtype=np.int8)
    C0 = rng.integers(-1000, 1000, (m, n)).astype(np.int32)
    a_d, b_d, c_d = to_dev(A), to_dev(B), to_dev(C0)
    d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    lo, hi = -2**31, 2**31 - 1
    for i, (k0, k1) in enumerate(_slabs(k, first)):
        last = k1 == k
        uk.run_gemm(m, n, k1 - k0, a_d.data_ptr() + uk.get_a_offset(0, k0, k), k, 0,
                    b_d.data_ptr() + uk.get_b_offset(0, k0, n), n, 0, c_d if i == 0 else d, n, d, n,
                    -30000 if last else lo, 25000 if last else hi)
    sync_and_check()
    want = oracle.gemm_clamp_i32_i8_i8(A, B, False, C0, (-30000, 25000))
    assert np.array_equal(d.cpu().numpy(), want)


@pytest.mark.parametrize("m,n,k,first", [(140, 270, 384, 128), (300, 130, 1000, 512), (32, 32, 256, 128)])
def test_ksplit_i32_packed_and_requant(oracle, m, n, k, first):
    """Packed int8 types: the first slab runs on gemm_clamp_i32_i8p_i8p into an int32 buffer (then in place,
    C == D); the last slab of the requantising type takes that buffer as C together with bias and clamp."""
    p = pkg()
    uk32, ukq = p.GemmClampI32I8pI8p(), p.GemmReqI8()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m * 3 + n + k)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    a_d, w_d = to_dev(A), to_dev(W)

    def packed(uk):
        ap = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
        bp = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        uk.run_a_pack(m, k, k, k, 0, a_d, ap)
        uk.run_bt_pack(n, k, k, k, 0, w_d, bp)
        return ap, bp

    ap, bp = packed(uk32)
    acc = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    # int32 type alone: two slabs, second in place
    for i, (k0, k1) in enumerate(_slabs(k, first)):
        uk32.run_gemm(m, n, k1 - k0, ap.data_ptr() + uk32.get_a_packed_offset(0, k0, k, m), k, 0,
                      bp.data_ptr() + uk32.get_b_packed_offset(0, k0, k, n), k, 0, None if i == 0 else acc, n, acc, n,
                      -2**31, 2**31 - 1)
    sync_and_check()
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_clamp_i32_i8_i8(A, W, True))
    # requantising type: int32 partial of the first slab, then the last slab with C, bias and clamp
    k0, k1 = _slabs(k, first)[0]
    uk32.run_gemm(m, n, k1 - k0, ap, k, 0, bp, k, 0, None, n, acc, n, -2**31, 2**31 - 1)
    apq, bpq = packed(ukq)
    out = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    sb_d, bias_d = to_dev(sb), to_dev(bias)
    params = p.QaI8QaI8QsI8CxParams(0.05, 0, sb_d.data_ptr(), 0, 20.0, -5)
    k0, k1 = _slabs(k, first)[1]
    ukq.run_gemm(m, n, k1 - k0, apq.data_ptr() + ukq.get_a_packed_offset(0, k0, k, m), k, 0,
                 bpq.data_ptr() + ukq.get_b_packed_offset(0, k0, k, n), k, 0, acc, n, out, n, bias_d, -100, 90, params)
    sync_and_check()
    want = oracle.gemm_reqi32toi8(A, W, True, 0.05, sb, 20.0, -5, bias, None, (-100, 90))
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("td", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("m,n,k,first", [(200, 300, 512, 256), (4, 260, 384, 128), (1, 512, 1024, 512), (130, 130, 320, 128)])
def test_ksplit_w4a8(oracle, td, m, n, k, first):
    """W4A8 packed (tensor-core GEMM for large m, GEMV for m <= 8): every packed block carries its own row
    sums, so a slab's zero-point correction is complete by itself.  The oracle is run through the same
    two calls; outputs bit for bit."""
    p = pkg()
    uk = p.GemmW4A8(td)
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + 2 * n + k)
    A = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    W = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    q, sa, zp = oracle.quantize_a_per_row_asym(A)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    C0 = rng.uniform(-2, 2, (m, n)).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    if td == "f16":
        C0, bias = C0.astype(np.float16).view(np.uint16), bias.astype(np.float16).view(np.uint16)
    elif td == "bf16":
        C0, bias = f32_to_bf16_bits(C0), f32_to_bf16_bits(bias)
    tdt = TD_TORCH[td]

    def dev_td(x):
        return to_dev(x) if td == "f32" else from_bits16(x, tdt)

    ap = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    bp = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(q), ap)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(nib), bp)
    sa_d, zp_d, sb_d = to_dev(sa), to_dev(zp), to_dev(sb)
    params = p.QaI8DxQsI4CxParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    c_d, bias_d = dev_td(C0), dev_td(bias)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)
    want = C0
    for i, (k0, k1) in enumerate(_slabs(k, first)):
        last = k1 == k
        cl = (-0.75, 0.5) if last else (-INF, INF)
        uk.run_gemm(m, n, k1 - k0, ap.data_ptr() + uk.get_a_packed_offset(0, k0, k, m), k, 0,
                    bp.data_ptr() + uk.get_b_packed_offset(0, k0, k, n), k, 0, c_d if i == 0 else d, n, d, n,
                    bias_d if last else None, cl[0], cl[1], params)
        want = oracle.gemm_w4a8(np.ascontiguousarray(q[:, k0:k1]), np.ascontiguousarray(nib[:, k0 // 2:k1 // 2]), sa, zp, sb,
                                TD_CODE[td], want, bias if last else None, cl)
    sync_and_check()
    got = d.cpu().numpy() if td == "f32" else bits16(d)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("td", ["f16", "f32"])
@pytest.mark.parametrize("m,n,k,first,bl", [(200, 300, 512, 256, 32), (130, 140, 384, 128, 64)])
def test_ksplit_w4a16(oracle, td, m, n, k, first, bl):
    """W4A16 packed: slabs start on multiples of the 128-element packed block and of bl; the block scales of
    a slab are found with get_scale_b_offset."""
    p = pkg()
    uk = p.GemmW4A16(td)
    p.use_current_torch_stream()
    rng = np.random.default_rng(m + n + k + bl)
    A = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    bias = rng.normal(0, 0.1, n).astype(np.float16 if td == "f16" else np.float32)
    tdt = TD_TORCH[td]
    ap = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    bp = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(A), ap)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(nib), bp)
    sc_d = from_bits16(sc, torch.float16)
    bias_d = to_dev(bias)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)
    ldsb = k // bl
    want = None
    for i, (k0, k1) in enumerate(_slabs(k, first)):
        last = k1 == k
        cl = (-2.0, 1.5) if last else (-INF, INF)
        uk.run_gemm(m, n, k1 - k0, bl, ap.data_ptr() + uk.get_a_packed_offset(0, k0, k, m), k, 0,
                    bp.data_ptr() + uk.get_b_packed_offset(0, k0, k, n), k, 0,
                    sc_d.data_ptr() + uk.get_scale_b_offset(0, k0 // bl, ldsb), ldsb, None if i == 0 else d, n, d, n,
                    bias_d if last else None, cl[0], cl[1])
        bias_o = None if not last else (bias.view(np.uint16) if td == "f16" else bias)
        want = oracle.gemm_w4a16(np.ascontiguousarray(A[:, k0:k1]).view(np.uint16), np.ascontiguousarray(nib[:, k0 // 2:k1 // 2]),
                                 np.ascontiguousarray(sc[:, k0 // bl:k1 // bl]), bl, TD_CODE[td], want, bias_o, cl)
    sync_and_check()
    if td == "f16":
        g, w = f16_bits_to_f32(bits16(d)), f16_bits_to_f32(want)
    else:
        g, w = d.cpu().numpy(), want
    assert rel_err(g, w) <= 2e-2
    assert np.max(np.abs(g - w)) <= 1.0 and cosine(g, w) >= 0.9999


def test_bf16_output_beyond_the_f16_range(oracle):
    """bf16 outputs have the f32 exponent range: an operator built without a clamp must not saturate them at
    the f16 maximum.  Large activation scales push the results past 65536."""
    from __graft_entry__ import load_linear
    lin = load_linear()
    rng = np.random.default_rng(9)
    m, n, k = 130, 256, 256
    A = (rng.normal(0, 1, (m, k)) * 3.0e4).astype(np.float32)
    W = rng.normal(0, 1.0, (n, k)).astype(np.float32)
    a_bits = f32_to_bf16_bits(A)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16")
    out = layer(from_bits16(a_bits, torch.bfloat16))
    sync_and_check()
    q, sa, zp = oracle.quantize_a_per_row_asym(a_bits, TD_BF16)
    bmax = 3.3895313892515355e38
    want = oracle.gemm_w4a8(q, nib, sa, zp, sb, TD_BF16, None, None, (-bmax, bmax))
    got = bits16(out)
    assert np.array_equal(got, want)
    vals = (want.astype(np.uint32) << 16).view(np.float32)
    assert (np.abs(vals) > 65536.0).mean() > 0.2
