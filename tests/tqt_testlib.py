"""Shared helpers of the GPU parity tests: seeded inputs and thin drivers that call the micro-kernels
through the C ABI the way the reference's own test runners drive its kernels
(test/common/quantized_gemm_test_runner.h, test/gemm/test_gemm_i8_i4_rvv.cpp:325-421)."""
from __future__ import annotations

import numpy as np
import torch

from __graft_entry__ import load, load_linear

FMAX = 3.4028234663852886e38
DEV = "cuda:0"


def pkg():
    return load()


def to_dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def bits16(t):
    """numpy uint16 view of a f16 / bf16 torch tensor."""
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits16(bits, dtype):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(DEV).view(dtype)


def sync_and_check():
    torch.cuda.synchronize()
    fault = pkg().read_device_fault()
    assert fault == 0, f"device watchdog fired: 0x{fault:x}"


TD_TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def run_w4a8(td, A_q, sa, zp, nib, sb, Cm=None, bias=None, clamp=None, tile=None, m_override=None):
    """Pack + run gemm_1xnbias_clamp_<td>_qai8dxp_qsi4cxp.  A_q int8 [m,k]; nib uint8 [n,k/2]; C/bias as
    numpy arrays already in the output type's bit representation (float32, or uint16 bits).
    tile=(tm, tn): drive it as a caller-side tile loop with the offset helpers; else one whole call."""
    p = pkg()
    uk = p.GemmW4A8(td)
    p.use_current_torch_stream()
    m, k = A_q.shape
    n = nib.shape[0]
    tdt = TD_TORCH[td]
    a_dev, nib_dev = to_dev(A_q), to_dev(nib)
    a_packed = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    b_packed = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, a_dev, a_packed)
    uk.run_bt_pack(n, k, k, k, 0, nib_dev, b_packed)
    sa_d, zp_d, sb_d = to_dev(sa), to_dev(zp), to_dev(sb)

    def as_td(x):
        if x is None:
            return None
        return to_dev(x) if td == "f32" else from_bits16(x, tdt)

    c_d, bias_d = as_td(Cm), as_td(bias)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)   # canary value in untouched cells
    if clamp is None:
        clamp = (-FMAX, FMAX) if td == "f32" else (-65504.0, 65504.0)
    es = 4 if td == "f32" else 2
    if tile is None:
        params = p.QaI8DxQsI4CxParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
        uk.run_gemm(m, n, k, a_packed, k, 0, b_packed, k, 0, c_d, n, d, n, bias_d, clamp[0], clamp[1], params)
    else:
        tm, tn = tile
        assert tm % uk.get_m_step() == 0 and tn % uk.get_n_step() == 0
        for m0 in range(0, m, tm):
            for n0 in range(0, n, tn):
                am, an = min(tm, m - m0), min(tn, n - n0)
                # params arrays are indexed from the call's own origin: pass offset pointers
                params = p.QaI8DxQsI4CxParams(sa_d.data_ptr() + 4 * m0, zp_d.data_ptr() + 4 * m0, sb_d.data_ptr() + 4 * n0)
                uk.run_gemm(am, an, k,
                            a_packed.data_ptr() + uk.get_a_packed_offset(m0, 0, k, am), k, 0,
                            b_packed.data_ptr() + uk.get_b_packed_offset(n0, 0, k, an), k, 0,
                            None if c_d is None else c_d.data_ptr() + uk.get_c_offset(m0, n0, n), n,
                            d.data_ptr() + uk.get_d_offset(m0, n0, n), n,
                            None if bias_d is None else bias_d.data_ptr() + uk.get_bias_offset(n0),
                            clamp[0], clamp[1], params)
    sync_and_check()
    return d.cpu().numpy() if td == "f32" else bits16(d)


def run_i32_packed(A, B, b_is_nk, Cm=None, clamp=(-2**31, 2**31 - 1)):
    p = pkg()
    uk = p.GemmClampI32I8pI8p()
    p.use_current_torch_stream()
    m, k = A.shape
    n = B.shape[0] if b_is_nk else B.shape[1]
    a_packed = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    b_packed = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(A), a_packed)
    if b_is_nk:
        uk.run_bt_pack(n, k, k, k, 0, to_dev(B), b_packed)
    else:
        uk.run_b_pack(n, k, n, k, 0, to_dev(B), b_packed)
    d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    c_d = None if Cm is None else to_dev(Cm)
    uk.run_gemm(m, n, k, a_packed, k, 0, b_packed, k, 0, c_d, n, d, n, int(clamp[0]), int(clamp[1]))
    sync_and_check()
    return d.cpu().numpy()


def run_i32_unpacked(A, B_kn, Cm=None, clamp=(-2**31, 2**31 - 1)):
    p = pkg()
    uk = p.GemmClampI32I8I8()
    p.use_current_torch_stream()
    m, k = A.shape
    n = B_kn.shape[1]
    d = torch.full((m, n), -77, dtype=torch.int32, device=DEV)
    c_d = None if Cm is None else to_dev(Cm)
    uk.run_gemm(m, n, k, to_dev(A), k, 0, to_dev(B_kn), n, 0, c_d, n, d, n, int(clamp[0]), int(clamp[1]))
    sync_and_check()
    return d.cpu().numpy()


def run_requant(A, B_nk, scale_a, scale_b, scale_d, zp_d, bias=None, Cm=None, clamp=(-128, 127), quant_channel_b=0,
                tile=None):
    p = pkg()
    uk = p.GemmReqI8()
    p.use_current_torch_stream()
    m, k = A.shape
    n = B_nk.shape[0]
    a_packed = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    b_packed = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(A), a_packed)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(B_nk), b_packed)
    sb_d = to_dev(scale_b)
    bias_d = None if bias is None else to_dev(bias)
    c_d = None if Cm is None else to_dev(Cm)
    d = torch.full((m, n), 99, dtype=torch.int8, device=DEV)
    if tile is None:
        params = p.QaI8QaI8QsI8CxParams(scale_a, 0, sb_d.data_ptr(), quant_channel_b, scale_d, zp_d)
        uk.run_gemm(m, n, k, a_packed, k, 0, b_packed, k, 0, c_d, n, d, n, bias_d, clamp[0], clamp[1], params)
    else:
        tm, tn = tile
        for m0 in range(0, m, tm):
            for n0 in range(0, n, tn):
                am, an = min(tm, m - m0), min(tn, n - n0)
                params = p.QaI8QaI8QsI8CxParams(scale_a, 0, sb_d.data_ptr() + 4 * n0, quant_channel_b, scale_d, zp_d)
                uk.run_gemm(am, an, k, a_packed.data_ptr() + uk.get_a_packed_offset(m0, 0, k, am), k, 0,
                            b_packed.data_ptr() + uk.get_b_packed_offset(n0, 0, k, an), k, 0,
                            None if c_d is None else c_d.data_ptr() + uk.get_c_offset(m0, n0, n), n,
                            d.data_ptr() + uk.get_d_offset(m0, n0, n), n,
                            None if bias_d is None else bias_d.data_ptr() + uk.get_bias_offset(n0),
                            clamp[0], clamp[1], params)
    sync_and_check()
    return d.cpu().numpy()


def run_w4a16(td, A_bits, nib, scale_bits, bl, Cm=None, bias=None, clamp=None):
    p = pkg()
    uk = p.GemmW4A16(td)
    p.use_current_torch_stream()
    m, k = A_bits.shape
    n = nib.shape[0]
    tdt = TD_TORCH[td]
    a_dev = from_bits16(A_bits, torch.float16)
    a_packed = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    b_packed = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, a_dev, a_packed)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(nib), b_packed)
    sc_d = from_bits16(scale_bits, torch.float16)

    def as_td(x):
        if x is None:
            return None
        return to_dev(x) if td == "f32" else from_bits16(x, tdt)

    c_d, bias_d = as_td(Cm), as_td(bias)
    d = torch.full((m, n), 7.0, dtype=tdt, device=DEV)
    if clamp is None:
        clamp = (-FMAX, FMAX) if td == "f32" else (-65504.0, 65504.0)
    uk.run_gemm(m, n, k, bl, a_packed, k, 0, b_packed, k, 0, sc_d, k // bl, c_d, n, d, n, bias_d, clamp[0], clamp[1])
    sync_and_check()
    return d.cpu().numpy() if td == "f32" else bits16(d)


def requant_acceptance_case(oracle, m, n, k):
    """Inputs of the reference's own test of the 1xN-bias requantising GEMM (run_1xnbias_reqi32toi8_gemm_test,
    test/common/quantized_gemm_test_runner.h:193-306): real-valued A, B ~ U(-1,1) from one mt19937(42) stream,
    bias ~ U(-10,10) seed 123; A quantised asymmetrically per tensor, B symmetrically per channel, bias to int32 at
    scale_a * scale_b[n] with the activation zero point fused in; the output scale / zero point from the range of
    the real-valued result.  Returns the quantised operands, the params and that real-valued result (no GPU)."""
    f32 = np.float32
    AB = oracle.fill_uniform((m * k + n * k,), np.float32, -1.0, 1.0, 42)
    A, B = AB[:m * k].reshape(m, k), AB[m * k:].reshape(n, k)
    bias = oracle.fill_uniform((n,), np.float32, -10.0, 10.0, 123)

    def asym(x):   # compute_asym_quant_params_i8 (:37-65)
        fmin, fmax = f32(min(x.min(), 0.0)), f32(max(x.max(), 0.0))
        sc = f32(f32(fmax - fmin) / f32(255.0))
        if sc == 0:
            return f32(1.0), 0
        zp = int(np.rint(f32(-128.0) - f32(fmin / sc)))
        return sc, (-127 if zp == -128 else zp)

    def quant(x, sc, zp):   # quantize_i8 (test_common.h:232-240)
        return np.clip(np.rint((x / f32(sc)).astype(f32)) + f32(zp), -128, 127).astype(np.int8)

    sa, zpa = asym(A)
    absmax = np.abs(B).max(axis=1).astype(f32)
    sb = (f32(2.0) * absmax / f32(255.0)).astype(f32)   # compute_sym_quant_params_i8 (:69-86)
    sb[sb == 0] = 1.0
    Aq = quant(A, sa, zpa)
    Bq = np.stack([quant(B[j], sb[j], 0) for j in range(n)])
    bias_i32 = np.clip(np.rint((bias / (f32(sa) * sb)).astype(f32)), -2147483648.0, 2147483647.0).astype(np.int64).astype(np.int32)
    fused = oracle.fuse_zp_to_bias(bias_i32, Bq, zpa)
    real = (A.astype(np.float64) @ B.T.astype(np.float64) + bias.astype(np.float64)[None, :]).astype(f32)
    sd, zpd = asym(real)
    return dict(A=Aq, B=Bq, scale_a=float(sa), zp_a=zpa, scale_b=sb, bias_fused=fused, scale_d=float(sd), zp_d=zpd, real=real)


def requant_acceptance_check(D_i8, case):
    """The reference's pass criterion: dequantised output against the real-valued GEMM, max abs error 1.0 and
    cosine similarity 0.999 (quantized_gemm_test_runner.h:294-302)."""
    deq = (D_i8.astype(np.float32) - np.float32(case["zp_d"])) * np.float32(case["scale_d"])
    assert np.max(np.abs(deq - case["real"])) <= 1.0
    assert cosine(deq, case["real"]) >= 0.999


def rel_err(got, want):
    """max |got - want| / max(|want|, rms(want)): relative error with an RMS floor against 0/0."""
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    rms = float(np.sqrt(np.mean(want * want))) or 1.0
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), rms)))


def cosine(got, want):
    a, b = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    d = np.linalg.norm(a) * np.linalg.norm(b)
    return 1.0 if d == 0 else float(a @ b / d)


def f16_bits_to_f32(bits):
    return np.ascontiguousarray(bits).view(np.float16).astype(np.float32)


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
