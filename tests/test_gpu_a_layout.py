"""GPU tests of the one-time layout kernels: packers (with their inverses) and the qai8dx quantiser."""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import DEV, bits16, f32_to_bf16_bits, from_bits16, pkg, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

SHAPES = [(1, 16), (3, 11), (5, 130), (17, 24), (60, 127), (128, 128), (129, 257), (300, 1000)]


@pytest.mark.parametrize("rows,k", SHAPES)
def test_i8_pack_roundtrip(rows, k):
    p = pkg()
    uk = p.GemmClampI32I8pI8p()
    p.use_current_torch_stream()
    rng = np.random.default_rng(rows * 1000 + k)
    A = rng.integers(-128, 128, (rows, k), dtype=np.int8)
    lda = k + 5   # non-trivial leading dimension, unaligned rows
    A_ld = np.zeros((rows, lda), np.int8)
    A_ld[:, :k] = A
    packed = torch.full((uk.get_a_packed_size(rows, k),), 0x55, dtype=torch.uint8, device=DEV)
    uk.run_a_pack(rows, k, lda, k, 0, to_dev(A_ld), packed)
    out = torch.zeros((rows, k), dtype=torch.int8, device=DEV)
    p.a_unpack_i8(rows, k, packed, k, out, k)
    sync_and_check()
    assert np.array_equal(out.cpu().numpy(), A)
    # run_b_pack takes the transposed source [k, rows] and must give the same packed bytes
    packed_t = torch.full_like(packed, 0x55)
    uk.run_b_pack(rows, k, rows, k, 0, to_dev(np.ascontiguousarray(A.T)), packed_t)
    packed_n = torch.full_like(packed, 0x55)
    uk.run_bt_pack(rows, k, k, k, 0, to_dev(A), packed_n)
    sync_and_check()
    assert torch.equal(packed_t, packed_n) and torch.equal(packed_n, packed)
    # padding inside the blocks is zero
    total = packed.cpu().numpy().astype(np.int64)
    assert total.sum() == A.astype(np.uint8).astype(np.int64).sum()


@pytest.mark.parametrize("rows,k", SHAPES)
def test_f16_pack_roundtrip(rows, k):
    p = pkg()
    uk = p.GemmW4A16("f16")
    p.use_current_torch_stream()
    rng = np.random.default_rng(rows * 7 + k)
    A = rng.normal(0, 1, (rows, k)).astype(np.float16)
    packed = torch.zeros(uk.get_a_packed_size(rows, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(rows, k, k, k, 0, to_dev(A), packed)
    out = torch.zeros((rows, k), dtype=torch.float16, device=DEV)
    p.a_unpack_f16(rows, k, packed, k, out, k)
    sync_and_check()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), A.view(np.uint16))


@pytest.mark.parametrize("n,k", [(1, 2), (3, 8), (11, 16), (19, 24), (35, 64), (61, 128), (128, 256), (130, 258), (300, 1000)])
@pytest.mark.parametrize("c2", [False, True])
def test_i4_pack_roundtrip_and_rowsums(n, k, c2):
    p = pkg()
    uk = p.GemmW4A16("f16") if c2 else p.GemmW4A8("f32")
    p.use_current_torch_stream()
    rng = np.random.default_rng(n * 31 + k)
    nib = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    packed = torch.full((uk.get_b_packed_size(n, k),), 0xAB, dtype=torch.uint8, device=DEV)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(nib), packed)
    out = torch.zeros((n, k // 2), dtype=torch.uint8, device=DEV)
    (p.bt_unpack_qsi4c2p if c2 else p.bt_unpack_qsi4cxp)(n, k, packed, k, out, k)
    sync_and_check()
    assert np.array_equal(out.cpu().numpy(), nib)
    if not c2:
        # every block carries the int16 partial row sums of its 128 x 128 signed values
        blocks = packed.cpu().numpy().reshape(-1, 8448)
        q = np.zeros((-(-n // 128) * 128, -(-k // 128) * 128), np.int32)
        q[:n, 0:k:2] = (nib & 0xF).astype(np.int32) - 8
        q[:n, 1:k:2] = (nib >> 4).astype(np.int32) - 8
        kb = q.shape[1] // 128
        for t in range(q.shape[0] // 128):
            for b in range(kb):
                want = q[t * 128:(t + 1) * 128, b * 128:(b + 1) * 128].sum(1)
                got = blocks[t * kb + b, 8192:].view(np.int16)
                assert np.array_equal(got, want)


def test_k_slab_packing_matches_whole_pack():
    """run_*_pack with k < ld_packed and k_idx > 0 writes a K slab into the full buffer when given the
    destination offset by get_*_packed_offset (reference: tqt_gemm_pack_rvv.h:786-793 semantics)."""
    p = pkg()
    uk = p.GemmW4A8("f32")
    p.use_current_torch_stream()
    rng = np.random.default_rng(9)
    n, m, k = 200, 150, 640
    nib = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    nib_d, a_d = to_dev(nib), to_dev(A)
    whole_b = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    whole_a = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    uk.run_bt_pack(n, k, k, k, 0, nib_d, whole_b)
    uk.run_a_pack(m, k, k, k, 0, a_d, whole_a)
    slab_b, slab_a = torch.zeros_like(whole_b), torch.zeros_like(whole_a)
    for k0, kl in ((0, 256), (256, 128), (384, 256)):
        uk.run_bt_pack(n, kl, k, k, k0, nib_d.data_ptr() + k0 // 2, slab_b.data_ptr() + uk.get_b_packed_offset(0, k0, k, n))
        uk.run_a_pack(m, kl, k, k, k0, a_d.data_ptr() + k0, slab_a.data_ptr() + uk.get_a_packed_offset(0, k0, k, m))
    sync_and_check()
    assert torch.equal(slab_b, whole_b) and torch.equal(slab_a, whole_a)


@pytest.mark.parametrize("m,k", [(1, 16), (1, 4096), (5, 11), (7, 130), (17, 24), (33, 1000), (130, 512)])
@pytest.mark.parametrize("ta", ["f32", "f16", "bf16"])
def test_quantiser_bit_exact(oracle, m, k, ta):
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(m * 13 + k)
    A = rng.normal(0, 1, (m, k)).astype(np.float32)
    if m > 2:
        A[1] = 0.0                   # scale 1, zero point 0
        A[2] = np.abs(A[2]) + 0.5    # all positive: fmin forced to 0
    if m > 4:
        A[3] = -np.abs(A[3]) - 0.5   # all negative: fmax forced to 0
        A[4] = A[4] * 1e-30          # tiny range
    tt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[ta]
    a_dev = torch.from_numpy(A).to(DEV).to(tt)
    if ta == "f32":
        q_o, s_o, z_o = oracle.quantize_a_per_row_asym(A, TD_F32)
    else:
        q_o, s_o, z_o = oracle.quantize_a_per_row_asym(bits16(a_dev), TD_F16 if ta == "f16" else TD_BF16)
    # plain layout
    q = torch.full((m, k), 77, dtype=torch.int8, device=DEV)
    s = torch.zeros(m, dtype=torch.float32, device=DEV)
    z = torch.zeros(m, dtype=torch.int32, device=DEV)
    p.quant_qai8dx(a_dev, q, s, z)
    sync_and_check()
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_o.view(np.uint32))
    assert np.array_equal(z.cpu().numpy(), z_o)
    assert np.array_equal(q.cpu().numpy(), q_o)
    # packed layout: unpack and compare
    uk = p.GemmW4A8("f32")
    packed = torch.full((uk.get_a_packed_size(m, k),), 0x33, dtype=torch.uint8, device=DEV)
    s2, z2 = torch.zeros_like(s), torch.zeros_like(z)
    p.quant_pack_qai8dxp(a_dev, packed, s2, z2)
    back = torch.zeros((m, k), dtype=torch.int8, device=DEV)
    p.a_unpack_i8(m, k, packed, k, back, k)
    sync_and_check()
    assert np.array_equal(back.cpu().numpy(), q_o)
    assert torch.equal(s2, s) and torch.equal(z2, z)


def test_quantiser_strided_rows(oracle):
    """lda > k and a row base that is not 16-byte aligned take the scalar load path."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(4)
    m, k, lda = 9, 50, 61
    buf = rng.normal(0, 2, (m, lda)).astype(np.float32)
    a_dev = to_dev(buf)[:, 3:3 + k]
    q_o, s_o, z_o = oracle.quantize_a_per_row_asym(np.ascontiguousarray(buf[:, 3:3 + k]), TD_F32)
    q = torch.zeros((m, k), dtype=torch.int8, device=DEV)
    s = torch.zeros(m, dtype=torch.float32, device=DEV)
    z = torch.zeros(m, dtype=torch.int32, device=DEV)
    p.quant_qai8dx(a_dev, q, s, z)
    sync_and_check()
    assert np.array_equal(q.cpu().numpy(), q_o) and np.array_equal(z.cpu().numpy(), z_o)


@pytest.mark.parametrize("ta", ["f16", "bf16"])
@pytest.mark.parametrize("m,k", [(256, 4096), (40, 1024), (33, 16), (128, 4080), (45, 2064), (50, 1040), (37, 3088), (20000, 1024)])
def test_quantiser_rows_in_registers_exact_division(oracle, m, k, ta):
    """Many 16-bit rows with k <= 4096 take the warp-per-row kernel, which divides by the row scale
    through a corrected reciprocal.  Values are planted next to the rounding boundaries (quotients
    near j + 0.5) and at the extremes of the row; every byte must still equal the reference's
    round(x / scale) + zero point."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(k * 7 + m)
    tt = torch.float16 if ta == "f16" else torch.bfloat16
    A = rng.normal(0, 1, (m, k)).astype(np.float32)
    A[:, 0] = rng.uniform(-6, -2, m)      # row minimum
    A[:, 1] = rng.uniform(2, 6, m)        # row maximum
    scale = (A[:, 1] - A[:, 0]) / 255.0
    half = rng.integers(-100, 100, (m, k)).astype(np.float32) + 0.5
    plant = rng.random((m, k)) < 0.5
    plant[:, :2] = False
    A = np.where(plant, np.clip(half * scale[:, None], A[:, :1], A[:, 1:2]), A)
    if m > 2:
        A[2] = 0.0
    a_dev = torch.from_numpy(A).to(DEV).to(tt)
    q_o, s_o, z_o = oracle.quantize_a_per_row_asym(bits16(a_dev), TD_F16 if ta == "f16" else TD_BF16)
    q = torch.full((m, k), 77, dtype=torch.int8, device=DEV)
    s = torch.zeros(m, dtype=torch.float32, device=DEV)
    z = torch.zeros(m, dtype=torch.int32, device=DEV)
    p.quant_qai8dx(a_dev, q, s, z)
    sync_and_check()
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_o.view(np.uint32))
    assert np.array_equal(z.cpu().numpy(), z_o)
    assert np.array_equal(q.cpu().numpy(), q_o)
    uk = p.GemmW4A8("f32")
    packed = torch.full((uk.get_a_packed_size(m, k),), 0x33, dtype=torch.uint8, device=DEV)
    s2, z2 = torch.zeros_like(s), torch.zeros_like(z)
    p.quant_pack_qai8dxp(a_dev, packed, s2, z2)
    back = torch.zeros((m, k), dtype=torch.int8, device=DEV)
    p.a_unpack_i8(m, k, packed, k, back, k)
    sync_and_check()
    assert np.array_equal(back.cpu().numpy(), q_o)
    assert np.array_equal(s2.cpu().numpy().view(np.uint32), s_o.view(np.uint32))


def test_quantiser_rows_with_extreme_scales(oracle):
    """bf16 rows whose range is far outside the normal f32 reciprocal range (scale below 2^-126, or a huge
    scale): the warp-per-row kernel's corrected reciprocal cannot be used there (1 / s overflows or goes
    subnormal), so such rows divide; every byte must equal the reference's nearbyint(x / scale) + zero point."""
    p = pkg()
    p.use_current_torch_stream()
    rng = np.random.default_rng(31)
    m, k = 64, 256
    A = rng.normal(0, 1, (m, k)).astype(np.float32)
    A[0] *= np.float32(1e-38)
    A[1] *= np.float32(3e-39)
    A[2] *= np.float32(1e-36)
    A[3] *= np.float32(1e37)
    A[4] *= np.float32(3e38) / np.abs(A[4]).max()
    A[5] *= np.float32(1e-33)
    A[6] = np.abs(A[6]) * np.float32(2e-39)
    bits = f32_to_bf16_bits(A)
    a_dev = from_bits16(bits, torch.bfloat16)
    q_o, s_o, z_o = oracle.quantize_a_per_row_asym(bits, TD_BF16)
    q = torch.full((m, k), 77, dtype=torch.int8, device=DEV)
    s = torch.zeros(m, dtype=torch.float32, device=DEV)
    z = torch.zeros(m, dtype=torch.int32, device=DEV)
    p.quant_qai8dx(a_dev, q, s, z)
    sync_and_check()
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_o.view(np.uint32))
    assert np.array_equal(z.cpu().numpy(), z_o)
    assert np.array_equal(q.cpu().numpy(), q_o)
