"""The unquantised GEMM kernel types (include/tqt_b200_gemm_float.h) against the oracle's restatement of the reference's
reference_gemm<TA, TD> (pinned to the reference's own code in tests/test_oracle_pins.py).  Inputs as in the reference's
runner (test/common/gemm_test_runner.h:326-365: U(-1,1), seed 42 for A then B, seed 43 for C then bias) on its shape
list plus tile-crossing shapes.  The generic CUDA-core kernel multiplies and adds in k order like the reference: bit-exact.
The tensor-core path (16-bit operands, packed or 16-byte-aligned row-major) accumulates in f32 in another order: within
the stated bars (rel 1e-3 for f32 outputs, 2e-2 for 16-bit outputs) and the reference's own thresholds."""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import DEV, FMAX, bf16_bits_to_f32, bits16, cosine, f16_bits_to_f32, f32_to_bf16_bits, pkg, rel_err, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

TDI = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}
TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
SIMT, PAIR_BLOCKS, PAIR_TMA = 1, 2, 3
# (m, n, k, bias, c, clamp): the reference's list (test/gemm/test_gemm_f32_f32_rvv.cpp:30-44), then shapes that cross tiles
SHAPES = [(32, 32, 32, 0, 0, None), (5, 11, 10, 0, 0, None), (17, 19, 23, 1, 0, None), (31, 35, 63, 0, 1, None),
          (60, 61, 127, 1, 1, (-100.0, 150.0)), (130, 260, 200, 1, 0, (-2.0, 2.5)), (300, 390, 520, 1, 1, None),
          (128, 256, 192, 0, 0, None)]


def _typed(oracle, shape, t, seed):
    """U(-1,1) from the reference's generator stream, rounded to type t: (numpy for the oracle, device tensor)."""
    x = oracle.fill_uniform(shape, np.float32, -1.0, 1.0, seed)
    if t == "f32":
        return x, to_dev(x)
    if t == "f16":
        h = x.astype(np.float16)
        return h.view(np.uint16), to_dev(h)
    b = f32_to_bf16_bits(x)
    return b, to_dev(b.view(np.int16)).view(torch.bfloat16)


def _as_f32(bits, t):
    return bits if t == "f32" else (f16_bits_to_f32(bits) if t == "f16" else bf16_bits_to_f32(bits))


@pytest.mark.parametrize("m,n,k,has_bias,has_c,clamp", SHAPES)
@pytest.mark.parametrize("type_idx", range(22))
def test_float_gemm(oracle, type_idx, m, n, k, has_bias, has_c, clamp):
    p = pkg()
    p.use_current_torch_stream()
    uk = p.FloatGemm(p.FLOAT_TYPES[type_idx])
    ta, td = uk.ta, uk.td
    AB, _ = _typed(oracle, (m * k + n * k,), ta, 42)
    A, Bt = AB[:m * k].reshape(m, k).copy(), AB[m * k:].reshape(n, k).copy()      # B drawn as [n, k]
    CB, _ = _typed(oracle, (m * n + max(m, n),), td, 43)
    Cm = CB[:m * n].reshape(m, n).copy() if has_c else None
    nb = m if uk.bias_per_row else n
    bias = CB[m * n:m * n + nb].copy() if has_bias else None
    cl = clamp if clamp else ((-FMAX, FMAX) if td == "f32" else ((-65504.0, 65504.0) if td == "f16" else (-3.0e38, 3.0e38)))
    if td == "bf16":   # the clamp arguments are bf16 values
        cl = tuple(float(bf16_bits_to_f32(f32_to_bf16_bits(np.array([c], np.float32)))[0]) for c in cl)
    want = oracle.gemm_float(TDI[ta], TDI[td], A, Bt, True, Cm, bias, uk.bias_per_row, cl)

    def dev(x, t):
        if x is None:
            return None
        return to_dev(x) if t == "f32" else to_dev(x.view(np.int16)).view(TORCH[t])

    a_d, c_d, bias_d = dev(A, ta), dev(Cm, td), dev(bias, td)
    if uk.a_packed:
        a_arg = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
        uk.run_a_pack(m, k, k, k, 0, a_d, a_arg)
    else:
        a_arg = a_d
    if uk.b_packed:
        b_arg = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        if (m + n) % 2:   # either packer: from [k, n] or from [n, k]
            uk.run_b_pack(n, k, n, k, 0, dev(np.ascontiguousarray(Bt.T), ta), b_arg)
        else:
            uk.run_bt_pack(n, k, k, k, 0, dev(Bt, ta), b_arg)
        ldb = k
    elif uk.b_transposed:
        b_arg, ldb = dev(Bt, ta), k
    else:
        b_arg, ldb = dev(np.ascontiguousarray(Bt.T), ta), n
    d = torch.full((m, n), 7.0, dtype=TORCH[td], device=DEV)
    uk.run_gemm(m, n, k, a_arg, k, 0, b_arg, ldb, 0, c_d, n, d, n, bias_d, cl[0], cl[1])
    sync_and_check()
    got = d.cpu().numpy() if td == "f32" else bits16(d)
    fam = p.debug_last_kernel()
    tensor_ok = ta != "f32"
    aligned = (uk.a_packed or (2 * k) % 16 == 0) and (uk.b_packed or (2 * (k if uk.b_transposed else n)) % 16 == 0)
    if not tensor_ok or not aligned:
        assert fam == SIMT
        assert np.array_equal(got.view(np.uint32) if td == "f32" else got, want.view(np.uint32) if td == "f32" else want)
    else:
        assert fam == (PAIR_BLOCKS if uk.a_packed and uk.b_packed else PAIR_TMA)
        g, w = _as_f32(got, td), _as_f32(want, td)
        assert rel_err(g, w) <= (1e-3 if td == "f32" else 2e-2)
        # the reference's DefaultThreshold for these suites is looser than the bars above; cosine as a second view
        assert cosine(g, w) >= 0.9999


def test_float_gemm_forced_generic_agrees(oracle, force_path):
    """A packed bf16 call on tensor cores and on the generic kernel (TQT_B200_PATH=simt): the generic one is bit-exact
    against the oracle, the tensor-core one within the bar of it."""
    p = pkg()
    p.use_current_torch_stream()
    uk = p.FloatGemm("gemm_1xnbias_clamp_bf16_bf16p_bf16p")
    m, n, k = 200, 272, 320
    AB, _ = _typed(oracle, (m * k + n * k,), "bf16", 42)
    A, Bt = AB[:m * k].reshape(m, k).copy(), AB[m * k:].reshape(n, k).copy()
    want = oracle.gemm_float(TD_BF16, TD_BF16, A, Bt, True, None, None, False, (-3.0e38, 3.0e38))
    a_p = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    b_p = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(A.view(np.int16)).view(torch.bfloat16), a_p)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(Bt.view(np.int16)).view(torch.bfloat16), b_p)
    outs = {}
    for path in ("simt", None):
        force_path(path, None)
        d = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
        uk.run_gemm(m, n, k, a_p, k, 0, b_p, k, 0, None, n, d, n, None, -3.0e38, 3.0e38)
        sync_and_check()
        outs[path] = bits16(d)
        assert p.debug_last_kernel() == (SIMT if path else PAIR_BLOCKS)
    assert np.array_equal(outs["simt"], want)
    assert rel_err(bf16_bits_to_f32(outs[None]), bf16_bits_to_f32(want)) <= 2e-2
