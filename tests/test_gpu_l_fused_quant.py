"""Quantise + W4A8 GEMM as one call (tqt_run_quant_gemm_1xnbias_clamp_<td>_qai8dxp_qsi4cxp, include/tqt_b200_ext.h): the
call must leave exactly what the quantiser followed by run_gemm leaves — packed activations, scales, zero points and the
output, bit for bit — whether the library runs it as one cooperative launch (16-bit activations, k <= 4096, m > 16) or
as the two kernels back to back (every other shape), and against the oracle's restatement of the reference's
quantisation (test/common/quantization_method.h) and GEMM."""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import DEV, bits16, f32_to_bf16_bits, from_bits16, load_linear, pkg, sync_and_check, to_dev

pytestmark = pytest.mark.gpu

TDI = {"f32": TD_F32, "f16": TD_F16, "bf16": TD_BF16}
TS_FUSED_QUANT = 5     # the family the fused launch reports


def _activations(oracle, m, k, ta, seed):
    x = oracle.fill_normal((m, k), 0.0, 1.0, seed)
    if ta == "f32":
        return x, to_dev(x), TD_F32
    if ta == "f16":
        h = x.astype(np.float16)
        return h.view(np.uint16), to_dev(h), TD_F16
    b = f32_to_bf16_bits(x)
    return b, from_bits16(b, torch.bfloat16), TD_BF16


def _layer(oracle, n, k, td, seed, with_bias):
    lin = load_linear()
    W = oracle.fill_normal((n, k), 0.0, 0.02, seed)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    bias = to_dev(oracle.fill_normal((n,), 0.0, 0.1, seed + 1)) if with_bias else None
    return lin.W4A8Linear(to_dev(nib), to_dev(sb), k, td, bias=bias), nib, sb


# (m, n, k, activation type, output type, fused launch expected)
CASES = [(512, 512, 1024, "bf16", "bf16", True), (300, 260, 528, "f16", "f32", True), (192, 3000, 4096, "bf16", "f16", True),
         (17, 130, 48, "f16", "bf16", True), (1000, 1100, 2000, "bf16", "f32", True),
         (256, 256, 4112, "bf16", "bf16", False),   # k above the fused form's row buffer
         (200, 384, 512, "f32", "f32", False),      # f32 activations
         (8, 512, 1024, "bf16", "bf16", False),     # decode: the GEMV
         (320, 256, 264, "f16", "f16", False)]      # k not a multiple of 16


@pytest.mark.parametrize("m,n,k,ta,td,fused", CASES)
def test_fused_equals_two_launches(oracle, m, n, k, ta, td, fused):
    p = pkg()
    layer, nib, sb = _layer(oracle, n, k, td, 77, with_bias=(m % 2 == 0))
    a_np, a_dev, ta_id = _activations(oracle, m, k, ta, 5)
    ws = layer.workspace(m)

    def snapshot():
        sync_and_check()
        return (ws["a_packed"].cpu().numpy().copy(), ws["scale_a"].cpu().numpy().copy(), ws["zp_a"].cpu().numpy().copy(),
                ws["out"].cpu().numpy().copy() if td == "f32" else bits16(ws["out"]).copy())

    def poison():
        ws["a_packed"].zero_()
        ws["scale_a"].fill_(float("nan"))
        ws["zp_a"].fill_(12345)
        ws["out"].fill_(float("nan"))

    poison()
    layer.fuse_quant = False
    layer(a_dev)
    two = snapshot()
    poison()
    layer.fuse_quant = True
    layer(a_dev)
    one = snapshot()
    fam = p.debug_last_kernel()
    for x, y in zip(one, two):
        assert np.array_equal(x, y)
    assert (fam == TS_FUSED_QUANT) == fused
    # and against the oracle on a sample of rows
    rows = np.unique(np.linspace(0, m - 1, min(m, 48)).astype(np.int64))
    q, sa, zp = oracle.quantize_a_per_row_asym(np.ascontiguousarray(a_np[rows]), ta_id)
    assert np.array_equal(one[1][rows], sa) and np.array_equal(one[2][rows], zp)
    bias = None
    if layer.bias is not None:
        bias = layer.bias.cpu().numpy() if td == "f32" else bits16(layer.bias)
    lo, hi = layer.clamp
    if td == "bf16":
        lo, hi = (float(torch.tensor(v).to(torch.bfloat16)) for v in (lo, hi))
    want = oracle.gemm_w4a8(q, nib, sa, zp, sb, TDI[td], None, bias, (lo, hi))
    assert np.array_equal(one[3][rows], want)


def test_fused_in_cuda_graph(oracle):
    """The cooperative launch captured into a CUDA graph and replayed on fresh activations each time: the barrier's
    state lives in device memory, so every replay finds it as the one before left it."""
    m, n, k = 640, 768, 1536
    layer, nib, sb = _layer(oracle, n, k, "bf16", 91, with_bias=True)
    _, a0, _ = _activations(oracle, m, k, "bf16", 6)
    a_in = a0.clone()
    layer.fuse_quant = True
    fn = layer.captured(a_in)
    plain, _, _ = _layer(oracle, n, k, "bf16", 91, with_bias=True)
    for seed in (6, 7, 8):
        _, a_new, _ = _activations(oracle, m, k, "bf16", seed)
        a_in.copy_(a_new)
        out = fn()
        sync_and_check()
        want = plain(a_new)
        sync_and_check()
        assert np.array_equal(bits16(out), bits16(want))


def test_fused_repeated_and_interleaved(oracle):
    """Fifty fused launches back to back with a two-launch call in between every tenth: the barrier words return to
    their resting state after every launch."""
    m, n, k = 400, 520, 1024
    layer, _, _ = _layer(oracle, n, k, "f16", 33, with_bias=False)
    _, a_dev, _ = _activations(oracle, m, k, "f16", 9)
    layer.fuse_quant = False
    want = bits16(layer(a_dev)).copy()
    sync_and_check()
    layer.fuse_quant = True
    for i in range(50):
        if i % 10 == 9:
            layer.fuse_quant = False
            layer(a_dev)
            layer.fuse_quant = True
        out = layer(a_dev)
    sync_and_check()
    assert np.array_equal(bits16(out), want)
