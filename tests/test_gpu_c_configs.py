"""The five benchmark configurations at their full sizes, on seeded synthetic inputs with the stated
distributions.  Inputs come from std::mt19937 with the seeds of the reference's runners (42 for
activations, 123 for weights and weight scales, 7 for bias; test/common/quantized_gemm_test_runner.h:136,
1051, 1060, 1082) through the oracle's generators: the uniform ones reproduce the reference's
UniformRandomGenerator stream for stream, the normal ones are std::normal_distribution<float> on the same
engine (the reference has no normal generator).

The CPU oracle finishes only a sample at these sizes, so each test compares at least 128 whole output rows
(first / last rows of the first and last tiles of every tile height in use, plus seeded random ones) and at
least 64 whole output columns (same choice) against the oracle, checks the quantised activations in full,
and checks that no output cell was left unwritten.
"""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import (DEV, FMAX, bf16_bits_to_f32, bits16, cosine, f16_bits_to_f32, f32_to_bf16_bits, from_bits16,
                         pkg, rel_err, run_i32_unpacked, sync_and_check, to_dev)
from __graft_entry__ import load_linear

pytestmark = pytest.mark.gpu

SEED_A, SEED_B, SEED_BIAS = 42, 123, 7


def _sample(extent, rng, total):
    """Indices along one output dimension: both edges of the first and last tiles (tile heights 128, 192
    and 256 are all in use), then seeded random ones up to ``total``."""
    fixed = [0, 1, 127, 128, 191, 192, 255, 256, extent - 257, extent - 256, extent - 193, extent - 192,
             extent - 129, extent - 128, extent - 2, extent - 1]
    idx = set(i for i in fixed if 0 <= i < extent)
    while len(idx) < min(total, extent):
        idx.add(int(rng.integers(0, extent)))
    return np.array(sorted(idx))


def test_config1_w8a8_i32(oracle):
    """M=64, K=512, N=256; the reference's generator: int8 U[-128,127], seed 42 for A, 123 for B."""
    A = oracle.fill_uniform((64, 512), np.int8, -128, 127, SEED_A)
    B = oracle.fill_uniform((512, 256), np.int8, -128, 127, SEED_B)
    assert np.array_equal(run_i32_unpacked(A, B), oracle.gemm_clamp_i32_i8_i8(A, B, False))


def test_config2_decode_gemv(oracle):
    """M=1, K=4096, N=4096: f32 activations ~N(0,1), weights ~N(0,0.02) -> int4, bias ~N(0,0.1), f32 out."""
    lin = load_linear()
    a = oracle.fill_normal((1, 4096), 0.0, 1.0, SEED_A)
    W = oracle.fill_normal((4096, 4096), 0.0, 0.02, SEED_B)
    bias = oracle.fill_normal((4096,), 0.0, 0.1, SEED_BIAS)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), 4096, "f32", bias=to_dev(bias))
    out = layer(to_dev(a))
    sync_and_check()
    q, sa, zp = oracle.quantize_a_per_row_asym(a)
    want = oracle.gemm_w4a8(q, nib, sa, zp, sb, TD_F32, None, bias, (-FMAX, FMAX))
    got = out.cpu().numpy()
    assert np.array_equal(got, want)
    assert rel_err(got, want) <= 1e-3      # the stated bar for f32 outputs
    assert pkg().lib().tqt_cuda_kernel_choice_w4a8(1, 4096, 4096) == 1


def test_config3_prefill_w4a8_bf16(oracle):
    """M=2048, K=4096, N=14336 (Llama-3-8B MLP up-projection shape), bf16 in / out, zero bias, clamp +-65504."""
    lin = load_linear()
    rng = np.random.default_rng(3)
    m, k, n = 2048, 4096, 14336
    a_bits = f32_to_bf16_bits(oracle.fill_normal((m, k), 0.0, 1.0, SEED_A))
    a_dev = from_bits16(a_bits, torch.bfloat16)
    W = oracle.fill_normal((n, k), 0.0, 0.02, SEED_B)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    del W
    bias = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16", bias=bias, clamp=(-65504.0, 65504.0))
    ws = layer.workspace(m)
    ws["out"].fill_(float("nan"))
    out = layer(a_dev)
    sync_and_check()
    # quantised activations: every element
    q, sa, zp = oracle.quantize_a_per_row_asym(a_bits, TD_BF16)
    back = torch.zeros((m, k), dtype=torch.int8, device=DEV)
    pkg().a_unpack_i8(m, k, ws["a_packed"], k, back, k)
    sync_and_check()
    assert np.array_equal(back.cpu().numpy(), q)
    assert np.array_equal(ws["scale_a"].cpu().numpy(), sa) and np.array_equal(ws["zp_a"].cpu().numpy(), zp)
    assert not torch.isnan(out).any()
    # bf16(65504) is 65536: the kernel clamps at the value the bf16 argument holds
    clamp = (-65536.0, 65536.0)
    rows = _sample(m, rng, 128)
    want = oracle.gemm_w4a8(np.ascontiguousarray(q[rows]), nib, np.ascontiguousarray(sa[rows]),
                            np.ascontiguousarray(zp[rows]), sb, TD_BF16, None, np.zeros(n, np.uint16), clamp)
    got = bits16(out[torch.from_numpy(rows).to(DEV)])
    assert np.array_equal(got, want)
    assert rel_err(bf16_bits_to_f32(got), bf16_bits_to_f32(want)) <= 2e-2      # the stated bar
    cols = _sample(n, rng, 64)
    want = oracle.gemm_w4a8(q, np.ascontiguousarray(nib[cols]), sa, zp, np.ascontiguousarray(sb[cols]), TD_BF16, None,
                            np.zeros(len(cols), np.uint16), clamp)
    got = bits16(out[:, torch.from_numpy(cols).to(DEV)])
    assert np.array_equal(got, want)


def test_config4_static_w8a8_requant(oracle):
    """M=K=N=4096, activations int8 U[-128,127] with scale_a 0.05, zp_a 3 (fused into the bias as the
    reference's callers do), weights int8 U[-127,127], per-channel scales U(0.001,0.01), int32 bias
    U(-1000,1000), output scale 0.1, zero point -5, clamp [-128,127]; plus the same problem with an output
    scale that keeps the results inside the int8 range."""
    lin = load_linear()
    rng = np.random.default_rng(4)
    m = k = n = 4096
    A = oracle.fill_uniform((m, k), np.int8, -128, 127, SEED_A)
    W = oracle.fill_uniform((n, k), np.int8, -127, 127, SEED_B)
    sb = oracle.fill_uniform((n,), np.float32, 0.001, 0.01, SEED_B)
    bias = oracle.fill_uniform((n,), np.int32, -1000, 1000, SEED_BIAS)
    fused = oracle.fuse_zp_to_bias(bias, W, 3)
    rows, cols = _sample(m, rng, 128), _sample(n, rng, 64)
    a_dev = to_dev(A)
    # the real-valued result the int8 output stands for, on the sampled rows; its range gives the third output scale
    # the way the reference's runner derives scale_d / zero_point_d (quantized_gemm_test_runner.h:37-65, 262-265)
    real = (A[rows].astype(np.float64) - 3.0) @ W.T.astype(np.float64) * np.float64(np.float32(0.05)) * sb.astype(np.float64)[None, :]
    real += bias.astype(np.float64)[None, :] * np.float64(np.float32(0.05)) * sb.astype(np.float64)[None, :]
    fmin, fmax = min(real.min(), 0.0), max(real.max(), 0.0)
    scale_fit = float(np.float32((fmax - fmin) / 255.0))
    zp_fit = int(np.rint(-128.0 - fmin / scale_fit))
    for scale_d, zp_d in ((0.1, -5), (30.0, -5), (scale_fit, zp_fit)):
        layer = lin.W8A8RequantLinear(to_dev(W), to_dev(sb), 0.05, 3, scale_d, zp_d, to_dev(fused))
        layer.workspace(m)["out"].fill_(99)
        out = layer(a_dev)
        sync_and_check()
        want = oracle.gemm_reqi32toi8(np.ascontiguousarray(A[rows]), W, True, 0.05, sb, scale_d, zp_d, fused)
        got = out[torch.from_numpy(rows).to(DEV)].cpu().numpy()
        assert np.array_equal(got, want)
        want_c = oracle.gemm_reqi32toi8(A, np.ascontiguousarray(W[cols]), True, 0.05, np.ascontiguousarray(sb[cols]),
                                        scale_d, zp_d, np.ascontiguousarray(fused[cols]))
        got_c = out[:, torch.from_numpy(cols).to(DEV)].cpu().numpy()
        assert np.array_equal(got_c, want_c)
        if scale_d == 30.0:
            assert (np.abs(want.astype(np.int32)) < 127).mean() > 0.9
        if scale_d == scale_fit:
            # the reference's own acceptance test of this kernel type (quantized_gemm_test_runner.h:193-306): the
            # dequantised int8 output against the real-valued GEMM, cosine 0.999 and a bound on the absolute error
            # (there 1.0 on results of magnitude ~10 with steps of ~0.05; here two output steps: the requantisation
            # floors twice, it does not round)
            deq = (got.astype(np.float64) - zp_fit) * scale_fit
            assert np.max(np.abs(deq - real)) <= 2.0 * scale_fit
            assert cosine(deq, real) >= 0.999


@pytest.mark.parametrize("shards", [1, 8])
def test_config5_w4a16_block_quant(oracle, shards):
    """M=8192, K=8192, N=28672 (Llama-3-70B MLP shape), bl=32, f16 in / out, bias ~N(0,0.1), clamp +-65504.
    shards=8 runs the per-GPU slice of the 8-way column split (N/8 = 3584) as rank 3 would."""
    lin = load_linear()
    rng = np.random.default_rng(5)
    m, k, n_full, bl = 8192, 8192, 28672, 32
    n0, n = pkg().shard_plan_n(n_full, shards, 3 % shards)
    A = oracle.fill_normal((m, k), 0.0, 1.0, SEED_A).astype(np.float16)
    # the weight stream is drawn for the whole matrix so that a shard holds the rows the full problem has
    W = oracle.fill_normal((n_full, k), 0.0, 0.02, SEED_B)[n0:n0 + n].astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    del W
    bias = oracle.fill_normal((n_full,), 0.0, 0.1, SEED_BIAS)[n0:n0 + n].astype(np.float16)
    layer = lin.W4A16Linear(to_dev(nib), from_bits16(sc, torch.float16), k, bl, "f16", bias=to_dev(bias))
    layer.workspace(m)["out"].fill_(float("nan"))
    out = layer(to_dev(A))
    sync_and_check()
    assert not torch.isnan(out).any()

    def check(got, want):
        g, w = f16_bits_to_f32(got), f16_bits_to_f32(want)
        assert rel_err(g, w) <= 2e-2                                   # the stated bar (RMS floor)
        assert np.max(np.abs(g - w)) <= 1.0 and cosine(g, w) >= 0.9999   # the reference's own thresholds

    rows = _sample(m, rng, 128)
    want = oracle.gemm_w4a16(np.ascontiguousarray(A[rows]).view(np.uint16), nib, sc, bl, TD_F16, None, bias.view(np.uint16))
    check(bits16(out[torch.from_numpy(rows).to(DEV)]), want)
    cols = _sample(n, rng, 64)
    want = oracle.gemm_w4a16(A.view(np.uint16), np.ascontiguousarray(nib[cols]), np.ascontiguousarray(sc[cols]), bl, TD_F16,
                             None, np.ascontiguousarray(bias[cols]).view(np.uint16))
    check(bits16(out[:, torch.from_numpy(cols).to(DEV)]), want)
