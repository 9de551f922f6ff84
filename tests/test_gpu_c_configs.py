"""The five benchmark configurations at their full sizes, on seeded synthetic inputs with the stated
distributions.  The CPU oracle finishes only a sample of rows at these sizes, so each test compares
a spread of output rows (first / last row of the first and last tile, and random ones) against the
oracle, checks the quantised activations in full, and checks that no output cell was left unwritten.
"""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16, TD_F16, TD_F32
from tqt_testlib import (DEV, FMAX, bits16, f16_bits_to_f32, from_bits16, pkg, rel_err, run_i32_unpacked, sync_and_check,
                         to_dev)
from __graft_entry__ import load_linear

pytestmark = pytest.mark.gpu


def _rows(m, rng, extra=8):
    fixed = [0, 1, 127, 128, m - 129, m - 128, m - 1]
    rows = sorted(set(r for r in fixed if 0 <= r < m) | set(int(x) for x in rng.integers(0, m, extra)))
    return np.array(rows)


def test_config1_w8a8_i32(oracle):
    rng = np.random.default_rng(42)
    A = rng.integers(-128, 128, (64, 512), dtype=np.int8)
    B = rng.integers(-128, 128, (512, 256), dtype=np.int8)
    assert np.array_equal(run_i32_unpacked(A, B), oracle.gemm_clamp_i32_i8_i8(A, B, False))


def test_config2_decode_gemv(oracle):
    """M=1, K=4096, N=4096: f32 activations ~N(0,1), weights ~N(0,0.02) -> int4, bias ~N(0,0.1), f32 out."""
    lin = load_linear()
    rng = np.random.default_rng(2)
    a = rng.normal(0, 1, (1, 4096)).astype(np.float32)
    W = rng.normal(0, 0.02, (4096, 4096)).astype(np.float32)
    bias = rng.normal(0, 0.1, 4096).astype(np.float32)
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
    """M=2048, K=4096, N=14336 (Llama-3-8B MLP up-projection shape), bf16 in / out, zero bias."""
    lin = load_linear()
    rng = np.random.default_rng(3)
    m, k, n = 2048, 4096, 14336
    a_dev = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    del W
    bias = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16", bias=bias)
    ws = layer.workspace(m)
    ws["out"].fill_(float("nan"))
    out = layer(a_dev)
    sync_and_check()
    # quantised activations: every element
    q, sa, zp = oracle.quantize_a_per_row_asym(bits16(a_dev), TD_BF16)
    back = torch.zeros((m, k), dtype=torch.int8, device=DEV)
    pkg().a_unpack_i8(m, k, ws["a_packed"], k, back, k)
    sync_and_check()
    assert np.array_equal(back.cpu().numpy(), q)
    assert np.array_equal(ws["scale_a"].cpu().numpy(), sa) and np.array_equal(ws["zp_a"].cpu().numpy(), zp)
    assert not torch.isnan(out).any()
    rows = _rows(m, rng)
    # bf16(65504) is 65536: the kernel clamps at the value the bf16 argument holds
    want = oracle.gemm_w4a8(np.ascontiguousarray(q[rows]), nib, np.ascontiguousarray(sa[rows]),
                            np.ascontiguousarray(zp[rows]), sb, TD_BF16, None, np.zeros(n, np.uint16), (-65536.0, 65536.0))
    got = bits16(out[torch.from_numpy(rows).to(DEV)])
    assert np.array_equal(got, want)


def test_config4_static_w8a8_requant(oracle):
    """M=K=N=4096, scale_a 0.05, zp_a 3 (fused into the bias), per-channel scales U(0.001,0.01),
    int32 bias U(-1000,1000), output scale 0.1, zero point -5, clamp [-128,127]; plus the same
    problem with an output scale that keeps the results inside the int8 range."""
    lin = load_linear()
    rng = np.random.default_rng(4)
    m = k = n = 4096
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    W = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sb = rng.uniform(0.001, 0.01, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    fused = oracle.fuse_zp_to_bias(bias, W, 3)
    rows = _rows(m, rng)
    a_dev = to_dev(A)
    for scale_d in (0.1, 30.0):
        layer = lin.W8A8RequantLinear(to_dev(W), to_dev(sb), 0.05, 3, scale_d, -5, to_dev(fused))
        layer.workspace(m)["out"].fill_(99)
        out = layer(a_dev)
        sync_and_check()
        want = oracle.gemm_reqi32toi8(np.ascontiguousarray(A[rows]), W, True, 0.05, sb, scale_d, -5, fused)
        got = out[torch.from_numpy(rows).to(DEV)].cpu().numpy()
        assert np.array_equal(got, want)
        if scale_d == 30.0:
            assert (np.abs(want.astype(np.int32)) < 127).mean() > 0.9


@pytest.mark.parametrize("shards", [1, 8])
def test_config5_w4a16_block_quant(oracle, shards):
    """M=8192, K=8192, N=28672 (Llama-3-70B MLP shape), bl=32, f16 in / out, bias ~N(0,0.1).
    shards=8 runs the per-GPU slice of the 8-way column split (N/8 = 3584) as rank 3 would."""
    lin = load_linear()
    rng = np.random.default_rng(5)
    m, k, n_full, bl = 8192, 8192, 28672, 32
    n0, n = pkg().shard_plan_n(n_full, shards, 3 % shards)
    A = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    W = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    nib, sc = oracle.quantize_fp16_to_int4(W.view(np.uint16), bl)
    del W
    bias = rng.normal(0, 0.1, n).astype(np.float16)
    layer = lin.W4A16Linear(to_dev(nib), from_bits16(sc, torch.float16), k, bl, "f16", bias=to_dev(bias))
    layer.workspace(m)["out"].fill_(float("nan"))
    out = layer(to_dev(A))
    sync_and_check()
    assert not torch.isnan(out).any()
    rows = _rows(m, rng, extra=2)[:6]
    want = oracle.gemm_w4a16(np.ascontiguousarray(A[rows]).view(np.uint16), nib, sc, bl, TD_F16, None, bias.view(np.uint16))
    got = bits16(out[torch.from_numpy(rows).to(DEV)])
    g, w = f16_bits_to_f32(got), f16_bits_to_f32(want)
    assert rel_err(g, w) <= 2e-2
    assert np.max(np.abs(g - w)) <= 1.0
