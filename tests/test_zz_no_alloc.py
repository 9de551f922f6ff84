"""The quantise + W4A8 GEMM entry point that allocates nothing and takes no workspace
(tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp, include/tqt_b200_ext.h).  It exists for plug-ins that cannot
get device memory of their own: code running inside a server whose memory pool has taken the whole GPU, or in a loop that
must not pay for cudaMalloc's synchronisation.  Its intermediates live in a static device array of the library, shared by
all calls, so the test runs two calls in a row (the second one smaller, over what the first one left behind) and wants
each output to equal, bit for bit, what the existing entry points (quantiser, then run_gemm, with caller-owned buffers)
produce.  Collected last on purpose: a run that stops at the first failure has then run every other test."""
import numpy as np
import pytest
import torch

from tqt_testlib import DEV, f32_to_bf16_bits, from_bits16, load_linear, pkg, sync_and_check, to_dev

pytestmark = pytest.mark.gpu


def _weights(oracle, n, k, seed):
    W = oracle.fill_normal((n, k), 0.0, 0.02, seed)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    return to_dev(nib), to_dev(sb)


def _acts(oracle, m, k, ta, seed):
    x = oracle.fill_normal((m, k), 0.0, 1.0, seed)
    if ta == "f32":
        return to_dev(x)
    if ta == "f16":
        return to_dev(x.astype(np.float16))
    return from_bits16(f32_to_bf16_bits(x), torch.bfloat16)


def test_static_entry_matches_existing_entry_on_two_calls(oracle):
    p = pkg()
    lin = load_linear()
    p.use_current_torch_stream()
    # (m, n, k, activation type): a prefill-sized call, then smaller ones that reuse the array (ragged sizes, the decode GEMV)
    calls = [(700, 520, 2048, "bf16"), (133, 260, 528, "f16"), (4, 384, 1024, "f32"), (700, 520, 2048, "bf16")]
    for i, (m, n, k, ta) in enumerate(calls):
        nib, sb = _weights(oracle, n, k, 100 + i)
        bias = to_dev(oracle.fill_normal((n,), 0.0, 0.1, 200 + i))
        a = _acts(oracle, m, k, ta, 300 + i)
        layer = lin.W4A8Linear(nib, sb, k, "f32", bias=bias, clamp=(-3.0, 4.0))
        want = layer(a).clone()                      # existing entry points, buffers owned by the caller
        sync_and_check()
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        p.quant_gemm_w4a8_static(m, n, k, a, a.stride(0), layer.b_packed, k, None, n, got, n, bias, -3.0, 4.0, sb)
        sync_and_check()
        assert torch.equal(got, want), f"call {i}"
        # tolerance of the f32-output tests, for the record: bit equality implies it
        assert float((got - want).abs().max()) <= 1e-3 * float(want.abs().max())


def test_static_entry_refuses_calls_beyond_its_array():
    p = pkg()
    p.use_current_torch_stream()
    n, k = 128, 4096
    for m in (8193, 4096):          # too many rows; packed activations of 16 MiB
        a = torch.zeros((m, k), dtype=torch.bfloat16, device=DEV)
        uk = p.GemmW4A8("f32")
        b_packed = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
        sb = torch.ones(n, dtype=torch.float32, device=DEV)
        out = torch.full((m, n), 5.0, dtype=torch.float32, device=DEV)
        with pytest.raises(p.TqtError, match="UNSUPPORTED"):
            p.quant_gemm_w4a8_static(m, n, k, a, k, b_packed, k, None, n, out, n, None, -1.0, 1.0, sb)
        sync_and_check()
        assert bool((out == 5.0).all())             # nothing was launched
