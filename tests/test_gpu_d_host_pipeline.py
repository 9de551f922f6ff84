"""forward_host(): the operators' pinned-host entry point (row chunks pipelined on three streams)
must give exactly what the device-resident call gives, also when called repeatedly (the chunk
buffers and events of one call are reused by the next)."""
import numpy as np
import pytest
import torch

from tqt_testlib import DEV, sync_and_check, to_dev
from __graft_entry__ import load_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,chunks", [(300, 2), (1024, 4), (130, 4), (64, 1)])
def test_w4a8_forward_host_matches_device_call(oracle, m, chunks):
    lin = load_linear()
    rng = np.random.default_rng(m)
    n, k = 384, 512
    W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16", bias=to_dev(rng.normal(0, 0.1, n).astype(np.float32)))
    out_host = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    a_host = torch.empty((m, k), dtype=torch.bfloat16).pin_memory()
    for rep in range(4):   # call 0 runs eagerly and captures, later calls replay the graph on new contents
        a_host.copy_(torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).to(torch.bfloat16))
        layer.forward_host(a_host, out_host, chunks=chunks, graph=(rep != 3))
        torch.cuda.current_stream().synchronize()
        got = out_host.clone()
        want = layer(a_host.to(DEV)).cpu()
        sync_and_check()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {rep}"


def test_requant_forward_host_matches_device_call():
    lin = load_linear()
    rng = np.random.default_rng(5)
    m, n, k = 520, 256, 384
    w = torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).to(DEV)
    sb = torch.from_numpy(rng.uniform(0.001, 0.01, n).astype(np.float32)).to(DEV)
    bias = torch.from_numpy(rng.integers(-1000, 1000, n, dtype=np.int32)).to(DEV)
    layer = lin.W8A8RequantLinear(w, sb, 0.05, 3, 0.1, -5, bias_fused=bias)
    a_host = torch.from_numpy(rng.integers(-128, 128, (m, k), dtype=np.int8)).pin_memory()
    out_host = torch.empty((m, n), dtype=torch.int8).pin_memory()
    for _ in range(3):
        out_host.zero_()
        layer.forward_host(a_host, out_host, chunks=3)
        torch.cuda.current_stream().synchronize()
        want = layer(a_host.to(DEV)).cpu()
        sync_and_check()
        assert torch.equal(out_host, want)


def test_captured_graph_matches_eager_call(oracle):
    """captured(A): CUDA-graph replay of prepare + run_gemm (and of run_gemm alone) on new contents of A."""
    lin = load_linear()
    rng = np.random.default_rng(11)
    m, n, k = 300, 384, 512
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16")
    a = torch.empty((m, k), dtype=torch.bfloat16, device=DEV)
    step = layer.captured(a)
    gemm = layer.captured(a, gemm_only=True)
    for _ in range(3):
        a.copy_(torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).to(torch.bfloat16))
        got = step().clone()
        again = gemm().clone()      # the packed activations of the step are still in the workspace
        want = layer(a).clone()
        sync_and_check()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        assert torch.equal(again.view(torch.int16), want.view(torch.int16))
