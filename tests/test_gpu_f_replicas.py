"""tqt_cuda_set_output_replicas: the tensor-core W4A8 / W4A16 kernels also store every output element at
the same offset inside each replica buffer (on one GPU the replicas are ordinary local buffers; across
GPUs they are peer-mapped copies of the output).  Other kernel paths must refuse loudly while replicas
are set."""
import numpy as np
import pytest
import torch

from tqt_testlib import DEV, sync_and_check, to_dev
from __graft_entry__ import load, load_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [40, 300])   # single-CTA and CTA-pair tensor-memory kernels
def test_w4a8_stores_replicas_of_a_column_shard(oracle, m):
    pkg, lin = load(), load_linear()
    rng = np.random.default_rng(m)
    n_total, n0, n, k = 640, 128, 384, 512   # this "rank" owns columns [128, 512) of a 640-column output
    W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(W)
    layer = lin.W4A8Linear(to_dev(nib), to_dev(sb), k, "bf16")
    a = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    want = layer(a).clone()
    bufs = [torch.full((m, n_total), 5.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    nbytes = bufs[0].numel() * 2
    with pkg.output_replicas(bufs[0].data_ptr(), nbytes, [b.data_ptr() for b in bufs[1:]]):
        layer.quantize(a)
        layer.gemm(m, out=bufs[0][:, n0:n0 + n])
        sync_and_check()
        # an output that is not inside the registered buffer is refused and nothing is launched
        stray = torch.full((m, n), 3.0, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(pkg.TqtError):
            layer.gemm(m, out=stray)
        sync_and_check()
        assert torch.all(stray == 3.0)
    for b in bufs:
        assert torch.equal(b[:, n0:n0 + n].view(torch.int16), want.view(torch.int16))
        assert torch.all(b[:, :n0] == 5.0) and torch.all(b[:, n0 + n:] == 5.0)


def test_other_paths_refuse_replicas():
    pkg = load()
    uk = pkg.GemmClampI32I8I8()
    a = torch.zeros((8, 16), dtype=torch.int8, device=DEV)
    b = torch.zeros((16, 8), dtype=torch.int8, device=DEV)
    d = torch.zeros((8, 8), dtype=torch.int32, device=DEV)
    other = torch.zeros((8, 8), dtype=torch.int32, device=DEV)
    with pkg.output_replicas(d.data_ptr(), d.numel() * 4, [other.data_ptr()]):
        with pytest.raises(pkg.TqtError):
            uk.run_gemm(8, 8, 16, a, 16, 0, b, 8, 0, None, 8, d, 8, -2**31, 2**31 - 1)
    uk.run_gemm(8, 8, 16, a, 16, 0, b, 8, 0, None, 8, d, 8, -2**31, 2**31 - 1)
    sync_and_check()
