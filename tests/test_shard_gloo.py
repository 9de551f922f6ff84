"""The N > 1 path on CPU: two gloo ranks shard the weight matrix by columns with tqt_shard_plan_n,
each computes its slice (the CPU oracle stands in for the device kernels, which need a GPU), and an
all-gather of the column shards must reproduce the unsharded result.  This checks the host-side
logic that bench.py --gpus N relies on: the plan, the per-shard params / bias slicing and the
staging layout of the gather."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, m, out_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load
    from oracle.tqo import TD_F32, Oracle
    pkg, orc = load(), Oracle()
    orc.set_threads(1)
    rng = np.random.default_rng(0)      # same inputs on every rank
    A = rng.normal(0, 1, (m, k)).astype(np.float32)
    W = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    bias = rng.normal(0, 0.1, n).astype(np.float32)
    q, sa, zp = orc.quantize_a_per_row_asym(A)
    nib, sb = orc.quantize_b_per_channel_sym_int4(W)
    n0, nc = pkg.shard_plan_n(n, world, rank)
    mine = orc.gemm_w4a8(q, np.ascontiguousarray(nib[n0:n0 + nc]), sa, zp, np.ascontiguousarray(sb[n0:n0 + nc]), TD_F32,
                         None, np.ascontiguousarray(bias[n0:n0 + nc]))
    # equal shard sizes here (n is a multiple of 128 * world): gather into [world * m, n/world]
    staging = torch.empty((world * m, nc), dtype=torch.float32)
    dist.all_gather_into_tensor(staging, torch.from_numpy(mine))
    full = staging.reshape(world, m, nc).permute(1, 0, 2).reshape(m, n).numpy()
    if rank == 0:
        want = orc.gemm_w4a8(q, nib, sa, zp, sb, TD_F32, None, bias)
        np.save(out_path, np.array([np.array_equal(full, want)]))
    dist.destroy_process_group()


def test_two_rank_column_shards_reassemble(tmp_path):
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(2, _free_port(), 512, 64, 9, out), nprocs=2, join=True)
    assert bool(np.load(out)[0])
