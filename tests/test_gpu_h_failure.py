"""Failure path of the tensor-core kernels: a bounded wait that runs out.

Every wait inside the kernels has a limit; when one runs out the kernel records a code, stops issuing work,
lets its copies land, frees its tensor memory and returns.  The failure is made on the host side of the
pipeline: a test knob (tqt_cuda_debug_inject_wait_failure) shortens the limits to about a millisecond and
makes one producer warp withhold the copies and the barrier arrive of its first stage, i.e. a flag that
nothing sets.  Nothing traps, faults or spins without a limit, and the context stays usable: the next call
must succeed and be correct.
"""
import numpy as np
import pytest
import torch

from oracle.tqo import TD_BF16
from tqt_testlib import DEV, bits16, from_bits16, f32_to_bf16_bits, pkg, to_dev

pytestmark = pytest.mark.gpu

WAIT_CODES = {0x200, 0x300, 0x400, 0x500}   # MMA issuer, epilogue or converter: whichever limit ran out first


@pytest.mark.parametrize("umma,m", [("pair", 300), ("ts", 200)])
def test_wait_runs_out_and_the_next_call_succeeds(oracle, force_path, umma, m):
    p = pkg()
    uk = p.GemmW4A8("bf16")
    p.use_current_torch_stream()
    force_path("umma", umma)
    rng = np.random.default_rng(m)
    n, k = 384, 512
    A = rng.integers(-128, 128, (m, k), dtype=np.int8)
    nib, sb = oracle.quantize_b_per_channel_sym_int4(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    sa = rng.uniform(0.01, 0.05, m).astype(np.float32)
    zp = rng.integers(-30, 30, m).astype(np.int32)
    ap = torch.zeros(uk.get_a_packed_size(m, k), dtype=torch.uint8, device=DEV)
    bp = torch.zeros(uk.get_b_packed_size(n, k), dtype=torch.uint8, device=DEV)
    uk.run_a_pack(m, k, k, k, 0, to_dev(A), ap)
    uk.run_bt_pack(n, k, k, k, 0, to_dev(nib), bp)
    sa_d, zp_d, sb_d = to_dev(sa), to_dev(zp), to_dev(sb)
    params = p.QaI8DxQsI4CxParams(sa_d.data_ptr(), zp_d.data_ptr(), sb_d.data_ptr())
    canary = f32_to_bf16_bits(np.full((m, n), 7.0, np.float32))
    d = from_bits16(canary, torch.bfloat16)

    def run():
        uk.run_gemm(m, n, k, ap, k, 0, bp, k, 0, None, n, d, n, None, -65504.0, 65504.0, params)
        torch.cuda.synchronize()

    assert p.read_device_fault() == 0
    p.debug_inject_wait_failure(10, 1)
    try:
        run()                                   # returns: the waits downstream of the withheld stage run out
    finally:
        p.debug_inject_wait_failure(0, 0)
    fault = p.read_device_fault()
    assert fault in WAIT_CODES, hex(fault)
    assert np.array_equal(bits16(d), canary)    # no tile was stored
    assert p.read_device_fault() == 0           # reading the fault word clears it
    run()                                       # same context, same buffers: normal operation again
    assert p.read_device_fault() == 0
    want = oracle.gemm_w4a8(A, nib, sa, zp, sb, TD_BF16, None, None, (-65536.0, 65536.0))
    assert np.array_equal(bits16(d), want)
