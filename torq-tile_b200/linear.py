"""Caller-side composition of the micro-kernels into linear operators.

The reference leaves memory, packing and tiling loops to its caller (an ML runtime; in-tree the
test runners, e.g. test/gemm/test_gemm_i8_i4_rvv.cpp:325-421: quantise A, size and fill the packed
buffers, one whole-problem run_gemm).  These classes are that caller for a GPU: they own the device
buffers (torch tensors), pack the weights once, and per call run  quantise+pack -> run_gemm  through
the C ABI.  They add no arithmetic of their own.
"""
from __future__ import annotations

import torch

from . import (GemmReqI8, GemmW4A8, GemmW4A16, QaI8DxQsI4CxParams, QaI8QaI8QsI8CxParams, quant_gemm_w4a8, quant_pack_qai8dxp,
               use_current_torch_stream)

_TORCH_TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
FLT_MAX = 3.4028234663852886e38
BF16_MAX = 3.3895313892515355e38   # largest finite bf16
F16_MAX = 65504.0
# "no clamp" per output type: the largest finite value of the type (bf16 has the f32 exponent range,
# so the f16 maximum would saturate it at +-65536)
_NO_CLAMP = {"f32": (-FLT_MAX, FLT_MAX), "f16": (-F16_MAX, F16_MAX), "bf16": (-BF16_MAX, BF16_MAX)}


class _HostPipelined:
    """Host-memory entry point shared by the operators: ``forward_host(a_host, out_host)``.

    The rows of A are processed in chunks on three streams (host->device copy, prepare + run_gemm,
    device->host copy), so the copies of one chunk overlap the kernels and the opposite-direction
    copies of its neighbours; PCIe is full duplex.  Stream-ordered like any asynchronous torch
    operation: the call returns once everything is enqueued, and the calling stream waits for the
    last copy, so ``torch.cuda.current_stream().synchronize()`` (or an event) completes the call.
    Both host tensors must be pinned.  ``prepare`` is the operator's quantise+pack or pack step.
    """

    def captured(self, A, gemm_only=False):
        """A callable that replays, on the current stream, a CUDA graph of ``prepare(A)`` + ``gemm`` (or of
        the GEMM alone) for this very input tensor: the per-call host work (argument marshalling, two
        launches) drops to one graph launch, which matters once a call takes less GPU time than the host
        needs to issue it (column shards on several GPUs).  The result is the workspace's output tensor,
        available as ``.out`` on the callable.  A must stay alive and in place."""
        m = A.shape[0]
        key = ("captured", A.data_ptr(), m, bool(gemm_only), bool(getattr(self, "fuse_quant", False)))
        fn = self._ws.get(key)
        if fn is None:
            self.prepare(A)          # allocates the workspace, leaves a valid packed A for a GEMM-only graph
            out = self.gemm(m)
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                if gemm_only:
                    self.gemm(m)
                else:
                    self.step(A)

            def fn():
                g.replay()
                return out
            fn.out = out
            fn.graph = g
            self._ws[key] = fn
        return fn

    def step(self, A):
        """prepare(A) + gemm: what one call of the operator enqueues."""
        self.prepare(A)
        return self.gemm(A.shape[0])

    def _pipe(self, m, chunks, in_dtype):
        key = ("pipe", m, chunks)
        st = self._ws.get(key)
        if st is None:
            dev = self.b_packed.device
            rows = -(-m // chunks)
            rows = -(-rows // 128) * 128   # whole row tiles per chunk
            bounds = [(r0, min(m, r0 + rows)) for r0 in range(0, m, rows)]
            st = dict(bounds=bounds,
                      a_dev=torch.empty((m, self.k), dtype=in_dtype, device=dev),
                      out_dev=torch.empty((m, self.n), dtype=self.out_dtype, device=dev),
                      s_in=torch.cuda.Stream(dev), s_run=torch.cuda.Stream(dev), s_out=torch.cuda.Stream(dev),
                      used=False)
            for mode in ("eager", "capture"):   # events recorded during a graph capture belong to that graph
                st[mode] = {name: [torch.cuda.Event() for _ in bounds] for name in ("loaded", "consumed", "computed", "copied")}
            self._ws[key] = st
        return st

    def _enqueue(self, a_host, out_host, st, cross_call):
        cur = torch.cuda.current_stream()
        st["s_in"].wait_stream(cur)
        st["s_run"].wait_stream(cur)
        st["s_out"].wait_stream(cur)
        chained = cross_call and st["used"]
        ev = st["eager" if cross_call else "capture"]
        for c, (r0, r1) in enumerate(st["bounds"]):
            with torch.cuda.stream(st["s_in"]):
                if chained:
                    st["s_in"].wait_event(ev["consumed"][c])   # the previous call has read this chunk
                st["a_dev"][r0:r1].copy_(a_host[r0:r1], non_blocking=True)
                ev["loaded"][c].record()
            with torch.cuda.stream(st["s_run"]):
                st["s_run"].wait_event(ev["loaded"][c])
                if chained:
                    st["s_run"].wait_event(ev["copied"][c])    # the previous call's result has left the device
                self.prepare(st["a_dev"][r0:r1])
                ev["consumed"][c].record()
                self.gemm(r1 - r0, out=st["out_dev"][r0:r1])
                ev["computed"][c].record()
            with torch.cuda.stream(st["s_out"]):
                st["s_out"].wait_event(ev["computed"][c])
                out_host[r0:r1].copy_(st["out_dev"][r0:r1], non_blocking=True)
                ev["copied"][c].record()
        if cross_call:
            st["used"] = True
        cur.wait_stream(st["s_out"])

    def forward_host(self, a_host, out_host, chunks=4, graph=True):
        """a_host [m, k] (pinned) -> out_host [m, n] (pinned).  With ``graph`` (default) the enqueued
        copies and kernels of a given (a_host, out_host) pair are captured once in a CUDA graph and
        replayed on later calls, which takes the per-chunk launch overhead off the host; the two
        tensors must then stay alive and in place for as long as the operator is used with them."""
        m = a_host.shape[0]
        st = self._pipe(m, chunks, a_host.dtype)
        if not graph:
            self._enqueue(a_host, out_host, st, cross_call=True)
            return out_host
        key = ("graph", a_host.data_ptr(), out_host.data_ptr(), m, chunks)
        g = self._ws.get(key)
        if g is None:
            self._enqueue(a_host, out_host, st, cross_call=True)   # allocates the workspaces; delivers this call
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue(a_host, out_host, st, cross_call=False)
            stale = [k2 for k2 in self._ws if isinstance(k2, tuple) and k2[0] == "graph"]
            for k2 in stale[:-7]:   # keep a handful of captured pairs
                del self._ws[k2]
            self._ws[key] = g
            return out_host
        g.replay()
        return out_host


class W4A8Linear(_HostPipelined):
    """D = clamp(dequant(quant(A)) * dequant(W)^T + bias): qai8dxp x qsi4cxp, float output.

    ``nib`` is the [n, k/2] uint8 weight in the reference's encoding (low nibble = even k, value
    q + 8); ``scale_b`` [n] f32; ``bias`` [n] in the output type.  Columns [n_begin, n_begin+n_count)
    only are packed when a shard is given (column-parallel use: each rank builds its own slice).
    """

    def __init__(self, nib, scale_b, k, out_dtype="bf16", bias=None, clamp=None):
        self.uk = GemmW4A8(out_dtype)
        self.out_name = out_dtype
        self.td = self.out_dtype = _TORCH_TD[out_dtype]
        self.n, self.k = nib.shape[0], k
        dev = nib.device
        use_current_torch_stream()
        self.b_packed = torch.empty(self.uk.get_b_packed_size(self.n, k), dtype=torch.uint8, device=dev)
        self.uk.run_bt_pack(self.n, k, k, k, 0, nib.contiguous(), self.b_packed)
        self.scale_b = scale_b.contiguous()
        self.bias = None if bias is None else bias.to(self.td).contiguous()
        self.clamp = _NO_CLAMP[out_dtype] if clamp is None else clamp
        self._ws = {}

    def workspace(self, m):
        ws = self._ws.get(m)
        if ws is None:
            dev = self.b_packed.device
            ws = dict(a_packed=torch.empty(self.uk.get_a_packed_size(m, self.k), dtype=torch.uint8, device=dev),
                      scale_a=torch.empty(m, dtype=torch.float32, device=dev),
                      zp_a=torch.empty(m, dtype=torch.int32, device=dev),
                      out=torch.empty((m, self.n), dtype=self.td, device=dev))
            ws["params"] = QaI8DxQsI4CxParams(ws["scale_a"].data_ptr(), ws["zp_a"].data_ptr(), self.scale_b.data_ptr())
            self._ws[m] = ws
        return ws

    def quantize(self, A):
        """Dynamic per-row quantisation + LHS pack of A [m, k] (f32 / f16 / bf16) into the workspace."""
        ws = self.workspace(A.shape[0])
        use_current_torch_stream()
        quant_pack_qai8dxp(A, ws["a_packed"], ws["scale_a"], ws["zp_a"])
        return ws

    def gemm(self, m, Cm=None, out=None):
        """run_gemm on the workspace of size m (after quantize()); returns the output tensor
        (the workspace's, or ``out`` [m, n] with any row stride)."""
        ws = self.workspace(m)
        out = ws["out"] if out is None else out
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, Cm, self.n, out,
                         out.stride(0), self.bias, self.clamp[0], self.clamp[1], ws["params"])
        return out

    prepare = quantize

    #: quantise + GEMM as ONE cooperative launch where the library has a fused form for the shape (16-bit activations,
    #: k <= 4096, more than 16 rows); the entry point runs the two kernels back to back otherwise
    fuse_quant = False

    def step(self, A, Cm=None):
        if not self.fuse_quant:
            self.quantize(A)
            return self.gemm(A.shape[0], Cm)
        m = A.shape[0]
        ws = self.workspace(m)
        use_current_torch_stream()
        quant_gemm_w4a8(self.out_name, m, self.n, self.k, A, A.stride(0), ws["a_packed"], ws["scale_a"], ws["zp_a"], self.b_packed,
                        self.k, Cm, self.n, ws["out"], ws["out"].stride(0), self.bias, self.clamp[0], self.clamp[1], self.scale_b)
        return ws["out"]

    def __call__(self, A, Cm=None):
        return self.step(A, Cm)


class W8A8RequantLinear(_HostPipelined):
    """Static W8A8 with int8 output: qai8 x qsi8cxp (weights [n, k] int8), int32 bias with the
    activation zero point already fused (bias - zp_a * sum_k w), as the reference's callers do."""

    def __init__(self, w_i8, scale_b, scale_a, zero_point_a, scale_d, zero_point_d, bias_fused=None, clamp=(-128, 127)):
        self.uk = GemmReqI8()
        self.out_dtype = torch.int8
        self.n, self.k = w_i8.shape
        dev = w_i8.device
        use_current_torch_stream()
        self.b_packed = torch.empty(self.uk.get_b_packed_size(self.n, self.k), dtype=torch.uint8, device=dev)
        self.uk.run_bt_pack(self.n, self.k, self.k, self.k, 0, w_i8.contiguous(), self.b_packed)
        self.scale_b = scale_b.contiguous()
        self.bias = bias_fused
        self.clamp = clamp
        self.params = QaI8QaI8QsI8CxParams(scale_a, zero_point_a, self.scale_b.data_ptr(), 0, scale_d, zero_point_d)
        self._ws = {}

    def workspace(self, m):
        ws = self._ws.get(m)
        if ws is None:
            dev = self.b_packed.device
            ws = dict(a_packed=torch.empty(self.uk.get_a_packed_size(m, self.k), dtype=torch.uint8, device=dev),
                      out=torch.empty((m, self.n), dtype=torch.int8, device=dev))
            self._ws[m] = ws
        return ws

    def pack(self, A_i8):
        ws = self.workspace(A_i8.shape[0])
        use_current_torch_stream()
        self.uk.run_a_pack(A_i8.shape[0], self.k, A_i8.stride(0), self.k, 0, A_i8, ws["a_packed"])
        return ws

    def gemm(self, m, Cm=None, out=None):
        ws = self.workspace(m)
        out = ws["out"] if out is None else out
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, Cm, self.n, out,
                         out.stride(0), self.bias, self.clamp[0], self.clamp[1], self.params)
        return out

    prepare = pack

    def __call__(self, A_i8, Cm=None):
        self.pack(A_i8)
        return self.gemm(A_i8.shape[0], Cm)


class W4A16Linear(_HostPipelined):
    """f16 activations x block-quantised int4 weights (qsi4c2, f16 scale per bl elements of k)."""

    def __init__(self, nib, scale_b, k, bl, out_dtype="f16", bias=None, clamp=None):
        self.uk = GemmW4A16(out_dtype)
        self.td = self.out_dtype = _TORCH_TD[out_dtype]
        self.n, self.k, self.bl = nib.shape[0], k, bl
        dev = nib.device
        use_current_torch_stream()
        self.b_packed = torch.empty(self.uk.get_b_packed_size(self.n, k), dtype=torch.uint8, device=dev)
        self.uk.run_bt_pack(self.n, k, k, k, 0, nib.contiguous(), self.b_packed)
        self.scale_b = scale_b.contiguous()   # [n, k/bl] f16, not packed
        self.bias = None if bias is None else bias.to(self.td).contiguous()
        self.clamp = _NO_CLAMP[out_dtype] if clamp is None else clamp
        self._ws = {}

    def workspace(self, m):
        ws = self._ws.get(m)
        if ws is None:
            dev = self.b_packed.device
            ws = dict(a_packed=torch.empty(self.uk.get_a_packed_size(m, self.k), dtype=torch.uint8, device=dev),
                      out=torch.empty((m, self.n), dtype=self.td, device=dev))
            self._ws[m] = ws
        return ws

    def pack(self, A_f16):
        ws = self.workspace(A_f16.shape[0])
        use_current_torch_stream()
        self.uk.run_a_pack(A_f16.shape[0], self.k, A_f16.stride(0), self.k, 0, A_f16, ws["a_packed"])
        return ws

    def gemm(self, m, Cm=None, out=None):
        ws = self.workspace(m)
        out = ws["out"] if out is None else out
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, self.bl, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, self.scale_b,
                         self.k // self.bl, Cm, self.n, out, out.stride(0), self.bias, self.clamp[0], self.clamp[1])
        return out

    prepare = pack

    def __call__(self, A_f16, Cm=None):
        self.pack(A_f16)
        return self.gemm(A_f16.shape[0], Cm)
