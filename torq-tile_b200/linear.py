"""Caller-side composition of the micro-kernels into linear operators.

The reference leaves memory, packing and tiling loops to its caller (an ML runtime; in-tree the
test runners, e.g. test/gemm/test_gemm_i8_i4_rvv.cpp:325-421: quantise A, size and fill the packed
buffers, one whole-problem run_gemm).  These classes are that caller for a GPU: they own the device
buffers (torch tensors), pack the weights once, and per call run  quantise+pack -> run_gemm  through
the C ABI.  They add no arithmetic of their own.
"""
from __future__ import annotations

import torch

from . import (GemmReqI8, GemmW4A8, GemmW4A16, QaI8DxQsI4CxParams, QaI8QaI8QsI8CxParams, quant_pack_qai8dxp,
               use_current_torch_stream)

_TORCH_TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
FLT_MAX = 3.4028234663852886e38


class W4A8Linear:
    """D = clamp(dequant(quant(A)) * dequant(W)^T + bias): qai8dxp x qsi4cxp, float output.

    ``nib`` is the [n, k/2] uint8 weight in the reference's encoding (low nibble = even k, value
    q + 8); ``scale_b`` [n] f32; ``bias`` [n] in the output type.  Columns [n_begin, n_begin+n_count)
    only are packed when a shard is given (column-parallel use: each rank builds its own slice).
    """

    def __init__(self, nib, scale_b, k, out_dtype="bf16", bias=None, clamp=None):
        self.uk = GemmW4A8(out_dtype)
        self.td = _TORCH_TD[out_dtype]
        self.n, self.k = nib.shape[0], k
        dev = nib.device
        use_current_torch_stream()
        self.b_packed = torch.empty(self.uk.get_b_packed_size(self.n, k), dtype=torch.uint8, device=dev)
        self.uk.run_bt_pack(self.n, k, k, k, 0, nib.contiguous(), self.b_packed)
        self.scale_b = scale_b.contiguous()
        self.bias = None if bias is None else bias.to(self.td).contiguous()
        if clamp is None:
            clamp = (-FLT_MAX, FLT_MAX) if out_dtype == "f32" else (-65504.0, 65504.0)
        self.clamp = clamp
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

    def gemm(self, m, Cm=None):
        """run_gemm on the workspace of size m (after quantize()); returns the output tensor."""
        ws = self.workspace(m)
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, Cm, self.n, ws["out"],
                         self.n, self.bias, self.clamp[0], self.clamp[1], ws["params"])
        return ws["out"]

    def __call__(self, A, Cm=None):
        self.quantize(A)
        return self.gemm(A.shape[0], Cm)


class W8A8RequantLinear:
    """Static W8A8 with int8 output: qai8 x qsi8cxp (weights [n, k] int8), int32 bias with the
    activation zero point already fused (bias - zp_a * sum_k w), as the reference's callers do."""

    def __init__(self, w_i8, scale_b, scale_a, zero_point_a, scale_d, zero_point_d, bias_fused=None, clamp=(-128, 127)):
        self.uk = GemmReqI8()
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

    def gemm(self, m, Cm=None):
        ws = self.workspace(m)
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, Cm, self.n, ws["out"],
                         self.n, self.bias, self.clamp[0], self.clamp[1], self.params)
        return ws["out"]

    def __call__(self, A_i8, Cm=None):
        self.pack(A_i8)
        return self.gemm(A_i8.shape[0], Cm)


class W4A16Linear:
    """f16 activations x block-quantised int4 weights (qsi4c2, f16 scale per bl elements of k)."""

    def __init__(self, nib, scale_b, k, bl, out_dtype="f16", bias=None, clamp=None):
        self.uk = GemmW4A16(out_dtype)
        self.td = _TORCH_TD[out_dtype]
        self.n, self.k, self.bl = nib.shape[0], k, bl
        dev = nib.device
        use_current_torch_stream()
        self.b_packed = torch.empty(self.uk.get_b_packed_size(self.n, k), dtype=torch.uint8, device=dev)
        self.uk.run_bt_pack(self.n, k, k, k, 0, nib.contiguous(), self.b_packed)
        self.scale_b = scale_b.contiguous()   # [n, k/bl] f16, not packed
        self.bias = None if bias is None else bias.to(self.td).contiguous()
        if clamp is None:
            clamp = (-FLT_MAX, FLT_MAX) if out_dtype == "f32" else (-65504.0, 65504.0)
        self.clamp = clamp
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

    def gemm(self, m, Cm=None):
        ws = self.workspace(m)
        use_current_torch_stream()
        self.uk.run_gemm(m, self.n, self.k, self.bl, ws["a_packed"], self.k, 0, self.b_packed, self.k, 0, self.scale_b,
                         self.k // self.bl, Cm, self.n, ws["out"], self.n, self.bias, self.clamp[0], self.clamp[1])
        return ws["out"]

    def __call__(self, A_f16, Cm=None):
        self.pack(A_f16)
        return self.gemm(A_f16.shape[0], Cm)
