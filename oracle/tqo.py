"""numpy/ctypes front-end of the CPU oracle (test infrastructure only).

Loads ``oracle/libtqt_oracle.so`` (the plain-C restatement, ``tqt_oracle.c``) and, when it has
been built, ``oracle/_ref/libtqt_ref.so`` (the reference's own portable C++ behind
``ref_shim.cpp``).  Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
TD_F32, TD_F16, TD_BF16 = 0, 1, 2

_sz = C.c_size_t
_vp = C.c_void_p


def _build_if_missing(name: str) -> str:
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", _HERE, "all"], stdout=subprocess.DEVNULL)
    return path


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(_vp)


class Oracle:
    """The restated oracle.  ``native=True`` loads the AVX2 build used only for timing."""

    def __init__(self, native: bool = False):
        lib = C.CDLL(_build_if_missing("libtqt_oracle_native.so" if native else "libtqt_oracle.so"))
        self.lib = lib
        lib.tqo_max_threads.restype = C.c_int
        lib.tqo_set_threads.argtypes = [C.c_int]
        lib.tqo_f32_to_bf16.restype = C.c_uint16
        lib.tqo_f32_to_bf16.argtypes = [C.c_float]
        lib.tqo_f32_to_f16.restype = C.c_uint16
        lib.tqo_f32_to_f16.argtypes = [C.c_float]
        lib.tqo_bf16_to_f32.restype = C.c_float
        lib.tqo_bf16_to_f32.argtypes = [C.c_uint16]
        lib.tqo_f16_to_f32.restype = C.c_float
        lib.tqo_f16_to_f32.argtypes = [C.c_uint16]
        lib.tqo_quantize_i8.restype = C.c_int8
        lib.tqo_quantize_i8.argtypes = [C.c_float, C.c_float, C.c_int32]
        lib.tqo_quantize_multiplier.argtypes = [C.c_double, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        lib.tqo_requantize_one.restype = C.c_int32
        lib.tqo_requantize_one.argtypes = [C.c_int32] * 4
        lib.tqo_gemm_clamp_i32_i8_i8.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz,
                                                 _vp, _sz, C.c_int32, C.c_int32]
        lib.tqo_fuse_zp_to_bias.argtypes = [_vp, _vp, _vp, C.c_int32, _sz, _sz]
        lib.tqo_quantize_a_per_row_asym.argtypes = [_vp, C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _vp]
        lib.tqo_quantize_b_per_channel_sym_int4.argtypes = [_vp, _sz, _sz, _vp, _vp]
        lib.tqo_gemm_w4a8.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _vp, _sz, _vp,
                                      _vp, _sz, C.c_float, C.c_float, C.c_int]
        lib.tqo_gemm_reqi32toi8.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz, _vp,
                                            _vp, _sz, C.c_int8, C.c_int8, C.c_float, _vp, C.c_int32,
                                            C.c_float, C.c_int32]
        lib.tqo_gemm_mx1bias_reqi32toi8.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _vp, _sz,
                                                    C.c_int8, C.c_int8, _vp, C.c_int32, C.c_float, C.c_float,
                                                    C.c_int32]
        lib.tqo_quantize_fp16_to_int4.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp, _sz]
        lib.tqo_gemm_w4a16.argtypes = [_sz, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp,
                                       _sz, _vp, C.c_float, C.c_float, C.c_int]
        lib.tqo_gemm_qai8dx_qsi8cx.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _vp,
                                               _vp, _vp, _vp, _sz, C.c_float, C.c_float, C.c_int]

        lib.tqo_im2col_i8.argtypes = [C.c_int, _sz, _vp, _vp, _vp]
        lib.tqo_gemm_float.argtypes = [C.c_int, C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz, _vp, _sz, _vp,
                                       C.c_int, C.c_float, C.c_float]
        lib.tqo_fill_uniform_f32.argtypes = [_vp, _sz, C.c_float, C.c_float, C.c_uint32]
        lib.tqo_fill_uniform_i8.argtypes = [_vp, _sz, C.c_int, C.c_int, C.c_uint32]
        lib.tqo_fill_uniform_i32.argtypes = [_vp, _sz, C.c_int32, C.c_int32, C.c_uint32]
        lib.tqo_fill_normal_f32.argtypes = [_vp, _sz, C.c_float, C.c_float, C.c_uint32]

    # ---- seeded generators (std::mt19937, the engine and seeds of the reference's suites) ----
    def fill_uniform(self, shape, dtype, lo, hi, seed):
        a = np.empty(shape, dtype)
        if dtype == np.float32:
            self.lib.tqo_fill_uniform_f32(_ptr(a), a.size, float(lo), float(hi), int(seed))
        elif dtype == np.int8:
            self.lib.tqo_fill_uniform_i8(_ptr(a), a.size, int(lo), int(hi), int(seed))
        elif dtype == np.int32:
            self.lib.tqo_fill_uniform_i32(_ptr(a), a.size, int(lo), int(hi), int(seed))
        else:
            raise TypeError(dtype)
        return a

    def fill_normal(self, shape, mean, sigma, seed):
        a = np.empty(shape, np.float32)
        self.lib.tqo_fill_normal_f32(_ptr(a), a.size, float(mean), float(sigma), int(seed))
        return a

    def gemm_float(self, ta, td, A, B, b_transposed, Cm=None, bias=None, bias_per_row=False,
                   clamp=(-3.4028234663852886e38, 3.4028234663852886e38)):
        """Unquantised GEMM: A [m, k], B [n, k] (b_transposed) or [k, n], as float32 arrays (ta / td TD_F32) or uint16
        bit patterns; C, bias and the result in the output type td."""
        m, k = A.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        self.lib.tqo_gemm_float(ta, td, m, n, k, _ptr(A), A.shape[1], _ptr(B), B.shape[1], int(b_transposed), _ptr(Cm), n,
                                _ptr(D), n, _ptr(bias), int(bias_per_row), float(clamp[0]), float(clamp[1]))
        return D

    def im2col_i8(self, activation, geom, channel_first, group_idx=0):
        """``geom``: ConvGeometry.  Returns [M, K] (channel-last) or [K, N] (channel-first)."""
        rows, k = geom.rows, geom.k
        out = np.empty((k, rows) if channel_first else (rows, k), np.int8)
        g = geom.as_array()
        self.lib.tqo_im2col_i8(int(channel_first), group_idx, _ptr(activation), _ptr(out), _ptr(g))
        return out

    # ---- helpers -----------------------------------------------------------------------
    def max_threads(self) -> int:
        return int(self.lib.tqo_max_threads())

    def set_threads(self, n: int) -> None:
        self.lib.tqo_set_threads(int(n))

    def quantize_multiplier(self, v: float):
        m, s = C.c_int32(), C.c_int32()
        self.lib.tqo_quantize_multiplier(float(v), C.byref(m), C.byref(s))
        return m.value, s.value

    # ---- kernels -----------------------------------------------------------------------
    def gemm_clamp_i32_i8_i8(self, A, B, b_transposed, Cm=None, clamp=(-2**31, 2**31 - 1)):
        m, k = A.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.int32)
        self.lib.tqo_gemm_clamp_i32_i8_i8(m, n, k, _ptr(A), A.shape[1], _ptr(B), B.shape[1],
                                          int(bool(b_transposed)), _ptr(Cm), n, _ptr(D), n,
                                          int(clamp[0]), int(clamp[1]))
        return D

    def fuse_zp_to_bias(self, bias, data, zp):
        out = np.empty_like(bias)
        self.lib.tqo_fuse_zp_to_bias(_ptr(out), _ptr(bias), _ptr(data), int(zp), data.shape[0], data.shape[1])
        return out

    def quantize_a_per_row_asym(self, A, ta=TD_F32):
        """A: f32 array, or uint16 array holding f16/bf16 bit patterns (per ``ta``)."""
        m, k = A.shape
        q = np.empty((m, k), np.int8)
        s = np.empty(m, np.float32)
        z = np.empty(m, np.int32)
        self.lib.tqo_quantize_a_per_row_asym(_ptr(A), ta, m, k, k, _ptr(q), k, _ptr(s), _ptr(z))
        return q, s, z

    def quantize_b_per_channel_sym_int4(self, B):
        n, k = B.shape
        nib = np.empty((n, k // 2), np.uint8)
        s = np.empty(n, np.float32)
        self.lib.tqo_quantize_b_per_channel_sym_int4(_ptr(B), n, k, _ptr(nib), _ptr(s))
        return nib, s

    def gemm_w4a8(self, A_i8, B_nib, scale_a, zp_a, scale_b, td, Cm=None, bias=None,
                  clamp=(-3.4028234663852886e38, 3.4028234663852886e38)):
        m, k = A_i8.shape
        n = B_nib.shape[0]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        self.lib.tqo_gemm_w4a8(m, n, k, _ptr(A_i8), k, _ptr(B_nib), B_nib.shape[1], _ptr(scale_a),
                               _ptr(zp_a), _ptr(scale_b), _ptr(Cm), n, _ptr(bias), _ptr(D), n,
                               float(clamp[0]), float(clamp[1]), td)
        return D

    def gemm_reqi32toi8(self, A, B, b_transposed, scale_a, scale_b, scale_d, zp_d, bias=None, Cm=None,
                        clamp=(-128, 127), quant_channel_b=0):
        m, k = A.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.int8)
        self.lib.tqo_gemm_reqi32toi8(m, n, k, _ptr(A), k, _ptr(B), B.shape[1], int(bool(b_transposed)),
                                     _ptr(Cm), n, _ptr(bias), _ptr(D), n, int(clamp[0]), int(clamp[1]),
                                     float(scale_a), _ptr(scale_b), int(quant_channel_b), float(scale_d),
                                     int(zp_d))
        return D

    def gemm_mx1bias_reqi32toi8(self, A, B_kn, scale_a, scale_b, scale_d, zp_d, bias=None, Cm=None,
                                clamp=(-128, 127), quant_channel_a=0):
        """A [m,k] int8, B [k,n] int8, scale_a [m] f32, bias [m] int32."""
        m, k = A.shape
        n = B_kn.shape[1]
        D = np.empty((m, n), np.int8)
        self.lib.tqo_gemm_mx1bias_reqi32toi8(m, n, k, _ptr(A), k, _ptr(B_kn), n, _ptr(Cm), n, _ptr(bias), _ptr(D), n,
                                             int(clamp[0]), int(clamp[1]), _ptr(scale_a), int(quant_channel_a),
                                             float(scale_b), float(scale_d), int(zp_d))
        return D

    def quantize_fp16_to_int4(self, W_f16_bits, bl):
        n, k = W_f16_bits.shape
        nib = np.empty((n, k // 2), np.uint8)
        sc = np.empty((n, k // bl), np.uint16)
        self.lib.tqo_quantize_fp16_to_int4(n, k, bl, _ptr(W_f16_bits), _ptr(nib), _ptr(sc), k // bl)
        return nib, sc

    def gemm_w4a16(self, A_bits, B_nib, scale_bits, bl, td=TD_F16, Cm=None, bias=None,
                   clamp=(-65504.0, 65504.0)):
        m, k = A_bits.shape
        n = B_nib.shape[0]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        self.lib.tqo_gemm_w4a16(m, n, k, bl, _ptr(A_bits), k, _ptr(B_nib), k, _ptr(scale_bits),
                                scale_bits.shape[1], _ptr(Cm), n, _ptr(D), n, _ptr(bias),
                                float(clamp[0]), float(clamp[1]), td)
        return D

    def gemm_qai8dx_qsi8cx(self, A_i8, B, b_transposed, scale_a, zp_a, scale_b, td, bias=None,
                           clamp=(-3.4028234663852886e38, 3.4028234663852886e38)):
        m, k = A_i8.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        self.lib.tqo_gemm_qai8dx_qsi8cx(m, n, k, _ptr(A_i8), k, _ptr(B), B.shape[1],
                                        int(bool(b_transposed)), _ptr(scale_a), _ptr(zp_a),
                                        _ptr(scale_b), _ptr(bias), _ptr(D), n, float(clamp[0]),
                                        float(clamp[1]), td)
        return D


class ConvGeometry:
    """The members of the reference's tqt_conv_params (src/common/tqt_conv.h:23-34); the output shape is computed
    the way the reference's test suites do (test/common/conv_test_runner.h:95-114)."""

    def __init__(self, input_channel, output_channel, groups, input_shape, kernel_shape, stride=(1, 1, 1),
                 dilation=(1, 1, 1), pad=(0, 0, 0)):
        self.input_channel, self.output_channel, self.groups = input_channel, output_channel, groups
        self.input_shape, self.kernel_shape = tuple(input_shape), tuple(kernel_shape)
        self.stride, self.dilation, self.pad = tuple(stride), tuple(dilation), tuple(pad)
        self.output_shape = tuple((self.input_shape[i] + 2 * self.pad[i] - self.dilation[i] * (self.kernel_shape[i] - 1) - 1)
                                  // self.stride[i] + 1 for i in range(3))

    @property
    def rows(self):
        return int(np.prod(self.output_shape))

    @property
    def k(self):
        return int(np.prod(self.kernel_shape)) * (self.input_channel // self.groups)

    def as_array(self):
        return np.array(list(self.input_shape) + list(self.output_shape) + list(self.kernel_shape) + list(self.stride)
                        + list(self.dilation) + list(self.pad) + [self.input_channel, self.output_channel, self.groups],
                        dtype=np.uint64)


class Reference:
    """The reference's own portable C++ (oracle/_ref).  ``available()`` is False on machines that
    have neither the prebuilt library nor the reference checkout."""

    def __init__(self, native: bool = False):
        name = "libtqt_ref_native.so" if native else "libtqt_ref.so"
        path = os.path.join(_HERE, "_ref", name)
        self.lib = C.CDLL(path) if os.path.exists(path) else None
        if self.lib is None:
            return
        lib = self.lib
        lib.ref_gemm_i32_i8.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz, _vp, _sz,
                                        C.c_int32, C.c_int32]
        for f in (lib.ref_gemm_w4a16_f16, lib.ref_gemm_w4a16_f32):
            f.argtypes = [_sz, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp,
                          C.c_float, C.c_float]
        lib.ref_quantize_fp16_to_int4.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp, _sz]
        lib.ref_quantize_multiplier.argtypes = [C.c_double, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        lib.ref_quantize_i8.restype = C.c_int8
        lib.ref_quantize_i8.argtypes = [C.c_float, C.c_float, C.c_int32]
        lib.ref_fuse_zp_to_bias.argtypes = [_vp, _vp, _vp, C.c_int32, _sz, _sz]
        lib.ref_f32_to_f16.restype = C.c_uint16
        lib.ref_f32_to_f16.argtypes = [C.c_float]
        lib.ref_f32_to_bf16.restype = C.c_uint16
        lib.ref_f32_to_bf16.argtypes = [C.c_float]
        lib.ref_f16_to_f32.restype = C.c_float
        lib.ref_f16_to_f32.argtypes = [C.c_uint16]
        lib.ref_bf16_to_f32.restype = C.c_float
        lib.ref_bf16_to_f32.argtypes = [C.c_uint16]
        lib.ref_fill_uniform_f32.argtypes = [_vp, _sz, _sz, C.c_float, C.c_float, C.c_uint32]
        lib.ref_fill_uniform_f16.argtypes = [_vp, _sz, _sz, C.c_float, C.c_float, C.c_uint32]
        lib.ref_fill_uniform_i8.argtypes = [_vp, _sz, _sz, C.c_int, C.c_int, C.c_uint32]
        lib.ref_fill_uniform_i32.argtypes = [_vp, _sz, _sz, C.c_int32, C.c_int32, C.c_uint32]
        if hasattr(lib, "ref_w4a8_gemm"):
            lib.ref_fill_uniform_bf16.argtypes = [_vp, _sz, _sz, C.c_float, C.c_float, C.c_uint32]
            lib.ref_w4a8_quantize_a_per_row_asym.argtypes = [_vp, _sz, _sz, _vp, _vp, _vp]
            lib.ref_w4a8_quantize_b_per_channel_sym_int4.argtypes = [_vp, _sz, _sz, _vp, _vp]
            lib.ref_w4a8_gemm.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_float,
                                          C.c_float, C.c_int]

    def has_float(self) -> bool:
        return self.lib is not None and hasattr(self.lib, "ref_gemm_float")

    def gemm_float(self, ta, td, A, B, b_transposed, Cm=None, bias=None, bias_per_row=False,
                   clamp=(-3.4028234663852886e38, 3.4028234663852886e38)):
        """reference_gemm<TA, TD> of the reference (same argument conventions as Oracle.gemm_float)."""
        m, k = A.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        f = self.lib.ref_gemm_float
        f.argtypes = [C.c_int, C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int, _vp, _sz, _vp, _sz, _vp, C.c_int,
                      C.c_float, C.c_float]
        f.restype = C.c_int
        rc = f(ta, td, m, n, k, _ptr(A), A.shape[1], _ptr(B), B.shape[1], int(b_transposed), _ptr(Cm), n, _ptr(D), n,
               _ptr(bias), int(bias_per_row), float(clamp[0]), float(clamp[1]))
        if rc != 0:
            raise ValueError("the reference does not instantiate this type combination")
        return D

    def has_conv(self) -> bool:
        return self.lib is not None and hasattr(self.lib, "ref_im2col_i8")

    def im2col_i8(self, activation, geom, channel_first, group_idx=0):
        """tqt_im2col_cf / tqt_im2col_cl of the reference on int8."""
        rows, k = geom.rows, geom.k
        out = np.empty((k, rows) if channel_first else (rows, k), np.int8)
        g = geom.as_array()
        self.lib.ref_im2col_i8.argtypes = [C.c_int, _sz, _vp, _vp, _vp]
        self.lib.ref_im2col_i8(int(channel_first), group_idx, _ptr(activation), _ptr(out), _ptr(g))
        return out

    def has_w4a8(self) -> bool:
        """True when the library carries the W4A8 helpers cut out of the reference's gtest suite."""
        return self.lib is not None and hasattr(self.lib, "ref_w4a8_gemm")

    def w4a8_quantize_a_per_row_asym(self, A_f32):
        m, k = A_f32.shape
        q = np.empty((m, k), np.int8)
        s = np.empty(m, np.float32)
        z = np.empty(m, np.int32)
        self.lib.ref_w4a8_quantize_a_per_row_asym(_ptr(A_f32), m, k, _ptr(q), _ptr(s), _ptr(z))
        return q, s, z

    def w4a8_quantize_b_per_channel_sym_int4(self, B_f32):
        n, k = B_f32.shape
        nib = np.empty((n, k // 2), np.uint8)
        s = np.empty(n, np.float32)
        self.lib.ref_w4a8_quantize_b_per_channel_sym_int4(_ptr(B_f32), n, k, _ptr(nib), _ptr(s))
        return nib, s

    def w4a8_gemm(self, A_i8, B_nib, scale_a, zp_a, scale_b, td, Cm=None, bias=None,
                  clamp=(-3.4028234663852886e38, 3.4028234663852886e38)):
        """w4a8_reference_fp32 narrowed through the output type; C, bias, result: f32 arrays or
        uint16 bit patterns per ``td``."""
        m, k = A_i8.shape
        n = B_nib.shape[0]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        self.lib.ref_w4a8_gemm(m, n, k, _ptr(A_i8), _ptr(B_nib), _ptr(scale_a), _ptr(zp_a), _ptr(scale_b),
                               _ptr(Cm), _ptr(bias), _ptr(D), float(clamp[0]), float(clamp[1]), td)
        return D

    def available(self) -> bool:
        return self.lib is not None

    def quantize_multiplier(self, v: float):
        m, s = C.c_int32(), C.c_int32()
        self.lib.ref_quantize_multiplier(float(v), C.byref(m), C.byref(s))
        return m.value, s.value

    def gemm_i32_i8(self, A, B, b_transposed, Cm=None, clamp=(-2**31, 2**31 - 1)):
        m, k = A.shape
        n = B.shape[0] if b_transposed else B.shape[1]
        D = np.empty((m, n), np.int32)
        self.lib.ref_gemm_i32_i8(m, n, k, _ptr(A), A.shape[1], _ptr(B), B.shape[1],
                                 int(bool(b_transposed)), _ptr(Cm), n, _ptr(D), n, int(clamp[0]),
                                 int(clamp[1]))
        return D

    def gemm_w4a16(self, A_bits, B_nib, scale_bits, bl, td=TD_F16, Cm=None, bias=None,
                   clamp=(-65504.0, 65504.0)):
        m, k = A_bits.shape
        n = B_nib.shape[0]
        D = np.empty((m, n), np.float32 if td == TD_F32 else np.uint16)
        f = self.lib.ref_gemm_w4a16_f32 if td == TD_F32 else self.lib.ref_gemm_w4a16_f16
        f(m, n, k, bl, _ptr(A_bits), k, _ptr(B_nib), k, _ptr(scale_bits), scale_bits.shape[1], _ptr(Cm),
          n, _ptr(D), n, _ptr(bias), float(clamp[0]), float(clamp[1]))
        return D

    def quantize_fp16_to_int4(self, W_f16_bits, bl):
        n, k = W_f16_bits.shape
        nib = np.empty((n, k // 2), np.uint8)
        sc = np.empty((n, k // bl), np.uint16)
        self.lib.ref_quantize_fp16_to_int4(n, k, bl, _ptr(W_f16_bits), _ptr(nib), _ptr(sc), k // bl)
        return nib, sc

    def fuse_zp_to_bias(self, bias, data, zp):
        out = np.empty_like(bias)
        self.lib.ref_fuse_zp_to_bias(_ptr(out), _ptr(bias), _ptr(data), int(zp), data.shape[0], data.shape[1])
        return out

    def fill_uniform(self, shape, dtype, lo, hi, seed):
        rows, cols = shape
        if dtype == np.float32:
            a = np.empty(shape, np.float32)
            self.lib.ref_fill_uniform_f32(_ptr(a), rows, cols, lo, hi, seed)
        elif dtype == np.float16:
            a = np.empty(shape, np.float16)
            self.lib.ref_fill_uniform_f16(_ptr(a), rows, cols, lo, hi, seed)
        elif dtype == "bf16":
            a = np.empty(shape, np.uint16)
            self.lib.ref_fill_uniform_bf16(_ptr(a), rows, cols, lo, hi, seed)
        elif dtype == np.int8:
            a = np.empty(shape, np.int8)
            self.lib.ref_fill_uniform_i8(_ptr(a), rows, cols, int(lo), int(hi), seed)
        elif dtype == np.int32:
            a = np.empty(shape, np.int32)
            self.lib.ref_fill_uniform_i32(_ptr(a), rows, cols, int(lo), int(hi), seed)
        else:
            raise TypeError(dtype)
        return a
