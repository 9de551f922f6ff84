"""Host-side mirror of the TORQ-Tile micro-kernel interface for the B200 library.

The product is ``libtorq_tile_b200.so`` (C ABI declared in ``include/*.h``).  This module binds it
with ctypes and offers, per kernel type, an object with the same members as the reference's
``struct tqt_<kernel-type>_ukernel`` function-pointer tables (``get_m_step``, ``get_n_step``, the
offset/size helpers, ``run_a_pack``, ``run_b[t]_pack``, ``run_gemm``), taking torch CUDA tensors (or
raw device addresses) where the C API takes device pointers.  PyTorch is used only for device
memory and streams.  There is no CPU fallback: importing works without a GPU (so that symbols and
host helpers can be checked), but every ``run_*`` call needs the CUDA library and a device.

The directory name contains a hyphen, so the package is loaded by path; see ``load()`` in
``__graft_entry__.py`` at the repository root.
"""
from __future__ import annotations

import ctypes as C
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TQT_B200_LIB") or os.path.join(HERE, "libtorq_tile_b200.so")   # override: A/B comparisons of builds
VARIANT = "128x128_sm100a"

_sz, _vp = C.c_size_t, C.c_void_p

STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "LAUNCH_FAILED", 3: "UNSUPPORTED"}


class TqtError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise TqtError(f"{LIB_PATH} is missing: build it with `python torq-tile_b200/build.py` "
                       "(there is no CPU fallback)")
    return C.CDLL(LIB_PATH)


_lib = None


def lib():
    """The loaded shared library (raises TqtError if it has not been built)."""
    global _lib
    if _lib is None:
        _lib = _load()
        _lib.tqt_cuda_set_stream.argtypes = [_vp]
        _lib.tqt_cuda_get_stream.restype = _vp
        _lib.tqt_cuda_get_last_status.restype = C.c_int
        _lib.tqt_cuda_get_last_cuda_error.restype = C.c_int
        _lib.tqt_cuda_read_device_fault.restype = C.c_int
        _lib.tqt_cuda_version.restype = C.c_char_p
        _lib.tqt_shard_plan_n.argtypes = [_sz, _sz, _sz, C.POINTER(_sz), C.POINTER(_sz)]
        _lib.tqt_cuda_kernel_choice_w4a8.argtypes = [_sz, _sz, _sz]
        _lib.tqt_cuda_kernel_choice_w4a8.restype = C.c_int
    return _lib


def _addr(x):
    """Device address of a torch tensor, or the integer itself, or NULL for None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def half_arg(bits: int):
    """A 16-bit float (given as its bit pattern) passed by value.

    The x86-64 SysV ABI passes ``_Float16`` / ``__bf16`` in the low 16 bits of an SSE register,
    which is where the low half of a C ``float`` argument travels too, so a ``c_float`` whose low
    16 bits hold the pattern is received unchanged (no arithmetic touches it on the way).
    """
    return C.c_float.from_buffer_copy(struct.pack("<HH", bits & 0xFFFF, 0))


def f16_bits(v: float) -> int:
    return struct.unpack("<H", struct.pack("<e", v))[0]


def bf16_bits(v: float) -> int:
    u = struct.unpack("<I", struct.pack("<f", v))[0]
    if (u & 0x7FFFFFFF) > 0x7F800000:
        return (u >> 16) | 0x40
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def check(what: str = "call"):
    """Raise if the calling thread's last run_* call was refused."""
    st = lib().tqt_cuda_get_last_status()
    if st != 0:
        raise TqtError(f"{what}: status {STATUS_NAMES.get(st, st)} "
                       f"(cudaError {lib().tqt_cuda_get_last_cuda_error()})")


def set_stream(stream) -> None:
    """Use a torch.cuda.Stream (or a raw cudaStream_t integer, or None) for this thread's calls."""
    h = None if stream is None else (stream if isinstance(stream, int) else stream.cuda_stream)
    lib().tqt_cuda_set_stream(h)


def use_current_torch_stream() -> None:
    import torch
    set_stream(torch.cuda.current_stream())


def set_output_replicas(local_base: int, local_bytes: int, replica_bases) -> None:
    """Also store the output of the following run_gemm calls at the same offsets inside the buffers that
    start at ``replica_bases`` (device addresses, e.g. peer-mapped copies, each at least ``local_bytes``
    long); the output of every such call must lie inside [local_base, local_base + local_bytes).  An empty
    list switches it off."""
    n = len(replica_bases)
    arr = (C.c_void_p * max(n, 1))(*[C.c_void_p(int(b)) for b in replica_bases])
    f = lib().tqt_cuda_set_output_replicas
    f.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t]
    f.restype = None
    f(C.c_void_p(int(local_base)) if n else None, int(local_bytes) if n else 0, arr if n else None, n)
    check("set_output_replicas")


class output_replicas:
    """Context manager around set_output_replicas: the setting is cleared on the way out, also when the body raises."""

    def __init__(self, local_base: int, local_bytes: int, replica_bases):
        self.args = (local_base, local_bytes, list(replica_bases))

    def __enter__(self):
        set_output_replicas(*self.args)
        return self

    def __exit__(self, *exc):
        set_output_replicas(0, 0, [])
        return False


def debug_inject_wait_failure(wait_shift: int = 0, flags: int = 0) -> None:
    """Test knob of the bounded waits (tqt_cuda_debug_inject_wait_failure); (0, 0) = normal operation."""
    f = lib().tqt_cuda_debug_inject_wait_failure
    f.argtypes = [C.c_uint, C.c_uint]
    f.restype = None
    f(int(wait_shift), int(flags))


def debug_set_path(path=None, umma=None) -> None:
    """Force a kernel path ("auto", "umma", "gemv", "simt") and a tensor-core kernel ("single", "pair", "ts")
    for all later run_gemm calls of the process; None = automatic choice."""
    f = lib().tqt_cuda_debug_set_path
    f.argtypes = [C.c_char_p, C.c_char_p]
    f.restype = None
    f(None if path is None else path.encode(), None if umma is None else umma.encode())


def debug_last_kernel() -> int:
    """0 none, 1 generic CUDA-core kernel, 2 tcgen05 CTA-pair kernel on packed blocks, 3 the same with tiled TMA loads."""
    return int(lib().tqt_cuda_debug_last_kernel())


def read_device_fault() -> int:
    return int(lib().tqt_cuda_read_device_fault())


def shard_plan_n(n: int, world: int, rank: int):
    b, c = _sz(), _sz()
    lib().tqt_shard_plan_n(n, world, rank, C.byref(b), C.byref(c))
    return int(b.value), int(c.value)


_PACK_SIG = [_sz, _sz, _sz, _sz, _sz, _vp, _vp]


class _UKernel:
    """Common part of the per-kernel-type tables."""

    type_name = ""
    helpers_size = ()      # names returning size_t with their argument counts
    td_size = 4

    def __init__(self):
        self._l = lib()
        for name, nargs in self.helpers_size:
            f = self._sym(name)
            f.argtypes = [_sz] * nargs
            f.restype = _sz
            setattr(self, name, f)

    def _name(self, action: str) -> str:
        # tqt_<action>_<kernel-type>_<variant>; the kernel type itself starts with "gemm", so the
        # GEMM entry point is tqt_run_<kernel-type>_<variant>
        if action == "run_gemm":
            return f"tqt_run_{self.type_name}_{VARIANT}"
        return f"tqt_{action}_{self.type_name}_{VARIANT}"

    def _sym(self, action: str):
        return getattr(self._l, self._name(action))

    def symbol_names(self):
        return [self._name(a) for a in self.actions]

    def _pack(self, action, rows, k, ld, ld_packed, k_idx, src, dst):
        f = self._sym(action)
        f.argtypes = _PACK_SIG
        f.restype = None
        f(rows, k, ld, ld_packed, k_idx, _addr(src), _addr(dst))
        check(f"{action} {self.type_name}")


_PACKED_HELPERS = (("get_m_step", 0), ("get_n_step", 0), ("get_a_packed_offset", 4), ("get_b_packed_offset", 4),
                   ("get_c_offset", 3), ("get_d_offset", 3), ("get_d_size", 2), ("get_a_packed_size", 2),
                   ("get_b_packed_size", 2))


class GemmClampI32I8I8(_UKernel):
    """gemm_clamp_i32_i8_i8: D = clamp(C + A*B), unpacked int8 operands, int32 output."""
    type_name = "gemm_clamp_i32_i8_i8"
    helpers_size = (("get_m_step", 0), ("get_n_step", 0), ("get_a_offset", 3), ("get_b_offset", 3),
                    ("get_c_offset", 3), ("get_d_offset", 3), ("get_d_size", 2))
    actions = [h[0] for h in helpers_size] + ["run_gemm"]

    def run_gemm(self, m, n, k, A, lda, k_idx_a, B, ldb, k_idx_b, Cm, ldc, D, ldd, clamp_min, clamp_max):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int32, C.c_int32]
        f.restype = None
        f(m, n, k, _addr(A), lda, k_idx_a, _addr(B), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd, clamp_min, clamp_max)
        check("run_gemm " + self.type_name)


class GemmClampI32I8pI8p(_UKernel):
    """gemm_clamp_i32_i8p_i8p: same result from packed operands (tensor cores)."""
    type_name = "gemm_clamp_i32_i8p_i8p"
    helpers_size = _PACKED_HELPERS
    actions = [h[0] for h in helpers_size] + ["run_a_pack", "run_b_pack", "run_bt_pack", "run_gemm"]

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_b_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_b_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_gemm(self, m, n, k, A_packed, lda, k_idx_a, B_packed, ldb, k_idx_b, Cm, ldc, D, ldd, clamp_min, clamp_max):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, C.c_int32, C.c_int32]
        f.restype = None
        f(m, n, k, _addr(A_packed), lda, k_idx_a, _addr(B_packed), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd,
          clamp_min, clamp_max)
        check("run_gemm " + self.type_name)


class QaI8QaI8QsI8CxParams(C.Structure):
    """struct tqt_qai8_qai8_qsi8cx_params (host struct; scale_b is a device array)."""
    _fields_ = [("scale_a", C.c_float), ("zero_point_a", C.c_int32), ("scale_b", _vp),
                ("quant_channel_b", C.c_int32), ("scale_d", C.c_float), ("zero_point_d", C.c_int32)]


class GemmReqI8(GemmClampI32I8pI8p):
    """gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp: static W8A8 with int8 requantised output."""
    type_name = "gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp"
    helpers_size = _PACKED_HELPERS + (("get_bias_offset", 1),)
    actions = [h[0] for h in helpers_size] + ["run_a_pack", "run_b_pack", "run_bt_pack", "run_gemm"]

    def run_gemm(self, m, n, k, A_packed, lda, k_idx_a, B_packed, ldb, k_idx_b, Cm, ldc, D, ldd, bias, clamp_min,
                 clamp_max, params):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, C.c_int8, C.c_int8,
                      C.POINTER(QaI8QaI8QsI8CxParams)]
        f.restype = None
        f(m, n, k, _addr(A_packed), lda, k_idx_a, _addr(B_packed), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd,
          _addr(bias), clamp_min, clamp_max, None if params is None else C.byref(params))
        check("run_gemm " + self.type_name)


class QaI8DxQsI4CxParams(C.Structure):
    """struct tqt_qai8dx_qsi4cx_params (host struct holding three device arrays)."""
    _fields_ = [("scale_a", _vp), ("zero_point_a", _vp), ("scale_b", _vp)]


class GemmW4A8(_UKernel):
    """gemm_1xnbias_clamp_<td>_qai8dxp_qsi4cxp, td in {"f32", "f16", "bf16"}."""
    helpers_size = _PACKED_HELPERS + (("get_bias_offset", 1),)
    actions = [h[0] for h in helpers_size] + ["run_a_pack", "run_bt_pack", "run_gemm"]

    def __init__(self, td: str):
        assert td in ("f32", "f16", "bf16")
        self.td = td
        self.td_size = 4 if td == "f32" else 2
        self.type_name = f"gemm_1xnbias_clamp_{td}_qai8dxp_qsi4cxp"
        super().__init__()

    def clamp_arg(self, v: float):
        if self.td == "f32":
            return C.c_float(v)
        return half_arg(f16_bits(v) if self.td == "f16" else bf16_bits(v))

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_gemm(self, m, n, k, A_packed, lda, k_idx_a, B_packed, ldb, k_idx_b, Cm, ldc, D, ldd, bias, clamp_min,
                 clamp_max, params):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, C.c_float, C.c_float,
                      C.POINTER(QaI8DxQsI4CxParams)]
        f.restype = None
        f(m, n, k, _addr(A_packed), lda, k_idx_a, _addr(B_packed), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd,
          _addr(bias), self.clamp_arg(clamp_min), self.clamp_arg(clamp_max),
          None if params is None else C.byref(params))
        check("run_gemm " + self.type_name)


class GemmW4A16(_UKernel):
    """gemm_1xnbias_clamp_<td>_f16p_qsi4c2p, td in {"f16", "f32"}."""
    helpers_size = _PACKED_HELPERS + (("get_bias_offset", 1), ("get_scale_b_offset", 3))
    actions = [h[0] for h in helpers_size] + ["run_a_pack", "run_bt_pack", "run_gemm"]

    def __init__(self, td: str = "f16"):
        assert td in ("f16", "f32")
        self.td = td
        self.td_size = 4 if td == "f32" else 2
        self.type_name = f"gemm_1xnbias_clamp_{td}_f16p_qsi4c2p"
        super().__init__()

    def clamp_arg(self, v: float):
        return C.c_float(v) if self.td == "f32" else half_arg(f16_bits(v))

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_gemm(self, m, n, k, bl, A_packed, lda, k_idx_a, B_packed, ldb, k_idx_b, scale_b, ldsb, Cm, ldc, D, ldd,
                 bias, clamp_min, clamp_max):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp,
                      C.c_float, C.c_float]
        f.restype = None
        f(m, n, k, bl, _addr(A_packed), lda, k_idx_a, _addr(B_packed), ldb, k_idx_b, _addr(scale_b), ldsb,
          _addr(Cm), ldc, _addr(D), ldd, _addr(bias), self.clamp_arg(clamp_min), self.clamp_arg(clamp_max))
        check("run_gemm " + self.type_name)


# ---- sibling kernel types (generic CUDA-core path) ------------------------------------------------
class QaI8QsI8DxQaI8Params(C.Structure):
    """struct tqt_qai8_qsi8dx_qai8_params (host struct; scale_a is a device array)."""
    _fields_ = [("scale_a", _vp), ("quant_channel_a", C.c_int32), ("scale_b", C.c_float),
                ("zero_point_b", C.c_int32), ("scale_d", C.c_float), ("zero_point_d", C.c_int32)]


class QaI8DxpQsI8CxpParams(C.Structure):
    """struct tqt_qai8dxp_qsi8cxp_params (host struct holding three device arrays)."""
    _fields_ = [("scale_a", _vp), ("zero_point_a", _vp), ("scale_b", _vp)]


_UNPACKED_HELPERS = (("get_m_step", 0), ("get_n_step", 0), ("get_a_offset", 3), ("get_b_offset", 3),
                     ("get_c_offset", 3), ("get_bias_offset", 1), ("get_d_offset", 3), ("get_d_size", 2))
_PACKED_HELPERS_B = _PACKED_HELPERS + (("get_bias_offset", 1),)


class SiblingGemm(_UKernel):
    """One of the sibling kernel types of include/tqt_b200_gemm_siblings.h.

    ``type_name`` selects it; the signature of run_gemm follows from the name:
    ``clamp`` "i8" / "f32" / "f16" / "bf16" (type of the two clamp arguments), ``params`` the ctypes
    struct class (None for the W4A16 types, which take bl / scale_b / ldsb instead)."""

    def __init__(self, type_name: str):
        self.type_name = type_name
        t = type_name
        self.w4a16 = "_f16_qsi4c2t" in t
        a_packed = "qai8dxp" in t or "qsi8dxp" in t
        b_packed = t.endswith("p")
        if self.w4a16:
            self.helpers_size = (("get_m_step", 0), ("get_n_step", 0), ("get_a_offset", 4), ("get_b_offset", 4),
                                 ("get_scale_b_offset", 3), ("get_c_offset", 3), ("get_bias_offset", 1),
                                 ("get_d_offset", 3), ("get_d_size", 2))
            packs = []
        elif a_packed and b_packed:
            self.helpers_size = _PACKED_HELPERS_B
            packs = ["run_a_pack", "run_b_pack", "run_bt_pack"]
        elif b_packed:   # A unpacked, B packed
            self.helpers_size = (("get_m_step", 0), ("get_n_step", 0), ("get_a_offset", 3), ("get_b_packed_offset", 4),
                                 ("get_c_offset", 3), ("get_bias_offset", 1), ("get_d_offset", 3), ("get_d_size", 2),
                                 ("get_b_packed_size", 2))
            packs = ["run_b_pack", "run_bt_pack"]
        else:
            self.helpers_size = _UNPACKED_HELPERS
            packs = []
        self.actions = [h[0] for h in self.helpers_size] + packs + ["run_gemm"]
        if "reqi32toi8" in t:
            self.clamp = "i8"
            self.params_cls = QaI8QsI8DxQaI8Params if "mx1bias" in t else QaI8QaI8QsI8CxParams
        else:
            self.clamp = t.split("_clamp_")[1].split("_")[0]
            self.params_cls = None if self.w4a16 else (QaI8DxQsI4CxParams if "qsi4cx" in t else QaI8DxpQsI8CxpParams)
        super().__init__()

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_b_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_b_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def _clamp_arg(self, v):
        if self.clamp == "i8":
            return C.c_int8(int(v))
        if self.clamp == "f32":
            return C.c_float(v)
        return half_arg(f16_bits(v) if self.clamp == "f16" else bf16_bits(v))

    def run_gemm(self, m, n, k, A, lda, k_idx_a, B, ldb, k_idx_b, Cm, ldc, D, ldd, bias, clamp_min, clamp_max,
                 params=None, bl=None, scale_b=None, ldsb=0):
        f = self._sym("run_gemm")
        ct = C.c_int8 if self.clamp == "i8" else C.c_float
        f.restype = None
        if self.w4a16:
            f.argtypes = [_sz, _sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, ct, ct]
            f(m, n, k, bl, _addr(A), lda, k_idx_a, _addr(B), ldb, k_idx_b, _addr(scale_b), ldsb, _addr(Cm), ldc,
              _addr(D), ldd, _addr(bias), self._clamp_arg(clamp_min), self._clamp_arg(clamp_max))
        else:
            f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, ct, ct,
                          C.POINTER(self.params_cls)]
            f(m, n, k, _addr(A), lda, k_idx_a, _addr(B), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd, _addr(bias),
              self._clamp_arg(clamp_min), self._clamp_arg(clamp_max), None if params is None else C.byref(params))
        check("run_gemm " + self.type_name)


SIBLING_TYPES = (
    [f"gemm_1xnbias_clamp_{t}_qai8dx_qsi4cxt" for t in ("f32", "f16", "bf16")]
    + ["gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt", "gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp",
       "gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8", "gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p"]
    + [f"gemm_1xnbias_clamp_{t}_qai8dx_qsi8cxt" for t in ("f32", "f16")]
    + [f"gemm_1xnbias_clamp_{t}_qai8dxp_qsi8cxp" for t in ("f32", "f16")]
    + [f"gemm_1xnbias_clamp_{t}_f16_qsi4c2t" for t in ("f16", "f32")]
)


# ---- int8 convolution wrappers (include/tqt_b200_conv_i8_i8.h) ---------------------------------------
class ConvParams(C.Structure):
    """struct tqt_conv_params (host struct; reference src/common/tqt_conv.h:23-34)."""
    _fields_ = [(n, _sz * 3) for n in ("input_shape", "output_shape", "kernel_shape", "stride", "dilation", "pad")] + \
               [("input_channel", _sz), ("output_channel", _sz), ("groups", _sz)]

    @classmethod
    def make(cls, input_channel, output_channel, groups, input_shape, kernel_shape, stride=(1, 1, 1), dilation=(1, 1, 1),
             pad=(0, 0, 0), output_shape=None):
        p = cls()
        if output_shape is None:   # the caller computes it; this is the usual formula
            output_shape = [(input_shape[i] + 2 * pad[i] - dilation[i] * (kernel_shape[i] - 1) - 1) // stride[i] + 1
                            for i in range(3)]
        for name, v in (("input_shape", input_shape), ("output_shape", output_shape), ("kernel_shape", kernel_shape),
                        ("stride", stride), ("dilation", dilation), ("pad", pad)):
            setattr(p, name, (_sz * 3)(*[int(x) for x in v]))
        p.input_channel, p.output_channel, p.groups = input_channel, output_channel, groups
        return p


CONV_TYPES = ("convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp", "convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt",
              "convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8", "convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p")


class ConvI8(_UKernel):
    """One of the int8 convolution wrappers: an im2col step (plain, or fused with the pack) and run_conv, which is the
    run_gemm of the requantising GEMM type of the same name."""

    def __init__(self, type_name: str):
        self.type_name = type_name
        self.channel_first = type_name.startswith("convcf")
        self.packed = type_name.endswith("p")
        common = (("get_m_step", 0), ("get_n_step", 0), ("get_c_offset", 3), ("get_bias_offset", 1), ("get_d_offset", 3),
                  ("get_d_size", 2))
        if self.channel_first and self.packed:
            own = (("get_a_packed_offset", 4), ("get_b_im2colpack_offset", 4), ("get_a_packed_size", 2),
                   ("get_b_im2colpack_size", 2))
            runs = ["run_a_pack", "run_b_im2colpack"]
        elif self.channel_first:
            own = (("get_a_offset", 3), ("get_b_im2col_size", 2), ("get_b_im2col_offset", 3))
            runs = ["run_im2col"]
        elif self.packed:
            own = (("get_a_im2colpack_offset", 4), ("get_b_packed_offset", 4), ("get_a_im2colpack_size", 2),
                   ("get_b_packed_size", 2))
            runs = ["run_bt_pack", "run_a_im2colpack"]
        else:
            own = (("get_b_offset", 3), ("get_a_im2col_size", 2), ("get_a_im2col_offset", 3))
            runs = ["run_im2col"]
        self.helpers_size = common + own
        self.actions = [h[0] for h in self.helpers_size] + runs + ["run_conv"]
        self.params_cls = QaI8QsI8DxQaI8Params if self.channel_first else QaI8QaI8QsI8CxParams
        super().__init__()

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_im2col(self, group_idx, activation, im2col_buf, params):
        f = self._sym("run_im2col")
        f.argtypes = [_sz, _vp, _vp, C.POINTER(ConvParams)]
        f.restype = None
        f(group_idx, _addr(activation), _addr(im2col_buf), None if params is None else C.byref(params))
        check("run_im2col " + self.type_name)

    def run_im2colpack(self, group_idx, activation, ld_packed, k_idx, packed, params):
        """run_a_im2colpack (channel-last) / run_b_im2colpack (channel-first)."""
        f = self._sym("run_b_im2colpack" if self.channel_first else "run_a_im2colpack")
        f.argtypes = [_sz, _vp, _sz, _sz, _vp, C.POINTER(ConvParams)]
        f.restype = None
        f(group_idx, _addr(activation), ld_packed, k_idx, _addr(packed), None if params is None else C.byref(params))
        check("run_im2colpack " + self.type_name)

    def run_conv(self, m, n, k, A, lda, k_idx_a, B, ldb, k_idx_b, Cm, ldc, D, ldd, bias, clamp_min, clamp_max, params):
        f = self._sym("run_conv")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, C.c_int8, C.c_int8,
                      C.POINTER(self.params_cls)]
        f.restype = None
        f(m, n, k, _addr(A), lda, k_idx_a, _addr(B), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd, _addr(bias),
          int(clamp_min), int(clamp_max), None if params is None else C.byref(params))
        check("run_conv " + self.type_name)


FLOAT_TYPES = (
    [f"gemm_1xnbias_clamp_{t}_{t}_{t}{s}" for t in ("f32", "f16", "bf16") for s in ("", "p", "t")]
    + [f"gemm_1xnbias_clamp_{t}_{t}p_{t}p" for t in ("f32", "f16", "bf16")]
    + [f"gemm_mx1bias_clamp_{t}_{t}_{t}" for t in ("f32", "f16")] + [f"gemm_mx1bias_clamp_{t}_{t}p_{t}p" for t in ("f32", "f16")]
    + [f"gemm_1xnbias_clamp_{td}_bf16{a}_bf16{b}" for td in ("f16", "f32") for a, b in (("", ""), ("", "t"), ("p", "p"))]
)


class FloatGemm(_UKernel):
    """One of the unquantised GEMM kernel types (include/tqt_b200_gemm_float.h): gemm_<bias>_clamp_<TD>_<TA>[p]_<TB>[p|t]."""

    def __init__(self, type_name: str):
        self.type_name = type_name
        parts = type_name.split("_")            # gemm, <bias>, clamp, TD, TA[p], TB[p|t]
        self.bias_per_row = parts[1] == "mx1bias"
        self.td = parts[3]
        self.ta = parts[4].rstrip("p")
        self.a_packed = parts[4].endswith("p")
        self.b_packed = parts[5].endswith("p")
        self.b_transposed = parts[5].endswith("t")
        common = (("get_m_step", 0), ("get_n_step", 0), ("get_c_offset", 3), ("get_bias_offset", 1), ("get_d_offset", 3),
                  ("get_d_size", 2))
        own, packs = (), []
        if self.a_packed:
            own += (("get_a_packed_offset", 4), ("get_a_packed_size", 2))
            packs.append("run_a_pack")
        else:
            own += (("get_a_offset", 3),)
        if self.b_packed:
            own += (("get_b_packed_offset", 4), ("get_b_packed_size", 2))
            packs += ["run_b_pack", "run_bt_pack"]
        else:
            own += (("get_b_offset", 3),)
        self.helpers_size = common + own
        self.actions = [h[0] for h in self.helpers_size] + packs + ["run_gemm"]
        super().__init__()

    def run_a_pack(self, m, k, lda, lda_packed, k_idx, A, A_packed):
        self._pack("run_a_pack", m, k, lda, lda_packed, k_idx, A, A_packed)

    def run_b_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_b_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_bt_pack(self, n, k, ldb, ldb_packed, k_idx, B, B_packed):
        self._pack("run_bt_pack", n, k, ldb, ldb_packed, k_idx, B, B_packed)

    def run_gemm(self, m, n, k, A, lda, k_idx_a, B, ldb, k_idx_b, Cm, ldc, D, ldd, bias, clamp_min, clamp_max):
        f = self._sym("run_gemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, C.c_float, C.c_float]
        f.restype = None
        if self.td == "f32":
            lo, hi = C.c_float(clamp_min), C.c_float(clamp_max)
        else:
            cv = f16_bits if self.td == "f16" else bf16_bits
            lo, hi = half_arg(cv(clamp_min)), half_arg(cv(clamp_max))
        f(m, n, k, _addr(A), lda, k_idx_a, _addr(B), ldb, k_idx_b, _addr(Cm), ldc, _addr(D), ldd, _addr(bias), lo, hi)
        check("run_gemm " + self.type_name)


IGEMM_TYPES = ("igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp", "igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt",
               "igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8", "igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8")


class IgemmI8(_UKernel):
    """One of the int8 implicit-GEMM convolution types: run_igemm gathers the activation operand from the input tensor."""

    def __init__(self, type_name: str):
        self.type_name = type_name
        self.channel_first = type_name.startswith("igemmcf")
        self.packed = "qsi8cxp" in type_name or "qsi8dxp" in type_name
        common = (("get_m_step", 0), ("get_n_step", 0), ("get_c_offset", 3), ("get_bias_offset", 1), ("get_d_offset", 3),
                  ("get_d_size", 2))
        if self.channel_first:
            own = (("get_a_packed_offset", 4), ("get_a_packed_size", 2)) if self.packed else (("get_a_offset", 3),)
            runs = ["run_a_pack"] if self.packed else []
        else:
            own = (("get_b_packed_offset", 4), ("get_b_packed_size", 2)) if self.packed else (("get_b_offset", 3),)
            runs = ["run_bt_pack"] if self.packed else []
        self.helpers_size = common + own
        self.actions = [h[0] for h in self.helpers_size] + runs + ["run_igemm"]
        self.params_cls = QaI8QsI8DxQaI8Params if self.channel_first else QaI8QaI8QsI8CxParams
        super().__init__()

    def run_a_pack(self, m, k, ldw, ldw_packed, k_idx, W, W_packed):
        self._pack("run_a_pack", m, k, ldw, ldw_packed, k_idx, W, W_packed)

    def run_bt_pack(self, n, k, ldw, ldw_packed, k_idx, W, W_packed):
        self._pack("run_bt_pack", n, k, ldw, ldw_packed, k_idx, W, W_packed)

    def run_igemm(self, m, n, k, inp, group_idx, pos_idx, weights, ldw, D, ldd, bias, clamp_min, clamp_max, conv_params,
                  quant_params):
        """pos_idx: first output position of the call (m_idx for channel-last, n_idx for channel-first)."""
        f = self._sym("run_igemm")
        f.argtypes = [_sz, _sz, _sz, _vp, _sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, C.c_int8, C.c_int8,
                      C.POINTER(ConvParams), C.POINTER(self.params_cls)]
        f.restype = None
        f(m, n, k, _addr(inp), group_idx, pos_idx, 0, _addr(weights), ldw, 0, None, 0, _addr(D), ldd, _addr(bias),
          int(clamp_min), int(clamp_max), None if conv_params is None else C.byref(conv_params),
          None if quant_params is None else C.byref(quant_params))
        check("run_igemm " + self.type_name)


# ---- extensions ------------------------------------------------------------------------------------
_TA_NAMES = {"float32": "f32", "float16": "f16", "bfloat16": "bf16"}


def quant_pack_qai8dxp(A, A_packed, scale_a, zero_point_a, m=None, k=None, lda=None):
    """Dynamic per-row asymmetric int8 quantisation of A (f32 / f16 / bf16) into the packed LHS layout."""
    ta = _TA_NAMES[str(A.dtype).replace("torch.", "")]
    f = getattr(lib(), f"tqt_run_quant_pack_qai8dxp_{ta}_{VARIANT}")
    f.argtypes = [_sz, _sz, _vp, _sz, _vp, _vp, _vp]
    f.restype = None
    m = A.shape[0] if m is None else m
    k = A.shape[1] if k is None else k
    lda = A.stride(0) if lda is None else lda
    f(m, k, _addr(A), lda, _addr(A_packed), _addr(scale_a), _addr(zero_point_a))
    check("quant_pack_qai8dxp")


_A_TYPE = {"f32": 0, "f16": 1, "bf16": 2}


def quant_gemm_w4a8(td, m, n, k, A, lda, A_packed, scale_a, zero_point_a, B_packed, ldb, Cm, ldc, D, ldd, bias, clamp_min,
                    clamp_max, scale_b):
    """tqt_run_quant_gemm_1xnbias_clamp_<td>_qai8dxp_qsi4cxp: quantise the activations A (f32 / f16 / bf16 tensor) and run
    the W4A8 GEMM on them; one cooperative launch where the library has a fused form for the shape."""
    f = getattr(lib(), f"tqt_run_quant_gemm_1xnbias_clamp_{td}_qai8dxp_qsi4cxp_{VARIANT}")
    f.argtypes = [_sz, _sz, _sz, _vp, _sz, C.c_int, _vp, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _sz, _vp, C.c_float, C.c_float, _vp]
    f.restype = None
    a_type = _A_TYPE[_TA_NAMES[str(A.dtype).replace("torch.", "")]]
    if td == "f32":
        lo, hi = C.c_float(clamp_min), C.c_float(clamp_max)
    else:
        cv = f16_bits if td == "f16" else bf16_bits
        lo, hi = half_arg(cv(clamp_min)), half_arg(cv(clamp_max))
    f(m, n, k, _addr(A), lda, a_type, _addr(A_packed), _addr(scale_a), _addr(zero_point_a), _addr(B_packed), ldb, _addr(Cm), ldc,
      _addr(D), ldd, _addr(bias), lo, hi, _addr(scale_b))
    check("quant_gemm_w4a8")


def quant_gemm_w4a8_static(m, n, k, A, lda, B_packed, ldb, Cm, ldc, D, ldd, bias, clamp_min, clamp_max, scale_b):
    """tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp: quantise + W4A8 GEMM (f32 output) for callers that
    cannot allocate: the intermediates live in a static device array of the library.  Status UNSUPPORTED (raised by
    ``check``) when the call exceeds the array."""
    f = getattr(lib(), f"tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp_{VARIANT}")
    f.argtypes = [_sz, _sz, _sz, _vp, _sz, C.c_int, _vp, _sz, _vp, _sz, _vp, _sz, _vp, C.c_float, C.c_float, _vp]
    f.restype = None
    a_type = _A_TYPE[_TA_NAMES[str(A.dtype).replace("torch.", "")]]
    f(m, n, k, _addr(A), lda, a_type, _addr(B_packed), ldb, _addr(Cm), ldc, _addr(D), ldd, _addr(bias), clamp_min, clamp_max,
      _addr(scale_b))
    check("quant_gemm_w4a8_static")


def quant_qai8dx(A, A_q, scale_a, zero_point_a):
    """Same quantiser with a plain row-major int8 result."""
    ta = _TA_NAMES[str(A.dtype).replace("torch.", "")]
    f = getattr(lib(), f"tqt_run_quant_qai8dx_{ta}_sm100a")
    f.argtypes = [_sz, _sz, _vp, _sz, _vp, _sz, _vp, _vp]
    f.restype = None
    f(A.shape[0], A.shape[1], _addr(A), A.stride(0), _addr(A_q), A_q.stride(0), _addr(scale_a), _addr(zero_point_a))
    check("quant_qai8dx")


def _unpack(name, rows, k, src, ld_packed, dst, ld):
    f = getattr(lib(), f"tqt_run_{name}_{VARIANT}")
    f.argtypes = [_sz, _sz, _vp, _sz, _vp, _sz]
    f.restype = None
    f(rows, k, _addr(src), ld_packed, _addr(dst), ld)
    check(name)


def a_unpack_i8(m, k, A_packed, lda_packed, A, lda):
    _unpack("a_unpack_i8", m, k, A_packed, lda_packed, A, lda)


def a_unpack_f16(m, k, A_packed, lda_packed, A, lda):
    _unpack("a_unpack_f16", m, k, A_packed, lda_packed, A, lda)


def bt_unpack_qsi4cxp(n, k, B_packed, ldb_packed, B, ldb):
    _unpack("bt_unpack_qsi4cxp", n, k, B_packed, ldb_packed, B, ldb)


def bt_unpack_qsi4c2p(n, k, B_packed, ldb_packed, B, ldb):
    _unpack("bt_unpack_qsi4c2p", n, k, B_packed, ldb_packed, B, ldb)


EXTENSION_SYMBOLS = (
    ["tqt_cuda_set_stream", "tqt_cuda_get_stream", "tqt_cuda_get_last_status", "tqt_cuda_get_last_cuda_error",
     "tqt_cuda_read_device_fault", "tqt_cuda_version", "tqt_shard_plan_n", "tqt_cuda_kernel_choice_w4a8",
     "tqt_cuda_debug_f16_bits", "tqt_cuda_debug_bf16_bits", "tqt_cuda_debug_set_timing_buffer",
     "tqt_cuda_debug_stream_read", "tqt_cuda_set_output_replicas", "tqt_cuda_debug_set_path", "tqt_cuda_debug_inject_wait_failure",
     "tqt_cuda_debug_last_kernel"]
    + [f"tqt_run_quant_pack_qai8dxp_{t}_{VARIANT}" for t in ("f32", "f16", "bf16")]
    + [f"tqt_run_quant_gemm_1xnbias_clamp_{t}_qai8dxp_qsi4cxp_{VARIANT}" for t in ("f32", "f16", "bf16")]
    + [f"tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp_{VARIANT}"]
    + [f"tqt_run_quant_qai8dx_{t}_sm100a" for t in ("f32", "f16", "bf16")]
    + [f"tqt_run_{n}_{VARIANT}" for n in ("a_unpack_i8", "a_unpack_f16", "bt_unpack_qsi4cxp", "bt_unpack_qsi4c2p")]
)


def all_ukernels():
    return [GemmClampI32I8I8(), GemmClampI32I8pI8p(), GemmReqI8(), GemmW4A8("f32"), GemmW4A8("f16"),
            GemmW4A8("bf16"), GemmW4A16("f16"), GemmW4A16("f32")] + [SiblingGemm(t) for t in SIBLING_TYPES] + \
           [ConvI8(t) for t in CONV_TYPES] + [IgemmI8(t) for t in IGEMM_TYPES] + [FloatGemm(t) for t in FLOAT_TYPES]
