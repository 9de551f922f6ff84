"""CPU-only checks of the C ABI: the library loads, exports every symbol the headers declare,
and its host-side helpers (steps, offsets, sizes, shard plan, half-by-value passing) compute what
the headers say.  No kernel is launched."""
import ctypes as C
import os
import re

import pytest

from __graft_entry__ import ROOT, load


@pytest.fixture(scope="module")
def pkg():
    import importlib.util
    spec = importlib.util.spec_from_file_location("tqt_b200_build", os.path.join(ROOT, "torq-tile_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build()
    return load()


def _declared_symbols():
    """Expand the declaration macros of include/*.h the way the preprocessor does (g++ -E)."""
    import subprocess
    names = set()
    for h in ("tqt_b200_common.h", "tqt_b200_gemm_i8_i8.h", "tqt_b200_gemm_i8_i4.h", "tqt_b200_gemm_f16_i4.h", "tqt_b200_gemm_siblings.h",
              "tqt_b200_conv_i8_i8.h", "tqt_b200_gemm_float.h", "tqt_b200_ext.h"):
        out = subprocess.check_output(["/usr/bin/g++", "-E", "-P", "-x", "c++", os.path.join(ROOT, "include", h)], text=True)
        names |= set(re.findall(r"\b(tqt_[a-z0-9_]+?)\s*\(", out))
    return {n for n in names if not n.endswith("_t")}


def test_exports_every_declared_symbol(pkg):
    lib = pkg.lib()
    declared = _declared_symbols()
    assert len(declared) > 100
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    for uk in pkg.all_ukernels():
        for s in uk.symbol_names():
            assert s in declared, s
    for s in pkg.EXTENSION_SYMBOLS:
        assert s in declared, s


def test_steps_and_plain_offsets(pkg):
    for uk in pkg.all_ukernels():
        assert uk.get_m_step() == 128 and uk.get_n_step() == 128
    u = pkg.GemmClampI32I8I8()
    # reference: (m_idx*lda + k_idx), (k_idx*ldb + n_idx), int32 C/D  (gemm_clamp_i32_i8_i8 ..._4x1vl_rvv.cpp:35-64)
    assert u.get_a_offset(128, 7, 512) == 128 * 512 + 7
    assert u.get_b_offset(256, 3, 1000) == 3 * 1000 + 256
    assert u.get_c_offset(128, 256, 300) == (128 * 300 + 256) * 4
    assert u.get_d_offset(128, 256, 300) == (128 * 300 + 256) * 4
    assert u.get_d_size(5, 7) == 140
    w = pkg.GemmW4A8("bf16")
    assert w.get_c_offset(128, 128, 1000) == (128 * 1000 + 128) * 2
    assert w.get_bias_offset(256) == 512 and w.get_d_size(3, 5) == 30
    assert pkg.GemmW4A8("f32").get_d_offset(128, 0, 10) == 128 * 10 * 4
    r = pkg.GemmReqI8()
    assert r.get_d_offset(128, 128, 4096) == 128 * 4096 + 128 and r.get_bias_offset(128) == 512
    assert r.get_c_offset(128, 0, 64) == 128 * 64 * 4


def test_packed_sizes_and_offsets(pkg):
    w = pkg.GemmW4A8("f32")
    assert w.get_a_packed_size(1, 4096) == 32 * 16384
    assert w.get_a_packed_size(2048, 4096) == 16 * 32 * 16384
    assert w.get_b_packed_size(4096, 4096) == 32 * 32 * 8448
    assert w.get_b_packed_size(129, 130) == 2 * 2 * 8448
    assert w.get_b_packed_offset(256, 0, 4096, 128) == 2 * 32 * 8448
    assert w.get_b_packed_offset(256, 384, 4096, 128) == (2 * 32 + 3) * 8448
    assert w.get_a_packed_offset(128, 256, 4096, 128) == (32 + 2) * 16384
    r = pkg.GemmReqI8()
    assert r.get_b_packed_size(4096, 4096) == 32 * 32 * 16384
    assert r.get_b_packed_offset(128, 128, 300, 128) == (3 + 1) * 16384
    h = pkg.GemmW4A16("f16")
    assert h.get_a_packed_size(8192, 8192) == 64 * 128 * 16384
    assert h.get_b_packed_size(28672, 8192) == 224 * 64 * 8192
    assert h.get_a_packed_offset(128, 64, 8192, 128) == (128 + 1) * 16384
    assert h.get_scale_b_offset(128, 3, 256) == (128 * 256 + 3) * 2


def test_shard_plan(pkg):
    # the N of the three sharded configurations, at 1/2/4/8 ranks: contiguous, 128-aligned, complete
    for n in (4096, 14336, 28672, 1000, 128, 130):
        for world in (1, 2, 4, 8):
            pos = 0
            sizes = []
            for rank in range(world):
                b, c = pkg.shard_plan_n(n, world, rank)
                assert b == pos and b % 128 == 0 or c == 0
                pos = b + c
                sizes.append(c)
            assert pos == n
            full = [s for s in sizes if s]
            assert max(sizes) - min(sizes) <= 128 or n % 128
    assert pkg.shard_plan_n(14336, 8, 3) == (3 * 1792, 1792)
    assert pkg.shard_plan_n(28672, 8, 7) == (7 * 3584, 3584)


def test_half_by_value_passing(pkg):
    lib = pkg.lib()
    lib.tqt_cuda_debug_f16_bits.restype = C.c_uint16
    lib.tqt_cuda_debug_f16_bits.argtypes = [C.c_float]
    lib.tqt_cuda_debug_bf16_bits.restype = C.c_uint16
    lib.tqt_cuda_debug_bf16_bits.argtypes = [C.c_float]
    for bits in (0x0000, 0x3C00, 0xBC00, 0x7BFF, 0xFBFF, 0x0001, 0x1234, 0xFFFF):
        assert lib.tqt_cuda_debug_f16_bits(pkg.half_arg(bits)) == bits
        assert lib.tqt_cuda_debug_bf16_bits(pkg.half_arg(bits)) == bits
    assert pkg.f16_bits(65504.0) == 0x7BFF and pkg.f16_bits(-0.5) == 0xB800
    assert pkg.bf16_bits(1.0) == 0x3F80 and pkg.bf16_bits(65504.0) == 0x4780 and pkg.bf16_bits(-65504.0) == 0xC780


def test_status_word_without_gpu(pkg):
    """params == NULL returns silently with status OK (reference ..._qsi4cxp_4x1vl_rvv.cpp:205-207); a
    NULL output with a non-empty problem is rejected before any launch."""
    w = pkg.GemmW4A8("f32")
    w.run_gemm(4, 4, 8, 0, 8, 0, 0, 8, 0, None, 4, 0, 4, None, -1.0, 1.0, None)
    assert pkg.lib().tqt_cuda_get_last_status() == 0
    p = pkg.QaI8DxQsI4CxParams(16, 16, 16)
    with pytest.raises(pkg.TqtError):
        w.run_gemm(4, 4, 8, 16, 8, 0, 16, 8, 0, None, 4, None, 4, None, -1.0, 1.0, p)
    assert pkg.lib().tqt_cuda_get_last_status() == 1
    # odd k is illegal for int4 weights ("Must be a multiple of 2")
    with pytest.raises(pkg.TqtError):
        w.run_gemm(4, 4, 7, 16, 7, 0, 16, 7, 0, None, 4, 16, 4, None, -1.0, 1.0, p)
    # empty problems are accepted
    w.run_gemm(0, 4, 8, None, 8, 0, None, 8, 0, None, 4, None, 4, None, -1.0, 1.0, p)
    assert pkg.lib().tqt_cuda_get_last_status() == 0
    assert pkg.lib().tqt_cuda_kernel_choice_w4a8(1, 4096, 4096) == 1
    assert pkg.lib().tqt_cuda_kernel_choice_w4a8(2048, 14336, 4096) == 0


def test_conv_wrappers_without_gpu(pkg, tmp_path):
    """The convolution wrappers' helpers are the GEMM types' helpers (reference: src/conv/conv_i8_i8/*/
    tqt_conv*_4x1vl_rvv.cpp forward the same way); a geometry that cannot be narrowed is rejected before any launch; a C
    caller fills every ukernel table positionally, which checks member order and signatures at compile time."""
    import subprocess
    g = pkg.GemmReqI8()
    for t in pkg.CONV_TYPES:
        c = pkg.ConvI8(t)
        assert c.get_m_step() == 128 and c.get_n_step() == 128
        assert c.get_d_size(5, 7) == 35 and c.get_c_offset(128, 256, 1000) == (128 * 1000 + 256) * 4
        assert c.get_bias_offset(128) == 512 and c.get_d_offset(128, 256, 1000) == 128 * 1000 + 256
    c = pkg.ConvI8(pkg.CONV_TYPES[0])
    assert c.get_a_im2colpack_size(200, 300) == g.get_a_packed_size(200, 300) == 2 * 3 * 16384
    assert c.get_a_im2colpack_offset(128, 256, 300, 72) == g.get_a_packed_offset(128, 256, 300, 72)
    assert c.get_b_packed_offset(256, 128, 300, 44) == g.get_b_packed_offset(256, 128, 300, 44)
    c = pkg.ConvI8(pkg.CONV_TYPES[1])
    assert c.get_a_im2col_size(10, 27) == 270 and c.get_a_im2col_offset(3, 5, 27) == 86 and c.get_b_offset(3, 5, 27) == 86
    c = pkg.ConvI8(pkg.CONV_TYPES[2])
    assert c.get_b_im2col_size(27, 10) == 270 and c.get_b_im2col_offset(3, 5, 10) == 53 and c.get_a_offset(3, 5, 27) == 86
    c = pkg.ConvI8(pkg.CONV_TYPES[3])
    assert c.get_b_im2colpack_size(200, 300) == 2 * 3 * 16384 and c.get_a_packed_size(1, 1) == 16384
    # rejected before any launch: group index out of range, channels not divisible by groups, k_idx off the K step,
    # an extent of 2^31; NULL geometry returns silently
    cp = pkg.ConvParams.make(8, 8, 2, (1, 4, 4), (1, 3, 3))
    for args in ((2, 16, 36, 0, 16, cp), (0, 16, 36, 64, 16, cp), (0, 16, 36, 0, 16, pkg.ConvParams.make(9, 8, 2, (1, 4, 4), (1, 3, 3))),
                 (0, 16, 36, 0, 16, pkg.ConvParams.make(8, 8, 2, (1, 4, 1 << 31), (1, 3, 3))), (0, None, 36, 0, 16, cp)):
        with pytest.raises(pkg.TqtError):
            pkg.ConvI8(pkg.CONV_TYPES[0]).run_im2colpack(*args)
        assert pkg.lib().tqt_cuda_get_last_status() == 1
    with pytest.raises(pkg.TqtError):
        pkg.ConvI8(pkg.CONV_TYPES[2]).run_im2col(5, 16, 16, cp)
    pkg.ConvI8(pkg.CONV_TYPES[0]).run_im2colpack(0, 16, 36, 0, 16, None)
    assert pkg.lib().tqt_cuda_get_last_status() == 0
    libdir = os.path.join(ROOT, "torq-tile_b200")
    S = "_128x128_sm100a"
    tables = []
    for t, members in ((pkg.CONV_TYPES[0], ("get_m_step get_n_step get_a_im2colpack_offset get_b_packed_offset get_c_offset get_bias_offset "
                                            "get_d_offset get_d_size get_a_im2colpack_size get_b_packed_size run_bt_pack run_a_im2colpack run_conv")),
                       (pkg.CONV_TYPES[1], ("get_m_step get_n_step get_b_offset get_c_offset get_bias_offset get_d_offset get_d_size "
                                            "get_a_im2col_size get_a_im2col_offset run_im2col run_conv")),
                       (pkg.CONV_TYPES[2], ("get_m_step get_n_step get_a_offset get_c_offset get_bias_offset get_d_offset get_d_size "
                                            "get_b_im2col_size get_b_im2col_offset run_im2col run_conv")),
                       (pkg.CONV_TYPES[3], ("get_m_step get_n_step get_a_packed_offset get_b_im2colpack_offset get_c_offset get_bias_offset "
                                            "get_d_offset get_d_size get_a_packed_size get_b_im2colpack_size run_a_pack run_b_im2colpack run_conv"))):
        tables.append(f"    struct tqt_{t}_ukernel u{len(tables)} = {{" + ", ".join(f"tqt_{m}_{t}{S}" for m in members.split()) + "};")
    for t, members in ((pkg.IGEMM_TYPES[0], "get_m_step get_n_step get_b_packed_offset get_c_offset get_bias_offset get_d_offset get_d_size "
                                            "get_b_packed_size run_bt_pack run_igemm"),
                       (pkg.IGEMM_TYPES[1], "get_m_step get_n_step get_b_offset get_c_offset get_bias_offset get_d_offset get_d_size run_igemm"),
                       (pkg.IGEMM_TYPES[2], "get_m_step get_n_step get_a_offset get_c_offset get_bias_offset get_d_offset get_d_size run_igemm"),
                       (pkg.IGEMM_TYPES[3], "get_m_step get_n_step get_a_packed_offset get_c_offset get_bias_offset get_d_offset get_d_size "
                                            "get_a_packed_size run_a_pack run_igemm")):
        tables.append(f"    struct tqt_{t}_ukernel u{len(tables)} = {{" + ", ".join(f"tqt_{m}_{t}{S}" for m in members.split()) + "};")
    tables.append("    if (!(u4.run_igemm && u5.run_igemm && u6.run_igemm && u7.run_a_pack)) return 1;")
    src = tmp_path / "conv_tables.c"
    src.write_text('#include "tqt_b200_conv_i8_i8.h"\nint main(void) {\n' + "\n".join(tables) +
                   "\n    return (int)u0.get_m_step() + (u1.run_conv && u2.run_im2col && u3.run_b_im2colpack);\n}\n")
    exe = tmp_path / "conv_tables"
    r = subprocess.run(["/usr/bin/gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                        "-L", libdir, "-ltorq_tile_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([str(exe)]).returncode == 129


def test_output_replicas_argument_checks(pkg):
    """tqt_cuda_set_output_replicas is host-side state: more than 7 replicas or missing pointers are refused,
    an empty list clears it (no GPU needed)."""
    import ctypes as C
    lib = pkg.lib()
    f = lib.tqt_cuda_set_output_replicas
    f.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t]
    f.restype = None
    arr = (C.c_void_p * 8)(*[C.c_void_p(1 << (20 + i)) for i in range(8)])
    f(C.c_void_p(4096), 4096, arr, 8)
    assert lib.tqt_cuda_get_last_status() != 0
    f(None, 4096, arr, 2)
    assert lib.tqt_cuda_get_last_status() != 0
    f(C.c_void_p(4096), 0, arr, 2)          # a registered buffer needs its size
    assert lib.tqt_cuda_get_last_status() != 0
    f(C.c_void_p(4096), 4096, arr, 7)
    assert lib.tqt_cuda_get_last_status() == 0
    f(None, 0, None, 0)
    assert lib.tqt_cuda_get_last_status() == 0


def test_output_replicas_refuse_an_output_outside_the_registered_buffer(pkg):
    """While replicas are set, a run_gemm whose output range is not inside [local_base, local_base + local_bytes)
    is refused before anything is launched (host-side check: fake addresses, no GPU needed).  The refusal is what
    is tested: the accepted case is covered on a GPU."""
    base, size = 1 << 30, 64 * 256 * 2          # a 64 x 256 bf16 output buffer
    peers = [1 << 31, (1 << 31) + (1 << 24)]
    w = pkg.GemmW4A8("bf16")
    p = pkg.QaI8DxQsI4CxParams(16, 16, 16)
    try:
        pkg.set_output_replicas(base, size, peers)
        for (m, n, D, ldd) in ((64, 256, base - 512, 256),          # starts before the buffer
                               (64, 256, base + 512, 256),          # runs past its end
                               (65, 256, base, 256),                # one row too many
                               (64, 128, base + 2 * 200, 256),      # column slice that overhangs the last row
                               (64, 256, 1 << 29, 256)):            # another buffer altogether
            with pytest.raises(pkg.TqtError):
                w.run_gemm(m, n, 128, 16, 128, 0, 16, 128, 0, None, n, D, ldd, None, -1.0, 1.0, p)
            assert pkg.lib().tqt_cuda_get_last_status() == 1
        w16 = pkg.GemmW4A16("f16")
        with pytest.raises(pkg.TqtError):
            w16.run_gemm(64, 256, 128, 32, 16, 128, 0, 16, 128, 0, 16, 4, None, 256, base + 512, 256, None, -1.0, 1.0)
        assert pkg.lib().tqt_cuda_get_last_status() == 1
    finally:
        pkg.set_output_replicas(0, 0, [])


def test_headers_compile_as_c_and_cxx(tmp_path):
    """The boundary is a C ABI: every header under include/ must be accepted by a C11 and a C++17 compiler,
    with the 16-bit float prototypes and without them (TQT_B200_NO_HALF_TYPES)."""
    import subprocess
    inc = os.path.join(ROOT, "include")
    headers = sorted(f for f in os.listdir(inc) if f.endswith(".h"))
    body = "".join(f'#include "{h}"\n' for h in headers) + \
        "int main(void) { return (int)tqt_get_m_step_gemm_clamp_i32_i8_i8_128x128_sm100a(); }\n"
    for name, cc, std in (("t.c", "/usr/bin/gcc", "-std=c11"), ("t.cpp", "/usr/bin/g++", "-std=c++17")):
        src = tmp_path / name
        src.write_text(body)
        for extra in ([], ["-DTQT_B200_NO_HALF_TYPES"]):
            r = subprocess.run([cc, std, "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-I", inc] + extra + [str(src)],
                               capture_output=True, text=True)
            assert r.returncode == 0, r.stderr


def test_c_program_links_and_calls_helpers(pkg, tmp_path):
    """A plain C caller links the library and uses the size / offset helpers (no GPU needed for those)."""
    import subprocess
    libdir = os.path.join(ROOT, "torq-tile_b200")
    src = tmp_path / "caller.c"
    src.write_text('''
#include <stdio.h>
#include "tqt_b200_gemm_i8_i4.h"
#include "tqt_b200_gemm_siblings.h"
int main(void) {
    printf("%zu %zu %zu %zu\\n",
           tqt_get_n_step_gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp_128x128_sm100a(),
           tqt_get_b_packed_size_gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp_128x128_sm100a(256, 256),
           tqt_get_b_packed_size_gemm_1xnbias_clamp_f32_qai8dxp_qsi8cxp_128x128_sm100a(128, 128),
           tqt_get_b_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a(128, 64, 512));
    return 0;
}
''')
    exe = tmp_path / "caller"
    r = subprocess.run(["/usr/bin/gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-L", libdir,
                        "-ltorq_tile_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    # 2 x 2 qsi4cx blocks of 8448 B; one int8 block with its row sums; nibble offset n_idx * (ldb / 2) + k_idx / 2
    assert out.stdout.split() == ["128", str(4 * 8448), str(16384 + 256), str(128 * 256 + 32)]


def test_sibling_ukernel_tables_fill_and_link(pkg, tmp_path):
    """Every sibling kernel type has a struct tqt_<type>_ukernel with the members of the reference's
    <type>_interface.h; a C caller fills the tables with this variant's symbols (positionally for one of them,
    which checks member order and signatures at compile time) and links.  Also accepted by a C++17 compiler."""
    import subprocess
    libdir = os.path.join(ROOT, "torq-tile_b200")
    src = tmp_path / "tables.c"
    src.write_text(r'''
#include "tqt_b200_gemm_siblings.h"
int main(void) {
    struct tqt_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_ukernel a = {
        tqt_get_m_step_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a, tqt_get_n_step_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a,
        tqt_get_a_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a, tqt_get_b_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a,
        tqt_get_c_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a, tqt_get_bias_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a,
        tqt_get_d_offset_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a, tqt_get_d_size_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a,
        tqt_run_gemm_1xnbias_clamp_f32_qai8dx_qsi4cxt_128x128_sm100a};
    struct tqt_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_ukernel b;
    b.run_gemm = tqt_run_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a;
    b.run_bt_pack = tqt_run_bt_pack_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a;
    struct tqt_gemm_1xnbias_clamp_f16_qai8dxp_qsi8cxp_ukernel c;
    c.run_gemm = tqt_run_gemm_1xnbias_clamp_f16_qai8dxp_qsi8cxp_128x128_sm100a;
    struct tqt_gemm_1xnbias_clamp_f16_f16_qsi4c2t_ukernel d;
    d.run_gemm = tqt_run_gemm_1xnbias_clamp_f16_f16_qsi4c2t_128x128_sm100a;
    struct tqt_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_ukernel e;
    e.run_gemm = tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a;
    struct tqt_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_ukernel f;
    f.run_gemm = tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a;
    struct tqt_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_ukernel g;
    g.run_gemm = tqt_run_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a;
    return (int)a.get_m_step() + (b.run_gemm && c.run_gemm && d.run_gemm && e.run_gemm && f.run_gemm && g.run_gemm && b.run_bt_pack);
}
''')
    exe = tmp_path / "tables"
    r = subprocess.run(["/usr/bin/gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                        "-L", libdir, "-ltorq_tile_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 129          # m_step 128 + all table members set
    r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-I",
                        os.path.join(ROOT, "include"), "-x", "c++", str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
