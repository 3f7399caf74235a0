"""The C++ operator surface (include/pto/pto-inst.hpp, include/pto/b200_launchers.hpp): it must compile as plain
host C++ against the C ABI (CPU check), and the reference's two GEMM tile programs written with it must give exact
results on the GPU (GPU check)."""
import os
import subprocess

import pytest

from pto_isa_mirror_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "examples", "gemm_tile_program.cpp")
EXE = os.path.join(ROOT, "examples", "gemm_tile_program")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def compile_example():
    build.build()
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           SRC, "-L", os.path.join(ROOT, "pto_isa_mirror_b200", "lib"), "-lpto_b200", "-L", os.path.join(CUDA, "lib64"),
           "-lcudart", "-Wl,-rpath," + os.path.join(ROOT, "pto_isa_mirror_b200", "lib"), "-o", EXE]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return EXE


def test_operator_surface_compiles_as_host_cpp():
    assert os.path.exists(compile_example())


def test_illegal_dtype_combination_is_a_compile_error(tmp_path):
    """CheckMadValid is a static_assert in the reference (include/pto/cpu/TMatmul.hpp:39-49); so it is here."""
    src = tmp_path / "bad.cpp"
    src.write_text('#include "pto/pto-inst.hpp"\nusing namespace pto;\nint main() {\n'
                   "  TileLeft<half, 128, 64> a; TileRight<half, 64, 256> b; TileAcc<int32_t, 128, 256> c;\n"
                   "  TMATMUL(c, a, b);\n  return 0;\n}\n")
    proc = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                          capture_output=True, text=True)
    assert proc.returncode != 0 and "Not supported data type" in proc.stderr


def test_one_row_and_bias_forms_compile(tmp_path):
    """TGEMV / TGEMV_ACC / TGEMV_BIAS / TMATMUL_BIAS exist with the reference's argument order, and a bias tile of the
    wrong type is a compile error (CheckBiasValid, include/pto/cpu/TMatmul.hpp:159-167)."""
    good = tmp_path / "good.cpp"
    good.write_text('#include "pto/pto-inst.hpp"\nusing namespace pto;\nint main() {\n'
                    "  TileLeft<half, 1, 64> a; TileRight<half, 64, 256> b; TileAcc<float, 1, 256> c;\n"
                    "  Tile<TileType::Bias, float, 1, 256, BLayout::RowMajor, 1, 256> bias;\n"
                    "  if (false) { TGEMV(c, a, b); TGEMV_ACC(c, c, a, b); TGEMV_BIAS(c, a, b, bias); "
                    "TMATMUL_BIAS(c, a, b, bias); }\n"
                    "  TileLeft<float8_e4m3_t, 1, 128> xa; TileRight<float8_e5m2_t, 128, 256> xb;\n"
                    "  TileLeftScale<float8_e8m0_t, 1, 4> xsa; TileRightScale<float8_e8m0_t, 4, 256> xsb;\n"
                    "  if (false) { TGEMV_MX(c, xa, xsa, xb, xsb); TGEMV_MX(c, c, xa, xsa, xb, xsb); "
                    "TGEMV_MX(c, xa, xsa, xb, xsb, bias); }\n  return 0;\n}\n")
    inc = ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include")]
    proc = subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", *inc, str(good)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    bad = tmp_path / "bad_bias.cpp"
    bad.write_text(good.read_text().replace("Tile<TileType::Bias, float,", "Tile<TileType::Bias, int32_t,"))
    proc = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", *inc, str(bad)], capture_output=True, text=True)
    assert proc.returncode != 0 and "No supported bias data type" in proc.stderr


REJECTIONS_CPP = r"""
#include <cstdio>
#include <cstring>
#include <string>
#include "pto/pto-inst.hpp"
using namespace pto;
static int fails = 0;
static std::string last;
static void handler(const char* what, int) { ++fails; last = what; }
static bool rejected(const char* fragment) {
    const bool ok = (fails == 1) && last.find(fragment) != std::string::npos;
    std::printf("%s: %s [%s]\n", fragment, ok ? "rejected" : "NOT rejected as expected", last.c_str());
    fails = 0; last.clear();
    return ok;
}
int main() {
    b200::error_handler() = handler;
    // device pointers are never dereferenced: every program below must be refused before anything is launched
    constexpr int M = 128, N = 256, K = 256, mxK = 128, KG = K / 32;
    auto* a = reinterpret_cast<float8_e4m3_t*>(0x10000000);
    auto* b = reinterpret_cast<float8_e4m3_t*>(0x20000000);
    auto* sa = reinterpret_cast<float8_e8m0_t*>(0x30000000);
    auto* sb = reinterpret_cast<float8_e8m0_t*>(0x40000000);
    auto* c = reinterpret_cast<float*>(0x50000000);
    using GlobalA = GlobalTensor<float8_e4m3_t, TileShape2D<float8_e4m3_t, M, mxK, Layout::ND>,
                                 BaseShape2D<float8_e4m3_t, M, K, Layout::ND>, Layout::ND>;
    using GlobalB = GlobalTensor<float8_e4m3_t, TileShape2D<float8_e4m3_t, mxK, N, Layout::DN>,
                                 BaseShape2D<float8_e4m3_t, K, N, Layout::DN>, Layout::DN>;
    using GlobalSA = GlobalTensor<float8_e8m0_t, TileShape2D<float8_e8m0_t, M, mxK / 32, Layout::MX_A_ND>,
                                  BaseShape2D<float8_e8m0_t, M, KG, Layout::MX_A_ND>, Layout::MX_A_ND>;
    using GlobalSB = GlobalTensor<float8_e8m0_t, TileShape2D<float8_e8m0_t, mxK / 32, N, Layout::MX_B_DN>,
                                  BaseShape2D<float8_e8m0_t, KG, N, Layout::MX_B_DN>, Layout::MX_B_DN>;
    using GlobalC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
    using SmallC = GlobalTensor<float, Shape<1, 1, 1, M, N / 2>, Stride<M * N, M * N, M * N, N, 1>>;
    TileLeft<float8_e4m3_t, M, mxK> at;
    TileRight<float8_e4m3_t, mxK, N> bt;
    TileLeftScale<float8_e8m0_t, M, mxK / 32> ast;
    TileRightScale<float8_e8m0_t, mxK / 32, N> bst;
    TileAcc<float, M, N> acc;
    bool ok = true;
    auto chain = [&](int sa_step, int sb_step) {
        for (int kIter = 0; kIter < 2; ++kIter) {
            GlobalA gA(a + kIter * mxK);
            GlobalB gB(b + kIter * mxK);
            GlobalSA gSA(sa + kIter * sa_step);
            GlobalSB gSB(sb + kIter * sb_step);
            TLOAD(at, gA); TLOAD(bt, gB); TLOAD(ast, gSA); TLOAD(bst, gSB);
            if (kIter == 0) TMATMUL_MX(acc, at, ast, bt, bst); else TMATMUL_MX(acc, acc, at, ast, bt, bst);
        }
    };
    GlobalC cG(c);
    chain(0, mxK / 32);                       // A's scale tile does not advance with K
    TSTORE(cG, acc);
    ok &= rejected("scale tiles");
    chain(mxK / 32, 0);                       // B's scale tile does not advance with K
    TSTORE(cG, acc);
    ok &= rejected("scale tiles");
    chain(mxK / 32, mxK / 32);                // a legal chain into a destination with too few columns
    SmallC smallG(c);
    TSTORE(smallG, acc);
    ok &= rejected("smaller than the accumulator");
    {                                         // the bias form of a block-scaled chain without scratch
        Tile<TileType::Bias, float, 1, N, BLayout::RowMajor, 1, N> bias;
        using GlobalBias = GlobalTensor<float, Shape<1, 1, 1, 1, N>, Stride<N, N, N, N, 1>>;
        GlobalBias bG(c);
        TLOAD(bias, bG);
        GlobalA gA(a); GlobalB gB(b); GlobalSA gSA(sa); GlobalSB gSB(sb);
        TLOAD(at, gA); TLOAD(bt, gB); TLOAD(ast, gSA); TLOAD(bst, gSB);
        TMATMUL_MX(acc, at, ast, bt, bst, bias);
        TSTORE(cG, acc);
        ok &= rejected("set_workspace");
    }
    {                                         // a scaling tile shorter than the accumulator is wide
        auto* a8 = reinterpret_cast<int8_t*>(0x10000000);
        auto* b8 = reinterpret_cast<int8_t*>(0x20000000);
        using GA = GlobalTensor<int8_t, TileShape2D<int8_t, M, 64, Layout::ND>, BaseShape2D<int8_t, M, K, Layout::ND>>;
        using GB = GlobalTensor<int8_t, TileShape2D<int8_t, 64, N, Layout::DN>, BaseShape2D<int8_t, K, N, Layout::DN>, Layout::DN>;
        using GOut = GlobalTensor<bfloat16_t, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
        using GWords = GlobalTensor<uint64_t, Shape<1, 1, 1, 1, N / 2>, Stride<N, N, N, N, 1>>;
        TileLeft<int8_t, M, 64> l; TileRight<int8_t, 64, N> r; TileAcc<int32_t, M, N> acc32;
        Tile<TileType::Scaling, uint64_t, 1, N / 2, BLayout::RowMajor, 1, N / 2, SLayout::NoneBox> fp;
        GA gA(a8); GB gB(b8); GWords gW(reinterpret_cast<uint64_t*>(0x60000000));
        GOut gO(reinterpret_cast<bfloat16_t*>(c));
        TLOAD(l, gA); TLOAD(r, gB); TLOAD(fp, gW);
        TMATMUL(acc32, l, r);
        TSTORE_FP(gO, acc32, fp);
        ok &= rejected("fewer words");
    }
    std::printf("%s\n", ok ? "rejections ok" : "rejections FAILED");
    return ok ? 0 : 1;
}
"""


def test_illegal_tile_programs_are_rejected_before_any_launch(tmp_path):
    """Chains that one GEMM cannot honour are refused through the error handler: scale tiles that do not follow the K
    slices, a destination smaller than the accumulator, a block-scaled bias chain without scratch, a scaling tile
    that is too short. Nothing here needs a GPU: each case must fail before the C ABI would touch the device."""
    build.build()
    src = tmp_path / "rejections.cpp"
    src.write_text(REJECTIONS_CPP)
    exe = tmp_path / "rejections"
    lib_dir = os.path.join(ROOT, "pto_isa_mirror_b200", "lib")
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           str(src), "-L", lib_dir, "-lpto_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + lib_dir, "-o", str(exe)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and "rejections ok" in run.stdout, run.stdout + run.stderr


@pytest.mark.gpu
def test_reference_tile_programs_run_exactly_on_gpu():
    exe = compile_example()
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "tile programs ok" in proc.stdout
    assert proc.stdout.count(": 0 mismatches") == 11
