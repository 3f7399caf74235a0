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
                    "TMATMUL_BIAS(c, a, b, bias); }\n  return 0;\n}\n")
    inc = ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include")]
    proc = subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", *inc, str(good)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    bad = tmp_path / "bad_bias.cpp"
    bad.write_text(good.read_text().replace("Tile<TileType::Bias, float,", "Tile<TileType::Bias, int32_t,"))
    proc = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", *inc, str(bad)], capture_output=True, text=True)
    assert proc.returncode != 0 and "No supported bias data type" in proc.stderr


@pytest.mark.gpu
def test_reference_tile_programs_run_exactly_on_gpu():
    exe = compile_example()
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "tile programs ok" in proc.stdout
    assert proc.stdout.count(": 0 mismatches") == 5
