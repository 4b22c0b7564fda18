"""Builds the C++ host driver (tests/cpp/test_cuda_backend.cpp) against the C-ABI library and
the oracle, and runs it on the GPU: the compiled-language view of the drop-in boundary."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _build(tmp: Path) -> Path:
    from agention_infer_b200.build import build_library
    from oracle import oracle as orc
    lib = build_library()
    orc.build()
    exe = tmp / "test_cuda_backend"
    cmd = ["g++", "-O1", "-std=c++17", "-I", str(ROOT / "include"), "-I", str(ROOT / "oracle"),
           str(ROOT / "tests" / "cpp" / "test_cuda_backend.cpp"), "-o", str(exe),
           f"-L{lib.parent}", "-lagention_b200", f"-L{orc.LIB.parent}", "-loracle",
           f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{orc.LIB.parent}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_cpp_host_compiles_and_links(tmp_path):
    assert _build(tmp_path).exists()


@pytest.mark.gpu
def test_cpp_host_parity(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "FAIL" not in res.stdout
