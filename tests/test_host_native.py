"""The host runtime from C++ alone (no GPU, no Python on its path): tests/native/host_runtime_test.cpp is
compiled against csrc/host and run."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_host_runtime_in_cpp(tmp_path):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "host_runtime_test"
    subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-Wextra", "-I", str(ROOT / "easy_gpt" / "cpp_b200" / "csrc" / "host"),
                    str(ROOT / "tests" / "native" / "host_runtime_test.cpp"), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "all checks passed" in out.stdout
