"""The host runtime from C++ alone (no GPU, no Python on its path): tests/native/host_runtime_test.cpp is
compiled against csrc/host and run, once plainly and once under the address and undefined-behaviour
sanitizers (a read past a block table's row, a page freed twice into the wrong list or a signed overflow
in the packing arithmetic stops the run)."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SANITIZE = ["-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all"]


@pytest.mark.parametrize("extra", [[], SANITIZE], ids=["plain", "asan_ubsan"])
def test_host_runtime_in_cpp(tmp_path, extra):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "host_runtime_test"
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-Wextra", *extra, "-I", str(ROOT / "easy_gpt" / "cpp_b200" / "csrc" / "host"),
                            str(ROOT / "tests" / "native" / "host_runtime_test.cpp"), "-o", str(exe)], capture_output=True, text=True)
    if build.returncode != 0 and extra and "sanitize" in build.stderr:
        pytest.skip("this compiler has no sanitizer runtime")
    assert build.returncode == 0, build.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "all checks passed" in out.stdout
