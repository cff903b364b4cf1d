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


@pytest.mark.parametrize("extra", [[], SANITIZE], ids=["plain", "asan_ubsan"])
def test_native_engine_host_side_in_cpp(tmp_path, extra):
    """The native engine's JSON reader, safetensors reader, manifest check, typed configuration, registry and
    run-order checks (csrc/engine), from C++ alone: tests/native/engine_host_test.cpp."""
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "engine_host_test"
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", "-Wextra", *extra, "-I", str(ROOT / "easy_gpt" / "cpp_b200" / "csrc" / "engine"),
                            str(ROOT / "tests" / "native" / "engine_host_test.cpp"), "-o", str(exe)], capture_output=True, text=True)
    if build.returncode != 0 and extra and "sanitize" in build.stderr:
        pytest.skip("this compiler has no sanitizer runtime")
    assert build.returncode == 0, build.stderr
    work = tmp_path / "files"
    work.mkdir()
    out = subprocess.run([str(exe), str(work)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all checks passed" in out.stdout


def test_kernel_interface_header_matches_the_launchers():
    """csrc/engine/kernels_api.h declares the kernel library's launchers for the native engine; extern "C" gives the
    linker nothing to check, so every declaration is compared with the launcher's definition."""
    import re

    csrc = ROOT / "easy_gpt" / "cpp_b200" / "csrc"
    header = " ".join((csrc / "engine" / "kernels_api.h").read_text().split())
    declared = dict(re.findall(r"int (eg_\w+)\((.*?)\);", header))
    assert len(declared) >= 17
    defined = {}
    for source in csrc.glob("*.cu"):
        for name, args in re.findall(r"EG_API int (eg_\w+)\((.*?)\)\s*\{", source.read_text(), re.S):
            defined[name] = " ".join(args.split())
    for name, args in declared.items():
        assert defined.get(name) == args, name
