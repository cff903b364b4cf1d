"""Builds the CUDA kernels into one shared library, in the tree, at first use.

Each ``.cu`` file is compiled by nvcc for sm_100a into ``_build/<name>.o`` and
the objects are linked into ``libeasygpt_kernels.so`` beside this file.  A stamp
records the hash of the sources and the flags, so a stale library is rebuilt
and a current one is loaded as it is.  If the tree is not writable, the build
goes to a per-user folder under the system's temporary directory.  A line is
printed to stderr for every file, so that a first call does not look hung.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libeasygpt_kernels.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _sources():
    return sorted(HERE.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(HERE.glob("*.cu")) + list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc was not found (set NVCC or put it on PATH); the CUDA kernels cannot be built")


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def _current(lib: Path, stamp: Path, fp: str) -> bool:
    try:
        return lib.is_file() and json.loads(stamp.read_text()).get("fingerprint") == fp
    except (OSError, ValueError):
        return False


def library_path(verbose: bool = True) -> Path:
    """Path of an up-to-date kernel library, building it if need be."""
    fp = _fingerprint()
    in_tree = (HERE / LIB_NAME, HERE / "_build" / "stamp.json")
    if _current(*in_tree, fp):
        return in_tree[0]
    if _writable(HERE / "_build") and _writable(HERE):
        out_dir, build_dir = HERE, HERE / "_build"
    else:
        base = Path(tempfile.gettempdir()) / f"easy_gpt_b200_build_{os.getuid()}"
        out_dir, build_dir = base, base / "_build"
        build_dir.mkdir(parents=True, exist_ok=True)
        if _current(out_dir / LIB_NAME, build_dir / "stamp.json", fp):
            return out_dir / LIB_NAME
    nvcc = _nvcc()
    sources = _sources()

    def say(msg):
        if verbose:
            print(f"[easy_gpt.cpp_b200] {msg}", file=sys.stderr, flush=True)

    say(f"building {len(sources)} CUDA files for sm_100a into {out_dir} (first call only)")

    def compile_one(src: Path) -> str:
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        say(f"compiled {src.name}")
        return str(obj)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp_lib = out_dir / (LIB_NAME + f".{os.getpid()}.tmp")
    r = subprocess.run([nvcc, "-shared", "-o", str(tmp_lib), *objects], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, out_dir / LIB_NAME)
    (build_dir / "stamp.json").write_text(json.dumps({"fingerprint": fp}))
    say(f"built {out_dir / LIB_NAME}")
    return out_dir / LIB_NAME


HOST_LIB_NAME = "libeasygpt_host.so"
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


def _host_fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list((HERE / "host").glob("*.cpp")) + list((HERE / "host").glob("*.hpp"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()


def host_library_path(verbose: bool = True) -> Path:
    """Path of an up-to-date library of the host runtime (``host/*.cpp``: page pools, cache
    bookkeeping, step packing, scheduler), built by the C++ compiler; no CUDA is involved."""
    fp = _host_fingerprint()
    in_tree = (HERE / HOST_LIB_NAME, HERE / "_build" / "host_stamp.json")
    if _current(*in_tree, fp):
        return in_tree[0]
    if _writable(HERE / "_build") and _writable(HERE):
        out_dir, build_dir = HERE, HERE / "_build"
    else:
        base = Path(tempfile.gettempdir()) / f"easy_gpt_b200_build_{os.getuid()}"
        out_dir, build_dir = base, base / "_build"
        build_dir.mkdir(parents=True, exist_ok=True)
        if _current(out_dir / HOST_LIB_NAME, build_dir / "host_stamp.json", fp):
            return out_dir / HOST_LIB_NAME
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler was found (set CXX or put g++ on PATH); the host runtime cannot be built")
    if verbose:
        print(f"[easy_gpt.cpp_b200] building the host runtime into {out_dir} (first call only)", file=sys.stderr, flush=True)
    tmp_lib = out_dir / (HOST_LIB_NAME + f".{os.getpid()}.tmp")
    sources = [str(p) for p in sorted((HERE / "host").glob("*.cpp"))]
    r = subprocess.run([cxx, *HOST_FLAGS, "-I", str(HERE / "host"), *sources, "-o", str(tmp_lib)], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {HOST_LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, out_dir / HOST_LIB_NAME)
    (build_dir / "host_stamp.json").write_text(json.dumps({"fingerprint": fp}))
    return out_dir / HOST_LIB_NAME


ENGINE_LIB_NAME = "libeasygpt_engine.so"
ENGINE_EXE_NAME = "easy_llm"
ENGINE_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall"]


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), str(Path(_nvcc()).resolve().parent.parent), "/usr/local/cuda"):
        if cand and (Path(cand) / "include" / "cuda_runtime.h").is_file():
            return Path(cand)
    raise BuildError("the CUDA toolkit's headers were not found (set CUDA_HOME); the native engine cannot be built")


def _engine_fingerprint(kernel_fp: str) -> str:
    h = hashlib.sha256()
    files = list((HERE / "engine").glob("*.cpp")) + list((HERE / "engine").glob("*.hpp")) + list((HERE / "engine").glob("*.h")) \
        + list((HERE / "host").glob("*.hpp"))
    for p in sorted(files):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ENGINE_FLAGS).encode())
    h.update(kernel_fp.encode())
    return h.hexdigest()


def engine_paths(verbose: bool = True):
    """(library, program): the native engine (``engine/*.hpp`` behind the C interface of ``engine/engine_api.cpp``) as a
    shared library, and the ``easy_llm`` program of ``engine/main.cpp`` linked against it.  Both are built by the C++
    compiler against the CUDA runtime and cuBLAS and linked to the kernel library beside them."""
    kernels = library_path(verbose)
    out_dir = kernels.parent
    build_dir = out_dir / "_build"
    fp = _engine_fingerprint(_fingerprint())
    lib, exe, stamp = out_dir / ENGINE_LIB_NAME, out_dir / ENGINE_EXE_NAME, build_dir / "engine_stamp.json"
    if _current(lib, stamp, fp) and exe.is_file():
        return lib, exe
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler was found (set CXX or put g++ on PATH); the native engine cannot be built")
    cuda = _cuda_home()
    lib_dirs = [d for d in (cuda / "lib64", cuda / "lib") if d.is_dir()]
    if verbose:
        print(f"[easy_gpt.cpp_b200] building the native engine into {out_dir} (first call only)", file=sys.stderr, flush=True)
    common = [*ENGINE_FLAGS, "-I", str(cuda / "include"), "-I", str(HERE / "host")]
    link = ["-L", str(out_dir), "-leasygpt_kernels", *[a for d in lib_dirs for a in ("-L", str(d))], "-lcudart", "-lcublas", "-lcublasLt", "-ldl",
            "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in lib_dirs]]
    tmp_lib = out_dir / (ENGINE_LIB_NAME + f".{os.getpid()}.tmp")
    r = subprocess.run([cxx, *common, "-shared", str(HERE / "engine" / "engine_api.cpp"), "-o", str(tmp_lib), *link], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {ENGINE_LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    tmp_exe = out_dir / (ENGINE_EXE_NAME + f".{os.getpid()}.tmp")
    r = subprocess.run([cxx, *common, str(HERE / "engine" / "main.cpp"), "-o", str(tmp_exe), *link],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {ENGINE_EXE_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_exe, exe)
    stamp.write_text(json.dumps({"fingerprint": fp}))
    return lib, exe


def build_plugin(source, output, verbose: bool = True) -> Path:
    """Builds a plugin of the native engine (a .cu or .cpp file that includes ``engine/plugin.hpp`` and exports
    ``easygpt_register``) into a shared library at ``output``."""
    library_path(verbose)
    cuda = _cuda_home()
    source, output = Path(source), Path(output)
    flags = ["-std=c++17", "-O2", "-I", str(HERE / "engine"), "-I", str(HERE), "-I", str(HERE / "host"), "-I", str(cuda / "include")]
    if source.suffix == ".cu":
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", *flags, str(source), "-o", str(output),
               "-L", str(library_path(False).parent), "-leasygpt_kernels", "-lcublas", "-lcublasLt"]
    else:
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        cmd = [cxx, "-shared", "-fPIC", *flags, str(source), "-o", str(output)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"building the plugin {source} failed:\n{r.stdout}\n{r.stderr}")
    return output


if __name__ == "__main__":
    print(library_path())
    print(host_library_path())
    print(*engine_paths())
