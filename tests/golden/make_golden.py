"""Builds the reference's CPU model code in true 32-bit (-DUSE_FP32, no CMake:
its CMakeLists.txt hard-codes the bfloat16 build), runs ref_harness.cpp on the
tiny golden model and stores the logits as ref_logits.npy beside this file.

    python tests/golden/make_golden.py /path/to/reference

The committed ref_logits.npy came from exactly this script.
"""
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
import golden_model  # noqa: E402


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference (a checkout of the reference's sources)")
    ref = Path(sys.argv[1])
    here = Path(__file__).resolve().parent
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        sources = [p for p in sorted((ref / "src").glob("*.cpp")) if p.name != "main.cpp"]
        sources += sorted((ref / "src" / "models").glob("*.cpp"))
        sources += sorted((ref / "src" / "third_party" / "spdlog").glob("*.cpp"))
        sources.append(here / "ref_harness.cpp")
        flags = ["-std=c++17", "-O2", "-DUSE_FP32", "-DSPDLOG_COMPILED_LIB", f"-I{ref}/include",
                 f"-I{ref}/include/third_party", f"-I{ref}/include/models"]

        def compile_one(src):
            obj = tmp / (src.parent.name + "_" + src.stem + ".o")
            subprocess.run(["g++", *flags, "-c", str(src), "-o", str(obj)], check=True)
            return str(obj)

        with ThreadPoolExecutor(8) as pool:
            objects = list(pool.map(compile_one, sources))
        subprocess.run(["g++", *objects, "-o", str(tmp / "harness"), "-lpthread"], check=True)
        golden_model.write_model_dir(tmp / "model")
        (tmp / "script.txt").write_text(golden_model.script_text())
        c = golden_model.CONFIG
        subprocess.run([str(tmp / "harness"), str(tmp / "model" / "model.safetensors"), str(tmp / "script.txt"),
                        str(tmp / "out.f32"), str(c["num_hidden_layers"]), str(c["num_attention_heads"]),
                        str(c["num_key_value_heads"]), str(c["hidden_size"]), str(c["vocab_size"]),
                        str(c["rope_theta"])], check=True)
        logits = np.fromfile(tmp / "out.f32", dtype="<f4").reshape(-1, c["vocab_size"])
    assert logits.shape[0] == len(golden_model.wanted_rows())
    np.save(here / "ref_logits.npy", logits)
    print("wrote", here / "ref_logits.npy", logits.shape)


if __name__ == "__main__":
    main()
