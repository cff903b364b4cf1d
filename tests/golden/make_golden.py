"""Builds the reference's CPU model code in true 32-bit (-DUSE_FP32, no CMake:
its CMakeLists.txt hard-codes the bfloat16 build), runs ref_harness.cpp on the
tiny golden model (and on its twin with RoPE base 1e6 over 2,100 positions) and
stores the logits as ref_logits.npy and ref_logits_long.npy beside this file;
runs ref_tokenizer_harness.cpp (the reference's own tokenizer) on the texts of
golden_tokenizer.py and stores its tokens and ids as ref_tokens.json.

    python tests/golden/make_golden.py /path/to/reference

The committed files came from exactly this script.
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
        def run(config, script, out_name):
            golden_model.write_model_dir(tmp / "model", config)
            (tmp / "script.txt").write_text(script)
            subprocess.run([str(tmp / "harness"), str(tmp / "model" / "model.safetensors"), str(tmp / "script.txt"),
                            str(tmp / out_name), str(config["num_hidden_layers"]), str(config["num_attention_heads"]),
                            str(config["num_key_value_heads"]), str(config["hidden_size"]), str(config["vocab_size"]),
                            str(config["rope_theta"])], check=True)
            return np.fromfile(tmp / out_name, dtype="<f4").reshape(-1, config["vocab_size"])

        logits = run(golden_model.CONFIG, golden_model.script_text(), "out.f32")
        long_logits = run(golden_model.CONFIG_LONG,
                          golden_model.script_text(golden_model.CALLS_LONG, {0: golden_model.long_request()}), "long.f32")
        tokenizer_golden(ref, tmp, objects)
    assert logits.shape[0] == len(golden_model.wanted_rows())
    np.save(here / "ref_logits.npy", logits)
    print("wrote", here / "ref_logits.npy", logits.shape)
    assert long_logits.shape[0] == golden_model.LONG_LENGTH
    np.save(here / "ref_logits_long.npy", long_logits[golden_model.KEPT_LONG])
    print("wrote", here / "ref_logits_long.npy", (len(golden_model.KEPT_LONG), long_logits.shape[1]))


def tokenizer_golden(ref, tmp, objects):
    """The reference's own Tokenizer (src/tokenizer.cpp, src/bpe.cpp) on the handmade vocabulary and the texts of
    golden_tokenizer.py; what it makes of them goes to ref_tokens.json."""
    import json

    import golden_tokenizer

    here = Path(__file__).resolve().parent
    flags = ["-std=c++17", "-O2", "-DUSE_FP32", "-DSPDLOG_COMPILED_LIB", f"-I{ref}/include",
             f"-I{ref}/include/third_party", f"-I{ref}/include/models"]
    subprocess.run(["g++", *flags, "-c", str(here / "ref_tokenizer_harness.cpp"), "-o", str(tmp / "tok_harness.o")], check=True)
    others = [o for o in objects if not o.endswith("_ref_harness.o")]
    subprocess.run(["g++", str(tmp / "tok_harness.o"), *others, "-o", str(tmp / "tok_harness"), "-lpthread"], check=True)
    folder = tmp / "tok"
    folder.mkdir()
    golden_tokenizer.write_files(folder)
    (tmp / "texts.json").write_text(json.dumps(golden_tokenizer.TEXTS))
    subprocess.run([str(tmp / "tok_harness"), str(folder / "tokenizer.json"), str(folder / "tokenizer_config.json"),
                    str(tmp / "texts.json"), str(tmp / "tokens.json")], check=True)
    result = json.loads((tmp / "tokens.json").read_text())
    assert len(result) == len(golden_tokenizer.TEXTS)
    (here / "ref_tokens.json").write_text(json.dumps(result, indent=0, ensure_ascii=True) + "\n")
    print("wrote", here / "ref_tokens.json", len(result), "texts")


if __name__ == "__main__":
    main()
