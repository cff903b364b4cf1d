"""The tiny model and the calls of the golden comparison with the reference's
own CPU code.  Weights come from an integer hash (no library random stream), so
the very same values can be rebuilt anywhere."""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 32, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 48, "vocab_size": 64, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 64, "bos_token_id": -1, "eos_token_id": -1,
}

# request 0: 8 tokens, then 1; request 1: 5 tokens, then a portion of 4 on a
# non-empty cache; then both decode one token in one batch (different lengths).
REQUESTS = {0: [3, 41, 7, 19, 60, 2, 33, 8, 27, 11], 1: [50, 1, 22, 9, 14, 37, 5, 48, 30, 6]}
CALLS = [
    [(0, 0, 8)], [(0, 8, 1)], [(1, 0, 5)], [(1, 5, 4)], [(0, 9, 1), (1, 9, 1)],
]


# A second case for what the first cannot show: rotation angles of thousands of radians.  The same sizes with
# RoPE base 1e6 (Qwen2.5's), one request of 2,100 tokens: 2,048 at once, a portion of 50 on that cache, two
# single tokens.  Only the rows of KEPT_LONG are stored (the others are computed and dropped).
CONFIG_LONG = dict(CONFIG, rope_theta=1000000.0, max_position_embeddings=4096)
LONG_LENGTH = 2100
CALLS_LONG = [[(0, 0, 2048)], [(0, 2048, 50)], [(0, 2098, 1)], [(0, 2099, 1)]]
KEPT_LONG = [0, 1, 1000, 2046, 2047, 2048, 2049, 2050, 2051, 2052, 2095, 2096, 2097, 2098, 2099]


def long_request() -> list:
    z = (np.arange(LONG_LENGTH, dtype=np.uint64) + np.uint64(77)) * np.uint64(0x9E3779B97F4A7C15)
    z ^= z >> np.uint64(29)
    z *= np.uint64(0xBF58476D1CE4E5B9)
    z ^= z >> np.uint64(32)
    return [int(t) for t in (z % np.uint64(CONFIG["vocab_size"]))]


def _hash_uniform(n: int, stream: int) -> np.ndarray:
    z = (np.arange(n, dtype=np.uint64) + np.uint64(stream) * np.uint64(0x100000001B3)) * np.uint64(0x9E3779B97F4A7C15)
    z ^= z >> np.uint64(30)
    z *= np.uint64(0xBF58476D1CE4E5B9)
    z ^= z >> np.uint64(27)
    z *= np.uint64(0x94D049BB133111EB)
    z ^= z >> np.uint64(31)
    return ((z >> np.uint64(40)).astype(np.float64) / float(1 << 24)).astype(np.float32)


def weights() -> dict[str, np.ndarray]:
    c = CONFIG
    H, NH, NKV, I, V = c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["intermediate_size"], c["vocab_size"]
    HD = H // NH
    out: dict[str, np.ndarray] = {}
    stream = [0]

    def mat(*shape, scale=0.2, centre=0.0):
        stream[0] += 1
        u = _hash_uniform(int(np.prod(shape)), stream[0]).reshape(shape)
        return (centre + (u - np.float32(0.5)) * np.float32(scale)).astype(np.float32)

    out["model.embed_tokens.weight"] = mat(V, H)
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out[p + "self_attn.q_proj.weight"] = mat(NH * HD, H)
        out[p + "self_attn.q_proj.bias"] = mat(NH * HD)
        out[p + "self_attn.k_proj.weight"] = mat(NKV * HD, H)
        out[p + "self_attn.k_proj.bias"] = mat(NKV * HD)
        out[p + "self_attn.v_proj.weight"] = mat(NKV * HD, H)
        out[p + "self_attn.v_proj.bias"] = mat(NKV * HD)
        out[p + "self_attn.o_proj.weight"] = mat(H, NH * HD)
        out[p + "input_layernorm.weight"] = mat(H, centre=1.0)
        out[p + "post_attention_layernorm.weight"] = mat(H, centre=1.0)
        out[p + "mlp.gate_proj.weight"] = mat(I, H)
        out[p + "mlp.up_proj.weight"] = mat(I, H)
        out[p + "mlp.down_proj.weight"] = mat(H, I)
    out["model.norm.weight"] = mat(H, centre=1.0)
    return out


def write_model_dir(folder, config=None) -> None:
    """The weights do not depend on the configuration's RoPE base: both cases share them."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config or CONFIG))
    header, blobs, off = {}, [], 0
    for k, v in weights().items():
        b = v.tobytes()
        header[k] = {"dtype": "F32", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hs = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hs)) + hs + b"".join(blobs))


def script_text(calls=None, requests=None) -> str:
    calls, requests = calls or CALLS, requests or REQUESTS
    lines = []
    for call in calls:
        parts = [str(len(call))]
        for rid, start, n in call:
            parts += [str(rid), str(start), str(n)] + [str(t) for t in requests[rid][start:start + n]]
        lines.append(" ".join(parts))
    return "\n".join(lines) + "\n"


def wanted_rows():
    """(request, position) of every logits row the calls produce, in order."""
    rows = []
    for call in CALLS:
        for rid, start, n in call:
            rows += [(rid, start + i) for i in range(n)]
    return rows
