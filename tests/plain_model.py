"""Plain, slow implementation of the Qwen2 dense decoder, written from the
reference's formulas (MarsPain/easy_gpt.cpp).  Whole sequences, no cache, one
function per part, float32 (or float64) on the CPU.  It shares no code with the
product package: it parses config.json and reads safetensors by itself.

It has been compared once with the reference's own CPU model code compiled in
true 32-bit (tests/golden/make_golden.py); the logits of that run are committed
under tests/golden/ and tests/test_plain_vs_golden.py replays the comparison.

Two things go beyond what the reference can express and rest on the formulas
alone: a sliding window (the reference ignores Qwen2's window keys) and an
untied lm_head / configurable eps (the reference hard-codes both).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------
# reading a model folder (own reader; not the product's)
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """u64 little-endian header length, JSON header, raw data
    (src/models/loader.cpp:213-227, 229-270)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(raw[base + lo:base + hi], dtype=np_dtype).reshape(meta["shape"]).copy()
        if meta["dtype"] == "BF16":
            t = torch.from_numpy(arr.astype(np.int32) << 16).view(torch.float32)
        else:
            t = torch.from_numpy(arr)
        out[name] = t
    return out


def read_model_dir(model_dir, dtype=torch.float32, round_to_bf16=False):
    """Returns (config dict, {name: tensor}).  With round_to_bf16 every floating
    tensor is rounded to bfloat16 first and widened again: this is what a
    bfloat16 engine holds, computed here in full precision."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = {}
    for k, v in read_safetensors(model_dir / "model.safetensors").items():
        if v.is_floating_point():
            v = v.float()
            if round_to_bf16:
                v = v.to(torch.bfloat16).float()
            v = v.to(dtype)
        weights[k] = v
    return cfg, weights


# --------------------------------------------------------------------------
# configuration (the keys of src/config.cpp:16-31 and the ones Qwen2 adds)
# --------------------------------------------------------------------------

def sizes(cfg: dict) -> dict:
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh  # src/models/self_attn.cpp:169-174
    layers = cfg["num_hidden_layers"]
    window = [None] * layers
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window"):
        first = cfg.get("max_window_layers", layers)
        for i in range(layers):
            if i >= first:
                window[i] = int(cfg["sliding_window"])
    return dict(L=layers, H=cfg["hidden_size"], NH=nh, NKV=cfg["num_key_value_heads"], HD=hd,
                I=cfg["intermediate_size"], V=cfg["vocab_size"], theta=float(cfg["rope_theta"]),
                eps=float(cfg.get("rms_norm_eps", 1e-6)), tied=bool(cfg.get("tie_word_embeddings", False)),
                window=window)


# --------------------------------------------------------------------------
# the parts
# --------------------------------------------------------------------------

def embed(table: torch.Tensor, ids) -> torch.Tensor:
    """x[t,:] = E[id[t],:], ids range-checked (src/models/embedding.cpp:54-76)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise IndexError("token id out of range")
    return table[ids]


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y = w * (x * 1/sqrt(mean(x^2) + eps)) (src/models/norm.cpp:46-60)."""
    mean_sq = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(mean_sq + eps)
    return gain.reshape(-1) * (x * inv)


def linear(x, weight, bias=None):
    """y = x W^T + b with W [out, in] (src/models/linear.cpp:42-44, src/ops.cpp:79-121)."""
    y = x @ weight.t()
    if bias is not None:
        y = y + bias.reshape(-1)
    return y


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[k] = 1 / theta^(2k/HD), k < HD/2 (src/ops.cpp:172-177).  Computed
    in double and rounded once to float32, so that every implementation that does
    the same holds the very same table."""
    k = np.arange(head_dim // 2, dtype=np.float64)
    return torch.from_numpy((1.0 / np.power(np.float64(theta), 2.0 * k / head_dim)).astype(np.float32))


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half rotation over the whole head (src/ops.cpp:404-421): the angle
    pos*inv_freq[k] is a float32 product; x'[k] = x[k] cos - x[k+HD/2] sin,
    x'[k+HD/2] = x[k] sin + x[k+HD/2] cos.  x is [T, heads, HD]."""
    hd = x.shape[-1]
    half = hd // 2
    inv = rope_inverse_frequencies(hd, theta)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]      # float32 angle
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def attention_core(q, k, v, positions, window=None, round_scores_like_reference=False):
    """q [T,NH,HD], k,v [T,NKV,HD] of one whole sequence.  Query head h reads
    KV head h // (NH/NKV) (src/tensor.cpp:246-253, src/models/self_attn.cpp:324-327);
    scores are masked causally (src/models/self_attn.cpp:75-98), scaled by
    1/sqrt(HD) (:253) and soft-maxed over the keys with the row maximum taken
    out first (src/tensor.cpp:116-142).  With a window w, the token at position
    p sees the keys at positions p-w+1 .. p."""
    T, NH, HD = q.shape
    rep = NH // k.shape[1]
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk)
    qpos = positions[:, None]
    kpos = positions[None, :]
    banned = kpos > qpos
    if window is not None:
        banned = banned | (kpos <= qpos - window)
    s = s.masked_fill(banned[None], float("-inf"))
    s = s * (1.0 / math.sqrt(HD))
    if round_scores_like_reference:
        # Tensor::scale_inplace rounds through bfloat16 even in the reference's
        # 32-bit build (src/tensor.cpp:95-99); only the golden comparison sets this
        s = s.to(torch.bfloat16).to(s.dtype)
    s = s - s.max(dim=-1, keepdim=True).values
    e = torch.exp(s)
    p = e / e.sum(dim=-1, keepdim=True)
    ctx = torch.einsum("hts,shd->thd", p, vv)
    return ctx.reshape(T, NH * HD)                                   # head-major concat (:255-258)


def attention(x, w, prefix, sz, positions, window=None, **core_options):
    """Q/K/V projections with bias, rotation of q and k, core, output projection
    (src/models/self_attn.cpp:224-258)."""
    T = x.shape[0]
    p = prefix + "self_attn."
    q = linear(x, w[p + "q_proj.weight"], w.get(p + "q_proj.bias")).reshape(T, sz["NH"], sz["HD"])
    k = linear(x, w[p + "k_proj.weight"], w.get(p + "k_proj.bias")).reshape(T, sz["NKV"], sz["HD"])
    v = linear(x, w[p + "v_proj.weight"], w.get(p + "v_proj.bias")).reshape(T, sz["NKV"], sz["HD"])
    q = rope(q, positions, sz["theta"])
    k = rope(k, positions, sz["theta"])
    ctx = attention_core(q, k, v, positions, window, **core_options)
    return linear(ctx, w[p + "o_proj.weight"], w.get(p + "o_proj.bias"))


def swiglu_mlp(x, w, prefix):
    """down( up(x) * silu(gate(x)) ), silu(g) = g / (1 + exp(-g))
    (src/models/mlp.cpp:41-49, src/tensor.cpp:159-174)."""
    p = prefix + "mlp."
    up = linear(x, w[p + "up_proj.weight"], w.get(p + "up_proj.bias"))
    gate = linear(x, w[p + "gate_proj.weight"], w.get(p + "gate_proj.bias"))
    gate = gate * (1.0 / (1.0 + torch.exp(-gate)))
    return linear(up * gate, w[p + "down_proj.weight"], w.get(p + "down_proj.bias"))


def block(x, w, layer, sz, positions, **core_options):
    """h = x + attn(norm_in(x)); y = h + mlp(norm_post(h)) (src/models/block.cpp:23-29)."""
    prefix = f"model.layers.{layer}."
    h = x + attention(rms_norm(x, w[prefix + "input_layernorm.weight"], sz["eps"]), w, prefix, sz,
                      positions, sz["window"][layer], **core_options)
    return h + swiglu_mlp(rms_norm(h, w[prefix + "post_attention_layernorm.weight"], sz["eps"]), w, prefix)


def lm_head(x, w, sz):
    """logits = norm(x) E^T (src/models/gpt_model.cpp:324-328, src/models/embedding.cpp:78-81);
    an untied model multiplies by lm_head.weight instead."""
    xf = rms_norm(x, w["model.norm.weight"], sz["eps"])
    table = w["model.embed_tokens.weight"] if sz["tied"] else w["lm_head.weight"]
    return xf @ table.t()


def forward_logits(cfg: dict, w: dict, ids, run_order=None, **core_options) -> torch.Tensor:
    """Logits [S, V] at every position of one whole sequence
    (src/models/gpt_model.cpp:310-333).  run_order lists the layers to run,
    by default 0..L-1 once each."""
    sz = sizes(cfg)
    positions = torch.arange(len(ids))
    x = embed(w["model.embed_tokens.weight"], ids)
    for layer in (run_order if run_order is not None else range(sz["L"])):
        x = block(x, w, layer, sz, positions, **core_options)
    return lm_head(x, w, sz)


# --------------------------------------------------------------------------
# generation and sampling
# --------------------------------------------------------------------------

def greedy_token(logits_row) -> int:
    """Lowest index among the maxima (std::max_element, src/sampler.cpp:13-20)."""
    return int(np.argmax(logits_row.detach().cpu().numpy()))


def greedy_generate(cfg, w, prompt, new_tokens, eos=None):
    """Whole-sequence recomputation for every new token; the token equal to eos
    is emitted and ends the request (src/models/gpt_model.cpp:279-280, 297-308)."""
    ids = list(prompt)
    out = []
    for _ in range(new_tokens):
        row = forward_logits(cfg, w, ids)[-1]
        t = greedy_token(row)
        out.append(t)
        ids.append(t)
        if eos is not None and eos >= 0 and t == eos:
            break
    return out


def uniform_from_counter(seed: int, request: int, index: int) -> float:
    """The counter-based uniform number of the engine's sampler, restated:
    three rounds of the splitmix64 finaliser over (seed, request, index),
    top 24 bits -> [0, 1).  (The reference draws from one shared mt19937,
    src/sampler.cpp:96-97; ours is keyed per request and token.)"""
    mask = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    z = mix(seed & mask)
    z = mix(z ^ (request & mask))
    z = mix(z ^ (index & mask))
    return (z >> 40) / float(1 << 24)


def sampling_distribution(logits_row, temperature, top_k=0, top_p=1.0):
    """Probabilities after temperature, top-k and top-p, in float64, over the
    whole vocabulary (zero outside the kept set).  p^(1/T) of the softmax, i.e.
    softmax(logits/T) (src/sampler.cpp:50-58); keep the top_k most probable if
    0 < k < V (:60-64), then the shortest prefix of the descending order whose
    normalised mass reaches top_p (:73-94).  Ties go to the lower index."""
    z = logits_row.double().numpy() / max(temperature, 1e-6)
    z = z - z.max()
    p = np.exp(z)
    p = p / p.sum()
    order = np.lexsort((np.arange(len(p)), -p))        # descending p, ascending index
    keep = order
    if 0 < top_k < len(p):
        keep = keep[:top_k]
    if 0.0 < top_p < 1.0:
        total = p[keep].sum()
        cum = np.cumsum(p[keep] / total)
        cutoff = int(np.searchsorted(cum, top_p, side="left")) + 1
        keep = keep[:max(1, min(cutoff, len(keep)))]
    out = np.zeros_like(p)
    out[keep] = p[keep]
    return out / out.sum()


def sample_token(logits_row, temperature, top_k, top_p, u):
    """Inverse CDF over the kept tokens in index order with the uniform u."""
    p = sampling_distribution(logits_row, temperature, top_k, top_p)
    cdf = np.cumsum(p)
    idx = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
    kept = np.nonzero(p)[0]
    return int(kept[np.searchsorted(kept, min(idx, kept[-1]), side="left")])
