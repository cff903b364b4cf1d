"""Text <-> token ids for the command line: a byte-level BPE read from ``tokenizer.json`` (and, for
special tokens, ``tokenizer_config.json``), with the reference's rules:

* the text is cut at special tokens (``added_tokens_decoder`` entries marked ``special``): the earliest
  match wins, the longest at the same place (src/tokenizer.cpp:58-75, 270-281);
* what lies between is split at whitespace; every word but the first gets one leading space, runs of
  whitespace and line breaks collapse (src/bpe.cpp:32-62) — simpler than the pre-tokeniser the model was
  trained with, and kept that way on purpose; a word that touches a special token on both sides
  without whitespace gets no space (src/tokenizer.cpp:85-92);
* a word's bytes are mapped to the printable stand-ins of the GPT-2 table (src/bpe.cpp:163-195) and
  merged pair by pair, lowest merge rank first (src/bpe.cpp:119-161);
* tokens that are not in the vocabulary are dropped; BOS is put in front if ``bos_token_id >= 0``
  (src/tokenizer.cpp:129-142).

The engine itself works on token ids; only ``bin/easy_llm`` with a text prompt needs this.  The rules
run in C++ (``csrc/host/bpe_tokenizer.hpp``); this module reads the JSON files and is its face in Python.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import host


def _blob(strings: Sequence[str]):
    """UTF-8 bytes of the strings in a row, and the n + 1 offsets that cut them apart."""
    encoded = [s.encode("utf-8") for s in strings]
    offsets = np.zeros(len(encoded) + 1, dtype=np.int64)
    if encoded:
        offsets[1:] = np.cumsum([len(e) for e in encoded])
    return b"".join(encoded), offsets


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]], specials: Optional[Dict[str, int]] = None,
                 bos_token_id: int = -1):
        self.token_to_id = dict(vocab)
        self.specials = []
        for token, idx in (specials or {}).items():
            self.specials.append(token)
            if token not in self.token_to_id and idx not in self.token_to_id.values():
                self.token_to_id[token] = idx
        self.specials.sort(key=lambda t: (-len(t), t))                       # longest first
        self.id_to_token = {i: t for t, i in self.token_to_id.items()}
        self.bos_token_id = bos_token_id
        self._lib = host.library()
        self._core = self._lib.egh_bpe_create()
        tokens = list(self.token_to_id)
        blob, offsets = _blob(tokens)
        ids = np.asarray([self.token_to_id[t] for t in tokens], dtype=np.int32)
        self._lib.egh_bpe_add_tokens(self._core, blob, offsets.ctypes.data, ids.ctypes.data, len(tokens))
        left, left_offsets = _blob([m[0] for m in merges])
        right, right_offsets = _blob([m[1] for m in merges])
        self._lib.egh_bpe_add_merges(self._core, left, left_offsets.ctypes.data, right, right_offsets.ctypes.data, len(merges))
        blob, offsets = _blob(self.specials)
        self._lib.egh_bpe_add_specials(self._core, blob, offsets.ctypes.data, len(self.specials))
        self._lib.egh_bpe_set_bos(self._core, int(bos_token_id))

    def __del__(self):
        core = getattr(self, "_core", None)
        if core:
            self._core = None
            self._lib.egh_bpe_destroy(core)

    @staticmethod
    def from_dir(model_dir, bos_token_id: int = -1) -> "Tokenizer":
        model_dir = Path(model_dir)
        path = model_dir / "tokenizer.json"
        if not path.is_file():
            raise FileNotFoundError(f"no tokenizer.json in {model_dir}")
        data = json.loads(path.read_text(encoding="utf-8"))
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else (m[0], m[1]) for m in data["model"]["merges"]]
        specials = {}
        cfg = model_dir / "tokenizer_config.json"
        if cfg.is_file():
            for idx, info in json.loads(cfg.read_text(encoding="utf-8")).get("added_tokens_decoder", {}).items():
                if info.get("special") and info.get("content"):
                    specials[info["content"]] = int(idx)
        return Tokenizer(data["model"]["vocab"], merges, specials, bos_token_id)

    def _twice(self, call, first_capacity: int, dtype):
        """Runs ``call(buffer, capacity)``, which returns how much there is; a second time if it did not fit."""
        cap = max(16, first_capacity)
        for _ in range(2):
            buf = np.empty(cap, dtype=dtype)
            n = int(call(buf.ctypes.data, cap))
            if n <= cap:
                return buf[:n]
            cap = n
        raise RuntimeError("the tokenizer's answer changed between two calls")

    # -- encoding -------------------------------------------------------------
    def tokenize(self, text: str) -> List[str]:
        raw = text.encode("utf-8")
        out = self._twice(lambda buf, cap: self._lib.egh_bpe_tokenize(self._core, raw, len(raw), buf, cap), 4 * len(raw) + 64, np.uint8)
        joined = out.tobytes()
        return [t.decode("utf-8") for t in joined.split(b"\0")[:-1]] if joined else []

    def encode(self, text: str) -> List[int]:
        raw = text.encode("utf-8")
        out = self._twice(lambda buf, cap: self._lib.egh_bpe_encode(self._core, raw, len(raw), buf, cap), len(raw) + 8, np.int32)
        return out.tolist()

    # -- decoding ---------------------------------------------------------------
    def decode(self, ids) -> str:
        arr = np.asarray([int(i) for i in ids], dtype=np.int32)
        out = self._twice(lambda buf, cap: self._lib.egh_bpe_decode(self._core, arr.ctypes.data, len(arr), buf, cap),
                          8 * len(arr) + 64, np.uint8)
        return out.tobytes().decode("utf-8", errors="replace")
