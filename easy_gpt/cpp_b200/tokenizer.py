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

The engine itself works on token ids; only ``bin/easy_llm`` with a text prompt needs this.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Tuple


def _byte_table() -> Dict[int, str]:
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table = {b: chr(b) for b in keep}
    extra = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + extra)
            extra += 1
    return table


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
        self.rank = {pair: r for r, pair in enumerate(merges)}
        self.bos_token_id = bos_token_id
        self.byte_to_char = _byte_table()
        self.char_to_byte = {c: b for b, c in self.byte_to_char.items()}
        self._cache: Dict[str, List[str]] = {}

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

    # -- encoding -------------------------------------------------------------
    def _merge_word(self, word: str) -> List[str]:
        if word in self._cache:
            return self._cache[word]
        parts = list(word)
        while len(parts) > 1:
            best, where = None, -1
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, where = r, i
            if where < 0:
                break
            parts[where:where + 2] = [parts[where] + parts[where + 1]]
        self._cache[word] = parts
        return parts

    def _plain(self, text: str, first_word: bool, out: List[str]) -> bool:
        """Tokens of a stretch without special tokens; returns whether it held a word."""
        saw = False
        for word in text.split():
            raw = word if first_word else " " + word
            first_word = False
            saw = True
            mapped = "".join(self.byte_to_char[b] for b in raw.encode("utf-8"))
            out.extend(self._merge_word(mapped))
        return saw

    def tokenize(self, text: str) -> List[str]:
        out: List[str] = []
        first_word, no_space_next, pos = True, False, 0
        while pos < len(text):
            hit, hit_at = None, len(text)
            for s in self.specials:                                             # longest first; earliest wins
                at = text.find(s, pos)
                if at != -1 and at < hit_at:
                    hit, hit_at = s, at
            if hit_at > pos:
                if self._plain(text[pos:hit_at], first_word or no_space_next, out):
                    first_word = False
            if hit is None:
                break
            out.append(hit)
            end = hit_at + len(hit)
            no_space_next = (hit_at > 0 and not text[hit_at - 1].isspace()) and (end < len(text) and not text[end].isspace())
            pos = end
        return out

    def encode(self, text: str) -> List[int]:
        ids = [self.bos_token_id] if self.bos_token_id >= 0 else []
        ids += [self.token_to_id[t] for t in self.tokenize(text) if t in self.token_to_id]
        return ids

    # -- decoding ---------------------------------------------------------------
    def decode(self, ids) -> str:
        text = "".join(self.id_to_token.get(int(i), "") for i in ids)
        raw = bytearray()
        for ch in text:
            if ch in self.char_to_byte:
                raw.append(self.char_to_byte[ch])
            else:
                raw += ch.encode("utf-8")
        return raw.decode("utf-8", errors="replace")
