"""The command line's tokenizer against the reference's rules, on a handmade vocabulary (no GPU)."""
import json
from pathlib import Path

from easy_gpt.cpp_b200.tokenizer import Tokenizer
from golden import golden_tokenizer


def make(tmp_path):
    golden_tokenizer.write_files(tmp_path)
    return Tokenizer.from_dir(tmp_path), golden_tokenizer.SPACE


def test_same_tokens_and_ids_as_the_references_own_tokenizer(tmp_path):
    """tests/golden/ref_tokens.json is what the reference's Tokenizer (src/tokenizer.cpp, src/bpe.cpp), compiled
    on the CPU by tests/golden/make_golden.py, made of these texts with this vocabulary."""
    tok, _ = make(tmp_path)
    golden = json.loads((Path(__file__).parent / "golden" / "ref_tokens.json").read_text())
    assert len(golden) == len(golden_tokenizer.TEXTS)
    for text, want in zip(golden_tokenizer.TEXTS, golden):
        assert tok.tokenize(text) == want["tokens"], repr(text)
        assert tok.encode(text) == want["ids"], repr(text)


def test_words_merges_and_spaces(tmp_path):
    tok, sp = make(tmp_path)
    assert tok.tokenize("hello world") == ["hello", sp + "wor", "ld"]          # lowest rank first, leading space on later words
    assert tok.tokenize("hello   \n\t world") == ["hello", sp + "wor", "ld"]   # runs of whitespace collapse
    assert tok.tokenize("  hello") == ["hello"]                                # the first word gets no space
    assert tok.encode("hello world") == [11, 14, 15]
    assert tok.decode([11, 14, 15]) == "hello world"
    assert tok.encode("hello xyz") == [11, 7]                                   # unknown pieces are dropped: only the space of " xyz" is known
    assert Tokenizer.from_dir(tmp_path, bos_token_id=9).encode("hello")[0] == 9


def test_special_tokens(tmp_path):
    tok, sp = make(tmp_path)
    assert tok.tokenize("<|im_start|>hello<|im_end|>") == ["<|im_start|>", "hello", "<|im_end|>"]
    # a word between text and a special token keeps its space unless it touches specials on both sides without whitespace
    assert tok.tokenize("hello <|im_end|> world") == ["hello", "<|im_end|>", sp + "wor", "ld"]
    assert tok.tokenize("hello<|im|>world") == ["hello", "<|im|>", "w", "or", "ld"]
    assert tok.encode("<|im_start|>hello") == [100, 11]
    assert tok.decode([100, 11, 101]) == "<|im_start|>hello<|im_end|>"
    assert tok.tokenize("<tool>") != ["<tool>"]                                # not special: goes through the merges


def test_bytes_round_trip(tmp_path):
    tok, _ = make(tmp_path)
    ids = tok.encode("é")                                                  # two UTF-8 bytes, each its own token
    assert ids == [17, 18] and tok.decode(ids) == "é"


def test_only_ascii_white_space_splits_words(tmp_path):
    """The reference splits on the classic locale's white space (src/bpe.cpp:32-62): space, tab, newline,
    vertical tab, form feed, carriage return.  Other Unicode spaces are bytes of the word they stand in."""
    tok, sp = make(tmp_path)
    for gap in (" ", "\t", "\n", "\v", "\f", "\r", " \r\n\t "):
        assert tok.tokenize("hello" + gap + "world") == ["hello", sp + "wor", "ld"], repr(gap)
    for gap in ("\u00a0", "\u2003", "\u3000", "\x85", "\x1c"):
        tokens = tok.tokenize("hello" + gap + "world")
        assert tokens[0] == "hello" and tokens[-3:] == ["w", "or", "ld"] and len(tokens) > 4, repr(gap)
    # white space beside a special token decides whether the next word gets its space
    assert tok.tokenize("hello<|im|> world") == ["hello", "<|im|>", sp + "wor", "ld"]
    assert tok.tokenize("") == [] and tok.encode("   ") == [] and tok.decode([]) == ""


def test_missing_file(tmp_path):
    import pytest

    with pytest.raises(FileNotFoundError, match="tokenizer.json"):
        Tokenizer.from_dir(tmp_path / "nowhere")
