"""The command line's tokenizer against the reference's rules, on a handmade vocabulary (no GPU)."""
import json

from easy_gpt.cpp_b200.tokenizer import Tokenizer


def make(tmp_path):
    space = "Ġ"                                                  # the stand-in of the space byte
    vocab = {t: i for i, t in enumerate(["h", "e", "l", "o", "w", "r", "d", space, "he", "ll", "hell", "hello",
                                         space + "w", "or", space + "wor", "ld", "!", "Ã", "©"])}
    merges = ["h e", "l l", "he ll", "hell o", space + " w", "o r", space + "w or", "l d"]
    (tmp_path / "tokenizer.json").write_text(json.dumps({"model": {"vocab": vocab, "merges": merges}}))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"added_tokens_decoder": {
        "100": {"content": "<|im_start|>", "special": True}, "101": {"content": "<|im_end|>", "special": True},
        "102": {"content": "<|im|>", "special": True}, "103": {"content": "<tool>", "special": False}}}))
    return Tokenizer.from_dir(tmp_path), space


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


def test_every_kind_of_white_space_splits_words(tmp_path):
    tok, sp = make(tmp_path)
    for gap in ("\u00a0", "\u2003", "\u3000", "\x85", "\x1c", " \u2028\t"):
        assert tok.tokenize("hello" + gap + "world") == ["hello", sp + "wor", "ld"], repr(gap)
    # white space beside a special token decides whether the next word gets its space
    assert tok.tokenize("hello<|im|>\u00a0world") == ["hello", "<|im|>", sp + "wor", "ld"]
    assert tok.tokenize("") == [] and tok.encode("   ") == [] and tok.decode([]) == ""


def test_missing_file(tmp_path):
    import pytest

    with pytest.raises(FileNotFoundError, match="tokenizer.json"):
        Tokenizer.from_dir(tmp_path / "nowhere")
