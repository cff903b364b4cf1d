"""The handmade vocabulary and the texts of the tokenizer's golden comparison with the
reference's own Tokenizer (tests/golden/make_golden.py runs it; tests/test_tokenizer.py holds
the package's tokenizer to what it produced)."""
import json
from pathlib import Path

SPACE = "Ġ"                                                 # the stand-in of the space byte
VOCAB = {t: i for i, t in enumerate(["h", "e", "l", "o", "w", "r", "d", SPACE, "he", "ll", "hell", "hello",
                                     SPACE + "w", "or", SPACE + "wor", "ld", "!", "Ã", "©", "Â", "ł"])}
MERGES = ["h e", "l l", "he ll", "hell o", SPACE + " w", "o r", SPACE + "w or", "l d"]
ADDED = {"100": {"content": "<|im_start|>", "special": True}, "101": {"content": "<|im_end|>", "special": True},
         "102": {"content": "<|im|>", "special": True}, "103": {"content": "<tool>", "special": False}}

TEXTS = [
    "hello world", "hello   \n\t world", "  hello", "hello xyz", "hello\vworld\fhello\rworld",
    "é", "hello world", "hello　world", "hello\u0085world", "hello\x1cworld", "hello  \tworld",
    "<|im_start|>hello<|im_end|>", "hello <|im_end|> world", "hello<|im|>world", "hello<|im|> world",
    "hello<|im|> world", "hello <|im|>world", "<tool>", "<|im_start|><|im|>hello world!<|im_end|>\n<|im_start|>world",
    "", "   ",
    "<|im_start|>system\nYou are Qwen, created by Alibaba Cloud. You are a helpful assistant.<|im_end|>\n"
    "<|im_start|>user\nhello world<|im_end|>\n<|im_start|>assistant\n",
]


def write_files(folder) -> None:
    folder = Path(folder)
    (folder / "tokenizer.json").write_text(json.dumps({"model": {"vocab": VOCAB, "merges": MERGES}}))
    (folder / "tokenizer_config.json").write_text(json.dumps({"added_tokens_decoder": ADDED}))
