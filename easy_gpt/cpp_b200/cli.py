"""The ``easy_llm`` command line, in the reference's manner (src/cli_options.cpp,
src/main.cpp): the same option names, meanings, defaults, checks and error
texts where the reference has them, plus the options this engine adds (a model
folder instead of a fixed path, token-id prompts, cache and batch sizes).
``--serve`` and its options are not provided: no server is built here.  Text prompts go through
``tokenizer.py`` (the reference's whitespace-split byte-level BPE) and the fixed Qwen chat template.
"""
from __future__ import annotations

import json
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Tuple

USAGE = """Usage: easy_llm [--model <dir>] [--prompt-file <path>] [--max-steps <n>]
                [--temperature <float>] [--top-p <float>] [--top-k <int>] [--seed <int>] [--greedy]
                [--token-ids] [--dtype <bfloat16|float32>] ["prompt"]
  -f, --prompt-file <path>  Read prompts from file (one per line, ignore empty lines)
  -m, --max-steps <n>        Maximum generation steps per request (default: 100)
      --temperature <float> Sampling temperature (default: 0.8)
      --top-p <float>        Nucleus sampling cutoff in (0,1] (default: 0.95)
      --top-k <int>          Top-K sampling cutoff, 0 disables (default: 20)
      --seed <int>           RNG seed for sampling (default: 42)
      --greedy               Use greedy decoding (override sampling)
      --model <dir>          Folder with config.json and model.safetensors (default: data/model)
      --dtype <name>         bfloat16 (default) or float32 (true 32-bit everywhere)
      --token-ids            Prompts are lists of token ids ("5 17 3" or "5,17,3"); outputs are ids too
      --random-weights <seed> Write random weights for --config into --model first
      --config <path>        config.json to use with --random-weights
      --page-size <n>        Tokens per cache page (default: 16)
      --cache-tokens <n>     Tokens the cache pool holds (default: max-active x 4096)
      --max-active <n>       Max concurrent requests (default: 16)
      --prefill-batch <n>    Max requests admitted per step (default: 4)
      --max-batch-tokens <n> Token budget of one step (default: 2048)
      --chunk-size <n>       Longest portion of a prompt in one step (default: 512)
      --no-chat-template     Do not wrap text prompts in the chat template
  -h, --help                Show this help message
Examples:
  easy_llm --model data/model --max-steps 128 "Hello"
  easy_llm --model m --token-ids --greedy "5 17 3"
  easy_llm --model m -f prompts.txt
"""


@dataclass
class CliOptions:
    prompt_file: str = ""
    prompt: str = ""
    max_steps: int = 100
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 20
    seed: int = 42
    use_greedy: bool = False
    show_help: bool = False
    model: str = "data/model"
    dtype: str = "bfloat16"
    token_ids: bool = False
    random_weights: Optional[int] = None
    config: str = ""
    page_size: int = 16
    cache_tokens: Optional[int] = None
    max_active: int = 16
    prefill_batch: int = 4
    max_batch_tokens: int = 2048
    chunk_size: int = 512
    chat_template: bool = True


def _number(kind, text):
    # std::stoi / std::stof accept a numeric prefix; a plain conversion is close enough here
    return kind(text)


def parse_args(argv: List[str]) -> Tuple[Optional[CliOptions], str]:
    """Returns (options, "") or (None, error text).  Error texts of the options the
    reference has are its own (src/cli_options.cpp:86-286)."""
    o = CliOptions()
    i = 0

    def value(after_what, arg):
        nonlocal i
        if i + 1 >= len(argv):
            return None, f"Missing {after_what} after {arg}"
        i += 1
        return argv[i], ""

    int_options = {
        # flag: (field, label in the error, check, complaint)
        "--max-steps": ("max_steps", "max steps", lambda v: v > 0, "Max steps must be greater than 0"),
        "-m": ("max_steps", "max steps", lambda v: v > 0, "Max steps must be greater than 0"),
        "--top-k": ("top_k", "top-k", lambda v: v >= 0, "Top-k must be >= 0"),
        "--seed": ("seed", "seed", lambda v: v >= 0, "Seed must be >= 0"),
        "--random-weights": ("random_weights", "random weights seed", lambda v: v >= 0, "random-weights seed must be >= 0"),
        "--page-size": ("page_size", "page size", lambda v: v > 0, "page-size must be greater than 0"),
        "--cache-tokens": ("cache_tokens", "cache tokens", lambda v: v > 0, "cache-tokens must be greater than 0"),
        "--max-active": ("max_active", "max active", lambda v: v > 0, "max-active must be greater than 0"),
        "--prefill-batch": ("prefill_batch", "prefill batch", lambda v: v > 0, "prefill-batch must be greater than 0"),
        "--max-batch-tokens": ("max_batch_tokens", "max batch tokens", lambda v: v > 0, "max-batch-tokens must be greater than 0"),
        "--chunk-size": ("chunk_size", "chunk size", lambda v: v > 0, "chunk-size must be greater than 0"),
    }
    float_options = {
        "--temperature": ("temperature", "temperature", lambda v: v > 0.0, "Temperature must be greater than 0"),
        "--top-p": ("top_p", "top-p", lambda v: 0.0 < v <= 1.0, "Top-p must be in (0, 1]"),
    }
    while i < len(argv):
        arg = argv[i]
        if arg in ("-h", "--help"):
            o.show_help = True
            return o, ""
        if arg in ("-f", "--prompt-file"):
            v, err = value("path", arg)
            if err:
                return None, err
            if o.prompt_file:
                return None, "Prompt file option specified multiple times"
            o.prompt_file = v
        elif arg in int_options or arg in float_options:
            fld, label, ok, complaint = (int_options.get(arg) or float_options[arg])
            v, err = value("number", arg)
            if err:
                return None, err
            try:
                num = _number(int if arg in int_options else float, v)
            except ValueError:
                return None, f"Invalid number for {label}: {v}"
            if not ok(num):
                return None, complaint
            setattr(o, fld, num)
        elif arg == "--greedy":
            o.use_greedy = True
        elif arg == "--token-ids":
            o.token_ids = True
        elif arg == "--no-chat-template":
            o.chat_template = False
        elif arg in ("--model", "--config", "--dtype"):
            v, err = value("value", arg)
            if err:
                return None, err
            if arg == "--dtype" and v not in ("bfloat16", "float32"):
                return None, "dtype must be bfloat16 or float32"
            setattr(o, arg[2:], v)
        elif arg.startswith("--serve"):
            return None, f"{arg}: the serving mode is not provided by this engine"
        elif arg.startswith("-") and len(arg) > 1 and not arg[1:].replace(",", "").replace(" ", "").isdigit():
            return None, f"Unknown option: {arg}"
        else:
            if o.prompt:
                return None, "Multiple prompts provided; use a single prompt or --prompt-file"
            o.prompt = arg
        i += 1
    return o, ""


def read_prompts_file(path: str) -> List[str]:
    """One prompt per non-empty trimmed line (src/cli_options.cpp:66-84)."""
    try:
        text = Path(path).read_text()
    except OSError:
        raise OSError(f"Failed to open prompt file: {path}") from None
    return [line.strip() for line in text.splitlines() if line.strip()]


def output_path_for(prompt_file: str) -> Path:
    """<stem>_output<ext> beside the prompt file (src/main.cpp:113-120)."""
    p = Path(prompt_file)
    return p.parent / f"{p.stem}_output{p.suffix}"


CHAT_TEMPLATE = ("<|im_start|>system\nYou are Qwen, created by Alibaba Cloud. You are a helpful assistant.<|im_end|>\n"
                 "<|im_start|>user\n{user_query}<|im_end|>\n<|im_start|>assistant\n")


def apply_chat_template(user_query: str) -> str:
    """The fixed Qwen template (src/cli_options.cpp:49-64)."""
    return CHAT_TEMPLATE.replace("{user_query}", user_query)


def parse_token_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def escape_single_line(text: str) -> str:
    return text.replace("\\", "\\\\").replace("\n", "\\n").replace("\r", "\\r")


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    opts, err = parse_args(argv)
    if opts is None:
        print(err, file=sys.stderr)
        print(USAGE, file=sys.stderr, end="")
        return 1
    if opts.show_help:
        print(USAGE, end="")
        return 0
    prompts: List[str] = []
    if opts.prompt_file:
        try:
            prompts += read_prompts_file(opts.prompt_file)
        except OSError as e:
            print(e, file=sys.stderr)
            return 1
    if opts.prompt:
        prompts.append(opts.prompt)
    if not prompts:
        print("No prompts provided", file=sys.stderr)
        print(USAGE, file=sys.stderr, end="")
        return 1

    from .engine.engine import GptEngine

    if opts.random_weights is not None:
        from .weights.random_init import write_random_model

        if not opts.config:
            print("--random-weights needs --config <config.json>", file=sys.stderr)
            return 1
        write_random_model(opts.model, json.loads(Path(opts.config).read_text()), opts.random_weights)

    tokenizer = None
    if opts.token_ids:
        try:
            token_prompts = [parse_token_ids(p) for p in prompts]
        except ValueError:
            print("--token-ids prompts must be lists of integers", file=sys.stderr)
            return 1
    else:
        from .tokenizer import Tokenizer

        try:
            bos = json.loads((Path(opts.model) / "config.json").read_text()).get("bos_token_id")
            tokenizer = Tokenizer.from_dir(opts.model, bos_token_id=-1 if bos is None else int(bos))
        except FileNotFoundError as e:
            print(f"{e}; text prompts need tokenizer.json (or pass --token-ids)", file=sys.stderr)
            return 1
        token_prompts = [tokenizer.encode(apply_chat_template(p) if opts.chat_template else p) for p in prompts]

    engine = GptEngine(opts.model, dtype=opts.dtype, page_size=opts.page_size, cache_tokens=opts.cache_tokens,
                       max_active=opts.max_active, prefill_batch=opts.prefill_batch,
                       max_batch_tokens=opts.max_batch_tokens, chunk_size=opts.chunk_size)
    outputs = engine.generate(token_prompts, max_steps=opts.max_steps, temperature=opts.temperature, top_p=opts.top_p,
                              top_k=opts.top_k, seed=opts.seed, greedy=opts.use_greedy)
    lines = [" ".join(map(str, out)) if tokenizer is None else escape_single_line(tokenizer.decode(out)) for out in outputs]
    if opts.prompt_file:
        path = output_path_for(opts.prompt_file)
        path.write_text("".join(line + "\n" for line in lines))
    for line in lines:
        print(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
