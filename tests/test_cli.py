"""The command line's parsing, after test/cli_options_test.cpp of the reference (no GPU)."""
import pytest

from easy_gpt.cpp_b200 import cli
from easy_gpt.cpp_b200.engine.engine import max_new_tokens_from_max_steps
from easy_gpt.cpp_b200.sampling import SamplingParams


def test_defaults_are_the_reference_ones():
    o, err = cli.parse_args(["hello"])
    assert err == "" and o.prompt == "hello"
    assert (o.max_steps, o.temperature, o.top_p, o.top_k, o.seed, o.use_greedy) == (100, 0.8, 0.95, 20, 42, False)


def test_options_parse():
    o, err = cli.parse_args(["-f", "p.txt", "-m", "7", "--temperature", "0.5", "--top-p", "0.9", "--top-k", "0",
                             "--seed", "3", "--greedy", "--model", "m", "--dtype", "float32", "--token-ids",
                             "--page-size", "8", "--cache-tokens", "4096", "--max-active", "2", "--chunk-size", "64"])
    assert err == ""
    assert (o.prompt_file, o.max_steps, o.temperature, o.top_p, o.top_k, o.seed) == ("p.txt", 7, 0.5, 0.9, 0, 3)
    assert o.use_greedy and o.model == "m" and o.dtype == "float32" and o.token_ids
    assert (o.page_size, o.cache_tokens, o.max_active, o.chunk_size) == (8, 4096, 2, 64)
    assert cli.parse_args(["--help"])[0].show_help and cli.parse_args(["-h", "--bogus"])[0].show_help


@pytest.mark.parametrize("argv, text", [
    (["-f"], "Missing path after -f"),
    (["-f", "a", "--prompt-file", "b"], "Prompt file option specified multiple times"),
    (["--max-steps"], "Missing number after --max-steps"),
    (["-m", "x"], "Invalid number for max steps: x"),
    (["-m", "0"], "Max steps must be greater than 0"),
    (["--temperature", "0"], "Temperature must be greater than 0"),
    (["--temperature", "hot"], "Invalid number for temperature: hot"),
    (["--top-p", "1.5"], "Top-p must be in (0, 1]"),
    (["--top-p", "0"], "Top-p must be in (0, 1]"),
    (["--top-k", "-1"], "Top-k must be >= 0"),
    (["--seed", "-4"], "Seed must be >= 0"),
    (["--bogus"], "Unknown option: --bogus"),
    (["a", "b"], "Multiple prompts provided; use a single prompt or --prompt-file"),
    (["--serve"], "--serve: the serving mode is not provided by this engine"),
    (["--dtype", "fp8"], "dtype must be bfloat16 or float32"),
])
def test_errors_name_the_problem(argv, text):
    o, err = cli.parse_args(argv)
    assert o is None and err == text


def test_prompt_file_and_output_path(tmp_path):
    f = tmp_path / "prompts.txt"
    f.write_text("  first prompt  \n\n\t\nsecond\n")
    assert cli.read_prompts_file(str(f)) == ["first prompt", "second"]
    assert cli.output_path_for(str(f)) == tmp_path / "prompts_output.txt"
    with pytest.raises(OSError, match="Failed to open prompt file"):
        cli.read_prompts_file(str(tmp_path / "none.txt"))


def test_helpers():
    assert cli.parse_token_ids("5, 17 3") == [5, 17, 3]
    assert cli.apply_chat_template("hi").endswith("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n")
    assert cli.escape_single_line("a\nb") == "a\\nb"
    # --max-steps caps prompt + generated, at least one token (src/continuous_batch_server.cpp:313)
    assert max_new_tokens_from_max_steps(100, 10) == 91 and max_new_tokens_from_max_steps(5, 50) == 1


def test_main_without_prompts_fails(capsys):
    assert cli.main([]) == 1
    assert "No prompts provided" in capsys.readouterr().err
    assert cli.main(["--help"]) == 0


def test_sampling_params_are_checked():
    with pytest.raises(ValueError, match="Temperature"):
        SamplingParams(temperature=0.0)
    with pytest.raises(ValueError, match="Top-p"):
        SamplingParams(top_p=0.0)
    assert SamplingParams(temperature=0.0, greedy=True).is_greedy


def test_log_levels(capsys, monkeypatch):
    """EASYGPT_LOG picks the level; lines below it are dropped, an unknown name falls back to warn."""
    import importlib

    from easy_gpt.cpp_b200 import log

    monkeypatch.setenv("EASYGPT_LOG", "debug")
    importlib.reload(log)
    log.debug("shown")
    log.trace("hidden")
    err = capsys.readouterr().err
    assert "[debug] shown" in err and "hidden" not in err
    monkeypatch.setenv("EASYGPT_LOG", "loud")
    importlib.reload(log)
    assert "is no level" in capsys.readouterr().err and log.level == log.LEVELS["warn"]
    log.info("hidden")
    log.warn("shown")
    err = capsys.readouterr().err
    assert "[warn] shown" in err and "hidden" not in err
    with log.nvtx_range("nothing"):                      # a no-op unless EASY_GPT_NVTX is set
        pass
    monkeypatch.delenv("EASYGPT_LOG")
    importlib.reload(log)
