"""The command line keeps the names, meanings and defaults of the reference's runner
(src/cpu_runner.cpp:9-26, 51-64; src/config.h:97-100, 106-108).  No GPU needed."""
import pytest

from vllm_cpp_b200.cli import build_parser, parse_token_ids


def test_the_reference_runners_options_and_defaults():
    a = build_parser().parse_args(["MODEL"])
    assert a.model_path == "MODEL" and a.prompt is None and a.tokens == []
    assert (a.max_new, a.temp, a.top_p, a.max_batch, a.max_tokens) == (2048, 0.7, 0.8, 4, 8192)
    assert a.repeat_penalty == 1.1 and a.paged is False and a.debug is False
    a = build_parser().parse_args(["MODEL", "--tokens", "1,2,3", "--tokens", "4", "--max-new", "5", "--temp", "0", "--top-p", "1",
                                   "--paged", "--max-batch", "2", "--max-tokens", "256", "--debug"])
    assert a.tokens == ["1,2,3", "4"] and (a.max_new, a.temp, a.top_p, a.max_batch, a.max_tokens) == (5, 0.0, 1.0, 2, 256)
    assert a.paged and a.debug


def test_the_engines_own_options():
    a = build_parser().parse_args(["MODEL", "--dtype", "float32", "--page-size", "8", "--max-step-tokens", "64", "--seed", "3",
                                   "--stop-id", "7", "--stop-id", "9", "--ignore-eos", "--repeat-penalty", "1.0"])
    assert (a.dtype, a.page_size, a.max_step_tokens, a.seed, a.stop_id, a.ignore_eos, a.repeat_penalty) == \
        ("float32", 8, 64, 3, [7, 9], True, 1.0)
    with pytest.raises(SystemExit):
        build_parser().parse_args(["MODEL", "--dtype", "float16"])


def test_token_ids_from_text():
    assert parse_token_ids("5,17, 3") == [5, 17, 3]
    assert parse_token_ids("42") == [42]
