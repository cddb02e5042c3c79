"""Command-line strictness: a bad flag fails before the model is touched (no GPU).
Cf. tests/cli_tests.zig:57-86 of the reference."""
import pytest

from hk_b200 import cli


def parse(*args):
    return cli.parse_run_args(list(args))


def test_options_have_the_references_names_and_defaults():
    g = parse("model_dir", "1,2,3")
    assert g["prompt_ids"] == [1, 2, 3]
    assert (g["max_tokens"], g["temperature"], g["top_k"], g["top_p"], g["min_p"], g["repeat_penalty"], g["seed"]) == \
        (128, 0.8, 40, 0.95, 0.05, 1.0, 0)
    g = parse("m", "-p", "5 6", "-n", "7", "--temp", "0", "--top-k", "3", "--top-p", "0.5", "--min-p", "0.1",
              "--repeat-penalty", "1.2", "--seed", "9", "--threads", "4", "-ngl", "99", "--backend", "cuda",
              "--dtype", "float32")
    assert g["prompt_ids"] == [5, 6] and g["max_tokens"] == 7 and g["temperature"] == 0 and g["dtype"] == "float32"
    assert (g["top_k"], g["top_p"], g["min_p"], g["repeat_penalty"], g["seed"]) == (3, 0.5, 0.1, 1.2, 9)
    assert parse("m", "--rep-pen", "2", "--max-tokens", "1", "4")["repeat_penalty"] == 2


@pytest.mark.parametrize("args,needle", [
    (["m", "1", "--bogus"], "unknown argument '--bogus'"),
    (["m", "1", "--temp"], "needs a value"),
    (["m", "1", "--temp", "warm"], "--temp"),
    (["m", "1", "--temp", "-1"], "--temp"),
    (["m", "1", "--top-p", "1.5"], "--top-p"),
    (["m", "1", "-n", "0"], "-n"),
    (["m", "1", "--top-k", "x"], "--top-k"),
    (["m", "1", "2"], "more than one prompt"),
    (["m", "-p", "1", "-p", "2"], "more than one prompt"),
    (["m"], "no prompt"),
    ([], "no model"),
    (["m", "one two"], "not a list of token ids"),
    (["m", "1", "--backend", "vulkan"], "vulkan"),
    (["m", "1", "--backend", "metal"], "--backend"),
    (["m", "1", "-ngl", "0"], "CPU"),
    (["m", "1", "--dtype", "int4"], "--dtype"),
])
def test_bad_usage_is_refused_before_any_model_is_opened(args, needle):
    with pytest.raises(cli.BadUsage) as e:
        cli.parse_run_args(args)
    assert needle in str(e.value)


def test_main_reports_usage_errors_with_exit_code_2(capsys):
    assert cli.main(["run", "/nonexistent", "1", "--wat"]) == 2
    err = capsys.readouterr().err
    assert "unknown argument '--wat'" in err and "Usage: hk run" in err
    assert cli.main(["fly"]) == 2
