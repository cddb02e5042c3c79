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


def test_prompt_of_a_given_length_and_page_size():
    g = parse("m", "--prompt-len", "12", "--page-tokens", "16", "--seed", "3")
    assert g["prompt_ids"] is None and g["prompt_len"] == 12 and g["page_tokens"] == 16
    with pytest.raises(cli.BadUsage) as e:
        parse("m", "1,2", "--prompt-len", "4")
    assert "both a prompt" in str(e.value)
    with pytest.raises(cli.BadUsage):
        parse("m", "--prompt-len", "0")


def test_random_command_writes_a_model_folder_that_loads(tmp_path, capsys):
    import json
    from hk_b200.config import load_config
    from hk_b200.weights.safetensors_io import SafetensorsFile

    def load_file(path):
        f = SafetensorsFile(path)
        return {n: f.tensor(n).clone() for n in f.names()}
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=48, num_hidden_layers=2, intermediate_size=80,
               num_attention_heads=3, num_key_value_heads=1, head_dim=16, vocab_size=70, rms_norm_eps=1e-6,
               rope_theta=10000.0, tie_word_embeddings=True, max_position_embeddings=64)
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    out = tmp_path / "model"
    assert cli.main(["random", str(tmp_path / "c.json"), str(out), "--seed", "5", "--dtype", "float32"]) == 0
    assert load_config(str(out)).hidden_size == 48
    a = load_file(str(out / "model.safetensors"))
    assert "model.layers.1.mlp.down_proj.weight" in a and "lm_head.weight" not in a
    # the same seed gives the same weights; an existing model is not overwritten
    assert cli.main(["random", str(out), str(tmp_path / "again"), "--seed", "5", "--dtype", "float32"]) == 0
    b = load_file(str(tmp_path / "again" / "model.safetensors"))
    assert all((a[k] == b[k]).all() for k in a)
    assert cli.main(["random", str(out), str(out)]) == 1
    assert cli.main(["random", str(out)]) == 2
    assert cli.main(["random", str(out), str(tmp_path / "x"), "--wat"]) == 2
