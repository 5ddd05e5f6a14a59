"""The command line's options: names, short forms and defaults are the reference's
(alpacca/cli.py:662-671, alpacca/sample.py:12-19), and a flag sets the sampler field it names."""
import argparse

import pytest

from alpacca_b200 import cli
from alpacca_b200.sampling import SamplerParams


def parse(words):
    ap = argparse.ArgumentParser()
    cli.add_run_flags(ap)
    return ap.parse_args(words)


def test_flags_not_given_leave_the_sampler_defaults():
    args = parse([])
    assert args.ctx == 0 and args.n_predict == -1 and args.dtype == "bfloat16"
    assert cli.sampler_params_from(args) == SamplerParams()
    assert SamplerParams() == SamplerParams(0.8, 40, 0.95, 1.1, 64, -1)


def test_each_flag_sets_its_field():
    args = parse(["--temp", "0", "--top-k", "7", "--top-p", "0.5", "--repeat-penalty", "1.0", "-s", "3",
                  "-c", "512", "-n", "9"])
    p = cli.sampler_params_from(args)
    assert (p.temperature, p.top_k, p.top_p, p.repeat_penalty, p.seed) == (0.0, 7, 0.5, 1.0, 3)
    assert p.repeat_last_n == 64 and args.ctx == 512 and args.n_predict == 9
    args = parse(["--seed", "11", "--ctx", "64", "--n-predict", "2"])
    assert cli.sampler_params_from(args).seed == 11 and (args.ctx, args.n_predict) == (64, 2)


def test_prompts_are_token_ids():
    assert cli.parse_prompts(["1", "2,3", "/", "4"]) == [[1, 2, 3], [4]]
    with pytest.raises(ValueError, match="no tokenizer"):
        cli.parse_prompts(["hello"])


def test_exit_codes(capsys):
    assert cli.main([]) == 0
    assert cli.main(["run", "/nonexistent/model", "1 2"]) == 1
    assert "alpacca_b200: error:" in capsys.readouterr().err


def test_show_reads_a_folder_without_a_gpu(tmp_path, capsys):
    import tiny
    from alpacca_b200.engine.loading import write_random_model_dir
    d = write_random_model_dir(tmp_path / "m", tiny.TINY_C, 3, dtype="bfloat16")
    assert cli.main(["show", str(d), "--tensors"]) == 0
    out = capsys.readouterr().out
    assert '"hidden_size": 120' in out and "model.safetensors" in out and "4 layers" in out
    assert "model.layers.3.self_attn.q_proj.bias" in out and "BF16" in out
    (d / "config.json").write_text((d / "config.json").read_text().replace('"hidden_size": 120', '"hidden_size": 128'))
    assert cli.main(["show", str(d)]) == 1
    assert "shape" in capsys.readouterr().err
