"""The command line's options (no GPU): names and defaults of the reference's flags."""
import json

from odin_infer_b200.cli import build_parser, main, parse_ids
from tests import tiny


def test_reference_flags_and_defaults():
    a = build_parser().parse_args(["model_dir"])
    # docs/ENVIRONMENT.md:50-62 of the reference
    assert (a.temperature, a.top_p, a.seed, a.repetition_penalty, a.max_ctx) == (0.6, 0.95, 0, 1.0, 4096)
    assert a.print_tps is False and a.print_ttft is False and a.max_new_tokens == 256
    a = build_parser().parse_args(["m", "-t", "0", "-p", "0.5", "-s", "7", "-x", "1.3", "-r", "-f", "-c", "512",
                                   "-j", "4", "-g", "1", "--prompt-ids", "1,2,3", "--prompt-ids", "4 5"])
    assert (a.temperature, a.top_p, a.seed, a.repetition_penalty, a.max_ctx) == (0.0, 0.5, 7, 1.3, 512)
    assert a.print_tps and a.print_ttft and a.prompt_ids == ["1,2,3", "4 5"]
    assert parse_ids("1, 2 3,4") == [1, 2, 3, 4]


def test_write_random_model(tmp_path, capsys):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(tiny.TINY_A))
    out = tmp_path / "model"
    assert main(["--random-config", str(cfg), "--weights-seed", "3", "--write-random-model", str(out)]) == 0
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    assert main([]) == 2
    assert main(["--write-random-model", str(out)]) == 2
