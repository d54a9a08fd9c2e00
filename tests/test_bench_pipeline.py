"""The pipeline benchmark scripts run (on CPU, with a tiny model) and compose valid commands."""

import json

from benchmarks import bench_pipeline as bp

SMALL = ["--tokens", "1200", "--query-tokens", "128", "--seq-len", "32", "--token-batch-size", "256", "--precision", "fp32",
         "--projection-dim", "4"]


def test_in_memory_benchmark_runs(tmp_path, capsys):
    rec = bp.main(["inmem", *SMALL, "--workdir", str(tmp_path)])
    assert rec["tokens"] == 37 * 32 and rec["scores"] == 37 * 4 and rec["build_tokens_per_s"] > 0 and rec["score_checksum"] > 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["bench"] == "inmem"


def test_cli_benchmark_composes_the_four_commands(tmp_path, monkeypatch):
    from bergson_b200.cli.commands import COMMANDS
    from bergson_b200.config.parsing import parse_command

    seen = []

    def fake_run(cmd):
        seen.append(cmd)
        return 2.0

    monkeypatch.setattr(bp, "_run", fake_run)
    out = bp.main(["cli", *SMALL, "--workdir", str(tmp_path), "--gpus", "2"])
    assert [r["command"] for r in out] == ["build_query", "build", "reduce", "score"]
    assert out[1]["tokens"] == 37 * 32 and out[1]["tokens_per_s"] == 37 * 32 / 2.0 and out[0]["n_gpus"] == 2
    for cmd in seen:  # every composed command line parses
        parsed = parse_command(COMMANDS, cmd[3:], prog="bergson")
        assert parsed.index_cfg.distributed.nproc_per_node == 2 and parsed.index_cfg.precision == "fp32"
    assert seen[3][3] == "score" and "--query_path" in seen[3]
