"""CLI smoke on the CPU path."""
import json

from antfly_b200.cli import main


def test_cli_embed_rerank_generate_list(capsys, tmp_path):
    assert main(["embed", "--model", "random:tiny", "--device", "cpu", "--text", "hello", "world", "--dimensions", "8"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(lines) == 2 and len(lines[0]["embedding"]) == 8
    assert main(["rerank", "--model", "random:tiny", "--device", "cpu", "--query", "q", "--doc", "a", "bb"]) == 0
    out = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert {o["index"] for o in out} == {0, 1} and out[0]["score"] >= out[1]["score"]
    assert main(["generate", "--model", "random:tiny", "--device", "cpu", "--kv-blocks", "64", "--prompt", "hi",
                 "--max-tokens", "4", "--print-timing", "--print-finish-reason", "--draft-layers", "1",
                 "--speculative-k", "2"]) == 0
    cap = capsys.readouterr()
    assert "generate_timing_ms:" in cap.err and "speculative: rounds=" in cap.err and "finish_reason:" in cap.err
    assert main(["list", "--models-dir", str(tmp_path)]) == 0
    assert "chunkers" in capsys.readouterr().out
