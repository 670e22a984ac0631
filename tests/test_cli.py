"""The command line: the reference's positional form and flags are parsed to the same fields."""
import json
import os
import subprocess
import sys

import pytest

from llm_steadyinfer_b200.cli.offline_batch_benchmark import parse_args

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_positional_form_and_flags():
    a = parse_args(["model_dir", "tok.json", "64", "16", "100", "out.csv", "2"])
    assert (a.checkpoint, a.tokenizer, a.num_requests, a.max_batch, a.max_gen, a.output_csv, a.iterations) == \
        ("model_dir", "tok.json", 64, 16, 100, "out.csv", 2)
    b = parse_args(["model_dir", "tok.json", "64", "16", "100", "--max-batch", "8", "--model-type", "llama3", "--seed", "7"])
    assert b.max_batch == 8 and b.num_requests == 64 and b.seed == 7
    c = parse_args(["--checkpoint", "m"])
    assert (c.num_requests, c.max_batch, c.max_gen, c.iterations, c.seed) == (512, 32, 256, 1, 42)    # the reference's defaults
    with pytest.raises(SystemExit):
        parse_args(["--checkpoint", "m", "--model-type", "qwen2"])
    with pytest.raises(SystemExit):
        parse_args([])


@pytest.mark.gpu
def test_cli_runs_the_1b_style_workload_small(tmp_path):
    """Lognormal lengths, Poisson arrivals, a shared prefix, sampling: through the program itself."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from tiny_configs import make_model_folder
    folder = make_model_folder(tmp_path, "B")
    out = tmp_path / "m.json"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "offline_batch_benchmark"), "--checkpoint", folder,
         "--num-requests", "24", "--max-batch", "6", "--max-gen", "12", "--prompt-len-dist", "lognormal:40,0.8,4,150",
         "--output-len-dist", "lognormal:8,0.5,1,12", "--prefix-share", "0.4,32", "--request-rate", "400",
         "--temperature", "0.7", "--top-p", "0.9", "--ignore-eos", "--kv-block-size", "8", "--num-kv-blocks", "80",
         "--max-num-batched-tokens", "48", "--output-csv", str(tmp_path / "m.csv"), "--output-json", str(out)],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    m = json.loads(out.read_text())[0]
    assert m["completed"] == 24 and m["rejected"] == 0 and m["output_tokens"] > 24
    assert m["prefix_hit_tokens"] > 0 and m["output_tps"] > 0 and m["ttft_p99_ms"] >= m["ttft_p50_ms"] > 0
    assert (tmp_path / "m.csv").read_text().startswith("run_id,")
