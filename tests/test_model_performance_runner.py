"""benchmarks/run_model_performance.py: the reference's JSON batch description, CSV output, layer ranges and the
two-rank communication mode, on CPU with the tiny model."""
import csv
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "benchmarks", "run_model_performance.py")


def _run(args, **kw):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=300, env=env, **kw)


def test_json_batches_per_dp_csv_and_layer_range(tmp_path):
    cfg = {"layer_forward_round": 3,
           "batch_0": {"dp_0": [{"forwarding_token_num": 24, "sequence_len": 40, "request_num": 2},
                                {"forwarding_token_num": 1, "sequence_len": 33, "request_num": 3}],
                       "dp_1": [{"forwarding_token_num": 1, "sequence_len": 20, "request_num": 4}]},
           "batch_1": {"dp_0": [{"forwarding_token_num": 16, "sequence_len": 16, "request_num": 1}]}}
    p = tmp_path / "perf.json"
    p.write_text(json.dumps(cfg))
    out = tmp_path / "perf.csv"
    r = _run([SCRIPT, "--model", "tiny-llama", "--device", "cpu", "--perf-config", str(p), "--warmup-round", "1",
              "--profile-round", "2", "--output", str(out), "--lower-layer-idx", "1", "--upper-layer-idx", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [(x["batch_id"], x["dp"]) for x in rows] == [(0, 0), (0, 1), (1, 0)]
    assert rows[0]["tokens"] == 2 * 24 + 3 and rows[0]["seqs"] == 5 and rows[0]["layers"] == 1
    assert rows[1]["tokens"] == 4 and rows[2]["tokens"] == 16
    assert all(x["layer_forward_round"] == 3 and x["forward_ms"] > 0 for x in rows)
    with open(out) as f:
        table = list(csv.reader(f))
    assert table[0][:3] == ["batch_id", "dp", "tokens"] and len(table) == 4
    # the same batch on every DP rank: only dp_0 entries run
    r2 = _run([SCRIPT, "--model", "tiny-llama", "--device", "cpu", "--perf-config", str(p), "--warmup-round", "1",
               "--profile-round", "1", "--same-batch-in-dps"])
    assert r2.returncode == 0, r2.stderr[-2000:]
    rows2 = [json.loads(l) for l in r2.stdout.splitlines() if l.startswith("{")]
    assert [(x["batch_id"], x["dp"]) for x in rows2] == [(0, 0), (1, 0)] and rows2[0]["layers"] == 2


def test_bad_perf_config_is_refused(tmp_path):
    p = tmp_path / "bad.json"
    p.write_text(json.dumps({"batch_0": {"dp_0": [{"forwarding_token_num": 50, "sequence_len": 40}]}}))
    r = _run([SCRIPT, "--model", "tiny-llama", "--device", "cpu", "--perf-config", str(p)])
    assert r.returncode != 0 and "forwarding_token_num" in r.stderr


def test_communication_mode_two_gloo_ranks():
    r = _run(["-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
              "29677", SCRIPT, "--comm", "--model", "tiny-llama", "--device", "cpu", "--max-step-tokens", "8",
              "--warmup-round", "1", "--profile-round", "3"])
    assert r.returncode == 0, r.stderr[-2000:]
    import re
    rows = [json.loads(m) for m in re.findall(r"\{[^{}]*\}", r.stdout)]  # the two ranks share one stdout
    assert sorted((x["role"], x["tokens"]) for x in rows) == sorted(
        (role, t) for role in ("master", "worker") for t in (1, 2, 4, 8))
    assert all(x["ms_per_round"] > 0 and x["hidden"] == 256 for x in rows)
