"""Benchmark drivers on CPU: the all-in-one latency CSV (reference schema) and sliding-window perplexity."""
import csv
import math
import os

import torch


def test_all_in_one_csv_schema(tmp_path, monkeypatch):
    import yaml
    from ipex_llm_b200.benchmark import all_in_one
    monkeypatch.chdir(tmp_path)
    conf = {"repo_id": ["synthetic:tiny"], "warm_up": 1, "num_trials": 2, "low_bit": "sym_int8", "batch_size": 2,
            "in_out_pairs": ["16-4", "24-3"], "test_api": ["transformer_int4"]}
    with open("config.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    rows = all_in_one.main(["config.yaml"])
    assert len(rows) == 2
    files = [n for n in os.listdir(".") if n.startswith("transformer_int4-results-") and n.endswith(".csv")]
    assert len(files) == 1
    with open(files[0]) as f:
        table = list(csv.reader(f))
    assert table[0][1:] == all_in_one.CSV_COLUMNS
    first = dict(zip(table[0][1:], table[1][1:]))
    assert first["input/output tokens"] == "16-4" and first["actual input/output tokens"] == "16-4"
    assert float(first["1st token avg latency (ms)"]) > 0 and float(first["2+ avg latency (ms/token)"]) > 0
    assert first["low_bit"] == "sym_int8" and first["batch_size"] == "2"


def test_perplexity_windows(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.benchmark.perplexity import BigDLPPL
    model = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
    ppl = BigDLPPL(model=model, device="cpu")
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (96,))
    # one window over everything = the plain definition
    s, c = ppl.nll(ids)
    assert c == 95
    whole = ppl.perplexity_hf(ids, seq_len=96)
    assert abs(whole - math.exp(s / c)) < 1e-6 * whole
    # a random model on random tokens is close to uniform over the vocabulary
    assert 0.3 * 32000 < whole < 3 * 32000
    # strided windows score every token exactly once and stay in the same range
    strided = ppl.perplexity_hf(ids, seq_len=48, stride=24)
    assert 0.3 * 32000 < strided < 3 * 32000


def test_check_results_and_stress(tmp_path, monkeypatch):
    import yaml
    from ipex_llm_b200.benchmark import all_in_one, check_results, stress_test
    monkeypatch.chdir(tmp_path)
    conf = {"repo_id": ["synthetic:tiny"], "warm_up": 0, "num_trials": 1, "low_bit": "sym_int8", "batch_size": 1,
            "in_out_pairs": ["8-2"], "test_api": ["transformer_int4"]}
    with open("config.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    all_in_one.main(["config.yaml"])
    assert check_results.main(["-c", "transformer_int4-results-", "-y", "config.yaml"]) == 0
    conf["in_out_pairs"].append("16-2")                 # a configured case without a row
    with open("config2.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    assert check_results.main(["-c", "transformer_int4-results-", "-y", "config2.yaml"]) == 1
    rc = stress_test.main(["--repo-id", "synthetic:tiny", "--test-api", "transformer_int4", "--low-bit", "sym_int8",
                           "--in-out", "8-3", "--rounds", "3", "--max-latency-drift", "100"])
    assert rc == 0
