"""Did every configured case produce a CSV row?  ``python -m ipex_llm_b200.benchmark.check_results -c <csv-prefix>
-y config.yaml`` (reference python/llm/test/benchmark/check_results.py:24-66: the nightly perf job fails when a
configured model / in-out pair is missing from the latency table)."""
from __future__ import annotations

import argparse
import csv
import glob
import sys


def missing_cases(csv_path: str, conf: dict):
    with open(csv_path) as f:
        rows = list(csv.DictReader(f))
    have = {(r["model"], r["input/output tokens"]) for r in rows}
    want = {(m, p) for m in conf["repo_id"] for p in conf["in_out_pairs"]}
    return sorted(want - have)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-c", "--csv_name", required=True, help="csv file or the prefix of <test_api>-results-<date>.csv")
    ap.add_argument("-y", "--yaml_name", required=True)
    a = ap.parse_args(argv)
    import yaml
    with open(a.yaml_name) as f:
        conf = yaml.safe_load(f)
    files = [a.csv_name] if a.csv_name.endswith(".csv") else sorted(glob.glob(a.csv_name + "*.csv"))
    if not files:
        print(f"no csv matches {a.csv_name}")
        return 1
    miss = missing_cases(files[-1], conf)
    for m, p in miss:
        print(f"missing: {m} {p}")
    print("All the test cases are completed." if not miss else f"{len(miss)} test case(s) missing.")
    return 1 if miss else 0


if __name__ == "__main__":
    sys.exit(main())
