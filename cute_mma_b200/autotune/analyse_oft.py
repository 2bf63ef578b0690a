"""Joins the sweep results with the parameter index and prints the best configurations
(the role of the reference's autotune/analyse_oft.py:11-18)."""
from __future__ import annotations

import argparse
import os

import pandas as pd

from .runner_oft import load_results


def table(configs: str, results: str) -> pd.DataFrame:
    params = pd.read_csv(os.path.join(configs, "config_csvs", "param.csv"))
    res = load_results(results)
    params["flops"] = [res.get(f"autotune_{c}", {}).get("value", float("nan")) for c in params["config"]]
    return params.sort_values("flops", ascending=False)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="autotune_configs")
    ap.add_argument("--results", default="results_oft.jsonl")
    a = ap.parse_args()
    print(table(a.configs, a.results).head(10).to_string(index=False))
