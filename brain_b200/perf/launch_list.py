"""Aggregate an ``ncu --metrics gpu__time_duration.sum --csv`` launch list by kernel.

    python -m brain_b200.perf.launch_list launches.csv [--top 25]

Durations in such a list are cold-cache and serialised, so compare SHARES, not absolute times."""
from __future__ import annotations

import argparse
import collections
import csv
import sys


def aggregate(path: str):
    with open(path) as f:
        lines = [l for l in f if l.startswith('"')]
    agg = collections.defaultdict(lambda: [0, 0.0])
    total = 0.0
    n = 0
    for row in csv.DictReader(lines):
        name = row["Kernel Name"].split("(")[0]
        v = float(row["Metric Value"].replace(",", ""))
        unit = row["Metric Unit"]
        us = v / 1e3 if unit in ("ns", "nsecond") else v * 1e3 if unit in ("ms", "msecond") else v
        agg[name][0] += 1
        agg[name][1] += us
        total += us
        n += 1
    return agg, total, n


def render(agg, total, n, top=25) -> str:
    out = [f"{n} launches, {total / 1e3:.2f} ms of kernel time", f"{'ms':>9} {'share':>7} {'n':>6} {'us/launch':>10}  kernel"]
    for name, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:top]:
        out.append(f"{t / 1e3:9.2f} {100 * t / total:6.1f}% {c:6d} {t / c:10.1f}  {name[:90]}")
    return "\n".join(out)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--top", type=int, default=25)
    a = ap.parse_args(argv)
    print(render(*aggregate(a.csv), top=a.top))


if __name__ == "__main__":
    main(sys.argv[1:])
