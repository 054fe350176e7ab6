"""Summarise a profile written by ``SessionOptions.enable_profiling`` (chrome-trace JSON).

Counterpart of the reference's tools/python/profile_explorer: per operator type (or per node with ``--by-node``) the
number of calls, total / average / share of the node time, split by execution provider; ``--csv`` writes the table."""
from __future__ import annotations

import argparse
import csv
import json
import sys
from collections import defaultdict
from typing import Dict, List, Tuple


def load_events(path: str) -> List[dict]:
    with open(path) as f:
        data = json.load(f)
    return data["traceEvents"] if isinstance(data, dict) else data


def summarise(events: List[dict], by_node: bool = False) -> List[Tuple[str, str, int, float, float, float]]:
    """[(key, provider, calls, total_us, avg_us, percent)] sorted by total time, for the node events of a profile."""
    acc: Dict[Tuple[str, str], List[float]] = defaultdict(lambda: [0, 0.0])
    for e in events:
        if e.get("cat") != "Node" or not str(e.get("name", "")).endswith("_kernel_time"):
            continue
        args = e.get("args", {})
        key = e["name"][: -len("_kernel_time")] if by_node else args.get("op_name", "?")
        slot = acc[(key, args.get("provider", "?"))]
        slot[0] += 1
        slot[1] += float(e.get("dur", 0))
    total = sum(v[1] for v in acc.values()) or 1.0
    rows = [(k[0], k[1], int(v[0]), v[1], v[1] / max(v[0], 1), 100.0 * v[1] / total) for k, v in acc.items()]
    return sorted(rows, key=lambda r: -r[3])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="profile_explorer")
    ap.add_argument("profile")
    ap.add_argument("--by-node", action="store_true")
    ap.add_argument("--top", type=int, default=20)
    ap.add_argument("--csv")
    args = ap.parse_args(argv)
    rows = summarise(load_events(args.profile), args.by_node)
    print(f"{'name':40s} {'provider':24s} {'calls':>7s} {'total us':>12s} {'avg us':>10s} {'%':>6s}")
    for r in rows[: args.top]:
        print(f"{r[0][:40]:40s} {r[1][:24]:24s} {r[2]:7d} {r[3]:12.1f} {r[4]:10.1f} {r[5]:6.2f}")
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["name", "provider", "calls", "total_us", "avg_us", "percent"])
            w.writerows(rows)
    return 0


if __name__ == "__main__":
    sys.exit(main())
