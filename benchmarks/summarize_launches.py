"""Sum an `ncu --metrics gpu__time_duration.sum --csv` launch list per kernel name: python benchmarks/summarize_launches.py file.csv"""
import csv
import re
import sys
from collections import defaultdict

rows = []
with open(sys.argv[1], newline="") as f:
    lines = [l for l in f if l.startswith('"')]
rd = csv.DictReader(lines)
tot = defaultdict(lambda: [0, 0.0])
for r in rd:
    if r.get("Metric Name") != "gpu__time_duration.sum":
        continue
    name = re.sub(r"\(.*", "", r["Kernel Name"])
    v = float(r["Metric Value"].replace(",", ""))
    unit = r["Metric Unit"]
    us = v / 1000.0 if unit in ("ns", "nsecond") else v * (1000.0 if unit in ("ms", "msecond") else 1.0)
    tot[name][0] += 1
    tot[name][1] += us
total = sum(v[1] for v in tot.values())
print(f"{'kernel':60s} {'count':>6s} {'total_us':>10s} {'avg_us':>8s} {'share':>6s}")
for k, (n, us) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
    print(f"{k[:60]:60s} {n:6d} {us:10.1f} {us / n:8.2f} {100 * us / total:5.1f}%")
print(f"{'total':60s} {sum(v[0] for v in tot.values()):6d} {total:10.1f}")
