"""Turn Nsight Compute output into the short tables kept under ``profiles/``.

    ncu -i prof.ncu-rep --page raw --csv > prof.csv
    python -m lorafusion_b200.cli.summarize_ncu prof.csv                 # one row per captured launch
    python -m lorafusion_b200.cli.summarize_ncu launches.csv --launches  # time share per kernel name

Two input kinds: the ``--page raw --csv`` export of a ``--set full`` (or sections) capture, and
the ``--metrics gpu__time_duration.sum --csv`` launch list.  Counterpart of
``benchmarks_paper/summarize_kernel_ncu_profile.py`` (DRAM bytes per NVTX range from
``scripts/kernel_perf/2_kernel_ncu_profile.sh:22-41``), extended with the tensor-pipe and
occupancy counters a Blackwell roofline needs.
"""

from __future__ import annotations

import argparse
import csv
import re
from collections import defaultdict

RAW_COLUMNS = [
    ("gpu__time_duration.sum", "duration"),
    ("sm__cycles_elapsed.avg.per_second", "SM clock"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM write"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM %"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe %"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "SM %"),
    ("lts__t_sector_hit_rate.pct", "L2 hit %"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active %"),
    ("launch__registers_per_thread", "regs"),
    ("launch__grid_size", "grid"),
]


def _short(name: str, width: int = 70) -> str:
    name = re.sub(r"^void\s+", "", name)
    name = re.sub(r"\(.*\)$", "", name)
    return name if len(name) <= width else name[:width - 3] + "..."


def _csv_rows(path: str) -> list:
    """ncu prefixes its CSV with ``==PROF==`` lines when the log and the CSV share a file."""
    with open(path, newline="") as f:
        lines = [ln for ln in f if not ln.startswith("==")]
    return list(csv.reader(lines))


def summarize_raw(path: str) -> str:
    rows = _csv_rows(path)
    hdr, units, body = rows[0], rows[1], rows[2:]
    idx = {h: i for i, h in enumerate(hdr)}
    cols = [(m, label) for m, label in RAW_COLUMNS if m in idx]
    out = ["| kernel | " + " | ".join(label for _, label in cols) + " |",
           "|---|" + "---|" * len(cols)]
    for r in body:
        cells = []
        for m, _ in cols:
            v, u = r[idx[m]], units[idx[m]]
            try:
                v = f"{float(v.replace(',', '')):.4g}"
            except ValueError:
                pass
            cells.append(f"{v} {u}".strip() if u not in ("", "%") else v)
        out.append(f"| `{_short(r[idx['Kernel Name']])}` | " + " | ".join(cells) + " |")
    return "\n".join(out)


def summarize_launches(path: str) -> str:
    rows = _csv_rows(path)
    hdr = rows[0]
    idx = {h: i for i, h in enumerate(hdr)}
    name_i, val_i = idx["Kernel Name"], idx["Metric Value"]
    unit_i = idx.get("Metric Unit")
    tot = defaultdict(float)
    cnt = defaultdict(int)
    for r in rows[1:]:
        if len(r) <= val_i or r[idx["Metric Name"]] != "gpu__time_duration.sum":
            continue
        v = float(r[val_i].replace(",", ""))
        unit = r[unit_i] if unit_i is not None else "ns"
        v *= {"ns": 1e-6, "us": 1e-3, "ms": 1.0, "s": 1e3}.get(unit, 1e-6)
        k = _short(r[name_i])
        tot[k] += v
        cnt[k] += 1
    total = sum(tot.values()) or 1.0
    out = [f"Total {total:.1f} ms over {sum(cnt.values())} launches.", "",
           "| kernel | launches | ms | share |", "|---|---|---|---|"]
    for k in sorted(tot, key=tot.get, reverse=True):
        out.append(f"| `{k}` | {cnt[k]} | {tot[k]:.3f} | {100 * tot[k] / total:.1f} % |")
    return "\n".join(out)


def main(argv=None) -> str:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("csv_file")
    ap.add_argument("--launches", action="store_true", help="input is a gpu__time_duration.sum launch list")
    args = ap.parse_args(argv)
    text = summarize_launches(args.csv_file) if args.launches else summarize_raw(args.csv_file)
    print(text)
    return text


if __name__ == "__main__":
    main()
