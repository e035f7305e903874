"""Turns an ncu report of one kernel into the two things the repository keeps of it:

* a short text summary (the counters the roofline figures use) and
* one entry of ``profiles/dram_traffic.json`` -- DRAM bytes per processed image -- which
  ``bench.py`` reads for ``roofline.traffic`` instead of carrying constants of its own.

    python -m fastertnn_b200.profile_summary REPORT.ncu-rep --workload tnn_conv_large --key f4_fused \
        --images 64 --summary profiles/NAME.txt --command "ncu ... (the command that made the report)"

Runs ``ncu -i REPORT --page raw --csv`` (works without a GPU).  With several captured launches
the figures are the mean over the launches.
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
TRAFFIC = ROOT / "profiles" / "dram_traffic.json"

COUNTERS = [
    "gpu__time_duration.sum", "launch__grid_size", "launch__block_size", "launch__registers_per_thread",
    "launch__shared_mem_per_block_dynamic", "dram__bytes_read.sum", "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "lts__t_sector_hit_rate.pct", "lts__t_bytes.sum",
    "lts__throughput.avg.pct_of_peak_sustained_elapsed", "l1tex__throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__warps_active.avg.pct_of_peak_sustained_active", "smsp__inst_executed.sum",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum", "l1tex__data_pipe_lsu_wavefronts_mem_shared.sum",
    "smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_wait_per_issue_active.ratio",
]
UNIT_SCALE = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "ns": 1e-3, "us": 1.0, "usecond": 1.0, "ms": 1e3, "msecond": 1e3, "nsecond": 1e-3}


def read_report(path: str):
    out = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], check=True, stdout=subprocess.PIPE, text=True).stdout
    rows = list(csv.reader(io.StringIO(out)))
    header, units, data = rows[0], rows[1], rows[2:]
    col = {h: i for i, h in enumerate(header)}
    launches = []
    for r in data:
        d = {"Kernel Name": r[col["Kernel Name"]]}
        for name in COUNTERS:
            if name in col and r[col[name]] not in ("", "n/a"):
                d[name] = (float(r[col[name]].replace(",", "")), units[col[name]])
        launches.append(d)
    return launches


def mean_of(launches, name):
    vals = [d[name] for d in launches if name in d]
    if not vals:
        return None, ""
    return sum(v for v, _ in vals) / len(vals), vals[0][1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("report")
    ap.add_argument("--workload", required=True)
    ap.add_argument("--key", required=True, help="kernel key bench.py looks up (f4_fused, f4_im2col, quantise_e2m1, ...)")
    ap.add_argument("--images", type=int, required=True, help="images one captured launch processed")
    ap.add_argument("--summary", help="text file to write")
    ap.add_argument("--command", default="", help="the command that produced the report")
    ap.add_argument("--note", default="")
    a = ap.parse_args()
    launches = read_report(a.report)
    if not launches:
        raise SystemExit("no launch in the report")
    rd, u1 = mean_of(launches, "dram__bytes_read.sum")
    wr, u2 = mean_of(launches, "dram__bytes_write.sum")
    rd_b, wr_b = rd * UNIT_SCALE.get(u1, 1.0), wr * UNIT_SCALE.get(u2, 1.0)
    table = json.loads(TRAFFIC.read_text()) if TRAFFIC.exists() else {}
    table.setdefault(a.workload, {})[a.key] = {
        "dram_bytes_per_image": (rd_b + wr_b) / a.images, "dram_read_bytes": rd_b, "dram_write_bytes": wr_b, "images_per_launch": a.images,
        "launches_averaged": len(launches), "kernel": launches[0]["Kernel Name"], "summary": a.summary or "", "command": a.command}
    TRAFFIC.write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
    if a.summary:
        lines = [f"ncu capture of {launches[0]['Kernel Name']}", f"workload: {a.workload} ({a.images} images per launch), {len(launches)} launch(es) averaged",
                 f"command: {a.command}", ""]
        for name in COUNTERS:
            v, u = mean_of(launches, name)
            if v is not None:
                lines.append(f"{name:<90s}{v:>16.6f} {u}")
        lines += ["", f"traffic = {rd_b / 1e6:.1f} MB read + {wr_b / 1e6:.1f} MB written = {(rd_b + wr_b) / 1e6:.1f} MB per launch "
                      f"= {(rd_b + wr_b) / a.images / 1e6:.3f} MB per image"]
        if a.note:
            lines += ["", a.note]
        Path(a.summary).write_text("\n".join(lines) + "\n")
    print(json.dumps(table[a.workload][a.key], indent=1))


if __name__ == "__main__":
    main()
