"""Turn an ``.ncu-rep`` file into the short text table kept under ``profiles/``.

    python benchmarks/ncu_summary.py prof.ncu-rep [--all-stalls]

Runs ``ncu -i <file> --page raw --csv`` (works without a GPU) and prints, per captured launch: duration, DRAM
bytes and throughput, tensor-pipe and SM throughput, registers / block / grid / shared memory, and the warp
stall reasons above 0.3 per issued instruction.
"""
import argparse
import csv
import io
import subprocess

KEEP = [
    ("gpu__time_duration.sum", "duration"),
    ("dram__bytes_read.sum", "dram read"),
    ("dram__bytes_write.sum", "dram write"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "dram throughput %"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active %"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "sm throughput %"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active %"),
    ("launch__registers_per_thread", "registers/thread"),
    ("launch__block_size", "block"),
    ("launch__grid_size", "grid"),
    ("launch__shared_mem_per_block_dynamic", "dynamic smem"),
]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("report")
    ap.add_argument("--all-stalls", action="store_true")
    args = ap.parse_args()
    raw = subprocess.run(["ncu", "-i", args.report, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    rows = list(csv.reader(io.StringIO(raw)))
    header, units = rows[0], rows[1]
    col = {h: i for i, h in enumerate(header)}
    for r in rows[2:]:
        print(f"### {r[col['Kernel Name']][:110]}")
        print("| metric | value |\n|---|---|")
        for key, label in KEEP:
            if key in col:
                print(f"| {label} | {r[col[key]]} {units[col[key]]} |")
        for h, i in col.items():
            if h.startswith("smsp__average_warps_issue_stalled_") and h.endswith("_per_issue_active.ratio"):
                try:
                    v = float(r[i])
                except ValueError:
                    continue
                if args.all_stalls or v >= 0.3:
                    print(f"| stall {h[len('smsp__average_warps_issue_stalled_'):-len('_per_issue_active.ratio')]} | {v:.2f} per issue |")
        print()


if __name__ == "__main__":
    try:
        main()
    except BrokenPipeError:      # output piped into head
        pass
