"""Analysis of exported traces: kernel classes, per-operator and per-communication-label time
and bytes, and exposed (not overlapped by compute) communication time.

Works on Kineto chrome traces (`rank_*.trace.json[.gz]`) and on `nsys export --type sqlite` files.
Kernels are classified by name into nccl / peer_comm / attention_fwd / attention_bwd / moe_transport /
grouped_gemm / dense_gemm / optimizer / elementwise / other, using this package's kernel names and the
usual library patterns. Communication labels follow `operator_trace.communication_label`.

Counterpart of dllm_parallel/core/profiling/trace_analysis.py:28-602.
"""
from __future__ import annotations

import gzip
import json
import re
import sqlite3
from collections import defaultdict

from .operator_trace import parse_communication_label

KERNEL_CLASSES = [
    ("nccl", re.compile(r"nccl", re.I)),
    ("peer_comm", re.compile(r"zero_reduce|zero_update|kv_gather|kv_scatter|barrier_kernel")),
    ("attention_fwd", re.compile(r"attn_fwd|flash.*fwd|fmha.*fwd", re.I)),
    ("attention_bwd", re.compile(r"attn_bwd|attn_delta|flash.*bwd|fmha.*bwd", re.I)),
    ("moe_transport", re.compile(r"dispatch|combine|all_to_all|alltoall", re.I)),
    ("grouped_gemm", re.compile(r"grouped", re.I)),
    ("dense_gemm", re.compile(r"gemm_bf16|gemm|cutlass|cublas|sm100.*mma", re.I)),
    ("optimizer", re.compile(r"adamw|sumsq", re.I)),
    ("elementwise", re.compile(r"rmsnorm|swiglu|qk_norm_rope|colsum|ce_finalize|kl_rows|merge|elementwise", re.I)),
]


def classify_kernel(name: str) -> str:
    for cls, pat in KERNEL_CLASSES:
        if pat.search(name):
            return cls
    return "other"


def _union_length(intervals) -> float:
    total, end = 0.0, None
    for s, e in sorted(intervals):
        if end is None or s > end:
            total += e - s
            end = e
        elif e > end:
            total += e - end
            end = e
    return total


def _subtract(a, b) -> float:
    """Length of the union of intervals `a` not covered by the union of `b`."""
    both = _union_length(list(a) + list(b))
    return both - _union_length(b)


def _short_name(name: str) -> str:
    """Kernel name without template arguments and parameter lists (one table row per kernel family)."""
    n = re.sub(r"\(.*$", "", name)
    n = re.sub(r"<.*$", "", n)
    n = n.replace("void ", "").strip()
    return n.split("::")[-1] if "::" in n and not n.startswith("at::") else n


def summarize(kernels: list[tuple[str, float, float]], ranges: list[tuple[str, float, float]],
              copies: list[tuple[str, float, float]] | None = None) -> dict:
    """kernels / ranges / copies: (name, start_us, end_us). `copies` are device memcpy / memset activities."""
    by_class = defaultdict(lambda: {"count": 0, "time_us": 0.0})
    by_name = defaultdict(lambda: {"count": 0, "time_us": 0.0, "class": ""})
    comm, compute = [], []
    for name, s, e in kernels:
        c = classify_kernel(name)
        by_class[c]["count"] += 1
        by_class[c]["time_us"] += e - s
        rec = by_name[_short_name(name)]
        rec["count"] += 1
        rec["time_us"] += e - s
        rec["class"] = c
        (comm if c in ("nccl", "peer_comm", "moe_transport") else compute).append((s, e))
    labels = defaultdict(lambda: {"count": 0, "time_us": 0.0, "input_bytes": 0, "logical_bytes": 0})
    operators = defaultdict(lambda: {"count": 0, "time_us": 0.0})
    for name, s, e in ranges:
        info = parse_communication_label(name)
        if info is not None:
            key = f"{info.get('domain')}/{info.get('phase')}/{info.get('collective')}"
            labels[key]["count"] += 1
            labels[key]["time_us"] += e - s
            labels[key]["input_bytes"] += int(info.get("input_bytes", 0))
            labels[key]["logical_bytes"] += int(info.get("logical_bytes", 0))
        elif name.startswith("dllm.operator.") or name.startswith("dllm.phase."):
            operators[name]["count"] += 1
            operators[name]["time_us"] += e - s
    copies = copies or []
    copy_classes = defaultdict(lambda: {"count": 0, "time_us": 0.0})
    for name, s, e in copies:
        key = ("host_to_device" if re.search(r"HtoD|Host.*Device", name) else
               "device_to_host" if re.search(r"DtoH|Device.*Host", name) else
               "device_to_device" if re.search(r"DtoD|Device.*Device", name) else
               "memset" if re.search(r"memset", name, re.I) else "other_copy")
        copy_classes[key]["count"] += 1
        copy_classes[key]["time_us"] += e - s
    all_k = [(s, e) for _, s, e in kernels]
    all_c = [(s, e) for _, s, e in copies]
    span = 0.0
    steps = [(s, e) for n, s, e in ranges if n.startswith("dllm.step.")]
    if steps:
        span = max(e for _, e in steps) - min(s for s, _ in steps)
    elif all_k:
        span = max(e for _, e in all_k) - min(s for s, _ in all_k)
    busy = _union_length(all_k)
    busy_or_copy = _union_length(all_k + all_c)
    top = sorted(by_name.items(), key=lambda kv: -kv[1]["time_us"])
    return {"kernel_classes": dict(by_class), "kernels_by_name": dict(top),
            "copy_classes": dict(copy_classes), "communication_labels": dict(labels), "operators": dict(operators),
            "compute_time_us": _union_length(compute), "communication_time_us": _union_length(comm),
            "exposed_communication_us": _subtract(comm, compute),
            "span_us": span, "kernel_busy_us": busy, "exposed_copy_us": _subtract(all_c, all_k),
            "idle_us": max(span - busy_or_copy, 0.0) if span else 0.0}


def analyze_kineto_trace(path: str) -> dict:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        data = json.load(f)
    events = data["traceEvents"] if isinstance(data, dict) else data
    kernels, ranges, copies = [], [], []
    for ev in events:
        if ev.get("ph") != "X":
            continue
        s, d = float(ev.get("ts", 0)), float(ev.get("dur", 0))
        cat = str(ev.get("cat", ""))
        if cat == "kernel":
            kernels.append((ev.get("name", ""), s, s + d))
        elif cat in ("gpu_memcpy", "gpu_memset"):
            copies.append((ev.get("name", ""), s, s + d))
        elif cat in ("user_annotation", "gpu_user_annotation", "cpu_op") and str(ev.get("name", "")).startswith("dllm."):
            ranges.append((ev["name"], s, s + d))
    return summarize(kernels, ranges, copies)


def analyze_nsys_sqlite(path: str) -> dict:
    con = sqlite3.connect(path)
    try:
        cur = con.cursor()
        names = dict(cur.execute("SELECT id, value FROM StringIds"))
        kernels = [(names.get(n, str(n)), s / 1e3, e / 1e3) for n, s, e in
                   cur.execute("SELECT demangledName, start, end FROM CUPTI_ACTIVITY_KIND_KERNEL")]
        ranges = []
        try:
            for text, tid, s, e in cur.execute("SELECT text, textId, start, end FROM NVTX_EVENTS WHERE end IS NOT NULL"):
                label = text if text is not None else names.get(tid, "")
                if label and label.startswith("dllm."):
                    ranges.append((label, s / 1e3, e / 1e3))
        except sqlite3.Error:
            pass
    finally:
        con.close()
    return summarize(kernels, ranges)


def write_summary(summary: dict, path: str) -> None:
    with open(path, "w") as f:
        json.dump(summary, f, indent=1, sort_keys=True)


def format_table(summary: dict, top: int = 25) -> str:
    """Markdown: device time per kernel family (share of the traced span), copies, exposed time and idle gaps."""
    span = summary.get("span_us") or 1.0
    lines = ["| kernel | class | launches | device ms | share of span |", "|---|---|---|---|---|"]
    for name, rec in list(summary["kernels_by_name"].items())[:top]:
        lines.append(f"| `{name}` | {rec['class']} | {rec['count']} | {rec['time_us'] / 1e3:.1f} | "
                     f"{100 * rec['time_us'] / span:.1f} % |")
    rest = list(summary["kernels_by_name"].items())[top:]
    if rest:
        t = sum(r["time_us"] for _, r in rest)
        lines.append(f"| {len(rest)} other kernels | | {sum(r['count'] for _, r in rest)} | {t / 1e3:.1f} | "
                     f"{100 * t / span:.1f} % |")
    lines.append("")
    lines.append("| quantity | ms | share of span |")
    lines.append("|---|---|---|")
    rows = [("traced span (dllm.step ranges)", span),
            ("kernels busy (union over streams)", summary["kernel_busy_us"]),
            ("copies not hidden behind kernels", summary["exposed_copy_us"]),
            ("device idle inside the span (launch gaps, host waits)", summary["idle_us"]),
            ("communication kernels not hidden behind compute", summary["exposed_communication_us"])]
    for k, rec in summary["copy_classes"].items():
        rows.append((f"copies: {k} ({rec['count']})", rec["time_us"]))
    for k, v in rows:
        lines.append(f"| {k} | {v / 1e3:.1f} | {100 * v / span:.1f} % |")
    labels = summary.get("communication_labels") or {}
    if labels:
        lines += ["", "| communication (domain/phase/op) | calls | host-range ms | input MB | logical MB | GB/s over the range |",
                  "|---|---|---|---|---|---|"]
        for key, rec in sorted(labels.items(), key=lambda kv: -kv[1]["time_us"]):
            moved = max(rec["input_bytes"], rec["logical_bytes"])
            rate = moved / (rec["time_us"] * 1e-6) / 1e9 if rec["time_us"] > 0 else 0.0
            lines.append(f"| {key} | {rec['count']} | {rec['time_us'] / 1e3:.2f} | {rec['input_bytes'] / 1e6:.1f} | "
                         f"{rec['logical_bytes'] / 1e6:.1f} | {rate:.1f} |")
    phases = {k: v for k, v in (summary.get("operators") or {}).items() if k.startswith("dllm.phase.")}
    if phases:
        lines += ["", "| step phase | count | ms | share of span |", "|---|---|---|---|"]
        for key, rec in sorted(phases.items(), key=lambda kv: -kv[1]["time_us"]):
            lines.append(f"| {key[len('dllm.phase.'):]} | {rec['count']} | {rec['time_us'] / 1e3:.1f} | "
                         f"{100 * rec['time_us'] / span:.1f} % |")
    return "\n".join(lines)


def analyze_directory(directory: str) -> dict:
    """Every `rank_*.trace.json[.gz]` of a run: per-rank span, busy share, exposed communication and idle time, and
    which rank is the slowest (the one the others wait for in every collective)."""
    import glob
    import os

    per_rank = {}
    for path in sorted(glob.glob(os.path.join(directory, "rank_*.trace.json*"))):
        m = re.search(r"rank_(\d+)\.trace", os.path.basename(path))
        if not m:
            continue
        sm = analyze_kineto_trace(path)
        span = sm["span_us"] or 1.0
        per_rank[int(m.group(1))] = {
            "span_ms": span / 1e3, "busy_pct": 100 * sm["kernel_busy_us"] / span,
            "compute_ms": sm["compute_time_us"] / 1e3, "exposed_communication_ms": sm["exposed_communication_us"] / 1e3,
            "exposed_copy_ms": sm["exposed_copy_us"] / 1e3, "idle_ms": sm["idle_us"] / 1e3}
    if not per_rank:
        raise FileNotFoundError(f"no rank_*.trace.json[.gz] under {directory}")
    compute = {r: v["compute_ms"] for r, v in per_rank.items()}
    slow = max(compute, key=compute.get)
    return {"ranks": per_rank, "slowest_rank_by_compute": slow,
            "compute_spread_pct": 100 * (max(compute.values()) - min(compute.values())) / max(min(compute.values()), 1e-9)}


def compare_summaries(a: dict, b: dict, top: int = 15) -> str:
    """Markdown table of the kernel families whose device time differs most between two summaries (a -> b), e.g. the
    same step on 2 and on 8 GPUs."""
    names = set(a["kernels_by_name"]) | set(b["kernels_by_name"])
    rows = []
    for n in names:
        ta = a["kernels_by_name"].get(n, {}).get("time_us", 0.0)
        tb = b["kernels_by_name"].get(n, {}).get("time_us", 0.0)
        rows.append((tb - ta, n, ta, tb))
    rows.sort(key=lambda r: -abs(r[0]))
    lines = ["| kernel | a ms | b ms | b - a ms |", "|---|---|---|---|"]
    for d, n, ta, tb in rows[:top]:
        lines.append(f"| `{n}` | {ta / 1e3:.1f} | {tb / 1e3:.1f} | {d / 1e3:+.1f} |")
    for key, label in (("span_us", "traced span"), ("kernel_busy_us", "kernels busy"), ("idle_us", "device idle"),
                       ("exposed_communication_us", "exposed communication"), ("exposed_copy_us", "exposed copies")):
        lines.append(f"| {label} | {a.get(key, 0) / 1e3:.1f} | {b.get(key, 0) / 1e3:.1f} | "
                     f"{(b.get(key, 0) - a.get(key, 0)) / 1e3:+.1f} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="python -m turbo_dllm_b200.profiling.trace_analysis",
                                 description="Summarise a Kineto chrome trace or an nsys sqlite export.")
    ap.add_argument("trace", help="a trace file, or a directory of rank_*.trace.json[.gz] files (per-rank table)")
    ap.add_argument("--json", help="write the full summary here")
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--compare", help="a second trace (or summary .json): print what changed from TRACE to it")
    a = ap.parse_args(argv)
    import os

    if os.path.isdir(a.trace):
        res = analyze_directory(a.trace)
        if a.json:
            write_summary(res, a.json)
        print("| rank | span ms | busy % | compute ms | exposed comm ms | exposed copies ms | idle ms |")
        print("|---|---|---|---|---|---|---|")
        for r, v in sorted(res["ranks"].items()):
            print(f"| {r} | {v['span_ms']:.1f} | {v['busy_pct']:.1f} | {v['compute_ms']:.1f} | "
                  f"{v['exposed_communication_ms']:.1f} | {v['exposed_copy_ms']:.1f} | {v['idle_ms']:.1f} |")
        print(f"\nslowest rank by compute time: {res['slowest_rank_by_compute']} "
              f"(spread {res['compute_spread_pct']:.1f} %)")
        return 0

    def load(path):
        if path.endswith(".json") and not path.endswith(".trace.json"):
            return json.load(open(path))
        return analyze_nsys_sqlite(path) if path.endswith(".sqlite") else analyze_kineto_trace(path)

    summary = load(a.trace)
    if a.compare:
        print(compare_summaries(summary, load(a.compare), a.top))
        return 0
    if a.json:
        write_summary(summary, a.json)
    print(format_table(summary, a.top))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
