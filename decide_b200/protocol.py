"""The measuring and checking protocol of the reference's `decide bench` and `decide check`, on this backend.

    python -m decide_b200.protocol bench [--json report.json] [--iters 20] [--warmup 3]

bench (crates/decide-cli/src/bench.rs:40-71, 96-112, 303-349, 440-514): per request a warm-up then
`iters` timed runs (half as many for the long request), spans `e2e_ms` (host ids -> host logits,
wall clock) and `gpu_ms` (CUDA events around the same call), p50 / p95 by linear interpolation
between closest ranks, the machine's state captured before and after (host load per core, free
memory, swap, top processes; and what plays the part of "AC power, low-power mode off" on a GPU
server: SM clock against its maximum, power draw against the limit, active throttle reasons, other
compute processes on the device), FLAG lines for handicapped runs, and a JSON report that carries
every sample. The reference flags GEMM pipelines built during the runs ("the warm-up missed them");
the same check here is on tensor maps encoded and allocations made during the timed runs.

check (`check_table`; crates/decide-cli/src/check.rs:22-25, 195-343): the parity table, one row per request
(tokens, rows computed, max|dlogit|, max|dp|, decisions agreeing, smallest gold top-2 margin,
forward ms) and the summary with the allowed near-tie flips listed. The reference checks its 58
gold files, which need the real checkpoint; here the gold is the fp32 CPU forward of the same
synthetic weights, supplied by the caller (tests, bench) as logits, so this module never imports
the CPU oracle.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import time

import numpy as np

from . import check as parity

STEADY_STATE = "every request is warmed up before it is timed; weights, tensor maps and workspace are resident"
SPANS = {
    "e2e_ms": "host token ids in -> candidate logits on the host (copies, every kernel, the wait)",
    "gpu_ms": "CUDA events around the same call on its stream",
}


def quantile(samples, p: float) -> float:
    """The p-quantile (0..1) by linear interpolation between the closest ranks (bench.rs:103-112)."""
    s = sorted(float(x) for x in samples)
    if not s:
        return float("nan")
    rank = p * (len(s) - 1)
    lo, hi = int(np.floor(rank)), int(np.ceil(rank))
    return s[lo] + (s[hi] - s[lo]) * (rank - lo)


def stats(samples) -> dict:
    """A sample's summary, every sample included (bench.rs's Stats::json)."""
    s = [float(x) for x in samples]
    return {"p50": quantile(s, 0.5), "p95": quantile(s, 0.95), "min": min(s) if s else None, "max": max(s) if s else None,
            "mean": sum(s) / len(s) if s else None, "samples": s}


def _run(cmd: list) -> str | None:
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=10)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return out.stdout if out.returncode == 0 else None


GPU_FIELDS = ("name,clocks.sm,clocks.max.sm,power.draw,power.limit,memory.used,memory.total,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def machine_state(gpu: int = 0, run=_run) -> dict:
    """What the machine is doing, as far as the timings are concerned (bench.rs:303-349). `run` executes a command and
    returns its standard output or None (tests pass a fake)."""
    cores = os.cpu_count() or 1
    try:
        load = list(os.getloadavg())
    except OSError:
        load = None
    per_core = load[0] / cores if load else None
    mem_free = swap_used = None
    try:
        info = {l.split(":")[0]: int(l.split()[1]) for l in open("/proc/meminfo") if len(l.split()) >= 2}
        mem_free = round(100.0 * info["MemAvailable"] / info["MemTotal"])
        swap_used = round((info["SwapTotal"] - info["SwapFree"]) / 1024.0)
    except (OSError, KeyError, ValueError):
        pass
    top = []
    for line in (run(["ps", "-Ao", "pcpu=,comm=", "--sort=-pcpu"]) or "").splitlines()[:5]:
        parts = line.split(None, 1)
        if len(parts) == 2:
            try:
                top.append({"cpu_percent": float(parts[0]), "process": parts[1].strip().rsplit("/", 1)[-1]})
            except ValueError:
                pass
    g = {"name": None, "sm_mhz": None, "sm_max_mhz": None, "power_w": None, "power_limit_w": None, "throttle_reasons": [], "other_processes": None}
    row = (run(["nvidia-smi", f"--id={gpu}", f"--query-gpu={GPU_FIELDS}", "--format=csv,noheader,nounits"]) or "").strip().split(", ")
    if len(row) >= 11:
        num = lambda v: float(v) if v.replace(".", "", 1).isdigit() else None
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        g.update(name=row[0], sm_mhz=num(row[1]), sm_max_mhz=num(row[2]), power_w=num(row[3]), power_limit_w=num(row[4]),
                 memory_used_mib=num(row[5]), memory_total_mib=num(row[6]),
                 throttle_reasons=[n for n, v in zip(names, row[7:11]) if v.strip().lower() == "active"])
    apps = run(["nvidia-smi", f"--id={gpu}", "--query-compute-apps=pid,used_memory", "--format=csv,noheader,nounits"])
    if apps is not None:
        pids = [int(l.split(",")[0]) for l in apps.splitlines() if l.strip() and l.split(",")[0].strip().isdigit()]
        g["other_processes"] = len([p for p in pids if p != os.getpid()])
    return {"load_average": load, "cores": cores, "load_per_core": round(per_core, 2) if per_core is not None else None,
            "load_flag": bool(per_core is not None and per_core > 1.0), "memory_free_percent": mem_free, "swap_used_mb": swap_used,
            "top_processes": top, "gpu": g,
            "gpu_flag": bool(set(g["throttle_reasons"]) & {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"} or (g["other_processes"] or 0) > 0)}


def describe_machine(m: dict) -> str:
    load = " ".join(f"{x:.2f}" for x in m["load_average"]) if m.get("load_average") else "unknown"
    top = ", ".join(f"{p['process']} {p['cpu_percent']:.0f}%" for p in m.get("top_processes", [])) or "-"
    g = m.get("gpu", {})
    return (f"load {load} on {m['cores']} cores, memory free {m.get('memory_free_percent')}%, swap {m.get('swap_used_mb')} MB; "
            f"{g.get('name')}: SM {g.get('sm_mhz')}/{g.get('sm_max_mhz')} MHz, {g.get('power_w')}/{g.get('power_limit_w')} W, "
            f"throttle {g.get('throttle_reasons') or 'none'}, other processes on the GPU {g.get('other_processes')}; top: {top}")


def flags(before: dict, after: dict, encoded_during_runs: int = 0, allocations_during_runs: int = 0) -> list:
    """The FLAG lines of a handicapped run (bench.rs:466-474)."""
    out = []
    if before.get("load_flag") or after.get("load_flag"):
        out.append("FLAG: load above 1 per core; these timings are not protocol numbers")
    for when, m in (("before", before), ("after", after)):
        g = m.get("gpu", {})
        bad = sorted(set(g.get("throttle_reasons") or []) & {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"})
        if bad:
            out.append(f"FLAG: the GPU was slowed down ({', '.join(bad)}) {when} the runs; these timings are not protocol numbers")
        if (g.get("other_processes") or 0) > 0:
            out.append(f"FLAG: {g['other_processes']} other compute process(es) on the GPU {when} the runs; these timings are not protocol numbers")
    if encoded_during_runs > 0:
        out.append(f"FLAG: {encoded_during_runs} tensor maps were encoded during the runs (the warm-up missed them)")
    if allocations_during_runs > 0:
        out.append(f"FLAG: {allocations_during_runs} device allocations were made during the runs (the warm-up missed them)")
    return out


def measure(eng, batch, iters: int, warmup: int) -> dict:
    """One request (or batch) through the public host-buffer call: warm-up, then `iters` timed runs of both spans."""
    import torch

    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        eng.logits(batch)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e, gpu = [], []
    for _ in range(iters):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record(stream)
        eng.logits(batch)
        e1.record(stream)
        torch.cuda.synchronize()
        e2e.append((time.perf_counter() - t0) * 1e3)
        gpu.append(e0.elapsed_time(e1))
    return {"e2e_ms": stats(e2e), "gpu_ms": stats(gpu), "rows_computed": eng.resident_rows}


def bench_report(eng, requests: list, iters: int = 20, warmup: int = 3, gpu: int = 0, engine_info: dict | None = None) -> tuple[dict, list]:
    """`decide bench`: `requests` = [(name, Batch)]. Returns (report, lines to print)."""
    dev = eng.dev
    before = machine_state(gpu)
    lines = [f"machine before: {describe_machine(before)}", "",
             f"{'request':<24} {'tokens':>7} {'rows':>7}  {'e2e p50':>9} {'p95':>9}  {'gpu p50':>9} {'p95':>9}"]
    results = []
    for name, batch in requests:
        n = max(1, iters // 2) if batch.rows >= 2000 and batch.n_seq == 1 else iters   # the long request runs half as often (bench.rs:60-64)
        for _ in range(warmup):
            eng.logits(batch)
        e_before, a_before = dev.tmap_encodes, dev.alloc_count
        m = measure(eng, batch, n, 0)
        m.update(name=name, tokens=batch.rows, requests=batch.n_seq, answers=len(batch.ans_rows),
                 tensor_maps_encoded=dev.tmap_encodes - e_before, allocations=dev.alloc_count - a_before)
        results.append(m)
        lines.append(f"{name:<24} {batch.rows:>7} {m['rows_computed']:>7}  {m['e2e_ms']['p50']:>9.3f} {m['e2e_ms']['p95']:>9.3f}  "
                     f"{m['gpu_ms']['p50']:>9.3f} {m['gpu_ms']['p95']:>9.3f}")
    after = machine_state(gpu)
    fl = flags(before, after, sum(r["tensor_maps_encoded"] for r in results), sum(r["allocations"] for r in results))
    lines += ["", f"machine after: {describe_machine(after)}"] + fl
    report = {"date": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"), "engine": engine_info or {},
              "protocol": {"warmup": warmup, "iters": iters, "percentiles": "linear interpolation between closest ranks", "spans": SPANS,
                           "steady_state": STEADY_STATE},
              "machine": {"before": before, "after": after}, "flags": fl, "requests": results}
    return report, lines


def measure_request(de, name: str, text: str, iters: int = 20, warmup: int = 3, primer: str | None = None) -> dict:
    """One request JSON through `DecisionEngine.decide`, timed as the reference's bench does (bench.rs:209-290): cold
    (`primer` None: the state cache is emptied before every run, outside the timed region) or as a follow-up (`primer`: that
    request runs once, untimed, to cache its state, and every run of `text` finds it). Spans per run: tokenize, forward
    (ids to logits on the host), head, end to end."""
    follow_up = primer is not None

    def reset():
        if not follow_up:
            de.engine.forget_states()

    if follow_up:
        de.decide(primer)
    reset()
    first = de.decide(text)   # the first warm-up run also records what the request is
    for _ in range(1, warmup):
        reset()
        de.decide(text)
    spans = {"tokenize": [], "forward": [], "head": [], "e2e": []}
    for _ in range(iters):
        reset()
        t0 = time.perf_counter()
        d = de.decide(text)
        spans["e2e"].append((time.perf_counter() - t0) * 1e3)
        for k in ("tokenize", "forward", "head"):
            spans[k].append(d.timings[f"{k}_ms"])
    return {"name": name, "kind": "follow-up" if follow_up else "cold", "tokens": len(first.prepared.ids), "rows": first.rows, "route": first.route,
            "decisions": {f: a["decision"] for f, a in first.response["answers"].items()},
            **{f"{k}_ms": stats(v) for k, v in spans.items()}}


def check_table(rows: list) -> tuple[bool, list]:
    """`decide check`'s table and summary (check.rs:270-343). rows = [{"name", "tokens", "rows", "got", "want", "ncand", "forward_ms"}]
    with got / want logits [n, max_cand]. Returns (pass, lines)."""
    lines = [f"criteria: decisions agree wherever the gold top-2 logit margin is >= {parity.MARGIN}; calibrated |dp| <= {parity.MAX_DP}; "
             f"|dlogit| <= {parity.MAX_DLOGIT}", "",
             f"{'request':<18} {'tokens':>6}  {'rows':>6}  {'max|dlogit|':>11}  {'max|dp|':>9}  {'decisions':>9}  {'gold margin':>11}  {'forward ms':>10}"]
    failures, small_flips, agree, fields, worst_dl, worst_dp, ms = [], [], 0, 0, (0.0, "-"), (0.0, "-"), []
    for r in rows:
        t = parity.compare(r["got"], r["want"], r["ncand"])
        margin = min(parity.top2_margin(r["want"][i, :int(n)]) for i, n in enumerate(r["ncand"]))
        lines.append(f"{r['name']:<18} {r['tokens']:>6}  {r['rows']:>6}  {t['max_dlogit']:>11.4f}  {t['max_dp']:>9.5f}  {t['agree']:>4}/{t['fields']:<4}  "
                     f"{margin:>11.3f}  {r['forward_ms']:>10.1f}")
        failures += [f"{r['name']}: {f}" for f in t["failures"]]
        small_flips += [f"{r['name']}: {f}" for f in t["small_flips"]]
        agree, fields = agree + t["agree"], fields + t["fields"]
        worst_dl = max(worst_dl, (t["max_dlogit"], r["name"]))
        worst_dp = max(worst_dp, (t["max_dp"], r["name"]))
        ms.append(r["forward_ms"])
    ok = not failures
    lines.append("")
    if failures:
        lines += ["failures:"] + [f"  {f}" for f in failures]
    lines += [f"summary: {len(rows)} requests, {fields} fields: {'PASS' if ok else 'FAIL'}",
              f"  decisions agree: {agree}/{fields}; flips below the {parity.MARGIN} gold margin (allowed): {'; '.join(small_flips) or 'none'}",
              f"  max |dlogit| {worst_dl[0]:.4f} at {worst_dl[1]}; max |dp| {worst_dp[0]:.5f} at {worst_dp[1]} (tolerance {parity.MAX_DP})",
              f"  forward mean {sum(ms) / max(len(ms), 1):.1f} ms, max {max(ms, default=0.0):.1f} ms"]
    return ok, lines


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("mode", choices=["bench"])
    ap.add_argument("--json", default=None, help="write the report with every sample here")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    import torch

    from .engine import Engine
    from .kernels import Device
    from .synth import synth_batch, synth_fused_on_device
    from .weights import BASELINE_DIMS as dims

    dev = Device(0)
    cuda = torch.device("cuda", 0)
    fused, embed, final_norm = synth_fused_on_device(dims, 1, cuda)
    eng = Engine(dims, dev=dev, max_rows=4096, max_seqs=4, max_answers=16, max_cand=16, fused_layers=fused, embed=embed, final_norm=final_norm)
    # stand-ins for the reference's card (276 tokens, 3 questions), ticket (603, 6) and long-document (2,307, 3) requests
    requests = [("card-like (276)", synth_batch(dims, 1, 276, seed=3, n_answers=3)), ("ticket-like (603)", synth_batch(dims, 1, 603, seed=4, n_answers=6)),
                ("long-document-like (2307)", synth_batch(dims, 1, 2307, seed=5, n_answers=3))]
    report, lines = bench_report(eng, requests, args.iters, args.warmup,
                                 engine_info={"backend": "decide-cuda", "dtype": dev.act.name.lower(), "model": "synthetic weights at the benchmark's dims", "layers": dims.n_layers})
    print("\n".join(lines))
    if args.json:
        with open(args.json, "w") as f:
            f.write(json.dumps(report, indent=2) + "\n")
        print(f"report: {args.json}")
    eng.close()


if __name__ == "__main__":
    main()
