"""Prefill throughput of the B200 engine on the benchmark's full-model config, and the CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one batched prefill of 64 requests x 603 seeded token ids through the full synthetic
36-layer hybrid model (3 Gated DeltaNet : 1 attention layer, hidden 2560, vocab 151936, tied bf16
embedding, random-init weights) ending in the candidate-row head over 6 answer rows x 16 candidate
ids per request. With N GPUs every rank runs its own 64 requests (requests share nothing: no
collective on the data path), so per-GPU work is fixed ("weak" scaling); `value` is the tokens all
ranks prefilled divided by the slowest rank's device time. At N > 1 the line also carries
`strong_scaling`: ONE set of 64 requests sharded 64/N over the ranks (every rank holds the same
weights), timed the same way, its logits gathered on rank 0 and compared bit for bit with rank 0's
own pass over the same shards.

`value` is timed with the batch resident in HBM; `e2e` is the same batch through the public
host-buffer call (`Engine.logits`: ids, offsets, answer rows and candidates copied in from host
memory, logits copied out, every step). `roofline` is the dominant kernel, the fused gate_up
projection GEMM (tensor-bound): 2*M*N*K per launch divided by its average CUDA-event duration inside
the timed steps, against the measured sustained bf16 peak. `cpu_baseline` times the reference's fp32
CPU forward (oracle/gold_synth.py) on one request with all host cores.

`--impl reference` times that CPU forward alone, one request per step.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

REQUESTS, TOKENS, ANSWERS, CANDS = 64, 603, 6, 16
METRIC, UNIT = "prefill_tokens_per_s", "tokens/s"
WORKLOAD = "configs[4]: full 36-layer hybrid model, 64 requests x 603 tokens, 6 answer rows x 16 candidates"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return {"bf16_tflops": j["bf16_tflops"], "bf16_tflops_sustained": j["bf16_tflops_sustained"], "hbm_gbs": j["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        self.gpu = gpu
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [l.split(", ") for l in Path(self.file.name).read_text().splitlines() if l.count(",") >= 8]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[5 + i].strip().lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "power_w_max": max(float(r[3]) for r in rows),
                "samples": len(rows), "reasons": reasons}


def sub_batch(batch, reqs: range):
    """The requests `reqs` of a batch of equal-length requests, as a batch of their own."""
    lo, hi = reqs.start, reqs.stop
    return type(batch)(batch.ids[lo * TOKENS:hi * TOKENS].copy(), (np.arange(hi - lo + 1) * TOKENS).astype(np.uint32),
                       (batch.ans_rows[lo * ANSWERS:hi * ANSWERS] - np.uint32(lo * TOKENS)).astype(np.uint32),
                       batch.cand[lo * ANSWERS:hi * ANSWERS].copy(), batch.ncand[lo * ANSWERS:hi * ANSWERS].copy())


def cpu_gold_setup(dims, seed):
    import torch

    from decide_b200.synth import synth_state_dict
    from oracle import gold_synth

    torch.set_num_threads(os.cpu_count() or 1)
    sd = synth_state_dict(dims, seed)
    return sd, gold_synth.build_model(dims, sd)


def run_reference(args):
    """The reference arm: the fp32 CPU forward the reference's gold generator runs, one request per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from decide_b200.synth import synth_batch
    from decide_b200.weights import BASELINE_DIMS as dims
    from oracle import gold_synth

    sd, model = cpu_gold_setup(dims, seed=1)
    cores = torch.get_num_threads()
    batch = synth_batch(dims, args.steps + args.warmup, TOKENS, seed=2, n_answers=ANSWERS, n_cand=CANDS, max_cand=CANDS)
    times = []
    for s in range(args.steps + args.warmup):
        one = type(batch)(batch.ids[s * TOKENS:(s + 1) * TOKENS], np.array([0, TOKENS], np.uint32),
                          batch.ans_rows[s * ANSWERS:(s + 1) * ANSWERS] - np.uint32(s * TOKENS), batch.cand[s * ANSWERS:(s + 1) * ANSWERS],
                          batch.ncand[s * ANSWERS:(s + 1) * ANSWERS])
        _, sec = gold_synth.gold_batch_logits(model, one, CANDS)
        if s >= args.warmup:
            times.append(sec)
    total = sum(times)
    value = TOKENS * len(times) / total
    sample = f"{len(times)} request(s) of {TOKENS} tokens, all 36 layers, fp32, torch {torch.__version__} CPU"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "step": "one 603-token request on the host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_engine(args):
    import torch
    import torch.distributed as dist

    from decide_b200 import check, dist as ddist
    from decide_b200.engine import Engine
    from decide_b200.kernels import Device
    from decide_b200.synth import synth_batch, synth_fused_on_device
    from decide_b200.weights import BASELINE_DIMS as dims, fuse_layer

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    if world > 1:   # a rank that fails must not leave the others waiting for the default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    dev = Device(local)
    cuda = torch.device("cuda", local)

    with_cpu = (world == 1 and rank == 0 and not args.no_cpu_baseline)
    cpu = None
    if with_cpu:
        t0 = time.perf_counter()
        sd, gold = cpu_gold_setup(dims, seed=1)
        fused = [{k: v.to(cuda) for k, v in fuse_layer(sd, l, dims).items()} for l in range(dims.n_layers)]
        embed, final_norm = sd["embed_tokens.weight"].to(cuda), sd["norm.weight"].to(cuda)
        cpu = {"setup_s": time.perf_counter() - t0}
    else:
        fused, embed, final_norm = synth_fused_on_device(dims, 1, cuda)   # the same weights on every rank
    rows = REQUESTS * TOKENS
    eng = Engine(dims, dev=dev, max_rows=rows, max_seqs=REQUESTS, max_answers=REQUESTS * ANSWERS, max_cand=CANDS,
                 fused_layers=fused, embed=embed, final_norm=final_norm)
    batch = synth_batch(dims, REQUESTS, TOKENS, seed=100 + rank, n_answers=ANSWERS, n_cand=CANDS, max_cand=CANDS)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        return ddist.max_over_ranks(ms, cuda)

    stream = torch.cuda.current_stream()
    # ---- warm-up (also fills the tensor-map cache and leaves the batch resident on the device)
    logits = None
    for _ in range(args.warmup):
        logits = eng.logits(batch)
    eng.profile()

    # ---- device-resident timing: the headline `value`
    sampler = ClockSampler(local)
    eng.set_profiling(True)
    barrier()
    sampler.start()
    launches0 = dev.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        eng.forward_resident(batch)
    e1.record(stream)
    barrier()
    launches = dev.launches - launches0
    ms_value = max_over_ranks(e0.elapsed_time(e1))
    prof = {name: (ms, calls) for name, ms, calls in eng.profile()}
    eng.set_profiling(False)

    # ---- end to end through the host-buffer call
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        logits = eng.logits(batch)
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    dev.check_status()
    rows_run_batch = eng.resident_rows

    # ---- single-request latency (p50 forward ms of the metric): one 2,307-token and one 603-token request,
    # host buffers in, logits out, 3 warm-up + 10 timed calls each; linear-interpolated median as the
    # reference's bench does (crates/decide-cli/src/bench.rs:103-112)
    latency = {}
    if rank == 0 and not args.no_latency:
        for toks, nans in ((2307, 3), (603, 6)):
            one = synth_batch(dims, 1, toks, seed=7, n_answers=nans, n_cand=CANDS, max_cand=CANDS)
            for _ in range(3):
                eng.logits(one)
            samples = []
            for _ in range(10):
                e0.record(stream)
                eng.logits(one)
                e1.record(stream)
                torch.cuda.synchronize()
                samples.append(e0.elapsed_time(e1))
            eng.profile()
            eng.set_profiling(True)     # one more, profiled run: where a single request's time goes (events around every op add a little)
            eng.logits(one)
            per_op = {name: round(ms, 4) for name, ms, _ in eng.profile()}
            eng.set_profiling(False)
            latency[f"tokens_{toks}"] = {"p50_ms": float(np.percentile(samples, 50)), "p95_ms": float(np.percentile(samples, 95)), "runs": len(samples),
                                         "rows_computed": eng.resident_rows, "per_op_ms": per_op}

        # follow-up questions about one state (the reference's follow-up demo, crates/decide-cli/src/race.rs:707-733, and
        # `decide bench`, bench.rs:224): a 2,491-token request cold from a 300-token prefix snapshot (the state cache
        # forgotten before every call, the new state captured inside it), then other questions about the same state, which
        # run only the 184 rows after it
        from decide_b200.synth import Batch
        rs = np.random.RandomState(11)
        marker = np.array([550, 39087, 10485, 198], np.uint32)        # the engine's default state marker
        prefix, state = rs.randint(0, dims.vocab, 300), rs.randint(0, dims.vocab, 2491 - 300 - 4 - 184)

        def ask(seed):
            q = np.random.RandomState(seed)
            ids = np.concatenate([prefix, state, marker, q.randint(0, dims.vocab, 184)]).astype(np.uint32)
            ans = np.array([len(ids) - o for o in (52, 33, 7)], np.uint32)
            cand = np.zeros((3, CANDS), np.uint32)
            for i in range(3):
                cand[i] = q.choice(dims.vocab, CANDS, replace=False)
            return Batch(ids, np.array([0, len(ids)], np.uint32), ans, cand, np.full(3, CANDS, np.uint32))

        def timed(req, forget):
            out = []
            for i in range(13):
                if forget:
                    eng.forget_states()
                e0.record(stream)
                got = eng.logits(req)
                e1.record(stream)
                torch.cuda.synchronize()
                if i >= 3:
                    out.append(e0.elapsed_time(e1))
            return got, {"p50_ms": float(np.percentile(out, 50)), "p95_ms": float(np.percentile(out, 95)), "runs": len(out),
                         "route": eng.last_route, "rows_computed": eng.resident_rows - eng.last_start}

        eng.build_snapshot(prefix)
        first, second = ask(1), ask(2)
        _, cold = timed(first, forget=True)
        cold_second, _ = timed(second, forget=True)
        eng.forget_states()
        eng.logits(first)                                   # leaves the state in the cache
        warm_second, follow = timed(second, forget=False)
        follow["max_abs_dlogit_vs_cold"] = float(np.abs(warm_second - cold_second).max())
        latency["follow_up"] = {"cold": cold, "follow_up": follow, "speedup_p50": cold["p50_ms"] / follow["p50_ms"]}
        eng.build_snapshot([])

    # ---- strong scaling (N > 1): the same 64 requests on every N, sharded by request; results checked across ranks
    strong = None
    if world > 1:
        whole = synth_batch(dims, REQUESTS, TOKENS, seed=100, n_answers=ANSWERS, n_cand=CANDS, max_cand=CANDS)
        mine = sub_batch(whole, ddist.shard(REQUESTS, world, rank))
        for _ in range(max(2, args.warmup)):
            local_logits = eng.logits(mine)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            eng.forward_resident(mine)
        e1.record(stream)
        barrier()
        ms_strong = max_over_ranks(e0.elapsed_time(e1))
        gathered = ddist.gather_rows(local_logits, cuda)
        if rank == 0:
            # rank 0 alone over the same shards, one after the other: same batches, same kernels, another GPU
            alone = np.concatenate([eng.logits(sub_batch(whole, ddist.shard(REQUESTS, world, r))) for r in range(world)], axis=0)
            together = eng.logits(whole)
            strong = {"tokens_per_s": REQUESTS * TOKENS * args.steps / (ms_strong / 1e3), "ms_per_step": ms_strong / args.steps,
                      "requests_per_gpu": REQUESTS // world, "rows_per_gpu": mine.rows,
                      "logits_bit_identical_to_one_gpu": bool(np.array_equal(gathered, alone)),
                      "max_abs_dlogit_vs_one_gpu": float(np.abs(gathered - alone).max()),
                      "max_abs_dlogit_vs_one_batch_of_64": float(np.abs(gathered - together).max()),
                      "note": "the one-GPU pass runs the same shard-sized batches; one batch of 64 differs in which rows fall into K-split tail tiles (fp32 summation order)"}
        barrier()

    tokens = world * rows * args.steps
    value = tokens / (ms_value / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    h2d = rows * 4 * 2 + (REQUESTS + 1) * 4 + REQUESTS * ANSWERS * 4 * 2 + REQUESTS * ANSWERS * CANDS * 4
    d2h = REQUESTS * ANSWERS * CANDS * 4

    peaks = measured_peaks()
    gu_ms, gu_calls = prof.get("gemm_gate_up", (0.0, 0))
    rows_run = rows_run_batch   # rows per step after tail truncation
    flops_per_launch = 2.0 * rows_run * (2 * dims.inter) * dims.hidden
    achieved = flops_per_launch / (gu_ms / gu_calls * 1e-3) / 1e12 if gu_calls else None
    gemm_ms = sum(ms for n, (ms, _) in prof.items() if n.startswith("gemm_"))
    gemm_tflops = dims.gemm_flops(rows_run, REQUESTS * ANSWERS, pruned=True) * args.steps / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None
    traffic = None
    tf = ROOT / "profiles" / "gemm_gate_up_traffic.json"
    if tf.exists():
        traffic = json.loads(tf.read_text()).get("dram_bytes_per_launch_at_bench_size")

    cpu_baseline = None
    if with_cpu and rank == 0:
        from oracle import gold_synth

        # the LAST request of the batch: its rows sit in the tiles of the GEMMs' partial last wave, which run K-split
        one = sub_batch(batch, range(REQUESTS - 1, REQUESTS))
        want, sec = gold_synth.gold_batch_logits(gold, one, CANDS)
        got = logits[-ANSWERS:]
        table = check.compare(got, want, one.ncand)
        cpu_baseline = {"value": TOKENS / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"1 request of {TOKENS} tokens (the last request of the batch), all 36 layers, fp32 CPU forward: {sec:.1f} s",
                        "parity_on_sample": {"max_abs_dlogit": table["max_dlogit"], "max_abs_dp": table["max_dp"],
                                             "decisions_agree": f"{table['agree']}/{table['fields']}", "near_tie_flips": len(table["small_flips"]),
                                             "failures": table["failures"]}}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_value / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16" if dev.act.name == "F16" else "bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests_per_gpu": REQUESTS, "tokens_per_request": TOKENS,
                       "work_skipping": f"as the reference: each request runs to its last answer row ({rows_run_batch} of {rows} rows per step, forward.rs:830-831) and the "
                                        "last layer runs q/attention/out-projection/MLP for the answer rows only (forward.rs:1150-1186); tokens/s counts the request's tokens",
                       "l2": "inputs larger than L2: 8.2 GB of weights stream through every step", "sharding": "by request, no collectives",
                       "sixteen_bit_type": "fp16 weights and activations, fp32 accumulate/residual/state (bf16 activations miss the 0.02 logit bar; DECIDE_ACT=bf16 selects them)"
                       if dev.act.name == "F16" else "bf16 weights and activations (misses the 0.02 logit bar over 36 layers)"},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"kernel": "gemm_tc_kernel<256, SwiGLU> (gate_up projection)", "bound": "tensor", "achieved": achieved,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"] if achieved else None,
                         "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)", "traffic": traffic,
                         "flops_per_launch": flops_per_launch, "launches_timed": gu_calls},
            "gemm_tflops_all_projections": gemm_tflops,
            "gemm_frac_of_peak": gemm_tflops / peaks["bf16_tflops_sustained"] if gemm_tflops else None,
            "per_op_ms_per_step": {n: ms / args.steps for n, (ms, _) in sorted(prof.items(), key=lambda kv: -kv[1][0])},
            "single_request_latency": latency,
            "strong_scaling": strong,
            "cpu_baseline": cpu_baseline,
        }))
    eng.close()
    if world > 1:
        dist.destroy_process_group()


def run_tp(args):
    """Latency mode of the benchmark's config: ONE 2,307-token request, tensor-parallel over all ranks of the launch
    (torch.distributed.run --nproc-per-node N bench.py --gpus N --tp). Prints its own JSON line: p50 / p95 of the forward
    from host ids to host logits (max over ranks), the share of the all-reduces, and the logits against rank 0's
    one-GPU engine on the same weights."""
    import torch
    import torch.distributed as dist

    from decide_b200 import dist as ddist
    from decide_b200.engine import Engine
    from decide_b200.kernels import Device
    from decide_b200.synth import synth_batch, synth_fused_on_device
    from decide_b200.weights import BASELINE_DIMS as dims, tp_shard_layer

    rank, local, world = ddist.env_rank()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    cuda = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=cuda, timeout=datetime.timedelta(seconds=180))
    uid = torch.zeros(128, dtype=torch.uint8, device=cuda)
    if rank == 0:
        uid = torch.frombuffer(bytearray(Device.tp_unique_id()), dtype=torch.uint8).to(cuda)
    if world > 1:
        dist.broadcast(uid, 0)
    dev = Device(local)
    dev.tp_init(bytes(uid.cpu().numpy().tobytes()), world, rank)
    whole, embed, final_norm = synth_fused_on_device(dims, 1, cuda)   # the same weights on every rank
    shard = [tp_shard_layer(whole[l], l, dims, world, rank) for l in range(dims.n_layers)] if world > 1 else whole
    toks, nans = 2307, 3
    one = synth_batch(dims, 1, toks, seed=7, n_answers=nans, n_cand=CANDS, max_cand=CANDS)
    eng = Engine(dims, dev=dev, max_rows=toks, max_seqs=1, max_answers=nans, max_cand=CANDS, fused_layers=shard, embed=embed, final_norm=final_norm)
    stream = torch.cuda.current_stream()
    for _ in range(max(3, args.warmup)):
        got = eng.logits(one)
    eng.profile()
    eng.set_profiling(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    samples = []
    runs = max(10, args.steps)
    for _ in range(runs):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record(stream)
        eng.logits(one)
        e1.record(stream)
        torch.cuda.synchronize()
        samples.append(ddist.max_over_ranks(e0.elapsed_time(e1), cuda))
    prof = {name: ms / runs for name, ms, _ in eng.profile()}
    eng.set_profiling(False)
    parity = None
    if rank == 0:
        ref_dev = Device(local)       # a second context on this GPU, outside the group: the one-GPU engine on the whole weights
        ref = Engine(dims, dev=ref_dev, max_rows=toks, max_seqs=1, max_answers=nans, max_cand=CANDS, fused_layers=whole, embed=embed, final_norm=final_norm)
        want = ref.logits(one)
        ref.close()
        parity = float(np.abs(got - want).max())
        print(json.dumps({
            "mode": "tensor-parallel single request", "tp": world, "tokens": toks, "runs": runs,
            "p50_ms": float(np.percentile(samples, 50)), "p95_ms": float(np.percentile(samples, 95)),
            "all_reduce_ms_per_forward": prof.get("all_reduce", 0.0), "per_op_ms": dict(sorted(prof.items(), key=lambda kv: -kv[1])),
            "max_abs_dlogit_vs_one_gpu": parity, "dtype": "f16" if dev.act.name == "F16" else "bf16",
            "exchange": "ncclAllReduce of the fp32 [rows, 2560] partial sums after each out / down projection (72 per forward)"}))
    eng.close()
    if world > 1:       # every rank leaves together; only then may rank 0 fail the run
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and parity > 0.02:
        raise SystemExit(f"tensor-parallel logits differ from the one-GPU engine by {parity}")


def cpu_config_seconds(cfg: int, gated: bool, repeats: int) -> tuple[float, int]:
    """The same op sequence as decide_b200.bench_ops.config_case(cfg) in fp32 on the host cores with torch (the arithmetic
    the reference's CPU gold path runs: F.linear in fp32, torch SDPA, the transformers chunk-64 delta rule). Best of `repeats`."""
    import math

    import torch
    import torch.nn.functional as F

    torch.set_num_threads(os.cpu_count() or 1)
    H, I, nq, nkv, hd, nk, nv = 2560, 9728, 32, 8, 128, 16, 16
    m = {0: 276, 1: 603, 2: 2307, 3: 2307}[cfg]
    g = torch.Generator().manual_seed(cfg)
    rn = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    x, nw = rn(m, H), rn(H, std=0.02)
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + w)
    if cfg in (0, 1):
        w_g, w_u, w_d = rn(I, H, std=0.02), rn(I, H, std=0.02), rn(H, I, std=0.02)
        if cfg == 0:
            fn = lambda: F.silu(F.linear(x, w_g)) * F.linear(x, w_u)
        else:
            def fn():
                h = rms(x, nw)
                return x + F.linear(F.silu(F.linear(h, w_g)) * F.linear(h, w_u), w_d)
    elif cfg == 2:
        qd, kvd = nq * hd, nkv * hd
        w_in, w_o = rn((2 if gated else 1) * qd + 2 * kvd, H, std=0.02), rn(H, qd, std=0.02)
        qw, kw = rn(hd, std=0.02), rn(hd, std=0.02)
        ang = torch.arange(m, dtype=torch.float32)[:, None] * torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)])
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
        rot = lambda t: t * cos + torch.cat([-t[..., hd // 2:], t[..., :hd // 2]], -1) * sin

        def fn():
            p = F.linear(rms(x, nw), w_in)
            q = rot(rms(p[:, :qd].view(m, nq, hd), qw)).transpose(0, 1)[None]
            kcol = (2 if gated else 1) * qd
            kk = rot(rms(p[:, kcol:kcol + kvd].view(m, nkv, hd), kw)).transpose(0, 1)[None]
            v = p[:, kcol + kvd:].view(m, nkv, hd).transpose(0, 1)[None]
            y = F.scaled_dot_product_attention(q, kk, v, is_causal=True, enable_gqa=True)[0].transpose(0, 1).reshape(m, qd)
            if gated:
                y = y * torch.sigmoid(p[:, qd:2 * qd])
            return x + F.linear(y, w_o)
    else:
        from transformers.models.qwen3_5.modeling_qwen3_5 import torch_chunk_gated_delta_rule

        conv_dim, vd = (2 * nk + nv) * 128, nv * 128
        w_in, w_out, cw = rn(conv_dim + vd + 2 * nv, H, std=0.02), rn(H, vd, std=0.02), rn(conv_dim, 1, 4, std=0.3)
        a_log, dt, gw = torch.rand(nv, generator=g) * math.log(16.0), torch.ones(nv), torch.ones(128)

        def fn():
            p = F.linear(rms(x, nw), w_in)
            qkv = F.silu(F.conv1d(p[:, :conv_dim].t()[None], cw, padding=3, groups=conv_dim)[0, :, :m]).t()
            q, kk, v = qkv[:, :nk * 128].view(1, m, nk, 128), qkv[:, nk * 128:2 * nk * 128].view(1, m, nk, 128), qkv[:, 2 * nk * 128:].view(1, m, nv, 128)
            beta = torch.sigmoid(p[:, conv_dim + vd:conv_dim + vd + nv])[None]
            gdecay = (-a_log.exp() * F.softplus(p[:, conv_dim + vd + nv:] + dt))[None]
            o, _ = torch_chunk_gated_delta_rule(q, kk, v, g=gdecay, beta=beta, initial_state=None, output_final_state=False, use_qk_l2norm_in_kernel=True)
            o = o[0]
            z = p[:, conv_dim:conv_dim + vd].view(m, nv, 128)
            gg = (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * gw * F.silu(z)).reshape(m, vd)
            return x + F.linear(gg, w_out)
    best = float("inf")
    with torch.inference_mode():
        fn()
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()


def run_config(args):
    """`--config k`: one of the benchmark's single-block configs (0: gate_up GEMM at M = 276; 1: MLP block at M = 603; 2: attention layer
    at M = 2,307, gated and un-gated; 3: Gated DeltaNet layer at M = 2,307), one JSON line each: GPU microseconds, TFLOP/s and the fraction
    of the measured burst peak, beside the fp32 CPU time of the same op sequence."""
    from decide_b200 import bench_ops
    from decide_b200.kernels import Device, Kernels

    dev = Device(0)
    k = Kernels(dev)
    peaks = measured_peaks()
    for gated in ((True, False) if args.config == 2 else (True,)):
        r = bench_ops.config_case(k, args.config, iters=max(args.steps, 10), warmup=max(args.warmup, 3), gated=gated)
        sec, cores = cpu_config_seconds(args.config, gated, repeats=3)
        print(json.dumps({
            "metric": "block_forward_us", "value": r["us"], "unit": "us", "n_gpus": 1, "higher_is_better": False, "dtype": "f16" if dev.act.name == "F16" else "bf16",
            "data": "synthetic", "config": {"workload": f"configs[{args.config}]: {r['what']}, M = {r['rows']}"},
            "roofline": {"bound": "tensor", "achieved": r["tflops"], "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": r["tflops"] / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['source']} (burst cuBLAS bf16; the sequence is timed alone)", "flops_per_pass": r["flops"],
                         "note": "whole op sequence (norms, RoPE, attention / delta rule included) against the GEMM peak"},
            "cpu_baseline": {"value": sec * 1e6, "unit": "us", "cores": cores, "kind": "port", "sample": "the same op sequence in fp32 with torch on the host cores, best of 3"},
            "speedup_vs_cpu": sec * 1e6 / r["us"]}))
    dev.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["engine", "reference"], default="engine")
    ap.add_argument("--no-latency", action="store_true", help="skip the single-request latency runs (for short profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU forward (weights are then drawn on the GPU)")
    ap.add_argument("--config", type=int, choices=[0, 1, 2, 3], default=None, help="measure one of the single-block configs instead of the full model")
    ap.add_argument("--tp", action="store_true", help="latency mode: one 2,307-token request, tensor-parallel over all ranks of the launch")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config is not None:
        run_config(args)
    elif args.tp:
        run_tp(args)
    else:
        run_engine(args)


if __name__ == "__main__":
    main()
