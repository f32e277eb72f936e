#!/usr/bin/env python
"""Encoder throughput benchmark (tokens/s) of the B200 block-sparse encoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload base|large|band]

Workload at any N: the full 12-layer BigBird-base encoder (embeddings included), fp16,
on a padding-free varlen batch of 8*N sequences with lengths uniform over multiples of 64
in [1024, 4096] and token ids uniform in [5, 50358) (seed 0), weights ~N(0, 0.02) (seed 0).
For N > 1 whole sequences are bin-packed over the ranks (weak scaling: 8 sequences per
GPU on average) and the final hidden states are all-gathered inside the timed step.

One step = per-batch metadata (block tables, work lists, varlen offsets) + embeddings +
12 layers.  `value` is timed with CUDA events with the token ids already in HBM; `e2e`
runs the same step through the host-buffer entry point (H2D of ids and tables, D2H of the
hidden states inside the timed region).  The L2 is flushed between timed steps.

--impl reference times the CPU restatement of the reference's validation model (the
oracle) on the host cores, one short sequence of the same workload per step.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (hidden, heads, ffn, layers, max_pos, dtype, pattern, seqs_per_gpu, min_blocks, max_blocks)
    "base": dict(hidden=768, heads=12, ffn=3072, layers=12, max_pos=4096, dtype="f16", pattern="bigbird",
                 seqs=8, lo=16, hi=64, desc="BigBird-base 12L fp16, 8 seqs/GPU, len U[1024,4096] step 64"),
    "band": dict(hidden=768, heads=12, ffn=3072, layers=12, max_pos=4096, dtype="bf16", pattern="band",
                 seqs=16, lo=8, hi=64, desc="Longformer-shaped band 12L bf16, 16 seqs/GPU, len U[512,4096] step 64"),
    "large": dict(hidden=1024, heads=16, ffn=4096, layers=24, max_pos=8192, dtype="bf16", pattern="bigbird",
                  seqs=32, lo=8, hi=128, desc="BigBird-large 24L bf16, 32 seqs/GPU, lognormal lengths"),
}
VOCAB, TYPE_VOCAB = 50358, 2


def make_lengths(w, n_seq, seed=0):
    rng = np.random.default_rng(seed)
    if w is WORKLOADS["large"]:
        raw = np.clip(rng.lognormal(np.log(2048), 0.6, size=n_seq), 512, 8192)
        lens = (np.ceil(raw / 64) * 64).astype(np.int64)
    else:
        lens = 64 * rng.integers(w["lo"], w["hi"] + 1, size=n_seq)
    lens[lens == 768] = 832  # 12 blocks: the reference's validation model cannot run this length
    ids = [rng.integers(5, VOCAB, size=int(n)).astype(np.int32) for n in lens]
    return [int(n) for n in lens], ids


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU on a background thread (NVML reads
    only, every 5 ms) while the timed loops run."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index):
        import threading
        self.sm, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and visible.split(",")[gpu_index].isdigit() else gpu_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            return
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def stop(self):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._stop.set()
        self.t.join(2)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


def ncu_traffic(kernel, units_here):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary
    (profiles/ncu_<kernel>_microbench.md: dram__bytes_read.sum + dram__bytes_write.sum of one captured
    launch), scaled to this run's launch by the algorithmic work ratio.  None when no summary exists."""
    import re
    path = os.path.join(ROOT, "profiles", f"ncu_{kernel}_microbench.md")
    ref_units = {"gemm": 2.0 * 16384 * 3072 * 768, "attention": 1048576.0 * 59712}[kernel]
    try:
        text = open(path).read()
        vals = []
        for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            m = re.search(r"`" + re.escape(key) + r"`\) \| ([0-9.]+) \| (\w+)", text)
            scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}[m.group(2)]
            vals.append(float(m.group(1)) * scale)
        return sum(vals) * units_here / ref_units
    except Exception:
        return None


def flops_per_step(w, lens, visits_per_head):
    T = sum(lens)
    gemm = w["layers"] * T * (8 * w["hidden"] ** 2 + 4 * w["hidden"] * w["ffn"])
    attn = w["layers"] * w["heads"] * 1048576 * visits_per_head
    return gemm, attn


# ------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the oracle on the host cores
# ------------------------------------------------------------------------------------------
def cpu_oracle_tokens_per_s(w, seq_ids, steps, warmup, threads):
    import oracle  # test infrastructure: used here only as the timed CPU baseline
    torch.set_num_threads(threads)
    cfg = oracle.EncoderConfig(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                               max_pos=w["max_pos"], vocab=VOCAB, type_vocab=TYPE_VOCAB, pattern=w["pattern"])
    P = oracle.make_weights(cfg, seed=0)
    seqs = [torch.from_numpy(s) for s in seq_ids]
    toks = sum(len(s) for s in seq_ids)
    for _ in range(warmup):
        oracle.encoder_ref(seqs, P, cfg)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.encoder_ref(seqs, P, cfg)
    dt = time.perf_counter() - t0
    return toks * steps / dt, dt / steps * 1e3


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lens, ids = make_lengths(w, w["seqs"] * args.gpus)
    i = int(np.argmin(lens))
    threads = os.cpu_count() or 1
    tps, ms = cpu_oracle_tokens_per_s(w, [ids[i]], args.steps, min(args.warmup, 1), threads)
    sample = f"sequence {i} of the workload ({lens[i]} tokens), all layers, fp32, per step"
    print(json.dumps({
        "impl": "reference", "metric": "encoder_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"]},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu(args, w):
    import torch.distributed as dist
    from raptor_t_b200 import capi, metadata, parallel
    from raptor_t_b200.engine import Encoder, kernel_launches
    from raptor_t_b200.weights import synthetic_weights

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n_gpus = world

    cfg = capi.make_config(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                           max_pos=w["max_pos"], vocab=VOCAB, type_vocab=TYPE_VOCAB, pattern=w["pattern"],
                           dtype=w["dtype"])
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    P = synthetic_weights(w["hidden"], w["ffn"], w["layers"], VOCAB, w["max_pos"], TYPE_VOCAB, seed=0)
    enc = Encoder(cfg).load_weights(P)
    del P

    lens_all, ids_all = make_lengths(w, w["seqs"] * n_gpus)
    assignment = parallel.partition_batch(cfg, lens_all, n_gpus) if n_gpus > 1 else [list(range(len(lens_all)))]
    mine = assignment[rank]
    lens = [lens_all[i] for i in mine]
    ids_np = np.concatenate([ids_all[i] for i in mine])
    T_local, T_total = int(sum(lens)), int(sum(lens_all))
    ids_dev = torch.from_numpy(ids_np).cuda()
    ids_pinned = torch.from_numpy(ids_np).pin_memory()
    out_dev = torch.empty(T_local, w["hidden"], dtype=dtype, device="cuda")
    out_pinned = torch.empty(T_local, w["hidden"], dtype=dtype).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB L2

    # N > 1: the all_gather of step i runs on a side stream under the kernels of the next two
    # steps (three output buffers rotate), so that the ranks are coupled loosely: a step's timed
    # window ends after the gather issued two steps earlier has finished, and the tail of the
    # last gathers is added to the total.
    DEPTH = 3
    gatherer = (parallel.OutputGatherer(assignment, lens_all, w["hidden"], dtype, "cuda", depth=DEPTH)
                if n_gpus > 1 else None)
    out_devs = [out_dev] + [torch.empty_like(out_dev) for _ in range(DEPTH - 1)]
    pipe = {"i": 0, "pending": []}

    def step():
        k = pipe["i"] % DEPTH
        pipe["i"] += 1
        enc.prepare(lens)
        enc.forward_ids(ids_dev, out=out_devs[k])
        if gatherer is not None:
            pipe["pending"].append(gatherer.start(out_devs[k]))
            if len(pipe["pending"]) >= DEPTH:
                gatherer.finish(pipe["pending"].pop(0))
        return out_devs[k]

    def drain():
        while gatherer is not None and pipe["pending"]:
            gatherer.finish(pipe["pending"].pop(0))

    def barrier():
        drain()
        torch.cuda.synchronize()
        if n_gpus > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------
    # Pass 1 (the reported value): no events between the kernels of a step, so that dependent
    # launches overlap (programmatic dependent launch).  Pass 2: the same K steps with CUDA
    # events around every launch for the per-kernel durations of the roofline; those events
    # serialise the launches and make a step ~15 % slower, which is why the value is not
    # taken from that pass.
    enc.enable_timing(False)
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = kernel_launches()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    host_t0 = time.perf_counter()
    for a, b in ev:
        flush.fill_(1)
        a.record()
        step()
        b.record()
    host_ms_per_step = (time.perf_counter() - host_t0) * 1e3 / args.steps  # launch time only: nothing waits here
    tail = torch.cuda.Event(enable_timing=True)
    drain()
    tail.record()
    barrier()
    launches = kernel_launches() - launches0
    t_ms = sum(a.elapsed_time(b) for a, b in ev) + ev[-1][1].elapsed_time(tail)
    t = torch.tensor([t_ms], dtype=torch.float64, device="cuda")
    if n_gpus > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    value = T_total / (ms_per_step * 1e-3)

    enc.enable_timing(True)
    stage_ms = {}
    step()
    for _ in range(args.steps):
        flush.fill_(1)
        step()
        for k, v in enc.timing().items():  # synchronises
            stage_ms[k] = stage_ms.get(k, 0.0) + v
    barrier()
    enc.enable_timing(False)

    # ---- end to end through the host-buffer entry points --------------------------------
    # Every step copies its token ids from pinned host memory and its hidden states back to
    # pinned host memory inside the timed region.  Throughput figure: two batches in flight
    # (submit_host / wait_host; the D2H of one step overlaps the kernels of the next, each step
    # with its own pair of host buffers).  Latency figure: one batch at a time (forward_host).
    ids_pin = [ids_pinned, ids_pinned.clone().pin_memory()]
    out_pin = [out_pinned, torch.empty_like(out_pinned).pin_memory()]
    for _ in range(min(args.warmup, 3)):
        enc.forward_host(lens, ids_pinned, out_pinned)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        enc.forward_host(lens, ids_pinned, out_pinned)
    torch.cuda.synchronize()
    e2e_sync_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    barrier()
    t0 = time.perf_counter()
    pending = None
    for i in range(args.steps):
        ticket = enc.submit_host(lens, ids_pin[i & 1], out_pin[i & 1])
        if pending is not None:
            enc.wait_host(pending)
        pending = ticket
    enc.wait_host(pending)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([e2e_ms], dtype=torch.float64, device="cuda")
    if n_gpus > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = t.item() / args.steps
    e2e_value = T_total / (e2e_ms_per_step * 1e-3)
    clocks = sampler.stop() if sampler else None
    stats = enc.plan_stats(0)
    visits_local = stats["visits"] // w["heads"]
    meta_bytes = w["layers"] * (stats["items"] * 32 + stats["entries"] * 4 + 297 * 4) + (len(lens) + 1) * 4
    h2d = T_local * 4 + meta_bytes
    d2h = T_local * w["hidden"] * 2

    if rank != 0:
        if n_gpus > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (this rank's share) ----------------------------
    pk = peaks()
    gemm_fl, attn_fl = flops_per_step(w, lens, visits_local)
    per = {k: v / args.steps for k, v in stage_ms.items()}
    n_gemm = 4 * w["layers"]
    gemm_ms, attn_ms = per.get("gemm", 0.0), per.get("attention", 0.0)
    ln_ms, tr_ms = per.get("add_bias_and_layernorm_kernel", 0.0), per.get("add_bias_and_transpose_kernel", 0.0)
    gemm_tf = gemm_fl / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    attn_tf = attn_fl / (attn_ms * 1e-3) / 1e12 if attn_ms else 0.0
    ln_gbs = (2 * w["layers"] * 3 * T_local * w["hidden"] * 2) / (ln_ms * 1e-3) / 1e9 if ln_ms else 0.0
    tr_gbs = (w["layers"] * 2 * T_local * 3 * w["hidden"] * 2) / (tr_ms * 1e-3) / 1e9 if tr_ms else 0.0
    dominant_is_gemm = gemm_ms >= attn_ms
    if dominant_is_gemm:
        roof = {"kernel": "gemm_pair_kernel (CTA-pair tcgen05 projection GEMMs, 4 per layer)", "bound": "tensor",
                "achieved": gemm_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                "frac": gemm_tf / pk["tf_sustained"], "traffic": ncu_traffic("gemm", gemm_fl / n_gemm),
                "launches_per_step": n_gemm, "avg_launch_ms": gemm_ms / n_gemm,
                "flops_per_launch": gemm_fl / n_gemm}
    else:
        roof = {"kernel": "sparse_attention_kernel (tcgen05 block-sparse attention, 1 per layer)", "bound": "tensor",
                "achieved": attn_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                "frac": attn_tf / pk["tf_sustained"], "traffic": ncu_traffic("attention", attn_fl / w["layers"]),
                "launches_per_step": w["layers"], "avg_launch_ms": attn_ms / w["layers"],
                "flops_per_launch": attn_fl / w["layers"]}
    roof["peak_source"] = pk["source"] + " (sustained bf16 dense, kernel timed inside a long step)"
    roof["traffic_source"] = ("ncu capture of the same kernel on the micro-benchmark shape (profiles/), "
                              "scaled by algorithmic work per launch")

    # ---- CPU baseline: oracle on a bounded sample of the same workload -----------------------
    cpu = None
    if n_gpus == 1 and not args.no_cpu_baseline:
        i = int(np.argmin(lens_all))
        threads = os.cpu_count() or 1
        tps, ms = cpu_oracle_tokens_per_s(w, [ids_all[i]], 2, 1, threads)
        cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"sequence {i} of the batch ({lens_all[i]} tokens), all {w['layers']} layers, fp32, "
                         f"2 timed runs after 1 warm-up ({ms:.0f} ms each)"}

    print(json.dumps({
        "metric": "encoder_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["desc"], "sequences": len(lens_all), "tokens": T_total,
                   "l2": "flushed between timed steps (256 MiB write)",
                   "stage_timing": "per-kernel durations (roofline, stages_ms_per_step) come from a second pass of the "
                                   "same steps with CUDA events around every launch",
                   "parallelism": f"replicas x{n_gpus}, whole-sequence bin packing, all_gather of outputs timed (the gather of "
                                  f"step i overlaps the kernels of steps i+1 and i+2; the last gathers' tail is added)"
                   if n_gpus > 1 else "single GPU"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms_per_step, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
                "mode": "submit_host/wait_host, two batches in flight, pinned host buffers; every step's H2D and "
                        "D2H copies are inside the timed region",
                "one_batch_at_a_time_ms_per_step": e2e_sync_ms},
        "gpu_launches": int(launches),
        "host_launch_ms_per_step": host_ms_per_step,
        "clocks": clocks,
        "roofline": roof,
        "stages_ms_per_step": per,
        "rooflines_other": {
            "attention_tflops": attn_tf, "attention_frac_of_tensor_peak": attn_tf / pk["tf_sustained"],
            "gemm_tflops": gemm_tf,
            "layernorm_gbs": ln_gbs, "layernorm_frac_of_hbm": ln_gbs / pk["hbm"],
            "qkv_transpose_gbs": tr_gbs, "qkv_transpose_frac_of_hbm": tr_gbs / pk["hbm"],
        },
        "cpu_baseline": cpu,
    }))
    if n_gpus > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="base", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--seqs", type=int, default=0, help="sequences per GPU (default: the workload's own count)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    if args.seqs > 0:
        w["seqs"] = args.seqs
        w["desc"] += f" (--seqs {args.seqs})"
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_gpu(args, w)


if __name__ == "__main__":
    main()
