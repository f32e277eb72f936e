#!/usr/bin/env python
"""Encoder throughput benchmark (tokens/s) of the B200 block-sparse encoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload base|large|band]

Workload at any N: the full 12-layer BigBird-base encoder (embeddings included), fp16,
on padding-free varlen batches of 8*N sequences with lengths uniform over multiples of 64
in [1024, 4096] and token ids uniform in [5, 50358), weights ~N(0, 0.02) (seed 0).  Four
different batches (seeds 0..3; seed 0 is the configuration the metric is quoted on) rotate
through the timed steps, so that per-batch metadata is really rebuilt every step.
For N > 1 whole sequences are bin-packed over the ranks (weak scaling: 8 sequences per
GPU on average) and the final hidden states are gathered to rank 0 inside the timed step.

One step = per-batch metadata (block tables, work lists, varlen offsets) + embeddings +
12 layers (+ the gather).  `value` is timed with CUDA events with the token ids already in HBM;
`e2e` copies every step's ids from pinned host memory and its hidden states back to pinned
host memory inside the timed region (at N > 1: the gathered tensor, on rank 0).  The L2 is
flushed between timed steps.

--impl reference times the reference's own validation module (oracle/_ref, when a reference
checkout was present at build time; else the CPU restatement in oracle/) on the host cores,
on the whole seed-0 batch per step.
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


N_ROTATE = 4  # different batches that rotate through the timed steps


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
# reference arm / cpu baseline: the reference's validation model on the host cores
# ------------------------------------------------------------------------------------------
def cpu_encoder(w):
    """-> (forward(list of id tensors) -> hidden states, kind): the reference's own module when
    oracle/_ref holds it (BigBird pattern only), else the restatement in oracle/bigbird.py."""
    import oracle  # test infrastructure: used here only as the timed CPU baseline
    cfg = oracle.EncoderConfig(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                               max_pos=w["max_pos"], vocab=VOCAB, type_vocab=TYPE_VOCAB, pattern=w["pattern"])
    P = oracle.make_weights(cfg, seed=0)
    from oracle import ref_runner
    if ref_runner.available() and w["pattern"] == "bigbird":
        try:
            enc = ref_runner.ReferenceEncoder(cfg, P)
            return (lambda seqs: enc.forward(seqs)), "reference"
        except Exception as exc:  # an incompatible transformers install: fall back to the restatement
            sys.stderr.write(f"bench.py: reference module unusable ({exc}); timing the restatement\n")
    return (lambda seqs: oracle.encoder_ref(seqs, P, cfg)), "port"


def cpu_tokens_per_s(w, seq_ids, steps, warmup_ids, threads):
    torch.set_num_threads(threads)
    fwd, kind = cpu_encoder(w)
    seqs = [torch.from_numpy(s) for s in seq_ids]
    toks = sum(len(s) for s in seq_ids)
    if warmup_ids is not None:
        fwd([torch.from_numpy(warmup_ids)])
    t0 = time.perf_counter()
    for _ in range(steps):
        fwd(seqs)
    dt = time.perf_counter() - t0
    return toks * steps / dt, dt / steps * 1e3, kind


MAX_CPU_STEPS = 3  # the CPU arm needs seconds per step: its step count is capped


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the sequences one GPU gets at N = 1: the whole seed-0 batch of the workload
    lens, ids = make_lengths(w, w["seqs"], seed=0)
    threads = os.cpu_count() or 1
    steps = max(1, min(args.steps, MAX_CPU_STEPS))
    warm = ids[int(np.argmin(lens))] if args.warmup > 0 else None
    tps, ms, kind = cpu_tokens_per_s(w, ids, steps, warm, threads)
    sample = (f"whole seed-0 batch ({len(lens)} sequences, {sum(lens)} tokens), all {w['layers']} layers, fp32, per step; "
              f"{steps} timed step(s) (capped at {MAX_CPU_STEPS})"
              + (" after a warm-up on its shortest sequence" if warm is not None else ", no warm-up"))
    print(json.dumps({
        "impl": "reference", "metric": "encoder_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": 1 if warm is not None else 0, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "sequences": len(lens), "tokens": int(sum(lens))},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class Batch:
    """One global batch and this rank's share of it."""

    def __init__(self, w, cfg, n_gpus, rank, seed, dtype):
        from raptor_t_b200 import parallel
        self.lens_all, ids_all = make_lengths(w, w["seqs"] * n_gpus, seed=seed)
        self.assignment = (parallel.partition_batch(cfg, self.lens_all, n_gpus) if n_gpus > 1
                           else [list(range(len(self.lens_all)))])
        mine = self.assignment[rank]
        self.lens = [self.lens_all[i] for i in mine]
        ids_np = np.concatenate([ids_all[i] for i in mine])
        self.ids_all = ids_all
        self.T_local, self.T_total = int(sum(self.lens)), int(sum(self.lens_all))
        self.ids_dev = torch.from_numpy(ids_np).cuda()
        self.ids_pinned = torch.from_numpy(ids_np).pin_memory()
        self.gatherer = (parallel.make_root_gatherer(self.assignment, self.lens_all, w["hidden"], dtype, "cuda", depth=DEPTH,
                                                     kind=w.get("gather"))
                         if n_gpus > 1 else None)


DEPTH = 3  # output buffers in rotation: the gather of step i runs under the kernels of steps i+1 and i+2


def run_gpu(args, w):
    import torch.distributed as dist
    from raptor_t_b200 import capi
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

    batches = [Batch(w, cfg, n_gpus, rank, seed, dtype) for seed in range(N_ROTATE)]
    T_max = max(b.T_local for b in batches)
    out_devs = [torch.empty(T_max, w["hidden"], dtype=dtype, device="cuda") for _ in range(DEPTH)]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB L2
    pipe = {"i": 0, "pending": [], "host_ms": 0.0}

    # N > 1: the gather of step i (grouped send/recv to rank 0) runs on a side stream under the
    # kernels of the next two steps, so that the ranks are coupled loosely: a step's timed window
    # ends after the gather issued two steps earlier has finished, and the tail of the last
    # gathers is added to the total.
    def step(h2d=False, d2h=None):
        i = pipe["i"]
        pipe["i"] += 1
        b, k = batches[i % N_ROTATE], i % DEPTH
        if h2d:
            b.ids_dev.copy_(b.ids_pinned, non_blocking=True)
        out = out_devs[k][: b.T_local]
        # host work of the step: metadata hand-off + ~90 kernel launches, without the time the thread sits
        # waiting for the GPU to release a metadata slot (it runs ahead of the GPU until the slots are used up)
        t0, blocked0 = time.perf_counter(), enc.host_blocked_ms()
        enc.prepare(b.lens)
        enc.forward_ids(b.ids_dev, out=out)
        pipe["host_ms"] += (time.perf_counter() - t0) * 1e3 - (enc.host_blocked_ms() - blocked0)
        if b.gatherer is not None:
            # d2h (rank 0 only): the gathered batch also goes to pinned host memory, on the gather's stream
            pipe["pending"].append((b, b.gatherer.start(out, host_out=d2h)))
            if len(pipe["pending"]) >= DEPTH:
                finish_one()
        return b

    def finish_one():
        b, ticket = pipe["pending"].pop(0)
        b.gatherer.finish(ticket)

    def drain():
        while pipe["pending"]:
            finish_one()

    def barrier():
        drain()
        torch.cuda.synchronize()
        if n_gpus > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        if n_gpus > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-resident timing ------------------------------------------------------
    # Pass 1 (the reported value): no events between the kernels of a step, so that dependent
    # launches overlap (programmatic dependent launch).  Pass 2: the same K steps with CUDA
    # events around every launch for the per-kernel durations of the roofline; those events
    # serialise the launches and make a step ~15 % slower, which is why the value is not
    # taken from that pass.
    warmup = max(args.warmup, N_ROTATE)  # every rotating batch is seen once before the clock starts
    enc.enable_timing(False)
    pipe["i"] = 0
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = kernel_launches()
    pipe["host_ms"] = 0.0
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    pipe["i"] = 0
    tokens_timed = 0
    for a, b in ev:
        flush.fill_(1)
        a.record()
        tokens_timed += step().T_total
        b.record()
    host_ms_per_step = pipe["host_ms"] / args.steps
    tail = torch.cuda.Event(enable_timing=True)
    drain()
    tail.record()
    barrier()
    launches = kernel_launches() - launches0
    t_ms_local = sum(a.elapsed_time(b) for a, b in ev) + ev[-1][1].elapsed_time(tail)
    rank_ms = torch.tensor([t_ms_local / args.steps], dtype=torch.float64, device="cuda")
    if n_gpus > 1:
        all_ms = [torch.zeros_like(rank_ms) for _ in range(n_gpus)]
        dist.all_gather(all_ms, rank_ms)
        per_rank_ms = [float(t.item()) for t in all_ms]
    else:
        per_rank_ms = [float(rank_ms.item())]
    ms_per_step = max(per_rank_ms)
    value = tokens_timed / args.steps / (ms_per_step * 1e-3)

    enc.enable_timing(True)
    stage_ms = {}
    pipe["i"] = 0
    stage_flops = [0.0, 0.0]
    stage_tokens = 0
    ln_in_ao, ln_in_down = enc.layernorm_in_projection()
    for i in range(args.steps):
        flush.fill_(1)
        b = step()
        for k, v in enc.timing().items():  # synchronises
            stage_ms[k] = stage_ms.get(k, 0.0) + v
        st = enc.plan_stats(0)
        g, a = flops_per_step(w, b.lens, st["visits"] // w["heads"])
        stage_flops[0] += g
        stage_flops[1] += a
        stage_tokens += b.T_local
    barrier()
    enc.enable_timing(False)

    # ---- end to end: host buffers in, host buffers out ---------------------------------
    # Every step copies its token ids from pinned host memory and its hidden states back to
    # pinned host memory inside the timed region.  N = 1: the library's host-buffer entry points
    # (submit_host / wait_host, two batches in flight: the D2H of one step overlaps the kernels of
    # the next; forward_host for the one-batch-at-a-time latency).  N > 1: per rank H2D of its ids,
    # forward, gather to rank 0, and on rank 0 the D2H of the whole gathered batch.
    e2e_sync_ms = None
    if n_gpus == 1:
        outs_pin = [torch.empty(T_max, w["hidden"], dtype=dtype).pin_memory() for _ in range(2)]
        for i in range(N_ROTATE):
            b = batches[i]
            enc.forward_host(b.lens, b.ids_pinned, outs_pin[0][: b.T_local])
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            b = batches[i % N_ROTATE]
            enc.forward_host(b.lens, b.ids_pinned, outs_pin[0][: b.T_local])
        torch.cuda.synchronize()
        e2e_sync_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        barrier()
        t0 = time.perf_counter()
        pending = None
        for i in range(args.steps):
            b = batches[i % N_ROTATE]
            ticket = enc.submit_host(b.lens, b.ids_pinned, outs_pin[i & 1][: b.T_local])
            if pending is not None:
                enc.wait_host(pending)
            pending = ticket
        enc.wait_host(pending)
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        d2h = float(np.mean([batches[i % N_ROTATE].T_local for i in range(args.steps)])) * w["hidden"] * 2
        e2e_mode = ("submit_host/wait_host, two batches in flight, pinned host buffers; every step's H2D and D2H "
                    "copies are inside the timed region")
    else:
        T_tot_max = max(b.T_total for b in batches)
        # non-root ranks take part in the gather and copy nothing back
        host_out = torch.empty(T_tot_max, w["hidden"], dtype=dtype).pin_memory() if rank == 0 else None
        pipe["i"] = 0
        for _ in range(N_ROTATE):
            step(h2d=True, d2h=host_out)
        barrier()
        pipe["i"] = 0
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step(h2d=True, d2h=host_out)
        drain()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        d2h = float(np.mean([batches[i % N_ROTATE].T_total for i in range(args.steps)])) * w["hidden"] * 2
        e2e_mode = ("per rank: H2D of its ids from pinned memory, forward, gather to rank 0 (grouped send/recv under "
                    "the next steps' kernels); rank 0: D2H of the whole gathered batch to pinned memory; all inside the "
                    "timed region")
    e2e_ms_per_step = max_over_ranks(e2e_ms) / args.steps
    e2e_value = tokens_timed / args.steps / (e2e_ms_per_step * 1e-3)
    clocks = sampler.stop() if sampler else None
    stats = enc.plan_stats(0)
    meta_bytes = w["layers"] * (stats["items"] * 32 + stats["entries"] * 4 + 297 * 4) + (len(batches[0].lens) + 1) * 4
    h2d = batches[0].T_local * 4 + meta_bytes

    if rank != 0:
        if n_gpus > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (this rank's share, summed over the timed steps) --------
    # gemm_pair_kernel = the projections whose span holds nothing but the GEMM and its bias / GELU / QKV
    # epilogue; a projection that carries its LayerNorm (gemm_ln_kernel) is reported beside it, because its
    # span also contains the LayerNorm's work, which is not counted as FLOPs.
    pk = peaks()
    H, F, L = w["hidden"], w["ffn"], w["layers"]
    fl = {"gemm.qkv": 2.0 * H * 3 * H, "gemm.attention_output": 2.0 * H * H, "gemm.ffn_up": 2.0 * H * F,
          "gemm.ffn_down": 2.0 * F * H}
    fl = {k: v * L * stage_tokens for k, v in fl.items()}
    fused_keys = [k for k, on in (("gemm.attention_output", ln_in_ao), ("gemm.ffn_down", ln_in_down)) if on]
    pair_keys = [k for k in fl if k not in fused_keys]
    gemm_fl, attn_fl = sum(fl[k] for k in pair_keys), stage_flops[1]
    gemm_ms = sum(stage_ms.get(k, 0.0) for k in pair_keys)
    n_gemm = len(pair_keys) * L * args.steps
    n_attn = L * args.steps
    attn_ms = stage_ms.get("attention", 0.0)
    ln_ms, tr_ms = stage_ms.get("add_bias_and_layernorm_kernel", 0.0), stage_ms.get("add_bias_and_transpose_kernel", 0.0)
    per = {k: v / args.steps for k, v in stage_ms.items()}
    gemm_tf = gemm_fl / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    attn_tf = attn_fl / (attn_ms * 1e-3) / 1e12 if attn_ms else 0.0
    fused_ms = sum(stage_ms.get(k, 0.0) for k in fused_keys)
    fused_tf = sum(fl[k] for k in fused_keys) / (fused_ms * 1e-3) / 1e12 if fused_ms else 0.0
    ln_launches = L * (2 - len(fused_keys))
    ln_gbs = (ln_launches * 3 * stage_tokens * H * 2) / (ln_ms * 1e-3) / 1e9 if ln_ms else 0.0
    tr_gbs = (L * 2 * stage_tokens * 3 * H * 2) / (tr_ms * 1e-3) / 1e9 if tr_ms else 0.0
    if gemm_ms >= attn_ms:
        roof = {"kernel": f"gemm_pair_kernel (CTA-pair tcgen05 projection GEMMs: {', '.join(k[5:] for k in pair_keys)})",
                "bound": "tensor", "achieved": gemm_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                "frac": gemm_tf / pk["tf_sustained"], "traffic": ncu_traffic("gemm", gemm_fl / n_gemm),
                "launches_per_step": n_gemm // args.steps, "avg_launch_ms": gemm_ms / n_gemm,
                "flops_per_launch": gemm_fl / n_gemm}
    else:
        roof = {"kernel": "sparse_attention_kernel (tcgen05 block-sparse attention, 1 per layer)", "bound": "tensor",
                "achieved": attn_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                "frac": attn_tf / pk["tf_sustained"], "traffic": ncu_traffic("attention", attn_fl / n_attn),
                "launches_per_step": n_attn // args.steps, "avg_launch_ms": attn_ms / n_attn,
                "flops_per_launch": attn_fl / n_attn}
    roof["peak_source"] = pk["source"] + " (sustained bf16 dense, kernel timed inside a long step)"
    roof["traffic_source"] = ("ncu capture of the same kernel on the micro-benchmark shape (profiles/), "
                              "scaled by algorithmic work per launch")

    # ---- CPU baseline: the reference's validation model on the whole seed-0 batch ------------
    cpu = None
    if n_gpus == 1 and not args.no_cpu_baseline:
        b0 = batches[0]
        threads = os.cpu_count() or 1
        tps, ms, kind = cpu_tokens_per_s(w, b0.ids_all, 1, b0.ids_all[int(np.argmin(b0.lens_all))], threads)
        cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": kind,
               "sample": f"whole seed-0 batch ({len(b0.lens_all)} sequences, {b0.T_total} tokens), all {w['layers']} layers, "
                         f"fp32, one timed pass ({ms / 1e3:.1f} s) after a warm-up on its shortest sequence"}

    print(json.dumps({
        "metric": "encoder_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": w.get("scaling", "weak"), "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["desc"], "sequences": len(batches[0].lens_all), "tokens": batches[0].T_total,
                   "rotation": f"{N_ROTATE} batches (seeds 0..{N_ROTATE - 1}, {[b.T_total for b in batches]} tokens) take turns; "
                               f"tokens/s counts the tokens of the steps actually timed",
                   "l2": "flushed between timed steps (256 MiB write)",
                   "stage_timing": "per-kernel durations (roofline, stages_ms_per_step) come from a second pass of the "
                                   "same steps with CUDA events around every launch",
                   "parallelism": f"replicas x{n_gpus}, whole-sequence bin packing, gather of outputs to rank 0 "
                                  f"({'copy-engine peer copies into symmetric memory' if type(batches[0].gatherer).__name__ == 'PeerGatherer' else 'NCCL send/recv'}) timed (the gather "
                                  f"of step i overlaps the kernels of steps i+1 and i+2; the last gathers' tail is added)"
                   if n_gpus > 1 else "single GPU"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms_per_step, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "mode": e2e_mode, "one_batch_at_a_time_ms_per_step": e2e_sync_ms},
        "gpu_launches": int(launches),
        "host_work_ms_per_step": host_ms_per_step,
        "rank_ms_per_step": {"max": max(per_rank_ms), "mean": float(np.mean(per_rank_ms)), "per_rank": per_rank_ms},
        "clocks": clocks,
        "roofline": roof,
        "stages_ms_per_step": per,
        "rooflines_other": {
            "attention_tflops": attn_tf, "attention_frac_of_tensor_peak": attn_tf / pk["tf_sustained"],
            "gemm_tflops": gemm_tf,
            "gemm_with_layernorm_tflops": fused_tf,
            "gemm_with_layernorm": [k[5:] for k in fused_keys],
            "layernorm_launches_per_step": ln_launches,
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
    ap.add_argument("--gather", default=None, choices=["peer", "nccl"],
                    help="N > 1: how outputs reach rank 0 (default: copy-engine peer copies where available, else NCCL send/recv)")
    ap.add_argument("--total-seqs", type=int, default=0,
                    help="strong scaling: this many sequences in the global batch whatever --gpus (must divide evenly)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    w["gather"] = args.gather
    if args.seqs > 0:
        w["seqs"] = args.seqs
        w["desc"] += f" (--seqs {args.seqs})"
    w["scaling"] = "weak"
    if args.total_seqs > 0:
        world = int(os.environ.get("WORLD_SIZE", "1")) if args.impl == "ours" else 1
        if args.total_seqs % world:
            raise SystemExit("--total-seqs must be a multiple of the number of GPUs")
        w["seqs"] = args.total_seqs // world
        w["scaling"] = "strong"
        w["desc"] += f" (fixed global batch of {args.total_seqs} sequences)"
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_gpu(args, w)


if __name__ == "__main__":
    main()
