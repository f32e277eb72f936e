"""Kernel micro-benchmarks (the reference's attention_test / mem_bound_op experiments,
python/benchmark/attention_test.py and mem_bound_op.py, re-stated for this library).

    python -m raptor_t_b200.microbench --kernel attention --seq 4096 --batch 8 [--dtype bf16]
    python -m raptor_t_b200.microbench --kernel layernorm --rows 32768 --cols 768
    python -m raptor_t_b200.microbench --kernel gelu --rows 32768 --cols 3072
    python -m raptor_t_b200.microbench --kernel transpose --seq 4096 --batch 8
    python -m raptor_t_b200.microbench --kernel gemm --m 16384 --n 3072 --k 768
    python -m raptor_t_b200.microbench --kernel gemm_ln --m 16384 --n 768 --k 3072
    python -m raptor_t_b200.microbench --kernel all

Each line of output is one JSON object: algorithmic FLOPs or bytes, the median CUDA-event
time over --iters launches (L2 flushed before each: 256 MiB written, then read back), and the achieved rate as a fraction
of the measured peaks in MEASURED_PEAKS.json (fallback 6650 GB/s / 1590 TFLOP/s).
Attention FLOPs count listed (query block, key block) pairs only: 4*64*64*64 per pair.
"""
import argparse
import json
import math
import os

import numpy as np
import torch

from . import capi, metadata, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_FLUSH = None


def _time(fn, iters, warmup=3, flush=True):
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            # write 256 MiB (evicts everything), then read it back: the read sweep forces the
            # dirty lines out, so the timed kernel starts on a cold L2 without write-back debt
            _FLUSH.fill_(0)
            _FLUSH.view(torch.int64).sum()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ops.check_device()
    return float(np.median(ts)), float(np.min(ts))


def _dtype(name):
    return torch.bfloat16 if name == "bf16" else torch.float16


def bench_attention(seq, batch, dtype, iters, heads=12, seed=0, pattern="bigbird"):
    hbm, tf, src = _peaks()
    cfg = capi.make_config(hidden=heads * 64, heads=heads, ffn=4 * heads * 64, layers=1, max_pos=max(4096, seq),
                           pattern=pattern, dtype=dtype)
    lens = [seq] * batch
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, seed, lens)
    plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx)
    T, H = seq * batch, heads * 64
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(T, H, device="cuda", generator=g).to(_dtype(dtype)) for _ in range(3))
    out = torch.empty_like(q)
    med, best = _time(lambda: ops.sparse_attention(q, k, v, plan, scale=0.125, out=out), iters)
    flops = 1048576.0 * plan.visits
    return {"kernel": "sparse_attention", "seq": seq, "batch": batch, "heads": heads, "dtype": dtype,
            "pattern": pattern, "visits": plan.visits, "issued_block_loads": plan.entries, "items": plan.items,
            "flops": flops, "ms": med, "ms_min": best, "tflops": flops / med / 1e9,
            "frac_of_tensor_peak": flops / med / 1e9 / tf, "peak": tf, "peak_source": src}


def bench_layernorm(rows, cols, dtype, iters):
    hbm, tf, src = _peaks()
    dt = _dtype(dtype)
    x = torch.randn(rows, cols, device="cuda").to(dt)
    r = torch.randn(rows, cols, device="cuda").to(dt)
    b, g, be = (torch.randn(cols, device="cuda").to(dt) for _ in range(3))
    med, best = _time(lambda: ops.bias_residual_layernorm(x, b, r, g, be, 1e-12), iters)
    nbytes = 3.0 * rows * cols * 2 + 3 * cols * 2
    return {"kernel": "bias_residual_layernorm", "rows": rows, "cols": cols, "dtype": dtype, "bytes": nbytes,
            "ms": med, "ms_min": best, "gbs": nbytes / med / 1e6, "frac_of_hbm_peak": nbytes / med / 1e6 / hbm,
            "peak": hbm, "peak_source": src}


def bench_gelu(rows, cols, dtype, iters):
    hbm, tf, src = _peaks()
    dt = _dtype(dtype)
    x = torch.randn(rows, cols, device="cuda").to(dt)
    b = torch.randn(cols, device="cuda").to(dt)
    med, best = _time(lambda: ops.bias_gelu_(x, b), iters)
    nbytes = 2.0 * rows * cols * 2 + cols * 2
    return {"kernel": "bias_gelu", "rows": rows, "cols": cols, "dtype": dtype, "bytes": nbytes, "ms": med,
            "ms_min": best, "gbs": nbytes / med / 1e6, "frac_of_hbm_peak": nbytes / med / 1e6 / hbm, "peak": hbm,
            "peak_source": src}


def bench_transpose(seq, batch, dtype, iters, heads=12):
    hbm, tf, src = _peaks()
    dt = _dtype(dtype)
    T, H = seq * batch, heads * 64
    qkv = torch.randn(T, 3 * H, device="cuda").to(dt)
    bias = torch.randn(3 * H, device="cuda").to(dt)
    prefix = torch.from_numpy(metadata.seq_block_prefix([seq] * batch)).cuda()
    outs = tuple(torch.empty(T, H, device="cuda", dtype=dt) for _ in range(3))
    med, best = _time(lambda: ops.qkv_bias_transpose(qkv, bias, prefix, heads, 0.125, out=outs), iters)
    nbytes = 2.0 * T * 3 * H * 2
    return {"kernel": "qkv_bias_transpose", "tokens": T, "heads": heads, "dtype": dtype, "bytes": nbytes, "ms": med,
            "ms_min": best, "gbs": nbytes / med / 1e6, "frac_of_hbm_peak": nbytes / med / 1e6 / hbm, "peak": hbm,
            "peak_source": src}


def bench_gemm(m, n, k, dtype, iters, epilogue=capi.RT_EPI_NONE):
    hbm, tf, src = _peaks()
    dt = _dtype(dtype)
    a = torch.randn(m, k, device="cuda").to(dt)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(dt)
    bias = torch.randn(n, device="cuda").to(dt)
    out = torch.empty(m, n, device="cuda", dtype=dt)
    med, best = _time(lambda: ops.gemm(a, w, bias if epilogue else None, epilogue, out=out), iters)
    flops = 2.0 * m * n * k
    return {"kernel": "gemm", "m": m, "n": n, "k": k, "epilogue": epilogue, "dtype": dtype, "flops": flops, "ms": med,
            "ms_min": best, "tflops": flops / med / 1e9, "frac_of_tensor_peak": flops / med / 1e9 / tf, "peak": tf,
            "peak_source": src}


def bench_gemm_ln(m, n, k, dtype, iters):
    """Projection + bias + residual + LayerNorm in one kernel, next to the two-kernel path it replaces."""
    hbm, tf, src = _peaks()
    dt = _dtype(dtype)
    a = torch.randn(m, k, device="cuda").to(dt)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(dt)
    bias, gamma, beta = (torch.randn(n, device="cuda").to(dt) for _ in range(3))
    res = torch.randn(m, n, device="cuda").to(dt)
    out = torch.empty(m, n, device="cuda", dtype=dt)
    dense = torch.empty(m, n, device="cuda", dtype=dt)
    med, best = _time(lambda: ops.gemm_bias_residual_layernorm(a, w, bias, res, gamma, beta, 1e-12, out=out), iters)

    def two():
        ops.gemm(a, w, out=dense)
        ops.bias_residual_layernorm(dense, bias, res, gamma, beta, 1e-12, out=out)
    med2, _ = _time(two, iters)
    flops = 2.0 * m * n * k
    return {"kernel": "gemm_bias_residual_layernorm", "m": m, "n": n, "k": k, "dtype": dtype, "flops": flops, "ms": med,
            "ms_min": best, "tflops": flops / med / 1e9, "frac_of_tensor_peak": flops / med / 1e9 / tf,
            "two_kernel_ms": med2, "peak": tf, "peak_source": src}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all",
                    choices=["all", "attention", "layernorm", "gelu", "transpose", "gemm", "gemm_ln", "attention_sweep"])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=768)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    ap.add_argument("--pattern", default="bigbird", choices=["bigbird", "band"])
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    out = []
    if a.kernel == "attention":
        out.append(bench_attention(a.seq, a.batch, a.dtype, a.iters, a.heads, pattern=a.pattern))
    if a.kernel in ("attention_sweep", "all"):
        for batch in (1, 8, 32):
            for seq in (1024, 2048, 4096, 8192, 16384):
                out.append(bench_attention(seq, batch, a.dtype, a.iters, a.heads))
                print(json.dumps(out[-1]), flush=True)
        out = [] if a.kernel == "attention_sweep" else out[:0]
    if a.kernel == "layernorm":
        out.append(bench_layernorm(a.rows, a.cols, a.dtype, a.iters))
    if a.kernel == "gelu":
        out.append(bench_gelu(a.rows, a.cols, a.dtype, a.iters))
    if a.kernel == "transpose":
        out.append(bench_transpose(a.seq, a.batch, a.dtype, a.iters, a.heads))
    if a.kernel == "gemm":
        out.append(bench_gemm(a.m, a.n, a.k, a.dtype, a.iters))
    if a.kernel == "gemm_ln":
        out.append(bench_gemm_ln(a.m, a.n, a.k, a.dtype, a.iters))
    if a.kernel == "all":
        out.append(bench_layernorm(32768, 768, a.dtype, a.iters))
        out.append(bench_layernorm(32768, 1024, a.dtype, a.iters))
        out.append(bench_gelu(32768, 3072, a.dtype, a.iters))
        out.append(bench_transpose(4096, 8, a.dtype, a.iters))
        for (m, n, k) in ((16384, 2304, 768), (16384, 768, 768), (16384, 3072, 768), (16384, 768, 3072)):
            out.append(bench_gemm(m, n, k, a.dtype, a.iters))
        out.append(bench_gemm(16384, 3072, 768, a.dtype, a.iters, capi.RT_EPI_BIAS_GELU))
        for (m, n, k) in ((16384, 768, 768), (16384, 768, 3072), (16384, 1024, 4096)):
            out.append(bench_gemm_ln(m, n, k, a.dtype, a.iters))
    for o in out:
        print(json.dumps(o), flush=True)


if __name__ == "__main__":
    main()
