"""GPU encoder vs the CPU oracle at the benchmark configurations' own sizes and depths.

* config 2: the exact batch bench.py times (8 sequences, 16 512 tokens, seed 0), embeddings +
  12 BigBird-base layers, fp16, the benchmark's seed-0 weights;
* config 3: band pattern (window of 9 blocks + first block global), 12 layers, bf16, four
  sequences spanning 512..4096 tokens;
* config 5: BigBird-large shape, all 24 layers, bf16, four sequences spanning 640..8192 tokens
  (640 tokens = 10 blocks runs full attention).

Checked: block tables of every layer bit-exact with the oracle, final hidden states within the
stated max-abs / mean-abs bounds.  fp16 is held to 2e-2 / 2e-3.  bf16 has 8 instead of 11
mantissa bits in every activation that crosses HBM (each LayerNorm output alone is rounded by
up to 2^-9 relative, twice per layer), so its bounds are wider; they are the measured errors on
a B200 plus a margin, and every run prints what it measured.

Set RAPTOR_B200_PARITY_LOG=<file> to append the measured errors as JSON lines.
"""
import json
import os
import time

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = {
    # name: (max_abs, mean_abs)
    "config2_fp16": (2e-2, 2e-3),
    # measured on a B200: config 3 max 0.072 / mean 0.0069, config 5 max 0.064 / mean 0.0090 - the fp16
    # figure (0.0097 / 0.00086) times the 8x coarser mantissa; these bounds are those plus ~50 %
    "config3_bf16": (1.1e-1, 1.0e-2),
    "config5_bf16": (1.0e-1, 1.4e-2),
}


def _report(name, err, extra):
    rec = {"case": name, "max_abs": err.max().item(), "mean_abs": err.mean().item(), **extra}
    print("PARITY " + json.dumps(rec))
    path = os.environ.get("RAPTOR_B200_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")
    return rec


def _run_case(name, w, lens, ids, P):
    import bench
    from raptor_t_b200 import capi, ops
    from raptor_t_b200.engine import Encoder
    ocfg = oracle.EncoderConfig(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                                max_pos=w["max_pos"], vocab=bench.VOCAB, type_vocab=bench.TYPE_VOCAB,
                                pattern=w["pattern"])
    cfg = capi.make_config(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                           max_pos=w["max_pos"], vocab=bench.VOCAB, type_vocab=bench.TYPE_VOCAB,
                           pattern=w["pattern"], band_half=ocfg.band_half, dtype=w["dtype"])
    enc = Encoder(cfg).load_weights(P)
    enc.prepare(lens)
    out = enc.forward_ids(torch.from_numpy(np.concatenate(ids)).cuda())
    ops.check_device()
    for layer in range(w["layers"]):
        ptr, idx = enc.table(layer)
        optr, oidx = oracle.build_block_csr(lens, ocfg, layer)
        assert np.array_equal(ptr, optr) and np.array_equal(idx, oidx), f"layer {layer}: block table differs"
    t0 = time.perf_counter()
    ref = oracle.encoder_ref([torch.from_numpy(s) for s in ids], P, ocfg)
    cpu_s = time.perf_counter() - t0
    err = (out.float().cpu() - ref).abs()
    rec = _report(name, err, {"dtype": w["dtype"], "layers": w["layers"], "tokens": int(sum(lens)),
                              "lens": [int(n) for n in lens], "oracle_seconds": round(cpu_s, 2)})
    mx, mean = TOL[name]
    assert rec["max_abs"] < mx and rec["mean_abs"] < mean, rec
    enc.close()


def _weights(w):
    import bench
    from raptor_t_b200.weights import synthetic_weights
    return synthetic_weights(w["hidden"], w["ffn"], w["layers"], bench.VOCAB, w["max_pos"], bench.TYPE_VOCAB, seed=0)


def _skip_no_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def test_config2_bench_batch_fp16_12_layers():
    _skip_no_gpu()
    import bench
    w = bench.WORKLOADS["base"]
    lens, ids = bench.make_lengths(w, 8)
    assert sum(lens) == 16512
    _run_case("config2_fp16", w, lens, ids, _weights(w))


def test_config3_band_bf16_12_layers():
    _skip_no_gpu()
    import bench
    w = bench.WORKLOADS["band"]
    lens = [512, 1536, 2880, 4096]
    rng = np.random.default_rng(3)
    ids = [rng.integers(5, bench.VOCAB, size=n).astype(np.int32) for n in lens]
    _run_case("config3_bf16", w, lens, ids, _weights(w))


def test_config5_large_bf16_24_layers():
    _skip_no_gpu()
    import bench
    w = bench.WORKLOADS["large"]
    lens = [640, 1088, 3200, 8192]
    rng = np.random.default_rng(5)
    ids = [rng.integers(5, bench.VOCAB, size=n).astype(np.int32) for n in lens]
    _run_case("config5_bf16", w, lens, ids, _weights(w))
