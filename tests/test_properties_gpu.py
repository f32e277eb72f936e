"""Size-independent properties at the benchmark's full size (BigBird-base, 8 sequences of
1024..4096 tokens, the lengths bench.py draws).  The comparison with the CPU oracle at this size
lives in test_parity_configs_gpu.py; here is what must hold for a correct padding-free varlen
encoder whatever its size, and what an oracle comparison within a tolerance would not catch
(races, stale scratch, dependence on batch position):

* the same batch twice gives bit-identical hidden states (no race, no stale scratch);
* a sequence's hidden states do not depend on its position in the batch (bit-exact under a
  permutation of the sequences) nor on its neighbours (each sequence alone: same result up to
  the summation order of split key/value lists);
* softmax rows are normalised: with V = 1 every context value is 1;
* attention is linear in V;
* splitting long key/value lists into merged parts does not change the result beyond rounding.

Small-size parity against the oracle itself lives in test_kernels_gpu.py / test_encoder_gpu.py.
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _skip_no_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _bench_batch():
    import bench
    w = bench.WORKLOADS["base"]
    lens, ids = bench.make_lengths(w, 8)
    return w, lens, ids


def _encoder(w):
    from raptor_t_b200 import capi
    from raptor_t_b200.engine import Encoder
    from raptor_t_b200.weights import synthetic_weights
    import bench
    cfg = capi.make_config(hidden=w["hidden"], heads=w["heads"], ffn=w["ffn"], layers=w["layers"],
                           max_pos=w["max_pos"], vocab=bench.VOCAB, type_vocab=bench.TYPE_VOCAB,
                           pattern=w["pattern"], dtype=w["dtype"])
    P = synthetic_weights(w["hidden"], w["ffn"], w["layers"], bench.VOCAB, w["max_pos"], bench.TYPE_VOCAB, seed=0,
                          nonzero_bias=True)
    return Encoder(cfg).load_weights(P)


def _run(enc, lens, ids):
    enc.prepare(lens)
    out = enc.forward_ids(torch.from_numpy(np.concatenate(ids)).cuda()).clone()
    torch.cuda.synchronize()
    return out


def test_full_size_encoder_is_deterministic_and_batch_invariant():
    _skip_no_gpu()
    from raptor_t_b200 import ops
    w, lens, ids = _bench_batch()
    assert sum(lens) == 16512 and len(lens) == 8
    enc = _encoder(w)
    full = _run(enc, lens, ids)
    assert torch.isfinite(full.float()).all()
    # LayerNorm output: every row has (close to) zero mean and unit variance before gamma/beta;
    # with the perturbed gamma/beta of the synthetic weights the rows are still O(1)
    assert 0.5 < full.float().std().item() < 2.0
    again = _run(enc, lens, ids)
    assert torch.equal(full, again)

    starts = np.concatenate([[0], np.cumsum(lens)])
    # permuted batch: same rows, moved
    perm = [5, 2, 7, 0, 3, 6, 1, 4]
    moved = _run(enc, [lens[i] for i in perm], [ids[i] for i in perm])
    off = 0
    for i in perm:
        assert torch.equal(moved[off:off + lens[i]], full[starts[i]:starts[i] + lens[i]]), i
        off += lens[i]
    # every sequence alone: the work-list split of its long lists may differ from the batch's
    # (another summation order in fp32), everything else is the same arithmetic
    worst = 0.0
    for i in (int(np.argmin(lens)), int(np.argmax(lens))):
        alone = _run(enc, [lens[i]], [ids[i]])
        d = (alone.float() - full[starts[i]:starts[i] + lens[i]].float()).abs()
        worst = max(worst, d.max().item())
        assert d.max().item() < 2e-2 and d.mean().item() < 1e-3, (i, d.max().item(), d.mean().item())
    ops.check_device()
    enc.close()


def _attention_inputs(lens, heads, dtype, seed):
    T, H = sum(lens), heads * 64
    g = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn(T, H, device="cuda", generator=g).to(dtype) for _ in range(3))


def test_full_size_attention_rows_are_normalised_and_linear_in_v():
    _skip_no_gpu()
    from raptor_t_b200 import capi, metadata, ops
    w, lens, _ = _bench_batch()
    dtype = torch.bfloat16
    cfg = capi.make_config(hidden=768, heads=12, ffn=3072, layers=1, max_pos=4096, dtype="bf16")
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 3, lens)
    plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx)
    q, k, v = _attention_inputs(lens, 12, dtype, seed=11)
    scale = 1.0 / math.sqrt(64)
    ones = ops.sparse_attention(q, k, torch.ones_like(v), plan, scale=scale)
    # probabilities are rounded to bf16 before the PV product: a row sums to 1 within 2^-8
    assert (ones.float() - 1.0).abs().max().item() < 8e-3
    v2 = torch.randn_like(v)
    a = ops.sparse_attention(q, k, v, plan, scale=scale).float()
    b = ops.sparse_attention(q, k, v2, plan, scale=scale).float()
    both = ops.sparse_attention(q, k, (v.float() * 0.5 + v2.float() * 0.25).to(dtype), plan, scale=scale).float()
    err = (both - (0.5 * a + 0.25 * b)).abs()
    assert err.max().item() < 3e-2 and err.mean().item() < 2e-3, (err.max().item(), err.mean().item())
    # a convex combination of V rows stays inside their range
    assert a.abs().max().item() <= v.float().abs().max().item() + 1e-2
    ops.check_device()


@pytest.mark.parametrize("lens", [[4096], [3136, 1024]])
def test_split_lists_equal_whole_lists(lens):
    _skip_no_gpu()
    from raptor_t_b200 import capi, metadata, ops
    dtype = torch.float16
    cfg = capi.make_config(hidden=768, heads=12, ffn=3072, layers=1, max_pos=4096, dtype="f16")
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 7, lens)
    q, k, v = _attention_inputs(lens, 12, dtype, seed=5)
    whole_plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx, split_entries=0)
    whole = ops.sparse_attention(q, k, v, whole_plan, scale=0.125)
    split_plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx, split_entries=16)
    assert split_plan.items > whole_plan.items          # the global blocks' lists were cut
    split = ops.sparse_attention(q, k, v, split_plan, scale=0.125)
    d = (split.float() - whole.float()).abs()
    assert d.max().item() < 4e-3, d.max().item()
    # only the split items' rows may differ at all: first and last block of every sequence
    t0 = 0
    for n in lens:
        assert torch.equal(split[t0 + 64:t0 + n - 64], whole[t0 + 64:t0 + n - 64])
        t0 += n
    ops.check_device()
