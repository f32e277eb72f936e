"""rt_sparse_attention_static: the attention entry point for callers that cannot allocate
device memory (their memory belongs to an external arena / caching allocator, or they run
where cudaMalloc's implicit synchronisation is not acceptable).  It must give the same
context tensor as the regular entry point (rt_sparse_attention with an rt_attn_plan), call
after call, although every call reuses one fixed device array that still holds the previous
call's work list.  Collected last on purpose: a failure here cannot hide other tests."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(cfg, lens, layer, seed, dtype):
    from raptor_t_b200 import metadata, ops
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, layer, lens)
    T, H = sum(lens), cfg.hidden
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(T, H, device="cuda", generator=g).to(dtype) for _ in range(3))
    plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx)
    ref = ops.sparse_attention(q, k, v, plan, scale=1.0 / math.sqrt(64))
    out = torch.empty_like(q)            # the caller owns inputs and outputs
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    ops.sparse_attention_static(q, k, v, cfg, lens, kv_ptr, kv_idx, scale=1.0 / math.sqrt(64), out=out)
    ops.check_device()
    free_after = torch.cuda.mem_get_info()[0]
    return ref, out, free_before - free_after


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    # the regular entry point cuts long lists into parts merged by a second kernel (another
    # summation order); the static one keeps lists whole.  With splitting off both run the
    # same work list, so the comparison can be exact.
    monkeypatch.setenv("RAPTOR_B200_ATTN_SPLIT", "0")
    from raptor_t_b200 import capi
    cfg = capi.make_config(hidden=768, heads=12, ffn=3072, layers=1, dtype="bf16")
    # first call: a larger batch; second call: a smaller, different one (stale work-list
    # entries of the first call stay in the array behind the second call's list)
    ref1, out1, _ = _case(cfg, [1024, 1856, 704], layer=0, seed=1, dtype=torch.bfloat16)
    ref2, out2, grew = _case(cfg, [832, 64], layer=5, seed=2, dtype=torch.bfloat16)
    for ref, out in ((ref1, out1), (ref2, out2)):
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= 4e-2, err              # same tolerance as the attention parity tests (bf16)
        assert torch.equal(out, ref)         # same kernel, same work list: bit-identical in practice
    assert grew == 0, f"device memory in use grew by {grew} bytes during a call that must not allocate"


def test_static_scratch_entry_rejects_oversized_batches():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi, metadata, ops
    cfg = capi.make_config(hidden=768, heads=12, ffn=3072, layers=1, dtype="bf16")
    lens = [4096] * 32                       # ~157k list entries > 131072
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 0, lens)
    T = sum(lens)
    q = torch.zeros(T, 768, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.RtError) as e:
        ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=torch.empty_like(q))
    assert e.value.code == 2 and "static scratch holds" in str(e.value)
    # and the entry point keeps working afterwards
    ref, out, _ = _case(cfg, [960], layer=1, seed=3, dtype=torch.float16)
    assert torch.equal(out, ref)
