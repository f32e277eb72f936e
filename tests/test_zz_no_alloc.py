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


def _case(cfg, lens, layer, seed, dtype, with_oracle=False):
    from raptor_t_b200 import metadata, ops
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, layer, lens)
    T, H = sum(lens), cfg.hidden
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(T, H, device="cuda", generator=g).to(dtype) for _ in range(3))
    # the regular entry point cuts long lists into parts merged by a second kernel (another
    # summation order); the static one keeps lists whole.  With splitting off both run the
    # same work list, so the comparison can be exact.
    plan = ops.AttentionPlan(cfg, lens, kv_ptr, kv_idx, split_entries=0)
    ref = ops.sparse_attention(q, k, v, plan, scale=1.0 / math.sqrt(64))
    out = torch.empty_like(q)            # the caller owns inputs and outputs
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    ops.sparse_attention_static(q, k, v, cfg, lens, kv_ptr, kv_idx, scale=1.0 / math.sqrt(64), out=out)
    ops.check_device()
    free_after = torch.cuda.mem_get_info()[0]
    if with_oracle:  # one direct comparison with the CPU oracle (q/k/v storage is head-major per sequence)
        import oracle
        ocfg = oracle.EncoderConfig(hidden=H, heads=cfg.heads, ffn=cfg.ffn, layers=1, max_pos=cfg.max_pos)
        nh, t0 = cfg.heads, 0
        for n in lens:
            qs, ks, vs = (t.view(-1)[t0 * H:(t0 + n) * H].view(nh, n, 64).float().cpu() for t in (q, k, v))
            L = n // 64
            rand = oracle.rand_block_table(layer, nh, L, cfg.num_rand, cfg.max_pos) if L > 5 + 2 * cfg.num_rand else None
            lists = [oracle.kv_block_lists(L, ocfg, rand, h) for h in range(nh)]
            want = oracle.sparse_attention_ref(qs, ks, vs, lists).permute(1, 0, 2).reshape(n, H)
            err = (out[t0:t0 + n].float().cpu() - want).abs().max().item()
            assert err < 4e-2, err
            t0 += n
    return ref, out, free_before - free_after


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi
    cfg = capi.make_config(hidden=768, heads=12, ffn=3072, layers=1, dtype="bf16")
    # first call: a larger batch; second call: a smaller, different one (stale work-list
    # entries of the first call stay in the array behind the second call's list)
    ref1, out1, _ = _case(cfg, [1024, 1856, 704], layer=0, seed=1, dtype=torch.bfloat16, with_oracle=True)
    ref2, out2, grew = _case(cfg, [832, 64], layer=5, seed=2, dtype=torch.bfloat16)
    for ref, out in ((ref1, out1), (ref2, out2)):
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= 4e-2, err              # same tolerance as the attention parity tests (bf16)
        assert torch.equal(out, ref)         # same kernel, same work list: bit-identical in practice
    assert grew == 0, f"device memory in use grew by {grew} bytes during a call that must not allocate"


def test_static_scratch_entry_on_a_side_stream():
    """Two calls in a row on a non-blocking side stream: the read-back of the previous call's
    status is ordered on that stream, and the results still match the regular entry point."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi
    cfg = capi.make_config(hidden=256, heads=4, ffn=1024, layers=1, dtype="f16")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for seed, lens in ((7, [1152, 640]), (8, [896])):
            ref, out, _ = _case(cfg, lens, layer=2, seed=seed, dtype=torch.float16)
            assert torch.equal(out, ref)
    side.synchronize()


def test_static_scratch_entry_reports_a_kernel_that_gave_up_and_recovers():
    """The status word of the static array is written by the library's self-test kernel (one
    wait that runs out after ~0.5 ms and returns normally); the next call of the entry point
    must report it, and the call after that must work."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi, metadata, ops
    cfg = capi.make_config(hidden=128, heads=2, ffn=256, layers=1, dtype="bf16")
    lens = [832]
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 0, lens)
    q = torch.randn(832, 128, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=out)    # sets the array up
        ops.selftest_bounded_wait(limit_cycles=1_000_000, target=1)
        with pytest.raises(capi.RtError) as e:
            ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=out)
        assert e.value.code == 4 and "901" in str(e.value)
        ref, got, _ = _case(cfg, lens, layer=0, seed=3, dtype=torch.bfloat16)
        assert torch.equal(got, ref)
    side.synchronize()


def test_static_scratch_entry_refuses_a_capturing_stream():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import capi, metadata, ops
    cfg = capi.make_config(hidden=128, heads=2, ffn=256, layers=1, dtype="bf16")
    lens = [832]
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 0, lens)
    q = torch.randn(832, 128, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=out)        # first call: set-up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        with pytest.raises(capi.RtError) as e:
            ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=out)
        assert e.value.code == 2
    torch.cuda.synchronize()
    ops.sparse_attention_static(q, q, q, cfg, lens, kv_ptr, kv_idx, out=out)        # still usable
    ops.check_device()


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
