"""Parity of every CUDA kernel (through the C ABI) with a torch fp32 reference / the oracle."""
import math

import numpy as np
import pytest
import torch

import oracle
from oracle import EncoderConfig

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16]


def _tol(dtype):
    return 2e-2 if dtype == torch.bfloat16 else 4e-3


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(1, 768), (257, 768), (4096, 1024), (130, 128), (64, 256)])
def test_layernorm(ops, dtype, rows, hidden):
    g = torch.Generator(device="cuda").manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
    res = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
    bias = (torch.randn(hidden, device="cuda", generator=g) * 0.1).to(dtype)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).to(dtype)
    beta = (0.1 * torch.randn(hidden, device="cuda", generator=g)).to(dtype)
    ref = torch.nn.functional.layer_norm(x.float() + bias.float() + res.float(), (hidden,), gamma.float(),
                                         beta.float(), 1e-12)
    out = ops.bias_residual_layernorm(x.clone(), bias, res, gamma, beta, 1e-12)
    assert (out.float() - ref).abs().max().item() < _tol(dtype) * 2
    # in place, no bias / residual
    out2 = ops.bias_residual_layernorm(x.clone(), None, None, gamma, beta, 1e-5)
    ref2 = torch.nn.functional.layer_norm(x.float(), (hidden,), gamma.float(), beta.float(), 1e-5)
    assert (out2.float() - ref2).abs().max().item() < _tol(dtype) * 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,cols", [(3, 3072), (1000, 3072), (513, 4096), (7, 256)])
def test_bias_gelu(ops, dtype, rows, cols):
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = (2 * torch.randn(rows, cols, device="cuda", generator=g)).to(dtype)
    b = torch.randn(cols, device="cuda", generator=g).to(dtype)
    ref = oracle.gelu_new(x.float().cpu() + b.float().cpu())
    out = ops.bias_gelu_(x.clone(), b)
    assert (out.float().cpu() - ref).abs().max().item() < _tol(dtype) * 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,lens", [(12, [1024, 64, 832]), (2, [128]), (16, [512, 2048])])
def test_qkv_bias_transpose(ops, dtype, heads, lens):
    H, T = heads * 64, sum(lens)
    g = torch.Generator(device="cuda").manual_seed(T)
    qkv = torch.randn(T, 3 * H, device="cuda", generator=g).to(dtype)
    bias = torch.randn(3 * H, device="cuda", generator=g).to(dtype)
    prefix = torch.tensor(oracle.seq_block_prefix(lens), dtype=torch.int32, device="cuda")
    q, k, v = ops.qkv_bias_transpose(qkv, bias, prefix, heads, 0.125)
    full = qkv.float() + bias.float()
    t0 = 0
    for n in lens:
        for part, got in enumerate((q, k, v)):
            ref = full[t0:t0 + n, part * H:(part + 1) * H].view(n, heads, 64).permute(1, 0, 2)
            if part == 0:
                ref = ref * 0.125
            blk = got.view(-1)[t0 * H:(t0 + n) * H].view(heads, n, 64).float()
            assert (blk - ref).abs().max().item() < _tol(dtype)
        t0 += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_embeddings(ops, dtype):
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=1, max_pos=4096, vocab=97)
    P = oracle.make_weights(cfg, seed=3, nonzero_bias=True)
    ids = torch.from_numpy(np.random.default_rng(5).integers(0, cfg.vocab, size=832)).int()
    pos = torch.arange(832, dtype=torch.int32)
    ref = oracle.embeddings_ref(ids, P, cfg)
    f = lambda k: P["embeddings." + k].cuda().float().contiguous()  # noqa: E731
    out = ops.embeddings(ids.cuda(), pos.cuda(), None, f("word_embeddings.weight"), f("position_embeddings.weight"),
                         f("token_type_embeddings.weight"), f("LayerNorm.weight"), f("LayerNorm.bias"), cfg.eps, dtype)
    assert (out.float().cpu() - ref).abs().max().item() < _tol(dtype) * 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (128, 256, 128), (200, 768, 768), (1024, 2304, 768),
                                   (4160, 768, 3072), (64, 128, 64), (20032, 3072, 768), (333, 384, 128)])
def test_gemm(ops, dtype, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(dtype)
    ref = a.float() @ w.float().t()
    out = ops.gemm(a, w)
    ops.check_device()
    err = (out.float() - ref).abs().max().item()
    assert err < _tol(dtype) * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_epilogues(ops, dtype):
    from raptor_t_b200 import capi
    M, N, K = 777, 3072, 768
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(dtype)
    b = torch.randn(N, device="cuda", generator=g).to(dtype)
    ref = a.float() @ w.float().t() + b.float()
    out = ops.gemm(a, w, b, capi.RT_EPI_BIAS)
    assert (out.float() - ref).abs().max().item() < _tol(dtype) * 4
    out = ops.gemm(a, w, b, capi.RT_EPI_BIAS_GELU)
    assert (out.float() - oracle.gelu_new(ref.cpu()).cuda()).abs().max().item() < _tol(dtype) * 4
    ops.check_device()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,lens", [(12, [1024, 64, 832]), (2, [128, 64]), (16, [512, 2048, 4096])])
def test_gemm_qkv_equals_gemm_plus_transpose(ops, dtype, heads, lens):
    H, T = heads * 64, sum(lens)
    g = torch.Generator(device="cuda").manual_seed(T)
    a = torch.randn(T, H, device="cuda", generator=g).to(dtype)
    w = (torch.randn(3 * H, H, device="cuda", generator=g) / math.sqrt(H)).to(dtype)
    bias = torch.randn(3 * H, device="cuda", generator=g).to(dtype)
    prefix = torch.tensor(oracle.seq_block_prefix(lens), dtype=torch.int32, device="cuda")
    q, k, v = ops.gemm_qkv(a, w, bias, ops.block_seq_table(lens), heads, 0.125)
    ops.check_device()
    full = (a.float() @ w.float().t() + bias.float())
    t0 = 0
    for n in lens:
        for part, got in enumerate((q, k, v)):
            ref = full[t0:t0 + n, part * H:(part + 1) * H].view(n, heads, 64).permute(1, 0, 2)
            if part == 0:
                ref = ref * 0.125
            blk = got.view(-1)[t0 * H:(t0 + n) * H].view(heads, n, 64).float()
            assert (blk - ref).abs().max().item() < _tol(dtype) * max(1.0, ref.abs().max().item())
        t0 += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(333, 768, 768), (20032, 768, 3072), (130, 128, 256)])
def test_gemm_residual(ops, dtype, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(dtype)
    b = torch.randn(N, device="cuda", generator=g).to(dtype)
    r = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    ref = a.float() @ w.float().t() + b.float() + r.float()
    out = ops.gemm_residual(a, w, b, r)
    assert (out.float() - ref).abs().max().item() < _tol(dtype) * 4
    inplace = ops.gemm_residual(a, w, b, r, out=r)   # output over the residual buffer
    assert torch.equal(inplace, out)
    ops.check_device()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,lens", [(768, [1024, 64, 832]), (1024, [128]), (128, [512, 2048, 64, 64])])
def test_pooler(ops, dtype, hidden, lens):
    """tanh(Linear(first token of every sequence)) on a packed varlen batch against torch fp32."""
    from raptor_t_b200 import metadata
    T = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(hidden + T)
    x = torch.randn(T, hidden, device="cuda", generator=g).to(dtype)
    w = (torch.randn(hidden, hidden, device="cuda", generator=g) / math.sqrt(hidden)).to(dtype)
    b = (0.1 * torch.randn(hidden, device="cuda", generator=g)).to(dtype)
    prefix = torch.from_numpy(metadata.seq_block_prefix(lens)).cuda()
    firsts = torch.tensor(np.concatenate([[0], np.cumsum(lens)[:-1]]), device="cuda")
    ref = torch.tanh(x[firsts].float() @ w.float().t() + b.float())
    out = ops.pooler(x, prefix, w, b)
    assert out.shape == (len(lens), hidden) and (out - ref).abs().max().item() < 2e-3
    from raptor_t_b200.modeling_bert import BertPooler
    assert torch.equal(BertPooler(w.t().contiguous(), b)(x, prefix), out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(256, 768, 768), (1000, 768, 3072), (16512, 768, 768), (64, 1024, 1024),
                                   (4100, 1024, 4096), (1, 768, 64)])
def test_gemm_bias_residual_layernorm(ops, dtype, M, N, K):
    """Projection + bias + residual + LayerNorm in one kernel (clusters of N/256 CTA pairs own whole
    rows) against torch fp32; also in place over the residual, and against the two-kernel path."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(dtype)
    b = (0.1 * torch.randn(N, device="cuda", generator=g)).to(dtype)
    r = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    gamma = (1 + 0.1 * torch.randn(N, device="cuda", generator=g)).to(dtype)
    beta = (0.1 * torch.randn(N, device="cuda", generator=g)).to(dtype)
    x = a.float() @ w.float().t() + b.float() + r.float()
    ref = torch.nn.functional.layer_norm(x, (N,), gamma.float(), beta.float(), 1e-12)
    out = ops.gemm_bias_residual_layernorm(a, w, b, r, gamma, beta, 1e-12)
    err = (out.float() - ref).abs()
    assert err.max().item() < _tol(dtype) * 2 and err.mean().item() < _tol(dtype) / 8, (err.max().item(), err.mean().item())
    two = ops.bias_residual_layernorm(ops.gemm(a, w), b, r, gamma, beta, 1e-12)   # rounds the projection to 16 bits first
    assert (out.float() - two.float()).abs().max().item() < _tol(dtype) * 2
    inplace = ops.gemm_bias_residual_layernorm(a, w, b, r, gamma, beta, 1e-12, out=r)   # output over the residual buffer
    assert torch.equal(inplace, out)
    again = ops.gemm_bias_residual_layernorm(a, w, b, out.clone(), gamma, beta, 1e-12)    # another launch, other data
    assert torch.isfinite(again.float()).all()
    ops.check_device()


def _attention_case(ops, dtype, cfg, lens, layer, seed, key_ramp=0.0):
    from raptor_t_b200 import capi, metadata
    rc = capi.make_config(hidden=cfg.hidden, heads=cfg.heads, ffn=cfg.ffn, layers=cfg.layers, max_pos=cfg.max_pos,
                          pattern=cfg.pattern, band_half=cfg.band_half,
                          dtype="bf16" if dtype == torch.bfloat16 else "f16")
    kv_ptr, kv_idx = metadata.build_block_csr(rc, layer, lens)
    plan = ops.AttentionPlan(rc, lens, kv_ptr, kv_idx)
    nh, T, H = cfg.heads, sum(lens), cfg.hidden
    g = torch.Generator().manual_seed(seed)
    # head-major per sequence storage
    q = torch.empty(T * H, dtype=dtype)
    k = torch.empty(T * H, dtype=dtype)
    v = torch.empty(T * H, dtype=dtype)
    refs, t0 = [], 0
    for n in lens:
        qs, ks, vs = (torch.randn(nh, n, 64, generator=g) for _ in range(3))
        if key_ramp != 0.0:
            # scores that climb (or fall) by 64 * |key_ramp| per key block, i.e. by more than 2^8 from one block to the
            # next: whatever order a list is walked in, the running maximum keeps moving and the accumulated output
            # has to be rescaled again and again
            blk = (torch.arange(n) // 64).float().view(1, n, 1)
            qs = 1.0 + 0.1 * qs
            ks = key_ramp * blk + 0.1 * ks
        qs, ks, vs = qs.to(dtype), ks.to(dtype), vs.to(dtype)
        for buf, src in ((q, qs), (k, ks), (v, vs)):
            buf[t0 * H:(t0 + n) * H] = src.reshape(-1)
        L = n // 64
        rand = None
        if cfg.pattern == "bigbird" and L > 5 + 2 * cfg.num_rand:
            rand = oracle.rand_block_table(layer, nh, L, cfg.num_rand, cfg.max_pos)
        lists = [oracle.kv_block_lists(L, cfg, rand, h) for h in range(nh)]
        r = oracle.sparse_attention_ref(qs.float(), ks.float(), vs.float(), lists)  # [nh, n, 64]
        refs.append(r.permute(1, 0, 2).reshape(n, H))
        t0 += n
    ref = torch.cat(refs, 0)
    out = ops.sparse_attention(q.cuda().view(T, H), k.cuda().view(T, H), v.cuda().view(T, H), plan,
                               scale=1.0 / math.sqrt(64))
    ops.check_device()
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() < _tol(dtype) * 2, (err.max().item(), err.mean().item())
    assert err.mean().item() < _tol(dtype) / 8
    assert plan.visits == cfg.heads * kv_ptr[-1]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lens", [[832], [1024], [512], [1088, 64, 1344], [4096, 960]])
def test_sparse_attention_bigbird(ops, dtype, lens):
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=1)
    _attention_case(ops, dtype, cfg, lens, layer=0, seed=len(lens))


def test_sparse_attention_12_heads_layer_seed(ops):
    cfg = EncoderConfig()
    _attention_case(ops, torch.bfloat16, cfg, [1024, 1856], layer=7, seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_ramp", [0.75, -0.75])
def test_sparse_attention_moving_maximum(ops, dtype, key_ramp):
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=1)
    _attention_case(ops, dtype, cfg, [1024, 2112], layer=0, seed=5, key_ramp=key_ramp)


@pytest.mark.parametrize("lens", [[1280], [512, 64, 2048]])
def test_sparse_attention_band(ops, lens):
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=1, pattern="band", band_half=4)
    _attention_case(ops, torch.bfloat16, cfg, lens, layer=0, seed=9)
