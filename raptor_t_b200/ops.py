"""Single CUDA kernels of the encoder on torch CUDA tensors (16-bit), through the C ABI.

torch is used for device memory and streams only; every function launches one
kernel of this library on the current torch stream and returns its output.
"""
import ctypes as C

import torch

from . import capi
from .capi import check, lib


def _dt(t):
    if t.dtype == torch.bfloat16:
        return capi.RT_BF16
    if t.dtype == torch.float16:
        return capi.RT_F16
    raise TypeError(f"expected float16 or bfloat16, got {t.dtype}")


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("raptor_t_b200 ops need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError("raptor_t_b200 ops need contiguous tensors")
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def bias_residual_layernorm(x, bias, residual, gamma, beta, eps, out=None):
    out = x if out is None else out
    rows, hidden = x.shape
    check(lib.rt_bias_residual_layernorm(_p(out), _p(x), _p(bias), _p(residual), _p(gamma), _p(beta), rows, hidden,
                                         float(eps), _dt(x), _stream()))
    return out


def bias_gelu_(x, bias):
    rows, cols = x.shape
    check(lib.rt_bias_gelu(_p(x), _p(bias), rows, cols, _dt(x), _stream()))
    return x


def qkv_bias_transpose(qkv, bias, seq_block_prefix_dev, heads, q_scale=0.125, out=None):
    T = qkv.shape[0]
    hidden = qkv.shape[1] // 3
    if out is None:
        out = tuple(torch.empty(T, hidden, dtype=qkv.dtype, device=qkv.device) for _ in range(3))
    q, k, v = out
    check(lib.rt_qkv_bias_transpose(_p(qkv), _p(bias), _p(q), _p(k), _p(v), _p(seq_block_prefix_dev),
                                    seq_block_prefix_dev.numel() - 1, T // 64, heads, float(q_scale), _dt(qkv),
                                    _stream()))
    return q, k, v


def embeddings(ids, pos_ids, type_ids, word, pos, typ, gamma, beta, eps, dtype, out=None):
    T, hidden = ids.numel(), word.shape[1]
    if out is None:
        out = torch.empty(T, hidden, dtype=dtype, device=ids.device)
    check(lib.rt_embeddings(_p(out), _p(ids), _p(pos_ids), _p(type_ids), _p(word), _p(pos), _p(typ), _p(gamma),
                            _p(beta), T, hidden, float(eps), _dt(out), _stream()))
    return out


def pooler(hidden, seq_block_prefix_dev, w, b, out=None):
    """pooled [n_seq, H] fp32 = tanh(hidden[first token of each sequence] @ w^T + b); w is [out, in]."""
    n_seq, H = seq_block_prefix_dev.numel() - 1, hidden.shape[1]
    if out is None:
        out = torch.empty(n_seq, H, dtype=torch.float32, device=hidden.device)
    check(lib.rt_pooler(_p(out), _p(hidden), _p(seq_block_prefix_dev), n_seq, _p(w), _p(b), H, _dt(hidden), _stream()))
    return out


def gemm(a, w, bias=None, epilogue=capi.RT_EPI_NONE, out=None):
    """out[M,N] = a[M,K] @ w[N,K]^T (+bias, +GELU); w is [out_features, in_features]."""
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    check(lib.rt_gemm(_p(out), _p(a), _p(w), _p(bias), M, N, K, epilogue, _dt(a), _stream()))
    return out


def gemm_residual(a, w, bias, residual, out=None):
    """out[M,N] = a @ w^T + bias + residual (pre-LayerNorm sum); out may alias residual."""
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    check(lib.rt_gemm_residual(_p(out), _p(a), _p(w), _p(bias), _p(residual), M, N, K, _dt(a), _stream()))
    return out


def gemm_bias_residual_layernorm(a, w, bias, residual, gamma, beta, eps, out=None):
    """out[M,N] = LayerNorm(a @ w^T + bias + residual) * gamma + beta in one kernel (N = 768 or 1024)."""
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    check(lib.rt_gemm_bias_residual_layernorm(_p(out), _p(a), _p(w), _p(bias), _p(residual), _p(gamma), _p(beta), M, N, K,
                                              float(eps), _dt(a), _stream()))
    return out


def block_seq_table(lens_tokens, device="cuda"):
    """int32 [N, 2]: for every packed 64-token block {first token of its sequence, sequence length}."""
    import numpy as np
    rows, t0 = [], 0
    for n in lens_tokens:
        rows += [[t0, int(n)]] * (int(n) // 64)
        t0 += int(n)
    return torch.from_numpy(np.asarray(rows, dtype=np.int32).reshape(-1, 2)).to(device)


def gemm_qkv(a, w, bias, block_seq, heads, q_scale=0.125, out=None):
    """Fused QKV projection + bias + query scale + head-major split (no [T,3H] intermediate)."""
    M, K = a.shape
    if out is None:
        out = tuple(torch.empty(M, heads * 64, dtype=a.dtype, device=a.device) for _ in range(3))
    q, k, v = out
    check(lib.rt_gemm_qkv(_p(q), _p(k), _p(v), _p(a), _p(w), _p(bias), _p(block_seq), M, heads, K, float(q_scale),
                          _dt(a), _stream()))
    return q, k, v


class AttentionPlan:
    """Device work list for rt_sparse_attention built from a CSR block table.
    split_entries: lists longer than this are cut into merged parts (0: never, -1: default)."""

    def __init__(self, cfg, lens_tokens, kv_ptr, kv_idx, n_ctas=0, split_entries=-1):
        import numpy as np
        lens = np.ascontiguousarray(lens_tokens, dtype=np.int32)
        kv_ptr = np.ascontiguousarray(kv_ptr, dtype=np.int32)
        kv_idx = np.ascontiguousarray(kv_idx, dtype=np.int32)
        self._h = C.c_void_p()
        i32p = C.POINTER(C.c_int32)
        check(lib.rt_attn_plan_create(C.byref(cfg), lens.ctypes.data_as(i32p), len(lens), kv_ptr.ctypes.data_as(i32p),
                                      kv_idx.ctypes.data_as(i32p), n_ctas, int(split_entries), _stream(),
                                      C.byref(self._h)))
        e, v, it = C.c_int64(), C.c_int64(), C.c_int32()
        check(lib.rt_attn_plan_stats(self._h, C.byref(e), C.byref(v), C.byref(it)))
        self.entries, self.visits, self.items = int(e.value), int(v.value), int(it.value)

    @property
    def handle(self):
        return self._h

    def close(self):
        if self._h:
            lib.rt_attn_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sparse_attention(q, k, v, plan, scale=1.0, out=None):
    """q,k,v head-major per sequence ([T, hidden] storage); returns token-major context [T, hidden]."""
    if out is None:
        out = torch.empty_like(q)
    check(lib.rt_sparse_attention(_p(out), _p(q), _p(k), _p(v), plan.handle, float(scale), _dt(q), _stream()))
    return out


def sparse_attention_static(q, k, v, cfg, lens_tokens, kv_ptr, kv_idx, scale=1.0, out=None):
    """Same result as sparse_attention, for callers that must not allocate device memory: the
    work list goes into the library's fixed device array instead of an AttentionPlan (see
    rt_sparse_attention_static in include/raptor_b200.h for the size limit and sharing rules).
    `out` must be given by such callers; it is only created here for convenience."""
    import numpy as np
    if out is None:
        out = torch.empty_like(q)
    lens = np.ascontiguousarray(lens_tokens, dtype=np.int32)
    kv_ptr = np.ascontiguousarray(kv_ptr, dtype=np.int32)
    kv_idx = np.ascontiguousarray(kv_idx, dtype=np.int32)
    i32p = C.POINTER(C.c_int32)
    check(lib.rt_sparse_attention_static(_p(out), _p(q), _p(k), _p(v), C.byref(cfg), lens.ctypes.data_as(i32p),
                                         len(lens), kv_ptr.ctypes.data_as(i32p), kv_idx.ctypes.data_as(i32p),
                                         float(scale), _dt(q), _stream()))
    return out


def check_device():
    """Synchronise and raise if any kernel gave up on a bounded device-side wait."""
    check(lib.rt_check_device())


def selftest_bounded_wait(limit_cycles=1_000_000, target=0):
    """Launch the library's self-test kernel whose only wait runs out after `limit_cycles` SM
    clocks; it returns normally and leaves site 901 in the error word (target 0: the word
    check_device() reads; 1: the status word of sparse_attention_static)."""
    check(lib.rt_selftest_bounded_wait(int(limit_cycles), int(target), _stream()))
