"""The reference's operator API (its pybind module `raptor_t`, python/pybind.cpp:11-80)
on top of this library's C ABI.

Same class names, constructor arguments, call arguments and in-place output
convention as the reference:

    BertAttention(qkv_weight[H,3H], qkv_bias, dense_weight[H,H], dense_bias, ln_weight, ln_bias,
                  num_attention_heads, layer_idx, async_)
        (input[T,H], attention_mask, output[T,H], seq_position_info, seq_len_info_tensor,
         partition_part_index_tensor, partition_part_tensor, block_limit, info,
         kernel_fusion=True, balanced=True) -> info
    BertIntermediate(dense_weight[H,F], dense_bias)(input, output, info, kernel_fusion=True) -> info
    BertOutput(dense_weight[F,H], dense_bias, ln_weight, ln_bias)
        (hidden_states[T,F], input_tensor[T,H], output[T,H], info, kernel_fusion=True) -> info
    TensorSet(total_seq_len, to_select_index_len, to_select_index_position_len)
    MetaData().update_meta_data(T, to_select_index_len, to_select_index_position_len, seq_len_info)
    multi_headed_attention = the base class of BertAttention (python/pybind.cpp:23-37)

Weights arrive [in, out] (python/modeling_bert.py:84-91,107-113,138-163) and are
re-laid-out once to [out, in] for the TMA-fed GEMM.  Differences on purpose: the
block table is the validation model's deterministic per-head table (seeded by
layer_idx) instead of a std::random_device shuffle; accumulation and LayerNorm
statistics are fp32; LayerNorm eps is a module attribute (default 1e-12, the model's
value) instead of the hard-coded 1e-5 of layers/bert_output.cpp:23; the context is
written token-major so that the output projection sees the layout it expects.
The partition tensors and block_limit are accepted for signature compatibility; the
kernel's own work list (pairs of query blocks per CTA) is built from the block table.
"""
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

from . import capi, metadata, ops

LAYER_NORM_EPS = 1e-12
_INFO_KEYS = ("pre_process", "attention", "add_bias_act_kernel", "add_bias_and_layernorm_kernel",
              "add_bias_and_transpose_kernel")


def _accumulate(info, key, fn):
    """Run fn(); if `info` carries `key`, add the kernel's device time in seconds
    (the reference adds host time under CUDA_LAUNCH_BLOCKING=1, layers/kernels/add_bias_act.cu:129-132)."""
    if info is None or key not in info:
        return fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = fn()
    b.record()
    b.synchronize()
    info[key] += a.elapsed_time(b) * 1e-3
    return out


class TensorSet:
    """Process-wide scratch buffers resized per batch (layers/tensor_set.h:36-65).
    Buffers are allocated on first use, so the bookkeeping also works without a GPU."""
    _instance = None
    _lock = threading.RLock()

    def __init__(self, total_seq_len=4096, to_select_index_len=622, to_select_index_position_len=65,
                 hidden=768, dtype=torch.float16):
        self.hidden, self.dtype = hidden, dtype
        self.total_seq_len = int(total_seq_len)
        self.capacity = 0
        self.seq_len_info = [0]
        self.to_select_index_len = to_select_index_len
        self.to_select_index_position_len = to_select_index_position_len
        self.tensors = {}
        self.generation = 0
        with TensorSet._lock:
            if TensorSet._instance is None:
                TensorSet._instance = self

    @staticmethod
    def get_instance():
        with TensorSet._lock:
            if TensorSet._instance is None:
                TensorSet._instance = TensorSet()
            return TensorSet._instance

    def configure(self, hidden, dtype):
        if (hidden, dtype) != (self.hidden, self.dtype):
            self.hidden, self.dtype = hidden, dtype
            self.tensors, self.capacity = {}, 0

    def _ensure(self):
        if self.tensors and self.capacity >= self.total_seq_len:
            return
        if not torch.cuda.is_available():
            raise RuntimeError("raptor_t needs a CUDA device (there is no CPU path)")
        T, H = max(self.total_seq_len, 1), self.hidden
        mk = lambda cols: torch.empty(T, cols, dtype=self.dtype, device="cuda")  # noqa: E731
        self.tensors = {"q_out": mk(H), "k_out": mk(H), "v_out": mk(H), "attention_out": mk(H),
                        "tmp_qkv_out1": mk(3 * H), "dense_out": mk(H)}
        self.capacity = T

    def update_tensor_set(self, total_seq_len, to_select_index_len, to_select_index_position_len, seq_len_info=None):
        self.total_seq_len = int(total_seq_len)
        self.to_select_index_len = to_select_index_len
        self.to_select_index_position_len = to_select_index_position_len
        if seq_len_info is not None:
            self.seq_len_info = [int(x) for x in seq_len_info]
        self.generation += 1

    _NAMES = ("q_out", "k_out", "v_out", "attention_out", "tmp_qkv_out1", "dense_out")

    def get_tensor(self, name):
        if name not in TensorSet._NAMES:
            print("no exists tensor")  # layers/tensor_set.cpp:30-33
            return torch.empty(0)
        self._ensure()
        return self.tensors[name][: self.total_seq_len]

    def lens_tokens(self):
        p = self.seq_len_info
        return [(p[i + 1] - p[i]) * 64 for i in range(len(p) - 1)]


class MetaData:
    """Per-batch kick of the metadata pipeline (layers/metadata.cpp:6-18).  Every
    registered attention layer gets a worker job that builds its block table and
    work list and uploads them; the layer waits for it right before its attention
    kernel, after the QKV GEMM has been queued."""
    _layers = []
    _pool = None
    _lock = threading.Lock()

    @classmethod
    def register_layer(cls, layer):
        with cls._lock:
            cls._layers.append(layer)

    def update_meta_data(self, total_seq_len, to_select_index_len, to_select_index_position_len, seq_len_info):
        ts = TensorSet.get_instance()
        ts.update_tensor_set(total_seq_len, to_select_index_len, to_select_index_position_len, seq_len_info)
        lens = ts.lens_tokens()
        if sum(lens) != int(total_seq_len):
            raise ValueError("update_meta_data: seq_len_info does not add up to total_seq_len")
        with MetaData._lock:
            layers = list(MetaData._layers)
            if MetaData._pool is None:
                MetaData._pool = ThreadPoolExecutor(max_workers=4, thread_name_prefix="raptor_meta")
        device = torch.cuda.current_device() if torch.cuda.is_available() else None
        for layer in layers:
            if layer.async_:
                layer._pending = MetaData._pool.submit(layer._build_plan, lens, device)
            else:
                layer._pending = None
                layer._lens = lens

    def terminate_thread(self):
        with MetaData._lock:
            if MetaData._pool is not None:
                MetaData._pool.shutdown(wait=True)
                MetaData._pool = None
            MetaData._layers = []


def _dtype_name(t):
    return "bf16" if t == torch.bfloat16 else "f16"


class multi_headed_attention:
    """layers/multi_headed_attention.{h,cpp}: QKV GEMM -> bias/scale/transpose -> block-sparse
    attention -> output GEMM -> residual + bias + LayerNorm."""

    def __init__(self, qkv_weight, qkv_bias, dense_weight, dense_bias, layer_norm_weight, layer_norm_bias,
                 num_attention_heads, layer_idx=0, async_=True, num_rand=3, max_pos=4096, pattern="bigbird",
                 band_half=4, eps=LAYER_NORM_EPS):
        self.heads = int(num_attention_heads)
        self.hidden = qkv_weight.shape[0]
        if self.hidden != self.heads * 64:
            raise ValueError("head size must be 64")
        self.dtype = qkv_weight.dtype
        self.qkv_w = qkv_weight.t().contiguous()      # [3H, H]
        self.qkv_b = qkv_bias.contiguous()
        self.dense_w = dense_weight.t().contiguous()  # [H, H] as [out, in]
        self.dense_b = dense_bias.contiguous()
        self.ln_w, self.ln_b = layer_norm_weight.contiguous(), layer_norm_bias.contiguous()
        self.layer_idx, self.async_, self.eps = int(layer_idx), bool(async_), eps
        self.cfg = capi.make_config(hidden=self.hidden, heads=self.heads, ffn=4 * self.hidden, layers=1,
                                    num_rand=num_rand, max_pos=max_pos, pattern=pattern, band_half=band_half,
                                    dtype=_dtype_name(self.dtype))
        self._pending, self._lens, self._plan, self._prefix = None, None, None, None
        self._side = None
        MetaData.register_layer(self)

    def _build_plan(self, lens, device):
        with torch.cuda.device(device):
            if self._side is None:
                self._side = torch.cuda.Stream()
            kv_ptr, kv_idx = metadata.build_block_csr(self.cfg, self.layer_idx, lens)
            with torch.cuda.stream(self._side):
                plan = ops.AttentionPlan(self.cfg, lens, kv_ptr, kv_idx)
                prefix = torch.from_numpy(metadata.seq_block_prefix(lens)).to("cuda", non_blocking=False)
                ready = torch.cuda.Event()
                ready.record(self._side)
            return plan, prefix, ready

    def __call__(self, input_tensor, attention_mask, output, seq_position_info, seq_len_info_tensor,
                 partition_part_index_tensor=None, partition_part_tensor=None, block_limit=0, info=None,
                 kernel_fusion=True, balanced=True):
        ts = TensorSet.get_instance()
        ts.configure(self.hidden, self.dtype)
        T = input_tensor.shape[0]
        qkv = ts.get_tensor("tmp_qkv_out1")[:T]
        q, k, v = (ts.get_tensor(n)[:T] for n in ("q_out", "k_out", "v_out"))
        ctx, dense = ts.get_tensor("attention_out")[:T], ts.get_tensor("dense_out")[:T]
        ops.gemm(input_tensor, self.qkv_w, out=qkv)
        _accumulate(info, "add_bias_and_transpose_kernel",
                    lambda: ops.qkv_bias_transpose(qkv, self.qkv_b, seq_len_info_tensor, self.heads, 0.125,
                                                   out=(q, k, v)))
        t0 = time.perf_counter()
        if self._pending is not None:
            self._plan, self._prefix, ready = self._pending.result()
            self._pending = None
            torch.cuda.current_stream().wait_event(ready)
        elif self._lens is not None:
            self._plan, self._prefix, ready = self._build_plan(self._lens, torch.cuda.current_device())
            self._lens = None
            torch.cuda.current_stream().wait_event(ready)
        if self._plan is None:
            raise RuntimeError("BertAttention called before MetaData.update_meta_data")
        if info is not None and "pre_process" in info:
            info["pre_process"] += time.perf_counter() - t0
        _accumulate(info, "attention", lambda: ops.sparse_attention(q, k, v, self._plan, scale=1.0, out=ctx))
        ops.gemm(ctx, self.dense_w, out=dense)
        _accumulate(info, "add_bias_and_layernorm_kernel",
                    lambda: ops.bias_residual_layernorm(dense, self.dense_b, input_tensor, self.ln_w, self.ln_b,
                                                        self.eps, out=output))
        return info


class BertAttention(multi_headed_attention):
    """layers/bert_attention.{h,cpp}: the attention sub-layer of one encoder layer."""


class BertIntermediate:
    """layers/bert_intermediate.{h,cpp}: GEMM [T,H]x[H,F] then bias + GELU."""

    def __init__(self, dense_weight, dense_bias):
        self.w = dense_weight.t().contiguous()  # [F, H]
        self.b = dense_bias.contiguous()

    def __call__(self, input_tensor, output, info=None, kernel_fusion=True):
        if kernel_fusion and (info is None or "add_bias_act_kernel" not in info):
            ops.gemm(input_tensor, self.w, self.b, capi.RT_EPI_BIAS_GELU, out=output)
        else:
            ops.gemm(input_tensor, self.w, out=output)
            _accumulate(info, "add_bias_act_kernel", lambda: ops.bias_gelu_(output, self.b))
        return info


class BertOutput:
    """layers/bert_output.{h,cpp}: GEMM [T,F]x[F,H] then residual + bias + LayerNorm;
    `output` may alias the layer's input buffer (python/modeling_bert.py:205-207)."""

    def __init__(self, dense_weight, dense_bias, layer_norm_weight, layer_norm_bias, eps=LAYER_NORM_EPS):
        self.w = dense_weight.t().contiguous()  # [H, F]
        self.b = dense_bias.contiguous()
        self.ln_w, self.ln_b, self.eps = layer_norm_weight.contiguous(), layer_norm_bias.contiguous(), eps

    def __call__(self, hidden_states, input_tensor, output, info=None, kernel_fusion=True):
        ts = TensorSet.get_instance()
        dense = ts.get_tensor("dense_out")[: hidden_states.shape[0]]
        ops.gemm(hidden_states, self.w, out=dense)
        _accumulate(info, "add_bias_and_layernorm_kernel",
                    lambda: ops.bias_residual_layernorm(dense, self.b, input_tensor, self.ln_w, self.ln_b, self.eps,
                                                        out=output))
        return info
