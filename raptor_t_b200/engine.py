"""Whole-encoder object: one C call per forward (weights, scratch, metadata pipeline in C++)."""
import ctypes as C

import numpy as np
import torch

from . import capi
from .capi import check, lib

_LAYER_KEYS = [
    "attention.self.query", "attention.self.key", "attention.self.value", "attention.output.dense",
    "attention.output.LayerNorm", "intermediate.dense", "output.dense", "output.LayerNorm",
]


def _ptr(t):
    return C.c_void_p(t.data_ptr())


class Encoder:
    """B200 encoder.  `cfg` is a capi.RtConfig; weights come as a dict with the parameter
    names of the reference's validation model (HuggingFace BigBird state_dict names,
    torch Linear layout [out, in])."""

    def __init__(self, cfg, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("raptor_t_b200.Encoder needs a CUDA device (there is no CPU path)")
        self.cfg = cfg
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dtype = torch.bfloat16 if cfg.dtype == capi.RT_BF16 else torch.float16
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.rt_encoder_create(C.byref(cfg), C.byref(self._h)))
        self.tokens = 0

    # ---- weights ------------------------------------------------------------
    def load_weights(self, P, layer_seeds=None):
        dev, dt = self.device, self.dtype
        with torch.cuda.device(dev):
            for i in range(self.cfg.layers):
                pre = f"encoder.layer.{i}."
                g = lambda k: P[pre + k].to(device=dev, dtype=dt).contiguous()  # noqa: E731
                qkv_w = torch.cat([g("attention.self.query.weight"), g("attention.self.key.weight"),
                                   g("attention.self.value.weight")], 0).contiguous()
                qkv_b = torch.cat([g("attention.self.query.bias"), g("attention.self.key.bias"),
                                   g("attention.self.value.bias")], 0).contiguous()
                ts = [qkv_w, qkv_b, g("attention.output.dense.weight"), g("attention.output.dense.bias"),
                      g("attention.output.LayerNorm.weight"), g("attention.output.LayerNorm.bias"),
                      g("intermediate.dense.weight"), g("intermediate.dense.bias"), g("output.dense.weight"),
                      g("output.dense.bias"), g("output.LayerNorm.weight"), g("output.LayerNorm.bias")]
                seed = i if layer_seeds is None else int(layer_seeds[i])
                check(lib.rt_encoder_set_layer(self._h, i, seed, 0, *[_ptr(t) for t in ts]))
            if "embeddings.word_embeddings.weight" in P:
                f = lambda k: P["embeddings." + k].to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
                ts = [f("word_embeddings.weight"), f("position_embeddings.weight"), f("token_type_embeddings.weight"),
                      f("LayerNorm.weight"), f("LayerNorm.bias")]
                check(lib.rt_encoder_set_embeddings(self._h, *[_ptr(t) for t in ts]))
            torch.cuda.synchronize()
        return self

    def set_option(self, name, value):
        check(lib.rt_encoder_set_option(self._h, name.encode(), int(value)))

    def get_option(self, name):
        v = C.c_int()
        check(lib.rt_encoder_get_option(self._h, name.encode(), C.byref(v)))
        return int(v.value)

    def layernorm_in_projection(self):
        """Which of the two hidden-wide projections carry their LayerNorm in the current configuration:
        (attention output, FFN down)."""
        mode, H, F = self.get_option("fuse_layernorm"), self.cfg.hidden, self.cfg.ffn
        both = mode == 2 and H in (768, 1024)
        return both, both or (mode == 1 and H == 768 and F >= 2048)

    # ---- per batch -------------------------------------------------------------
    def prepare(self, lens_tokens):
        lens = np.ascontiguousarray(lens_tokens, dtype=np.int32)
        with torch.cuda.device(self.device):
            check(lib.rt_encoder_prepare_batch(self._h, lens.ctypes.data_as(C.POINTER(C.c_int32)), len(lens)))
        self.tokens = int(lens.sum())
        return self

    def forward_hidden(self, hidden, layer_begin=0, layer_end=None):
        """hidden [T, H] CUDA tensor, updated in place."""
        assert hidden.is_cuda and hidden.is_contiguous() and hidden.dtype == self.dtype
        assert hidden.shape == (self.tokens, self.cfg.hidden)
        end = self.cfg.layers if layer_end is None else layer_end
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.rt_encoder_forward_hidden(self._h, _ptr(hidden), layer_begin, end, st))
        return hidden

    def forward_ids(self, ids, out=None, pos_ids=None, type_ids=None):
        assert ids.is_cuda and ids.dtype == torch.int32 and ids.numel() == self.tokens
        if out is None:
            out = torch.empty(self.tokens, self.cfg.hidden, dtype=self.dtype, device=ids.device)
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.rt_encoder_forward_ids(self._h, _ptr(ids), None if pos_ids is None else _ptr(pos_ids),
                                         None if type_ids is None else _ptr(type_ids), _ptr(out), st))
        return out

    def forward_host(self, lens_tokens, ids_host, out_host):
        """End to end on HOST buffers: ids_host int32 CPU tensor (pinned for speed),
        out_host 16-bit CPU tensor [T, H]; returns when out_host is filled."""
        lens = np.ascontiguousarray(lens_tokens, dtype=np.int32)
        assert not ids_host.is_cuda and ids_host.dtype == torch.int32 and not out_host.is_cuda
        self.tokens = int(lens.sum())
        with torch.cuda.device(self.device):
            check(lib.rt_encoder_forward_host(self._h, lens.ctypes.data_as(C.POINTER(C.c_int32)), len(lens),
                                              _ptr(ids_host), _ptr(out_host)))
        return out_host

    def submit_host(self, lens_tokens, ids_host, out_host):
        """First half of forward_host: enqueues the batch and returns a ticket at once.  Up to
        two batches are in flight; the device-to-host copy of one overlaps the kernels of the
        next.  ids_host / out_host (pinned) must stay untouched until wait_host(ticket)."""
        lens = np.ascontiguousarray(lens_tokens, dtype=np.int32)
        assert not ids_host.is_cuda and ids_host.dtype == torch.int32 and not out_host.is_cuda
        self.tokens = int(lens.sum())
        ticket = C.c_uint64(0)
        with torch.cuda.device(self.device):
            check(lib.rt_encoder_submit_host(self._h, lens.ctypes.data_as(C.POINTER(C.c_int32)), len(lens),
                                             _ptr(ids_host), _ptr(out_host), C.byref(ticket)))
        return ticket.value

    def wait_host(self, ticket):
        """Second half: returns when the output of that batch is in its out_host buffer."""
        with torch.cuda.device(self.device):
            check(lib.rt_encoder_wait_host(self._h, C.c_uint64(ticket)))

    # ---- the three operators of the reference's pybind module -------------------------
    def attention(self, layer, x, out):
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.rt_encoder_attention(self._h, layer, _ptr(x), _ptr(out), st))
        return out

    def intermediate(self, layer, x, out):
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.rt_encoder_intermediate(self._h, layer, _ptr(x), _ptr(out), st))
        return out

    def output(self, layer, ffn, residual, out):
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.rt_encoder_output(self._h, layer, _ptr(ffn), _ptr(residual), _ptr(out), st))
        return out

    # ---- introspection ----------------------------------------------------------
    def table(self, layer):
        kp, ki, v = C.POINTER(C.c_int32)(), C.POINTER(C.c_int32)(), C.c_int64()
        check(lib.rt_encoder_get_table(self._h, layer, C.byref(kp), C.byref(ki), C.byref(v)))
        n_blocks = self.tokens // 64
        kv_ptr = np.ctypeslib.as_array(kp, shape=(n_blocks + 1,)).copy()
        kv_idx = np.ctypeslib.as_array(ki, shape=(self.cfg.heads, int(v.value))).copy()
        return kv_ptr, kv_idx

    def plan_stats(self, layer=0):
        e, v, it = C.c_int64(), C.c_int64(), C.c_int32()
        check(lib.rt_encoder_plan_stats(self._h, layer, C.byref(e), C.byref(v), C.byref(it)))
        return {"entries": int(e.value), "visits": int(v.value), "items": int(it.value)}

    def enable_timing(self, on=True):
        check(lib.rt_encoder_enable_timing(self._h, int(on)))

    def timing(self):
        out = {}
        for key in ("gemm", "gemm.qkv", "gemm.attention_output", "gemm.ffn_up", "gemm.ffn_down",
                    "add_bias_and_transpose_kernel", "attention", "add_bias_and_layernorm_kernel",
                    "add_bias_act_kernel", "embeddings", "pre_process"):
            ms = C.c_float()
            check(lib.rt_encoder_get_timing(self._h, key.encode(), C.byref(ms)))
            out[key] = float(ms.value)
        return out

    def host_blocked_ms(self):
        """Cumulative time the calling thread spent waiting for the GPU to release a slot or buffer."""
        ms = C.c_float()
        check(lib.rt_encoder_get_timing(self._h, b"host_blocked", C.byref(ms)))
        return float(ms.value)

    def close(self):
        if self._h:
            lib.rt_encoder_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def kernel_launches():
    return int(lib.rt_kernel_launches())
