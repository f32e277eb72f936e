"""ctypes binding of the C ABI declared in include/raptor_b200.h.

The shared library is built in-tree by raptor_t_b200.build.  There is no CPU
implementation behind these calls: if the library is missing and cannot be
built, importing this module raises.
"""
import ctypes as C
import os

from . import build as _build

RT_OK = 0
RT_F16, RT_BF16 = 0, 1
RT_PATTERN_BIGBIRD, RT_PATTERN_BAND = 0, 1
RT_EPI_NONE, RT_EPI_BIAS, RT_EPI_BIAS_GELU = 0, 1, 2


class RtConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("heads", C.c_int32), ("ffn", C.c_int32), ("layers", C.c_int32),
        ("block", C.c_int32), ("num_rand", C.c_int32), ("max_pos", C.c_int32), ("vocab", C.c_int32),
        ("type_vocab", C.c_int32), ("pattern", C.c_int32), ("band_half", C.c_int32), ("dtype", C.c_int32),
        ("eps", C.c_float), ("reserved", C.c_int32),
    ]


class RtError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"raptor_b200 error {code}: {msg}")
        self.code = code


def _load():
    # RAPTOR_B200_LIB selects an explicitly built library (e.g. an instrumented build);
    # otherwise build() is a no-op when the library is newer than every source file
    path = os.environ.get("RAPTOR_B200_LIB") or _build.build(force=bool(os.environ.get("RAPTOR_B200_REBUILD")))
    return C.CDLL(path)


lib = _load()

_vp, _i32p, _i64p = C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64)
_cfgp = C.POINTER(RtConfig)

_SIGS = {
    "rt_last_error": (C.c_char_p, []),
    "rt_version": (C.c_int, []),
    "rt_check_device": (C.c_int, []),
    "rt_selftest_bounded_wait": (C.c_int, [C.c_int64, C.c_int, _vp]),
    "rt_kernel_launches": (C.c_int64, []),
    "rt_rand_block_table": (C.c_int, [C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p]),
    "rt_count_visits": (C.c_int, [_cfgp, _i32p, C.c_int, _i64p]),
    "rt_build_block_csr": (C.c_int, [_cfgp, C.c_uint32, _i32p, C.c_int, _i32p, _i32p]),
    "rt_seq_block_prefix": (C.c_int, [_i32p, C.c_int, C.c_int, _i32p]),
    "rt_lpt_partition": (C.c_int, [_i32p, C.c_int, _i32p, C.c_int, C.c_int, C.c_int, _i32p, _i32p]),
    "rt_binpack_sequences": (C.c_int, [C.POINTER(C.c_double), C.c_int, C.c_int, _i32p]),
    "rt_bias_residual_layernorm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_float, C.c_int, _vp]),
    "rt_bias_gelu": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "rt_qkv_bias_transpose": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _vp]),
    "rt_embeddings": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_float, C.c_int, _vp]),
    "rt_pooler": (C.c_int, [_vp, _vp, _vp, C.c_int, _vp, _vp, C.c_int, C.c_int, _vp]),
    "rt_gemm": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "rt_gemm_residual": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "rt_gemm_bias_residual_layernorm": (C.c_int, [_vp] * 7 + [C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _vp]),
    "rt_gemm_qkv": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _vp]),
    "rt_attn_plan_create": (C.c_int, [_cfgp, _i32p, C.c_int, _i32p, _i32p, C.c_int, C.c_int, _vp, C.POINTER(_vp)]),
    "rt_attn_plan_destroy": (C.c_int, [_vp]),
    "rt_attn_plan_build_host": (C.c_int, [_cfgp, C.c_uint32, _i32p, C.c_int, C.c_int, C.c_int, _i32p, C.c_int64, _i32p,
                                          C.c_int64, _i32p, _i64p, _i64p, _i64p]),
    "rt_attn_plan_stats": (C.c_int, [_vp, _i64p, _i64p, _i32p]),
    "rt_attn_plan_bounds": (C.c_int, [_cfgp, _i32p, C.c_int, C.c_int, _i64p, _i64p, _i64p, _i64p]),
    "rt_sparse_attention": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_float, C.c_int, _vp]),
    "rt_sparse_attention_static": (C.c_int, [_vp, _vp, _vp, _vp, _cfgp, _i32p, C.c_int, _i32p, _i32p, C.c_float, C.c_int,
                                             _vp]),
    "rt_encoder_create": (C.c_int, [_cfgp, C.POINTER(_vp)]),
    "rt_encoder_destroy": (C.c_int, [_vp]),
    "rt_encoder_set_layer": (C.c_int, [_vp, C.c_int, C.c_uint32, C.c_int] + [_vp] * 12),
    "rt_encoder_set_embeddings": (C.c_int, [_vp] * 6),
    "rt_encoder_set_option": (C.c_int, [_vp, C.c_char_p, C.c_int]),
    "rt_encoder_get_option": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_int)]),
    "rt_encoder_prepare_batch": (C.c_int, [_vp, _i32p, C.c_int]),
    "rt_encoder_forward_hidden": (C.c_int, [_vp, _vp, C.c_int, C.c_int, _vp]),
    "rt_encoder_forward_ids": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "rt_encoder_forward_host": (C.c_int, [_vp, _i32p, C.c_int, _vp, _vp]),
    "rt_encoder_submit_host": (C.c_int, [_vp, _i32p, C.c_int, _vp, _vp, C.POINTER(C.c_uint64)]),
    "rt_encoder_wait_host": (C.c_int, [_vp, C.c_uint64]),
    "rt_encoder_attention": (C.c_int, [_vp, C.c_int, _vp, _vp, _vp]),
    "rt_encoder_intermediate": (C.c_int, [_vp, C.c_int, _vp, _vp, _vp]),
    "rt_encoder_output": (C.c_int, [_vp, C.c_int, _vp, _vp, _vp, _vp]),
    "rt_encoder_get_table": (C.c_int, [_vp, C.c_int, C.POINTER(_i32p), C.POINTER(_i32p), _i64p]),
    "rt_encoder_plan_stats": (C.c_int, [_vp, C.c_int, _i64p, _i64p, _i32p]),
    "rt_encoder_get_scratch": (C.c_int, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(C.c_size_t)]),
    "rt_encoder_get_timing": (C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "rt_encoder_enable_timing": (C.c_int, [_vp, C.c_int]),
    "rt_encoder_kernel_launches": (C.c_int, [_vp, _i64p]),
}

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(status):
    if status != RT_OK:
        raise RtError(status, lib.rt_last_error().decode("utf-8", "replace"))


def i32_array(values):
    arr = (C.c_int32 * len(values))(*[int(v) for v in values])
    return arr


def make_config(hidden=768, heads=12, ffn=3072, layers=12, num_rand=3, max_pos=4096, vocab=50358, type_vocab=2,
                pattern="bigbird", band_half=4, dtype="bf16", eps=1e-12):
    return RtConfig(hidden=hidden, heads=heads, ffn=ffn, layers=layers, block=64, num_rand=num_rand, max_pos=max_pos,
                    vocab=vocab, type_vocab=type_vocab,
                    pattern=RT_PATTERN_BIGBIRD if pattern == "bigbird" else RT_PATTERN_BAND, band_half=band_half,
                    dtype=RT_BF16 if dtype in ("bf16", RT_BF16) else RT_F16, eps=eps, reserved=0)
