"""Host metadata through the C ABI (numpy in / numpy out, no GPU needed).

Mirrors python/util.py of the reference (generate_data_metainfo,
generate_parition_plan) and the block-table generator of
layers/multi_headed_attention.cpp, with tables that are bit-exact with the
reference's validation model.
"""
import ctypes as C

import numpy as np

from . import capi
from .capi import check, lib


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def rand_block_table(seed, heads, n_blocks, num_rand=3, max_pos=4096, block=64):
    out = np.zeros((heads, n_blocks - 2, num_rand), dtype=np.int32)
    check(lib.rt_rand_block_table(int(seed), heads, n_blocks, num_rand, max_pos, block,
                                  out.ctypes.data_as(C.POINTER(C.c_int32))))
    return out


def count_visits(cfg, lens_tokens):
    lens, lp = _i32(lens_tokens)
    v = C.c_int64(0)
    check(lib.rt_count_visits(C.byref(cfg), lp, len(lens), C.byref(v)))
    return int(v.value)


def build_block_csr(cfg, layer_seed, lens_tokens):
    """-> (kv_ptr int32 [N+1], kv_idx int32 [heads, visits])"""
    lens, lp = _i32(lens_tokens)
    visits = count_visits(cfg, lens)
    n_blocks = int(lens.sum()) // cfg.block
    kv_ptr = np.zeros(n_blocks + 1, dtype=np.int32)
    kv_idx = np.zeros((cfg.heads, visits), dtype=np.int32)
    check(lib.rt_build_block_csr(C.byref(cfg), int(layer_seed), lp, len(lens),
                                 kv_ptr.ctypes.data_as(C.POINTER(C.c_int32)),
                                 kv_idx.ctypes.data_as(C.POINTER(C.c_int32))))
    return kv_ptr, kv_idx


def seq_block_prefix(lens_tokens, block=64):
    lens, lp = _i32(lens_tokens)
    out = np.zeros(len(lens) + 1, dtype=np.int32)
    check(lib.rt_seq_block_prefix(lp, len(lens), block, out.ctypes.data_as(C.POINTER(C.c_int32))))
    return out


def lpt_partition(cost_per_qblock, seq_prefix, n_parts, heads):
    cost, cp = _i32(cost_per_qblock)
    pref, pp = _i32(seq_prefix)
    off = np.zeros(n_parts + 1, dtype=np.int32)
    ids = np.zeros(heads * len(cost), dtype=np.int32)
    check(lib.rt_lpt_partition(cp, len(cost), pp, len(pref) - 1, n_parts, heads,
                               off.ctypes.data_as(C.POINTER(C.c_int32)), ids.ctypes.data_as(C.POINTER(C.c_int32))))
    return off, ids


def binpack_sequences(costs, n_bins):
    c = np.ascontiguousarray(costs, dtype=np.float64)
    out = np.zeros(len(c), dtype=np.int32)
    check(lib.rt_binpack_sequences(c.ctypes.data_as(C.POINTER(C.c_double)), len(c), n_bins,
                                   out.ctypes.data_as(C.POINTER(C.c_int32))))
    return out


def generate_data_metainfo(seq_lens_tokens, block_size=64, thread_block_limit=160, heads=12):
    """python/util.py:36-50: (seq_position_info list, total_comp_block_num,
    partition_part_index int32 [limit+1], partition_part int32 [heads*N]) - host arrays."""
    blocks = [int(n) // block_size for n in seq_lens_tokens]
    cost = []
    for L in blocks:
        cost += [L, 7] + [8] * (L - 4) + [7, L]
    prefix = seq_block_prefix(seq_lens_tokens, block_size)
    off, ids = lpt_partition(cost, prefix, thread_block_limit, heads)
    return [int(x) for x in prefix], int(sum(cost)), off, ids


def sequence_cost(n_tokens, hidden, ffn, heads, visits_per_head):
    """FLOPs of one sequence in one layer: GEMMs + listed attention blocks."""
    return float(n_tokens) * (8 * hidden * hidden + 4 * hidden * ffn) + float(heads) * 1048576.0 * visits_per_head


def attention_plan_host(cfg, layer_seed, lens_tokens, n_ctas, use_templates=True):
    """Host-only work list: dict(items [n,8], entries [m], cta_ptr [n_ctas+1], visits)."""
    lens, lp = _i32(lens_tokens)
    ni, ne, vis = C.c_int64(), C.c_int64(), C.c_int64()
    i32p = C.POINTER(C.c_int32)
    check(lib.rt_attn_plan_build_host(C.byref(cfg), int(layer_seed), lp, len(lens), n_ctas, int(use_templates), None, 0,
                                      None, 0, None, C.byref(ni), C.byref(ne), C.byref(vis)))
    items = np.zeros((ni.value, 8), dtype=np.int32)
    entries = np.zeros(ne.value, dtype=np.int32)
    cta_ptr = np.zeros(n_ctas + 1, dtype=np.int32)
    check(lib.rt_attn_plan_build_host(C.byref(cfg), int(layer_seed), lp, len(lens), n_ctas, int(use_templates),
                                      items.ctypes.data_as(i32p), ni.value, entries.ctypes.data_as(i32p), ne.value,
                                      cta_ptr.ctypes.data_as(i32p), C.byref(ni), C.byref(ne), C.byref(vis)))
    return {"items": items, "entries": entries, "cta_ptr": cta_ptr, "visits": int(vis.value)}


def attention_plan_bounds(cfg, lens_tokens, split_entries=-1):
    """Upper bounds of a batch's work-list sizes for any table seed: dict(items, entries, slots, groups)."""
    lens, lp = _i32(lens_tokens)
    out = [C.c_int64() for _ in range(4)]
    check(lib.rt_attn_plan_bounds(C.byref(cfg), lp, len(lens), int(split_entries), *[C.byref(o) for o in out]))
    return dict(zip(("items", "entries", "slots", "groups"), (int(o.value) for o in out)))
