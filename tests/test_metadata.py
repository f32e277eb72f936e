"""Host metadata of the CUDA library (C++ through the C ABI) against the oracle and
the reference-generated golden tables.  Bit-exact; runs without a GPU."""
import os

import numpy as np
import pytest

import oracle
from oracle import EncoderConfig
from raptor_t_b200 import capi, metadata


def _cfg(o: EncoderConfig):
    return capi.make_config(hidden=o.hidden, heads=o.heads, ffn=o.ffn, layers=o.layers, num_rand=o.num_rand,
                            max_pos=o.max_pos, vocab=o.vocab, pattern=o.pattern, band_half=o.band_half)


def test_tables_match_reference_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "tables.npz"))
    n = 0
    for key in z.files:
        s, h, L, m = key.split("_")
        seed, heads, L, max_pos = int(s[1:]), int(h[1:]), int(L[1:]), int(m[1:])
        ref = z[key]
        if int(ref.max()) >= L:
            with pytest.raises(capi.RtError):
                metadata.rand_block_table(seed, heads, L, 3, max_pos)
            continue
        got = metadata.rand_block_table(seed, heads, L, 3, max_pos)
        assert np.array_equal(got, ref), key
        n += 1
    assert n > 200


@pytest.mark.parametrize("L", [13, 14, 15, 16, 17, 24, 33, 64, 100, 128])
def test_tables_match_oracle_other_seeds(L):
    for seed in (2, 11, 12345):
        for heads, max_pos in ((12, 8192), (16, 8192)):
            assert np.array_equal(metadata.rand_block_table(seed, heads, L, 3, max_pos),
                                  oracle.rand_block_table(seed, heads, L, 3, max_pos))


def test_rejected_lengths():
    with pytest.raises(capi.RtError):
        metadata.rand_block_table(0, 12, 12, 3, 4096)          # 768 tokens: ids beyond the sequence
    with pytest.raises(capi.RtError):
        metadata.rand_block_table(0, 12, 8, 3, 4096)           # full-attention length: no table
    cfg = _cfg(EncoderConfig())
    with pytest.raises(capi.RtError):
        metadata.build_block_csr(cfg, 0, [1000])               # not a multiple of 64
    with pytest.raises(capi.RtError):
        metadata.build_block_csr(cfg, 0, [8192])               # beyond max_pos
    with pytest.raises(capi.RtError):
        metadata.build_block_csr(cfg, 0, [])                   # empty batch


@pytest.mark.parametrize("pattern", ["bigbird", "band"])
def test_csr_matches_oracle(pattern):
    o = EncoderConfig(pattern=pattern)
    cfg = _cfg(o)
    lens = [1024, 832, 4096, 512, 704, 1984, 64, 128]
    for layer in (0, 5):
        ptr, idx = metadata.build_block_csr(cfg, layer, lens)
        optr, oidx = oracle.build_block_csr(lens, o, layer)
        assert np.array_equal(ptr, optr) and np.array_equal(idx, oidx)
    assert metadata.count_visits(cfg, lens) == oracle.visits_per_head(lens, o)
    assert list(metadata.seq_block_prefix(lens)) == oracle.seq_block_prefix(lens)


def test_csr_large_heads16():
    o = EncoderConfig(hidden=1024, heads=16, ffn=4096, max_pos=8192)
    cfg = _cfg(o)
    lens = [8192, 6400, 832, 2048]
    ptr, idx = metadata.build_block_csr(cfg, 3, lens)
    optr, oidx = oracle.build_block_csr(lens, o, 3)
    assert np.array_equal(ptr, optr) and np.array_equal(idx, oidx)


def test_reference_structural_fixture():
    # layers/test.cpp:80-107: one 64-block sequence, 160 CTAs
    cfg = _cfg(EncoderConfig())
    ptr, idx = metadata.build_block_csr(cfg, 0, [4096])
    assert ptr.shape == (65,) and idx.shape == (12, 622) and ptr[-1] == 622
    prefix, total, off, ids = metadata.generate_data_metainfo([4096], 64, 160, 12)
    assert prefix == [0, 64] and total == 622 and off.shape == (161,) and ids.shape == (768,)
    assert sorted(ids.tolist()) == list(range(768))


@pytest.mark.parametrize("lens,parts", [([4096], 160), ([1024, 2048, 832, 4096], 160), ([3584] * 8, 720)])
def test_lpt_partition_matches_oracle(lens, parts):
    cost = []
    for n in lens:
        L = n // 64
        cost += [L, 7] + [8] * (L - 4) + [7, L]
    prefix = oracle.seq_block_prefix(lens)
    off, ids = metadata.lpt_partition(cost, prefix, parts, 12)
    ooff, oids = oracle.lpt_partition(cost, prefix, parts, 12)
    assert off.tolist() == ooff and ids.tolist() == oids


def test_binpack_matches_oracle():
    rng = np.random.default_rng(1)
    costs = rng.lognormal(7.6, 0.6, size=256)
    for n in (1, 2, 4, 8):
        bins = metadata.binpack_sequences(costs, n)
        obins = oracle.binpack_sequences(list(costs), n)
        for b, members in enumerate(obins):
            assert sorted(np.nonzero(bins == b)[0].tolist()) == sorted(members)
        loads = [costs[bins == b].sum() for b in range(n)]
        assert max(loads) / (costs.sum() / n) < 1.05


@pytest.mark.parametrize("pattern,lens", [("bigbird", [1024, 832, 4096, 512, 704, 1984, 64, 128]),
                                          ("band", [1280, 64, 512, 2048]), ("bigbird", [960]),
                                          ("bigbird", [4096]), ("bigbird", [2048, 4096])])
@pytest.mark.parametrize("use_templates", [0, 1, 2])
def test_attention_work_list_covers_every_block_list_once(pattern, lens, use_templates):
    """Every (sequence, head, query block) appears in exactly one work item and the masked
    entries of that item reproduce its key/value list as a multiset."""
    from collections import Counter
    o = EncoderConfig(pattern=pattern)
    cfg = _cfg(o)
    layer, n_ctas = 3, 296
    plan = metadata.attention_plan_host(cfg, layer, lens, n_ctas, use_templates)
    items, entries, cta_ptr = plan["items"], plan["entries"], plan["cta_ptr"]
    assert cta_ptr[0] == 0 and cta_ptr[-1] == len(items) and np.all(np.diff(cta_ptr) >= 0)
    starts = np.concatenate([[0], np.cumsum(lens)])
    seen = set()
    visits = 0
    expected = {}
    for s, n in enumerate(lens):
        L = n // 64
        rand = None
        if pattern == "bigbird" and L > 11:
            rand = oracle.rand_block_table(layer, o.heads, L, 3, o.max_pos)
        for h in range(o.heads):
            for q, lst in enumerate(oracle.kv_block_lists(L, o, rand, h)):
                expected[(s, h, q)] = Counter(lst)
    got = {}
    slots = set()
    for q_row0, q_row1, kv_row0, off, n_ent, tok0, tok1, head_field in items.tolist():
        head, slot = head_field & 255, (head_field >> 8) - 1
        if slot >= 0:
            # one part of a split list: no longer than 24 entries or one CTA's share of the batch
            # (+1: parts are whole two-entry steps), and with a scratch slot of its own
            assert n_ent <= max(24, -(-(len(entries) + 2 * len(items)) // n_ctas)) + 1 and slot not in slots
            slots.add(slot)
        s = int(np.searchsorted(starts, tok0, side="right") - 1)
        n = lens[s]
        assert kv_row0 == starts[s] * o.heads + head * n
        qa = (tok0 - starts[s]) // 64
        assert q_row0 == kv_row0 + qa * 64
        ent = entries[off:off + n_ent]
        blocks, masks = ent >> 2, ent & 3
        assert np.all(masks > 0) and np.all(blocks < n // 64)
        got.setdefault((s, head, qa), Counter()).update(blocks[(masks & 1) != 0].tolist())
        if slot < 0:
            assert (s, head, qa) not in seen
        seen.add((s, head, qa))
        if tok1 >= 0:
            qb = (tok1 - starts[s]) // 64
            assert q_row1 == kv_row0 + qb * 64
            got.setdefault((s, head, qb), Counter()).update(blocks[(masks & 2) != 0].tolist())
            seen.add((s, head, qb))
        else:
            assert q_row1 == q_row0 and not np.any(masks & 2)
    assert got == expected
    visits = sum(sum(c.values()) for c in got.values())
    assert slots == set(range(len(slots)))
    if lens in ([4096], [2048, 4096]):
        assert len(slots) >= 2 * o.heads     # the global query blocks' lists were cut
    assert len(seen) == len(expected) and visits == plan["visits"]
    # load balance of the longest-processing-time assignment
    loads = [int(items[cta_ptr[c]:cta_ptr[c + 1], 4].sum()) for c in range(n_ctas)]
    if len(items) >= 4 * n_ctas:
        assert max(loads) <= 1.25 * (sum(loads) / n_ctas) + 64


def test_template_and_csr_work_lists_agree():
    o = EncoderConfig()
    cfg = _cfg(o)
    lens = [1024, 832, 4096, 704]
    a = metadata.attention_plan_host(cfg, 1, lens, 296, 0)
    b = metadata.attention_plan_host(cfg, 1, lens, 296, 1)
    assert np.array_equal(a["items"], b["items"]) and np.array_equal(a["entries"], b["entries"])
    assert np.array_equal(a["cta_ptr"], b["cta_ptr"]) and a["visits"] == b["visits"]


@pytest.mark.parametrize("pattern,band_half,lens", [
    ("bigbird", 4, [1024, 832, 4096, 512, 704, 1984, 64, 128]), ("bigbird", 4, [4096]), ("bigbird", 4, [832] * 40),
    ("band", 4, [1280, 64, 512, 2048]), ("band", 11, [2048]), ("band", 16, [2048, 640]), ("band", 40, [4096, 64]),
    ("band", 0, [1024])])
def test_work_list_size_bounds_hold(pattern, band_half, lens):
    """The encoder sizes its metadata regions before the tables exist: the bounds must cover the
    work list of every layer seed, also for band windows so wide that most lists are cut."""
    o = EncoderConfig(pattern=pattern, band_half=band_half)
    cfg = _cfg(o)
    bounds = metadata.attention_plan_bounds(cfg, lens)
    for seed in (0, 5):
        for n_ctas in (296, 16):
            plan = metadata.attention_plan_host(cfg, seed, lens, n_ctas, 1)
            items = plan["items"]
            slots = {(h >> 8) - 1 for h in items[:, 7].tolist() if (h >> 8) > 0}
            groups = {(int(t0), int(h) & 255) for t0, h in zip(items[:, 5], items[:, 7]) if (h >> 8) > 0}
            assert len(items) <= bounds["items"] and len(plan["entries"]) <= bounds["entries"]
            assert len(slots) <= bounds["slots"] and len(groups) <= bounds["groups"], (len(slots), len(groups), bounds)


def test_static_entry_capacity_statement():
    """The no-allocation attention entry point documents room for 25 sequences of 4096 tokens with
    12 heads (10240 work items, 131072 list entries, lists never cut): check it against the builder."""
    o = EncoderConfig()
    cfg = _cfg(o)
    lens = [4096] * 25
    kv_ptr, kv_idx = metadata.build_block_csr(cfg, 0, lens)
    ni, ne = 0, 0
    plan = metadata.attention_plan_host(cfg, 0, lens, 296, 0)
    whole = {}
    for q0, q1, kv0, off, n, t0, t1, h in plan["items"].tolist():   # undo the cuts: count whole lists
        whole[(t0, h & 255)] = whole.get((t0, h & 255), 0) + n
    assert len(whole) <= 10240 and sum(whole.values()) <= 131072
