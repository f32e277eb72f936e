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
