"""Generate the golden fixtures in this folder FROM THE REFERENCE ITSELF.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference [tables small embeddings base config1]

(no group names = all groups)

It imports the reference's validation model (python/modeling_big_bird.py, the
patched HuggingFace BigBird) as a sub-module of the installed `transformers`
package, with the one symbol that newer transformers dropped
(`pytorch_utils.torch_int_div`) injected, and records

* tables.npz   - random-block tables produced by the reference's
                 BigBirdBlockSparseAttention code path for many
                 (layer seed, block count, max_position_embeddings);
* hidden_small.npz - every 4th row of the per-layer hidden states of a 2-layer,
                 hidden-128 model on sequences of 8 (full attention), 13, 16
                 and 20 blocks;
* hidden_base.npz  - every 16th row of one BigBird-base-shaped layer's output
                 for 13- and 16-block sequences, plus a float64 checksum;
* embeddings.npz   - embedding output for a tiny vocabulary;
* hidden_config1.npz - one BigBird-base layer on ONE 4096-token sequence (64 blocks: the
                 first and last query block attend to all 64 blocks), hidden states ~ N(0, 1),
                 weights and table seed 0: every 64th row, eight rows of the first and of the
                 last block, and float64 row sums of all 4096 rows.

The fixtures are inputs to the CPU tests of the oracle (tests/test_oracle.py);
nothing here is read by the GPU library.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


from oracle.ref_runner import hf_config, ref_layer  # noqa: E402
from oracle.ref_runner import load_reference as _load_reference  # noqa: E402


def load_reference(ref_root):
    return _load_reference(os.path.join(ref_root, "python", "modeling_big_bird.py"))


@torch.no_grad()
def run_ref_layers(mbb, cfg, P, x, n_layers):
    """x [S, hidden] -> list of per-layer outputs, using the reference's modules."""
    S = x.shape[0]
    L = S // cfg.block
    full = L <= 5 + 2 * cfg.num_rand
    outs = []
    h = x[None]
    if not full:
        bm, band, fm, tm = mbb.BigBirdModel.create_masks_for_block_sparse_attn(torch.ones(1, S), cfg.block)
    for i in range(n_layers):
        layer = ref_layer(mbb, cfg, P, i, "original_full" if full else "block_sparse")
        if full:
            h = layer(h)[0]
        else:
            h = layer(h, band_mask=band, from_mask=fm, to_mask=tm, blocked_encoder_mask=bm)[0]
        outs.append(h[0].clone())
    return outs


def ref_table(mbb, seed, heads, L, r, max_pos, block=64):
    """Drive exactly the table branch of bigbird_block_sparse_attention
    (python/modeling_big_bird.py:573-600) on the reference's own methods."""
    A = mbb.BigBirdBlockSparseAttention
    np.random.seed(seed)
    S = L * block
    if S % 256 == 0:
        rows = [A._bigbird_block_rand_mask(max_pos, max_pos, block, block, r, last_idx=1024)[: L - 2]
                for _ in range(heads)]
    else:
        plan_len, plan_r = A._get_rand_attn_plan(S, block, r)
        rows = A._bigbird_block_rand_mask_with_head(
            A, from_seq_length=S, to_seq_length=S, from_block_size=block, to_block_size=block,
            num_heads=heads, plan_from_length=plan_len, plan_num_rand_blocks=plan_r)
    return np.stack(rows, axis=0).astype(np.int32)


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref_root = sys.argv[1]
    groups = set(sys.argv[2:]) or {"tables", "small", "embeddings", "base", "config1"}
    mbb = load_reference(ref_root)
    from oracle import EncoderConfig, make_weights

    if "config1" in groups:
        cfg1 = EncoderConfig(layers=1)
        P1 = make_weights(cfg1, seed=0, nonzero_bias=False, embeddings=False)
        x = torch.randn(4096, cfg1.hidden, generator=torch.Generator().manual_seed(264))
        o = run_ref_layers(mbb, cfg1, P1, x, 1)[0]
        edge = list(range(0, 64, 8)) + list(range(4032, 4096, 8))
        np.savez_compressed(os.path.join(HERE, "hidden_config1.npz"), rows=o[::64].numpy(), edge_rows=o[edge].numpy(),
                            edge_index=np.array(edge), row_sums=o.double().sum(dim=1).numpy())
        print("hidden_config1.npz written")
    if not groups & {"tables", "small", "embeddings", "base"}:
        return

    # ---- tables ----------------------------------------------------------
    tables = {}
    for seed in (0, 1, 7, 23):
        for L in range(13, 65):
            tables[f"s{seed}_h12_L{L}_m4096"] = ref_table(mbb, seed, 12, L, 3, 4096)
    for seed in (0, 3):
        for L in (13, 16, 20, 31, 64, 65, 96, 100, 127, 128):
            tables[f"s{seed}_h16_L{L}_m8192"] = ref_table(mbb, seed, 16, L, 3, 8192)
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **tables)

    # ---- small model hidden states ----------------------------------------
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=2, max_pos=4096, vocab=97)
    P = make_weights(cfg, seed=3, nonzero_bias=True)
    small = {}
    for L in (8, 13, 16, 20):
        g = torch.Generator().manual_seed(100 + L)
        x = torch.randn(L * 64, cfg.hidden, generator=g)
        outs = run_ref_layers(mbb, cfg, P, x, cfg.layers)
        for i, o in enumerate(outs):
            small[f"L{L}_layer{i}"] = o[::4].numpy()
    np.savez_compressed(os.path.join(HERE, "hidden_small.npz"), **small)

    # ---- embeddings --------------------------------------------------------
    emb = mbb.BigBirdEmbeddings(hf_config(cfg)).eval()
    sd = {k[len("embeddings."):]: v for k, v in P.items() if k.startswith("embeddings.")}
    emb.load_state_dict(sd, strict=False)
    ids = torch.from_numpy(np.random.default_rng(5).integers(0, cfg.vocab, size=832))
    with torch.no_grad():
        e = emb(input_ids=ids[None])[0]
    np.savez_compressed(os.path.join(HERE, "embeddings.npz"), ids=ids.numpy(), out=e.numpy())

    # ---- base-shaped single layer -----------------------------------------
    cfgb = EncoderConfig(layers=1)
    Pb = make_weights(cfgb, seed=0, nonzero_bias=False, embeddings=False)
    base = {}
    for L in (13, 16):
        g = torch.Generator().manual_seed(200 + L)
        x = torch.randn(L * 64, cfgb.hidden, generator=g)
        o = run_ref_layers(mbb, cfgb, Pb, x, 1)[0]
        base[f"L{L}_rows"] = o[::16].numpy()
        base[f"L{L}_sum"] = np.array([o.double().sum().item(), o.double().abs().sum().item()])
    np.savez_compressed(os.path.join(HERE, "hidden_base.npz"), **base)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
