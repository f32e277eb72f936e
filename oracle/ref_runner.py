"""Drives the reference's OWN validation module (python/modeling_big_bird.py of
WongHuLin/Raptor-T) on the host cores.  TEST / BASELINE INFRASTRUCTURE ONLY: nothing in the
product package may import this.

The module file is not part of this repository.  oracle/build_ref.py copies it from a
reference checkout into oracle/_ref/ (git-ignored); when it is there, the CPU baseline of the
benchmark times the reference's real code ("kind": "reference"), otherwise the restatement in
oracle/bigbird.py ("kind": "port").  tests/golden/make_golden.py uses the same loader to
produce the fixtures the restatement is pinned to.

The file imports under the installed transformers once the single symbol newer releases dropped
(`pytorch_utils.torch_int_div`) is put back.  BigBirdModel.forward itself no longer runs there
(it calls get_head_mask, removed since), so the encoder is driven layer by layer with the
module's own BigBirdEmbeddings / BigBirdLayer / create_masks_for_block_sparse_attn, the way
python/benchmark/end2end.py:94-112 drives it, one un-padded sequence at a time.
"""
import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_FILE = os.path.join(HERE, "_ref", "modeling_big_bird.py")


def available():
    return os.path.exists(REF_FILE)


def load_reference(path=None):
    """Import the reference's modeling_big_bird.py as a sub-module of transformers.models.big_bird."""
    import transformers.pytorch_utils as pu
    pu.torch_int_div = lambda a, b: torch.div(a, b, rounding_mode="floor")
    import transformers.models.big_bird  # noqa: F401
    name = "transformers.models.big_bird.reference_modeling_big_bird"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path or REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def hf_config(cfg, attention_type="block_sparse"):
    from transformers import BigBirdConfig
    return BigBirdConfig(
        hidden_size=cfg.hidden, num_attention_heads=cfg.heads, intermediate_size=cfg.ffn,
        num_hidden_layers=cfg.layers, hidden_act="gelu_new", layer_norm_eps=cfg.eps, block_size=cfg.block,
        num_random_blocks=cfg.num_rand, max_position_embeddings=cfg.max_pos, attention_type=attention_type,
        vocab_size=cfg.vocab, type_vocab_size=cfg.type_vocab, hidden_dropout_prob=0.0,
        attention_probs_dropout_prob=0.0, rescale_embeddings=False, use_bias=True)


def ref_layer(mbb, cfg, P, i, attention_type):
    """One BigBirdLayer of the reference with the parameters of layer i of P (seed = layer index,
    python/modeling_big_bird.py:1577)."""
    layer = mbb.BigBirdLayer(hf_config(cfg, attention_type), seed=cfg.seed_of(i)).eval()
    pre = f"encoder.layer.{i}."
    sd = {k[len(pre):]: v for k, v in P.items() if k.startswith(pre)}
    missing, unexpected = layer.load_state_dict(sd, strict=False)
    assert not unexpected and all("position_ids" in m for m in missing), (missing, unexpected)
    return layer


class ReferenceEncoder:
    """Embeddings + all layers built ONCE from the reference's modules (both attention types: the
    reference switches to full attention for sequences of at most 5 + 2r blocks,
    python/modeling_big_bird.py:2076-2094); forward() then runs a varlen batch sequence by sequence."""

    def __init__(self, cfg, P, mbb=None):
        if cfg.pattern != "bigbird":
            raise ValueError("the reference's validation model only has the BigBird pattern")
        self.cfg, self.mbb = cfg, mbb or load_reference()
        self.sparse = [ref_layer(self.mbb, cfg, P, i, "block_sparse") for i in range(cfg.layers)]
        self.full = None
        self._P = P
        self.emb = None
        if "embeddings.word_embeddings.weight" in P:
            self.emb = self.mbb.BigBirdEmbeddings(hf_config(cfg)).eval()
            sd = {k[len("embeddings."):]: v for k, v in P.items() if k.startswith("embeddings.")}
            self.emb.load_state_dict(sd, strict=False)

    @torch.no_grad()
    def forward_one(self, seq, from_ids=True):
        cfg = self.cfg
        h = self.emb(input_ids=seq.long()[None]) if from_ids else seq.float()[None]
        S = h.shape[1]
        if S // cfg.block <= 5 + 2 * cfg.num_rand:
            if self.full is None:
                self.full = [ref_layer(self.mbb, cfg, self._P, i, "original_full") for i in range(cfg.layers)]
            for layer in self.full:
                h = layer(h)[0]
            return h[0]
        bm, band, fm, tm = self.mbb.BigBirdModel.create_masks_for_block_sparse_attn(torch.ones(1, S), cfg.block)
        for layer in self.sparse:
            h = layer(h, band_mask=band, from_mask=fm, to_mask=tm, blocked_encoder_mask=bm)[0]
        return h[0]

    def forward(self, seqs, from_ids=True):
        return torch.cat([self.forward_one(s, from_ids) for s in seqs], dim=0)
