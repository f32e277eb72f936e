"""Seeded synthetic parameters with the names of the reference's validation model
(HuggingFace BigBird state_dict names, torch Linear layout [out, in]).  There is no
network access for checkpoints, so benchmarks and tests use these: weights ~ N(0, 0.02),
biases 0, LayerNorm gamma 1 / beta 0 (nonzero_bias=True perturbs all three)."""
import torch

_LAYER = [
    ("attention.self.query.weight", "hh"), ("attention.self.query.bias", "bh"),
    ("attention.self.key.weight", "hh"), ("attention.self.key.bias", "bh"),
    ("attention.self.value.weight", "hh"), ("attention.self.value.bias", "bh"),
    ("attention.output.dense.weight", "hh"), ("attention.output.dense.bias", "bh"),
    ("attention.output.LayerNorm.weight", "g"), ("attention.output.LayerNorm.bias", "be"),
    ("intermediate.dense.weight", "fh"), ("intermediate.dense.bias", "bf"),
    ("output.dense.weight", "hf"), ("output.dense.bias", "bh"),
    ("output.LayerNorm.weight", "g"), ("output.LayerNorm.bias", "be"),
]


def synthetic_weights(hidden, ffn, layers, vocab, max_pos, type_vocab, seed=0, nonzero_bias=False, embeddings=True):
    g = torch.Generator().manual_seed(seed)
    H, F = hidden, ffn
    w = lambda *s: torch.randn(*s, generator=g) * 0.02  # noqa: E731
    bias = lambda n: torch.randn(n, generator=g) * 0.02 if nonzero_bias else torch.zeros(n)  # noqa: E731
    gamma = lambda n: 1.0 + torch.randn(n, generator=g) * 0.1 if nonzero_bias else torch.ones(n)  # noqa: E731
    beta = lambda n: torch.randn(n, generator=g) * 0.1 if nonzero_bias else torch.zeros(n)  # noqa: E731
    P = {}
    if embeddings:
        P["embeddings.word_embeddings.weight"] = w(vocab, H)
        P["embeddings.position_embeddings.weight"] = w(max_pos, H)
        P["embeddings.token_type_embeddings.weight"] = w(type_vocab, H)
        P["embeddings.LayerNorm.weight"] = gamma(H)
        P["embeddings.LayerNorm.bias"] = beta(H)
    for i in range(layers):
        for name, kind in _LAYER:
            key = f"encoder.layer.{i}.{name}"
            if kind == "hh":
                P[key] = w(H, H)
            elif kind == "fh":
                P[key] = w(F, H)
            elif kind == "hf":
                P[key] = w(H, F)
            elif kind == "bh":
                P[key] = bias(H)
            elif kind == "bf":
                P[key] = bias(F)
            elif kind == "g":
                P[key] = gamma(H)
            else:
                P[key] = beta(H)
    return P
