"""The reference's Python model layer (python/modeling_bert.py) on this library's
operator API: BertEmbeddings, BertLayer, BertEncoder, BertModelNoPooler, with the same call
order and buffer reuse (the FFN-down output is written into the layer's input buffer,
python/modeling_bert.py:205-207).  Weights come from a HuggingFace-style module
(from_torch) or from a dict with the same parameter names (from_weights)."""
from typing import Optional, Sequence

import torch

from . import ops, raptor_t as cxx


class BertEmbeddings:
    """python/modeling_bert.py:27-69.  fp32 tables, one fused gather + add + LayerNorm kernel."""

    def __init__(self, word, position, token_type, ln_weight, ln_bias, eps=1e-12, dtype=torch.float16):
        f = lambda t: t.detach().to("cuda", torch.float32).contiguous()  # noqa: E731
        self.word, self.position, self.token_type = f(word), f(position), f(token_type)
        self.ln_w, self.ln_b, self.eps, self.dtype = f(ln_weight), f(ln_bias), eps, dtype

    def __call__(self, input_ids, position_ids=None, token_type_ids=None, output=None):
        if position_ids is None or token_type_ids is None:
            raise ValueError("Missing parameters")
        return ops.embeddings(input_ids.int(), position_ids.int(), token_type_ids.int(), self.word, self.position,
                              self.token_type, self.ln_w, self.ln_b, self.eps, self.dtype, out=output)


class BertLayer:
    """python/modeling_bert.py:165-216."""

    def __init__(self, attention, intermediate, output):
        self.attention, self.intermediate, self.output = attention, intermediate, output

    def __call__(self, hidden_states, seq_position_info, seq_position_info_tensor, partition_part_index_tensor,
                 partition_part_tensor, intermediate_temp, output_layer_temp, attention_output, block_limit,
                 attention_mask=None, head_mask=None, output_attentions=False, kernel_fusion=True, test_info=None,
                 balanced=True):
        test_info = self.attention(hidden_states, attention_mask, attention_output, seq_position_info,
                                   seq_position_info_tensor, partition_part_index_tensor, partition_part_tensor,
                                   block_limit, test_info, kernel_fusion, balanced)
        test_info = self.intermediate(attention_output, intermediate_temp, test_info, kernel_fusion)
        test_info = self.output(intermediate_temp, attention_output, hidden_states, test_info, kernel_fusion)
        return hidden_states, test_info


class BertEncoder:
    """python/modeling_bert.py:218-269."""

    def __init__(self, layer: Sequence[BertLayer]):
        self.layer = layer

    def __call__(self, hidden_states, total_seq_len, thread_block_limit, seq_position_info, seq_position_info_tensor,
                 partition_part_index_tensor, partition_part_tensor, output_layer_temp, intermediate_temp,
                 attention_output, test_info=None, kernel_fusion=True, balanced=True, attention_mask=None,
                 head_mask=None, output_attentions=False, output_hidden_states=False):
        for l in self.layer:
            hidden_states, test_info = l(hidden_states, seq_position_info, seq_position_info_tensor,
                                         partition_part_index_tensor, partition_part_tensor, intermediate_temp,
                                         output_layer_temp, attention_output, thread_block_limit, attention_mask,
                                         head_mask, output_attentions, kernel_fusion, test_info, balanced)
        return hidden_states, test_info


class BertPooler:
    """The pooler the reference sketches and leaves commented out (python/modeling_bert.py:281-300):
    tanh(dense(first token of every sequence)), the head of its validation model
    (python/modeling_big_bird.py:1964, 2179).  weight is [in, out] as the reference's from_torch would pass it."""

    def __init__(self, dense_weight, dense_bias):
        self.w = dense_weight.t().contiguous()  # [out, in]
        self.b = dense_bias.contiguous()

    def __call__(self, input_tensor, seq_position_info_tensor, output=None):
        return ops.pooler(input_tensor, seq_position_info_tensor, self.w, self.b, out=output)


class BertModelNoPooler:
    """python/modeling_bert.py:318-394."""

    def __init__(self, embeddings: BertEmbeddings, encoder: BertEncoder):
        self.embeddings, self.encoder = embeddings, encoder

    def __call__(self, inputs, total_seq_len, thread_block_limit, seq_position_info, seq_position_info_tensor,
                 partition_part_index_tensor=None, partition_part_tensor=None, attention_masks=None,
                 token_type_ids=None, position_ids=None, output_layer_temp=None, intermediate_temp=None,
                 attention_output=None, test_info=None, kernel_fusion=True, balanced=True, **_):
        dev = inputs.device
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(inputs)
        if position_ids is None:
            raise ValueError("position_ids are required (token index within its sequence)")
        hidden = self.embeddings(inputs, position_ids=position_ids, token_type_ids=token_type_ids)
        H = hidden.shape[1]
        if attention_output is None:
            attention_output = torch.empty(total_seq_len, H, dtype=hidden.dtype, device=dev)
        if intermediate_temp is None:
            intermediate_temp = torch.empty(total_seq_len, self.ffn, dtype=hidden.dtype, device=dev)
        return self.encoder(hidden, total_seq_len, thread_block_limit, seq_position_info, seq_position_info_tensor,
                            partition_part_index_tensor, partition_part_tensor, output_layer_temp,
                            intermediate_temp[:total_seq_len], attention_output[:total_seq_len], test_info,
                            kernel_fusion, balanced)

    @staticmethod
    def from_weights(P, hidden, heads, ffn, layers, dtype=torch.float16, async_=True, eps=1e-12, max_pos=4096,
                     pattern="bigbird", band_half=4, backend=None) -> "BertModelNoPooler":
        """P: dict with HuggingFace BigBird parameter names (torch Linear layout [out, in]); the
        re-layout to [in, out] + q|k|v concatenation is the reference's (python/modeling_bert.py:138-163).
        backend: the operator module - the compiled pybind11 module (raptor_t_b200.compiled.load())
        or, by default, its ctypes twin raptor_t_b200.raptor_t."""
        cxx_mod = cxx if backend is None else backend
        compiled = backend is not None and not hasattr(backend, "LAYER_NORM_EPS")
        if compiled:
            backend.set_model_options(num_rand=3, max_pos=max_pos, pattern=pattern, band_half=band_half, eps=eps)
        g = lambda k: P[k].detach().to("cuda", dtype)  # noqa: E731
        emb = BertEmbeddings(P["embeddings.word_embeddings.weight"], P["embeddings.position_embeddings.weight"],
                             P["embeddings.token_type_embeddings.weight"], P["embeddings.LayerNorm.weight"],
                             P["embeddings.LayerNorm.bias"], eps, dtype)
        ls = []
        for i in range(layers):
            pre = f"encoder.layer.{i}."
            qkv_w = torch.cat([g(pre + "attention.self.query.weight"), g(pre + "attention.self.key.weight"),
                               g(pre + "attention.self.value.weight")], 0).t().contiguous()
            qkv_b = torch.cat([g(pre + "attention.self.query.bias"), g(pre + "attention.self.key.bias"),
                               g(pre + "attention.self.value.bias")], 0).contiguous()
            extra = {} if compiled else dict(max_pos=max_pos, pattern=pattern, band_half=band_half, eps=eps)
            att = cxx_mod.BertAttention(qkv_w, qkv_b, g(pre + "attention.output.dense.weight").t().contiguous(),
                                        g(pre + "attention.output.dense.bias"),
                                        g(pre + "attention.output.LayerNorm.weight"),
                                        g(pre + "attention.output.LayerNorm.bias"), heads, i, async_, **extra)
            inter = cxx_mod.BertIntermediate(g(pre + "intermediate.dense.weight").t().contiguous(),
                                             g(pre + "intermediate.dense.bias"))
            out = cxx_mod.BertOutput(g(pre + "output.dense.weight").t().contiguous(), g(pre + "output.dense.bias"),
                                     g(pre + "output.LayerNorm.weight"), g(pre + "output.LayerNorm.bias"),
                                     **({} if compiled else {"eps": eps}))
            ls.append(BertLayer(att, inter, out))
        m = BertModelNoPooler(emb, BertEncoder(ls))
        m.ffn = ffn
        return m

    @staticmethod
    def from_torch(model, async_: bool = True, dtype=torch.float16) -> "BertModelNoPooler":
        """model: a HuggingFace BigBirdModel-like module (state_dict names as in from_weights)."""
        cfg = model.config
        P = {k: v for k, v in model.state_dict().items()}
        return BertModelNoPooler.from_weights(P, cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size,
                                              cfg.num_hidden_layers, dtype, async_, cfg.layer_norm_eps,
                                              cfg.max_position_embeddings)
