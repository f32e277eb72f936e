"""The reference's operator API (BertAttention / BertIntermediate / BertOutput / TensorSet /
MetaData and the Python model layer on top) against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from oracle import EncoderConfig

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("binding", ["ctypes", "pybind"])
def test_model_layer_matches_oracle(binding):
    """The reference's Python model layer on the operator classes, bound with ctypes
    (raptor_t_b200.raptor_t) and as the compiled pybind11 module `raptor_t`: both must match the
    oracle, with and without the per-layer metadata tasks (async)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from raptor_t_b200 import metadata
    from raptor_t_b200.modeling_bert import BertModelNoPooler
    if binding == "ctypes":
        from raptor_t_b200 import raptor_t
        backend = None
    else:
        from raptor_t_b200 import compiled
        raptor_t = backend = compiled.load()
    cfg = EncoderConfig(hidden=128, heads=2, ffn=256, layers=2, max_pos=4096, vocab=97)
    P = oracle.make_weights(cfg, seed=3, nonzero_bias=True)
    lens = [832, 1024, 512]
    rng = np.random.default_rng(0)
    seqs = [torch.from_numpy(rng.integers(0, cfg.vocab, size=n)).int() for n in lens]
    ref = oracle.encoder_ref(seqs, P, cfg)
    for async_ in (True, False):
        model = BertModelNoPooler.from_weights(P, cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, torch.bfloat16, async_,
                                               backend=backend)
        prefix, total_comp, part_off, part_ids = metadata.generate_data_metainfo(lens, 64, 160, cfg.heads)
        T = sum(lens)
        md = raptor_t.MetaData()
        md.update_meta_data(T, prefix[-1] + 1, total_comp, prefix)
        ids = torch.cat(seqs).cuda()
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).cuda()
        info = {"pre_process": 0.0, "attention": 0.0, "add_bias_act_kernel": 0.0,
                "add_bias_and_layernorm_kernel": 0.0, "add_bias_and_transpose_kernel": 0.0}
        out, info = model(ids, T, 160, prefix, torch.tensor(prefix, dtype=torch.int32, device="cuda"),
                          torch.from_numpy(part_off).cuda(), torch.from_numpy(part_ids).cuda(),
                          position_ids=pos, test_info=info)
        err = (out.float().cpu() - ref).abs()
        print(f"PARITY operator_api[{binding}, async={async_}] max_abs={err.max().item():.4f} "
              f"mean_abs={err.mean().item():.5f}")
        assert err.max().item() < 6e-2 and err.mean().item() < 6e-3  # bf16, 2 layers of hidden 128
        assert info["attention"] > 0 and info["add_bias_and_layernorm_kernel"] > 0
        # without timing keys the fused epilogues run (kernel_fusion=True): same result within rounding
        out2, _ = model(ids, T, 160, prefix, torch.tensor(prefix, dtype=torch.int32, device="cuda"),
                        torch.from_numpy(part_off).cuda(), torch.from_numpy(part_ids).cuda(),
                        position_ids=pos, test_info={})
        assert (out2.float().cpu() - ref).abs().max().item() < 6e-2
        if binding == "pybind":  # the pooler the reference leaves commented out, on the batch MetaData describes
            w = (torch.randn(cfg.hidden, cfg.hidden, device="cuda") / 11.0).to(torch.bfloat16)
            b = torch.zeros(cfg.hidden, device="cuda", dtype=torch.bfloat16)
            pooled = raptor_t.BertPooler(w, b)(out, torch.empty(len(lens), cfg.hidden, device="cuda"))
            firsts = torch.tensor(np.concatenate([[0], np.cumsum(lens)[:-1]]), device="cuda")
            want = torch.tanh(out[firsts].float() @ w.float())
            assert (pooled - want).abs().max().item() < 2e-3
        md.terminate_thread()
        del model
    ts = raptor_t.TensorSet.get_instance()
    assert ts.get_tensor("q_out").shape[0] == T and ts.get_tensor("nope").numel() == 0
