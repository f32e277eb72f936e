"""Bookkeeping of the operator-API mirror that needs no GPU (TensorSet / MetaData)."""
import threading

import torch

from raptor_t_b200 import raptor_t


def test_tensor_set_singleton_and_metadata_bookkeeping():
    done = []

    def run():
        ts = raptor_t.TensorSet.get_instance()
        assert ts is raptor_t.TensorSet.get_instance()
        md = raptor_t.MetaData()
        md.update_meta_data(2880, 46, 400, [0, 13, 29, 45])
        assert ts.total_seq_len == 2880 and ts.lens_tokens() == [832, 1024, 1024]
        assert ts.get_tensor("unknown").numel() == 0
        md.terminate_thread()
        done.append(True)

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(20)
    assert done, "TensorSet / MetaData bookkeeping deadlocked"
    if not torch.cuda.is_available():
        try:
            raptor_t.TensorSet.get_instance().get_tensor("q_out")
            raise AssertionError("expected a loud failure without CUDA")
        except RuntimeError:
            pass


def test_compiled_module_exports_the_reference_classes():
    """The pybind11 module `raptor_t` builds, imports without a GPU and carries every class and
    method of the reference's extension module (python/pybind.cpp:11-80)."""
    import sys

    from raptor_t_b200 import compiled
    mod = compiled.load()
    assert sys.modules["raptor_t"] is mod
    for name in ("BertAttention", "BertIntermediate", "BertOutput", "TensorSet", "MetaData", "multi_headed_attention"):
        assert hasattr(mod, name), name
    assert mod.multi_headed_attention is mod.BertAttention
    for cls in (mod.BertAttention, mod.BertIntermediate, mod.BertOutput):
        assert callable(getattr(cls, "__call__"))
    ts = mod.TensorSet.get_instance()
    ts.update_tensor_set(2880, 46, 400, [0, 13, 29, 45])
    assert ts.get_tensor("nope").numel() == 0          # "no exists tensor", as the reference prints
    md = mod.MetaData()
    assert hasattr(md, "update_meta_data") and hasattr(md, "terminate_thread")
    md.terminate_thread()
    if not torch.cuda.is_available():
        w = torch.zeros(128, 384, dtype=torch.float16)
        try:
            mod.BertAttention(w, w[0], w[:, :128], w[0, :128], w[0, :128], w[0, :128], 2, 0, True)
            raise AssertionError("expected a loud failure for CPU tensors")
        except RuntimeError:
            pass
