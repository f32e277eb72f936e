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
