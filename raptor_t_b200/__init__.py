"""raptor_t_b200 - B200 (sm_100a) block-sparse transformer encoder.

Layout:
  capi        ctypes binding of the C ABI (include/raptor_b200.h)
  metadata    host metadata: random-block tables, CSR lists, varlen offsets, partitions
  ops         single-kernel wrappers on torch tensors (device memory only)
  raptor_t    the reference's operator API (BertAttention, BertIntermediate, BertOutput,
              TensorSet, MetaData, multi_headed_attention)
  modeling_bert  the reference's Python model layer on top of raptor_t
  engine      whole-encoder object (one C call per forward)
  parallel    whole-sequence partitioning across GPUs + output gather
"""
__all__ = ["capi", "metadata", "ops", "engine", "raptor_t", "modeling_bert", "parallel", "weights", "build"]
