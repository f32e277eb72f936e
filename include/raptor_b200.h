/*
 * raptor_b200 - C ABI of the B200 (sm_100a) block-sparse encoder library.
 *
 * Every entry point is extern "C", takes plain pointers and sizes, and returns
 * an rt_status (0 = ok).  rt_last_error() gives the message of the last
 * failure on the calling thread.  Pointers named *_dev are device pointers,
 * *_host are host pointers; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  dtype: RT_F16 or RT_BF16 for every
 * 16-bit activation / weight buffer of a call.
 *
 * Each declaration cites the interface of the reference project
 * (WongHuLin/Raptor-T, paths relative to its root) that it stands in for.
 */
#ifndef RAPTOR_B200_H_
#define RAPTOR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int rt_status;
enum {
  RT_OK = 0,
  RT_ERR_INVALID = 1,      /* bad argument (size, alignment, null pointer)        */
  RT_ERR_UNSUPPORTED = 2,  /* shape / length the path does not support            */
  RT_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed                 */
  RT_ERR_DEVICE_WAIT = 4,  /* a bounded device-side wait ran out (kernel aborted) */
  RT_ERR_STATE = 5         /* call order violated (e.g. forward before prepare)   */
};

enum { RT_F16 = 0, RT_BF16 = 1 };
enum { RT_PATTERN_BIGBIRD = 0, RT_PATTERN_BAND = 1 };
enum { RT_EPI_NONE = 0, RT_EPI_BIAS = 1, RT_EPI_BIAS_GELU = 2 };
/* (3 is the internal QKV scatter of rt_gemm_qkv) */
enum { RT_EPI_BIAS_RESIDUAL = 4 };  /* C = A W^T + bias + residual (rt_gemm_residual) */

/* Model shape.  Replaces the constants hard-coded in layers/bert_attention.h:37-40
 * (12 heads, 768, block 64), layers/tensor_set.h:40-44 and layers/bert_output.cpp:23 (eps). */
typedef struct rt_config {
  int32_t hidden;      /* heads * 64                                        */
  int32_t heads;
  int32_t ffn;
  int32_t layers;
  int32_t block;       /* must be 64                                        */
  int32_t num_rand;    /* random blocks per query block (BigBird pattern)   */
  int32_t max_pos;     /* max_position_embeddings (also sizes the old-plan random table) */
  int32_t vocab;
  int32_t type_vocab;
  int32_t pattern;     /* RT_PATTERN_*                                      */
  int32_t band_half;   /* RT_PATTERN_BAND: window = 2*band_half+1 blocks    */
  int32_t dtype;       /* RT_F16 / RT_BF16                                  */
  float   eps;         /* LayerNorm epsilon                                 */
  int32_t reserved;
} rt_config;

const char* rt_last_error(void);
int rt_version(void);

/* ------------------------------------------------------------------------------------------
 * Host metadata (no GPU needed)
 * ---------------------------------------------------------------------------------------- */

/* Random-block table of one (layer seed, block count): out_host int32 [heads][n_blocks-2][num_rand].
 * Bit-exact with the reference's validation model, python/modeling_big_bird.py:573-600,
 * 1072-1125, 1127-1314 (numpy legacy RNG seeded with the layer index).  Replaces the
 * non-deterministic generator layers/multi_headed_attention.cpp:15-140. */
rt_status rt_rand_block_table(uint32_t seed, int heads, int n_blocks, int num_rand, int max_pos, int block,
                              int32_t* out_host);

/* Number of key/value block visits per head for a batch (= last entry of kv_ptr). */
rt_status rt_count_visits(const rt_config* cfg, const int32_t* lens_tokens, int n_seq, int64_t* visits_out);

/* CSR block table of one layer: kv_ptr_host int32 [N+1], kv_idx_host int32 [heads][visits]
 * (sequence-local block ids).  Counterpart of to_select_index_position / to_select_index,
 * layers/multi_headed_attention.cpp:124-132, with a head dimension. */
rt_status rt_build_block_csr(const rt_config* cfg, uint32_t layer_seed, const int32_t* lens_tokens, int n_seq,
                             int32_t* kv_ptr_host, int32_t* kv_idx_host);

/* Varlen offsets in blocks, out_host int32 [n_seq+1] (python/util.py:37,45 seq_position_info). */
rt_status rt_seq_block_prefix(const int32_t* lens_tokens, int n_seq, int block, int32_t* out_host);

/* Longest-processing-time partition of heads*N (head, query block) work items over n_parts
 * CTAs; python/util.py:11-34 (generate_parition_plan).  offsets_host [n_parts+1], ids_host [heads*N]. */
rt_status rt_lpt_partition(const int32_t* cost_per_qblock, int n_qblocks, const int32_t* seq_block_prefix,
                           int n_seq, int n_parts, int heads, int32_t* offsets_host, int32_t* ids_host);

/* Whole-sequence bin packing over n_bins GPUs (same greedy, lifted from CTAs to GPUs):
 * bin_of_seq_host int32 [n_seq]. */
rt_status rt_binpack_sequences(const double* cost, int n_seq, int n_bins, int32_t* bin_of_seq_host);

/* ------------------------------------------------------------------------------------------
 * Single kernels (device pointers).  Launchers of layers/kernels/kernel.h:12-42.
 * ---------------------------------------------------------------------------------------- */

/* out = LayerNorm(x + bias + residual) * gamma + beta, rows x hidden, out may alias x.
 * layers/kernels/add_bias_and_layernorm.cu:191-285 (add_bias_and_layernorm_kernel).
 * bias_dev / residual_dev may be NULL. */
rt_status rt_bias_residual_layernorm(void* out_dev, const void* x_dev, const void* bias_dev,
                                     const void* residual_dev, const void* gamma_dev, const void* beta_dev,
                                     int rows, int hidden, float eps, int dtype, void* stream);

/* x = gelu_tanh(x + bias) in place, rows x cols.
 * layers/kernels/add_bias_act.cu:86-133 (add_bias_act_kernel). */
rt_status rt_bias_gelu(void* x_dev, const void* bias_dev, int rows, int cols, int dtype, void* stream);

/* q = (x_q + b_q) * q_scale, k = x_k + b_k, v = x_v + b_v, split and written head-major per
 * sequence: q/k/v_dev[(first_token_of_seq*heads + head*len_seq + token_in_seq) * 64 + d].
 * qkv_dev is [T][3*hidden] (q | k | v along columns).  seq_block_prefix_dev int32 [n_seq+1].
 * layers/kernels/add_bias_and_transpose.cu:118-233 (add_bias_and_transpose_kernel). */
rt_status rt_qkv_bias_transpose(const void* qkv_dev, const void* bias_dev, void* q_dev, void* k_dev,
                                void* v_dev, const int32_t* seq_block_prefix_dev, int n_seq,
                                int total_blocks, int heads, float q_scale, int dtype, void* stream);

/* word + token-type + position embedding gather, sum, LayerNorm -> out [T][hidden] (16-bit).
 * The three tables [vocab|max_pos|type_vocab][hidden] and gamma/beta are fp32: the reference keeps
 * its embeddings in fp32 torch.nn modules and casts the result (python/modeling_bert.py:45-60).
 * pos_ids_dev / type_ids_dev may be NULL (= all zero). */
rt_status rt_embeddings(void* out_dev, const int32_t* ids_dev, const int32_t* pos_ids_dev,
                        const int32_t* type_ids_dev, const void* word_dev, const void* pos_dev,
                        const void* type_dev, const void* gamma_dev, const void* beta_dev, int tokens,
                        int hidden, float eps, int dtype, void* stream);

/* Pooler of the model head: pooled_dev fp32 [n_seq][hidden] = tanh(W hidden[first token of each sequence] + b),
 * W 16-bit [hidden][hidden] in torch Linear layout [out][in], hidden_dev the packed [T][hidden] encoder output,
 * seq_block_prefix_dev int32 [n_seq+1] (offsets in 64-token blocks).  The reference's own binding is commented
 * out (python/pybind.cpp:58-64); the math is its validation model's, python/modeling_big_bird.py:1964, 2179. */
rt_status rt_pooler(float* pooled_dev, const void* hidden_dev, const int32_t* seq_block_prefix_dev, int n_seq,
                    const void* w_dev, const void* b_dev, int hidden, int dtype, void* stream);

/* C[M][N] = A[M][K] * W[N][K]^T (+ bias, + GELU), fp32 accumulation on tcgen05 tensor cores.
 * A, W, C 16-bit row-major; K % 64 == 0, N % 64 == 0; A, W, bias 16-byte and C 32-byte aligned.
 * layers/kernels/mat_mul.cpp:9-96 (MatMul; note W here is [out][in], i.e. B transposed). */
rt_status rt_gemm(void* c_dev, const void* a_dev, const void* w_dev, const void* bias_dev, int M, int N,
                  int K, int epilogue, int dtype, void* stream);

/* C[M][N] = A W^T + bias + residual[M][N]: the pre-LayerNorm sum of the attention-output and
 * FFN-down projections, so that the LayerNorm that follows reads one tensor instead of two
 * (layers/multi_headed_attention.cpp:206-210, layers/bert_output.cpp:19-23).  C may alias residual. */
rt_status rt_gemm_residual(void* c_dev, const void* a_dev, const void* w_dev, const void* bias_dev,
                           const void* residual_dev, int M, int N, int K, int dtype, void* stream);

/* out[M][N] = LayerNorm(A W^T + bias + residual) * gamma + beta in ONE kernel, N = 768 or 1024: the
 * projection and the add_bias_and_layernorm kernel that follows it in both sub-layers
 * (layers/multi_headed_attention.cpp:206-210, layers/bert_output.cpp:19-23).  A cluster of N/256 CTA
 * pairs owns 256 whole rows; the pre-LayerNorm sum stays in fp32 in TMEM and never reaches HBM.
 * All pointers 32-byte aligned, K % 64 == 0; out may alias residual. */
rt_status rt_gemm_bias_residual_layernorm(void* out_dev, const void* a_dev, const void* w_dev, const void* bias_dev,
                                          const void* residual_dev, const void* gamma_dev, const void* beta_dev,
                                          int M, int N, int K, float eps, int dtype, void* stream);

/* Fused QKV projection: (A[M][K] * W[3*heads*64][K]^T + bias), query part scaled by q_scale,
 * written head-major per sequence straight into q/k/v (the layout of rt_qkv_bias_transpose) -
 * the [T][3H] intermediate of layers/multi_headed_attention.cpp:143-152 (FuseGemm012AddBIasTranspose)
 * never touches HBM.  block_seq_dev: int32 pairs {first token of the sequence, sequence length}
 * for every packed 64-token block. */
rt_status rt_gemm_qkv(void* q_dev, void* k_dev, void* v_dev, const void* a_dev, const void* w_dev,
                      const void* bias_dev, const int32_t* block_seq_dev, int M, int heads, int K, float q_scale,
                      int dtype, void* stream);

/* Attention work list of one layer, built on the host from a CSR block table.
 * A work item covers up to two query blocks of one (sequence, head) so that the tensor-core
 * tile has 128 rows; its key/value list is the multiset union of the two blocks' lists, each
 * entry tagged with the query blocks that use it.  Opaque handle; holds host + device copies. */
typedef struct rt_attn_plan rt_attn_plan;
/* n_ctas <= 0: as many CTAs as the current device keeps resident.  split_entries: key/value lists
 * longer than this (and than one CTA's share of the batch) are cut into parts whose partial
 * results a second kernel merges; 0 = never split, < 0 = the library's default. */
rt_status rt_attn_plan_create(const rt_config* cfg, const int32_t* lens_tokens, int n_seq,
                              const int32_t* kv_ptr_host, const int32_t* kv_idx_host, int n_ctas,
                              int split_entries, void* stream, rt_attn_plan** plan_out);
rt_status rt_attn_plan_destroy(rt_attn_plan* plan);
/* issued key/value block loads (work-list entries) and useful visits, for roofline accounting */
rt_status rt_attn_plan_stats(const rt_attn_plan* plan, int64_t* entries_out, int64_t* visits_out,
                             int32_t* items_out);

/* The same work list built on the host only (no GPU; for validation and tooling).
 * use_templates = 1 takes the cached per-sequence template path the encoder object uses for the
 * first layer of a batch; 2 its path for the other layers (items, cuts and CTA assignment taken
 * from another seed's lists, entries refilled from this seed's).
 * items_out: 8 int32 per item {q_row0, q_row1, kv_row0, entry_off, n_entries, out_tok0, out_tok1, head};
 * entries_out: (sequence-local block id << 2) | mask (bit 0: first query block, bit 1: second);
 * cta_ptr_out [n_ctas+1].  Pass items_out = NULL to query the sizes.  No reference counterpart
 * (the reference partitions single query blocks, python/util.py:11-34). */
rt_status rt_attn_plan_build_host(const rt_config* cfg, uint32_t layer_seed, const int32_t* lens_tokens, int n_seq,
                                  int n_ctas, int use_templates, int32_t* items_out, int64_t items_cap,
                                  int32_t* entries_out, int64_t entries_cap, int32_t* cta_ptr_out,
                                  int64_t* n_items, int64_t* n_entries, int64_t* visits);

/* Upper bounds, valid for every table seed, of the sizes of a batch's work list: work items, list
 * entries, partial-result slots (one 128 x 64 fp32 tile each) and groups of split lists.  The
 * encoder object sizes its per-batch metadata regions with these before the tables exist.
 * split_entries as in rt_attn_plan_create.  No reference counterpart (the reference sizes
 * to_select_index for one fixed 4096-token sequence, layers/tensor_set.h:61). */
rt_status rt_attn_plan_bounds(const rt_config* cfg, const int32_t* lens_tokens, int n_seq, int split_entries,
                              int64_t* items_out, int64_t* entries_out, int64_t* slots_out, int64_t* groups_out);

/* ctx[token][head*64 + d] = softmax(scale * q k_listed^T) v_listed, online softmax, per work item.
 * q/k/v in the head-major layout of rt_qkv_bias_transpose; ctx_dev is token-major [T][heads*64].
 * layers/kernels/sparse_attention.cu:2953-3228 (sparse_attention_lastest / test_gemm_1). */
rt_status rt_sparse_attention(void* ctx_dev, const void* q_dev, const void* k_dev, const void* v_dev,
                              const rt_attn_plan* plan, float scale, int dtype, void* stream);

/* Block-sparse attention WITHOUT any device allocation.  No counterpart in the reference.
 * For callers that may not call cudaMalloc (memory owned by an external arena or caching
 * allocator, a fixed start-up budget, a thread that must not hit an implicit device
 * synchronisation): the work list and the status word live in a file-scope device array of
 * about 0.84 MB that each GPU holds from library load until exit.  Same math and layouts as
 * rt_sparse_attention; the block table is given as HOST CSR arrays (rt_build_block_csr).
 * Limits: at most 10240 work items and 131072 list entries per call (25 sequences of 4096
 * tokens with 12 heads fit), else RT_ERR_UNSUPPORTED and nothing runs.  The array is shared by all
 * calls on a device and keeps the last call's contents; calls whose GPU work overlaps race on
 * it, so issue them on one stream.  The first call on a device resolves the array's address
 * and sets kernel attributes: make it before any stream capture.  Each call first reads back
 * (4 bytes, queued on `stream`; the host waits for it) and clears the status of the previous call,
 * so a kernel that gave up on a bounded wait is reported by the following call.  Because of that
 * wait, and because the work list is copied from host memory that is released on return, a call
 * whose `stream` is being captured is refused with RT_ERR_UNSUPPORTED. */
rt_status rt_sparse_attention_static(void* ctx_dev, const void* q_dev, const void* k_dev, const void* v_dev,
                                     const rt_config* cfg, const int32_t* lens_tokens_host, int n_seq,
                                     const int32_t* kv_ptr_host, const int32_t* kv_idx_host, float scale,
                                     int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Encoder object: weights, scratch (the TensorSet), metadata pipeline, streams and events.
 * ---------------------------------------------------------------------------------------- */
typedef struct rt_encoder rt_encoder;

rt_status rt_encoder_create(const rt_config* cfg, rt_encoder** enc_out);
rt_status rt_encoder_destroy(rt_encoder* enc);

/* Weights of one layer, 16-bit device pointers, copied into the object (re-laid-out once).
 * qkv_w [hidden][3*hidden] and the other matrices are [in][out] exactly as the reference's
 * Python wrappers pass them (python/modeling_bert.py:138-163, 84-91, 107-113);
 * in_out_layout = 0 means the torch Linear layout [out][in] instead. */
rt_status rt_encoder_set_layer(rt_encoder* enc, int layer, uint32_t table_seed, int in_out_layout,
                               const void* qkv_w, const void* qkv_b, const void* attn_out_w,
                               const void* attn_out_b, const void* attn_ln_g, const void* attn_ln_b,
                               const void* ffn_up_w, const void* ffn_up_b, const void* ffn_down_w,
                               const void* ffn_down_b, const void* out_ln_g, const void* out_ln_b);
rt_status rt_encoder_set_embeddings(rt_encoder* enc, const void* word, const void* pos, const void* type,
                                    const void* ln_g, const void* ln_b);

/* Per-batch metadata: varlen offsets, block tables and attention work lists of every layer are
 * built by a host worker thread and uploaded on a side stream, one event per layer; the
 * forward pass waits on layer i's event right before layer i's attention kernel.
 * layers/metadata.cpp:6-18 (MetaData::update_meta_data) + layers/semaphore.cpp:16-37 +
 * layers/tensor_set.cpp:10-25 (scratch resize). */
rt_status rt_encoder_prepare_batch(rt_encoder* enc, const int32_t* lens_tokens, int n_seq);

/* hidden_dev [T][hidden] in/out: runs layers [layer_begin, layer_end) in place.
 * python/modeling_bert.py:244-261 (BertEncoder.__call__). */
rt_status rt_encoder_forward_hidden(rt_encoder* enc, void* hidden_dev, int layer_begin, int layer_end,
                                    void* stream);
/* ids -> embeddings -> all layers -> out_dev [T][hidden].  python/modeling_bert.py:324-383. */
rt_status rt_encoder_forward_ids(rt_encoder* enc, const int32_t* ids_dev, const int32_t* pos_ids_dev,
                                 const int32_t* type_ids_dev, void* out_dev, void* stream);
/* End to end with HOST buffers (pinned or pageable): prepare_batch + H2D of ids + forward +
 * D2H of the final hidden states; returns after the output is in out_host. */
rt_status rt_encoder_forward_host(rt_encoder* enc, const int32_t* lens_tokens, int n_seq,
                                  const int32_t* ids_host, void* out_host);
/* The same in two halves, so that a caller keeps two batches in flight: submit enqueues
 * prepare_batch + forward on the encoder's own stream, the H2D of the ids on a second stream
 * (into a per-batch buffer, under the previous batch's kernels) and the D2H of the result on a
 * third (the copy of batch i overlaps the kernels of batch i+1) and returns at once
 * with a ticket; wait blocks until that batch's output is in out_host.  ids_host and out_host
 * belong to the library between the two calls (pinned memory, or the copies block).  A third
 * submit first waits for the oldest batch.  rt_encoder_forward_host == submit + wait.
 * For drivers shaped like the batch loop of python/benchmark/end2end.py:79-89 (one
 * update_meta_data + one model call per batch) that feed from and return to host memory. */
rt_status rt_encoder_submit_host(rt_encoder* enc, const int32_t* lens_tokens, int n_seq, const int32_t* ids_host,
                                 void* out_host, uint64_t* ticket);
rt_status rt_encoder_wait_host(rt_encoder* enc, uint64_t ticket);

/* The three operators of python/pybind.cpp:12-56 on one layer's weights.
 * attention: layers/multi_headed_attention.cpp:154-216; intermediate: layers/bert_intermediate.cpp:7-29;
 * output: layers/bert_output.cpp:7-44 (out_dev may alias the layer input). */
rt_status rt_encoder_attention(rt_encoder* enc, int layer, const void* input_dev, void* output_dev, void* stream);
rt_status rt_encoder_intermediate(rt_encoder* enc, int layer, const void* input_dev, void* output_dev, void* stream);
rt_status rt_encoder_output(rt_encoder* enc, int layer, const void* ffn_dev, const void* residual_dev,
                            void* out_dev, void* stream);

/* Accessors used by tests and the Python shim. */
rt_status rt_encoder_get_table(rt_encoder* enc, int layer, const int32_t** kv_ptr_host,
                               const int32_t** kv_idx_host, int64_t* visits);
rt_status rt_encoder_get_scratch(rt_encoder* enc, const char* name, void** ptr_dev, size_t* bytes);
/* device milliseconds of the last forward per stage: "gemm","transpose","attention","layernorm","gelu",
 * "embeddings","pre_process" (host wait for metadata) - the keys of the reference's info dict;
 * "host_blocked": cumulative milliseconds the calling thread has waited for the GPU to release a
 * metadata slot or a host-pipeline buffer (host time that is not host work). */
rt_status rt_encoder_get_timing(rt_encoder* enc, const char* key, float* ms_out);
rt_status rt_encoder_enable_timing(rt_encoder* enc, int on);
rt_status rt_encoder_kernel_launches(rt_encoder* enc, int64_t* launches_out);
/* options: "fuse_gelu" (1: bias+GELU in the FFN-up GEMM epilogue, 0: separate rt_bias_gelu kernel);
 * "fuse_qkv" (1: rt_gemm_qkv, 0: rt_gemm + rt_qkv_bias_transpose); "fuse_layernorm" (LayerNorm in the epilogue of
 * the hidden-wide projections, rt_gemm_bias_residual_layernorm: 0 never; 1 where it measured faster, i.e.
 * the FFN-down projection of a 768-wide model; 2 both projections of 768- and 1024-wide models);
 * "fuse_residual" (1: bias + residual added in the projection GEMM's epilogue, LayerNorm reads one tensor;
 * default 0: it costs one more 16-bit rounding and measured slower; ignored where fuse_layernorm applies).
 * fuse_gelu, fuse_qkv and fuse_layernorm default to 1. */
rt_status rt_encoder_set_option(rt_encoder* enc, const char* name, int value);
rt_status rt_encoder_get_option(rt_encoder* enc, const char* name, int* value_out);
/* work-list statistics of one layer of the prepared batch */
rt_status rt_encoder_plan_stats(rt_encoder* enc, int layer, int64_t* entries_out, int64_t* visits_out,
                                int32_t* items_out);
/* Synchronises the device and reports (then clears) a kernel that gave up on a bounded wait. */
rt_status rt_check_device(void);
/* Self-test of that error path: launches one CTA that waits, for at most limit_cycles SM clocks
 * (1 .. 2e8), on a barrier nothing arrives on.  The kernel then returns normally and leaves wait
 * site 901 in the error word: target 0 = the per-device word rt_check_device() reads, target 1 =
 * the status word of rt_sparse_attention_static (reported by that entry point's next call).
 * Nothing faults or traps; the device stays usable.  The reference has no error reporting at all
 * (layers/kernels/mat_mul.cpp:50-55 prints and exits), so this has no counterpart there. */
rt_status rt_selftest_bounded_wait(int64_t limit_cycles, int target, void* stream);
/* Kernel launches made by this library in this process so far. */
int64_t rt_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* RAPTOR_B200_H_ */
