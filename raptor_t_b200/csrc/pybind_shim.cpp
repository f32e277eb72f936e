// pybind11 module `raptor_t`: the operator API of the reference's extension module
// (python/pybind.cpp:11-80, built by python/setup.py:4-19) on top of this library's C ABI.
//
// Same classes, constructor arguments, call arguments and in-place output convention:
//   BertAttention(qkv_weight[H,3H], qkv_bias, dense_weight[H,H], dense_bias, ln_weight, ln_bias,
//                 num_attention_heads, layer_idx, async)
//     (input[T,H], attention_mask, output[T,H], seq_position_info, seq_len_info_tensor,
//      partition_part_index_tensor, partition_part_tensor, block_limit, info,
//      kernel_fusion=True, balanced=True) -> info                     python/pybind.cpp:12-21
//   multi_headed_attention  = the same class under its base-class name (python/pybind.cpp:23-37)
//   BertIntermediate(dense_weight[H,F], dense_bias)(input, output, info, kernel_fusion=True)   :40-46
//   BertOutput(dense_weight[F,H], dense_bias, ln_weight, ln_bias)
//     (hidden_states[T,F], input_tensor[T,H], output[T,H], info, kernel_fusion=True)           :48-56
//   TensorSet(total_seq_len, to_select_index_len, to_select_index_position_len)
//     .update_tensor_set(...), TensorSet.get_instance()                                         :66-71
//   MetaData().update_meta_data(T, to_select_index_len, to_select_index_position_len,
//     seq_len_info), .terminate_thread()                                                        :73-78
//
// Every body is a sequence of calls into include/raptor_b200.h; torch is used for the tensors'
// memory and for the current stream only.  Weights arrive [in, out] (python/modeling_bert.py:
// 84-91, 107-113, 138-163) and are re-laid-out once to [out, in] for the TMA-fed GEMMs.
// As in the reference, MetaData::update_meta_data starts one host task per registered
// attention layer (layers/multi_headed_attention.h:72-110) that builds that layer's block table
// and work list and uploads them on a side stream while the main thread issues the QKV GEMM;
// the layer joins its task right before the attention kernel ("pre_process" in info).
// The partition tensors and block_limit are accepted for signature compatibility: the kernel's
// own work list (pairs of query blocks per CTA) is built from the block table.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <chrono>
#include <future>
#include <map>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/raptor_b200.h"

namespace {

using InfoMap = std::map<std::string, float>;

void check(rt_status s) {
  if (s != RT_OK) throw std::runtime_error(std::string("raptor_b200 error ") + std::to_string(s) + ": " + rt_last_error());
}

int dtype_of(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return RT_BF16;
  if (t.scalar_type() == torch::kFloat16) return RT_F16;
  throw std::runtime_error("raptor_t: expected a float16 or bfloat16 tensor");
}

void* stream_of_current() { return at::cuda::getCurrentCUDAStream().stream(); }

void require_cuda(const torch::Tensor& t, const char* what) {
  if (!t.is_cuda() || !t.is_contiguous())
    throw std::runtime_error(std::string("raptor_t: ") + what + " must be a contiguous CUDA tensor (there is no CPU path)");
}

// Module-wide model options the reference hard-codes (layers/bert_attention.h:37-40,
// layers/bert_output.cpp:23): settable once from Python through set_model_options().
struct ModelOptions {
  int num_rand = 3, max_pos = 4096, pattern = RT_PATTERN_BIGBIRD, band_half = 4;
  float eps = 1e-12f;
};
ModelOptions& options() {
  static ModelOptions o;
  return o;
}

// Adds the device time of fn() in seconds to info[key] when the caller asked for that key
// (the reference adds host time around a blocking launch, layers/kernels/add_bias_act.cu:129-132).
template <typename F>
void timed(InfoMap& info, const char* key, F&& fn) {
  auto it = info.find(key);
  if (it == info.end()) {
    fn();
    return;
  }
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  cudaEventRecord(a, st);
  fn();
  cudaEventRecord(b, st);
  cudaEventSynchronize(b);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, b);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  it->second += ms * 1e-3f;
}

// ---------------------------------------------------------------------------------------------
// TensorSet: process-wide scratch buffers resized per batch (layers/tensor_set.h:36-65)
// ---------------------------------------------------------------------------------------------
class TensorSet {
 public:
  TensorSet(int64_t total_seq_len, int64_t to_select_index_len, int64_t to_select_index_position_len)
      : total_seq_len_(total_seq_len), index_len_(to_select_index_len), position_len_(to_select_index_position_len) {
    std::lock_guard<std::mutex> lk(mu());
    if (!instance()) instance() = this;
  }
  static TensorSet* get_instance() {
    std::lock_guard<std::mutex> lk(mu());
    if (!instance()) instance() = new TensorSet(4096, 622, 65, 0);
    return instance();
  }
  void update_tensor_set(int64_t total_seq_len, int64_t to_select_index_len, int64_t to_select_index_position_len,
                         std::vector<int> seq_len_info) {
    total_seq_len_ = total_seq_len;
    index_len_ = to_select_index_len;
    position_len_ = to_select_index_position_len;
    seq_len_info_ = std::move(seq_len_info);
  }
  // [total_seq_len, cols] view of the named buffer; (re)allocated when the batch or model grows
  torch::Tensor get(const std::string& name, int64_t cols, torch::ScalarType dtype) {
    auto& t = tensors_[name];
    if (!t.defined() || t.size(0) < total_seq_len_ || t.size(1) != cols || t.scalar_type() != dtype)
      t = torch::empty({std::max<int64_t>(total_seq_len_, 1), cols}, torch::dtype(dtype).device(torch::kCUDA));
    return t.narrow(0, 0, total_seq_len_);
  }
  torch::Tensor get_tensor(const std::string& name) {
    auto it = tensors_.find(name);
    if (it == tensors_.end() || !it->second.defined()) {
      printf("no exists tensor\n");  // layers/tensor_set.cpp:30-33
      return torch::empty({0});
    }
    return it->second.narrow(0, 0, total_seq_len_);
  }
  std::vector<int32_t> lens_tokens() const {
    std::vector<int32_t> lens;
    for (size_t i = 0; i + 1 < seq_len_info_.size(); ++i) lens.push_back((seq_len_info_[i + 1] - seq_len_info_[i]) * 64);
    return lens;
  }
  int64_t total_seq_len() const { return total_seq_len_; }

 private:
  TensorSet(int64_t a, int64_t b, int64_t c, int) : total_seq_len_(a), index_len_(b), position_len_(c) {}
  static TensorSet*& instance() {
    static TensorSet* p = nullptr;
    return p;
  }
  static std::mutex& mu() {
    static std::mutex m;
    return m;
  }
  int64_t total_seq_len_, index_len_, position_len_;
  std::vector<int> seq_len_info_{0};
  std::map<std::string, torch::Tensor> tensors_;
};

// ---------------------------------------------------------------------------------------------
// Attention layer + MetaData
// ---------------------------------------------------------------------------------------------
class BertAttention;

struct LayerRegistry {
  std::mutex mu;
  std::vector<BertAttention*> layers;
  torch::Tensor block_seq;  // per packed 64-token block {first token of its sequence, length}: the fused QKV epilogue's map
  torch::Tensor seq_prefix; // int32 [B+1] block offsets of the sequences (device): the pooler's "first token" map
  static LayerRegistry& get() {
    static LayerRegistry r;
    return r;
  }
};

struct PlanResult {
  rt_attn_plan* plan = nullptr;
  std::string error;
};

class BertAttention {
 public:
  BertAttention(torch::Tensor qkv_weight, torch::Tensor qkv_bias, torch::Tensor dense_weight, torch::Tensor dense_bias,
                torch::Tensor layer_norm_weight, torch::Tensor layer_norm_bias, int64_t num_attention_heads,
                int layer_idx, bool async)
      : heads_(static_cast<int>(num_attention_heads)), layer_idx_(layer_idx), async_(async) {
    require_cuda(qkv_weight, "qkv_weight");
    hidden_ = static_cast<int>(qkv_weight.size(0));
    if (hidden_ != heads_ * 64) throw std::runtime_error("raptor_t: head size must be 64");
    dtype_ = dtype_of(qkv_weight);
    qkv_w_ = qkv_weight.t().contiguous();  // [3H, H]
    qkv_b_ = qkv_bias.contiguous();
    dense_w_ = dense_weight.t().contiguous();
    dense_b_ = dense_bias.contiguous();
    ln_w_ = layer_norm_weight.contiguous();
    ln_b_ = layer_norm_bias.contiguous();
    auto& reg = LayerRegistry::get();
    std::lock_guard<std::mutex> lk(reg.mu);
    reg.layers.push_back(this);
  }
  ~BertAttention() {
    drop_plan();
    auto& reg = LayerRegistry::get();
    std::lock_guard<std::mutex> lk(reg.mu);
    for (auto& p : reg.layers)
      if (p == this) p = nullptr;
  }

  rt_config config() const {
    const ModelOptions& o = options();
    rt_config c{};
    c.hidden = hidden_;
    c.heads = heads_;
    c.ffn = 4 * hidden_;
    c.layers = 1;
    c.block = 64;
    c.num_rand = o.num_rand;
    c.max_pos = o.max_pos;
    c.vocab = 1;
    c.type_vocab = 1;
    c.pattern = o.pattern;
    c.band_half = o.band_half;
    c.dtype = dtype_;
    c.eps = o.eps;
    return c;
  }

  // Host task of one batch: block table of this layer (seeded by its index) -> work list -> upload.
  PlanResult build_plan(std::vector<int32_t> lens, int device) const {
    PlanResult r;
    try {
      c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
      const rt_config c = config();
      int64_t visits = 0;
      check(rt_count_visits(&c, lens.data(), static_cast<int>(lens.size()), &visits));
      int64_t n_blocks = 0;
      for (int32_t n : lens) n_blocks += n / 64;
      std::vector<int32_t> kv_ptr(n_blocks + 1), kv_idx(static_cast<size_t>(visits) * heads_);
      check(rt_build_block_csr(&c, static_cast<uint32_t>(layer_idx_), lens.data(), static_cast<int>(lens.size()),
                               kv_ptr.data(), kv_idx.data()));
      auto side = c10::cuda::getStreamFromPool(false, static_cast<c10::DeviceIndex>(device));
      check(rt_attn_plan_create(&c, lens.data(), static_cast<int>(lens.size()), kv_ptr.data(), kv_idx.data(), 0, -1,
                                side.stream(), &r.plan));
    } catch (const std::exception& e) {
      r.error = e.what();
    }
    return r;
  }

  void kick(const std::vector<int32_t>& lens, int device) {
    drop_plan();
    if (async_) pending_ = std::async(std::launch::async, &BertAttention::build_plan, this, lens, device);
    else sync_lens_ = lens;
    device_ = device;
  }

  void join() {
    if (pending_.valid()) pending_.wait();
  }

  // attention_mask and the two partition tensors are not read (the batch is padding-free and the kernel
  // builds its own work list), so None is accepted for them as well as the tensors the reference passes
  InfoMap call(const torch::Tensor& input_tensor, const std::optional<torch::Tensor>& /*attention_mask*/,
               torch::Tensor& output, const std::vector<int> /*seq_position_info*/, torch::Tensor& seq_len_info_tensor,
               const std::optional<torch::Tensor>& /*partition_part_index_tensor*/,
               const std::optional<torch::Tensor>& /*partition_part_tensor*/, const int /*block_limit*/, InfoMap& info,
               bool kernel_fusion, bool /*balanced*/) {
    require_cuda(input_tensor, "input_tensor");
    require_cuda(output, "output");
    TensorSet* ts = TensorSet::get_instance();
    const int T = static_cast<int>(input_tensor.size(0));
    const auto st_dtype = input_tensor.scalar_type();
    torch::Tensor q = ts->get("q_out", hidden_, st_dtype), k = ts->get("k_out", hidden_, st_dtype);
    torch::Tensor v = ts->get("v_out", hidden_, st_dtype), ctx = ts->get("attention_out", hidden_, st_dtype);
    torch::Tensor dense = ts->get("dense_out", hidden_, st_dtype);
    void* st = stream_of_current();
    auto& reg = LayerRegistry::get();
    if (kernel_fusion && reg.block_seq.defined() && info.find("add_bias_and_transpose_kernel") == info.end()) {
      check(rt_gemm_qkv(q.data_ptr(), k.data_ptr(), v.data_ptr(), input_tensor.data_ptr(), qkv_w_.data_ptr(),
                        qkv_b_.data_ptr(), reg.block_seq.data_ptr<int32_t>(), T, heads_, hidden_, 0.125f, dtype_, st));
    } else {
      torch::Tensor qkv = ts->get("tmp_qkv_out1", 3 * hidden_, st_dtype);
      check(rt_gemm(qkv.data_ptr(), input_tensor.data_ptr(), qkv_w_.data_ptr(), nullptr, T, 3 * hidden_, hidden_,
                    RT_EPI_NONE, dtype_, st));
      require_cuda(seq_len_info_tensor, "seq_len_info_tensor");
      timed(info, "add_bias_and_transpose_kernel", [&] {
        check(rt_qkv_bias_transpose(qkv.data_ptr(), qkv_b_.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                    seq_len_info_tensor.data_ptr<int32_t>(),
                                    static_cast<int>(seq_len_info_tensor.numel()) - 1, T / 64, heads_, 0.125f, dtype_, st));
      });
    }
    // the layer's table: wait for the host task started by MetaData.update_meta_data
    const auto t0 = std::chrono::steady_clock::now();
    if (pending_.valid()) {
      PlanResult r = pending_.get();
      if (!r.error.empty()) throw std::runtime_error(r.error);
      plan_ = r.plan;
    } else if (!sync_lens_.empty()) {
      PlanResult r = build_plan(sync_lens_, device_);
      sync_lens_.clear();
      if (!r.error.empty()) throw std::runtime_error(r.error);
      plan_ = r.plan;
    }
    if (!plan_) throw std::runtime_error("raptor_t: BertAttention called before MetaData.update_meta_data");
    auto pre = info.find("pre_process");
    if (pre != info.end())
      pre->second += std::chrono::duration<float>(std::chrono::steady_clock::now() - t0).count();
    timed(info, "attention", [&] {
      check(rt_sparse_attention(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), plan_, 1.0f, dtype_, st));
    });
    check(rt_gemm(dense.data_ptr(), ctx.data_ptr(), dense_w_.data_ptr(), nullptr, T, hidden_, hidden_, RT_EPI_NONE,
                  dtype_, st));
    timed(info, "add_bias_and_layernorm_kernel", [&] {
      check(rt_bias_residual_layernorm(output.data_ptr(), dense.data_ptr(), dense_b_.data_ptr(), input_tensor.data_ptr(),
                                       ln_w_.data_ptr(), ln_b_.data_ptr(), T, hidden_, options().eps, dtype_, st));
    });
    return info;
  }

 private:
  void drop_plan() {
    if (pending_.valid()) {
      PlanResult r = pending_.get();
      if (r.plan) rt_attn_plan_destroy(r.plan);
    }
    if (plan_) {
      cudaDeviceSynchronize();  // the previous batch's attention kernel may still read it
      rt_attn_plan_destroy(plan_);
      plan_ = nullptr;
    }
  }

  int heads_, hidden_ = 0, layer_idx_, dtype_ = RT_F16, device_ = 0;
  bool async_;
  torch::Tensor qkv_w_, qkv_b_, dense_w_, dense_b_, ln_w_, ln_b_;
  std::future<PlanResult> pending_;
  std::vector<int32_t> sync_lens_;
  rt_attn_plan* plan_ = nullptr;
};

class MetaData {
 public:
  // layers/metadata.cpp:6-18: once per batch, before the forward pass
  void update_meta_data(int64_t total_seq_len, int64_t to_select_index_len, int64_t to_select_index_position_len,
                        std::vector<int> seq_len_info) {
    TensorSet* ts = TensorSet::get_instance();
    ts->update_tensor_set(total_seq_len, to_select_index_len, to_select_index_position_len, seq_len_info);
    const std::vector<int32_t> lens = ts->lens_tokens();
    int64_t sum = 0;
    for (int32_t n : lens) sum += n;
    if (sum != total_seq_len) throw std::runtime_error("update_meta_data: seq_len_info does not add up to total_seq_len");
    int device = 0;
    cudaGetDevice(&device);
    // per-block {first token, length} for the fused QKV epilogue
    std::vector<int32_t> bs;
    int32_t t0 = 0;
    for (int32_t n : lens) {
      for (int i = 0; i < n / 64; ++i) {
        bs.push_back(t0);
        bs.push_back(n);
      }
      t0 += n;
    }
    auto& reg = LayerRegistry::get();
    std::lock_guard<std::mutex> lk(reg.mu);
    reg.block_seq = torch::from_blob(bs.data(), {static_cast<int64_t>(bs.size())}, torch::kInt32).clone().to(torch::kCUDA);
    reg.seq_prefix = torch::from_blob(seq_len_info.data(), {static_cast<int64_t>(seq_len_info.size())}, torch::kInt32)
                         .clone().to(torch::kCUDA);
    for (BertAttention* l : reg.layers)
      if (l) l->kick(lens, device);
  }
  // layers/metadata.cpp:20-27: shutdown; here: join every pending host task
  void terminate_thread() {
    auto& reg = LayerRegistry::get();
    std::lock_guard<std::mutex> lk(reg.mu);
    for (BertAttention* l : reg.layers)
      if (l) l->join();
  }
};

class BertIntermediate {
 public:
  BertIntermediate(torch::Tensor dense_weight, torch::Tensor dense_bias) {
    require_cuda(dense_weight, "dense_weight");
    dtype_ = dtype_of(dense_weight);
    hidden_ = static_cast<int>(dense_weight.size(0));
    ffn_ = static_cast<int>(dense_weight.size(1));
    w_ = dense_weight.t().contiguous();  // [F, H]
    b_ = dense_bias.contiguous();
  }
  InfoMap call(const torch::Tensor& input_tensor, torch::Tensor& output, InfoMap& info, bool kernel_fusion) {
    require_cuda(input_tensor, "input_tensor");
    require_cuda(output, "output");
    const int T = static_cast<int>(input_tensor.size(0));
    void* st = stream_of_current();
    if (kernel_fusion && info.find("add_bias_act_kernel") == info.end()) {
      check(rt_gemm(output.data_ptr(), input_tensor.data_ptr(), w_.data_ptr(), b_.data_ptr(), T, ffn_, hidden_,
                    RT_EPI_BIAS_GELU, dtype_, st));
    } else {
      check(rt_gemm(output.data_ptr(), input_tensor.data_ptr(), w_.data_ptr(), nullptr, T, ffn_, hidden_, RT_EPI_NONE,
                    dtype_, st));
      timed(info, "add_bias_act_kernel", [&] { check(rt_bias_gelu(output.data_ptr(), b_.data_ptr(), T, ffn_, dtype_, st)); });
    }
    return info;
  }

 private:
  int dtype_, hidden_, ffn_;
  torch::Tensor w_, b_;
};

class BertOutput {
 public:
  BertOutput(torch::Tensor dense_weight, torch::Tensor dense_bias, torch::Tensor layer_norm_weight,
             torch::Tensor layer_norm_bias) {
    require_cuda(dense_weight, "dense_weight");
    dtype_ = dtype_of(dense_weight);
    ffn_ = static_cast<int>(dense_weight.size(0));
    hidden_ = static_cast<int>(dense_weight.size(1));
    w_ = dense_weight.t().contiguous();  // [H, F]
    b_ = dense_bias.contiguous();
    ln_w_ = layer_norm_weight.contiguous();
    ln_b_ = layer_norm_bias.contiguous();
  }
  InfoMap call(const torch::Tensor& hidden_states, const torch::Tensor& input_tensor, torch::Tensor& output,
               InfoMap& info, bool /*kernel_fusion*/) {
    require_cuda(hidden_states, "hidden_states");
    require_cuda(input_tensor, "input_tensor");
    require_cuda(output, "output");
    const int T = static_cast<int>(hidden_states.size(0));
    void* st = stream_of_current();
    torch::Tensor dense = TensorSet::get_instance()->get("dense_out", hidden_, hidden_states.scalar_type());
    check(rt_gemm(dense.data_ptr(), hidden_states.data_ptr(), w_.data_ptr(), nullptr, T, hidden_, ffn_, RT_EPI_NONE, dtype_,
                  st));
    timed(info, "add_bias_and_layernorm_kernel", [&] {
      check(rt_bias_residual_layernorm(output.data_ptr(), dense.data_ptr(), b_.data_ptr(), input_tensor.data_ptr(),
                                       ln_w_.data_ptr(), ln_b_.data_ptr(), T, hidden_, options().eps, dtype_, st));
    });
    return info;
  }

 private:
  int dtype_, hidden_, ffn_;
  torch::Tensor w_, b_, ln_w_, ln_b_;
};

// The pooler the reference declares and leaves commented out (python/pybind.cpp:58-64):
// output fp32 [B, H] = tanh(dense(first token of every sequence of the current batch)).
class BertPooler {
 public:
  BertPooler(torch::Tensor dense_weight, torch::Tensor dense_bias) {
    require_cuda(dense_weight, "dense_weight");
    dtype_ = dtype_of(dense_weight);
    hidden_ = static_cast<int>(dense_weight.size(0));
    w_ = dense_weight.t().contiguous();  // [out, in]
    b_ = dense_bias.contiguous();
  }
  torch::Tensor call(const torch::Tensor& input_tensor, torch::Tensor& output) {
    require_cuda(input_tensor, "input_tensor");
    require_cuda(output, "output");
    auto& reg = LayerRegistry::get();
    if (!reg.seq_prefix.defined()) throw std::runtime_error("raptor_t: BertPooler called before MetaData.update_meta_data");
    if (output.scalar_type() != torch::kFloat32) throw std::runtime_error("raptor_t: BertPooler writes a float32 output");
    check(rt_pooler(output.data_ptr<float>(), input_tensor.data_ptr(), reg.seq_prefix.data_ptr<int32_t>(),
                    static_cast<int>(reg.seq_prefix.numel()) - 1, w_.data_ptr(), b_.data_ptr(), hidden_, dtype_,
                    stream_of_current()));
    return output;
  }

 private:
  int dtype_, hidden_;
  torch::Tensor w_, b_;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.doc() = "Operator API of WongHuLin/Raptor-T's extension module on the raptor_b200 C ABI (B200, sm_100a)";

  auto attention = py::class_<BertAttention>(m, "BertAttention")
      .def(py::init<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int,
                    bool>(),
           py::arg("qkv_weight"), py::arg("qkv_bias"), py::arg("dense_weight"), py::arg("dense_bias"),
           py::arg("layer_norm_weight"), py::arg("layer_norm_bias"), py::arg("num_attention_heads"), py::arg("layer_idx"),
           py::arg("async") = true)
      .def("__call__", &BertAttention::call, py::arg("input_tensor"), py::arg("attention_mask"), py::arg("output"),
           py::arg("seq_position_info"), py::arg("seq_len_info_tensor"), py::arg("partition_part_index_tensor"),
           py::arg("partition_part_tensor"), py::arg("block_limit"), py::arg("info"), py::arg("kernel_fusion") = true,
           py::arg("balanced") = true);
  m.attr("multi_headed_attention") = attention;

  py::class_<BertIntermediate>(m, "BertIntermediate")
      .def(py::init<torch::Tensor, torch::Tensor>(), py::arg("dense_weight"), py::arg("dense_bias"))
      .def("__call__", &BertIntermediate::call, py::arg("input_tensor"), py::arg("output"), py::arg("info"),
           py::arg("kernel_fusion") = true);

  py::class_<BertOutput>(m, "BertOutput")
      .def(py::init<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>(), py::arg("dense_weight"),
           py::arg("dense_bias"), py::arg("layer_norm_weight"), py::arg("layer_norm_bias"))
      .def("__call__", &BertOutput::call, py::arg("hidden_states"), py::arg("input_tensor"), py::arg("output"),
           py::arg("info"), py::arg("kernel_fusion") = true);

  py::class_<BertPooler>(m, "BertPooler")
      .def(py::init<torch::Tensor, torch::Tensor>(), py::arg("dense_weight"), py::arg("dense_bias"))
      .def("__call__", &BertPooler::call, py::arg("input_tensor"), py::arg("output"));

  py::class_<TensorSet, std::unique_ptr<TensorSet, py::nodelete>>(m, "TensorSet")
      .def(py::init<int64_t, int64_t, int64_t>(), py::arg("total_seq_len"), py::arg("to_select_index_len"),
           py::arg("to_select_index_position_len"))
      .def("update_tensor_set", &TensorSet::update_tensor_set)
      .def("get_tensor", &TensorSet::get_tensor)
      .def_static("get_instance", &TensorSet::get_instance, py::return_value_policy::reference);

  py::class_<MetaData>(m, "MetaData")
      .def(py::init<>())
      .def("update_meta_data", &MetaData::update_meta_data)
      .def("terminate_thread", &MetaData::terminate_thread);

  // Not in the reference: the model constants it hard-codes (3 random blocks, 4096 positions,
  // LayerNorm eps) for models of another shape.
  m.def("set_model_options",
        [](int num_rand, int max_pos, const std::string& pattern, int band_half, float eps) {
          ModelOptions& o = options();
          o.num_rand = num_rand;
          o.max_pos = max_pos;
          o.pattern = pattern == "band" ? RT_PATTERN_BAND : RT_PATTERN_BIGBIRD;
          o.band_half = band_half;
          o.eps = eps;
        },
        py::arg("num_rand") = 3, py::arg("max_pos") = 4096, py::arg("pattern") = "bigbird", py::arg("band_half") = 4,
        py::arg("eps") = 1e-12f);
}
