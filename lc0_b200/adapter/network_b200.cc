// lc0 plug-in for the B200 backend: the one translation unit that includes lc0 headers.
//
// It derives lczero::Network / lczero::NetworkComputation (src/neural/network.h:56-126), flattens the
// decoded weights (lczero::MultiHeadWeights, src/neural/network_legacy.h:178-229) into the named tensors
// the C ABI of include/b200nn.h expects, and registers the factory with REGISTER_NETWORK
// (src/neural/factory.h:111-142) under the names "b200" (fp16), "b200-bf16" and "b200-fp32".
// It also registers "b200-native", a direct lczero::Backend (src/neural/backend.h:64-133) that skips the
// Network-to-Backend wrapper of src/neural/wrapper.cc: the legal-move policy softmax of that wrapper runs on the
// device and only the legal moves' probabilities come back to the host.
// Build: add this file to lc0's source list and link libb200nn.so; this file is GPL-3
// like lc0 because it includes lc0 headers, the library behind the C ABI contains no lc0 code.
//
// Options (parsed like the reference CUDA backend's, src/neural/backends/cuda/network_cuda.cc:210-254):
//   gpu=<id>  max_batch=<n> (default 1024)  slots=<n> (concurrent computations, default 2)
//   policy_head=<name>  value_head=<name>  mlh=<bool>  tensor_cores=<bool>  graph_capture=<bool>
// "b200-native" only: precision=<fp16|bf16|fp32>  device_encode=<bool> (default true: the game history goes to the
//   device and EncodePositionForNN's planes are produced there)
#include <memory>
#include <string>
#include <vector>

#include <mutex>

#include "chess/position.h"
#include "include/b200nn.h"
#include "neural/backend.h"
#include "neural/encoder.h"
#include "neural/factory.h"
#include "neural/loader.h"
#include "neural/network_legacy.h"
#include "neural/register.h"
#include "neural/shared_params.h"
#include "neural/tables/activation_function.h"
#include "utils/exception.h"

namespace lczero {
namespace {

void Check(int rc) {
  if (rc != B200_OK) throw Exception(std::string("b200 backend: ") + b200_last_error());
}

class B200Network;

class B200Computation : public NetworkComputation {
 public:
  explicit B200Computation(b200_net* net, bool wdl, bool mlh) : wdl_(wdl), mlh_(mlh) {
    Check(b200_comp_create(net, &comp_));
  }
  ~B200Computation() override { b200_comp_destroy(comp_); }

  void AddInput(InputPlanes&& input) override {
    if (input.size() != static_cast<size_t>(kInputPlanes)) throw Exception("b200 backend: expected 112 input planes");
    uint64_t masks[kInputPlanes];
    float values[kInputPlanes];
    for (int i = 0; i < kInputPlanes; ++i) {
      masks[i] = input[i].mask;
      values[i] = input[i].value;
    }
    Check(b200_comp_add_input(comp_, masks, values));
  }
  void ComputeBlocking() override { Check(b200_comp_compute(comp_)); }
  int GetBatchSize() const override { return b200_comp_batch_size(comp_); }
  float GetQVal(int sample) const override { return b200_comp_q(comp_, sample); }
  float GetDVal(int sample) const override { return wdl_ ? b200_comp_d(comp_, sample) : 0.0f; }
  float GetMVal(int sample) const override { return mlh_ ? b200_comp_m(comp_, sample) : 0.0f; }
  float GetPVal(int sample, int move_id) const override { return b200_comp_p(comp_, sample, move_id); }

 private:
  b200_comp* comp_ = nullptr;
  bool wdl_, mlh_;
};

class Builder {
 public:
  Builder() { Check(b200_builder_create(&b_)); }
  ~Builder() { b200_builder_destroy(b_); }
  void Int(const char* key, long long v) { Check(b200_builder_set_int(b_, key, v)); }
  void Tensor(const std::string& name, const std::vector<float>& v) {
    if (!v.empty()) Check(b200_builder_add_tensor(b_, name.c_str(), v.data(), v.size()));
  }
  void Conv(const std::string& p, const BaseWeights::ConvBlock& c) {
    Tensor(p + ".weights", c.weights);  // batch norm is already folded by ConvBlock's constructor
    Tensor(p + ".biases", c.biases);
  }
  void Encoder(const std::string& p, const BaseWeights::EncoderLayer& e) {
    Tensor(p + ".mha.q_w", e.mha.q_w);
    Tensor(p + ".mha.q_b", e.mha.q_b);
    Tensor(p + ".mha.k_w", e.mha.k_w);
    Tensor(p + ".mha.k_b", e.mha.k_b);
    Tensor(p + ".mha.v_w", e.mha.v_w);
    Tensor(p + ".mha.v_b", e.mha.v_b);
    Tensor(p + ".mha.dense_w", e.mha.dense_w);
    Tensor(p + ".mha.dense_b", e.mha.dense_b);
    if (e.mha.has_smolgen) {
      const auto& s = e.mha.smolgen;
      Tensor(p + ".mha.smolgen.compress", s.compress);
      Tensor(p + ".mha.smolgen.dense1_w", s.dense1_w);
      Tensor(p + ".mha.smolgen.dense1_b", s.dense1_b);
      Tensor(p + ".mha.smolgen.ln1_gammas", s.ln1_gammas);
      Tensor(p + ".mha.smolgen.ln1_betas", s.ln1_betas);
      Tensor(p + ".mha.smolgen.dense2_w", s.dense2_w);
      Tensor(p + ".mha.smolgen.dense2_b", s.dense2_b);
      Tensor(p + ".mha.smolgen.ln2_gammas", s.ln2_gammas);
      Tensor(p + ".mha.smolgen.ln2_betas", s.ln2_betas);
    }
    Tensor(p + ".ln1_gammas", e.ln1_gammas);
    Tensor(p + ".ln1_betas", e.ln1_betas);
    Tensor(p + ".ffn.dense1_w", e.ffn.dense1_w);
    Tensor(p + ".ffn.dense1_b", e.ffn.dense1_b);
    Tensor(p + ".ffn.dense2_w", e.ffn.dense2_w);
    Tensor(p + ".ffn.dense2_b", e.ffn.dense2_b);
    Tensor(p + ".ln2_gammas", e.ln2_gammas);
    Tensor(p + ".ln2_betas", e.ln2_betas);
  }
  b200_builder* get() const { return b_; }

 private:
  b200_builder* b_ = nullptr;
};

// Describes the network of `file` to the library: format integers and every weight tensor by name.
void FillBuilder(const WeightsFile& file, const OptionsDict& options, Builder& b) {
  const auto nf = file.format().network_format();
  using NF = pblczero::NetworkFormat;
  const MultiHeadWeights weights(file.weights());

  const std::string policy_head = options.GetOrDefault<std::string>("policy_head", "vanilla");
  if (weights.policy_heads.count(policy_head) == 0)
    throw Exception("The policy head you specified '" + policy_head + "' does not exist in this net.");
  const std::string value_head = options.GetOrDefault<std::string>("value_head", "winner");
  if (weights.value_heads.count(value_head) == 0)
    throw Exception("The value head you specified '" + value_head + "' does not exist in this net.");
  const auto& ph = weights.policy_heads.at(policy_head);
  const auto& vh = weights.value_heads.at(value_head);

  // Activation resolution as in the reference backends (network_blas.cc:1010-1028).
  const int default_act =
      nf.default_activation() == NF::DEFAULT_ACTIVATION_MISH ? ACTIVATION_MISH : ACTIVATION_RELU;
  const int smolgen_act =
      nf.smolgen_activation() == NF::ACTIVATION_DEFAULT ? default_act : static_cast<int>(nf.smolgen_activation());
  const int ffn_act =
      nf.ffn_activation() == NF::ACTIVATION_DEFAULT ? default_act : static_cast<int>(nf.ffn_activation());

  b.Int("input_format", nf.input());
  b.Int("output_format", nf.output());
  b.Int("network", nf.network());
  b.Int("policy", nf.policy());
  b.Int("value", nf.value());
  b.Int("moves_left", nf.moves_left());
  b.Int("input_embedding", nf.input_embedding());
  b.Int("default_activation", default_act);
  b.Int("smolgen_activation", smolgen_act);
  b.Int("ffn_activation", ffn_act);
  b.Int("headcount", weights.encoder_head_count);
  b.Int("pol_headcount", ph.pol_encoder_head_count);

  b.Conv("input", weights.input);
  for (size_t i = 0; i < weights.residual.size(); ++i) {
    const auto& r = weights.residual[i];
    const std::string p = "residual." + std::to_string(i);
    b.Conv(p + ".conv1", r.conv1);
    b.Conv(p + ".conv2", r.conv2);
    if (r.has_se) {
      b.Tensor(p + ".se.w1", r.se.w1);
      b.Tensor(p + ".se.b1", r.se.b1);
      b.Tensor(p + ".se.w2", r.se.w2);
      b.Tensor(p + ".se.b2", r.se.b2);
    }
  }
  b.Tensor("ip_emb_preproc_w", weights.ip_emb_preproc_w);
  b.Tensor("ip_emb_preproc_b", weights.ip_emb_preproc_b);
  b.Tensor("ip_emb_w", weights.ip_emb_w);
  b.Tensor("ip_emb_b", weights.ip_emb_b);
  b.Tensor("ip_emb_ln_gammas", weights.ip_emb_ln_gammas);
  b.Tensor("ip_emb_ln_betas", weights.ip_emb_ln_betas);
  b.Tensor("ip_mult_gate", weights.ip_mult_gate);
  b.Tensor("ip_add_gate", weights.ip_add_gate);
  b.Tensor("ip_emb_ffn.dense1_w", weights.ip_emb_ffn.dense1_w);
  b.Tensor("ip_emb_ffn.dense1_b", weights.ip_emb_ffn.dense1_b);
  b.Tensor("ip_emb_ffn.dense2_w", weights.ip_emb_ffn.dense2_w);
  b.Tensor("ip_emb_ffn.dense2_b", weights.ip_emb_ffn.dense2_b);
  b.Tensor("ip_emb_ffn_ln_gammas", weights.ip_emb_ffn_ln_gammas);
  b.Tensor("ip_emb_ffn_ln_betas", weights.ip_emb_ffn_ln_betas);
  for (size_t i = 0; i < weights.encoder.size(); ++i) b.Encoder("encoder." + std::to_string(i), weights.encoder[i]);
  b.Tensor("smolgen_w", weights.smolgen_w);
  b.Conv("moves_left", weights.moves_left);
  b.Tensor("ip_mov_w", weights.ip_mov_w);
  b.Tensor("ip_mov_b", weights.ip_mov_b);
  b.Tensor("ip1_mov_w", weights.ip1_mov_w);
  b.Tensor("ip1_mov_b", weights.ip1_mov_b);
  b.Tensor("ip2_mov_w", weights.ip2_mov_w);
  b.Tensor("ip2_mov_b", weights.ip2_mov_b);

  b.Tensor("policy.ip_pol_w", ph.ip_pol_w);
  b.Tensor("policy.ip_pol_b", ph.ip_pol_b);
  b.Tensor("policy.ip2_pol_w", ph.ip2_pol_w);
  b.Tensor("policy.ip2_pol_b", ph.ip2_pol_b);
  b.Tensor("policy.ip3_pol_w", ph.ip3_pol_w);
  b.Tensor("policy.ip3_pol_b", ph.ip3_pol_b);
  b.Tensor("policy.ip4_pol_w", ph.ip4_pol_w);
  b.Conv("policy.policy1", ph.policy1);
  b.Conv("policy.policy", ph.policy);
  for (size_t i = 0; i < ph.pol_encoder.size(); ++i)
    b.Encoder("policy.pol_encoder." + std::to_string(i), ph.pol_encoder[i]);
  b.Conv("value.value", vh.value);
  b.Tensor("value.ip_val_w", vh.ip_val_w);
  b.Tensor("value.ip_val_b", vh.ip_val_b);
  b.Tensor("value.ip1_val_w", vh.ip1_val_w);
  b.Tensor("value.ip1_val_b", vh.ip1_val_b);
  b.Tensor("value.ip2_val_w", vh.ip2_val_w);
  b.Tensor("value.ip2_val_b", vh.ip2_val_b);

}

b200_net_options MakeNetOptions(const OptionsDict& options, int precision) {
  b200_net_options opt{};
  opt.gpu = options.GetOrDefault<int>("gpu", 0);
  opt.max_batch = options.GetOrDefault<int>("max_batch", 1024);
  opt.slots = options.GetOrDefault<int>("slots", 2);
  opt.precision = precision;
  opt.mlh = options.GetOrDefault<bool>("mlh", true) ? 1 : 0;
  opt.flags = (options.GetOrDefault<bool>("tensor_cores", true) ? 0 : B200_FLAG_NO_TENSOR_CORES) |
              (options.GetOrDefault<bool>("graph_capture", true) ? 0 : B200_FLAG_NO_GRAPHS) |
              (options.GetOrDefault<bool>("fold_ln", true) ? 0 : B200_FLAG_NO_LN_FOLD) |
              (options.GetOrDefault<bool>("merge_compress", true) ? 0 : B200_FLAG_NO_MERGED_COMPRESS) |
              (options.GetOrDefault<bool>("split_last_wave", true) ? 0 : B200_FLAG_NO_SPLIT_LAST_WAVE) |
              (options.GetOrDefault<bool>("fused_se", true) ? 0 : B200_FLAG_NO_FUSED_SE) |
              (options.GetOrDefault<bool>("winograd", false) ? B200_FLAG_WINOGRAD : 0) |
              (options.GetOrDefault<bool>("side_stream", true) ? 0 : B200_FLAG_NO_SIDE_STREAM) |
              (options.GetOrDefault<bool>("dependent_launch", true) ? 0 : B200_FLAG_NO_DEPENDENT_LAUNCH) |
              (options.GetOrDefault<bool>("tower", true) ? 0 : B200_FLAG_NO_TOWER_KERNEL);
  return opt;
}

class B200Network : public Network {
 public:
  B200Network(const WeightsFile& file, const OptionsDict& options, int precision)
      : capabilities_{file.format().network_format().input(), file.format().network_format().output(),
                      file.format().network_format().moves_left()} {
    Builder b;
    FillBuilder(file, options, b);
    const b200_net_options opt = MakeNetOptions(options, precision);
    Check(b200_net_create(b.get(), &opt, &net_));
    Check(b200_net_get_info(net_, &info_));
    if (!info_.has_mlh) capabilities_.moves_left = pblczero::NetworkFormat::MOVES_LEFT_NONE;
  }
  ~B200Network() override { b200_net_destroy(net_); }

  const NetworkCapabilities& GetCapabilities() const override { return capabilities_; }
  std::unique_ptr<NetworkComputation> NewComputation() override {
    return std::make_unique<B200Computation>(net_, info_.wdl != 0, info_.has_mlh != 0);
  }
  int GetThreads() const override { return 2; }  // one thread fills a batch while the other computes
  bool IsCpu() const override { return false; }
  int GetMiniBatchSize() const override { return 2 * info_.sm_count; }
  int GetPreferredBatchStep() const override { return 1; }
  b200_net* net() const { return net_; }
  const b200_net_info& info() const { return info_; }

 private:
  NetworkCapabilities capabilities_;
  b200_net* net_ = nullptr;
  b200_net_info info_{};
};

template <int kPrecision>
std::unique_ptr<Network> MakeB200Network(const std::optional<WeightsFile>& w, const OptionsDict& options) {
  if (!w) throw Exception("The b200 backend requires a network file.");
  return std::make_unique<B200Network>(*w, options, kPrecision);
}

// Below the reference's own GPU backends (cuda-auto is 104) so that adding the plug-in never changes the default.
REGISTER_NETWORK("b200", MakeB200Network<B200_PREC_FP16>, 90)
REGISTER_NETWORK("b200-bf16", MakeB200Network<B200_PREC_BF16>, 89)
REGISTER_NETWORK("b200-fp32", MakeB200Network<B200_PREC_FP32>, 88)


// ---- batch aggregation inside the plug-in -----------------------------------------------------------------------
// "b200-mux": what `multiplexing` over `b200` gives (MuxingComputation and MuxingNetwork, src/neural/backends/network_mux.cc:39-245), with
// the merging done by the library's aggregator (b200_mux_*): every computation keeps its inputs and results in host
// vectors of its own, ComputeBlocking() queues them and blocks until a worker has evaluated them together with the
// requests of the other search threads or games.  For selfplay with many games of small batches.
// Options: the ones of `b200` plus precision=fp16|bf16|fp32 and mux_wait_us (how long a worker that finds fewer than
// max_batch positions waits for more; default 200).
class B200MuxComputation : public NetworkComputation {
 public:
  B200MuxComputation(b200_mux* mux, bool wdl, bool mlh) : mux_(mux), wdl_(wdl), mlh_(mlh) {}
  void AddInput(InputPlanes&& input) override {
    if (input.size() != static_cast<size_t>(kInputPlanes)) throw Exception("b200 backend: expected 112 input planes");
    for (int i = 0; i < kInputPlanes; ++i) {
      masks_.push_back(input[i].mask);
      values_.push_back(input[i].value);
    }
    ++n_;
  }
  void ComputeBlocking() override {
    if (n_ == 0) return;
    policy_.resize(static_cast<size_t>(n_) * kPolicySize);
    q_.resize(n_);
    d_.resize(n_);
    m_.resize(n_);
    Check(b200_mux_eval(mux_, masks_.data(), values_.data(), n_, policy_.data(), q_.data(), d_.data(), m_.data()));
  }
  int GetBatchSize() const override { return n_; }
  float GetQVal(int sample) const override { return q_[sample]; }
  float GetDVal(int sample) const override { return wdl_ ? d_[sample] : 0.0f; }
  float GetMVal(int sample) const override { return mlh_ ? m_[sample] : 0.0f; }
  float GetPVal(int sample, int move_id) const override {
    return policy_[static_cast<size_t>(sample) * kPolicySize + move_id];
  }

 private:
  static constexpr int kPolicySize = 1858;
  b200_mux* mux_;
  bool wdl_, mlh_;
  int n_ = 0;
  std::vector<uint64_t> masks_;
  std::vector<float> values_, policy_, q_, d_, m_;
};

class B200MuxNetwork : public Network {
 public:
  B200MuxNetwork(const WeightsFile& file, const OptionsDict& options)
      : net_(file, options, PrecisionOption(options)) {
    Check(b200_mux_create(net_.net(), options.GetOrDefault<int>("max_batch", 1024),
                          options.GetOrDefault<int>("mux_wait_us", 200), &mux_));
  }
  ~B200MuxNetwork() override { b200_mux_destroy(mux_); }  // before net_, which the aggregator uses

  const NetworkCapabilities& GetCapabilities() const override { return net_.GetCapabilities(); }
  std::unique_ptr<NetworkComputation> NewComputation() override {
    return std::make_unique<B200MuxComputation>(mux_, net_.info().wdl != 0, net_.info().has_mlh != 0);
  }
  int GetThreads() const override { return 8; }  // callers only queue and wait; the aggregator owns the GPU
  bool IsCpu() const override { return false; }
  int GetMiniBatchSize() const override { return 32; }
  int GetPreferredBatchStep() const override { return 1; }

 private:
  static int PrecisionOption(const OptionsDict& options) {
    const std::string p = options.GetOrDefault<std::string>("precision", "fp16");
    if (p == "fp16") return B200_PREC_FP16;
    if (p == "bf16") return B200_PREC_BF16;
    if (p == "fp32") return B200_PREC_FP32;
    throw Exception("b200-mux: precision must be fp16, bf16 or fp32");
  }
  B200Network net_;
  b200_mux* mux_ = nullptr;
};

std::unique_ptr<Network> MakeB200MuxNetwork(const std::optional<WeightsFile>& w, const OptionsDict& options) {
  if (!w) throw Exception("The b200-mux backend requires a network file.");
  return std::make_unique<B200MuxNetwork>(*w, options);
}
REGISTER_NETWORK("b200-mux", MakeB200MuxNetwork, 86)


// ---- one batch over several GPUs ----------------------------------------------------------------------------------
// "b200-multi": what `demux` over per-GPU `b200` backends gives (DemuxingNetwork, src/neural/backends/network_demux.cc),
// with the split done by the library (b200_multi_*): a computation keeps its planes and results in host vectors and
// ComputeBlocking() hands the whole batch to b200_multi_eval_host, which cuts it into one contiguous slice per GPU.
// Options: the ones of `b200` plus precision=fp16|bf16|fp32, gpus=<count> (default 2) and first_gpu (default 0);
// max_batch is per GPU.
class B200MultiComputation : public NetworkComputation {
 public:
  B200MultiComputation(b200_multi* multi, bool wdl, bool mlh) : multi_(multi), wdl_(wdl), mlh_(mlh) {}
  void AddInput(InputPlanes&& input) override {
    if (input.size() != static_cast<size_t>(kInputPlanes)) throw Exception("b200 backend: expected 112 input planes");
    for (int i = 0; i < kInputPlanes; ++i) {
      masks_.push_back(input[i].mask);
      values_.push_back(input[i].value);
    }
    ++n_;
  }
  void ComputeBlocking() override {
    if (n_ == 0) return;
    policy_.resize(static_cast<size_t>(n_) * kPolicySize);
    q_.resize(n_);
    d_.resize(n_);
    m_.resize(n_);
    Check(b200_multi_eval_host(multi_, masks_.data(), values_.data(), n_, policy_.data(), q_.data(), d_.data(),
                               m_.data()));
  }
  int GetBatchSize() const override { return n_; }
  float GetQVal(int sample) const override { return q_[sample]; }
  float GetDVal(int sample) const override { return wdl_ ? d_[sample] : 0.0f; }
  float GetMVal(int sample) const override { return mlh_ ? m_[sample] : 0.0f; }
  float GetPVal(int sample, int move_id) const override {
    return policy_[static_cast<size_t>(sample) * kPolicySize + move_id];
  }

 private:
  static constexpr int kPolicySize = 1858;
  b200_multi* multi_;
  bool wdl_, mlh_;
  int n_ = 0;
  std::vector<uint64_t> masks_;
  std::vector<float> values_, policy_, q_, d_, m_;
};

int PrecisionByName(const OptionsDict& options, const char* backend) {
  const std::string p = options.GetOrDefault<std::string>("precision", "fp16");
  if (p == "fp16") return B200_PREC_FP16;
  if (p == "bf16") return B200_PREC_BF16;
  if (p == "fp32") return B200_PREC_FP32;
  throw Exception(std::string(backend) + ": precision must be fp16, bf16 or fp32");
}

class B200MultiNetwork : public Network {
 public:
  B200MultiNetwork(const WeightsFile& file, const OptionsDict& options)
      : capabilities_{file.format().network_format().input(), file.format().network_format().output(),
                      file.format().network_format().moves_left()} {
    Builder b;
    FillBuilder(file, options, b);
    const b200_net_options opt = MakeNetOptions(options, PrecisionByName(options, "b200-multi"));
    const int count = options.GetOrDefault<int>("gpus", 2);
    const int first = options.GetOrDefault<int>("first_gpu", 0);
    if (count < 1 || count > 64) throw Exception("b200-multi: gpus must be between 1 and 64");
    std::vector<int> ids;
    for (int i = 0; i < count; ++i) ids.push_back(first + i);
    Check(b200_multi_create(b.get(), &opt, ids.data(), count, &multi_));
    Check(b200_net_get_info(b200_multi_net(multi_, 0), &info_));
    if (!info_.has_mlh) capabilities_.moves_left = pblczero::NetworkFormat::MOVES_LEFT_NONE;
    gpus_ = count;
  }
  ~B200MultiNetwork() override { b200_multi_destroy(multi_); }

  const NetworkCapabilities& GetCapabilities() const override { return capabilities_; }
  std::unique_ptr<NetworkComputation> NewComputation() override {
    return std::make_unique<B200MultiComputation>(multi_, info_.wdl != 0, info_.has_mlh != 0);
  }
  int GetThreads() const override { return 2; }
  bool IsCpu() const override { return false; }
  int GetMiniBatchSize() const override { return 2 * info_.sm_count * gpus_; }
  int GetPreferredBatchStep() const override { return gpus_; }

 private:
  NetworkCapabilities capabilities_;
  b200_multi* multi_ = nullptr;
  b200_net_info info_{};
  int gpus_ = 1;
};

std::unique_ptr<Network> MakeB200MultiNetwork(const std::optional<WeightsFile>& w, const OptionsDict& options) {
  if (!w) throw Exception("The b200-multi backend requires a network file.");
  return std::make_unique<B200MultiNetwork>(*w, options);
}
REGISTER_NETWORK("b200-multi", MakeB200MultiNetwork, 85)


// ---- native Backend ---------------------------------------------------------------------------------------------
// Same contract as NetworkAsBackend (src/neural/wrapper.cc:48-101) with two differences: the batch limit is the
// network's max_batch option instead of the wrapper's fixed 1024, and EvalResultPtr::p is filled from the device's
// legal-move softmax (same FastExp arithmetic and summation order, so the numbers are bit-identical to the wrapper's).

FillEmptyHistory ParseHistoryFill(const std::string& s) {
  if (s == "fen_only") return FillEmptyHistory::FEN_ONLY;
  if (s == "always") return FillEmptyHistory::ALWAYS;
  return FillEmptyHistory::NO;
}

class B200Backend : public Backend {
 public:
  B200Backend(std::unique_ptr<B200Network> network, const OptionsDict& options, bool device_encode)
      : network_(std::move(network)),
        device_encode_(device_encode),
        backend_opts_(options.Get<std::string>(SharedBackendParams::kBackendOptionsId)),
        weights_path_(options.Get<std::string>(SharedBackendParams::kWeightsId)) {
    UpdateConfiguration(options);
  }

  BackendAttributes GetAttributes() const override {
    const NetworkCapabilities& caps = network_->GetCapabilities();
    BackendAttributes a;
    a.has_mlh = caps.has_mlh();
    a.has_wdl = caps.has_wdl();
    a.runs_on_cpu = false;
    a.suggested_num_search_threads = network_->GetThreads();
    a.recommended_batch_size = network_->GetMiniBatchSize();
    a.maximum_batch_size = network_->info().max_batch;
    return a;
  }
  std::unique_ptr<BackendComputation> CreateComputation() override;

  UpdateConfigurationResult UpdateConfiguration(const OptionsDict& options) override {
    Backend::UpdateConfiguration(options);
    if (backend_opts_ != options.Get<std::string>(SharedBackendParams::kBackendOptionsId)) return NEED_RESTART;
    if (weights_path_ != options.Get<std::string>(SharedBackendParams::kWeightsId)) return NEED_RESTART;
    inv_temperature_ = 1.0f / options.Get<float>(SharedBackendParams::kPolicySoftmaxTemp);
    history_fill_ = ParseHistoryFill(options.Get<std::string>(SharedBackendParams::kHistoryFill));
    return UPDATE_OK;
  }

 private:
  friend class B200BackendComputation;
  std::unique_ptr<B200Network> network_;
  const std::string backend_opts_;
  const std::string weights_path_;
  const bool device_encode_;
  float inv_temperature_ = 1.0f;
  FillEmptyHistory history_fill_ = FillEmptyHistory::NO;
};

// One position of the history in the layout of include/b200nn.h.
b200_board ToRecord(const Position& p) {
  const ChessBoard& b = p.GetBoard();
  b200_board r{};
  r.ours = b.ours().as_int();
  r.theirs = b.theirs().as_int();
  r.pawns = b.pawns().as_int();
  r.knights = b.knights().as_int();
  r.bishops = b.bishops().as_int();
  r.rooks = b.rooks().as_int();
  r.queens = b.queens().as_int();
  r.kings = b.kings().as_int();
  r.en_passant = b.en_passant().as_int();
  const auto& c = b.castlings();
  r.castling = c.as_int();
  r.rook_files[0] = c.our_queenside_rook.idx;
  r.rook_files[1] = c.our_kingside_rook.idx;
  r.rook_files[2] = c.their_queenside_rook.idx;
  r.rook_files[3] = c.their_kingside_rook.idx;
  r.flags = (b.flipped() ? 1 : 0) | (b == ChessBoard::kStartposBoard ? 2 : 0);
  r.rule50 = static_cast<uint16_t>(p.GetRule50Ply());
  r.repetitions = static_cast<uint8_t>(p.GetRepetitions());
  return r;
}

class B200BackendComputation : public BackendComputation {
 public:
  explicit B200BackendComputation(B200Backend* backend)
      : backend_(backend),
        input_format_(backend->network_->GetCapabilities().input_format),
        wdl_(backend->network_->info().wdl != 0),
        mlh_(backend->network_->info().has_mlh != 0) {
    Check(b200_comp_create(backend->network_->net(), &comp_));
    Check(b200_comp_set_policy_options(comp_, backend->inv_temperature_, /*compact=*/1));
    Check(b200_comp_set_encoding(comp_, 0, static_cast<int>(backend->history_fill_)));
    results_.reserve(256);
  }
  ~B200BackendComputation() override { b200_comp_destroy(comp_); }

  size_t UsedBatchSize() const override { return results_.size(); }

  AddInputResult AddInput(const EvalPosition& pos, EvalResultPtr result) override {
    uint16_t ids[256];
    int n_moves = 0;
    const bool with_policy = !result.p.empty();
    if (with_policy && (pos.legal_moves.size() > 256 || result.p.size() != pos.legal_moves.size()))
      throw Exception("b200 backend: bad legal-move list");
    if (by_history_allowed_ && AddByHistory(pos, result, with_policy, ids)) return ENQUEUED_FOR_EVAL;
    int transform;
    const InputPlanes planes =
        EncodePositionForNN(input_format_, pos.pos, 8, backend_->history_fill_, &transform);
    uint64_t masks[kInputPlanes];
    float values[kInputPlanes];
    for (int i = 0; i < kInputPlanes; ++i) {
      masks[i] = planes[i].mask;
      values[i] = planes[i].value;
    }
    if (with_policy)
      for (const Move& m : pos.legal_moves) ids[n_moves++] = MoveToNNIndex(m, transform);
    // The search may add inputs to one computation from several threads (the wrapper uses an atomic vector).
    std::lock_guard<std::mutex> lock(mutex_);
    if (by_history_) throw Exception("b200 backend: mixed input kinds in one computation");
    Check(b200_comp_add_input_with_moves(comp_, masks, values, ids, n_moves));
    results_.push_back(result);
    return ENQUEUED_FOR_EVAL;
  }

  // Hands the history to the library instead of the planes.  The transform that maps the legal moves to policy
  // indices is a few bit operations on the last board and stays on the host (TransformForPosition's rule,
  // src/neural/encoder.cc:124-132).  Returns false when the history does not fit (the planes are then encoded here).
  bool AddByHistory(const EvalPosition& pos, EvalResultPtr result, bool with_policy, uint16_t* ids) {
    const auto& h = pos.pos;
    // The encoder looks at most 8 positions back (the two V2 formats, which may walk back to the last irreversible
    // move, keep the host encoder: their histories would not fit the per-computation staging in the worst case).
    const size_t first = h.size() > 8 ? h.size() - 8 : 0;
    const size_t count = h.size() - first;
    if (count > B200_MAX_HISTORY) return false;
    b200_board records[B200_MAX_HISTORY];
    for (size_t i = 0; i < count; ++i) records[i] = ToRecord(h[first + i]);
    int n_moves = -1;
    if (with_policy) {
      const int transform = IsCanonicalFormat(input_format_) ? TransformOf(h.back().GetBoard()) : 0;
      n_moves = 0;
      for (const Move& m : pos.legal_moves) ids[n_moves++] = MoveToNNIndex(m, transform);
    }
    std::lock_guard<std::mutex> lock(mutex_);
    if (!results_.empty() && !by_history_) return false;
    const int rc = b200_comp_add_position(comp_, records, static_cast<int>(count), first == 0 ? 1 : 0, ids,
                                          with_policy ? n_moves : 0);
    if (rc != B200_OK) {
      if (results_.empty()) return false;  // e.g. staging capacity: fall back before anything was added this way
      Check(rc);
    }
    by_history_ = true;
    results_.push_back(result);
    return true;
  }

  // ChooseTransform needs a PositionHistory in the reference's public API; EncodePositionForNN on the last position
  // alone returns the same transform (it only looks at that board).
  static int TransformOf(const ChessBoard& board) {
    PositionHistory one;
    one.Reset(board, 0, 1);
    return TransformForPosition(pblczero::NetworkFormat::INPUT_112_WITH_CANONICALIZATION, one);
  }

  void ComputeBlocking() override {
    if (results_.empty()) return;
    Check(b200_comp_compute(comp_));
    for (size_t i = 0; i < results_.size(); ++i) {
      const EvalResultPtr& r = results_[i];
      if (r.q) *r.q = b200_comp_q(comp_, i);
      if (r.d) *r.d = wdl_ ? b200_comp_d(comp_, i) : 0.0f;
      if (r.m) *r.m = mlh_ ? b200_comp_m(comp_, i) : 0.0f;
      if (!r.p.empty()) {
        const float* probs = nullptr;
        int n = 0;
        Check(b200_comp_legal_policy(comp_, i, &probs, &n));
        std::copy(probs, probs + n, r.p.begin());
      }
    }
  }

 private:
  B200Backend* backend_;
  pblczero::NetworkFormat::InputFormat input_format_;
  bool wdl_, mlh_;
  b200_comp* comp_ = nullptr;
  std::mutex mutex_;
  std::vector<EvalResultPtr> results_;
  bool by_history_ = false;
  const bool by_history_allowed_ =
      backend_->device_encode_ && input_format_ != pblczero::NetworkFormat::INPUT_112_WITH_CANONICALIZATION_V2 &&
      input_format_ != pblczero::NetworkFormat::INPUT_112_WITH_CANONICALIZATION_V2_ARMAGEDDON;
};

std::unique_ptr<BackendComputation> B200Backend::CreateComputation() {
  return std::make_unique<B200BackendComputation>(this);
}

class B200BackendFactory : public BackendFactory {
 public:
  int GetPriority() const override { return 87; }
  std::string_view GetName() const override { return "b200-native"; }
  // Option handling as in NetworkAsBackendFactory::Create (src/neural/wrapper.cc:182-198); precision=<fp16|bf16|fp32>.
  std::unique_ptr<Backend> Create(const OptionsDict& options) override {
    OptionsDict network_options;
    network_options.AddSubdictFromString(options.Get<std::string>(SharedBackendParams::kBackendOptionsId));
    const std::optional<WeightsFile> weights = LoadWeights(options.Get<std::string>(SharedBackendParams::kWeightsId));
    if (!weights) throw Exception("The b200 backend requires a network file.");
    const std::string prec = network_options.GetOrDefault<std::string>("precision", "fp16");
    int precision;
    if (prec == "fp16") precision = B200_PREC_FP16;
    else if (prec == "bf16") precision = B200_PREC_BF16;
    else if (prec == "fp32") precision = B200_PREC_FP32;
    else throw Exception("b200 backend: unknown precision '" + prec + "'");
    const bool device_encode = network_options.GetOrDefault<bool>("device_encode", true);
    auto network = std::make_unique<B200Network>(*weights, network_options, precision);
    network_options.CheckAllOptionsRead("b200-native");
    return std::make_unique<B200Backend>(std::move(network), options, device_encode);
  }
};

[[maybe_unused]] static BackendManager::Register reg_b200_native(std::make_unique<B200BackendFactory>());

}  // namespace
}  // namespace lczero
