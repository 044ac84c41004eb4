// Host side of the backend: network construction from named tensors, the evaluation schedule
// (which kernel runs on which buffer), computation objects, and the C ABI of include/b200nn.h.
//
// The schedule restates BlasComputation::ComputeBlocking / ForwardEncoderLayer
// (src/neural/backends/blas/network_blas.cc:271-971) as a sequence of CUDA kernel launches on one stream
// per workspace slot.  Activations are token-major ([position*64 + square][channels]) for both attention
// and residual bodies, so every dense layer and every 1x1 convolution is a plain row-major GEMM.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/b200nn.h"
#include "kernels.cuh"

namespace b200 {

static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }
int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  set_error(std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what + " (" + file + ":" +
            std::to_string(line) + ")");
  return B200_ERR_CUDA;
}

struct Fail {
  int code;
  std::string msg;
};
#define CK(call)                                                                   \
  do {                                                                             \
    cudaError_t e__ = (call);                                                      \
    if (e__ != cudaSuccess)                                                        \
      throw Fail{B200_ERR_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e__) + " in " #call + \
                                    " (" __FILE__ ":" + std::to_string(__LINE__) + ")"};            \
  } while (0)

// NetworkFormat enum values (proto/net.proto:275-367).
enum { NET_CLASSICAL_HF = 3, NET_SE_HF = 4, NET_ATTN_HF = 6, NET_ATTN_MHF = 7 };
enum { POLICY_CLASSICAL = 1, POLICY_CONVOLUTION = 2, POLICY_ATTENTION = 3 };
enum { VALUE_CLASSICAL = 1, VALUE_WDL = 2 };
enum { EMB_NONE = 0, EMB_PE_MAP = 1, EMB_PE_DENSE = 2 };

// ---- policy tables, generated from chess geometry (reference arrays: neural/encoder.cc:339,
// neural/tables/attention_policy_map.h:24 and :386, neural/tables/policy_map.h:24) ----------------
struct Tables {
  std::vector<short> attn_src;   // [1858] slot in the 64*64 + 8*24 attention-policy vector
  std::vector<short> conv_src;   // [1858] plane*64 + square of the convolutional policy output
  std::vector<float> pos_enc;    // [64][64]
};
static bool reachable(int a, int b) {
  if (a == b) return false;
  const int dx = b % 8 - a % 8, dy = b / 8 - a / 8;
  if (dx == 0 || dy == 0 || std::abs(dx) == std::abs(dy)) return true;
  return (std::abs(dx) == 1 && std::abs(dy) == 2) || (std::abs(dx) == 2 && std::abs(dy) == 1);
}
static const Tables& tables() {
  static const Tables t = [] {
    Tables t;
    // Policy index of a plain move from a to b, and of promotion (file f -> file g, piece i in q,r,b).
    std::vector<int> plain(64 * 64, -1);
    int idx = 0;
    for (int a = 0; a < 64; ++a)
      for (int b = 0; b < 64; ++b)
        if (reachable(a, b)) plain[a * 64 + b] = idx++;
    int promo[8][8][3];
    for (int f = 0; f < 8; ++f)
      for (int g = 0; g < 8; ++g)
        for (int i = 0; i < 3; ++i) promo[f][g][i] = -1;
    for (int f = 0; f < 8; ++f)
      for (int g = f - 1; g <= f + 1; ++g)
        if (g >= 0 && g < 8)
          for (int i = 0; i < 3; ++i) promo[f][g][i] = idx++;
    t.attn_src.assign(1858, 0);
    for (int a = 0; a < 64; ++a)
      for (int b = 0; b < 64; ++b)
        if (plain[a * 64 + b] >= 0) t.attn_src[plain[a * 64 + b]] = short(a * 64 + b);
    for (int f = 0; f < 8; ++f)
      for (int g = 0; g < 8; ++g)
        for (int i = 0; i < 3; ++i)
          if (promo[f][g][i] >= 0) t.attn_src[promo[f][g][i]] = short(4096 + 24 * f + 3 * g + i);
    // Convolutional policy planes: 8 directions x 7 distances, 8 knight jumps, 3 directions x (r, b, q).
    static const int qd[8][2] = {{0, 1}, {1, 1}, {1, 0}, {1, -1}, {0, -1}, {-1, -1}, {-1, 0}, {-1, 1}};
    static const int kn[8][2] = {{1, 2}, {2, 1}, {2, -1}, {1, -2}, {-1, -2}, {-2, -1}, {-2, 1}, {-1, 2}};
    t.conv_src.assign(1858, 0);
    for (int sq = 0; sq < 64; ++sq) {
      const int x = sq % 8, y = sq / 8;
      for (int d = 0; d < 8; ++d)
        for (int dist = 1; dist < 8; ++dist) {
          const int tx = x + qd[d][0] * dist, ty = y + qd[d][1] * dist;
          if (tx >= 0 && tx < 8 && ty >= 0 && ty < 8)
            t.conv_src[plain[sq * 64 + ty * 8 + tx]] = short((d * 7 + dist - 1) * 64 + sq);
        }
      for (int k = 0; k < 8; ++k) {
        const int tx = x + kn[k][0], ty = y + kn[k][1];
        if (tx >= 0 && tx < 8 && ty >= 0 && ty < 8)
          t.conv_src[plain[sq * 64 + ty * 8 + tx]] = short((56 + k) * 64 + sq);
      }
      if (y == 6)
        for (int d = 0; d < 3; ++d) {
          const int tx = x + d - 1;
          if (tx < 0 || tx >= 8) continue;
          static const int piece_of_plane[3] = {1, 2, 0};  // planes are ordered r, b, q; indices q, r, b
          for (int i = 0; i < 3; ++i)
            t.conv_src[promo[x][tx][piece_of_plane[i]]] = short((64 + 3 * d + i) * 64 + sq);
        }
    }
    t.pos_enc.assign(64 * 64, 0.f);
    for (int a = 0; a < 64; ++a)
      for (int b = 0; b < 64; ++b) t.pos_enc[a * 64 + b] = a == b ? -1.f : (reachable(a, b) ? 1.f : 0.f);
    return t;
  }();
  return t;
}

// Host copy of the attention-policy gather table (1858 slots), shared with other translation units.
const short* attn_policy_src_table() { return tables().attn_src.data(); }

}  // namespace b200

using namespace b200;

struct b200_builder {
  std::map<std::string, std::vector<float>> tensors;
  std::map<std::string, long long> ints;
};

namespace b200 {

// ---- device memory bookkeeping --------------------------------------------------------------------
struct DeviceAllocs {
  std::vector<void*> ptrs;
  long long bytes = 0;
  void* alloc(size_t n) {
    void* p = nullptr;
    if (n == 0) n = 16;
    CK(cudaMalloc(&p, n));
    ptrs.push_back(p);
    bytes += (long long)n;
    return p;
  }
  void release() {
    for (void* p : ptrs) cudaFree(p);
    ptrs.clear();
  }
};

template <typename T> static T host_cast(float v);
template <> float host_cast<float>(float v) { return v; }
template <> __half host_cast<__half>(float v) {
  return __float2half_rn(std::min(std::max(v, -65504.f), 65504.f));
}
template <> __nv_bfloat16 host_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> struct Dense {
  T* w = nullptr;        // [out][in]
  float* b = nullptr;    // [out] or nullptr
  int out = 0, in = 0;
  // Set when the LayerNorm that feeds this layer is folded into it: w holds W * gamma (per input column),
  // b holds b + beta . W^T, and colsum[n] = sum_k (W * gamma)[n][k] of the stored (rounded) weights.
  float* colsum = nullptr;
};

template <typename T> struct EncoderW {
  Dense<T> qkv, proj, ffn1, ffn2;
  float *ln1g = nullptr, *ln1b = nullptr, *ln2g = nullptr, *ln2b = nullptr;
  bool smolgen = false;
  Dense<T> sg_compress, sg_d1, sg_d2;
  int qkvc_out = 0;  // > 0: qkv.w holds this many rows, the smolgen compression's appended to Q, K, V's
  float *sg_ln1g = nullptr, *sg_ln1b = nullptr, *sg_ln2g = nullptr, *sg_ln2b = nullptr;
};

template <typename T> struct ConvW {
  T* w = nullptr;  // [9][Cout][Cin]
  T* u = nullptr;  // [36][Cout][Cin]: Winograd-transformed filters (only with the winograd option)
  float* b = nullptr;
  int cout = 0, cin = 0;
};

template <typename T> struct ResidualW {
  ConvW<T> c1, c2;
  bool se = false;
  float *se_w1 = nullptr, *se_b1 = nullptr, *se_w2 = nullptr, *se_b2 = nullptr;
  int se_k = 0;
};

struct NetBase {
  virtual ~NetBase() {}
  b200_net_info info{};
  b200_net_options opt{};
  std::atomic<long long> launches{0};
  // Optional per-kernel-class timing with CUDA events on the evaluation stream.
  enum { K_GEMM_TC = 0, K_GEMM_FMA = 1, K_ATTENTION = 2, K_LAYERNORM = 3, K_OTHER = 4, K_CLASSES = 5 };
  std::atomic<bool> profiling{false};
  // `tag` names the launch within its class (the products of an encoder layer: see b200_net_get_profile_tagged)
  struct Span { int cls, tag; cudaEvent_t a, b; double work; };
  std::mutex prof_mu;  // computations of several slots may record spans at the same time
  std::vector<Span> spans;
  std::vector<cudaEvent_t> event_pool;
  double prof_ms[K_CLASSES] = {0}, prof_work[K_CLASSES] = {0};
  long long prof_launches[K_CLASSES] = {0};
  enum { K_TAGS = 16 };
  // Tags: which product of an encoder layer (or which other part of the evaluation) a tensor-core launch belongs to.
  enum { TAG_NONE = 0, TAG_QKV = 1, TAG_OUT_PROJ = 2, TAG_FFN1 = 3, TAG_FFN2 = 4, TAG_SMOLGEN_DENSE = 5,
         TAG_SMOLGEN_BIAS = 6, TAG_ATTENTION = 7, TAG_EMBEDDING = 8, TAG_HEADS = 9 };
  double tag_ms[K_TAGS] = {0}, tag_work[K_TAGS] = {0};
  long long tag_launches[K_TAGS] = {0};
  cudaEvent_t get_event() {  // prof_mu held
    if (!event_pool.empty()) {
      cudaEvent_t e = event_pool.back();
      event_pool.pop_back();
      return e;
    }
    cudaEvent_t e;
    cudaEventCreate(&e);
    return e;
  }
  // Brackets one launch: begin() before, end(index begin() returned) after (no-ops unless profiling is on).
  int span_begin(cudaStream_t st, int cls, double work, int tag = 0) {
    if (!profiling) return -1;
    std::lock_guard<std::mutex> l(prof_mu);
    Span sp{cls, tag, get_event(), get_event(), work};
    cudaEventRecord(sp.a, st);
    spans.push_back(sp);
    return (int)spans.size() - 1;
  }
  void span_end(cudaStream_t st, int idx) {
    if (idx < 0) return;
    std::lock_guard<std::mutex> l(prof_mu);
    if (idx < (int)spans.size()) cudaEventRecord(spans[idx].b, st);
  }
  void collect_spans() {
    std::lock_guard<std::mutex> l(prof_mu);
    for (auto& sp : spans) {
      float ms = 0.f;
      if (cudaEventSynchronize(sp.b) == cudaSuccess && cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
        prof_ms[sp.cls] += ms;
        prof_work[sp.cls] += sp.work;
        prof_launches[sp.cls]++;
        if (sp.tag > 0 && sp.tag < K_TAGS) {
          tag_ms[sp.tag] += ms;
          tag_work[sp.tag] += sp.work;
          tag_launches[sp.tag]++;
        }
      }
      event_pool.push_back(sp.a);
      event_pool.push_back(sp.b);
    }
    spans.clear();
  }
  virtual int eval_device(int slot, const void* d_masks, const void* d_values, int n, void* d_policy,
                          void* d_qdm, bool sync) = 0;
  // Pinned host staging of one computation: inputs are written here by AddInput, results are read from here,
  // so a computation costs no host-side copies beyond the caller's own (the reference pools its InputsOutputs
  // the same way, backends/cuda/network_cuda.cc:1066-1083).
  struct HostSet {
    uint64_t* masks = nullptr;
    float *values = nullptr, *policy = nullptr, *qdm = nullptr;
    // legal-move policy: per position up to kLegalStride policy indices in, probabilities out
    unsigned short* move_ids = nullptr;
    int* n_moves = nullptr;
    float* probs = nullptr;
    // device-side position encoding: the histories of the positions (allocated at the first b200_comp_add_position)
    b200_board* boards = nullptr;
    int* offsets = nullptr;
    uint8_t* from_start = nullptr;
    int id = 0;
  };
  // Board records a computation may stage: an average of kBoardsPerPosition per position of the largest batch.
  static constexpr int kBoardsPerPosition = 16;
  size_t board_capacity() const { return (size_t)opt.max_batch * kBoardsPerPosition; }
  void ensure_board_staging(HostSet& h) {
    if (h.boards) return;
    const size_t nb = (size_t)opt.max_batch;
    if (cudaSetDevice(opt.gpu) != cudaSuccess ||
        cudaMallocHost(&h.boards, board_capacity() * sizeof(b200_board)) != cudaSuccess ||
        cudaMallocHost(&h.offsets, (nb + 1) * sizeof(int)) != cudaSuccess ||
        cudaMallocHost(&h.from_start, nb) != cudaSuccess) {
      if (h.boards) cudaFreeHost(h.boards);
      if (h.offsets) cudaFreeHost(h.offsets);
      h.boards = nullptr;
      h.offsets = nullptr;
      cudaGetLastError();
      throw Fail{B200_ERR_NOMEM, "cannot allocate pinned host staging for position histories"};
    }
    h.offsets[0] = 0;
  }
  std::mutex host_mu;
  std::vector<HostSet*> host_free, host_all;
  HostSet* acquire_host() {
    {
      std::lock_guard<std::mutex> l(host_mu);
      if (!host_free.empty()) {
        HostSet* h = host_free.back();
        host_free.pop_back();
        return h;
      }
    }
    const size_t nb = (size_t)opt.max_batch;
    auto h = std::make_unique<HostSet>();
    if (cudaSetDevice(opt.gpu) != cudaSuccess || cudaMallocHost(&h->masks, nb * 112 * 8) != cudaSuccess ||
        cudaMallocHost(&h->values, nb * 112 * 4) != cudaSuccess ||
        cudaMallocHost(&h->policy, nb * 1858 * 4) != cudaSuccess || cudaMallocHost(&h->qdm, nb * 3 * 4) != cudaSuccess ||
        cudaMallocHost(&h->move_ids, nb * kLegalStride * 2) != cudaSuccess ||
        cudaMallocHost(&h->n_moves, nb * 4) != cudaSuccess ||
        cudaMallocHost(&h->probs, nb * kLegalStride * 4) != cudaSuccess) {
      if (h->masks) cudaFreeHost(h->masks);
      if (h->values) cudaFreeHost(h->values);
      if (h->policy) cudaFreeHost(h->policy);
      if (h->qdm) cudaFreeHost(h->qdm);
      if (h->move_ids) cudaFreeHost(h->move_ids);
      if (h->n_moves) cudaFreeHost(h->n_moves);
      cudaGetLastError();
      throw Fail{B200_ERR_NOMEM, "cannot allocate pinned host staging for a computation"};
    }
    std::lock_guard<std::mutex> l(host_mu);
    h->id = (int)host_all.size() + 1;
    host_all.push_back(h.get());
    return h.release();
  }
  void release_host(HostSet* h) {
    std::lock_guard<std::mutex> l(host_mu);
    host_free.push_back(h);
  }
  void free_host_sets() {
    for (HostSet* h : host_all) {
      cudaFreeHost(h->masks);
      cudaFreeHost(h->values);
      cudaFreeHost(h->policy);
      cudaFreeHost(h->qdm);
      cudaFreeHost(h->move_ids);
      cudaFreeHost(h->n_moves);
      cudaFreeHost(h->probs);
      if (h->boards) cudaFreeHost(h->boards);
      if (h->offsets) cudaFreeHost(h->offsets);
      if (h->from_start) cudaFreeHost(h->from_start);
      delete h;
    }
    host_all.clear();
    host_free.clear();
  }
  // policy_mode: 0 full 1858-logit policy, 1 full policy + legal-move probabilities, 2 legal-move probabilities
  // only (the 1858-logit vectors stay on the device).
  // enc_format > 0: the planes are produced on the device from hs.boards (n_boards records) in that input format
  virtual int eval_staged(int slot, HostSet& hs, int n, int policy_mode, float inv_temperature, int enc_format = 0,
                          int enc_fill = 0, int n_boards = 0) = 0;
  virtual cudaStream_t stream(int slot) = 0;
  virtual int device_status() = 0;
  virtual int sync_slot(int slot) = 0;
  virtual void inject_status(int code) = 0;
  // slot pool
  std::mutex mu;
  std::condition_variable cv;
  std::vector<int> free_slots;
  int acquire() {
    std::unique_lock<std::mutex> l(mu);
    cv.wait(l, [&] { return !free_slots.empty(); });
    int s = free_slots.back();
    free_slots.pop_back();
    return s;
  }
  void release(int s) {
    {
      std::lock_guard<std::mutex> l(mu);
      free_slots.push_back(s);
    }
    cv.notify_all();
  }
  // The device-pointer entry points (b200_net_eval_device / _enqueue_device) run on slot 0, whose stream
  // b200_net_stream exposes.  They take that slot out of the pool like a computation does; the enqueue form keeps it
  // until b200_net_sync, so that a computation of another thread never shares the workspace of work still in flight.
  bool dev_holds_slot0 = false;  // guarded by mu
  void hold_slot0() {
    std::unique_lock<std::mutex> l(mu);
    if (dev_holds_slot0) return;
    cv.wait(l, [&] { return std::find(free_slots.begin(), free_slots.end(), 0) != free_slots.end(); });
    free_slots.erase(std::find(free_slots.begin(), free_slots.end(), 0));
    dev_holds_slot0 = true;
  }
  void unhold_slot0() {
    {
      std::lock_guard<std::mutex> l(mu);
      if (!dev_holds_slot0) return;
      dev_holds_slot0 = false;
      free_slots.push_back(0);
    }
    cv.notify_all();
  }
};

template <typename T>
struct Net : NetBase {
  DeviceAllocs walloc, salloc;
  int sm_count = 148;
  bool use_tc = false;
  // LayerNorms of the encoder stack folded into the neighbouring tensor-core products (16-bit storage only).
  bool fold_ln = false;
  bool fold_emb_ln = false;  // the embedding block's last LayerNorm is folded into the first encoder layer
  bool merge_compress = true;  // false (B200_FLAG_NO_MERGED_COMPRESS): smolgen compression as a launch of its own
  bool fold_heads = false;  // the heads' first products fold the last LayerNorm too (else it is materialised)
  bool winograd = false;    // 3x3 convolutions as Winograd F(4x4, 3x3) transforms around 36 stacked products
  int* d_status = nullptr;  // one status word per slot
  // Status word of the evaluation being enqueued on this thread (the slot's), handed to every kernel with bounded waits.
  static inline thread_local int* t_status = nullptr;
  static inline thread_local void* t_slot_ptr = nullptr;  // the slot of that evaluation
  // > 0: the tensor-core launches that follow on this thread use at most this many SMs (persistent grids are sized
  // from it), so that two launches on different streams can share the GPU
  static inline thread_local int t_sm_limit = 0;
  struct DependentLaunchScope {
    bool prev;
    explicit DependentLaunchScope(bool on) : prev(t_dependent_launch) { t_dependent_launch = on; }
    ~DependentLaunchScope() { t_dependent_launch = prev; }
  };
  // smolgen's two small dense layers and their LayerNorms run on a second stream on kSideSms SMs while the QKV product
  // has the rest of the GPU: they are launch- and latency-bound (a quarter of a layer's time at batch 256), not
  // throughput-bound
  bool side_stream = false;
  bool dependent_launch = false;  // tensor-core products, attention and LayerNorms launched with launch_dependent()
  bool heads_side = false;        // value and moves-left heads on the side stream beside the policy head
  int heads_side_max = 0;         // ... up to this many positions
  bool tower = false;             // residual towers: all 3x3 convolutions in one launch up to tower_max_batch positions
  int tower_max_batch = 0;
  static constexpr int kSideSms = 8;

  // format
  int network = 0, policy_fmt = 0, value_fmt = 0, emb_fmt = 0;
  int act_default = ACT_RELU, act_smolgen = ACT_SWISH, act_ffn = ACT_RELU_2;
  bool attn_body = false, wdl = false, mlh = false;

  // attention body
  int E = 0, H = 0, cin = 0, pe_ch = 0, layers = 0, emb_dff = 0, max_dff = 0;
  int sg_hc = 0, sg_hid = 0, sg_gen = 0;  // sg_gen = heads * per-head generator width
  float alpha = 1.f, ln_eps = 1e-6f;
  Dense<T> emb_pre, emb, emb_ffn1, emb_ffn2, smolgen_w;
  float *emb_lng = nullptr, *emb_lnb = nullptr, *emb_ffn_lng = nullptr, *emb_ffn_lnb = nullptr;
  float *gate_mult = nullptr, *gate_add = nullptr, *pos_enc = nullptr;
  std::vector<EncoderW<T>> enc;

  // residual body
  int C = 0;
  ConvW<T> conv_in;
  std::vector<ResidualW<T>> res;

  // heads
  Dense<T> pol_emb, pol_q, pol_k, pol_fc;  // attention policy (emb, wq, wk) / classical FC
  std::vector<EncoderW<T>> pol_enc;        // encoder layers of the attention policy head
  int pol_heads = 0;
  float* pol_w4 = nullptr;
  int pol_dm = 0;
  ConvW<T> pol_conv1, pol_conv2;
  Dense<T> pol_c1x1;
  short *d_attn_src = nullptr, *d_conv_src = nullptr;
  int pol_planes = 0;
  Dense<T> val_emb, val_fc1, mov_emb, mov_fc1;
  float *val_w2 = nullptr, *val_b2 = nullptr, *mov_w2 = nullptr, *mov_b2 = nullptr;

  struct Slot {
    cudaStream_t stream = nullptr;
    cudaStream_t stream2 = nullptr;      // side stream of the smolgen dense layers
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaEvent_t compute_done = nullptr;  // recorded after the last kernel of an evaluation, before its result copies
    int* h_status = nullptr;             // pinned copy of the device status word, refreshed by every evaluation
    uint64_t* d_masks = nullptr;
    float *d_values = nullptr, *d_policy = nullptr, *d_qdm = nullptr;
    void* tower_layers = nullptr;  // device table of the tower kernel (one entry per convolution), or null
    int tower_n = 0;
    unsigned short* d_move_ids = nullptr;
    int* d_n_moves = nullptr;
    float* d_probs = nullptr;
    b200_board* d_boards = nullptr;  // histories for the device-side position encoding
    int* d_offsets = nullptr;
    uint8_t* d_from_start = nullptr;
    T *tokens = nullptr, *pre = nullptr, *pe = nullptr;
    T *x = nullptr, *x1 = nullptr, *y = nullptr, *qkv = nullptr, *att = nullptr, *ffn = nullptr;
    T *sg_c = nullptr, *sg_h1 = nullptr, *sg_h2 = nullptr, *sg_bias = nullptr;
    T *wino_v = nullptr, *wino_m = nullptr;  // [36][rows_padded][channels]: transformed input / product output
    // per-row (sum, sum of squares; double) of the folded LayerNorm inputs, laid out [stats2[0] | stats1 | stats2[1]] so that
    // one memset at the start of a layer clears stats1 and the stats2 buffer that layer writes (layers alternate)
    double *stats1 = nullptr, *stats2[2] = {nullptr, nullptr};
    int stats_parity = 0;
    size_t stats_stride = 0;  // floats between consecutive buffers of that block
    T *pemb = nullptr, *pq = nullptr, *pk = nullptr, *praw = nullptr;
    T *p_qkv = nullptr, *p_att = nullptr, *p_ffn = nullptr, *p_x1 = nullptr, *p_y = nullptr;  // policy-head encoders
    float* logits = nullptr;
    T *vtok = nullptr, *vhid = nullptr, *mtok = nullptr, *mhid = nullptr;
  };
  std::vector<Slot> slots;

  ~Net() override {
    for (auto& cache : graph_cache)
      for (auto& kv : cache)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    for (auto& s : slots) {
      if (s.stream) cudaStreamDestroy(s.stream);
      if (s.stream2) cudaStreamDestroy(s.stream2);
      if (s.ev_fork) cudaEventDestroy(s.ev_fork);
      if (s.ev_join) cudaEventDestroy(s.ev_join);
      if (s.compute_done) cudaEventDestroy(s.compute_done);
      if (s.h_status) cudaFreeHost(s.h_status);
    }
    free_host_sets();
    walloc.release();
    salloc.release();
  }

  // ---- weight upload helpers ----
  const b200_builder* bld = nullptr;
  const std::vector<float>* find(const std::string& name) const {
    auto it = bld->tensors.find(name);
    return it == bld->tensors.end() ? nullptr : &it->second;
  }
  const std::vector<float>& need(const std::string& name, size_t count = 0) const {
    const std::vector<float>* v = find(name);
    if (!v || v->empty()) throw Fail{B200_ERR_INVALID, "weights: missing tensor '" + name + "'"};
    if (count && v->size() != count)
      throw Fail{B200_ERR_INVALID, "weights: tensor '" + name + "' has " + std::to_string(v->size()) +
                                       " values, expected " + std::to_string(count)};
    return *v;
  }
  size_t size_of(const std::string& name) const {
    const std::vector<float>* v = find(name);
    return v ? v->size() : 0;
  }
  float* up_f32(const std::vector<float>& v) {
    float* d = (float*)walloc.alloc(v.size() * sizeof(float));
    CK(cudaMemcpy(d, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice));
    return d;
  }
  float* up_f32(const std::string& name, size_t count) { return up_f32(need(name, count)); }
  T* up_T(const std::vector<float>& v) {
    std::vector<T> h(v.size());
    for (size_t i = 0; i < v.size(); ++i) h[i] = host_cast<T>(v[i]);
    T* d = (T*)walloc.alloc(h.size() * sizeof(T));
    CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
  }
  Dense<T> dense(const std::string& wname, const std::string& bname, int out, int in) {
    Dense<T> d;
    d.out = out;
    d.in = in;
    d.w = up_T(need(wname, (size_t)out * in));
    if (!bname.empty()) d.b = up_f32(bname, out);
    return d;
  }
  // Dense layer whose input LayerNorm (gamma, beta) is folded into the weights (see Dense::colsum).
  Dense<T> dense_folded(const std::vector<float>& w, const std::vector<float>* b, int out, int in,
                        const std::vector<float>& gamma, const std::vector<float>& beta) {
    if (w.size() != (size_t)out * in || gamma.size() != (size_t)in || beta.size() != (size_t)in)
      throw Fail{B200_ERR_INVALID, "weights: size mismatch while folding a LayerNorm"};
    std::vector<T> wt((size_t)out * in);
    std::vector<float> cs(out), bias(out);
    for (int o = 0; o < out; ++o) {
      double sum = 0.0, bsum = b ? (double)(*b)[o] : 0.0;
      for (int k = 0; k < in; ++k) {
        const float orig = w[(size_t)o * in + k];
        const T q = host_cast<T>(orig * gamma[k]);
        wt[(size_t)o * in + k] = q;
        sum += (double)static_cast<float>(q);
        bsum += (double)beta[k] * orig;
      }
      cs[o] = (float)sum;
      bias[o] = (float)bsum;
    }
    Dense<T> d;
    d.out = out;
    d.in = in;
    d.w = (T*)walloc.alloc(wt.size() * sizeof(T));
    CK(cudaMemcpy(d.w, wt.data(), wt.size() * sizeof(T), cudaMemcpyHostToDevice));
    d.b = up_f32(bias);
    d.colsum = up_f32(cs);
    return d;
  }
  Dense<T> dense_maybe_folded(const std::string& wname, const std::string& bname, int out, int in,
                              const std::vector<float>* gamma, const std::vector<float>* beta) {
    if (!gamma) return dense(wname, bname, out, in);
    return dense_folded(need(wname, (size_t)out * in), bname.empty() ? nullptr : &need(bname, out), out, in, *gamma,
                        *beta);
  }
  // FC that consumes a channel-major flatten [c*64 + sq] in the file; our activations are square-major.
  Dense<T> dense_chw(const std::string& wname, const std::string& bname, int out, int planes) {
    const std::vector<float>& w = need(wname, (size_t)out * planes * 64);
    std::vector<float> p(w.size());
    for (int o = 0; o < out; ++o)
      for (int c = 0; c < planes; ++c)
        for (int sq = 0; sq < 64; ++sq)
          p[(size_t)o * planes * 64 + sq * planes + c] = w[(size_t)o * planes * 64 + c * 64 + sq];
    Dense<T> d;
    d.out = out;
    d.in = planes * 64;
    d.w = up_T(p);
    if (!bname.empty()) d.b = up_f32(bname, out);
    return d;
  }
  ConvW<T> conv3(const std::string& prefix, int cout, int cin_) {
    const std::vector<float>& w = need(prefix + ".weights", (size_t)cout * cin_ * 9);
    std::vector<float> p(w.size());
    for (int o = 0; o < cout; ++o)
      for (int c = 0; c < cin_; ++c)
        for (int t = 0; t < 9; ++t) p[((size_t)t * cout + o) * cin_ + c] = w[((size_t)o * cin_ + c) * 9 + t];
    ConvW<T> cw;
    cw.cout = cout;
    cw.cin = cin_;
    cw.w = up_T(p);
    if (winograd) {
      std::vector<float> u((size_t)36 * cout * cin_);
      wino_transform_filters(w.data(), cout, cin_, u.data());
      cw.u = up_T(u);
    }
    cw.b = up_f32(prefix + ".biases", cout);
    return cw;
  }
  Dense<T> conv1(const std::string& prefix, int cout, int cin_) {
    return dense(prefix + ".weights", prefix + ".biases", cout, cin_);
  }
  void add_flops(double rows_per_pos, const Dense<T>& d, bool encoder_gemm = false) {
    const double f = 2.0 * rows_per_pos * d.out * d.in;
    info.flops_per_position += f;
    if (encoder_gemm) info.gemm_flops_per_position += f;
  }

  // LayerNorm parameters folded into the heads' first products: the last encoder layer's second LayerNorm.
  const std::vector<float>* head_gamma() const {
    return (fold_heads && layers > 0) ? &need("encoder." + std::to_string(layers - 1) + ".ln2_gammas", E) : nullptr;
  }
  const std::vector<float>* head_beta() const {
    return (fold_heads && layers > 0) ? &need("encoder." + std::to_string(layers - 1) + ".ln2_betas", E) : nullptr;
  }
  long long geti(const std::string& k, long long def = 0) const {
    auto it = bld->ints.find(k);
    return it == bld->ints.end() ? def : it->second;
  }

  // in_gamma / in_beta: parameters of the LayerNorm whose output feeds this layer when that LayerNorm is folded
  // into the consuming products (nullptr: the layer input is a materialised activation).
  // body = false: a policy-head encoder layer (no folding, no smolgen, not counted among the encoder products)
  EncoderW<T> load_encoder(const std::string& p, int emb, int heads, const std::vector<float>* in_gamma,
                           const std::vector<float>* in_beta, bool body = true) {
    const bool fold_ffn1 = fold_ln && body;
    EncoderW<T> e;
    const int dm = (int)size_of(p + ".mha.q_b");
    if (dm <= 0 || dm % heads) throw Fail{B200_ERR_INVALID, "weights: bad attention width in " + p};
    if (dm != emb) throw Fail{B200_ERR_UNSUPPORTED, "attention width different from the embedding is not supported"};
    std::vector<float> w, b;
    for (const char* n : {"q", "k", "v"}) {
      const auto& ww = need(p + ".mha." + n + "_w", (size_t)dm * emb);
      const auto& bb = need(p + ".mha." + n + "_b", dm);
      w.insert(w.end(), ww.begin(), ww.end());
      b.insert(b.end(), bb.begin(), bb.end());
    }
    // The smolgen compression reads the same layer input as Q, K, V: its rows are appended to theirs so that one
    // launch of the CTA-pair kernel can compute both (second output, narrow last tile); sg_compress below is a view
    // of those rows for the cases that run it as a product of its own.
    const size_t cw_size = size_of(p + ".mha.smolgen.compress");
    const int hc_rows = cw_size ? (int)(cw_size / emb) : 0;
    const bool merge = hc_rows > 0 && sizeof(T) == 2 && use_tc && (3 * dm) % 256 == 0 && hc_rows <= 256 && hc_rows % 8 == 0;
    if (merge) {
      const auto& cw = need(p + ".mha.smolgen.compress", (size_t)hc_rows * emb);
      w.insert(w.end(), cw.begin(), cw.end());
      b.resize((size_t)3 * dm + hc_rows, 0.f);
    }
    const int qkv_rows = 3 * dm + (merge ? hc_rows : 0);
    if (in_gamma) {
      e.qkv = dense_folded(w, &b, qkv_rows, emb, *in_gamma, *in_beta);
    } else {
      e.qkv.in = emb;
      e.qkv.w = up_T(w);
      e.qkv.b = up_f32(b);
    }
    e.qkv.out = 3 * dm;
    if (merge) e.qkvc_out = qkv_rows;
    e.proj = dense(p + ".mha.dense_w", p + ".mha.dense_b", emb, dm);
    const int dff = (int)size_of(p + ".ffn.dense1_b");
    if (fold_ffn1)
      e.ffn1 = dense_folded(need(p + ".ffn.dense1_w", (size_t)dff * emb), &need(p + ".ffn.dense1_b", dff), dff, emb,
                            need(p + ".ln1_gammas", emb), need(p + ".ln1_betas", emb));
    else
      e.ffn1 = dense(p + ".ffn.dense1_w", p + ".ffn.dense1_b", dff, emb);
    e.ffn2 = dense(p + ".ffn.dense2_w", p + ".ffn.dense2_b", emb, dff);
    e.ln1g = up_f32(p + ".ln1_gammas", emb);
    e.ln1b = up_f32(p + ".ln1_betas", emb);
    e.ln2g = up_f32(p + ".ln2_gammas", emb);
    e.ln2b = up_f32(p + ".ln2_betas", emb);
    add_flops(64, e.qkv, body);
    add_flops(64, e.proj, body);
    add_flops(64, e.ffn1, body);
    add_flops(64, e.ffn2, body);
    info.flops_per_position += 2.0 * 2.0 * heads * 64 * 64 * (dm / heads);
    if (!body && size_of(p + ".mha.smolgen.compress"))
      throw Fail{B200_ERR_UNSUPPORTED, "smolgen in policy-head encoder layers is not supported"};
    if (size_of(p + ".mha.smolgen.compress")) {
      e.smolgen = true;
      const int hc = (int)size_of(p + ".mha.smolgen.compress") / emb;
      const int hid = (int)size_of(p + ".mha.smolgen.dense1_b");
      const int gen = (int)size_of(p + ".mha.smolgen.dense2_b");
      if (e.qkvc_out) {
        e.sg_compress.out = hc;
        e.sg_compress.in = emb;
        e.sg_compress.w = e.qkv.w + (size_t)3 * dm * emb;
        e.sg_compress.b = e.qkv.b + 3 * dm;  // zeros, or beta . W^T of the folded LayerNorm
        e.sg_compress.colsum = e.qkv.colsum ? e.qkv.colsum + 3 * dm : nullptr;
      } else {
        e.sg_compress = dense_maybe_folded(p + ".mha.smolgen.compress", "", hc, emb, in_gamma, in_beta);
      }
      e.sg_d1 = dense(p + ".mha.smolgen.dense1_w", p + ".mha.smolgen.dense1_b", hid, 64 * hc);
      e.sg_d2 = dense(p + ".mha.smolgen.dense2_w", p + ".mha.smolgen.dense2_b", gen, hid);
      e.sg_ln1g = up_f32(p + ".mha.smolgen.ln1_gammas", hid);
      e.sg_ln1b = up_f32(p + ".mha.smolgen.ln1_betas", hid);
      e.sg_ln2g = up_f32(p + ".mha.smolgen.ln2_gammas", gen);
      e.sg_ln2b = up_f32(p + ".mha.smolgen.ln2_betas", gen);
      if (gen % heads) throw Fail{B200_ERR_INVALID, "weights: smolgen width not divisible by heads"};
      if (sg_hc == 0) { sg_hc = hc; sg_hid = hid; sg_gen = gen; }
      if (hc != sg_hc || hid != sg_hid || gen != sg_gen)
        throw Fail{B200_ERR_UNSUPPORTED, "smolgen sizes differ between layers"};
      add_flops(64, e.sg_compress);
      add_flops(1, e.sg_d1);
      add_flops(1, e.sg_d2);
      info.flops_per_position += 2.0 * heads * (gen / heads) * 4096;
    }
    return e;
  }

  void build(const b200_builder* b, const b200_net_options& o) {
    bld = b;
    opt = o;
    network = (int)geti("network");
    policy_fmt = (int)geti("policy");
    value_fmt = (int)geti("value");
    emb_fmt = (int)geti("input_embedding");
    act_default = (int)geti("default_activation", ACT_RELU);
    act_smolgen = (int)geti("smolgen_activation", act_default);
    act_ffn = (int)geti("ffn_activation", act_default);
    if (network != NET_CLASSICAL_HF && network != NET_SE_HF && network != NET_ATTN_HF && network != NET_ATTN_MHF)
      throw Fail{B200_ERR_UNSUPPORTED, "Network format " + std::to_string(network) + " is not supported by the b200 backend."};
    if (policy_fmt < POLICY_CLASSICAL || policy_fmt > POLICY_ATTENTION)
      throw Fail{B200_ERR_UNSUPPORTED, "Policy format " + std::to_string(policy_fmt) + " is not supported by the b200 backend."};
    if (value_fmt != VALUE_CLASSICAL && value_fmt != VALUE_WDL)
      throw Fail{B200_ERR_UNSUPPORTED, "Value format " + std::to_string(value_fmt) + " is not supported by the b200 backend."};
    if (geti("moves_left") != 0 && geti("moves_left") != 1)
      throw Fail{B200_ERR_UNSUPPORTED, "Moves left head format is not supported by the b200 backend."};
    for (int a : {act_default, act_smolgen, act_ffn})
      if (a < ACT_MISH || a > ACT_RELU_2) throw Fail{B200_ERR_UNSUPPORTED, "unsupported activation function"};
    attn_body = network == NET_ATTN_HF || network == NET_ATTN_MHF;
    wdl = value_fmt == VALUE_WDL;
    mlh = geti("moves_left") == 1 && opt.mlh != 0;

    CK(cudaSetDevice(opt.gpu));
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, opt.gpu));
    sm_count = prop.multiProcessorCount;
    use_tc = sizeof(T) == 2 && !(opt.flags & B200_FLAG_NO_TENSOR_CORES);
    if (use_tc) {
      if (prop.major != 10)
        throw Fail{B200_ERR_UNSUPPORTED, "the tensor-core path needs an sm_100 device, found sm_" +
                                             std::to_string(prop.major) + std::to_string(prop.minor)};
      CK(gemm_tc_init());
    }
    merge_compress = !(opt.flags & B200_FLAG_NO_MERGED_COMPRESS);
    winograd = use_tc && !attn_body && (opt.flags & B200_FLAG_WINOGRAD);
    side_stream = use_tc && attn_body && !(opt.flags & B200_FLAG_NO_SIDE_STREAM) && sm_count >= 4 * kSideSms;
    dependent_launch = use_tc && !(opt.flags & B200_FLAG_NO_DEPENDENT_LAUNCH);
    heads_side = use_tc && !(opt.flags & B200_FLAG_NO_SIDE_STREAM) && sm_count >= 4 * kSideSms;
    // measured: +8 % at batch 64 on a 10 x 128 residual net, +2 % at 256 on a 20 x 256 one, +1.7 % at 64 on the BT4-class net,
    // nothing from 1024 on (the products then fill the GPU on their own)
    heads_side_max = 512;
    tower = use_tc && !attn_body && !(opt.flags & B200_FLAG_NO_TOWER_KERNEL) && !(opt.flags & B200_FLAG_NO_FUSED_SE) &&
            !(opt.flags & B200_FLAG_WINOGRAD);
    fold_ln = use_tc && attn_body && !(opt.flags & B200_FLAG_NO_LN_FOLD);
    // Folding needs every product that consumes or produces a folded LayerNorm to be eligible for the tensor-core
    // kernel's TMA epilogue: output widths that are multiples of 8.
    auto foldable = [](size_t width) { return width >= 8 && width % 8 == 0; };
    if (fold_ln) {
      if (!foldable(size_of("ip_emb_b"))) fold_ln = false;
      for (int i = 0; fold_ln && size_of("encoder." + std::to_string(i) + ".mha.q_w"); ++i) {
        const std::string p = "encoder." + std::to_string(i);
        if (!foldable(size_of(p + ".ffn.dense1_b")) || size_of(p + ".mha.q_b") != size_of("ip_emb_b")) fold_ln = false;
        const size_t cs = size_of(p + ".mha.smolgen.compress");
        if (cs && !foldable(cs / size_of("ip_emb_b"))) fold_ln = false;
      }
    }
    fold_heads = fold_ln && foldable(size_of("value.ip_val_b")) &&
                 (!mlh || foldable(size_of("ip_mov_b"))) &&
                 (policy_fmt != POLICY_ATTENTION || foldable(size_of("policy.ip_pol_b")));
    if (opt.slots > 64) throw Fail{B200_ERR_INVALID, "at most 64 slots"};
    d_status = (int*)walloc.alloc(64 * sizeof(int));
    CK(cudaMemset(d_status, 0, 64 * sizeof(int)));

    const Tables& tb = tables();
    d_attn_src = (short*)walloc.alloc(1858 * sizeof(short));
    CK(cudaMemcpy(d_attn_src, tb.attn_src.data(), 1858 * sizeof(short), cudaMemcpyHostToDevice));

    // ---- residual tower ----
    int res_blocks = 0;
    while (size_of("residual." + std::to_string(res_blocks) + ".conv1.weights")) ++res_blocks;
    if (res_blocks > 0 || !attn_body) {
      C = (int)size_of("input.biases");
      if (C <= 0) throw Fail{B200_ERR_INVALID, "weights: missing input convolution"};
      conv_in = conv3("input", C, 112);
      info.flops_per_position += 2.0 * 64 * 9 * 112 * C;
      for (int i = 0; i < res_blocks; ++i) {
        const std::string p = "residual." + std::to_string(i);
        ResidualW<T> r;
        r.c1 = conv3(p + ".conv1", C, C);
        r.c2 = conv3(p + ".conv2", C, C);
        info.flops_per_position += 2.0 * 2.0 * 64 * 9 * C * C;
        if (size_of(p + ".se.w1")) {
          r.se = true;
          r.se_k = (int)size_of(p + ".se.b1");
          r.se_w1 = up_f32(p + ".se.w1", (size_t)r.se_k * C);
          r.se_b1 = up_f32(p + ".se.b1", r.se_k);
          r.se_w2 = up_f32(p + ".se.w2", (size_t)2 * C * r.se_k);
          r.se_b2 = up_f32(p + ".se.b2", 2 * C);
        }
        res.push_back(r);
      }
    }
    const int body_ch = attn_body ? (int)size_of("ip_emb_b") : C;
    // The reference's CPU path for an attention body on top of a residual tower (network_blas.cc:603-659) feeds the
    // embedding from a buffer that nothing filled for that topology, so there is no reference result to match;
    // refused at load rather than at the first evaluation.
    if (attn_body && res_blocks > 0)
      throw Fail{B200_ERR_UNSUPPORTED, "attention body on top of a residual tower is not supported"};

    // ---- attention body ----
    if (attn_body) {
      E = (int)size_of("ip_emb_b");
      H = (int)geti("headcount");
      if (E <= 0 || H <= 0 || E % H) throw Fail{B200_ERR_INVALID, "weights: bad embedding size / head count"};
      if (E % 8 || E > 8192) throw Fail{B200_ERR_UNSUPPORTED, "embedding size must be a multiple of 8 and at most 8192"};
      int in_ch;
      if (res_blocks == 0) {
        if (emb_fmt == EMB_PE_DENSE) {
          pe_ch = (int)size_of("ip_emb_preproc_b") / 64;
          emb_pre = dense("ip_emb_preproc_w", "ip_emb_preproc_b", 64 * pe_ch, 64 * 12);
          add_flops(1, emb_pre);
        } else {
          pe_ch = 64;
          pos_enc = up_f32(tb.pos_enc);
        }
        in_ch = 112 + pe_ch;
      } else {
        in_ch = C;
      }
      cin = (in_ch + 7) / 8 * 8;
      {  // embedding weight, columns zero padded to cin
        const std::vector<float>& w = need("ip_emb_w", (size_t)E * in_ch);
        std::vector<float> p((size_t)E * cin, 0.f);
        for (int o = 0; o < E; ++o) std::copy(&w[(size_t)o * in_ch], &w[(size_t)o * in_ch] + in_ch, &p[(size_t)o * cin]);
        emb.out = E;
        emb.in = cin;
        emb.w = up_T(p);
        emb.b = up_f32("ip_emb_b", E);
        add_flops(64, emb);
      }
      if (emb_fmt == EMB_PE_DENSE) {
        emb_lng = up_f32("ip_emb_ln_gammas", E);
        emb_lnb = up_f32("ip_emb_ln_betas", E);
      }
      if (size_of("ip_mult_gate") && size_of("ip_add_gate")) {
        const auto& m = need("ip_mult_gate", (size_t)E * 64);
        const auto& a = need("ip_add_gate", (size_t)E * 64);
        std::vector<float> mt((size_t)64 * E), at((size_t)64 * E);
        for (int c = 0; c < E; ++c)
          for (int sq = 0; sq < 64; ++sq) {
            mt[(size_t)sq * E + c] = m[(size_t)c * 64 + sq];
            at[(size_t)sq * E + c] = a[(size_t)c * 64 + sq];
          }
        gate_mult = up_f32(mt);
        gate_add = up_f32(at);
      }
      while (size_of("encoder." + std::to_string(layers) + ".mha.q_w")) ++layers;
      alpha = (float)std::pow(2.0 * layers, -0.25);
      ln_eps = emb_fmt == EMB_PE_DENSE ? 1e-3f : 1e-6f;
      if (emb_fmt == EMB_PE_DENSE) {
        emb_dff = (int)size_of("ip_emb_ffn.dense1_b");
        emb_ffn1 = dense("ip_emb_ffn.dense1_w", "ip_emb_ffn.dense1_b", emb_dff, E);
        emb_ffn2 = dense("ip_emb_ffn.dense2_w", "ip_emb_ffn.dense2_b", E, emb_dff);
        emb_ffn_lng = up_f32("ip_emb_ffn_ln_gammas", E);
        emb_ffn_lnb = up_f32("ip_emb_ffn_ln_betas", E);
        add_flops(64, emb_ffn1);
        add_flops(64, emb_ffn2);
      }
      max_dff = emb_dff;
      for (int i = 0; i < layers; ++i) {
        const std::vector<float>*g = nullptr, *bt = nullptr;
        if (fold_ln && i > 0) {
          g = &need("encoder." + std::to_string(i - 1) + ".ln2_gammas", E);
          bt = &need("encoder." + std::to_string(i - 1) + ".ln2_betas", E);
        } else if (fold_ln && emb_fmt == EMB_PE_DENSE) {
          // the LayerNorm that ends the embedding block is folded into the first layer the same way
          fold_emb_ln = true;
          g = &need("ip_emb_ffn_ln_gammas", E);
          bt = &need("ip_emb_ffn_ln_betas", E);
        }
        enc.push_back(load_encoder("encoder." + std::to_string(i), E, H, g, bt));
        max_dff = std::max(max_dff, enc.back().ffn1.out);
      }
      if (sg_gen) {
        // the LayerNorm kernels read rows in vectors of 8 elements and keep a row of at most 8192 in registers
        if (sg_hid % 8 || sg_gen % 8 || sg_hid > 8192 || sg_gen > 8192)
          throw Fail{B200_ERR_UNSUPPORTED, "smolgen widths must be multiples of 8 and at most 8192"};
        smolgen_w = dense("smolgen_w", "", 4096, sg_gen / H);
      }
    }

    // ---- policy head ----
    if (policy_fmt == POLICY_ATTENTION) {
      const int pe = (int)size_of("policy.ip_pol_b");
      pol_dm = (int)size_of("policy.ip2_pol_b");
      pol_emb = dense_maybe_folded("policy.ip_pol_w", "policy.ip_pol_b", pe, body_ch, head_gamma(), head_beta());
      // encoder layers of the policy head (network_blas.cc:832-838): alpha 1, epsilon 1e-6, explicit LayerNorms
      int n_pol = 0;
      while (size_of("policy.pol_encoder." + std::to_string(n_pol) + ".mha.q_w")) ++n_pol;
      if (n_pol > 0) {
        pol_heads = (int)geti("pol_headcount");
        if (pol_heads <= 0 || pe % pol_heads || pe % 8)
          throw Fail{B200_ERR_INVALID, "weights: bad policy-head encoder width / head count"};
        for (int i = 0; i < n_pol; ++i) {
          pol_enc.push_back(load_encoder("policy.pol_encoder." + std::to_string(i), pe, pol_heads, nullptr, nullptr, false));
          max_dff = std::max(max_dff, pol_enc.back().ffn1.out);
        }
      }
      pol_q = dense("policy.ip2_pol_w", "policy.ip2_pol_b", pol_dm, pe);
      pol_k = dense("policy.ip3_pol_w", "policy.ip3_pol_b", pol_dm, pe);
      pol_w4 = up_f32("policy.ip4_pol_w", (size_t)4 * pol_dm);
      add_flops(64, pol_emb);
      add_flops(64, pol_q);
      add_flops(64, pol_k);
      info.flops_per_position += 2.0 * 64 * 64 * pol_dm;
    } else if (policy_fmt == POLICY_CONVOLUTION) {
      if (attn_body) throw Fail{B200_ERR_UNSUPPORTED, "convolutional policy with an attention body is not supported"};
      pol_planes = (int)size_of("policy.policy.biases");
      if (pol_planes < 73) throw Fail{B200_ERR_INVALID, "weights: convolutional policy needs at least 73 planes"};
      pol_conv1 = conv3("policy.policy1", C, C);
      pol_conv2 = conv3("policy.policy", pol_planes, C);
      info.flops_per_position += 2.0 * 64 * 9 * C * (C + pol_planes);
      std::vector<short> src(1858);
      for (int j = 0; j < 1858; ++j) {
        const int plane = tb.conv_src[j] / 64, sq = tb.conv_src[j] % 64;
        src[j] = short(sq * pol_planes + plane);
      }
      d_conv_src = (short*)walloc.alloc(1858 * sizeof(short));
      CK(cudaMemcpy(d_conv_src, src.data(), 1858 * sizeof(short), cudaMemcpyHostToDevice));
    } else {
      if (attn_body) throw Fail{B200_ERR_UNSUPPORTED, "classical policy with an attention body is not supported"};
      pol_planes = (int)size_of("policy.policy.biases");
      pol_c1x1 = conv1("policy.policy", pol_planes, C);
      pol_fc = dense_chw("policy.ip_pol_w", "policy.ip_pol_b", 1858, pol_planes);
      add_flops(64, pol_c1x1);
      add_flops(1, pol_fc);
    }

    // ---- value head ----
    {
      const int vh = (int)size_of("value.ip1_val_b");
      int vp;
      if (attn_body) {
        vp = (int)size_of("value.ip_val_b");
        val_emb = dense_maybe_folded("value.ip_val_w", "value.ip_val_b", vp, E, head_gamma(), head_beta());
        val_fc1 = dense("value.ip1_val_w", "value.ip1_val_b", vh, vp * 64);
      } else {
        vp = (int)size_of("value.value.biases");
        val_emb = conv1("value.value", vp, C);
        val_fc1 = dense_chw("value.ip1_val_w", "value.ip1_val_b", vh, vp);
      }
      const int outs = wdl ? 3 : 1;
      val_w2 = up_f32("value.ip2_val_w", (size_t)outs * vh);
      val_b2 = up_f32("value.ip2_val_b", outs);
      add_flops(64, val_emb);
      add_flops(1, val_fc1);
    }
    // ---- moves-left head ----
    if (mlh) {
      const int mh = (int)size_of("ip1_mov_b");
      int mp;
      if (attn_body) {
        mp = (int)size_of("ip_mov_b");
        mov_emb = dense_maybe_folded("ip_mov_w", "ip_mov_b", mp, E, head_gamma(), head_beta());
        mov_fc1 = dense("ip1_mov_w", "ip1_mov_b", mh, mp * 64);
      } else {
        mp = (int)size_of("moves_left.biases");
        mov_emb = conv1("moves_left", mp, C);
        mov_fc1 = dense_chw("ip1_mov_w", "ip1_mov_b", mh, mp);
      }
      mov_w2 = up_f32("ip2_mov_w", mh);
      mov_b2 = up_f32("ip2_mov_b", 1);
      add_flops(64, mov_emb);
      add_flops(1, mov_fc1);
    }

    alloc_slots();
    build_towers();
    // The uploads above are copies from pageable memory and the slots' streams are non-blocking: everything must have
    // landed before the first evaluation is enqueued.
    CK(cudaDeviceSynchronize());

    info.input_format = (int)geti("input_format");
    info.output_format = (int)geti("output_format");
    info.moves_left_format = (int)geti("moves_left");
    info.wdl = wdl;
    info.has_mlh = mlh;
    info.attention_body = attn_body;
    info.embedding = E;
    info.encoder_layers = layers;
    info.heads = H;
    info.dff = enc.empty() ? 0 : enc[0].ffn1.out;
    info.filters = C;
    info.residual_blocks = (int)res.size();
    info.max_batch = opt.max_batch;
    info.precision = opt.precision;
    info.sm_count = sm_count;
    info.weight_bytes = walloc.bytes;
    info.workspace_bytes = salloc.bytes;
    bld = nullptr;
  }

  void alloc_slots() {
    const size_t nb = (size_t)opt.max_batch, R = nb * 64;
    slots.resize(opt.slots);
    graph_cache.resize(opt.slots);
    auto A = [&](size_t elems) { return (T*)salloc.alloc(elems * sizeof(T)); };
    for (int si = 0; si < opt.slots; ++si) {
      Slot& s = slots[si];
      int prio_low = 0, prio_high = 0;
      CK(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
      CK(cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, prio_high));
      CK(cudaStreamCreateWithPriority(&s.stream2, cudaStreamNonBlocking, prio_low));
      CK(cudaEventCreateWithFlags(&s.ev_fork, cudaEventDisableTiming));
      CK(cudaEventCreateWithFlags(&s.ev_join, cudaEventDisableTiming));
      CK(cudaEventCreateWithFlags(&s.compute_done, cudaEventDisableTiming));
      CK(cudaMallocHost(&s.h_status, sizeof(int)));
      *s.h_status = 0;
      s.d_masks = (uint64_t*)salloc.alloc(nb * 112 * 8);
      s.d_values = (float*)salloc.alloc(nb * 112 * 4);
      s.d_policy = (float*)salloc.alloc(nb * 1858 * 4);
      s.d_qdm = (float*)salloc.alloc(nb * 3 * 4);
      s.d_move_ids = (unsigned short*)salloc.alloc(nb * kLegalStride * 2);
      s.d_n_moves = (int*)salloc.alloc(nb * 4);
      s.d_probs = (float*)salloc.alloc(nb * kLegalStride * 4);
      s.d_boards = (b200_board*)salloc.alloc(board_capacity() * sizeof(b200_board));
      s.d_offsets = (int*)salloc.alloc((nb + 1) * sizeof(int));
      s.d_from_start = (uint8_t*)salloc.alloc(nb);
      const int body_ch = attn_body ? E : C;
      if (!res.empty() || !attn_body) {
        s.tokens = A(R * 112);
        s.x = A(R * C);
        s.x1 = A(R * C);
        s.y = A(R * C);
        if (winograd) {
          const size_t rows = (nb * 4 + 255) / 256 * 256;
          const size_t ch = (size_t)std::max(std::max(C, 112), pol_planes);
          s.wino_v = A(36 * rows * ch);
          s.wino_m = A(36 * rows * ch);
        }
      }
      if (attn_body) {
        if (res.empty()) s.tokens = A(R * cin);
        if (emb_fmt == EMB_PE_DENSE && res.empty()) {
          s.pre = A(nb * 768);
          s.pe = A(nb * 64 * pe_ch);
        }
        if (!s.x || E > C) {
          s.x = A(R * E);
          s.x1 = A(R * E);
          s.y = A(R * E);
        }
        s.qkv = A(R * 3 * E);
        if (fold_ln) {
          double* blk = (double*)salloc.alloc(3 * R * 2 * sizeof(double));
          s.stats2[0] = blk;
          s.stats1 = blk + R * 2;
          s.stats2[1] = blk + 2 * R * 2;
          s.stats_stride = (size_t)R * 2;
        }
        s.att = A(R * E);
        s.ffn = A(R * std::max(max_dff, 8));
        if (sg_gen) {
          s.sg_c = A(R * sg_hc);
          s.sg_h1 = A(nb * sg_hid);
          s.sg_h2 = A(nb * sg_gen);
          s.sg_bias = A(nb * H * 4096);
        }
      }
      if (policy_fmt == POLICY_ATTENTION) {
        s.pemb = A(R * pol_emb.out);
        if (!pol_enc.empty()) {
          int pdff = 8;
          for (const auto& e : pol_enc) pdff = std::max(pdff, e.ffn1.out);
          s.p_qkv = A(R * 3 * pol_emb.out);
          s.p_att = A(R * pol_emb.out);
          s.p_x1 = A(R * pol_emb.out);
          s.p_y = A(R * pol_emb.out);
          s.p_ffn = A(R * pdff);
        }
        s.pq = A(R * pol_dm);
        s.pk = A(R * pol_dm);
        s.logits = (float*)salloc.alloc(nb * 4096 * 4);
      } else if (policy_fmt == POLICY_CONVOLUTION) {
        s.praw = A(R * pol_planes);
      } else {
        s.praw = A(R * pol_planes);
      }
      (void)body_ch;
      s.vtok = A(R * val_emb.out);
      s.vhid = A(nb * val_fc1.out);
      if (mlh) {
        s.mtok = A(R * mov_emb.out);
        s.mhid = A(nb * mov_fc1.out);
      }
      free_slots.push_back(si);
    }
  }

  // ---- launch helpers ----
  void gemm(cudaStream_t st, const T* A, long long lda, const Dense<T>& d, T* Cout, long long ldc, int M, int act,
            const T* skip = nullptr, long long ldskip = 0, float alpha_ = 1.f, bool out_f32 = false,
            void* cf32 = nullptr) {
    GemmParams p;
    p.A = A; p.lda = lda; p.W = d.w; p.ldw = d.in; p.bias = d.b;
    p.C = out_f32 ? cf32 : (void*)Cout; p.ldc = ldc; p.M = M; p.N = d.out; p.K = d.in; p.act = act;
    p.skip = skip; p.ldskip = ldskip; p.alpha = alpha_; p.out_f32 = out_f32;
    p.whole_tiles = (opt.flags & B200_FLAG_NO_SPLIT_LAST_WAVE) != 0;
    run_gemm(st, p);
  }
  // A LayerNorm output that is either materialised (stats == nullptr) or kept as its un-normalised input `u`
  // with per-row statistics and the LayerNorm's parameters.
  struct LNState {
    const T* u = nullptr;
    const double* stats = nullptr;
    const float* gamma = nullptr;
    const float* beta = nullptr;
  };
  // Product whose A operand is `in` (folded when in.stats is set); optional residual `res` added as
  // alpha * act(...) + LN(res) and optional accumulation of output row statistics.
  void gemm_ln(cudaStream_t st, const LNState& in, long long lda, const Dense<T>& d, T* Cout, long long ldc, int M,
               int act, const LNState* res = nullptr, float alpha_ = 1.f, double* out_stats = nullptr,
               T* C2 = nullptr, long long ldc2 = 0, int n_split = 0, bool zero_stats = true) {
    GemmParams p;
    p.C2 = C2; p.ldc2 = ldc2; p.n_split = n_split;
    p.A = in.u; p.lda = lda; p.W = d.w; p.ldw = d.in; p.bias = d.b;
    p.C = Cout; p.ldc = ldc; p.M = M; p.N = d.out; p.K = d.in; p.act = act;
    if (in.stats) {
      if (!d.colsum) throw Fail{B200_ERR_INVALID, "internal: folded input for a layer without folded weights"};
      p.a_stats = in.stats; p.colsum = d.colsum; p.a_inv_c = 1.0f / d.in; p.a_eps = ln_eps;
    }
    if (res) {
      p.res = res->u; p.ldres = d.out; p.alpha = alpha_;
      if (res->stats) {
        p.res_stats = res->stats; p.res_gamma = res->gamma; p.res_beta = res->beta;
        p.res_inv_c = 1.0f / d.out; p.res_eps = ln_eps;
      }
    }
    if (out_stats) {
      if (zero_stats) CK(cudaMemsetAsync(out_stats, 0, (size_t)M * 2 * sizeof(double), st));
      p.out_stats = out_stats;
    }
    p.whole_tiles = (opt.flags & B200_FLAG_NO_SPLIT_LAST_WAVE) != 0;
    run_gemm(st, p);
  }
  // Tag of the launches that follow on this thread (which product of the layer they are), for the tagged profile.
  static inline thread_local int t_tag = 0;
  void run_gemm(cudaStream_t st, const GemmParams& p) {
    launches++;
    const double flops = 2.0 * p.M * (double)p.N * p.K * p.batch;
    if constexpr (sizeof(T) == 2) {
      if (use_tc && p.M >= 64 && gemm_tc_supported(p)) {
        const int sp_ = span_begin(st, K_GEMM_TC, flops, t_tag);
        CK(launch_gemm_tc<T>(p, t_status, t_sm_limit > 0 ? t_sm_limit : sm_count, st));
        span_end(st, sp_);
        return;
      }
    }
    if (p.a_stats || p.res || p.out_stats)
      throw Fail{B200_ERR_UNSUPPORTED, "internal: folded LayerNorm product outside the tensor-core kernel"};
    const int sp_ = span_begin(st, K_GEMM_FMA, flops);
    CK(launch_gemm_simt<T>(p, st));
    span_end(st, sp_);
  }
  // Any other kernel: counted, and timed under the class "other" (work = algorithmic bytes).
  template <typename F>
  void other(cudaStream_t st, double bytes, F&& launch) {
    launches++;
    const int sp_ = span_begin(st, K_OTHER, bytes);
    CK(launch());
    span_end(st, sp_);
  }
  // 3x3 convolution: tensor-core kernel (TMA board tiles with zero-filled halo) for 16-bit storage, FMA otherwise.
  // Winograd form of the same convolution (winograd.cu): transform, 36 stacked products, transform back with bias,
  // optional squeeze-excitation (r != nullptr), optional skip and the activation.
  bool conv3_wino(cudaStream_t st, const T* x, const ConvW<T>& c, const float* bias, T* y, int n, int act,
                  const T* skip = nullptr, const ResidualW<T>* r = nullptr) {
    if constexpr (sizeof(T) == 2) {
      if (!winograd || !c.u || (c.cin % 8) || (c.cout % 8) || c.cout > 256) return false;
      Slot& s = *static_cast<Slot*>(t_slot_ptr);
      const long long rows = ((long long)n * 4 + 255) / 256 * 256;
      GemmParams p;
      p.A = s.wino_v; p.lda = c.cin; p.W = c.u; p.ldw = c.cin; p.C = s.wino_m; p.ldc = c.cout;
      p.M = (int)(36 * rows); p.N = c.cout; p.K = c.cin; p.batch_rows = (int)rows;
      if (!gemm_tc_supported(p)) return false;
      other(st, (double)n * 64 * c.cin * sizeof(T) * (1.0 + 36.0 / 16.0),
            [&] { return launch_wino_input<T>(x, s.wino_v, c.cin, n, rows, st); });
      launches++;
      const int sp_ = span_begin(st, K_GEMM_TC, 2.0 * 36 * n * 4 * (double)c.cin * c.cout);  // Winograd-domain FLOPs
      CK(launch_gemm_tc<T>(p, t_status, sm_count, st));
      span_end(st, sp_);
      other(st, (double)n * 64 * c.cout * sizeof(T) * (1.0 + 36.0 / 16.0 + (skip ? 1.0 : 0.0)), [&] {
        return launch_wino_output<T>(s.wino_m, bias, skip, r ? r->se_w1 : nullptr, r ? r->se_b1 : nullptr,
                                     r ? r->se_w2 : nullptr, r ? r->se_b2 : nullptr, r ? r->se_k : 0, y, c.cout, n, rows,
                                     act, st);
      });
      return true;
    }
    return false;
  }
  static GemmParams conv_params(const T* x, const ConvW<T>& c, const float* bias, T* y, int n, int act) {
    GemmParams p;
    p.A = x; p.W = c.w; p.bias = bias; p.C = y; p.ldc = c.cout; p.M = n * 64; p.N = c.cout; p.K = 9 * c.cin;
    p.act = act; p.conv_cin = c.cin; p.lda = c.cin; p.ldw = c.cin;
    return p;
  }
  GemmParams conv_se_params(const T* x, const ResidualW<T>& r, const T* skip, T* y, int n) const {
    const ConvW<T>& c = r.c2;
    GemmParams p = conv_params(x, c, nullptr, y, n, act_default);
    p.res = skip; p.ldres = c.cout;
    p.se_w1 = r.se_w1; p.se_b1 = r.se_b1; p.se_w2 = r.se_w2; p.se_b2 = r.se_b2; p.se_bias = c.b; p.se_k = r.se_k;
    return p;
  }
  // Residual towers whose blocks all carry a squeeze-excitation unit: the table of the tower kernel, once per slot
  // (its descriptors cover the buffers' full extent, so it serves every batch size).  The buffers rotate exactly as in
  // forward().
  void build_towers() {
    if constexpr (sizeof(T) == 2) {
      // Measured (evaluations per second, tower / per-layer launches): 10 blocks of 128 filters 176 100 / 161 400 at
      // batch 64 and 670 800 / 589 000 at batch 256; 20 blocks of 256 filters 57 100 / 55 300 at batch 64 and 210 100 /
      // 212 300 at batch 256: the wide tower stays on one launch per convolution (CTA pairs from 150 positions on).
      if (!tower || res.empty() || C > 128) { tower = false; return; }
      for (const auto& r : res)
        if (!r.se) { tower = false; return; }
      const int nb = opt.max_batch;
      for (size_t si = 0; si < slots.size(); ++si) {
        Slot& s = slots[si];
        std::vector<GemmParams> g;
        g.push_back(conv_params(s.tokens, conv_in, conv_in.b, s.x, nb, act_default));
        T *cur = s.x, *tmp = s.x1, *tmp2 = s.y;
        for (const auto& r : res) {
          g.push_back(conv_params(cur, r.c1, r.c1.b, tmp, nb, act_default));
          g.push_back(conv_se_params(tmp, r, cur, tmp2, nb));
          std::swap(cur, tmp2);
        }
        if (!gemm_tc_tower_supported(g.data(), (int)g.size())) { tower = false; return; }
        std::vector<unsigned char> host(g.size() * gemm_tc_tower_layer_bytes());
        CK(gemm_tc_tower_build<T>(g.data(), (int)g.size(), d_status + si, host.data()));
        s.tower_layers = salloc.alloc(host.size());
        CK(cudaMemcpy(s.tower_layers, host.data(), host.size(), cudaMemcpyHostToDevice));
        s.tower_n = (int)g.size();
      }
      // one CTA per two boards walks all layers: worth it while the launches it replaces are latency-bound
      tower_max_batch = 16 * sm_count;
    } else {
      tower = false;
    }
  }
  void conv3(cudaStream_t st, const T* x, const ConvW<T>& c, const float* bias, T* y, int n, int act) {
    if (conv3_wino(st, x, c, bias, y, n, act)) return;
    if constexpr (sizeof(T) == 2) {
      GemmParams p = conv_params(x, c, bias, y, n, act);
      if (use_tc && (c.cout % 8) == 0 && gemm_tc_supported(p)) {
        launches++;
        const int sp_ = span_begin(st, K_GEMM_TC, 2.0 * p.M * (double)p.N * p.K);
        CK(launch_gemm_tc<T>(p, t_status, sm_count, st));
        span_end(st, sp_);
        return;
      }
    }
    launches++;
    const int sp_ = span_begin(st, K_GEMM_FMA, 2.0 * n * 64 * (double)c.cout * 9 * c.cin);
    CK(launch_conv3x3<T>(x, c.cin, c.w, bias, y, c.cout, n, act, st));
    span_end(st, sp_);
  }
  // Second convolution of a residual block with its squeeze-excitation unit, the skip connection and the activation
  // in the tensor-core kernel's epilogue (network_blas.cc:584-597); false when the shape does not qualify.
  bool conv3_se(cudaStream_t st, const T* x, const ResidualW<T>& r, const T* skip, T* y, int n) {
    if constexpr (sizeof(T) == 2) {
      if (!use_tc || (opt.flags & B200_FLAG_NO_FUSED_SE)) return false;
      const GemmParams p = conv_se_params(x, r, skip, y, n);
      if (!gemm_tc_supported(p) || !gemm_tc_se_supported(p)) return false;
      launches++;
      const int sp_ = span_begin(st, K_GEMM_TC, 2.0 * p.M * (double)p.N * p.K);
      CK(launch_gemm_tc<T>(p, t_status, sm_count, st));
      span_end(st, sp_);
      return true;
    }
    return false;
  }
  void ln(cudaStream_t st, T* out, const T* x, const T* skip, const float* g, const float* b, int rows, int Cc,
          float a, float eps, const float* gm = nullptr, const float* ga = nullptr) {
    launches++;
    // algorithmic bytes: read x (+ skip), write out
    const int sp_ = span_begin(st, K_LAYERNORM, (double)rows * Cc * sizeof(T) * (skip ? 3 : 2));
    CK(launch_layer_norm<T>(out, x, skip, g, b, gm, ga, rows, Cc, a, eps, st));
    span_end(st, sp_);
  }

  // softmax(Q K^T / sqrt(depth) + bias) V for every (position, head); q, k, v are consecutive column blocks of `qkv`
  void run_attention(cudaStream_t st, const T* qkv, int ld, const T* bias, T* out, int width, int n, int heads) {
    const int depth = width / heads;
    const float scale = 1.0f / sqrtf((float)depth);
    launches++;
    // algorithmic bytes: read Q, K, V (+ bias), write the head outputs
    const int sp_ = span_begin(st, K_ATTENTION, (double)n * 64 * width * sizeof(T) * 4 +
                                                    (bias ? (double)n * heads * 4096 * sizeof(T) : 0.0), TAG_ATTENTION);
    bool done = false;
    if constexpr (sizeof(T) == 2) {
      if (use_tc && attention_tc_supported(ld, width, depth, qkv, qkv + width, qkv + 2 * width, bias, out)) {
        CK(launch_attention_tma<T>(qkv, qkv + width, qkv + 2 * width, ld, bias, out, width, n, heads, depth, scale,
                                   t_status, sm_count, st));
        done = true;
      }
    }
    if (!done) CK(launch_attention<T>(qkv, qkv + width, qkv + 2 * width, ld, bias, out, width, n, heads, depth, scale, st));
    span_end(st, sp_);
  }
  // One encoder layer of the attention policy head (network_blas.cc:832-838: ForwardEncoderLayer with alpha 1 and
  // epsilon 1e-6 on the policy embedding), LayerNorms as kernels; x [n*64][pe] is the layer's input and output.
  void policy_encoder_layer(Slot& s, const EncoderW<T>& e, int n, T* x) {
    cudaStream_t st = s.stream;
    const int R = n * 64, pe = pol_emb.out;
    const int act = attn_body ? act_ffn : ACT_SELU;
    gemm(st, x, pe, e.qkv, s.p_qkv, 3 * pe, R, ACT_NONE);
    run_attention(st, s.p_qkv, 3 * pe, nullptr, s.p_att, pe, n, pol_heads);
    gemm(st, s.p_att, pe, e.proj, s.p_y, pe, R, ACT_NONE);
    ln(st, s.p_x1, s.p_y, x, e.ln1g, e.ln1b, R, pe, 1.f, 1e-6f);
    gemm(st, s.p_x1, pe, e.ffn1, s.p_ffn, e.ffn1.out, R, act);
    gemm(st, s.p_ffn, e.ffn1.out, e.ffn2, s.p_y, pe, R, ACT_NONE);
    ln(st, x, s.p_y, s.p_x1, e.ln2g, e.ln2b, R, pe, 1.f, 1e-6f);
  }
  // `in` describes the layer input: buffer x, materialised for the first layer, afterwards the un-normalised
  // sum of the previous layer with its statistics.  With folding the two LayerNorms of the layer never run as
  // kernels: out-proj and FFN2 add the (normalised-on-the-fly) residual and accumulate row statistics, QKV,
  // the smolgen compression and FFN1 apply the normalisation as a row scale plus a rank-1 correction.
  void encoder_layer(Slot& s, const EncoderW<T>& e, int n, T*& x, T*& x1, LNState& in) {
    cudaStream_t st = s.stream;
    const int R = n * 64;
    const int depth = E / H;
    const T* bias = nullptr;
    // The statistics this layer accumulates are cleared here, in one memset ahead of all its launches, so that no
    // memset sits between two products.  The layer input may refer to the other stats2 buffer.
    double* stats2 = nullptr;
    if (fold_ln) {
      const int par = s.stats_parity;
      s.stats_parity ^= 1;
      stats2 = s.stats2[par];
      CK(cudaMemsetAsync(par == 0 ? s.stats2[0] : s.stats1, 0, (s.stats_stride + (size_t)R * 2) * sizeof(double), st));
    }
    // With per-launch event pairs on (profiling) the layer runs in line: a span around a launch that shares the GPU
    // with another stream measures the sharing, not the kernel.
    if (side_stream && !profiling && e.smolgen && R >= 2048) {
      // compression first (it reads the whole layer input: memory-bound, all SMs), then the two small dense layers
      // with their LayerNorms on the side stream while Q, K, V are computed on the other SMs
      cudaStream_t st2 = s.stream2;
      t_tag = TAG_SMOLGEN_DENSE;
      gemm_ln(st, in, E, e.sg_compress, s.sg_c, sg_hc, R, ACT_NONE);
      CK(cudaEventRecord(s.ev_fork, st));
      // Q, K, V first and on the higher-priority stream: its CTA pairs take whole TPCs, the side stream's CTAs then
      // land on the SMs it leaves free
      t_sm_limit = (sm_count - kSideSms) & ~1;
      t_tag = TAG_QKV;
      gemm_ln(st, in, E, e.qkv, s.qkv, 3 * E, R, ACT_NONE);
      CK(cudaStreamWaitEvent(st2, s.ev_fork, 0));
      t_sm_limit = kSideSms;
      t_tag = TAG_SMOLGEN_DENSE;
      {  // the first launch behind an event of the other stream is an ordinary one
        DependentLaunchScope ordinary(false);
        gemm(st2, s.sg_c, 64 * sg_hc, e.sg_d1, s.sg_h1, sg_hid, n, act_smolgen);
      }
      ln(st2, s.sg_h1, s.sg_h1, nullptr, e.sg_ln1g, e.sg_ln1b, n, sg_hid, 1.f, 1e-3f);
      gemm(st2, s.sg_h1, sg_hid, e.sg_d2, s.sg_h2, sg_gen, n, act_smolgen);
      ln(st2, s.sg_h2, s.sg_h2, nullptr, e.sg_ln2g, e.sg_ln2b, n, sg_gen, 1.f, 1e-3f);
      CK(cudaEventRecord(s.ev_join, st2));
      t_sm_limit = 0;
      CK(cudaStreamWaitEvent(st, s.ev_join, 0));
      t_tag = TAG_SMOLGEN_BIAS;
      {
        DependentLaunchScope ordinary(false);
        gemm(st, s.sg_h2, sg_gen / H, smolgen_w, s.sg_bias, 4096, n * H, ACT_NONE);
      }
      bias = s.sg_bias;
      run_attention(st, s.qkv, 3 * E, bias, s.att, E, n, H);
      finish_layer(s, e, R, x, x1, in, stats2);
      return;
    }
    // One launch for Q, K, V and the smolgen compression when the CTA-pair kernel takes the product.
    bool merged = false;
    if (e.smolgen && e.qkvc_out && merge_compress) {
      GemmParams probe;
      probe.A = in.u; probe.lda = E; probe.W = e.qkv.w; probe.ldw = E; probe.C = s.qkv; probe.ldc = 3 * E;
      probe.M = R; probe.N = e.qkvc_out; probe.K = E; probe.C2 = s.sg_c; probe.ldc2 = sg_hc; probe.n_split = 3 * E;
      merged = gemm_tc_split_supported(probe, sm_count);
    }
    t_tag = TAG_QKV;
    if (merged) {
      Dense<T> both = e.qkv;
      both.out = e.qkvc_out;
      gemm_ln(st, in, E, both, s.qkv, 3 * E, R, ACT_NONE, nullptr, 1.f, nullptr, s.sg_c, sg_hc, 3 * E);
    } else {
      gemm_ln(st, in, E, e.qkv, s.qkv, 3 * E, R, ACT_NONE);  // :341-350, :408-412
    }
    if (e.smolgen) {  // network_blas.cc:300-339
      t_tag = TAG_SMOLGEN_DENSE;
      if (!merged) gemm_ln(st, in, E, e.sg_compress, s.sg_c, sg_hc, R, ACT_NONE);
      gemm(st, s.sg_c, 64 * sg_hc, e.sg_d1, s.sg_h1, sg_hid, n, act_smolgen);
      ln(st, s.sg_h1, s.sg_h1, nullptr, e.sg_ln1g, e.sg_ln1b, n, sg_hid, 1.f, 1e-3f);
      gemm(st, s.sg_h1, sg_hid, e.sg_d2, s.sg_h2, sg_gen, n, act_smolgen);
      ln(st, s.sg_h2, s.sg_h2, nullptr, e.sg_ln2g, e.sg_ln2b, n, sg_gen, 1.f, 1e-3f);
      t_tag = TAG_SMOLGEN_BIAS;
      gemm(st, s.sg_h2, sg_gen / H, smolgen_w, s.sg_bias, 4096, n * H, ACT_NONE);
      bias = s.sg_bias;
    }
    run_attention(st, s.qkv, 3 * E, bias, s.att, E, n, H);  // :352-439
    finish_layer(s, e, R, x, x1, in, stats2);
  }
  // Output projection, first LayerNorm, FFN, second LayerNorm of an encoder layer (network_blas.cc:441-470).
  void finish_layer(Slot& s, const EncoderW<T>& e, int R, T*& x, T*& x1, LNState& in, double* stats2) {
    cudaStream_t st = s.stream;
    if (fold_ln) {
      LNState att{s.att, nullptr, nullptr, nullptr}, ffn{s.ffn, nullptr, nullptr, nullptr};
      t_tag = TAG_OUT_PROJ;
      gemm_ln(st, att, E, e.proj, x1, E, R, ACT_NONE, &in, alpha, s.stats1, nullptr, 0, 0, false);  // u1 = alpha * proj + x
      LNState mid{x1, s.stats1, e.ln1g, e.ln1b};
      t_tag = TAG_FFN1;
      gemm_ln(st, mid, E, e.ffn1, s.ffn, e.ffn1.out, R, act_ffn);                  // relu2(LN1(u1) W1 + b1)
      t_tag = TAG_FFN2;
      gemm_ln(st, ffn, e.ffn1.out, e.ffn2, x, E, R, ACT_NONE, &mid, alpha, stats2, nullptr, 0, 0, false);  // u2 = alpha * ffn + LN1(u1)
      t_tag = TAG_NONE;
      in = LNState{x, stats2, e.ln2g, e.ln2b};
      return;
    }
    t_tag = TAG_OUT_PROJ;
    gemm(st, s.att, E, e.proj, s.y, E, R, ACT_NONE);           // :441-445
    ln(st, x1, s.y, x, e.ln1g, e.ln1b, R, E, alpha, ln_eps);   // :447-452
    t_tag = TAG_FFN1;
    gemm(st, x1, E, e.ffn1, s.ffn, e.ffn1.out, R, act_ffn);    // :454-458
    t_tag = TAG_FFN2;
    gemm(st, s.ffn, e.ffn1.out, e.ffn2, s.y, E, R, ACT_NONE);  // :460-463
    ln(st, x, s.y, x1, e.ln2g, e.ln2b, R, E, alpha, ln_eps);   // :465-470
    t_tag = TAG_NONE;
    in = LNState{x, nullptr, nullptr, nullptr};
  }

  void forward(Slot& s, const uint64_t* d_masks, const float* d_values, int n, float* d_policy, float* d_qdm) {
    cudaStream_t st = s.stream;
    const int R = n * 64;
    T* flow = nullptr;  // output of the body, [R][body_ch]
    int body_ch = 0;
    LNState body_in;    // attention bodies: how the heads must read `flow` (folded LayerNorm or materialised)
    s.stats_parity = 0;
    t_status = d_status + (&s - slots.data());
    t_slot_ptr = &s;
    // not with per-launch event pairs: the spans would then time the overlap with the neighbours
    DependentLaunchScope launch_scope(dependent_launch && !profiling);
    CK(cudaMemsetAsync(d_qdm, 0, (size_t)n * 3 * sizeof(float), st));
    if (!res.empty() || !attn_body) {  // network_blas.cc:564-601
      other(st, (double)R * 112 * sizeof(T), [&] {
        return launch_expand_tokens<T>(d_masks, d_values, n, nullptr, (const T*)nullptr, 0, 112, s.tokens, st);
      });
      T *cur = s.x, *tmp = s.x1, *tmp2 = s.y;
      bool in_one = false;
      if constexpr (sizeof(T) == 2) {
        if (tower && s.tower_layers && n <= tower_max_batch) {
          // input convolution and every block of the tower in one launch (gemm_tc.cu, tower kernel)
          launches++;
          double flops = 2.0 * R * (double)C * 9 * 112;
          for (const auto& r : res) flops += 2.0 * R * (double)C * 9 * (r.c1.cin + r.c2.cin);
          const int sp_ = span_begin(st, K_GEMM_TC, flops);
          CK(launch_gemm_tower<T>(s.tower_layers, s.tower_n, C, (n + 1) / 2, t_status, sm_count, st));
          span_end(st, sp_);
          if (res.size() & 1) cur = s.y;  // the blocks' outputs alternate between y and x
          in_one = true;
        }
      }
      if (!in_one) conv3(st, s.tokens, conv_in, conv_in.b, s.x, n, act_default);
      for (const auto& r : res) {
        if (in_one) break;
        conv3(st, cur, r.c1, r.c1.b, tmp, n, act_default);
        if (winograd && conv3_wino(st, tmp, r.c2, r.c2.b, tmp2, n, act_default, cur, r.se ? &r : nullptr)) {
          std::swap(cur, tmp2);  // output transform with SE / skip / activation
          continue;
        }
        if (r.se && conv3_se(st, tmp, r, cur, tmp2, n)) {  // second convolution, SE, skip and activation in one launch
          std::swap(cur, tmp2);
          continue;
        }
        conv3(st, tmp, r.c2, nullptr, tmp2, n, ACT_NONE);
        other(st, 3.0 * R * C * sizeof(T), [&] {
          return r.se ? launch_se<T>(tmp2, r.c2.b, cur, r.se_w1, r.se_b1, r.se_w2, r.se_b2, tmp, C, r.se_k, n,
                                     act_default, st)
                      : launch_bias_skip_act<T>(tmp2, r.c2.b, cur, tmp, C, R, act_default, st);
        });
        std::swap(cur, tmp);
      }
      flow = cur;
      body_ch = C;
    }
    if (attn_body) {  // network_blas.cc:603-721
      if (emb_fmt == EMB_PE_DENSE) {
        other(st, (double)n * 768 * sizeof(T), [&] { return launch_expand_pre12<T>(d_masks, d_values, n, s.pre, st); });
        gemm(st, s.pre, 768, emb_pre, s.pe, 64 * pe_ch, n, ACT_NONE);
        other(st, (double)R * (cin + pe_ch) * sizeof(T), [&] {
          return launch_expand_tokens<T>(d_masks, d_values, n, nullptr, s.pe, pe_ch, cin, s.tokens, st);
        });
      } else {
        other(st, (double)R * cin * sizeof(T), [&] {
          return launch_expand_tokens<T>(d_masks, d_values, n, pos_enc, (const T*)nullptr, pe_ch, cin, s.tokens, st);
        });
      }
      T *x = s.x, *x1 = s.x1;
      t_tag = TAG_EMBEDDING;
      gemm(st, s.tokens, cin, emb, x, E, R, act_default);
      if (emb_fmt == EMB_PE_DENSE) {
        ln(st, x, x, nullptr, emb_lng, emb_lnb, R, E, 1.f, 1e-3f, gate_mult, gate_add);
        gemm(st, x, E, emb_ffn1, s.ffn, emb_dff, R, act_ffn);
        if (fold_emb_ln) {
          // u = alpha * ffn2 + x with row statistics; the first layer reads LN(u) through its folded products.  The
          // statistics live in the stats2 buffer that the first layer does not write.
          LNState ffn{s.ffn, nullptr, nullptr, nullptr}, skip{x, nullptr, nullptr, nullptr};
          gemm_ln(st, ffn, emb_dff, emb_ffn2, x1, E, R, ACT_NONE, &skip, alpha, s.stats2[1]);
          std::swap(x, x1);
          body_in = LNState{x, s.stats2[1], emb_ffn_lng, emb_ffn_lnb};
        } else {
          gemm(st, s.ffn, emb_dff, emb_ffn2, s.y, E, R, ACT_NONE);
          ln(st, x1, s.y, x, emb_ffn_lng, emb_ffn_lnb, R, E, alpha, 1e-3f);
          std::swap(x, x1);
          body_in = LNState{x, nullptr, nullptr, nullptr};
        }
      } else {
        if (gate_mult)
          other(st, 2.0 * R * E * sizeof(T), [&] { return launch_gate<T>(x, gate_mult, gate_add, R, E, st); });
        body_in = LNState{x, nullptr, nullptr, nullptr};
      }
      t_tag = TAG_NONE;
      for (const auto& e : enc) encoder_layer(s, e, n, x, x1, body_in);
      if (body_in.stats && !fold_heads) {  // materialise the last LayerNorm for heads that cannot fold it
        ln(st, x1, x, nullptr, body_in.gamma, body_in.beta, R, E, 1.f, ln_eps);
        std::swap(x, x1);
        body_in = LNState{x, nullptr, nullptr, nullptr};
      }
      flow = x;
      body_ch = E;
    }

    // ---- value head (network_blas.cc:725-772) ----
    LNState head_in = attn_body ? body_in : LNState{flow, nullptr, nullptr, nullptr};
    t_tag = TAG_HEADS;
    // The value and moves-left heads do not depend on the policy head: at small batches, where their products are a
    // few tiles of latency each, they run on the side stream beside it (fork here, join after the policy head).
    const bool heads_beside = heads_side && !profiling && n <= heads_side_max;
    cudaStream_t hs = heads_beside ? s.stream2 : st;
    if (heads_beside) {
      CK(cudaEventRecord(s.ev_fork, st));
      CK(cudaStreamWaitEvent(hs, s.ev_fork, 0));
    }
    {
      DependentLaunchScope first(heads_beside ? false : t_dependent_launch);  // ordinary launch behind the event
      gemm_ln(hs, head_in, body_ch, val_emb, s.vtok, val_emb.out, R, act_default);
    }
    gemm(hs, s.vtok, 64 * val_emb.out, val_fc1, s.vhid, val_fc1.out, n, act_default);
    other(hs, (double)n * val_fc1.out * sizeof(T), [&] {
      return launch_head_final<T>(s.vhid, val_fc1.out, val_w2, val_b2, wdl ? 0 : 1, n, d_qdm, hs);
    });
    // ---- moves-left head (:775-803) ----
    if (mlh) {
      gemm_ln(hs, head_in, body_ch, mov_emb, s.mtok, mov_emb.out, R, act_default);
      gemm(hs, s.mtok, 64 * mov_emb.out, mov_fc1, s.mhid, mov_fc1.out, n, act_default);
      other(hs, (double)n * mov_fc1.out * sizeof(T), [&] {
        return launch_head_final<T>(s.mhid, mov_fc1.out, mov_w2, mov_b2, 2, n, d_qdm, hs);
      });
    }
    // ---- policy head (:806-968) ----
    if (policy_fmt == POLICY_ATTENTION) {
      gemm_ln(st, head_in, body_ch, pol_emb, s.pemb, pol_emb.out, R, attn_body ? act_default : ACT_SELU);
      for (const auto& e : pol_enc) policy_encoder_layer(s, e, n, s.pemb);
      gemm(st, s.pemb, pol_emb.out, pol_q, s.pq, pol_dm, R, ACT_NONE);
      gemm(st, s.pemb, pol_emb.out, pol_k, s.pk, pol_dm, R, ACT_NONE);
      bool done = false;
      if constexpr (sizeof(T) == 2) {
        if (use_tc && policy_attn_tc_supported(pol_dm, s.pq, s.pk)) {
          launches++;
          const int sp_ = span_begin(st, K_OTHER, 2.0 * R * pol_dm * sizeof(T) + (double)n * 1858 * 4);
          CK(launch_policy_attn_tc<T>(s.pq, s.pk, pol_w4, pol_dm, d_attn_src, n, d_policy, st));
          span_end(st, sp_);
          done = true;
        }
      }
      if (!done) {
        GemmParams p;  // per-position Q.K^T, scaled
        p.A = s.pq; p.lda = pol_dm; p.strideA = 64LL * pol_dm;
        p.W = s.pk; p.ldw = pol_dm; p.strideW = 64LL * pol_dm;
        p.C = s.logits; p.ldc = 64; p.strideC = 4096; p.out_f32 = true;
        p.M = 64; p.N = 64; p.K = pol_dm; p.batch = n; p.scale = 1.0f / sqrtf((float)pol_dm);
        run_gemm(st, p);
        other(st, (double)n * (4096 + 1858) * 4, [&] {
          return launch_policy_attn_gather<T>(s.logits, s.pk, pol_w4, pol_dm, d_attn_src, n, d_policy, st);
        });
      }
    } else if (policy_fmt == POLICY_CONVOLUTION) {
      T* t1 = flow == s.y ? s.x : s.y;  // any tower buffer that does not hold the tower's output
      conv3(st, flow, pol_conv1, pol_conv1.b, t1, n, act_default);
      conv3(st, t1, pol_conv2, pol_conv2.b, s.praw, n, ACT_NONE);
      other(st, (double)n * 1858 * (4 + sizeof(T)), [&] {
        return launch_policy_gather<T>(s.praw, 64LL * pol_planes, d_conv_src, n, d_policy, st);
      });
    } else {
      gemm(st, flow, C, pol_c1x1, s.praw, pol_planes, R, act_default);
      gemm(st, s.praw, 64 * pol_planes, pol_fc, nullptr, 1858, n, ACT_NONE, nullptr, 0, 1.f, true, d_policy);
    }
    if (heads_beside) {
      CK(cudaEventRecord(s.ev_join, hs));
      CK(cudaStreamWaitEvent(st, s.ev_join, 0));
    }
    t_tag = TAG_NONE;
  }

  // ---- CUDA graphs: the launch sequence of one evaluation is captured per (batch size, buffers) the second
  // time it is requested and replayed afterwards (the reference captures per batch size too,
  // backends/cuda/network_cuda.cc:690-706).  Profiling needs event records between kernels, so it bypasses graphs.
  struct GraphKey {
    int n, staged;
    const void *a, *b, *c, *d;
    bool operator<(const GraphKey& o) const {
      return std::tie(n, staged, a, b, c, d) < std::tie(o.n, o.staged, o.a, o.b, o.c, o.d);
    }
  };
  struct GraphEntry {
    int seen = 0;
    cudaGraphExec_t exec = nullptr;
    long long launches = 0;
  };
  std::vector<std::map<GraphKey, GraphEntry>> graph_cache;  // per slot

  void enqueue_staged(Slot& s, HostSet& hs, int n, int policy_mode, float inv_t, int enc_format, int enc_fill) {
    if (enc_format > 0) {
      // the histories were copied ahead of this (their size varies from call to call, a captured copy could not)
      other(s.stream, (double)n * 112 * 12, [&] {
        return launch_encode_positions(s.d_boards, s.d_offsets, s.d_from_start, n, enc_format, enc_fill, s.d_masks,
                                       s.d_values, nullptr, s.stream);
      });
    } else {
      CK(cudaMemcpyAsync(s.d_masks, hs.masks, (size_t)n * 112 * 8, cudaMemcpyHostToDevice, s.stream));
      CK(cudaMemcpyAsync(s.d_values, hs.values, (size_t)n * 112 * 4, cudaMemcpyHostToDevice, s.stream));
    }
    if (policy_mode) {
      CK(cudaMemcpyAsync(s.d_move_ids, hs.move_ids, (size_t)n * kLegalStride * 2, cudaMemcpyHostToDevice, s.stream));
      CK(cudaMemcpyAsync(s.d_n_moves, hs.n_moves, (size_t)n * 4, cudaMemcpyHostToDevice, s.stream));
    }
    // Evaluations of different slots take turns on the GPU: the kernels of this one start after the kernels of the
    // others (as of their latest launch), while its input copies above and their result copies overlap with the
    // other's kernels.  Interleaving the kernels of two batches was slower than running the batches one at a time.
    // Inside a stream capture the waits and the record become external event nodes.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CK(cudaStreamIsCapturing(s.stream, &cap));
    const bool capturing = cap == cudaStreamCaptureStatusActive;
    for (auto& o : slots)
      if (&o != &s) CK(cudaStreamWaitEvent(s.stream, o.compute_done, capturing ? cudaEventWaitExternal : 0));
    forward(s, s.d_masks, s.d_values, n, s.d_policy, s.d_qdm);
    if (policy_mode) {
      other(s.stream, (double)n * kLegalStride * 6, [&] {
        return launch_legal_softmax(s.d_policy, s.d_move_ids, s.d_n_moves, n, inv_t, s.d_probs, s.stream);
      });
    }
    CK(cudaEventRecordWithFlags(s.compute_done, s.stream, capturing ? cudaEventRecordExternal : 0));
    if (policy_mode) {
      CK(cudaMemcpyAsync(hs.probs, s.d_probs, (size_t)n * kLegalStride * 4, cudaMemcpyDeviceToHost, s.stream));
    }
    if (policy_mode != 2)
      CK(cudaMemcpyAsync(hs.policy, s.d_policy, (size_t)n * 1858 * 4, cudaMemcpyDeviceToHost, s.stream));
    CK(cudaMemcpyAsync(hs.qdm, s.d_qdm, (size_t)n * 3 * 4, cudaMemcpyDeviceToHost, s.stream));
    copy_status(s);
  }
  // The slot's status word follows the results to the host (inside a captured graph too), so that an evaluation
  // whose kernels gave up on a bounded wait is reported by the call that ran it.
  void copy_status(Slot& s) {
    CK(cudaMemcpyAsync(s.h_status, d_status + (&s - slots.data()), sizeof(int), cudaMemcpyDeviceToHost, s.stream));
  }
  // After the stream has been synchronised: B200_ERR_TIMEOUT if a kernel of this slot gave up; the word is cleared so
  // that the next evaluation starts clean.
  void check_status(Slot& s) {
    const int code = *s.h_status;
    if (!code) return;
    *s.h_status = 0;
    CK(cudaMemsetAsync(d_status + (&s - slots.data()), 0, sizeof(int), s.stream));
    CK(cudaStreamSynchronize(s.stream));
    throw Fail{B200_ERR_TIMEOUT, "a bounded device-side wait gave up (kernel status " + std::to_string(code) +
                                     "); the results of this evaluation are not valid"};
  }

  template <typename F>
  void run_or_replay(int slot, const GraphKey& key, F&& enqueue) {
    Slot& s = slots[slot];
    const bool use_graphs = !(opt.flags & B200_FLAG_NO_GRAPHS) && !profiling;
    if (!use_graphs) {
      enqueue();
      return;
    }
    auto& cache = graph_cache[slot];
    auto it = cache.find(key);
    if (it == cache.end()) {
      if (cache.size() >= 64) {  // bounded: beyond that, new shapes simply run eagerly
        enqueue();
        return;
      }
      it = cache.emplace(key, GraphEntry{}).first;
    }
    GraphEntry& e = it->second;
    if (e.exec) {
      CK(cudaGraphLaunch(e.exec, s.stream));
      launches += e.launches;
      return;
    }
    if (++e.seen < 2) {  // first request: plain launches (also performs every one-time attribute set-up)
      enqueue();
      return;
    }
    const long long before = launches.load();
    CK(cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeThreadLocal));
    cudaGraph_t graph = nullptr;
    try {
      enqueue();
    } catch (...) {
      cudaStreamEndCapture(s.stream, &graph);
      if (graph) cudaGraphDestroy(graph);
      throw;
    }
    CK(cudaStreamEndCapture(s.stream, &graph));
    cudaGraphExec_t exec = nullptr;
    cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
      cudaGetLastError();
      e.seen = -1000000;  // do not try again
      launches = before;
      enqueue();
      return;
    }
    e.exec = exec;
    e.launches = launches.load() - before;
    launches = before;
    CK(cudaGraphLaunch(e.exec, s.stream));
    launches += e.launches;
  }

  int eval_device(int slot, const void* d_masks, const void* d_values, int n, void* d_policy, void* d_qdm,
                  bool sync) override {
    Slot& s = slots[slot];
    run_or_replay(slot, GraphKey{n, 0, d_masks, d_values, d_policy, d_qdm}, [&] {
      forward(s, (const uint64_t*)d_masks, (const float*)d_values, n, (float*)d_policy, (float*)d_qdm);
      copy_status(s);
    });
    if (sync) {
      CK(cudaStreamSynchronize(s.stream));
      check_status(s);
    }
    return B200_OK;
  }
  int eval_staged(int slot, HostSet& hs, int n, int policy_mode, float inv_t, int enc_format, int enc_fill,
                  int n_boards) override {
    Slot& s = slots[slot];
    if (enc_format > 0) {
      CK(cudaMemcpyAsync(s.d_boards, hs.boards, (size_t)n_boards * sizeof(b200_board), cudaMemcpyHostToDevice, s.stream));
      CK(cudaMemcpyAsync(s.d_offsets, hs.offsets, (size_t)(n + 1) * sizeof(int), cudaMemcpyHostToDevice, s.stream));
      CK(cudaMemcpyAsync(s.d_from_start, hs.from_start, (size_t)n, cudaMemcpyHostToDevice, s.stream));
    }
    // The captured copy nodes embed the host set's addresses and the softmax launch its temperature, so each
    // (host set, policy mode, temperature) gets its own graph; the temperature's bits ride in a pointer field.
    uint32_t tbits;
    memcpy(&tbits, &inv_t, 4);
    const int enc_code = enc_format > 0 ? enc_format * 4 + enc_fill : 0;  // below 1024
    run_or_replay(slot,
                  GraphKey{n, (hs.id * 4 + policy_mode) * 1024 + enc_code, nullptr, nullptr, nullptr,
                           (const void*)(uintptr_t)tbits},
                  [&] { enqueue_staged(s, hs, n, policy_mode, inv_t, enc_format, enc_fill); });
    CK(cudaStreamSynchronize(s.stream));
    check_status(s);
    return B200_OK;
  }
  cudaStream_t stream(int slot) override { return slots[slot].stream; }
  int device_status() override {
    int v[64] = {0};
    cudaMemcpy(v, d_status, sizeof(v), cudaMemcpyDeviceToHost);
    for (int i = 0; i < 64; ++i)
      if (v[i]) return v[i];
    return 0;
  }
  int sync_slot(int slot) override {
    Slot& s = slots[slot];
    CK(cudaStreamSynchronize(s.stream));
    check_status(s);
    return B200_OK;
  }
  void inject_status(int code) override {
    int v[64];
    for (int i = 0; i < 64; ++i) v[i] = code;
    CK(cudaMemcpy(d_status, v, sizeof(v), cudaMemcpyHostToDevice));
  }
};

}  // namespace b200

struct b200_net {
  // Shared with the computations created from it: a computation that is destroyed after b200_net_destroy keeps
  // the network's resources alive until it is gone too (lc0 never does this, garbage-collected hosts may).
  std::shared_ptr<NetBase> impl;
};

// A computation owns host copies of its inputs and, after compute, of its outputs; the device
// workspace slot is held only while computing.
struct b200_comp {
  std::shared_ptr<NetBase> net;
  NetBase::HostSet* hs = nullptr;  // pinned staging, taken from the network's pool at the first AddInput
  int n = 0;
  int with_moves = 0;    // inputs added together with their legal moves
  bool compact = false;  // return only legal-move probabilities (no 1858-logit vectors)
  float inv_temperature = 1.0f;
  bool computed = false;
  // device-side position encoding
  int positions = 0;     // inputs added by their history
  int n_boards = 0;      // records staged
  int enc_format = 0;    // 0: the network's input format
  int enc_fill = B200_FILL_FEN_ONLY;
};

template <typename F>
static int guarded(F&& f) {
  try {
    return f();
  } catch (const Fail& e) {
    set_error(e.msg);
    return e.code;
  } catch (const std::bad_alloc&) {
    set_error("out of host memory");
    return B200_ERR_NOMEM;
  } catch (const std::exception& e) {
    set_error(e.what());
    return B200_ERR_INVALID;
  }
}

template <typename F32, typename F16, typename BF16>
static int by_precision(int precision, F32&& f32, F16&& f16, BF16&& bf16) {
  if (precision == B200_PREC_FP32) return f32();
  if (precision == B200_PREC_FP16) return f16();
  if (precision == B200_PREC_BF16) return bf16();
  set_error("unknown precision");
  return B200_ERR_INVALID;
}

extern "C" {

const char* b200_last_error(void) { return g_last_error.c_str(); }

int b200_builder_create(b200_builder** out) {
  if (!out) return B200_ERR_INVALID;
  *out = new b200_builder();
  return B200_OK;
}
int b200_builder_set_int(b200_builder* b, const char* key, long long value) {
  if (!b || !key) return B200_ERR_INVALID;
  b->ints[key] = value;
  return B200_OK;
}
int b200_builder_add_tensor(b200_builder* b, const char* name, const float* data, size_t count) {
  if (!b || !name || (!data && count)) {
    set_error("b200_builder_add_tensor: null argument");
    return B200_ERR_INVALID;
  }
  return guarded([&] {
    b->tensors[name].assign(data, data + count);
    return B200_OK;
  });
}
void b200_builder_destroy(b200_builder* b) { delete b; }

int b200_net_create(const b200_builder* b, const b200_net_options* opt, b200_net** out) {
  if (!b || !opt || !out) {
    set_error("b200_net_create: null argument");
    return B200_ERR_INVALID;
  }
  *out = nullptr;
  return guarded([&] {
    b200_net_options o = *opt;
    if (o.max_batch <= 0) o.max_batch = 1024;
    if (o.slots <= 0) o.slots = 1;
    if (o.max_batch > 65536) throw Fail{B200_ERR_INVALID, "max_batch too large (limit 65536)"};
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
      throw Fail{B200_ERR_CUDA, std::string("no usable CUDA device: ") + cudaGetErrorString(e)};
    if (o.gpu < 0 || o.gpu >= ndev)
      throw Fail{B200_ERR_INVALID, "Invalid GPU Id: " + std::to_string(o.gpu)};
    std::unique_ptr<NetBase> impl;
    if (o.precision == B200_PREC_FP32) {
      auto n = std::make_unique<Net<float>>();
      n->build(b, o);
      impl = std::move(n);
    } else if (o.precision == B200_PREC_FP16) {
      auto n = std::make_unique<Net<__half>>();
      n->build(b, o);
      impl = std::move(n);
    } else if (o.precision == B200_PREC_BF16) {
      auto n = std::make_unique<Net<__nv_bfloat16>>();
      n->build(b, o);
      impl = std::move(n);
    } else {
      throw Fail{B200_ERR_INVALID, "unknown precision " + std::to_string(o.precision)};
    }
    *out = new b200_net{std::shared_ptr<NetBase>(std::move(impl))};
    return B200_OK;
  });
}
int b200_net_get_info(const b200_net* net, b200_net_info* info) {
  if (!net || !info) return B200_ERR_INVALID;
  *info = net->impl->info;
  return B200_OK;
}
void b200_net_destroy(b200_net* net) {
  if (!net) return;
  cudaSetDevice(net->impl->opt.gpu);
  delete net;
}

int b200_comp_create(b200_net* net, b200_comp** out) {
  if (!net || !out) return B200_ERR_INVALID;
  return guarded([&] {
    *out = new b200_comp();
    (*out)->net = net->impl;
    return B200_OK;
  });
}
int b200_comp_add_inputs(b200_comp* c, const uint64_t* masks, const float* values, int n) {
  if (!c || !masks || !values || n < 0) return B200_ERR_INVALID;
  return guarded([&] {
    if (c->n + n > c->net->opt.max_batch)
      throw Fail{B200_ERR_INVALID, "computation exceeds max_batch=" + std::to_string(c->net->opt.max_batch)};
    if (n == 0) return (int)B200_OK;
    if (c->positions) throw Fail{B200_ERR_INVALID, "a computation takes either planes or position histories, not both"};
    if (!c->hs) c->hs = c->net->acquire_host();
    memcpy(c->hs->masks + (size_t)c->n * 112, masks, (size_t)n * 112 * 8);
    memcpy(c->hs->values + (size_t)c->n * 112, values, (size_t)n * 112 * 4);
    for (int i = 0; i < n; ++i) c->hs->n_moves[c->n + i] = 0;
    c->n += n;
    return (int)B200_OK;
  });
}
int b200_comp_add_input(b200_comp* c, const uint64_t* masks, const float* values) {
  return b200_comp_add_inputs(c, masks, values, 1);
}
int b200_comp_compute(b200_comp* c) {
  if (!c) return B200_ERR_INVALID;
  return guarded([&] {
    NetBase* nb = c->net.get();
    if (c->n == 0) {
      c->computed = true;
      return (int)B200_OK;
    }
    CK(cudaSetDevice(nb->opt.gpu));
    const int slot = nb->acquire();
    int rc;
    try {
      const int mode = c->with_moves ? (c->compact ? 2 : 1) : 0;
      if (c->positions) {
        const int fmt = c->enc_format ? c->enc_format : nb->info.input_format;
        rc = nb->eval_staged(slot, *c->hs, c->n, mode, c->inv_temperature, fmt, c->enc_fill, c->n_boards);
      } else {
        rc = nb->eval_staged(slot, *c->hs, c->n, mode, c->inv_temperature);
      }
    } catch (...) {
      nb->release(slot);
      throw;
    }
    nb->release(slot);
    c->computed = rc == B200_OK;
    return rc;
  });
}
int b200_comp_batch_size(const b200_comp* c) { return c ? c->n : 0; }
// Accessors are valid after b200_comp_compute for 0 <= sample < batch size.
float b200_comp_q(const b200_comp* c, int s) { return c->hs->qdm[(size_t)s * 3 + 0]; }
float b200_comp_d(const b200_comp* c, int s) { return c->hs->qdm[(size_t)s * 3 + 1]; }
float b200_comp_m(const b200_comp* c, int s) { return c->hs->qdm[(size_t)s * 3 + 2]; }
float b200_comp_p(const b200_comp* c, int s, int move_id) { return c->hs->policy[(size_t)s * 1858 + move_id]; }
const float* b200_comp_policy(const b200_comp* c, int s) { return c->hs->policy + (size_t)s * 1858; }
int b200_comp_add_input_with_moves(b200_comp* c, const uint64_t* masks, const float* values,
                                   const uint16_t* move_ids, int n_moves) {
  if (!c || !move_ids || n_moves < 0 || n_moves > kLegalStride) {
    set_error("b200_comp_add_input_with_moves: bad argument (at most 256 legal moves per position)");
    return B200_ERR_INVALID;
  }
  for (int i = 0; i < n_moves; ++i)
    if (move_ids[i] >= 1858) {
      set_error("b200_comp_add_input_with_moves: policy index out of range");
      return B200_ERR_INVALID;
    }
  const int rc = b200_comp_add_inputs(c, masks, values, 1);
  if (rc != B200_OK) return rc;
  const int idx = c->n - 1;
  memcpy(c->hs->move_ids + (size_t)idx * kLegalStride, move_ids, (size_t)n_moves * 2);
  c->hs->n_moves[idx] = n_moves;
  c->with_moves++;
  return B200_OK;
}
int b200_comp_add_inputs_with_moves(b200_comp* c, const uint64_t* masks, const float* values,
                                    const uint16_t* move_ids, const int* n_moves, int n) {
  if (!c || !masks || !values || !move_ids || !n_moves || n < 0) return B200_ERR_INVALID;
  for (int i = 0; i < n; ++i) {
    const int rc = b200_comp_add_input_with_moves(c, masks + (size_t)i * 112, values + (size_t)i * 112,
                                                  move_ids + (size_t)i * kLegalStride, n_moves[i]);
    if (rc != B200_OK) return rc;
  }
  return B200_OK;
}
int b200_comp_set_encoding(b200_comp* c, int input_format, int fill_empty_history) {
  if (!c || fill_empty_history < B200_FILL_NO || fill_empty_history > B200_FILL_ALWAYS ||
      (input_format != 0 && !encode_format_supported(input_format))) {
    set_error("b200_comp_set_encoding: unsupported input format or fill policy");
    return B200_ERR_INVALID;
  }
  c->enc_format = input_format;
  c->enc_fill = fill_empty_history;
  return B200_OK;
}
int b200_comp_add_position(b200_comp* c, const b200_board* history, int count, int from_start,
                           const uint16_t* move_ids, int n_moves) {
  if (!c || !history || count < 1 || count > B200_MAX_HISTORY || n_moves > kLegalStride || (n_moves > 0 && !move_ids)) {
    set_error("b200_comp_add_position: bad argument (1..128 history entries, at most 256 legal moves)");
    return B200_ERR_INVALID;
  }
  for (int i = 0; i < n_moves; ++i)
    if (move_ids[i] >= 1858) {
      set_error("b200_comp_add_position: policy index out of range");
      return B200_ERR_INVALID;
    }
  return guarded([&] {
    NetBase* nb = c->net.get();
    if (c->n != c->positions)
      throw Fail{B200_ERR_INVALID, "a computation takes either planes or position histories, not both"};
    if (c->n + 1 > nb->opt.max_batch)
      throw Fail{B200_ERR_INVALID, "computation exceeds max_batch=" + std::to_string(nb->opt.max_batch)};
    if (!encode_format_supported(c->enc_format ? c->enc_format : nb->info.input_format))
      throw Fail{B200_ERR_UNSUPPORTED, "the network's input format has no device-side encoder"};
    if (!c->hs) c->hs = nb->acquire_host();
    nb->ensure_board_staging(*c->hs);
    if ((size_t)c->n_boards + count > nb->board_capacity())
      throw Fail{B200_ERR_INVALID, "position histories exceed the staging capacity of a computation (" +
                                       std::to_string(nb->board_capacity()) + " boards); add planes instead"};
    if (c->n == 0) c->hs->offsets[0] = 0;
    memcpy(c->hs->boards + c->n_boards, history, (size_t)count * sizeof(b200_board));
    c->n_boards += count;
    c->hs->offsets[c->n + 1] = c->n_boards;
    c->hs->from_start[c->n] = from_start ? 1 : 0;
    if (n_moves >= 0) {
      if (c->with_moves != c->n) throw Fail{B200_ERR_INVALID, "either every position of a computation has a move list or none"};
      if (n_moves > 0) memcpy(c->hs->move_ids + (size_t)c->n * kLegalStride, move_ids, (size_t)n_moves * 2);
      c->hs->n_moves[c->n] = n_moves;
      c->with_moves++;
    } else {
      c->hs->n_moves[c->n] = 0;
    }
    c->n++;
    c->positions++;
    return (int)B200_OK;
  });
}
int b200_comp_add_positions(b200_comp* c, const b200_board* boards, const int* offsets, const uint8_t* from_start,
                            const uint16_t* move_ids, const int* n_moves, int n) {
  if (!c || n < 0 || (n > 0 && (!boards || !offsets || !from_start)) || ((move_ids == nullptr) != (n_moves == nullptr))) {
    set_error("b200_comp_add_positions: bad argument");
    return B200_ERR_INVALID;
  }
  for (int i = 0; i < n; ++i) {
    const int rc = b200_comp_add_position(c, boards + offsets[i], offsets[i + 1] - offsets[i], from_start[i],
                                          move_ids ? move_ids + (size_t)i * kLegalStride : nullptr,
                                          n_moves ? n_moves[i] : -1);
    if (rc != B200_OK) return rc;
  }
  return B200_OK;
}
int b200_comp_set_policy_options(b200_comp* c, float inv_temperature, int compact) {
  if (!c || !(inv_temperature > 0.f)) return B200_ERR_INVALID;
  c->inv_temperature = inv_temperature;
  c->compact = compact != 0;
  return B200_OK;
}
int b200_comp_legal_policy(const b200_comp* c, int sample, const float** probs, int* n_moves) {
  if (!c || !probs || !n_moves || !c->computed || !c->with_moves || sample < 0 || sample >= c->n) return B200_ERR_INVALID;
  *probs = c->hs->probs + (size_t)sample * kLegalStride;
  *n_moves = c->hs->n_moves[sample];
  return B200_OK;
}
void b200_comp_destroy(b200_comp* c) {
  if (!c) return;
  if (c->hs) c->net->release_host(c->hs);
  if (c->net.use_count() == 1) cudaSetDevice(c->net->opt.gpu);  // this computation frees the network's device memory
  delete c;
}

int b200_net_eval_host(b200_net* net, const uint64_t* masks, const float* values, int n, float* policy,
                       float* q, float* d, float* m) {
  if (!net || n < 0 || (n > 0 && (!masks || !values))) return B200_ERR_INVALID;
  return guarded([&] {
    NetBase* nb = net->impl.get();
    if (n > nb->opt.max_batch)
      throw Fail{B200_ERR_INVALID, "batch " + std::to_string(n) + " exceeds max_batch=" + std::to_string(nb->opt.max_batch)};
    if (n == 0) return (int)B200_OK;
    CK(cudaSetDevice(nb->opt.gpu));
    NetBase::HostSet* hs = nb->acquire_host();
    memcpy(hs->masks, masks, (size_t)n * 112 * 8);
    memcpy(hs->values, values, (size_t)n * 112 * 4);
    const int slot = nb->acquire();
    int rc;
    try {
      rc = nb->eval_staged(slot, *hs, n, 0, 1.0f);
      if (rc == B200_OK) {
        if (policy) memcpy(policy, hs->policy, (size_t)n * 1858 * 4);
        for (int i = 0; i < n; ++i) {
          if (q) q[i] = hs->qdm[i * 3];
          if (d) d[i] = hs->qdm[i * 3 + 1];
          if (m) m[i] = hs->qdm[i * 3 + 2];
        }
      }
    } catch (...) {
      nb->release(slot);
      nb->release_host(hs);
      throw;
    }
    nb->release(slot);
    nb->release_host(hs);
    return rc;
  });
}

static int eval_dev(b200_net* net, const void* d_masks, const void* d_values, int n, void* d_policy, void* d_qdm,
                    bool sync) {
  if (!net || n < 0 || (n > 0 && (!d_masks || !d_values || !d_policy || !d_qdm))) return B200_ERR_INVALID;
  return guarded([&] {
    NetBase* nb = net->impl.get();
    if (n > nb->opt.max_batch)
      throw Fail{B200_ERR_INVALID, "batch " + std::to_string(n) + " exceeds max_batch=" + std::to_string(nb->opt.max_batch)};
    if (n == 0) return (int)B200_OK;
    CK(cudaSetDevice(nb->opt.gpu));
    nb->hold_slot0();
    if (!sync) return nb->eval_device(0, d_masks, d_values, n, d_policy, d_qdm, false);
    int rc;
    try {
      rc = nb->eval_device(0, d_masks, d_values, n, d_policy, d_qdm, true);
    } catch (...) {
      nb->unhold_slot0();
      throw;
    }
    nb->unhold_slot0();
    return rc;
  });
}
int b200_net_eval_device(b200_net* net, const void* d_masks, const void* d_values, int n, void* d_policy,
                         void* d_qdm) {
  return eval_dev(net, d_masks, d_values, n, d_policy, d_qdm, true);
}
int b200_net_enqueue_device(b200_net* net, const void* d_masks, const void* d_values, int n, void* d_policy,
                            void* d_qdm) {
  return eval_dev(net, d_masks, d_values, n, d_policy, d_qdm, false);
}
int b200_net_sync(b200_net* net) {
  if (!net) return B200_ERR_INVALID;
  return guarded([&] {
    NetBase* nb = net->impl.get();
    CK(cudaSetDevice(nb->opt.gpu));
    int rc;
    try {
      rc = nb->sync_slot(0);
    } catch (...) {
      nb->unhold_slot0();
      throw;
    }
    nb->unhold_slot0();
    return rc;
  });
}
void* b200_net_stream(b200_net* net) { return net ? (void*)net->impl->stream(0) : nullptr; }
long long b200_net_launch_count(const b200_net* net) { return net ? net->impl->launches.load() : 0; }
int b200_net_device_status(b200_net* net) { return net ? net->impl->device_status() : 0; }
int b200_net_inject_device_status(b200_net* net, int code) {
  if (!net) return B200_ERR_INVALID;
  return guarded([&] {
    CK(cudaSetDevice(net->impl->opt.gpu));
    net->impl->inject_status(code);
    return (int)B200_OK;
  });
}

int b200_net_set_profiling(b200_net* net, int enabled) {
  if (!net) return B200_ERR_INVALID;
  net->impl->collect_spans();
  net->impl->profiling = enabled != 0;
  return B200_OK;
}
int b200_net_get_profile(b200_net* net, double* ms, double* work, long long* launches, int reset) {
  if (!net || !ms || !work || !launches) return B200_ERR_INVALID;
  NetBase* nb = net->impl.get();
  cudaSetDevice(nb->opt.gpu);
  nb->collect_spans();
  for (int i = 0; i < NetBase::K_CLASSES; ++i) {
    ms[i] = nb->prof_ms[i];
    work[i] = nb->prof_work[i];
    launches[i] = nb->prof_launches[i];
    if (reset) {
      nb->prof_ms[i] = 0;
      nb->prof_work[i] = 0;
      nb->prof_launches[i] = 0;
    }
  }
  return B200_OK;
}

int b200_net_get_profile_tagged(b200_net* net, double* ms, double* work, long long* launches, int reset) {
  if (!net || !ms || !work || !launches) return B200_ERR_INVALID;
  NetBase* nb = net->impl.get();
  cudaSetDevice(nb->opt.gpu);
  nb->collect_spans();
  std::lock_guard<std::mutex> l(nb->prof_mu);
  for (int i = 0; i < NetBase::K_TAGS; ++i) {
    ms[i] = nb->tag_ms[i];
    work[i] = nb->tag_work[i];
    launches[i] = nb->tag_launches[i];
    if (reset) {
      nb->tag_ms[i] = 0;
      nb->tag_work[i] = 0;
      nb->tag_launches[i] = 0;
    }
  }
  return B200_OK;
}

// ---- stand-alone operators ----------------------------------------------------------------------
int b200_op_expand_planes(const void* d_masks, const void* d_values, int n, void* d_out, int precision,
                          void* stream) {
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    B200_CUDA(launch_expand_planes<T>((const uint64_t*)d_masks, (const float*)d_values, n, (T*)d_out,
                                      (cudaStream_t)stream));
    return B200_OK;
  };
  return by_precision(precision, [&] { return run(float()); }, [&] { return run(__half()); },
                      [&] { return run(__nv_bfloat16()); });
}

int b200_op_gemm(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int activation,
                 int precision, int use_tc, void* stream) {
  GemmParams p;
  p.A = A; p.lda = K; p.W = W; p.ldw = K; p.bias = bias; p.C = C; p.ldc = N;
  p.M = M; p.N = N; p.K = K; p.act = activation;
  if (use_tc) {
    if (precision == B200_PREC_FP32 || !gemm_tc_supported(p)) {
      set_error("b200_op_gemm: shape or precision not supported by the tensor-core kernel");
      return B200_ERR_UNSUPPORTED;
    }
    B200_CUDA(gemm_tc_init());
    int dev = 0, sms = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static int* status = nullptr;  // one status word per process for the stand-alone operator
    if (!status) {
      B200_CUDA(cudaMalloc(&status, sizeof(int)));
      B200_CUDA(cudaMemset(status, 0, sizeof(int)));
    }
    if (precision == B200_PREC_FP16) B200_CUDA(launch_gemm_tc<__half>(p, status, sms, (cudaStream_t)stream));
    else B200_CUDA(launch_gemm_tc<__nv_bfloat16>(p, status, sms, (cudaStream_t)stream));
    B200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int st = 0;
    B200_CUDA(cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st) {
      cudaMemset(status, 0, sizeof(int));
      set_error("tensor-core GEMM: a bounded device-side wait gave up, status " + std::to_string(st));
      return B200_ERR_TIMEOUT;
    }
    return B200_OK;
  }
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    B200_CUDA(launch_gemm_simt<T>(p, (cudaStream_t)stream));
    return B200_OK;
  };
  return by_precision(precision, [&] { return run(float()); }, [&] { return run(__half()); },
                      [&] { return run(__nv_bfloat16()); });
}

int b200_op_gemm_ex(const b200_gemm_desc* d, void* stream) {
  if (!d || !d->A || !d->W || !d->C || d->M < 0 || d->N <= 0 || d->K <= 0) {
    set_error("b200_op_gemm_ex: bad argument");
    return B200_ERR_INVALID;
  }
  if (d->precision != B200_PREC_FP16 && d->precision != B200_PREC_BF16) {
    set_error("b200_op_gemm_ex: the tensor-core kernel takes fp16 or bf16");
    return B200_ERR_UNSUPPORTED;
  }
  GemmParams p;
  p.A = d->A; p.lda = d->lda ? d->lda : d->K; p.W = d->W; p.ldw = d->ldw ? d->ldw : d->K; p.bias = d->bias;
  p.C = d->C; p.ldc = d->ldc ? d->ldc : (d->n_split > 0 ? d->n_split : d->N);
  p.M = d->M; p.N = d->N; p.K = d->K; p.act = d->activation;
  p.scale = d->scale; p.alpha = d->alpha;
  p.a_stats = d->a_stats; p.colsum = d->colsum; p.a_inv_c = d->a_inv_c; p.a_eps = d->a_eps;
  p.res = d->res; p.ldres = d->ldres ? d->ldres : d->N;
  p.res_stats = d->res_stats; p.res_gamma = d->res_gamma; p.res_beta = d->res_beta;
  p.res_inv_c = d->res_inv_c; p.res_eps = d->res_eps;
  p.out_stats = d->out_stats;
  p.C2 = d->C2; p.ldc2 = d->ldc2; p.n_split = d->n_split;
  p.whole_tiles = d->whole_tiles != 0;
  if ((p.a_stats && !p.colsum) || (p.res_stats && (!p.res || !p.res_gamma || !p.res_beta)) || !gemm_tc_supported(p)) {
    set_error("b200_op_gemm_ex: inconsistent description or shape not supported by the tensor-core kernel");
    return B200_ERR_UNSUPPORTED;
  }
  B200_CUDA(gemm_tc_init());
  int dev = 0, sms = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (p.n_split > 0 && !gemm_tc_split_supported(p, sms)) {
    set_error("b200_op_gemm_ex: the second output needs a product large enough for the CTA-pair kernel, n_split a "
              "multiple of 256 and at most 256 columns beyond it");
    return B200_ERR_UNSUPPORTED;
  }
  int* status = nullptr;
  B200_CUDA(cudaMalloc(&status, sizeof(int)));
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t err = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (err == cudaSuccess)
    err = d->precision == B200_PREC_FP16 ? launch_gemm_tc<__half>(p, status, sms, st)
                                         : launch_gemm_tc<__nv_bfloat16>(p, status, sms, st);
  if (err == cudaSuccess) err = cudaStreamSynchronize(st);
  int code = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(status);
  B200_CUDA(err);
  if (code) {
    set_error("tensor-core GEMM: a bounded device-side wait gave up, status " + std::to_string(code));
    return B200_ERR_TIMEOUT;
  }
  return B200_OK;
}

int b200_op_gemm_timed(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int activation,
                       int precision, int launches, float* ms_per_launch, void* stream) {
  GemmParams p;
  p.A = A; p.lda = K; p.W = W; p.ldw = K; p.bias = bias; p.C = C; p.ldc = N;
  p.M = M; p.N = N; p.K = K; p.act = activation;
  if (launches < 1 || !ms_per_launch) {
    set_error("b200_op_gemm_timed: bad argument");
    return B200_ERR_INVALID;
  }
  if (precision == B200_PREC_FP32 || !gemm_tc_supported(p)) {
    set_error("b200_op_gemm_timed: shape or precision not supported by the tensor-core kernel");
    return B200_ERR_UNSUPPORTED;
  }
  B200_CUDA(gemm_tc_init());
  int dev = 0, sms = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int* status = nullptr;
  B200_CUDA(cudaMalloc(&status, sizeof(int)));
  B200_CUDA(cudaMemset(status, 0, sizeof(int)));
  cudaEvent_t e0, e1;
  B200_CUDA(cudaEventCreate(&e0));
  B200_CUDA(cudaEventCreate(&e1));
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t err = cudaEventRecord(e0, s);
  for (int i = 0; i < launches && err == cudaSuccess; ++i)
    err = precision == B200_PREC_FP16 ? launch_gemm_tc<__half>(p, status, sms, s)
                                      : launch_gemm_tc<__nv_bfloat16>(p, status, sms, s);
  if (err == cudaSuccess) err = cudaEventRecord(e1, s);
  if (err == cudaSuccess) err = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
  int st = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(status);
  B200_CUDA(err);
  if (st) {
    set_error("tensor-core GEMM: a bounded device-side wait gave up, status " + std::to_string(st));
    return B200_ERR_TIMEOUT;
  }
  *ms_per_launch = ms / launches;
  return B200_OK;
}

int b200_op_encode_positions(const b200_board* d_boards, const int* d_offsets, const uint8_t* d_from_start, int n,
                             int input_format, int fill_empty_history, uint64_t* d_masks, float* d_values,
                             int* d_transforms, void* stream) {
  if (n < 0 || (n > 0 && (!d_boards || !d_offsets || !d_from_start || !d_masks || !d_values)) ||
      fill_empty_history < B200_FILL_NO || fill_empty_history > B200_FILL_ALWAYS) {
    set_error("b200_op_encode_positions: bad argument");
    return B200_ERR_INVALID;
  }
  if (!encode_format_supported(input_format)) {
    set_error("Unsupported input plane encoding " + std::to_string(input_format));  // the reference's message
    return B200_ERR_UNSUPPORTED;
  }
  B200_CUDA(launch_encode_positions(d_boards, d_offsets, d_from_start, n, input_format, fill_empty_history, d_masks,
                                    d_values, d_transforms, (cudaStream_t)stream));
  return B200_OK;
}

int b200_op_planes_from_training_data(const void* d_records, int n, long long record_stride, int undo_transform,
                                      uint64_t* d_masks, float* d_values, int* d_unsupported, void* stream) {
  if (n < 0 || (n > 0 && (!d_records || !d_masks || !d_values)) || record_stride < 8280 || (record_stride & 3) ||
      (reinterpret_cast<uintptr_t>(d_records) & 3)) {
    set_error("b200_op_planes_from_training_data: bad argument (records of at least 8280 bytes, 4-byte aligned)");
    return B200_ERR_INVALID;
  }
  B200_CUDA(launch_planes_from_training_data(d_records, n, record_stride, undo_transform != 0, d_masks, d_values,
                                             d_unsupported, (cudaStream_t)stream));
  return B200_OK;
}

int b200_op_policy_attention(const void* q, const void* k, const float* w4, int dm, int n, float* scratch_logits,
                             float* policy, int precision, void* stream) {
  if (n < 0 || dm <= 0 || (n > 0 && (!q || !k || !w4 || !scratch_logits || !policy))) {
    set_error("b200_op_policy_attention: bad argument");
    return B200_ERR_INVALID;
  }
  if (n == 0) return B200_OK;
  // Gather table in device memory, uploaded once per device.
  static std::mutex mu;
  static short* d_src[64] = {nullptr};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!d_src[dev & 63]) {
      B200_CUDA(cudaMalloc(&d_src[dev & 63], 1858 * sizeof(short)));
      B200_CUDA(cudaMemcpy(d_src[dev & 63], attn_policy_src_table(), 1858 * sizeof(short), cudaMemcpyHostToDevice));
      B200_CUDA(cudaDeviceSynchronize());  // the caller's stream may be non-blocking: the table must have landed
    }
  }
  const short* src = d_src[dev & 63];
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    GemmParams p;
    p.A = q; p.lda = dm; p.strideA = 64LL * dm;
    p.W = k; p.ldw = dm; p.strideW = 64LL * dm;
    p.C = scratch_logits; p.ldc = 64; p.strideC = 4096; p.out_f32 = true;
    p.M = 64; p.N = 64; p.K = dm; p.batch = n; p.scale = 1.0f / sqrtf((float)dm);
    B200_CUDA(launch_gemm_simt<T>(p, (cudaStream_t)stream));
    B200_CUDA(launch_policy_attn_gather<T>(scratch_logits, (const T*)k, w4, dm, src, n, policy, (cudaStream_t)stream));
    return B200_OK;
  };
  return by_precision(precision, [&] { return run(float()); }, [&] { return run(__half()); },
                      [&] { return run(__nv_bfloat16()); });
}

int b200_op_layer_norm(void* out, const void* x, const void* skip, const float* gamma, const float* beta, int rows,
                       int C, float alpha, float eps, int precision, void* stream) {
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    B200_CUDA(launch_layer_norm<T>((T*)out, (const T*)x, (const T*)skip, gamma, beta, nullptr, nullptr, rows, C,
                                   alpha, eps, (cudaStream_t)stream));
    return B200_OK;
  };
  return by_precision(precision, [&] { return run(float()); }, [&] { return run(__half()); },
                      [&] { return run(__nv_bfloat16()); });
}

int b200_op_attention(const void* q, const void* k, const void* v, long long ld, const void* bias, void* out,
                      long long ldo, int n, int heads, int depth, int precision, int variant, void* stream) {
  if (n < 0 || heads < 1 || depth < 1 || (n > 0 && (!q || !k || !v || !out)) || variant < 0 || variant > 1) {
    set_error("b200_op_attention: bad argument");
    return B200_ERR_INVALID;
  }
  const float scale = 1.0f / sqrtf((float)depth);
  cudaStream_t st = (cudaStream_t)stream;
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    if (variant == 0) {
      B200_CUDA(launch_attention<T>((const T*)q, (const T*)k, (const T*)v, ld, (const T*)bias, (T*)out, ldo, n, heads,
                                    depth, scale, st));
      return B200_OK;
    }
    if constexpr (sizeof(T) == 2) {
      if (!attention_tc_supported(ld, ldo, depth, q, k, v, bias, out)) {
        set_error("b200_op_attention: layout not supported by the tensor-core kernels");
        return B200_ERR_UNSUPPORTED;
      }
      B200_CUDA(gemm_tc_init());
      int dev = 0, sms = 0;
      B200_CUDA(cudaGetDevice(&dev));
      B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      int* status = nullptr;
      B200_CUDA(cudaMalloc(&status, sizeof(int)));
      B200_CUDA(cudaMemset(status, 0, sizeof(int)));
      cudaError_t err = launch_attention_tma<T>((const T*)q, (const T*)k, (const T*)v, ld, (const T*)bias, (T*)out,
                                                ldo, n, heads, depth, scale, status, sms, st);
      if (err == cudaSuccess) err = cudaStreamSynchronize(st);
      int code = 0;
      if (err == cudaSuccess) err = cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost);
      cudaFree(status);
      B200_CUDA(err);
      if (code) {
        set_error("attention: a bounded device-side wait gave up, status " + std::to_string(code));
        return B200_ERR_TIMEOUT;
      }
      return B200_OK;
    } else {
      set_error("b200_op_attention: the tensor-core kernels take fp16 or bf16");
      return B200_ERR_UNSUPPORTED;
    }
  };
  return by_precision(precision, [&] { return run(float()); }, [&] { return run(__half()); },
                      [&] { return run(__nv_bfloat16()); });
}

}  // extern "C"
