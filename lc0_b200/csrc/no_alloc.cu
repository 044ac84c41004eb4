// Allocation-free variant of the attention-policy tail operator.
//
// b200_op_policy_attention needs n * 4096 floats of scratch for the per-position 64x64 logits between its two
// kernels.  Some callers cannot provide or obtain that memory at call time: an engine that evaluates from
// search threads must not call cudaMalloc there (it synchronises the whole device and stalls every other
// stream), and a host that has handed all remaining device memory to its own pool has nothing left to give.
// For them the scratch lives in a file-scope __device__ array below, reserved when the library is loaded on
// a GPU and held until the process exits.
#include <mutex>

#include "../../include/b200nn.h"
#include "kernels.cuh"

namespace {

constexpr int kMaxPositions = B200_STATIC_POLICY_MAX_POSITIONS;

// 256 positions x 4096 logits x 4 bytes = 4 MiB per GPU that loads the library.
static __device__ __align__(256) float g_logits_scratch[(size_t)kMaxPositions * 4096];
static __device__ __align__(256) short g_gather_table[1864];  // 1858 entries, padded

struct DeviceSetup {
  bool ready = false;
  float* logits = nullptr;  // device address of g_logits_scratch on this device
  short* table = nullptr;   // device address of g_gather_table on this device
};
std::mutex g_mu;
DeviceSetup g_setup[64];

// In host code the array names above are only handles; the kernels need the real device addresses, which
// cudaGetSymbolAddress returns for the device that is current.  Done once per device.
int setup_device(int dev, DeviceSetup** out) {
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceSetup& s = g_setup[dev & 63];
  if (!s.ready) {
    void* p = nullptr;
    B200_CUDA(cudaGetSymbolAddress(&p, g_logits_scratch));
    s.logits = static_cast<float*>(p);
    B200_CUDA(cudaGetSymbolAddress(&p, g_gather_table));
    s.table = static_cast<short*>(p);
    B200_CUDA(cudaMemcpy(s.table, b200::attn_policy_src_table(), 1858 * sizeof(short), cudaMemcpyHostToDevice));
    // A copy from pageable memory may return before the data has landed, and a non-blocking caller stream is not
    // ordered behind it: wait once here so that the first launch on any stream reads the finished table.
    B200_CUDA(cudaDeviceSynchronize());
    s.ready = true;
  }
  *out = &s;
  return B200_OK;
}

}  // namespace

extern "C" int b200_op_policy_attention_static(const void* q, const void* k, const float* w4, int dm, int n,
                                               float* policy, int precision, void* stream) {
  using namespace b200;
  if (n < 0 || dm <= 0 || (n > 0 && (!q || !k || !w4 || !policy))) {
    set_error("b200_op_policy_attention_static: bad argument");
    return B200_ERR_INVALID;
  }
  if (n > kMaxPositions) {
    set_error("b200_op_policy_attention_static: " + std::to_string(n) + " positions exceed the built-in scratch of " +
              std::to_string(kMaxPositions) + " positions; split the batch or use b200_op_policy_attention");
    return B200_ERR_INVALID;
  }
  if (n == 0) return B200_OK;
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  DeviceSetup* s = nullptr;
  const int rc = setup_device(dev, &s);
  if (rc != B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Every one of the n * 4096 scratch entries is overwritten by the first kernel before the second reads it,
  // so nothing has to be cleared between calls.
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    GemmParams p;
    p.A = q; p.lda = dm; p.strideA = 64LL * dm;
    p.W = k; p.ldw = dm; p.strideW = 64LL * dm;
    p.C = s->logits; p.ldc = 64; p.strideC = 4096; p.out_f32 = true;
    p.M = 64; p.N = 64; p.K = dm; p.batch = n; p.scale = 1.0f / sqrtf((float)dm);
    B200_CUDA(launch_gemm_simt<T>(p, st));
    B200_CUDA(launch_policy_attn_gather<T>(s->logits, static_cast<const T*>(k), w4, dm, s->table, n, policy, st));
    return B200_OK;
  };
  if (precision == B200_PREC_FP32) return run(float());
  if (precision == B200_PREC_FP16) return run(__half());
  if (precision == B200_PREC_BF16) return run(__nv_bfloat16());
  set_error("unknown precision");
  return B200_ERR_INVALID;
}
