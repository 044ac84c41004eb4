// Shared device helpers: storage-type conversion, activation functions, error plumbing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace b200 {

// lczero::ActivationFunction values (src/neural/tables/activation_function.h:24-35).
enum Act : int {
  ACT_DEFAULT = 0, ACT_MISH = 1, ACT_RELU = 2, ACT_NONE = 3, ACT_TANH = 4, ACT_SIGMOID = 5,
  ACT_SELU = 6, ACT_SWISH = 7, ACT_RELU_2 = 8, ACT_SOFTMAX = 9
};

// Thread-local last-error string behind b200_last_error().
void set_error(const std::string& msg);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define B200_CUDA(call)                                                        \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) return ::b200::cuda_fail(e__, #call, __FILE__, __LINE__); \
  } while (0)

// ---- programmatic dependent launch --------------------------------------------------------------------------
// A kernel launched through launch_dependent() may be made resident, and run its prologue (barrier initialisation,
// tensor-memory allocation, descriptor prefetch), while the kernel before it in the stream is still running.  Such a
// kernel calls grid_dependency_wait() in every thread before its first access to global memory: the call returns
// when the kernels before it have completed and their writes are visible.  grid_launch_dependents() lets the kernel
// after it do the same in turn.  Both are no-ops in a kernel that was launched the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// Whether launch_dependent() asks for the overlap (off: an ordinary launch).  Set by the host schedule per thread.
extern thread_local bool t_dependent_launch;

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = t_dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> struct TypeTag;
template <> struct TypeTag<float> { static constexpr int prec = 0; };
template <> struct TypeTag<__half> { static constexpr int prec = 1; };
template <> struct TypeTag<__nv_bfloat16> { static constexpr int prec = 2; };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
// fp16 stores saturate instead of producing inf (the reference clamps in its fp16 kernels too,
// src/neural/backends/cuda/common_kernels.cu:768-811).
template <> __device__ __forceinline__ __half from_f<__half>(float v) {
  return __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
}
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Activations in fp32, formulas as in src/neural/backends/shared/activation.cc:51-94.
// Fast variant for 16-bit storage: one ex2.approx and one rcp.approx per element.
__device__ __forceinline__ float mish_f(float v) {
  const float e = __expf(fminf(v, 30.0f));  // keeps n finite; mish(v) == v to fp32 precision beyond that
  const float n = e * e + 2.0f * e;
  const float d = __fdividef(v, n + 2.0f);
  return v <= -0.125f ? n * d : v - 2.0f * d;
}
__device__ __forceinline__ float swish_f(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
// Accurate variants (expf) are used in the fp32 verification mode.
template <bool kFast>
__device__ __forceinline__ float activate(float v, int act) {
  switch (act) {
    case ACT_RELU: return v > 0.f ? v : 0.f;
    case ACT_RELU_2: return v > 0.f ? v * v : 0.f;
    case ACT_MISH: {
      if (kFast) return mish_f(v);
      const float e = expf(v);
      const float n = e * e + 2.0f * e;
      const float d = v / (n + 2.0f);
      return v <= -0.125f ? n * d : v - 2.0f * d;
    }
    case ACT_TANH: return tanhf(v);
    case ACT_SIGMOID: return 1.0f / (1.0f + (kFast ? __expf(-v) : expf(-v)));
    case ACT_SELU: {
      const float alpha = 1.67326324f, scale = 1.05070098f;
      return v > 0.f ? scale * v : scale * alpha * ((kFast ? __expf(v) : expf(v)) - 1.0f);
    }
    case ACT_SWISH: return kFast ? swish_f(v) : v / (1.0f + expf(-v));
    default: return v;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

inline int ceil_div(long long a, long long b) { return int((a + b - 1) / b); }

}  // namespace b200
