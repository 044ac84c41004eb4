// L2 residency probe (profiling surface, not on the evaluation path).
//
// Question it answers: can a kernel keep a per-CTA scratch tensor out of HBM by writing it and reading it back while it
// streams other data, the way a fused "produce the smolgen bias, consume it in the attention" kernel would?  Every CTA
// (one per SM) repeats: write its private slice, stream a chunk of a large buffer (stands for Q, K, V), read the slice
// back.  Under ncu, dram__bytes_read / dram__bytes_write tell how much of the scratch traffic reached HBM.
//   mode bit 0: L2 evict_last policy on the scratch stores and loads      bit 1: evict_first policy on the stream loads
//        bit 2: discard.global.L2 of the slice after it was read          bit 3: no scratch traffic (stream only)
#include "../../include/b200nn.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void st_hint(uint4* a, uint4 v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(a), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w), "l"(pol)
               : "memory");
}
__device__ __forceinline__ uint4 ld_hint(const uint4* a, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.L2::cache_hint.v4.b32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(a), "l"(pol));
  return v;
}
__device__ __forceinline__ uint4 ld_plain(const uint4* a) {
  uint4 v;
  asm volatile("ld.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a));
  return v;
}

// slice16 / stream16: sizes in 16-byte units, both multiples of 4 * blockDim.x
__global__ void __launch_bounds__(1024)
scratch_residency_kernel(uint4* scratch, const uint4* stream, size_t slice16, size_t stream16_per_iter,
                         size_t stream16_total, int iters, int mode, unsigned* sink) {
  uint4* mine = scratch + (size_t)blockIdx.x * slice16;
  const uint64_t pl = policy_evict_last(), pf = policy_evict_first();
  unsigned acc = 0;
  size_t spos = ((size_t)blockIdx.x * 7919u * stream16_per_iter) % stream16_total;
  for (int it = 0; it < iters; ++it) {
    if (!(mode & 8)) {
      for (size_t i = threadIdx.x; i < slice16; i += blockDim.x) {
        const uint4 v = make_uint4(it, (unsigned)i, acc, 7);
        if (mode & 1) st_hint(mine + i, v, pl);
        else mine[i] = v;
      }
      __syncthreads();
    }
    for (size_t i = threadIdx.x; i < stream16_per_iter; i += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        size_t idx = spos + i + u * blockDim.x;
        if (idx >= stream16_total) idx -= stream16_total;
        v[u] = (mode & 2) ? ld_hint(stream + idx, pf) : ld_plain(stream + idx);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc += v[u].x ^ v[u].w;
    }
    spos += stream16_per_iter * gridDim.x;
    while (spos >= stream16_total) spos -= stream16_total;
    if (!(mode & 8)) {
      for (size_t i = threadIdx.x; i < slice16; i += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[u] = (mode & 1) ? ld_hint(mine + i + u * blockDim.x, pl) : ld_plain(mine + i + u * blockDim.x);
#pragma unroll
        for (int u = 0; u < 4; ++u) acc += v[u].y + v[u].x;
      }
      __syncthreads();
      if (mode & 4) {
        for (size_t i = (size_t)threadIdx.x * 8; i < slice16; i += (size_t)blockDim.x * 8)
          asm volatile("discard.global.L2 [%0], 128;" ::"l"(mine + i) : "memory");
        __syncthreads();
      }
    }
  }
  if (acc == 0x12345678u) *sink = acc;
}

}  // namespace

extern "C" int b200_op_scratch_residency_probe(int slice_kb, int stream_kb, int iters, int mode, float* ms_out) {
  using namespace b200;
  if (slice_kb < 64 || slice_kb > 4096 || (slice_kb % 64) || stream_kb < 64 || stream_kb > 65536 || (stream_kb % 64) ||
      iters < 1 || iters > 1000 || mode < 0 || mode > 15 || !ms_out) {
    set_error("b200_op_scratch_residency_probe: slice 64..4096 KB and stream 64..65536 KB in multiples of 64 KB, "
              "1..1000 iterations, mode 0..15");
    return B200_ERR_INVALID;
  }
  int dev = 0, sms = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const size_t slice16 = (size_t)slice_kb * 64, stream16 = (size_t)stream_kb * 64;
  const size_t stream_total = (size_t)2 << 30;  // 2 GiB, far larger than L2
  uint4 *scratch = nullptr, *stream = nullptr;
  unsigned* sink = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t err = cudaMalloc(&scratch, (size_t)sms * slice16 * 16);
  if (err == cudaSuccess) err = cudaMalloc(&stream, stream_total);
  if (err == cudaSuccess) err = cudaMalloc(&sink, sizeof(unsigned));
  if (err == cudaSuccess) err = cudaMemset(stream, 1, stream_total);
  if (err == cudaSuccess) err = cudaMemset(scratch, 0, (size_t)sms * slice16 * 16);
  if (err == cudaSuccess) err = cudaEventCreate(&e0);
  if (err == cudaSuccess) err = cudaEventCreate(&e1);
  float best = 1e30f;
  for (int rep = 0; rep < 4 && err == cudaSuccess; ++rep) {
    err = cudaEventRecord(e0);
    scratch_residency_kernel<<<sms, 1024>>>(scratch, stream, slice16, stream16, stream_total / 16, iters, mode, sink);
    if (err == cudaSuccess) err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaEventRecord(e1);
    if (err == cudaSuccess) err = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && ms < best) best = ms;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(sink);
  cudaFree(stream);
  cudaFree(scratch);
  B200_CUDA(err);
  *ms_out = best;
  return B200_OK;
}
