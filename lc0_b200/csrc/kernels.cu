// Memory-bound and small-matrix kernels of the evaluation path, plus the plain FMA matrix kernel
// used by the fp32 verification mode and for shapes the tensor-core kernel does not take.
#include "kernels.cuh"

namespace b200 {

thread_local bool t_dependent_launch = false;

// ------------------------------------------------------------------------------------------------
// Plane expansion (reference: BlasComputation::EncodePlanes, backends/blas/network_blas.cc:973-981;
// GPU twin expandPlanes_kernel_NCHW, backends/cuda/common_kernels.cu:484-521).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void expand_planes_kernel(const uint64_t* __restrict__ masks, const float* __restrict__ values,
                                     long long total_planes, T* __restrict__ out) {
  // One thread writes 8 consecutive squares (one 16-byte store for 16-bit types).
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long plane = idx >> 3;
  if (plane >= total_planes) return;
  const int part = int(idx & 7);
  const uint64_t m = masks[plane] >> (part * 8);
  const float v = values[plane];
  __align__(16) T vals[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) vals[i] = from_f<T>(((m >> i) & 1) ? v : 0.f);
  T* dst = out + plane * 64 + part * 8;
  if (sizeof(T) == 2) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
  } else {
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(vals)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(vals)[1];
  }
}

template <typename T>
cudaError_t launch_expand_planes(const uint64_t* masks, const float* values, int n, T* out, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const long long planes = (long long)n * 112;
  const long long threads = planes * 8;
  expand_planes_kernel<T><<<ceil_div(threads, 256), 256, 0, s>>>(masks, values, planes, out);
  return cudaGetLastError();
}

// Token-major expansion with positional-encoding concat (reference: network_blas.cc:631-652; GPU twin
// preprocess_for_attention_body_kernel, backends/cuda/common_kernels.cu:1203-1244).
template <typename T> struct __align__(16) Vec8 { T v[8]; };

template <typename T>
__global__ void expand_tokens_kernel(const uint64_t* __restrict__ masks, const float* __restrict__ values,
                                     const float* __restrict__ pe_static, const T* __restrict__ pe_dense,
                                     int pe_ch, int cin, T* __restrict__ out) {
  __shared__ uint64_t sm[112];
  __shared__ float sv[112];
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < 112; i += blockDim.x) {
    sm[i] = masks[(long long)n * 112 + i];
    sv[i] = values[(long long)n * 112 + i];
  }
  __syncthreads();
  T* o = out + (long long)n * 64 * cin;
  const int total = 64 * cin;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int sq = idx / cin, c = idx - sq * cin;
    float v = 0.f;
    if (c < 112) {
      v = ((sm[c] >> sq) & 1) ? sv[c] : 0.f;
    } else if (c < 112 + pe_ch) {
      const int j = c - 112;
      v = pe_dense ? to_f(pe_dense[((long long)n * 64 + sq) * pe_ch + j]) : pe_static[sq * pe_ch + j];
    }
    o[idx] = from_f<T>(v);
  }
}

// Same for row widths and encoding widths that are multiples of 8: a thread writes 8 channels (16 bytes for
// 16-bit storage) at a time, dense positional encodings are copied as 16-byte pieces.
template <typename T>
__global__ void __launch_bounds__(256)
expand_tokens_vec_kernel(const uint64_t* __restrict__ masks, const float* __restrict__ values,
                         const float* __restrict__ pe_static, const T* __restrict__ pe_dense, int pe_ch, int cin,
                         T* __restrict__ out) {
  __shared__ uint64_t sm[112];
  __shared__ float sv[112];
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < 112; i += blockDim.x) {
    sm[i] = masks[(long long)n * 112 + i];
    sv[i] = values[(long long)n * 112 + i];
  }
  __syncthreads();
  T* o = out + (long long)n * 64 * cin;
  const int vec_per_row = cin >> 3;
  for (int idx = threadIdx.x; idx < 64 * vec_per_row; idx += blockDim.x) {
    const int sq = idx / vec_per_row, c = (idx - sq * vec_per_row) << 3;
    Vec8<T> r;
    if (c < 112) {
#pragma unroll
      for (int i = 0; i < 8; ++i) r.v[i] = from_f<T>(((sm[c + i] >> sq) & 1) ? sv[c + i] : 0.f);
    } else if (c < 112 + pe_ch) {
      const int j = c - 112;
      if (pe_dense) {
        r = *reinterpret_cast<const Vec8<T>*>(pe_dense + ((long long)n * 64 + sq) * pe_ch + j);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) r.v[i] = from_f<T>(pe_static[sq * pe_ch + j + i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) r.v[i] = from_f<T>(0.f);
    }
    *reinterpret_cast<Vec8<T>*>(o + (long long)sq * cin + c) = r;
  }
}

template <typename T>
cudaError_t launch_expand_tokens(const uint64_t* masks, const float* values, int n, const float* pe_static,
                                 const T* pe_dense, int pe_ch, int cin, T* out, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(pe_dense) & 15) == 0;
  if ((cin & 7) == 0 && (pe_ch & 7) == 0 && aligned)
    expand_tokens_vec_kernel<T><<<n, 256, 0, s>>>(masks, values, pe_static, pe_dense, pe_ch, cin, out);
  else
    expand_tokens_kernel<T><<<n, 256, 0, s>>>(masks, values, pe_static, pe_dense, pe_ch, cin, out);
  return cudaGetLastError();
}

// First 12 planes, square-major (reference: network_blas.cc:613-621).
template <typename T>
__global__ void expand_pre12_kernel(const uint64_t* __restrict__ masks, const float* __restrict__ values, int n,
                                    T* __restrict__ out) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * 768) return;
  const int s = int(idx / 768), r = int(idx - (long long)s * 768);
  const int sq = r / 12, j = r - sq * 12;
  const uint64_t m = masks[(long long)s * 112 + j];
  out[idx] = from_f<T>(((m >> sq) & 1) ? values[(long long)s * 112 + j] : 0.f);
}

template <typename T>
cudaError_t launch_expand_pre12(const uint64_t* masks, const float* values, int n, T* out, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  expand_pre12_kernel<T><<<ceil_div((long long)n * 768, 256), 256, 0, s>>>(masks, values, n, out);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Plain FMA GEMM: 64x64 tile, 16-deep k-steps, 256 threads x (4x4) outputs, fp32 accumulation.
// (reference: FullyConnectedLayer::Forward1D, backends/blas/fully_connected_layer.cc:50-106)
// ------------------------------------------------------------------------------------------------
template <typename T, bool kFast>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmParams p) {
  __shared__ float As[16][64 + 4];
  __shared__ float Ws[16][64 + 4];
  const int b = blockIdx.z;
  const T* A = reinterpret_cast<const T*>(p.A) + (long long)b * p.strideA;
  const T* W = reinterpret_cast<const T*>(p.W) + (long long)b * p.strideW;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int lr = tid >> 2;        // 0..63 tile row
  const int lc = (tid & 3) * 4;   // 0,4,8,12 k offset
  for (int k0 = 0; k0 < p.K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lc + i;
      const int m = m0 + lr, n = n0 + lr;
      As[lc + i][lr] = (m < p.M && k < p.K) ? to_f(A[(long long)m * p.lda + k]) : 0.f;
      Ws[lc + i][lr] = (n < p.N && k < p.K) ? to_f(W[(long long)n * p.ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
  const T* skip = reinterpret_cast<const T*>(p.skip);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j] * p.scale;
      if (p.bias) v += p.bias[n];
      v = activate<kFast>(v, p.act);
      if (skip) v = p.alpha * v + to_f(skip[(long long)m * p.ldskip + n]);
      const long long o = (long long)b * p.strideC + (long long)m * p.ldc + n;
      if (p.out_f32) reinterpret_cast<float*>(p.C)[o] = v;
      else reinterpret_cast<T*>(p.C)[o] = from_f<T>(v);
    }
  }
}

template <typename T>
cudaError_t launch_gemm_simt(const GemmParams& p, cudaStream_t s) {
  if (p.M <= 0 || p.N <= 0 || p.batch <= 0) return cudaSuccess;
  dim3 grid(ceil_div(p.N, 64), ceil_div(p.M, 64), p.batch);
  gemm_simt_kernel<T, (sizeof(T) == 2)><<<grid, 256, 0, s>>>(p);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// LayerNorm with skip connection (reference: LayerNorm2DWithSkipConnection, backends/blas/encoder.h:29-78;
// GPU twin layer_norm_kernel, backends/cuda/common_kernels.cu:932-1081).  One CTA per row, the row is held
// in registers (8 contiguous elements per thread per step), two-pass mean / variance, warp-shuffle sums.
// ------------------------------------------------------------------------------------------------
template <int kThreads>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < kThreads / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}


template <typename T, int kThreads, int kSteps>
__global__ void __launch_bounds__(kThreads)
layer_norm_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ skip,
                  const float* __restrict__ gamma, const float* __restrict__ beta,
                  const float* __restrict__ gate_mult, const float* __restrict__ gate_add, int C,
                  float alpha, float eps) {
  __shared__ float red[32];
  grid_dependency_wait();
  grid_launch_dependents();
  const long long row = blockIdx.x;
  const T* xr = x + row * C;
  const T* sr = skip ? skip + row * C : nullptr;
  float v[kSteps][8];
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int c = (s * kThreads + threadIdx.x) * 8;
    if (c < C) {
      Vec8<T> a = *reinterpret_cast<const Vec8<T>*>(xr + c);
      Vec8<T> b;
      if (sr) b = *reinterpret_cast<const Vec8<T>*>(sr + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = to_f(a.v[i]) * alpha;
        if (sr) t += to_f(b.v[i]);
        v[s][i] = t;
        sum += t;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[s][i] = 0.f;
    }
  }
  const float mean = block_sum<kThreads>(sum, red) / C;
  float var = 0.f;
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int c = (s * kThreads + threadIdx.x) * 8;
    if (c < C) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = v[s][i] - mean;
        var += d * d;
      }
    }
  }
  var = block_sum<kThreads>(var, red) / C;
  const float den = 1.0f / sqrtf(var + eps);
  const int sq = int(row & 63);
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int c = (s * kThreads + threadIdx.x) * 8;
    if (c < C) {
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(beta + c), b1 = *reinterpret_cast<const float4*>(beta + c + 4);
      const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      Vec8<T> o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = bb[i] + gg[i] * (v[s][i] - mean) * den;
        if (gate_mult) t = t * gate_mult[(long long)sq * C + c + i] + gate_add[(long long)sq * C + c + i];
        o.v[i] = from_f<T>(t);
      }
      *reinterpret_cast<Vec8<T>*>(out + row * C + c) = o;
    }
  }
}

// Warp-per-row variant for C <= 2048: a lane holds kChunks 16-byte pieces of the row (piece index
// lane + 32 * i), the reductions are pure shuffles and a 128-thread CTA normalises four rows.
template <typename T, int kChunks>
__global__ void __launch_bounds__(128)
layer_norm_warp_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ skip,
                       const float* __restrict__ gamma, const float* __restrict__ beta,
                       const float* __restrict__ gate_mult, const float* __restrict__ gate_add, int rows, int C,
                       float alpha, float eps) {
  grid_dependency_wait();
  grid_launch_dependents();
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + row * C;
  const T* sr = skip ? skip + row * C : nullptr;
  Vec8<T> a[kChunks], b[kChunks];
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int c = (lane + 32 * i) * 8;
    if (c < C) {
      a[i] = *reinterpret_cast<const Vec8<T>*>(xr + c);
      if (sr) b[i] = *reinterpret_cast<const Vec8<T>*>(sr + c);
    }
  }
  float v[kChunks][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int c = (lane + 32 * i) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f;
      if (c < C) {
        t = to_f(a[i].v[j]) * alpha;
        if (sr) t += to_f(b[i].v[j]);
      }
      v[i][j] = t;
      sum += t;
    }
  }
  const float mean = warp_sum(sum) / C;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int c = (lane + 32 * i) * 8;
    if (c < C) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        var += d * d;
      }
    }
  }
  var = warp_sum(var) / C;
  const float den = 1.0f / sqrtf(var + eps);
  const int sq = int(row & 63);
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int c = (lane + 32 * i) * 8;
    if (c < C) {
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(beta + c), b1 = *reinterpret_cast<const float4*>(beta + c + 4);
      const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      float gm[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f}, ga[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (gate_mult) {
        const float4 m0 = *reinterpret_cast<const float4*>(gate_mult + (long long)sq * C + c);
        const float4 m1 = *reinterpret_cast<const float4*>(gate_mult + (long long)sq * C + c + 4);
        const float4 a0 = *reinterpret_cast<const float4*>(gate_add + (long long)sq * C + c);
        const float4 a1 = *reinterpret_cast<const float4*>(gate_add + (long long)sq * C + c + 4);
        gm[0] = m0.x; gm[1] = m0.y; gm[2] = m0.z; gm[3] = m0.w; gm[4] = m1.x; gm[5] = m1.y; gm[6] = m1.z; gm[7] = m1.w;
        ga[0] = a0.x; ga[1] = a0.y; ga[2] = a0.z; ga[3] = a0.w; ga[4] = a1.x; ga[5] = a1.y; ga[6] = a1.z; ga[7] = a1.w;
      }
      Vec8<T> o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = bb[j] + gg[j] * (v[i][j] - mean) * den;
        t = t * gm[j] + ga[j];
        o.v[j] = from_f<T>(t);
      }
      *reinterpret_cast<Vec8<T>*>(out + row * C + c) = o;
    }
  }
}

template <typename T>
cudaError_t launch_layer_norm(T* out, const T* x, const T* skip, const float* gamma, const float* beta,
                              const float* gate_mult, const float* gate_add, int rows, int C, float alpha,
                              float eps, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if (C % 8 != 0 || C > 8192) return cudaErrorInvalidValue;
#define LNW_LAUNCH(CH)                                                                                      \
  le = launch_dependent(layer_norm_warp_kernel<T, CH>, dim3(ceil_div(rows, 4)), dim3(128), 0, s, out, x, skip, \
                        gamma, beta, gate_mult, gate_add, rows, C, alpha, eps)
#define LN_LAUNCH(TH, ST)                                                                                     \
  le = launch_dependent(layer_norm_kernel<T, TH, ST>, dim3(rows), dim3(TH), 0, s, out, x, skip, gamma, beta, \
                        gate_mult, gate_add, C, alpha, eps)
  cudaError_t le = cudaSuccess;
  if (C <= 256) LNW_LAUNCH(1);
  else if (C <= 512) LNW_LAUNCH(2);
  else if (C <= 1024) LNW_LAUNCH(4);
  else if (C <= 2048) LNW_LAUNCH(8);
  else if (C <= 4096) LN_LAUNCH(256, 2);  // few, wide rows (smolgen): 256 threads, several 16-byte pieces each
  else LN_LAUNCH(256, 4);
#undef LN_LAUNCH
#undef LNW_LAUNCH
  return le;
}

// Input gating x * mult + add (reference: network_blas.cc:669-682; gates re-laid out [64][C] at load).
template <typename T>
__global__ void gate_kernel(T* __restrict__ x, const float* __restrict__ mult, const float* __restrict__ add,
                            long long total, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / C;
  const int c = int(idx - row * C);
  const long long g = (row & 63) * C + c;
  x[idx] = from_f<T>(to_f(x[idx]) * mult[g] + add[g]);
}

template <typename T>
cudaError_t launch_gate(T* x, const float* gate_mult, const float* gate_add, int rows, int C, cudaStream_t s) {
  const long long total = (long long)rows * C;
  if (total <= 0) return cudaSuccess;
  gate_kernel<T><<<ceil_div(total, 256), 256, 0, s>>>(x, gate_mult, gate_add, total, C);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// 64-token attention, one CTA per (sample, head), fp32 arithmetic in shared memory
// (reference: network_blas.cc:352-439; GPU twins are two batched cuBLAS calls + softmax_opt_64_kernel).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
attention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                 const T* __restrict__ bias, T* __restrict__ out, long long ldo, int heads, int depth,
                 float scale) {
  extern __shared__ float smem[];
  const int dp = depth + 1;
  float* sq = smem;             // [64][dp]
  float* sk = sq + 64 * dp;     // [64][dp]
  float* sv = sk + 64 * dp;     // [64][dp]
  float* sp = sv + 64 * dp;     // [64][65]
  const int n = blockIdx.x / heads, h = blockIdx.x - n * heads;
  const long long base = (long long)n * 64 * ld + (long long)h * depth;
  for (int i = threadIdx.x; i < 64 * depth; i += 256) {
    const int r = i / depth, c = i - r * depth;
    sq[r * dp + c] = to_f(q[base + r * ld + c]);
    sk[r * dp + c] = to_f(k[base + r * ld + c]);
    sv[r * dp + c] = to_f(v[base + r * ld + c]);
  }
  __syncthreads();
  const int row = threadIdx.x >> 2, part = threadIdx.x & 3;
  float sc[16];
  const T* brow = bias ? bias + (((long long)n * heads + h) * 64 + row) * 64 : nullptr;
  float mx = -3.0e38f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int col = part + 4 * j;  // interleaved so the 4 lanes of a row hit different banks
    float a = 0.f;
    for (int c = 0; c < depth; ++c) a = fmaf(sq[row * dp + c], sk[col * dp + c], a);
    a *= scale;
    if (brow) a += to_f(brow[col]);
    sc[j] = a;
    mx = fmaxf(mx, a);
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    sc[j] = __expf(sc[j] - mx);
    sum += sc[j];
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int j = 0; j < 16; ++j) sp[row * 65 + part + 4 * j] = sc[j] * inv;
  __syncthreads();
  // O[row][c] for c = part, part+4, ...
  for (int c = part; c < depth; c += 4) {
    float a = 0.f;
#pragma unroll 8
    for (int j = 0; j < 64; ++j) a = fmaf(sp[row * 65 + j], sv[j * dp + c], a);
    out[((long long)n * 64 + row) * ldo + (long long)h * depth + c] = from_f<T>(a);
  }
}

// fp32 mode uses expf for parity with the CPU oracle.
template <>
__global__ void __launch_bounds__(256)
attention_kernel<float>(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                        long long ld, const float* __restrict__ bias, float* __restrict__ out, long long ldo,
                        int heads, int depth, float scale) {
  extern __shared__ float smem[];
  const int dp = depth + 1;
  float* sq = smem;
  float* sk = sq + 64 * dp;
  float* sv = sk + 64 * dp;
  float* sp = sv + 64 * dp;
  const int n = blockIdx.x / heads, h = blockIdx.x - n * heads;
  const long long base = (long long)n * 64 * ld + (long long)h * depth;
  for (int i = threadIdx.x; i < 64 * depth; i += 256) {
    const int r = i / depth, c = i - r * depth;
    sq[r * dp + c] = q[base + r * ld + c];
    sk[r * dp + c] = k[base + r * ld + c];
    sv[r * dp + c] = v[base + r * ld + c];
  }
  __syncthreads();
  const int row = threadIdx.x >> 2, part = threadIdx.x & 3;
  float sc[16];
  const float* brow = bias ? bias + (((long long)n * heads + h) * 64 + row) * 64 : nullptr;
  float mx = -3.0e38f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int col = part + 4 * j;
    float a = 0.f;
    for (int c = 0; c < depth; ++c) a = fmaf(sq[row * dp + c], sk[col * dp + c], a);
    a *= scale;
    if (brow) a += brow[col];
    sc[j] = a;
    mx = fmaxf(mx, a);
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    sc[j] = expf(sc[j] - mx);
    sum += sc[j];
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
#pragma unroll
  for (int j = 0; j < 16; ++j) sp[row * 65 + part + 4 * j] = sc[j] / sum;
  __syncthreads();
  for (int c = part; c < depth; c += 4) {
    float a = 0.f;
    for (int j = 0; j < 64; ++j) a = fmaf(sp[row * 65 + j], sv[j * dp + c], a);
    out[((long long)n * 64 + row) * ldo + (long long)h * depth + c] = a;
  }
}

template <typename T>
cudaError_t launch_attention(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                             long long ldo, int n, int heads, int depth, float scale, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (depth > 128) return cudaErrorInvalidValue;
  const size_t smem = (size_t)(3 * 64 * (depth + 1) + 64 * 65) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  attention_kernel<T><<<n * heads, 256, smem, s>>>(q, k, v, ld, bias, out, ldo, heads, depth, scale);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Attention policy tail: promotion offsets + gather of the 1858 move logits
// (reference: network_blas.cc:873-914; GPU twins promotion_logits_kernel and policyMap_kernel,
// backends/cuda/common_kernels.cu:1116-1201 and :703-734).  One CTA per sample.
// src_slot[j] is the slot (0..4287) of the 64*64 + 8*24 raw vector that feeds policy index j.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
policy_attn_gather_kernel(const float* __restrict__ logits, const T* __restrict__ kp,
                          const float* __restrict__ w4, int dm, const short* __restrict__ src_slot,
                          float* __restrict__ policy) {
  __shared__ float off[4][8];
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 32 dot products (4 promotion rows x 8 files), 4 per warp.
  for (int t = warp * 4; t < warp * 4 + 4; ++t) {
    const int i = t >> 3, j = t & 7;
    const T* key = kp + ((long long)n * 64 + 56 + j) * dm;
    float a = 0.f;
    for (int c = lane; c < dm; c += 32) a = fmaf(to_f(key[c]), w4[i * dm + c], a);
    a = warp_sum(a);
    if (lane == 0) off[i][j] = a;
  }
  __syncthreads();
  const float* lg = logits + (long long)n * 4096;
  for (int j = threadIdx.x; j < 1858; j += 256) {
    const int slot = src_slot[j];
    float v;
    if (slot < 4096) {
      v = lg[slot];
    } else {
      const int r = slot - 4096;  // 24*k + 3*file + i
      const int kf = r / 24, rem = r - kf * 24, jf = rem / 3, i = rem - jf * 3;
      v = lg[(48 + kf) * 64 + 56 + jf] + off[i][jf] + off[3][jf];
    }
    policy[(long long)n * 1858 + j] = v;
  }
}

template <typename T>
cudaError_t launch_policy_attn_gather(const float* logits, const T* kp, const float* w4, int dm,
                                      const short* src_slot, int n, float* policy, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  policy_attn_gather_kernel<T><<<n, 256, 0, s>>>(logits, kp, w4, dm, src_slot, policy);
  return cudaGetLastError();
}

template <typename T>
__global__ void policy_gather_kernel(const T* __restrict__ raw, long long ld, const short* __restrict__ src,
                                     float* __restrict__ policy) {
  const int n = blockIdx.x;
  for (int j = threadIdx.x; j < 1858; j += blockDim.x)
    policy[(long long)n * 1858 + j] = to_f(raw[(long long)n * ld + src[j]]);
}

template <typename T>
cudaError_t launch_policy_gather(const T* raw, long long ld, const short* src_slot, int n, float* policy,
                                 cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  policy_gather_kernel<T><<<n, 256, 0, s>>>(raw, ld, src_slot, policy);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Last layer of the value / moves-left heads (reference: network_blas.cc:747-772 and :797-802;
// the reference CUDA backend leaves the WDL softmax to the host, network_cuda.cc:991-1014).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void head_final_kernel(const T* __restrict__ h, int k, const float* __restrict__ w,
                                  const float* __restrict__ b, int mode, int n, float* __restrict__ qdm) {
  const int sample = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (sample >= n) return;
  const T* hr = h + (long long)sample * k;
  const int outs = mode == 0 ? 3 : 1;
  float o[3] = {0.f, 0.f, 0.f};
  for (int i = 0; i < outs; ++i) {
    float a = 0.f;
    for (int c = lane; c < k; c += 32) a = fmaf(to_f(hr[c]), w[i * k + c], a);
    o[i] = warp_sum(a) + b[i];
  }
  if (lane != 0) return;
  float* dst = qdm + (long long)sample * 3;
  if (mode == 0) {
    const float mx = fmaxf(o[0], fmaxf(o[1], o[2]));
    const float e0 = expf(o[0] - mx), e1 = expf(o[1] - mx), e2 = expf(o[2] - mx);
    const float s = e0 + e1 + e2;
    dst[0] = e0 / s - e2 / s;
    dst[1] = e1 / s;
  } else if (mode == 1) {
    dst[0] = tanhf(o[0]);
    dst[1] = 0.f;
  } else {
    dst[2] = o[0] > 0.f ? o[0] : 0.f;
  }
}

template <typename T>
cudaError_t launch_head_final(const T* h, int k, const float* w, const float* b, int mode, int n, float* qdm,
                              cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  head_final_kernel<T><<<ceil_div(n, 4), 128, 0, s>>>(h, k, w, b, mode, n, qdm);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Residual tower on NHWC activations [n*64][C].
// 3x3 convolution as an implicit GEMM over (tap, cin): same 64x64x16 FMA tiling as gemm_simt_kernel;
// the A tile gathers the shifted board square (zero outside the board).
// (reference: WinogradConvolution3::Forward, backends/blas/winograd_convolution3.cc:47-57, computes the
// same sums through F(2x2,3x3) transforms.)
// ------------------------------------------------------------------------------------------------
template <typename T, bool kFast>
__global__ void __launch_bounds__(256)
conv3x3_kernel(const T* __restrict__ x, int cin, const T* __restrict__ w, const float* __restrict__ bias,
               T* __restrict__ y, int cout, int rows, int act) {
  __shared__ float As[16][64 + 4];
  __shared__ float Ws[16][64 + 4];
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lc = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int m = m0 + lr;  // this thread's A row: (sample, square)
  const int sq = m & 63, sx = sq & 7, sy = sq >> 3;
  for (int tap = 0; tap < 9; ++tap) {
    const int dy = tap / 3 - 1, dx = tap % 3 - 1;
    const int yy = sy + dy, xx = sx + dx;
    const bool inside = m < rows && yy >= 0 && yy < 8 && xx >= 0 && xx < 8;
    const T* arow = x + ((long long)(m - sq) + yy * 8 + xx) * cin;
    const T* wt = w + (long long)tap * cout * cin;
    for (int k0 = 0; k0 < cin; k0 += 16) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = k0 + lc + i;
        const int n = n0 + lr;
        As[lc + i][lr] = (inside && k < cin) ? to_f(arow[k]) : 0.f;
        Ws[lc + i][lr] = (n < cout && k < cin) ? to_f(wt[(long long)n * cin + k]) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        float a[4], ww[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) ww[j] = Ws[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], ww[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mm = m0 + ty * 4 + i;
    if (mm >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= cout) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      y[(long long)mm * cout + n] = from_f<T>(activate<kFast>(v, act));
    }
  }
}

template <typename T>
cudaError_t launch_conv3x3(const T* x, int cin, const T* w, const float* bias, T* y, int cout, int n, int act,
                           cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  dim3 grid(ceil_div(cout, 64), n);
  conv3x3_kernel<T, (sizeof(T) == 2)><<<grid, 256, 0, s>>>(x, cin, w, bias, y, cout, n * 64, act);
  return cudaGetLastError();
}

// Squeeze-excitation block, one CTA per sample (reference: ApplySEUnit, backends/blas/se_unit.cc:31-91;
// GPU twin SE_Layer_NHWC, backends/cuda/fp16_kernels.cu:55-136).
template <typename T, bool kFast>
__global__ void __launch_bounds__(256)
se_kernel(const T* __restrict__ x, const float* __restrict__ conv_bias, const T* __restrict__ skip,
          const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ w2,
          const float* __restrict__ b2, T* __restrict__ y, int C, int se_k, int act) {
  extern __shared__ float sm[];
  float* pool = sm;           // [C]
  float* hid = pool + C;      // [se_k]
  float* z = hid + se_k;      // [2C]
  const int n = blockIdx.x;
  const T* xs = x + (long long)n * 64 * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f;
    for (int sq = 0; sq < 64; ++sq) a += to_f(xs[sq * C + c]);
    pool[c] = a / 64.0f + conv_bias[c];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int o = warp; o < se_k; o += nw) {
    float a = 0.f;
    for (int c = lane; c < C; c += 32) a = fmaf(pool[c], w1[o * C + c], a);
    a = warp_sum(a);
    if (lane == 0) hid[o] = activate<false>(a + b1[o], act);
  }
  __syncthreads();
  for (int o = threadIdx.x; o < 2 * C; o += blockDim.x) {
    float a = b2[o];
    for (int c = 0; c < se_k; ++c) a = fmaf(hid[c], w2[o * se_k + c], a);
    z[o] = a;
  }
  __syncthreads();
  const T* ss = skip + (long long)n * 64 * C;
  T* ys = y + (long long)n * 64 * C;
  for (int i = threadIdx.x; i < 64 * C; i += blockDim.x) {
    const int c = i % C;
    const float g = 1.0f / (1.0f + expf(-z[c]));
    const float v = g * to_f(xs[i]) + to_f(ss[i]) + z[C + c] + g * conv_bias[c];
    ys[i] = from_f<T>(activate<kFast>(v, act));
  }
}

// Vectorised variant (C % 8 == 0): 16-byte loads, the sample's 64 x C tile is kept in shared memory between the
// pooling pass and the scaling pass, partial sums over square groups are reduced through shared memory.
template <typename T, bool kFast>
__global__ void __launch_bounds__(256)
se_vec_kernel(const T* __restrict__ x, const float* __restrict__ conv_bias, const T* __restrict__ skip,
              const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ w2,
              const float* __restrict__ b2, T* __restrict__ y, int C, int se_k, int act) {
  extern __shared__ __align__(16) uint8_t se_sm[];
  T* xs = reinterpret_cast<T*>(se_sm);                          // [64][C]
  float* partial = reinterpret_cast<float*>(xs + 64 * C);       // [nsqg][C]  (nsqg * C == 2048)
  float* pool = partial + 2048;                                 // [C]
  float* hid = pool + C;                                        // [se_k]
  float* z = hid + se_k;                                        // [2C]
  const int n = blockIdx.x, tid = threadIdx.x;
  const int cgs = C / 8;            // channel groups of 8
  const int nsqg = 256 / cgs;       // square groups working in parallel
  const int cg = tid % cgs, sqg = tid / cgs;
  const T* xg = x + (long long)n * 64 * C;
  if (sqg < nsqg) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int sq = sqg; sq < 64; sq += nsqg) {
      const Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(xg + sq * C + cg * 8);
      *reinterpret_cast<Vec8<T>*>(xs + sq * C + cg * 8) = v;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += to_f(v.v[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) partial[sqg * C + cg * 8 + j] = acc[j];
  }
  __syncthreads();
  for (int c = tid; c < C; c += 256) {
    float a = 0.f;
    for (int g = 0; g < nsqg; ++g) a += partial[g * C + c];
    pool[c] = a / 64.0f + conv_bias[c];
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int o = warp; o < se_k; o += 8) {
    float a = 0.f;
    for (int c = lane; c < C; c += 32) a = fmaf(pool[c], w1[o * C + c], a);
    a = warp_sum(a);
    if (lane == 0) hid[o] = activate<false>(a + b1[o], act);
  }
  __syncthreads();
  for (int o = tid; o < 2 * C; o += 256) {
    float a = b2[o];
    for (int c = 0; c < se_k; ++c) a = fmaf(hid[c], w2[o * se_k + c], a);
    // first C outputs become the sigmoid gate, the rest the shift (with the gate times the conv bias folded in)
    z[o] = a;
  }
  __syncthreads();
  for (int c = tid; c < C; c += 256) {
    const float g = 1.0f / (1.0f + expf(-z[c]));
    z[C + c] += g * conv_bias[c];
    z[c] = g;
  }
  __syncthreads();
  const T* sg = skip + (long long)n * 64 * C;
  T* yg = y + (long long)n * 64 * C;
  if (sqg < nsqg) {
    float g[8], sh[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      g[j] = z[cg * 8 + j];
      sh[j] = z[C + cg * 8 + j];
    }
    for (int sq = sqg; sq < 64; sq += nsqg) {
      const Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(xs + sq * C + cg * 8);
      const Vec8<T> r = *reinterpret_cast<const Vec8<T>*>(sg + sq * C + cg * 8);
      Vec8<T> o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = from_f<T>(activate<kFast>(g[j] * to_f(v.v[j]) + to_f(r.v[j]) + sh[j], act));
      *reinterpret_cast<Vec8<T>*>(yg + sq * C + cg * 8) = o;
    }
  }
}

template <typename T>
cudaError_t launch_se(const T* x, const float* conv_bias, const T* skip, const float* w1, const float* b1,
                      const float* w2, const float* b2, T* y, int C, int se_k, int n, int act, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int cgs = C / 8;
  if (C % 8 == 0 && cgs <= 256 && 256 % cgs == 0) {
    const size_t smem = (size_t)64 * C * sizeof(T) + (size_t)(2048 + 3 * C + se_k) * sizeof(float);
    if (smem <= 200 * 1024) {
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(se_vec_kernel<T, (sizeof(T) == 2)>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
      }
      se_vec_kernel<T, (sizeof(T) == 2)><<<n, 256, smem, s>>>(x, conv_bias, skip, w1, b1, w2, b2, y, C, se_k, act);
      return cudaGetLastError();
    }
  }
  const size_t smem = (size_t)(3 * C + se_k) * sizeof(float);
  se_kernel<T, (sizeof(T) == 2)><<<n, 256, smem, s>>>(x, conv_bias, skip, w1, b1, w2, b2, y, C, se_k, act);
  return cudaGetLastError();
}

template <typename T, bool kFast>
__global__ void bias_skip_act_kernel(const T* __restrict__ x, const float* __restrict__ bias,
                                     const T* __restrict__ skip, T* __restrict__ y, int C, long long total,
                                     int act) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float v = to_f(x[idx]) + bias[idx % C];
  if (skip) v += to_f(skip[idx]);
  y[idx] = from_f<T>(activate<kFast>(v, act));
}

template <typename T>
cudaError_t launch_bias_skip_act(const T* x, const float* bias, const T* skip, T* y, int C, int rows, int act,
                                 cudaStream_t s) {
  const long long total = (long long)rows * C;
  if (total <= 0) return cudaSuccess;
  bias_skip_act_kernel<T, (sizeof(T) == 2)><<<ceil_div(total, 256), 256, 0, s>>>(x, bias, skip, y, C, total, act);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Legal-move softmax (reference: NetworkAsBackendComputation::SoftmaxPolicy, neural/wrapper.cc:135-156).
// One warp per position.  The exponential is the reference's FastExp restated with explicitly unfused
// multiplies and adds, and the total is accumulated sequentially in move order, so that the result is
// bit-identical to the host formula applied to the same logits.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp_ref(float x) {
  const float a = __fmul_rn(1.442695040f, x);
  int e;
  if (a < 0.f) {
    if (a < -126.f) return 0.f;
    e = (int)__fadd_rn(a, -1.0f);
  } else {
    e = (int)a;
  }
  float out = __fadd_rn(a, -(float)e);
  out = __fadd_rn(1.0f, __fmul_rn(out, __fadd_rn(0.6602339f, __fmul_rn(0.33976606f, out))));
  return __int_as_float(__float_as_int(out) + (int)((unsigned)e << 23));
}

__global__ void __launch_bounds__(128)
legal_softmax_kernel(const float* __restrict__ policy, const unsigned short* __restrict__ move_ids,
                     const int* __restrict__ n_moves, int n, float inv_t, float* __restrict__ probs) {
  __shared__ float vals[4][kLegalStride];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sample = blockIdx.x * 4 + w;
  if (sample >= n) return;
  int cnt = n_moves[sample];
  cnt = cnt < 0 ? 0 : (cnt > kLegalStride ? kLegalStride : cnt);
  const unsigned short* ids = move_ids + (long long)sample * kLegalStride;
  const float* pol = policy + (long long)sample * 1858;
  float mx = -INFINITY;
  for (int i = lane; i < cnt; i += 32) {
    const int id = ids[i] < 1858 ? ids[i] : 1857;
    const float v = pol[id];
    vals[w][i] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  __syncwarp();
  for (int i = lane; i < cnt; i += 32) vals[w][i] = fast_exp_ref(__fmul_rn(__fadd_rn(vals[w][i], -mx), inv_t));
  __syncwarp();
  float total = 0.f;
  if (lane == 0)
    for (int i = 0; i < cnt; ++i) total = __fadd_rn(total, vals[w][i]);
  total = __shfl_sync(0xffffffffu, total, 0);
  const float scale = total > 0.f ? __fdiv_rn(1.0f, total) : 1.0f;
  float* out = probs + (long long)sample * kLegalStride;
  for (int i = lane; i < cnt; i += 32) out[i] = __fmul_rn(vals[w][i], scale);
}

cudaError_t launch_legal_softmax(const float* policy, const unsigned short* move_ids, const int* n_moves, int n,
                                 float inv_temperature, float* probs, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  legal_softmax_kernel<<<ceil_div(n, 4), 128, 0, s>>>(policy, move_ids, n_moves, n, inv_temperature, probs);
  return cudaGetLastError();
}

#define INSTANTIATE(T)                                                                                        \
  template cudaError_t launch_gemm_simt<T>(const GemmParams&, cudaStream_t);                                  \
  template cudaError_t launch_expand_planes<T>(const uint64_t*, const float*, int, T*, cudaStream_t);         \
  template cudaError_t launch_expand_tokens<T>(const uint64_t*, const float*, int, const float*, const T*,    \
                                               int, int, T*, cudaStream_t);                                   \
  template cudaError_t launch_expand_pre12<T>(const uint64_t*, const float*, int, T*, cudaStream_t);          \
  template cudaError_t launch_layer_norm<T>(T*, const T*, const T*, const float*, const float*, const float*, \
                                            const float*, int, int, float, float, cudaStream_t);              \
  template cudaError_t launch_gate<T>(T*, const float*, const float*, int, int, cudaStream_t);                \
  template cudaError_t launch_attention<T>(const T*, const T*, const T*, long long, const T*, T*, long long,  \
                                           int, int, int, float, cudaStream_t);                               \
  template cudaError_t launch_policy_attn_gather<T>(const float*, const T*, const float*, int, const short*,  \
                                                    int, float*, cudaStream_t);                               \
  template cudaError_t launch_policy_gather<T>(const T*, long long, const short*, int, float*, cudaStream_t); \
  template cudaError_t launch_head_final<T>(const T*, int, const float*, const float*, int, int, float*,      \
                                            cudaStream_t);                                                    \
  template cudaError_t launch_conv3x3<T>(const T*, int, const T*, const float*, T*, int, int, int,            \
                                         cudaStream_t);                                                       \
  template cudaError_t launch_se<T>(const T*, const float*, const T*, const float*, const float*,             \
                                    const float*, const float*, T*, int, int, int, int, cudaStream_t);        \
  template cudaError_t launch_bias_skip_act<T>(const T*, const float*, const T*, T*, int, int, int,           \
                                               cudaStream_t);

INSTANTIATE(float)
INSTANTIATE(__half)
INSTANTIATE(__nv_bfloat16)

}  // namespace b200
