// Winograd F(4x4, 3x3) path for the 3x3 convolutions of residual networks on the 8x8 board (16-bit storage).
//
//   V = B^T d B      input transform: four overlapping 6x6 patches per board and channel -> 36 matrices [boards*4][Cin]
//   M = V . U^T      36 independent products [boards*4][Cin] x [Cin][Cout] on the tensor-core kernel (gemm_tc.cu,
//                    batched-rows mode), U = G g G^T transformed once at load
//   Y = A^T M A      output transform: 4x4 outputs per patch, + bias, squeeze-excitation, skip, activation
//
// The same decomposition as the reference's GPU path (InputTransform / OutputTransform kernels,
// src/neural/backends/cuda/winograd_helper.inc:194-428, driven by FusedWinogradConvSELayer::Eval,
// backends/cuda/layers.cc:940-1013) and, with 2x2 tiles, its CPU path
// (backends/blas/winograd_convolution3.cc:47-324); the filter transform is WinogradFilterTransformF's
// (backends/shared/winograd_filter.cc:54-90) with the F(4x4, 3x3) matrices.  The transform kernels are memory-bound:
// one thread owns two channels of one patch (input) or of one board (output), so that a warp reads and writes 128
// contiguous bytes per square.
#include "kernels.cuh"

namespace b200 {
namespace {

// d[0..5] -> B^T d   (Lavin & Gray, F(4x4, 3x3))
__device__ __forceinline__ void wino_in_1d(const float (&d)[6], float (&o)[6]) {
  o[0] = 4.f * d[0] - 5.f * d[2] + d[4];
  o[1] = -4.f * d[1] - 4.f * d[2] + d[3] + d[4];
  o[2] = 4.f * d[1] - 4.f * d[2] - d[3] + d[4];
  o[3] = -2.f * d[1] - d[2] + 2.f * d[3] + d[4];
  o[4] = 2.f * d[1] - d[2] - 2.f * d[3] + d[4];
  o[5] = 4.f * d[1] - 5.f * d[3] + d[5];
}
// m[0..5] -> A^T m
__device__ __forceinline__ void wino_out_1d(const float (&m)[6], float (&o)[4]) {
  o[0] = m[0] + m[1] + m[2] + m[3] + m[4];
  o[1] = m[1] - m[2] + 2.f * (m[3] - m[4]);
  o[2] = m[1] + m[2] + 4.f * (m[3] + m[4]);
  o[3] = m[1] - m[2] + 8.f * (m[3] - m[4]) + m[5];
}

template <typename T> struct Pair;
template <> struct Pair<__half> {
  static __device__ __forceinline__ float2 load(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
  static __device__ __forceinline__ void store(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

// x: [boards*64][C] token-major.  v: [36][rows_padded][C], row = board * 4 + patch (patch = 2 * (rank / 4) + file / 4).
// One thread per (patch, channel pair): a warp reads and writes 128 contiguous bytes per square.  (One channel per
// thread, a third of the registers and three times the occupancy, measured 20 % slower: the 2-byte accesses cost more
// than the occupancy buys.)
template <typename T>
__global__ void __launch_bounds__(256)
wino_input_kernel(const T* __restrict__ x, T* __restrict__ v, int C, long long patches, long long rows_padded) {
  const int pairs = C >> 1;
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  if (idx >= patches * pairs) return;
  const long long row = idx / pairs;
  const int c = int(idx - row * pairs) * 2;
  const long long board = row >> 2;
  const int py = int(row & 3) >> 1, px = int(row & 1);
  const T* xb = x + board * 64 * C + c;
  float t[6][6][2];  // B^T d, columns transformed
#pragma unroll
  for (int j = 0; j < 6; ++j) {  // patch column j
    const int xx = 4 * px - 1 + j;
    float d0[6], d1[6], o0[6], o1[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const int yy = 4 * py - 1 + i;
      float2 e = make_float2(0.f, 0.f);
      if (xx >= 0 && xx < 8 && yy >= 0 && yy < 8) e = Pair<T>::load(xb + (long long)(yy * 8 + xx) * C);
      d0[i] = e.x;
      d1[i] = e.y;
    }
    wino_in_1d(d0, o0);
    wino_in_1d(d1, o1);
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      t[i][j][0] = o0[i];
      t[i][j][1] = o1[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    float r0[6], r1[6], o0[6], o1[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      r0[j] = t[i][j][0];
      r1[j] = t[i][j][1];
    }
    wino_in_1d(r0, o0);
    wino_in_1d(r1, o1);
#pragma unroll
    for (int j = 0; j < 6; ++j)
      Pair<T>::store(v + ((long long)(i * 6 + j) * rows_padded + row) * C + c, o0[j], o1[j]);
  }
}

// m: [36][rows_padded][C] (row = board * 4 + patch).  One CTA per board, one thread per channel pair; a thread ends up
// with all 64 squares of its two channels in registers, so the squeeze-excitation pooling is a local sum.
//   no SE:  y = act(conv + bias [+ skip])                                  (BiasActivate / BiasResidual)
//   SE:     y = act(gate * conv + skip + shift + gate * bias)              (ApplySEUnit, backends/blas/se_unit.cc:31-91)
template <typename T, bool kSe>
__global__ void __launch_bounds__(256)
wino_output_kernel(const T* __restrict__ m, const float* __restrict__ bias, const T* __restrict__ skip,
                   const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ w2,
                   const float* __restrict__ b2, T* __restrict__ y, int C, int se_k, long long rows_padded, int act) {
  extern __shared__ float wsm[];
  float* pool = wsm;          // [C]
  float* hid = pool + C;      // [se_k]
  float* z = hid + se_k;      // [2C]
  const long long board = blockIdx.x;
  const int c = threadIdx.x * 2;
  const bool live = c < C;
  float o[64][2];
  if (live) {
#pragma unroll
    for (int patch = 0; patch < 4; ++patch) {
      const long long row = board * 4 + patch;
      float t[4][6][2];  // A^T M, columns transformed
#pragma unroll
      for (int j = 0; j < 6; ++j) {
        float m0[6], m1[6], r0[4], r1[4];
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const float2 e = Pair<T>::load(m + ((long long)(i * 6 + j) * rows_padded + row) * C + c);
          m0[i] = e.x;
          m1[i] = e.y;
        }
        wino_out_1d(m0, r0);
        wino_out_1d(m1, r1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          t[i][j][0] = r0[i];
          t[i][j][1] = r1[i];
        }
      }
      const int py = patch >> 1, px = patch & 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a0[6], a1[6], r0[4], r1[4];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
          a0[j] = t[i][j][0];
          a1[j] = t[i][j][1];
        }
        wino_out_1d(a0, r0);
        wino_out_1d(a1, r1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[(4 * py + i) * 8 + 4 * px + j][0] = r0[j];
          o[(4 * py + i) * 8 + 4 * px + j][1] = r1[j];
        }
      }
    }
  }
  float g0 = 1.f, g1 = 1.f, s0 = 0.f, s1 = 0.f;  // gate and shift of this thread's two channels
  if (live && bias) {
    s0 = bias[c];
    s1 = bias[c + 1];
  }
  if (kSe) {
    if (live) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int sq = 0; sq < 64; ++sq) {
        a0 += o[sq][0];
        a1 += o[sq][1];
      }
      pool[c] = a0 * (1.0f / 64.0f) + s0;
      pool[c + 1] = a1 * (1.0f / 64.0f) + s1;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int k = warp; k < se_k; k += nw) {
      float a = 0.f;
      for (int cc = lane; cc < C; cc += 32) a = fmaf(pool[cc], w1[(long long)k * C + cc], a);
      a = warp_sum(a);
      if (lane == 0) hid[k] = activate<false>(a + b1[k], act);
    }
    __syncthreads();
    for (int j = threadIdx.x; j < 2 * C; j += blockDim.x) {
      float a = b2[j];
      for (int k = 0; k < se_k; ++k) a = fmaf(hid[k], w2[(long long)j * se_k + k], a);
      z[j] = a;
    }
    __syncthreads();
    if (live) {
      g0 = 1.0f / (1.0f + expf(-z[c]));
      g1 = 1.0f / (1.0f + expf(-z[c + 1]));
      s0 = z[C + c] + g0 * s0;
      s1 = z[C + c + 1] + g1 * s1;
    }
  }
  if (!live) return;
  const T* sk = skip ? skip + board * 64 * C + c : nullptr;
  T* yb = y + board * 64 * C + c;
#pragma unroll
  for (int sq = 0; sq < 64; ++sq) {
    float v0 = fmaf(g0, o[sq][0], s0), v1 = fmaf(g1, o[sq][1], s1);
    if (sk) {
      const float2 e = Pair<T>::load(sk + (long long)sq * C);
      v0 += e.x;
      v1 += e.y;
    }
    Pair<T>::store(yb + (long long)sq * C, activate<true>(v0, act), activate<true>(v1, act));
  }
}

}  // namespace

template <typename T>
cudaError_t launch_wino_input(const T* x, T* v, int C, int boards, long long rows_padded, cudaStream_t s) {
  if (boards <= 0) return cudaSuccess;
  if (C % 2) return cudaErrorInvalidValue;
  const long long patches = (long long)boards * 4, work = patches * (C / 2);
  wino_input_kernel<T><<<(unsigned)((work + 255) / 256), 256, 0, s>>>(x, v, C, patches, rows_padded);
  return cudaGetLastError();
}
template cudaError_t launch_wino_input<__half>(const __half*, __half*, int, int, long long, cudaStream_t);
template cudaError_t launch_wino_input<__nv_bfloat16>(const __nv_bfloat16*, __nv_bfloat16*, int, int, long long,
                                                      cudaStream_t);

template <typename T>
cudaError_t launch_wino_output(const T* m, const float* bias, const T* skip, const float* se_w1, const float* se_b1,
                               const float* se_w2, const float* se_b2, int se_k, T* y, int C, int boards,
                               long long rows_padded, int act, cudaStream_t s) {
  if (boards <= 0) return cudaSuccess;
  if (C % 2 || C > 512) return cudaErrorInvalidValue;  // one thread per channel pair, at most 256 threads
  const int threads = ((C / 2 + 31) / 32) * 32;
  if (se_k > 0) {
    const size_t smem = (size_t)(3 * C + se_k) * sizeof(float);
    wino_output_kernel<T, true><<<boards, threads, smem, s>>>(m, bias, skip, se_w1, se_b1, se_w2, se_b2, y, C, se_k,
                                                              rows_padded, act);
  } else {
    wino_output_kernel<T, false><<<boards, threads, 0, s>>>(m, bias, skip, nullptr, nullptr, nullptr, nullptr, y, C, 0,
                                                            rows_padded, act);
  }
  return cudaGetLastError();
}
template cudaError_t launch_wino_output<__half>(const __half*, const float*, const __half*, const float*, const float*,
                                                const float*, const float*, int, __half*, int, int, long long, int,
                                                cudaStream_t);
template cudaError_t launch_wino_output<__nv_bfloat16>(const __nv_bfloat16*, const float*, const __nv_bfloat16*,
                                                       const float*, const float*, const float*, const float*, int,
                                                       __nv_bfloat16*, int, int, long long, int, cudaStream_t);

// Filter transform U = G g G^T on the host in fp32: w [Cout][Cin][3][3] (the file's order) -> u [36][Cout][Cin].
void wino_transform_filters(const float* w, int cout, int cin, float* u) {
  static const float G[6][3] = {{1.f / 4, 0.f, 0.f},          {-1.f / 6, -1.f / 6, -1.f / 6}, {-1.f / 6, 1.f / 6, -1.f / 6},
                                {1.f / 24, 1.f / 12, 1.f / 6}, {1.f / 24, -1.f / 12, 1.f / 6}, {0.f, 0.f, 1.f}};
  for (int o = 0; o < cout; ++o)
    for (int c = 0; c < cin; ++c) {
      const float* g = w + ((size_t)o * cin + c) * 9;
      float t[6][3];
      for (int i = 0; i < 6; ++i)
        for (int k = 0; k < 3; ++k) t[i][k] = G[i][0] * g[k] + G[i][1] * g[3 + k] + G[i][2] * g[6 + k];
      for (int i = 0; i < 6; ++i)
        for (int l = 0; l < 6; ++l)
          u[((size_t)(i * 6 + l) * cout + o) * cin + c] = t[i][0] * G[l][0] + t[i][1] * G[l][1] + t[i][2] * G[l][2];
    }
}

}  // namespace b200
