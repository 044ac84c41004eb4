// Fused 64-token multi-head attention for 16-bit activations: one CTA (4 warps) per (position, head).
//
//   S = scale * Q K^T + bias   (bias = the smolgen-generated 64x64 logits of this head, optional)
//   P = softmax_rows(S)
//   O = P V
//
// Q, K, V (64 x depth each) and the bias tile are brought into padded shared memory with 16-byte
// cp.async copies; each warp owns 16 query rows, computes its 16x64 slab of S with m16n8k16 tensor-core
// MMAs (fp32 accumulation), does the softmax in registers (row reductions by quad shuffles), reuses the
// probabilities as the A operand of the second product and writes its 16 x depth slab of O through shared
// memory with 16-byte stores.  The problem is 64x64x32 per head, far below one tcgen05 tile, and the kernel
// is bound by the HBM traffic of Q/K/V/bias, so the warp-level MMA shape is the right granularity here.
//
// Reference: BlasComputation::ForwardEncoderLayer, src/neural/backends/blas/network_blas.cc:352-439
// (per-head sgemm, SoftmaxActivation, sgemm); the reference CUDA backend does this with two batched
// cuBLAS calls and softmax_opt_64_kernel (backends/cuda/layers.cc:1803-1850, common_kernels.cu:775-835).
#include "kernels.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

// Shared-memory rows are padded by 16 bytes so that the eight 16-byte rows an ldmatrix phase (or a quad-row
// bias read) touches fall into distinct bank groups.
template <int D> struct AttnSmem {
  static constexpr int kRow = D * 2 + 16;       // bytes per Q/K/V row
  static constexpr int kBiasRow = 64 * 2 + 16;  // bytes per bias row
  static constexpr int kBytes = 3 * 64 * kRow + 64 * kBiasRow;
};

template <typename T, int D>
__global__ void __launch_bounds__(128)
attention_tc_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                    const T* __restrict__ bias, T* __restrict__ out, long long ldo, int heads, float scale) {
  using L = AttnSmem<D>;
  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* sq = sm;
  uint8_t* sk = sq + 64 * L::kRow;
  uint8_t* sv = sk + 64 * L::kRow;
  uint8_t* sb = sv + 64 * L::kRow;
  const int n = blockIdx.x / heads, h = blockIdx.x - n * heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long base = (long long)n * 64 * ld + (long long)h * D;
  constexpr int kChunks = D / 8;  // 16-byte chunks per row
  for (int i = tid; i < 64 * kChunks; i += 128) {
    const int r = i / kChunks, c = i - r * kChunks;
    const long long g = base + r * ld + c * 8;
    cp_async16(sq + r * L::kRow + c * 16, q + g);
    cp_async16(sk + r * L::kRow + c * 16, k + g);
    cp_async16(sv + r * L::kRow + c * 16, v + g);
  }
  if (bias) {
    const T* bsrc = bias + ((long long)n * heads + h) * 4096;
    for (int i = tid; i < 64 * 8; i += 128) {
      const int r = i >> 3, c = i & 7;
      cp_async16(sb + r * L::kBiasRow + c * 16, bsrc + r * 64 + c * 8);
    }
  }
  cp_async_wait_all();
  __syncthreads();

  const int m0 = warp * 16;
  const int g = lane >> 2, t = lane & 3;
  // ---- S = Q K^T : 8 key tiles of 8, fp32 accumulators ----
  float s[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(a, sq + (m0 + (lane & 15)) * L::kRow + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, sk + (np * 16 + (lane & 7) + (lane >> 4) * 8) * L::kRow + (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
      mma16816<T>(s[2 * np], a, b[0], b[1]);
      mma16816<T>(s[2 * np + 1], a, b[2], b[3]);
    }
  }
  // ---- scale, bias, row softmax (rows g and g+8 of this warp's slab) ----
  float mx0 = -3.0e38f, mx1 = -3.0e38f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    float2 b0 = make_float2(0.f, 0.f), b1 = make_float2(0.f, 0.f);
    if (bias) {
      b0 = unpack2<T>(*reinterpret_cast<const uint32_t*>(sb + (m0 + g) * L::kBiasRow + (nt * 8 + 2 * t) * 2));
      b1 = unpack2<T>(*reinterpret_cast<const uint32_t*>(sb + (m0 + g + 8) * L::kBiasRow + (nt * 8 + 2 * t) * 2));
    }
    s[nt][0] = fmaf(s[nt][0], scale, b0.x);
    s[nt][1] = fmaf(s[nt][1], scale, b0.y);
    s[nt][2] = fmaf(s[nt][2], scale, b1.x);
    s[nt][3] = fmaf(s[nt][3], scale, b1.y);
    mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
    mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = __expf(s[nt][0] - mx0);
    s[nt][1] = __expf(s[nt][1] - mx0);
    s[nt][2] = __expf(s[nt][2] - mx1);
    s[nt][3] = __expf(s[nt][3] - mx1);
    sum0 += s[nt][0] + s[nt][1];
    sum1 += s[nt][2] + s[nt][3];
  }
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
  const float inv0 = 1.0f / sum0, inv1 = 1.0f / sum1;
  // ---- O = P V : probabilities become the A operand (normalised first, like the reference) ----
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {  // 16 keys per step
    uint32_t a[4];
    a[0] = pack2<T>(s[2 * j][0] * inv0, s[2 * j][1] * inv0);
    a[1] = pack2<T>(s[2 * j][2] * inv1, s[2 * j][3] * inv1);
    a[2] = pack2<T>(s[2 * j + 1][0] * inv0, s[2 * j + 1][1] * inv0);
    a[3] = pack2<T>(s[2 * j + 1][2] * inv1, s[2 * j + 1][3] * inv1);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, sv + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * L::kRow + (np * 16 + (lane >> 4) * 8) * 2);
      mma16816<T>(o[2 * np], a, b[0], b[1]);
      mma16816<T>(o[2 * np + 1], a, b[2], b[3]);
    }
  }
  // ---- write the 16 x D slab through this warp's (now unused) Q rows ----
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    *reinterpret_cast<uint32_t*>(sq + (m0 + g) * L::kRow + (nt * 8 + 2 * t) * 2) = pack2<T>(o[nt][0], o[nt][1]);
    *reinterpret_cast<uint32_t*>(sq + (m0 + g + 8) * L::kRow + (nt * 8 + 2 * t) * 2) = pack2<T>(o[nt][2], o[nt][3]);
  }
  __syncwarp();
  for (int i = lane; i < 16 * kChunks; i += 32) {
    const int r = i / kChunks, c = i - r * kChunks;
    const uint4 val = *reinterpret_cast<const uint4*>(sq + (m0 + r) * L::kRow + c * 16);
    *reinterpret_cast<uint4*>(out + ((long long)n * 64 + m0 + r) * ldo + (long long)h * D + c * 8) = val;
  }
}


// ------------------------------------------------------------------------------------------------
// Attention policy head tail on tensor cores, one CTA (4 warps) per position:
//   logits = Q K^T / sqrt(dm)  (64 x 64, dm streamed through shared memory in 64-wide double-buffered chunks),
//   promotion offsets from the rank-8 keys, and the gather of the 1858 move logits, written as fp32.
// Reference: network_blas.cc:850-914; GPU twins: a batched cuBLAS call, promotion_logits_kernel and
// policyMap_kernel (backends/cuda/layers.cc:1898-1979, common_kernels.cu:1116-1201, :703-734).
// ------------------------------------------------------------------------------------------------
constexpr int kPolRow = 64 * 2 + 16;          // bytes per staged row (64 values + padding)
constexpr int kPolStage = 2 * 64 * kPolRow;   // Q chunk + K chunk

template <typename T>
__global__ void __launch_bounds__(128)
policy_attn_tc_kernel(const T* __restrict__ q, const T* __restrict__ k, const float* __restrict__ w4, int dm,
                      const short* __restrict__ src_slot, float scale, float* __restrict__ policy) {
  extern __shared__ __align__(16) uint8_t sm[];
  __shared__ float off[4][8];
  const int n = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* qn = q + (long long)n * 64 * dm;
  const T* kn = k + (long long)n * 64 * dm;
  const int chunks = (dm + 63) / 64;
  auto stage_load = [&](int c, int st) {
    uint8_t* sq = sm + st * kPolStage;
    uint8_t* sk = sq + 64 * kPolRow;
    for (int i = tid; i < 64 * 8; i += 128) {
      const int r = i >> 3, ch = i & 7;
      const int col = c * 64 + ch * 8;
      if (col < dm) {  // dm is a multiple of 8
        cp_async16(sq + r * kPolRow + ch * 16, qn + (long long)r * dm + col);
        cp_async16(sk + r * kPolRow + ch * 16, kn + (long long)r * dm + col);
      } else {
        *reinterpret_cast<uint4*>(sq + r * kPolRow + ch * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sk + r * kPolRow + ch * 16) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float s[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
  stage_load(0, 0);
  const int m0 = warp * 16;
  for (int c = 0; c < chunks; ++c) {
    if (c + 1 < chunks) {
      stage_load(c + 1, (c + 1) & 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint8_t* sq = sm + (c & 1) * kPolStage;
    const uint8_t* sk = sq + 64 * kPolRow;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, sq + (m0 + (lane & 15)) * kPolRow + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, sk + (np * 16 + (lane & 7) + (lane >> 4) * 8) * kPolRow + (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
        mma16816<T>(s[2 * np], a, b[0], b[1]);
        mma16816<T>(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // the stage may be overwritten by the load issued in the next iteration
  }
  // promotion offsets: 4 x 8 dot products of the rank-8 keys with w4 (4 per warp... 8 per warp over 4 warps)
  for (int t = warp * 8; t < warp * 8 + 8; ++t) {
    const int i = t >> 3, j = t & 7;
    const T* key = kn + (long long)(56 + j) * dm;
    float a = 0.f;
    for (int cc = lane; cc < dm; cc += 32) a = fmaf(to_f(key[cc]), w4[i * dm + cc], a);
    a = warp_sum(a);
    if (lane == 0) off[i][j] = a;
  }
  // logits to shared memory (fp32 [64][65]), reusing the staging area
  float* lg = reinterpret_cast<float*>(sm);
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    lg[(m0 + g) * 65 + nt * 8 + 2 * t4] = s[nt][0] * scale;
    lg[(m0 + g) * 65 + nt * 8 + 2 * t4 + 1] = s[nt][1] * scale;
    lg[(m0 + g + 8) * 65 + nt * 8 + 2 * t4] = s[nt][2] * scale;
    lg[(m0 + g + 8) * 65 + nt * 8 + 2 * t4 + 1] = s[nt][3] * scale;
  }
  __syncthreads();
  for (int j = tid; j < 1858; j += 128) {
    const int slot = src_slot[j];
    float v;
    if (slot < 4096) {
      v = lg[(slot >> 6) * 65 + (slot & 63)];
    } else {
      const int r = slot - 4096;  // 24 * from_file + 3 * to_file + piece
      const int kf = r / 24, rem = r - kf * 24, jf = rem / 3, i = rem - jf * 3;
      v = lg[(48 + kf) * 65 + 56 + jf] + off[i][jf] + off[3][jf];
    }
    policy[(long long)n * 1858 + j] = v;
  }
}

}  // namespace

bool attention_tc_supported(long long ld, long long ldo, int depth, const void* q, const void* k, const void* v,
                            const void* bias, const void* out) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return (depth == 32 || depth == 64) && (ld % 8) == 0 && (ldo % 8) == 0 && al(q) && al(k) && al(v) && al(bias) &&
         al(out);
}

template <typename T>
cudaError_t launch_attention_tc(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                                long long ldo, int n, int heads, int depth, float scale, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (depth == 32) {
    attention_tc_kernel<T, 32><<<n * heads, 128, AttnSmem<32>::kBytes, s>>>(q, k, v, ld, bias, out, ldo, heads, scale);
  } else if (depth == 64) {
    attention_tc_kernel<T, 64><<<n * heads, 128, AttnSmem<64>::kBytes, s>>>(q, k, v, ld, bias, out, ldo, heads, scale);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template cudaError_t launch_attention_tc<__half>(const __half*, const __half*, const __half*, long long,
                                                 const __half*, __half*, long long, int, int, int, float,
                                                 cudaStream_t);
template cudaError_t launch_attention_tc<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*,
                                                        const __nv_bfloat16*, long long, const __nv_bfloat16*,
                                                        __nv_bfloat16*, long long, int, int, int, float,
                                                        cudaStream_t);

}  // namespace b200

namespace b200 {

bool policy_attn_tc_supported(int dm, const void* q, const void* k) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return dm >= 8 && (dm % 8) == 0 && al(q) && al(k);
}

template <typename T>
cudaError_t launch_policy_attn_tc(const T* q, const T* k, const float* w4, int dm, const short* src_slot, int n,
                                  float* policy, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  policy_attn_tc_kernel<T><<<n, 128, 2 * kPolStage, s>>>(q, k, w4, dm, src_slot, 1.0f / sqrtf((float)dm), policy);
  return cudaGetLastError();
}
template cudaError_t launch_policy_attn_tc<__half>(const __half*, const __half*, const float*, int, const short*, int,
                                                   float*, cudaStream_t);
template cudaError_t launch_policy_attn_tc<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, const float*, int,
                                                          const short*, int, float*, cudaStream_t);

}  // namespace b200
