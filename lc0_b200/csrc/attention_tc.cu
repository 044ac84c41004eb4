// Fused 64-token multi-head attention for 16-bit activations, per (position, head):
//
//   S = scale * Q K^T + bias   (bias = the smolgen-generated 64x64 logits of this head, optional)
//   P = softmax_rows(S)
//   O = P V
//
// A warp owns 16 query rows, computes its 16x64 slab of S with m16n8k16 tensor-core MMAs (fp32 accumulation), does
// the softmax in registers (row reductions by quad shuffles) and reuses the probabilities as the A operand of the
// second product.  The problem is 64x64x32 per head, far below one tcgen05 tile, and the operator is bound by the
// HBM traffic of Q/K/V/bias, so the warp-level MMA shape is the right granularity here.
// attention_tma_kernel: persistent CTAs; a producer lane streams the tiles of successive (position, head) items
// into a ring of swizzled shared-memory stages with TMA loads, the compute warps only touch shared memory and hand
// their slab of O to a TMA store.
//
// Reference: BlasComputation::ForwardEncoderLayer, src/neural/backends/blas/network_blas.cc:352-439
// (per-head sgemm, SoftmaxActivation, sgemm); the reference CUDA backend does this with two batched
// cuBLAS calls and softmax_opt_64_kernel (backends/cuda/layers.cc:1803-1850, common_kernels.cu:775-835).
#include <cuda.h>

#include <type_traits>

#include "kernels.cuh"
#include "tma_mma.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// ------------------------------------------------------------------------------------------------
// A CTA is four compute warps and one producer warp and walks over (position, head) items
// blockIdx.x, blockIdx.x + gridDim.x, ...  The producer's elected lane brings the bias tile (64 x 64) and the Q, K, V
// tiles (64 x D) of an item into one stage of a shared-memory ring with four TMA loads (swizzled: 128-byte rows for
// the bias, D*2-byte rows for Q, K, V) that complete on the stage's `full` mbarrier; each compute warp owns 16 query
// rows, releases the stage with an arrival on its `empty` mbarrier after its last read, and writes its 16 x D slab
// of O with a TMA store of its own from one of two swizzled staging slabs.  The compute warps never issue a
// global-memory instruction: a version whose compute warps did their own loads and stores was limited by
// instruction issue (its time followed the SM clock), not by HBM.
// Every mbarrier wait is bounded; a wait that gives up raises the CTA's abort flag and the status word.
// ------------------------------------------------------------------------------------------------
template <int D, int NS> struct AttnTma {
  static constexpr int kRow = D * 2;              // bytes per Q/K/V/O row = the swizzle span
  static constexpr int kTile = 64 * kRow;         // Q, K, V or O tile
  static constexpr int kBias = 64 * 128;          // bias tile, 128-byte rows
  static constexpr int kStage = kBias + 3 * kTile;
  static constexpr int kThreads = 160;
  static constexpr int kBytes = NS * kStage + 2 * kTile + 1024 /*alignment*/ + 128 /*barriers*/;
};
template <typename T, int D, int NS>
__global__ void __launch_bounds__(160, D == 32 ? 4 : 2)
attention_tma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_o, int items, int heads, int has_bias, float scale,
                     int* status) {
  using L = AttnTma<D, NS>;
  extern __shared__ uint8_t sm_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sm_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* outb = sm + NS * L::kStage;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(outb + 2 * L::kTile);
  uint64_t* empty_bar = full_bar + NS;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + NS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid == 128) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    tma_prefetch_map(&map_o);
    if (has_bias) tma_prefetch_map(&map_b);
  }
  __syncthreads();
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
        const int s = it % NS;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / NS) & 1) ^ 1, abort_flag, 1)) break;
        const int n = item / heads, h = item - n * heads;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t base = smem_u32(sm + s * L::kStage);
        mbar_expect_tx(bar, has_bias ? L::kStage : 3 * L::kTile);
        if (has_bias) tma_load_2d(base, &map_b, 0, item * 64, bar);
        tma_load_2d(base + L::kBias, &map_q, h * D, n * 64, bar);
        tma_load_2d(base + L::kBias + L::kTile, &map_k, h * D, n * 64, bar);
        tma_load_2d(base + L::kBias + 2 * L::kTile, &map_v, h * D, n * 64, bar);
      }
    }
  } else {
    // ---------------- compute: warp w owns query rows 16 w .. 16 w + 15 ----------------
    const int m0 = warp * 16;
    const int g = lane >> 2, t = lane & 3;
    // Per-lane offsets of the ldmatrix rows in a swizzled tile (the same for every item).  Moving 16 rows down adds
    // 16 * kRow bytes (the swizzle term depends on the row modulo 8 only) and moving two 16-byte chunks to the right
    // flips bit 5 of the offset, so one offset per operand is enough.
    const int a0 = swz<L::kRow>(m0 + (lane & 15), lane >> 4);
    const int k0 = swz<L::kRow>((lane & 7) + (lane >> 4) * 8, (lane >> 3) & 1);
    const int v0 = swz<L::kRow>((lane & 7) + ((lane >> 3) & 1) * 8, lane >> 4);
    const float kLog2e = 1.4426950408889634f;
    uint32_t it = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
      const int s = it % NS;
      const uint8_t* sb = sm + s * L::kStage;
      const uint8_t* sq = sb + L::kBias;
      const uint8_t* sk = sq + L::kTile;
      const uint8_t* sv = sk + L::kTile;
      if (!mbar_wait(smem_u32(&full_bar[s]), (it / NS) & 1, abort_flag, 2)) break;
      // ---- S = Q K^T ----
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, sq + (a0 ^ (ks * 32)));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, sk + np * 16 * L::kRow + (k0 ^ (ks * 32)));
          mma16816<T>(sc[2 * np], a, b[0], b[1]);
          mma16816<T>(sc[2 * np + 1], a, b[2], b[3]);
        }
      }
      // ---- scale, bias, row softmax (rows g and g + 8 of the slab; both have (row & 7) == g) ----
      float mx0 = -3.0e38f, mx1 = -3.0e38f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float2 b0 = make_float2(0.f, 0.f), b1 = make_float2(0.f, 0.f);
        if (has_bias) {
          const int off = ((nt ^ g) << 4) + t * 4;
          b0 = unpack2<T>(*reinterpret_cast<const uint32_t*>(sb + (m0 + g) * 128 + off));
          b1 = unpack2<T>(*reinterpret_cast<const uint32_t*>(sb + (m0 + g + 8) * 128 + off));
        }
        sc[nt][0] = fmaf(sc[nt][0], scale, b0.x);
        sc[nt][1] = fmaf(sc[nt][1], scale, b0.y);
        sc[nt][2] = fmaf(sc[nt][2], scale, b1.x);
        sc[nt][3] = fmaf(sc[nt][3], scale, b1.y);
        mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float nm0 = -mx0 * kLog2e, nm1 = -mx1 * kLog2e;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sc[nt][0] = ex2_approx(fmaf(sc[nt][0], kLog2e, nm0));
        sc[nt][1] = ex2_approx(fmaf(sc[nt][1], kLog2e, nm0));
        sc[nt][2] = ex2_approx(fmaf(sc[nt][2], kLog2e, nm1));
        sc[nt][3] = ex2_approx(fmaf(sc[nt][3], kLog2e, nm1));
        sum0 += sc[nt][0] + sc[nt][1];
        sum1 += sc[nt][2] + sc[nt][3];
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      const float inv0 = 1.0f / sum0, inv1 = 1.0f / sum1;
      // ---- O = P V (probabilities normalised first, like the reference) ----
      float o[D / 8][4];
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a[4];
        a[0] = pack2<T>(sc[2 * j][0] * inv0, sc[2 * j][1] * inv0);
        a[1] = pack2<T>(sc[2 * j][2] * inv1, sc[2 * j][3] * inv1);
        a[2] = pack2<T>(sc[2 * j + 1][0] * inv0, sc[2 * j + 1][1] * inv0);
        a[3] = pack2<T>(sc[2 * j + 1][2] * inv1, sc[2 * j + 1][3] * inv1);
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, sv + j * 16 * L::kRow + (v0 ^ (np * 32)));
          mma16816<T>(o[2 * np], a, b[0], b[1]);
          mma16816<T>(o[2 * np + 1], a, b[2], b[3]);
        }
      }
      // the stage may be refilled once all four warps are past their last read of it
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
      // ---- this warp's 16 x D slab: swizzled staging slab (one of two) -> TMA store of its own ----
      uint8_t* ob = outb + (it & 1) * L::kTile + warp * (16 * L::kRow);
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // the store of two items ago
      __syncwarp();
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<uint32_t*>(ob + swz<L::kRow>(g, nt) + t * 4) = pack2<T>(o[nt][0], o[nt][1]);
        *reinterpret_cast<uint32_t*>(ob + swz<L::kRow>(g + 8, nt) + t * 4) = pack2<T>(o[nt][2], o[nt][3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        const int n = item / heads, h = item - n * heads;
        tma_store_2d(&map_o, h * D, n * 64 + m0, smem_u32(ob));
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    // the staging slabs must outlive the stores' reads of them; the grid's end completes the writes
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  __syncthreads();
  if (*abort_flag) {
    // Give loads that may still be in flight time to land before the CTA's shared memory is released.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (tid == 0 && status) atomicCAS(status, 0, 300 + *abort_flag);
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

template <typename T, int D, int NS>
static cudaError_t launch_attention_tma_cfg(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                                            long long ldo, int n, int heads, float scale, int* status, int sm_count,
                                            int ctas_per_sm, cudaStream_t s) {
  using L = AttnTma<D, NS>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (!attr_done[dev & 63]) {
    e = cudaFuncSetAttribute(attention_tma_kernel<T, D, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  const int prec = sizeof(T) == 2 && std::is_same<T, __half>::value ? 1 : 2;
  const long long rows = (long long)n * 64;
  CUtensorMap mq, mk, mv, mb, mo;
  if ((e = tma_encode_2d(q, ld, rows, heads * D, D, 64, D * 2, prec, &mq)) != cudaSuccess) return e;
  if ((e = tma_encode_2d(k, ld, rows, heads * D, D, 64, D * 2, prec, &mk)) != cudaSuccess) return e;
  if ((e = tma_encode_2d(v, ld, rows, heads * D, D, 64, D * 2, prec, &mv)) != cudaSuccess) return e;
  if ((e = tma_encode_2d(out, ldo, rows, heads * D, D, 16, D * 2, prec, &mo)) != cudaSuccess) return e;
  mb = mq;
  if (bias && (e = tma_encode_2d(bias, 64, rows * heads, 64, 64, 64, 128, prec, &mb)) != cudaSuccess) return e;
  const int items = n * heads;
  const int max_ctas = sm_count * ctas_per_sm;
  const int grid = items < max_ctas ? items : max_ctas;
  return launch_dependent(attention_tma_kernel<T, D, NS>, dim3(grid), dim3(L::kThreads), L::kBytes, s, mq, mk, mv, mb, mo,
                          items, heads, bias ? 1 : 0, scale, status);
}

template <typename T>
cudaError_t launch_attention_tma(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                                 long long ldo, int n, int heads, int depth, float scale, int* status, int sm_count,
                                 cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  // depth 32: two 20 KB stages and four CTAs per SM (sixteen compute warps) measured best: with three or two CTAs
  // the kernel waits on its compute warps, more stages per CTA buy nothing.
  if (depth == 32) return launch_attention_tma_cfg<T, 32, 2>(q, k, v, ld, bias, out, ldo, n, heads, scale, status,
                                                             sm_count, 4, s);
  if (depth == 64) return launch_attention_tma_cfg<T, 64, 2>(q, k, v, ld, bias, out, ldo, n, heads, scale, status,
                                                             sm_count, 2, s);
  return cudaErrorInvalidValue;
}
template cudaError_t launch_attention_tma<__half>(const __half*, const __half*, const __half*, long long,
                                                  const __half*, __half*, long long, int, int, int, float, int*, int,
                                                  cudaStream_t);
template cudaError_t launch_attention_tma<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*,
                                                         const __nv_bfloat16*, long long, const __nv_bfloat16*,
                                                         __nv_bfloat16*, long long, int, int, int, float, int*, int,
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
