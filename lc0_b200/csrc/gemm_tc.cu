// Tensor-core GEMM for sm_100a: C[M][N] = epilogue(A[M][K] . W[N][K]^T), 16-bit inputs, fp32 accumulation.
//
// Structure (one persistent CTA per SM, warp-specialised):
//   TMA producer   cp.async.bulk.tensor 2D loads (no multicast) of a 128x64 A tile and a BNx64 W tile per k-block
//                  into a ring of 128B-swizzled shared-memory stages
//   MMA issuer     tcgen05.mma kind::f16, 128xBNx16 (cta_group::1) or 256xNx16 (cta_group::2) per instruction,
//                  accumulating in tensor memory (TMEM); two accumulators so the epilogue of tile i overlaps the
//                  MMAs of tile i+1
//   epilogue       groups of four warps, one 64-column slab at a time: tcgen05.ld TMEM -> registers, scale, folded
//                  LayerNorm, bias, activation, residual, row statistics, pack -> swizzled staging buffer
//   store warp(s)  TMA stores of the staged slabs, hand-back of the staging buffers, prefetch of residual tiles
// Synchronisation is by mbarriers (full/empty per stage, full/empty per accumulator, full/free per staging
// buffer).  Every wait is bounded by wall-clock time; a wait that gives up raises a status word and all roles leave the kernel.
//
// It computes what the reference obtains from cuBLAS for every dense layer
// (cublasXgemm call sites, src/neural/backends/cuda/layers.cc:1587-1605) fused with the bias/activation
// kernels that follow them there (addBiasBatched / addVectors, backends/cuda/common_kernels.cu:47-309).
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "kernels.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 16-bit elements = one 128-byte swizzle row
constexpr int kThreads = 352;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two groups of four), warp 10 stores
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Same with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds (it is woken when the
// phase completes), so a long wait costs few issue slots of the warps that share its scheduler.
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting (this or another role timed out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    if ((it & 63) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        *abort_flag = code;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// 4D tile load (channels, file, rank, position); coordinates may lie outside the tensor, those elements are
// zero-filled, which is exactly the zero padding of a same-padded convolution on the 8x8 board.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// Brings a tensor map into the descriptor cache ahead of its first use (the first TMA store of a launch otherwise
// waited about three microseconds for it).
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most one of this thread's bulk groups still reads its shared-memory source.
__device__ __forceinline__ void tma_store_wait_read1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


// ---- CTA-pair (cta_group::2) helpers -------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of a CTA of the cluster.  Relaxed: the arrivals of this kernel only hand tensor memory back
// to the MMA issuer (ordered by tcgen05.fence), no generic-proxy data is published through them; a release at
// cluster scope here stalled the arriving thread for 2-3 thousand cycles per tile.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is signalled on a barrier that may live in the peer CTA of the pair (no multicast:
// each CTA of the pair fetches its own half of the operands).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 64 16-bit elements x R rows with CU_TENSOR_MAP_SWIZZLE_128B produces):
// start address >> 4 in bits [0,14), stride between 8-row groups (1024 B) >> 4 in bits [32,46),
// descriptor version 1 in bits [46,48), layout type 2 (SWIZZLE_128B) in bits [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Activation of a register array with the selection hoisted out of the element loop.
template <int N>
__device__ __forceinline__ void apply_activation(float (&v)[N], int act) {
  switch (act) {
    case ACT_RELU:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = fmaxf(v[j], 0.f);
      break;
    case ACT_RELU_2:
#pragma unroll
      for (int j = 0; j < N; ++j) { const float t = fmaxf(v[j], 0.f); v[j] = t * t; }
      break;
    case ACT_MISH:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = mish_f(v[j]);
      break;
    case ACT_SWISH:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = swish_f(v[j]);
      break;
    case ACT_NONE:
      break;
    default:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = activate<true>(v[j], act);
      break;
  }
}

template <typename T> struct FmtCode;
template <> struct FmtCode<__half> { static constexpr uint32_t v = 0; };
template <> struct FmtCode<__nv_bfloat16> { static constexpr uint32_t v = 1; };

// Instruction descriptor of tcgen05.mma.kind::f16: D format fp32 (bits 4-5 = 1), A/B format (bits 7-9,
// 10-12: 0 = f16, 1 = bf16), both operands K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
template <typename T, int BN>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (1u << 4) | (FmtCode<T>::v << 7) | (FmtCode<T>::v << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

struct TcParams {
  const float* bias;
  void* C;
  long long ldc;
  int M, N, K;
  int act;
  float scale, alpha;
  int out_f32;
  int* status;
  int tma_store;  // 1: 16-bit output staged in shared memory and written with TMA stores
  // CTA-pair kernel: the tiles from split_from on are computed as two half-width tiles each (tiles_v virtual tiles in
  // all), so that a last, less than half filled wave spreads over all pairs; split_from >= tiles_v means no split
  int split_from, tiles_v;
  int conv_cblocks;  // > 0: 3x3 convolution, number of 64-channel blocks of the input (k_blocks = 9 * conv_cblocks)
  // folded LayerNorm (see GemmParams)
  const double* a_stats; const float* colsum; float a_inv_c, a_eps;
  int res_mode;  // 0 none, 1 add the residual tile, 2 add the normalised residual tile
  const double* res_stats; const float* res_gamma; const float* res_beta; float res_inv_c, res_eps;
  double* out_stats;
  int n_split;  // > 0: columns from here on are stored through the second output map
  // Squeeze-excitation unit fused into the epilogue of a convolution whose tile holds two whole boards and every
  // output channel (se_k > 0; see GemmParams).
  const float* se_w1; const float* se_b1; const float* se_w2; const float* se_b2; const float* se_bias; int se_k;
  int batch_rows;  // > 0: stacked products, rows [b * batch_rows, (b + 1) * batch_rows) use W rows [b * N, (b + 1) * N)
};

// Per-thread (= per output row) state of the folded-LayerNorm epilogue.
// The sums are kept in double: a row whose mean is a hundred standard deviations from zero loses the variance's
// leading digits in fp32 (sum of squares minus squared mean), which the two-pass reference does not.
struct RowCtx {
  float mean_a = 0.f, rstd_a = 1.f, mean_r = 0.f, rstd_r = 1.f;
  double sum = 0.0, sumsq = 0.0;
};
__device__ __forceinline__ void mean_rstd(const double* stats, long long m, float inv_c, float eps, float& mean,
                                          float& rstd) {
  const double2 st = *reinterpret_cast<const double2*>(stats + 2 * m);
  const double mu = st.x * (double)inv_c;
  const double var = fmax(st.y * (double)inv_c - mu * mu, 0.0);
  mean = (float)mu;
  rstd = rsqrtf((float)var + eps);
}
__device__ __forceinline__ void load_row_ctx(const TcParams& p, int m, RowCtx& rc) {
  rc.sum = 0.0;
  rc.sumsq = 0.0;
  if (p.a_stats && m < p.M) mean_rstd(p.a_stats, m, p.a_inv_c, p.a_eps, rc.mean_a, rc.rstd_a);
  if (p.res_mode == 2 && m < p.M) mean_rstd(p.res_stats, m, p.res_inv_c, p.res_eps, rc.mean_r, rc.rstd_r);
}
__device__ __forceinline__ void flush_row_ctx(const TcParams& p, int m, const RowCtx& rc) {
  if (p.out_stats && m < p.M) {
    atomicAdd(p.out_stats + 2 * (long long)m, rc.sum);
    atomicAdd(p.out_stats + 2 * (long long)m + 1, rc.sumsq);
  }
}

// Packs two floats into one 32-bit pair of T; fp16 saturates to the largest finite value.
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));  // first source -> upper half
  return r;
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One 64-column slab of the epilogue fast path, executed by one group of four warps: TMEM -> registers ->
// scale / folded-LayerNorm correction / bias / activation / residual -> 128B-swizzled staging buffer, which the
// store warp then writes out with a TMA store.  A group alternates between two buffers; `free_bar` completes when
// the store that last used `buf` has finished reading it, `full_bar` (four arrivals, one per warp) tells the
// store warp that the slab is staged.  No named barriers: the four warps only meet on those two barriers.
// Per-column vectors (bias, colsum, residual gamma / beta) are fetched with coalesced loads one slab ahead
// (`cr`) and redistributed through a per-warp shared-memory scratch (`wvec`, 4 x 64 floats) as broadcast float4 reads.  The residual tile
// is fetched by TMA into the staging buffer itself (completion on `res_bar`) and combined in place.
// Per-lane slice of the per-column vectors of one slab (columns lane and 32 + lane), fetched one slab ahead.
struct ColRegs {
  float bias0 = 0.f, bias1 = 0.f, cs0 = 0.f, cs1 = 0.f, g0 = 0.f, g1 = 0.f, be0 = 0.f, be1 = 0.f;
};
__device__ __forceinline__ void load_col_regs(const TcParams& p, int nb, int lane, ColRegs& c) {
  auto col = [&](const float* src, int i) { return (src && nb + i < p.N) ? __ldg(src + nb + i) : 0.f; };
  if (p.bias) { c.bias0 = col(p.bias, lane); c.bias1 = col(p.bias, 32 + lane); }
  if (p.a_stats) { c.cs0 = col(p.colsum, lane); c.cs1 = col(p.colsum, 32 + lane); }
  if (p.res_mode == 2) {
    c.g0 = col(p.res_gamma, lane); c.g1 = col(p.res_gamma, 32 + lane);
    c.be0 = col(p.res_beta, lane); c.be1 = col(p.res_beta, 32 + lane);
  }
}

// kMixed (the tower kernel, whose tiles alternate between layers with and without a residual input): the store thread
// arrives on `free_bar` after every store and the group always waits for it; a slab with a residual also waits for
// `res_bar`, whose phase is counted by `res_use` (the number of residual tiles this staging buffer has received).
template <typename T, bool kSe = false, bool kMixed = false>
__device__ __forceinline__ void epilogue_slab(const TcParams& p, uint8_t* buf, uint32_t res_bar, uint32_t free_bar,
                                              uint32_t full_bar, uint32_t use, bool leader, uint32_t taddr, int row,
                                              int lane, int nb, int next_nb, ColRegs& cr, float* wvec, RowCtx& rc,
                                              volatile int* abort_flag, const float* se_arg = nullptr,
                                              uint32_t res_use = 0) {
  const float* se = kSe ? se_arg : nullptr;  // compiled out of the kernels that never fuse squeeze-excitation
  // se != nullptr: gate (se[0..63]) and shift (se[256..319]) of this row's sample for the slab's 64 columns; the
  // activation then follows the residual: act(gate * v + shift + residual)   (se_unit.cc:54-61)
  __syncwarp();  // the previous slab's reads of wvec are done
  if (p.bias) { wvec[lane] = cr.bias0; wvec[32 + lane] = cr.bias1; }
  if (p.a_stats) { wvec[64 + lane] = cr.cs0; wvec[96 + lane] = cr.cs1; }
  if (p.res_mode == 2) {
    wvec[128 + lane] = cr.g0; wvec[160 + lane] = cr.g1;
    wvec[192 + lane] = cr.be0; wvec[224 + lane] = cr.be1;
  }
  __syncwarp();
  if (next_nb >= 0) load_col_regs(p, next_nb, lane, cr);  // in flight during the arithmetic below
  uint8_t* srow = buf + row * 128;
  // The slab is processed as two halves of 32 columns (keeps the register footprint of an epilogue thread small
  // enough for sixteen epilogue warps per CTA).
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    uint32_t r[32];
    tmem_ld32(taddr + 32 * h, r);
    tmem_ld_wait();
    float v[32];
    if (p.scale != 1.0f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.scale;
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    }
    if (p.a_stats) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 cs = *reinterpret_cast<const float4*>(wvec + 64 + 32 * h + j);
        v[j] = rc.rstd_a * (v[j] - rc.mean_a * cs.x);
        v[j + 1] = rc.rstd_a * (v[j + 1] - rc.mean_a * cs.y);
        v[j + 2] = rc.rstd_a * (v[j + 2] - rc.mean_a * cs.z);
        v[j + 3] = rc.rstd_a * (v[j + 3] - rc.mean_a * cs.w);
      }
    }
    if (se) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 g = *reinterpret_cast<const float4*>(se + 32 * h + j);
        const float4 b = *reinterpret_cast<const float4*>(se + 256 + 32 * h + j);
        v[j] = fmaf(g.x, v[j], b.x); v[j + 1] = fmaf(g.y, v[j + 1], b.y);
        v[j + 2] = fmaf(g.z, v[j + 2], b.z); v[j + 3] = fmaf(g.w, v[j + 3], b.w);
      }
    } else {
      if (p.bias) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 b = *reinterpret_cast<const float4*>(wvec + 32 * h + j);
          v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
        }
      }
      apply_activation(v, p.act);
    }
    if (h == 0) {
      // Every thread does its own bounded wait (after a failed wait the result is meaningless and the status word
      // says so): for the residual tile, which the store warp fetched into `buf` once the buffer was free, or
      // for the buffer itself.
      if (kMixed) {
        mbar_wait(free_bar, (use & 1) ^ 1, abort_flag, 6);
        if (p.res_mode) mbar_wait(res_bar, res_use & 1, abort_flag, 5);
      } else {
        if (p.res_mode) mbar_wait(res_bar, use & 1, abort_flag, 5);
        else mbar_wait(free_bar, (use & 1) ^ 1, abort_flag, 6);
      }
    }
    if (p.res_mode) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int cc = 4 * h + c;
        const uint4 u = *reinterpret_cast<const uint4*>(srow + ((cc ^ (row & 7)) << 4));
        const T* e = reinterpret_cast<const T*>(&u);
        float s[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = to_f(e[i]);
        if (p.res_mode == 2) {
          const float4 g0 = *reinterpret_cast<const float4*>(wvec + 128 + cc * 8);
          const float4 g1 = *reinterpret_cast<const float4*>(wvec + 132 + cc * 8);
          const float4 b0 = *reinterpret_cast<const float4*>(wvec + 192 + cc * 8);
          const float4 b1 = *reinterpret_cast<const float4*>(wvec + 196 + cc * 8);
          const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
          const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          const float sh = -rc.mean_r * rc.rstd_r;
#pragma unroll
          for (int i = 0; i < 8; ++i) s[i] = fmaf(fmaf(s[i], rc.rstd_r, sh), gg[i], bb[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c * 8 + i] = fmaf(p.alpha, v[c * 8 + i], s[i]);
      }
    }
    if (se) apply_activation(v, p.act);
    if (p.out_stats) {
      float a = 0.f, q = 0.f;
      const int nh = nb + 32 * h;
      if (nh + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 32; ++j) { a += v[j]; q = fmaf(v[j], v[j], q); }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (nh + j < p.N) { a += v[j]; q = fmaf(v[j], v[j], q); }
      }
      rc.sum += (double)a;  // 32-column partial sums in fp32, their total in double
      rc.sumsq += (double)q;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int cc = 4 * h + c;
      uint4 o;
      o.x = pack_pair<T>(v[c * 8 + 0], v[c * 8 + 1]);
      o.y = pack_pair<T>(v[c * 8 + 2], v[c * 8 + 3]);
      o.z = pack_pair<T>(v[c * 8 + 4], v[c * 8 + 5]);
      o.w = pack_pair<T>(v[c * 8 + 6], v[c * 8 + 7]);
      *reinterpret_cast<uint4*>(srow + ((cc ^ (row & 7)) << 4)) = o;
    }
  }
  fence_async_smem();  // this thread's writes are visible to the TMA store the store warp will issue
  __syncwarp();
  if (lane == 0) mbar_arrive(full_bar);
}

// Sum over the warp's 32 lanes of each of 32 per-lane values: afterwards v[0] of lane j is the sum of column j.
// Halving exchange (16 + 8 + 4 + 2 + 1 shuffles) instead of 32 full reductions.
__device__ __forceinline__ void warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = upper ? v[i] : v[i + off];
      const float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

// Barrier among the 256 epilogue threads of a CTA on an mbarrier, with the bounded wait of every other wait here.
__device__ __forceinline__ void epilogue_barrier(uint32_t bar, uint32_t& phase, volatile int* abort_flag) {
  mbar_arrive(bar);
  mbar_wait(bar, phase & 1, abort_flag, 8);
  ++phase;
}

// Squeeze-excitation vectors of the two boards of a convolution tile (ApplySEUnit, backends/blas/se_unit.cc:31-63):
// pool = mean over the 64 squares of the accumulator + conv bias, hid = act(W1 pool + b1), z = W2 hid + b2,
// gate = sigmoid(z[:C]), shift = z[C:] + gate * conv bias.  Runs on the eight epilogue warps while the accumulator
// stays in tensor memory; `gb` receives [2 boards][gate 256 | shift 256].  `tmp` is the per-warp scratch area of the
// slabs (2048 floats), free between two tiles.
template <int BN>
__device__ __forceinline__ void se_prepare(const TcParams& p, uint32_t trow, int quarter, int group, int lane, int eid,
                                           float* tmp, float* gb, uint32_t bar, uint32_t& phase,
                                           volatile int* abort_flag, const float* w_smem = nullptr,
                                           const float* v_smem = nullptr) {
  // w_smem: se_w1 [se_k][C] and se_w2 [2C][se_k]; v_smem: se_bias [C], se_b1 [se_k], se_b2 [2C]: copies in shared
  // memory, made while the tile was computed.  What is not there is read from global memory, and each of the five
  // is then one more round trip in a chain of dependent ones.
  const float* g_w1 = w_smem ? w_smem : p.se_w1;
  const float* g_w2 = w_smem ? g_w1 + p.se_k * p.N : p.se_w2;
  const float* g_bias = v_smem ? v_smem : p.se_bias;
  const float* g_b1 = v_smem ? g_bias + p.N : p.se_b1;
  const float* g_b2 = v_smem ? g_b1 + p.se_k : p.se_b2;
  auto ld = [&](const float* q) { return v_smem ? *q : __ldg(q); };
  auto ld4 = [&](const float4* q) { return w_smem ? *q : __ldg(q); };
  float* part = tmp;          // [4 quarters][256] column sums over 32 rows
  float* pool = tmp + 1024;   // [2][256]
  float* hid = tmp + 1536;    // [2][64]
  const int C = p.N;
  epilogue_barrier(bar, phase, abort_flag);  // nobody still reads the previous tile's per-warp vectors in `tmp`
#pragma unroll 1
  for (int c0 = group * 64; c0 < BN; c0 += 128) {
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      tmem_ld32(trow + c0 + 32 * h, r);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      warp_column_sums(v, lane);
      part[quarter * 256 + c0 + 32 * h + lane] = v[0];
    }
  }
  epilogue_barrier(bar, phase, abort_flag);
  {
    const int c = eid;  // 256 threads, one channel each
    const float b = c < C ? ld(g_bias + c) : 0.f;
    pool[c] = (part[c] + part[256 + c]) * (1.0f / 64.0f) + b;
    pool[256 + c] = (part[512 + c] + part[768 + c]) * (1.0f / 64.0f) + b;
  }
  epilogue_barrier(bar, phase, abort_flag);
  // hid[s][k]: four threads per output, a quarter of the channels each (C is a multiple of 16 and se_k of 4, so the
  // quads of a warp run the same trip count).  The weights come from L2: 16-byte loads, several in flight, so that
  // the whole dot product costs about one round trip.
  for (int o = eid >> 2; o < 2 * p.se_k; o += 64) {
    const int sidx = o / p.se_k, k = o - sidx * p.se_k;
    // the four threads of an output take every fourth 16-byte piece of the row: consecutive addresses (no bank
    // conflicts in shared memory, whole lines per quad in global memory)
    const float4* w = reinterpret_cast<const float4*>(g_w1 + (long long)k * C) + (eid & 3);
    const float4* x = reinterpret_cast<const float4*>(pool + sidx * 256) + (eid & 3);
    float a = 0.f;
#pragma unroll 8
    for (int i = 0; i < (C >> 2); i += 4) {
      const float4 wv = ld4(w + i), xv = x[i];
      a = fmaf(wv.x, xv.x, fmaf(wv.y, xv.y, fmaf(wv.z, xv.z, fmaf(wv.w, xv.w, a))));
    }
    a += __shfl_xor_sync(0xffffffffu, a, 1);
    a += __shfl_xor_sync(0xffffffffu, a, 2);
    if ((eid & 3) == 0) hid[sidx * 64 + k] = activate<false>(a + ld(g_b1 + k), p.act);
  }
  epilogue_barrier(bar, phase, abort_flag);
  if (eid < C) {
    const int c = eid;
    float z0a = ld(g_b2 + c), z1a = ld(g_b2 + C + c), z0b = z0a, z1b = z1a;
    const float4* w0 = reinterpret_cast<const float4*>(g_w2 + (long long)c * p.se_k);
    const float4* w1 = reinterpret_cast<const float4*>(g_w2 + (long long)(C + c) * p.se_k);
    // in shared memory the 16-byte pieces of row r sit at position k ^ (r & 7) (eight or more pieces per row): thread c
    // reads row c, and without the swizzle every lane of a warp would hit the same banks
    const int swz = (w_smem && p.se_k >= 32) ? (c & 7) : 0;  // (C + c) & 7 == c & 7: C is a multiple of 16
    const float4* ha = reinterpret_cast<const float4*>(hid);
    const float4* hb = reinterpret_cast<const float4*>(hid + 64);
#pragma unroll 8
    for (int k = 0; k < (p.se_k >> 2); ++k) {
      const float4 a = ld4(w0 + (k ^ swz)), b = ld4(w1 + (k ^ swz)), xa = ha[k], xb = hb[k];
      z0a = fmaf(a.x, xa.x, fmaf(a.y, xa.y, fmaf(a.z, xa.z, fmaf(a.w, xa.w, z0a))));
      z1a = fmaf(b.x, xa.x, fmaf(b.y, xa.y, fmaf(b.z, xa.z, fmaf(b.w, xa.w, z1a))));
      z0b = fmaf(a.x, xb.x, fmaf(a.y, xb.y, fmaf(a.z, xb.z, fmaf(a.w, xb.w, z0b))));
      z1b = fmaf(b.x, xb.x, fmaf(b.y, xb.y, fmaf(b.z, xb.z, fmaf(b.w, xb.w, z1b))));
    }
    const float cb = ld(g_bias + c);
    const float ga = 1.0f / (1.0f + expf(-z0a)), gbb = 1.0f / (1.0f + expf(-z0b));
    gb[c] = ga; gb[256 + c] = z1a + ga * cb;
    gb[512 + c] = gbb; gb[768 + c] = z1b + gbb * cb;
  } else {
    gb[eid] = 0.f; gb[256 + eid] = 0.f; gb[512 + eid] = 0.f; gb[768 + eid] = 0.f;
  }
  epilogue_barrier(bar, phase, abort_flag);
}

// A store thread's side of the fast path: for every slab of this CTA's tiles that belongs to the epilogue groups
// [g_lo, g_hi), in the order the groups produce them, wait until the slab is staged, write it out with a TMA store,
// and hand the staging buffer back once the store has finished reading shared memory (with two buffers per group
// one store stays in flight, with one buffer the thread waits for the read right away).  With a residual input the
// same thread fetches the residual tiles: kBufs slabs ahead per group, each into the staging buffer its slab will
// use, as soon as that buffer is free; the epilogue threads then only wait for the tile to have landed.
struct SlabWalk {
  const TcParams& p;
  int first_tile, tile_step, tiles, n_tiles, tile_rows, row_offset, bn, groups;
  int split_from;  // virtual tiles from here on are half-width halves of the tiles split_from, split_from + 1, ...
  __device__ __forceinline__ int tile(int t) const { return t < split_from ? t : split_from + ((t - split_from) >> 1); }
  __device__ __forceinline__ int width(int t) const { return t < split_from ? bn : bn / 2; }
  __device__ __forceinline__ int n0(int t) const {
    return (tile(t) % n_tiles) * bn + (t < split_from ? 0 : ((t - split_from) & 1) * (bn / 2));
  }
  __device__ __forceinline__ int m0(int t) const { return (tile(t) / n_tiles) * tile_rows + row_offset; }
  // cursor over the slabs of one epilogue group (columns g*64, (g + groups)*64, ... of each tile)
  struct Cursor { int t, c0; };
  __device__ __forceinline__ void settle(Cursor& c, int g) const {
    while (c.t < tiles && (c.c0 >= width(c.t) || n0(c.t) + c.c0 >= p.N)) { c.t += tile_step; c.c0 = g * 64; }
  }
  __device__ __forceinline__ Cursor begin(int g) const {
    Cursor c{first_tile, g * 64};
    settle(c, g);
    return c;
  }
  __device__ __forceinline__ void next(Cursor& c, int g) const {
    c.c0 += 64 * groups;
    if (c.c0 >= width(c.t) || n0(c.t) + c.c0 >= p.N) { c.t += tile_step; c.c0 = g * 64; }
    settle(c, g);
  }
};

template <int kGroups, int kBufs>
__device__ __forceinline__ void store_warp_loop(const TcParams& p, const CUtensorMap* tmap_c, const CUtensorMap* tmap_c2,
                                                const CUtensorMap* tmap_r, uint8_t* epi_mem, uint64_t* stg_full, uint64_t* stg_free,
                                                uint64_t* res_bar, int g_lo, int g_hi, int first_tile, int tile_step,
                                                int tiles, int n_tiles, int tile_rows, int row_offset, int bn,
                                                int split_from, volatile int* abort_flag) {
  const SlabWalk w{p, first_tile, tile_step, tiles, n_tiles, tile_rows, row_offset, bn, kGroups, split_from};
  SlabWalk::Cursor pf[kGroups];
  uint32_t pf_count[kGroups], count[kGroups];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    pf[g] = w.begin(g);
    pf_count[g] = 0;
    count[g] = 0;
  }
  auto fetch_residual = [&](int g) {
    if (pf[g].t >= tiles) return;
    const int idx = g * kBufs + (int)(pf_count[g] % kBufs);
    const uint32_t bar = smem_u32(&res_bar[idx]);
    mbar_expect_tx(bar, BM * 128);
    tma_load_2d(smem_u32(epi_mem + idx * (BM * 128)), tmap_r, w.n0(pf[g].t) + pf[g].c0, w.m0(pf[g].t), bar);
    ++pf_count[g];
    w.next(pf[g], g);
  };
  // a staging buffer has been read out by its store: fetch the next residual tile into it, or tell the group
  auto release = [&](int idx) {
    if (p.res_mode) fetch_residual(idx / kBufs);
    else mbar_arrive(smem_u32(&stg_free[idx]));
  };
  if (p.res_mode)
    for (int k = 0; k < kBufs; ++k)
      for (int g = g_lo; g < g_hi; ++g) fetch_residual(g);
  int prev = -1;
  bool ok = true;
  for (int t = first_tile; t < tiles && ok; t += tile_step) {
    const int m0 = w.m0(t), n0 = w.n0(t), width = w.width(t);
    for (int c0 = 0; c0 < width; c0 += 64) {
      if (n0 + c0 >= p.N) break;
      const int g = (c0 >> 6) % kGroups;
      if (g < g_lo || g >= g_hi) continue;
      const uint32_t s = count[g]++;
      const int idx = g * kBufs + (int)(s % kBufs);
      if (!mbar_wait(smem_u32(&stg_full[idx]), (s / kBufs) & 1, abort_flag, 7)) { ok = false; break; }
      if (p.n_split > 0 && n0 >= p.n_split)
        tma_store_2d(tmap_c2, n0 + c0 - p.n_split, m0, smem_u32(epi_mem + idx * (BM * 128)));
      else
        tma_store_2d(tmap_c, n0 + c0, m0, smem_u32(epi_mem + idx * (BM * 128)));
      tma_store_commit();
      if (kBufs == 1) {
        tma_store_wait_read0();
        release(idx);
      } else {
        if (prev >= 0) {
          tma_store_wait_read1();
          release(prev);
        }
        prev = idx;
      }
    }
  }
  // The CTA's shared memory must outlive the stores' reads of it; the writes themselves are complete, and visible to
  // the next kernel of the stream, when the grid has finished.
  tma_store_wait_read0();
}

template <int BN> struct TileCfg {
  // stages + 64 KB of epilogue staging + 3.3 KB must stay below the 227 KB a CTA may use
  static constexpr int kStageBytes = (BM + BN) * BK * 2;
  static constexpr int kStages = BN == 256 ? 3 : (BN == 128 ? 4 : 6);
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kEpiBytes = 4 * BM * 128;  // 2 groups x 2 staging buffers of 128 rows x 128 bytes
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 512 /*barriers*/ +
                                    8192 /*per-warp column vectors*/ + 4096 /*squeeze-excitation gate and shift*/ +
                                    4096 /*squeeze-excitation bias vectors*/;
};


template <typename T, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
               const TcParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_mem = smem + S * Cfg::kStageBytes;
  uint8_t* bar_mem = epi_mem + Cfg::kEpiBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);       // [S]
  uint64_t* empty_bar = full_bar + S;                               // [S]
  uint64_t* tfull_bar = empty_bar + S;                              // [2]
  uint64_t* tempty_bar = tfull_bar + 2;                             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* res_bar = reinterpret_cast<uint64_t*>(bar_mem + 192);   // [2 groups][2 buffers] residual tile landed
  uint64_t* stg_full = reinterpret_cast<uint64_t*>(bar_mem + 256);  // [2 groups][2 buffers] slab staged (4 warps)
  uint64_t* stg_free = stg_full + 4;                                // [2 groups][2 buffers] store has read the buffer
  float* wvec_all = reinterpret_cast<float*>(bar_mem + 512);                                // 8 warps x 256 floats
  float* wvec = wvec_all + ((threadIdx.x >> 5) & 7) * 256;                                  // per-warp scratch
  uint64_t* se_bar = reinterpret_cast<uint64_t*>(bar_mem + 384);    // barrier of the 256 epilogue threads
  float* se_gb = reinterpret_cast<float*>(bar_mem + 512 + 8192);    // [2 boards][gate 256 | shift 256]
  float* se_vec = se_gb + 1024;                                     // se_bias [N], se_b1 [se_k], se_b2 [2N]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = p.conv_cblocks > 0 ? 9 * p.conv_cblocks : (p.K + BK - 1) / BK;

  if (threadIdx.x == 32) {
    tma_prefetch_map(&tmap_a);
    tma_prefetch_map(&tmap_w);
    tma_prefetch_map(&tmap_c);
    if (p.res_mode) tma_prefetch_map(&tmap_r);
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&res_bar[i]), 1);
      mbar_init(smem_u32(&stg_full[i]), 4);
      mbar_init(smem_u32(&stg_free[i]), 1);
    }
    mbar_init(smem_u32(se_bar), 256);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();  // everything above overlapped the kernel before this one
  grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        const int m0 = (t / n_tiles) * BM, n0 = (t % n_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, 1)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, Cfg::kStageBytes);
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          if (p.conv_cblocks > 0) {
            // k-block = (filter tap, 64-channel block): the A tile is the board shifted by the tap.
            const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
            tma_load_4d(sa, &tmap_a, cb * BK, tap % 3 - 1, tap / 3 - 1, m0 >> 6, fb);
            tma_load_2d(sa + BM * BK * 2, &tmap_w, cb * BK, tap * p.N + n0, fb);
          } else {
            tma_load_2d(sa, &tmap_a, kb * BK, m0, fb);
            tma_load_2d(sa + BM * BK * 2, &tmap_w, kb * BK, n0 + (p.batch_rows > 0 ? (m0 / p.batch_rows) * p.N : 0), fb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<T, BN>();
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_it) {
        const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abort_flag, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + BM * BK * 2);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advancing 16 elements (32 bytes) along K inside the swizzle row = +2 in the address field
            tcgen05_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));  // frees the stage once the MMAs have read it
        }
        if (ok) tcgen05_commit(smem_u32(&tfull_bar[acc]));
      }
    }
  } else if (warp == 10) {
    // ---------------- store warp: TMA stores of the staged slabs ----------------
    if (lane == 0 && p.tma_store)
      store_warp_loop<2, 2>(p, &tmap_c, &tmap_c, &tmap_r, epi_mem, stg_full, stg_free, res_bar, 0, 2, blockIdx.x, gridDim.x,
                            tiles, n_tiles, BM, 0, BN, 0x7fffffff, abort_flag);
  } else {
    // ---------------- epilogue (warps 2..9: two groups of four warps, alternating 64-column slabs) ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
    const int group = (warp - 2) >> 2;
    const bool leader = ((warp - 2) & 3) == 0 && lane == 0;
    uint8_t* gbuf = epi_mem + group * (2 * BM * 128);
    uint32_t tile_it = 0, slab_it = 0, se_phase = 0;
    ColRegs cr;
    int cr_nb = -1;  // first column of the slab whose vectors `cr` holds
    bool se_vec_ok = false;
    if constexpr (BN == 256) {
      if (p.se_k > 0 && 3 * p.N + p.se_k <= 1024) {
        // the squeeze-excitation bias vectors into shared memory while the first tile is computed (the first
        // barrier of se_prepare orders these stores before the reads)
        const int eid = (int)threadIdx.x - 64;
        for (int i = eid; i < p.N; i += 256) se_vec[i] = __ldg(p.se_bias + i);
        for (int i = eid; i < p.se_k; i += 256) se_vec[p.N + i] = __ldg(p.se_b1 + i);
        for (int i = eid; i < 2 * p.N; i += 256) se_vec[p.N + p.se_k + i] = __ldg(p.se_b2 + i);
        se_vec_ok = true;
      }
    }
    if ((int)blockIdx.x < tiles && ((int)blockIdx.x % n_tiles) * BN + group * 64 < p.N) {
      cr_nb = ((int)blockIdx.x % n_tiles) * BN + group * 64;  // first slab: fetched while the first tile is computed
      load_col_regs(p, cr_nb, lane, cr);
    }
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
      const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
      const int m0 = (t / n_tiles) * BM, n0 = (t % n_tiles) * BN;
      // Every thread does its own bounded wait; the roles only meet on mbarriers, so a thread that gives up
      // (the abort flag is then set and every other wait returns soon) leaves nobody behind at a barrier.
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag, 4)) break;
      tcgen05_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if (p.tma_store) {
        // Fast path: 64-column slabs -> registers -> swizzled shared memory -> TMA store (clips the M/N tails).
        RowCtx rc;
        load_row_ctx(p, m, rc);
        const float* se_row = nullptr;
        if constexpr (BN == 256) {
          if (p.se_k > 0) {  // one tile = two boards x all channels: the squeeze-excitation vectors of both boards
            se_prepare<BN>(p, trow, quarter, group, lane, (int)threadIdx.x - 64, wvec_all, se_gb, smem_u32(se_bar),
                           se_phase, abort_flag, nullptr, se_vec_ok ? se_vec : nullptr);
            se_row = se_gb + (quarter >> 1) * 512;
          }
        }
#pragma unroll 1
        for (int c0 = group * 64; c0 < BN; c0 += 128) {
          if (n0 + c0 >= p.N) break;  // uniform over the group
          const int idx = group * 2 + (int)(slab_it & 1);
          if (cr_nb != n0 + c0) load_col_regs(p, n0 + c0, lane, cr);
          // the slab this group handles next: further right in this tile, else the first one of its next tile
          int next_nb = -1;
          if (c0 + 128 < BN && n0 + c0 + 128 < p.N) {
            next_nb = n0 + c0 + 128;
          } else if (t + (int)gridDim.x < tiles) {
            const int nn = ((t + (int)gridDim.x) % n_tiles) * BN + group * 64;
            if (nn < p.N) next_nb = nn;
          }
          cr_nb = next_nb;
          epilogue_slab<T, BN == 256>(p, gbuf + (slab_it & 1) * (BM * 128), smem_u32(&res_bar[idx]), smem_u32(&stg_free[idx]),
                           smem_u32(&stg_full[idx]), slab_it >> 1, leader, trow + c0, quarter * 32 + lane, lane,
                           n0 + c0, next_nb, cr, wvec, rc, abort_flag, se_row ? se_row + c0 : nullptr);
          ++slab_it;
        }
        flush_row_ctx(p, m, rc);
      } else {
#pragma unroll 1
      for (int c0 = group * 32; c0 < BN; c0 += 64) {
        uint32_t r[32];
        tmem_ld32(trow + c0, r);
        tmem_ld_wait();
        const int nb = n0 + c0;
        if (m < p.M && nb < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nb + j;
            float x = __uint_as_float(r[j]) * p.scale;
            if (p.bias && n < p.N) x += __ldg(p.bias + n);
            v[j] = activate<true>(x, p.act);
          }
          if (p.out_f32) {
            float* crow = reinterpret_cast<float*>(p.C) + (long long)m * p.ldc + nb;
            if (nb + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(crow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
              for (int j = 0; j < 32 && nb + j < p.N; ++j) crow[j] = v[j];
            }
          } else {
            T* crow = reinterpret_cast<T*>(p.C) + (long long)m * p.ldc + nb;
            if (nb + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __align__(16) T o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = from_f<T>(v[j + i]);
                *reinterpret_cast<uint4*>(crow + j) = *reinterpret_cast<const uint4*>(o);
              }
            } else {
              for (int j = 0; j < 32 && nb + j < p.N; ++j) crow[j] = from_f<T>(v[j]);
            }
          }
        }
      }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before the CTA's shared memory is released.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, 100 + *abort_flag);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}


// ------------------------------------------------------------------------------------------------
// Tower kernel: every 3x3 convolution of a residual tower in ONE launch.  A CTA owns 128 rows = two whole boards and
// walks the layers for them: a convolution only mixes squares of the same board, and the squeeze-excitation unit
// only pools over a board, so a CTA never needs another CTA's output and the only dependency is its own: the A
// operand of layer l (and its skip input) are rows this CTA stored for an earlier layer.  The store thread waits for
// those stores to complete (cp.async.bulk.wait_group 0) and arrives on a shared-memory barrier that the producer
// waits on before it loads the next layer's A tiles; nothing is waited for across CTAs.  What it removes is the fixed
// cost of 2 x blocks + 1 launches (drain, dependency resolution, prologue, first loads: about 10 us each), which is
// most of the evaluation of a small residual net at the batch sizes a search sends.
//   layers: device array, one entry per convolution (tensor maps of A as boards, W as [9][N][Cin] with boxes of BN
//           rows, C and the skip input; the epilogue parameters incl. the squeeze-excitation unit).
// Roles and barriers are those of gemm_tc_kernel; the staging buffers follow the mixed protocol of epilogue_slab.
// ------------------------------------------------------------------------------------------------
struct alignas(64) TowerLayer {
  CUtensorMap a, w, c, r;
  TcParams p;
};
// Towers of at most 128 output channels: 128x128 tiles, one 64-column slab per epilogue group and tile, so one staging
// buffer per group is enough (the next tile's epilogue is a whole main loop away) and the shared memory goes to the
// pipeline: a CTA alone on its rows is bound by the bytes it has in flight.
struct TowerCfg {
  static constexpr int BN = 128;
  static constexpr int kStageBytes = (BM + BN) * BK * 2;  // 32 KB
  static constexpr int kStages = 4;  // a fifth did not pay, and its 32 KB hold the squeeze-excitation parameters
  static constexpr int kBufs = 1;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kEpiBytes = 2 * kBufs * BM * 128;
  // a layer's squeeze-excitation parameters: two matrices of 128 channels x 32 hidden units and three vectors (fp32)
  static constexpr int kSeWBytes = 48 * 1024 + 2048;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 512 /*barriers*/ +
                                    8192 /*per-warp column vectors*/ + 4096 /*squeeze-excitation gate and shift*/ +
                                    kSeWBytes;
};

// The tiles of one CTA in the order it computes them.  With more row blocks than CTAs (gridDim.x * 2 <= row blocks
// + 1) a CTA takes its blocks two at a time and, for such a pair, goes layer by layer, alternating between the two
// blocks: a tile then depends on the tile before the previous one, so the wait for a block's stores and for the next
// layer's first loads falls under the other block's main loop (9.3 us per tile against 13.8; measured on a tower of 128
// filters).  With fewer blocks each CTA has one: all layers of a block take 21 x 13.8 us, of a pair 21 x 18.5 us.
struct TowerWalk {
  int n_layers, first, step, nb;  // nb: row blocks of this CTA
  int i0 = 0, l = 0, j = 0;       // index of the pair's first block among the CTA's blocks, layer, block of the pair
  __device__ TowerWalk(int n_layers_, int row_blocks) : n_layers(n_layers_), first(blockIdx.x), step(gridDim.x) {
    nb = first < row_blocks ? (row_blocks - first + step - 1) / step : 0;
  }
  __device__ bool valid() const { return i0 < nb; }
  __device__ int rb() const { return first + (i0 + j) * step; }
  __device__ int cnt() const { return nb - i0 >= 2 ? 2 : 1; }  // a CTA with one block (grid = row blocks) never pairs
  __device__ void next() {
    if (++j >= cnt()) {
      j = 0;
      if (++l >= n_layers) { l = 0; i0 += 2; }
    }
  }
};

// Store thread: writes the slabs of this CTA's tiles out in order (two groups, kBufs staging buffers each), counts a
// tile as complete when its stores have landed, and then fetches the skip input of the next tile's slabs into the
// buffers those slabs will use (all are free at that point, and the rows it reads were completed two tiles ago).
__device__ __forceinline__ void tower_store_loop(const TowerLayer* layers, int n_layers, int row_blocks, uint8_t* epi_mem,
                                                 uint64_t* stg_full, uint64_t* stg_free, uint64_t* res_bar,
                                                 uint64_t* done_bar, volatile int* abort_flag) {
  constexpr int BN = TowerCfg::BN, kBufs = TowerCfg::kBufs;
  uint32_t count[2] = {0, 0};  // slabs stored per group
  auto fetch_tile = [&](int rb, int l) {  // skip input of tile (rb, l), slab by slab, into the buffers they will use
    const TowerLayer& L = layers[l];
    if (!L.p.res_mode) return;
    uint32_t k[2] = {count[0], count[1]};
    for (int c0 = 0; c0 < BN && c0 < L.p.N; c0 += 64) {
      const int g = (c0 >> 6) & 1;
      const int idx = g * kBufs + (int)(k[g]++ % kBufs);
      const uint32_t bar = smem_u32(&res_bar[idx]);
      mbar_expect_tx(bar, BM * 128);
      tma_load_2d(smem_u32(epi_mem + idx * (BM * 128)), &L.r, c0, rb * BM, bar);
    }
  };
  bool ok = true;
  for (TowerWalk w(n_layers, row_blocks); w.valid() && ok; w.next()) {
    const TowerLayer& L = layers[w.l];
    const int rb = w.rb();
    for (int c0 = 0; c0 < BN && c0 < L.p.N; c0 += 64) {
      const int g = (c0 >> 6) & 1;
      const uint32_t k = count[g]++;
      const int idx = g * kBufs + (int)(k % kBufs);
      if (!mbar_wait(smem_u32(&stg_full[idx]), (k / kBufs) & 1, abort_flag, 7)) { ok = false; break; }
      tma_store_2d(&L.c, c0, rb * BM, smem_u32(epi_mem + idx * (BM * 128)));
      tma_store_commit();
      tma_store_wait_read0();
      mbar_arrive(smem_u32(&stg_free[idx]));
    }
    if (!ok) break;
    tma_store_wait_all0();    // the tile's rows are in memory
    fence_proxy_async_all();  // ... before the loads of the block's next layer, which the producer issues after the arrival
    mbar_arrive(smem_u32(&done_bar[w.j]));
    TowerWalk nx = w;
    nx.next();
    if (nx.valid()) fetch_tile(nx.rb(), nx.l);  // its source is that block's output of two layers ago
  }
  tma_store_wait_read0();
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_tower_kernel(const TowerLayer* __restrict__ layers, int n_layers, int row_blocks, int* status) {
  using Cfg = TowerCfg;
  constexpr int S = Cfg::kStages, BN = Cfg::BN, kBufs = Cfg::kBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_mem = smem + S * Cfg::kStageBytes;
  uint8_t* bar_mem = epi_mem + Cfg::kEpiBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);       // [S]
  uint64_t* empty_bar = full_bar + S;                               // [S]
  uint64_t* tfull_bar = empty_bar + S;                              // [2]
  uint64_t* tempty_bar = tfull_bar + 2;                             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* res_bar = reinterpret_cast<uint64_t*>(bar_mem + 192);   // [2 groups][2 buffers] skip tile landed
  uint64_t* stg_full = reinterpret_cast<uint64_t*>(bar_mem + 256);  // [2 groups][2 buffers] slab staged (4 warps)
  uint64_t* stg_free = stg_full + 4;                                // [2 groups][2 buffers] store has read the buffer
  uint64_t* se_bar = reinterpret_cast<uint64_t*>(bar_mem + 384);    // barrier of the 256 epilogue threads
  uint64_t* done_bar = se_bar + 1;                                  // [2] the latest tile of block 0 / 1 of the pair is in memory
  float* wvec_all = reinterpret_cast<float*>(bar_mem + 512);        // 8 warps x 256 floats
  float* wvec = wvec_all + ((threadIdx.x >> 5) & 7) * 256;
  float* se_gb = reinterpret_cast<float*>(bar_mem + 512 + 8192);    // [2 boards][gate 256 | shift 256]
  float* se_w = se_gb + 1024;                                       // the layer's squeeze-excitation parameters (kSeWBytes)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    for (int l = 0; l < n_layers; ++l) {
      tma_prefetch_map(&layers[l].a);
      tma_prefetch_map(&layers[l].w);
      tma_prefetch_map(&layers[l].c);
      if (layers[l].p.res_mode) tma_prefetch_map(&layers[l].r);
    }
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&res_bar[i]), 1);
      mbar_init(smem_u32(&stg_full[i]), 4);
      mbar_init(smem_u32(&stg_free[i]), 1);
    }
    mbar_init(smem_u32(se_bar), 256);
    mbar_init(smem_u32(&done_bar[0]), 1);
    mbar_init(smem_u32(&done_bar[1]), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0, nslot[2] = {0, 0};  // nslot: tiles issued per block of the pair
      bool ok = true;
      for (TowerWalk w(n_layers, row_blocks); w.valid() && ok; w.next()) {
        const TowerLayer& L = layers[w.l];
        const int rb = w.rb();
        const int cblocks = L.p.conv_cblocks, k_blocks = 9 * cblocks, N = L.p.N;
        // The filters do not depend on this CTA's earlier output: those of the first stages are requested before
        // the wait for it.
        const int early = k_blocks < S ? k_blocks : S;
        for (int kb = 0; kb < early && ok; ++kb) {
          const int s = (it + kb) % S;
          const uint32_t ph = ((it + kb) / S) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, 1)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, Cfg::kStageBytes);
          const int tap = kb / cblocks, cb = kb - tap * cblocks;
          tma_load_2d(smem_u32(smem + s * Cfg::kStageBytes) + BM * BK * 2, &L.w, cb * BK, tap * N, fb);
        }
        if (!ok) break;
        const uint32_t nth = nslot[w.j]++;
        if (w.l > 0) {  // the block's previous layer (the first layer reads what was complete before the launch)
          if (!mbar_wait(smem_u32(&done_bar[w.j]), (nth - 1) & 1, abort_flag, 9)) break;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t fb = smem_u32(&full_bar[s]);
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          const int tap = kb / cblocks, cb = kb - tap * cblocks;
          if (kb >= early) {
            const uint32_t ph = (it / S) & 1;
            if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, 1)) { ok = false; break; }
            mbar_expect_tx(fb, Cfg::kStageBytes);
            tma_load_2d(sa + BM * BK * 2, &L.w, cb * BK, tap * N, fb);
          }
          tma_load_4d(sa, &L.a, cb * BK, tap % 3 - 1, tap / 3 - 1, rb * 2, fb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<T, BN>();
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (TowerWalk w(n_layers, row_blocks); w.valid() && ok; w.next(), ++tile_it) {
        const int k_blocks = 9 * layers[w.l].p.conv_cblocks;
        const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abort_flag, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + BM * BK * 2);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tcgen05_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit(smem_u32(&empty_bar[s]));
        }
        if (ok) tcgen05_commit(smem_u32(&tfull_bar[acc]));
      }
    }
  } else if (warp == 10) {
    // ---------------- store warp ----------------
    if (lane == 0)
      tower_store_loop(layers, n_layers, row_blocks, epi_mem, stg_full, stg_free, res_bar, done_bar, abort_flag);
  } else {
    // ---------------- epilogue (warps 2..9: two groups of four warps, alternating 64-column slabs) ----------------
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const bool leader = ((warp - 2) & 3) == 0 && lane == 0;
    uint8_t* gbuf = epi_mem + group * (kBufs * BM * 128);
    uint32_t tile_it = 0, slab_it = 0, se_phase = 0;
    uint32_t res_use0 = 0, res_use1 = 0;  // skip tiles each of the group's two staging buffers has received
    ColRegs cr;
    int se_layer = -1;  // layer whose squeeze-excitation parameters sit in shared memory
    {
      for (TowerWalk w(n_layers, row_blocks); w.valid(); w.next(), ++tile_it) {
        const TcParams& P = layers[w.l].p;
        const int rb = w.rb();
        const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (group * 64 < P.N) load_col_regs(P, group * 64, lane, cr);  // in flight while the tile is computed
        const bool se_in_smem = P.se_k > 0 && (12 * P.se_k * P.N + 4 * (3 * P.N + P.se_k)) <= Cfg::kSeWBytes;
        if (se_in_smem && se_layer != w.l) {
          // This layer's squeeze-excitation parameters into shared memory while the tile is computed: the epilogue
          // warps are idle and all their loads are in flight at once.  se_prepare then reads shared memory where it
          // otherwise walks a chain of dependent round trips to L2 (pooling bias, first matrix and bias, second matrix
          // and bias: 6 us per layer at batch 64).  The previous user of the region finished behind the last barrier
          // of its se_prepare; the first barrier of this one orders the stores below before the reads.
          const int eid = (int)threadIdx.x - 64;
          const int n1 = P.se_k * P.N / 4, n2 = 2 * n1;  // float4 of se_w1, se_w2
          const float4* g1 = reinterpret_cast<const float4*>(P.se_w1);
          const float4* g2 = reinterpret_cast<const float4*>(P.se_w2);
          float4* s1 = reinterpret_cast<float4*>(se_w);
          float4* s2 = s1 + n1;
          float* sv = se_w + 12 * n1;  // se_bias [N], se_b1 [se_k], se_b2 [2N]
          for (int i = eid; i < n1; i += 256) s1[i] = __ldg(g1 + i);
          const int L = P.se_k >> 2;  // 16-byte pieces per row of se_w2; swizzled within the row (see se_prepare)
#pragma unroll 4
          for (int i = eid; i < n2; i += 256) {
            const int r = i / L, k = i - r * L;
            s2[r * L + (P.se_k >= 32 ? (k ^ (r & 7)) : k)] = __ldg(g2 + i);
          }
          for (int i = eid; i < P.N; i += 256) sv[i] = __ldg(P.se_bias + i);
          for (int i = eid; i < P.se_k; i += 256) sv[P.N + i] = __ldg(P.se_b1 + i);
          for (int i = eid; i < 2 * P.N; i += 256) sv[P.N + P.se_k + i] = __ldg(P.se_b2 + i);
          se_layer = w.l;
        }
        if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag, 4)) break;
        tcgen05_fence_after();
        const int m = rb * BM + quarter * 32 + lane;
        const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
        RowCtx rc;
        load_row_ctx(P, m, rc);
        const float* se_row = nullptr;
        if (P.se_k > 0) {
          se_prepare<BN>(P, trow, quarter, group, lane, (int)threadIdx.x - 64, wvec_all, se_gb, smem_u32(se_bar), se_phase,
                         abort_flag, se_in_smem ? se_w : nullptr, se_in_smem ? se_w + 3 * P.se_k * P.N : nullptr);
          se_row = se_gb + (quarter >> 1) * 512;
        }
#pragma unroll 1
        for (int c0 = group * 64; c0 < BN; c0 += 128) {
          if (c0 >= P.N) break;  // uniform over the group
          const int b = (int)(slab_it % kBufs);
          const int idx = group * kBufs + b;
          const int next_nb = (c0 + 128 < BN && c0 + 128 < P.N) ? c0 + 128 : -1;
          epilogue_slab<T, true, true>(P, gbuf + b * (BM * 128), smem_u32(&res_bar[idx]), smem_u32(&stg_free[idx]),
                                       smem_u32(&stg_full[idx]), slab_it / kBufs, leader, trow + c0, quarter * 32 + lane, lane,
                                       c0, next_nb, cr, wvec, rc, abort_flag, se_row ? se_row + c0 : nullptr,
                                       b ? res_use1 : res_use0);
          if (P.res_mode) {
            if (b) ++res_use1; else ++res_use0;
          }
          ++slab_it;
        }
        flush_row_ctx(P, m, rc);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      }
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 400 + *abort_flag);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (one TPC) computes a 256x256 tile with
// tcgen05.mma.cta_group::2 (M = 256: 128 rows per CTA; each CTA stages its 128 rows of A and its 128
// of the 256 W rows, so a CTA moves 32 KB per k-block instead of 48 KB).  The MMAs are issued by the
// even CTA; operand arrival from both CTAs is counted on its `full` barriers, stage release and
// accumulator hand-over are signalled to both CTAs with one tcgen05.commit per CTA, and the odd CTA's
// epilogue warps release the accumulator with remote mbarrier arrivals.
// ------------------------------------------------------------------------------------------------
// N of the MMA that computes a tile of which `remaining` columns exist: full width, or the remainder rounded up to 32.
__host__ __device__ __forceinline__ int pair_mma_n(int remaining, int bn) {
  return remaining >= bn ? bn : ((remaining + 31) & ~31);
}

template <int kGroupsT> struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int kStageBytes = (BM + BN / 2) * BK * 2;  // 32 KB per CTA
  static constexpr int kTmemCols = 512;
  // warp 0 TMA, warp 1 MMA, warps 2 and 3 stores (half of the epilogue groups each), then kGroups epilogue groups of
  // four warps, each with one staging buffer of 128 rows x 128 bytes: two groups (138 registers per thread; best when
  // the main loop dominates) or four groups (96 registers; twice the epilogue throughput, for products with few
  // k-blocks per tile).  The two-group form spends the 32 KB it saves on staging on a fifth pipeline stage: a stage
  // is refilled only after the MMAs that read it have completed, so with four stages a load has three k-blocks of MMA
  // time to arrive.  Measured against four stages and two buffers per group, in the network at batch 1024 / 256:
  // FFN2 (24 k-blocks per tile) 1040 -> 1084 and 872 -> 923 TFLOP/s, out-projection 868 -> 853 and 688 -> 670 (the
  // residual tile is prefetched one slab ahead instead of two), the whole evaluation +0.9 % and +1.0 %.  Run for
  // seconds under the power cap the two forms are equal: the clock settles where the power does.
  static constexpr int kGroups = kGroupsT;
  static constexpr int kStages = kGroupsT == 2 ? 5 : 4;
  static constexpr int kBufs = 1;
  static constexpr int kThreads = 128 + 128 * kGroupsT;
  static constexpr int kEpiBytes = kGroups * kBufs * BM * 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + 512 + 16 * 1024 /*column vectors*/ +
                                    4096 /*squeeze-excitation gate and shift*/ + 4096 /*... bias vectors*/;
};

template <typename T, int kGroups>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<kGroups>::kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
                    const __grid_constant__ CUtensorMap tmap_c2, const __grid_constant__ CUtensorMap tmap_wh,
                    const TcParams p) {
  using Cfg = PairCfg<kGroups>;
  constexpr int kBufs = Cfg::kBufs;
  constexpr int S = Cfg::kStages;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_mem = smem + S * Cfg::kStageBytes;
  uint8_t* bar_mem = epi_mem + Cfg::kEpiBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);  // [S]  waited on by the even CTA only
  uint64_t* empty_bar = full_bar + S;                          // [S]  per CTA
  uint64_t* tfull_bar = empty_bar + S;                         // [2]  per CTA
  uint64_t* tempty_bar = tfull_bar + 2;                        // [2]  even CTA: one arrival per epilogue warp of both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* res_bar = reinterpret_cast<uint64_t*>(bar_mem + 192);   // [kGroups][kBufs]
  uint64_t* stg_full = reinterpret_cast<uint64_t*>(bar_mem + 256);  // [kGroups][kBufs]
  uint64_t* stg_free = stg_full + 4;                                // [kGroups][kBufs]
  float* wvec_all = reinterpret_cast<float*>(bar_mem + 512);                                 // 16 warps x 256 floats
  float* wvec = wvec_all + ((threadIdx.x >> 5) & 15) * 256;                                  // per-warp scratch
  uint64_t* se_bar = reinterpret_cast<uint64_t*>(bar_mem + 384);        // barrier of this CTA's epilogue threads
  float* se_gb = reinterpret_cast<float*>(bar_mem + 512 + 16 * 1024);   // [2 boards][gate 256 | shift 256]
  float* se_vec = se_gb + 1024;                                         // se_bias [N], se_b1 [se_k], se_b2 [2N]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + 2 * BM - 1) / (2 * BM), n_tiles = (p.N + BN - 1) / BN;
  // virtual tiles: the tiles from split_from on count twice, as a left and a right half of 128 columns
  const int split_from = p.split_from < m_tiles * n_tiles ? p.split_from : 0x7fffffff;
  const int tiles = split_from < m_tiles * n_tiles ? p.tiles_v : m_tiles * n_tiles;
  auto tile_of = [&](int t) { return t < split_from ? t : split_from + ((t - split_from) >> 1); };
  auto col_of = [&](int t) {
    return (tile_of(t) % n_tiles) * BN + (t < split_from ? 0 : ((t - split_from) & 1) * (BN / 2));
  };
  auto width_of = [&](int t) { return t < split_from ? BN : BN / 2; };
  // N of the MMA that computes virtual tile t: the tile's width, or what is left of N rounded up to 32
  auto mma_n_of = [&](int t) { return pair_mma_n(p.N - col_of(t), width_of(t)); };
  const int k_blocks = p.conv_cblocks > 0 ? 9 * p.conv_cblocks : (p.K + BK - 1) / BK;

  if (threadIdx.x == 64) {
    tma_prefetch_map(&tmap_a);
    tma_prefetch_map(&tmap_w);
    tma_prefetch_map(&tmap_c);
    if (p.res_mode) tma_prefetch_map(&tmap_r);
    if (p.n_split > 0) tma_prefetch_map(&tmap_c2);
    if (p.split_from < p.tiles_v) tma_prefetch_map(&tmap_wh);
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8 * kGroups);
    }
    mbar_init(smem_u32(se_bar), 128 * kGroups);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&res_bar[i]), 1);
      mbar_init(smem_u32(&stg_full[i]), 4);
      mbar_init(smem_u32(&stg_free[i]), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // one warp of each CTA of the pair takes part in the allocation
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();  // everything above overlapped the kernel before this one
  grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += pairs) {
        const int m0 = (tile_of(t) / n_tiles) * (2 * BM) + (int)rank * BM;
        // a narrower tile is computed with a narrower MMA, of which each CTA supplies half the W rows
        const int n0 = col_of(t) + (int)rank * (mma_n_of(t) / 2) + (p.batch_rows > 0 ? (m0 / p.batch_rows) * p.N : 0);
        const bool half = t >= split_from;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, 1)) { ok = false; break; }
          const uint32_t fb_local = smem_u32(&full_bar[s]);
          // both CTAs' bytes land on this barrier; a half-width tile takes 64 W rows per CTA instead of 128
          if (rank == 0) mbar_expect_tx(fb_local, half ? 2 * (BM + BN / 4) * BK * 2 : 2 * Cfg::kStageBytes);
          const uint32_t fb = mapa(fb_local, 0);
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          if (p.conv_cblocks > 0) {
            // k-block = (filter tap, 64-channel block): this CTA's two boards shifted by the tap (the halo is zero
            // filled by TMA) and its half of the tap's filter rows
            const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
            tma_load_4d_pair(sa, &tmap_a, cb * BK, tap % 3 - 1, tap / 3 - 1, m0 >> 6, fb);
            tma_load_2d_pair(sa + BM * BK * 2, &tmap_w, cb * BK, tap * p.N + n0, fb);
          } else {
            tma_load_2d_pair(sa, &tmap_a, kb * BK, m0, fb);
            tma_load_2d_pair(sa + BM * BK * 2, half ? &tmap_wh : &tmap_w, kb * BK, n0, fb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_base = (1u << 4) | (FmtCode<T>::v << 7) | (FmtCode<T>::v << 10) |
                                      ((uint32_t)((2 * BM) >> 4) << 24);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += pairs, ++tile_it) {
        const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abort_flag, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const uint32_t idesc = idesc_base | ((uint32_t)(mma_n_of(t) >> 3) << 17);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + BM * BK * 2);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tcgen05_mma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          const uint32_t eb = smem_u32(&empty_bar[s]);
          tcgen05_commit_pair(mapa(eb, 0));  // frees the stage in both CTAs once the MMAs have read it
          tcgen05_commit_pair(mapa(eb, 1));
        }
        if (ok) {
          const uint32_t tb = smem_u32(&tfull_bar[acc]);
          tcgen05_commit_pair(mapa(tb, 0));
          tcgen05_commit_pair(mapa(tb, 1));
        }
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ---------------- store warps (both CTAs): TMA stores of the staged slabs, half of the groups each ----------
    if (lane == 0)
      store_warp_loop<kGroups, kBufs>(p, &tmap_c, &tmap_c2, &tmap_r, epi_mem, stg_full, stg_free, res_bar,
                                      (warp - 2) * (kGroups / 2), (warp - 1) * (kGroups / 2), pair, pairs, tiles, n_tiles,
                                      2 * BM, (int)rank * BM, BN, split_from, abort_flag);
  } else {
    // ---------------- epilogue (warps 4.. of both CTAs): group g handles the 64-column slabs g, g + kGroups, ... of
    // every tile ----------------
    const int quarter = warp & 3;
    const int group = (warp - 4) >> 2;
    const bool leader = ((warp - 4) & 3) == 0 && lane == 0;
    uint32_t tile_it = 0, slab_it = 0, se_phase = 0;
    ColRegs cr;
    int cr_nb = -1;
    bool se_vec_ok = false;
    if constexpr (kGroups == 2) {
      if (p.se_k > 0 && 3 * p.N + p.se_k <= 1024) {
        // the squeeze-excitation bias vectors into shared memory while the first tile is computed
        const int eid = (int)threadIdx.x - 128;
        for (int i = eid; i < p.N; i += 256) se_vec[i] = __ldg(p.se_bias + i);
        for (int i = eid; i < p.se_k; i += 256) se_vec[p.N + i] = __ldg(p.se_b1 + i);
        for (int i = eid; i < 2 * p.N; i += 256) se_vec[p.N + p.se_k + i] = __ldg(p.se_b2 + i);
        se_vec_ok = true;
      }
    }
    if (pair < tiles && group * 64 < width_of(pair) && col_of(pair) + group * 64 < p.N) {
      cr_nb = col_of(pair) + group * 64;  // first slab: fetched while the first tile is computed
      load_col_regs(p, cr_nb, lane, cr);
    }
    for (int t = pair; t < tiles; t += pairs, ++tile_it) {
      const uint32_t acc = tile_it & 1, aph = (tile_it >> 1) & 1;
      const int m0 = (tile_of(t) / n_tiles) * (2 * BM) + (int)rank * BM, n0 = col_of(t), width = width_of(t);
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag, 4)) break;
      tcgen05_fence_after();
      const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      const int m = m0 + quarter * 32 + lane;
      RowCtx rc;
      load_row_ctx(p, m, rc);
      const float* se_row = nullptr;
      if constexpr (kGroups == 2) {
        if (p.se_k > 0) {  // this CTA's 128 rows are two boards with all their channels
          se_prepare<BN>(p, trow, quarter, group, lane, (int)threadIdx.x - 128, wvec_all, se_gb, smem_u32(se_bar),
                         se_phase, abort_flag, nullptr, se_vec_ok ? se_vec : nullptr);
          se_row = se_gb + (quarter >> 1) * 512;
        }
      }
#pragma unroll 1
      for (int c0 = group * 64; c0 < width; c0 += 64 * kGroups) {
        if (n0 + c0 >= p.N) break;  // uniform over the group
        const int idx = group * kBufs + (int)(slab_it % kBufs);
        if (cr_nb != n0 + c0) load_col_regs(p, n0 + c0, lane, cr);
        // the slab this group handles next: further right in this tile, else the first one of its next tile
        int next_nb = -1;
        if (c0 + 64 * kGroups < width && n0 + c0 + 64 * kGroups < p.N) {
          next_nb = n0 + c0 + 64 * kGroups;
        } else if (t + pairs < tiles && group * 64 < width_of(t + pairs)) {
          const int nn = col_of(t + pairs) + group * 64;
          if (nn < p.N) next_nb = nn;
        }
        cr_nb = next_nb;
        epilogue_slab<T, kGroups == 2>(p, epi_mem + idx * (BM * 128), smem_u32(&res_bar[idx]), smem_u32(&stg_free[idx]),
                                       smem_u32(&stg_full[idx]), slab_it / kBufs, leader, trow + c0, quarter * 32 + lane,
                                       lane, n0 + c0, next_nb, cr, wvec, rc, abort_flag,
                                       se_row ? se_row + c0 : nullptr);
        ++slab_it;
      }
      flush_row_ctx(p, m, rc);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&tempty_bar[acc]), 0));
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, 200 + *abort_flag);
    __syncthreads();
  }
  cluster_sync_all();  // neither CTA releases tensor or shared memory while its peer may still touch it
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;

struct MapKey {
  const void* ptr; long long ld; int rows, cols, box_rows, prec;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && ld == o.ld && rows == o.rows && cols == o.cols && box_rows == o.box_rows && prec == o.prec;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long long>()(k.ld);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)(k.box_rows * 4 + k.prec);
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// 2D map over a row-major [rows][cols] 16-bit matrix with leading dimension ld; box = 64 columns x box_rows.
cudaError_t get_map(const void* ptr, long long ld, int rows, int cols, int box_rows, int prec, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_encode) return cudaErrorNotReady;
  MapKey key{ptr, ld, rows, cols, box_rows, prec};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, prec == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return cudaErrorInvalidValue;
  }
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return cudaSuccess;
}

void fill_folded(TcParams& p, const GemmParams& g) {
  p.a_stats = g.a_stats; p.colsum = g.colsum; p.a_inv_c = g.a_inv_c; p.a_eps = g.a_eps;
  p.res_mode = g.res ? (g.res_stats ? 2 : 1) : 0;
  p.res_stats = g.res_stats; p.res_gamma = g.res_gamma; p.res_beta = g.res_beta;
  p.res_inv_c = g.res_inv_c; p.res_eps = g.res_eps;
  p.out_stats = g.out_stats;
  p.n_split = 0;
  p.se_w1 = g.se_w1; p.se_b1 = g.se_b1; p.se_w2 = g.se_w2; p.se_b2 = g.se_b2; p.se_bias = g.se_bias;
  p.se_k = g.se_k;
  p.batch_rows = g.batch_rows;
}

// 4D map over a token-major activation [positions][8][8][channels]; box = 64 channels x 8 x 8 x 2 boards
// (128 GEMM rows).  Not cached: convolution inputs are few and the encode call is a host-side pure function.
cudaError_t make_board_map(const void* ptr, int channels, int positions, int prec, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_encode) return cudaErrorNotReady;
  cuuint64_t dims[4] = {(cuuint64_t)channels, 8, 8, (cuuint64_t)positions};
  cuuint64_t strides[3] = {(cuuint64_t)channels * 2, (cuuint64_t)channels * 16, (cuuint64_t)channels * 128};
  cuuint32_t box[4] = {(cuuint32_t)BK, 8, 8, 2};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(out, prec == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                        const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (4D) failed with CUresult " + std::to_string((int)r));
    return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

template <typename T, int BN>
cudaError_t launch_bn(const GemmParams& g, int* status, int sm_count, cudaStream_t s) {
  using Cfg = TileCfg<BN>;
  // The opt-in to large dynamic shared memory is per device.
  static std::atomic<unsigned long long> attr_mask{0};
  int dev = 0;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return de;
  if (!(attr_mask.load() >> (dev & 63) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_mask.fetch_or(1ull << (dev & 63));
  }
  CUtensorMap ma, mw;
  const int prec = TypeTag<T>::prec;
  cudaError_t e;
  if (g.conv_cin > 0) {
    e = make_board_map(g.A, g.conv_cin, g.M / 64, prec, &ma);
    if (e != cudaSuccess) return e;
    e = get_map(g.W, g.conv_cin, 9 * g.N, g.conv_cin, BN, prec, &mw);
  } else {
    e = get_map(g.A, g.lda, g.M, g.K, BM, prec, &ma);
    if (e != cudaSuccess) return e;
    e = get_map(g.W, g.ldw, g.batch_rows > 0 ? g.N * (g.M / g.batch_rows) : g.N, g.K, BN, prec, &mw);
  }
  if (e != cudaSuccess) return e;
  const bool tma_store = !g.out_f32 && (g.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(g.C) & 15) == 0;
  CUtensorMap mc = ma;
  if (tma_store) {
    e = get_map(g.C, g.ldc, g.M, g.N, BM, prec, &mc);
    if (e != cudaSuccess) return e;
  }
  const bool folded = g.a_stats || g.res || g.out_stats || g.se_k > 0;
  if (folded && !tma_store) return cudaErrorInvalidValue;  // the folded-LayerNorm modes live in the TMA-store epilogue
  if (g.se_k > 0 && (BN != 256 || !gemm_tc_se_supported(g))) return cudaErrorInvalidValue;
  CUtensorMap mr = mc;
  if (g.res) {
    if ((g.ldres % 8) != 0 || (reinterpret_cast<uintptr_t>(g.res) & 15) != 0) return cudaErrorInvalidValue;
    e = get_map(g.res, g.ldres, g.M, g.N, BM, prec, &mr);
    if (e != cudaSuccess) return e;
  }
  TcParams p;
  fill_folded(p, g);
  p.tma_store = tma_store ? 1 : 0;
  p.split_from = 0x7fffffff; p.tiles_v = 0;
  p.bias = g.bias; p.C = g.C; p.ldc = g.ldc;
  p.M = g.M; p.N = g.N; p.K = g.K; p.act = g.act; p.scale = g.scale; p.alpha = g.alpha;
  p.out_f32 = g.out_f32 ? 1 : 0; p.status = status;
  p.conv_cblocks = g.conv_cin > 0 ? ceil_div(g.conv_cin, BK) : 0;
  const int tiles = ceil_div(g.M, BM) * ceil_div(g.N, BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  return launch_dependent(gemm_tc_kernel<T, BN>, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, s, ma, mw, mc, mr, p);
}


template <typename T, int kGroups>
cudaError_t launch_pair(const GemmParams& g, int* status, int sm_count, cudaStream_t s) {
  using Cfg = PairCfg<kGroups>;
  static std::atomic<unsigned long long> attr_mask{0};
  int dev = 0;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return de;
  if (!(attr_mask.load() >> (dev & 63) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<T, kGroups>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_mask.fetch_or(1ull << (dev & 63));
  }
  CUtensorMap ma, mw, mc;
  const int prec = TypeTag<T>::prec;
  const bool conv = g.conv_cin > 0;
  cudaError_t e = conv ? make_board_map(g.A, g.conv_cin, g.M / 64, prec, &ma) : get_map(g.A, g.lda, g.M, g.K, BM, prec, &ma);
  if (e != cudaSuccess) return e;
  const int w_rows = conv ? 9 * g.N : (g.batch_rows > 0 ? g.N * (g.M / g.batch_rows) : g.N);
  e = get_map(g.W, conv ? g.conv_cin : g.ldw, w_rows, conv ? g.conv_cin : g.K, Cfg::BN / 2, prec, &mw);
  if (e != cudaSuccess) return e;
  if (g.se_k > 0 && (kGroups != 2 || !gemm_tc_se_supported(g))) return cudaErrorInvalidValue;
  e = get_map(g.C, g.ldc, g.M, g.n_split > 0 ? g.n_split : g.N, BM, prec, &mc);
  if (e != cudaSuccess) return e;
  CUtensorMap mr = mc, mc2 = mc;
  if (g.res) {
    if ((g.ldres % 8) != 0 || (reinterpret_cast<uintptr_t>(g.res) & 15) != 0) return cudaErrorInvalidValue;
    e = get_map(g.res, g.ldres, g.M, g.N, BM, prec, &mr);
    if (e != cudaSuccess) return e;
  }
  if (g.n_split > 0) {
    e = get_map(g.C2, g.ldc2, g.M, g.N - g.n_split, BM, prec, &mc2);
    if (e != cudaSuccess) return e;
  }
  TcParams p;
  fill_folded(p, g);
  p.n_split = g.n_split;
  p.tma_store = 1;
  p.bias = g.bias; p.C = g.C; p.ldc = g.ldc;
  p.M = g.M; p.N = g.N; p.K = g.K; p.act = g.act; p.scale = g.scale; p.alpha = g.alpha;
  p.out_f32 = 0; p.status = status;
  p.conv_cblocks = conv ? ceil_div(g.conv_cin, BK) : 0;
  const int tiles = ceil_div(g.M, 2 * BM) * ceil_div(g.N, Cfg::BN);
  const int max_pairs = sm_count / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  // A last wave that fills at most half of the pairs is computed as half-width tiles (twice as many, half as long), so
  // that it costs about half a tile time instead of a whole one: 13-16 % of a product of three to six waves.
  // Full-width tiles only; GemmParams::whole_tiles switches it off.
  const bool split_enabled = !g.whole_tiles;
  const int rem = tiles % pairs;
  p.split_from = 0x7fffffff;
  p.tiles_v = tiles;
  if (split_enabled && !conv && g.n_split == 0 && (g.N % Cfg::BN) == 0 && tiles > pairs && rem > 0 && 2 * rem <= pairs) {
    p.split_from = tiles - rem;
    p.tiles_v = tiles + rem;
  }
  CUtensorMap mwh = mw;  // W in boxes of 64 rows, for the half-width tiles
  if (p.split_from < p.tiles_v) {
    e = get_map(g.W, g.ldw, w_rows, g.K, Cfg::BN / 4, prec, &mwh);
    if (e != cudaSuccess) return e;
  }
  return launch_dependent(gemm_tc_pair_kernel<T, kGroups>, dim3(2 * pairs), dim3(Cfg::kThreads), Cfg::kSmemBytes, s, ma,
                          mw, mc, mr, mc2, mwh, p);
}

}  // namespace

cudaError_t gemm_tc_init() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode) return cudaSuccess;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return cudaSuccess;
}

cudaError_t tma_encode_2d(const void* ptr, long long ld, long long rows, int cols, int box_cols, int box_rows,
                          int swizzle_bytes, int prec, void* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_encode) return cudaErrorNotReady;
  if (box_cols * 2 != swizzle_bytes || (swizzle_bytes != 64 && swizzle_bytes != 128)) return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(reinterpret_cast<CUtensorMap*>(out),
                        prec == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

bool gemm_tc_supported(const GemmParams& p) {
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (p.conv_cin > 0)
    return p.batch == 1 && p.M >= 64 && (p.M % 64) == 0 && p.N >= 8 && (p.conv_cin % 8) == 0 && al16(p.A) && al16(p.W);
  if (p.batch_rows > 0 && ((p.batch_rows % 256) != 0 || (p.M % p.batch_rows) != 0 || p.res || p.a_stats || p.out_stats ||
                           p.n_split > 0 || p.bias))
    return false;
  return p.batch == 1 && p.M >= 1 && p.N >= 8 && p.K >= 8 && (p.K % 8) == 0 && (p.lda % 8) == 0 &&
         (p.ldw % 8) == 0 && al16(p.A) && al16(p.W);
}

// Squeeze-excitation in the convolution's epilogue: a 128-row tile is two boards, so all output channels must fit one
// 256-column tile; the residual arrives through `res`, the hidden width must suit the quad-wise reduction.
bool gemm_tc_se_supported(const GemmParams& p) {
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return p.conv_cin > 0 && p.N <= 256 && (p.N % 16) == 0 && al16(p.se_w1) && al16(p.se_w2) && p.se_k >= 4 && p.se_k <= 64 && (p.se_k % 4) == 0 &&
         p.res && !p.res_stats && !p.a_stats && !p.out_stats && !p.bias && p.n_split == 0 && !p.out_f32 &&
         p.se_w1 && p.se_b1 && p.se_w2 && p.se_b2 && p.se_bias && p.alpha == 1.0f && p.scale == 1.0f;
}

namespace {
// Large problems with 16-bit output go to the CTA-pair kernel (256x256 tiles).
bool pair_eligible(const GemmParams& p, int sm_count) {
  const bool tma_store_ok = !p.out_f32 && (p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
  // a convolution qualifies when one 256-wide tile holds all its output channels (each CTA of a pair then loads half
  // of every tap's filter rows instead of all of them)
  if (p.conv_cin > 0 && (p.N > 256 || p.n_split > 0)) return false;
  return tma_store_ok && p.M >= 512 && p.N > 128 &&
         (long long)ceil_div(p.M, 2 * BM) * ceil_div(p.N, 256) >= sm_count / 4;
}
}  // namespace

bool gemm_tc_split_supported(const GemmParams& p, int sm_count) {
  return gemm_tc_supported(p) && pair_eligible(p, sm_count) && p.n_split > 0 && (p.n_split % 256) == 0 &&
         p.N > p.n_split && p.N - p.n_split <= 256 && p.C2 && (p.ldc2 % 8) == 0 &&
         (reinterpret_cast<uintptr_t>(p.C2) & 15) == 0 && !p.res && !p.out_stats && !p.skip;
}

// ---- tower kernel, host side ----
size_t gemm_tc_tower_layer_bytes() { return sizeof(TowerLayer); }

bool gemm_tc_tower_supported(const GemmParams* g, int n) {
  if (n < 2) return false;
  for (int i = 0; i < n; ++i) {
    const GemmParams& p = g[i];
    const bool tma_ok = !p.out_f32 && (p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
    if (p.conv_cin <= 0 || !gemm_tc_supported(p) || !tma_ok || p.skip || p.n_split > 0 || p.batch_rows > 0 || p.a_stats ||
        p.out_stats || p.res_stats)
      return false;
    if (p.M != g[0].M || p.N != g[0].N || p.N > TowerCfg::BN || (p.N % 64) != 0) return false;
    if (p.se_k > 0 && !gemm_tc_se_supported(p)) return false;
    if (p.res && ((p.ldres % 8) != 0 || (reinterpret_cast<uintptr_t>(p.res) & 15) != 0)) return false;
    // a layer reads what an earlier layer of the same CTA wrote, or something complete before the launch; the skip
    // input must be at least two layers old (it is fetched while the layer before is still being computed)
    if (i > 0 && p.res && p.res == g[i - 1].C) return false;
  }
  return true;
}

// Fills `host_layers` (n entries of gemm_tc_tower_layer_bytes() each) for a later launch; the caller copies them to
// the device.  The descriptors cover the buffers' full extent (M rows), so one table serves every batch size: a launch
// only walks the row blocks it is given.
template <typename T>
cudaError_t gemm_tc_tower_build(const GemmParams* g, int n, int* status, void* host_layers) {
  if (!gemm_tc_tower_supported(g, n)) return cudaErrorInvalidValue;
  const int prec = TypeTag<T>::prec;
  const int bn = TowerCfg::BN;
  TowerLayer* out = static_cast<TowerLayer*>(host_layers);
  for (int i = 0; i < n; ++i) {
    const GemmParams& q = g[i];
    TowerLayer& L = out[i];
    memset(&L, 0, sizeof(L));
    cudaError_t e = make_board_map(q.A, q.conv_cin, q.M / 64, prec, &L.a);
    if (e != cudaSuccess) return e;
    if ((e = get_map(q.W, q.conv_cin, 9 * q.N, q.conv_cin, bn, prec, &L.w)) != cudaSuccess) return e;
    if ((e = get_map(q.C, q.ldc, q.M, q.N, BM, prec, &L.c)) != cudaSuccess) return e;
    L.r = L.c;
    if (q.res && (e = get_map(q.res, q.ldres, q.M, q.N, BM, prec, &L.r)) != cudaSuccess) return e;
    TcParams& p = L.p;
    fill_folded(p, q);
    p.tma_store = 1;
    p.split_from = 0x7fffffff; p.tiles_v = 0;
    p.bias = q.bias; p.C = q.C; p.ldc = q.ldc;
    p.M = q.M; p.N = q.N; p.K = q.K; p.act = q.act; p.scale = q.scale; p.alpha = q.alpha;
    p.out_f32 = 0; p.status = status;
    p.conv_cblocks = ceil_div(q.conv_cin, BK);
  }
  return cudaSuccess;
}
template cudaError_t gemm_tc_tower_build<__half>(const GemmParams*, int, int*, void*);
template cudaError_t gemm_tc_tower_build<__nv_bfloat16>(const GemmParams*, int, int*, void*);

// One launch for `n_layers` convolutions over the first `row_blocks` blocks of 128 rows (two boards).
template <typename T>
cudaError_t launch_gemm_tower(const void* d_layers, int n_layers, int channels, int row_blocks, int* status, int sm_count,
                              cudaStream_t s) {
  if (row_blocks <= 0) return cudaSuccess;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  // one row block per CTA while there are SMs for that, two at a time beyond (see TowerWalk)
  const int want = row_blocks <= sm_count ? row_blocks : (row_blocks + 1) / 2;
  const int grid = want < sm_count ? want : sm_count;
  const TowerLayer* layers = static_cast<const TowerLayer*>(d_layers);
  if (channels > TowerCfg::BN) return cudaErrorInvalidValue;
  static std::atomic<unsigned long long> mask{0};
  if (!(mask.load() >> (dev & 63) & 1ull)) {
    e = cudaFuncSetAttribute(gemm_tc_tower_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, TowerCfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    mask.fetch_or(1ull << (dev & 63));
  }
  return launch_dependent(gemm_tc_tower_kernel<T>, dim3(grid), dim3(kThreads), TowerCfg::kSmemBytes, s, layers, n_layers,
                          row_blocks, status);
}
template cudaError_t launch_gemm_tower<__half>(const void*, int, int, int, int*, int, cudaStream_t);
template cudaError_t launch_gemm_tower<__nv_bfloat16>(const void*, int, int, int, int*, int, cudaStream_t);

template <typename T>
cudaError_t launch_gemm_tc(const GemmParams& p, int* status, int sm_count, cudaStream_t s) {
  if (p.M <= 0 || p.N <= 0) return cudaSuccess;
  if (!gemm_tc_supported(p) || p.skip) return cudaErrorInvalidValue;  // residuals go through `res`
  if (p.n_split > 0 && !gemm_tc_split_supported(p, sm_count)) return cudaErrorInvalidValue;
  if (pair_eligible(p, sm_count))
  {
    // Four epilogue groups when a tile has few k-blocks (the epilogue then sets the pace), two otherwise (fewer
    // warps compete with the MMA issuer and the producer).  With a residual input or row statistics a slab costs a
    // residual fetch, the epilogue and a store in a row, which two groups only hide behind more than 16 k-blocks: the
    // out-projection (16 k-blocks) went from 838 to 873 TFLOP/s at batch 1024 and from 668 to 723 at batch 256 on four.
    const bool heavy = p.res != nullptr || p.out_stats != nullptr;
    const bool four = p.conv_cin == 0 && p.se_k == 0 && (p.K <= 8 * BK || (heavy && p.K <= 16 * BK));
    return four ? launch_pair<T, 4>(p, status, sm_count, s) : launch_pair<T, 2>(p, status, sm_count, s);
  }
  if (p.se_k > 0) return launch_bn<T, 256>(p, status, sm_count, s);  // the tile must hold every channel of two boards
  // Wide tiles amortise the A-tile loads; narrow problems take the smallest tile that covers N, and skinny
  // problems (few rows) the widest tile that still yields at least half an SM count of CTAs.
  auto tiles = [&](int bn) { return (long long)ceil_div(p.M, BM) * ceil_div(p.N, bn); };
  if (p.N > 128 && (tiles(256) >= sm_count / 2 || p.N <= 128)) return launch_bn<T, 256>(p, status, sm_count, s);
  if (p.N > 64 && (tiles(128) >= sm_count / 2 || p.N <= 64)) return launch_bn<T, 128>(p, status, sm_count, s);
  if (p.N > 128 && tiles(64) < sm_count / 8) return launch_bn<T, 256>(p, status, sm_count, s);
  return launch_bn<T, 64>(p, status, sm_count, s);
}

template cudaError_t launch_gemm_tc<__half>(const GemmParams&, int*, int, cudaStream_t);
template cudaError_t launch_gemm_tc<__nv_bfloat16>(const GemmParams&, int*, int, cudaStream_t);

}  // namespace b200
