// Launchers of the hand-written kernels (one explicit instantiation per storage type).
#pragma once
#include "common.cuh"

struct b200_board;  // include/b200nn.h

namespace b200 {

struct GemmParams {
  // C[b][M][N] = epilogue(scale * A[b][M][K] . W[b][N][K]^T)
  // epilogue(v): v += bias[n]; v = act(v); if (skip) v = alpha * v + skip[m][n]
  const void* A = nullptr; long long lda = 0, strideA = 0;
  const void* W = nullptr; long long ldw = 0, strideW = 0;
  const float* bias = nullptr;
  void* C = nullptr; long long ldc = 0, strideC = 0;
  const void* skip = nullptr; long long ldskip = 0;
  int M = 0, N = 0, K = 0, batch = 1;
  int act = ACT_NONE;
  float scale = 1.0f, alpha = 1.0f;
  bool out_f32 = false;  // C holds float even when the storage type is 16-bit
  // 3x3 convolution mode of the tensor-core kernel (conv_cin > 0): A is the token-major activation
  // [M = positions*64][conv_cin] (8x8 boards), W is [9][N][conv_cin] (tap-major filters), K is ignored.
  int conv_cin = 0;
  // ---- folded LayerNorm (tensor-core kernel only) ----------------------------------------------------------
  // The rows of A are LayerNorm *inputs* u whose normalisation x = (u - mean) * rstd * gamma + beta was folded
  // into this product: W holds W * gamma, `colsum[n]` = sum_k (W * gamma)[n][k], `bias` holds beta . W^T + b and
  // `a_stats` the per-row (sum, sum of squares) of u.  Then x . W^T + b = rstd * (u . (W gamma)^T - mean * colsum) + bias.
  const double* a_stats = nullptr;
  const float* colsum = nullptr;
  float a_inv_c = 0.f, a_eps = 0.f;
  // Residual input added after the activation: out = alpha * act(...) + s, where s is read from `res`
  // ([M][N], leading dimension ldres) and, when res_stats is set, normalised on the fly:
  // s = (res - mean) * rstd * res_gamma[n] + res_beta[n].
  const void* res = nullptr; long long ldres = 0;
  const double* res_stats = nullptr;
  const float* res_gamma = nullptr;
  const float* res_beta = nullptr;
  float res_inv_c = 0.f, res_eps = 0.f;
  // Per-row (sum, sum of squares) of the outputs, accumulated in double with atomic adds into out_stats[M][2]
  // (the caller zeroes it), so that the next product can fold the LayerNorm of this output.
  double* out_stats = nullptr;
  // Second output of the CTA-pair kernel: columns [n_split, N) go to C2 (leading dimension ldc2, column n - n_split)
  // instead of C.  n_split must be a multiple of 256 and the remainder at most 256 columns wide; the last tile is then
  // computed with a narrower MMA.  Lets a narrow product share the operand traffic of a wide one (same A, same folded
  // LayerNorm); no residual / statistics in this mode.
  void* C2 = nullptr; long long ldc2 = 0;
  int n_split = 0;
  // Squeeze-excitation unit fused into a convolution (tensor-core kernel, convolution mode, at most 256 output
  // channels): out = act(gate * conv + shift + res) with gate / shift from the board's pooled conv output
  // (ApplySEUnit, backends/blas/se_unit.cc:31-91).  se_w1 [se_k][N], se_b1 [se_k], se_w2 [2N][se_k], se_b2 [2N],
  // se_bias [N] = the convolution's own bias (it enters through the pooled mean and the shift); `bias` stays null and
  // `act` is applied after the residual.  See gemm_tc_se_supported.
  const float* se_w1 = nullptr; const float* se_b1 = nullptr; const float* se_w2 = nullptr;
  const float* se_b2 = nullptr; const float* se_bias = nullptr;
  int se_k = 0;
  // Stacked products in one launch (tensor-core kernel): A and C are [batches * batch_rows][..], W is [batches * N][K];
  // rows of batch b meet the W rows of batch b.  batch_rows must be a multiple of 256 (a tile never spans two
  // batches); M = batches * batch_rows.  No bias, residual or statistics.  The 36 products of a Winograd convolution.
  int batch_rows = 0;
  // CTA-pair kernel: compute a sparsely filled last wave as whole 256x256 tiles instead of half-width ones
  // (verification switch; the split is on by default).
  bool whole_tiles = false;
};

template <typename T> cudaError_t launch_gemm_simt(const GemmParams& p, cudaStream_t s);
// tcgen05 / TMEM / TMA kernel (gemm_tc.cu); T is __half or __nv_bfloat16, batch must be 1.
// `status` is a device int the kernel sets non-zero when a bounded wait gives up.
template <typename T> cudaError_t launch_gemm_tc(const GemmParams& p, int* status, int sm_count, cudaStream_t s);
bool gemm_tc_supported(const GemmParams& p);
bool gemm_tc_se_supported(const GemmParams& p);
// Whether launch_gemm_tc would run `p` (with C2 / n_split set) on the CTA-pair kernel, the only one that splits.
bool gemm_tc_split_supported(const GemmParams& p, int sm_count);
// Tower kernel (gemm_tc.cu): the 3x3 convolutions of a residual tower (conv_cin > 0, optional fused squeeze-excitation
// and skip input), all with the same rows and output channels (at most 256), in one launch.  gemm_tc_tower_build fills
// a host table of n entries of gemm_tc_tower_layer_bytes() bytes, which the caller copies to the device once;
// launch_gemm_tower runs the first `row_blocks` blocks of 128 rows (two boards) through all layers.
bool gemm_tc_tower_supported(const GemmParams* g, int n);
size_t gemm_tc_tower_layer_bytes();
template <typename T> cudaError_t gemm_tc_tower_build(const GemmParams* g, int n, int* status, void* host_layers);
template <typename T>
cudaError_t launch_gemm_tower(const void* d_layers, int n_layers, int channels, int row_blocks, int* status, int sm_count,
                              cudaStream_t s);
cudaError_t gemm_tc_init();  // resolves the driver entry point used to encode TMA descriptors
// TMA descriptor over a row-major 16-bit matrix [rows][cols] with leading dimension ld (elements), box
// box_cols x box_rows, shared-memory swizzle of 64 or 128 bytes (= box_cols * 2); `out` is a CUtensorMap.
// prec: 1 = fp16, 2 = bf16.  Needs gemm_tc_init().
cudaError_t tma_encode_2d(const void* ptr, long long ld, long long rows, int cols, int box_cols, int box_rows,
                          int swizzle_bytes, int prec, void* out);

template <typename T>
cudaError_t launch_expand_planes(const uint64_t* masks, const float* values, int n, T* out, cudaStream_t s);
// tokens[n*64][cin]: columns 0..111 expanded planes (NHWC), columns 112.. positional encoding taken
// from pe_static [64][pe_ch] (fp32 table) or pe_dense [n][64][pe_ch] (T), zero padded to cin.
template <typename T>
cudaError_t launch_expand_tokens(const uint64_t* masks, const float* values, int n, const float* pe_static,
                                 const T* pe_dense, int pe_ch, int cin, T* out, cudaStream_t s);
// pre[n][64*12]: first 12 planes, square-major (input of the PE_DENSE preprocessing layer).
template <typename T>
cudaError_t launch_expand_pre12(const uint64_t* masks, const float* values, int n, T* out, cudaStream_t s);

// out = LN(alpha * x + skip) * gamma + beta, then optional gating out * mult[r%64][c] + add[r%64][c].
template <typename T>
cudaError_t launch_layer_norm(T* out, const T* x, const T* skip, const float* gamma, const float* beta,
                              const float* gate_mult, const float* gate_add, int rows, int C, float alpha,
                              float eps, cudaStream_t s);
template <typename T>
cudaError_t launch_gate(T* x, const float* gate_mult, const float* gate_add, int rows, int C, cudaStream_t s);

// 64-token multi-head attention: per (sample, head) softmax(scale * Q K^T + bias) V.
// q/k/v point into one row-major activation with leading dimension ld; head h uses columns h*d...
// bias: [n][heads][64][64] or nullptr.
template <typename T>
cudaError_t launch_attention(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                             long long ldo, int n, int heads, int depth, float scale, cudaStream_t s);

// Tensor-core version of the same operator for 16-bit storage and depth 32 or 64 (attention_tc.cu).
bool attention_tc_supported(long long ld, long long ldo, int depth, const void* q, const void* k, const void* v,
                            const void* bias, const void* out);
// Persistent kernel: TMA loads into a ring of swizzled shared-memory stages, TMA stores of the result; `status`
// receives 300 + code if a bounded device-side wait gives up.
template <typename T>
cudaError_t launch_attention_tma(const T* q, const T* k, const T* v, long long ld, const T* bias, T* out,
                                 long long ldo, int n, int heads, int depth, float scale, int* status, int sm_count,
                                 cudaStream_t s);

// Attention policy: promotion logits + gather to 1858 (network_blas.cc:873-914).
// logits: fp32 [n][64*64] (already scaled), kp: [n*64][dm] keys, w4: fp32 [4][dm].
template <typename T>
cudaError_t launch_policy_attn_gather(const float* logits, const T* kp, const float* w4, int dm,
                                      const short* src_slot, int n, float* policy, cudaStream_t s);
// Tensor-core version of the whole tail (Q K^T, promotion offsets, gather) for 16-bit storage (attention_tc.cu).
bool policy_attn_tc_supported(int dm, const void* q, const void* k);
template <typename T>
cudaError_t launch_policy_attn_tc(const T* q, const T* k, const float* w4, int dm, const short* src_slot, int n,
                                  float* policy, cudaStream_t s);
// Generic gather for conv policy: policy[n][j] = raw[n][src[j]] (raw row stride ld), T -> fp32.
template <typename T>
cudaError_t launch_policy_gather(const T* raw, long long ld, const short* src_slot, int n, float* policy,
                                 cudaStream_t s);

// Legal-move policy softmax on the device: probs[n][i] = FastExp((logit[move_ids[n][i]] - max) * inv_t) / total for
// the first n_moves[n] entries (stride kLegalStride), same arithmetic and order as the reference's caller-side
// SoftmaxPolicy (src/neural/wrapper.cc:135-156) with FastExp of src/utils/fastmath.h:59-86.
constexpr int kLegalStride = 256;
cudaError_t launch_legal_softmax(const float* policy, const unsigned short* move_ids, const int* n_moves, int n,
                                 float inv_temperature, float* probs, cudaStream_t s);

// Final tiny layers of the value / moves-left heads, one warp per sample:
// mode 0: 3 logits -> softmax -> (q = w - l, d); mode 1: 1 output -> tanh -> q, d = 0;
// mode 2: 1 output -> relu -> m.  h: [n][k]; w: fp32 [outs][k]; b: fp32 [outs]; qdm: [n][3].
template <typename T>
cudaError_t launch_head_final(const T* h, int k, const float* w, const float* b, int mode, int n,
                              float* qdm, cudaStream_t s);

// ---- residual tower (NHWC activations [n*64][C]) ----
// 3x3 same-padded convolution as an implicit GEMM; w: [9][Cout][Cin] (tap-major).
template <typename T>
cudaError_t launch_conv3x3(const T* x, int cin, const T* w, const float* bias, T* y, int cout, int n,
                           int act, cudaStream_t s);
// Squeeze-excitation + skip + activation (se_unit.cc:31-91) on NHWC: y = act(sig(z0)*x + skip + z1 + sig(z0)*b).
template <typename T>
cudaError_t launch_se(const T* x, const float* conv_bias, const T* skip, const float* w1, const float* b1,
                      const float* w2, const float* b2, T* y, int C, int se_k, int n, int act, cudaStream_t s);
template <typename T>
cudaError_t launch_bias_skip_act(const T* x, const float* bias, const T* skip, T* y, int C, int rows, int act,
                                 cudaStream_t s);

// Winograd F(4x4, 3x3) convolution pieces (winograd.cu): input transform x [boards*64][C] -> v [36][rows_padded][C]
// (row = board * 4 + patch), output transform m [36][rows_padded][C] -> y [boards*64][C] with bias, optional
// squeeze-excitation (se_k > 0), optional skip and the activation, and the host-side filter transform
// w [Cout][Cin][3][3] -> u [36][Cout][Cin].
template <typename T>
cudaError_t launch_wino_input(const T* x, T* v, int C, int boards, long long rows_padded, cudaStream_t s);
template <typename T>
cudaError_t launch_wino_output(const T* m, const float* bias, const T* skip, const float* se_w1, const float* se_b1,
                               const float* se_w2, const float* se_b2, int se_k, T* y, int C, int boards,
                               long long rows_padded, int act, cudaStream_t s);
void wino_transform_filters(const float* w, int cout, int cin, float* u);

// Position encoding on the device (encoder.cu): game histories -> 112 packed planes per position, the work of the
// reference's host-side EncodePositionForNN (src/neural/encoder.cc:134-328).  boards/offsets/from_start as in
// b200_op_encode_positions (include/b200nn.h).
bool encode_format_supported(int input_format);
cudaError_t launch_encode_positions(const b200_board* boards, const int* offsets, const uint8_t* from_start, int n,
                                    int input_format, int fill, uint64_t* masks, float* values, int* transforms,
                                    cudaStream_t s);

// Packed V6 training-data records -> 112 packed planes each (PlanesFromTrainingData, src/trainingdata/reader.cc:32-118).
cudaError_t launch_planes_from_training_data(const void* records, int n, long long stride, int undo, uint64_t* masks,
                                             float* values, int* unsupported, cudaStream_t s);

// Host copy of the 1858-entry attention-policy gather table (slot in the 64*64 + 8*24 raw vector per move).
const short* attn_policy_src_table();

}  // namespace b200
