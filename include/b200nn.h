/*
 * b200nn - C ABI of the B200 (sm_100a) neural-network evaluation backend for lc0.
 *
 * This is the boundary an lc0 backend plug-in binds: everything above it (the
 * `lczero::Network` / `NetworkComputation` classes registered with
 * REGISTER_NETWORK, or a Python/ctypes harness) is host glue; everything below
 * it is hand-written CUDA.  Plain pointers and sizes only; no C++ or torch types.
 *
 * Every function returns B200_OK (0) or an error code; `b200_last_error()`
 * returns a thread-local description of the last failure.  Nothing here falls
 * back to a CPU implementation: without a usable CUDA device the create call fails.
 */
#ifndef B200NN_H_
#define B200NN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200_OK = 0,
  B200_ERR_INVALID = 1,     /* bad argument, unknown key, inconsistent weight sizes */
  B200_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed */
  B200_ERR_UNSUPPORTED = 3, /* network format the backend does not implement */
  B200_ERR_NOMEM = 4,
  B200_ERR_TIMEOUT = 5      /* a bounded device-side wait gave up (kernel status word) */
};

/* Arithmetic/storage type of activations and matrices on the device. */
enum { B200_PREC_FP32 = 0, B200_PREC_FP16 = 1, B200_PREC_BF16 = 2 };

#define B200_INPUT_PLANES 112  /* lczero::kInputPlanes, src/neural/network.h:38 */
#define B200_POLICY_SIZE 1858  /* policy vector length, src/neural/backends/blas/network_blas.cc:130 */

typedef struct b200_builder b200_builder;
typedef struct b200_net b200_net;
typedef struct b200_comp b200_comp;

const char* b200_last_error(void);

/* ---- Network description -------------------------------------------------------------
 * Replaces the `WeightsFile` + `MultiHeadWeights` hand-over of the reference's backend
 * constructors (src/neural/backends/blas/network_blas.cc:983-1072,
 * src/neural/network_legacy.h:178-229): the host flattens the decoded weights into named
 * fp32 tensors ("encoder.3.mha.q_w", "policy.ip2_pol_w", "residual.0.se.w1", ...; dense
 * weights [out][in] row-major, conv weights [Cout][Cin][3][3], batch norm already folded)
 * and integer attributes:
 *   network, policy, value, moves_left, input_embedding, input_format, output_format
 *       -- pblczero::NetworkFormat enum values (proto/net.proto:275-367)
 *   default_activation, smolgen_activation, ffn_activation
 *       -- resolved lczero::ActivationFunction values (src/neural/tables/activation_function.h)
 *   headcount, pol_headcount
 */
int b200_builder_create(b200_builder** out);
int b200_builder_set_int(b200_builder* b, const char* key, long long value);
int b200_builder_add_tensor(b200_builder* b, const char* name, const float* data, size_t count);
void b200_builder_destroy(b200_builder* b);

/* ---- Network (lczero::Network, src/neural/network.h:116-126) ----------------------------
 * b200_net_create uploads and re-lays-out the weights on device `gpu` and allocates
 * `slots` evaluation workspaces of `max_batch` positions each (no allocation happens
 * during evaluation).  Options mirror the reference CUDA backend's `gpu` / `max_batch`
 * keys (src/neural/backends/cuda/network_cuda.cc:210-254). */
typedef struct b200_net_options {
  int gpu;        /* CUDA device ordinal */
  int max_batch;  /* largest batch one computation may hold */
  int precision;  /* B200_PREC_* */
  int slots;      /* concurrent computations (>= 1) */
  int mlh;        /* 0 disables the moves-left head like the reference's mlh=false */
  int flags;      /* B200_FLAG_* */
} b200_net_options;

enum {
  B200_FLAG_NO_TENSOR_CORES = 1, /* force the plain FMA matrix kernels in fp16/bf16 mode */
  B200_FLAG_NO_GRAPHS = 2,       /* launch kernels one by one instead of replaying captured CUDA graphs */
  /* Verification switches: each turns one fusion of the 16-bit tensor-core schedule off, so that a test can compare
   * the fused schedule with the plain one on the same network (results agree to rounding). */
  B200_FLAG_NO_LN_FOLD = 4,          /* run the encoder LayerNorms as kernels instead of folding them into the products */
  B200_FLAG_NO_MERGED_COMPRESS = 8,  /* smolgen compression as a product of its own instead of riding on the QKV launch */
  B200_FLAG_NO_SPLIT_LAST_WAVE = 16, /* whole 256x256 tiles in the last wave of the CTA-pair kernel */
  B200_FLAG_NO_FUSED_SE = 32,        /* squeeze-excitation as a kernel of its own instead of the convolution's epilogue */
  /* Residual networks in fp16 / bf16: 3x3 convolutions as Winograd F(4x4, 3x3) (transform kernels around 36 stacked
   * tensor-core products, the reference GPU backend's decomposition) instead of the direct tensor-core convolution.
   * Off by default: a quarter of the multiplications, but about ten times the rounding error in 16-bit storage. */
  B200_FLAG_WINOGRAD = 64,
  B200_FLAG_NO_SIDE_STREAM = 128,    /* smolgen's small dense layers in line instead of on a second stream beside the QKV
                                      * product; value and moves-left heads in line instead of beside the policy head */
  /* Ordinary launches instead of programmatic dependent launches: by default the tensor-core products, the attention
   * kernel and the LayerNorms are launched so that a kernel's prologue (barrier set-up, tensor-memory allocation,
   * descriptor prefetch) runs under the tail of the kernel before it; each waits for its predecessors' results
   * (griddepcontrol.wait) before its first global-memory access. */
  B200_FLAG_NO_DEPENDENT_LAUNCH = 256,
  /* One launch per convolution instead of the tower kernel.  By default a residual tower of at most 128 filters whose
   * blocks all carry a squeeze-excitation unit runs, in fp16 / bf16 and for batches up to a few hundred positions, as
   * ONE launch: a CTA owns two boards and walks the input convolution and every block for them (a convolution and the
   * squeeze-excitation unit only mix squares of one board), waiting only for its own stores between layers. */
  B200_FLAG_NO_TOWER_KERNEL = 512
};

typedef struct b200_net_info {
  int input_format, output_format, moves_left_format; /* NetworkCapabilities, network.h:85-113 */
  int wdl;            /* 1: q = W - L and d = D; 0: q = tanh(value), d = 0 */
  int has_mlh;        /* GetMVal returns 0 when 0 */
  int attention_body; /* 1 for NETWORK_ATTENTIONBODY_* */
  int embedding, encoder_layers, heads, dff, filters, residual_blocks;
  int max_batch, precision, sm_count;
  long long weight_bytes, workspace_bytes;
  double flops_per_position;      /* all matrix products, 2 * MACs */
  double gemm_flops_per_position; /* encoder QKV / out-projection / FFN products only */
} b200_net_info;

int b200_net_create(const b200_builder* b, const b200_net_options* opt, b200_net** out);
int b200_net_get_info(const b200_net* net, b200_net_info* info);
void b200_net_destroy(b200_net* net);

/* ---- Computation (lczero::NetworkComputation, src/neural/network.h:56-71) -----------------
 * create -> add_input x n -> compute -> read results -> destroy; the heavy buffers are
 * pooled in the network like the reference does (network_cuda.cc:1066-1083). */
int b200_comp_create(b200_net* net, b200_comp** out);                       /* NewComputation */
int b200_comp_add_input(b200_comp* c, const uint64_t* masks, const float* values); /* AddInput: 112 + 112 */
int b200_comp_add_inputs(b200_comp* c, const uint64_t* masks, const float* values, int n);
int b200_comp_compute(b200_comp* c);                                        /* ComputeBlocking */
int b200_comp_batch_size(const b200_comp* c);                               /* GetBatchSize */
float b200_comp_q(const b200_comp* c, int sample);                          /* GetQVal */
float b200_comp_d(const b200_comp* c, int sample);                          /* GetDVal */
float b200_comp_m(const b200_comp* c, int sample);                          /* GetMVal */
float b200_comp_p(const b200_comp* c, int sample, int move_id);             /* GetPVal: raw logit */
const float* b200_comp_policy(const b200_comp* c, int sample);              /* 1858 raw logits */
void b200_comp_destroy(b200_comp* c);

/* Legal-move policy on the device: what lc0's new-API wrapper does on the host after ComputeBlocking
 * (NetworkAsBackendComputation::SoftmaxPolicy, src/neural/wrapper.cc:135-156: gather GetPVal for every legal move,
 * subtract the maximum, FastExp((p - max) * inv_temperature) of src/utils/fastmath.h:59-86, normalise).
 * b200_comp_add_input_with_moves adds one position together with the policy indices of its legal moves
 * (MoveToNNIndex(move, transform), at most 256); b200_comp_legal_policy returns a pointer to that position's
 * probabilities in move order.  With compact != 0 the 1858-logit vectors are not copied to the host at all
 * (GetPVal / b200_comp_policy are then undefined): 1 KB instead of 7.4 KB per position crosses PCIe. */
int b200_comp_add_input_with_moves(b200_comp* c, const uint64_t* masks, const float* values,
                                   const uint16_t* move_ids, int n_moves);
/* n positions at once: move_ids is [n][256] (rows padded), n_moves [n]. */
int b200_comp_add_inputs_with_moves(b200_comp* c, const uint64_t* masks, const float* values,
                                    const uint16_t* move_ids, const int* n_moves, int n);
int b200_comp_set_policy_options(b200_comp* c, float inv_temperature, int compact);
int b200_comp_legal_policy(const b200_comp* c, int sample, const float** probs, int* n_moves);

/* ---- Whole-batch entry points ----------------------------------------------------------------
 * b200_net_eval_host: one call = add n inputs, compute, copy results out.  Host pointers;
 *   H2D and D2H copies are part of the call.  policy [n][1858], q/d/m [n]; any may be NULL.
 * b200_net_eval_device: inputs and outputs already in device memory of the net's GPU
 *   (masks [n][112] u64, values [n][112] f32, policy [n][1858] f32, qdm [n][3] f32 as q,d,m);
 *   enqueues on the slot's stream and synchronises before returning.
 * b200_net_enqueue_device / b200_net_sync: the same without the final synchronisation, so a
 *   caller can time many evaluations with events on b200_net_stream().  These entry points run on workspace slot 0
 *   and take it out of the pool the computations draw from: the enqueue form holds it until b200_net_sync (which also
 *   reports a kernel time-out of the enqueued evaluations), so every b200_net_enqueue_device must be followed by a
 *   b200_net_sync before a network with a single slot can serve a computation again. */
int b200_net_eval_host(b200_net* net, const uint64_t* masks, const float* values, int n,
                       float* policy, float* q, float* d, float* m);
int b200_net_eval_device(b200_net* net, const void* d_masks, const void* d_values, int n,
                         void* d_policy, void* d_qdm);
int b200_net_enqueue_device(b200_net* net, const void* d_masks, const void* d_values, int n,
                            void* d_policy, void* d_qdm);
int b200_net_sync(b200_net* net);
void* b200_net_stream(b200_net* net); /* cudaStream_t of slot 0 */

/* Number of kernels this library launched on behalf of `net` since creation. */
long long b200_net_launch_count(const b200_net* net);
/* Device status word written by kernels whose bounded waits gave up (0 = none).  Every evaluation call reads its own
 * slot's word with its results and returns B200_ERR_TIMEOUT (and clears the word) when it is set; this accessor is for
 * diagnostics. */
int b200_net_device_status(b200_net* net);
/* Failure-injection hook for tests of that error path: writes `code` into the status words from the host, as a kernel
 * that gave up would; the next evaluation of each slot then fails with B200_ERR_TIMEOUT.  No kernel is disturbed. */
int b200_net_inject_device_status(b200_net* net, int code);

/* Per-kernel-class timing with CUDA events recorded on the evaluation stream around every launch
 * (off by default).  Classes: 0 tensor-core GEMM, 1 FMA GEMM, 2 attention, 3 LayerNorm, 4 other.
 * b200_net_get_profile waits for the recorded events and returns, per class, the summed device time
 * in ms, the summed algorithmic work (FLOPs for the GEMM classes, bytes for the others) and the number
 * of launches; arrays of B200_PROFILE_CLASSES entries.  The reference has the DEBUG_RAW_NPS timing
 * ifdef in its forward pass for the same purpose (src/neural/backends/cuda/network_cuda.cc:715-717). */
#define B200_PROFILE_CLASSES 5
int b200_net_set_profiling(b200_net* net, int enabled);
int b200_net_get_profile(b200_net* net, double* ms, double* work, long long* launches, int reset);
/* The same sums by tag, for the launches that carry one (arrays of B200_PROFILE_TAGS entries): 1 QKV (+ smolgen
 * compression), 2 attention output projection, 3 FFN dense 1, 4 FFN dense 2, 5 smolgen dense layers, 6 smolgen bias
 * product, 7 attention, 8 embedding block, 9 heads; the products of ForwardEncoderLayer
 * (src/neural/backends/blas/network_blas.cc:271-471) one by one. */
#define B200_PROFILE_TAGS 16
int b200_net_get_profile_tagged(b200_net* net, double* ms, double* work, long long* launches, int reset);

/* ---- Batch aggregation across caller threads ------------------------------------------------------------------
 * Many threads with a few positions each, one GPU batch: the role of the reference's `multiplexing` decorator
 * (MuxingNetwork::Worker, src/neural/backends/network_mux.cc:169-205).  b200_mux_eval blocks until its positions
 * have been evaluated together with whatever other callers queued meanwhile; two worker threads alternate, a worker
 * that finds fewer than max_batch positions queued waits up to wait_us microseconds for more.  Outputs as in
 * b200_net_eval_host (any may be NULL).  The network must outlive the aggregator; destroying the aggregator fails the
 * requests still queued. */
typedef struct b200_mux b200_mux;
int b200_mux_create(b200_net* net, int max_batch, int wait_us, b200_mux** out);
int b200_mux_eval(b200_mux* mux, const uint64_t* masks, const float* values, int n, float* policy, float* q, float* d,
                  float* m);
int b200_mux_stats(b200_mux* mux, long long* requests, long long* batches, long long* positions);
void b200_mux_destroy(b200_mux* mux);

/* ---- One batch over several GPUs of the box ---------------------------------------------------------------------
 * Positions are independent: the batch is cut into contiguous slices whose sizes differ by at most one (b200_multi_slice),
 * one per GPU, the weights are replicated, nothing is exchanged.  The role of the reference's `demux` decorator
 * (DemuxingComputation::ComputeBlocking, src/neural/backends/network_demux.cc:279-334) without its per-slice
 * computations: one persistent host thread per GPU evaluates its slice with b200_net_eval_host and writes the results
 * into the caller's arrays at the slice's offset.  `opt->gpu` is ignored, `opt->max_batch` is per GPU; the same GPU may
 * be listed more than once.  Calls are serialised. */
typedef struct b200_multi b200_multi;
void b200_multi_slice(int n, int parts, int part, int* begin, int* count);
int b200_multi_create(const b200_builder* b, const b200_net_options* opt, const int* gpus, int n_gpus,
                      b200_multi** out);
int b200_multi_gpu_count(const b200_multi* mg);
b200_net* b200_multi_net(b200_multi* mg, int i);
int b200_multi_eval_host(b200_multi* mg, const uint64_t* masks, const float* values, int n, float* policy, float* q,
                         float* d, float* m);
void b200_multi_destroy(b200_multi* mg);

/* ---- Position encoding on the device ------------------------------------------------------------------------
 * What lc0 does on the host before AddInput: EncodePositionForNN (src/neural/encoder.cc:134-328) turns the game
 * history into the 112 packed planes, with ChooseTransform (encoder.cc:50-104) for the canonical formats.  Here the
 * caller passes the history itself, 88 bytes per position of the history instead of 1344 bytes of planes per evaluated
 * position, and a kernel produces the planes where the network reads them.
 *
 * b200_board is one position of the history as Position::GetBoard() stores it (from the point of view of the side to
 * move; bit i of a board = square i, a1 = 0, h8 = 63):
 *   ours .. kings       ChessBoard::ours(), theirs(), pawns(), knights(), bishops(), rooks(), queens(), kings()
 *   en_passant          ChessBoard::en_passant()
 *   castling            ChessBoard::Castlings::as_int(): bit 0 we O-O, 1 we O-O-O, 2 they O-O, 3 they O-O-O
 *   rook_files          our queenside, our kingside, their queenside, their kingside rook file (0 = a)
 *   flags               bit 0 ChessBoard::flipped() (black to move), bit 1 the board equals ChessBoard::kStartposBoard
 *   rule50, repetitions Position::GetRule50Ply(), GetRepetitions()
 * A history is given oldest first with the position to encode last; `from_start` says that its first entry is the
 * first position of the game history (the encoder may then repeat it to fill missing planes, as fill_empty_history
 * asks).  A history that does not start there must hold at least 8 entries or, for the two V2 input formats, reach
 * back to an entry with rule50 == 0; the walk stops at its beginning. */
typedef struct b200_board {
  uint64_t ours, theirs, pawns, knights, bishops, rooks, queens, kings, en_passant;
  uint8_t castling;
  uint8_t rook_files[4];
  uint8_t flags;
  uint16_t rule50;
  uint8_t repetitions;
  uint8_t reserved[7];
} b200_board; /* 88 bytes */
#define B200_FILL_NO 0        /* FillEmptyHistory::NO (src/neural/encoder.h:42) */
#define B200_FILL_FEN_ONLY 1
#define B200_FILL_ALWAYS 2
/* Stand-alone operator: n positions; the history of position i is boards[offsets[i] .. offsets[i+1]) (offsets has
 * n + 1 entries), from_start[i] as above.  Writes masks [n][112], values [n][112] and, when not NULL, transforms [n]
 * (the value EncodePositionForNN returns through transform_out).  All pointers are device pointers. */
int b200_op_encode_positions(const b200_board* d_boards, const int* d_offsets, const uint8_t* d_from_start, int n,
                             int input_format, int fill_empty_history, uint64_t* d_masks, float* d_values,
                             int* d_transforms, void* stream);
/* Computation-level entry (instead of b200_comp_add_input): adds one position by its history (host memory, at most
 * B200_MAX_HISTORY entries) and optionally the policy indices of its legal moves (n_moves < 0: none; see
 * b200_comp_add_input_with_moves).  The planes are produced on the device at b200_comp_compute.  All positions of a
 * computation must be added the same way.  b200_comp_set_encoding chooses the input format (default: the network's)
 * and the fill policy (default B200_FILL_FEN_ONLY, lc0's default). */
#define B200_MAX_HISTORY 128
int b200_comp_set_encoding(b200_comp* c, int input_format, int fill_empty_history);
int b200_comp_add_position(b200_comp* c, const b200_board* history, int count, int from_start,
                           const uint16_t* move_ids, int n_moves);
/* n positions at once: histories concatenated in `boards` with n + 1 `offsets` (as in b200_op_encode_positions, host
 * memory), from_start [n]; move_ids [n][256] (rows padded) and n_moves [n], or both NULL for no move lists. */
int b200_comp_add_positions(b200_comp* c, const b200_board* boards, const int* offsets, const uint8_t* from_start,
                            const uint16_t* move_ids, const int* n_moves, int n);

/* ---- Training-data records -> planes -------------------------------------------------------------------------
 * PlanesFromTrainingData (src/trainingdata/reader.cc:32-118) for n packed V6TrainingData records
 * (src/trainingdata/trainingdata_v6.h:36-87, 8356 bytes; V7 records start with the same fields) that lie
 * `record_stride` bytes apart in device memory (4-byte aligned).  Writes masks [n][112] and values [n][112], the
 * input of b200_net_eval_device / b200_op_expand_planes.  undo_transform = 0 gives the planes as a network is fed
 * them (what EncodePositionForNN produced when the record was written); 1 takes the canonical formats' board transform
 * back, which is what the reference function returns to the rescorer.  Records with an input format the reference
 * rejects get empty planes and are counted in *d_unsupported (device int, may be NULL; the caller zeroes it). */
int b200_op_planes_from_training_data(const void* d_records, int n, long long record_stride, int undo_transform,
                                      uint64_t* d_masks, float* d_values, int* d_unsupported, void* stream);

/* ---- Stand-alone operators (unit-test and profiling surface of the same kernels) --------------
 * All pointers are device pointers on the current device; `stream` is a cudaStream_t or NULL.
 * b200_op_expand_planes: 112 (mask,value) pairs per position -> dense [n][112][64] values of
 *   `precision` type (BlasComputation::EncodePlanes, network_blas.cc:973-981).
 * b200_op_gemm: C[M][N] = act(A[M][K] . W[N][K]^T + bias) in the given precision, using the
 *   tcgen05 tensor-core kernel when use_tc != 0 (fp16/bf16 only) else the FMA kernel
 *   (FullyConnectedLayer::Forward1D, fully_connected_layer.cc:50-106).
 * b200_op_layer_norm: out = LN(alpha * x + skip) * gamma + beta over rows of width C
 *   (LayerNorm2DWithSkipConnection, backends/blas/encoder.h:29-78). */
int b200_op_expand_planes(const void* d_masks, const void* d_values, int n, void* d_out,
                          int precision, void* stream);
int b200_op_gemm(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                 int activation, int precision, int use_tc, void* stream);
/* b200_op_gemm_ex: the tensor-core product with every epilogue the network's schedule uses, for tests of those
 *   epilogues on their own.  out = alpha * act(rstd_a * (scale * A . W^T - mean_a * colsum) + bias) + residual, where
 *   - a_stats [M][2] (double; per-row sum and sum of squares of A's rows over K columns, with a_inv_c = 1/K and a_eps) and
 *     colsum [N] describe a LayerNorm of A folded into the product (W then holds W * gamma, bias holds
 *     beta . W^T + b): LayerNorm2DWithSkipConnection followed by Forward1D (backends/blas/encoder.h:29-78,
 *     fully_connected_layer.cc:50-106) in one launch; NULL: plain product;
 *   - res [M][N] is added after the activation, normalised on the fly with res_stats / res_gamma / res_beta
 *     (res_inv_c = 1/N, res_eps) when those are given;
 *   - out_stats [M][2] (double) accumulates the per-row sum and sum of squares of the outputs (the caller zeroes it);
 *   - columns [n_split, N) go to C2 (leading dimension ldc2) instead of C when n_split > 0.
 *   Leading dimensions of 0 mean dense.  fp16 / bf16 only; synchronises the stream before returning. */
typedef struct b200_gemm_desc {
  const void* A; const void* W; const float* bias; void* C;
  int M, N, K;
  long long lda, ldw, ldc;
  int activation, precision;
  float scale, alpha;
  const double* a_stats; const float* colsum; float a_inv_c, a_eps;
  const void* res; long long ldres;
  const double* res_stats; const float* res_gamma; const float* res_beta; float res_inv_c, res_eps;
  double* out_stats;
  void* C2; long long ldc2; int n_split;
  int whole_tiles;
} b200_gemm_desc;
int b200_op_gemm_ex(const b200_gemm_desc* d, void* stream);
/* b200_op_attention: out = softmax(Q K^T / sqrt(depth) + bias) V for every (position, head) of n positions of 64
 *   tokens (BlasComputation::ForwardEncoderLayer, network_blas.cc:352-439).  q, k, v: [n*64] rows with leading
 *   dimension ld (elements), head h in columns [h*depth, (h+1)*depth); bias: [n][heads][64][64] or NULL; out:
 *   [n*64] rows with leading dimension ldo.  variant 0: FMA kernel (any precision); 1: persistent TMA +
 *   tensor-core kernel (the one the network uses; fp16 / bf16, depth 32 or 64). */
int b200_op_attention(const void* q, const void* k, const void* v, long long ld, const void* bias, void* out,
                      long long ldo, int n, int heads, int depth, int precision, int variant, void* stream);
/* b200_op_gemm_timed: the tensor-core product of b200_op_gemm queued `launches` times back to back on `stream`
 *   between two CUDA events; *ms_per_launch = elapsed / launches.  With enough launches the host's launch latency
 *   drops out, which is what a launch costs inside a replayed graph (profiling surface only). */
int b200_op_gemm_timed(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                       int activation, int precision, int launches, float* ms_per_launch, void* stream);
/* b200_op_scratch_residency_probe (profiling surface): every SM's CTA writes a private scratch slice of slice_kb, streams
 *   stream_kb of a 2 GiB buffer and reads the slice back, `iters` times; *ms_out = best of three timed launches.  mode
 *   bit 0: L2 evict_last policy on the scratch accesses, bit 1: evict_first on the stream loads, bit 2: discard the
 *   slice after reading, bit 3: stream only.  Under ncu the DRAM byte counters of this launch show whether a scratch
 *   tensor of that footprint stays in L2 (the question behind keeping the smolgen bias a materialised tensor). */
int b200_op_scratch_residency_probe(int slice_kb, int stream_kb, int iters, int mode, float* ms_out);
/* b200_op_policy_attention: tail of the attention policy head for n positions: logits = Q K^T / sqrt(dm)
 *   per position (64x64), promotion offsets from the rank-8 keys and `w4` ([4][dm], fp32), and the gather of
 *   the 1858 move logits (network_blas.cc:850-914).  q, k: [n*64][dm] in `precision`; scratch_logits: n*4096
 *   floats of device memory the caller provides; policy: [n][1858] fp32. */
int b200_op_policy_attention(const void* q, const void* k, const float* w4, int dm, int n, float* scratch_logits,
                             float* policy, int precision, void* stream);
/* b200_op_policy_attention_static: the same operator for callers that cannot hand over scratch memory.
 *   It has no counterpart in the reference.  lc0's search threads call the backend from a hot loop where a
 *   cudaMalloc would synchronise the device, and some hosts give every free byte to their own pool at
 *   start-up; neither can allocate n*4096 floats per call.  Here the scratch is a fixed array inside the
 *   library (4 MiB, held by every GPU that loads the library until the process exits), so the call
 *   allocates nothing, on the device or through any allocating library routine.
 *   Limit: n <= B200_STATIC_POLICY_MAX_POSITIONS, larger batches are refused with B200_ERR_INVALID.
 *   The first call on each device looks up the array's device address and uploads the gather table; make
 *   that first call before any stream capture begins.  All calls share the one array (it keeps the last
 *   call's logits; nothing in it needs clearing), so two calls whose kernels may overlap on the GPU race:
 *   issue them on one stream or order them yourself. */
#define B200_STATIC_POLICY_MAX_POSITIONS 256
int b200_op_policy_attention_static(const void* q, const void* k, const float* w4, int dm, int n, float* policy,
                                    int precision, void* stream);
int b200_op_layer_norm(void* out, const void* x, const void* skip, const float* gamma,
                       const float* beta, int rows, int C, float alpha, float eps, int precision,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NN_H_ */
