// Position encoding on the device: game history -> the 112 packed input planes (mask, value) of a position.
//
// Same decisions, in the same order, as the reference's host-side encoder: EncodePositionForNN
// (src/neural/encoder.cc:134-328) with history_planes = 8 and ChooseTransform (encoder.cc:50-104); the bit tricks are
// those of src/utils/bititer.h:66-89 and ChessBoard::Mirror (src/chess/board.cc:57-69).  Integer work, bit-exact.
// One warp per position: lane 0 walks the history (a short, branchy, sequential loop) into shared memory, the warp
// writes the planes out coalesced.
#include "../../include/b200nn.h"
#include "kernels.cuh"

namespace b200 {
namespace {

constexpr int kAux = 104;  // kAuxPlaneBase = 13 planes per board x 8 boards (src/neural/encoder.h:38-40)
constexpr uint64_t kAll = ~0ull;

__device__ __forceinline__ uint64_t reverse_bits_in_bytes(uint64_t v) {  // horizontal mirror
  v = ((v >> 1) & 0x5555555555555555ull) | ((v & 0x5555555555555555ull) << 1);
  v = ((v >> 2) & 0x3333333333333333ull) | ((v & 0x3333333333333333ull) << 2);
  v = ((v >> 4) & 0x0F0F0F0F0F0F0F0Full) | ((v & 0x0F0F0F0F0F0F0F0Full) << 4);
  return v;
}
__device__ __forceinline__ uint64_t reverse_bytes_in_bytes(uint64_t v) {  // vertical mirror
  const uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
  return ((uint64_t)__byte_perm(lo, 0, 0x0123) << 32) | (uint64_t)__byte_perm(hi, 0, 0x0123);
}
__device__ __forceinline__ uint64_t transpose_bits_in_bytes(uint64_t v) {  // across the h1-a8 diagonal
  v = (v & 0xAA00AA00AA00AA00ull) >> 9 | (v & 0x0055005500550055ull) << 9 | (v & 0x55AA55AA55AA55AAull);
  v = (v & 0xCCCC0000CCCC0000ull) >> 18 | (v & 0x0000333300003333ull) << 18 | (v & 0x3333CCCC3333CCCCull);
  v = (v & 0xF0F0F0F000000000ull) >> 36 | (v & 0x000000000F0F0F0Full) << 36 | (v & 0x0F0F0F0FF0F0F0F0ull);
  return v;
}

__device__ __forceinline__ bool is_canonical(int f) { return f >= 3; }   // encoder.cc:107-110
__device__ __forceinline__ bool is_hectoplies(int f) { return f >= 4; }  // encoder.cc:119-122
__device__ __forceinline__ bool is_armageddon(int f) { return f == 132 || f == 133; }
__device__ __forceinline__ bool is_v2(int f) { return f == 5 || f == 133; }

__device__ int compare_transposing(uint64_t value, int transform) {  // encoder.cc:36-48
  if (transform & 1) value = reverse_bits_in_bytes(value);
  if (transform & 2) value = reverse_bytes_in_bytes(value);
  const uint64_t alt = transpose_bits_in_bytes(value);
  return value < alt ? -1 : (value > alt ? 1 : 0);
}

__device__ int choose_transform(const b200_board& b) {  // encoder.cc:50-104
  if (b.castling != 0) return 0;
  uint64_t our_king = b.kings & b.ours;
  int transform = 0;
  if (our_king & 0x0F0F0F0F0F0F0F0Full) {
    transform |= 1;
    our_king = reverse_bits_in_bytes(our_king);
  }
  if (b.pawns != 0) return transform;
  if (our_king & 0xFFFFFFFF00000000ull) {
    transform |= 2;
    our_king = reverse_bytes_in_bytes(our_king);
  }
  if (our_king & 0xE0C08000ull) {
    transform |= 4;
  } else if (our_king & 0x10204080ull) {
    const uint64_t order[7] = {b.ours | b.theirs, b.ours, b.kings, b.queens, b.rooks, b.knights, b.bishops};
    for (int i = 0; i < 7; ++i) {
      const int outcome = compare_transposing(order[i], transform);
      if (outcome == -1) return transform;
      if (outcome == 1) return transform | 4;
    }
  }
  return transform;
}

__device__ void mirror(b200_board& b) {  // ChessBoard::Mirror, Castlings::Mirror (src/chess/board.h:148-152)
  const uint64_t ours = reverse_bytes_in_bytes(b.theirs), theirs = reverse_bytes_in_bytes(b.ours);
  b.ours = ours;
  b.theirs = theirs;
  b.pawns = reverse_bytes_in_bytes(b.pawns);
  b.knights = reverse_bytes_in_bytes(b.knights);
  b.bishops = reverse_bytes_in_bytes(b.bishops);
  b.rooks = reverse_bytes_in_bytes(b.rooks);
  b.queens = reverse_bytes_in_bytes(b.queens);
  b.kings = reverse_bytes_in_bytes(b.kings);
  b.en_passant = reverse_bytes_in_bytes(b.en_passant);
  b.castling = (uint8_t)(((b.castling & 3) << 2) | ((b.castling & 12) >> 2));
  const uint8_t q = b.rook_files[0], k = b.rook_files[1];
  b.rook_files[0] = b.rook_files[2];
  b.rook_files[1] = b.rook_files[3];
  b.rook_files[2] = q;
  b.rook_files[3] = k;
  b.flags ^= 1;
}

__device__ int encode_one(const b200_board* history, int size, bool from_start, int fmt, int fill, uint64_t* masks,
                          float* values) {
  const b200_board& last = history[size - 1];
  const bool we_are_black = last.flags & 1;
  const bool canonical = is_canonical(fmt);
  const int transform = canonical ? choose_transform(last) : 0;
  const uint8_t c = last.castling;
  if (fmt == 1) {  // encoder.cc:155-168
    if (c & 2) masks[kAux + 0] = kAll;
    if (c & 1) masks[kAux + 1] = kAll;
    if (c & 8) masks[kAux + 2] = kAll;
    if (c & 4) masks[kAux + 3] = kAll;
  } else {  // encoder.cc:170-203: the rooks that still have castling rights
    masks[kAux + 0] = ((c & 2) ? 1ull << last.rook_files[0] : 0) | ((c & 8) ? 1ull << (56 + last.rook_files[2]) : 0);
    masks[kAux + 1] = ((c & 1) ? 1ull << last.rook_files[1] : 0) | ((c & 4) ? 1ull << (56 + last.rook_files[3]) : 0);
  }
  if (canonical) masks[kAux + 4] = last.en_passant;
  else if (we_are_black) masks[kAux + 4] = kAll;
  masks[kAux + 5] = kAll;
  values[kAux + 5] = is_hectoplies(fmt) ? (float)last.rule50 / 100.0f : (float)last.rule50;
  if (is_armageddon(fmt) && we_are_black) masks[kAux + 6] = kAll;
  masks[kAux + 7] = kAll;

  const bool stop_early = canonical, skip_non_repeats = is_v2(fmt);
  bool flip = false;
  int history_idx = size - 1;
  for (int i = 0; i < 8;) {  // encoder.cc:234-308
    if (history_idx < 0 && !from_start) break;  // the caller's list does not reach further back
    const b200_board& position = history[history_idx < 0 ? 0 : history_idx];
    b200_board board = position;
    if (flip) mirror(board);
    if (stop_early && board.castling != c) break;
    if (stop_early && history_idx != size - 1 && board.en_passant != 0) break;
    if (fill == B200_FILL_NO && (history_idx < -1 || (history_idx == -1 && board.en_passant == 0))) break;
    if (history_idx < 0 && fill == B200_FILL_FEN_ONLY && (position.flags & 2)) break;
    if (skip_non_repeats && position.repetitions == 0 && i > 0) {
      if (history_idx > 0) flip = !flip;
      if (position.rule50 == 0) break;
      if (history_idx < 0) break;  // nothing further back can differ (the reference does not terminate here)
      --history_idx;
      continue;
    }
    const int base = i * 13;
    masks[base + 0] = board.ours & board.pawns;
    masks[base + 1] = board.ours & board.knights;
    masks[base + 2] = board.ours & board.bishops;
    masks[base + 3] = board.ours & board.rooks;
    masks[base + 4] = board.ours & board.queens;
    masks[base + 5] = board.ours & board.kings;
    masks[base + 6] = board.theirs & board.pawns;
    masks[base + 7] = board.theirs & board.knights;
    masks[base + 8] = board.theirs & board.bishops;
    masks[base + 9] = board.theirs & board.rooks;
    masks[base + 10] = board.theirs & board.queens;
    masks[base + 11] = board.theirs & board.kings;
    if (position.repetitions >= 1) masks[base + 12] = kAll;
    if (history_idx < 0 && board.en_passant != 0) {  // encoder.cc:290-300: take the double pawn push back
      const int idx = __ffsll((long long)board.en_passant) - 1;
      if (idx < 8) masks[base + 0] += (0x0000000000000100ull - 0x0000000001000000ull) << idx;
      else masks[base + 6] += (0x0001000000000000ull - 0x0000000100000000ull) << (idx - 56);
    }
    if (history_idx > 0) flip = !flip;
    if (stop_early && position.rule50 == 0) break;
    ++i;
    --history_idx;
  }
  if (transform != 0) {  // encoder.cc:309-325
    for (int p = 0; p <= kAux + 4; ++p) {
      uint64_t v = masks[p];
      if (v == 0 || v == kAll) continue;
      if (transform & 1) v = reverse_bits_in_bytes(v);
      if (transform & 2) v = reverse_bytes_in_bytes(v);
      if (transform & 4) v = transpose_bits_in_bytes(v);
      masks[p] = v;
    }
  }
  return transform;
}

__global__ void __launch_bounds__(128)
encode_positions_kernel(const b200_board* __restrict__ boards, const int* __restrict__ offsets,
                        const uint8_t* __restrict__ from_start, int n, int fmt, int fill, uint64_t* __restrict__ masks,
                        float* __restrict__ values, int* __restrict__ transforms) {
  __shared__ uint64_t sm[4][112];
  __shared__ float sv[4][112];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = blockIdx.x * 4 + warp;
  if (pos >= n) return;
  for (int i = lane; i < 112; i += 32) {
    sm[warp][i] = 0;
    sv[warp][i] = 1.0f;  // InputPlane's default value
  }
  __syncwarp();
  if (lane == 0) {
    const int first = offsets[pos], size = offsets[pos + 1] - first;
    int t = 0;
    if (size > 0) t = encode_one(boards + first, size, from_start[pos] != 0, fmt, fill, sm[warp], sv[warp]);
    if (transforms) transforms[pos] = t;
  }
  __syncwarp();
  for (int i = lane; i < 112; i += 32) {
    masks[(long long)pos * 112 + i] = sm[warp][i];
    values[(long long)pos * 112 + i] = sv[warp][i];
  }
}

// Training-data records -> planes: PlanesFromTrainingData (src/trainingdata/reader.cc:32-118).  One warp per packed
// V6 record (src/trainingdata/trainingdata_v6.h:36-87), one plane per lane and step.  undo = 0 leaves the planes as
// a network is fed them (what EncodePositionForNN produced when the record was written), undo = 1 takes the canonical
// formats' board transform back as the reference function does for the rescorer.
constexpr int kTdPlanes = 8 + 1858 * 4;        // byte offset of planes[104]
constexpr int kTdBytes = kTdPlanes + 104 * 8;  // castling x4, side to move / en passant, rule50, invariance info

__global__ void __launch_bounds__(128)
planes_from_training_data_kernel(const uint8_t* __restrict__ records, int n, long long stride, int undo,
                                 uint64_t* __restrict__ masks, float* __restrict__ values,
                                 int* __restrict__ unsupported) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rec = blockIdx.x * 4 + warp;
  if (rec >= n) return;
  const uint8_t* r = records + (long long)rec * stride;
  const int fmt = (int)*reinterpret_cast<const uint32_t*>(r + 4);  // records are 4-byte aligned (8356 = 4 * 2089)
  const bool known = (fmt >= 1 && fmt <= 5) || fmt == 132 || fmt == 133;
  if (!known && lane == 0 && unsupported) atomicAdd(unsupported, 1);
  const uint64_t us_ooo = r[kTdBytes + 0], us_oo = r[kTdBytes + 1], them_ooo = r[kTdBytes + 2], them_oo = r[kTdBytes + 3];
  const uint64_t stm_ep = r[kTdBytes + 4];
  const int rule50 = r[kTdBytes + 5], inv = r[kTdBytes + 6];
  for (int i = lane; i < 112; i += 32) {
    uint64_t m = 0;
    float v = 1.0f;
    if (known) {
      if (i < 104) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(r + kTdPlanes + i * 8);
        m = reverse_bits_in_bytes((uint64_t)p[0] | ((uint64_t)p[1] << 32));
      } else if (fmt == 1) {
        if (i == 104) m = us_ooo ? kAll : 0;
        else if (i == 105) m = us_oo ? kAll : 0;
        else if (i == 106) m = them_ooo ? kAll : 0;
        else if (i == 107) m = them_oo ? kAll : 0;
      } else {
        if (i == 104) m = us_ooo | (them_ooo << 56);
        else if (i == 105) m = us_oo | (them_oo << 56);
      }
      if (i == 108) m = is_canonical(fmt) ? stm_ep << 56 : (stm_ep ? kAll : 0);
      if (i == 109) {
        m = kAll;
        v = is_hectoplies(fmt) ? (float)rule50 / 100.0f : (float)rule50;
      }
      if (i == 110) m = (is_armageddon(fmt) && inv >= 128) ? kAll : 0;
      if (i == 111) m = kAll;
      if (undo && is_canonical(fmt) && inv != 0 && m != 0 && m != kAll) {
        if (inv & 4) m = transpose_bits_in_bytes(m);
        if (inv & 2) m = reverse_bytes_in_bytes(m);
        if (inv & 1) m = reverse_bits_in_bytes(m);
      }
    }
    masks[(long long)rec * 112 + i] = m;
    values[(long long)rec * 112 + i] = v;
  }
}

}  // namespace

cudaError_t launch_planes_from_training_data(const void* records, int n, long long stride, int undo, uint64_t* masks,
                                             float* values, int* unsupported, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  planes_from_training_data_kernel<<<ceil_div(n, 4), 128, 0, s>>>(static_cast<const uint8_t*>(records), n, stride,
                                                                   undo, masks, values, unsupported);
  return cudaGetLastError();
}

bool encode_format_supported(int input_format) {
  return (input_format >= 1 && input_format <= 5) || input_format == 132 || input_format == 133;
}

cudaError_t launch_encode_positions(const b200_board* boards, const int* offsets, const uint8_t* from_start, int n,
                                    int input_format, int fill, uint64_t* masks, float* values, int* transforms,
                                    cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  encode_positions_kernel<<<ceil_div(n, 4), 128, 0, s>>>(boards, offsets, from_start, n, input_format, fill, masks,
                                                          values, transforms);
  return cudaGetLastError();
}

}  // namespace b200
