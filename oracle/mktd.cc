// mktd: V6 training-data records for seeded game histories and the planes the reference reconstructs from them, for
// pinning the restatement (oracle/encoder.py planes_from_training_data) and the device-side reader.  Test
// infrastructure only.  The records are filled the way the reference's writer fills them
// (src/trainingdata/trainingdata.cc:118-214: planes, castling bytes, side to move / en passant, rule-50 counter,
// invariance info); the planes come from the reference's own PlanesFromTrainingData (src/trainingdata/reader.cc:32-118)
// and, for the form a network is fed, from EncodePositionForNN itself.
//
// usage: mktd <out.td> <count>
// Output (little endian): char magic[8] = "LC0TDV6\0"; int32 n_records; then per record: uint32 input_format;
// uint64 planes[104]; uint8 castling_us_ooo, castling_us_oo, castling_them_ooo, castling_them_oo,
// side_to_move_or_enpassant, rule50_count, invariance_info; uint8 pad; uint64 reader_masks[112]; float
// reader_values[112] (PlanesFromTrainingData); uint64 encoder_masks[112]; float encoder_values[112]
// (EncodePositionForNN).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <random>

#include "chess/board.h"
#include "chess/position.h"
#include "neural/encoder.h"
#include "trainingdata/reader.h"
#include "trainingdata/trainingdata_v6.h"

using namespace lczero;

int main(int argc, char** argv) {
  if (argc < 3) {
    std::cerr << "usage: mktd <out.td> <count>\n";
    return 2;
  }
  const int count = atoi(argv[2]);
  InitializeMagicBitboards();
  const char* fens[] = {
      ChessBoard::kStartposFen,
      "rnbqkbnr/ppp1pppp/8/8/3pP3/8/PPPP1PPP/RNBQKBNR b KQkq e3 0 3",
      "4k3/8/8/8/8/8/4P3/4K3 w - - 0 1",
      "8/8/8/8/8/2k5/8/K1Q5 w - - 10 40",
      "K7/8/2k5/8/8/8/8/6Q1 w - - 7 60",
      "7K/8/5k2/8/8/8/8/1Q6 b - - 7 60",
      "8/6K1/8/4k3/8/8/8/R7 b - - 12 50",
      "bnrqkrnb/pppppppp/8/8/8/8/PPPPPPPP/BNRQKRNB w FCfc - 0 1",
  };
  const int n_fens = sizeof(fens) / sizeof(fens[0]);
  const int formats[] = {1, 2, 3, 4, 132};
  FILE* f = fopen(argv[1], "wb");
  if (!f) return 1;
  const char magic[8] = {'L', 'C', '0', 'T', 'D', 'V', '6', 0};
  fwrite(magic, 1, 8, f);
  const int32_t n_records = count * 5;
  fwrite(&n_records, 4, 1, f);
  for (int s = 0; s < count; ++s) {
    std::mt19937_64 rng(88000000ull + uint64_t(s));
    const int which = (s % 3 == 0) ? 0 : int(rng() % n_fens);
    const int target = which == 0 ? int(rng() % 100) : int(rng() % 14);
    ChessBoard board;
    int rule50 = 0, moves = 1;
    board.SetFromFen(fens[which], &rule50, &moves);
    PositionHistory history;
    history.Reset(board, rule50, 2 * (moves - 1) + (board.flipped() ? 1 : 0));
    for (int ply = 0; ply < target; ++ply) {
      const MoveList legal = history.Last().GetBoard().GenerateLegalMoves();
      if (legal.empty()) break;
      history.Append(legal[rng() % legal.size()]);
      if (history.ComputeGameResult() != GameResult::UNDECIDED) {
        history.Pop();
        break;
      }
    }
    const Position& position = history.Last();
    const auto& castlings = position.GetBoard().castlings();
    for (int fm : formats) {
      const auto input_format = static_cast<pblczero::NetworkFormat::InputFormat>(fm);
      V6TrainingData r;
      memset(&r, 0, sizeof(r));
      r.version = 6;
      r.input_format = fm;
      int transform = 0;
      const InputPlanes planes = EncodePositionForNN(input_format, history, 8, FillEmptyHistory::FEN_ONLY, &transform);
      for (int i = 0; i < 104; ++i) r.planes[i] = ReverseBitsInBytes(planes[i].mask);
      uint8_t oq = 1, ok = 1, tq = 1, tk = 1;
      if (fm >= 2) {  // Is960CastlingFormat
        oq <<= castlings.our_queenside_rook.idx;
        ok <<= castlings.our_kingside_rook.idx;
        tq <<= castlings.their_queenside_rook.idx;
        tk <<= castlings.their_kingside_rook.idx;
      }
      r.castling_us_ooo = castlings.we_can_000() ? oq : 0;
      r.castling_us_oo = castlings.we_can_00() ? ok : 0;
      r.castling_them_ooo = castlings.they_can_000() ? tq : 0;
      r.castling_them_oo = castlings.they_can_00() ? tk : 0;
      if (IsCanonicalFormat(input_format)) {
        r.side_to_move_or_enpassant = position.GetBoard().en_passant().as_int() >> 56;
        if (transform & FlipTransform) r.side_to_move_or_enpassant = ReverseBitsInBytes(r.side_to_move_or_enpassant);
        r.invariance_info = transform | (position.IsBlackToMove() ? (1u << 7) : 0u);
      } else {
        r.side_to_move_or_enpassant = position.IsBlackToMove() ? 1 : 0;
        r.invariance_info = 0;
      }
      r.rule50_count = position.GetRule50Ply();
      const InputPlanes back = PlanesFromTrainingData(r);
      fwrite(&r.input_format, 4, 1, f);
      fwrite(r.planes, 8, 104, f);
      const uint8_t bytes[8] = {r.castling_us_ooo, r.castling_us_oo, r.castling_them_ooo, r.castling_them_oo,
                                r.side_to_move_or_enpassant, r.rule50_count, r.invariance_info, 0};
      fwrite(bytes, 1, 8, f);
      for (int i = 0; i < 112; ++i) fwrite(&back[i].mask, 8, 1, f);
      for (int i = 0; i < 112; ++i) fwrite(&back[i].value, 4, 1, f);
      for (int i = 0; i < 112; ++i) fwrite(&planes[i].mask, 8, 1, f);
      for (int i = 0; i < 112; ++i) fwrite(&planes[i].value, 4, 1, f);
    }
  }
  fclose(f);
  return 0;
}
