// mkenc: game histories and the reference encoder's planes for them, for pinning the encoder restatement
// (oracle/encoder.py) and the device-side encoder.  Test infrastructure only.  It drives the reference's own chess
// rules and EncodePositionForNN (chess/position.h, neural/encoder.cc:134-328).
//
// usage: mkenc <out.enc> <count>
// Output (little endian): char magic[8] = "LC0ENC1\0"; int32 n; int32 n_combos; int32 combos[n_combos][2]
// (input format, fill policy); then per sample: int32 count; int32 from_start; b200_board boards[count] (oldest
// first); per combo: uint64 masks[112]; float values[112]; int32 transform.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <random>
#include <vector>

#include "chess/board.h"
#include "chess/position.h"
#include "include/b200nn.h"
#include "neural/encoder.h"

using namespace lczero;

static b200_board Record(const Position& p) {
  const ChessBoard& b = p.GetBoard();
  b200_board r{};
  r.ours = b.ours().as_int();
  r.theirs = b.theirs().as_int();
  r.pawns = b.pawns().as_int();
  r.knights = b.knights().as_int();
  r.bishops = b.bishops().as_int();
  r.rooks = b.rooks().as_int();
  r.queens = b.queens().as_int();
  r.kings = b.kings().as_int();
  r.en_passant = b.en_passant().as_int();
  const auto& c = b.castlings();
  r.castling = c.as_int();
  r.rook_files[0] = c.our_queenside_rook.idx;
  r.rook_files[1] = c.our_kingside_rook.idx;
  r.rook_files[2] = c.their_queenside_rook.idx;
  r.rook_files[3] = c.their_kingside_rook.idx;
  r.flags = (b.flipped() ? 1 : 0) | (b == ChessBoard::kStartposBoard ? 2 : 0);
  r.rule50 = static_cast<uint16_t>(p.GetRule50Ply());
  r.repetitions = static_cast<uint8_t>(p.GetRepetitions());
  return r;
}

int main(int argc, char** argv) {
  if (argc < 3) {
    std::cerr << "usage: mkenc <out.enc> <count>\n";
    return 2;
  }
  const int count = atoi(argv[2]);
  InitializeMagicBitboards();
  // Starting positions: the standard one (most samples) and positions that reach what random playouts from it rarely
  // do: an en-passant square in the first position of the history, no castling rights, pawnless boards with the side to
  // move's king in each quadrant and on the long diagonal (every transform), Chess960 rook files.
  const char* fens[] = {
      ChessBoard::kStartposFen,
      "rnbqkbnr/ppp1pppp/8/8/3pP3/8/PPPP1PPP/RNBQKBNR b KQkq e3 0 3",
      "rnbqkbnr/pppp1ppp/8/4pP2/8/8/PPPPP1PP/RNBQKBNR w KQkq e6 0 3",
      "4k3/8/8/8/8/8/4P3/4K3 w - - 0 1",
      "8/8/8/8/8/2k5/8/K1Q5 w - - 10 40",
      "8/8/8/8/8/5k2/8/2Q4K w - - 3 40",
      "K7/8/2k5/8/8/8/8/6Q1 w - - 7 60",
      "7K/8/5k2/8/8/8/8/1Q6 b - - 7 60",
      "8/8/8/4k3/8/8/1K6/7R w - - 0 50",
      "8/6K1/8/4k3/8/8/8/R7 b - - 12 50",
      "8/8/2k5/8/8/5K2/8/3R1B2 w - - 5 30",
      "bnrqkrnb/pppppppp/8/8/8/8/PPPPPPPP/BNRQKRNB w FCfc - 0 1",
      "r3k2r/8/8/8/8/8/8/R3K2R b Kq - 4 20",
  };
  const int n_fens = sizeof(fens) / sizeof(fens[0]);
  const int formats[] = {1, 2, 3, 4, 132, 5, 133};
  const FillEmptyHistory fills[] = {FillEmptyHistory::NO, FillEmptyHistory::FEN_ONLY, FillEmptyHistory::ALWAYS};

  FILE* f = fopen(argv[1], "wb");
  if (!f) return 1;
  const char magic[8] = {'L', 'C', '0', 'E', 'N', 'C', '1', 0};
  fwrite(magic, 1, 8, f);
  const int32_t n_combos = 21;
  fwrite(&count, 4, 1, f);
  fwrite(&n_combos, 4, 1, f);
  for (int fm : formats)
    for (int fl = 0; fl < 3; ++fl) {
      const int32_t pair[2] = {fm, fl};
      fwrite(pair, 4, 2, f);
    }

  for (int s = 0; s < count; ++s) {
    std::mt19937_64 rng(77000000ull + uint64_t(s));
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
      // prefer shuffling pieces back and forth now and then so that repetitions occur
      Move mv = legal[rng() % legal.size()];
      history.Append(mv);
      if (history.ComputeGameResult() != GameResult::UNDECIDED) {
        history.Pop();
        break;
      }
    }
    const auto positions = history.GetPositions();
    const int size = int(positions.size());
    // Odd samples pass a truncated history: the last 8 entries, extended back to the latest entry with rule50 == 0
    // at or before that point (what the V2 formats may walk to).
    int first = 0;
    if (s % 2 == 1 && size > 8) {
      first = size - 8;
      while (first > 0 && positions[first].GetRule50Ply() != 0) --first;
      if (size - first > B200_MAX_HISTORY) first = 0;
    }
    const int32_t cnt = size - first, from_start = first == 0 ? 1 : 0;
    fwrite(&cnt, 4, 1, f);
    fwrite(&from_start, 4, 1, f);
    for (int i = first; i < size; ++i) {
      const b200_board r = Record(positions[i]);
      fwrite(&r, sizeof(r), 1, f);
    }
    for (int fm : formats)
      for (int fl = 0; fl < 3; ++fl) {
        // The reference does not terminate when a V2 format walks past the first position of a history whose
        // rule-50 counter is not zero (a FEN start with a half-move clock) and the fill policy lets it continue:
        // such combinations are marked with transform = -1 and left out of the comparison.
        const bool v2 = fm == 5 || fm == 133;
        if (v2 && fl != 0 && positions[0].GetRule50Ply() != 0) {
          const uint64_t zm = 0;
          const float zv = 0.f;
          for (int i = 0; i < 112; ++i) fwrite(&zm, 8, 1, f);
          for (int i = 0; i < 112; ++i) fwrite(&zv, 4, 1, f);
          const int32_t t = -1;
          fwrite(&t, 4, 1, f);
          continue;
        }
        int transform = 0;
        const InputPlanes planes = EncodePositionForNN(static_cast<pblczero::NetworkFormat::InputFormat>(fm),
                                                       history, 8, fills[fl], &transform);
        for (int i = 0; i < 112; ++i) fwrite(&planes[i].mask, 8, 1, f);
        for (int i = 0; i < 112; ++i) fwrite(&planes[i].value, 4, 1, f);
        const int32_t t = transform;
        fwrite(&t, 4, 1, f);
      }
  }
  fclose(f);
  return 0;
}
