// mkpos: seeded random legal playouts -> position file of 112 packed input planes.
// Test infrastructure only. It drives the reference's own chess rules and
// position encoder (chess/board.h, chess/position.h, neural/encoder.cc:134)
// so that the planes fed to both the reference backend and the CUDA backend
// are exactly what lc0's search would produce.
//
// usage: mkpos <out.pos> <count> <input_format:int> <mix:uniform|split> [first_sample]
//   uniform: target ply uniform in [1,60]
//   split  : even samples ply in [1,20], odd samples ply in [40,120]
#include <cstdlib>
#include <iostream>
#include <random>

#include "chess/board.h"
#include "chess/position.h"
#include "neural/encoder.h"
#include "oracle/posfile.h"

using namespace lczero;

int main(int argc, char** argv) {
  if (argc < 5) {
    std::cerr << "usage: mkpos <out.pos> <count> <input_format> <uniform|split> [first]\n";
    return 2;
  }
  const std::string out = argv[1];
  const int count = atoi(argv[2]);
  const int fmt = atoi(argv[3]);
  const std::string mix = argv[4];
  const long first = argc > 5 ? atol(argv[5]) : 0;
  InitializeMagicBitboards();
  const auto input_format = static_cast<pblczero::NetworkFormat::InputFormat>(fmt);

  PosFile pf;
  pf.n = count;
  pf.input_format = fmt;
  pf.masks.resize(size_t(count) * 112);
  pf.values.resize(size_t(count) * 112);
  pf.transform.resize(count);
  pf.n_legal.resize(count);
  pf.legal.assign(size_t(count) * 256, -1);

  for (int s = 0; s < count; ++s) {
    std::mt19937_64 rng(42000000ull + uint64_t(first + s));
    int target;
    if (mix == "split") {
      target = ((first + s) % 2 == 0) ? 1 + int(rng() % 20) : 40 + int(rng() % 81);
    } else {
      target = 1 + int(rng() % 60);
    }
    PositionHistory history;
    ChessBoard board(ChessBoard::kStartposFen);
    history.Reset(board, 0, 1);
    for (int ply = 0; ply < target; ++ply) {
      const MoveList moves = history.Last().GetBoard().GenerateLegalMoves();
      if (moves.empty()) break;
      const Move mv = moves[rng() % moves.size()];
      history.Append(mv);
      if (history.ComputeGameResult() != GameResult::UNDECIDED) {
        history.Pop();
        break;
      }
    }
    int transform = 0;
    const InputPlanes planes = EncodePositionForNN(input_format, history, 8,
                                                   FillEmptyHistory::FEN_ONLY, &transform);
    for (int i = 0; i < 112; ++i) {
      pf.masks[size_t(s) * 112 + i] = planes[i].mask;
      pf.values[size_t(s) * 112 + i] = planes[i].value;
    }
    pf.transform[s] = transform;
    const MoveList legal = history.Last().GetBoard().GenerateLegalMoves();
    pf.n_legal[s] = int(legal.size());
    for (size_t i = 0; i < legal.size() && i < 256; ++i)
      pf.legal[size_t(s) * 256 + i] = int16_t(MoveToNNIndex(legal[i], transform));
  }
  WritePosFile(out, pf);
  return 0;
}
