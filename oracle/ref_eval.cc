// ref_eval: run one of the reference's own registered backends ("blas",
// "eigen", or any other name linked into this binary) on a weights file and a
// position file through lc0's public plug-in API
// (NetworkFactory::Create -> Network::NewComputation -> AddInput ->
// ComputeBlocking -> GetQVal/GetDVal/GetMVal/GetPVal, neural/network.h:56-126)
// and dump the raw outputs. Test infrastructure / CPU baseline only.
//
// usage: ref_eval <backend> <net.pb[.gz]> <in.pos> <out.bin|-> [opts-string] [repeat] [limit]
//   repeat > 0: time <repeat> evaluations after one warm-up and print
//               "evals_per_s=<v> n=<n> repeat=<r> seconds=<s> p50_ms=<..> p99_ms=<..>" on stdout
//               (per-evaluation wall time: AddInput x n, ComputeBlocking, result reads).
#include <chrono>
#include <cstdlib>
#include <algorithm>
#include <iostream>
#include <limits>

#include "chess/board.h"
#include "neural/factory.h"
#include "neural/loader.h"
#include "oracle/posfile.h"
#include "utils/fastmath.h"
#include "utils/optionsdict.h"

using namespace lczero;

static std::unique_ptr<NetworkComputation> Run(Network* net, const PosFile& pf, int n) {
  auto comp = net->NewComputation();
  for (int s = 0; s < n; ++s) {
    InputPlanes planes(112);
    for (int i = 0; i < 112; ++i) {
      planes[i].mask = pf.masks[size_t(s) * 112 + i];
      planes[i].value = pf.values[size_t(s) * 112 + i];
    }
    comp->AddInput(std::move(planes));
  }
  comp->ComputeBlocking();
  return comp;
}

int main(int argc, char** argv) {
  if (argc < 5) {
    std::cerr << "usage: ref_eval <backend> <net> <in.pos> <out.bin|-> [opts] [repeat] [limit]\n";
    return 2;
  }
  try {
    InitializeMagicBitboards();
    const std::string backend = argv[1];
    const WeightsFile weights = LoadWeightsFromFile(argv[2]);
    const PosFile pf = ReadPosFile(argv[3]);
    const std::string out = argv[4];
    OptionsDict opts;
    if (argc > 5 && argv[5][0]) opts.AddSubdictFromString(argv[5]);
    const int repeat = argc > 6 ? atoi(argv[6]) : 0;
    int n = pf.n;
    if (argc > 7 && atoi(argv[7]) > 0 && atoi(argv[7]) < n) n = atoi(argv[7]);
    auto net = NetworkFactory::Get()->Create(backend, weights, opts);

    auto comp = Run(net.get(), pf, n);
    if (out != "-") {
      FILE* f = fopen(out.c_str(), "wb");
      if (!f) throw std::runtime_error("cannot write " + out);
      const char magic[8] = {'L', 'C', '0', 'O', 'U', 'T', '1', 0};
      fwrite(magic, 1, 8, f);
      int32_t nn = n;
      fwrite(&nn, 4, 1, f);
      std::vector<float> buf(size_t(n) * 1858);
      for (int s = 0; s < n; ++s)
        for (int k = 0; k < 1858; ++k) buf[size_t(s) * 1858 + k] = comp->GetPVal(s, k);
      fwrite(buf.data(), 4, buf.size(), f);
      std::vector<float> v(n);
      for (int s = 0; s < n; ++s) v[s] = comp->GetQVal(s);
      fwrite(v.data(), 4, n, f);
      for (int s = 0; s < n; ++s) v[s] = comp->GetDVal(s);
      fwrite(v.data(), 4, n, f);
      for (int s = 0; s < n; ++s) v[s] = comp->GetMVal(s);
      fwrite(v.data(), 4, n, f);
      // Legal-move softmax at temperature 1 with the reference's own FastExp, in the order and arithmetic of
      // NetworkAsBackendComputation::SoftmaxPolicy (neural/wrapper.cc:135-156); float probs[n][256].
      std::vector<float> probs(size_t(n) * 256, 0.0f);
      for (int s = 0; s < n; ++s) {
        const int cnt = std::min(pf.n_legal[s], 256);
        float* dst = &probs[size_t(s) * 256];
        float max_p = -std::numeric_limits<float>::infinity();
        for (int i = 0; i < cnt; ++i) max_p = std::max(max_p, dst[i] = comp->GetPVal(s, pf.legal[size_t(s) * 256 + i]));
        float total = 0.0f;
        for (int i = 0; i < cnt; ++i) total = total + (dst[i] = FastExp((dst[i] - max_p) * 1.0f));
        const float scale = total > 0.0f ? 1.0f / total : 1.0f;
        for (int i = 0; i < cnt; ++i) dst[i] *= scale;
      }
      fwrite(probs.data(), 4, probs.size(), f);
      fclose(f);
    }
    if (repeat > 0) {
      std::vector<double> each;
      const auto t0 = std::chrono::steady_clock::now();
      auto prev = t0;
      for (int r = 0; r < repeat; ++r) {
        Run(net.get(), pf, n);
        const auto now = std::chrono::steady_clock::now();
        each.push_back(std::chrono::duration<double, std::milli>(now - prev).count());
        prev = now;
      }
      const double sec = std::chrono::duration<double>(prev - t0).count();
      std::sort(each.begin(), each.end());
      const double p50 = each[each.size() / 2];
      const double p99 = each[std::min(each.size() - 1, size_t(each.size() * 0.99))];
      std::cout << "evals_per_s=" << double(n) * repeat / sec << " n=" << n
                << " repeat=" << repeat << " seconds=" << sec << " p50_ms=" << p50 << " p99_ms=" << p99 << std::endl;
    }
  } catch (const std::exception& e) {
    std::cerr << "ref_eval error: " << e.what() << std::endl;
    return 1;
  }
  return 0;
}
