// Position-file and result-file formats shared by the oracle tools.
// Test infrastructure only (never linked into the product library).
//
// Position file (little endian):
//   char magic[8] = "LC0POS1\0"; int32 n; int32 input_format;
//   uint64 masks[n][112]; float values[n][112]; int32 transform[n];
//   int32 n_legal[n]; int16 legal[n][256]  (policy indices of the legal moves, -1 padded)
// Result file:
//   char magic[8] = "LC0OUT1\0"; int32 n;
//   float policy[n][1858]; float q[n]; float d[n]; float m[n];
//   float legal_probs[n][256]  (legal-move softmax at temperature 1, zero padded)
#pragma once
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

struct PosFile {
  int32_t n = 0, input_format = 0;
  std::vector<uint64_t> masks;    // n*112
  std::vector<float> values;      // n*112
  std::vector<int32_t> transform, n_legal;
  std::vector<int16_t> legal;     // n*256
};

inline void WritePosFile(const std::string& path, const PosFile& p) {
  FILE* f = fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("cannot write " + path);
  const char magic[8] = {'L', 'C', '0', 'P', 'O', 'S', '1', 0};
  fwrite(magic, 1, 8, f);
  fwrite(&p.n, 4, 1, f);
  fwrite(&p.input_format, 4, 1, f);
  fwrite(p.masks.data(), 8, p.masks.size(), f);
  fwrite(p.values.data(), 4, p.values.size(), f);
  fwrite(p.transform.data(), 4, p.transform.size(), f);
  fwrite(p.n_legal.data(), 4, p.n_legal.size(), f);
  fwrite(p.legal.data(), 2, p.legal.size(), f);
  fclose(f);
}

inline PosFile ReadPosFile(const std::string& path) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("cannot read " + path);
  char magic[8];
  PosFile p;
  if (fread(magic, 1, 8, f) != 8 || std::string(magic, 7) != "LC0POS1")
    throw std::runtime_error("bad position file " + path);
  if (fread(&p.n, 4, 1, f) != 1 || fread(&p.input_format, 4, 1, f) != 1)
    throw std::runtime_error("truncated position file");
  const size_t n = p.n;
  p.masks.resize(n * 112);
  p.values.resize(n * 112);
  p.transform.resize(n);
  p.n_legal.resize(n);
  p.legal.resize(n * 256);
  bool ok = fread(p.masks.data(), 8, n * 112, f) == n * 112 &&
            fread(p.values.data(), 4, n * 112, f) == n * 112 &&
            fread(p.transform.data(), 4, n, f) == n &&
            fread(p.n_legal.data(), 4, n, f) == n &&
            fread(p.legal.data(), 2, n * 256, f) == n * 256;
  fclose(f);
  if (!ok) throw std::runtime_error("truncated position file");
  return p;
}
