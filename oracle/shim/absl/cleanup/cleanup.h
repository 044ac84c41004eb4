// Scope-guard stand-in for absl::Cleanup (the only abseil facility the chess
// rules code needs).
#pragma once
#include <utility>
namespace absl {
template <typename F>
class Cleanup {
 public:
  Cleanup(F f) : f_(std::move(f)) {}
  Cleanup(const Cleanup&) = delete;
  ~Cleanup() { f_(); }
 private:
  F f_;
};
template <typename F> Cleanup(F) -> Cleanup<F>;
}  // namespace absl
