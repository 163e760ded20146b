// C-ABI bridge over the reference's own CPU convolutions, compiled together with
// test/ReferenceConvolutions.cpp taken from the reference checkout where it lies.
// TEST INFRASTRUCTURE ONLY: used to validate the fp64 restatement in refconv.c,
// to generate the golden fixtures under tests/golden/, and as the timed CPU
// baseline of the benchmark.  Nothing in the product path may link or load it.
//
// The reference functions are single-threaded (test/ReferenceConvolutions.cpp:85-554).
// `threads > 1` runs the unmodified functions on independent batch slices, one
// slice per thread; for the weight gradient (a reduction over the batch,
// :452-554) the per-slice results are summed afterwards in fp32.
#include "test/ReferenceConvolutions.h"

#include <algorithm>
#include <cstring>
#include <thread>
#include <tuple>
#include <vector>

using facebook::deeplearning::torch::Tensor;
namespace ref = facebook::deeplearning::torch::test;

namespace {

using Pad = folly::Optional<std::tuple<long, long, long, long>>;

Pad makePad(long padH, long padW) {
  if (padH == 0 && padW == 0) return folly::none;
  return std::make_tuple(padH, padH, padW, padW);  // <top, bottom, left, right>
}

Tensor<float> load(const float* src, long a, long b, long c, long d) {
  Tensor<float> t{{a, b, c, d}};
  std::memcpy(t.data(), src, sizeof(float) * t.numel());
  return t;
}

template <class Fn>
void forSlices(long batch, int threads, Fn fn) {
  threads = std::max(1, std::min<int>(threads, static_cast<int>(batch)));
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    const long b0 = batch * t / threads, b1 = batch * (t + 1) / threads;
    pool.emplace_back([=] { if (b1 > b0) fn(t, b0, b1); });
  }
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// updateOutput: crossCorrelationValidOnly (test/ReferenceConvolutions.cpp:85-200).
int ref_update_output(const float* input, const float* weight, float* output,
                      long B, long P, long F, long iH, long iW, long kH, long kW,
                      long padH, long padW, int threads) {
  const long oH = iH + 2 * padH - kH + 1, oW = iW + 2 * padW - kW + 1;
  auto w = load(weight, F, P, kH, kW);
  forSlices(B, threads, [&](int, long b0, long b1) {
    auto in = load(input + b0 * P * iH * iW, b1 - b0, P, iH, iW);
    auto out = ref::crossCorrelationValidOnly(in, w, 1, 1, makePad(padH, padW));
    std::memcpy(output + b0 * F * oH * oW, out.data(), sizeof(float) * out.numel());
  });
  return 0;
}

// updateGradInput: convolutionFull (test/ReferenceConvolutions.cpp:338-450).
int ref_update_grad_input(const float* gradOutput, const float* weight, float* gradInput,
                          long B, long P, long F, long iH, long iW, long kH, long kW,
                          long padH, long padW, int threads) {
  const long oH = iH + 2 * padH - kH + 1, oW = iW + 2 * padW - kW + 1;
  auto w = load(weight, F, P, kH, kW);
  forSlices(B, threads, [&](int, long b0, long b1) {
    auto go = load(gradOutput + b0 * F * oH * oW, b1 - b0, F, oH, oW);
    auto gi = ref::convolutionFull(go, w, 1, 1, makePad(padH, padW));
    std::memcpy(gradInput + b0 * P * iH * iW, gi.data(), sizeof(float) * gi.numel());
  });
  return 0;
}

// accGradParameters (weights): crossCorrelationReverseValidOnly (:452-554).
int ref_acc_grad_weight(const float* input, const float* gradOutput, float* gradWeight,
                        long B, long P, long F, long iH, long iW, long kH, long kW,
                        long padH, long padW, float scale, int threads) {
  const long oH = iH + 2 * padH - kH + 1, oW = iW + 2 * padW - kW + 1;
  threads = std::max(1, std::min<int>(threads, static_cast<int>(B)));
  std::vector<std::vector<float>> partial(threads);
  forSlices(B, threads, [&](int t, long b0, long b1) {
    auto in = load(input + b0 * P * iH * iW, b1 - b0, P, iH, iW);
    auto go = load(gradOutput + b0 * F * oH * oW, b1 - b0, F, oH, oW);
    auto gw = ref::crossCorrelationReverseValidOnly(in, go, 1, 1, scale, makePad(padH, padW));
    partial[t].assign(gw.data(), gw.data() + gw.numel());
  });
  const size_t n = static_cast<size_t>(F) * P * kH * kW;
  std::fill(gradWeight, gradWeight + n, 0.0f);
  for (auto& p : partial)
    for (size_t i = 0; i < p.size() && i < n; ++i) gradWeight[i] += p[i];
  return 0;
}

}  // extern "C"
