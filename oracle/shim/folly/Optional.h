// Stand-in for folly::Optional / folly::none on top of std::optional, enough for
// the optional padding tuple of the reference's CPU convolution signatures.
// TEST INFRASTRUCTURE ONLY.
#pragma once
#include <optional>

namespace folly {
template <class T>
using Optional = std::optional<T>;
constexpr std::nullopt_t none = std::nullopt;
}  // namespace folly
