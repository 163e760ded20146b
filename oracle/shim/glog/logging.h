// Stand-in for the glog macros named by the reference's CPU convolution file.
// TEST INFRASTRUCTURE ONLY.
#pragma once
#include <cstdlib>
#include <iostream>

namespace oracle_shim {
struct Voidify {
  void operator&(std::ostream&) {}
};
struct Fatal {
  std::ostream& stream() { return std::cerr; }
  ~Fatal() { std::cerr << std::endl; std::abort(); }
};
}  // namespace oracle_shim

#define ORACLE_SHIM_CHECK(cond) \
  (cond) ? (void)0 : oracle_shim::Voidify() & oracle_shim::Fatal().stream() << "Check failed: " #cond " "
#define CHECK(c) ORACLE_SHIM_CHECK(c)
#define CHECK_EQ(a, b) ORACLE_SHIM_CHECK((a) == (b))
#define CHECK_NE(a, b) ORACLE_SHIM_CHECK((a) != (b))
#define CHECK_LE(a, b) ORACLE_SHIM_CHECK((a) <= (b))
#define CHECK_LT(a, b) ORACLE_SHIM_CHECK((a) < (b))
#define CHECK_GE(a, b) ORACLE_SHIM_CHECK((a) >= (b))
#define CHECK_GT(a, b) ORACLE_SHIM_CHECK((a) > (b))
#define DCHECK(c) ORACLE_SHIM_CHECK(c)
#define LOG(x) std::cerr
#define VLOG(x) if (false) std::cerr
