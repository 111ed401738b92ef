// Architecture predicates with the names the reference offers to callers
// (reference include/ccglib/common/arch.h:8-93: isCDNA1..4, isRDNA4, isCDNA, isVolta, isAda,
// isHopper, isBlackwell, hasFP8, hasFP4, isUnsupported); its tests use them to skip cases a GPU
// cannot run (test/gemm/mma.cpp:530-591).  They classify the architecture string of a
// cu::Device ("sm_100", "gfx942", ...).  This library itself runs on sm_100 only: every other
// architecture, NVIDIA or AMD, is reported as unsupported.
#pragma once

#include <initializer_list>
#include <string>

#include <cudawrappers/cu.hpp>

namespace ccglib {

namespace detail {
inline bool arch_matches(const std::string &arch, std::initializer_list<const char *> prefixes) {
  for (const char *prefix : prefixes) {
    if (arch.find(prefix) != std::string::npos) return true;
  }
  return false;
}
inline std::string arch_of(cu::Device &device) { return std::string(device.getArch()); }
} // namespace detail

static inline bool isCDNA1(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx908"});
}
static inline bool isCDNA2(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx90a"});
}
static inline bool isCDNA3(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx94"});
}
static inline bool isCDNA4(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx95"});
}
static inline bool isRDNA4(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx12"});
}
static inline bool isCDNA(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"gfx908", "gfx90a", "gfx94", "gfx95"});
}
static inline bool isVolta(cu::Device &device) {
  return detail::arch_matches(detail::arch_of(device), {"sm_70"});
}
static inline bool isAda(const std::string &arch) { return detail::arch_matches(arch, {"sm_89"}); }
static inline bool isHopper(const std::string &arch) {
  return detail::arch_matches(arch, {"sm_90"});
}
static inline bool isBlackwell(const std::string &arch) {
  return detail::arch_matches(arch, {"sm_100", "sm_101", "sm_120"});
}
static inline bool hasFP8(cu::Device &device) {
  const std::string arch = detail::arch_of(device);
  return isBlackwell(arch) || isHopper(arch) || isAda(arch) ||
         detail::arch_matches(arch, {"gfx12", "gfx94"});
}
static inline bool hasFP4(cu::Device &device) {
  const std::string arch = detail::arch_of(device);
  return isBlackwell(arch) || isHopper(arch) || isAda(arch);
}
// The kernels of this library are tcgen05 code for sm_100 and nothing else.
static inline bool isUnsupported(cu::Device &device) {
  return !detail::arch_matches(detail::arch_of(device), {"sm_100"});
}

} // namespace ccglib
