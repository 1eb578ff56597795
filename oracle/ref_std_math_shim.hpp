// Test infrastructure only (checker / CPU baseline), never part of the product path.
//
// libstdc++ 13 does not declare the float-suffixed C math functions inside
// namespace std, but the reference header include/kernels_cpu.hpp calls
// std::expf, std::sqrtf, std::powf, std::cosf, std::sinf and std::tanhf
// (lines 87-91, 130, 152, 182-186). This force-included shim makes those
// names visible so the header compiles unmodified.
#pragma once
#include <cmath>
namespace std {
using ::cosf;
using ::expf;
using ::powf;
using ::sinf;
using ::sqrtf;
using ::tanhf;
}  // namespace std
