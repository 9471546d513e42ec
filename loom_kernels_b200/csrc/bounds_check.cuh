// The checked build (-DLB_DEBUG_BOUNDS=1, `python loom_kernels_b200/build.py --debug-bounds`): every
// index a kernel computes into one of its global operands is compared with the length of that
// operand before the access.  An index outside its operand is never dereferenced: the check
// records 0x1000 | site in the kernel's status word (read through the provider's device-status
// call) and the access is skipped -- nothing traps, nothing faults.  The GPU suites run against
// this build in tests/test_gpu_debug_bounds.py and must leave the status word at zero; it stands in
// for the memory checker of a sanitizer where none can be run.  In the product build the check
// is the constant `true` and costs nothing.
#pragma once

#include <cstdint>

namespace lb {
namespace dev {

#ifdef LB_DEBUG_BOUNDS
constexpr bool kCheckBounds = true;
#else
constexpr bool kCheckBounds = false;
#endif

// Sites (the low bits of the recorded word).
enum BoundsSite : int {
    kSiteIndptr = 1,
    kSiteLast,
    kSiteIndices,
    kSiteQuery,
    kSiteOutput,
    kSiteLse,
    kSiteWorkspace,
    kSitePage,
    kSiteDestRows,
    kSiteAppendToken,
    kSiteAppendPool,
    kSiteAppendWorkspace,
};

// true when [index, index + count) lies inside [0, bound)
__device__ __forceinline__ bool in_bounds(long long index, long long bound, int32_t *status,
                                          int site, long long count = 1) {
    if (!kCheckBounds) return true;
    if (count == 0) return true; // nothing is accessed
    if (index >= 0 && count > 0 && index + count <= bound) return true;
    if (status != nullptr) atomicExch(status, 0x1000 | site);
    return false;
}

} // namespace dev
} // namespace lb
