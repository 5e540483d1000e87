// Compiled against the reference's own src/runtime/device_probe.h (never together with sca_b200.h: both headers
// define ScaDeviceProbe, on purpose, so that src/runtime/capability.cpp links against libsca_b200.so unchanged).
// The numbers asserted here are asserted again for this repository's struct in ref_launch_bindings.cpp; equal
// numbers in both translation units mean equal layouts.
#include <cstddef>

#include "runtime/device_probe.h"

static_assert(sizeof(ScaDeviceProbe) == 352, "reference probe struct size");
static_assert(offsetof(ScaDeviceProbe, major) == 256 && offsetof(ScaDeviceProbe, smem_per_sm) == 272 &&
                  offsetof(ScaDeviceProbe, free_mem_bytes) == 328 && offsetof(ScaDeviceProbe, cuda_available) == 336 &&
                  offsetof(ScaDeviceProbe, binary_has_sm90) == 344,
              "reference probe struct offsets");

// Referenced so that the link of the host library fails if the C ABI stops exporting the reference's probe symbols.
extern "C" int sca_dropin_probe_symbols_present() {
    return (reinterpret_cast<void*>(&sca_probe_device) != nullptr && reinterpret_cast<void*>(&sca_mem_get_info) != nullptr) ? 1 : 0;
}
