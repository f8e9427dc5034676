// Host-side runtime services private to the library.
#pragma once

#include <cuda.h>

namespace vtp {

// Address of the current device's status word (a __device__ int owned by the library);
// kernels with bounded waits receive it as an argument.  Null if no device is current.
int* device_status_ptr();

// cuTensorMapEncodeTiled resolved through the runtime (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// bf16 tensor map with 128-byte swizzle: dims/strides innermost first; strides in bytes
// for dims 1.. (dim 0 is dense).  Returns 0 or a CUresult.
int make_tmap_bf16(CUtensorMap* map, const void* base, int rank, const unsigned long long* dims,
                   const unsigned long long* strides_bytes, const unsigned* box);

}  // namespace vtp
