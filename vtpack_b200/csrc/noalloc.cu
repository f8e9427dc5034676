// Gate + patch-list compaction for callers that cannot give the library any scratch memory.
//
// vtp_router_gate followed by vtp_index_to_patch needs two small intermediates (the grain
// index of every region and the query count of every image) that the caller normally
// allocates.  Some hosts have no way to do that: a plugin that is handed only its input
// and output buffers by an inference server, a host runtime in another language that can
// pass device pointers through its FFI but owns no CUDA allocator, or a latency-critical
// loop that must not call cudaMalloc because it synchronises the device.  For them the
// intermediates live in a fixed array inside the library's device image.
#include "region_ops.h"

namespace vtp {

constexpr int kStaticMaxRegions = 65536;   // B * (H/region) * (W/region)
constexpr int kStaticMaxImages = 4096;     // B
constexpr size_t kStaticBytes = (size_t)(kStaticMaxRegions + kStaticMaxImages) * sizeof(int32_t);

// 278,528 bytes of device memory per GPU that loads the library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the
// address kernels can use comes from cudaGetSymbolAddress, once per device, with that device
// current.
static int static_scratch(int32_t** idx, int32_t** counts) {
    static unsigned char* cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail((int)e, "gate_compact_static: no current device: %s", cudaGetErrorString(e));
    VTP_REQUIRE(dev >= 0 && dev < 64, VTP_ERR_SHAPE, "gate_compact_static: device ordinal %d out of range", dev);
    if (!cached[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(e != cudaSuccess ? (int)e : VTP_ERR_DRIVER,
                        "gate_compact_static: cannot resolve the static scratch array: %s", cudaGetErrorString(e));
        }
        cached[dev] = static_cast<unsigned char*>(p);
    }
    *idx = reinterpret_cast<int32_t*>(cached[dev]);
    *counts = reinterpret_cast<int32_t*>(cached[dev] + (size_t)kStaticMaxRegions * sizeof(int32_t));
    return VTP_OK;
}

}  // namespace vtp

using namespace vtp;

extern "C" int vtp_gate_compact_static(const void* x, int dtype, int B, int H, int W, int C, int num_extra,
                                       int region, const float* gate_w, const float* gate_b, const int* splits,
                                       int n_splits, int32_t* offsets, int32_t* patches, void* stream) {
    // Every argument check of the two calls below is repeated here, in front of the first launch, so that a
    // rejected call has launched nothing and has not touched the shared array.
    VTP_REQUIRE(x && gate_w && gate_b && splits && offsets && patches, VTP_ERR_NULL,
                "gate_compact_static: null pointer");
    VTP_REQUIRE(dtype == VTP_F32 || dtype == VTP_BF16, VTP_ERR_DTYPE, "gate_compact_static: dtype %d", dtype);
    VTP_REQUIRE(B > 0 && H > 0 && W > 0 && region > 0 && H % region == 0 && W % region == 0, VTP_ERR_SHAPE,
                "gate_compact_static: grid %dx%d not divisible by region %d", H, W, region);
    VTP_REQUIRE(num_extra >= 0, VTP_ERR_SHAPE, "gate_compact_static: num_extra %d", num_extra);
    VTP_REQUIRE(C > 0 && C % (16 / (int)elem_size(dtype)) == 0 && C % 4 == 0, VTP_ERR_SHAPE,
                "gate_compact_static: C=%d must be a multiple of 16 bytes", C);
    const long long regions = (long long)B * (H / region) * (W / region);
    VTP_REQUIRE(B <= kStaticMaxImages && regions <= kStaticMaxRegions, VTP_ERR_SHAPE,
                "gate_compact_static: %d images / %lld regions exceed the static scratch (at most %d images and %d "
                "regions); use vtp_router_gate + vtp_index_to_patch with caller-provided buffers",
                B, regions, kStaticMaxImages, kStaticMaxRegions);
    VTP_REQUIRE((H / region) * (W / region) <= 8192, VTP_ERR_SHAPE, "gate_compact_static: %d regions per image (at most 8192)",
                (H / region) * (W / region));
    Splits sp;
    if (int rc = make_splits(&sp, splits, n_splits, region)) return rc;
    VTP_REQUIRE(aligned16(x) && aligned16(gate_w) && aligned16(patches), VTP_ERR_ALIGN,
                "gate_compact_static: unaligned pointer");
    int32_t *idx = nullptr, *counts = nullptr;
    if (int rc = static_scratch(&idx, &counts)) return rc;
    // Nothing in the scratch has to start at zero: every entry read below is written first.
    if (int rc = vtp_router_gate(x, dtype, B, H, W, C, num_extra, region, gate_w, gate_b, n_splits, nullptr, idx,
                                 stream))
        return rc;
    return vtp_index_to_patch(idx, 0, splits, n_splits, B, H / region, W / region, region, num_extra, counts, offsets,
                              patches, nullptr, stream);
}
