/* Token matvec for callers that cannot give the library a scratch buffer.
 *
 * nwc_linear_bf16 keeps its fp32 partial sums in a buffer the caller allocates.  Some hosts cannot do that: an
 * inference server that hands every byte of HBM to its own KV-cache pool when it starts, a plugin sandbox that is
 * denied the CUDA allocator, firmware-style loops that must not touch the allocator once they run.  For them this
 * file carries a fixed scratch area inside the library image itself: every GPU that loads nwc_ops.so holds
 * NWC_STATIC_SCRATCH_FLOATS floats (4 MiB) of it until the process exits.
 *
 * The array's name below is only a host-side handle.  The address the kernels need is looked up once per device with
 * cudaGetSymbolAddress while that device is current, and only that address is ever passed to a launch.
 */
#include <atomic>
#include <mutex>
#include "../../include/nwc_ops.h"
#include "nwc_launch.h"

#define NWC_EXPORT extern "C" __attribute__((visibility("default")))

static __device__ __align__(256) float g_static_scratch[NWC_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<float *> g_scratch_address[kMaxDevices];      /* device address of g_static_scratch on each device, null until looked up */
std::mutex g_lookup_lock;

/* device address of the scratch array on the current device; null (and *err set) when it cannot be had */
float *scratch_on_current_device(int *err) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = e != cudaSuccess ? (int)e : (int)cudaErrorInvalidDevice; return nullptr; }
    if (float *known = g_scratch_address[dev].load(std::memory_order_acquire)) return known;
    std::lock_guard<std::mutex> hold(g_lookup_lock);
    float *known = g_scratch_address[dev].load(std::memory_order_relaxed);
    if (!known) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) { *err = e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol; return nullptr; }
        known = static_cast<float *>(p);
        g_scratch_address[dev].store(known, std::memory_order_release);
    }
    return known;
}
}  // namespace

namespace nwc {
/* Called when a device is prepared (nwc_setup and the first call of any entry point on that device): looks the area's
   address up right away, so that a later nwc_linear_bf16_static - even one made while a stream is being captured - finds
   it cached.  A failure here is not fatal; the entry point reports it when it is used. */
void prepare_static_scratch() { int ignored = 0; scratch_on_current_device(&ignored); }
}  // namespace nwc

NWC_EXPORT int nwc_linear_bf16_static(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                                      const uint8_t *low, const float *x, const uint16_t *bias, const float *scale, uint16_t *y,
                                      uint64_t n, uint32_t block, uint32_t K, int elem) {
    using namespace nwc;
    if (block != kBlockWeights || !K || !n || n % K || n / K > 0xFFFFFFFFull || layout_of(elem) > 2 || type_of(elem) > 1) return -1;
    const uintptr_t misaligned = (uintptr_t)data | (uintptr_t)low | (uintptr_t)lut | (uintptr_t)x;
    if (misaligned & 15u) return -1;
    const Geometry g((uint32_t)(n / K), K, layout_of(elem));
    if (g.scratch_floats() > (uint64_t)NWC_STATIC_SCRATCH_FLOATS) return NWC_ERR_STATIC_SCRATCH;     /* matrix too large for the built-in area */
    const int sms = nwc_setup();
    if (sms <= 0) return (int)cudaErrorNoDevice;
    int err = 0;
    float *scratch = scratch_on_current_device(&err);
    if (!scratch) return err;
    /* nothing in the area has to start at zero: every partial sum the finalize step reads is written by this call first */
    SegmentArgs a{data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, g.M, K, 0, 0, 0};
    return (int)launch_segments(0, elem, sms, (cudaStream_t)stream, a);
}
