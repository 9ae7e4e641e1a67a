// linf_inf_dist_forward_noalloc: the split-k inf-dist forward for callers that may not allocate.
//
// Some hosts of this library run under a fixed device-memory plan: a framework that owns all
// device memory through its own pool and forbids its plug-ins to call the CUDA allocator, or a
// deployment that sizes its memory once at start-up and treats any later cudaMalloc as an error.
// Such a caller cannot produce the scratch buffer that linf_inf_dist_forward_ws asks for.  For
// them the scratch lives inside the library image: one fixed, 256-byte aligned device array per
// GPU that has loaded the library (it stays resident until the process exits).
//
// The array below is declared with `static __device__`.  In host code its name only stands for
// the symbol -- it is not a device address and must never be handed to a kernel.  The real
// address comes from cudaGetSymbolAddress, asked once per device with that device current, and
// it is that pointer which travels to the kernel as its workspace argument.
#include <mutex>

#include "common.cuh"

namespace {

// 30 MiB: the parked partial tiles of 3 CTAs per SM on up to 152 SMs (29.9 MB) plus the tile
// tickets of any layer whose tensors fit the int32 element limit of the library.
constexpr size_t kScratchBytes = (size_t)LINF_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_forward_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of g_forward_scratch on the CURRENT device (looked up on first use).
int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return LINF_ERR_LAUNCH;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_forward_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return LINF_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return LINF_OK;
}

}  // namespace

extern "C" int linf_inf_dist_forward_noalloc(const float* input, const float* weight,
                                             int B, int CO, int CI, int G, int HW,
                                             float* output, int* pos, void* stream) {
    if (!input || !weight || !output || !pos) return LINF_ERR_NULL;
    linf::Dims d;
    int rc = linf::make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    const size_t need = linf::inf_forward_workspace(d);
    if (need > kScratchBytes) return LINF_ERR_TOO_LARGE;      // layer (or GPU) too large for the fixed array
    void* scratch = nullptr;
    if (need != 0) {
        rc = scratch_for_current_device(&scratch);
        if (rc) return rc;
    }
    // same launcher as linf_inf_dist_forward_ws; it zeroes the tile tickets it needs on `stream`
    // and ignores whatever else the previous call left in the array
    return linf::inf_forward(input, weight, d, output, pos, scratch, need ? kScratchBytes : 0,
                             reinterpret_cast<cudaStream_t>(stream));
}
