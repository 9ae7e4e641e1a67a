// Shared declarations of the distance-neuron kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include <atomic>

#include "../../include/linfdist.h"

namespace linf {

// Problem sizes of one call.  R = B*HW is the number of "rows" (one per batch element and
// spatial position); per group the work is an R x COg x CIg reduction over CIg.
struct Dims {
    int B, CO, CI, G, HW;
    int COg, CIg;   // per-group channel counts
    int R;          // B * HW
};

// Validates sizes; fills d.  Every product that is later used as an element count has to
// fit in int32 (the tensors of a layer are far below that).
inline int make_dims(int B, int CO, int CI, int G, int HW, Dims* d) {
    if (B <= 0 || CO <= 0 || CI <= 0 || G <= 0 || HW <= 0) return LINF_ERR_DIMS;
    if (CI % G != 0 || CO % G != 0) return LINF_ERR_GROUP;
    const long long lim = 0x7fffffffLL;
    if ((long long)B * HW > lim || (long long)B * HW * CO > lim ||
        (long long)B * HW * CI > lim || (long long)CO * (CI / G) > lim)
        return LINF_ERR_DIMS;
    d->B = B; d->CO = CO; d->CI = CI; d->G = G; d->HW = HW;
    d->COg = CO / G; d->CIg = CI / G; d->R = B * HW;
    return LINF_OK;
}

// Kernel launches of this library in this process (linf_launch_count): every launcher ends in launch_status.
extern std::atomic<unsigned long long> g_launches;

inline int launch_status(int launched = 1) {
    g_launches.fetch_add((unsigned long long)launched, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? LINF_OK : LINF_ERR_LAUNCH;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device id; read-only after first use).
// Device ids beyond the table (kMaxDevices) are asked from the runtime on every call.
constexpr int kMaxDevices = 64;
int sm_count();

// The library owns one helper stream per device for work that runs beside the caller's stream
// (the second kernel of the ordered backward).  A
// SideLease holds the per-device lock from construction to destruction, so that the
// record / wait pairs of one fork ... join sequence are never interleaved with those of another
// host thread; kernels of several leases simply queue behind each other on the helper stream.
class SideLease {
public:
    SideLease();
    ~SideLease();
    SideLease(const SideLease&) = delete;
    SideLease& operator=(const SideLease&) = delete;
    bool ok() const { return side_ != nullptr; }
    cudaStream_t stream() const;
    // helper stream waits for everything queued on `from` so far
    int fork(cudaStream_t from);
    // `into` waits for everything queued on the helper stream so far
    int join(cudaStream_t into);
private:
    void* side_;
};

// ---- element addressing ------------------------------------------------------------
// row r = b*HW + hw of group g, channel c of that group, in a [B, C, HW] tensor whose
// per-group channel count is Cg.
__device__ __forceinline__ size_t act_index(int r, int g, int c, int Cg, int G, int HW) {
    int b = r / HW, hw = r - b * HW;
    return ((size_t)(b * G + g) * Cg + c) * HW + hw;
}

// ---- Blackwell packed / 3-input fp32 instructions ------------------------------------
// Two IEEE round-to-nearest fp32 subtractions in one instruction (no flush-to-zero).
__device__ __forceinline__ unsigned long long sub_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// max(a, b, c) in one instruction; a NaN operand is ignored (same rule as fmaxf).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- cp.async (16-byte, L2-only caching) ----------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// ---- optional per-output-channel epilogue of the forward and bound kernels -------------------
//   v' = (v - sub[c]) + add[c]      either vector may be null: that step is skipped
//   v' = -v'                        if negate; the bound kernels then also exchange lower and upper
// c is the output channel (0 .. CO-1).  This is what follows an inf-dist layer in eval mode -- the
// mean shift by the running mean, the bias, the sign flip of the classifier layer -- applied in the
// same two fp32 operations and the same order as the separate elementwise passes it replaces.
struct Post {
    const float* sub; const float* add; int negate;
};
__device__ __forceinline__ float post_apply(const Post& q, float v, int c) {
    if (q.sub != nullptr) v = v - __ldg(q.sub + c);
    if (q.add != nullptr) v = v + __ldg(q.add + c);
    return q.negate ? -v : v;
}
inline Post no_post() { return Post{nullptr, nullptr, 0}; }

// ---- launchers implemented in the .cu files -----------------------------------------
int inf_forward(const float* x, const float* w, const Dims& d, float* y, int* pos,
                void* ws, size_t ws_bytes, cudaStream_t st, const Post& post = Post{nullptr, nullptr, 0});
size_t inf_forward_workspace(const Dims& d);
int inf_bound(const float* xl, const float* xu, const float* w, const Dims& d,
              float* yl, float* yu, cudaStream_t st, const Post& post = Post{nullptr, nullptr, 0});
// batch-mean shift of a [rows, cols] activation (epilogue.cu)
// sparse_exchange.cu: row lists of a sparse gradient, merged across ranks over peer memory
int grad_rows_compact(float* grad, int rows, int cols, int cap, int* cnt, void* ent, int* err, cudaStream_t st);
int flag_publish(int* flag, int value, cudaStream_t st);
int flags_wait(const int* const* flags, int n, int value, int timeout_ms, int* err, cudaStream_t st);
int grad_rows_merge(float* grad, int rows, int cols, int cap, const int* const* cnts, const void* const* ents,
                    int world, float scale, const int* err, cudaStream_t st);
int mean_shift(const float* in, int rows, int cols, float* running_mean, float momentum, float* out,
               float* mean_out, cudaStream_t st);
int inf_backward_input(const float* g, const int* pos, const Dims& d, float* gx, cudaStream_t st);
int inf_backward_weight(const float* g, const int* pos, const Dims& d, float* gw, cudaStream_t st);
int inf_backward_atomic(const float* g, const int* pos, const Dims& d, float* gx, float* gw,
                        cudaStream_t st);
// sort-free ordered grad_weight for dense layers (inf_backward_accum.cu); -1 = shape not taken
int inf_backward_weight_accum(const float* g, const int* pos, const Dims& d, float* gw, cudaStream_t st);
// direct accumulation in shared memory for dense layers (inf_backward_direct.cu); -1 = shape not taken
// The verdict of the grad_input probe (inf_backward_direct.cu): one word per probed row.
constexpr int kGxProbeRows = 8;
__device__ __forceinline__ bool probe_says_contested(const int* __restrict__ words) {
    int any = 0;
#pragma unroll
    for (int k = 0; k < kGxProbeRows; ++k) any |= words[k];
    return any != 0;
}
int inf_backward_input_direct(const float* g, const int* pos, const Dims& d, float* gx, cudaStream_t st,
                              const int** decided_by = nullptr);
extern int inf_backward_path;
int inf_backward_ordered_both(const float* g, const int* pos, const Dims& d, float* gx, float* gw,
                              cudaStream_t st);
// few output channels per group (skinny.cu)
bool skinny_ok(const Dims& d, const void* a, const void* b, const void* c);
int inf_forward_skinny(const float* x, const float* w, const Dims& d, float* y, int* pos, cudaStream_t st,
                       const Post& post);
int inf_bound_skinny(const float* xl, const float* xu, const float* w, const Dims& d, float* yl, float* yu,
                     cudaStream_t st, const Post& post);
// register-tiled finite-p kernels for dense, aligned layers (lp_tiled.cu)
bool lp_tiled_ok(const Dims& d, const void* a, const void* b, const void* c, const void* e, const void* f);
int lp_forward_tiled(const float* x, const float* w, const Dims& d, float* y, float p, cudaStream_t st);
int lp_backward_tiled(const float* g, const float* x, const float* w, const float* y, const Dims& d,
                      float* out, float p, bool wrt_weight, cudaStream_t st);
int lp_forward(const float* x, const float* w, const Dims& d, float* y, float p, cudaStream_t st);
int lp_backward_input(const float* g, const float* x, const float* w, const float* y,
                      const Dims& d, float* gx, float p, cudaStream_t st);
int lp_backward_weight(const float* g, const float* x, const float* w, const float* y,
                       const Dims& d, float* gw, float p, cudaStream_t st);

}  // namespace linf
