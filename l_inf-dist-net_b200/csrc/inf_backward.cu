// inf-dist backward: scatter of grad_output through the saved arg-max.
//
//   grad_input [b, g*CIg + idx, hw] += s * g      s = +1 if pos >= 0 else -1
//   grad_weight[o, idx]             -= s * g      g = grad_output[b, o, hw], idx = pos & 0x7fffffff
//
// Ordered kernels (the default): one warp owns one destination ROW -- a (b, group, hw) row of
// grad_input or an output-channel row of grad_weight -- keeps that row's bins in shared
// memory, walks the row's contributions 32 at a time in ascending source order, and lets the
// lowest lane of every set of lanes that hit the same bin add that set's values one by one in
// lane order.  Every bin therefore sees its contributions as sequential fp32 adds in ascending
// source order starting from +0: a fixed, reproducible order.  The finished row is written out
// whole, so the destination needs no zero fill.
//
// Atomic kernel: one pass over (grad_output, pos) produces both gradients with fp32 atomics;
// for grad_weight a 32 x 32 tile is transposed through shared memory so that the lanes of a
// warp run over the batch for one output channel, equal bins are combined inside the warp and
// one atomic is issued per distinct bin.
#include "common.cuh"

namespace linf {
namespace {

constexpr unsigned FULL = 0xffffffffu;

// Adds the values of all lanes that share a bin into that bin, in lane order.
__device__ __forceinline__ void ordered_warp_add(float* bins, bool active, int idx, float val, int lane) {
    const unsigned act = __ballot_sync(FULL, active);
    if (act == 0) return;
    unsigned grp = 0;
    if (active) grp = __match_any_sync(act, idx);
    const bool leader = active && ((grp & ((1u << lane) - 1u)) == 0);
    const int cnt = __popc(grp);
    const int maxcnt = __reduce_max_sync(FULL, cnt);
    if (maxcnt == 1) {
        if (active) bins[idx] += val;
    } else {
        float acc = leader ? bins[idx] : 0.f;
        unsigned rem = grp;
        for (int it = 0; it < maxcnt; ++it) {
            const int src = rem ? (__ffs(rem) - 1) : lane;
            const float v = __shfl_sync(FULL, val, src);
            if (leader && rem) acc += v;
            rem &= rem - 1;
        }
        if (leader) bins[idx] = acc;
    }
    __syncwarp();
}

// mode 0: rows of grad_input  -- row = (r, g), sources o = 0..COg-1
// mode 1: rows of grad_weight -- row = (g, o), sources r = 0..R-1
template <int MODE>
__global__ void __launch_bounds__(256)
inf_backward_ordered_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                            float* __restrict__ dst, int warps_per_cta, int n_rows) {
    extern __shared__ __align__(16) float bins_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * warps_per_cta + warp;
    if (row >= n_rows) return;
    float* bins = bins_all + (size_t)warp * d.CIg;
    for (int i = lane; i < d.CIg; i += 32) bins[i] = 0.f;
    __syncwarp();

    int r = 0, g = 0, o = 0, n_src;
    if (MODE == 0) { r = row / d.G; g = row - r * d.G; n_src = d.COg; }
    else { g = row / d.COg; o = row - g * d.COg; n_src = d.R; }

    // source element e -> offset in [B, CO, HW]
    auto src_off = [&](int e) -> size_t {
        return MODE == 0 ? act_index(r, g, e, d.COg, d.G, d.HW) : act_index(e, g, o, d.COg, d.G, d.HW);
    };
    int e = lane;
    bool act = e < n_src;
    int pv = 0; float gv = 0.f;
    if (act) { size_t a = src_off(e); pv = __ldg(pos + a); gv = __ldg(gout + a); }
    for (int base = 0; base < n_src; base += 32) {
        // prefetch the next 32 sources before the dependent bin update of this batch
        const int e2 = base + 32 + lane;
        const bool act2 = e2 < n_src;
        int pv2 = 0; float gv2 = 0.f;
        if (act2) { size_t a = src_off(e2); pv2 = __ldg(pos + a); gv2 = __ldg(gout + a); }

        const int idx = pv & 0x7fffffff;
        float val = (pv >= 0) ? gv : -gv;
        if (MODE == 1) val = -val;
        // an index outside the group (corrupt pos) is dropped rather than written out of bounds
        ordered_warp_add(bins, act && idx < d.CIg, idx, val, lane);

        act = act2; pv = pv2; gv = gv2;
    }
    __syncwarp();
    if (MODE == 0) {
        for (int i = lane; i < d.CIg; i += 32) dst[act_index(r, g, i, d.CIg, d.G, d.HW)] = bins[i];
    } else {
        float* out = dst + (size_t)(g * d.COg + o) * d.CIg;
        for (int i = lane; i < d.CIg; i += 32) out[i] = bins[i];
    }
}

// Both gradients with atomics; tile = 32 rows (r) x 32 output channels of one group.
template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
inf_backward_atomic_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                           float* __restrict__ gx, float* __restrict__ gw) {
    __shared__ int ps[32][33];
    __shared__ float gs[32][33];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = blockIdx.z, r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;

    for (int e = tid; e < 1024; e += 256) {
        int rl, cl;
        if (ROW_FAST) { rl = e & 31; cl = e >> 5; } else { cl = e & 31; rl = e >> 5; }
        const int r = r0 + rl, c = c0 + cl;
        int pv = 0; float gv = 0.f;
        if (r < d.R && c < d.COg) {
            size_t a = act_index(r, g, c, d.COg, d.G, d.HW);
            pv = __ldg(pos + a); gv = __ldg(gout + a);
            const int idx = pv & 0x7fffffff;
            if (gx != nullptr && idx < d.CIg)
                atomicAdd(gx + act_index(r, g, idx, d.CIg, d.G, d.HW), pv >= 0 ? gv : -gv);
        } else {
            pv = -1;   // idx = 0x7fffffff: never a valid bin
        }
        ps[rl][cl] = pv; gs[rl][cl] = gv;
    }
    if (gw == nullptr) return;
    __syncthreads();
    // warp `wid` handles output channels wid, wid+8, ...; lane = row of the tile
    for (int cl = wid; cl < 32; cl += 8) {
        const int c = c0 + cl;
        if (c >= d.COg) break;
        const int pv = ps[lane][cl];
        const float gv = gs[lane][cl];
        const int idx = pv & 0x7fffffff;
        const bool active = idx < d.CIg;
        const float val = (pv < 0) ? gv : -gv;
        const unsigned act = __ballot_sync(FULL, active);
        if (act == 0) continue;
        unsigned grp = 0;
        if (active) grp = __match_any_sync(act, idx);
        const bool leader = active && ((grp & ((1u << lane) - 1u)) == 0);
        const int maxcnt = __reduce_max_sync(FULL, __popc(grp));
        float acc = 0.f;
        unsigned rem = grp;
        for (int it = 0; it < maxcnt; ++it) {
            const int src = rem ? (__ffs(rem) - 1) : lane;
            const float v = __shfl_sync(FULL, val, src);
            if (leader && rem) acc += v;
            rem &= rem - 1;
        }
        if (leader) atomicAdd(gw + (size_t)(g * d.COg + c) * d.CIg + idx, acc);
    }
}

constexpr size_t BIN_SMEM_LIMIT = 200 * 1024;

template <int MODE>
int launch_ordered(const float* g, const int* pos, const Dims& d, float* dst, cudaStream_t st) {
    const size_t row_bytes = (size_t)d.CIg * sizeof(float);
    if (row_bytes > BIN_SMEM_LIMIT) return LINF_ERR_TOO_LARGE;
    const int n_rows = (MODE == 0) ? d.R * d.G : d.CO;
    int wpc = (int)(BIN_SMEM_LIMIT / row_bytes);
    if (wpc > 8) wpc = 8;
    // spread the rows over the SMs before stacking warps into one CTA
    const int sms = sm_count();
    while (wpc > 1 && (n_rows + wpc - 1) / wpc < sms) wpc >>= 1;
    const size_t smem = row_bytes * wpc;
    auto kern = inf_backward_ordered_kernel<MODE>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BIN_SMEM_LIMIT) !=
            cudaSuccess)
            return LINF_ERR_LAUNCH;
    }
    const int grid = (n_rows + wpc - 1) / wpc;
    kern<<<grid, wpc * 32, smem, st>>>(g, pos, d, dst, wpc, n_rows);
    return launch_status();
}

}  // namespace

int inf_backward_input(const float* g, const int* pos, const Dims& d, float* gx, cudaStream_t st) {
    return launch_ordered<0>(g, pos, d, gx, st);
}

int inf_backward_weight(const float* g, const int* pos, const Dims& d, float* gw, cudaStream_t st) {
    return launch_ordered<1>(g, pos, d, gw, st);
}

int inf_backward_atomic(const float* g, const int* pos, const Dims& d, float* gx, float* gw,
                        cudaStream_t st) {
    dim3 grid((d.R + 31) / 32, (d.COg + 31) / 32, d.G);
    if (grid.y > 65535u || grid.z > 65535u) return LINF_ERR_DIMS;
    if (d.HW > 1) inf_backward_atomic_kernel<true><<<grid, 256, 0, st>>>(g, pos, d, gx, gw);
    else inf_backward_atomic_kernel<false><<<grid, 256, 0, st>>>(g, pos, d, gx, gw);
    return launch_status();
}

}  // namespace linf
