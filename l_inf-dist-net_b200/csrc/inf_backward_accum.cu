// Ordered grad_weight of the inf-dist backward for dense layers (HW == 1) without a sort.
//
// One warp owns an output-channel row of grad_weight, keeps the whole row (CIg floats, all +0 at
// the start) in shared memory, and walks the row's sources -- the batch rows r = 0..R-1 -- 32 at
// a time in ascending order.  Lanes of one batch that hit the same bin are found with match_any;
// the lowest of them adds the bin's old value and then the lanes' values, one by one in lane
// order, and writes the bin back.  Every bin therefore sees exactly the sequential fp32 adds
// from +0 in ascending source order that the sort-based kernels (inf_backward.cu) produce, but
// the histogram, the scan over all bins and the per-bin loops of the sort are gone: what is left
// per row is 16 batches (R = 512) plus zeroing and copying the row.  The finished row is written
// out whole, so the destination needs no zero fill.
//
// The sources of a row lie CO floats apart.  The CTA therefore first copies a block of sources
// of its (up to 8) neighbouring rows into shared memory, 8 consecutive threads reading 8
// consecutive channels, so that every 32-byte sector of grad_output / pos is fetched once.
//
// grad_input keeps the sort: its rows are few (R) and long (COg sources), one warp per row is
// latency bound (measured 64 us at R = 512, COg = 5120, against 28 us for the sort), and sharing
// a row between warps by bin ownership multiplies the scan of the sources by the warp count.
#include "common.cuh"

namespace linf {
namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr int SB_MAX = 512;      // sources per staged block (template parameter SB: 512 or 256); a row's staged block
                                 // has a pitch of SB + 4 words: neighbouring rows land 4 banks apart, so the staging
                                 // stores of a warp (8 rows x 4 sources) touch 32 different banks

// One batch of up to 32 sources, one per lane: bin `idx` (idx >= nb = no source / dropped) and
// signed value `v`.
struct Batch {
    int idx; float v;
    unsigned grp;       // lanes with the same bin as this one (0 = no source here)
    unsigned dup;       // lanes that are not the lowest of their bin (same for the whole warp)
};

// match_any costs one pass per DISTINCT value among the lanes; rows of grad_weight have few (one
// bin usually takes most of a row's sources).  One vote per bit of the bin index -- a cost
// independent of the data -- measured slower on such rows (43 us against 35 us at B = 512,
// Din = 784, Dout = 5120).
__device__ __forceinline__ Batch classify(int idx, float v, int nb, int lane) {
    Batch b;
    b.idx = idx; b.v = v; b.grp = 0;
    const bool active = idx < nb;
    const unsigned act = __ballot_sync(FULL, active);
    if (active) b.grp = __match_any_sync(act, idx);
    b.dup = __ballot_sync(FULL, (b.grp & ((1u << lane) - 1u)) != 0);
    return b;
}

// `staged_v`: the 32 signed values of this batch in shared memory (16-byte aligned).
__device__ __forceinline__ void add_batch(float* __restrict__ acc, const Batch& b, int lane,
                                          const float* __restrict__ staged_v) {
    const bool active = b.grp != 0;
    const bool leader = active && (b.grp & ((1u << lane) - 1u)) == 0;
    float a = active ? acc[b.idx] + b.v : 0.f;       // only the leader's sum is kept
    if (b.dup != 0) {
        if (__popc(b.dup) > 8) {
            // many lanes share bins: every leader reads the batch's 32 signed values from shared
            // memory, 4 at a time, and adds those of its own group -- a fixed cost, where one
            // shuffle per duplicate lane would not be
            const unsigned rest = b.grp & ~(1u << lane);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 w4 = *reinterpret_cast<const float4*>(staged_v + 4 * q);
                if ((rest >> (4 * q + 0)) & 1u) a += w4.x;
                if ((rest >> (4 * q + 1)) & 1u) a += w4.y;
                if ((rest >> (4 * q + 2)) & 1u) a += w4.z;
                if ((rest >> (4 * q + 3)) & 1u) a += w4.w;
            }
        } else {
            unsigned todo = b.dup;
            while (todo) {
                const int l = __ffs(todo) - 1;
                todo &= todo - 1;
                const float vl = __shfl_sync(FULL, b.v, l);
                if ((b.grp >> l) & 1u) a += vl;
            }
        }
    }
    if (leader) acc[b.idx] = a;
    __syncwarp();
}

// COMPACT (rows much longer than their number of sources, all sources in one staged block): the
// warp does not keep the whole row but one accumulator per bin that OCCURS -- a bitmap of the
// row's bins, its running popcount, and dense accumulators addressed through them -- and expands
// to the full row (zeros elsewhere) when it writes it out.  Shared memory per row drops from
// 4 * CIg bytes to CIg / 4 + 4 * sources, which keeps 24 warps per SM at CIg = 5120.
template <bool COMPACT, int SB>
__global__ void __launch_bounds__(SB == 512 ? 256 : 640)
inf_backward_weight_accum_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                                 float* __restrict__ dst, int nbp, int vec_out) {
    constexpr int SBP = SB + 4;
    extern __shared__ __align__(16) float smem_f[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rpc = blockDim.x >> 5;
    const int n_rows = d.CO, n_src = d.R, nb = d.CIg;
    const int row0 = blockIdx.x * rpc, row = row0 + warp;    // row = g * COg + o
    // per-row area: the row itself, or (COMPACT) bitmap words | running popcounts | SB dense accumulators
    const int nbw = (nb + 31) >> 5;
    const int row_words = COMPACT ? 2 * ((nbw + 3) & ~3) + SB : nbp;
    float* acc = smem_f + (size_t)warp * row_words;
    unsigned* bits = reinterpret_cast<unsigned*>(acc);                 // COMPACT only
    int* before = reinterpret_cast<int*>(acc) + ((nbw + 3) & ~3);      // COMPACT only
    if (COMPACT) {
        for (int i = lane; i < nbw; i += 32) bits[i] = 0u;
        acc += 2 * ((nbw + 3) & ~3);
        for (int i = lane; i < SB; i += 32) acc[i] = 0.f;
    } else {
        for (int i = lane * 4; i < nbp; i += 128) *reinterpret_cast<float4*>(acc + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncwarp();

    // staging area behind the rows: [rpc][SBP] pos words, [rpc][SBP] signed values
    int* spos = reinterpret_cast<int*>(smem_f + (size_t)rpc * row_words);
    float* sval = reinterpret_cast<float*>(spos + (size_t)rpc * SBP);
    int occupied = 0;                                                  // COMPACT: bins of this row that occur
    const int sj = threadIdx.x % rpc, se = threadIdx.x / rpc;          // staging: this thread's row and first source
    const size_t srow = (size_t)min(row0 + sj, n_rows - 1);
    for (int s0 = 0; s0 < n_src; s0 += SB) {
        const int cnt = min(SB, n_src - s0);
        constexpr int SU = 8;                             // loads in flight per thread
        // element q = e * rpc + j of the block (source e of row j) goes to thread q mod blockDim; blockDim is
        // 32 * rpc, so a thread keeps its row j = sj and meets the sources se, se + 32, se + 64, ...
        for (int eb = se; eb < cnt; eb += 32 * SU) {
            int pp[SU]; float pg[SU];
#pragma unroll
            for (int u = 0; u < SU; ++u) {
                const int e = eb + 32 * u;
                pp[u] = -1; pg[u] = 0.f;
                if (e < cnt) {
                    // source r of row (g, o): element (r * G + g) * COg + o = r * CO + row
                    const size_t a = (size_t)(s0 + e) * d.CO + srow;
                    pp[u] = __ldg(pos + a); pg[u] = __ldg(gout + a);
                }
            }
#pragma unroll
            for (int u = 0; u < SU; ++u) {
                const int e = eb + 32 * u;
                if (e < cnt) {
                    spos[sj * SBP + e] = pp[u];
                    sval[sj * SBP + e] = (pp[u] >= 0) ? -pg[u] : pg[u];    // grad_weight takes -s * g
                }
            }
        }
        __syncthreads();
        if (row < n_rows) {
            const int* mp = spos + warp * SBP;
            const float* mv = sval + warp * SBP;
            if (COMPACT) {
                // which bins occur, and how many occurring bins lie before each 32-bin word
                for (int e = lane; e < cnt; e += 32) {
                    const int idx = mp[e] & 0x7fffffff;
                    if (idx < nb && mv[e] != 0.f) atomicOr(&bits[idx >> 5], 1u << (idx & 31));
                }
                __syncwarp();
                int run = 0;
                for (int w0 = 0; w0 < nbw; w0 += 32) {
                    const int c = (w0 + lane < nbw) ? __popc(bits[w0 + lane]) : 0;
                    int incl = c;
#pragma unroll
                    for (int sh = 1; sh < 32; sh <<= 1) {
                        const int up = __shfl_up_sync(FULL, incl, sh);
                        if (lane >= sh) incl += up;
                    }
                    if (w0 + lane < nbw) before[w0 + lane] = run + incl - c;
                    run += __shfl_sync(FULL, incl, 31);
                }
                occupied = run;
                __syncwarp();
            }
            // groups of 4 batches: the grouping of all four is issued before the first is added
            for (int b0 = 0; b0 * 32 < cnt; b0 += 4) {
                Batch bt[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int e = (b0 + u) * 32 + lane;
                    const float val = e < cnt ? mv[e] : 0.f;
                    // a source whose value is +-0 changes no sum (the accumulators start at +0 and can never become -0):
                    // it is dropped, which is most sources of most rows in a training step
                    int idx = (e < cnt && val != 0.f) ? (mp[e] & 0x7fffffff) : 0x7fffffff;
                    if (COMPACT) {
                        // dense number of the bin among the occurring ones (equal bins, equal numbers)
                        idx = idx < nb ? before[idx >> 5] + __popc(bits[idx >> 5] & ((1u << (idx & 31)) - 1u)) : 0x7fffffff;
                    }
                    bt[u] = classify(idx, val, COMPACT ? SB : nb, lane);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if ((b0 + u) * 32 < cnt) add_batch(acc, bt[u], lane, mv + (b0 + u) * 32);
            }
        }
        __syncthreads();
    }
    if (row >= n_rows) return;
    float* out = dst + (size_t)row * nb;
    if (COMPACT) {
        __syncwarp();
        if (vec_out && occupied <= 64) {
            // few bins occur (the usual case in training: the sources of a row agree on their arg-max position):
            // four bins per lane and store, nearly all of them zero (53 against 57 us at B = 512, Din = Dout = 5120;
            // with hundreds of occurring bins the word-by-word loop below is the faster one, 63 against 69 us)
            for (int i = lane * 4; i < nb; i += 128) {
                const unsigned word = bits[i >> 5];
                const unsigned nib = (word >> (i & 31)) & 0xfu;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (nib) {
                    int at = before[i >> 5] + __popc(word & ((1u << (i & 31)) - 1u));
                    if (nib & 1u) v.x = acc[at++];
                    if (nib & 2u) v.y = acc[at++];
                    if (nib & 4u) v.z = acc[at++];
                    if (nib & 8u) v.w = acc[at];
                }
                *reinterpret_cast<float4*>(out + i) = v;
            }
            return;
        }
        for (int i0 = 0; i0 < nb; i0 += 32) {
            const unsigned word = bits[i0 >> 5];
            const int i = i0 + lane;
            const float v = ((word >> lane) & 1u) ? acc[before[i0 >> 5] + __popc(word & ((1u << lane) - 1u))] : 0.f;
            if (i < nb) out[i] = v;
        }
        return;
    }
    if (vec_out) {
        for (int i = lane * 4; i < nb; i += 128)
            *reinterpret_cast<float4*>(out + i) = *reinterpret_cast<const float4*>(acc + i);
    } else {
        for (int i = lane; i < nb; i += 32) out[i] = acc[i];
    }
}

}  // namespace

// Returns -1 when the shape is not one this kernel takes (the caller falls back to the sort).
int inf_backward_weight_accum(const float* g, const int* pos, const Dims& d, float* gw, cudaStream_t st) {
    if (d.HW != 1) return -1;
    const int nbp = (d.CIg + 3) & ~3;
    const size_t limit = 200 * 1024;
    // long rows with few sources, and enough rows for occupancy to matter: accumulators only for
    // the bins that occur (measured at R = 512, CO = 5120: 61 us vs 76 us at CIg = 5120, but
    // 59 us vs 50 us at CIg = 3072 and 23 us vs 16 us for the 10 rows of a classifier layer)
    const bool compact = d.CIg >= 4096 && d.R <= SB_MAX && d.CO >= 1024;
    const int nbw4 = (((d.CIg + 31) >> 5) + 3) & ~3;
    if (!compact) {
        // Short rows: when the rows one SM has to produce (CO / SMs) fit its shared memory at once, they are
        // dealt to two CTAs per SM with one warp per row and half-size staging blocks, so that the whole
        // launch is ONE wave of CTAs with all of an SM's rows in flight together (at B = 512, Din = 784,
        // Dout = 5120: 285 CTAs of 18 warps on 296 slots, instead of 640 CTAs of 8 warps on 444 slots).
        constexpr int SBS = 256;
        const int sms = sm_count();
        const int rows_per_sm = (d.CO + sms - 1) / sms;
        const int rpc_w = (rows_per_sm + 1) / 2;
        const size_t per_row_w = (size_t)nbp * 4 + (size_t)(SBS + 4) * 8;
        if (rpc_w >= 4 && rpc_w <= 20 && 2 * rpc_w * per_row_w <= 220 * 1024 && d.CO >= 4 * sms) {
            const size_t smem_w = (size_t)rpc_w * per_row_w;
            auto kern_w = inf_backward_weight_accum_kernel<false, SBS>;
            if (cudaFuncSetAttribute(kern_w, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit) != cudaSuccess)
                return LINF_ERR_LAUNCH;
            const int vec = ((d.CIg & 3) == 0 && (reinterpret_cast<uintptr_t>(gw) & 15u) == 0) ? 1 : 0;
            kern_w<<<(d.CO + rpc_w - 1) / rpc_w, 32 * rpc_w, smem_w, st>>>(g, pos, d, gw, nbp, vec);
            return launch_status();
        }
    }
    constexpr int SBP = SB_MAX + 4;
    const size_t per_row = (compact ? (size_t)(2 * nbw4 + SB_MAX) * 4 : (size_t)nbp * 4) + (size_t)SBP * 8;
    if (per_row > limit) return -1;
    // Rows per CTA.  Neighbouring rows share the sectors of the strided sources: 8 rows use every
    // sector whole, but two CTAs per SM (one staging while the other adds) are worth more.
    int rpc = 8;
    while (rpc > 1 && (size_t)rpc * per_row > limit) rpc >>= 1;
    while (rpc > 2 && (size_t)rpc * per_row > 100 * 1024) rpc >>= 1;
    const size_t smem = (size_t)rpc * per_row;
    auto kern = compact ? inf_backward_weight_accum_kernel<true, SB_MAX> : inf_backward_weight_accum_kernel<false, SB_MAX>;
    if (smem > 40 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    const int vec_out = ((d.CIg & 3) == 0 && (reinterpret_cast<uintptr_t>(gw) & 15u) == 0) ? 1 : 0;
    const int grid = (d.CO + rpc - 1) / rpc;
    kern<<<grid, 32 * rpc, smem, st>>>(g, pos, d, gw, nbp, vec_out);
    return launch_status();
}

}  // namespace linf
