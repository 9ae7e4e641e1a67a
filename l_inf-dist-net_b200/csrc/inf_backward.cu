// inf-dist backward: scatter of grad_output through the saved arg-max.
//
//   grad_input [b, g*CIg + idx, hw] += s * g      s = +1 if pos >= 0 else -1
//   grad_weight[o, idx]             -= s * g      g = grad_output[b, o, hw], idx = pos & 0x7fffffff
//
// Ordered kernels (the default): every destination ROW -- a (b, group, hw) row of grad_input or
// an output-channel row of grad_weight -- is produced by one group of threads as a stable
// counting sort followed by per-bin sequential sums, all in shared memory:
//   1. histogram of the row's bin indices;
//   2. exclusive scan -> first slot of every bin;
//   3. placement of every (signed) gradient value into the next free slot of its bin, in
//      ascending source order;
//   4. one thread per bin adds the bin's values one by one, in slot (= source) order, from +0,
//      and the finished row is written out whole (no zero fill of the destination needed).
// Every bin therefore sees sequential fp32 adds in ascending source order: a fixed,
// reproducible order, and one of the orders the reference's atomicAdd scatter can produce.
// Implementations: inf_backward_rows_kernel keeps the row's sources in registers (grad_input rows
// of up to 12288 sources); inf_backward_ordered_kernel is the general one (any row length, sparse
// rows through a bitmap of occurring bins, conv-shaped tensors).  Dense grad_weight rows do not
// sort at all: inf_backward_accum.cu.
//
// Atomic kernel: one pass over (grad_output, pos) produces both gradients with fp32 atomics;
// for grad_weight a 32 x 32 tile is transposed through shared memory so that the lanes of a
// warp run over the batch for one output channel, equal bins are combined inside the warp and
// one atomic is issued per distinct bin.
#include "common.cuh"

namespace linf {

int inf_backward_path = 0;   // benchmarking knob: 0 = grad_input by the direct or the sort kernel as a probe of the positions decides;
                             // 1 = never the direct kernel; 2 = the direct kernel wherever it fits, no probe

namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Shared-memory footprint (in 4-byte words) of one row group.
__host__ __device__ inline int group_words(int W, int nb, int n_src, bool compact, bool staged, bool aplace) {
    const int nbw = (nb + 31) / 32;
    const int DM = compact ? min(nb, n_src) : nb;
    return (compact ? (2 * nbw + 1 + DM) : 0) + W * DM + (DM + 1) + 8 + n_src + (staged ? 2 * n_src : 0) +
           (aplace ? (n_src + 1) / 2 : 0);
}

// In-place exclusive scan of arr[0..n) by a group of GS threads (one warp, or the whole CTA);
// the total lands in arr[n].  Every thread of the group must call it.
template <bool CTA_ROW>
__device__ __forceinline__ void group_exclusive_scan(int* arr, int n, int gt, int GS, int lane, int gwp,
                                                     int* wsum) {
    const int blk = (n + GS - 1) / GS;
    const int b0 = min(n, gt * blk), b1 = min(n, b0 + blk);
    int local = 0;
    for (int i = b0; i < b1; ++i) local += arr[i];
    int incl = local;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        int t = __shfl_up_sync(FULL, incl, s);
        if (lane >= s) incl += t;
    }
    if (CTA_ROW) {
        if (lane == 31) wsum[gwp] = incl;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < gwp; ++w) before += wsum[w];
        incl += before;
    }
    int run = incl - local;
    for (int i = b0; i < b1; ++i) { int t = arr[i]; arr[i] = run; run += t; }
    if (gt == GS - 1) arr[n] = run;
    if (CTA_ROW) __syncthreads(); else __syncwarp();
}

// mode 0: rows of grad_input  -- row = (r, g), sources o = 0..COg-1
// mode 1: rows of grad_weight -- row = (g, o), sources r = 0..R-1
// CTA_ROW = true : the whole CTA (blockDim.x / 32 warps) works on one row
// CTA_ROW = false: every warp of the CTA works on a row of its own
// COMPACT        : dense bin ids through a bitmap (rows with fewer sources than bins)
// STAGED         : (warp-per-row only) the CTA first copies the sources of all its rows into
//                  shared memory with sector-friendly loads; the passes then read from there
// APLACE         : slots inside a bin are handed out by a shared-memory atomic instead of
//                  match_any (which costs one pass per DISTINCT bin of the 32 lanes); the source
//                  index travels with the value and step 4 restores ascending source order with
//                  an insertion sort that only has to untangle lanes of one 32-source batch
template <int MODE, bool CTA_ROW, bool COMPACT, bool STAGED, bool APLACE>
__global__ void __launch_bounds__(256)
inf_backward_ordered_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                            float* __restrict__ dst, int n_rows, int n_src) {
    extern __shared__ __align__(16) int smem_i[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int GS = CTA_ROW ? blockDim.x : 32;            // threads in the row's group
    const int W = GS >> 5;                               // warps in the group
    const int gt = CTA_ROW ? threadIdx.x : lane;         // thread index inside the group
    const int gwp = CTA_ROW ? warp : 0;                  // warp index inside the group
    const int rpc = CTA_ROW ? 1 : (blockDim.x >> 5);     // rows per CTA
    const int row0 = blockIdx.x * rpc;
    const int row = row0 + (CTA_ROW ? 0 : warp);
    const int nb = d.CIg;                                // bins per row
    const int nbw = (nb + 31) / 32;
    const int DM = COMPACT ? min(nb, n_src) : nb;        // most distinct bins a row can have
    const int gwords = group_words(W, nb, n_src, COMPACT, STAGED, APLACE);
    int* base = smem_i + (CTA_ROW ? 0 : (size_t)warp * gwords);
    int* bitmap = base;                                  // [nbw]      (COMPACT)
    int* wp = bitmap + (COMPACT ? nbw : 0);              // [nbw + 1]  (COMPACT) bins before each word
    int* keys = wp + (COMPACT ? nbw + 1 : 0);            // [DM]       (COMPACT) bin of a dense id
    int* hist = keys + (COMPACT ? DM : 0);               // [W][DM]
    int* seg = hist + W * DM;                            // [DM + 1]
    int* wsum = seg + DM + 1;                            // [8]
    float* sorted = reinterpret_cast<float*>(wsum + 8);  // [n_src]
    int* st_pos = reinterpret_cast<int*>(sorted + n_src);            // [n_src] (STAGED)
    float* st_g = reinterpret_cast<float*>(st_pos + n_src);          // [n_src] (STAGED)
    unsigned short* skey = reinterpret_cast<unsigned short*>(sorted + n_src + (STAGED ? 2 * n_src : 0));  // [n_src] (APLACE)
    const int HW = d.HW;

    // Element offsets without divisions inside the loops.  Source e of this row sits at
    // s_base + e * s_step (+ a correction when a row of grad_weight walks over (b, hw) pairs
    // with HW > 1, handled in src_off); bin i of the destination at d_base + i * d_step.
    size_t s_base, d_base; int s_step, d_step;
    int g = 0, o = 0;
    if (MODE == 0) {
        const int r = row / d.G; g = row - r * d.G;
        const int b = r / HW, hw = r - b * HW;
        s_base = ((size_t)(b * d.G + g) * d.COg) * HW + hw; s_step = HW;
        d_base = ((size_t)(b * d.G + g) * d.CIg) * HW + hw; d_step = HW;
    } else {
        g = row / d.COg; o = row - g * d.COg;
        s_base = (size_t)(g * d.COg + o) * HW; s_step = d.CO * HW;      // exact for HW == 1
        d_base = (size_t)(g * d.COg + o) * d.CIg; d_step = 1;
    }
    auto src_off = [&](int e) -> size_t {
        if (MODE == 0 || HW == 1) return s_base + (size_t)e * s_step;
        const int b = e / HW, hw = e - b * HW;                            // conv-shaped grad_weight rows
        return s_base + (size_t)b * s_step + hw;
    };

    if (STAGED) {
        // all threads of the CTA copy the sources of its rpc neighbouring rows: consecutive threads
        // read consecutive rows (channels) of one source, i.e. whole 32-byte sectors when HW == 1
        const int total = rpc * n_src;
        for (int q = threadIdx.x; q < total; q += blockDim.x) {
            const int j = q % rpc, e = q / rpc;
            if (row0 + j < n_rows) {
                const int rowj = row0 + j;                                // rows of a CTA may straddle groups
                const int gj = rowj / d.COg, ojj = rowj - gj * d.COg;
                size_t a;
                if (HW == 1) a = (size_t)e * d.CO + (size_t)gj * d.COg + ojj;
                else { const int b = e / HW, hw = e - b * HW; a = ((size_t)(b * d.G + gj) * d.COg + ojj) * HW + hw; }
                int* sp = smem_i + (size_t)j * gwords + (gwords - 2 * n_src - (APLACE ? (n_src + 1) / 2 : 0));
                sp[e] = __ldg(pos + a);
                reinterpret_cast<float*>(sp + n_src)[e] = __ldg(gout + a);
            }
        }
        __syncthreads();
    }
    if (row >= n_rows) return;                           // whole warps only, and only when !CTA_ROW

    auto sync = [&]() { if (CTA_ROW) __syncthreads(); else __syncwarp(); };
    auto get_pos = [&](int e) -> int { return STAGED ? st_pos[e] : __ldg(pos + src_off(e)); };
    auto get_g = [&](int e) -> float { return STAGED ? st_g[e] : __ldg(gout + src_off(e)); };
    auto dense = [&](int idx) -> int {
        if (!COMPACT) return idx;
        return wp[idx >> 5] + __popc((unsigned)bitmap[idx >> 5] & ((1u << (idx & 31)) - 1u));
    };
    // contiguous share of the sources for this warp, a multiple of 32 long
    const int per_warp = ((n_src + W - 1) / W + 31) & ~31;
    const int e_begin = gwp * per_warp, e_end = min(n_src, e_begin + per_warp);
    constexpr int U = 4;                                 // 32-source batches fetched together

    int D = nb;
    if (COMPACT) {
        // ---- 0. which bins occur; zero-fill the destination row ----
        for (int i = gt; i < nbw; i += GS) bitmap[i] = 0;
        if (d_step == 1 && (nb & 3) == 0 && ((d_base & 3) == 0) && aligned16_dev(dst)) {
            float4* row4 = reinterpret_cast<float4*>(dst + d_base);
            for (int i = gt; i < (nb >> 2); i += GS) row4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int i = gt; i < nb; i += GS) dst[d_base + (size_t)i * d_step] = 0.f;
        }
        sync();
        for (int eb = e_begin; eb < e_end; eb += 32 * U) {
            int pv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) { int e = eb + 32 * u + lane; pv[u] = e < e_end ? get_pos(e) : -1; }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = pv[u] & 0x7fffffff;
                if (idx < nb) atomicOr(&bitmap[idx >> 5], 1 << (idx & 31));
            }
        }
        sync();
        for (int i = gt; i < nbw; i += GS) wp[i] = __popc((unsigned)bitmap[i]);
        sync();
        group_exclusive_scan<CTA_ROW>(wp, nbw, gt, GS, lane, gwp, wsum);
        D = wp[nbw];
    }
    // ---- 1. histogram of dense ids, per warp of the group ----
    for (int w = 0; w < W; ++w)
        for (int i = gt; i < D; i += GS) hist[w * DM + i] = 0;
    sync();
    for (int eb = e_begin; eb < e_end; eb += 32 * U) {
        int pv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { int e = eb + 32 * u + lane; pv[u] = e < e_end ? get_pos(e) : -1; }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = pv[u] & 0x7fffffff;
            if (idx < nb) {                                          // an index outside the group is dropped
                const int did = dense(idx);
                atomicAdd(&hist[gwp * DM + did], 1);
                if (COMPACT) keys[did] = idx;
            }
        }
    }
    sync();
    // ---- 2. scans: offsets of the warps inside each bin, then first slot of each bin ----
    for (int i = gt; i < D; i += GS) {
        int run = 0;
        for (int w = 0; w < W; ++w) { int t = hist[w * DM + i]; hist[w * DM + i] = run; run += t; }
        seg[i] = run;
    }
    sync();
    group_exclusive_scan<CTA_ROW>(seg, D, gt, GS, lane, gwp, wsum);
    for (int w = 0; w < W; ++w)
        for (int i = gt; i < D; i += GS) hist[w * DM + i] += seg[i];
    sync();
    // ---- 3. stable placement ----
    for (int eb = e_begin; eb < e_end; eb += 32 * U) {
        int pv[U]; float gv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            int e = eb + 32 * u + lane;
            pv[u] = -1; gv[u] = 0.f;
            if (e < e_end) { pv[u] = get_pos(e); gv[u] = get_g(e); }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = pv[u] & 0x7fffffff;
            float val = (pv[u] >= 0) ? gv[u] : -gv[u];
            if (MODE == 1) val = -val;
            const bool active = idx < nb;
            const unsigned act = __ballot_sync(FULL, active);
            if (act == 0) continue;
            if (APLACE) {
                if (active) {
                    const int slot = atomicAdd(&hist[gwp * DM + dense(idx)], 1);
                    sorted[slot] = val;
                    skey[slot] = (unsigned short)(eb + 32 * u + lane);
                }
                continue;
            }
            // lanes with the same bin get consecutive slots in lane order.  The shuffle uses the
            // warp-wide mask on purpose: a per-group mask would be executed once per group.
            int did = 0, rank = 0, leader = lane, cur = 0;
            if (active) {
                did = dense(idx);
                const unsigned grp = __match_any_sync(act, did);
                rank = __popc(grp & ((1u << lane) - 1u));
                leader = __ffs(grp) - 1;
                if (rank == 0) { cur = hist[gwp * DM + did]; hist[gwp * DM + did] = cur + __popc(grp); }
            }
            cur = __shfl_sync(FULL, cur, leader);
            if (active) sorted[cur + rank] = val;
            __syncwarp();
        }
    }
    sync();
    // ---- 4. per-bin sequential sums ----
    for (int i = gt; i < D; i += GS) {
        float acc = 0.f;
        const int s0 = seg[i], s1 = seg[i + 1];
        if (APLACE) {
            // slots of one batch may be permuted among lanes: restore ascending source order
            for (int j = s0 + 1; j < s1; ++j) {
                const unsigned short k = skey[j];
                if (skey[j - 1] > k) {
                    const float v = sorted[j];
                    int q = j - 1;
                    while (q >= s0 && skey[q] > k) { skey[q + 1] = skey[q]; sorted[q + 1] = sorted[q]; --q; }
                    skey[q + 1] = k; sorted[q + 1] = v;
                }
            }
        }
        for (int j = s0; j < s1; ++j) acc += sorted[j];
        dst[d_base + (size_t)(COMPACT ? keys[i] : i) * d_step] = acc;
    }
}

// --------------------------------------------------------------------------------------------
// Fast ordered path for grad_input rows: same four steps, but every thread keeps its share of the
// row's sources (EPT of them) in registers from the first load to the placement, slots inside a
// bin come from one shared-memory atomic per source, and step 4 restores ascending source order
// with an insertion sort on the source indices that travel with the values (only sources that
// were in flight at the same time can be out of order, so the sort is close to a no-op).
// One CTA of 16 warps per row, sources read straight from global memory.
// --------------------------------------------------------------------------------------------
// C = number of copies of the count array: warps of different copies place in parallel
__host__ __device__ inline int fast_copies(int nb) {
    int c = 1;
    while (c < 8 && (2 * c - 1) * (nb + 1) * 4 <= 16 * 1024) c <<= 1;
    return c;
}
__host__ __device__ inline int fast_group_words(int nb, int n_src) {
    return (fast_copies(nb) + 1) * (nb + 1) + 32 + n_src + (n_src + 1) / 2;
}

template <int MODE, int EPT>
__global__ void __launch_bounds__(512)
inf_backward_rows_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                         float* __restrict__ dst, int n_rows, int n_src, const int* __restrict__ only_if) {
    if (only_if != nullptr && !probe_says_contested(only_if)) return;     // the direct-accumulation kernel did these rows
    extern __shared__ __align__(16) int smem_i[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int GS = blockDim.x, gt = threadIdx.x;
    const int row = blockIdx.x;
    const int nb = d.CIg, HW = d.HW;
    const int C = fast_copies(nb);                       // copies of the count / cursor array
    const int WPC = max(1, (int)(blockDim.x >> 5) / C);  // warps that share a copy
    int* hist = smem_i;                                  // [C][nb + 1] counts, then cursors
    int* seg = hist + C * (nb + 1);                      // [nb + 1] first slot of every bin
    int* myhist = hist + (warp / WPC) * (nb + 1);
    int* wsum = smem_i + (C + 1) * (nb + 1);             // [32]: warp sums of the scan; [24] = work-list length
    float* sorted = reinterpret_cast<float*>(wsum + 32); // [n_src]
    unsigned short* skey = reinterpret_cast<unsigned short*>(sorted + n_src);   // [n_src] source index of a slot

    int pv[EPT]; float gv[EPT];
    {
        size_t s_base; int s_step;
        if (MODE == 0) {
            const int r = row / d.G, g = row - r * d.G, b = r / HW, hw = r - b * HW;
            s_base = ((size_t)(b * d.G + g) * d.COg) * HW + hw; s_step = HW;
        } else {
            const int g = row / d.COg, o = row - g * d.COg;
            s_base = (size_t)(g * d.COg + o) * HW; s_step = d.CO * HW;
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int e = (warp * EPT + j) * 32 + lane;  // warp w owns sources [w*EPT*32, (w+1)*EPT*32)
            pv[j] = -1; gv[j] = 0.f;
            if (e < n_src) {
                size_t a;
                if (MODE == 0 || HW == 1) a = s_base + (size_t)e * s_step;
                else { const int b = e / HW, hw = e - b * HW; a = s_base + (size_t)b * s_step + hw; }
                pv[j] = __ldg(pos + a); gv[j] = __ldg(gout + a);
            }
        }
    }

    size_t d_base; int d_step;
    if (MODE == 0) {
        const int r = row / d.G, g = row - r * d.G, b = r / HW, hw = r - b * HW;
        d_base = ((size_t)(b * d.G + g) * d.CIg) * HW + hw; d_step = HW;
    } else {
        d_base = (size_t)row * d.CIg; d_step = 1;
    }

    // ---- 1. histogram ----
    for (int i = gt; i < C * (nb + 1); i += GS) hist[i] = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        // a source that adds +-0 changes no sum (every bin starts at +0 and can never become -0): it is dropped
        // here and at the placement, like an index outside the group
        if (gv[j] == 0.f) pv[j] = 0x7fffffff;
        const int idx = pv[j] & 0x7fffffff;
        if (idx < nb) atomicAdd(&myhist[idx], 1);
    }
    __syncthreads();
    // ---- 2. first slot of every bin (and of every copy's share of the bin) ----
    if (C > 1) {
        for (int i = gt; i < nb; i += GS) {
            int run = 0;
            for (int c = 0; c < C; ++c) { const int t = hist[c * (nb + 1) + i]; hist[c * (nb + 1) + i] = run; run += t; }
            seg[i] = run;
        }
        __syncthreads();
        group_exclusive_scan<true>(seg, nb, gt, GS, lane, warp, wsum);
        for (int c = 0; c < C; ++c)
            for (int i = gt; i < nb; i += GS) hist[c * (nb + 1) + i] += seg[i];
    } else {
        group_exclusive_scan<true>(hist, nb, gt, GS, lane, warp, wsum);
        for (int i = gt; i <= nb; i += GS) seg[i] = hist[i];
    }
    __syncthreads();
    // ---- 3. placement: value and source index into the next free slot of the bin ----
    // The warps own ascending source ranges.  Warps that share a copy of the cursor array take
    // their slots one warp after the other, each warp in ascending batches; warps of different
    // copies own disjoint slot ranges of a bin and run in parallel.  A bin then fills in
    // ascending source order provided the lanes of one atomic instruction are served in lane
    // order.  That last point is hardware behaviour, not a guarantee, so the source index
    // travels along and step 4 checks it.
    for (int w = 0; w < WPC; ++w) {
        if (warp % WPC == w) {
            int slot[EPT];
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int idx = pv[j] & 0x7fffffff;
                slot[j] = idx < nb ? atomicAdd(&myhist[idx], 1) : -1;
            }
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (slot[j] >= 0) {
                    float val = (pv[j] >= 0) ? gv[j] : -gv[j];
                    if (MODE == 1) val = -val;
                    sorted[slot[j]] = val;
                    skey[slot[j]] = (unsigned short)((warp * EPT + j) * 32 + lane);
                }
            }
        }
        __syncthreads();
    }
    // ---- 4. per bin: ascending source order, then sequential fp32 adds from +0 ----
    // First pass: one thread per bin adds in slot order while checking that the source indices
    // ascend; a bin that fails the check goes on a work list (kept in the cursor array, which
    // is dead now).  Second pass: the listed bins are sorted by source index and added again.
    if (gt == 0) wsum[24] = 0;
    __syncthreads();
    for (int i = gt; i < nb; i += GS) {
        const int s0 = seg[i], s1 = seg[i + 1];
        float acc = 0.f;
        bool ordered = true;
        int prev = -1, j = s0;
        for (; j + 2 <= s1; j += 2) {
            const int k0 = skey[j], k1 = skey[j + 1];
            const float v0 = sorted[j], v1 = sorted[j + 1];
            ordered = ordered && (k0 > prev) && (k1 > k0);
            prev = k1;
            acc += v0; acc += v1;
        }
        if (j < s1) { ordered = ordered && ((int)skey[j] > prev); acc += sorted[j]; }
        if (ordered) dst[d_base + (size_t)i * d_step] = acc;
        else hist[atomicAdd(&wsum[24], 1)] = i;
    }
    __syncthreads();
    const int n_list = wsum[24];
    for (int q = gt; q < n_list; q += GS) {
        const int i = hist[q];
        const int s0 = seg[i], s1 = seg[i + 1];
        for (int a = s0 + 1; a < s1; ++a) {
            const unsigned short k = skey[a];
            const float v = sorted[a];
            int b2 = a - 1;
            while (b2 >= s0 && skey[b2] > k) { skey[b2 + 1] = skey[b2]; sorted[b2 + 1] = sorted[b2]; --b2; }
            skey[b2 + 1] = k; sorted[b2 + 1] = v;
        }
        float acc = 0.f;
        for (int a = s0; a < s1; ++a) acc += sorted[a];
        dst[d_base + (size_t)i * d_step] = acc;
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

constexpr size_t SMEM_LIMIT = 200 * 1024;

template <int MODE, bool CTA_ROW, bool COMPACT, bool STAGED, bool APLACE>
int launch_ordered_as(const float* g, const int* pos, const Dims& d, float* dst, cudaStream_t st,
                      int n_rows, int n_src, int warps, size_t smem) {
    auto kern = inf_backward_ordered_kernel<MODE, CTA_ROW, COMPACT, STAGED, APLACE>;
    if (smem > 40 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    const int grid = CTA_ROW ? n_rows : (n_rows + warps - 1) / warps;
    kern<<<grid, 32 * warps, smem, st>>>(g, pos, d, dst, n_rows, n_src);
    return launch_status();
}

template <int MODE, int EPT>
int launch_fast(const float* g, const int* pos, const Dims& d, float* dst, cudaStream_t st,
                int n_rows, int n_src, int warps, size_t smem, const int* only_if) {
    auto kern = inf_backward_rows_kernel<MODE, EPT>;
    if (smem > 40 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    kern<<<n_rows, 32 * warps, smem, st>>>(g, pos, d, dst, n_rows, n_src, only_if);
    return launch_status();
}

template <int MODE>
int launch_ordered(const float* g, const int* pos, const Dims& d, float* dst, cudaStream_t st) {
    const int n_rows = (MODE == 0) ? d.R * d.G : d.CO;
    const int n_src = (MODE == 0) ? d.COg : d.R;
    const int nb = d.CIg;
    // grad_input: the sort kernel with the sources held in registers applies whenever the row fits its thread group
    const size_t fast_bytes = (size_t)fast_group_words(nb, n_src) * 4;
    const bool fast_ok = MODE == 0 && n_src <= 512 * 24 && fast_bytes <= SMEM_LIMIT;
    const int* only_if = nullptr;
    if (MODE == 0 && inf_backward_path != 1) {
        // Dense layers with many bins per source: direct accumulation (inf_backward_direct.cu).  Where its speed
        // depends on how the positions are spread, a probe decides between it and the sort kernel below.
        int rc = inf_backward_input_direct(g, pos, d, dst, st, fast_ok ? &only_if : nullptr);
        if (rc > 0 || (rc == 0 && only_if == nullptr)) return rc;
    }
    if (MODE == 1) {
        // dense layers with longer rows: the warp-per-row kernel (inf_backward_accum.cu)
        int rc = inf_backward_weight_accum(g, pos, d, dst, st);
        if (rc >= 0) return rc;
    }
    if (fast_ok && n_src > 512 * 8 && n_src <= 256 * 24 && nb < 1536) {
        // 4097 ... 6144 sources into few bins: a CTA of 8 warps with 24 sources per thread spends less time in the
        // barriers between the phases of the sort than 16 warps with 12 each (28.7 against 30.7 us at B = 512,
        // Din = 784, Dout = 5120; 84 against 88 us at B = 2048); with fewer sources, or with thousands of bins to
        // scan (46 against 42 us at Din = 5120), the wider CTA wins
        return launch_fast<MODE, 24>(g, pos, d, dst, st, n_rows, n_src, 8, fast_bytes, only_if);
    }
    if (fast_ok) {
        // one CTA of 16 warps per row; the smallest per-thread share that covers the row
        if (n_src <= 512 * 4) return launch_fast<MODE, 4>(g, pos, d, dst, st, n_rows, n_src, 16, fast_bytes, only_if);
        if (n_src <= 512 * 8) return launch_fast<MODE, 8>(g, pos, d, dst, st, n_rows, n_src, 16, fast_bytes, only_if);
        if (n_src <= 512 * 12) return launch_fast<MODE, 12>(g, pos, d, dst, st, n_rows, n_src, 16, fast_bytes, only_if);
        if (n_src <= 512 * 16) return launch_fast<MODE, 16>(g, pos, d, dst, st, n_rows, n_src, 16, fast_bytes, only_if);
        return launch_fast<MODE, 24>(g, pos, d, dst, st, n_rows, n_src, 16, fast_bytes, only_if);
    }
    const bool compact = n_src < nb;                 // fewer sources than bins: go through dense ids
    if ((size_t)group_words(1, nb, n_src, compact, false, false) * 4 > SMEM_LIMIT) return LINF_ERR_TOO_LARGE;
    if (n_src >= 2048) {
        // long rows: one CTA per row; as many warps as there are sources to share, within a
        // shared-memory budget that leaves room for several CTAs per SM.  Dense rows spread their
        // sources over many bins, where match_any is at its slowest: they place with atomics.
        const bool aplace = !compact && n_src <= 65535;
        auto bytes = [&](int W) { return (size_t)group_words(W, nb, n_src, compact, false, aplace) * 4; };
        int W = 8;
        while (W > 1 && (bytes(W) > 100 * 1024 || n_src < 64 * W)) W >>= 1;
        if (bytes(W) > SMEM_LIMIT) return LINF_ERR_TOO_LARGE;
        if (compact) return launch_ordered_as<MODE, true, true, false, false>(g, pos, d, dst, st, n_rows, n_src, W, bytes(W));
        return aplace ? launch_ordered_as<MODE, true, false, false, true>(g, pos, d, dst, st, n_rows, n_src, W, bytes(W))
                      : launch_ordered_as<MODE, true, false, false, false>(g, pos, d, dst, st, n_rows, n_src, W, bytes(W));
    }
    // short rows: one warp per row, up to 8 neighbouring rows per CTA; the rows of grad_weight
    // read their sources with a stride, so the CTA stages them in shared memory first
    const bool staged = (MODE == 1) && (size_t)group_words(1, nb, n_src, compact, true, false) * 4 * 8 <= 110 * 1024;
    const size_t gb = (size_t)group_words(1, nb, n_src, compact, staged, false) * 4;
    int rpc = (int)(SMEM_LIMIT / gb);
    if (rpc > 8) rpc = 8;
#define LINF_GO(C, S) launch_ordered_as<MODE, false, C, S, false>(g, pos, d, dst, st, n_rows, n_src, rpc, gb * rpc)
    if (compact) return staged ? LINF_GO(true, true) : LINF_GO(true, false);
    return staged ? LINF_GO(false, true) : LINF_GO(false, false);
#undef LINF_GO
}

}  // namespace

int inf_backward_input(const float* g, const int* pos, const Dims& d, float* gx, cudaStream_t st) {
    return launch_ordered<0>(g, pos, d, gx, st);
}

int inf_backward_weight(const float* g, const int* pos, const Dims& d, float* gw, cudaStream_t st) {
    return launch_ordered<1>(g, pos, d, gw, st);
}

// Both ordered gradients.  The two kernels are independent and each of them is bound by the
// latency of its sort phases rather than by throughput, so they are run side by side: grad_weight
// on the library's helper stream, which forks from, and joins back into, the caller's stream.  The
// lease keeps other host threads out of the helper stream's events until the join is queued.
int inf_backward_ordered_both(const float* g, const int* pos, const Dims& d, float* gx, float* gw,
                              cudaStream_t st) {
    SideLease side;
    if (!side.ok()) {            // no helper stream on this device: one after the other
        const int rc = launch_ordered<1>(g, pos, d, gw, st);
        const int rc2 = launch_ordered<0>(g, pos, d, gx, st);
        return rc ? rc : rc2;
    }
    if (side.fork(st) != LINF_OK) return LINF_ERR_LAUNCH;
    const int rc = launch_ordered<1>(g, pos, d, gw, side.stream());
    const int rc2 = launch_ordered<0>(g, pos, d, gx, st);
    if (side.join(st) != LINF_OK) return LINF_ERR_LAUNCH;
    return rc ? rc : rc2;
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
