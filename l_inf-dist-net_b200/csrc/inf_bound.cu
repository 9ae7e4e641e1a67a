// Interval propagation through an inf-dist layer: from elementwise input bounds
// lower <= x <= upper to bounds on y = max_i |x_i - w_i|, both outputs in one pass.
//
//   literal rule (always valid):  tL = lower - w, tU = upper - w
//       U = max_i max(|tL|, |tU|)
//       L = max_i ( (tL < 0 && tU > 0) ? 0 : min(|tL|, |tU|) )
//   fast rule (valid when lower <= upper and both are finite):  with nL = w - lower (= -tL exactly)
//       U = max(0, max_i nL, max_i tU)          -- since tL <= tU, max(|tL|,|tU|) = max(-tL, tU)
//       L = 0 - min(0, min_i nL, min_i tU)      -- straddling terms have nL > 0 and tU > 0
//     i.e. one 3-input max and one 3-input min over the SAME two differences per term.
//
// The tiled kernel runs the fast rule and, while the operand tiles pass through shared
// memory, checks the precondition on every element of its own rows; a CTA that saw a
// violation recomputes its tile with the literal rule, so the result is bit-identical to
// the literal rule for every input.
#include "common.cuh"

namespace linf {
namespace {

__device__ __forceinline__ float min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ void literal_term(float xl, float xu, float w, float& L, float& U) {
    const float tL = xl - w, tU = xu - w;
    const float aL = fabsf(tL), aU = fabsf(tU);
    U = fmaxf(U, fmaxf(aL, aU));
    if (!(tL < 0.f && tU > 0.f)) L = fmaxf(L, fminf(aL, aU));
}

// ------------------------------------------------------------------------------------
// generic path: 32 x 32 tile, literal rule, any G / HW / alignment
// ------------------------------------------------------------------------------------
constexpr int GT = 32;

template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
inf_bound_generic_kernel(const float* __restrict__ xl, const float* __restrict__ xu,
                         const float* __restrict__ w, Dims d,
                         float* __restrict__ yl, float* __restrict__ yu, Post post) {
    __shared__ float ls[GT][GT + 1], us[GT][GT + 1], ws[GT][GT + 1];
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int g = blockIdx.z, r0 = blockIdx.x * GT, c0 = blockIdx.y * GT;
    float L[4] = {0.f, 0.f, 0.f, 0.f}, U[4] = {0.f, 0.f, 0.f, 0.f};

    for (int k0 = 0; k0 < d.CIg; k0 += GT) {
        for (int e = tid; e < GT * GT; e += 256) {
            int kl, rl;
            if (ROW_FAST) { rl = e & 31; kl = e >> 5; } else { kl = e & 31; rl = e >> 5; }
            int r = r0 + rl, k = k0 + kl;
            bool in = r < d.R && k < d.CIg;
            size_t a = in ? act_index(r, g, k, d.CIg, d.G, d.HW) : 0;
            ls[kl][rl] = in ? xl[a] : 0.f;
            us[kl][rl] = in ? xu[a] : 0.f;
            int kw = e & 31, cl = e >> 5, c = c0 + cl, k2 = k0 + kw;
            ws[kw][cl] = (c < d.COg && k2 < d.CIg) ? w[(size_t)(g * d.COg + c) * d.CIg + k2] : 0.f;
        }
        __syncthreads();
        const int kmax = min(GT, d.CIg - k0);
        for (int kk = 0; kk < kmax; ++kk) {
            const float wv = ws[kk][tx];
#pragma unroll
            for (int j = 0; j < 4; ++j) literal_term(ls[kk][ty + 8 * j], us[kk][ty + 8 * j], wv, L[j], U[j]);
        }
        __syncthreads();
    }
    const int c = c0 + tx;
    if (c < d.COg) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int r = r0 + ty + 8 * j;
            if (r < d.R) {
                size_t o = act_index(r, g, c, d.COg, d.G, d.HW);
                const float lo = post_apply(post, L[j], g * d.COg + c), up = post_apply(post, U[j], g * d.COg + c);
                yl[o] = post.negate ? up : lo;
                yu[o] = post.negate ? lo : up;
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// tiled path (HW == 1, CI/G % 4 == 0, 16-byte aligned): 64 x 64 tile, 128 threads,
// 8 x 4 outputs (x 2 bounds) per thread, cp.async ring, 3 CTAs per SM.
// ------------------------------------------------------------------------------------
constexpr int BM = 64, BN = 64, NT = 128, BK = 16, LD = BK + 4, STAGES = 4, TN = 4, NO = 8 * TN;
constexpr int STAGE_FLOATS = (2 * BM + BN) * LD;
constexpr int SMEM_BYTES = STAGES * STAGE_FLOATS * 4;

struct BoundParams {
    const float* xl; const float* xu; const float* w; float* yl; float* yu;
    int M, N, K, G, lda, ldo, tiles_m, tiles_n, KT;
    int ksplit;            // CTAs per output tile, each with an equal share of the k-tiles (1 or 2)
    Post post;             // per-channel epilogue of the stored bounds (all null: none; ksplit == 1 only)
};

__device__ __forceinline__ void load_stage(float* stage, const BoundParams& p, int g, int m0, int n0,
                                           int kt, int tid) {
    constexpr int CH = BK / 4;
    const int k0 = kt * BK;
    float* Ls = stage;
    float* Us = stage + BM * LD;
    float* Bs = stage + 2 * BM * LD;
#pragma unroll
    for (int q = tid; q < BM * CH; q += NT) {
        int row = q / CH, ch = q % CH;
        int m = min(m0 + row, p.M - 1);
        int k = k0 + ch * 4;
        bool in = k < p.K;
        size_t off = (size_t)m * p.lda + (size_t)g * p.K + (in ? k : 0);
        cp_async16(Ls + row * LD + ch * 4, p.xl + off, in ? 16 : 0);
        cp_async16(Us + row * LD + ch * 4, p.xu + off, in ? 16 : 0);
    }
#pragma unroll
    for (int q = tid; q < BN * CH; q += NT) {
        int row = q / CH, ch = q % CH;
        int n = min(n0 + row, p.N - 1);
        int k = k0 + ch * 4;
        bool in = k < p.K;
        cp_async16(Bs + row * LD + ch * 4, p.w + ((size_t)g * p.N + n) * p.K + (in ? k : 0), in ? 16 : 0);
    }
}

// One k-tile.  FAST: accU = running max, accL = running MIN (negated lower bound).
// !FAST: literal rule, accL = running lower bound.
template <bool FAST>
__device__ __forceinline__ void tile_step(const float* __restrict__ Ls, const float* __restrict__ Us,
                                          const float* __restrict__ Bs, float (&accL)[NO], float (&accU)[NO]) {
#pragma unroll
    for (int k4 = 0; k4 < BK / 4; ++k4) {
        ulonglong2 bf[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) bf[j] = *reinterpret_cast<const ulonglong2*>(Bs + (8 * j) * LD + k4 * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const ulonglong2 al = *reinterpret_cast<const ulonglong2*>(Ls + (4 * i) * LD + k4 * 4);
            const ulonglong2 au = *reinterpret_cast<const ulonglong2*>(Us + (4 * i) * LD + k4 * 4);
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                if (FAST) {
                    float n0, n1, n2, n3, u0, u1, u2, u3;
                    unpack_f32x2(sub_f32x2(bf[j].x, al.x), n0, n1);   // w - lower
                    unpack_f32x2(sub_f32x2(bf[j].y, al.y), n2, n3);
                    unpack_f32x2(sub_f32x2(au.x, bf[j].x), u0, u1);   // upper - w
                    unpack_f32x2(sub_f32x2(au.y, bf[j].y), u2, u3);
                    float U = accU[i * TN + j], L = accL[i * TN + j];
                    U = max3(U, n0, u0); L = min3(L, n0, u0);
                    U = max3(U, n1, u1); L = min3(L, n1, u1);
                    U = max3(U, n2, u2); L = min3(L, n2, u2);
                    U = max3(U, n3, u3); L = min3(L, n3, u3);
                    accU[i * TN + j] = U; accL[i * TN + j] = L;
                } else {
                    float l0, l1, l2, l3, u0, u1, u2, u3, w0, w1, w2, w3;
                    unpack_f32x2(al.x, l0, l1); unpack_f32x2(al.y, l2, l3);
                    unpack_f32x2(au.x, u0, u1); unpack_f32x2(au.y, u2, u3);
                    unpack_f32x2(bf[j].x, w0, w1); unpack_f32x2(bf[j].y, w2, w3);
                    literal_term(l0, u0, w0, accL[i * TN + j], accU[i * TN + j]);
                    literal_term(l1, u1, w1, accL[i * TN + j], accU[i * TN + j]);
                    literal_term(l2, u2, w2, accL[i * TN + j], accU[i * TN + j]);
                    literal_term(l3, u3, w3, accL[i * TN + j], accU[i * TN + j]);
                }
            }
        }
    }
}

// Runs the k loop of one output tile.  Returns (FAST only) whether this thread saw an
// element of the tile's rows that breaks "lower <= upper, both finite".
template <bool FAST>
__device__ __forceinline__ bool run_tile(float* smem, const BoundParams& p, int g, int m0, int n0,
                                         int kt_begin, int kt_end, int tid, int row_off, int col_off,
                                         float (&accL)[NO], float (&accU)[NO]) {
    bool bad = false;
#pragma unroll
    for (int e = 0; e < NO; ++e) { accL[e] = 0.f; accU[e] = 0.f; }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (kt_begin + s < kt_end) load_stage(smem + s * STAGE_FLOATS, p, g, m0, n0, kt_begin + s, tid);
        cp_async_commit();
    }
    int rd = 0, wr = STAGES - 1;
    for (int kt = kt_begin; kt < kt_end; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (kt + STAGES - 1 < kt_end) load_stage(smem + wr * STAGE_FLOATS, p, g, m0, n0, kt + STAGES - 1, tid);
        cp_async_commit();
        const float* st = smem + rd * STAGE_FLOATS;
        if (FAST) {
            // each thread checks 8 of the 64 x 16 staged (lower, upper) pairs
            const int row = tid >> 1, h = (tid & 1) * 8;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float4 lo = *reinterpret_cast<const float4*>(st + row * LD + h + 4 * q);
                const float4 up = *reinterpret_cast<const float4*>(st + (BM + row) * LD + h + 4 * q);
                const float ninf = -__int_as_float(0x7f800000), pinf = __int_as_float(0x7f800000);
                bad |= !(lo.x <= up.x && lo.x > ninf && up.x < pinf);
                bad |= !(lo.y <= up.y && lo.y > ninf && up.y < pinf);
                bad |= !(lo.z <= up.z && lo.z > ninf && up.z < pinf);
                bad |= !(lo.w <= up.w && lo.w > ninf && up.w < pinf);
            }
        }
        tile_step<FAST>(st + row_off * LD, st + (BM + row_off) * LD, st + (2 * BM + col_off) * LD, accL, accU);
        rd = (rd + 1 == STAGES) ? 0 : rd + 1;
        wr = (wr + 1 == STAGES) ? 0 : wr + 1;
    }
    cp_async_wait<0>();
    return bad;
}

__global__ void __launch_bounds__(NT, 3)
inf_bound_tiled_kernel(const BoundParams p) {
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 1, wn = warp >> 1, lm = lane >> 3, ln = lane & 7;
    const int row_off = wm * 32 + lm, col_off = wn * (8 * TN) + ln;

    const int tiles_per_group = p.tiles_m * p.tiles_n;
    // With ksplit = 2 two CTAs share an output tile, each over one half of the k-tiles.  Both bounds are maxima of
    // non-negative numbers that start from 0, so the halves are combined with an integer atomicMax on the zero-filled
    // outputs (non-negative floats order like their bit patterns): exact, whichever CTA comes first.
    const int tile = (int)blockIdx.x / p.ksplit, part = (int)blockIdx.x - tile * p.ksplit;
    const int kt_begin = p.KT * part / p.ksplit, kt_end = p.KT * (part + 1) / p.ksplit;
    const int g = tile / tiles_per_group, tg = tile - g * tiles_per_group;
    const int n0 = (tg / p.tiles_m) * BN, m0 = (tg % p.tiles_m) * BM;

    float accL[NO], accU[NO];
    const bool bad = run_tile<true>(smem, p, g, m0, n0, kt_begin, kt_end, tid, row_off, col_off, accL, accU);
    const bool any_bad = __syncthreads_or(bad);
    if (!any_bad) {
#pragma unroll
        for (int e = 0; e < NO; ++e) accL[e] = 0.f - accL[e];
    } else {
        run_tile<false>(smem, p, g, m0, n0, kt_begin, kt_end, tid, row_off, col_off, accL, accU);
    }
    if (p.ksplit > 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = m0 + row_off + 4 * i;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + col_off + 8 * j;
                if (m < p.M && n < p.N) {
                    const size_t o = (size_t)m * p.ldo + (size_t)g * p.N + n;
                    atomicMax(reinterpret_cast<int*>(p.yl + o), __float_as_int(accL[i * TN + j]));
                    atomicMax(reinterpret_cast<int*>(p.yu + o), __float_as_int(accU[i * TN + j]));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + row_off + 4 * i;
        if (m < p.M) {
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + col_off + 8 * j;
                if (n < p.N) {
                    const size_t o = (size_t)m * p.ldo + (size_t)g * p.N + n;
                    const float lo = post_apply(p.post, accL[i * TN + j], g * p.N + n);
                    const float up = post_apply(p.post, accU[i * TN + j], g * p.N + n);
                    p.yl[o] = p.post.negate ? up : lo;       // a negated upper bound is the new lower bound
                    p.yu[o] = p.post.negate ? lo : up;
                }
            }
        }
    }
}

// The per-channel epilogue as a pass of its own, for launches that combined partial results in memory.
__global__ void __launch_bounds__(256)
inf_bound_post_kernel(float* __restrict__ yl, float* __restrict__ yu, size_t n, int CO, Post post) {
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < n; e += (size_t)gridDim.x * 256) {
        const int c = (int)(e % (size_t)CO);
        const float lo = post_apply(post, yl[e], c), up = post_apply(post, yu[e], c);
        yl[e] = post.negate ? up : lo;
        yu[e] = post.negate ? lo : up;
    }
}

}  // namespace

int inf_bound(const float* xl, const float* xu, const float* w, const Dims& d,
              float* yl, float* yu, cudaStream_t st, const Post& post) {
    const bool tiled = d.HW == 1 && (d.CIg % 4) == 0 && aligned16(xl) && aligned16(xu) && aligned16(w) &&
                       d.COg >= 32;
    if (!tiled) {
        if (skinny_ok(d, xl, xu, w)) return inf_bound_skinny(xl, xu, w, d, yl, yu, st, post);
        dim3 grid((d.R + GT - 1) / GT, (d.COg + GT - 1) / GT, d.G);
        if (grid.y > 65535u || grid.z > 65535u) return LINF_ERR_DIMS;
        if (d.HW > 1) inf_bound_generic_kernel<true><<<grid, 256, 0, st>>>(xl, xu, w, d, yl, yu, post);
        else inf_bound_generic_kernel<false><<<grid, 256, 0, st>>>(xl, xu, w, d, yl, yu, post);
        return launch_status();
    }
    BoundParams p;
    p.xl = xl; p.xu = xu; p.w = w; p.yl = yl; p.yu = yu;
    p.M = d.R; p.N = d.COg; p.K = d.CIg; p.G = d.G; p.lda = d.CI; p.ldo = d.CO;
    p.post = post;
    p.ksplit = 1;
    p.tiles_m = (d.R + BM - 1) / BM; p.tiles_n = (d.COg + BN - 1) / BN;
    p.KT = (d.CIg + BK - 1) / BK;
    int grid = p.tiles_m * p.tiles_n * d.G;
    {
        // Output tiles that leave much of their last wave of CTAs idle, with long rows: two CTAs per tile (1.58 ->
        // 1.2 ms at B = 512, Din = 3072, Dout = 5120: 640 tiles on 444 CTA slots).
        const int slots = 3 * sm_count();
        auto fill = [&](int n) { return (double)n / ((double)((n + slots - 1) / slots) * slots); };
        if (p.KT >= 64 && fill(2 * grid) > 1.15 * fill(grid)) {
            const size_t bytes = (size_t)d.R * d.CO * sizeof(float);
            if (cudaMemsetAsync(yl, 0, bytes, st) != cudaSuccess || cudaMemsetAsync(yu, 0, bytes, st) != cudaSuccess)
                return LINF_ERR_LAUNCH;
            p.ksplit = 2;
            grid *= 2;
        }
    }
    // opting in to > 48 KB of dynamic shared memory is per function and per device; repeating it on
    // every call is cheap and keeps the launcher free of per-device state
    if (cudaFuncSetAttribute(inf_bound_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    inf_bound_tiled_kernel<<<grid, NT, SMEM_BYTES, st>>>(p);
    int launched = 1;
    if (p.ksplit > 1 && (post.sub != nullptr || post.add != nullptr || post.negate)) {
        const size_t n = (size_t)d.R * d.CO;
        inf_bound_post_kernel<<<2 * sm_count(), 256, 0, st>>>(yl, yu, n, d.CO, post);
        launched = 2;
    }
    return launch_status(launched);
}

}  // namespace linf
