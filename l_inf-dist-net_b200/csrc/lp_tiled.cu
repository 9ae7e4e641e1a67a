// Register-tiled kernels for the finite-p distance neuron on dense layers (HW == 1, channel
// counts per group multiples of 4, 16-byte aligned tensors).  64 x 64 output tile per CTA of 128
// threads, 8 x 4 outputs per thread, operand tiles staged through shared memory with cp.async in a
// multi-stage ring (the geometry of the inf-dist forward).
//
//   forward          S[b,o] = sum_i (|x[b,i] - w[o,i]| / M[b,o])^p        reduce over i
//                    (M is read from `y`, which the caller filled with max_i |x - w|; y := M * S^(1/p))
//   backward input   gx[b,i] = sum_o g[b,o] * s * |s|^(p-2),  s = (x[b,i] - w[o,i]) / y[b,o]   reduce over o
//   backward weight  gw[o,i] = sum_b g[b,o] * s * |s|^(p-2),  s = (w[o,i] - x[b,i]) / y[b,o]   reduce over b
//
// s * |s|^(p-2) equals |t/y|^(p-1) * sign(t) and keeps the sign for free.  IP > 0 instantiates an
// integer p known at compile time (8, 16, 64: the powers are a handful of multiplies on the FP32
// pipe); IP == 0 takes p at run time (integer part by square-and-multiply, fractional part by one
// log2/exp2 pair on the special-function unit, skipped when p is an integer).
#include <math.h>

#include "common.cuh"

namespace linf {
namespace {

constexpr int TM = 64, TN = 64, NT = 128, BK = 16, LDK = BK + 4, STAGES = 3;

struct Pw {          // run-time exponent q = n + f
    int n; float f;
};

__device__ __forceinline__ float lg2_approx(float a) {
    float r; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r;
}
__device__ __forceinline__ float ex2_approx(float a) {
    float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r;
}

// a^(n + f) for 0 <= a <= ~1 with the integer part n < 2^NB: square-and-multiply unrolled over the
// NB low bits of n (the bit tests are uniform across the grid), fractional part by log2/exp2
template <int NB>
__device__ __forceinline__ float pow_bits(float a, const Pw q) {
    float r = 1.f, b = a;
#pragma unroll
    for (int k = 0; k < NB; ++k) {
        if ((q.n >> k) & 1) r *= b;
        if (k + 1 < NB) b *= b;
    }
    if (q.f != 0.f) r *= ex2_approx(q.f * lg2_approx(a));     // a = 0: exp2(-inf) = 0
    return r;
}

// a^E for a compile-time non-negative integer E
template <int E>
__device__ __forceinline__ float pow_ct(float a) {
    if (E == 0) return 1.f;
    if (E == 1) return a;
    const float h = pow_ct<E / 2>(a);
    return (E & 1) ? h * h * a : h * h;
}

// Template parameter IP of the kernels: IP > 0 is an integer p fixed at compile time; IP <= 0 takes
// p at run time (backward: -IP = number of bits of the integer part of p - 1).

// term of the forward sum: u^p, u >= 0.  The run-time path is one log2/exp2 pair: its relative
// error of about p * 2e-7 per term shrinks by 1/p again in the final S^(1/p).
template <int IP>
__device__ __forceinline__ float fwd_term(float u, const Pw q, float p) {
    if (IP > 0) return pow_ct<(IP > 0 ? IP : 1)>(u);
    return ex2_approx(p * lg2_approx(u));
}

// backward factor s * |s|^(p-2) (q holds p - 1 for the run-time path)
template <int IP>
__device__ __forceinline__ float bwd_factor(float s, const Pw q) {
    if (IP > 0) return s * pow_ct<(IP > 1 ? IP - 2 : 0)>(fabsf(s));
    return copysignf(pow_bits<(IP < 0 ? -IP : 2)>(fabsf(s), q), s);
}

// cp.async copy of a ROWS x COLS tile of a row-major matrix into shared memory (row pitch LD
// floats); rows/columns beyond the valid extent are zero-filled.  COLS % 4 == 0.
template <int ROWS, int COLS, int LD>
__device__ __forceinline__ void load_tile(float* dst, const float* __restrict__ src, size_t ld_src,
                                          int row0, int rows_valid, int col0, int cols_valid, int tid) {
    constexpr int CH = COLS / 4;
#pragma unroll
    for (int q = tid; q < ROWS * CH; q += NT) {
        const int r = q / CH, c = (q % CH) * 4;
        const bool in = (row0 + r < rows_valid) && (col0 + c < cols_valid);
        const float* s = src + (size_t)(in ? row0 + r : 0) * ld_src + (in ? col0 + c : 0);
        cp_async16(dst + r * LD + c, s, in ? 16 : 0);
    }
}

struct LpParams {
    const float* x; const float* w; const float* g; float* y; float* out;
    int B, COg, CIg, G, CI, CO;
    Pw q; float inv_p, pf;
    int ksplit;        // backward: CTAs per output tile, each with an equal share of the reduction (1 or 2)
};

// ------------------------------------------------------------------------------------------------
// forward: tile = 64 rows (b) x 64 outputs (o), reduce over i; x and w tiles are K-contiguous
// ------------------------------------------------------------------------------------------------
// TJ = output columns per thread (4: 64-wide tiles; 3: 48-wide tiles, for shapes whose 64-wide tiles
// leave much of their last wave of CTAs idle)
template <int IP, int TJ>
__global__ void __launch_bounds__(NT, 3)
lp_forward_tiled_kernel(const LpParams p) {
    extern __shared__ __align__(16) float smem[];
    constexpr int TNF = 16 * TJ, NO = 8 * TJ;
    constexpr int STAGE = (TM + TNF) * LDK;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 1, wn = warp >> 1, lm = lane >> 3, ln = lane & 7;
    const int row_off = wm * 32 + lm, col_off = wn * (8 * TJ) + ln;       // + 4i rows, + 8j columns
    const int tiles_m = (p.B + TM - 1) / TM, tiles_n = (p.COg + TNF - 1) / TNF;
    const int g = blockIdx.x / (tiles_m * tiles_n), tg = blockIdx.x % (tiles_m * tiles_n);
    const int n0 = (tg / tiles_m) * TNF, m0 = (tg % tiles_m) * TM;
    const float* xg = p.x + (size_t)g * p.CIg;
    const float* wg = p.w + (size_t)g * p.COg * p.CIg;
    const int KT = (p.CIg + BK - 1) / BK;

    float S[NO], rM[NO];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < TJ; ++j) {
            const int m = min(m0 + row_off + 4 * i, p.B - 1), n = min(n0 + col_off + 8 * j, p.COg - 1);
            const float M = p.y[(size_t)m * p.CO + (size_t)g * p.COg + n];
            rM[i * TJ + j] = M > 0.f ? 1.f / M : 0.f;
            S[i * TJ + j] = 0.f;
        }
    auto load = [&](int s, int kt) {
        float* st = smem + s * STAGE;
        load_tile<TM, BK, LDK>(st, xg, p.CI, m0, p.B, kt * BK, p.CIg, tid);
        load_tile<TNF, BK, LDK>(st + TM * LDK, wg, p.CIg, n0, p.COg, kt * BK, p.CIg, tid);
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) { if (s < KT) load(s, s); cp_async_commit(); }
    int rd = 0, wr = STAGES - 1;
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (kt + STAGES - 1 < KT) load(wr, kt + STAGES - 1);
        cp_async_commit();
        const float* As = smem + rd * STAGE + row_off * LDK;
        const float* Bs = smem + rd * STAGE + (TM + col_off) * LDK;
        // two of the four k4 steps per loop trip: the fully unrolled body (4 x 128 power sums) ran into instruction
        // fetch stalls (p = 64: 6.7 ms unrolled, 4.6 ms so)
#pragma unroll 2
        for (int k4 = 0; k4 < BK / 4; ++k4) {
            ulonglong2 bf[TJ];
#pragma unroll
            for (int j = 0; j < TJ; ++j) bf[j] = *reinterpret_cast<const ulonglong2*>(Bs + (8 * j) * LDK + k4 * 4);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const ulonglong2 af = *reinterpret_cast<const ulonglong2*>(As + (4 * i) * LDK + k4 * 4);
#pragma unroll
                for (int j = 0; j < TJ; ++j) {
                    float t0, t1, t2, t3;
                    unpack_f32x2(sub_f32x2(af.x, bf[j].x), t0, t1);
                    unpack_f32x2(sub_f32x2(af.y, bf[j].y), t2, t3);
                    const float r = rM[i * TJ + j];
                    float s = S[i * TJ + j];
                    s += fwd_term<IP>(fabsf(t0) * r, p.q, p.pf);
                    s += fwd_term<IP>(fabsf(t1) * r, p.q, p.pf);
                    s += fwd_term<IP>(fabsf(t2) * r, p.q, p.pf);
                    s += fwd_term<IP>(fabsf(t3) * r, p.q, p.pf);
                    S[i * TJ + j] = s;
                }
            }
        }
        rd = (rd + 1 == STAGES) ? 0 : rd + 1;
        wr = (wr + 1 == STAGES) ? 0 : wr + 1;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + row_off + 4 * i;
#pragma unroll
        for (int j = 0; j < TJ; ++j) {
            const int n = n0 + col_off + 8 * j;
            if (m < p.B && n < p.COg) {
                float* yo = p.y + (size_t)m * p.CO + (size_t)g * p.COg + n;
                const float M = *yo;                     // still the normaliser: nobody else writes this element
                *yo = M > 0.f ? powf(S[i * TJ + j], p.inv_p) * M : 0.f;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// backward: one kernel for both gradients.
//   WRT_W == false: tile = 64 rows (b) x 64 inputs (i), reduce over outputs o.
//       per k-tile: g, y tiles [64 b][16 o] (K-contiguous), w tile [16 o][64 i]; x[b,i] in registers
//   WRT_W == true : tile = 64 outputs (o) x 64 inputs (i), reduce over rows b.
//       per k-tile: g, y tiles [16 b][64 o], x tile [16 b][64 i]; w[o,i] in registers
// The y tile is turned into 1/y in shared memory once per stage (0 where y == 0).
// ------------------------------------------------------------------------------------------------
constexpr int LDN = TN + 4;

template <int IP, bool WRT_W>
__global__ void __launch_bounds__(NT, 3)
lp_backward_tiled_kernel(const LpParams p) {
    extern __shared__ __align__(16) float smem[];
    // stage layout: !WRT_W: G[64][LDK], Y[64][LDK], W[16][LDN];  WRT_W: G[16][LDN], Y[16][LDN], X[16][LDN]
    constexpr int GY = WRT_W ? BK * LDN : TM * LDK;
    constexpr int STAGE = 2 * GY + BK * LDN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 1, wn = warp >> 1, lm = lane >> 3, ln = lane & 7;
    const int MT = WRT_W ? p.COg : p.B;                 // extent of the tile's row dimension
    const int KD = WRT_W ? p.B : p.COg;                 // extent of the reduction
    const int tiles_m = (MT + TM - 1) / TM, tiles_n = (p.CIg + TN - 1) / TN;
    // With ksplit = 2 two CTAs share an output tile, each reducing over one half of the k-tiles and adding
    // its sum to the zero-filled output with one atomic per element: the two additions commute, so the
    // result does not depend on which CTA comes first.
    const int bid = (int)blockIdx.x / p.ksplit, part = (int)blockIdx.x - bid * p.ksplit;
    const int g = bid / (tiles_m * tiles_n), tg = bid % (tiles_m * tiles_n);
    const int n0 = (tg / tiles_m) * TN, m0 = (tg % tiles_m) * TM;
    const int KT_all = (KD + BK - 1) / BK;
    const int kt_begin = KT_all * part / p.ksplit, KT = KT_all * (part + 1) / p.ksplit;
    const float* xg = p.x + (size_t)g * p.CIg;                       // [B][CI]
    const float* wg = p.w + (size_t)g * p.COg * p.CIg;               // [COg][CIg]
    const float* gg = p.g + (size_t)g * p.COg;                       // [B][CO]
    const float* yg = p.y + (size_t)g * p.COg;
    // rows owned: !WRT_W: b = m0 + wm*32 + lm + 4i (strided, K-contiguous fragments)
    //             WRT_W : o = m0 + wm*32 + lm*8 + i (8 consecutive, read as two 16-byte fragments)
    // columns owned: i = n0 + wn*32 + ln*4 + j (4 consecutive)
    const int col_off = wn * 32 + ln * 4;
    float fixed[32], acc[32];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = min(n0 + col_off + j, p.CIg - 1);
            float v;
            if (WRT_W) v = wg[(size_t)min(m0 + wm * 32 + lm * 8 + i, p.COg - 1) * p.CIg + c];
            else v = xg[(size_t)min(m0 + wm * 32 + lm + 4 * i, p.B - 1) * p.CI + c];
            fixed[i * 4 + j] = v; acc[i * 4 + j] = 0.f;
        }
    auto load = [&](int s, int kt) {
        float* st = smem + s * STAGE;
        if (WRT_W) {
            load_tile<BK, TM, LDN>(st, gg, p.CO, kt * BK, p.B, m0, p.COg, tid);
            load_tile<BK, TM, LDN>(st + GY, yg, p.CO, kt * BK, p.B, m0, p.COg, tid);
            load_tile<BK, TN, LDN>(st + 2 * GY, xg, p.CI, kt * BK, p.B, n0, p.CIg, tid);
        } else {
            load_tile<TM, BK, LDK>(st, gg, p.CO, m0, p.B, kt * BK, p.COg, tid);
            load_tile<TM, BK, LDK>(st + GY, yg, p.CO, m0, p.B, kt * BK, p.COg, tid);
            load_tile<BK, TN, LDN>(st + 2 * GY, wg, p.CIg, kt * BK, p.COg, n0, p.CIg, tid);
        }
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) { if (kt_begin + s < KT) load(s, kt_begin + s); cp_async_commit(); }
    int rd = 0, wr = STAGES - 1;
    for (int kt = kt_begin; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (kt + STAGES - 1 < KT) load(wr, kt + STAGES - 1);
        cp_async_commit();
        float* st = smem + rd * STAGE;
        {   // y -> 1/y, once per element of the stage
            float* ys = st + GY;
            constexpr int ROWS = WRT_W ? BK : TM, COLS = WRT_W ? TM : BK, LD = WRT_W ? LDN : LDK;
#pragma unroll
            for (int q = tid; q < ROWS * COLS; q += NT) {
                float* e = ys + (q / COLS) * LD + (q % COLS);
                const float v = *e;
                *e = v > 0.f ? 1.f / v : 0.f;
            }
        }
        __syncthreads();
        if (WRT_W) {
            const float* Gs = st + wm * 32 + lm * 8;
            const float* Ys = st + GY + wm * 32 + lm * 8;
            const float* Xs = st + 2 * GY + col_off;
#pragma unroll 4
            for (int k = 0; k < BK; ++k) {
                const float4 g0 = *reinterpret_cast<const float4*>(Gs + k * LDN), g1 = *reinterpret_cast<const float4*>(Gs + k * LDN + 4);
                const float4 y0 = *reinterpret_cast<const float4*>(Ys + k * LDN), y1 = *reinterpret_cast<const float4*>(Ys + k * LDN + 4);
                const float4 xv = *reinterpret_cast<const float4*>(Xs + k * LDN);
                const float gr[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                const float yr[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
                const float xc[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float s = (fixed[i * 4 + j] - xc[j]) * yr[i];
                        acc[i * 4 + j] = fmaf(gr[i], bwd_factor<IP>(s, p.q), acc[i * 4 + j]);
                    }
            }
        } else {
            const float* Gs = st + (wm * 32 + lm) * LDK;
            const float* Ys = st + GY + (wm * 32 + lm) * LDK;
            const float* Ws = st + 2 * GY + col_off;
            // not unrolled: the body of one k4 step is 128 power evaluations; four copies of it do not fit the
            // instruction cache (the profile of the fully unrolled loop showed instruction fetch as its top stall)
#pragma unroll 1
            for (int k4 = 0; k4 < BK / 4; ++k4) {
                float4 wv[4];
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) wv[kk] = *reinterpret_cast<const float4*>(Ws + (k4 * 4 + kk) * LDN);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 gv = *reinterpret_cast<const float4*>(Gs + (4 * i) * LDK + k4 * 4);
                    const float4 yv = *reinterpret_cast<const float4*>(Ys + (4 * i) * LDK + k4 * 4);
                    const float gk[4] = {gv.x, gv.y, gv.z, gv.w}, yk[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const float wc[4] = {wv[kk].x, wv[kk].y, wv[kk].z, wv[kk].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float s = (fixed[i * 4 + j] - wc[j]) * yk[kk];
                            acc[i * 4 + j] = fmaf(gk[kk], bwd_factor<IP>(s, p.q), acc[i * 4 + j]);
                        }
                    }
                }
            }
        }
        rd = (rd + 1 == STAGES) ? 0 : rd + 1;
        wr = (wr + 1 == STAGES) ? 0 : wr + 1;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = WRT_W ? m0 + wm * 32 + lm * 8 + i : m0 + wm * 32 + lm + 4 * i;
        if (r < MT) {
            float* orow = WRT_W ? p.out + ((size_t)g * p.COg + r) * p.CIg : p.out + (size_t)r * p.CI + (size_t)g * p.CIg;
            const int c = n0 + col_off;
            if (p.ksplit > 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (c + j < p.CIg) atomicAdd(orow + c + j, acc[i * 4 + j]);
            } else if (c + 3 < p.CIg) {
                *reinterpret_cast<float4*>(orow + c) = make_float4(acc[i * 4], acc[i * 4 + 1], acc[i * 4 + 2], acc[i * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (c + j < p.CIg) orow[c + j] = acc[i * 4 + j];
            }
        }
    }
}

Pw make_pw(float q) {
    Pw r; const float fl = floorf(q);
    r.n = (int)fl; r.f = q - fl;
    return r;
}

template <class K>
int set_smem(K kern, int bytes) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? LINF_OK
                                                                                                         : LINF_ERR_LAUNCH;
}

constexpr int BWD_X_SMEM = STAGES * (2 * TM * LDK + BK * LDN) * 4;
constexpr int BWD_W_SMEM = STAGES * (3 * BK * LDN) * 4;

}  // namespace

bool lp_tiled_ok(const Dims& d, const void* a, const void* b, const void* c, const void* e, const void* f) {
    return d.HW == 1 && (d.CIg % 4) == 0 && (d.COg % 4) == 0 && (d.CI % 4) == 0 && (d.CO % 4) == 0 &&
           d.COg >= 32 && d.CIg >= 32 && aligned16(a) && aligned16(b) && aligned16(c) &&
           (e == nullptr || aligned16(e)) && (f == nullptr || aligned16(f));
}

static LpParams make_params(const float* x, const float* w, const float* g, float* y, float* out,
                            const Dims& d, float q, float p) {
    LpParams P;
    P.x = x; P.w = w; P.g = g; P.y = y; P.out = out;
    P.B = d.R; P.COg = d.COg; P.CIg = d.CIg; P.G = d.G; P.CI = d.CI; P.CO = d.CO;
    P.q = make_pw(q); P.inv_p = 1.f / p; P.pf = p;
    P.ksplit = 1;
    return P;
}

int lp_forward_width = 0;   // 0: tile width by shape; 1: 64 columns; 2: 48 columns (benchmarking knob)

// `y` holds max_i |x - w| on entry and the L_p distance on exit
int lp_forward_tiled(const float* x, const float* w, const Dims& d, float* y, float p, cudaStream_t st) {
    const LpParams P = make_params(x, w, nullptr, y, nullptr, d, p, p);
    // The kernel is bound by FP32 throughput: an SM of the last, partial wave takes a third of a full wave per CTA
    // it holds.  48-wide tiles cost 3/4 of 64-wide ones and are taken when that buys a shorter launch
    // (B = 512, Dout = 5120: 640 tiles on 444 slots = 1 + 2/3 waves, against 856 tiles = 2 x 3/4).
    const int tiles_m = (d.R + TM - 1) / TM, slots = 3 * sm_count(), sms = sm_count();
    auto cost = [&](int tn) {
        const int tiles = tiles_m * ((d.COg + tn - 1) / tn) * d.G, rest = tiles % slots;
        return (tn / 64.0) * ((tiles / slots) + ((rest + sms - 1) / sms) / 3.0);
    };
    const bool narrow = lp_forward_width == 2 || (lp_forward_width == 0 && d.COg >= 48 && cost(48) < 0.97 * cost(64));
    const int tn = narrow ? 48 : 64;
    const int grid = tiles_m * ((d.COg + tn - 1) / tn) * d.G;
    const int smem = STAGES * (TM + tn) * LDK * 4;
#define LINF_FWD(IPV)                                                                                       \
    { if (narrow) {                                                                                         \
          if (set_smem(lp_forward_tiled_kernel<IPV, 3>, smem)) return LINF_ERR_LAUNCH;                      \
          lp_forward_tiled_kernel<IPV, 3><<<grid, NT, smem, st>>>(P);                                       \
      } else {                                                                                              \
          if (set_smem(lp_forward_tiled_kernel<IPV, 4>, smem)) return LINF_ERR_LAUNCH;                      \
          lp_forward_tiled_kernel<IPV, 4><<<grid, NT, smem, st>>>(P);                                       \
      }                                                                                                     \
      return launch_status(); }
    if (p == 8.f) LINF_FWD(8)
    if (p == 16.f) LINF_FWD(16)
    if (p == 64.f) LINF_FWD(64)
    LINF_FWD(0)
#undef LINF_FWD
}

int lp_backward_tiled(const float* g, const float* x, const float* w, const float* y, const Dims& d,
                      float* out, float p, bool wrt_weight, cudaStream_t st) {
    LpParams P = make_params(x, w, g, const_cast<float*>(y), out, d, p - 1.f, p);
    const int mt = wrt_weight ? d.COg : d.R;
    int grid = ((mt + TM - 1) / TM) * ((d.CIg + TN - 1) / TN) * d.G;
    {
        // Output tiles that leave much of their last wave of CTAs idle, with a long reduction: two CTAs per
        // tile, each with half of the reduction (4.6 -> 3.4 ms for grad_input at B = 512, Din = Dout = 5120, p = 8:
        // 640 tiles on 444 CTA slots).
        const int slots = 3 * sm_count();
        auto fill = [&](int n) { return (double)n / ((double)((n + slots - 1) / slots) * slots); };
        const int kd = wrt_weight ? d.R : d.COg;
        if (kd >= 64 * BK && fill(2 * grid) > 1.15 * fill(grid)) {
            const size_t bytes = (wrt_weight ? (size_t)d.CO * d.CIg : (size_t)d.R * d.CI) * sizeof(float);
            if (cudaMemsetAsync(out, 0, bytes, st) != cudaSuccess) return LINF_ERR_LAUNCH;
            P.ksplit = 2;
            grid *= 2;
        }
    }
#define LINF_BWD(IPV, W, SM)                                                                   \
    { if (set_smem(lp_backward_tiled_kernel<IPV, W>, SM)) return LINF_ERR_LAUNCH;              \
      lp_backward_tiled_kernel<IPV, W><<<grid, NT, SM, st>>>(P); return launch_status(); }
    // run-time p: instantiate for the bit length of the integer part of p - 1 (rounded up to even)
    const int n = P.q.n;
    const int nb = n < 4 ? 2 : n < 16 ? 4 : n < 64 ? 6 : n < 256 ? 8 : n < 1024 ? 10 : 0;
    if (wrt_weight) {
        if (p == 8.f) LINF_BWD(8, true, BWD_W_SMEM)
        if (p == 16.f) LINF_BWD(16, true, BWD_W_SMEM)
        if (p == 64.f) LINF_BWD(64, true, BWD_W_SMEM)
        if (nb == 2) LINF_BWD(-2, true, BWD_W_SMEM)
        if (nb == 4) LINF_BWD(-4, true, BWD_W_SMEM)
        if (nb == 6) LINF_BWD(-6, true, BWD_W_SMEM)
        if (nb == 8) LINF_BWD(-8, true, BWD_W_SMEM)
        if (nb == 10) LINF_BWD(-10, true, BWD_W_SMEM)
        return -1;
    }
    if (p == 8.f) LINF_BWD(8, false, BWD_X_SMEM)
    if (p == 16.f) LINF_BWD(16, false, BWD_X_SMEM)
    if (p == 64.f) LINF_BWD(64, false, BWD_X_SMEM)
    if (nb == 2) LINF_BWD(-2, false, BWD_X_SMEM)
    if (nb == 4) LINF_BWD(-4, false, BWD_X_SMEM)
    if (nb == 6) LINF_BWD(-6, false, BWD_X_SMEM)
    if (nb == 8) LINF_BWD(-8, false, BWD_X_SMEM)
    if (nb == 10) LINF_BWD(-10, false, BWD_X_SMEM)
    return -1;
#undef LINF_BWD
}

}  // namespace linf
