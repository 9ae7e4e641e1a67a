// inf-dist forward: y[r,o] = max_i |x[r,i] - w[o,i]| with capture of the lowest arg-max index.
//
// Three paths:
//   * tiled path (dense layers: HW == 1, CI/G a multiple of 4, 16-byte aligned pointers, at
//     least 32 outputs per group): a register-tiled (max, |a-b|) "GEMM" on the FP32 cores.  A
//     CTA of 128 threads owns a 64 x 64 output tile, a thread an 8 x 4 sub-tile, three CTAs share
//     an SM.  Operand tiles are staged through shared memory with cp.async in a 4-stage ring and
//     read back with 128-bit loads along k, so that two neighbouring k-terms of one output sit in
//     one 64-bit register pair: one packed `sub.f32x2` produces both differences and one 3-input
//     `max.f32` folds both |differences| into the running maximum.  Both are half-rate
//     instructions, i.e. two issue cycles per pair of terms each -- the same two cycles per term
//     as a scalar subtract plus a scalar max, but with half the instructions to fetch and decode.
//     The arg-max is NOT tracked per term.  The loop only records, once per tracking window (a
//     k-tile or a fraction of one), which window last raised the maximum; after the loop the
//     winning window alone is rescanned for the first index whose |difference| equals the
//     maximum (strict ">" between windows plus first-match inside a window = lowest index among
//     exact ties).
//     With scratch memory the k-tiles of all output tiles are dealt out evenly to the CTAs that
//     fit the GPU at once; an output tile cut by a CTA boundary is finished by whichever of its
//     CTAs arrives last (ticket counter, nobody waits).
//     Without k-splitting, a CTA is bound by latency, not by what its neighbours on the SM do
//     (measured at B = 512, Din = 784, Dout = 5120: 444 tiles, three per SM, take 108 us; the 196
//     tiles left over, one or two per SM, still take 87 us).  So when whole waves of tiles are
//     followed by a partial one, the columns of the partial wave are cut into tiles of half the
//     width and run as a second launch of twice as many CTAs, which fills the GPU again.
//   * few outputs per group (skinny.cu): the reduction is spread over the threads of a CTA.
//   * generic path (any G, HW, alignment): 32 x 32 tile, index tracked per term.
#include <cuda.h>   // CUtensorMap and the enums of cuTensorMapEncodeTiled (types only: no libcuda link)

#include "common.cuh"

namespace linf {

// =====================================================================================
// generic path
// =====================================================================================
namespace {

constexpr int GT = 32;  // generic tile edge

template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
inf_forward_generic_kernel(const float* __restrict__ x, const float* __restrict__ w, Dims d,
                           float* __restrict__ y, int* __restrict__ pos, Post post) {
    __shared__ float xs[GT][GT + 1];  // [k][row]
    __shared__ float ws[GT][GT + 1];  // [k][col]
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int g = blockIdx.z, r0 = blockIdx.x * GT, c0 = blockIdx.y * GT;

    float best[4] = {0.f, 0.f, 0.f, 0.f};
    int arg[4] = {0, 0, 0, 0};

    for (int k0 = 0; k0 < d.CIg; k0 += GT) {
        for (int e = tid; e < GT * GT; e += 256) {
            int kl, rl;
            if (ROW_FAST) { rl = e & 31; kl = e >> 5; } else { kl = e & 31; rl = e >> 5; }
            int r = r0 + rl, k = k0 + kl;
            xs[kl][rl] = (r < d.R && k < d.CIg) ? x[act_index(r, g, k, d.CIg, d.G, d.HW)] : 0.f;
            int kw = e & 31, cl = e >> 5, c = c0 + cl, k2 = k0 + kw;
            ws[kw][cl] = (c < d.COg && k2 < d.CIg) ? w[(size_t)(g * d.COg + c) * d.CIg + k2] : 0.f;
        }
        __syncthreads();
        const int kmax = min(GT, d.CIg - k0);
        for (int kk = 0; kk < kmax; ++kk) {
            const float wv = ws[kk][tx];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t = xs[kk][ty + 8 * j] - wv;
                float a = fabsf(t);
                if (a > best[j]) {
                    best[j] = a;
                    arg[j] = (k0 + kk) | (t >= 0.f ? 0 : (int)0x80000000);
                }
            }
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
                y[o] = post_apply(post, best[j], g * d.COg + c);
                if (pos) pos[o] = arg[j];
            }
        }
    }
}

// =====================================================================================
// tiled path
// =====================================================================================
// Geometry of one kernel variant.  A thread owns 8 rows x TN columns; a warp (4 x 8 lanes)
// owns 32 rows x 8*TN columns; a CTA has 2 warps along m and NT/64 along n.
template <int NT_, int TN_, int BK_, int MINB_, int TW_ = BK_, int PAD_ = 4, int STAGES_ = 0>
struct Geo {
    static constexpr int NT = NT_, TN = TN_, BK = BK_, MINB = MINB_;
    static constexpr int TW = TW_;                      // terms per arg-max tracking window
    static constexpr int NSUB = BK / TW;                // tracking windows per k-tile (1, or even)
    static constexpr int BM = 64, BN = (NT / 64) * 8 * TN;
    static constexpr int NOUT = 8 * TN;                 // outputs per thread
    static constexpr int TILE_OUT = BM * BN;
    static constexpr int LD = BK + PAD_;                // row length in shared memory, in floats (PAD_ = 0: swizzled rows)
    static constexpr int STAGES = STAGES_ > 0 ? STAGES_ : (BK <= 16) ? 4 : 3;
    static constexpr int STAGE_FLOATS = (BM + BN) * LD;
    static constexpr int SMEM_BYTES = STAGES * STAGE_FLOATS * 4;
    static_assert(BK % TW == 0 && TW % 4 == 0 && (NSUB == 1 || NSUB % 2 == 0), "tracking window");
};

struct TiledParams {
    const float* x; const float* w; float* y; int* pos;
    int M, N, K, G;        // rows, per-group outputs, per-group inputs, groups
    int lda;               // floats between consecutive rows of x (= CI)
    int ldo;               // floats between consecutive rows of y (= CO)
    int tiles_m, tiles_n;  // per group
    int KT;                // k-tiles per output tile
    int n_cta;             // CTAs of the launch (units are dealt evenly to them)
    int slots_cta;         // CTAs the partial-result area was sized for
    int tile0;             // whole mode: CTA b owns output tile tile0 + b
    Post post;             // per-channel epilogue of the stored values (all null: none)
    int* tickets;          // one counter per output tile (split mode), else nullptr
    float* part_val;       // [slots_cta][2][TILE_OUT]
    int* part_cid;         // [slots_cta][2][TILE_OUT]
    CUtensorMap tm_x, tm_w; // TMA loader only: x as [R][CI], w as [CO][CIg], boxes of (BK + 4) x 64 floats
};

__device__ __forceinline__ long long unit_begin(const TiledParams& p, int c) {
    long long total = (long long)p.tiles_m * p.tiles_n * p.G * p.KT;
    return total * c / p.n_cta;
}

// cp.async sources of one thread for the k-tiles of an output tile.  A thread always copies the
// same 16-byte column `ch` of the same rows (RPP rows apart) of x and of w; only k advances from
// tile to tile.  The row part of the address is worked out once per output tile and kept as a
// 32-bit element offset (tensors of the tiled path have fewer than 2^31 elements), so that a
// k-tile costs one add and one copy instruction per 16 bytes.
template <class GEO>
struct StageSrc {
    static constexpr int CH = GEO::BK / 4;             // 16-byte chunks per row
    static constexpr int RPP = GEO::NT / CH;           // rows per pass of the CTA
    static constexpr int PA = GEO::BM / RPP, PB = GEO::BN / RPP;
    unsigned a[PA], b[PB];                             // element offsets of (row, 4 * ch) in x and w
    int kin;                                           // 4 * ch: first k this thread copies in a tile
    int dst;                                           // float offset of (row0, ch) in a stage's A block
};

template <class GEO>
__device__ __forceinline__ StageSrc<GEO> stage_src(const TiledParams& p, int g, int m0, int n0, int tid) {
    StageSrc<GEO> s;
    const int row = tid / s.CH, ch = tid % s.CH;
    s.kin = 4 * ch;
    s.dst = row * GEO::LD + 4 * ch;
#pragma unroll
    for (int u = 0; u < s.PA; ++u)
        s.a[u] = (unsigned)min(m0 + row + u * s.RPP, p.M - 1) * (unsigned)p.lda + (unsigned)g * (unsigned)p.K + 4u * ch;
#pragma unroll
    for (int u = 0; u < s.PB; ++u)
        s.b[u] = ((unsigned)g * (unsigned)p.N + (unsigned)min(n0 + row + u * s.RPP, p.N - 1)) * (unsigned)p.K + 4u * ch;
    return s;
}

template <class GEO>
__device__ __forceinline__ void load_stage(float* stage, const TiledParams& p, const StageSrc<GEO>& s, int kt) {
    const int k0 = kt * GEO::BK;
    const bool in = k0 + s.kin < p.K;                  // past the end of the row: zero fill
    const unsigned kk = in ? (unsigned)k0 : 0u;
    const int bytes = in ? 16 : 0;
    float* As = stage + s.dst;
    float* Bs = As + GEO::BM * GEO::LD;
#pragma unroll
    for (int u = 0; u < s.PA; ++u) cp_async16(As + u * s.RPP * GEO::LD, p.x + (size_t)(s.a[u] + kk), bytes);
#pragma unroll
    for (int u = 0; u < s.PB; ++u) cp_async16(Bs + u * s.RPP * GEO::LD, p.w + (size_t)(s.b[u] + kk), bytes);
}

// Columns [4*K4B, 4*K4E) of one k-tile of the (max, |a-b|) product for the 8 x TN sub-tile of this
// thread.  `in` holds the running maxima before, `out` after (they may alias).
// Where the fragments of a thread lie in a stage.  Padded rows (cp.async loader, first TMA loader):
// row pitch LD = BK + 4 floats, chunk k4 of a row at k4 * 4.
template <class GEO>
struct FragPadded {
    const float* As; const float* Bs;     // first row of the thread's x / w fragments
    __device__ __forceinline__ ulonglong2 a(int i, int k4) const {
        return *reinterpret_cast<const ulonglong2*>(As + (4 * i) * GEO::LD + k4 * 4);
    }
    __device__ __forceinline__ ulonglong2 b(int j, int k4) const {
        return *reinterpret_cast<const ulonglong2*>(Bs + (8 * j) * GEO::LD + k4 * 4);
    }
};
__device__ __forceinline__ ulonglong2 lds128(unsigned addr) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(addr));
    return v;
}
// Swizzled rows (TMA loader with the 128-byte swizzle; BK = 32, rows of exactly 128 bytes): the copy
// engine stores 16-byte chunk c of row r at chunk position c ^ (r & 7).  The rows of a thread's x
// fragments are r = (multiple of 32) + lm + 4 * i, so r & 7 = lm | ((i & 1) << 2); those of its w fragments
// are r = (multiple of 8) + ln + 8 * j, so r & 7 = ln.  The run-time part of the exclusive-or is folded
// into four (x) and eight (w) base pointers per k-tile; everything else is a compile-time offset.
template <class GEO>
struct FragSwizzled {
    unsigned Aq[4], Bc[8];                 // shared-memory byte addresses
    __device__ __forceinline__ void set(const float* As, const float* Bs, int lm, int ln) {
        const unsigned a0 = (unsigned)__cvta_generic_to_shared(As), b0 = (unsigned)__cvta_generic_to_shared(Bs);
#pragma unroll
        for (int q = 0; q < 4; ++q) Aq[q] = a0 + ((unsigned)(q ^ lm) << 4);
#pragma unroll
        for (int c = 0; c < 8; ++c) Bc[c] = b0 + ((unsigned)(c ^ ln) << 4);
    }
    __device__ __forceinline__ ulonglong2 a(int i, int k4) const {
        return lds128(Aq[k4 & 3] + (unsigned)((4 * i) * 128 + ((((k4 >> 2) ^ (i & 1)) & 1) << 6)));
    }
    __device__ __forceinline__ ulonglong2 b(int j, int k4) const { return lds128(Bc[k4] + (unsigned)((8 * j) * 128)); }
};

template <class GEO, int K4B, int K4E, class FRAG>
__device__ __forceinline__ void tile_step(const FRAG& fr,
                                          const float (&in)[GEO::NOUT], float (&out)[GEO::NOUT]) {
    constexpr int TN = GEO::TN;
#pragma unroll
    for (int k4 = K4B; k4 < K4E; ++k4) {
        ulonglong2 bf[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j)
            bf[j] = fr.b(j, k4);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const ulonglong2 af = fr.a(i, k4);
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                float a = (k4 == K4B) ? in[i * TN + j] : out[i * TN + j];
                float t0, t1, t2, t3;
                unpack_f32x2(sub_f32x2(af.x, bf[j].x), t0, t1);
                unpack_f32x2(sub_f32x2(af.y, bf[j].y), t2, t3);
                a = max3(a, fabsf(t0), fabsf(t1));
                a = max3(a, fabsf(t2), fabsf(t3));
                out[i * TN + j] = a;
            }
        }
    }
}

// After a tracking window: every output whose maximum rose remembers the window number.  Two
// 16-bit window numbers share a register; `dup` holds the number in both halves.
template <int NOUT>
__device__ __forceinline__ void note_raises(const float (&before)[NOUT], const float (&after)[NOUT],
                                            unsigned (&cid)[NOUT / 2], unsigned dup) {
#pragma unroll
    for (int e = 0; e < NOUT; e += 2) {
        if (after[e] > before[e]) cid[e >> 1] = __byte_perm(cid[e >> 1], dup, 0x3254);
        if (after[e + 1] > before[e + 1]) cid[e >> 1] = __byte_perm(cid[e >> 1], dup, 0x7610);
    }
}

// The NSUB tracking windows of one k-tile, ping-ponging between the two accumulator sets; NSUB is
// even here, so the tile starts and ends in accA.
template <class GEO, int S, class FRAG>
__device__ __forceinline__ void tracked_windows(const FRAG& fr,
                                                float (&accA)[GEO::NOUT], float (&accB)[GEO::NOUT],
                                                unsigned (&cid)[GEO::NOUT / 2], unsigned win0) {
    if constexpr (S < GEO::NSUB) {
        constexpr int K4B = S * GEO::TW / 4, K4E = (S + 1) * GEO::TW / 4;
        const unsigned dup = (win0 + S) * 0x10001u;
        if constexpr ((S & 1) == 0) {
            tile_step<GEO, K4B, K4E>(fr, accA, accB);
            note_raises<GEO::NOUT>(accA, accB, cid, dup);
        } else {
            tile_step<GEO, K4B, K4E>(fr, accB, accA);
            note_raises<GEO::NOUT>(accB, accA, cid, dup);
        }
        tracked_windows<GEO, S + 1>(fr, accA, accB, cid, win0);
    }
}

template <int H>
__device__ __forceinline__ void cid_set(unsigned (&cid)[H], int e, unsigned v) {
    v &= 0xffffu;
    cid[e >> 1] = (e & 1) ? ((cid[e >> 1] & 0x0000ffffu) | (v << 16)) : ((cid[e >> 1] & 0xffff0000u) | v);
}

template <int H>
__device__ __forceinline__ int cid_get(const unsigned (&cid)[H], int e) {
    return (e & 1) ? (int)(cid[e >> 1] >> 16) : (int)(cid[e >> 1] & 0xffffu);
}

// Finds the first index in tracking window `win` (TW terms) whose |x - w| equals yv, and the sign
// there.  (A window that reaches past the end of a split segment is harmless: a match inside the
// segment comes first.)
template <int TW>
__device__ __forceinline__ int resolve_pos(const float* __restrict__ xrow, const float* __restrict__ wrow,
                                           int win, int K, float yv) {
    if (!(yv > 0.f)) return 0;
    const int kbase = win * TW;
    int best = 0;
    float tb = 0.f;
#pragma unroll
    for (int q = TW / 4 - 1; q >= 0; --q) {
        if (kbase + 4 * q < K) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xrow + kbase + 4 * q));
            const float4 wv = __ldg(reinterpret_cast<const float4*>(wrow + kbase + 4 * q));
            float t;
            t = xv.w - wv.w; if (fabsf(t) == yv) { best = 4 * q + 3; tb = t; }
            t = xv.z - wv.z; if (fabsf(t) == yv) { best = 4 * q + 2; tb = t; }
            t = xv.y - wv.y; if (fabsf(t) == yv) { best = 4 * q + 1; tb = t; }
            t = xv.x - wv.x; if (fabsf(t) == yv) { best = 4 * q + 0; tb = t; }
        }
    }
    return (kbase + best) | (tb < 0.f ? (int)0x80000000 : 0);
}

// ---- TMA loader (LOADER == 1) ---------------------------------------------------------------
// One thread per CTA issues two tiled bulk copies per k-tile: (BK + 4) x BM floats of x and
// (BK + 4) x BN floats of w.  The four extra columns are fetched only so that the rows land in
// shared memory with the same padded pitch the cp.async loader produces (conflict-free 128-bit
// fragment loads without a swizzle); out-of-range rows and columns arrive as zeros.  Completion is
// signalled on one mbarrier per stage; every wait is bounded: a thread that gives up sets
// g_tma_gave_up, marks the CTA dead (later waits return at once) and the launch finishes with
// meaningless results instead of hanging.
__device__ int g_tma_gave_up = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, int parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, int parity, volatile int* dead) {
    if (mbar_try_wait(bar, parity)) return;
    if (*dead) return;
    for (int spin = 0; spin < (1 << 20); ++spin)
        if (mbar_try_wait(bar, parity)) return;
    *dead = 1;
    atomicExch(&g_tma_gave_up, 1);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, int c0, int c1, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// One thread fills a stage: the x box at (column xc, row xr) and the w box at (column wc, row wr).
template <class GEO>
__device__ __forceinline__ void tma_stage(float* stage, unsigned long long* bar, const CUtensorMap* tm_x,
                                          const CUtensorMap* tm_w, int xc, int xr, int wc, int wr, int tid) {
    if (tid == 0) {
        mbar_expect_tx(bar, GEO::STAGE_FLOATS * 4);
        tma_load_2d(stage, tm_x, xc, xr, bar);
        tma_load_2d(stage + GEO::BM * GEO::LD, tm_w, wc, wr, bar);
    }
}

template <class GEO, bool TRACK, int LOADER>
__global__ void __launch_bounds__(GEO::NT, GEO::MINB)
inf_forward_tiled_kernel(const __grid_constant__ TiledParams p) {
    constexpr int NT = GEO::NT, TN = GEO::TN, NOUT = GEO::NOUT, BK = GEO::BK, TILE_OUT = GEO::TILE_OUT;
    constexpr int BM = GEO::BM, BN = GEO::BN, STAGES = GEO::STAGES, STAGE_FLOATS = GEO::STAGE_FLOATS;
    constexpr int NSUB = GEO::NSUB;
    constexpr int NB = TRACK ? NOUT : 2;        // size of the second accumulator set / window-number set
    extern __shared__ __align__(16) float smem_raw[];
    __shared__ int s_last;
    __shared__ int s_dead;
    __shared__ __align__(8) unsigned long long s_full[STAGES];   // TMA loader: "stage filled" barriers
    // TMA writes want a 128-byte aligned destination, swizzled ones (LOADER == 2) a 1024-byte aligned one
    // (the swizzle pattern repeats every eight 128-byte rows): the launcher reserves the bytes for the round-up
    constexpr uintptr_t ALIGN = LOADER == 2 ? 1024 : 128;
    float* smem = LOADER >= 1
        ? reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(smem_raw) + ALIGN - 1) & ~(ALIGN - 1)) : smem_raw;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if constexpr (LOADER >= 1) {
        if (tid == 0) {
            s_dead = 0;
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(&s_full[s], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }
    [[maybe_unused]] unsigned filled = 0;   // TMA loader: k-tiles consumed so far (stage = filled % STAGES, parity from filled / STAGES)
    const int wm = warp & 1, wn = warp >> 1, lm = lane >> 3, ln = lane & 7;
    const int row_off = wm * 32 + lm;            // + 4*i
    const int col_off = wn * (8 * TN) + ln;      // + 8*j

    const int tiles_per_group = p.tiles_m * p.tiles_n;
    // Work of this CTA, in units of one k-tile of one output tile.  Split mode (tickets set): an
    // even share of all units, whatever tiles it cuts through.  Whole mode: output tile
    // tile0 + blockIdx.x (the launcher gives every tile a CTA of its own: starting the CTAs of an SM
    // staggered so that their rescans do not coincide was measured and lost, 215 us against 207 us
    // at B = 512, Din = 784, Dout = 5120).
    const bool whole = p.tickets == nullptr;
    long long u = whole ? (long long)(p.tile0 + (int)blockIdx.x) * p.KT : unit_begin(p, blockIdx.x);
    const long long u_end = whole ? u + p.KT : unit_begin(p, blockIdx.x + 1);
    int seg = 0;

    // (Doing a CTA's partial segments first and its whole tiles last, so that the merges of cut tiles
    // happen early in the launch instead of behind every CTA's last k-tile, was measured and changed
    // nothing: 195 us either way in split mode at B = 512, Din = 784, Dout = 5120.)
    while (u < u_end) {
        const int tile = (int)(u / p.KT);
        const int kt0 = (int)(u - (long long)tile * p.KT);
        const int kt1 = whole ? p.KT : (int)min((long long)p.KT, kt0 + (u_end - u));
        const int g = tile / tiles_per_group;
        const int tg = tile - g * tiles_per_group;
        const int n0 = (tg / p.tiles_m) * BN, m0 = (tg % p.tiles_m) * BM;

        float accA[NOUT];
        float accB[NB];
        unsigned cid[NB / 2];
#pragma unroll
        for (int e = 0; e < NOUT; ++e) accA[e] = 0.f;
#pragma unroll
        for (int e = 0; e < NB / 2; ++e) cid[e] = (unsigned)(kt0 * NSUB) * 0x10001u;

        // ---- software pipeline over the k-tiles of this segment ----
        const StageSrc<GEO> src = stage_src<GEO>(p, g, m0, n0, tid);
        __syncthreads();   // previous segment is done with the ring
        int rd = 0, wr = STAGES - 1;
        if constexpr (LOADER >= 1) {
            // the ring position carries over from segment to segment (the barriers' phases depend on it)
            rd = (int)(filled % STAGES); wr = (rd + STAGES - 1) % STAGES;
        }
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if constexpr (LOADER == 0) {
                if (kt0 + s < kt1) load_stage<GEO>(smem + s * STAGE_FLOATS, p, src, kt0 + s);
                cp_async_commit();
            } else {
                if (kt0 + s < kt1) tma_stage<GEO>(smem + ((rd + s) % STAGES) * STAGE_FLOATS, &s_full[(rd + s) % STAGES],
                                                  &p.tm_x, &p.tm_w, g * p.K + (kt0 + s) * BK, m0, (kt0 + s) * BK, g * p.N + n0, tid);
            }
        }
        // consume one k-tile: wait for its stage, refill the stage freed by the previous k-tile
        auto next_stage = [&](int ktc) {
            if constexpr (LOADER == 0) {
                cp_async_wait<STAGES - 2>();
            } else {
                mbar_wait(&s_full[rd], (int)((filled / STAGES) & 1u), &s_dead);
                ++filled;
            }
            __syncthreads();   // every thread is done with the stage about to be refilled
            if constexpr (LOADER == 0) {
                if (ktc + STAGES - 1 < kt1) load_stage<GEO>(smem + wr * STAGE_FLOATS, p, src, ktc + STAGES - 1);
                cp_async_commit();
            } else {
                if (ktc + STAGES - 1 < kt1)
                    tma_stage<GEO>(smem + wr * STAGE_FLOATS, &s_full[wr], &p.tm_x, &p.tm_w,
                                   g * p.K + (ktc + STAGES - 1) * BK, m0, (ktc + STAGES - 1) * BK, g * p.N + n0, tid);
            }
        };
        auto advance = [&]() {
            rd = (rd + 1 == STAGES) ? 0 : rd + 1;
            wr = (wr + 1 == STAGES) ? 0 : wr + 1;
        };
        if constexpr (TRACK && NSUB > 1) {
            // several tracking windows per k-tile: every k-tile starts and ends in accA
            for (int kt = kt0; kt < kt1; ++kt) {
                next_stage(kt);
                const float* As = smem + rd * STAGE_FLOATS + row_off * GEO::LD;
                const float* Bs = smem + rd * STAGE_FLOATS + (BM + col_off) * GEO::LD;
                if constexpr (LOADER == 2) {
                    FragSwizzled<GEO> fr;
                    fr.set(As, Bs, lm, ln);
                    tracked_windows<GEO, 0>(fr, accA, accB, cid, (unsigned)(kt * NSUB));
                } else {
                    const FragPadded<GEO> fr{As, Bs};
                    tracked_windows<GEO, 0>(fr, accA, accB, cid, (unsigned)(kt * NSUB));
                }
                advance();
            }
        } else {
            // one tracking window per k-tile: two k-tiles per trip, accA -> accB -> accA
            for (int kt = kt0; kt < kt1; kt += 2) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int ktc = kt + h;
                    if (ktc < kt1) {
                        next_stage(ktc);
                        const float* As = smem + rd * STAGE_FLOATS + row_off * GEO::LD;
                        const float* Bs = smem + rd * STAGE_FLOATS + (BM + col_off) * GEO::LD;
                        auto body = [&](const auto& fr) {
                            if constexpr (TRACK) {
                                if (h == 0) {
                                    tile_step<GEO, 0, BK / 4>(fr, accA, accB);
                                    note_raises<NOUT>(accA, accB, cid, (unsigned)ktc * 0x10001u);
                                } else {
                                    tile_step<GEO, 0, BK / 4>(fr, accB, accA);
                                    note_raises<NOUT>(accB, accA, cid, (unsigned)ktc * 0x10001u);
                                }
                            } else {
                                tile_step<GEO, 0, BK / 4>(fr, accA, accA);
                            }
                        };
                        if constexpr (LOADER == 2) {
                            FragSwizzled<GEO> fr;
                            fr.set(As, Bs, lm, ln);
                            body(fr);
                        } else {
                            body(FragPadded<GEO>{As, Bs});
                        }
                        advance();
                    } else if (TRACK && h == 1) {
                        // the last k-tile ended in the second set
                        if constexpr (TRACK) {
#pragma unroll
                            for (int e = 0; e < NOUT; ++e) accA[e] = accB[e];
                        }
                    }
                }
            }
        }
        if constexpr (LOADER == 0) cp_async_wait<0>();

        // ---- finish the segment ----
        const bool complete = (kt0 == 0 && kt1 == p.KT);
        bool finish = complete;
        if (!complete) {
            // park the partial result, then take a ticket: the last arrival merges
            const size_t slot = ((size_t)blockIdx.x * 2 + (seg ? 1 : 0)) * TILE_OUT;
#pragma unroll
            for (int e = 0; e < NOUT; ++e) {
                p.part_val[slot + e * NT + tid] = accA[e];
                if constexpr (TRACK) p.part_cid[slot + e * NT + tid] = cid_get(cid, e);
            }
            __threadfence();
            __syncthreads();
            // CTAs that share this tile: consecutive block ids
            const long long t_begin = (long long)tile * p.KT, t_end = t_begin + p.KT;
            int c_lo = blockIdx.x, c_hi = blockIdx.x;
            while (c_lo > 0 && unit_begin(p, c_lo) > t_begin) --c_lo;
            while (c_hi + 1 < p.n_cta && unit_begin(p, c_hi + 1) < t_end) ++c_hi;
            if (tid == 0) {
                int old = atomicAdd(&p.tickets[tile], 1);
                int last = (old == c_hi - c_lo);
                if (last) p.tickets[tile] = 0;   // leave the counter clean for the next call
                s_last = last;
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                // Merge the parked partial results of the other CTAs of this tile into the
                // registers.  A partial from an EARLIER k-range wins ties (lowest index rule),
                // one from a LATER k-range must be strictly larger.
                for (int c = (int)blockIdx.x - 1; c >= c_lo; --c) {
                    const int s2 = ((int)(unit_begin(p, c) / p.KT) == tile) ? 0 : 1;
                    const size_t sl = ((size_t)c * 2 + s2) * TILE_OUT;
#pragma unroll
                    for (int e = 0; e < NOUT; ++e) {
                        const float v = __ldcg(p.part_val + sl + e * NT + tid);
                        if (v >= accA[e]) {
                            accA[e] = v;
                            if constexpr (TRACK) cid_set(cid, e, (unsigned)__ldcg(p.part_cid + sl + e * NT + tid));
                        }
                    }
                }
                for (int c = (int)blockIdx.x + 1; c <= c_hi; ++c) {
                    const size_t sl = ((size_t)c * 2 + 0) * TILE_OUT;   // always that CTA's first segment
#pragma unroll
                    for (int e = 0; e < NOUT; ++e) {
                        const float v = __ldcg(p.part_val + sl + e * NT + tid);
                        if (v > accA[e]) {
                            accA[e] = v;
                            if constexpr (TRACK) cid_set(cid, e, (unsigned)__ldcg(p.part_cid + sl + e * NT + tid));
                        }
                    }
                }
                finish = true;
            }
        }
        if (finish) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int m = m0 + row_off + 4 * i;
                if (m < p.M) {
                    const float* xrow = p.x + (size_t)m * p.lda + (size_t)g * p.K;
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        const int n = n0 + col_off + 8 * j;
                        if (n < p.N) {
                            const float yv = accA[i * TN + j];
                            const size_t o = (size_t)m * p.ldo + (size_t)g * p.N + n;
                            p.y[o] = post_apply(p.post, yv, g * p.N + n);
                            if constexpr (TRACK) {
                                const float* wrow = p.w + ((size_t)g * p.N + n) * p.K;
                                p.pos[o] = resolve_pos<GEO::TW>(xrow, wrow, cid_get(cid, i * TN + j), p.K, yv);
                            }
                        }
                    }
                }
            }
        }
        u += (long long)(kt1 - kt0);
        ++seg;   // only the first and the last segment of a CTA can be partial
    }
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// ---- variant table ------------------------------------------------------------------------
struct Kernels {
    int bm, bn, bk, nt, min_blocks, smem;
    void (*track)(const TiledParams);
    void (*plain)(const TiledParams);
};
struct Variant {
    Kernels main;      // 64 x 64 output tiles (8 x 4 outputs per thread), 3 CTAs per SM
    Kernels tail;      // 64 x 32 output tiles (8 x 2 outputs per thread) for a partial last wave
    int tma;           // 0: cp.async loader; 1: TMA, padded boxes; 2: TMA, 128-byte swizzle
    Kernels narrow;    // 64 x 48 output tiles (8 x 3 outputs per thread), 3 CTAs per SM, loader of `main`; nt == 0: none
    Kernels main_long, narrow_long;   // the same two with 16-term tracking windows, for long rows; nt == 0: none
};
constexpr Kernels kNoKernels{0, 0, 0, 0, 0, 0, nullptr, nullptr};

template <class GEO, int LOADER = 0>
constexpr Kernels make_kernels() {
    return Kernels{GEO::BM, GEO::BN, GEO::BK, GEO::NT, GEO::MINB, GEO::SMEM_BYTES + (LOADER == 1 ? 128 : LOADER == 2 ? 1024 : 0),
                   inf_forward_tiled_kernel<GEO, true, LOADER>, inf_forward_tiled_kernel<GEO, false, LOADER>};
}

// All variants: CTAs of 128 threads, 8 x 4 outputs per thread, 3 CTAs per SM.  Measured on one B200, us per
// forward with arg-max at B = 512, Dout = 5120 and Din = 784 / 1024 / 3072 / 5120 (whole 64 x 64 tiles + tail
// launch below 1536, k-split above), same box:
//   0: 196 / 238 / 592 / 942      1: 202 / 242 / 606 / 965      (0 with 4 stages: 200 / 239 / 600 / 950)
// and on another box   1: 192 / 230 / 596 / 954      2: 190 / 237 / 620 / 997      3: 204 / 247 / 611 / 962
// (variants 1-3 with the register budget of 4 CTAs per SM: 206-218 / 249-263 / 653-678 / 1022-1085).
// Variant 0 with 64 x 48 tiles (`narrow`, 149 registers, whole tiles, no tail): 178 / 217 / 584 / 951; the same
// with the register budget of 4 CTAs per SM (spills 108 bytes): 189 / 232 / 617 / 1004.
const Variant kVariants[] = {
    // 0: 32-term k-tiles fetched by TMA with the 128-byte swizzle (unpadded rows, 3 stages), 8-term windows (default)
    //    Rows of 2048 terms and more: 16-term windows (half the tracking instructions, a rescan of 128 instead of
    //    64 bytes per output): 565 / 907 us at Din = 3072 / 5120 against 586 / 952 us, 1081 against 1153 us at
    //    B = 256, Din = 12288; equal at Din = 1536, 8 % slower at Din = 784.  32-term windows lose everywhere
    //    (625 / 947 us; 257 us at Din = 784).
    {make_kernels<Geo<128, 4, 32, 3, 8, 0>, 2>(), make_kernels<Geo<128, 2, 32, 4, 8>>(), 2,
     make_kernels<Geo<128, 3, 32, 3, 8, 0>, 2>(),
     make_kernels<Geo<128, 4, 32, 3, 16, 0>, 2>(), make_kernels<Geo<128, 3, 32, 3, 16, 0>, 2>()},
    // 1: 32-term k-tiles (cp.async, 3 stages), 8-term tracking windows
    {make_kernels<Geo<128, 4, 32, 3, 8>>(), make_kernels<Geo<128, 2, 32, 4, 8>>(), 0, kNoKernels, kNoKernels, kNoKernels},
    // 2: 16-term k-tiles (cp.async, 4 stages), 8-term tracking windows
    {make_kernels<Geo<128, 4, 16, 3, 8>>(), make_kernels<Geo<128, 2, 16, 4, 8>>(), 0, kNoKernels, kNoKernels, kNoKernels},
    // 3: 16-term k-tiles, one tracking window per k-tile
    {make_kernels<Geo<128, 4, 16, 3, 16>>(), make_kernels<Geo<128, 2, 16, 4, 16>>(), 0, kNoKernels, kNoKernels, kNoKernels},
    // 4: as 3 with TMA and padded boxes (measured 7-14 % slower than 3: the extra four columns per row cost L2
    //    traffic)
    {make_kernels<Geo<128, 4, 16, 3, 16>, 1>(), make_kernels<Geo<128, 2, 16, 4, 16>>(), 1, kNoKernels, kNoKernels, kNoKernels},
};
constexpr int kLongRow = 2048;      // rows from this length on take the kernels with 16-term tracking windows
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);

}  // namespace

// Reads the flag a TMA-loader kernel sets when one of its bounded waits ran out (diagnostics only:
// synchronises the device).
int inf_forward_tma_gave_up() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tma_gave_up, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int inf_forward_variant = 0;   // index into kVariants (benchmarking knob)
int inf_forward_tail = 1;      // 1: a partial last wave runs as half-width tiles; 0: never
int inf_forward_split = 0;     // 0: k-splitting by the rule of make_plan; 1: whenever scratch is given; 2: never
int inf_forward_windows = 0;   // 0: 16-term tracking windows for long rows; 1: 8-term windows always (benchmarking knob)
int inf_forward_width = 0;     // 0: tile width by the rule of make_plan; 1: 64 columns always; 2: 48 wherever they exist

// Shapes the tiled path accepts (window numbers travel as 16 bits: at most 65535 windows per row).
static bool tiled_ok(const float* x, const float* w, const Dims& d) {
    return d.HW == 1 && (d.CIg % 4) == 0 && aligned16(x) && aligned16(w) &&
           d.COg >= 32 && (d.CIg + 7) / 8 < 65000 &&
           (size_t)d.R * d.CI < ((size_t)1 << 31) && (size_t)d.CO * d.CIg < ((size_t)1 << 31);
}

static const Variant& cur_variant() {
    int v = inf_forward_variant;
    return kVariants[(v >= 0 && v < kNumVariants) ? v : 0];
}

static int tiled_tiles(const Dims& d, const Kernels& k) {
    return ((d.R + k.bm - 1) / k.bm) * ((d.COg + k.bn - 1) / k.bn) * d.G;
}

// The TMA loader zero-fills past the END OF A ROW OF THE MATRIX.  With groups the k-tiles of one
// group are followed by the next group's columns, so a ragged last k-tile is only right for G = 1.
static bool tma_shape_ok(const Dims& d, int bk) { return (d.G == 1 || d.CIg % bk == 0) && d.CIg >= 32 && d.R >= 1; }

// How a shape is run: which tile geometry, whole tiles or k-tiles dealt evenly to the CTAs (scratch).
// A warp issues its subtract / max pairs every 5.5 cycles when it is alone on its scheduler and the
// scheduler one pair every 2.9 cycles when it has three or four warps, so what a wave of CTAs costs
// depends on how many CTAs share an SM and on the outputs per thread, not on how full the wave is.
// kWave: time of a wave with c CTAs per SM, in units of a full wave of 64 x 64 tiles (which takes
// about 12 + 0.115 * Din microseconds), fitted to measurements on one B200 over 21 shapes
// (B = 64 ... 2048, Din = 784 ... 12288, Dout = 512 ... 10240; the pick is within 4 % of the best of
// the three on all but one of them, 8 % there).  The k-split costs its share of a full wave plus
// 20 + 0.006 * Din microseconds for the parked partial results, the merge and an arg-max rescan that
// all CTAs reach at the same moment; it has to win by 3 %.
struct Plan { bool narrow, split; };

constexpr double kWaveMain[5] = {0, 0.387, 0.624, 1.0, 1.0};       // 8 x 4 outputs per thread, at most 3 CTAs per SM
constexpr double kWaveNarrow[5] = {0, 0.29, 0.468, 0.765, 0.765};  // 8 x 3
constexpr double kWaveTail[5] = {0, 0.22, 0.33, 0.60, 0.72};       // 8 x 2, at most 4 CTAs per SM, cp.async loader

static double waves_cost(int ctas, int per_sm, const double (&wave)[5]) {
    const int sms = sm_count(), slots = per_sm * sms;
    const int rest = ctas % slots;
    return (ctas / slots) * wave[per_sm] + (rest ? wave[(rest + sms - 1) / sms] : 0.0);
}

// CTAs of the tail launch that the launcher would use for this shape with 64 x 64 tiles (0: none),
// and the tiles left to the main launch.
static int tail_split(const Dims& d, const Variant& v, int* main_tiles) {
    const int tiles_m = (d.R + v.main.bm - 1) / v.main.bm;
    const int tiles = tiled_tiles(d, v.main), slots = v.main.min_blocks * sm_count();
    *main_tiles = tiles;
    if (inf_forward_tail == 0 || d.G != 1 || v.tail.bk != v.main.bk) return 0;
    const int cols_main = ((tiles / slots) * slots) / tiles_m;
    const int full = cols_main * tiles_m, rest = tiles - full;
    const int tail_ctas = ((d.COg + v.tail.bn - 1) / v.tail.bn - (v.main.bn / v.tail.bn) * cols_main) * tiles_m;
    if (!(rest > 0 && rest * 10 <= slots * 8 && tail_ctas > 0 && tail_ctas <= v.tail.min_blocks * sm_count())) return 0;
    *main_tiles = full;
    return tail_ctas;
}

static Plan make_plan(const Dims& d, const Variant& v, bool scratch) {
    const int slots = v.main.min_blocks * sm_count();
    const int tiles = tiled_tiles(d, v.main);
    const bool can_narrow = v.narrow.nt != 0 && inf_forward_width != 1 && d.COg >= v.narrow.bn &&
                            (v.tma == 0 || tma_shape_ok(d, v.narrow.bk));
    const bool can_split = scratch && inf_forward_split != 2;
    const double wave_us = 12.0 + 0.115 * d.CIg;
    int main_tiles;
    const int tail_ctas = tail_split(d, v, &main_tiles);
    double c_main = wave_us * (waves_cost(main_tiles, v.main.min_blocks, kWaveMain) +
                               (tail_ctas ? waves_cost(tail_ctas, v.tail.min_blocks, kWaveTail) : 0.0));
    double c_narrow = can_narrow ? wave_us * waves_cost(tiled_tiles(d, v.narrow), v.narrow.min_blocks, kWaveNarrow) : 1e30;
    double c_split = can_split ? 1.03 * (wave_us * tiles / slots + 20.0 + 0.006 * d.CIg) : 1e30;
    if (can_narrow && inf_forward_width == 2) c_narrow = 0.0;
    if (can_split && inf_forward_split == 1) c_split = -1.0;
    Plan pl;
    pl.split = c_split < c_main && c_split < c_narrow;
    pl.narrow = !pl.split && c_narrow < c_main;
    return pl;
}

size_t inf_forward_workspace(const Dims& d) {
    if (d.HW != 1 || (d.CIg % 4) != 0 || d.COg < 32) return 0;
    const Variant& v = cur_variant();
    if (!make_plan(d, v, true).split) return 0;
    const size_t n_cta = (size_t)v.main.min_blocks * sm_count();
    return align256((size_t)tiled_tiles(d, v.main) * sizeof(int)) +
           n_cta * 2 * v.main.bm * v.main.bn * (sizeof(float) + sizeof(int));
}

// ---- tensor maps for the TMA loader ----------------------------------------------------------
// cuTensorMapEncodeTiled is a host-only driver routine; it is looked up through the runtime so
// that the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tma_encoder() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// A row-major fp32 matrix [rows][cols] with `pitch` floats between rows, fetched in boxes of
// box_cols x box_rows.  The rules of the copy engine: base and pitch multiples of 16 bytes, box
// width a multiple of 16 bytes; the kernel only ever starts a box at a column that is a multiple
// of 16 floats.
static bool tma_matrix(const float* base, size_t rows, size_t cols, size_t pitch, int box_cols, int box_rows,
                       CUtensorMap* out, bool swizzle128 = false) {
    EncodeTiledFn fn = tma_encoder();
    if (fn == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) || (pitch & 3u) || (box_cols & 3)) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int launch_tiled(const Kernels& k, const TiledParams& p, bool track, cudaStream_t st) {
    auto kern = track ? k.track : k.plain;
    // opting in to > 48 KB of dynamic shared memory is per function and per device; it is cheap
    // enough to repeat on every call and keeps the library free of mutable global state
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    kern<<<p.n_cta, k.nt, k.smem, st>>>(p);
    return launch_status();
}

int inf_forward(const float* x, const float* w, const Dims& d, float* y, int* pos,
                void* ws, size_t ws_bytes, cudaStream_t st, const Post& post) {
    if (!tiled_ok(x, w, d)) {
        if (skinny_ok(d, x, w, nullptr)) return inf_forward_skinny(x, w, d, y, pos, st, post);
        dim3 grid((d.R + GT - 1) / GT, (d.COg + GT - 1) / GT, d.G);
        if (grid.y > 65535u || grid.z > 65535u) return LINF_ERR_DIMS;
        if (d.HW > 1) inf_forward_generic_kernel<true><<<grid, 256, 0, st>>>(x, w, d, y, pos, post);
        else inf_forward_generic_kernel<false><<<grid, 256, 0, st>>>(x, w, d, y, pos, post);
        return launch_status();
    }
    const Variant& v = cur_variant();
    const size_t need = inf_forward_workspace(d);
    const bool scratch = ws != nullptr && need != 0;
    if (scratch && (ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u))) return LINF_ERR_WORKSPACE;
    Plan plan = make_plan(d, v, scratch);
    TiledParams p;
    p.x = x; p.w = w; p.y = y; p.pos = pos;
    p.M = d.R; p.N = d.COg; p.K = d.CIg; p.G = d.G;
    p.lda = d.CI; p.ldo = d.CO;
    // (not with the k-split: 430 against 416 us at B = 512, Din = 5120, Dout = 2048, 311 against 291 us at B = 128)
    const bool long_rows = d.CIg >= kLongRow && v.main_long.nt != 0 && inf_forward_windows != 1 && !plan.split;
    const Kernels* use = plan.narrow ? (long_rows ? &v.narrow_long : &v.narrow) : (long_rows ? &v.main_long : &v.main);
    if (v.tma) {
        const int pad = v.tma == 1 ? 4 : 0;
        const bool ok = tma_shape_ok(d, use->bk) &&
                        tma_matrix(x, (size_t)d.R, (size_t)d.CI, (size_t)d.CI, use->bk + pad, use->bm, &p.tm_x, v.tma == 2) &&
                        tma_matrix(w, (size_t)d.CO, (size_t)d.CIg, (size_t)d.CIg, use->bk + pad, use->bn, &p.tm_w, v.tma == 2);
        if (!ok) {      // 64 x 64 tiles with the cp.async loader
            use = &kVariants[v.tma == 1 ? 3 : 1].main;
            plan.narrow = false;
        }
    }
    p.tiles_m = (d.R + use->bm - 1) / use->bm; p.tiles_n = (d.COg + use->bn - 1) / use->bn;
    p.KT = (d.CIg + use->bk - 1) / use->bk;
    const int tiles = p.tiles_m * p.tiles_n * d.G;
    p.tickets = nullptr; p.part_val = nullptr; p.part_cid = nullptr;
    p.n_cta = tiles;       // whole mode: one CTA per output tile
    p.slots_cta = 0;
    p.tile0 = 0;
    p.post = post;
    const int slots = use->min_blocks * sm_count();
    if (plan.split) {
        const size_t tick_bytes = align256((size_t)tiles * sizeof(int));
        const long long total = (long long)tiles * p.KT;
        p.slots_cta = slots;
        p.n_cta = (int)min((long long)p.slots_cta, total);
        p.tickets = reinterpret_cast<int*>(ws);
        p.part_val = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + tick_bytes);
        p.part_cid = reinterpret_cast<int*>(p.part_val + (size_t)p.slots_cta * 2 * use->bm * use->bn);
        if (cudaMemsetAsync(p.tickets, 0, tick_bytes, st) != cudaSuccess) return LINF_ERR_LAUNCH;
    }
    // Whole tiles that end in a partial wave of CTAs (or never fill one): the columns of that
    // partial wave are run as tiles of half the width by the tail kernels, twice as many CTAs.
    // Only whole columns of tiles change hands, so the two launches cover disjoint column ranges.
    if (p.tickets == nullptr && !plan.narrow) {
        int full;
        const int tail_ctas = tail_split(d, v, &full);
        if (tail_ctas > 0 && v.tail.bk == use->bk) {
            int rc = LINF_OK;
            if (full > 0) {
                p.n_cta = full;
                rc = launch_tiled(*use, p, pos != nullptr, st);
                if (rc) return rc;
            }
            TiledParams q = p;
            q.tiles_n = (d.COg + v.tail.bn - 1) / v.tail.bn;
            q.tile0 = (use->bn / v.tail.bn) * full;     // whole tile columns changed hands: tile index scales with the width
            q.n_cta = tail_ctas;
            return launch_tiled(v.tail, q, pos != nullptr, st);
        }
    }
    return launch_tiled(*use, p, pos != nullptr, st);
}

}  // namespace linf
