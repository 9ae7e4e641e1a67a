// L_p-distance neuron for finite p > 1.
//
//   forward   y = M * (sum_i (|x_i - w_i| / M)^p)^(1/p),  M = max_i |x_i - w_i|
//   backward  T[r,o,i] = g[r,o] * (|t| / y[r,o])^(p-1) * sign(t),  t = x[r,i] - w[o,i]
//             grad_x[r,i] = sum_o T,   grad_w[o,i] = -sum_r T
//
// Powers.  Every base u = |t| / M (or |t| / y) lies in [0, 1].  The exponent q is split as
// q = n + f with integer n and 0 <= f < 1: u^n comes from square-and-multiply on the FP32
// pipe (the loop is uniform: q is a launch constant), u^f from one log2/exp2 pair on the
// special-function unit and only when f != 0.  The approximation error of log2 is thereby
// multiplied by f < 1 instead of by q, which keeps the gradients of p = 64 ... 1000 within a
// few ulp of correctly rounded arithmetic; integer p (the common test points 8, 16, 64) never
// touches the special-function unit at all.
//
// Forward normalisation.  M is produced first by the inf-dist forward kernel (value-only mode)
// straight into `output`; the power-sum kernel reads it from there and overwrites it with y.
#include <math.h>

#include "common.cuh"

namespace linf {
namespace {

struct PowPlan {
    int n;      // integer part of the exponent
    float f;    // fractional part, 0 <= f < 1
};

inline PowPlan make_plan(float q) {
    PowPlan pl;
    float fl = floorf(q);
    pl.n = (int)fl;
    pl.f = q - fl;
    return pl;
}

// u^(n+f) for 0 <= u <= 1 (u = 0 gives 0 because n >= 1 on every path that calls this).
__device__ __forceinline__ float pow_unit(float u, const PowPlan pl) {
    float r = 1.f, b = u;
    for (int n = pl.n; n != 0; n >>= 1) {
        if (n & 1) r *= b;
        b *= b;
    }
    if (pl.f != 0.f) r *= exp2f(pl.f * __log2f(u));   // u = 0: exp2(-inf) = 0
    return r;
}

constexpr int GT = 32;

// ---- forward: y holds M on entry, the L_p distance on exit ---------------------------------
template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
lp_forward_generic_kernel(const float* __restrict__ x, const float* __restrict__ w, Dims d,
                          float* __restrict__ y, PowPlan pl, float inv_p) {
    __shared__ float xs[GT][GT + 1], ws[GT][GT + 1];
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int g = blockIdx.z, r0 = blockIdx.x * GT, c0 = blockIdx.y * GT;
    const int c = c0 + tx;

    float M[4], rM[4], S[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int r = r0 + ty + 8 * j;
        M[j] = (r < d.R && c < d.COg) ? y[act_index(r, g, c, d.COg, d.G, d.HW)] : 0.f;
        rM[j] = M[j] > 0.f ? 1.f / M[j] : 0.f;
        S[j] = 0.f;
    }
    for (int k0 = 0; k0 < d.CIg; k0 += GT) {
        for (int e = tid; e < GT * GT; e += 256) {
            int kl, rl;
            if (ROW_FAST) { rl = e & 31; kl = e >> 5; } else { kl = e & 31; rl = e >> 5; }
            int r = r0 + rl, k = k0 + kl;
            xs[kl][rl] = (r < d.R && k < d.CIg) ? x[act_index(r, g, k, d.CIg, d.G, d.HW)] : 0.f;
            int kw = e & 31, cl = e >> 5, cc = c0 + cl, k2 = k0 + kw;
            ws[kw][cl] = (cc < d.COg && k2 < d.CIg) ? w[(size_t)(g * d.COg + cc) * d.CIg + k2] : 0.f;
        }
        __syncthreads();
        const int kmax = min(GT, d.CIg - k0);
        for (int kk = 0; kk < kmax; ++kk) {
            const float wv = ws[kk][tx];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float u = fminf(fabsf(xs[kk][ty + 8 * j] - wv) * rM[j], 1.f);
                S[j] += pow_unit(u, pl);
            }
        }
        __syncthreads();
    }
    if (c < d.COg) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int r = r0 + ty + 8 * j;
            if (r < d.R) y[act_index(r, g, c, d.COg, d.G, d.HW)] = M[j] > 0.f ? powf(S[j], inv_p) * M[j] : 0.f;
        }
    }
}

// ---- forward for very few outputs per group (the 5120 -> 10 classifier layer) ------------------
// The 32 x 32 tiles above would give a handful of CTAs that each walk all of K alone (2.3 ms at
// B = 512, K = 5120, 10 outputs).  As in the inf-dist kernel for such layers the reduction dimension is
// spread over the threads of a CTA that owns R rows: thread t walks the 16-byte chunks t, t + 256, ...
// of those rows and of every weight row; the partial sums are added over the lanes by a butterfly and
// over the warps in warp order (a fixed order: same bits on every run).
template <int NMAX, int R>
__global__ void __launch_bounds__(256)
lp_forward_skinny_kernel(const float* __restrict__ x, const float* __restrict__ w, Dims d,
                         float* __restrict__ y, PowPlan pl, float inv_p) {
    __shared__ float s_s[8][R][NMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
    const int N = d.COg, K = d.CIg;
    const int row_blocks = (d.R + R - 1) / R;
    const int g = blockIdx.x / row_blocks, r0 = (blockIdx.x - g * row_blocks) * R;
    float S[R][NMAX], rM[R][NMAX];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            const float M = (n < N) ? y[(size_t)min(r0 + r, d.R - 1) * d.CO + (size_t)g * N + n] : 0.f;
            rM[r][n] = M > 0.f ? 1.f / M : 0.f;
            S[r][n] = 0.f;
        }
    const float* xr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) xr[r] = x + (size_t)min(r0 + r, d.R - 1) * d.CI + (size_t)g * K;
    const float* wg = w + (size_t)g * N * K;
    for (int k = threadIdx.x * 4; k < K; k += 4 * blockDim.x) {
        float4 xv[R];
#pragma unroll
        for (int r = 0; r < R; ++r) xv[r] = __ldg(reinterpret_cast<const float4*>(xr[r] + k));
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                const float4 wv = __ldg(reinterpret_cast<const float4*>(wg + (size_t)n * K + k));
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float m = rM[r][n];
                    float a = S[r][n];
                    a += pow_unit(fminf(fabsf(xv[r].x - wv.x) * m, 1.f), pl);
                    a += pow_unit(fminf(fabsf(xv[r].y - wv.y) * m, 1.f), pl);
                    a += pow_unit(fminf(fabsf(xv[r].z - wv.z) * m, 1.f), pl);
                    a += pow_unit(fminf(fabsf(xv[r].w - wv.w) * m, 1.f), pl);
                    S[r][n] = a;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                float a = S[r][n];
#pragma unroll
                for (int sft = 16; sft >= 1; sft >>= 1) a += __shfl_xor_sync(0xffffffffu, a, sft);
                if (lane == 0) s_s[warp][r][n] = a;
            }
        }
    __syncthreads();
    for (int q = threadIdx.x; q < R * NMAX; q += blockDim.x) {
        const int r = q / NMAX, n = q % NMAX;
        if (n < N && r0 + r < d.R) {
            float a = s_s[0][r][n];
            for (int wv = 1; wv < wpc; ++wv) a += s_s[wv][r][n];
            float* yo = y + (size_t)(r0 + r) * d.CO + (size_t)g * N + n;
            const float M = *yo;
            *yo = M > 0.f ? powf(a, inv_p) * M : 0.f;
        }
    }
}

// ---- backward w.r.t. the weight for very few outputs per group --------------------------------
// A CTA owns 32 input channels (one per lane) and all N outputs; its 8 warps share the batch rows
// (warp w takes rows w, w + 8, ...), the partial sums are added in warp order.  The 32 x 32 tiles of the
// generic kernel leave 160 CTAs walking all rows alone (265 us at B = 512, K = 5120, 10 outputs).
template <int NMAX>
__global__ void __launch_bounds__(256)
lp_backward_weight_skinny_kernel(const float* __restrict__ gout, const float* __restrict__ x,
                                 const float* __restrict__ w, const float* __restrict__ y, Dims d,
                                 float* __restrict__ gw, PowPlan pl) {
    __shared__ float part[8][NMAX][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int N = d.COg, K = d.CIg, g = blockIdx.y;
    const int i = blockIdx.x * 32 + lane;
    const bool in = i < K;
    float wv[NMAX], acc[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
        wv[n] = (n < N && in) ? w[(size_t)(g * N + n) * K + i] : 0.f;
        acc[n] = 0.f;
    }
    for (int b = warp; b < d.R; b += 8) {
        const float xv = in ? __ldg(x + (size_t)b * d.CI + (size_t)g * K + i) : 0.f;
        const float* gr = gout + (size_t)b * d.CO + (size_t)g * N;
        const float* yr = y + (size_t)b * d.CO + (size_t)g * N;
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                const float yv = __ldg(yr + n);
                const float ry = yv > 0.f ? 1.f / yv : 0.f;
                const float t = wv[n] - xv;
                const float term = __ldg(gr + n) * pow_unit(fminf(fabsf(t) * ry, 1.f), pl);
                acc[n] += (t > 0.f) ? term : -term;
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NMAX; ++n) part[warp][n][lane] = acc[n];
    __syncthreads();
    for (int q = threadIdx.x; q < NMAX * 32; q += 256) {
        const int n = q >> 5, l = q & 31, ii = blockIdx.x * 32 + l;
        if (n < N && ii < K) {
            float a = part[0][n][l];
#pragma unroll
            for (int wv2 = 1; wv2 < 8; ++wv2) a += part[wv2][n][l];
            gw[(size_t)(g * N + n) * K + ii] = a;
        }
    }
}

template <int NMAX, int R>
int launch_lp_skinny(const float* x, const float* w, const Dims& d, float* y, float p, cudaStream_t st) {
    const int items = ((d.R + R - 1) / R) * d.G;
    const int wpc = min(8, max(1, d.CIg / 512));
    lp_forward_skinny_kernel<NMAX, R><<<items, 32 * wpc, 0, st>>>(x, w, d, y, make_plan(p), 1.f / p);
    return launch_status();
}

// ---- backward w.r.t. the input: tile = 32 rows x 32 input channels, loop over outputs -------
template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
lp_backward_input_generic_kernel(const float* __restrict__ gout, const float* __restrict__ x,
                                 const float* __restrict__ w, const float* __restrict__ y, Dims d,
                                 float* __restrict__ gx, PowPlan pl) {
    __shared__ float gs[GT][GT + 1], ys[GT][GT + 1], ws[GT][GT + 1];   // [o][row], [o][row], [o][i]
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int g = blockIdx.z, r0 = blockIdx.x * GT, i0 = blockIdx.y * GT;
    const int i = i0 + tx;

    float xv[4], acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int r = r0 + ty + 8 * j;
        xv[j] = (r < d.R && i < d.CIg) ? x[act_index(r, g, i, d.CIg, d.G, d.HW)] : 0.f;
        acc[j] = 0.f;
    }
    for (int o0 = 0; o0 < d.COg; o0 += GT) {
        for (int e = tid; e < GT * GT; e += 256) {
            int ol, rl;
            if (ROW_FAST) { rl = e & 31; ol = e >> 5; } else { ol = e & 31; rl = e >> 5; }
            int r = r0 + rl, o = o0 + ol;
            bool in = r < d.R && o < d.COg;
            size_t a = in ? act_index(r, g, o, d.COg, d.G, d.HW) : 0;
            float yv = in ? y[a] : 0.f;
            gs[ol][rl] = in ? gout[a] : 0.f;
            ys[ol][rl] = yv > 0.f ? 1.f / yv : 0.f;
            int il = e & 31, ow = e >> 5, ii = i0 + il, oo = o0 + ow;
            ws[ow][il] = (ii < d.CIg && oo < d.COg) ? w[(size_t)(g * d.COg + oo) * d.CIg + ii] : 0.f;
        }
        __syncthreads();
        const int omax = min(GT, d.COg - o0);
        for (int oo = 0; oo < omax; ++oo) {
            const float wv = ws[oo][tx];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t = xv[j] - wv;
                float u = fminf(fabsf(t) * ys[oo][ty + 8 * j], 1.f);
                float term = gs[oo][ty + 8 * j] * pow_unit(u, pl);
                acc[j] += (t > 0.f) ? term : -term;
            }
        }
        __syncthreads();
    }
    if (i < d.CIg) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int r = r0 + ty + 8 * j;
            if (r < d.R) gx[act_index(r, g, i, d.CIg, d.G, d.HW)] = acc[j];
        }
    }
}

// ---- backward w.r.t. the weight: tile = 32 outputs x 32 input channels, loop over rows ------
template <bool ROW_FAST>
__global__ void __launch_bounds__(256)
lp_backward_weight_generic_kernel(const float* __restrict__ gout, const float* __restrict__ x,
                                  const float* __restrict__ w, const float* __restrict__ y, Dims d,
                                  float* __restrict__ gw, PowPlan pl) {
    __shared__ float gs[GT][GT + 1], ys[GT][GT + 1], xs[GT][GT + 1];   // [row][o], [row][o], [row][i]
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int g = blockIdx.z, o0 = blockIdx.x * GT, i0 = blockIdx.y * GT;
    const int i = i0 + tx;

    float wv[4], acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int o = o0 + ty + 8 * j;
        wv[j] = (o < d.COg && i < d.CIg) ? w[(size_t)(g * d.COg + o) * d.CIg + i] : 0.f;
        acc[j] = 0.f;
    }
    for (int rb = 0; rb < d.R; rb += GT) {
        for (int e = tid; e < GT * GT; e += 256) {
            {   // grad_output / output tile [row][o]
                int ol, rl;
                if (ROW_FAST) { rl = e & 31; ol = e >> 5; } else { ol = e & 31; rl = e >> 5; }
                int r = rb + rl, o = o0 + ol;
                bool in = r < d.R && o < d.COg;
                size_t a = in ? act_index(r, g, o, d.COg, d.G, d.HW) : 0;
                float yv = in ? y[a] : 0.f;
                gs[rl][ol] = in ? gout[a] : 0.f;
                ys[rl][ol] = yv > 0.f ? 1.f / yv : 0.f;
            }
            {   // input tile [row][i]
                int il, rl;
                if (ROW_FAST) { rl = e & 31; il = e >> 5; } else { il = e & 31; rl = e >> 5; }
                int r = rb + rl, ii = i0 + il;
                xs[rl][il] = (r < d.R && ii < d.CIg) ? x[act_index(r, g, ii, d.CIg, d.G, d.HW)] : 0.f;
            }
        }
        __syncthreads();
        const int rmax = min(GT, d.R - rb);
        for (int rr = 0; rr < rmax; ++rr) {
            const float xvv = xs[rr][tx];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t = wv[j] - xvv;
                float u = fminf(fabsf(t) * ys[rr][ty + 8 * j], 1.f);
                float term = gs[rr][ty + 8 * j] * pow_unit(u, pl);
                acc[j] += (t > 0.f) ? term : -term;
            }
        }
        __syncthreads();
    }
    if (i < d.CIg) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int o = o0 + ty + 8 * j;
            if (o < d.COg) gw[(size_t)(g * d.COg + o) * d.CIg + i] = acc[j];
        }
    }
}

bool grid_ok(const dim3& g) { return g.y <= 65535u && g.z <= 65535u; }

}  // namespace

int lp_forward(const float* x, const float* w, const Dims& d, float* y, float p, cudaStream_t st) {
    int rc = inf_forward(x, w, d, y, nullptr, nullptr, 0, st);
    if (rc != LINF_OK) return rc;
    if (lp_tiled_ok(d, x, w, y, nullptr, nullptr)) return lp_forward_tiled(x, w, d, y, p, st);
    if (skinny_ok(d, x, w, nullptr)) {
        if (d.COg <= 4) return launch_lp_skinny<4, 4>(x, w, d, y, p, st);
        if (d.COg <= 8) return launch_lp_skinny<8, 2>(x, w, d, y, p, st);
        if (d.COg <= 16) return launch_lp_skinny<16, 2>(x, w, d, y, p, st);
        return launch_lp_skinny<32, 1>(x, w, d, y, p, st);
    }
    dim3 grid((d.R + GT - 1) / GT, (d.COg + GT - 1) / GT, d.G);
    if (!grid_ok(grid)) return LINF_ERR_DIMS;
    const PowPlan pl = make_plan(p);
    const float inv_p = 1.f / p;
    if (d.HW > 1) lp_forward_generic_kernel<true><<<grid, 256, 0, st>>>(x, w, d, y, pl, inv_p);
    else lp_forward_generic_kernel<false><<<grid, 256, 0, st>>>(x, w, d, y, pl, inv_p);
    return launch_status();
}

int lp_backward_input(const float* g, const float* x, const float* w, const float* y,
                      const Dims& d, float* gx, float p, cudaStream_t st) {
    if (lp_tiled_ok(d, x, w, y, g, gx)) {
        const int rc = lp_backward_tiled(g, x, w, y, d, gx, p, false, st);
        if (rc >= 0) return rc;             // negative: exponent beyond the tiled instantiations
    }
    dim3 grid((d.R + GT - 1) / GT, (d.CIg + GT - 1) / GT, d.G);
    if (!grid_ok(grid)) return LINF_ERR_DIMS;
    const PowPlan pl = make_plan(p - 1.f);
    if (d.HW > 1) lp_backward_input_generic_kernel<true><<<grid, 256, 0, st>>>(g, x, w, y, d, gx, pl);
    else lp_backward_input_generic_kernel<false><<<grid, 256, 0, st>>>(g, x, w, y, d, gx, pl);
    return launch_status();
}

int lp_backward_weight(const float* g, const float* x, const float* w, const float* y,
                       const Dims& d, float* gw, float p, cudaStream_t st) {
    if (lp_tiled_ok(d, x, w, y, g, gw)) {
        const int rc = lp_backward_tiled(g, x, w, y, d, gw, p, true, st);
        if (rc >= 0) return rc;
    }
    if (skinny_ok(d, x, w, nullptr) && d.G <= 65535) {
        const dim3 sg((d.CIg + 31) / 32, d.G);
        const PowPlan spl = make_plan(p - 1.f);
        if (d.COg <= 16) lp_backward_weight_skinny_kernel<16><<<sg, 256, 0, st>>>(g, x, w, y, d, gw, spl);
        else lp_backward_weight_skinny_kernel<32><<<sg, 256, 0, st>>>(g, x, w, y, d, gw, spl);
        return launch_status();
    }
    dim3 grid((d.COg + GT - 1) / GT, (d.CIg + GT - 1) / GT, d.G);
    if (!grid_ok(grid)) return LINF_ERR_DIMS;
    const PowPlan pl = make_plan(p - 1.f);
    if (d.HW > 1) lp_backward_weight_generic_kernel<true><<<grid, 256, 0, st>>>(g, x, w, y, d, gw, pl);
    else lp_backward_weight_generic_kernel<false><<<grid, 256, 0, st>>>(g, x, w, y, d, gw, pl);
    return launch_status();
}

}  // namespace linf
