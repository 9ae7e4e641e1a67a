// Dense layers with very few output channels per group (the 5120 -> 10 classifier layer): the
// 64 x 64 output tiles of the tiled kernels would be almost empty and there are too few of them to
// fill the GPU, so the reduction dimension is spread over the threads of a CTA instead.  A CTA owns
// R input rows; thread t walks the 16-byte chunks t, t+256, ... of those rows and of every weight
// row, keeps its running best per output in registers; a butterfly over the lanes and a pass over
// the warps through shared memory merge them (larger |t| wins, equal |t| goes to the lower index
// -- the reference's tie rule).
// Needs HW == 1, CI/G a multiple of 4 and 16-byte aligned rows; memory-bound (the input is read
// once, the small weight matrix stays in L1/L2).
#include "common.cuh"

namespace linf {
namespace {

constexpr unsigned FULL = 0xffffffffu;

template <int NMAX, int R>
__global__ void __launch_bounds__(256)
inf_forward_skinny_kernel(const float* __restrict__ x, const float* __restrict__ w, Dims d,
                          float* __restrict__ y, int* __restrict__ pos, Post post) {
    __shared__ float s_t[8][R][NMAX];
    __shared__ int s_i[8][R][NMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    const int N = d.COg, K = d.CIg;
    // work item = (group, block of R rows), one CTA each
    const int row_blocks = (d.R + R - 1) / R;
    const int item = blockIdx.x;
    const int g = item / row_blocks, r0 = (item - g * row_blocks) * R;

    float tb[R][NMAX];      // signed difference of the best term so far
    int ib[R][NMAX];        // its index
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) { tb[r][n] = 0.f; ib[r][n] = 0; }

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
                    float t;
                    t = xv[r].x - wv.x; if (fabsf(t) > fabsf(tb[r][n])) { tb[r][n] = t; ib[r][n] = k; }
                    t = xv[r].y - wv.y; if (fabsf(t) > fabsf(tb[r][n])) { tb[r][n] = t; ib[r][n] = k + 1; }
                    t = xv[r].z - wv.z; if (fabsf(t) > fabsf(tb[r][n])) { tb[r][n] = t; ib[r][n] = k + 2; }
                    t = xv[r].w - wv.w; if (fabsf(t) > fabsf(tb[r][n])) { tb[r][n] = t; ib[r][n] = k + 3; }
                }
            }
        }
    }
    // merge the lanes: larger magnitude wins, equal magnitudes go to the lower index
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                float t = tb[r][n]; int i = ib[r][n];
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) {
                    const float t2 = __shfl_xor_sync(FULL, t, s);
                    const int i2 = __shfl_xor_sync(FULL, i, s);
                    const float a = fabsf(t), a2 = fabsf(t2);
                    if (a2 > a || (a2 == a && i2 < i)) { t = t2; i = i2; }
                }
                if (lane == 0) { s_t[warp][r][n] = t; s_i[warp][r][n] = i; }
            }
        }
    __syncthreads();
    for (int q = threadIdx.x; q < R * NMAX; q += blockDim.x) {
        const int r = q / NMAX, n = q % NMAX;
        if (n < N && r0 + r < d.R) {
            float t = s_t[0][r][n]; int i = s_i[0][r][n];
            for (int wv = 1; wv < wpc; ++wv) {
                const float t2 = s_t[wv][r][n]; const int i2 = s_i[wv][r][n];
                const float a = fabsf(t), a2 = fabsf(t2);
                if (a2 > a || (a2 == a && i2 < i)) { t = t2; i = i2; }
            }
            const size_t o = (size_t)(r0 + r) * d.CO + (size_t)g * N + n;
            const float yv = fabsf(t);
            y[o] = post_apply(post, yv, g * N + n);
            if (pos) pos[o] = (yv > 0.f) ? (i | (t < 0.f ? (int)0x80000000 : 0)) : 0;
        }
    }
}

// Interval bounds, literal rule (model/inf_dist_cuda.cu:106-110): max / min are order independent.
template <int NMAX, int R>
__global__ void __launch_bounds__(256)
inf_bound_skinny_kernel(const float* __restrict__ xl, const float* __restrict__ xu,
                        const float* __restrict__ w, Dims d, float* __restrict__ yl, float* __restrict__ yu, Post post) {
    __shared__ float s_l[8][R][NMAX], s_u[8][R][NMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    const int N = d.COg, K = d.CIg;
    const int row_blocks = (d.R + R - 1) / R;
    const int item = blockIdx.x;
    const int g = item / row_blocks, r0 = (item - g * row_blocks) * R;

    float L[R][NMAX], U[R][NMAX];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) { L[r][n] = 0.f; U[r][n] = 0.f; }
    size_t xo[R];
#pragma unroll
    for (int r = 0; r < R; ++r) xo[r] = (size_t)min(r0 + r, d.R - 1) * d.CI + (size_t)g * K;
    const float* wg = w + (size_t)g * N * K;

    auto term = [](float lo, float up, float wv, float& Lr, float& Ur) {
        const float tL = lo - wv, tU = up - wv;
        const float aL = fabsf(tL), aU = fabsf(tU);
        Ur = fmaxf(Ur, fmaxf(aL, aU));
        if (!(tL < 0.f && tU > 0.f)) Lr = fmaxf(Lr, fminf(aL, aU));
    };
    for (int k = threadIdx.x * 4; k < K; k += 4 * blockDim.x) {
        float4 lo[R], up[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            lo[r] = __ldg(reinterpret_cast<const float4*>(xl + xo[r] + k));
            up[r] = __ldg(reinterpret_cast<const float4*>(xu + xo[r] + k));
        }
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                const float4 wv = __ldg(reinterpret_cast<const float4*>(wg + (size_t)n * K + k));
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    term(lo[r].x, up[r].x, wv.x, L[r][n], U[r][n]);
                    term(lo[r].y, up[r].y, wv.y, L[r][n], U[r][n]);
                    term(lo[r].z, up[r].z, wv.z, L[r][n], U[r][n]);
                    term(lo[r].w, up[r].w, wv.w, L[r][n], U[r][n]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
            if (n < N) {
                float l = L[r][n], u = U[r][n];
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) {
                    l = fmaxf(l, __shfl_xor_sync(FULL, l, s));
                    u = fmaxf(u, __shfl_xor_sync(FULL, u, s));
                }
                if (lane == 0) { s_l[warp][r][n] = l; s_u[warp][r][n] = u; }
            }
        }
    __syncthreads();
    for (int q = threadIdx.x; q < R * NMAX; q += blockDim.x) {
        const int r = q / NMAX, n = q % NMAX;
        if (n < N && r0 + r < d.R) {
            float l = s_l[0][r][n], u = s_u[0][r][n];
            for (int wv = 1; wv < wpc; ++wv) { l = fmaxf(l, s_l[wv][r][n]); u = fmaxf(u, s_u[wv][r][n]); }
            const size_t o = (size_t)(r0 + r) * d.CO + (size_t)g * N + n;
            l = post_apply(post, l, g * N + n); u = post_apply(post, u, g * N + n);
            yl[o] = post.negate ? u : l; yu[o] = post.negate ? l : u;
        }
    }
}

template <int NMAX, int R>
int launch_fwd(const float* x, const float* w, const Dims& d, float* y, int* pos, cudaStream_t st, const Post& post) {
    const int items = ((d.R + R - 1) / R) * d.G;
    // warps that share a row block: as many as there are 128-float chunks to hand out, up to 8
    int wpc = min(8, max(1, d.CIg / 512));
    inf_forward_skinny_kernel<NMAX, R><<<items, 32 * wpc, 0, st>>>(x, w, d, y, pos, post);
    return launch_status();
}

template <int NMAX, int R>
int launch_bound(const float* xl, const float* xu, const float* w, const Dims& d, float* yl, float* yu,
                 cudaStream_t st, const Post& post) {
    const int items = ((d.R + R - 1) / R) * d.G;
    int wpc = min(8, max(1, d.CIg / 512));
    inf_bound_skinny_kernel<NMAX, R><<<items, 32 * wpc, 0, st>>>(xl, xu, w, d, yl, yu, post);
    return launch_status();
}

}  // namespace

bool skinny_ok(const Dims& d, const void* a, const void* b, const void* c) {
    return d.HW == 1 && d.COg < 32 && (d.CIg % 4) == 0 && (d.CI % 4) == 0 && d.CIg >= 128 &&
           aligned16(a) && aligned16(b) && (c == nullptr || aligned16(c));
}

int inf_forward_skinny(const float* x, const float* w, const Dims& d, float* y, int* pos, cudaStream_t st,
                       const Post& post) {
    if (d.COg <= 4) return launch_fwd<4, 4>(x, w, d, y, pos, st, post);
    if (d.COg <= 8) return launch_fwd<8, 2>(x, w, d, y, pos, st, post);
    if (d.COg <= 16) return launch_fwd<16, 2>(x, w, d, y, pos, st, post);
    return launch_fwd<32, 1>(x, w, d, y, pos, st, post);
}

int inf_bound_skinny(const float* xl, const float* xu, const float* w, const Dims& d, float* yl, float* yu,
                     cudaStream_t st, const Post& post) {
    if (d.COg <= 4) return launch_bound<4, 4>(xl, xu, w, d, yl, yu, st, post);
    if (d.COg <= 8) return launch_bound<8, 2>(xl, xu, w, d, yl, yu, st, post);
    if (d.COg <= 16) return launch_bound<16, 2>(xl, xu, w, d, yl, yu, st, post);
    return launch_bound<32, 1>(xl, xu, w, d, yl, yu, st, post);
}

}  // namespace linf
