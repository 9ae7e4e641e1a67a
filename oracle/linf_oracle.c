/*
 * linf_oracle.c -- CPU restatement of the distance-neuron path of zbh2047/L_inf-dist-net.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared with and
 * the CPU baseline that bench.py times; the product (liblinfdist.so and the Python package)
 * never calls it.
 *
 * Each function restates the semantics of one reference CUDA kernel (cited per function),
 * element by element, with plain loops.  Tensor layout as in the reference: input
 * [B, CI, HW], weight [CO, CI/G], output / pos / grad_output [B, CO, HW], all contiguous.
 *
 * Parity pins (tests/test_oracle_golden.py): the p = inf forward values, the interval bounds
 * and the finite-p forward / gradients are checked against outputs of the reference's own
 * pure-PyTorch branch (model/norm_dist.py:52-57, 66-75) stored under tests/golden/.  The
 * arg-max encoding and the scatter backward have no executable CPU counterpart in the
 * reference (its CPU branch never materialises indices, and autograd splits ties); for those
 * two this file IS the definition: the kernel's scan rule for the index, and sequential fp32
 * adds in ascending source order for the scatter.
 *
 * OpenMP parallelises over rows; every output element is still produced by one thread with a
 * fixed operation order, so results do not depend on the thread count.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define IDX_ACT(b, g, c, Cg, G, HW, hw) ((((size_t)(b) * (G) + (g)) * (Cg) + (c)) * (HW) + (hw))

/* model/inf_dist_cuda.cu:10-68 -- ascending scan, strict '>' update (lowest index wins ties),
 * start value 0 / pos 0, pos = index | (t < 0) << 31 with the index relative to the group. */
void oracle_inf_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                             float* y, int32_t* pos) {
    const int COg = CO / G, CIg = CI / G;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < CO; ++o) {
            const int g = o / COg;
            const float* wr = w + (size_t)o * CIg;
            for (int hw = 0; hw < HW; ++hw) {
                float best = 0.f;
                int32_t p = 0;
                for (int i = 0; i < CIg; ++i) {
                    float t = x[IDX_ACT(b, g, i, CIg, G, HW, hw)] - wr[i];
                    float a = fabsf(t);
                    if (a > best) {
                        best = a;
                        p = (int32_t)((uint32_t)i | (t >= 0.f ? 0u : 0x80000000u));
                    }
                }
                size_t oo = ((size_t)b * CO + o) * HW + hw;
                y[oo] = best;
                if (pos) pos[oo] = p;
            }
        }
}

/* fmaxf / fminf of CUDA: a NaN operand is ignored. */
static inline float mx(float a, float b) { return fmaxf(a, b); }
static inline float mn(float a, float b) { return fminf(a, b); }

/* model/inf_dist_cuda.cu:73-141 -- literal lower/upper rule, both start at 0. */
void oracle_inf_dist_bound_forward(const float* xl, const float* xu, const float* w,
                                   int B, int CO, int CI, int G, int HW, float* yl, float* yu) {
    const int COg = CO / G, CIg = CI / G;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < CO; ++o) {
            const int g = o / COg;
            const float* wr = w + (size_t)o * CIg;
            for (int hw = 0; hw < HW; ++hw) {
                float L = 0.f, U = 0.f;
                for (int i = 0; i < CIg; ++i) {
                    size_t a = IDX_ACT(b, g, i, CIg, G, HW, hw);
                    float tL = xl[a] - wr[i], tU = xu[a] - wr[i];
                    float aL = fabsf(tL), aU = fabsf(tU);
                    U = mx(U, mx(aL, aU));
                    if (!(tL < 0.f && tU > 0.f)) L = mx(L, mn(aL, aU));
                }
                size_t oo = ((size_t)b * CO + o) * HW + hw;
                yl[oo] = L;
                yu[oo] = U;
            }
        }
}

/* model/inf_dist_cuda.cu:143-156 -- grad_input[b, g*CIg+idx, hw] += (pos >= 0 ? g : -g).
 * The reference uses atomicAdd (order undefined); this fixes ASCENDING o, sequential fp32
 * adds from +0.  Indices outside the group are dropped. */
void oracle_inf_dist_backward_input(const float* gout, const int32_t* pos,
                                    int B, int CO, int CI, int G, int HW, float* gx) {
    const int COg = CO / G, CIg = CI / G;
    memset(gx, 0, (size_t)B * CI * HW * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b)
        for (int g = 0; g < G; ++g)
            for (int hw = 0; hw < HW; ++hw)
                for (int o = 0; o < COg; ++o) {
                    size_t a = IDX_ACT(b, g, o, COg, G, HW, hw);
                    int32_t p = pos[a];
                    uint32_t idx = (uint32_t)p & 0x7fffffffu;
                    if (idx >= (uint32_t)CIg) continue;
                    float v = gout[a];
                    float* dst = gx + IDX_ACT(b, g, idx, CIg, G, HW, hw);
                    *dst = *dst + (p >= 0 ? v : -v);
                }
}

/* model/inf_dist_cuda.cu:158-171 -- grad_weight[o, idx] += (pos < 0 ? g : -g); fixed here to
 * ASCENDING b*HW + hw, sequential fp32 adds from +0. */
void oracle_inf_dist_backward_weight(const float* gout, const int32_t* pos,
                                     int B, int CO, int CI, int G, int HW, float* gw) {
    const int COg = CO / G, CIg = CI / G;
    memset(gw, 0, (size_t)CO * CIg * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int o = 0; o < CO; ++o) {
        const int g = o / COg, og = o % COg;
        float* row = gw + (size_t)o * CIg;
        for (int b = 0; b < B; ++b)
            for (int hw = 0; hw < HW; ++hw) {
                size_t a = IDX_ACT(b, g, og, COg, G, HW, hw);
                int32_t p = pos[a];
                uint32_t idx = (uint32_t)p & 0x7fffffffu;
                if (idx >= (uint32_t)CIg) continue;
                float v = gout[a];
                row[idx] = row[idx] + (p < 0 ? v : -v);
            }
    }
}

/* Finite p, in double precision (the reference's arithmetic, model/norm_dist.py:52-57 and
 * model/norm_dist_cuda.cu:228-292, carried out exactly enough to serve as ground truth):
 * y = M * (sum (|t|/M)^p)^(1/p), M = max |t|; y = 0 when M = 0. */
void oracle_norm_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                              float p, float* y) {
    const int COg = CO / G, CIg = CI / G;
    const double pd = (double)p;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < CO; ++o) {
            const int g = o / COg;
            const float* wr = w + (size_t)o * CIg;
            for (int hw = 0; hw < HW; ++hw) {
                double M = 0.0;
                for (int i = 0; i < CIg; ++i) {
                    float t = x[IDX_ACT(b, g, i, CIg, G, HW, hw)] - wr[i];
                    double a = fabs((double)t);
                    if (a > M) M = a;
                }
                double S = 0.0;
                if (M > 0.0)
                    for (int i = 0; i < CIg; ++i) {
                        float t = x[IDX_ACT(b, g, i, CIg, G, HW, hw)] - wr[i];
                        S += pow(fabs((double)t) / M, pd);
                    }
                y[((size_t)b * CO + o) * HW + hw] = (M > 0.0) ? (float)(pow(S, 1.0 / pd) * M) : 0.f;
            }
        }
}

/* model/norm_dist_cuda.cu:294-361 -- grad_input = sum_o g * (|t|/y)^(p-1) * (t > 0 ? 1 : -1),
 * double accumulation; a zero output contributes nothing. */
void oracle_norm_dist_backward_input(const float* gout, const float* x, const float* w, const float* y,
                                     int B, int CO, int CI, int G, int HW, float p, float* gx) {
    const int COg = CO / G, CIg = CI / G;
    const double q = (double)p - 1.0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < CI; ++c) {
            const int g = c / CIg, i = c % CIg;
            for (int hw = 0; hw < HW; ++hw) {
                const float xv = x[((size_t)b * CI + c) * HW + hw];
                double acc = 0.0;
                for (int o = 0; o < COg; ++o) {
                    size_t a = IDX_ACT(b, g, o, COg, G, HW, hw);
                    double yv = (double)y[a];
                    if (!(yv > 0.0)) continue;
                    float t = xv - w[((size_t)g * COg + o) * CIg + i];
                    double term = (double)gout[a] * pow(fabs((double)t) / yv, q);
                    acc += (t > 0.f) ? term : -term;
                }
                gx[((size_t)b * CI + c) * HW + hw] = (float)acc;
            }
        }
}

/* model/norm_dist_cuda.cu:363-425 -- grad_weight = sum_{b,hw} g * (|t|/y)^(p-1) * (w - x > 0 ? 1 : -1). */
void oracle_norm_dist_backward_weight(const float* gout, const float* x, const float* w, const float* y,
                                      int B, int CO, int CI, int G, int HW, float p, float* gw) {
    const int COg = CO / G, CIg = CI / G;
    const double q = (double)p - 1.0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int o = 0; o < CO; ++o)
        for (int i = 0; i < CIg; ++i) {
            const int g = o / COg, og = o % COg;
            const float wv = w[(size_t)o * CIg + i];
            double acc = 0.0;
            for (int b = 0; b < B; ++b)
                for (int hw = 0; hw < HW; ++hw) {
                    size_t a = IDX_ACT(b, g, og, COg, G, HW, hw);
                    double yv = (double)y[a];
                    if (!(yv > 0.0)) continue;
                    float t = wv - x[IDX_ACT(b, g, i, CIg, G, HW, hw)];
                    double term = (double)gout[a] * pow(fabs((double)t) / yv, q);
                    acc += (t > 0.f) ? term : -term;
                }
            gw[(size_t)o * CIg + i] = (float)acc;
        }
}

int oracle_version(void) { return 100; }
