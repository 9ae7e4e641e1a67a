// Batch-mean shift of a dense activation [rows, cols] in one launch: the training-mode half of the
// mean-shift normalisation that follows a distance layer (MeanNorm, model/norm_dist.py:85-97 of
// zbh2047/L_inf-dist-net) -- per-column mean over the batch, exponential running mean, subtraction
// -- which as separate elementwise / reduction passes costs four launches and three trips of the
// activation through L2.  The same kernel without a running mean is the backward pass of that
// normalisation (grad_in = grad_out - column mean of grad_out).
//
// A CTA of NW warps owns 32 neighbouring columns (one 128-byte line per row) and all rows: warp w adds
// the rows w, w + NW, w + 2 NW, ... of its column one by one (a fixed order; eight rows in flight), the NW
// partial sums of a column are added in warp order, the sum is divided by the row count, and the CTA then
// walks its rows a second time (they are still in L1/L2) to subtract.  NW = 32 for batches of 256 rows and
// more: with 8 warps a 512 x 5120 activation kept 9 warps per SM busy waiting for memory, 16 us; with 32
// it takes a third of that.  The order of the additions is fixed, so the result is the same on every run;
// it is not the order of any other library's reduction, so the mean agrees with e.g. torch.mean to fp32
// rounding, not bit for bit.  The subtraction and the running-mean update are exact functions of that mean.
#include "common.cuh"

namespace linf {
namespace {

template <int NW>
__global__ void __launch_bounds__(32 * NW)
mean_shift_kernel(const float* __restrict__ in, int rows, int cols, float* __restrict__ running_mean,
                  float keep, float momentum, float* __restrict__ out, float* __restrict__ mean_out) {
    __shared__ float part[NW][32];
    __shared__ float mean_s[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (c < cols) {
        int r = warp;
        for (; r + 7 * NW < rows; r += 8 * NW) {          // eight rows in flight, added in row order
            float a[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = __ldg(in + (size_t)(r + u * NW) * cols + c);
#pragma unroll
            for (int u = 0; u < 8; ++u) s += a[u];
        }
        for (; r < rows; r += NW) s += __ldg(in + (size_t)r * cols + c);
    }
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0) {
        float t = part[0][lane];
#pragma unroll
        for (int w = 1; w < NW; ++w) t += part[w][lane];
        const float m = t / (float)rows;
        mean_s[lane] = m;
        if (c < cols) {
            if (mean_out != nullptr) mean_out[c] = m;
            // running = running * (1 - momentum) + momentum * mean: the product is rounded, the
            // multiply-add is fused -- the arithmetic of `running.mul_(1 - momentum).add_(mean, alpha=momentum)`
            if (running_mean != nullptr) running_mean[c] = fmaf(momentum, m, running_mean[c] * keep);
        }
    }
    __syncthreads();
    if (c < cols) {
        const float m = mean_s[lane];
        int r = warp;
        for (; r + 7 * NW < rows; r += 8 * NW) {           // eight loads, then eight stores (out may be in)
            float a[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = in[(size_t)(r + u * NW) * cols + c];
#pragma unroll
            for (int u = 0; u < 8; ++u) out[(size_t)(r + u * NW) * cols + c] = a[u] - m;
        }
        for (; r < rows; r += NW) out[(size_t)r * cols + c] = in[(size_t)r * cols + c] - m;
    }
}

}  // namespace

int mean_shift(const float* in, int rows, int cols, float* running_mean, float momentum, float* out,
               float* mean_out, cudaStream_t st) {
    if (rows >= 256)
        mean_shift_kernel<32><<<(cols + 31) / 32, 1024, 0, st>>>(in, rows, cols, running_mean, 1.f - momentum, momentum, out, mean_out);
    else
        mean_shift_kernel<8><<<(cols + 31) / 32, 256, 0, st>>>(in, rows, cols, running_mean, 1.f - momentum, momentum, out, mean_out);
    return launch_status();
}

}  // namespace linf
