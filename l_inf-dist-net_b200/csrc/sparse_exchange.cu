// Gradient exchange of a data-parallel step for p = inf distance layers, over peer memory.
//
// The weight gradient of an inf-dist layer is a scatter: sample b adds g[b, o] to ONE column of row o
// (model/inf_dist_cuda.cu:158-171 of zbh2047/L_inf-dist-net), so a row of grad_weight holds at most
// B non-zeros however wide it is -- in the CIFAR-shape training step a few hundred non-zeros in
// 26 M cells.  The reference averages the dense gradient (torch DistributedDataParallel,
// main.py:290-291: 378 MB per step through an all-reduce); here every rank lists the non-zeros of
// its rows, and every rank adds up the lists of all ranks, read straight from the peers' memory
// over NVLink.  Sizes are known on the device only, which is why this is a kernel reading peer
// pointers and not a collective with host-side counts.
//
//   list of one rank for one parameter:  cnt[rows] (int32)  +  ent[rows][cap] ({int32 col, fp32 value})
//   cap >= the largest possible number of non-zeros of a row (the caller passes the batch size).
//
//   compact:  one warp per row scans the row of the dense gradient, writes its non-zeros in ascending
//             column order, and zeroes them in the dense gradient (which is all zero afterwards).
//   publish:  one thread stores the step number to this rank's flag (system scope, after a fence).
//   wait:     one thread per peer polls that peer's flag until it has reached the step number or a
//             time limit runs out (then an error word is set and every later kernel of the exchange
//             does nothing: no wait here is unbounded, nothing traps).
//   merge:    one warp per row adds, rank by rank in rank order, value * scale of every listed entry
//             to the (zeroed) dense row: the sum is the same on every rank, bit for bit, because every
//             rank adds the same numbers in the same order.  With scale = 1 / world and a power-of-two
//             world this is the average an all-reduce gives.
//
// A list is read by the peers during their merge of step t and overwritten by its owner at step t + 2
// (two lists per parameter, used alternately): the owner's compaction of step t + 2 is stream-ordered
// behind its merge of step t + 1, which waited for every peer's flag of step t + 1, which that peer
// raised after its own merge of step t.  No further barrier is needed.
#include "common.cuh"

namespace linf {
namespace {

struct __align__(8) Entry { int col; float val; };

__global__ void __launch_bounds__(256)
grad_rows_compact_kernel(float* __restrict__ grad, int rows, int cols, int cap,
                         int* __restrict__ cnt, Entry* __restrict__ ent, int* __restrict__ err) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* g = grad + (size_t)row * cols;
    Entry* out = ent + (size_t)row * cap;
    int n = 0;
    const bool vec = (cols % 4) == 0 && ((reinterpret_cast<uintptr_t>(g) & 15u) == 0);
    if (vec) {
        // four 512-byte pieces of the row in flight per warp before the first vote
        for (int c00 = 0; c00 < cols; c00 += 512) {
            float4 vs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c00 + 128 * u + 4 * lane;
                vs[u] = c < cols ? *reinterpret_cast<const float4*>(g + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c00 + 128 * u + 4 * lane;
                const float e[4] = {vs[u].x, vs[u].y, vs[u].z, vs[u].w};
                const int mine = (e[0] != 0.f) + (e[1] != 0.f) + (e[2] != 0.f) + (e[3] != 0.f);
                if (__any_sync(0xffffffffu, mine != 0)) {
                    // exclusive prefix of `mine` over the lanes: ascending column order
                    int incl = mine;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const int t = __shfl_up_sync(0xffffffffu, incl, d);
                        if (lane >= d) incl += t;
                    }
                    int at = n + incl - mine;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (e[k] != 0.f) {
                            if (at < cap) out[at] = Entry{c + k, e[k]};
                            ++at;
                        }
                    if (mine) *reinterpret_cast<float4*>(g + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                    n += __shfl_sync(0xffffffffu, incl, 31);
                }
            }
        }
    } else {
        for (int c0 = 0; c0 < cols; c0 += 32) {
            const int c = c0 + lane;
            const float v = c < cols ? g[c] : 0.f;
            const unsigned m = __ballot_sync(0xffffffffu, v != 0.f);
            if (v != 0.f) {
                const int at = n + __popc(m & ((1u << lane) - 1u));
                if (at < cap) out[at] = Entry{c, v};
                g[c] = 0.f;
            }
            n += __popc(m);
        }
    }
    if (lane == 0) {
        cnt[row] = n;
        if (n > cap) atomicExch(err, 2);      // more non-zeros than the caller said a row can have
    }
}

__global__ void flag_publish_kernel(int* flag, int value) {
    __threadfence_system();
    *reinterpret_cast<volatile int*>(flag) = value;
    __threadfence_system();
}

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__global__ void flags_wait_kernel(const int* const* __restrict__ flags, int n, int value,
                                  unsigned long long limit_ns, int* __restrict__ err) {
    const int q = threadIdx.x;
    if (q >= n) return;
    const volatile int* f = flags[q];
    const unsigned long long t0 = now_ns();
    // the step numbers only grow; a flag beyond `value` means that peer is already a step ahead
    for (long long spin = 0; spin < (1ll << 40); ++spin) {
        if (*f - value >= 0) { __threadfence_system(); return; }
        if ((spin & 63) == 63 && now_ns() - t0 > limit_ns) break;
    }
    atomicExch(err, 1);
}

__global__ void __launch_bounds__(256)
grad_rows_merge_kernel(float* __restrict__ grad, int rows, int cols, int cap,
                       const int* const* __restrict__ cnts, const Entry* const* __restrict__ ents,
                       int world, float scale, const int* __restrict__ err) {
    if (*reinterpret_cast<const volatile int*>(err) != 0) return;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* g = grad + (size_t)row * cols;
    for (int q0 = 0; q0 < world; q0 += 32) {
        // the counts of up to 32 ranks in one round trip
        int mine = 0;
        if (q0 + lane < world) mine = *reinterpret_cast<const volatile int*>(cnts[q0 + lane] + row);
        const int span = min(32, world - q0);
        for (int j = 0; j < span; ++j) {
            const int n = min(__shfl_sync(0xffffffffu, mine, j), cap);
            if (n == 0) continue;
            const Entry* src = ents[q0 + j] + (size_t)row * cap;
            for (int e = lane; e < n; e += 32) {
                const unsigned long long raw = *reinterpret_cast<const volatile unsigned long long*>(src + e);
                const int col = (int)(unsigned)(raw & 0xffffffffull);
                const float val = __uint_as_float((unsigned)(raw >> 32));
                // (the product and the sum are rounded separately: the value an all-reduce of pre-scaled inputs gives)
                if (col >= 0 && col < cols) g[col] = __fadd_rn(g[col], __fmul_rn(val, scale));   // columns of one rank's row are distinct
            }
            __syncwarp();
        }
    }
}

}  // namespace

int grad_rows_compact(float* grad, int rows, int cols, int cap, int* cnt, void* ent, int* err, cudaStream_t st) {
    grad_rows_compact_kernel<<<(rows + 7) / 8, 256, 0, st>>>(grad, rows, cols, cap, cnt, static_cast<Entry*>(ent), err);
    return launch_status();
}

int flag_publish(int* flag, int value, cudaStream_t st) {
    flag_publish_kernel<<<1, 1, 0, st>>>(flag, value);
    return launch_status();
}

int flags_wait(const int* const* flags, int n, int value, int timeout_ms, int* err, cudaStream_t st) {
    flags_wait_kernel<<<1, ((n + 31) / 32) * 32, 0, st>>>(flags, n, value, (unsigned long long)timeout_ms * 1000000ull, err);
    return launch_status();
}

int grad_rows_merge(float* grad, int rows, int cols, int cap, const int* const* cnts, const void* const* ents,
                    int world, float scale, const int* err, cudaStream_t st) {
    grad_rows_merge_kernel<<<(rows + 7) / 8, 256, 0, st>>>(grad, rows, cols, cap, cnts,
                                                          reinterpret_cast<const Entry* const*>(ents), world, scale, err);
    return launch_status();
}

}  // namespace linf
