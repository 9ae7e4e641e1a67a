// Ordered grad_input of the inf-dist backward for dense layers (HW == 1) by direct accumulation in
// shared memory: no sort, no histogram.  The destination row lives in shared memory, starts at +0
// and receives its contributions one fp32 add at a time in ascending source order -- the order the
// CPU checker and the sort-based kernels (inf_backward.cu) define -- and is then written out whole,
// so the destination needs no zero fill.
//
// Rows = batch rows, sources = the COg channels of a group (contiguous).  One CTA per row takes the
// sources S = blockDim.x at a time, in ascending order.  Inside such a step the only ordering that
// matters is between sources of the SAME bin; they are peeled off in rounds: every pending thread
// offers its thread id to a per-bin tag with a shared-memory atomicMin, the lowest id of each bin
// wins the round, adds its value and clears the tag, the others try again.  A step needs as many
// rounds as its most frequent bin has sources; after MAX_ROUNDS the winner of the next round
// finishes its bin alone, walking the rest of the step's sources in order, so that a row whose
// sources all share one bin still costs a bounded number of barriers.
//
// (The same idea with one THREAD per grad_weight row -- program order is source order, nothing to
// detect -- was measured and dropped: the chain of 512 dependent shared-memory updates per row runs
// behind the latency of its strided loads, 108 us against 35 us for the warp-per-row kernel of
// inf_backward_accum.cu at B = 512, Din = 784, Dout = 5120.)
#include "common.cuh"

namespace linf {
namespace {

constexpr int NO_TAG = 0x7fffffff;

template <int S>
__global__ void __launch_bounds__(S)
inf_backward_input_direct_kernel(const float* __restrict__ gout, const int* __restrict__ pos, Dims d,
                                 float* __restrict__ dst, int nbp, const int* __restrict__ skip_if) {
    constexpr int MAX_ROUNDS = 6;
    if (skip_if != nullptr && probe_says_contested(skip_if)) return;      // the sort kernel runs instead
    extern __shared__ __align__(16) float smem_d[];
    float* acc = smem_d;                                        // [nbp]
    int* tag = reinterpret_cast<int*>(smem_d + nbp);            // [nbp]
    int* sidx = tag + nbp;                                      // [S]  fallback only
    float* sval = reinterpret_cast<float*>(sidx + S);           // [S]  fallback only
    const int tid = threadIdx.x;
    const int nb = d.CIg, n_src = d.COg;
    const int row = blockIdx.x;                                 // row = r * G + g
    const float* g_row = gout + (size_t)row * n_src;            // [R, G, COg] with HW == 1
    const int* p_row = pos + (size_t)row * n_src;
    for (int i = tid; i < nbp; i += S) { acc[i] = 0.f; tag[i] = NO_TAG; }
    int p_next = 0; float g_next = 0.f;
    if (tid < n_src) { p_next = __ldg(p_row + tid); g_next = __ldg(g_row + tid); }
    __syncthreads();
    for (int s0 = 0; s0 < n_src; s0 += S) {
        const int p = p_next; const float gv = g_next;
        const bool have = s0 + tid < n_src;
        if (s0 + S + tid < n_src) { p_next = __ldg(p_row + s0 + S + tid); g_next = __ldg(g_row + s0 + S + tid); }
        const int idx = p & 0x7fffffff;
        const float v = (p >= 0) ? gv : -gv;                    // grad_input takes +s * g
        bool pending = have && idx < nb && v != 0.f;           // +-0 changes no sum (accumulators start at +0, never become -0)
        int more = 1;
#pragma unroll 1
        for (int round = 0; round < MAX_ROUNDS && more; ++round) {
            if (pending) atomicMin(&tag[idx], tid);
            __syncthreads();
            if (pending && tag[idx] == tid) {
                acc[idx] += v;
                tag[idx] = NO_TAG;
                pending = false;
            }
            more = __syncthreads_or(pending ? 1 : 0);
        }
        if (more) {
            // some bin still has sources left in this step: its lowest pending thread takes them all
            sidx[tid] = pending ? idx : -1;
            sval[tid] = v;
            if (pending) atomicMin(&tag[idx], tid);
            __syncthreads();
            if (pending && tag[idx] == tid) {
                float a = acc[idx] + v;
                for (int t2 = tid + 1; t2 < S; ++t2)
                    if (sidx[t2] == idx) a += sval[t2];
                acc[idx] = a;
                tag[idx] = NO_TAG;
            }
            __syncthreads();
        }
    }
    float* out = dst + (size_t)row * nb;
    if ((nb & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        for (int i = tid * 4; i < nb; i += S * 4)
            *reinterpret_cast<float4*>(out + i) = *reinterpret_cast<const float4*>(acc + i);
    } else {
        for (int i = tid; i < nb; i += S) out[i] = acc[i];
    }
}

// How contested are the bins?  The rounds of a step are as many as the sources of its fullest bin: three or
// four when the arg-max positions of a row are spread (22 us at B = 512, Din = Dout = 5120), twenty to
// thirty-four when a few hundred input coordinates attract most of them (x ~ N(0,1): 141 us, where the sort
// kernel takes 56 us).  Only the data can tell, so a probe looks at it: PROBE_ROWS rows, two steps of S
// sources each, a shared-memory histogram per step; a bin with more than PROBE_LIMIT sources sets the flag
// that makes the direct kernel return at once and lets the sort kernel, launched right behind it, run.
constexpr int PROBE_ROWS = kGxProbeRows, PROBE_LIMIT = 8, PROBE_S = 512;

__global__ void __launch_bounds__(PROBE_S)
gx_probe_kernel(const int* __restrict__ pos, Dims d, int n_rows, int* __restrict__ contested) {
    extern __shared__ int cnt[];                                // [nb]
    const int tid = threadIdx.x, nb = d.CIg, n_src = d.COg;
    const int row = (int)((long long)blockIdx.x * n_rows / gridDim.x);
    const int* p_row = pos + (size_t)row * n_src;
    for (int i = tid; i < nb; i += PROBE_S) cnt[i] = 0;
    __syncthreads();
    int full = 0;
    const int last = ((n_src - 1) / PROBE_S) * PROBE_S;
    for (int pass = 0; pass < 2; ++pass) {
        const int s0 = pass == 0 ? 0 : (last / 2 / PROBE_S) * PROBE_S;
        if (pass == 1 && s0 == 0) break;
        const int e = s0 + tid;
        const int idx = e < n_src ? (__ldg(p_row + e) & 0x7fffffff) : nb;
        if (idx < nb) atomicAdd(&cnt[idx], 1);
        __syncthreads();
        if (idx < nb && cnt[idx] > PROBE_LIMIT) full = 1;
        __syncthreads();
        if (idx < nb) cnt[idx] = 0;
        __syncthreads();
    }
    full = __syncthreads_or(full);
    if (tid == 0) contested[blockIdx.x] = full;                 // every probe CTA owns a word: nothing to clear beforehand
}

// PROBE_ROWS words per call in flight; a slot comes round again after 256 calls.
__device__ int g_gx_contested[256 * PROBE_ROWS];
std::atomic<unsigned> g_gx_slot{0};

}  // namespace

// Returns -1 when the shape is not one this kernel takes (the caller goes on to the sort-based
// kernels).  Taken: dense layers whose rows have many bins for their sources -- the rounds of a step
// are few then -- or few sources altogether.  Measured at B = 512, Dout = 5120: 22 us against 37 us
// (sort) at Din = 3072, 22 us against 43 us at Din = 5120, but 35 us against 31 us at Din = 784,
// where every step of 512 sources meets the 784 bins with four to five sources in the fullest bin;
// 8 us against 20 us for the 10 sources per row of a classifier layer.
// `decided_by`: where the caller has a sort kernel ready for the same rows, it passes a pointer here; for the
// shapes whose speed depends on the data the direct kernel is then launched behind a probe, *decided_by
// receives the address of the probe's flag, and the caller launches its sort kernel conditional on that flag
// (exactly one of the two does the work; both give the same bits).
int inf_backward_input_direct(const float* g, const int* pos, const Dims& d, float* gx, cudaStream_t st,
                              const int** decided_by) {
    if (decided_by != nullptr) *decided_by = nullptr;
    if (d.HW != 1) return -1;
    if (d.COg > 128 && d.CIg < 1536) return -1;
    const int nbp = (d.CIg + 3) & ~3;
    const long long n_rows = (long long)d.R * d.G;
    if (n_rows > 0x7fffffffLL) return -1;
    if (d.COg > 128) {
        constexpr int S = 512;
        const size_t smem = (size_t)nbp * 8 + (size_t)S * 8;
        if (smem > 96 * 1024) return -1;
        if (cudaFuncSetAttribute(inf_backward_input_direct_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 96 * 1024) != cudaSuccess)
            return LINF_ERR_LAUNCH;
        int* flag = nullptr;
        int launched = 1;
        if (decided_by != nullptr && inf_backward_path == 0 && (size_t)d.CIg * 4 <= 48 * 1024) {
            void* base = nullptr;
            if (cudaGetSymbolAddress(&base, g_gx_contested) != cudaSuccess) return LINF_ERR_LAUNCH;
            flag = static_cast<int*>(base) + (size_t)(g_gx_slot.fetch_add(1, std::memory_order_relaxed) & 255u) * PROBE_ROWS;
            gx_probe_kernel<<<PROBE_ROWS, PROBE_S, (size_t)d.CIg * 4, st>>>(pos, d, (int)n_rows, flag);
            *decided_by = flag;
            launched = 2;
        }
        inf_backward_input_direct_kernel<S><<<(int)n_rows, S, smem, st>>>(g, pos, d, gx, nbp, flag);
        return launch_status(launched);
    } else {
        constexpr int S = 128;
        const size_t smem = (size_t)nbp * 8 + (size_t)S * 8;
        if (smem > 96 * 1024) return -1;
        if (cudaFuncSetAttribute(inf_backward_input_direct_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 96 * 1024) != cudaSuccess)
            return LINF_ERR_LAUNCH;
        inf_backward_input_direct_kernel<S><<<(int)n_rows, S, smem, st>>>(g, pos, d, gx, nbp, nullptr);
    }
    return launch_status();
}

}  // namespace linf
