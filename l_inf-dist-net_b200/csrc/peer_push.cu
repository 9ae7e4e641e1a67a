// Host-side helpers of the copy-engine gradient exchange of the data-parallel training step: a
// group of asynchronous copies (into peers' memory or local) followed by 32-bit flag writes, and
// a group of 32-bit flag waits, each queued on a stream with ONE call from the host.  Neither
// launches a kernel: the copies run on the copy engines, the flag operations are stream memory
// operations of the driver (cuStreamBatchMemOp, looked up through the runtime so that the library
// does not link libcuda).  They exist to keep the host cost of an exchange with W-1 peers low.
#include <cuda.h>

#include "common.cuh"

namespace {

typedef CUresult (*BatchMemOpFn)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);

BatchMemOpFn batch_mem_op() {
    static BatchMemOpFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<BatchMemOpFn>(f);
    }();
    return fn;
}

constexpr int MAX_FLAGS = 64;

}  // namespace

extern "C" int linf_peer_push(int n_copies, void* const* dst, const void* const* src, const size_t* bytes,
                              int n_flags, void* const* flag_addr, unsigned int flag_value, void* stream) {
    using namespace linf;
    if (n_copies < 0 || n_flags < 0 || n_flags > MAX_FLAGS) return LINF_ERR_DIMS;
    if ((n_copies > 0 && (!dst || !src || !bytes)) || (n_flags > 0 && !flag_addr)) return LINF_ERR_NULL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    for (int i = 0; i < n_copies; ++i) {
        if (!dst[i] || !src[i]) return LINF_ERR_NULL;
        if (bytes[i] == 0) continue;
        if (cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDefault, st) != cudaSuccess) return LINF_ERR_LAUNCH;
    }
    if (n_flags == 0) return LINF_OK;
    BatchMemOpFn fn = batch_mem_op();
    if (fn == nullptr) return LINF_ERR_LAUNCH;
    CUstreamBatchMemOpParams ops[MAX_FLAGS];
    for (int i = 0; i < n_flags; ++i) {
        if (!flag_addr[i] || (reinterpret_cast<uintptr_t>(flag_addr[i]) & 3u)) return LINF_ERR_WORKSPACE;
        ops[i] = CUstreamBatchMemOpParams();
        ops[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_32;
        ops[i].writeValue.address = reinterpret_cast<CUdeviceptr>(flag_addr[i]);
        ops[i].writeValue.value = flag_value;
        ops[i].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT;    // ordered behind the copies above
    }
    return fn(reinterpret_cast<CUstream>(st), (unsigned)n_flags, ops, 0) == CUDA_SUCCESS ? LINF_OK : LINF_ERR_LAUNCH;
}

extern "C" int linf_flags_wait(int n_flags, void* const* flag_addr, unsigned int value, void* stream) {
    using namespace linf;
    if (n_flags < 0 || n_flags > MAX_FLAGS) return LINF_ERR_DIMS;
    if (n_flags == 0) return LINF_OK;
    if (!flag_addr) return LINF_ERR_NULL;
    BatchMemOpFn fn = batch_mem_op();
    if (fn == nullptr) return LINF_ERR_LAUNCH;
    CUstreamBatchMemOpParams ops[MAX_FLAGS];
    for (int i = 0; i < n_flags; ++i) {
        if (!flag_addr[i] || (reinterpret_cast<uintptr_t>(flag_addr[i]) & 3u)) return LINF_ERR_WORKSPACE;
        ops[i] = CUstreamBatchMemOpParams();
        ops[i].waitValue.operation = CU_STREAM_MEM_OP_WAIT_VALUE_32;
        ops[i].waitValue.address = reinterpret_cast<CUdeviceptr>(flag_addr[i]);
        ops[i].waitValue.value = value;
        ops[i].waitValue.flags = CU_STREAM_WAIT_VALUE_GEQ;          // cyclic comparison: (int)(*addr - value) >= 0
    }
    return fn(reinterpret_cast<CUstream>(reinterpret_cast<cudaStream_t>(stream)), (unsigned)n_flags, ops, 0) == CUDA_SUCCESS
               ? LINF_OK : LINF_ERR_LAUNCH;
}
