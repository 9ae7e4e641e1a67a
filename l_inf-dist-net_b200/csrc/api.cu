// extern "C" surface of liblinfdist.so: argument validation, then the launchers.
#include <math.h>

#include <mutex>

#include "common.cuh"

namespace linf {

namespace {
// per-device state of the library: read-only attributes and the helper stream
struct DeviceSlot {
    std::mutex lock;            // held by a SideLease for a whole fork ... join sequence
    int sms = 0;
    bool side_ready = false;
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
DeviceSlot g_slots[kMaxDevices];
std::mutex g_attr_lock;

int current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return -1; }
    return dev;
}
}  // namespace

int sm_count() {
    const int dev = current_device();
    auto ask = [](int d) {
        int n = 0;
        if (d < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148;
        }
        return n;
    };
    if (dev < 0 || dev >= kMaxDevices) return ask(dev);
    std::lock_guard<std::mutex> hold(g_attr_lock);
    if (g_slots[dev].sms == 0) g_slots[dev].sms = ask(dev);
    return g_slots[dev].sms;
}

SideLease::SideLease() : side_(nullptr) {
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return;
    DeviceSlot* s = &g_slots[dev];
    s->lock.lock();
    if (!s->side_ready) {
        if (cudaStreamCreateWithFlags(&s->side, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->join, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            s->lock.unlock();
            return;
        }
        s->side_ready = true;
    }
    side_ = s;
}

SideLease::~SideLease() {
    if (side_ != nullptr) static_cast<DeviceSlot*>(side_)->lock.unlock();
}

cudaStream_t SideLease::stream() const { return static_cast<DeviceSlot*>(side_)->side; }

int SideLease::fork(cudaStream_t from) {
    DeviceSlot* s = static_cast<DeviceSlot*>(side_);
    if (cudaEventRecord(s->fork, from) != cudaSuccess || cudaStreamWaitEvent(s->side, s->fork, 0) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    return LINF_OK;
}

int SideLease::join(cudaStream_t into) {
    DeviceSlot* s = static_cast<DeviceSlot*>(side_);
    if (cudaEventRecord(s->join, s->side) != cudaSuccess || cudaStreamWaitEvent(into, s->join, 0) != cudaSuccess)
        return LINF_ERR_LAUNCH;
    return LINF_OK;
}

std::atomic<unsigned long long> g_launches{0};

extern int inf_forward_variant;
extern int inf_forward_tail;
extern int inf_forward_split;
extern int inf_forward_width;
extern int inf_forward_windows;
extern int lp_forward_width;
int inf_forward_tma_gave_up();

}  // namespace linf

using namespace linf;

namespace {
inline bool bad_p(float p) { return !(p > 1.f) || isinf(p); }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

extern "C" {

int linf_version(void) { return 100; }

unsigned long long linf_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* linf_error_string(int code) {
    switch (code) {
        case LINF_OK: return "ok";
        case LINF_ERR_NULL: return "a required pointer is NULL";
        case LINF_ERR_DIMS: return "a dimension is not positive or a tensor is too large";
        case LINF_ERR_GROUP: return "channel counts must be multiples of the group count";
        case LINF_ERR_P: return "p must be finite and greater than 1";
        case LINF_ERR_LAUNCH: return "CUDA reported an error at kernel launch";
        case LINF_ERR_WORKSPACE: return "workspace is missing, misaligned or too small";
        case LINF_ERR_TOO_LARGE: return "size exceeds a fixed maximum of this entry point";
        default: return "unknown error code";
    }
}

// Process-wide benchmarking knob: key 0 selects the tiled inf-dist forward variant (tile
// geometry / instruction mix, see the table in inf_forward.cu).  Not part of the drop-in
// surface; not thread safe.
int linf_tune_set(int key, int value) {
    if (key == 0 && value >= 0 && value < 16) { inf_forward_variant = value; return LINF_OK; }
    if (key == 1 && (value == 0 || value == 1)) { inf_forward_tail = value; return LINF_OK; }
    if (key == 3 && value >= 0 && value <= 2) { inf_backward_path = value; return LINF_OK; }
    if (key == 4 && value >= 0 && value <= 2) { inf_forward_split = value; return LINF_OK; }
    if (key == 5 && value >= 0 && value <= 2) { inf_forward_width = value; return LINF_OK; }
    if (key == 6 && value >= 0 && value <= 2) { lp_forward_width = value; return LINF_OK; }
    if (key == 7 && value >= 0 && value <= 1) { inf_forward_windows = value; return LINF_OK; }
    if (key == 2) return inf_forward_tma_gave_up();   // 1 = a bounded wait of the TMA loader ran out since the library was loaded
    return LINF_ERR_DIMS;
}

int linf_inf_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                          float* output, int* pos, void* stream) {
    if (!input || !weight || !output || !pos) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_forward(input, weight, d, output, pos, nullptr, 0, as_stream(stream));
}

size_t linf_inf_dist_forward_workspace_bytes(int B, int CO, int CI, int G, int HW) {
    Dims d;
    if (make_dims(B, CO, CI, G, HW, &d)) return 0;
    return inf_forward_workspace(d);
}

int linf_inf_dist_forward_ws(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                             float* output, int* pos, void* workspace, size_t workspace_bytes, void* stream) {
    if (!input || !weight || !output || !pos) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    if (inf_forward_workspace(d) != 0 && workspace == nullptr) return LINF_ERR_WORKSPACE;
    return inf_forward(input, weight, d, output, pos, workspace, workspace_bytes, as_stream(stream));
}

int linf_inf_dist_bound_forward(const float* input_lower, const float* input_upper, const float* weight,
                                int B, int CO, int CI, int G, int HW,
                                float* output_lower, float* output_upper, void* stream) {
    if (!input_lower || !input_upper || !weight || !output_lower || !output_upper) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_bound(input_lower, input_upper, weight, d, output_lower, output_upper, as_stream(stream));
}

int linf_inf_dist_forward_post(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                               const float* sub, const float* add, int negate, float* output,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (!input || !weight || !output) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    const Post post{sub, add, negate ? 1 : 0};
    return inf_forward(input, weight, d, output, nullptr, workspace, workspace_bytes, as_stream(stream), post);
}

int linf_inf_dist_bound_forward_post(const float* input_lower, const float* input_upper, const float* weight,
                                     int B, int CO, int CI, int G, int HW,
                                     const float* sub, const float* add, int negate,
                                     float* output_lower, float* output_upper, void* stream) {
    if (!input_lower || !input_upper || !weight || !output_lower || !output_upper) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    const Post post{sub, add, negate ? 1 : 0};
    return inf_bound(input_lower, input_upper, weight, d, output_lower, output_upper, as_stream(stream), post);
}

int linf_mean_shift(const float* input, int rows, int cols, float* running_mean, float momentum,
                    float* output, float* mean_out, void* stream) {
    if (!input || !output) return LINF_ERR_NULL;
    if (rows <= 0 || cols <= 0 || (long long)rows * cols > 0x7fffffffLL) return LINF_ERR_DIMS;
    return mean_shift(input, rows, cols, running_mean, momentum, output, mean_out, as_stream(stream));
}

int linf_grad_rows_compact(float* grad, int rows, int cols, int cap, int* cnt, void* ent, int* err, void* stream) {
    if (!grad || !cnt || !ent || !err) return LINF_ERR_NULL;
    if (rows <= 0 || cols <= 0 || cap <= 0 || (long long)rows * cap > 0x7fffffffLL) return LINF_ERR_DIMS;
    return grad_rows_compact(grad, rows, cols, cap, cnt, ent, err, as_stream(stream));
}

int linf_flag_publish(int* flag, int value, void* stream) {
    if (!flag) return LINF_ERR_NULL;
    return flag_publish(flag, value, as_stream(stream));
}

int linf_flags_wait(const int* const* flags, int n, int value, int timeout_ms, int* err, void* stream) {
    if (!flags || !err) return LINF_ERR_NULL;
    if (n <= 0 || n > 1024 || timeout_ms <= 0) return LINF_ERR_DIMS;
    return flags_wait(flags, n, value, timeout_ms, err, as_stream(stream));
}

int linf_grad_rows_merge(float* grad, int rows, int cols, int cap, const int* const* cnts, const void* const* ents,
                         int world, float scale, const int* err, void* stream) {
    if (!grad || !cnts || !ents || !err) return LINF_ERR_NULL;
    if (rows <= 0 || cols <= 0 || cap <= 0 || world <= 0 || (long long)rows * cap > 0x7fffffffLL) return LINF_ERR_DIMS;
    return grad_rows_merge(grad, rows, cols, cap, cnts, ents, world, scale, err, as_stream(stream));
}

int linf_inf_dist_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                                 float* grad_input, void* stream) {
    if (!grad_output || !pos || !grad_input) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_backward_input(grad_output, pos, d, grad_input, as_stream(stream));
}

int linf_inf_dist_backward_weight(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                                  float* grad_weight, void* stream) {
    if (!grad_output || !pos || !grad_weight) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_backward_weight(grad_output, pos, d, grad_weight, as_stream(stream));
}

int linf_inf_dist_backward(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                           float* grad_input, float* grad_weight, void* stream) {
    if (!grad_output || !pos || !grad_input || !grad_weight) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_backward_ordered_both(grad_output, pos, d, grad_input, grad_weight, as_stream(stream));
}

int linf_inf_dist_backward_atomic(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                                  float* grad_input, float* grad_weight, void* stream) {
    if (!grad_output || !pos) return LINF_ERR_NULL;
    if (!grad_input && !grad_weight) return LINF_ERR_NULL;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return inf_backward_atomic(grad_output, pos, d, grad_input, grad_weight, as_stream(stream));
}

int linf_norm_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                           float* output, float p, void* stream) {
    if (!input || !weight || !output) return LINF_ERR_NULL;
    if (bad_p(p)) return LINF_ERR_P;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return lp_forward(input, weight, d, output, p, as_stream(stream));
}

int linf_norm_dist_backward_input(const float* grad_output, const float* input, const float* weight,
                                  const float* output, int B, int CO, int CI, int G, int HW,
                                  float* grad_input, float p, void* stream) {
    if (!grad_output || !input || !weight || !output || !grad_input) return LINF_ERR_NULL;
    if (bad_p(p)) return LINF_ERR_P;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return lp_backward_input(grad_output, input, weight, output, d, grad_input, p, as_stream(stream));
}

int linf_norm_dist_backward_weight(const float* grad_output, const float* input, const float* weight,
                                   const float* output, int B, int CO, int CI, int G, int HW,
                                   float* grad_weight, float p, void* stream) {
    if (!grad_output || !input || !weight || !output || !grad_weight) return LINF_ERR_NULL;
    if (bad_p(p)) return LINF_ERR_P;
    Dims d;
    int rc = make_dims(B, CO, CI, G, HW, &d);
    if (rc) return rc;
    return lp_backward_weight(grad_output, input, weight, output, d, grad_weight, p, as_stream(stream));
}

}  // extern "C"
