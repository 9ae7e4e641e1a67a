/*
 * linfdist.h -- C ABI of liblinfdist.so: the L_p / L_inf-distance neuron on B200 (sm_100a).
 *
 * The library is the device-side replacement for the torch extension `norm_dist_cpp`
 * of zbh2047/L_inf-dist-net (binding file model/norm_dist.cpp).  Every entry point takes
 * plain device pointers and integer sizes; nothing in a signature is a torch type.
 *
 * Tensor layout (identical to the reference, all contiguous, fp32 unless noted):
 *     input / lower / upper / grad_input   [B, CI, HW]
 *     weight / grad_weight                 [CO, CI/G]
 *     output / pos(int32) / grad_output    [B, CO, HW]
 * B batch, CI input channels, CO output channels, G groups, HW spatial positions
 * (1 for a dense layer).  Group g maps input channels [g*CI/G, (g+1)*CI/G) to output
 * channels [g*CO/G, (g+1)*CO/G).
 *
 * Common rules
 *   - every pointer is a DEVICE pointer on the current device; the caller owns all
 *     buffers; the entry points of this header that take no workspace allocate nothing;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream); calls
 *     are asynchronous with respect to the host;
 *   - the return value is 0 on success or one of the LINF_ERR_* codes; no entry point
 *     ever traps or asserts on the device;
 *   - besides cached per-device attributes the library keeps one helper stream per device
 *     (linf_inf_dist_backward runs its second kernel there); its fork / join events are queued
 *     under a per-device lock, so calls from several host threads are safe.  The grad_input
 *     kernels of wide dense layers pick their algorithm from a probe of the data; the probe's
 *     verdict travels in a slot of a small array inside the library, one slot per call, reused
 *     after 256 calls (so at most 256 such calls may be in flight on a device at once).  The
 *     tuning hook linf_tune_set at the end of this header is the exception: it is process-wide
 *     and not thread safe.
 */
#ifndef LINFDIST_H_
#define LINFDIST_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LINF_OK             0
#define LINF_ERR_NULL       1   /* a required pointer is NULL                           */
#define LINF_ERR_DIMS       2   /* a dimension is <= 0 or a product overflows int32     */
#define LINF_ERR_GROUP      3   /* CI or CO is not a multiple of G                      */
#define LINF_ERR_P          4   /* p is NaN, infinite or <= 1 (finite-p entry points)   */
#define LINF_ERR_LAUNCH     5   /* the CUDA runtime reported an error at launch         */
#define LINF_ERR_WORKSPACE  6   /* workspace missing, misaligned or too small           */
#define LINF_ERR_TOO_LARGE  7   /* size beyond a documented fixed maximum               */

/* Library version as major*10000 + minor*100 + patch. */
int linf_version(void);

/* Static text for a LINF_ERR_* code (never NULL). */
const char* linf_error_string(int code);

/* ---------------------------------------------------------------------------------
 * p = inf
 * --------------------------------------------------------------------------------- */

/*
 * output[b,o,hw] = max_i |input[b,g,i,hw] - weight[o,i]|
 * pos[b,o,hw]    = i* | (sign << 31), i* = LOWEST index (within the group) attaining the
 *                  maximum, sign = 1 iff input - weight < 0 there; an all-zero (or all-NaN)
 *                  row gives output 0, pos 0.
 * Replaces inf_dist_forward_cuda (model/norm_dist.cpp:13-14, called at :54-62; kernel
 * model/inf_dist_cuda.cu:10-68, launcher :173-180).  Values and pos are bit-identical.
 */
int linf_inf_dist_forward(const float* input, const float* weight,
                          int B, int CO, int CI, int G, int HW,
                          float* output, int* pos, void* stream);

/*
 * Same result, but the caller lends scratch memory so that the k-range of a layer can be
 * split across SMs when there are too few output tiles to fill the GPU.  `workspace`
 * must be 256-byte aligned and at least linf_inf_dist_forward_workspace_bytes(...) long
 * (the query returns 0 when the shape never needs scratch; then workspace may be NULL).
 * The workspace is written and read inside this call only; two calls that overlap on the
 * GPU must not share it.
 */
size_t linf_inf_dist_forward_workspace_bytes(int B, int CO, int CI, int G, int HW);
int linf_inf_dist_forward_ws(const float* input, const float* weight,
                             int B, int CO, int CI, int G, int HW,
                             float* output, int* pos,
                             void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same forward for callers that are not allowed to allocate device memory -- for example a
 * plug-in of a framework that owns all device memory through its own pool, or a deployment whose
 * memory is sized once at start-up and where a later cudaMalloc counts as a fault.  Such a caller
 * cannot supply the workspace of linf_inf_dist_forward_ws, so the scratch lives in the library
 * itself: a fixed device array of LINF_NOALLOC_SCRATCH_BYTES that every GPU which loads the
 * library keeps resident until the process exits.  The call itself allocates nothing (no
 * cudaMalloc / cudaFree, no allocating library routine); inputs and outputs are the caller's.
 *   - Limit: returns LINF_ERR_TOO_LARGE when the layer would need more scratch than the array
 *     holds (the need grows with the SM count of the GPU and, slowly, with the number of output
 *     tiles; on a 148-SM B200 every layer the library accepts fits).
 *   - The first call on each device looks up the device address of the array (with that device
 *     current); later calls on that device reuse it.  That first call may also be the moment the
 *     CUDA runtime loads the library's device code onto that GPU, which is what makes the array
 *     exist there; make it before any stream capture begins.
 *   - All calls on one GPU share the one array, and it keeps whatever the last call left there;
 *     the call clears the part that has to start at zero.  Two calls that overlap on the same
 *     GPU (different streams or threads) race on it: run them one after the other.
 * Results are identical to linf_inf_dist_forward.  This entry point has no counterpart in the
 * reference, whose kernels use no scratch memory.
 */
#define LINF_NOALLOC_SCRATCH_BYTES (30u * 1024u * 1024u)
int linf_inf_dist_forward_noalloc(const float* input, const float* weight,
                                  int B, int CO, int CI, int G, int HW,
                                  float* output, int* pos, void* stream);

/*
 * Interval propagation through an inf-dist layer in one pass:
 *   tL = lower - w, tU = upper - w
 *   output_upper = max_i max(|tL|, |tU|)
 *   output_lower = max_i ( (tL < 0 && tU > 0) ? 0 : min(|tL|, |tU|) )
 * Both start from 0.  Replaces inf_dist_bound_forward_cuda (model/norm_dist.cpp:15-16,
 * :64-74; kernel model/inf_dist_cuda.cu:73-141, launcher :181-188).  Bit-identical for
 * every input, including lower > upper.
 */
int linf_inf_dist_bound_forward(const float* input_lower, const float* input_upper,
                                const float* weight,
                                int B, int CO, int CI, int G, int HW,
                                float* output_lower, float* output_upper, void* stream);

/*
 * What follows an inf-dist layer at inference and certification time, folded into the kernel's store:
 *     v' = (v - sub[c]) + add[c]      c = output channel; a NULL vector skips that step
 *     v' = -v'                        if negate != 0
 * sub is the running mean of the layer's mean-shift normalisation, add its bias (MeanNorm in eval mode
 * and the bias add, model/norm_dist.py:95-97, :137-140, :150-155), negate the sign flip of the
 * classifier layer (model/mlp.py:22).  The two operations are the fp32 subtraction and addition of
 * the separate elementwise passes, in their order, so the result is theirs bit for bit.
 *
 * linf_inf_dist_forward_post: values only (no arg-max: the path that needs no gradient); workspace
 * as for linf_inf_dist_forward_ws, or NULL / 0.
 * linf_inf_dist_bound_forward_post: both bounds; with negate the outputs are also exchanged
 * (output_lower receives the negated upper bound), as model/mlp.py:22 reorders them.
 * No counterpart in the reference's binding, which runs these steps as torch operations.
 */
int linf_inf_dist_forward_post(const float* input, const float* weight,
                               int B, int CO, int CI, int G, int HW,
                               const float* sub, const float* add, int negate, float* output,
                               void* workspace, size_t workspace_bytes, void* stream);
int linf_inf_dist_bound_forward_post(const float* input_lower, const float* input_upper,
                                     const float* weight,
                                     int B, int CO, int CI, int G, int HW,
                                     const float* sub, const float* add, int negate,
                                     float* output_lower, float* output_upper, void* stream);

/*
 * Training-mode mean shift of a dense activation input[rows, cols] (rows = batch) in one launch:
 *     mean[c] = (sum over rows, fixed order) / rows
 *     running_mean[c] = running_mean[c] * (1 - momentum) + momentum * mean[c]     (skipped if NULL)
 *     output[r, c] = input[r, c] - mean[c]                                       (output may be input)
 * mean_out (cols floats) receives the means if not NULL.  Replaces the torch passes of MeanNorm.forward
 * (model/norm_dist.py:85-97); with running_mean == NULL it is also that layer's backward
 * (grad_in = grad_out - column mean of grad_out).  The mean agrees with another library's reduction to
 * fp32 rounding (different summation order); subtraction and running-mean update are exact given it.
 */
int linf_mean_shift(const float* input, int rows, int cols, float* running_mean, float momentum,
                    float* output, float* mean_out, void* stream);

/*
 * grad_input[b, g*CI/G + idx, hw] = sum over o of (pos >= 0 ? +g : -g), g = grad_output[b,o,hw],
 * idx = pos & 0x7fffffff.  The sum runs in ASCENDING o, one fp32 add at a time starting from
 * +0, so the result is the same on every run.  grad_input is fully overwritten (it need
 * not be zeroed).  Replaces inf_dist_backward_input_cuda (model/norm_dist.cpp:17-18,
 * :76-82; kernel model/inf_dist_cuda.cu:143-156, launcher :189-196), whose atomicAdd
 * order is undefined: this is one of the orders it can produce.
 */
int linf_inf_dist_backward_input(const float* grad_output, const int* pos,
                                 int B, int CO, int CI, int G, int HW,
                                 float* grad_input, void* stream);

/*
 * grad_weight[o, idx] = sum over (b, hw) of (pos < 0 ? +g : -g), in ASCENDING b*HW + hw
 * order, sequential fp32 adds from +0.  grad_weight is fully overwritten.  Replaces
 * inf_dist_backward_weight_cuda (model/norm_dist.cpp:19-20, :84-90; kernel
 * model/inf_dist_cuda.cu:158-171, launcher :197-204).
 */
int linf_inf_dist_backward_weight(const float* grad_output, const int* pos,
                                  int B, int CO, int CI, int G, int HW,
                                  float* grad_weight, void* stream);

/*
 * Both ordered gradients in one call: the same results, bit for bit, as
 * linf_inf_dist_backward_input followed by linf_inf_dist_backward_weight, but the two kernels run
 * side by side (grad_weight on a library-owned helper stream that forks from and joins back into
 * `stream`, so to the caller the call is ordered on `stream` like any other).  Replaces the pair of
 * launches at model/norm_dist.py:34-38.
 */
int linf_inf_dist_backward(const float* grad_output, const int* pos,
                           int B, int CO, int CI, int G, int HW,
                           float* grad_input, float* grad_weight, void* stream);

/*
 * Both gradients in one pass over (grad_output, pos) with warp-aggregated fp32 atomics:
 * contributions of one warp that hit the same address are summed in lane order first and
 * issued as one atomic.  The buffers are ACCUMULATED into, exactly like the reference
 * kernels (model/inf_dist_cuda.cu:143-171): the caller zero-fills them.  Either gradient
 * pointer may be NULL to skip it.  The order of atomics across warps is undefined, so a
 * cell that receives three or more contributions may differ in the last bit from the
 * ordered entry points above.
 */
int linf_inf_dist_backward_atomic(const float* grad_output, const int* pos,
                                  int B, int CO, int CI, int G, int HW,
                                  float* grad_input, float* grad_weight, void* stream);

/* ---------------------------------------------------------------------------------
 * finite p  (1 < p < inf)
 * --------------------------------------------------------------------------------- */

/*
 * output[b,o,hw] = M * ( sum_i (|input - weight| / M)^p )^(1/p),  M = max_i |input - weight|
 * (0 when M == 0).  Replaces norm_dist_forward_cuda (model/norm_dist.cpp:7-8, :22-28; kernel
 * model/norm_dist_cuda.cu:228-292, launcher :427-437).  Agrees with the reference's
 * arithmetic to 1e-5 relative; it is not bit-identical (the reference itself uses
 * approximate intrinsics).
 */
int linf_norm_dist_forward(const float* input, const float* weight,
                           int B, int CO, int CI, int G, int HW,
                           float* output, float p, void* stream);

/*
 * grad_input[b,i,hw] = sum_o g * (|t| / output)^(p-1) * sign(t), t = input - weight.
 * Fully overwrites grad_input.  Replaces norm_dist_backward_input_cuda
 * (model/norm_dist.cpp:9-10, :30-40; kernel model/norm_dist_cuda.cu:299-361, launcher :438-448).
 */
int linf_norm_dist_backward_input(const float* grad_output, const float* input,
                                  const float* weight, const float* output,
                                  int B, int CO, int CI, int G, int HW,
                                  float* grad_input, float p, void* stream);

/*
 * grad_weight[o,i] = sum_{b,hw} g * (|t| / output)^(p-1) * sign(-t).  Fully overwrites
 * grad_weight with a fixed summation order (no atomics).  Replaces
 * norm_dist_backward_weight_cuda (model/norm_dist.cpp:11-12, :42-52; kernel
 * model/norm_dist_cuda.cu:368-425, launcher :449-459).
 */
int linf_norm_dist_backward_weight(const float* grad_output, const float* input,
                                   const float* weight, const float* output,
                                   int B, int CO, int CI, int G, int HW,
                                   float* grad_weight, float p, void* stream);

/* ---------------------------------------------------------------------------------
 * optimiser step (next to the distance neuron on the training path)
 * --------------------------------------------------------------------------------- */

/*
 * One fused AdamW step on a parameter viewed as [rows, cols] with the reference's l_p-norm weight
 * decay per row, then the Adam update:
 *   p_norm = +inf     only the entry of largest magnitude of each row decays by lr*weight_decay
 *                     (lowest column among equal magnitudes);
 *   1 < p_norm < inf  x_i -= lr*wd * (|x_i| / ||x||_p)^(p-2) * x_i, with eps added to x_i^2 and the
 *                     row normalised by its maximum exactly as the reference computes it;
 *   p_norm <= 0       x_i *= 1 - lr*wd (parameters of modules that carry no norm).
 *   m = beta1*m + (1-beta1)*g;  v = beta2*v + (1-beta2)*g^2;
 *   x -= lr/(1-beta1^step) * m / (sqrt(v)/sqrt(1-beta2^step) + eps)
 * param, exp_avg, exp_avg_sq are updated in place; step counts from 1.  Replaces the per-tensor
 * loop body of AdamW.step (adamw.py:37-84: about fifteen torch launches per tensor) with one
 * launch; results agree with it to rounding.  cols is limited by shared memory (51200).
 */
int linf_adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq,
                    int rows, int cols, float p_norm, float lr, float beta1, float beta2,
                    float eps, float weight_decay, int step, void* stream);

/* ---------------------------------------------------------------------------------
 * sparse gradient exchange of a data-parallel step (no counterpart in the reference, whose data
 * parallelism is torch DistributedDataParallel, main.py:290-291: a dense all-reduce of every gradient)
 * --------------------------------------------------------------------------------- */

/*
 * A row of an inf-dist layer's weight gradient has at most B non-zeros (every sample adds to one
 * column).  These four calls turn the dense gradient of one rank into per-row lists, and add up the
 * lists of all ranks, read directly from the peers' device memory (buffers that every rank can
 * address, e.g. symmetric memory):
 *     list of one rank:  cnt[rows] int32,  ent[rows][cap] pairs {int32 column, float value}
 *
 * linf_grad_rows_compact  lists the non-zeros of grad[rows, cols] in ascending column order (cnt, ent
 *                         of THIS rank) and zeroes them in grad; a row with more than cap non-zeros
 *                         stores 2 to *err.
 * linf_flag_publish       stores `value` (the step number) to this rank's flag, after a system fence.
 * linf_flags_wait         flags: device array of n pointers, one flag per rank; returns when every flag
 *                         has reached `value`, or after timeout_ms stores 1 to *err.  Bounded; never traps.
 * linf_grad_rows_merge    cnts / ents: device arrays of `world` pointers (rank order).  Adds, rank by
 *                         rank, value * scale of every listed entry to grad (which compact left zero).
 *                         Every rank adds the same numbers in the same order: identical bits on all
 *                         ranks.  Does nothing if *err != 0.
 * err may be device memory or mapped pinned host memory.  Call order per parameter and step, on one
 * stream: compact, publish, wait, merge.  Use two lists per parameter alternately (odd / even steps);
 * then the stream order of these four calls is all the synchronisation the ranks need.
 */
int linf_grad_rows_compact(float* grad, int rows, int cols, int cap, int* cnt, void* ent, int* err, void* stream);
int linf_flag_publish(int* flag, int value, void* stream);
int linf_flags_wait(const int* const* flags, int n, int value, int timeout_ms, int* err, void* stream);
int linf_grad_rows_merge(float* grad, int rows, int cols, int cap, const int* const* cnts, const void* const* ents,
                         int world, float scale, const int* err, void* stream);

/* ---------------------------------------------------------------------------------
 * tuning hook (benchmarks and tests only; no counterpart in the reference)
 * --------------------------------------------------------------------------------- */

/*
 * Process-wide switches between kernel variants that give identical results.  NOT thread safe, and
 * keys 0, 4 and 5 change what linf_inf_dist_forward_workspace_bytes answers: set it while no call is in flight.
 *   key 0  tiled inf-dist forward variant (0 = default; the table is in csrc/inf_forward.cu)
 *   key 1  1 = run a partial last wave of output tiles as half-width tiles (default), 0 = never
 *   key 2  (value ignored) returns 1 if a bounded wait of the TMA-loader variant ever ran out, else 0
 *   key 3  grad_input of dense layers: 0 = direct-accumulation or sort kernel as a probe of the positions decides
 *          (default), 1 = never the direct kernel, 2 = the direct kernel wherever it fits, without the probe
 *   key 4  k-splitting of the forward: 0 = by shape (default), 1 = whenever scratch is given, 2 = never
 *   key 5  width of the forward's output tiles: 0 = by shape (default), 1 = 64 columns, 2 = 48 columns wherever
 *          that kernel applies
 *   key 6  the same for the finite-p forward
 *   key 7  arg-max tracking windows of the forward: 0 = 16 terms for rows of 2048 terms and more, else 8 (default),
 *          1 = 8 terms always
 * Returns LINF_OK, the answer of key 2, or LINF_ERR_DIMS for an unknown key / value.
 */
int linf_tune_set(int key, int value);

/*
 * Number of CUDA kernels this library has launched in this process since it was loaded (all devices, all
 * threads).  Diagnostics: a caller that wants to know that its step really ran on the library's kernels
 * reads it before and after.  No counterpart in the reference.
 */
unsigned long long linf_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* LINFDIST_H_ */
