// C entry points around the reference's own CUDA launchers, so that the unmodified reference
// kernels can be called from the GPU tests and timed by bench.py as "the kernel to beat".
//
// TEST INFRASTRUCTURE ONLY.  This file holds no reference code: it declares the seven C++
// launchers whose prototypes the reference's binding lists (model/norm_dist.cpp:7-20) and
// forwards to them.  oracle/build.py compiles it TOGETHER WITH the reference's two .cu files
// where they lie (model/inf_dist_cuda.cu, model/norm_dist_cuda.cu) into
// oracle/_ref/libref_norm_dist.so.  The reference launches on the legacy default stream and
// expects zero-filled gradient buffers for its atomicAdd kernels.
void norm_dist_forward_cuda(const float*, const float*, int, int, int, int, int, float*, float);
void norm_dist_backward_input_cuda(const float*, const float*, const float*, const float*,
                                   int, int, int, int, int, float*, float);
void norm_dist_backward_weight_cuda(const float*, const float*, const float*, const float*,
                                    int, int, int, int, int, float*, float);
void inf_dist_forward_cuda(const float*, const float*, int, int, int, int, int, float*, int*);
void inf_dist_bound_forward_cuda(const float*, const float*, const float*, int, int, int, int, int,
                                 float*, float*);
void inf_dist_backward_input_cuda(const float*, const int*, int, int, int, int, int, float*);
void inf_dist_backward_weight_cuda(const float*, const int*, int, int, int, int, int, float*);

extern "C" {
void ref_norm_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                           float* y, float p) { norm_dist_forward_cuda(x, w, B, CO, CI, G, HW, y, p); }
void ref_norm_dist_backward_input(const float* g, const float* x, const float* w, const float* y,
                                  int B, int CO, int CI, int G, int HW, float* gx, float p) {
    norm_dist_backward_input_cuda(g, x, w, y, B, CO, CI, G, HW, gx, p);
}
void ref_norm_dist_backward_weight(const float* g, const float* x, const float* w, const float* y,
                                   int B, int CO, int CI, int G, int HW, float* gw, float p) {
    norm_dist_backward_weight_cuda(g, x, w, y, B, CO, CI, G, HW, gw, p);
}
void ref_inf_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                          float* y, int* pos) { inf_dist_forward_cuda(x, w, B, CO, CI, G, HW, y, pos); }
void ref_inf_dist_bound_forward(const float* xl, const float* xu, const float* w,
                                int B, int CO, int CI, int G, int HW, float* yl, float* yu) {
    inf_dist_bound_forward_cuda(xl, xu, w, B, CO, CI, G, HW, yl, yu);
}
void ref_inf_dist_backward_input(const float* g, const int* pos, int B, int CO, int CI, int G, int HW,
                                 float* gx) { inf_dist_backward_input_cuda(g, pos, B, CO, CI, G, HW, gx); }
void ref_inf_dist_backward_weight(const float* g, const int* pos, int B, int CO, int CI, int G, int HW,
                                  float* gw) { inf_dist_backward_weight_cuda(g, pos, B, CO, CI, G, HW, gw); }
}
