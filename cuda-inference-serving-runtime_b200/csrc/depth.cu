// Depth-weighted average of the residual stream: every layer's result is kept for the step, and what goes on to the
// next layer is a weighted sum of all results so far,
//     X_0 = the embedding,   X_(i+1) = the result of layer i,   x <- sum_(j <= i+1) w_i[j] * X_j.
//
// depth_mix_norm, a CTA per token, is the seam between two layers in one pass: it closes layer i (X_(i+1) = x + the
// pending output of the layer's last sub-block, stored as entry i + 1 of the history), forms the weighted sum in the
// order of j, stores it as the stream of the next layer, and norms it (RMS with one weight per channel) into the operand
// type of the next layer's first product.  With `rows` it does the same for picked tokens and stores nothing (the
// model's final norm).  Sums and statistics are float.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_depth_set_pdl(int on) { g_pdl = on != 0; }

namespace {
// hist [entries][tokens][hidden]; x, pending [tokens][hidden]; w [n_new + 1]; norm_w [hidden] or null (no norm: h unused)
template <typename OT>
__global__ void __launch_bounds__(256)
depth_mix_norm_kernel(float* __restrict__ hist, size_t entry_stride, float* __restrict__ x, const float* __restrict__ pending,
                      const float* __restrict__ w, int n_new, const float* __restrict__ norm_w, float eps,
                      OT* __restrict__ h, float* __restrict__ mixed_out, const int* __restrict__ rows, int hidden, int store) {
    extern __shared__ float row[];            // the mixed row
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = rows ? rows[blockIdx.x] : blockIdx.x;
    const size_t at = (size_t)t * hidden;
    float sq = 0.f;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        const float latest = pending ? x[at + d] + pending[at + d] : x[at + d];
        if (store) hist[(size_t)n_new * entry_stride + at + d] = latest;
        float acc = 0.f;
        for (int j = 0; j < n_new; ++j) acc = fmaf(w[j], hist[(size_t)j * entry_stride + at + d], acc);
        acc = fmaf(w[n_new], latest, acc);
        row[d] = acc;
        sq = fmaf(acc, acc, sq);
        if (store) x[at + d] = acc;
        if (mixed_out) mixed_out[(size_t)blockIdx.x * hidden + d] = acc;
    }
    if (!norm_w) return;
    sq = block_sum(sq, scratch);
    const float inv = 1.f / sqrtf(sq / (float)hidden + eps);
    OT* dst = h + (size_t)blockIdx.x * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = from_float<OT>(row[d] * inv * norm_w[d]);
}
}  // namespace

CISR_EXPORT int cisr_depth_mix_norm(float* hist, long long entry_stride, float* x, const float* pending, const float* w, int n_new,
                                    const float* norm_w, float eps, void* h, int h_dtype, float* mixed_out, const int* rows,
                                    int n_rows, int hidden, int store, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_new < 1 || hidden <= 0 || (size_t)hidden * sizeof(float) > 200 * 1024) return -2;
    const size_t smem = (size_t)hidden * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == CISR_BF16) {
        static size_t configured = 48 * 1024;
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(depth_mix_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = smem;
        }
        return launch_kernel(depth_mix_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), smem, s, g_pdl, hist, (size_t)entry_stride, x,
                             pending, w, n_new, norm_w, eps, (__nv_bfloat16*)h, mixed_out, rows, hidden, store);
    }
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(depth_mix_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    return launch_kernel(depth_mix_norm_kernel<float>, dim3(n_rows), dim3(256), smem, s, g_pdl, hist, (size_t)entry_stride, x, pending, w,
                         n_new, norm_w, eps, (float*)h, mixed_out, rows, hidden, store);
}
