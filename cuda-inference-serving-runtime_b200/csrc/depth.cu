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
// VEC numbers of a row per thread and access (4: rows of whole 16-byte groups; 1: any width).
template <int VEC> struct Pack;
template <> struct Pack<1> { float v[1]; };
template <> struct __align__(16) Pack<4> { float v[4]; };

template <int VEC, typename OT> __device__ __forceinline__ void store_rounded(OT* dst, const float* y);
template <> __device__ __forceinline__ void store_rounded<1, float>(float* dst, const float* y) { dst[0] = y[0]; }
template <> __device__ __forceinline__ void store_rounded<1, __nv_bfloat16>(__nv_bfloat16* dst, const float* y) { dst[0] = __float2bfloat16_rn(y[0]); }
template <> __device__ __forceinline__ void store_rounded<4, float>(float* dst, const float* y) {
    *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
}
template <> __device__ __forceinline__ void store_rounded<4, __nv_bfloat16>(__nv_bfloat16* dst, const float* y) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
    uint2 bits;
    bits.x = *reinterpret_cast<unsigned*>(&lo);
    bits.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst) = bits;
}

// hist [entries][tokens][hidden]; x, pending [tokens][hidden]; w [n_new + 1]; norm_w [hidden] or null (no norm: h unused)
template <int VEC, typename OT>
__global__ void __launch_bounds__(1024)
depth_mix_norm_kernel(float* __restrict__ hist, size_t entry_stride, float* __restrict__ x, const float* __restrict__ pending,
                      const float* __restrict__ w, int n_new, const float* __restrict__ norm_w, float eps,
                      OT* __restrict__ h, float* __restrict__ mixed_out, const int* __restrict__ rows, int hidden, int store) {
    extern __shared__ __align__(16) float row[];            // the mixed row
    __shared__ float scratch[32];
    using P = Pack<VEC>;
    pdl_trigger();
    pdl_wait();
    const int t = rows ? rows[blockIdx.x] : blockIdx.x;
    const size_t at = (size_t)t * hidden;
    float sq = 0.f;
    for (int d = threadIdx.x * VEC; d < hidden; d += blockDim.x * VEC) {
        P latest = *reinterpret_cast<const P*>(x + at + d);
        if (pending) {
            const P p = *reinterpret_cast<const P*>(pending + at + d);
#pragma unroll
            for (int i = 0; i < VEC; ++i) latest.v[i] += p.v[i];
        }
        P acc;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc.v[i] = 0.f;
#pragma unroll 4
        for (int j = 0; j < n_new; ++j) {                   // in the order of j, whatever the access width
            const P e = *reinterpret_cast<const P*>(hist + (size_t)j * entry_stride + at + d);
            const float wj = w[j];
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc.v[i] = fmaf(wj, e.v[i], acc.v[i]);
        }
        if (store) *reinterpret_cast<P*>(hist + (size_t)n_new * entry_stride + at + d) = latest;      // after the loads of the older entries
        const float wl = w[n_new];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            acc.v[i] = fmaf(wl, latest.v[i], acc.v[i]);
            sq = fmaf(acc.v[i], acc.v[i], sq);
        }
        *reinterpret_cast<P*>(row + d) = acc;
        if (store) *reinterpret_cast<P*>(x + at + d) = acc;
        if (mixed_out) *reinterpret_cast<P*>(mixed_out + (size_t)blockIdx.x * hidden + d) = acc;
    }
    if (!norm_w) return;
    sq = block_sum(sq, scratch);
    const float inv = 1.f / sqrtf(sq / (float)hidden + eps);
    OT* dst = h + (size_t)blockIdx.x * hidden;
    for (int d = threadIdx.x * VEC; d < hidden; d += blockDim.x * VEC) {
        const P m = *reinterpret_cast<const P*>(row + d), g = *reinterpret_cast<const P*>(norm_w + d);
        float y[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) y[i] = m.v[i] * inv * g.v[i];
        store_rounded<VEC, OT>(dst + d, y);
    }
}

template <int VEC, typename OT>
int launch_depth(float* hist, long long entry_stride, float* x, const float* pending, const float* w, int n_new, const float* norm_w,
                 float eps, void* h, float* mixed_out, const int* rows, int n_rows, int hidden, int store, cudaStream_t s) {
    const size_t smem = (size_t)hidden * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(depth_mix_norm_kernel<VEC, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    int threads = ((hidden / VEC + 31) / 32) * 32;         // one access per thread where the row allows it
    threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
    return launch_kernel(depth_mix_norm_kernel<VEC, OT>, dim3(n_rows), dim3(threads), smem, s, g_pdl, hist, (size_t)entry_stride, x,
                         pending, w, n_new, norm_w, eps, (OT*)h, mixed_out, rows, hidden, store);
}
}  // namespace

CISR_EXPORT int cisr_depth_mix_norm(float* hist, long long entry_stride, float* x, const float* pending, const float* w, int n_new,
                                    const float* norm_w, float eps, void* h, int h_dtype, float* mixed_out, const int* rows,
                                    int n_rows, int hidden, int store, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_new < 1 || hidden <= 0 || (size_t)hidden * sizeof(float) > 200 * 1024) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    // rows of whole 16-byte groups on 16-byte boundaries take the four-wide form
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool wide = hidden % 4 == 0 && entry_stride % 4 == 0 && aligned(hist) && aligned(x) && aligned(pending) && aligned(norm_w)
                      && aligned(h) && aligned(mixed_out);
    if (h_dtype == CISR_BF16)
        return wide ? launch_depth<4, __nv_bfloat16>(hist, entry_stride, x, pending, w, n_new, norm_w, eps, h, mixed_out, rows, n_rows, hidden, store, s)
                    : launch_depth<1, __nv_bfloat16>(hist, entry_stride, x, pending, w, n_new, norm_w, eps, h, mixed_out, rows, n_rows, hidden, store, s);
    return wide ? launch_depth<4, float>(hist, entry_stride, x, pending, w, n_new, norm_w, eps, h, mixed_out, rows, n_rows, hidden, store, s)
                : launch_depth<1, float>(hist, entry_stride, x, pending, w, n_new, norm_w, eps, h, mixed_out, rows, n_rows, hidden, store, s);
}
