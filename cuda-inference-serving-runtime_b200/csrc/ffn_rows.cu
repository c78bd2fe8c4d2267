// Row kernels of feed-forward layers whose activation needs a token's whole row, or pairs two products.
//
//   polynorm     act(z) = a N(z) + b N(z^2) + c N(z^3) + e over a token's row of ff values, powers element by element,
//                N(u) = u / sqrt(mean(u^2) + eps).  One pass finds the three mean squares (of z, z^2 and z^3), a second
//                writes the row.  A CTA per token.
//   gated_clamp  y = g' * sigmoid(alpha * g') * (u' + 1),  g' = min(g, limit),  u' = clamp(u, -limit, limit), from a row
//                [gate: ff | up: ff | ...]; an optional per-token logit at column `scale_col` multiplies the row by its
//                sigmoid (a gated shared expert: the product is linear, so the factor may be applied before it).
// Float arithmetic on the products' float sums; one rounding to the operand type of the next product.  Output rows may
// be wider than ff (zero-filled), where the next product wants its K in whole 16-byte groups.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_ffn_rows_set_pdl(int on) { g_pdl = on != 0; }

namespace {
template <typename OT>
__global__ void __launch_bounds__(256)
polynorm_kernel(const float* __restrict__ z, int row_stride, const float* __restrict__ coef, float eps, OT* __restrict__ out,
                int ff, int out_cols) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* src = z + (size_t)blockIdx.x * row_stride;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        const float v = src[i], v2 = v * v, v3 = v2 * v;
        s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float n = (float)ff;
    const float r1 = coef[0] / sqrtf(s1 / n + eps), r2 = coef[1] / sqrtf(s2 / n + eps), r3 = coef[2] / sqrtf(s3 / n + eps);
    const float e = coef[3];
    OT* dst = out + (size_t)blockIdx.x * out_cols;
    for (int i = threadIdx.x; i < out_cols; i += blockDim.x) {
        float y = 0.f;
        if (i < ff) { const float v = src[i], v2 = v * v; y = fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))); }
        dst[i] = from_float<OT>(y);
    }
}

template <typename OT>
__global__ void gated_clamp_kernel(const float* __restrict__ gu, int row_stride, int ff, float limit, float alpha, int scale_col,
                                   OT* __restrict__ out, int out_cols, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / out_cols;
    const int f = (int)(i - t * out_cols);
    float y = 0.f;
    if (f < ff) {
        const float* row = gu + t * row_stride;
        const float g = fminf(row[f], limit), u = fminf(fmaxf(row[ff + f], -limit), limit);
        y = g / (1.f + expf(-alpha * g)) * (u + 1.f);
        if (scale_col >= 0) y /= 1.f + expf(-row[scale_col]);
    }
    out[i] = from_float<OT>(y);
}
}  // namespace

CISR_EXPORT int cisr_polynorm(const float* z, int row_stride, const float* coef, float eps, void* out, int out_dtype, int tokens, int ff,
                              int out_cols, void* stream) {
    if (tokens <= 0) return 0;
    if (ff <= 0 || out_cols < ff) return -2;
    if (out_dtype == CISR_BF16)
        return launch_kernel(polynorm_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, g_pdl, z, row_stride, coef, eps,
                             (__nv_bfloat16*)out, ff, out_cols);
    return launch_kernel(polynorm_kernel<float>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, g_pdl, z, row_stride, coef, eps,
                         (float*)out, ff, out_cols);
}

CISR_EXPORT int cisr_gated_clamp(const float* gu, int row_stride, int ff, float limit, float alpha, int scale_col, void* out, int out_dtype,
                                 int rows, int out_cols, void* stream) {
    if (rows <= 0) return 0;
    if (ff <= 0 || out_cols < ff) return -2;
    const size_t total = (size_t)rows * out_cols;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (out_dtype == CISR_BF16)
        return launch_kernel(gated_clamp_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, g_pdl, gu, row_stride, ff, limit,
                             alpha, scale_col, (__nv_bfloat16*)out, out_cols, total);
    return launch_kernel(gated_clamp_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, g_pdl, gu, row_stride, ff, limit, alpha,
                         scale_col, (float*)out, out_cols, total);
}
