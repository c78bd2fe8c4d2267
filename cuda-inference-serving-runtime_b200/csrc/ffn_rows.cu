// Row kernels of feed-forward layers whose activation needs a token's whole row, or pairs two products.
//
//   polynorm     act(z) = a N(z) + b N(z^2) + c N(z^3) + e over a token's row of ff values, powers element by element,
//                N(u) = u / sqrt(mean(u^2) + eps).  One pass finds the three mean squares (of z, z^2 and z^3), a second
//                writes the row.  A CTA per token, four numbers per access where the rows allow it.
//   gated_clamp  y = g' * sigmoid(alpha * g') * (u' + 1),  g' = min(g, limit),  u' = clamp(u, -limit, limit), from a row
//                [gate: ff | up: ff | ...]; an optional per-token logit at column `scale_col` multiplies the row by its
//                sigmoid (a gated shared expert: the product is linear, so the factor may be applied before it).
// Float arithmetic on the products' float sums; one rounding to the operand type of the next product.  Output rows may
// be wider than ff (zero-filled), where the next product wants its K in whole 16-byte groups.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_ffn_rows_set_pdl(int on) { g_pdl = on != 0; }

namespace {
// VEC numbers per thread and access (4: rows of whole 16-byte groups on 16-byte boundaries; 1: any width)
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

template <int VEC, typename OT>
__global__ void __launch_bounds__(1024)
polynorm_kernel(const float* __restrict__ z, int row_stride, const float* __restrict__ coef, float eps, OT* __restrict__ out,
                int ff, int out_cols) {
    __shared__ float scratch[32];
    using P = Pack<VEC>;
    pdl_trigger();
    pdl_wait();
    const float* src = z + (size_t)blockIdx.x * row_stride;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x * VEC; i < ff; i += blockDim.x * VEC) {
        const P p = *reinterpret_cast<const P*>(src + i);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float v = p.v[k], v2 = v * v, v3 = v2 * v;
            s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
        }
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float n = (float)ff;
    const float r1 = coef[0] / sqrtf(s1 / n + eps), r2 = coef[1] / sqrtf(s2 / n + eps), r3 = coef[2] / sqrtf(s3 / n + eps);
    const float e = coef[3];
    OT* dst = out + (size_t)blockIdx.x * out_cols;
    for (int i = threadIdx.x * VEC; i < out_cols; i += blockDim.x * VEC) {      // ff is a multiple of VEC: a group is inside or outside
        float y[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) y[k] = 0.f;
        if (i < ff) {
            const P p = *reinterpret_cast<const P*>(src + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) { const float v = p.v[k], v2 = v * v; y[k] = fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))); }
        }
        store_rounded<VEC, OT>(dst + i, y);
    }
}

template <int VEC, typename OT>
int launch_polynorm(const float* z, int row_stride, const float* coef, float eps, void* out, int tokens, int ff, int out_cols, cudaStream_t s) {
    int threads = ((out_cols / VEC + 31) / 32) * 32;       // one access per thread where the row allows it
    threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
    return launch_kernel(polynorm_kernel<VEC, OT>, dim3(tokens), dim3(threads), 0, s, g_pdl, z, row_stride, coef, eps, (OT*)out, ff, out_cols);
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
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = ff % 4 == 0 && out_cols % 4 == 0 && row_stride % 4 == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (out_dtype == CISR_BF16)
        return wide ? launch_polynorm<4, __nv_bfloat16>(z, row_stride, coef, eps, out, tokens, ff, out_cols, s)
                    : launch_polynorm<1, __nv_bfloat16>(z, row_stride, coef, eps, out, tokens, ff, out_cols, s);
    return wide ? launch_polynorm<4, float>(z, row_stride, coef, eps, out, tokens, ff, out_cols, s)
                : launch_polynorm<1, float>(z, row_stride, coef, eps, out, tokens, ff, out_cols, s);
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
