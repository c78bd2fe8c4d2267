// Row kernels of differential attention: two softmax maps per head over the same values, combined as
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale,   o <- o * sigmoid(gate)
// with q, k and v passing a short causal convolution over time right after their projection.
//
// The two maps run on the engine's paged attention kernels as two query heads each (2 * heads query heads over kv_heads
// key heads of one width D): a key row of the cache holds [k of map 1 | k of map 2 | zeros], a query row of map m holds
// its dk numbers at columns [m * dk, (m + 1) * dk) and zeros elsewhere, so q' . k' is exactly q_m . k_m (products with
// zero add nothing), and the values are stored once per key head.
//
//   diff_rows     per token: convolution of the q (, k, v) channels of the step's stacked projection (inputs before the
//                 portion come from the request's kept inputs, zeros before the sequence), query rows in the layout
//                 above, key and value rows into the request's cache pages.
//   conv_keep     per request: the last taps - 1 convolution inputs become the request's kept inputs.
//   diff_combine  per (token, head): the combination, the norm over the head's values and the gate, rounded once to the
//                 operand type of the output projection.
// Convolution, norm, sigmoid and the combination are float whatever the storage type.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_diff_set_pdl(int on) { g_pdl = on != 0; }

namespace {
// y_t[c] = sum_j w[j][c] * u_(t - taps + 1 + j)[c], w stored tap by tap [taps][channels] so that a warp's lanes read
// neighbouring weights; `local` is the token's index inside its portion.
__device__ __forceinline__ float conv_at(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w,
                                         const float* __restrict__ keep, int channels, int taps, int t, int local, int c) {
    float acc = 0.f;
    for (int j = taps - 1; j >= 0; --j) {                 // oldest input first
        const int at = local - j;
        const float x = at >= 0 ? proj[(size_t)(t - j) * row_stride + c] : keep[(size_t)(taps - 1 + at) * channels + c];
        acc = fmaf(conv_w[(size_t)(taps - 1 - j) * channels + c], x, acc);
    }
    return acc;
}

template <typename T> __device__ __forceinline__ void store_pair(T* dst, float a, float b);
template <> __device__ __forceinline__ void store_pair<float>(float* dst, float a, float b) { *reinterpret_cast<float2*>(dst) = make_float2(a, b); }
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
}

// proj [tokens, row_stride] float; its first `channels` columns are the convolved ones: [q: hq * 2 * dk] and, when
// write_kv, [k: hkv * 2 * dk][v: hkv * dv].  keep: the request's row of the state tensor, [taps - 1][channels].
// A warp per row of `width` numbers (2 * hq query rows, then hkv key rows with their value rows), two neighbouring
// numbers per lane; blockIdx.y shares a token's rows among CTAs where a step has few tokens.  width is even.
template <typename T>
__global__ void __launch_bounds__(256)
diff_rows_kernel(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w, int taps,
                 const float* __restrict__ state, long long state_stride, const int* __restrict__ token_req,
                 const int* __restrict__ req_slot, const int* __restrict__ q_start, const int* __restrict__ positions,
                 T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                 int table_width, int page_size, int hq, int hkv, int dk, int dv, int width, int write_kv) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int req = token_req[t];
    const int slot = req_slot[req];
    const int local = t - q_start[req];
    const int pos = positions[t];
    const float* keep = state + (size_t)slot * state_stride;
    const int nq = hq * 2 * dk, nk = hkv * 2 * dk;
    const int channels = nq + (write_kv ? nk + hkv * dv : 0);
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    pdl_wait();
    int page = -1;                                         // a padding row of a fixed-size batch: its slot holds no pages
    if (write_kv) page = block_table[(size_t)slot * table_width + pos / page_size];
    const int rows = 2 * hq + (page >= 0 ? hkv : 0);
    T* q_row = q_out + (size_t)t * 2 * hq * width;
    for (int row = blockIdx.y * warps + (threadIdx.x >> 5); row < rows; row += gridDim.y * warps) {
        if (row < 2 * hq) {
            // query rows: head pair (h, m) is row 2 h + m, its numbers at columns [m * dk, (m + 1) * dk)
            const int first = (row & 1) * dk;
            for (int d = 2 * lane; d < width; d += 64) {
                float y[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int at = d + i - first;
                    y[i] = at >= 0 && at < dk ? conv_at(proj, row_stride, conv_w, keep, channels, taps, t, local, row * dk + at) : 0.f;
                }
                store_pair<T>(q_row + (size_t)row * width + d, y[0], y[1]);
            }
        } else {
            const int g = row - 2 * hq;
            const size_t dst = ((size_t)page * hkv * page_size + (size_t)g * page_size + pos % page_size) * width;
            for (int d = 2 * lane; d < width; d += 64) {
                float kk[2], vv[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int e = d + i;
                    kk[i] = e < 2 * dk ? conv_at(proj, row_stride, conv_w, keep, channels, taps, t, local, nq + g * 2 * dk + e) : 0.f;
                    vv[i] = e < dv ? conv_at(proj, row_stride, conv_w, keep, channels, taps, t, local, nq + nk + g * dv + e) : 0.f;
                }
                store_pair<T>(k_cache + dst + d, kk[0], kk[1]);
                store_pair<T>(v_cache + dst + d, vv[0], vv[1]);
            }
        }
    }
}

// keep [taps - 1][channels], oldest first; a channel is one thread's: it reads what it needs of the old rows before it
// overwrites them (rows move towards 0).
__global__ void conv_keep_kernel(const float* __restrict__ proj, int row_stride, float* __restrict__ state, long long state_stride,
                                 const int* __restrict__ req_slot, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                 int taps, int channels) {
    pdl_trigger();
    pdl_wait();
    const int req = blockIdx.x;
    float* keep = state + (size_t)req_slot[req] * state_stride;
    const int n = q_len[req], first = q_start[req], kept = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        for (int i = 0; i < kept; ++i) {
            const int at = n - kept + i;                  // index in the portion of the input that lands in row i
            keep[(size_t)i * channels + c] = at >= 0 ? proj[(size_t)(first + at) * row_stride + c] : keep[(size_t)(i + n) * channels + c];
        }
    }
}

// mixed [tokens, 2 * hq, width]: rows 2 h and 2 h + 1 are head h's two maps (their first dv columns count).
// gate: float, row_stride apart, head h's dv logits at gate_col + h * dv.  out [tokens, hq * dv].  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ mixed, const float* __restrict__ gate, int row_stride, int gate_col,
                    T* __restrict__ out, int tokens, int hq, int dv, int width, float lambda, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= tokens * hq) return;
    const int t = pair / hq, h = pair - t * hq;
    const T* a1 = mixed + ((size_t)t * 2 * hq + 2 * h) * width;
    const T* a2 = a1 + width;
    float sq = 0.f;
    for (int d = lane; d < dv; d += 32) {
        const float o = to_float(a1[d]) - lambda * to_float(a2[d]);
        sq = fmaf(o, o, sq);
    }
    sq = warp_sum(sq);
    const float inv = out_scale / sqrtf(sq / (float)dv + eps);
    const float* g = gate + (size_t)t * row_stride + gate_col + h * dv;
    T* dst = out + ((size_t)t * hq + h) * dv;
    for (int d = lane; d < dv; d += 32) {
        const float o = to_float(a1[d]) - lambda * to_float(a2[d]);
        dst[d] = from_float<T>(o * inv / (1.f + expf(-g[d])));
    }
}
}  // namespace

CISR_EXPORT int cisr_diff_rows(const float* proj, int row_stride, const float* conv_w, int taps, const float* state,
                               long long state_stride, const int* token_req, const int* req_slot, const int* q_start,
                               const int* positions, void* q_out, void* k_cache, void* v_cache, int dtype, const int* block_table,
                               int table_width, int page_size, int tokens, int hq, int hkv, int dk, int dv, int width, int write_kv,
                               void* stream) {
    if (tokens <= 0) return 0;
    if (taps < 1 || width < 2 * dk || width < dv || width % 2 || hq <= 0 || hkv <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    // eight rows per CTA; as many CTAs per token as bring a small step to about two per SM
    const int rows = 2 * hq + (write_kv ? hkv : 0);
    int share = (rows + 7) / 8, want = (296 + tokens - 1) / tokens;
    share = share < want ? share : want;
    const dim3 grid(tokens, share < 1 ? 1 : share);
    if (dtype == CISR_BF16)
        return launch_kernel(diff_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w, taps, state,
                             state_stride, token_req, req_slot, q_start, positions, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, block_table, table_width, page_size, hq, hkv, dk, dv, width, write_kv);
    return launch_kernel(diff_rows_kernel<float>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w, taps, state, state_stride,
                         token_req, req_slot, q_start, positions, (float*)q_out, (float*)k_cache, (float*)v_cache, block_table,
                         table_width, page_size, hq, hkv, dk, dv, width, write_kv);
}

CISR_EXPORT int cisr_conv_keep(const float* proj, int row_stride, float* state, long long state_stride, const int* req_slot,
                               const int* q_start, const int* q_len, int n_req, int taps, int channels, void* stream) {
    if (n_req <= 0 || taps <= 1) return 0;
    const int blocks_y = (channels + 255) / 256;
    return launch_kernel(conv_keep_kernel, dim3(n_req, blocks_y < 64 ? blocks_y : 64), dim3(256), 0, (cudaStream_t)stream, g_pdl, proj,
                         row_stride, state, state_stride, req_slot, q_start, q_len, taps, channels);
}

CISR_EXPORT int cisr_diff_combine(const void* mixed, const float* gate, int row_stride, int gate_col, void* out, int dtype, int tokens,
                                  int hq, int dv, int width, float lambda, float eps, float out_scale, void* stream) {
    if (tokens <= 0) return 0;
    const int pairs = tokens * hq;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CISR_BF16)
        return launch_kernel(diff_combine_kernel<__nv_bfloat16>, dim3((pairs + 3) / 4), dim3(128), 0, s, g_pdl, (const __nv_bfloat16*)mixed,
                             gate, row_stride, gate_col, (__nv_bfloat16*)out, tokens, hq, dv, width, lambda, eps, out_scale);
    return launch_kernel(diff_combine_kernel<float>, dim3((pairs + 3) / 4), dim3(128), 0, s, g_pdl, (const float*)mixed, gate, row_stride,
                         gate_col, (float*)out, tokens, hq, dv, width, lambda, eps, out_scale);
}
