// Row kernels of differential attention: two softmax maps per head over the same values, combined as
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale,   o <- o * sigmoid(gate)   (the gate may be absent)
// with q, k and v passing a short causal convolution over time right after their projection, or (no convolution) with the
// leading coordinates of each map of q and k turned to the token's position.
//
// The two maps run on the engine's paged attention kernels as two query heads each (2 * heads query heads over kv_heads
// key heads of one width D): a key row of the cache holds [k of map 1 | k of map 2 | zeros], a query row of map m holds
// its dk numbers at columns [m * dk, (m + 1) * dk) and zeros elsewhere, so q' . k' is exactly q_m . k_m (products with
// zero add nothing), and the values are stored once per key head.
//
//   diff_rows     per token: convolution of the q (, k, v) channels of the step's stacked projection (inputs before the
//                 portion come from the request's kept inputs, zeros before the sequence), query rows in the layout
//                 above, key and value rows into the request's cache pages.
//   diff_rope_rows  the same rows without a convolution: each map's first 2 * rot_half coordinates of q and k turn by the
//                 step's rotary tables (either pairing); values pass as they are.
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

constexpr int kSlideTaps = 8;   // most taps whose inputs a lane carries from token to token in registers

// One lane's two neighbouring outputs (channels c0 and c1 of proj; a negative channel is a zero of the padded row) for
// the n_tok <= CHUNK tokens from t0 on, handed to dst(i, y0, y1), which stores them.  The lane first issues the loads
// of all its inputs of the run (the tokens' and the taps - 1 before them), so that a warp has a run of loads in flight
// and not one, and then forms every token's sum from registers.  A token whose bit in `refill` is set (its portion began
// fewer than taps - 1 tokens before it; with CHUNK 1, every token) is left to a second pass that fetches its inputs from
// the portion or from the request's kept rows.  Lane i of the warp holds token i's request and place in its portion.
// The taps are added oldest first in both passes.  TAPS < kSlideTaps: exactly TAPS taps; TAPS == kSlideTaps: `taps` of
// them, up to kSlideTaps.  Every lane of the warp calls this together.
template <typename T, int TAPS, int CHUNK, typename Dst>
__device__ __forceinline__ void conv_pair_run(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w,
                                              const float* __restrict__ state, long long state_stride,
                                              const int* __restrict__ req_slot, int channels, int taps, int t0, int n_tok,
                                              unsigned refill, int my_req, int my_local, int c0, int c1, Dst dst) {
    const int n = TAPS < kSlideTaps ? TAPS : taps;
    constexpr int HALO = TAPS - 1;
    float w0[TAPS], w1[TAPS];                              // index j: the weight of the input j tokens back
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
        const bool tap = j < n;
        w0[j] = tap && c0 >= 0 ? conv_w[(size_t)(n - 1 - j) * channels + c0] : 0.f;
        w1[j] = tap && c1 >= 0 ? conv_w[(size_t)(n - 1 - j) * channels + c1] : 0.f;
    }
    if (CHUNK > 1) {
        const bool both = c0 >= 0 && c1 == c0 + 1 && ((c0 | row_stride) & 1) == 0 && (reinterpret_cast<uintptr_t>(proj) & 7) == 0;
        float x0[CHUNK + HALO], x1[CHUNK + HALO];          // index HALO + i: token i's input; below HALO: those before t0
#pragma unroll
        for (int k = 0; k < CHUNK + HALO; ++k) {
            const int i = k - HALO;
            const bool in = i >= 0 ? i < n_tok : (-i < n && t0 + i >= 0);
            x0[k] = 0.f; x1[k] = 0.f;
            if (in && (c0 >= 0 || c1 >= 0)) {
                const float* row = proj + (size_t)(t0 + i) * row_stride;
                if (both) {
                    const float2 v = *reinterpret_cast<const float2*>(row + c0);
                    x0[k] = v.x; x1[k] = v.y;
                } else {
                    if (c0 >= 0) x0[k] = row[c0];
                    if (c1 >= 0) x1[k] = row[c1];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) {
            if (i < n_tok && !((refill >> i) & 1u)) {
                float y0 = 0.f, y1 = 0.f;
#pragma unroll
                for (int j = TAPS - 1; j >= 0; --j) {
                    if (j < n) { y0 = fmaf(w0[j], x0[HALO + i - j], y0); y1 = fmaf(w1[j], x1[HALO + i - j], y1); }
                }
                dst(i, y0, y1);
            }
        }
    }
    for (unsigned left = refill & (n_tok >= 32 ? 0xffffffffu : (1u << n_tok) - 1u); left != 0; left &= left - 1) {
        const int i = __ffs(left) - 1;
        const int req = __shfl_sync(0xffffffffu, my_req, i);
        const int local = __shfl_sync(0xffffffffu, my_local, i);
        const float* keep = state + (size_t)req_slot[req] * state_stride;
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int j = TAPS - 1; j >= 0; --j) {
            if (j < n) {
                const int at = local - j;
                const float* src = at >= 0 ? proj + (size_t)(t0 + i - j) * row_stride : keep + (size_t)(n - 1 + at) * channels;
                if (c0 >= 0) y0 = fmaf(w0[j], src[c0], y0);
                if (c1 >= 0) y1 = fmaf(w1[j], src[c1], y1);
            }
        }
        dst(i, y0, y1);
    }
}

// proj [tokens, row_stride] float; its first `channels` columns are the convolved ones: [q: hq * 2 * dk] and, when
// write_kv, [k: hkv * 2 * dk][v: hkv * dv].  state: a request's row is [taps - 1][channels].
// A CTA takes `chunk` <= CHUNK neighbouring tokens of the step (of whichever requests).  A warp per run of `width` columns
// (the query rows, then hkv key rows with their value rows), two neighbouring numbers per lane, token after token;
// blockIdx.y shares the runs among CTAs.  width is even.
template <typename T, int TAPS, int CHUNK>
__global__ void __launch_bounds__(256, 3)
diff_rows_kernel(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w, int taps,
                 const float* __restrict__ state, long long state_stride, const int* __restrict__ token_req,
                 const int* __restrict__ req_slot, const int* __restrict__ q_start, const int* __restrict__ positions,
                 T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                 int table_width, int page_size, int tokens, int chunk, int hq, int hkv, int dk, int dv, int width, int write_kv) {
    pdl_trigger();
    const int t0 = blockIdx.x * chunk;
    const int n_tok = (t0 + chunk < tokens ? t0 + chunk : tokens) - t0;
    const int nq = hq * 2 * dk, nk = hkv * 2 * dk;
    const int channels = nq + (write_kv ? nk + hkv * dv : 0);
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // with an even dk one run of a warp makes both maps' rows of a head (their channels are neighbours in proj)
    const bool packed = (dk & 1) == 0;
    const int q_runs = packed ? hq : 2 * hq;
    const int rows = q_runs + (write_kv ? hkv : 0);
    pdl_wait();
    // lane i learns of token i: its request, its place in the portion and the row of the pages that is its own
    // (none for a padding row of a fixed-size batch, whose slot has no pages)
    int my_req = 0, my_local = 0, my_place = -1;
    if (lane < n_tok) {
        const int t = t0 + lane;
        my_req = token_req[t];
        my_local = t - q_start[my_req];
        if (write_kv) {
            const int pos = positions[t];
            const int page = block_table[(size_t)req_slot[my_req] * table_width + pos / page_size];
            if (page >= 0) my_place = page * hkv * page_size + pos % page_size;
        }
    }
    const unsigned refill = CHUNK > 1 ? __ballot_sync(0xffffffffu, lane < n_tok && my_local < taps - 1) : 0xffffffffu;
    const size_t step = (size_t)2 * hq * width;            // from a token's query rows to the next token's
    for (int row = blockIdx.y * warps + (threadIdx.x >> 5); row < rows; row += gridDim.y * warps) {
#pragma unroll 1
        for (int d0 = 0; d0 < width; d0 += 64) {
            const int d = d0 + 2 * lane;
            const bool mine = d < width;
            if (row < q_runs && packed) {
                // head `row`: column d < dk belongs to map 1 (query row 2 h), dk <= d < 2 dk to map 2 (row 2 h + 1); the
                // lane writes its numbers into the row of their map and zeros into the other row's same columns
                const bool real = mine && d < 2 * dk;
                const int m = real && d >= dk ? 1 : 0;
                T* value = q_out + ((size_t)t0 * 2 * hq + 2 * row + m) * width + d;
                T* zeros = q_out + ((size_t)t0 * 2 * hq + 2 * row + 1 - m) * width + d;
                conv_pair_run<T, TAPS, CHUNK>(proj, row_stride, conv_w, state, state_stride, req_slot, channels, taps, t0, n_tok, refill,
                                              my_req, my_local, real ? 2 * row * dk + d : -1, real ? 2 * row * dk + d + 1 : -1,
                                              [&](int i, float y0, float y1) {
                                                  if (!mine) return;
                                                  store_pair<T>(value + i * step, y0, y1);
                                                  store_pair<T>(zeros + i * step, 0.f, 0.f);
                                              });
            } else if (row < q_runs) {
                // query rows: head pair (h, m) is row 2 h + m, its numbers at columns [m * dk, (m + 1) * dk)
                const int a0 = d - (row & 1) * dk, a1 = a0 + 1;
                T* to = q_out + ((size_t)t0 * 2 * hq + row) * width + d;
                conv_pair_run<T, TAPS, CHUNK>(proj, row_stride, conv_w, state, state_stride, req_slot, channels, taps, t0, n_tok, refill,
                                              my_req, my_local, mine && a0 >= 0 && a0 < dk ? row * dk + a0 : -1,
                                              mine && a1 >= 0 && a1 < dk ? row * dk + a1 : -1,
                                              [&](int i, float y0, float y1) { if (mine) store_pair<T>(to + i * step, y0, y1); });
            } else {
                const int g = row - q_runs;
                const int kc = nq + g * 2 * dk, vc = nq + nk + g * dv;
                auto place = [&](T* cache, int i, float y0, float y1) {
                    const int at = __shfl_sync(0xffffffffu, my_place, i);
                    if (mine && at >= 0) store_pair<T>(cache + ((size_t)at + (size_t)g * page_size) * width + d, y0, y1);
                };
                conv_pair_run<T, TAPS, CHUNK>(proj, row_stride, conv_w, state, state_stride, req_slot, channels, taps, t0, n_tok, refill,
                                              my_req, my_local, mine && d < 2 * dk ? kc + d : -1, mine && d + 1 < 2 * dk ? kc + d + 1 : -1,
                                              [&](int i, float y0, float y1) { place(k_cache, i, y0, y1); });
                conv_pair_run<T, TAPS, CHUNK>(proj, row_stride, conv_w, state, state_stride, req_slot, channels, taps, t0, n_tok, refill,
                                              my_req, my_local, mine && d < dv ? vc + d : -1, mine && d + 1 < dv ? vc + d + 1 : -1,
                                              [&](int i, float y0, float y1) { place(v_cache, i, y0, y1); });
            }
        }
    }
}

// Any number of taps: a CTA per token (blockIdx.y shares its rows), every input fetched for every token that reads it.
template <typename T>
__global__ void __launch_bounds__(256)
diff_rows_long_kernel(const float* __restrict__ proj, int row_stride, const float* __restrict__ conv_w, int taps,
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
    const float* g = gate ? gate + (size_t)t * row_stride + gate_col + h * dv : nullptr;      // no gate: the factor is 1
    T* dst = out + ((size_t)t * hq + h) * dv;
    for (int d = lane; d < dv; d += 32) {
        const float o = to_float(a1[d]) - lambda * to_float(a2[d]);
        dst[d] = from_float<T>(g ? o * inv / (1.f + expf(-g[d])) : o * inv);
    }
}

// The same with two neighbouring numbers per lane and access (dv, width, row_stride and gate_col even): a head's
// combination stays in registers between the sum of squares and the store, up to kCombineKeep pairs per lane.
constexpr int kCombineKeep = 4;
template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
};

template <typename T>
__global__ void __launch_bounds__(256)
diff_combine_pairs_kernel(const T* __restrict__ mixed, const float* __restrict__ gate, int row_stride, int gate_col,
                          T* __restrict__ out, int tokens, int hq, int dv, int width, float lambda, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= tokens * hq) return;
    const int t = pair / hq, h = pair - t * hq;
    const T* a1 = mixed + ((size_t)t * 2 * hq + 2 * h) * width;
    const T* a2 = a1 + width;
    const float* g = gate ? gate + (size_t)t * row_stride + gate_col + h * dv : nullptr;      // no gate: a logit of +inf, a factor of 1
    float2 o[kCombineKeep], gl[kCombineKeep];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kCombineKeep; ++i) {
        const int d = 2 * lane + 64 * i;
        o[i] = make_float2(0.f, 0.f); gl[i] = o[i];
        if (d < dv) {
            const float2 x = Pair<T>::load(a1 + d), y = Pair<T>::load(a2 + d);
            gl[i] = g ? *reinterpret_cast<const float2*>(g + d) : make_float2(INFINITY, INFINITY);
            o[i] = make_float2(x.x - lambda * y.x, x.y - lambda * y.y);
            sq = fmaf(o[i].x, o[i].x, sq);
            sq = fmaf(o[i].y, o[i].y, sq);
        }
    }
    sq = warp_sum(sq);
    const float inv = out_scale / sqrtf(sq / (float)dv + eps);
    T* dst = out + ((size_t)t * hq + h) * dv;
#pragma unroll
    for (int i = 0; i < kCombineKeep; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < dv) store_pair<T>(dst + d, o[i].x * inv / (1.f + expf(-gl[i].x)), o[i].y * inv / (1.f + expf(-gl[i].y)));
    }
}

// Coordinate d of a map whose float coordinates are src[0 ..): turned by the token's tables when d < 2 * rot_half.
__device__ __forceinline__ float turned(const float* __restrict__ src, int d, int rot_half, int interleaved,
                                        const float* __restrict__ cs, const float* __restrict__ sn) {
    if (d >= 2 * rot_half) return src[d];
    int f, other; bool first;
    if (interleaved) { f = d >> 1; first = !(d & 1); other = first ? d + 1 : d - 1; }
    else { first = d < rot_half; f = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
    const float c = cs[f], s = sn[f], v = src[d], o = src[other];
    return first ? v * c - o * s : v * c + o * s;
}

// A CTA per token.  proj [T, row_stride] float: q (hq x 2 x dk) from column 0, and where the layer has keys and values of
// its own k (hkv x 2 x dk) from k_col and v (hkv x dv) from v_col.
template <typename T>
__global__ void __launch_bounds__(256)
diff_rope_rows_kernel(const float* __restrict__ proj, int row_stride, int k_col, int v_col, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int rot_half, int interleaved, const int* __restrict__ token_req,
                      const int* __restrict__ req_slot, const int* __restrict__ positions, T* __restrict__ q_out, T* __restrict__ k_cache,
                      T* __restrict__ v_cache, const int* __restrict__ block_table, int table_width, int page_size, int hq, int hkv,
                      int dk, int dv, int width, int write_kv) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * row_stride;
    const float* cs = cos_t + (size_t)t * rot_half;
    const float* sn = sin_t + (size_t)t * rot_half;
    T* q_dst = q_out + (size_t)t * 2 * hq * width;
    for (int i = threadIdx.x; i < 2 * hq * width; i += blockDim.x) {
        const int r = i / width, col = i - r * width, m = r & 1, d = col - m * dk;      // row r: map m of head r / 2
        q_dst[i] = from_float<T>(d >= 0 && d < dk ? turned(row + (size_t)r * dk, d, rot_half, interleaved, cs, sn) : 0.f);
    }
    if (!write_kv) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)req_slot[token_req[t]] * table_width + pos / page_size];
    if (page < 0) return;      // the host reserves a page before every write; never follow a missing entry
    for (int i = threadIdx.x; i < hkv * width; i += blockDim.x) {
        const int g = i / width, col = i - g * width;
        const size_t at = (((size_t)page * hkv + g) * page_size + pos % page_size) * width + col;
        float k = 0.f;
        if (col < 2 * dk) { const int m = col / dk; k = turned(row + k_col + (size_t)(2 * g + m) * dk, col - m * dk, rot_half, interleaved, cs, sn); }
        k_cache[at] = from_float<T>(k);
        v_cache[at] = from_float<T>(col < dv ? row[v_col + g * dv + col] : 0.f);
    }
}
}  // namespace

CISR_EXPORT int cisr_diff_rope_rows(const float* proj, int row_stride, int k_col, int v_col, const float* cos_t, const float* sin_t,
                                    int rot_half, int interleaved, const int* token_req, const int* req_slot, const int* positions,
                                    void* q_out, void* k_cache, void* v_cache, int dtype, const int* block_table, int table_width,
                                    int page_size, int tokens, int hq, int hkv, int dk, int dv, int width, int write_kv, void* stream) {
    if (tokens <= 0) return 0;
    if (width < 2 * dk || width < dv || 2 * rot_half > dk || rot_half < 0 || hq <= 0 || hkv <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CISR_BF16)
        return launch_kernel(diff_rope_rows_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, s, g_pdl, proj, row_stride, k_col, v_col, cos_t,
                             sin_t, rot_half, interleaved, token_req, req_slot, positions, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, block_table, table_width, page_size, hq, hkv, dk, dv, width, write_kv);
    return launch_kernel(diff_rope_rows_kernel<float>, dim3(tokens), dim3(256), 0, s, g_pdl, proj, row_stride, k_col, v_col, cos_t, sin_t,
                         rot_half, interleaved, token_req, req_slot, positions, (float*)q_out, (float*)k_cache, (float*)v_cache, block_table,
                         table_width, page_size, hq, hkv, dk, dv, width, write_kv);
}

CISR_EXPORT int cisr_diff_rows(const float* proj, int row_stride, const float* conv_w, int taps, const float* state,
                               long long state_stride, const int* token_req, const int* req_slot, const int* q_start,
                               const int* positions, void* q_out, void* k_cache, void* v_cache, int dtype, const int* block_table,
                               int table_width, int page_size, int tokens, int hq, int hkv, int dk, int dv, int width, int write_kv,
                               void* stream) {
    if (tokens <= 0) return 0;
    if (taps < 1 || width < 2 * dk || width < dv || width % 2 || hq <= 0 || hkv <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    // eight rows per CTA.  A large step gives a CTA up to sixteen neighbouring tokens, whose inputs it then reads once;
    // a small one keeps a token per CTA and shares its rows among as many CTAs as bring the launch to about two per SM.
    int share = (2 * hq + (write_kv ? hkv : 0) + 7) / 8;
    if (taps > kSlideTaps) {
        const int want = (296 + tokens - 1) / tokens;
        const dim3 grid(tokens, share < want ? share : want);
        if (dtype == CISR_BF16)
            return launch_kernel(diff_rows_long_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w, taps,
                                 state, state_stride, token_req, req_slot, q_start, positions, (__nv_bfloat16*)q_out,
                                 (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, block_table, table_width, page_size, hq, hkv, dk, dv,
                                 width, write_kv);
        return launch_kernel(diff_rows_long_kernel<float>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w, taps, state,
                             state_stride, token_req, req_slot, q_start, positions, (float*)q_out, (float*)k_cache, (float*)v_cache,
                             block_table, table_width, page_size, hq, hkv, dk, dv, width, write_kv);
    }
    share = (((dk & 1) == 0 ? hq : 2 * hq) + (write_kv ? hkv : 0) + 7) / 8;   // an even dk: a run per head makes both maps' rows
    long long chunk = (long long)tokens * share / 592;
    chunk = chunk > 16 ? 16 : chunk < 1 ? 1 : chunk;
    if (chunk == 1) {
        const int want = (296 + tokens - 1) / tokens;
        share = share < want ? share : want;
    }
    const dim3 grid((unsigned)((tokens + chunk - 1) / chunk), share < 1 ? 1 : share);
#define CISR_DIFF_ROWS_OF(TAPS, CHUNK)                                                                                          \
    return dtype == CISR_BF16                                                                                                   \
        ? launch_kernel(diff_rows_kernel<__nv_bfloat16, TAPS, CHUNK>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w,   \
                        taps, state, state_stride, token_req, req_slot, q_start, positions, (__nv_bfloat16*)q_out,              \
                        (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, block_table, table_width, page_size, tokens,          \
                        (int)chunk, hq, hkv, dk, dv, width, write_kv)                                                           \
        : launch_kernel(diff_rows_kernel<float, TAPS, CHUNK>, grid, dim3(256), 0, s, g_pdl, proj, row_stride, conv_w, taps,     \
                        state, state_stride, token_req, req_slot, q_start, positions, (float*)q_out, (float*)k_cache,           \
                        (float*)v_cache, block_table, table_width, page_size, tokens, (int)chunk, hq, hkv, dk, dv, width,       \
                        write_kv)
#define CISR_DIFF_ROWS(TAPS)                        \
    if (chunk > 1) { CISR_DIFF_ROWS_OF(TAPS, 16); } \
    CISR_DIFF_ROWS_OF(TAPS, 1)
    switch (taps) {
        case 1: CISR_DIFF_ROWS(1);
        case 2: CISR_DIFF_ROWS(2);
        case 3: CISR_DIFF_ROWS(3);
        case 4: CISR_DIFF_ROWS(4);
        default: CISR_DIFF_ROWS(kSlideTaps);
    }
#undef CISR_DIFF_ROWS
#undef CISR_DIFF_ROWS_OF
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
    const bool even = ((dv | width | row_stride | gate_col) & 1) == 0 && dv <= 64 * kCombineKeep &&
                      ((reinterpret_cast<uintptr_t>(mixed) | reinterpret_cast<uintptr_t>(out)) & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(gate) & 7) == 0;
    if (even) {
        if (dtype == CISR_BF16)
            return launch_kernel(diff_combine_pairs_kernel<__nv_bfloat16>, dim3((pairs + 7) / 8), dim3(256), 0, s, g_pdl,
                                 (const __nv_bfloat16*)mixed, gate, row_stride, gate_col, (__nv_bfloat16*)out, tokens, hq, dv, width,
                                 lambda, eps, out_scale);
        return launch_kernel(diff_combine_pairs_kernel<float>, dim3((pairs + 7) / 8), dim3(256), 0, s, g_pdl, (const float*)mixed, gate,
                             row_stride, gate_col, (float*)out, tokens, hq, dv, width, lambda, eps, out_scale);
    }
    if (dtype == CISR_BF16)
        return launch_kernel(diff_combine_kernel<__nv_bfloat16>, dim3((pairs + 3) / 4), dim3(128), 0, s, g_pdl, (const __nv_bfloat16*)mixed,
                             gate, row_stride, gate_col, (__nv_bfloat16*)out, tokens, hq, dv, width, lambda, eps, out_scale);
    return launch_kernel(diff_combine_kernel<float>, dim3((pairs + 3) / 4), dim3(128), 0, s, g_pdl, (const float*)mixed, gate, row_stride,
                         gate_col, (float*)out, tokens, hq, dv, width, lambda, eps, out_scale);
}
