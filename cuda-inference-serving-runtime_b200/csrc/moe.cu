// Routed experts: a router that scores every expert per token, picks a few, and the chosen experts' small
// feed-forward layers, summed with the router's weights.
//
//   scores s = sigmoid(W_router h), or softmax(W_router h) over all router outputs
//                                                        (float sums and float arithmetic whatever the storage type)
//   a choice bias (one number per router output, may be absent) is added to the scores for the choice only
//   experts form n_groups equal groups of neighbours; a group's score is the sum of its two best members; only members
//   of the `keep` best groups can be chosen (n_groups 0: all can)
//   the `top` best open experts are chosen, weight = s * route_scale; with `renormalize` the chosen scores are first
//   divided by their sum (+ 1e-20)
//   y = sum over chosen e of weight_e * W_down_e act(W_up_e h),   act(z) = max(z, 0)^2, the exact gelu z Phi(z), or the gated form
//       act = g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit), where W_up_e stacks the
//       gate rows on the up rows ([2 ff, hidden]) and alpha = 1.702
//   router outputs beyond the experts that have matrices are identity experts: their output is the token's input h
//
// Two shapes of the expert products.  Few tokens (and the float path): a warp per output feature, each chosen expert's
// rows streamed once per token that chose it (moe_up_rows / moe_down_rows).  Many tokens in bfloat16: the pairs are
// sorted by expert on the device (moe_sort), the activations gathered into that order (moe_gather), the two products run
// as grouped tcgen05 products (gemm_tcgen05.cu, the first with the activation as its epilogue), and each token's rows
// are summed with the router's weights (moe_combine).
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_moe_set_pdl(int on) { g_pdl = on != 0; }

// Dot product of two rows of n values, the warp's lanes striding over them; 16-byte loads where the rows allow.
__device__ __forceinline__ float warp_dot(const float* __restrict__ a, const float* __restrict__ b, int n, int lane) {
    float acc = 0.f;
    if (!(n & 3) && !(((uintptr_t)a | (uintptr_t)b) & 15)) {
        const float4* a4 = reinterpret_cast<const float4*>(a);
        const float4* b4 = reinterpret_cast<const float4*>(b);
        for (int i = lane; i < (n >> 2); i += 32) {
            const float4 x = a4[i], y = b4[i];
            acc += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
        }
    } else {
        for (int i = lane; i < n; i += 32) acc += a[i] * b[i];
    }
    return warp_sum(acc);
}
__device__ __forceinline__ float warp_dot(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, int n, int lane) {
    float acc = 0.f;
    if (!(n & 7) && !(((uintptr_t)a | (uintptr_t)b) & 15)) {
        const uint4* a4 = reinterpret_cast<const uint4*>(a);
        const uint4* b4 = reinterpret_cast<const uint4*>(b);
        for (int i = lane; i < (n >> 3); i += 32) {
            const uint4 x = a4[i], y = b4[i];
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
            const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 xf = __bfloat1622float2(xp[j]), yf = __bfloat1622float2(yp[j]);
                acc += xf.x * yf.x + xf.y * yf.y;
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc += __bfloat162float(a[i]) * __bfloat162float(b[i]);
    }
    return warp_sum(acc);
}

// ---------------------------------------------------------------- router: from logits to the chosen experts
// The logits z = W_router h come from the engine's matrix products (float sums of bfloat16 or float operands).  A warp
// per token: its lanes turn the logits into scores and score the groups, then keep the best groups and take the best
// open experts one after the other (ties go to the lower index).  Shared memory per warp: n_experts scores,
// n_experts flags, n_experts ranks, n_groups group scores.
constexpr int SELECT_WARPS = 4;
__global__ void __launch_bounds__(32 * SELECT_WARPS)
moe_select_kernel(const float* __restrict__ logits, int tokens, int n_experts, int top, int n_groups, int keep, float route_scale,
                  int softmax, int renormalize, const float* __restrict__ choice_bias, int* __restrict__ chosen, float* __restrict__ weight) {
    extern __shared__ float select_smem[];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = blockIdx.x * SELECT_WARPS + warp;
    if (t >= tokens) return;
    const int per_warp = 3 * n_experts + n_groups;
    float* score = select_smem + (size_t)warp * per_warp;       // what the weights are made of
    int* open_ = reinterpret_cast<int*>(score + n_experts);
    float* rank = score + 2 * n_experts;                        // what the choice goes by: the score plus the choice bias
    float* group_score = score + 3 * n_experts;
    const float* z = logits + (size_t)t * n_experts;
    float z_max = -INFINITY, z_sum = 1.f;
    if (softmax) {
        for (int e = lane; e < n_experts; e += 32) z_max = fmaxf(z_max, z[e]);
        z_max = warp_max(z_max);
        z_sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) z_sum += expf(z[e] - z_max);
        z_sum = warp_sum(z_sum);
    }
    for (int e = lane; e < n_experts; e += 32) {
        const float sc = softmax ? expf(z[e] - z_max) / z_sum : 1.f / (1.f + expf(-z[e]));
        score[e] = sc;
        rank[e] = choice_bias ? sc + choice_bias[e] : sc;
        open_[e] = n_groups > 0 ? 0 : 1;
    }
    __syncwarp();
    if (n_groups > 0) {
        const int per = n_experts / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY, second = -INFINITY;
            for (int i = 0; i < per; ++i) {
                const float s = rank[g * per + i];
                if (s > best) { second = best; best = s; }
                else if (s > second) second = s;
            }
            group_score[g] = per > 1 ? best + second : best;
        }
        __syncwarp();
    }
    // The best of the warp's candidates: each lane looks at every 32nd, then the lanes compare (the larger score wins, the
    // lower index among equals), so every round costs a few shuffles instead of a walk over all experts by one lane.
    auto warp_best = [&](const float* value, const int* allowed, int n, float& best_value) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = lane; i < n; i += 32)
            if ((!allowed || allowed[i]) && value[i] > bv) { bv = value[i]; bi = i; }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        best_value = bv;
        return bi;
    };
    if (n_groups > 0) {
        const int per = n_experts / n_groups;
        for (int k = 0; k < keep; ++k) {
            float v;
            const int best = warp_best(group_score, nullptr, n_groups, v);
            if (best == 0x7fffffff) break;
            __syncwarp();
            if (lane == 0) group_score[best] = -INFINITY;            // never the best again ("nothing found" compares > -inf)
            for (int i = lane; i < per; i += 32) open_[best * per + i] = 1;
            __syncwarp();
        }
    }
    float chosen_sum = 0.f;                                          // lane 0's: the chosen scores, added best first
    for (int k = 0; k < top; ++k) {
        float v;
        int best = warp_best(rank, open_, n_experts, v);
        __syncwarp();
        if (lane == 0) {
            if (best == 0x7fffffff) best = 0;                        // fewer open experts than `top`: the host refuses such a configuration
            else open_[best] = 0;
            chosen[(size_t)t * top + k] = best;
            chosen_sum += score[best];
            weight[(size_t)t * top + k] = renormalize ? score[best] : score[best] * route_scale;
        }
        __syncwarp();
    }
    if (renormalize && lane == 0) {
        const float den = chosen_sum + 1e-20f;
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] = weight[(size_t)t * top + k] / den * route_scale;
    }
}

CISR_EXPORT int cisr_moe_select(const float* logits, int tokens, int n_experts, int top, int n_groups, int keep, float route_scale,
                                int softmax, int renormalize, const float* choice_bias, int* chosen, float* weight, void* stream) {
    if (tokens <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || top > n_experts || (n_groups > 0 && (n_experts % n_groups || keep <= 0 || keep > n_groups)))
        return -2;
    const size_t smem = (size_t)SELECT_WARPS * (3 * n_experts + (n_groups > 0 ? n_groups : 0)) * sizeof(float);
    if (smem > 48 * 1024) return -3;
    return launch_kernel(moe_select_kernel, dim3((tokens + SELECT_WARPS - 1) / SELECT_WARPS), dim3(32 * SELECT_WARPS), smem,
                         (cudaStream_t)stream, g_pdl, logits, tokens, n_experts, top, n_groups > 0 ? n_groups : 0, keep, route_scale, softmax,
                         renormalize, choice_bias, chosen, weight);
}

// ---------------------------------------------------------------- few tokens: a warp per output feature
// act[t * top + k, f] = a(W_up[e][f] . h[t]) with e = chosen[t, k] and a = max(z, 0)^2 (act 0) or the exact gelu (act 1);
// W_up [experts, ff, hidden].  gated: W_up
// [experts, 2 ff, hidden] (gate rows, then up rows) and act = g' sigmoid(alpha g') (u' + 1), g and u clamped by `limit`.
// Pairs whose expert has no matrices (e >= n_real: an identity expert) are skipped.
constexpr int ROW_WARPS = 8;
constexpr float GATE_ALPHA = 1.702f;
enum : int { ACT_RELU2 = 0, ACT_GELU_ERF = 1 };
__device__ __forceinline__ float expert_act(float z, int act) {
    if (act == ACT_GELU_ERF) return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
    const float r = fmaxf(z, 0.f);
    return r * r;
}
template <typename T>
__global__ void __launch_bounds__(32 * ROW_WARPS)
moe_up_rows_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ chosen, int hidden, int ff,
                   int top, int n_real, int gated, float limit, int act_kind, T* __restrict__ act) {
    pdl_trigger();
    pdl_wait();
    const int pair = blockIdx.x, lane = threadIdx.x & 31, f = blockIdx.y * ROW_WARPS + (threadIdx.x >> 5);
    if (f >= ff) return;
    const int e = chosen[pair];
    if (e >= n_real) return;
    const T* x = h + (size_t)(pair / top) * hidden;
    if (gated) {
        const T* w = w_up + (size_t)e * 2 * ff * hidden;
        const float g = fminf(warp_dot(w + (size_t)f * hidden, x, hidden, lane), limit);
        const float u = fminf(fmaxf(warp_dot(w + (size_t)(ff + f) * hidden, x, hidden, lane), -limit), limit);
        if (lane == 0) act[(size_t)pair * ff + f] = from_float<T>(g / (1.f + expf(-GATE_ALPHA * g)) * (u + 1.f));
        return;
    }
    const float z = warp_dot(w_up + ((size_t)e * ff + f) * hidden, x, hidden, lane);
    if (lane == 0) act[(size_t)pair * ff + f] = from_float<T>(expert_act(z, act_kind));
}

// out[t, c] = out_scale[c] * sum_k weight[t, k] * (W_down[e_k][c] . act[t * top + k]);   W_down [experts, hidden, ff];
// experts in the order the router chose them; out_scale (a layer scale, one factor per channel) may be null.
template <typename T>
__global__ void __launch_bounds__(32 * ROW_WARPS)
moe_down_rows_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ chosen,
                     const float* __restrict__ weight, int hidden, int ff, int top, int n_real, const T* __restrict__ h,
                     const float* __restrict__ out_scale, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, c = blockIdx.y * ROW_WARPS + (threadIdx.x >> 5);
    if (c >= hidden) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const int e = chosen[(size_t)t * top + k];
        if (e >= n_real) { acc += weight[(size_t)t * top + k] * to_float(h[(size_t)t * hidden + c]); continue; }     // an identity expert
        acc += weight[(size_t)t * top + k] * warp_dot(w_down + ((size_t)e * hidden + c) * ff, act + ((size_t)t * top + k) * ff, ff, lane);
    }
    if (lane == 0) out[(size_t)t * hidden + c] = out_scale ? acc * out_scale[c] : acc;
}

CISR_EXPORT int cisr_moe_rows(const void* h, const void* w_up, const void* w_down, int dtype, const int* chosen,
                              const float* weight, int tokens, int hidden, int ff, int top, int n_real, int gated, float limit,
                              int act_kind, void* act, const float* out_scale, float* out, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 up_grid(tokens * top, (ff + ROW_WARPS - 1) / ROW_WARPS), down_grid(tokens, (hidden + ROW_WARPS - 1) / ROW_WARPS);
    int st;
    if (dtype == CISR_BF16) {
        st = launch_kernel(moe_up_rows_kernel<__nv_bfloat16>, up_grid, dim3(32 * ROW_WARPS), 0, s, g_pdl, (const __nv_bfloat16*)h,
                           (const __nv_bfloat16*)w_up, chosen, hidden, ff, top, n_real, gated, limit, act_kind, (__nv_bfloat16*)act);
        if (st) return st;
        return launch_kernel(moe_down_rows_kernel<__nv_bfloat16>, down_grid, dim3(32 * ROW_WARPS), 0, s, g_pdl,
                             (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, chosen, weight, hidden, ff, top, n_real,
                             (const __nv_bfloat16*)h, out_scale, out);
    }
    st = launch_kernel(moe_up_rows_kernel<float>, up_grid, dim3(32 * ROW_WARPS), 0, s, g_pdl, (const float*)h, (const float*)w_up,
                       chosen, hidden, ff, top, n_real, gated, limit, act_kind, (float*)act);
    if (st) return st;
    return launch_kernel(moe_down_rows_kernel<float>, down_grid, dim3(32 * ROW_WARPS), 0, s, g_pdl, (const float*)act,
                         (const float*)w_down, chosen, weight, hidden, ff, top, n_real, (const float*)h, out_scale, out);
}

// ---------------------------------------------------------------- many tokens: rows sorted by expert
// The (token, chosen expert) pairs of a step are laid out expert by expert, each expert's rows padded to whole tiles of
// `tile` rows, so that one grouped product serves all experts:
//   row_of[pair]        the row of pair t * top + k in the sorted layout
//   src_token[row]      the token whose activations row `row` holds, -1 for padding (and for rows beyond the last tile used)
//   tile_group[i]       the expert of row tile i, -1 for tiles beyond the last one used
// Pairs whose expert has no matrices (chosen >= n_experts: an identity expert) get row_of = -1 and no row.
// One CTA; shared memory: 3 * n_experts ints.  Which row inside its expert's block a pair gets depends on the order the
// atomics happen to run in; every row is computed by itself and a token's experts are summed in the router's order, so
// the result does not.
__global__ void moe_sort_kernel(const int* __restrict__ chosen, int n_pairs, int top, int n_experts, int tile, int max_rows,
                                int* __restrict__ row_of, int* __restrict__ src_token, int* __restrict__ tile_group) {
    extern __shared__ int sort_smem[];
    int* count = sort_smem;
    int* offset = sort_smem + n_experts;
    int* fill = sort_smem + 2 * n_experts;
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) src_token[r] = -1;
    for (int i = threadIdx.x; i < max_rows / tile; i += blockDim.x) tile_group[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x)
        if (chosen[p] < n_experts) atomicAdd(&count[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; ++e) { offset[e] = at; at += (count[e] + tile - 1) / tile * tile; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        for (int i = offset[e] / tile; i < (offset[e] + count[e] + tile - 1) / tile; ++i) tile_group[i] = e;
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= n_experts) { row_of[p] = -1; continue; }
        const int row = offset[e] + atomicAdd(&fill[e], 1);
        row_of[p] = row;
        src_token[row] = p / top;
    }
}

// sorted[row, :] = h[src_token[row], :], zeros where src_token[row] < 0.  16-byte copies (hidden * 2 bytes % 16 == 0).
__global__ void moe_gather_kernel(const uint4* __restrict__ h, const int* __restrict__ src_token, uint4* __restrict__ sorted, int row_vec) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, src = src_token[row];
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x)
        sorted[(size_t)row * row_vec + i] = src >= 0 ? h[(size_t)src * row_vec + i] : make_uint4(0, 0, 0, 0);
}

// out[t, c] = out_scale[c] * sum_k weight[t, k] * sorted_out[row_of[t * top + k], c], k in the router's order (out_scale null: 1);
// a pair without a row (row_of < 0: an identity expert) adds weight * h[t, c].
__global__ void moe_combine_kernel(const float* __restrict__ sorted_out, const int* __restrict__ row_of, const float* __restrict__ weight,
                                   int top, int hidden, const __nv_bfloat16* __restrict__ h, const float* __restrict__ out_scale,
                                   float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of[(size_t)t * top + k];
            acc += weight[(size_t)t * top + k] * (row >= 0 ? sorted_out[(size_t)row * hidden + c] : to_float(h[(size_t)t * hidden + c]));
        }
        out[(size_t)t * hidden + c] = out_scale ? acc * out_scale[c] : acc;
    }
}

CISR_EXPORT int cisr_moe_sort(const int* chosen, int tokens, int top, int n_experts, int tile, int max_rows, int* row_of,
                              int* src_token, int* tile_group, void* stream) {
    if (tokens <= 0) return 0;
    // the padded blocks of all experts together: at most pairs + (experts in use) * (tile - 1) rows, in whole tiles
    const long long pairs = (long long)tokens * top, in_use = pairs < n_experts ? pairs : n_experts;
    if (tile <= 0 || max_rows % tile || max_rows < (pairs + in_use * (tile - 1)) / tile * tile) return -2;
    const size_t smem = (size_t)3 * n_experts * sizeof(int);
    if (smem > 48 * 1024) return -3;
    return launch_kernel(moe_sort_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, g_pdl, chosen, tokens * top, top, n_experts, tile,
                         max_rows, row_of, src_token, tile_group);
}

CISR_EXPORT int cisr_moe_gather(const void* h, const int* src_token, void* sorted, int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    if ((hidden * 2) % 16 || (((uintptr_t)h | (uintptr_t)sorted) & 15)) return -2;
    return launch_kernel(moe_gather_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)stream, g_pdl, (const uint4*)h, src_token, (uint4*)sorted,
                         hidden * 2 / 16);
}

CISR_EXPORT int cisr_moe_combine(const float* sorted_out, const int* row_of, const float* weight, int tokens, int top, int hidden,
                                 const void* h, const float* out_scale, float* out, void* stream) {
    if (tokens <= 0) return 0;
    return launch_kernel(moe_combine_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, g_pdl, sorted_out, row_of, weight, top,
                         hidden, (const __nv_bfloat16*)h, out_scale, out);
}
