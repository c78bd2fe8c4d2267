// Lightning attention: linear attention with one fixed decay per head and a matrix state per head.
//
//   q = silu(W_q h), k = silu(W_k h) [heads x key_dim], v = silu(W_v h) [heads x value_dim]
//   per head:  S <- decay_h S + k v^T;  o = S^T q          (S [key_dim, value_dim], zero when the request starts)
//   out = o / sqrt(mean(o^2) + eps) * w_norm * sigmoid(W_g h), the mean over all heads of the token at once
//
// The projections arrive as float sums (proj [tokens, columns]: q | k | v | gate from given columns); silu, the decay and
// its powers, the state and every step of its recurrence, the norm and the gate are float arithmetic.  A request's state
// is one float row of a state tensor, laid out [heads, value_dim, key_dim] (a column of S is contiguous).
//
// Two forms of the same recurrence, which differ by rounding only:
//   walk    single tokens and short portions: a warp per column of S, its lanes holding the column's rows in registers,
//           token after token.
//   chunks  portions of LIGHTNING_CHUNK tokens and more, C = LIGHTNING_CHUNK tokens at a time.  With t, i counted inside a
//           chunk of n tokens and S0 the state before it:
//               o_t = decay^(t+1) S0^T q_t + sum_{i <= t} decay^(t-i) (q_t . k_i) v_i
//               S   = decay^n S0 + sum_i decay^(n-1-i) k_i v_i^T
//           three small float products per chunk in shared memory (scores, read-out, state), register tiles of 4 x 4 and
//           4 x CPT.  The columns of S are independent: a CTA takes CB = 16 CPT value columns of one head and recomputes
//           the chunk's scores for them.
#include "common.cuh"

static bool g_pdl = false;
CISR_EXPORT void cisr_lightning_set_pdl(int on) { g_pdl = on != 0; }

constexpr int LIGHTNING_CHUNK = 64;
constexpr int WALK_WARPS = 8;
constexpr int MAX_KEY_DIM = 256;
CISR_EXPORT int cisr_lightning_chunk_tokens() { return LIGHTNING_CHUNK; }
CISR_EXPORT int cisr_lightning_max_key_dim() { return MAX_KEY_DIM; }

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ---------------------------------------------------------------- token by token
// grid (requests, heads, value columns / WALK_WARPS); a warp owns column c of its head's state, lane l the rows l, l + 32, ...
// `least` > 0: requests that bring at least that many tokens are left to the chunked kernel.
template <int R>
__global__ void __launch_bounds__(32 * WALK_WARPS)
lightning_walk_kernel(const float* __restrict__ proj, int stride, int q_col, int k_col, int v_col, const float* __restrict__ decay,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ req_slot,
                      const int* __restrict__ q_start, const int* __restrict__ q_len, float* __restrict__ o, int heads, int key_dim,
                      int value_dim, int least) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, c = blockIdx.z * WALK_WARPS + (threadIdx.x >> 5);
    const int n = q_len[r];
    if (n <= 0 || (least > 0 && n >= least) || c >= value_dim) return;
    float* column = state + (size_t)req_slot[r] * state_stride + ((size_t)h * value_dim + c) * key_dim;
    float S[R], k_now[R], q_now[R], k_next[R], q_next[R], v_now, v_next = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) { const int row = lane + 32 * i; S[i] = row < key_dim ? column[row] : 0.f; k_next[i] = q_next[i] = 0.f; }
    const float dec = decay[h];
    const int t0 = q_start[r];
    auto fetch = [&](int t) {
        const float* row_p = proj + (size_t)(t0 + t) * stride;
        v_next = row_p[v_col + h * value_dim + c];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int row = lane + 32 * i;
            k_next[i] = row < key_dim ? row_p[k_col + h * key_dim + row] : 0.f;
            q_next[i] = row < key_dim ? row_p[q_col + h * key_dim + row] : 0.f;
        }
    };
    fetch(0);
    for (int t = 0; t < n; ++t) {
        v_now = v_next;
#pragma unroll
        for (int i = 0; i < R; ++i) { k_now[i] = k_next[i]; q_now[i] = q_next[i]; }
        if (t + 1 < n) fetch(t + 1);                  // the next token's operands are on their way during this token's sums
        const float v = silu_f(v_now);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            S[i] = dec * S[i] + silu_f(k_now[i]) * v;
            acc += S[i] * silu_f(q_now[i]);
        }
        acc = warp_sum(acc);
        if (lane == 0) o[(size_t)(t0 + t) * heads * value_dim + h * value_dim + c] = acc;
    }
#pragma unroll
    for (int i = 0; i < R; ++i) { const int row = lane + 32 * i; if (row < key_dim) column[row] = S[i]; }
}

// ---------------------------------------------------------------- chunk by chunk
// grid (requests, heads, value columns / CB), 256 threads as 16 x 16: thread (ty, tx) owns rows 4 ty .. 4 ty + 3 of a
// 64-row tile and columns 4 tx .. (scores) or CPT tx .. (read-out, state).  Shared memory (floats), LD = C + 4:
//   Qt, Kt [dP][LD]   silu(q), silu(k) of the chunk, coordinate-major (dP: key_dim rounded up to 4), zero beyond the portion
//   P [C][LD]         decayed scores, zero above the diagonal
//   V [C][CB]         silu(v) of the CTA's columns
//   S [dP][CB]        the state's columns
//   pw [C + 1]        powers of the decay
constexpr int C = LIGHTNING_CHUNK, LD = C + 4;
template <int CPT>
__global__ void __launch_bounds__(256)
lightning_chunk_kernel(const float* __restrict__ proj, int stride, int q_col, int k_col, int v_col, const float* __restrict__ decay,
                       float* __restrict__ state, long long state_stride, const int* __restrict__ req_slot,
                       const int* __restrict__ q_start, const int* __restrict__ q_len, float* __restrict__ o, int heads, int key_dim,
                       int value_dim, int least) {
    constexpr int CB = 16 * CPT;
    extern __shared__ __align__(16) float lightning_smem[];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int n_all = q_len[r];
    if (n_all < least) return;
    const int dP = (key_dim + 3) & ~3;
    float* Qt = lightning_smem;
    float* Kt = Qt + (size_t)dP * LD;
    float* P = Kt + (size_t)dP * LD;
    float* V = P + (size_t)C * LD;
    float* S = V + (size_t)C * CB;
    float* pw = S + (size_t)dP * CB;
    float* slot_state = state + (size_t)req_slot[r] * state_stride + (size_t)h * value_dim * key_dim;
    for (int i = tid; i < dP * CB; i += 256) {
        const int c = i / dP, row = i - c * dP;          // a column of the state is contiguous in memory
        S[row * CB + c] = (row < key_dim && c0 + c < value_dim) ? slot_state[(size_t)(c0 + c) * key_dim + row] : 0.f;
    }
    const float lg = logf(decay[h]);
    for (int j = tid; j <= C; j += 256) pw[j] = j ? expf((float)j * lg) : 1.f;
    const int t_first = q_start[r];
    for (int t0 = 0; t0 < n_all; t0 += C) {
        const int n = min(C, n_all - t0);
        __syncthreads();                                  // the chunk before is done with Qt, Kt, V; S and pw are written
        for (int i = tid; i < C * dP; i += 256) {
            const int t = i / dP, kk = i - t * dP;
            float q = 0.f, k = 0.f;
            if (t < n && kk < key_dim) {
                const float* row_p = proj + (size_t)(t_first + t0 + t) * stride + h * key_dim + kk;
                q = silu_f(row_p[q_col]);
                k = silu_f(row_p[k_col]);
            }
            Qt[kk * LD + t] = q;
            Kt[kk * LD + t] = k;
        }
        for (int i = tid; i < C * CB; i += 256) {
            const int t = i / CB, c = i - t * CB;
            V[i] = (t < n && c0 + c < value_dim) ? silu_f(proj[(size_t)(t_first + t0 + t) * stride + v_col + h * value_dim + c0 + c]) : 0.f;
        }
        __syncthreads();
        // scores of the chunk: P[t][i] = decay^(t - i) (q_t . k_i) for i <= t
        {
            float acc[4][4] = {};
            if (tx <= ty) {                                // tiles above the diagonal hold nothing
                for (int kk = 0; kk < dP; ++kk) {
                    const float4 a = *reinterpret_cast<const float4*>(Qt + kk * LD + 4 * ty);
                    const float4 b = *reinterpret_cast<const float4*>(Kt + kk * LD + 4 * tx);
                    const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int x = 0; x < 4; ++x)
#pragma unroll
                        for (int y = 0; y < 4; ++y) acc[x][y] += av[x] * bv[y];
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int t = 4 * ty + x;
                float4 out;
                float* ov = reinterpret_cast<float*>(&out);
#pragma unroll
                for (int y = 0; y < 4; ++y) { const int i = 4 * tx + y; ov[y] = i <= t ? acc[x][y] * pw[t - i] : 0.f; }
                *reinterpret_cast<float4*>(P + t * LD + 4 * tx) = out;
            }
        }
        __syncthreads();
        // read-out: o_t = decay^(t+1) S0^T q_t + sum_i P[t][i] v_i
        {
            float acc[4][CPT] = {}, carried[4][CPT] = {};
            for (int i = 0; i < 4 * ty + 4; i += 4) {      // P holds nothing right of the diagonal
                float4 p[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) p[x] = *reinterpret_cast<const float4*>(P + (4 * ty + x) * LD + i);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v[CPT];
#pragma unroll
                    for (int y = 0; y < CPT; ++y) v[y] = V[(i + j) * CB + CPT * tx + y];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float pv = reinterpret_cast<const float*>(&p[x])[j];
#pragma unroll
                        for (int y = 0; y < CPT; ++y) acc[x][y] += pv * v[y];
                    }
                }
            }
            for (int row = 0; row < dP; ++row) {
                const float4 a = *reinterpret_cast<const float4*>(Qt + row * LD + 4 * ty);
                const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int y = 0; y < CPT; ++y) {
                    const float s = S[row * CB + CPT * tx + y];
#pragma unroll
                    for (int x = 0; x < 4; ++x) carried[x][y] += av[x] * s;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int t = 4 * ty + x;
                if (t >= n) continue;
#pragma unroll
                for (int y = 0; y < CPT; ++y) {
                    const int c = c0 + CPT * tx + y;
                    if (c < value_dim)
                        o[(size_t)(t_first + t0 + t) * heads * value_dim + h * value_dim + c] = pw[t + 1] * carried[x][y] + acc[x][y];
                }
            }
        }
        __syncthreads();                                  // every read-out has used the old state
        // state: S = decay^n S0 + sum_i decay^(n-1-i) k_i v_i^T   (v_i is scaled in place first)
        for (int i = tid; i < C * CB; i += 256) { const int t = i / CB; V[i] = t < n ? V[i] * pw[n - 1 - t] : 0.f; }
        __syncthreads();
        for (int row0 = 0; row0 < dP; row0 += 64) {
            const int row = row0 + 4 * ty;
            if (row >= dP) continue;                       // dP is a multiple of 4: a thread's four rows exist together
            float acc[4][CPT] = {};
            for (int i = 0; i < C; i += 4) {
                float4 k[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) k[x] = *reinterpret_cast<const float4*>(Kt + (row + x) * LD + i);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v[CPT];
#pragma unroll
                    for (int y = 0; y < CPT; ++y) v[y] = V[(i + j) * CB + CPT * tx + y];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float kv = reinterpret_cast<const float*>(&k[x])[j];
#pragma unroll
                        for (int y = 0; y < CPT; ++y) acc[x][y] += kv * v[y];
                    }
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < CPT; ++y) {
                    float* s = S + (row + x) * CB + CPT * tx + y;
                    *s = pw[n] * *s + acc[x][y];
                }
        }
    }
    __syncthreads();
    for (int i = tid; i < dP * CB; i += 256) {
        const int c = i / dP, row = i - c * dP;
        if (row < key_dim && c0 + c < value_dim) slot_state[(size_t)(c0 + c) * key_dim + row] = S[row * CB + c];
    }
}

static size_t chunk_smem(int key_dim, int cb) {
    const size_t dP = (size_t)((key_dim + 3) & ~3);
    return sizeof(float) * (2 * dP * LD + (size_t)C * LD + (size_t)C * cb + dP * cb + C + 1 + 3);
}

template <int CPT>
static int launch_chunks(const float* proj, int stride, int q_col, int k_col, int v_col, const float* decay, float* state,
                         long long state_stride, const int* req_slot, const int* q_start, const int* q_len, float* o, int heads,
                         int key_dim, int value_dim, int n_req, int least, cudaStream_t s) {
    const size_t smem = chunk_smem(key_dim, 16 * CPT);
    static size_t allowed = 0;
    if (smem > allowed) {
        if (cudaFuncSetAttribute(lightning_chunk_kernel<CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return -3;
        }
        allowed = smem;
    }
    return launch_kernel(lightning_chunk_kernel<CPT>, dim3(n_req, heads, (value_dim + 16 * CPT - 1) / (16 * CPT)), dim3(256), smem, s, g_pdl,
                         proj, stride, q_col, k_col, v_col, decay, state, state_stride, req_slot, q_start, q_len, o, heads, key_dim,
                         value_dim, least);
}

// The recurrence for a step: `n_long` requests bring at least `least` tokens (they run chunk by chunk), `n_short` fewer
// (token by token); least <= 0: every request token by token.  o float [tokens, heads * value_dim].
CISR_EXPORT int cisr_lightning_recurrence(const float* proj, int stride, int q_col, int k_col, int v_col, const float* decay, float* state,
                                          long long state_stride, const int* req_slot, const int* q_start, const int* q_len, float* o,
                                          int heads, int key_dim, int value_dim, int n_req, int least, int n_long, int n_short,
                                          int columns_per_cta, void* stream) {
    if (n_req <= 0) return 0;
    if (key_dim <= 0 || key_dim > MAX_KEY_DIM || value_dim <= 0 || heads <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    int st = 0;
    if (least > 0 && n_long > 0) {
        // as many value columns per CTA as still leave the device's SMs a CTA each (the scores are recomputed per CTA)
        int cb = columns_per_cta;
        if (cb <= 0) {
            cb = 64;
            while (cb > 16 && ((long long)n_long * heads * ((value_dim + cb - 1) / cb) < 148 || cb / 2 >= value_dim)) cb /= 2;
        }
        while (cb > 16 && chunk_smem(key_dim, cb) > 200 * 1024) cb /= 2;
        if (chunk_smem(key_dim, cb) > 227 * 1024) return -3;
#define LIGHTNING_CHUNKS(CPT) launch_chunks<CPT>(proj, stride, q_col, k_col, v_col, decay, state, state_stride, req_slot, q_start, q_len, o, \
                                                 heads, key_dim, value_dim, n_req, least, s)
        st = cb >= 64 ? LIGHTNING_CHUNKS(4) : cb >= 32 ? LIGHTNING_CHUNKS(2) : LIGHTNING_CHUNKS(1);
#undef LIGHTNING_CHUNKS
        if (st) return st;
    }
    if (least <= 0 || n_short > 0) {
        const dim3 grid(n_req, heads, (value_dim + WALK_WARPS - 1) / WALK_WARPS), block(32 * WALK_WARPS);
        const int rows = (key_dim + 31) / 32;
#define LIGHTNING_WALK(R) launch_kernel(lightning_walk_kernel<R>, grid, block, 0, s, g_pdl, proj, stride, q_col, k_col, v_col, decay, state, \
                                        state_stride, req_slot, q_start, q_len, o, heads, key_dim, value_dim, least > 0 ? least : 0)
        switch (rows) {
            case 1: st = LIGHTNING_WALK(1); break;
            case 2: st = LIGHTNING_WALK(2); break;
            case 3: st = LIGHTNING_WALK(3); break;
            case 4: st = LIGHTNING_WALK(4); break;
            case 5: case 6: st = LIGHTNING_WALK(6); break;
            default: st = LIGHTNING_WALK(8); break;
        }
#undef LIGHTNING_WALK
    }
    return st;
}

// ---------------------------------------------------------------- output: norm over all heads, weight, gate
// out[t, j] = o[t, j] / sqrt(mean_j(o[t, :]^2) + eps) * norm_w[j] * sigmoid(gate[t, gate_col + j]), rounded once.
template <typename CT>
__global__ void lightning_output_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride, int gate_col,
                                        const float* __restrict__ norm_w, float eps, CT* __restrict__ out, int out_stride, int width) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = o + (size_t)t * width;
    float sq = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) { const float v = row[j]; sq += v * v; }
    const float unit = rsqrtf(block_sum(sq, scratch) / (float)width + eps);
    const float* g = gate + (size_t)t * gate_stride + gate_col;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        out[(size_t)t * out_stride + j] = from_float<CT>(row[j] * unit * norm_w[j] * (1.f / (1.f + expf(-g[j]))));
}

CISR_EXPORT int cisr_lightning_output(const float* o, const float* gate, int gate_stride, int gate_col, const float* norm_w, float eps,
                                      void* out, int dtype, int out_stride, int width, int tokens, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == CISR_BF16)
        return launch_kernel(lightning_output_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, s, g_pdl, o, gate, gate_stride, gate_col,
                             norm_w, eps, (__nv_bfloat16*)out, out_stride, width);
    return launch_kernel(lightning_output_kernel<float>, dim3(tokens), dim3(threads), 0, s, g_pdl, o, gate, gate_stride, gate_col, norm_w,
                         eps, (float*)out, out_stride, width);
}
