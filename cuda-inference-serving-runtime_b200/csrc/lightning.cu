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
//           The second sum of S (a chunk's gain) needs no state, so it is made for every chunk of the step at once; a short
//           scan then carries the state from chunk to chunk, element by element; and the read-outs of every chunk are made
//           at once from the state before each.  Small float products in shared memory, register tiles of 4 x 4 and
//           4 x CPT; a CTA takes CB = 16 CPT value columns of one head and one chunk.
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
// Three launches over the chunks of the step's long portions (chunk_req, chunk_t0: a chunk's request and its first token
// inside the portion; req_chunk0: a request's first chunk), with a scratch of one state-sized block per (chunk, head):
//   gains   (chunk, head, CB value columns): the chunk's own contribution to the state, sum_i decay^(n-1-i) k_i v_i^T,
//           into the chunk's scratch block [key_dim][value_dim].  Every chunk at once.
//   scan    (request, head): walks the request's chunks element by element: the scratch block receives the state BEFORE
//           its chunk, the running state becomes decay^n S + gain; the last one goes back to the request's slot.
//   reads   (chunk, head, CB value columns): the read-outs, decay^(t+1) S0^T q_t + sum_{i<=t} decay^(t-i) (q_t . k_i) v_i
//           with S0 from the scratch.  Every chunk at once.
// 256 threads as 16 x 16: thread (ty, tx) owns rows 4 ty .. 4 ty + 3 of a 64-row tile and columns 4 tx .. (scores) or
// CPT tx .. (read-outs, gains).  Shared memory (floats), LD = C + 4:
//   Qt, Kt [dP][LD]   silu(q), silu(k) of the chunk, coordinate-major (dP: key_dim rounded up to 4), zero beyond the portion
//   P [C][LD]         decayed scores, zero above the diagonal
//   V [C][CB]         silu(v) of the CTA's columns
//   S [dP][CB]        the state's columns before the chunk (in Kt's place once the scores are made)
//   pw [C + 1]        powers of the decay
constexpr int C = LIGHTNING_CHUNK, LD = C + 4;

struct ChunkArgs {
    const float* proj; int stride, q_col, k_col, v_col;
    const float* decay;
    float* state; long long state_stride;
    const int* req_slot; const int* q_start; const int* q_len;
    const int* chunk_req; const int* chunk_t0; const int* req_chunk0;
    float* scratch;                       // [chunks][heads][key_dim][value_dim]
    float* o; int heads, key_dim, value_dim, least;
};

// silu of one projection of the chunk's tokens, coordinate-major into dst [dP][LD]; zero beyond the portion and the width
// (a thread asks for eight of its numbers before it uses the first: eight loads in flight instead of one)
__device__ __forceinline__ void stage_transposed(const ChunkArgs& a, int col0, int token0, int n, int dP, float* dst) {
    const float* __restrict__ src = a.proj + (size_t)token0 * a.stride + col0;
    for (int i0 = threadIdx.x; i0 < C * dP; i0 += 8 * 256) {
        float raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 256, t = i / dP, kk = i - t * dP;
            raw[u] = (i < C * dP && t < n && kk < a.key_dim) ? src[(size_t)t * a.stride + kk] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 256, t = i / dP, kk = i - t * dP;
            if (i < C * dP) dst[kk * LD + t] = silu_f(raw[u]);       // silu(0) = 0: beyond the portion and the width
        }
    }
}
// silu(v) of the CTA's columns into V [C][CB], each row times weight(t) (zero beyond the portion and the width)
template <int CB, typename W>
__device__ __forceinline__ void stage_values(const ChunkArgs& a, int h, int c0, int token0, int n, float* V, W weight) {
    const float* __restrict__ src = a.proj + (size_t)token0 * a.stride + a.v_col + h * a.value_dim + c0;
    for (int i0 = threadIdx.x; i0 < C * CB; i0 += 4 * 256) {      // C * CB is a multiple of 1024
        float raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 256, t = i / CB, c = i - t * CB;
            raw[u] = (t < n && c0 + c < a.value_dim) ? src[(size_t)t * a.stride + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 256, t = i / CB;
            V[i] = t < n ? silu_f(raw[u]) * weight(t) : 0.f;
        }
    }
}
__device__ __forceinline__ void stage_powers(float decay, float* pw) {
    const float lg = logf(decay);
    for (int j = threadIdx.x; j <= C; j += 256) pw[j] = j ? expf((float)j * lg) : 1.f;
}

// CPT neighbouring floats of shared memory in one access (the address is a multiple of 4 CPT bytes)
template <int CPT>
__device__ __forceinline__ void load_run(const float* __restrict__ p, float (&v)[CPT]) {
    if (CPT == 4) { const float4 x = *reinterpret_cast<const float4*>(p); v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; }
    else if (CPT == 2) { const float2 x = *reinterpret_cast<const float2*>(p); v[0] = x.x; v[1] = x.y; }
    else v[0] = p[0];
}

template <int CPT>
__global__ void __launch_bounds__(256) lightning_gains_kernel(ChunkArgs a) {
    constexpr int CB = 16 * CPT;
    extern __shared__ __align__(16) float lightning_smem[];
    pdl_trigger();
    pdl_wait();
    const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB, ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int r = a.chunk_req[chunk], t0 = a.chunk_t0[chunk], n = min(C, a.q_len[r] - t0), token0 = a.q_start[r] + t0;
    const int dP = (a.key_dim + 3) & ~3;
    float* Kt = lightning_smem;
    float* V = Kt + (size_t)dP * LD;
    float* pw = V + (size_t)C * CB;
    stage_powers(a.decay[h], pw);
    stage_transposed(a, a.k_col + h * a.key_dim, token0, n, dP, Kt);
    __syncthreads();
    stage_values<CB>(a, h, c0, token0, n, V, [&](int t) { return pw[n - 1 - t]; });
    __syncthreads();
    float* block = a.scratch + ((size_t)chunk * a.heads + h) * a.key_dim * a.value_dim;
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
                load_run<CPT>(V + (i + j) * CB + CPT * tx, v);
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
                const int c = c0 + CPT * tx + y;
                if (row + x < a.key_dim && c < a.value_dim) block[(size_t)(row + x) * a.value_dim + c] = acc[x][y];
            }
    }
}

// grid (requests, heads, elements / (256 VEC)): a thread owns VEC neighbouring elements (row, col .. col + VEC - 1) of the
// head's state (VEC 4 where value_dim is a multiple of 4, so that a CTA reads 4 KB in one piece from every block; else 1)
template <int VEC>
__global__ void __launch_bounds__(256) lightning_scan_kernel(ChunkArgs a) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y, e = (blockIdx.z * 256 + threadIdx.x) * VEC;
    const int n_all = a.q_len[r];
    if (n_all < a.least || e >= a.key_dim * a.value_dim) return;
    const int row = e / a.value_dim, col = e - row * a.value_dim;
    float* kept = a.state + (size_t)a.req_slot[r] * a.state_stride + ((size_t)h * a.value_dim + col) * a.key_dim + row;
    float S[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) S[j] = kept[(size_t)j * a.key_dim];
    const float lg = logf(a.decay[h]), whole = expf((float)C * lg);
    const size_t step = (size_t)a.heads * a.key_dim * a.value_dim;
    float* block = a.scratch + ((size_t)a.req_chunk0[r] * a.heads + h) * a.key_dim * a.value_dim + e;
    const int chunks = (n_all + C - 1) / C;
    constexpr int AHEAD = VEC == 1 ? 8 : 4;               // gains requested together: the walk itself is one multiply-add per chunk
    for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
        float gain[AHEAD][VEC];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            if (VEC == 4) {
                const float4 g = c0 + u < chunks ? *reinterpret_cast<const float4*>(block + (size_t)(c0 + u) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
                gain[u][0] = g.x; gain[u][1 % VEC] = g.y; gain[u][2 % VEC] = g.z; gain[u][3 % VEC] = g.w;
            } else {
                gain[u][0] = c0 + u < chunks ? block[(size_t)(c0 + u) * step] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int c = c0 + u;
            if (c < chunks) {
                const int n = min(C, n_all - c * C);
                const float f = n == C ? whole : expf((float)n * lg);
                if (VEC == 4) *reinterpret_cast<float4*>(block + (size_t)c * step) = make_float4(S[0], S[1 % VEC], S[2 % VEC], S[3 % VEC]);
                else block[(size_t)c * step] = S[0];
#pragma unroll
                for (int j = 0; j < VEC; ++j) S[j] = f * S[j] + gain[u][j];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) kept[(size_t)j * a.key_dim] = S[j];
}

template <int CPT>
__global__ void __launch_bounds__(256) lightning_reads_kernel(ChunkArgs a) {
    constexpr int CB = 16 * CPT;
    extern __shared__ __align__(16) float lightning_smem[];
    pdl_trigger();
    pdl_wait();
    const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int r = a.chunk_req[chunk], t0 = a.chunk_t0[chunk], n = min(C, a.q_len[r] - t0), token0 = a.q_start[r] + t0;
    const int dP = (a.key_dim + 3) & ~3;
    float* Qt = lightning_smem;
    float* Kt = Qt + (size_t)dP * LD;                     // later S [dP][CB], CB <= LD
    float* P = Kt + (size_t)dP * LD;
    float* V = P + (size_t)C * LD;
    float* pw = V + (size_t)C * CB;
    float* S = Kt;
    stage_powers(a.decay[h], pw);
    stage_transposed(a, a.q_col + h * a.key_dim, token0, n, dP, Qt);
    stage_transposed(a, a.k_col + h * a.key_dim, token0, n, dP, Kt);
    stage_values<CB>(a, h, c0, token0, n, V, [](int) { return 1.f; });
    __syncthreads();
    // scores of the chunk: P[t][i] = decay^(t - i) (q_t . k_i) for i <= t.  The 136 tiles of 4 x 4 on and below the diagonal go
    // to the first 136 threads (tile k = py (py + 1) / 2 + px), so five warps work and three wait instead of all eight walking
    // the keys for a few lanes each; the tiles above the diagonal are zeroed by the other threads.
    {
        constexpr int TILES = (C / 4) * (C / 4 + 1) / 2;
        if (tid < TILES) {
            int py = (int)((sqrtf(8.f * (float)tid + 1.f) - 1.f) * 0.5f);
            while (py * (py + 1) / 2 > tid) --py;
            while ((py + 1) * (py + 2) / 2 <= tid) ++py;
            const int px = tid - py * (py + 1) / 2;
            float acc[4][4] = {};
            for (int kk = 0; kk < dP; ++kk) {
                const float4 q = *reinterpret_cast<const float4*>(Qt + kk * LD + 4 * py);
                const float4 k = *reinterpret_cast<const float4*>(Kt + kk * LD + 4 * px);
                const float qv[4] = {q.x, q.y, q.z, q.w}, kv[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) acc[x][y] += qv[x] * kv[y];
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int t = 4 * py + x;
                float4 out;
                float* ov = reinterpret_cast<float*>(&out);
#pragma unroll
                for (int y = 0; y < 4; ++y) { const int i = 4 * px + y; ov[y] = i <= t ? acc[x][y] * pw[t - i] : 0.f; }
                *reinterpret_cast<float4*>(P + t * LD + 4 * px) = out;
            }
        }
        if (tx > ty) {
#pragma unroll
            for (int x = 0; x < 4; ++x) *reinterpret_cast<float4*>(P + (4 * ty + x) * LD + 4 * tx) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncthreads();                                      // the scores are made: the keys' place takes the state's columns
    const float* block = a.scratch + ((size_t)chunk * a.heads + h) * a.key_dim * a.value_dim;
    for (int i0 = tid; i0 < dP * CB; i0 += 8 * 256) {
        float raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 256, row = i / CB, c = i - row * CB;
            raw[u] = (i < dP * CB && row < a.key_dim && c0 + c < a.value_dim) ? block[(size_t)row * a.value_dim + c0 + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (i0 + u * 256 < dP * CB) S[i0 + u * 256] = raw[u];
    }
    __syncthreads();
    float acc[4][CPT] = {}, carried[4][CPT] = {};
    for (int i = 0; i < 4 * ty + 4; i += 4) {             // P holds nothing right of the diagonal
        float4 p[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) p[x] = *reinterpret_cast<const float4*>(P + (4 * ty + x) * LD + i);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[CPT];
            load_run<CPT>(V + (i + j) * CB + CPT * tx, v);
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float pv = reinterpret_cast<const float*>(&p[x])[j];
#pragma unroll
                for (int y = 0; y < CPT; ++y) acc[x][y] += pv * v[y];
            }
        }
    }
    for (int row = 0; row < dP; ++row) {
        const float4 q = *reinterpret_cast<const float4*>(Qt + row * LD + 4 * ty);
        const float qv[4] = {q.x, q.y, q.z, q.w};
        float sv[CPT];
        load_run<CPT>(S + row * CB + CPT * tx, sv);
#pragma unroll
        for (int y = 0; y < CPT; ++y)
#pragma unroll
            for (int x = 0; x < 4; ++x) carried[x][y] += qv[x] * sv[y];
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const int t = 4 * ty + x;
        if (t >= n) continue;
#pragma unroll
        for (int y = 0; y < CPT; ++y) {
            const int c = c0 + CPT * tx + y;
            if (c < a.value_dim) a.o[(size_t)(token0 + t) * a.heads * a.value_dim + h * a.value_dim + c] = pw[t + 1] * carried[x][y] + acc[x][y];
        }
    }
}

static size_t gains_smem(int key_dim, int cb) {
    const size_t dP = (size_t)((key_dim + 3) & ~3);
    return sizeof(float) * (dP * LD + (size_t)C * cb + C + 1 + 3);
}
static size_t reads_smem(int key_dim, int cb) {
    const size_t dP = (size_t)((key_dim + 3) & ~3);
    return sizeof(float) * (2 * dP * LD + (size_t)C * LD + (size_t)C * cb + C + 1 + 3);
}

template <int CPT>
static int launch_chunks(const ChunkArgs& a, int n_req, int n_chunks, cudaStream_t s) {
    const int cb = 16 * CPT, slabs = (a.value_dim + cb - 1) / cb;
    const size_t smem_g = gains_smem(a.key_dim, cb), smem_r = reads_smem(a.key_dim, cb);
    static size_t allowed_g = 0, allowed_r = 0;
    if (smem_g > allowed_g) {
        if (cudaFuncSetAttribute(lightning_gains_kernel<CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_g) != cudaSuccess) { cudaGetLastError(); return -3; }
        allowed_g = smem_g;
    }
    if (smem_r > allowed_r) {
        if (cudaFuncSetAttribute(lightning_reads_kernel<CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_r) != cudaSuccess) { cudaGetLastError(); return -3; }
        allowed_r = smem_r;
    }
    int st = launch_kernel(lightning_gains_kernel<CPT>, dim3(n_chunks, a.heads, slabs), dim3(256), smem_g, s, g_pdl, a);
    if (st) return st;
    const int elements = a.key_dim * a.value_dim;
    if (a.value_dim % 4 == 0 && ((uintptr_t)a.scratch & 15) == 0)
        st = launch_kernel(lightning_scan_kernel<4>, dim3(n_req, a.heads, (elements / 4 + 255) / 256), dim3(256), 0, s, g_pdl, a);
    else
        st = launch_kernel(lightning_scan_kernel<1>, dim3(n_req, a.heads, (elements + 255) / 256), dim3(256), 0, s, g_pdl, a);
    if (st) return st;
    return launch_kernel(lightning_reads_kernel<CPT>, dim3(n_chunks, a.heads, slabs), dim3(256), smem_r, s, g_pdl, a);
}

CISR_EXPORT long long cisr_lightning_scratch_floats(int n_chunks, int heads, int key_dim, int value_dim) {
    return (long long)n_chunks * heads * key_dim * value_dim;
}

// The recurrence for a step: the requests that bring at least `least` tokens run chunk by chunk (`n_chunks` chunks listed in
// chunk_req / chunk_t0, a request's first one in req_chunk0; scratch as cisr_lightning_scratch_floats says), the `n_short`
// others token by token; least <= 0: every request token by token.  o float [tokens, heads * value_dim].
CISR_EXPORT int cisr_lightning_recurrence(const float* proj, int stride, int q_col, int k_col, int v_col, const float* decay, float* state,
                                          long long state_stride, const int* req_slot, const int* q_start, const int* q_len, float* o,
                                          int heads, int key_dim, int value_dim, int n_req, int least, int n_chunks, int n_short,
                                          const int* chunk_req, const int* chunk_t0, const int* req_chunk0, float* scratch,
                                          int columns_per_cta, void* stream) {
    if (n_req <= 0) return 0;
    if (key_dim <= 0 || key_dim > MAX_KEY_DIM || value_dim <= 0 || heads <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    int st = 0;
    if (least > 0 && n_chunks > 0) {
        if (!chunk_req || !chunk_t0 || !req_chunk0 || !scratch) return -2;
        ChunkArgs a;
        a.proj = proj; a.stride = stride; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col; a.decay = decay; a.state = state;
        a.state_stride = state_stride; a.req_slot = req_slot; a.q_start = q_start; a.q_len = q_len; a.chunk_req = chunk_req;
        a.chunk_t0 = chunk_t0; a.req_chunk0 = req_chunk0; a.scratch = scratch; a.o = o; a.heads = heads; a.key_dim = key_dim;
        a.value_dim = value_dim; a.least = least;
        // as many value columns per CTA as the head has (the scores are made once per CTA), fewer while the launch would
        // leave SMs without a CTA
        int cb = columns_per_cta;
        if (cb <= 0) {
            cb = 64;
            while (cb > 16 && ((long long)n_chunks * heads * ((value_dim + cb - 1) / cb) < 148 || cb / 2 >= value_dim)) cb /= 2;
        }
        while (cb > 16 && reads_smem(key_dim, cb) > 110 * 1024 && reads_smem(key_dim, cb / 2) <= 110 * 1024) cb /= 2;   // two CTAs per SM
        if (reads_smem(key_dim, cb) > 227 * 1024) return -3;
        st = cb >= 64 ? launch_chunks<4>(a, n_req, n_chunks, s) : cb >= 32 ? launch_chunks<2>(a, n_req, n_chunks, s) : launch_chunks<1>(a, n_req, n_chunks, s);
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
