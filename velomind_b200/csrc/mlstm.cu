// The matrix-memory recurrence of an mLSTM layer (Beck et al., "xLSTM: Extended Long Short-Term Memory", 2024), with its
// output stage, over the fixed-size per-sequence state of the cache.
//
// Per head, with q already scaled by dim^-1/2, log gates i_t and f_t, and a running maximum m (m_-1 = 0, S_-1 = 0, n_-1 = 0):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          S: [dim, vdim]
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// The gates are soft-capped: i_t = cap tanh(x_i / cap), f_t = logsigmoid(cap tanh(x_f / cap)), x = projection + bias.
// Output stage: each head's o_t divided by its root mean square, times a learned scale over all heads, times sigmoid(g_t).
//
// Everything here is float32 whatever the activation dtype: gates, decays, the state, the sums, the unit norm.
//
// Input: the stacked projections' float32 result [T, ld] with columns q | k | v | g | x_i | x_f (H*D, H*D, H*V, H*V, H, H).
// State of a sequence (float32, indexed by the sequence's slot): per head S [D, V], n [D], m.
//
// Three forms: a token-by-token scan (the smallest pieces; the plain statement of the recurrence), a chunkwise form for
// prompts that turns the recurrence inside a chunk of tokens into small matrix products, and a decode step that streams
// the state once.
#include "common.cuh"

namespace {

__device__ __forceinline__ float soft_cap(float x, float cap) { return cap * tanhf(x / cap); }
__device__ __forceinline__ float log_sigmoid(float x) { return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------------ token by token
// One block per (head, sequence).  Thread v owns column v of S (in shared memory), thread d owns n[d].  Two barriers per token.
template <typename T>
__global__ void mlstm_scan_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                                  const float* __restrict__ norm_w, float* __restrict__ state, const int* __restrict__ cu_tokens,
                                  const int* __restrict__ slots, T* __restrict__ out, int H, int D, int V, float cap, float eps) {
    extern __shared__ float sm[];
    float* S = sm;                        // [D, V]
    float* qs = S + (size_t)D * V;        // [2, D]
    float* ks = qs + 2 * D;               // [2, D]
    float* gs = ks + 2 * D;               // [2, 4]: decay of the old state, weight of the new token, exp(-m)
    float* red = gs + 8;                  // [2, warps]
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
    if (t1 <= t0) return;
    const size_t head_floats = (size_t)D * V + D + 1;
    float* st = state + ((size_t)slots[s] * H + h) * head_floats;
    for (int i = tid; i < D * V; i += blockDim.x) S[i] = st[i];
    float n_d = tid < D ? st[(size_t)D * V + tid] : 0.f;
    float m = st[(size_t)D * V + D];
    const int off_k = H * D, off_v = 2 * H * D, off_g = off_v + H * V, off_i = off_g + H * V, off_f = off_i + H;
    const float q_scale = rsqrtf((float)D);
    const float bi = bias_i[h], bf = bias_f[h];
    const float nwt = tid < V ? norm_w[h * V + tid] : 0.f;
    __syncthreads();
    int buf = 0;
    for (int t = t0; t < t1; ++t, buf ^= 1) {
        const float* row = proj + (size_t)t * ld;
        if (tid < D) {
            qs[buf * D + tid] = row[h * D + tid] * q_scale;
            ks[buf * D + tid] = row[off_k + h * D + tid];
        }
        float vv = 0.f, gate = 0.f;
        if (tid < V) {
            vv = row[off_v + h * V + tid];
            gate = row[off_g + h * V + tid];
        }
        // every thread derives the token's three scalars itself (the same arithmetic, the same result)
        const float ig = soft_cap(row[off_i + h] + bi, cap);
        const float fg = log_sigmoid(soft_cap(row[off_f + h] + bf, cap));
        const float m_new = fmaxf(fg + m, ig);
        const float a = expf(fg + m - m_new), b = expf(ig - m_new);
        m = m_new;
        __syncthreads();
        const float* qb = qs + buf * D;
        const float* kb = ks + buf * D;
        float num = 0.f, nq = 0.f;
        if (tid < V) {
            const float bv = b * vv;
            for (int d = 0; d < D; ++d) {
                const float sv = fmaf(a, S[d * V + tid], kb[d] * bv);
                S[d * V + tid] = sv;
                num = fmaf(sv, qb[d], num);
            }
        }
        if (tid < D) {
            n_d = fmaf(a, n_d, b * kb[tid]);
            nq = n_d * qb[tid];
        }
        float r0 = vm_warp_sum(nq), r1 = vm_warp_sum(num * num);
        if (lane == 0) { red[(buf * nw + warp) * 2] = r0; red[(buf * nw + warp) * 2 + 1] = r1; }
        __syncthreads();
        float tot_nq = 0.f, tot_sq = 0.f;
        for (int w = 0; w < nw; ++w) { tot_nq += red[(buf * nw + w) * 2]; tot_sq += red[(buf * nw + w) * 2 + 1]; }
        if (tid < V) {
            const float den = fmaxf(fabsf(tot_nq), expf(-m)) + 1e-6f;
            const float o = num / den;
            const float ms = tot_sq / (den * den) / (float)V;
            const float y = o * (1.0f / sqrtf(ms + eps)) * nwt * (1.0f / (1.0f + expf(-gate)));
            out[(size_t)t * H * V + h * V + tid] = vm_from_float<T>(y);
        }
    }
    __syncthreads();
    for (int i = tid; i < D * V; i += blockDim.x) st[i] = S[i];
    if (tid < D) st[(size_t)D * V + tid] = n_d;
    if (tid == 0) st[(size_t)D * V + D] = m;
}

template <typename T>
int launch_scan(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                const int* slots, void* out, int B, int H, int D, int V, float cap, float eps, cudaStream_t stream) {
    int threads = ((D > V ? D : V) + 31) / 32 * 32;
    if (threads < 64) threads = 64;
    if (threads > 1024) return VM_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)D * V + 4 * D + 8 + 4 * (threads / 32)) * sizeof(float);
    if (smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        static size_t raised = 0;       // per instantiation
        if (smem > raised) {
            if (cudaFuncSetAttribute(mlstm_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return vm_launch_status();
            raised = smem;
        }
    }
    vm_launch_pdl(mlstm_scan_kernel<T>, dim3(H, B), dim3(threads), smem, stream, proj, ld, bias_i, bias_f, norm_w, state, cu_tokens, slots, (T*)out, H, D,
                  V, cap, eps);
    return vm_launch_status();
}

// ------------------------------------------------------------------------------------------------ chunk by chunk
// Inside a chunk of L tokens that starts from (S', n', m') the recurrence has a closed form.  With F_j the sum of the log
// forget gates up to token j of the chunk, a_s = i_s - F_s, c_j = max_{s<=j} a_s and g_j = max(m', c_j):
//     m_j       = F_j + g_j
//     S_j^T q_j = exp(m' - g_j) S'^T q_j + exp(c_j - g_j) sum_{s<=j} exp(a_s - c_j) (k_s . q_j) v_s
//     n_j . q_j = exp(m' - g_j) n' . q_j + exp(c_j - g_j) sum_{s<=j} exp(a_s - c_j) (k_s . q_j)
//     S_end     = exp(m' - g_L) S'       + exp(c_L - g_L) sum_s exp(a_s - c_L) k_s v_s^T
// (every exponent is <= 0).  The sums over s need nothing from earlier chunks, so prompts run in three passes:
//   local   every chunk of every sequence at once: the weighted scores, their products with v, and the chunk's own
//           contribution to the state (grid: value slices x heads x chunks)
//   carry   per sequence, chunk after chunk, elementwise: the state at every chunk's start, the state at the prompt's end
//   finish  every chunk at once again: the old state's share of the answer, the denominator
// and the output stage.  F, a, c and g are float64, so that a chunk of strong forget gates does not cost the weights their
// float32 digits; everything else is float32.  The products are register-tiled (4 x 4 per thread) from shared memory.
constexpr int CHUNK_THREADS = 256;

struct ChunkSizes {
    int L, VS, slices, Dp, VSp;
    size_t smem;
};

inline ChunkSizes chunk_sizes(int D, int V) {
    ChunkSizes c;
    c.VS = V <= 64 ? V : 64;
    c.slices = (V + c.VS - 1) / c.VS;
    c.Dp = (D + 3) / 4 * 4;
    c.VSp = (c.VS + 3) / 4 * 4;
    c.L = 64;
    auto floats = [&](int L) {
        // Qt [Dp, L + 8], Kt [Dp, L + 8] (finish: S' [Dp, VSp] in its place), Vs [L, VSp], Pt [L, L], 6 float rows of L, 3 double rows of L
        const size_t second = (size_t)c.Dp * (L + 8) > (size_t)c.Dp * c.VSp ? (size_t)c.Dp * (L + 8) : (size_t)c.Dp * c.VSp;
        return (size_t)c.Dp * (L + 8) + second + (size_t)L * c.VSp + (size_t)L * L + c.Dp + 6 * (size_t)L + 6 * (size_t)L;
    };
    while (c.L > 8 && floats(c.L) * sizeof(float) + 64 > 200 * 1024) c.L /= 2;
    c.smem = floats(c.L) * sizeof(float) + 64;
    return c;
}

// which sequence and which of its chunks block z works on (-1: none); sequences have ceil(n / L) chunks each
__device__ __forceinline__ void find_chunk(const int* __restrict__ cu_tokens, int B, int L, int z, int* seq, int* first, int* count) {
    int at = 0;
    *seq = -1;
    for (int s = 0; s < B; ++s) {
        const int n = cu_tokens[s + 1] - cu_tokens[s];
        const int chunks = (n + L - 1) / L;
        if (z < at + chunks) {
            *seq = s;
            *first = cu_tokens[s] + (z - at) * L;
            *count = min(L, cu_tokens[s + 1] - *first);
            return;
        }
        at += chunks;
    }
}

// the gates of a chunk, by warp 0: a_s, c_s, F_s (float64, shared memory) for j < L (j >= Lc: weightless)
__device__ __forceinline__ void chunk_gates(const float* __restrict__ proj, int ld, int c0, int Lc, int L, int off_i, int off_f, int h, float bi, float bf,
                                            float cap, double* a_s, double* c_s, double* F_s, int lane) {
    double run_f = 0.0, run_c = -1e300;
    for (int base = 0; base < L; base += 32) {
        const int j = base + lane;
        double fg = 0.0, ig = 0.0;
        if (j < Lc) {
            const float* row = proj + (size_t)(c0 + j) * ld;
            ig = (double)soft_cap(row[off_i + h] + bi, cap);
            fg = (double)log_sigmoid(soft_cap(row[off_f + h] + bf, cap));
        }
        double F = fg;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const double up = __shfl_up_sync(0xffffffffu, F, o); if (lane >= o) F += up; }
        F += run_f;
        const double a = j < Lc ? ig - F : -1e300;
        double mx = a;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const double up = __shfl_up_sync(0xffffffffu, mx, o); if (lane >= o) mx = fmax(mx, up); }
        mx = fmax(mx, run_c);
        if (j < L) { a_s[j] = a; c_s[j] = mx; F_s[j] = F; }
        run_f = __shfl_sync(0xffffffffu, F, 31);
        run_c = __shfl_sync(0xffffffffu, mx, 31);
    }
}

struct ChunkSmem {
    float *Qt, *Kt, *Vs, *Pt, *nprev, *r0, *r1, *r2, *r3, *r4, *r5;
    double *a_s, *c_s, *F_s;
};
__device__ __forceinline__ ChunkSmem carve(float* sm, int L, int Dp, int VSp) {
    ChunkSmem m;
    const size_t second = (size_t)Dp * (L + 8) > (size_t)Dp * VSp ? (size_t)Dp * (L + 8) : (size_t)Dp * VSp;
    m.Qt = sm;
    m.Kt = m.Qt + (size_t)Dp * (L + 8);
    m.Vs = m.Kt + second;
    m.Pt = m.Vs + (size_t)L * VSp;
    m.nprev = m.Pt + (size_t)L * L;
    m.r0 = m.nprev + Dp; m.r1 = m.r0 + L; m.r2 = m.r1 + L; m.r3 = m.r2 + L; m.r4 = m.r3 + L; m.r5 = m.r4 + L;
    float* d = m.r5 + L;
    d += (reinterpret_cast<uintptr_t>(d) & 7) ? 1 : 0;
    m.a_s = reinterpret_cast<double*>(d);
    m.c_s = m.a_s + L;
    m.F_s = m.c_s + L;
    return m;
}

// ---- pass 1
__global__ void __launch_bounds__(CHUNK_THREADS)
mlstm_chunk_local_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                         const int* __restrict__ cu_tokens, int B, float* __restrict__ o_raw, float* __restrict__ nq_buf, float* __restrict__ dS,
                         float* __restrict__ dn, double* __restrict__ chunk_fc, int H, int D, int V, int L, int VS, int Dp, int VSp, float cap) {
    extern __shared__ __align__(16) float sm[];
    const ChunkSmem m = carve(sm, L, Dp, VSp);
    __shared__ int where[3];
    const int slice = blockIdx.x, h = blockIdx.y, z = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) find_chunk(cu_tokens, B, L, z, &where[0], &where[1], &where[2]);
    __syncthreads();
    if (where[0] < 0) return;
    const int c0 = where[1], Lc = where[2];
    const int v0 = slice * VS, vs = min(VS, V - v0);
    const int off_k = H * D, off_v = 2 * H * D, off_i = 2 * H * D + 2 * H * V, off_f = off_i + H;
    const float q_scale = rsqrtf((float)D);
    // q and k transposed into rows of L + 8 floats: a warp takes 4 values of d for 8 tokens, which lands in 32 different banks
    const int LS = L + 8;
    for (int i = tid; i < L * Dp; i += CHUNK_THREADS) {
        const int tile = i >> 5, dt = tile % (Dp / 4), d = 4 * dt + (i & 3), j = 8 * (tile / (Dp / 4)) + ((i & 31) >> 2);
        float q = 0.f, k = 0.f;
        if (j < Lc && d < D) {
            const float* row = proj + (size_t)(c0 + j) * ld;
            q = row[h * D + d] * q_scale;
            k = row[off_k + h * D + d];
        }
        m.Qt[d * LS + j] = q;
        m.Kt[d * LS + j] = k;
    }
    for (int i = tid; i < L * VSp; i += CHUNK_THREADS) {
        const int j = i / VSp, v = i - j * VSp;
        m.Vs[i] = (j < Lc && v < vs) ? proj[(size_t)(c0 + j) * ld + off_v + h * V + v0 + v] : 0.f;
    }
    if (warp == 0) chunk_gates(proj, ld, c0, Lc, L, off_i, off_f, h, bias_i[h], bias_f[h], cap, m.a_s, m.c_s, m.F_s, lane);
    __syncthreads();
    float* wend = m.r0;                   // exp(a_s - c_last): the tokens' weights in the chunk's contribution to the state
    for (int j = tid; j < L; j += CHUNK_THREADS) wend[j] = j < Lc ? expf((float)(m.a_s[j] - m.c_s[Lc - 1])) : 0.f;
    // weighted scores, transposed: Pt[s][j] = exp(a_s - c_j) (q_j . k_s) for s <= j, else 0
    const int LT = L / 4;
    for (int tt = tid; tt < LT * LT; tt += CHUNK_THREADS) {
        const int jt = tt / LT, st = tt - jt * LT;
        if (st > jt) continue;
        float acc[4][4] = {};
        for (int d = 0; d < Dp; ++d) {
            const float4 q4 = *reinterpret_cast<const float4*>(m.Qt + d * LS + 4 * jt);
            const float4 k4 = *reinterpret_cast<const float4*>(m.Kt + d * LS + 4 * st);
            const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, kb[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], kb[b], acc[a][b]);
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int ss = 4 * st + b;
            float p[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int j = 4 * jt + a;
                p[a] = (ss <= j && j < Lc) ? acc[a][b] * expf((float)(m.a_s[ss] - m.c_s[j])) : 0.f;
            }
            *reinterpret_cast<float4*>(m.Pt + ss * L + 4 * jt) = make_float4(p[0], p[1], p[2], p[3]);
        }
    }
    __syncthreads();
    if (slice == 0) {
        for (int j = tid; j < Lc; j += CHUNK_THREADS) {
            float acc = 0.f;
            for (int ss = 0; ss <= j; ++ss) acc += m.Pt[ss * L + j];
            nq_buf[(size_t)(c0 + j) * H + h] = acc;
        }
    }
    // the scores' products with v
    const int VT = VSp / 4;
    for (int tt = tid; tt < LT * VT; tt += CHUNK_THREADS) {
        const int jt = tt / VT, vt = tt - jt * VT;
        float acc[4][4] = {};
        const int last = min(4 * jt + 3, Lc - 1);
        for (int ss = 0; ss <= last; ++ss) {
            const float4 p4 = *reinterpret_cast<const float4*>(m.Pt + ss * L + 4 * jt);
            const float4 v4 = *reinterpret_cast<const float4*>(m.Vs + ss * VSp + 4 * vt);
            const float pa[4] = {p4.x, p4.y, p4.z, p4.w}, vb[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(pa[a], vb[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int j = 4 * jt + a;
            if (j >= Lc) continue;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (4 * vt + b < vs) o_raw[(size_t)(c0 + j) * H * V + h * V + v0 + 4 * vt + b] = acc[a][b];
        }
    }
    // the chunk's contribution to the state: dS[d][v] = sum_s wend[s] k_s[d] v_s[v], dn[d] = sum_s wend[s] k_s[d]
    float* dS_c = dS + ((size_t)z * H + h) * (size_t)D * V;
    const int DT = Dp / 4;
    for (int tt = tid; tt < DT * VT; tt += CHUNK_THREADS) {
        const int dt = tt / VT, vt = tt - dt * VT;
        float acc[4][4] = {};
        for (int ss = 0; ss < Lc; ++ss) {
            const float w = wend[ss];
            const float4 v4 = *reinterpret_cast<const float4*>(m.Vs + ss * VSp + 4 * vt);
            const float vb[4] = {v4.x * w, v4.y * w, v4.z * w, v4.w * w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float k = m.Kt[(4 * dt + a) * LS + ss];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(k, vb[b], acc[a][b]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (4 * dt + a < D && 4 * vt + b < vs) dS_c[(size_t)(4 * dt + a) * V + v0 + 4 * vt + b] = acc[a][b];
    }
    if (slice == 0) {
        for (int d = tid; d < D; d += CHUNK_THREADS) {
            float acc = 0.f;
            for (int ss = 0; ss < Lc; ++ss) acc = fmaf(wend[ss], m.Kt[d * LS + ss], acc);
            dn[((size_t)z * H + h) * D + d] = acc;
        }
        if (tid == 0) {
            chunk_fc[((size_t)z * H + h) * 2] = m.F_s[Lc - 1];
            chunk_fc[((size_t)z * H + h) * 2 + 1] = m.c_s[Lc - 1];
        }
    }
}

// ---- pass 2: one thread per element of S and of n; dS / dn come in as the chunks' contributions and go out as the state at each
// chunk's START; m at each chunk's start goes to chunk_m; the prompt's last n and m go to end_nm (the output stage commits them)
__global__ void mlstm_chunk_carry_kernel(float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int B,
                                         float* __restrict__ dS, float* __restrict__ dn, const double* __restrict__ chunk_fc,
                                         double* __restrict__ chunk_m, float* __restrict__ end_nm, int H, int D, int V, int L) {
    const int h = blockIdx.y, s = blockIdx.z;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int n_tok = cu_tokens[s + 1] - cu_tokens[s];
    if (n_tok <= 0 || e >= D * V + D) return;
    int z = 0;
    for (int r = 0; r < s; ++r) z += (cu_tokens[r + 1] - cu_tokens[r] + L - 1) / L;
    const int chunks = (n_tok + L - 1) / L;
    float* st = state + ((size_t)slots[s] * H + h) * ((size_t)D * V + D + 1);
    const bool is_n = e >= D * V;
    float x = st[e];                                   // S elements, then n, lie in this order
    double m = (double)st[(size_t)D * V + D];
    // eight chunks at a time: their contributions are fetched together (independent loads), then the state walks through them
    constexpr int AT_ONCE = 8;
    const size_t stride = is_n ? (size_t)H * D : (size_t)H * D * V;           // from one chunk's entry to the next chunk's
    float* base = is_n ? dn + ((size_t)z * H + h) * D + (e - D * V) : dS + ((size_t)z * H + h) * (size_t)D * V + e;
    for (int c = 0; c < chunks; c += AT_ONCE, z += AT_ONCE, base += AT_ONCE * stride) {
        float add[AT_ONCE];
#pragma unroll
        for (int i = 0; i < AT_ONCE; ++i) add[i] = c + i < chunks ? base[i * stride] : 0.f;
#pragma unroll
        for (int i = 0; i < AT_ONCE; ++i) {
            if (c + i >= chunks) break;
            const size_t zh = (size_t)(z + i) * H + h;
            base[i * stride] = x;
            if (e == 0) chunk_m[zh] = m;
            const double F = chunk_fc[zh * 2], c_last = chunk_fc[zh * 2 + 1];
            const double g = fmax(m, c_last);
            x = expf((float)(m - g)) * x + expf((float)(c_last - g)) * add[i];
            m = F + g;
        }
    }
    if (!is_n) st[e] = x;
    else end_nm[((size_t)s * H + h) * (D + 1) + (e - D * V)] = x;
    if (e == 0) end_nm[((size_t)s * H + h) * (D + 1) + D] = (float)m;
}

// ---- pass 3
__global__ void __launch_bounds__(CHUNK_THREADS)
mlstm_chunk_finish_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                          const int* __restrict__ cu_tokens, int B, float* __restrict__ o_raw, const float* __restrict__ nq_buf,
                          const float* __restrict__ S_start, const float* __restrict__ n_start, const double* __restrict__ chunk_m, int H, int D, int V,
                          int L, int VS, int Dp, int VSp, float cap) {
    extern __shared__ __align__(16) float sm[];
    const ChunkSmem m = carve(sm, L, Dp, VSp);
    __shared__ int where[3];
    const int slice = blockIdx.x, h = blockIdx.y, z = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) find_chunk(cu_tokens, B, L, z, &where[0], &where[1], &where[2]);
    __syncthreads();
    if (where[0] < 0) return;
    const int c0 = where[1], Lc = where[2];
    const int v0 = slice * VS, vs = min(VS, V - v0);
    const int off_i = 2 * H * D + 2 * H * V, off_f = off_i + H;
    const float q_scale = rsqrtf((float)D);
    const size_t zh = (size_t)z * H + h;
    const int LS = L + 8;
    for (int i = tid; i < L * Dp; i += CHUNK_THREADS) {
        const int tile = i >> 5, dt = tile % (Dp / 4), d = 4 * dt + (i & 3), j = 8 * (tile / (Dp / 4)) + ((i & 31) >> 2);
        m.Qt[d * LS + j] = (j < Lc && d < D) ? proj[(size_t)(c0 + j) * ld + h * D + d] * q_scale : 0.f;
    }
    float* Ss = m.Kt;                     // [Dp, VSp]: the slice's columns of the state at the chunk's start
    for (int i = tid; i < Dp * VSp; i += CHUNK_THREADS) {
        const int d = i / VSp, v = i - d * VSp;
        Ss[i] = (d < D && v < vs) ? S_start[zh * (size_t)D * V + (size_t)d * V + v0 + v] : 0.f;
    }
    for (int d = tid; d < Dp; d += CHUNK_THREADS) m.nprev[d] = d < D ? n_start[zh * D + d] : 0.f;
    if (warp == 0) chunk_gates(proj, ld, c0, Lc, L, off_i, off_f, h, bias_i[h], bias_f[h], cap, m.a_s, m.c_s, m.F_s, lane);
    __syncthreads();
    const double m_prev = chunk_m[zh];
    float *w_loc = m.r0, *w_old = m.r1, *den = m.r2;
    for (int j = tid; j < Lc; j += CHUNK_THREADS) {
        const double g = fmax(m_prev, m.c_s[j]);
        const float wl = expf((float)(m.c_s[j] - g)), wo = expf((float)(m_prev - g));
        float old = 0.f;
        for (int d = 0; d < D; ++d) old = fmaf(m.nprev[d], m.Qt[d * LS + j], old);
        const float nq = fmaf(wl, nq_buf[(size_t)(c0 + j) * H + h], wo * old);
        w_loc[j] = wl;
        w_old[j] = wo;
        den[j] = fmaxf(fabsf(nq), expf((float)(-(m.F_s[j] + g)))) + 1e-6f;
    }
    __syncthreads();
    const int LT = L / 4, VT = VSp / 4;
    for (int tt = tid; tt < LT * VT; tt += CHUNK_THREADS) {
        const int jt = tt / VT, vt = tt - jt * VT;
        if (4 * jt >= Lc) continue;
        float acc[4][4] = {};
        for (int d = 0; d < Dp; ++d) {
            const float4 q4 = *reinterpret_cast<const float4*>(m.Qt + d * LS + 4 * jt);
            const float4 s4 = *reinterpret_cast<const float4*>(Ss + d * VSp + 4 * vt);
            const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, sb[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], sb[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int j = 4 * jt + a;
            if (j >= Lc) continue;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (4 * vt + b >= vs) continue;
                float* o = o_raw + (size_t)(c0 + j) * H * V + h * V + v0 + 4 * vt + b;
                *o = fmaf(w_loc[j], *o, w_old[j] * acc[a][b]) / den[j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ one token per sequence
// A decode step streams the state through the SMs once: a block per (64 value columns, head, sequence) reads its columns of
// S, moves them on by one token and sums its share of S^T q on the way.  n and m go to the scratch row (every slice needs the
// OLD n; the output stage commits the new one), o to the float32 buffer.
__global__ void __launch_bounds__(256)
mlstm_step_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias_i, const float* __restrict__ bias_f, float* __restrict__ state,
                  const int* __restrict__ slots, float* __restrict__ o_raw, float* __restrict__ end_nm, int H, int D, int V, float cap) {
    extern __shared__ float sm[];          // q [D], k [D], partial sums [4][64], 8 warp sums
    float* qs = sm;
    float* ks = sm + D;
    float* part = ks + D;
    float* red = part + 256;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int slice = blockIdx.x, h = blockIdx.y, s = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v = slice * 64 + (tid & 63), dg = tid >> 6;
    const float* row = proj + (size_t)s * ld;          // one token per sequence: token s belongs to sequence s
    float* st = state + ((size_t)slots[s] * H + h) * ((size_t)D * V + D + 1);
    const int off_k = H * D, off_v = 2 * H * D, off_i = 2 * H * D + 2 * H * V, off_f = off_i + H;
    const float q_scale = rsqrtf((float)D);
    for (int d = tid; d < D; d += 256) {
        qs[d] = row[h * D + d] * q_scale;
        ks[d] = row[off_k + h * D + d];
    }
    const float m_old = st[(size_t)D * V + D];
    const float ig = soft_cap(row[off_i + h] + bias_i[h], cap);
    const float fg = log_sigmoid(soft_cap(row[off_f + h] + bias_f[h], cap));
    const float m_new = fmaxf(fg + m_old, ig);
    const float a = expf(fg + m_old - m_new), b = expf(ig - m_new);
    __syncthreads();
    // n . q with the new n (every slice the same); slice 0 leaves the new n and m in the scratch row
    float nq = 0.f;
    for (int d = tid; d < D; d += 256) {
        const float n_new = fmaf(a, st[(size_t)D * V + d], b * ks[d]);
        nq = fmaf(n_new, qs[d], nq);
        if (slice == 0) end_nm[((size_t)s * H + h) * (D + 1) + d] = n_new;
    }
    if (slice == 0 && tid == 0) end_nm[((size_t)s * H + h) * (D + 1) + D] = m_new;
    nq = vm_warp_sum(nq);
    if (lane == 0) red[warp] = nq;
    float num = 0.f;
    if (v < V) {
        const float bv = b * row[off_v + h * V + v];
        constexpr int AT_ONCE = 8;                     // the state's values are fetched eight at a time, then moved on and stored
        for (int d0 = dg; d0 < D; d0 += 4 * AT_ONCE) {
            float old[AT_ONCE];
#pragma unroll
            for (int i = 0; i < AT_ONCE; ++i) old[i] = d0 + 4 * i < D ? st[(size_t)(d0 + 4 * i) * V + v] : 0.f;
#pragma unroll
            for (int i = 0; i < AT_ONCE; ++i) {
                const int d = d0 + 4 * i;
                if (d >= D) break;
                const float sv = fmaf(a, old[i], ks[d] * bv);
                st[(size_t)d * V + v] = sv;
                num = fmaf(sv, qs[d], num);
            }
        }
    }
    part[tid] = num;
    __syncthreads();
    if (tid < 64 && v < V) {
        float tot_nq = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot_nq += red[w];
        const float den = fmaxf(fabsf(tot_nq), expf(-m_new)) + 1e-6f;
        o_raw[(size_t)s * H * V + h * V + v] = (part[tid] + part[tid + 64] + part[tid + 128] + part[tid + 192]) / den;
    }
}

// The output stage after the chunk kernel: a warp per (token, head) divides o by its root mean square, applies the learned
// scale and the sigmoid gate; the first warps also move the sequences' new n and m from the scratch rows into the state.
template <typename T>
__global__ void mlstm_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, const float* __restrict__ norm_w,
                                    T* __restrict__ out, int n_tokens, int H, int D, int V, float eps, const float* __restrict__ end_nm,
                                    float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int B) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w < (long long)B * H) {
        const int s = (int)(w / H), h = (int)(w % H);
        if (cu_tokens[s + 1] > cu_tokens[s]) {
            const float* e = end_nm + ((size_t)s * H + h) * (D + 1);
            float* st = state + ((size_t)slots[s] * H + h) * ((size_t)D * V + D + 1) + (size_t)D * V;
            for (int d = lane; d <= D; d += 32) st[d] = e[d];
        }
    }
    if (w >= (long long)n_tokens * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    const float* o = o_raw + (size_t)t * H * V + h * V;
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) ss = fmaf(o[v], o[v], ss);
    ss = vm_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    const float* gate = proj + (size_t)t * ld + 2 * H * D + H * V + h * V;
    for (int v = lane; v < V; v += 32)
        out[(size_t)t * H * V + h * V + v] = vm_from_float<T>(o[v] * inv * norm_w[h * V + v] * (1.0f / (1.0f + expf(-gate[v]))));
}


}  // namespace

// scratch floats of the chunkwise form: the un-normalised o [T, H*V], a row of n, m per (sequence, head), n . q per (token, head), and per
// (chunk, head) the state S, n at the chunk's start and (as float64) its gate sums and m
VM_API long long vm_mlstm_chunk_scratch_floats(int T, int B, int H, int D, int V) {
    const ChunkSizes c = chunk_sizes(D, V);
    const long long chunks = (long long)T / c.L + B + 1;
    return (long long)T * H * V + (long long)B * H * (D + 1) + (long long)T * H + chunks * H * ((long long)D * V + D) + 2 + chunks * H * 6;
}

VM_API int vm_mlstm_chunks(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                           const int* slots, void* out, float* scratch, int T, int B, int H, int D, int V, float cap, float eps, int act_dtype,
                           cudaStream_t stream) {
    if (B <= 0 || T <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + 2 * H * V + 2 * H || !(cap > 0.f)) return VM_ERR_BAD_ARG;
    if (act_dtype != VM_F32 && act_dtype != VM_BF16) return VM_ERR_UNSUPPORTED;
    const ChunkSizes c = chunk_sizes(D, V);
    if (c.smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    static size_t raised = 0;
    if (c.smem > 48 * 1024 && c.smem > raised) {
        if (cudaFuncSetAttribute(mlstm_chunk_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess ||
            cudaFuncSetAttribute(mlstm_chunk_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess)
            return vm_launch_status();
        raised = c.smem;
    }
    const long long chunks = (long long)T / c.L + B + 1;          // at least sum over sequences of ceil(n / L)
    if (chunks > 65535) return VM_ERR_UNSUPPORTED;
    float* o_raw = scratch;
    float* end_nm = o_raw + (size_t)T * H * V;
    float* nq_buf = end_nm + (size_t)B * H * (D + 1);
    float* dS = nq_buf + (size_t)T * H;
    float* dn = dS + (size_t)chunks * H * D * V;
    float* after = dn + (size_t)chunks * H * D;
    after += (reinterpret_cast<uintptr_t>(after) & 7) ? 1 : 0;
    double* chunk_fc = reinterpret_cast<double*>(after);
    double* chunk_m = chunk_fc + (size_t)chunks * H * 2;
    mlstm_chunk_local_kernel<<<dim3(c.slices, H, (unsigned)chunks), CHUNK_THREADS, c.smem, stream>>>(proj, ld, bias_i, bias_f, cu_tokens, B, o_raw, nq_buf, dS,
                                                                                                   dn, chunk_fc, H, D, V, c.L, c.VS, c.Dp, c.VSp, cap);
    int st = vm_launch_status();
    if (st) return st;
    mlstm_chunk_carry_kernel<<<dim3((D * V + D + 255) / 256, H, B), 256, 0, stream>>>(state, cu_tokens, slots, B, dS, dn, chunk_fc, chunk_m, end_nm, H, D, V,
                                                                                    c.L);
    st = vm_launch_status();
    if (st) return st;
    mlstm_chunk_finish_kernel<<<dim3(c.slices, H, (unsigned)chunks), CHUNK_THREADS, c.smem, stream>>>(proj, ld, bias_i, bias_f, cu_tokens, B, o_raw, nq_buf, dS,
                                                                                                    dn, chunk_m, H, D, V, c.L, c.VS, c.Dp, c.VSp, cap);
    st = vm_launch_status();
    if (st) return st;
    const long long warps = (long long)T * H > (long long)B * H ? (long long)T * H : (long long)B * H;
    const int blocks = (int)((warps + 7) / 8);
    if (act_dtype == VM_F32)
        mlstm_output_kernel<float><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (float*)out, T, H, D, V, eps, end_nm, state, cu_tokens, slots, B);
    else
        mlstm_output_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (__nv_bfloat16*)out, T, H, D, V, eps, end_nm, state,
                                                                       cu_tokens, slots, B);
    return vm_launch_status();
}

// One token per sequence (token s is sequence s): scratch of B * H * (V + D + 1) floats.
VM_API int vm_mlstm_step(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                         const int* slots, void* out, float* scratch, int B, int H, int D, int V, float cap, float eps, int act_dtype,
                         cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + 2 * H * V + 2 * H || !(cap > 0.f)) return VM_ERR_BAD_ARG;
    if (act_dtype != VM_F32 && act_dtype != VM_BF16) return VM_ERR_UNSUPPORTED;
    if ((size_t)(2 * D + 256 + 8) * sizeof(float) > 48 * 1024 || B > 65535) return VM_ERR_UNSUPPORTED;
    float* o_raw = scratch;
    float* end_nm = scratch + (size_t)B * H * V;
    vm_launch_pdl(mlstm_step_kernel, dim3((V + 63) / 64, H, B), dim3(256), (size_t)(2 * D + 256 + 8) * sizeof(float), stream, proj, ld, bias_i, bias_f,
                  state, slots, o_raw, end_nm, H, D, V, cap);
    int st = vm_launch_status();
    if (st) return st;
    const int blocks = (int)(((long long)B * H + 7) / 8);
    if (act_dtype == VM_F32)
        mlstm_output_kernel<float><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (float*)out, B, H, D, V, eps, end_nm, state, cu_tokens, slots, B);
    else
        mlstm_output_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (__nv_bfloat16*)out, B, H, D, V, eps, end_nm, state,
                                                                       cu_tokens, slots, B);
    return vm_launch_status();
}

// whether the token-by-token kernel takes heads of these sizes (its block holds a head's whole S in shared memory)
VM_API int vm_mlstm_scan_fits(int D, int V) {
    const int widest = D > V ? D : V;
    return widest <= 1024 && ((size_t)D * V + 4 * D + 8 + 4 * 32) * sizeof(float) <= 200 * 1024 ? 1 : 0;
}

VM_API int vm_mlstm_scan(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                         const int* slots, void* out, int B, int H, int D, int V, float cap, float eps, int act_dtype, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + 2 * H * V + 2 * H || !(cap > 0.f)) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_F32) return launch_scan<float>(proj, ld, bias_i, bias_f, norm_w, state, cu_tokens, slots, out, B, H, D, V, cap, eps, stream);
    if (act_dtype == VM_BF16)
        return launch_scan<__nv_bfloat16>(proj, ld, bias_i, bias_f, norm_w, state, cu_tokens, slots, out, B, H, D, V, cap, eps, stream);
    return VM_ERR_UNSUPPORTED;
}
