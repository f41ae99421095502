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
// Two kernels: a token-by-token scan (decode steps, short pieces, and the exact reference of the other one), and a
// chunkwise form for prompts that turns the recurrence inside a chunk of tokens into small matrix products.
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
// forget gates up to token j of the chunk, a_s = i_s - F_s and g_j = max(m', max_{s<=j} a_s):
//     m_j   = F_j + g_j
//     S_j   = exp(m' - g_j) S' + sum_{s<=j} exp(a_s - g_j) k_s v_s^T          (every exponent is <= 0)
//     S_j^T q_j = exp(m' - g_j) S'^T q_j + sum_{s<=j} exp(a_s - g_j) (k_s . q_j) v_s
//     n_j . q_j = exp(m' - g_j) n' . q_j + sum_{s<=j} exp(a_s - g_j) (k_s . q_j)
// so a chunk is three small matrix products (q k^T, weights times v, q times the old state) and the state moves on once per
// chunk.  F, a and g are summed in float64 and differences are taken there, so that a long chunk of strong forget gates does
// not cost the weights their float32 digits; everything else is float32.
//
// One block per (slice of value columns, head, sequence): the slice's columns of S live in shared memory for the whole
// prompt.  Every slice needs the scores and n . q, and computes them itself.  The un-normalised o goes to a float32 buffer
// (the unit norm needs all slices of a head), n and m of the sequence's end to a scratch row; the output kernel that follows
// finishes both.
constexpr int CHUNK_THREADS = 256;

struct ChunkSizes {
    int L, VS, slices;
    size_t smem;
};

__host__ __device__ inline size_t chunk_smem_floats(int L, int D, int VS) {
    // Q [L, D+1], Kt [D, L], Vs [L, VS], P [L, L], S [D, VS], n [D], nq [L], wdec [L], wend [L], doubles a [L], g [L] (as 4 L floats)
    return (size_t)L * (D + 1) + (size_t)D * L + (size_t)L * VS + (size_t)L * L + (size_t)D * VS + D + 3 * (size_t)L + 4 * (size_t)L;
}

__global__ void __launch_bounds__(CHUNK_THREADS)
mlstm_chunk_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                   float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots, float* __restrict__ o_raw,
                   float* __restrict__ end_nm, int H, int D, int V, int L, int VS, float cap) {
    extern __shared__ __align__(16) float sm[];
    float* Q = sm;                                   // [L, D + 1]
    float* Kt = Q + (size_t)L * (D + 1);             // [D, L]
    float* Vs = Kt + (size_t)D * L;                  // [L, VS]
    float* P = Vs + (size_t)L * VS;                  // [L, L]
    float* S = P + (size_t)L * L;                    // [D, VS]
    float* nv = S + (size_t)D * VS;                  // [D]
    float* nq = nv + D;                              // [L]
    float* wdec = nq + L;                            // [L] exp(m' - g_j)
    float* wend = wdec + L;                          // [L] exp(a_s - g_last)
    double* a_s = reinterpret_cast<double*>(wend + L + ((reinterpret_cast<uintptr_t>(wend + L) & 7) ? 1 : 0));   // [L]
    double* g_s = a_s + L;                           // [L]
    __shared__ double m_carry;
    const int slice = blockIdx.x, h = blockIdx.y, s = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
    if (t1 <= t0) return;
    const int v0 = slice * VS, vs = min(VS, V - v0);
    const size_t head_floats = (size_t)D * V + D + 1;
    float* st = state + ((size_t)slots[s] * H + h) * head_floats;
    for (int i = tid; i < D * vs; i += CHUNK_THREADS) { const int d = i / vs, v = i - d * vs; S[d * VS + v] = st[(size_t)d * V + v0 + v]; }
    for (int d = tid; d < D; d += CHUNK_THREADS) nv[d] = st[(size_t)D * V + d];
    if (tid == 0) m_carry = (double)st[(size_t)D * V + D];
    const int off_k = H * D, off_v = 2 * H * D, off_i = 2 * H * D + 2 * H * V, off_f = off_i + H;
    const float q_scale = rsqrtf((float)D);
    const float bi = bias_i[h], bf = bias_f[h];
    __syncthreads();
    for (int c0 = t0; c0 < t1; c0 += L) {
        const int Lc = min(L, t1 - c0);
        // ---- the chunk's q, k, v
        for (int i = tid; i < Lc * D; i += CHUNK_THREADS) {
            const int j = i / D, d = i - j * D;
            const float* row = proj + (size_t)(c0 + j) * ld;
            Q[j * (D + 1) + d] = row[h * D + d] * q_scale;
            Kt[d * L + j] = row[off_k + h * D + d];
        }
        for (int i = tid; i < Lc * vs; i += CHUNK_THREADS) {
            const int j = i / vs, v = i - j * vs;
            Vs[j * VS + v] = proj[(size_t)(c0 + j) * ld + off_v + h * V + v0 + v];
        }
        // ---- gates: F (inclusive sums of the log forget gates), a = i - F, g = max(m', running max of a); one warp, float64
        if (warp == 0) {
            const double m_prev = m_carry;
            double run_f = 0.0, run_a = -1e300;
            for (int base = 0; base < Lc; base += 32) {
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
                double a = j < Lc ? ig - F : -1e300;
                double mx = a;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const double up = __shfl_up_sync(0xffffffffu, mx, o); if (lane >= o) mx = fmax(mx, up); }
                mx = fmax(mx, run_a);
                if (j < Lc) {
                    a_s[j] = a;
                    g_s[j] = fmax(m_prev, mx);
                    wdec[j] = expf((float)(m_prev - fmax(m_prev, mx)));
                }
                run_f = __shfl_sync(0xffffffffu, F, 31);
                run_a = __shfl_sync(0xffffffffu, mx, 31);
                if (base + 32 >= Lc && lane == ((Lc - 1) & 31)) m_carry = F + fmax(m_prev, mx);     // m after the chunk's last token
            }
        }
        __syncthreads();
        // ---- weighted scores P[j][s] = exp(a_s - g_j) (q_j . k_s), s <= j; and the weights of the chunk's tokens in the new state
        for (int i = tid; i < Lc * Lc; i += CHUNK_THREADS) {
            const int j = i / Lc, ss = i - j * Lc;
            float p = 0.f;
            if (ss <= j) {
                const float* qj = Q + j * (D + 1);
                float acc = 0.f;
                for (int d = 0; d < D; ++d) acc = fmaf(qj[d], Kt[d * L + ss], acc);
                p = acc * expf((float)(a_s[ss] - g_s[j]));
            }
            P[j * L + ss] = p;
        }
        for (int j = tid; j < Lc; j += CHUNK_THREADS) wend[j] = expf((float)(a_s[j] - g_s[Lc - 1]));
        __syncthreads();
        // ---- n_j . q_j, a warp per row
        for (int j = warp; j < Lc; j += CHUNK_THREADS / 32) {
            float acc = 0.f;
            for (int ss = lane; ss <= j; ss += 32) acc += P[j * L + ss];
            float old = 0.f;
            for (int d = lane; d < D; d += 32) old = fmaf(nv[d], Q[j * (D + 1) + d], old);
            acc = vm_warp_sum(fmaf(wdec[j], old, acc));
            if (lane == 0) nq[j] = acc;
        }
        __syncthreads();
        // ---- o_j[v] = (exp(m' - g_j) S'^T q_j + sum_s P[j][s] v_s) / (max(|n_j . q_j|, exp(-m_j)) + 1e-6)
        for (int i = tid; i < Lc * vs; i += CHUNK_THREADS) {
            const int j = i / vs, v = i - j * vs;
            const float* qj = Q + j * (D + 1);
            float old = 0.f;
            for (int d = 0; d < D; ++d) old = fmaf(qj[d], S[d * VS + v], old);
            float acc = 0.f;
            for (int ss = 0; ss <= j; ++ss) acc = fmaf(P[j * L + ss], Vs[ss * VS + v], acc);
            const float num = fmaf(wdec[j], old, acc);
            // m_j = F_j + g_j and F_j = i_j - a_j are not kept; exp(-m_j) from the float64 pieces
            const float* row = proj + (size_t)(c0 + j) * ld;
            const double m_j = ((double)soft_cap(row[off_i + h] + bi, cap) - a_s[j]) + g_s[j];
            const float den = fmaxf(fabsf(nq[j]), expf((float)(-m_j))) + 1e-6f;
            o_raw[(size_t)(c0 + j) * H * V + h * V + v0 + v] = num / den;
        }
        __syncthreads();
        // ---- the state after the chunk
        const float keep = wdec[Lc - 1];
        for (int i = tid; i < D * vs; i += CHUNK_THREADS) {
            const int d = i / vs, v = i - d * vs;
            float acc = keep * S[d * VS + v];
            const float* kd = Kt + d * L;
            for (int ss = 0; ss < Lc; ++ss) acc = fmaf(wend[ss] * kd[ss], Vs[ss * VS + v], acc);
            S[d * VS + v] = acc;
        }
        for (int d = tid; d < D; d += CHUNK_THREADS) {
            float acc = keep * nv[d];
            const float* kd = Kt + d * L;
            for (int ss = 0; ss < Lc; ++ss) acc = fmaf(wend[ss], kd[ss], acc);
            nv[d] = acc;
        }
        __syncthreads();
    }
    for (int i = tid; i < D * vs; i += CHUNK_THREADS) { const int d = i / vs, v = i - d * vs; st[(size_t)d * V + v0 + v] = S[d * VS + v]; }
    if (slice == 0) {
        float* e = end_nm + ((size_t)s * H + h) * (D + 1);
        for (int d = tid; d < D; d += CHUNK_THREADS) e[d] = nv[d];
        if (tid == 0) e[D] = (float)m_carry;
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

ChunkSizes chunk_sizes(int D, int V) {
    ChunkSizes c;
    c.VS = V <= 64 ? V : 64;
    c.slices = (V + c.VS - 1) / c.VS;
    c.L = 64;
    while (c.L > 8 && chunk_smem_floats(c.L, D, c.VS) * sizeof(float) + 64 > 200 * 1024) c.L /= 2;
    c.smem = chunk_smem_floats(c.L, D, c.VS) * sizeof(float) + 64;
    return c;
}

}  // namespace

// scratch floats the chunkwise form needs: the un-normalised o [T, H*V] and a row of n, m per (sequence, head)
VM_API long long vm_mlstm_chunk_scratch_floats(int T, int B, int H, int D, int V) { return (long long)T * H * V + (long long)B * H * (D + 1); }

VM_API int vm_mlstm_chunks(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                           const int* slots, void* out, float* scratch, int T, int B, int H, int D, int V, float cap, float eps, int act_dtype,
                           cudaStream_t stream) {
    if (B <= 0 || T <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + 2 * H * V + 2 * H || !(cap > 0.f)) return VM_ERR_BAD_ARG;
    const ChunkSizes c = chunk_sizes(D, V);
    if (c.smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    static size_t raised = 0;
    if (c.smem > 48 * 1024 && c.smem > raised) {
        if (cudaFuncSetAttribute(mlstm_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess) return vm_launch_status();
        raised = c.smem;
    }
    float* o_raw = scratch;
    float* end_nm = scratch + (size_t)T * H * V;
    mlstm_chunk_kernel<<<dim3(c.slices, H, B), CHUNK_THREADS, c.smem, stream>>>(proj, ld, bias_i, bias_f, state, cu_tokens, slots, o_raw, end_nm, H, D, V,
                                                                                  c.L, c.VS, cap);
    int st = vm_launch_status();
    if (st) return st;
    const long long warps = (long long)T * H > (long long)B * H ? (long long)T * H : (long long)B * H;
    const int blocks = (int)((warps + 7) / 8);
    if (act_dtype == VM_F32)
        mlstm_output_kernel<float><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (float*)out, T, H, D, V, eps, end_nm, state, cu_tokens, slots, B);
    else if (act_dtype == VM_BF16)
        mlstm_output_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(o_raw, proj, ld, norm_w, (__nv_bfloat16*)out, T, H, D, V, eps, end_nm, state,
                                                                       cu_tokens, slots, B);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
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
