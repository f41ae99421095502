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

}  // namespace

VM_API int vm_mlstm_scan(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state, const int* cu_tokens,
                         const int* slots, void* out, int B, int H, int D, int V, float cap, float eps, int act_dtype, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + 2 * H * V + 2 * H || !(cap > 0.f)) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_F32) return launch_scan<float>(proj, ld, bias_i, bias_f, norm_w, state, cu_tokens, slots, out, B, H, D, V, cap, eps, stream);
    if (act_dtype == VM_BF16)
        return launch_scan<__nv_bfloat16>(proj, ld, bias_i, bias_f, norm_w, state, cu_tokens, slots, out, B, H, D, V, cap, eps, stream);
    return VM_ERR_UNSUPPORTED;
}
