// A selective state-space mixer in the manner of Mamba-2: a short causal convolution per channel, the recurrence of a
// matrix state per head, and the gated, group-normed output stage.
//
//   u_t [C]   the convolution's input (C = H * P + 2 * G * N channels: x | B | C), c_t = silu(bias + sum_k taps[:, k] u_(t - K + 1 + k))
//   dt_t,h  = softplus(dt_raw + dt_bias_h)                      a_t,h = exp(-exp(A_log_h) dt_t,h)
//   S_t,h   = a_t,h S_(t-1),h + dt_t,h B_t,g x_t,h^T            S is N x P, g = h / (H / G)
//   y_t,h   = S_t,h^T C_t,g + D_h x_t,h
//   out_t   = unit-rms over each of `parts` equal parts of (y_t * silu(z_t)), times w
//
// What a sequence keeps (float32, in its slot's state area): S [H, N, P], then the last K - 1 convolution inputs [K - 1, C].
// The state is zero when a slot is opened, which is also what "zeros before the start" asks of the convolution.
// Step sizes, decays, the state and the sums over it are float32 whatever the activation dtype.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------ convolution
// A thread per (token, channel).  u: columns [u_col, u_col + C) of proj [T, ld].
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ proj, int ld, int u_col, const float* __restrict__ taps, const float* __restrict__ bias,
                                 const float* __restrict__ state, int state_floats, int conv_off, const int* __restrict__ positions,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int n_tokens,
                                 int C, int K, T* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * C) return;
    const int t = (int)(i / C), c = (int)(i - (long long)t * C);
    const int seq = seq_of_token[t];
    const int local = t - cu_tokens[seq];                  // place of the token among its sequence's new tokens
    const float* kept = state + (size_t)slots[seq] * state_floats + conv_off;      // [K - 1, C]: inputs of the K - 1 tokens before this step
    float acc = bias ? bias[c] : 0.f;
    for (int k = 0; k < K; ++k) {
        const int back = K - 1 - k;                        // tap k reads the input `back` tokens ago
        float u;
        if (local - back >= 0) u = vm_to_float(proj[(size_t)(t - back) * ld + u_col + c]);
        else u = kept[(size_t)(K - 1 + local - back) * C + c];
        acc = fmaf(taps[(size_t)c * K + k], u, acc);
    }
    out[(size_t)t * C + c] = vm_from_float<T>(silu_f(acc));
}

// A block per sequence, a thread per channel: the last K - 1 inputs after this step (older ones move up, new ones come in).
template <typename T>
__global__ void conv_keep_kernel(const T* __restrict__ proj, int ld, int u_col, float* __restrict__ state, int state_floats, int conv_off,
                                 const int* __restrict__ cu_tokens, const int* __restrict__ slots, int C, int K) {
    const int seq = blockIdx.x;
    const int t0 = cu_tokens[seq], n = cu_tokens[seq + 1] - t0;
    if (n <= 0) return;
    float* kept = state + (size_t)slots[seq] * state_floats + conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        // new row j holds the input at local place n - (K - 1) + j; a negative place is old row j + n
        for (int j = 0; j < K - 1; ++j) {                  // ascending j reads only rows >= j: nothing it still needs is overwritten
            const int local = n - (K - 1) + j;
            kept[(size_t)j * C + c] = local >= 0 ? vm_to_float(proj[(size_t)(t0 + local) * ld + u_col + c]) : kept[(size_t)(j + n) * C + c];
        }
    }
}

// ------------------------------------------------------------------------------------------------ recurrence
// A block per (sequence, head, slice of P).  Thread (p, s) keeps S[n, p] for the n of its slice s (NPT values in registers) through all
// the sequence's new tokens; tokens are taken TOK at a time: their B, C, x and step sizes are staged in shared memory, every thread
// runs the TOK updates without a barrier, and the slices' partial sums of y are added up afterwards.
constexpr int SCAN_TOK = 8;

template <typename T, int NPT>
__global__ void ssm_scan_kernel(const T* __restrict__ xbc, int C, const T* __restrict__ proj, int ld, int dt_col, const float* __restrict__ dt_bias,
                                const float* __restrict__ A_log, const float* __restrict__ Dskip, float* __restrict__ state, int state_floats,
                                const int* __restrict__ cu_tokens, const int* __restrict__ slots, float* __restrict__ y, int H, int P, int N, int G,
                                int PB) {
    extern __shared__ float sm[];
    const int seq = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PB;
    const int g = h / (H / G);
    const int n_slices = (N + NPT - 1) / NPT;
    const int p_local = threadIdx.x % PB, slice = threadIdx.x / PB;
    const int p = p0 + p_local;
    const bool live = p < P && slice < n_slices;
    float* sB = sm;                                        // [TOK, N]
    float* sC = sB + SCAN_TOK * N;                         // [TOK, N]
    float* sx = sC + SCAN_TOK * N;                         // [TOK, PB]
    float* sdt = sx + SCAN_TOK * PB;                       // [TOK] step sizes, [TOK] decays
    float* sy = sdt + 2 * SCAN_TOK;                        // [TOK, n_slices, PB]
    const int t0 = cu_tokens[seq], n_new = cu_tokens[seq + 1] - t0;
    if (n_new <= 0) return;
    float* S = state + (size_t)slots[seq] * state_floats + (size_t)h * N * P;
    float s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = slice * NPT + i;
        s[i] = (live && n < N) ? S[(size_t)n * P + p] : 0.f;
    }
    const float rate = -expf(A_log[h]), skip = Dskip ? Dskip[h] : 0.f, bias = dt_bias ? dt_bias[h] : 0.f;
    const int inner = H * P;
    for (int base = 0; base < n_new; base += SCAN_TOK) {
        const int cnt = min(SCAN_TOK, n_new - base);
        __syncthreads();                                   // the previous round's sums are read
        for (int i = threadIdx.x; i < cnt * N; i += blockDim.x) {
            const int k = i / N, n = i - k * N;
            const T* row = xbc + (size_t)(t0 + base + k) * C;
            sB[k * N + n] = vm_to_float(row[inner + g * N + n]);
            sC[k * N + n] = vm_to_float(row[inner + G * N + g * N + n]);
        }
        for (int i = threadIdx.x; i < cnt * PB; i += blockDim.x) {
            const int k = i / PB, pp = i - k * PB;
            sx[k * PB + pp] = p0 + pp < P ? vm_to_float(xbc[(size_t)(t0 + base + k) * C + h * P + p0 + pp]) : 0.f;
        }
        if (threadIdx.x < cnt) {
            const float dt = softplus_f(vm_to_float(proj[(size_t)(t0 + base + threadIdx.x) * ld + dt_col + h]) + bias);
            sdt[threadIdx.x] = dt;
            sdt[SCAN_TOK + threadIdx.x] = expf(rate * dt);
        }
        __syncthreads();
        if (live) {
            for (int k = 0; k < cnt; ++k) {
                const float dt = sdt[k], a = sdt[SCAN_TOK + k];
                const float dx = dt * sx[k * PB + p_local];
                const float* Bk = sB + k * N + slice * NPT;
                const float* Ck = sC + k * N + slice * NPT;
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < NPT; ++i) {
                    if (slice * NPT + i < N) {
                        s[i] = fmaf(a, s[i], dx * Bk[i]);
                        part = fmaf(s[i], Ck[i], part);
                    }
                }
                sy[(k * n_slices + slice) * PB + p_local] = part;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cnt * PB; i += blockDim.x) {
            const int k = i / PB, pp = i - k * PB;
            if (p0 + pp >= P) continue;
            float sum = 0.f;
            for (int sl = 0; sl < n_slices; ++sl) sum += sy[(k * n_slices + sl) * PB + pp];       // slices in order: the same sum for every cut
            y[(size_t)(t0 + base + k) * inner + h * P + p0 + pp] = fmaf(skip, sx[k * PB + pp], sum);
        }
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = slice * NPT + i;
        if (live && n < N) S[(size_t)n * P + p] = s[i];
    }
}

// ------------------------------------------------------------------------------------------------ output stage
// A block per token: (y * silu(z)) normed over each of `parts` equal parts, times w.  y float32 [T, inner]; z: columns [z_col, z_col + inner) of proj.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col, const float* __restrict__ w, float eps,
                                        int inner, int parts, T* __restrict__ out) {
    extern __shared__ float gs[];                          // [inner]
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int per = inner / parts;
    for (int i = threadIdx.x; i < inner; i += blockDim.x) gs[i] = y[(size_t)t * inner + i] * silu_f(vm_to_float(proj[(size_t)t * ld + z_col + i]));
    __syncthreads();
    for (int part = 0; part < parts; ++part) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < per; i += blockDim.x) { const float v = gs[part * per + i]; ss += v * v; }
        ss = vm_block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)per + eps);
        for (int i = threadIdx.x; i < per; i += blockDim.x) {
            const int c = part * per + i;
            out[(size_t)t * inner + c] = vm_from_float<T>(gs[c] * inv * w[c]);
        }
    }
}

template <typename T>
int launch_scan(const void* xbc, int C, const void* proj, int ld, int dt_col, const float* dt_bias, const float* A_log, const float* Dskip, float* state,
                int state_floats, const int* cu_tokens, const int* slots, float* y, int B, int H, int P, int N, int G, int sm_count, cudaStream_t stream) {
    // registers per thread for the state: 16 values while the block stays within 1,024 threads, more for the largest heads
    int npt = 16;
    while (npt < 64 && (long long)((N + npt - 1) / npt) * min(P, 64) > 1024) npt *= 2;
    // columns of P per block: all of them, or fewer when the step has too few (sequence, head) pairs to fill the GPU
    int PB = P;
    while (PB > 8 && PB % 2 == 0 && (long long)B * H * (P / PB) < 2ll * sm_count) PB /= 2;
    int n_slices = (N + npt - 1) / npt;
    while ((long long)n_slices * PB > 1024 && PB % 2 == 0) PB /= 2;
    if ((long long)n_slices * PB > 1024) return VM_ERR_UNSUPPORTED;
    int threads = n_slices * PB;
    threads = (threads + 31) / 32 * 32;
    const size_t smem = ((size_t)2 * SCAN_TOK * N + (size_t)SCAN_TOK * PB + 2 * SCAN_TOK + (size_t)SCAN_TOK * n_slices * PB) * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    const dim3 grid(B, H, (P + PB - 1) / PB);
#define VM_SCAN(NPT)                                                                                                                             \
    ssm_scan_kernel<T, NPT><<<grid, threads, smem, stream>>>((const T*)xbc, C, (const T*)proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, \
                                                             cu_tokens, slots, y, H, P, N, G, PB)
    if (npt == 16) VM_SCAN(16);
    else if (npt == 32) VM_SCAN(32);
    else VM_SCAN(64);
#undef VM_SCAN
    return vm_launch_status();
}

}  // namespace

VM_API long long vm_ssm_state_floats(int H, int P, int N, int G, int K) { return (long long)H * N * P + (long long)(K - 1) * ((long long)H * P + 2ll * G * N); }

// proj [T, ld] in the activation dtype holds z | x | B | C | dt_raw side by side (H * P, H * P, G * N, G * N, H columns, from z_col on);
// taps float32 [C, K] with the current token's tap last, conv_bias float32 [C] (or null); dt_bias, A_log, Dskip float32 [H]; norm_w float32
// [H * P].  Scratch: xbc [T, C] in the activation dtype, y float32 [T, H * P].  out [T, H * P] in the activation dtype.
// state float32 [slots, state_floats] with state_floats >= vm_ssm_state_floats(...).
VM_API int vm_ssm_mixer(const void* proj, int ld, const float* taps, const float* conv_bias, const float* dt_bias, const float* A_log, const float* Dskip,
                        const float* norm_w, float eps, float* state, int state_floats, const int* positions, const int* seq_of_token,
                        const int* cu_tokens, const int* slots, void* xbc, float* y, void* out, int T, int B, int H, int P, int N, int G, int K,
                        int parts, int act_dtype, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || K < 1 || K > 64 || parts <= 0 || (H * P) % parts) return VM_ERR_BAD_ARG;
    if (state_floats < vm_ssm_state_floats(H, P, N, G, K)) return VM_ERR_BAD_ARG;
    const int inner = H * P, C = inner + 2 * G * N;
    if (ld < 2 * inner + 2 * G * N + H) return VM_ERR_BAD_ARG;
    const int u_col = inner, dt_col = 2 * inner + 2 * G * N, conv_off = H * N * P;
    if ((size_t)inner * sizeof(float) > 48 * 1024) return VM_ERR_UNSUPPORTED;
    const long long n = (long long)T * C;
    const int conv_blocks = (int)((n + 255) / 256);
    int st;
    if (act_dtype == VM_F32) {
        using Tt = float;
        conv_silu_kernel<Tt><<<conv_blocks, 256, 0, stream>>>((const Tt*)proj, ld, u_col, taps, conv_bias, state, state_floats, conv_off, positions,
                                                              seq_of_token, cu_tokens, slots, T, C, K, (Tt*)xbc);
        if (K > 1) conv_keep_kernel<Tt><<<B, 256, 0, stream>>>((const Tt*)proj, ld, u_col, state, state_floats, conv_off, cu_tokens, slots, C, K);
        st = launch_scan<Tt>(xbc, C, proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, cu_tokens, slots, y, B, H, P, N, G, vm_sm_count(), stream);
        if (st) return st;
        gated_group_norm_kernel<Tt><<<T, 256, (size_t)inner * sizeof(float), stream>>>(y, (const Tt*)proj, ld, 0, norm_w, eps, inner, parts, (Tt*)out);
    } else if (act_dtype == VM_BF16) {
        using Tt = __nv_bfloat16;
        conv_silu_kernel<Tt><<<conv_blocks, 256, 0, stream>>>((const Tt*)proj, ld, u_col, taps, conv_bias, state, state_floats, conv_off, positions,
                                                              seq_of_token, cu_tokens, slots, T, C, K, (Tt*)xbc);
        if (K > 1) conv_keep_kernel<Tt><<<B, 256, 0, stream>>>((const Tt*)proj, ld, u_col, state, state_floats, conv_off, cu_tokens, slots, C, K);
        st = launch_scan<Tt>(xbc, C, proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, cu_tokens, slots, y, B, H, P, N, G, vm_sm_count(), stream);
        if (st) return st;
        gated_group_norm_kernel<Tt><<<T, 256, (size_t)inner * sizeof(float), stream>>>(y, (const Tt*)proj, ld, 0, norm_w, eps, inner, parts, (Tt*)out);
    } else {
        return VM_ERR_UNSUPPORTED;
    }
    return vm_launch_status();
}
