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
// grid (channel tiles, tokens): a thread per (token, channel).  u: columns [u_col, u_col + C) of proj [T, ld].
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ proj, int ld, int u_col, const float* __restrict__ taps, const float* __restrict__ bias,
                                 const float* __restrict__ state, int state_floats, int conv_off, const int* __restrict__ positions,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int n_tokens,
                                 int C, int K, T* __restrict__ out) {
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
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
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        // new row j holds the input at local place n - (K - 1) + j; a negative place is old row j + n
        for (int j = 0; j < K - 1; ++j) {                  // ascending j reads only rows >= j: nothing it still needs is overwritten
            const int local = n - (K - 1) + j;
            kept[(size_t)j * C + c] = local >= 0 ? vm_to_float(proj[(size_t)(t0 + local) * ld + u_col + c]) : kept[(size_t)(j + n) * C + c];
        }
    }
}


// One new token per sequence (token s belongs to sequence s): the convolution and its memory in one pass; a thread per (sequence, channel).
template <typename T>
__global__ void conv_step_kernel(const T* __restrict__ proj, int ld, int u_col, const float* __restrict__ taps, const float* __restrict__ bias,
                                 float* __restrict__ state, int state_floats, int conv_off, const int* __restrict__ slots, int B, int C, int K,
                                 T* __restrict__ out) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * C) return;
    const int seq = (int)(i / C), c = (int)(i - (long long)seq * C);
    float* kept = state + (size_t)slots[seq] * state_floats + conv_off;
    const float u = vm_to_float(proj[(size_t)seq * ld + u_col + c]);
    float acc = fmaf(taps[(size_t)c * K + K - 1], u, bias ? bias[c] : 0.f);
    for (int j = 0; j < K - 1; ++j) {
        const float v = kept[(size_t)j * C + c];
        acc = fmaf(taps[(size_t)c * K + j], v, acc);
        if (j > 0) kept[(size_t)(j - 1) * C + c] = v;      // the memory moves up by one token
    }
    if (K > 1) kept[(size_t)(K - 2) * C + c] = u;
    out[(size_t)seq * C + c] = vm_from_float<T>(silu_f(acc));
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
    vm_pdl_launch_dependents();
    vm_pdl_wait();
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


// ------------------------------------------------------------------------------------------------ recurrence, chunk by chunk (prompts)
// Inside a chunk of CL tokens the recurrence has a closed form.  With c_t the running sum of the log decays (rate * dt) inside the chunk:
//   y_t = sum_{s <= t} exp(c_t - c_s) dt_s (C_t . B_s) x_s  +  exp(c_t) C_t^T S_start  +  D x_t
//   S_end = exp(c_last) S_start + sum_s exp(c_last - c_s) dt_s B_s x_s^T
// Pass 1 (all chunks of all sequences and heads at once): the first sum and the second line's sum (dS).  Pass 2 (elementwise over the
// state, chunk after chunk): S_start of every chunk, left where dS was, and the sequence's new state.  Pass 3 (all chunks at once): the
// old state's share and the skip term.  All products are float32 register tiles fed from shared memory: thread (ty, tx) of 16 x 16 owns
// rows 4 ty .. 4 ty + 3 and columns tx, tx + 16, ...; every exponent is <= 0.
constexpr int CL = 64;       // tokens per chunk
constexpr int NT = 64;       // state values per tile
constexpr int LDT = 65;      // padded row of a 64-wide tile

__device__ __forceinline__ bool chunk_where(const int* __restrict__ cu_tokens, int B, int chunk, int& seq, int& t0, int& len) {
    for (seq = 0; seq < B; ++seq) {
        const int a = cu_tokens[seq], b = cu_tokens[seq + 1];
        const int nc = (b - a + CL - 1) / CL;
        if (chunk < nc) { t0 = a + chunk * CL; len = min(CL, b - t0); return true; }
        chunk -= nc;
    }
    return false;
}

// scratch layout (floats): dS / S_start [n_chunks, H, N, P], then cum [T, H], then decay [n_chunks, H]
template <typename T, int PC>
__global__ void __launch_bounds__(256)
ssm_chunk_local_kernel(const T* __restrict__ xbc, int C, const T* __restrict__ proj, int ld, int dt_col, const float* __restrict__ dt_bias,
                       const float* __restrict__ A_log, const int* __restrict__ cu_tokens, int B, float* __restrict__ y, float* __restrict__ dS,
                       float* __restrict__ cum_out, float* __restrict__ decay_out, int H, int P, int N, int G) {
    constexpr int XP = PC * 16;
    extern __shared__ float sm[];
    float* sC = sm;                       // [CL][LDT]
    float* sB = sC + CL * LDT;            // [CL][LDT]
    float* sG = sB + CL * LDT;            // [CL][LDT]
    float* sX = sG + CL * LDT;            // [CL][XP]
    float* sXw = sX + CL * XP;            // [CL][XP]
    float* scum = sXw + CL * XP;          // [CL]
    float* sdt = scum + CL;               // [CL]
    int seq, t0, len;
    if (!chunk_where(cu_tokens, B, blockIdx.x, seq, t0, len)) return;
    const int h = blockIdx.y, g = h / (H / G), tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int inner = H * P;
    const float rate = -expf(A_log[h]), bias = dt_bias ? dt_bias[h] : 0.f;
    if (tid < CL) {
        const float dt = tid < len ? softplus_f(vm_to_float(proj[(size_t)(t0 + tid) * ld + dt_col + h]) + bias) : 0.f;
        sdt[tid] = dt;
        scum[tid] = rate * dt;
    }
    __syncthreads();
    if (tid == 0) {
        float c = 0.f;
        for (int i = 0; i < CL; ++i) { c += scum[i]; scum[i] = c; }
    }
    __syncthreads();
    const float c_last = scum[CL - 1];
    for (int i = tid; i < CL * XP; i += 256) {
        const int s_ = i / XP, p = i - s_ * XP;
        const float x = (s_ < len && p < P) ? vm_to_float(xbc[(size_t)(t0 + s_) * C + h * P + p]) : 0.f;
        sX[i] = x;
        sXw[i] = x * sdt[s_] * expf(c_last - scum[s_]);
    }
    if (tid < CL && tid < len) cum_out[(size_t)(t0 + tid) * H + h] = scum[tid];
    if (tid == 0) decay_out[(size_t)blockIdx.x * H + h] = expf(c_last);
    float gacc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) gacc[i][j] = 0.f;
    float* dS_out = dS + ((size_t)blockIdx.x * H + h) * N * P;
    for (int n0 = 0; n0 < N; n0 += NT) {
        __syncthreads();                  // the previous tile is read
        for (int i = tid; i < CL * NT; i += 256) {
            const int s_ = i / NT, k = i - s_ * NT;
            const bool in = s_ < len && n0 + k < N;
            const T* row = xbc + (size_t)(t0 + (in ? s_ : 0)) * C + inner + g * N + n0 + (in ? k : 0);
            sB[s_ * LDT + k] = in ? vm_to_float(row[0]) : 0.f;
            sC[s_ * LDT + k] = in ? vm_to_float(row[(size_t)G * N]) : 0.f;
        }
        __syncthreads();
        // scores of the chunk: G[t, s] += sum_k C[t, k] B[s, k]
#pragma unroll 4
        for (int k = 0; k < NT; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sC[(ty * 4 + i) * LDT + k];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sB[(tx + 16 * j) * LDT + k];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) gacc[i][j] = fmaf(a[i], b[j], gacc[i][j]);
        }
        // the chunk's contribution to the state: dS[n, p] = sum_s B[s, n] (w_s x_s)[p]
        float dacc[4][PC];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < PC; ++j) dacc[i][j] = 0.f;
#pragma unroll 2
        for (int s_ = 0; s_ < CL; ++s_) {
            float a[4], b[PC];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sB[s_ * LDT + ty * 4 + i];
#pragma unroll
            for (int j = 0; j < PC; ++j) b[j] = sXw[s_ * XP + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < PC; ++j) dacc[i][j] = fmaf(a[i], b[j], dacc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + ty * 4 + i;
            if (n >= N) continue;
#pragma unroll
            for (int j = 0; j < PC; ++j) {
                const int p = tx + 16 * j;
                if (p < P) dS_out[(size_t)n * P + p] = dacc[i][j];
            }
        }
    }
    // decays, step sizes and the causal mask on the scores
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = ty * 4 + i, s_ = tx + 16 * j;
            sG[t * LDT + s_] = (s_ <= t && t < len) ? gacc[i][j] * expf(scum[t] - scum[s_]) * sdt[s_] : 0.f;
        }
    __syncthreads();
    float yacc[4][PC];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < PC; ++j) yacc[i][j] = 0.f;
#pragma unroll 2
    for (int s_ = 0; s_ < CL; ++s_) {
        float a[4], b[PC];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = sG[(ty * 4 + i) * LDT + s_];
#pragma unroll
        for (int j = 0; j < PC; ++j) b[j] = sX[s_ * XP + tx + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < PC; ++j) yacc[i][j] = fmaf(a[i], b[j], yacc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = ty * 4 + i;
        if (t >= len) continue;
#pragma unroll
        for (int j = 0; j < PC; ++j) {
            const int p = tx + 16 * j;
            if (p < P) y[(size_t)(t0 + t) * inner + h * P + p] = yacc[i][j];
        }
    }
}

// grid (B * H, ceil(N * P / 256)): a thread carries one value of the state through its sequence's chunks
__global__ void ssm_chunk_carry_kernel(float* __restrict__ dS, const float* __restrict__ decay, float* __restrict__ state, int state_floats,
                                       const int* __restrict__ cu_tokens, const int* __restrict__ slots, int B, int H, int P, int N) {
    const int seq = blockIdx.x / H, h = blockIdx.x - seq * H;
    const int e = blockIdx.y * blockDim.x + threadIdx.x;
    if (e >= N * P) return;
    int first = 0;
    for (int b = 0; b < seq; ++b) first += (cu_tokens[b + 1] - cu_tokens[b] + CL - 1) / CL;
    const int nc = (cu_tokens[seq + 1] - cu_tokens[seq] + CL - 1) / CL;
    if (nc <= 0) return;
    float* S = state + (size_t)slots[seq] * state_floats + (size_t)h * N * P + e;
    float cur = *S;
    const size_t stride = (size_t)H * N * P;
    float* d0 = dS + ((size_t)first * H + h) * N * P + e;
    const float* dec = decay + (size_t)first * H + h;
    for (int c0 = 0; c0 < nc; c0 += 8) {
        // eight chunks' values are fetched before the first store (the compiler must not move a load over a store to the same array)
        float add[8], a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool in = c0 + k < nc;
            add[k] = in ? d0[(size_t)(c0 + k) * stride] : 0.f;
            a[k] = in ? dec[(size_t)(c0 + k) * H] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k >= nc) break;
            d0[(size_t)(c0 + k) * stride] = cur;          // the state at this chunk's start
            cur = fmaf(a[k], cur, add[k]);
        }
    }
    *S = cur;
}

template <typename T, int PC>
__global__ void __launch_bounds__(256)
ssm_chunk_finish_kernel(const T* __restrict__ xbc, int C, const float* __restrict__ Dskip, const int* __restrict__ cu_tokens, int B,
                        float* __restrict__ y, const float* __restrict__ S_start, const float* __restrict__ cum, int H, int P, int N, int G) {
    constexpr int XP = PC * 16;
    extern __shared__ float sm[];
    float* sC = sm;                       // [CL][LDT]
    float* sS = sC + CL * LDT;            // [NT][XP]
    int seq, t0, len;
    if (!chunk_where(cu_tokens, B, blockIdx.x, seq, t0, len)) return;
    const int h = blockIdx.y, g = h / (H / G), tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int inner = H * P;
    const float* S = S_start + ((size_t)blockIdx.x * H + h) * N * P;
    float acc[4][PC];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < PC; ++j) acc[i][j] = 0.f;
    for (int n0 = 0; n0 < N; n0 += NT) {
        __syncthreads();
        for (int i = tid; i < CL * NT; i += 256) {
            const int s_ = i / NT, k = i - s_ * NT;
            const bool in = s_ < len && n0 + k < N;
            sC[s_ * LDT + k] = in ? vm_to_float(xbc[(size_t)(t0 + s_) * C + inner + (size_t)G * N + g * N + n0 + k]) : 0.f;
        }
        for (int i = tid; i < NT * XP; i += 256) {
            const int k = i / XP, p = i - k * XP;
            sS[i] = (n0 + k < N && p < P) ? S[(size_t)(n0 + k) * P + p] : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int k = 0; k < NT; ++k) {
            float a[4], b[PC];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sC[(ty * 4 + i) * LDT + k];
#pragma unroll
            for (int j = 0; j < PC; ++j) b[j] = sS[k * XP + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < PC; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
    const float skip = Dskip ? Dskip[h] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = ty * 4 + i;
        if (t >= len) continue;
        const float w = expf(cum[(size_t)(t0 + t) * H + h]);
#pragma unroll
        for (int j = 0; j < PC; ++j) {
            const int p = tx + 16 * j;
            if (p >= P) continue;
            const size_t at = (size_t)(t0 + t) * inner + h * P + p;
            y[at] = y[at] + w * acc[i][j] + skip * vm_to_float(xbc[(size_t)(t0 + t) * C + h * P + p]);
        }
    }
}

template <typename T, int PC>
int launch_chunks_pc(const void* xbc, int C, const void* proj, int ld, int dt_col, const float* dt_bias, const float* A_log, const float* Dskip,
                     float* state, int state_floats, const int* cu_tokens, const int* slots, float* y, float* scratch, int T_, int B, int n_chunks,
                     int H, int P, int N, int G, cudaStream_t stream) {
    constexpr int XP = PC * 16;
    float* dS = scratch;
    float* cum = dS + (size_t)n_chunks * H * N * P;
    float* decay = cum + (size_t)T_ * H;
    const size_t smem1 = ((size_t)3 * CL * LDT + (size_t)2 * CL * XP + 2 * CL) * sizeof(float);
    const size_t smem3 = ((size_t)CL * LDT + (size_t)NT * XP) * sizeof(float);
    static bool raised = false;           // per instantiation
    if (!raised) {
        if (cudaFuncSetAttribute(ssm_chunk_local_kernel<T, PC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1) != cudaSuccess) return vm_launch_status();
        if (cudaFuncSetAttribute(ssm_chunk_finish_kernel<T, PC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3) != cudaSuccess) return vm_launch_status();
        raised = true;
    }
    ssm_chunk_local_kernel<T, PC><<<dim3(n_chunks, H), 256, smem1, stream>>>((const T*)xbc, C, (const T*)proj, ld, dt_col, dt_bias, A_log, cu_tokens, B, y,
                                                                            dS, cum, decay, H, P, N, G);
    int st = vm_launch_status();
    if (st) return st;
    ssm_chunk_carry_kernel<<<dim3(B * H, (N * P + 255) / 256), 256, 0, stream>>>(dS, decay, state, state_floats, cu_tokens, slots, B, H, P, N);
    st = vm_launch_status();
    if (st) return st;
    ssm_chunk_finish_kernel<T, PC><<<dim3(n_chunks, H), 256, smem3, stream>>>((const T*)xbc, C, Dskip, cu_tokens, B, y, dS, cum, H, P, N, G);
    return vm_launch_status();
}

template <typename T>
int launch_chunks(const void* xbc, int C, const void* proj, int ld, int dt_col, const float* dt_bias, const float* A_log, const float* Dskip, float* state,
                  int state_floats, const int* cu_tokens, const int* slots, float* y, float* scratch, int T_, int B, int n_chunks, int H, int P, int N,
                  int G, cudaStream_t stream) {
#define VM_CH(PC)                                                                                                                                  \
    return launch_chunks_pc<T, PC>(xbc, C, proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, cu_tokens, slots, y, scratch, T_, B, n_chunks, H, \
                                   P, N, G, stream)
    if (P <= 32) VM_CH(2);
    if (P <= 64) VM_CH(4);
    if (P <= 128) VM_CH(8);
#undef VM_CH
    return VM_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------------ output stage
// A block per token: (y * silu(z)) normed over each of `parts` equal parts, times w.  y float32 [T, inner]; z: columns [z_col, z_col + inner) of proj.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col, const float* __restrict__ w, float eps,
                                        int inner, int parts, T* __restrict__ out) {
    extern __shared__ float gs[];                          // [inner]
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
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
    vm_launch_pdl(ssm_scan_kernel<T, NPT>, grid, dim3(threads), smem, stream, (const T*)xbc, C, (const T*)proj, ld, dt_col, dt_bias, A_log, Dskip, state, \
                  state_floats, cu_tokens, slots, y, H, P, N, G, PB)
    if (npt == 16) VM_SCAN(16);
    else if (npt == 32) VM_SCAN(32);
    else VM_SCAN(64);
#undef VM_SCAN
    return vm_launch_status();
}

template <typename T>
int launch_mixer(const void* proj, int ld, const float* taps, const float* conv_bias, const float* dt_bias, const float* A_log, const float* Dskip,
                 const float* norm_w, float eps, float* state, int state_floats, const int* positions, const int* seq_of_token, const int* cu_tokens,
                 const int* slots, void* xbc, float* y, void* out, float* chunk_scratch, int n_chunks, int one_token_each, int T_, int B, int H, int P,
                 int N, int G, int K, int parts, cudaStream_t stream) {
    const int inner = H * P, C = inner + 2 * G * N;
    const int u_col = inner, dt_col = 2 * inner + 2 * G * N, conv_off = H * N * P;
    const long long n = (long long)T_ * C;
    const int conv_blocks = (int)((n + 255) / 256);
    int st;
    if (one_token_each) {
        vm_launch_pdl(conv_step_kernel<T>, dim3(conv_blocks), dim3(256), 0, stream, (const T*)proj, ld, u_col, taps, conv_bias, state, state_floats, conv_off,
                      slots, B, C, K, (T*)xbc);
    } else {
        if (T_ > 65535) return VM_ERR_UNSUPPORTED;
        conv_silu_kernel<T><<<dim3((C + 255) / 256, T_), 256, 0, stream>>>((const T*)proj, ld, u_col, taps, conv_bias, state, state_floats, conv_off,
                                                                           positions, seq_of_token, cu_tokens, slots, T_, C, K, (T*)xbc);
        if (K > 1)
            conv_keep_kernel<T><<<dim3(B, (C + 255) / 256), 256, 0, stream>>>((const T*)proj, ld, u_col, state, state_floats, conv_off, cu_tokens, slots, C, K);
    }
    st = vm_launch_status();
    if (st) return st;
    if (chunk_scratch && n_chunks > 0 && !one_token_each && P <= 128)
        st = launch_chunks<T>(xbc, C, proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, cu_tokens, slots, y, chunk_scratch, T_, B, n_chunks, H, P, N,
                              G, stream);
    else
        st = launch_scan<T>(xbc, C, proj, ld, dt_col, dt_bias, A_log, Dskip, state, state_floats, cu_tokens, slots, y, B, H, P, N, G, vm_sm_count(), stream);
    if (st) return st;
    vm_launch_pdl(gated_group_norm_kernel<T>, dim3(T_), dim3(256), (size_t)inner * sizeof(float), stream, (const float*)y, (const T*)proj, ld, 0, norm_w, eps,
                  inner, parts, (T*)out);
    return vm_launch_status();
}

}  // namespace

VM_API long long vm_ssm_state_floats(int H, int P, int N, int G, int K) { return (long long)H * N * P + (long long)(K - 1) * ((long long)H * P + 2ll * G * N); }

// floats of scratch the chunkwise recurrence needs for T tokens in n_chunks chunks of 64 (a sequence's last chunk may be shorter)
VM_API long long vm_ssm_chunk_scratch_floats(int T, int n_chunks, int H, int P, int N) {
    return (long long)n_chunks * H * N * P + (long long)T * H + (long long)n_chunks * H;
}

// proj [T, ld] in the activation dtype holds z | x | B | C | dt_raw side by side (H * P, H * P, G * N, G * N, H columns, from z_col on);
// taps float32 [C, K] with the current token's tap last, conv_bias float32 [C] (or null); dt_bias, A_log, Dskip float32 [H]; norm_w float32
// [H * P].  Scratch: xbc [T, C] in the activation dtype, y float32 [T, H * P].  out [T, H * P] in the activation dtype.
// state float32 [slots, state_floats] with state_floats >= vm_ssm_state_floats(...).
// chunk_scratch (vm_ssm_chunk_scratch_floats) with n_chunks = sum over the sequences of ceil(new tokens / 64): the recurrence runs chunk by
// chunk (values of up to 128 per head); null: token by token.  one_token_each: token s is sequence s's one new token.
VM_API int vm_ssm_mixer(const void* proj, int ld, const float* taps, const float* conv_bias, const float* dt_bias, const float* A_log, const float* Dskip,
                        const float* norm_w, float eps, float* state, int state_floats, const int* positions, const int* seq_of_token,
                        const int* cu_tokens, const int* slots, void* xbc, float* y, void* out, float* chunk_scratch, int n_chunks, int one_token_each,
                        int T, int B, int H, int P, int N, int G, int K, int parts, int act_dtype, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || K < 1 || K > 64 || parts <= 0 || (H * P) % parts) return VM_ERR_BAD_ARG;
    if (state_floats < vm_ssm_state_floats(H, P, N, G, K)) return VM_ERR_BAD_ARG;
    if (one_token_each && T != B) return VM_ERR_BAD_ARG;
    const int inner = H * P;
    if (ld < 2 * inner + 2 * G * N + H) return VM_ERR_BAD_ARG;
    if ((size_t)inner * sizeof(float) > 48 * 1024) return VM_ERR_UNSUPPORTED;
    if (act_dtype == VM_F32)
        return launch_mixer<float>(proj, ld, taps, conv_bias, dt_bias, A_log, Dskip, norm_w, eps, state, state_floats, positions, seq_of_token, cu_tokens,
                                   slots, xbc, y, out, chunk_scratch, n_chunks, one_token_each, T, B, H, P, N, G, K, parts, stream);
    if (act_dtype == VM_BF16)
        return launch_mixer<__nv_bfloat16>(proj, ld, taps, conv_bias, dt_bias, A_log, Dskip, norm_w, eps, state, state_floats, positions, seq_of_token,
                                           cu_tokens, slots, xbc, y, out, chunk_scratch, n_chunks, one_token_each, T, B, H, P, N, G, K, parts, stream);
    return VM_ERR_UNSUPPORTED;
}
