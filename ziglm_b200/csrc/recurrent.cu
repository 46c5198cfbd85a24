// A gated linear recurrence behind a short causal convolution, per channel:
//   u_t   = cb + sum_j taps[K-1-j] * x_{t-j}                 (j = 0 is the current token; zeros before the start;
//                                                              taps are kept one row per tap, [K, C])
//   a_t   = exp(-rate * r_t * softplus(lam)),   r_t, i_t: gates in (0, 1) computed from u_t by the caller
//   S_t   = a_t * S_{t-1} + sqrt(1 - a_t^2) * i_t * u_t      (S = 0 before the first token, no special case)
//   out_t = S_t * gelu_tanh(y_t)
// What a sequence carries from step to step is [K, C] floats per sequence: rows 0..K-2 hold the last K-1
// inputs x (oldest first), row K-1 holds S.  Decays, gates, the state and every product that enters the
// recurrence are float in both precisions; sqrt(1 - a^2) is taken as sqrt(-expm1(2 log a)), which stays exact
// when a is close to 1.
//
// The recurrence is a composition of affine maps S -> a S + b, which is associative: a block takes one
// sequence and 32 (or 16) channels, cuts the sequence's tokens of this step into as many chunks as it has rows of
// threads, every thread composes the maps of its chunk, the chunks' maps are folded in order to give each
// chunk its incoming state, and a second pass over the chunk writes the outputs.
#include "common.cuh"

namespace zlm {

constexpr int RC_CH = 32;        // channels a block takes
constexpr int RC_MAX_CHUNKS = 64;
constexpr int RC_MAX_THREADS = 1024;

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// u[t, c] for every token of the step; reads the inputs before the step from the sequence's state.
template <typename T>
__global__ void conv_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ taps,
                            const float* __restrict__ bias, const float* __restrict__ state, long state_stride,
                            const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ slots, T* __restrict__ u, int n_tokens, int C, int K, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * C) return;
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int b = seq_of_token[t];
    const int i = t - cu_seqlens[b];                  // index of the token among its sequence's tokens of this step
    const float* st = state + (long)slots[b] * state_stride;
    float acc = bias[c];
    for (int j = K - 1; j >= 0; --j) {                // oldest input first
        const float xv = (i - j >= 0) ? to_float(x[(long)(t - j) * x_stride + c])
                                      : st[(long)(K - 1 + i - j) * C + c];
        acc = fmaf(taps[(long)(K - 1 - j) * C + c], xv, acc);
    }
    if (act == 1) acc = silu_f(round_to<T>(acc));       // the convolution's sum is rounded as a result of its own
    u[idx] = from_float<T>(acc);
}

// The same for bf16 rows with C and the strides multiples of 8: a thread takes eight channels of a token and
// moves sixteen bytes at a time.
__global__ void conv_vec_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, const float* __restrict__ taps,
                                const float* __restrict__ bias, const float* __restrict__ state, long state_stride,
                                const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ slots, __nv_bfloat16* __restrict__ u, int n_tokens, int C, int K,
                                int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = C / 8;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * groups) return;
    const int t = (int)(idx / groups), c = (int)(idx % groups) * 8;
    const int b = seq_of_token[t];
    const int i = t - cu_seqlens[b];
    const float* st = state + (long)slots[b] * state_stride;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias[c + e];
    for (int j = K - 1; j >= 0; --j) {
        float xv[8];
        if (i - j >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (long)(t - j) * x_stride + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 v = __bfloat1622float2(h[e]);
                xv[2 * e] = v.x; xv[2 * e + 1] = v.y;
            }
        } else {
            const float* row = st + (long)(K - 1 + i - j) * C + c;
#pragma unroll
            for (int e = 0; e < 8; ++e) xv[e] = row[e];
        }
        const float4 w0 = *reinterpret_cast<const float4*>(taps + (long)(K - 1 - j) * C + c);
        const float4 w1 = *reinterpret_cast<const float4*>(taps + (long)(K - 1 - j) * C + c + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wv[e], xv[e], acc[e]);
    }
    if (act == 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = silu_f(round_to<__nv_bfloat16>(acc[e]));
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(u + (long)t * C + c) = o;
}

// grid (sequences, ceil(C / channels a block takes)), block (channels: 32 or 16, chunks)
template <typename T>
__global__ void __launch_bounds__(RC_MAX_THREADS)
scan_kernel(const T* __restrict__ u, const float* __restrict__ gates, int gate_block, const T* __restrict__ y,
            long y_stride, const T* __restrict__ x, long x_stride, const float* __restrict__ lam, float rate,
            float* __restrict__ state, long state_stride, const int* __restrict__ cu_seqlens,
            const int* __restrict__ slots, T* __restrict__ out, int C, int K) {
    __shared__ float agg_a[RC_MAX_CHUNKS][RC_CH], agg_b[RC_MAX_CHUNKS][RC_CH];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int chunk = threadIdx.y, n_chunks = blockDim.y;
    const int first = cu_seqlens[b], n_new = cu_seqlens[b + 1] - first;
    const int per = (n_new + n_chunks - 1) / n_chunks;
    const int lo = first + min(n_new, chunk * per), hi = first + min(n_new, (chunk + 1) * per);
    const bool live = c < C;
    float* st = state + (long)slots[b] * state_stride;
    float sp = 0.f;
    long g_r = 0;
    if (live) {
        sp = rate * softplus_f(lam[c]);
        g_r = (long)(c / gate_block) * 2 * gate_block + c % gate_block;     // its input gate lies gate_block further
    }
    const long g_stride = 2L * C;
    // pass 1: the chunk's map S -> A S + B
    float A = 1.f, B = 0.f;
    if (live) {
#pragma unroll 4
        for (int t = lo; t < hi; ++t) {
            const float r = gates[(long)t * g_stride + g_r], ig = gates[(long)t * g_stride + g_r + gate_block];
            const float uv = to_float(u[(long)t * C + c]);
            const float log_a = -sp * r;
            const float a = expf(log_a);
            const float bb = sqrtf(-expm1f(2.f * log_a)) * (ig * uv);
            A *= a;
            B = fmaf(a, B, bb);
        }
    }
    agg_a[chunk][threadIdx.x] = A;
    agg_b[chunk][threadIdx.x] = B;
    __syncthreads();
    if (!live) return;
    // the state that enters this chunk: the earlier chunks' maps applied in order to the carried state
    float S = st[(long)(K - 1) * C + c];
    for (int j = 0; j < chunk; ++j) S = fmaf(agg_a[j][threadIdx.x], S, agg_b[j][threadIdx.x]);
    // pass 2: the outputs
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
        const float r = gates[(long)t * g_stride + g_r], ig = gates[(long)t * g_stride + g_r + gate_block];
        const float uv = to_float(u[(long)t * C + c]);
        const float log_a = -sp * r;
        const float a = expf(log_a);
        S = fmaf(a, S, sqrtf(-expm1f(2.f * log_a)) * (ig * uv));
        out[(long)t * C + c] = from_float<T>(S * gelu_tanh_f(to_float(y[(long)t * y_stride + c])));
    }
    if (chunk != n_chunks - 1) return;
    // the last chunk leaves the state: S after the last token, and the last K-1 inputs (rows in ascending order:
    // row j takes what row j + n_new held, which is overwritten only later)
    st[(long)(K - 1) * C + c] = S;
    for (int j = 0; j < K - 1; ++j) {
        const int i = n_new - (K - 1) + j;           // index among the step's tokens, negative: an older input
        st[(long)j * C + c] = i >= 0 ? to_float(x[(long)(first + i) * x_stride + c]) : st[(long)(j + n_new) * C + c];
    }
}

// ------------------------------------------------------------------ selective scan
// Per channel c with N states (the recurrence of a selective state-space layer):
//   dt_t      = softplus(dtp[t, c])                                    (dtp: the step-size projection with its bias)
//   S_t[n]    = exp(dt_t A[c, n]) S_(t-1)[n] + dt_t u[t, c] B_t[n]     (A < 0; B_t, C_t: N numbers a token; the kernel is
//                                                                       given A log2(e) and takes exp2)
//   y_t       = sum_n S_t[n] C_t[n] + D[c] u[t, c];   out[t, c] = y_t * silu(z[t, c])
// What a sequence carries is float [K - 1 + N, C]: rows 0..K-2 the last K-1 inputs of the convolution before the
// scan (oldest first), row K-1+n the states S[n] of all channels.  Step sizes, decays, products and states are
// float in both precisions.  A block takes one sequence and SS_CH channels and cuts the sequence's tokens of the
// step into chunks; the map of a chunk on a state is S -> exp(A sum dt) S + Q, so a chunk's first pass sums its
// step sizes and composes Q, the maps are folded in order to give each chunk its incoming states, and a second
// pass writes the outputs.  A step of one token a sequence is one chunk and one pass.
constexpr int SS_CH = 32;           // channels a block takes
constexpr int SS_MAX_N = 256;       // states a channel, when their number is not one the kernel is compiled for
// chunks a block cuts a sequence into: as many as the registers of a thread's states allow threads
constexpr int ss_max_chunks(int ns) { return ns > 0 && ns <= 16 ? 16 : 8; }

// Eight consecutive numbers of a row as floats: sixteen bytes at a time where the row allows it (``wide``: the address
// is a multiple of 16 bytes for every token), else one by one.  The same for all threads of a warp: a broadcast.
__device__ __forceinline__ void ss_load8(const float* __restrict__ p, float (&f)[8], bool wide) {
    if (wide) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = p[i];
    }
}
__device__ __forceinline__ void ss_load8(const __nv_bfloat16* __restrict__ p, float (&f)[8], bool wide) {
    if (wide) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __bfloat1622float2(h[i]);
            f[2 * i] = v.x; f[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(p[i]);
    }
}

// ROOMY: the grid has no more blocks than the GPU has SMs, so a block may have an SM's registers to itself (no spills,
// more loads in flight); else two blocks share an SM (but for 64 states, whose registers fill one).
template <typename T, int NS, bool ROOMY>
__global__ void __launch_bounds__(SS_CH * ss_max_chunks(NS), (NS == 64 || ROOMY) ? 1 : 2)
selective_scan_kernel(const T* __restrict__ u, const float* __restrict__ dtp, const T* __restrict__ bc, long bc_stride,
                      int b_off, int c_off, const T* __restrict__ z, long z_stride, const T* __restrict__ x,
                      long x_stride, const float* __restrict__ a2_t, const float* __restrict__ dvec,
                      float* __restrict__ state, long state_stride, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ slots, T* __restrict__ out, int C, int N_rt, int K, int wide) {
    extern __shared__ float ss_sm[];
    constexpr int NA = NS > 0 ? NS : SS_MAX_N;
    const int N = NS > 0 ? NS : N_rt;
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * SS_CH + threadIdx.x;
    const int chunk = threadIdx.y, n_chunks = blockDim.y;
    float* agg_q = ss_sm;                                   // [n_chunks][N][SS_CH]
    float* agg_dt = ss_sm + (long)n_chunks * N * SS_CH;     // [n_chunks][SS_CH]
    const int first = cu_seqlens[b], n_new = cu_seqlens[b + 1] - first;
    const int per = (n_new + n_chunks - 1) / n_chunks;
    const int lo = first + min(n_new, chunk * per), hi = first + min(n_new, (chunk + 1) * per);
    const bool live = c < C;
    float* st = state + (long)slots[b] * state_stride;
    float A[NA], S[NA];
    if (live) {
#pragma unroll (NS > 0 ? NS : 1)
        for (int n = 0; n < N; ++n)
            A[n] = a2_t[(long)n * C + c];              // A log2(e): exp(dt A) is one multiplication and one exp2
    }
    if (n_chunks > 1) {
        // pass 1: the chunk's map on every state
        float dt_sum = 0.f;
        if (live) {
#pragma unroll (NS > 0 ? NS : 1)
            for (int n = 0; n < N; ++n) S[n] = 0.f;
            // the step size and the input of the next token are requested before this token's arithmetic begins
            float dtp_next = lo < hi ? dtp[(long)lo * C + c] : 0.f;
            float u_next = lo < hi ? to_float(u[(long)lo * C + c]) : 0.f;
            for (int t = lo; t < hi; ++t) {
                const float dt = softplus_f(dtp_next);
                const float dx = dt * u_next;
                if (t + 1 < hi) {
                    dtp_next = dtp[(long)(t + 1) * C + c];
                    u_next = to_float(u[(long)(t + 1) * C + c]);
                }
                const T* bt = bc + (long)t * bc_stride + b_off;
                dt_sum += dt;
                if constexpr (NS > 0) {
#pragma unroll
                    for (int n0 = 0; n0 < NS; n0 += 8) {
                        float b8[8];
                        ss_load8(bt + n0, b8, wide != 0);
#pragma unroll
                        for (int i = 0; i < 8; ++i) S[n0 + i] = fmaf(exp2f(dt * A[n0 + i]), S[n0 + i], dx * b8[i]);
                    }
                } else {
                    for (int n = 0; n < N; ++n)
                        S[n] = fmaf(exp2f(dt * A[n]), S[n], dx * to_float(bt[n]));
                }
            }
#pragma unroll (NS > 0 ? NS : 1)
            for (int n = 0; n < N; ++n)
                agg_q[((long)chunk * N + n) * SS_CH + threadIdx.x] = S[n];
            agg_dt[chunk * SS_CH + threadIdx.x] = dt_sum;
        }
        __syncthreads();
    }
    if (!live) return;
    // the states that enter this chunk: the earlier chunks' maps applied in order to the carried states
#pragma unroll (NS > 0 ? NS : 1)
    for (int n = 0; n < N; ++n)
        S[n] = st[(long)(K - 1 + n) * C + c];
    for (int j = 0; j < chunk; ++j) {
        const float ds = agg_dt[j * SS_CH + threadIdx.x];
#pragma unroll (NS > 0 ? NS : 1)
        for (int n = 0; n < N; ++n)
            S[n] = fmaf(exp2f(ds * A[n]), S[n], agg_q[((long)j * N + n) * SS_CH + threadIdx.x]);
    }
    // pass 2: the outputs
    const float dc = dvec[c];
    float dtp_next = lo < hi ? dtp[(long)lo * C + c] : 0.f;
    float u_next = lo < hi ? to_float(u[(long)lo * C + c]) : 0.f;
    for (int t = lo; t < hi; ++t) {
        const float dt = softplus_f(dtp_next);
        const float uv = u_next;
        const float dx = dt * uv;
        if (t + 1 < hi) {
            dtp_next = dtp[(long)(t + 1) * C + c];
            u_next = to_float(u[(long)(t + 1) * C + c]);
        }
        const T* bt = bc + (long)t * bc_stride + b_off;
        const T* ct = bc + (long)t * bc_stride + c_off;
        float y = 0.f;
        if constexpr (NS > 0) {
#pragma unroll
            for (int n0 = 0; n0 < NS; n0 += 8) {
                float b8[8], c8[8];
                ss_load8(bt + n0, b8, wide != 0);
                ss_load8(ct + n0, c8, wide != 0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    S[n0 + i] = fmaf(exp2f(dt * A[n0 + i]), S[n0 + i], dx * b8[i]);
                    y = fmaf(S[n0 + i], c8[i], y);
                }
            }
        } else {
            for (int n = 0; n < N; ++n) {
                S[n] = fmaf(exp2f(dt * A[n]), S[n], dx * to_float(bt[n]));
                y = fmaf(S[n], to_float(ct[n]), y);
            }
        }
        y = fmaf(dc, uv, y);
        out[(long)t * C + c] = from_float<T>(y * silu_f(to_float(z[(long)t * z_stride + c])));
    }
    if (chunk != n_chunks - 1) return;
    // the last chunk leaves the states after the last token, and the convolution's last K-1 inputs (rows in
    // ascending order: row j takes what row j + n_new held, which is overwritten only later)
#pragma unroll (NS > 0 ? NS : 1)
    for (int n = 0; n < N; ++n)
        st[(long)(K - 1 + n) * C + c] = S[n];
    for (int j = 0; j < K - 1; ++j) {
        const int i = n_new - (K - 1) + j;           // index among the step's tokens, negative: an older input
        st[(long)j * C + c] = i >= 0 ? to_float(x[(long)(first + i) * x_stride + c]) : st[(long)(j + n_new) * C + c];
    }
}

}  // namespace zlm

using namespace zlm;

// x: [T, C] rows with stride x_stride (the convolution's inputs); taps: float [K, C], the row of the current
// token last; bias: float [C];
// state: float [slots, rows, C], of which rows 0..K-2 are the inputs before the step; u: [T, C] contiguous.
// act: 0 none, 1 silu on the convolution's output.
ZLM_EXPORT int zlm_causal_conv(const void* x, int dtype, long x_stride, const float* taps, const float* bias,
                               const float* state, long state_stride, const int* seq_of_token, const int* cu_seqlens,
                               const int* slots, void* u, int n_tokens, int C, int K, int act, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (C <= 0 || K <= 0) return ZLM_ERR_BAD_ARG;
    const long total = (long)n_tokens * C;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(conv_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, x_stride, taps, bias, state,
                       state_stride, seq_of_token, cu_seqlens, slots, (float*)u, n_tokens, C, K, act);
    else if (dtype == ZLM_BF16 && C % 8 == 0 && x_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)u % 16 == 0)
        e = launch_pdl(conv_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream,
                       (const __nv_bfloat16*)x, x_stride, taps, bias, state, state_stride, seq_of_token, cu_seqlens, slots,
                       (__nv_bfloat16*)u, n_tokens, C, K, act);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(conv_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, x_stride,
                       taps, bias, state, state_stride, seq_of_token, cu_seqlens, slots, (__nv_bfloat16*)u, n_tokens, C, K,
                       act);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// u: [T, C]; gates: float [T, 2C], for each block of gate_block channels first its recurrence gates then its
// input gates; y, x: [T, C] rows with strides; lam: float [C]; out: [T, C]; max_new: the most tokens a sequence
// brings (sizes the chunks).
ZLM_EXPORT int zlm_gated_scan(const void* u, int dtype, const float* gates, int gate_block, const void* y, long y_stride,
                              const void* x, long x_stride, const float* lam, float rate, float* state,
                              long state_stride, const int* cu_seqlens, const int* slots, void* out, int n_seqs,
                              int max_new, int C, int K, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (C <= 0 || K <= 0 || gate_block <= 0 || C % gate_block || max_new <= 0) return ZLM_ERR_BAD_ARG;
    if ((C + 15) / 16 > 65535) return ZLM_ERR_UNSUPPORTED;
    // few sequences with many tokens: half as many channels a block and twice the chunks, so that the blocks fill the GPU
    const int ch = (long)n_seqs * ((C + RC_CH - 1) / RC_CH) < 148 && max_new >= 512 ? RC_CH / 2 : RC_CH;
    int chunks = (max_new + 15) / 16;                 // a chunk of fewer than 16 tokens is not worth a thread
    if (chunks > RC_MAX_THREADS / ch) chunks = RC_MAX_THREADS / ch;
    if (chunks > RC_MAX_CHUNKS) chunks = RC_MAX_CHUNKS;
    dim3 grid(n_seqs, (C + ch - 1) / ch), block(ch, chunks);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(scan_kernel<float>, grid, block, 0, stream, (const float*)u, gates, gate_block, (const float*)y,
                       y_stride, (const float*)x, x_stride, lam, rate, state, state_stride, cu_seqlens, slots,
                       (float*)out, C, K);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(scan_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)u, gates, gate_block,
                       (const __nv_bfloat16*)y, y_stride, (const __nv_bfloat16*)x, x_stride, lam, rate, state,
                       state_stride, cu_seqlens, slots, (__nv_bfloat16*)out, C, K);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// u: [T, C] contiguous (the convolution's output); dtp: float [T, C], the step-size projection with its bias, before
// the softplus; bc: rows with stride bc_stride that hold B_t at b_off and C_t at c_off (N numbers each); z, x: [T, C]
// rows with strides (the gate, and the convolution's inputs, which the state keeps); a2_t: float [N, C], A transposed and
// multiplied by log2(e);
// dvec: float [C]; state: float [slots, K - 1 + N, C]; out: [T, C] contiguous; max_new: the most tokens a sequence
// brings (sizes the chunks).
ZLM_EXPORT int zlm_selective_scan(const void* u, int dtype, const float* dtp, const void* bc, long bc_stride, int b_off,
                                  int c_off, const void* z, long z_stride, const void* x, long x_stride,
                                  const float* a2_t, const float* dvec, float* state, long state_stride,
                                  const int* cu_seqlens, const int* slots, void* out, int n_seqs, int max_new, int C,
                                  int N, int K, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (C <= 0 || N <= 0 || K <= 0 || max_new <= 0 || b_off < 0 || c_off < 0) return ZLM_ERR_BAD_ARG;
    if (N > SS_MAX_N || (C + SS_CH - 1) / SS_CH > 65535) return ZLM_ERR_UNSUPPORTED;
    int chunks = (max_new + 15) / 16;                 // a chunk of fewer than 16 tokens is not worth a thread
    const int compiled = (N == 8 || N == 16 || N == 24 || N == 32 || N == 64) ? N : 0;       // the template the switch below picks
    if (chunks > ss_max_chunks(compiled)) chunks = ss_max_chunks(compiled);
    while (chunks > 1 && (size_t)chunks * (N + 1) * SS_CH * sizeof(float) > 48 * 1024) --chunks;
    const size_t smem = chunks > 1 ? (size_t)chunks * (N + 1) * SS_CH * sizeof(float) : 0;
    dim3 grid(n_seqs, (C + SS_CH - 1) / SS_CH), block(SS_CH, chunks);
    // B and C of a token can be read sixteen bytes at a time when every token's B and C start on such a boundary
    const int per16 = dtype == ZLM_F32 ? 4 : 8;
    const int wide = (b_off % per16 == 0 && c_off % per16 == 0 && bc_stride % per16 == 0 && (uintptr_t)bc % 16 == 0) ? 1 : 0;
    static int n_sms = 0;
    if (n_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n_sms = 1;
    }
    const bool roomy = (long)grid.x * grid.y <= n_sms;
    cudaError_t e;
#define ZLM_SS(TT, NS)                                                                                                \
    e = roomy ? launch_pdl(selective_scan_kernel<TT, NS, true>, grid, block, smem, stream, (const TT*)u, dtp, (const TT*)bc, \
                           bc_stride, b_off, c_off, (const TT*)z, z_stride, (const TT*)x, x_stride, a2_t, dvec, state,   \
                           state_stride, cu_seqlens, slots, (TT*)out, C, N, K, wide)                                     \
              : launch_pdl(selective_scan_kernel<TT, NS, false>, grid, block, smem, stream, (const TT*)u, dtp, (const TT*)bc, \
                           bc_stride, b_off, c_off, (const TT*)z, z_stride, (const TT*)x, x_stride, a2_t, dvec, state,   \
                           state_stride, cu_seqlens, slots, (TT*)out, C, N, K, wide)
#define ZLM_SS_N(TT)                                                                                                  \
    switch (N) {                                                                                                      \
        case 8: ZLM_SS(TT, 8); break;                                                                                 \
        case 16: ZLM_SS(TT, 16); break;                                                                               \
        case 24: ZLM_SS(TT, 24); break;                                                                               \
        case 32: ZLM_SS(TT, 32); break;                                                                               \
        case 64: ZLM_SS(TT, 64); break;                                                                               \
        default: ZLM_SS(TT, 0); break;                                                                                \
    }
    if (dtype == ZLM_F32) { ZLM_SS_N(float) }
    else if (dtype == ZLM_BF16) { ZLM_SS_N(__nv_bfloat16) }
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_SS_N
#undef ZLM_SS
    return e == cudaSuccess ? launch_status() : (int)e;
}
