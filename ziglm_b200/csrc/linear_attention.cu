// Linear attention with a fixed decay per head, over a step's sequences, with the state carried in float:
//     S_t = a S_(t-1) + k_t v_t^T          (S: [D, V] per sequence and head, zero at the start)
//     o_t = S_t^T q_t
// q, k, v are read from the rows of a projection (optionally through silu).  Unrolled over a chunk of n tokens
// that starts behind the state S:
//     o_i = sum_{j <= i} a^(i-j) (q_i . k_j) v_j  +  a^(i+1) S^T q_i
//     S'  = a^n S + sum_j a^(n-1-j) k_j v_j^T
// so a chunk is three small matrix products instead of n steps, and a prompt of thousands of tokens is
// T/32 steps of a loop.  A decoded token is a chunk of one.  A block owns one (sequence, head, tile of 32 value
// columns): the columns of S are independent of one another, so the tiles of a head need nothing from each other
// but the scores q_i . k_j, which each computes for itself.  Every product is float FMA in a fixed order: the
// scores and their weights, the state and the outputs never pass through a 16-bit type.
//
// A long prompt is cut into segments of LA_SEG tokens that run side by side (a sequence alone would be a handful
// of blocks that walk its chunks one after the other):
//   1. every segment but a sequence's last sums its own tokens into a state that starts at zero;
//   2. per sequence and head, an element-wise scan turns those into the states the segments start from,
//      S_(s+1) = a^LA_SEG S_s + local_s;
//   3. every segment runs the chunked form from its start state; the last one of a sequence writes the state back.
// The state update is computed twice (steps 1 and 3), which costs a third more arithmetic and buys T / LA_SEG times
// the blocks.
#include "common.cuh"

namespace zlm {

constexpr int LA_C = 32;          // tokens of a chunk
constexpr int LA_VT = 32;         // value columns of a block
constexpr int LA_THREADS = 256;
constexpr int LA_WARPS = LA_THREADS / 32;
constexpr int LA_MAX_D = 512;
constexpr int LA_SEG = 128;       // tokens of a segment: a multiple of the chunk

// The sequence and the segment of it that block g works on, sequences counted in order with ceil(len / LA_SEG)
// segments each.  False: g lies behind the last segment.
__device__ __forceinline__ bool la_find_segment(int g, const int* __restrict__ cu_seqlens, int n_seqs, int& b, int& seg,
                                                int& n_segs) {
    for (b = 0; b < n_seqs; ++b) {
        n_segs = (cu_seqlens[b + 1] - cu_seqlens[b] + LA_SEG - 1) / LA_SEG;
        if (g < n_segs) { seg = g; return true; }
        g -= n_segs;
    }
    return false;
}

__device__ __forceinline__ float la_act(float x, int act) { return act == 1 ? x / (1.0f + expf(-x)) : x; }

// Rotary positions on q and k and a factor on k, applied to the float copies of a chunk in shared memory, so that what
// enters the recurrence never passes through a 16-bit type again: the first `rot` dimensions of a head are turned,
// dimension i together with i + rot/2, by the angle position * inv_freq[i]; k is then multiplied by k_scale.
// inv_freq null and k_scale 1: nothing to do (``active`` says which).
struct LaTurn {
    const float* inv_freq;      // [rot / 2], or null
    const int* positions;       // the position of every token of the step
    int rot;
    float k_scale;
    __device__ __forceinline__ bool active() const { return inv_freq != nullptr || k_scale != 1.0f; }
};

// Rows 0..n-1 of a chunk: q at q_s[j * q_row + d] (null: there are no queries), k at k_s[j * k_row + d * k_el].  Every
// element is touched by one thread; the caller synchronises before (the copies are complete) and after.
__device__ __forceinline__ void la_turn(const LaTurn& r, const int* __restrict__ pos, float* q_s, int q_row, float* k_s,
                                        int k_row, int k_el, int n, int D) {
    const int half = r.inv_freq != nullptr ? r.rot / 2 : 0;
    for (int idx = threadIdx.x; idx < n * half; idx += blockDim.x) {
        const int j = idx / half, i = idx - j * half;
        float sn, cs;
        sincosf((float)pos[j] * r.inv_freq[i], &sn, &cs);
        float* ka = k_s + j * k_row + i * k_el;
        float* kb = k_s + j * k_row + (i + half) * k_el;
        const float u = *ka, v = *kb;
        *ka = (u * cs - v * sn) * r.k_scale;
        *kb = (v * cs + u * sn) * r.k_scale;
        if (q_s != nullptr) {
            float* qa = q_s + j * q_row + i;
            const float qu = qa[0], qv = qa[half];
            qa[0] = qu * cs - qv * sn;
            qa[half] = qv * cs + qu * sn;
        }
    }
    if (r.k_scale != 1.0f) {
        const int rest = D - 2 * half;
        for (int idx = threadIdx.x; idx < n * rest; idx += blockDim.x) {
            const int j = idx / rest, d = 2 * half + idx - j * rest;
            k_s[j * k_row + d * k_el] *= r.k_scale;
        }
    }
}

// Shared memory, in floats, for a key size padded to Dp (a multiple of 4):
//   q_s [C][Dp], kT_s [Dp][C+1], v_s [C][VT], a_s [C][C+1], S_s [Dp][VT]
static inline size_t la_smem_floats(int Dp) {
    return (size_t)LA_C * Dp + (size_t)Dp * (LA_C + 1) + (size_t)LA_C * LA_VT + (size_t)LA_C * (LA_C + 1) + (size_t)Dp * LA_VT;
}

// pows: float [H][C+1], pows[h][n] = decay_h^n.  state: float [slots][H][D][V].  out: float rows [T][H*V].
// seg_state null: a block owns a whole sequence (blockIdx.x).  Else blockIdx.x counts segments and seg_state is
// float [segments][H][D][V]: with STATE_ONLY the block leaves the sum of its segment there (started at zero; a
// sequence's last segment does nothing), without it the block starts from the entry before its own (the scan wrote
// the segment's start state there; a sequence's first segment starts from ``state``) and only a sequence's last
// segment writes ``state``.
template <typename T, bool STATE_ONLY>
__global__ void __launch_bounds__(LA_THREADS)
decayed_linear_attention_kernel(const T* __restrict__ proj, long row_stride, int q_off, int k_off, int v_off, int H,
                                int D, int Dp, int V, int act, LaTurn turn, const float* __restrict__ pows,
                                float* __restrict__ state, const int* __restrict__ slots,
                                const int* __restrict__ cu_seqlens, int n_seqs, float* __restrict__ seg_state,
                                float* __restrict__ out, long out_stride) {
    extern __shared__ __align__(16) float la_smem[];
    float* q_s = la_smem;                              // [C][Dp]
    float* kT_s = q_s + LA_C * Dp;                     // [Dp][C+1]
    float* v_s = kT_s + Dp * (LA_C + 1);               // [C][VT]
    float* a_s = v_s + LA_C * LA_VT;                   // [C][C+1]
    float* S_s = a_s + LA_C * (LA_C + 1);              // [Dp][VT]
    __shared__ float pw[LA_C + 1];

    pdl_launch_dependents();
    const int h = blockIdx.y, v0 = blockIdx.z * LA_VT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nv = min(LA_VT, V - v0);                 // value columns of this tile
    for (int i = threadIdx.x; i <= LA_C; i += LA_THREADS) pw[i] = pows[h * (LA_C + 1) + i];
    pdl_wait();
    int b = blockIdx.x, seg = 0, n_segs = 1;
    if (seg_state != nullptr && !la_find_segment(blockIdx.x, cu_seqlens, n_seqs, b, seg, n_segs)) return;
    if (STATE_ONLY && seg == n_segs - 1) return;
    int first = cu_seqlens[b], last = cu_seqlens[b + 1];
    if (seg_state != nullptr) {
        first += seg * LA_SEG;
        last = min(last, first + LA_SEG);
    }
    const long hdv = (long)H * D * V;
    float* st = state + (((long)slots[b] * H + h) * D) * V;                       // where the sequence's state lives
    const float* from = seg == 0 ? st : seg_state + (long)(blockIdx.x - 1) * hdv + (long)h * D * V;
    float* to = STATE_ONLY ? seg_state + (long)blockIdx.x * hdv + (long)h * D * V : st;
    for (int i = threadIdx.x; i < Dp * LA_VT; i += LA_THREADS) {
        const int d = i / LA_VT, v = i % LA_VT;
        S_s[i] = (!STATE_ONLY && d < D && v < nv) ? from[(long)d * V + v0 + v] : 0.f;
    }

    for (int c0 = first; c0 < last; c0 += LA_C) {
        const int n = min(LA_C, last - c0);
        __syncthreads();                               // the chunk before is done with q_s, kT_s, v_s, a_s
        for (int i = threadIdx.x; i < LA_C * Dp; i += LA_THREADS) {
            const int j = i / Dp, d = i % Dp;
            float qv = 0.f, kv = 0.f;
            if (j < n && d < D) {
                const T* row = proj + (long)(c0 + j) * row_stride + (long)h * D + d;
                qv = la_act(to_float(row[q_off]), act);
                kv = la_act(to_float(row[k_off]), act);
            }
            q_s[j * Dp + d] = qv;
            kT_s[d * (LA_C + 1) + j] = kv;
        }
        for (int i = threadIdx.x; i < LA_C * LA_VT; i += LA_THREADS) {
            const int j = i / LA_VT, v = i % LA_VT;
            v_s[i] = (j < n && v < nv) ? la_act(to_float(proj[(long)(c0 + j) * row_stride + v_off + (long)h * V + v0 + v]), act)
                                       : 0.f;
        }
        __syncthreads();
        if (turn.active()) {
            la_turn(turn, turn.positions + c0, STATE_ONLY ? nullptr : q_s, Dp, kT_s, 1, LA_C + 1, n, D);
            __syncthreads();
        }
        // scores with their decay: a_s[i][j] = a^(i-j) (q_i . k_j) for j <= i.  A thread: rows warp, warp+8, .., column lane.
        if (!STATE_ONLY) {
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            for (int d = 0; d < Dp; d += 4) {
                const float k0 = kT_s[(d + 0) * (LA_C + 1) + lane], k1 = kT_s[(d + 1) * (LA_C + 1) + lane];
                const float k2 = kT_s[(d + 2) * (LA_C + 1) + lane], k3 = kT_s[(d + 3) * (LA_C + 1) + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp + LA_WARPS * r) * Dp + d);
                    s[r] = fmaf(qv.x, k0, s[r]); s[r] = fmaf(qv.y, k1, s[r]);
                    s[r] = fmaf(qv.z, k2, s[r]); s[r] = fmaf(qv.w, k3, s[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = warp + LA_WARPS * r;
                a_s[i * (LA_C + 1) + lane] = lane <= i ? s[r] * pw[i - lane] : 0.f;
            }
        }
        if (!STATE_ONLY) __syncthreads();
        // outputs: o_i = sum_j a_s[i][j] v_j + a^(i+1) S^T q_i.  A thread: rows warp, warp+8, .., value column lane.
        if (!STATE_ONLY) {
            float o[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n; ++j) {
                const float vv = v_s[j * LA_VT + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) o[r] = fmaf(a_s[(warp + LA_WARPS * r) * (LA_C + 1) + j], vv, o[r]);
            }
            for (int d = 0; d < Dp; d += 4) {
                const float s0 = S_s[(d + 0) * LA_VT + lane], s1 = S_s[(d + 1) * LA_VT + lane];
                const float s2 = S_s[(d + 2) * LA_VT + lane], s3 = S_s[(d + 3) * LA_VT + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp + LA_WARPS * r) * Dp + d);
                    p[r] = fmaf(qv.x, s0, p[r]); p[r] = fmaf(qv.y, s1, p[r]);
                    p[r] = fmaf(qv.z, s2, p[r]); p[r] = fmaf(qv.w, s3, p[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = warp + LA_WARPS * r;
                if (i < n && lane < nv)
                    out[(long)(c0 + i) * out_stride + (long)h * V + v0 + lane] = fmaf(pw[i + 1], p[r], o[r]);
            }
        }
        if (!STATE_ONLY) __syncthreads();              // everyone has read the old state and v_s
        // the values weighted for the state: v_j a^(n-1-j)
        for (int i = threadIdx.x; i < LA_C * LA_VT; i += LA_THREADS) {
            const int j = i / LA_VT;
            if (j < n) v_s[i] *= pw[n - 1 - j];
        }
        __syncthreads();
        // S' = a^n S + sum_j k_j (v_j a^(n-1-j))^T.  A thread: key dimensions warp, warp+8, .., value column lane.
        {
            const float an = pw[n];
            for (int d0 = warp; d0 < Dp; d0 += LA_WARPS * 8) {
                float acc[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) acc[r] = 0.f;
                for (int j = 0; j < n; ++j) {
                    const float vv = v_s[j * LA_VT + lane];
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const int d = d0 + LA_WARPS * r;
                        if (d < Dp) acc[r] = fmaf(kT_s[d * (LA_C + 1) + j], vv, acc[r]);
                    }
                }
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const int d = d0 + LA_WARPS * r;
                    if (d < Dp) S_s[d * LA_VT + lane] = fmaf(an, S_s[d * LA_VT + lane], acc[r]);
                }
            }
        }
    }
    __syncthreads();
    if (!STATE_ONLY && seg != n_segs - 1) return;      // the next segment starts from what the scan left it
    for (int i = threadIdx.x; i < Dp * LA_VT; i += LA_THREADS) {
        const int d = i / LA_VT, v = i % LA_VT;
        if (d < D && v < nv) to[(long)d * V + v0 + v] = S_s[i];
    }
}


// The same work for bf16 rows whose key size is a multiple of 32 up to 128 and whose offsets, strides and value size
// are multiples of 8 elements.  q, k and v are read 16 bytes a thread, and the rows of the next chunk are requested
// before the arithmetic on this one begins; a key is a row of D + 4 floats, so that a lane reads four dimensions of its
// own key in one instruction without a bank conflict (the scores) and a warp four dimensions of one key as a broadcast
// (the state); the decay of a value rides on the multiplication that uses it.  With STATE_ONLY neither queries nor scores exist.
static inline size_t la_fast_smem_floats(int D, bool state_only) {
    size_t n = (size_t)LA_C * (D + 4) + (size_t)LA_C * LA_VT + (size_t)D * LA_VT;            // k_s, v_s, S_s
    if (!state_only) n += (size_t)LA_C * D + (size_t)LA_C * (LA_C + 1);                       // q_s, a_s
    return n;
}

template <bool STATE_ONLY>
__global__ void __launch_bounds__(LA_THREADS, 3)
la_fast_kernel(const __nv_bfloat16* __restrict__ proj, long row_stride, int q_off, int k_off, int v_off, int H, int D, int V,
               int act, LaTurn turn, const float* __restrict__ pows, float* __restrict__ state, const int* __restrict__ slots,
               const int* __restrict__ cu_seqlens, int n_seqs, float* __restrict__ seg_state, float* __restrict__ out,
               long out_stride) {
    extern __shared__ __align__(16) float la_smem[];
    const int KS = D + 4;                              // floats of a key's row
    float* k_s = la_smem;                              // [C][D + 4]
    float* v_s = k_s + LA_C * KS;                      // [C][VT]
    float* S_s = v_s + LA_C * LA_VT;                   // [D][VT]
    float* q_s = S_s + D * LA_VT;                      // [C][D]
    float* a_s = q_s + LA_C * D;                       // [C][C+1]
    __shared__ float pw[LA_C + 1];

    pdl_launch_dependents();
    const int h = blockIdx.y, v0 = blockIdx.z * LA_VT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nv = min(LA_VT, V - v0);                 // value columns of this tile (a multiple of 8)
    for (int i = threadIdx.x; i <= LA_C; i += LA_THREADS) pw[i] = pows[h * (LA_C + 1) + i];
    pdl_wait();
    int b = blockIdx.x, seg = 0, n_segs = 1;
    if (seg_state != nullptr && !la_find_segment(blockIdx.x, cu_seqlens, n_seqs, b, seg, n_segs)) return;
    if (STATE_ONLY && seg == n_segs - 1) return;
    int first = cu_seqlens[b], last = cu_seqlens[b + 1];
    if (seg_state != nullptr) {
        first += seg * LA_SEG;
        last = min(last, first + LA_SEG);
    }
    const long hdv = (long)H * D * V;
    float* st = state + (((long)slots[b] * H + h) * D) * V;
    const float* from = seg == 0 ? st : seg_state + (long)(blockIdx.x - 1) * hdv + (long)h * D * V;
    float* to = STATE_ONLY ? seg_state + (long)blockIdx.x * hdv + (long)h * D * V : st;
    for (int i = threadIdx.x; i < D * LA_VT; i += LA_THREADS) {
        const int d = i / LA_VT, v = i % LA_VT;
        S_s[i] = (!STATE_ONLY && v < nv) ? from[(long)d * V + v0 + v] : 0.f;
    }

    // what a thread fetches of a chunk: two vectors of q and of k (the chunk holds C * D/8 <= 512), one of v
    const int D8 = D >> 3;
    int qj[2], qd[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int idx = threadIdx.x + u * LA_THREADS;
        qj[u] = idx < LA_C * D8 ? idx / D8 : -1;
        qd[u] = (idx - (idx / D8) * D8) * 8;
    }
    const int vj = threadIdx.x < LA_C * (LA_VT / 8) ? threadIdx.x / (LA_VT / 8) : -1;
    const int vd = (threadIdx.x % (LA_VT / 8)) * 8;
    uint4 rq[2], rk[2], rv;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    auto fetch = [&](int c0) {
        const int n = min(LA_C, last - c0);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            rq[u] = zero4; rk[u] = zero4;
            if (qj[u] >= 0 && qj[u] < n) {
                const __nv_bfloat16* row = proj + (long)(c0 + qj[u]) * row_stride + (long)h * D + qd[u];
                if (!STATE_ONLY) rq[u] = *reinterpret_cast<const uint4*>(row + q_off);
                rk[u] = *reinterpret_cast<const uint4*>(row + k_off);
            }
        }
        rv = zero4;
        if (vj >= 0 && vj < n && vd < nv)
            rv = *reinterpret_cast<const uint4*>(proj + (long)(c0 + vj) * row_stride + v_off + (long)h * V + v0 + vd);
    };
    auto unpack = [&](const uint4& r, float* f) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __bfloat1622float2(p[e]);
            f[2 * e] = la_act(x.x, act);
            f[2 * e + 1] = la_act(x.y, act);
        }
    };
    auto stash = [&]() {
        float f[8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (qj[u] < 0) continue;
            unpack(rk[u], f);
            *reinterpret_cast<float4*>(k_s + qj[u] * KS + qd[u]) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(k_s + qj[u] * KS + qd[u] + 4) = make_float4(f[4], f[5], f[6], f[7]);
            if (!STATE_ONLY) {
                unpack(rq[u], f);
                *reinterpret_cast<float4*>(q_s + qj[u] * D + qd[u]) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(q_s + qj[u] * D + qd[u] + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
        if (vj >= 0) {
            unpack(rv, f);
            *reinterpret_cast<float4*>(v_s + vj * LA_VT + vd) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(v_s + vj * LA_VT + vd + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
    };

    if (first < last) fetch(first);
    const int rpw = D >> 3;                            // key dimensions of a warp in the state update: 4, 8, 12 or 16
    for (int c0 = first; c0 < last; c0 += LA_C) {
        const int n = min(LA_C, last - c0);
        __syncthreads();                               // the chunk before is done with the rows; its state is written
        stash();
        if (c0 + LA_C < last) fetch(c0 + LA_C);
        __syncthreads();
        if (turn.active()) {
            la_turn(turn, turn.positions + c0, STATE_ONLY ? nullptr : q_s, D, k_s, KS, 1, n, D);
            __syncthreads();
        }
        if (!STATE_ONLY) {
            // scores with their decay: a_s[i][j] = a^(i-j) (q_i . k_j) for j <= i.  A thread: rows warp, warp+8, .., column lane.
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            for (int d = 0; d < D; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(k_s + lane * KS + d);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp + LA_WARPS * r) * D + d);
                    s[r] = fmaf(qv.x, kv.x, s[r]); s[r] = fmaf(qv.y, kv.y, s[r]);
                    s[r] = fmaf(qv.z, kv.z, s[r]); s[r] = fmaf(qv.w, kv.w, s[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = warp + LA_WARPS * r;
                a_s[i * (LA_C + 1) + lane] = lane <= i ? s[r] * pw[i - lane] : 0.f;
            }
            __syncthreads();
            // outputs: o_i = sum_j a_s[i][j] v_j + a^(i+1) S^T q_i.  A thread: rows warp, warp+8, .., value column lane.
            float o[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n; ++j) {
                const float vv = v_s[j * LA_VT + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) o[r] = fmaf(a_s[(warp + LA_WARPS * r) * (LA_C + 1) + j], vv, o[r]);
            }
            for (int d = 0; d < D; d += 4) {
                const float s0 = S_s[(d + 0) * LA_VT + lane], s1 = S_s[(d + 1) * LA_VT + lane];
                const float s2 = S_s[(d + 2) * LA_VT + lane], s3 = S_s[(d + 3) * LA_VT + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp + LA_WARPS * r) * D + d);
                    p[r] = fmaf(qv.x, s0, p[r]); p[r] = fmaf(qv.y, s1, p[r]);
                    p[r] = fmaf(qv.z, s2, p[r]); p[r] = fmaf(qv.w, s3, p[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = warp + LA_WARPS * r;
                if (i < n && lane < nv)
                    out[(long)(c0 + i) * out_stride + (long)h * V + v0 + lane] = fmaf(pw[i + 1], p[r], o[r]);
            }
            __syncthreads();                           // everyone has read the old state
        }
        // S' = a^n S + sum_j k_j (v_j a^(n-1-j))^T.  A thread: key dimensions warp * rpw .. + rpw, value column lane.
        {
            const float an = pw[n];
            const int dbase = warp * rpw;
            for (int g = 0; g < rpw; g += 8) {
                const bool two = g + 4 < rpw;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < n; ++j) {
                    const float vw = v_s[j * LA_VT + lane] * pw[n - 1 - j];
                    const float4 ka = *reinterpret_cast<const float4*>(k_s + j * KS + dbase + g);
                    acc[0] = fmaf(ka.x, vw, acc[0]); acc[1] = fmaf(ka.y, vw, acc[1]);
                    acc[2] = fmaf(ka.z, vw, acc[2]); acc[3] = fmaf(ka.w, vw, acc[3]);
                    if (two) {
                        const float4 kb = *reinterpret_cast<const float4*>(k_s + j * KS + dbase + g + 4);
                        acc[4] = fmaf(kb.x, vw, acc[4]); acc[5] = fmaf(kb.y, vw, acc[5]);
                        acc[6] = fmaf(kb.z, vw, acc[6]); acc[7] = fmaf(kb.w, vw, acc[7]);
                    }
                }
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (r < 4 || two) {
                        float* sp = S_s + (dbase + g + r) * LA_VT + lane;
                        *sp = fmaf(an, *sp, acc[r]);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (!STATE_ONLY && seg != n_segs - 1) return;      // the next segment starts from what the scan left it
    for (int i = threadIdx.x; i < D * LA_VT; i += LA_THREADS) {
        const int d = i / LA_VT, v = i % LA_VT;
        if (v < nv) to[(long)d * V + v0 + v] = S_s[i];
    }
}

// Step 2: seg_state[g] holds the local sum of segment g (entries of last segments are unused).  Afterwards entry g
// holds the state segment g + 1 starts from.  One thread an element of [D, V], one block row a (sequence, head).
__global__ void __launch_bounds__(256)
la_segment_scan_kernel(const float* __restrict__ pows, const float* __restrict__ state, const int* __restrict__ slots,
                       const int* __restrict__ cu_seqlens, int n_seqs, int H, int DV, float* __restrict__ seg_state) {
    pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y, e = blockIdx.z * blockDim.x + threadIdx.x;
    pdl_wait();
    if (e >= DV) return;
    int g0 = 0;                                        // the sequence's first segment
    for (int i = 0; i < b; ++i) g0 += (cu_seqlens[i + 1] - cu_seqlens[i] + LA_SEG - 1) / LA_SEG;
    const int n_segs = (cu_seqlens[b + 1] - cu_seqlens[b] + LA_SEG - 1) / LA_SEG;
    if (n_segs < 2) return;
    const float ac = pows[h * (LA_C + 1) + LA_C];      // the decay over a chunk, applied chunk by chunk as step 3 does
    float run = state[((long)slots[b] * H + h) * DV + e];
    for (int s = 0; s + 1 < n_segs; ++s) {
        float* p = seg_state + ((long)(g0 + s) * H + h) * DV + e;
#pragma unroll
        for (int c = 0; c < LA_SEG / LA_C; ++c) run *= ac;
        run += *p;
        *p = run;
    }
}


// A step in which every sequence brings one token: S' = a S + k v^T and o = S'^T q straight on the state in global
// memory.  A block owns a (sequence, head, tile of 32 value columns); lane l owns column l, warp w the key dimensions
// w, w + 8, ...  The state's elements are requested before q and k are in shared memory, a batch of
// LA_DEC_ROWS key dimensions a thread at a time; the warps' partial outputs are summed in a fixed order.
constexpr int LA_DEC_ROWS = 16;

template <typename T>
__global__ void __launch_bounds__(LA_THREADS)
la_decode_kernel(const T* __restrict__ proj, long row_stride, int q_off, int k_off, int v_off, int H, int D, int V, int act,
                 LaTurn turn, const float* __restrict__ pows, float* __restrict__ state, const int* __restrict__ slots,
                 const int* __restrict__ cu_seqlens, float* __restrict__ out, long out_stride) {
    __shared__ float q_s[LA_MAX_D], k_s[LA_MAX_D], red[LA_WARPS][LA_VT];
    pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v = blockIdx.z * LA_VT + lane;
    const float a = pows[h * (LA_C + 1) + 1];
    pdl_wait();
    float* st = state + (((long)slots[b] * H + h) * D) * V + v;
    float s_reg[LA_DEC_ROWS];
#pragma unroll
    for (int u = 0; u < LA_DEC_ROWS; ++u) {
        const int d = warp + u * LA_WARPS;
        s_reg[u] = (v < V && d < D) ? st[(long)d * V] : 0.f;
    }
    const long t = cu_seqlens[b];
    const T* row = proj + t * row_stride;
    for (int i = threadIdx.x; i < D; i += LA_THREADS) {
        q_s[i] = la_act(to_float(row[q_off + h * D + i]), act);
        k_s[i] = la_act(to_float(row[k_off + h * D + i]), act);
    }
    const float vv = v < V ? la_act(to_float(row[v_off + h * V + v]), act) : 0.f;
    __syncthreads();
    if (turn.active()) {
        la_turn(turn, turn.positions + t, q_s, 0, k_s, 0, 1, 1, D);
        __syncthreads();
    }
    float acc = 0.f;
    for (int base = 0; base < D; base += LA_DEC_ROWS * LA_WARPS) {
        if (base > 0) {
#pragma unroll
            for (int u = 0; u < LA_DEC_ROWS; ++u) {
                const int d = base + warp + u * LA_WARPS;
                s_reg[u] = (v < V && d < D) ? st[(long)d * V] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < LA_DEC_ROWS; ++u) {
            const int d = base + warp + u * LA_WARPS;
            if (v < V && d < D) {
                const float s = fmaf(a, s_reg[u], k_s[d] * vv);
                st[(long)d * V] = s;
                acc = fmaf(s, q_s[d], acc);
            }
        }
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && v < V) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) o += red[w][lane];
        out[t * out_stride + h * V + v] = o;
    }
}

}  // namespace zlm

using namespace zlm;

// The chunk length the table of powers must cover: pows is float [H][zlm_linear_attention_chunk() + 1].
ZLM_EXPORT int zlm_linear_attention_chunk() { return LA_C; }

// proj: rows [T][row_stride] of the step's type; head h's query lies at columns q_off + h*D, its key at k_off + h*D,
// its value at v_off + h*V.  act 0: as they are, 1: through silu.  pows: float [H][chunk + 1] with decay_h^n.
// state: float [n_slots][H][D][V]; slots, cu_seqlens: the step's sequences.  out: float rows [T][out_stride].
// seg_state: null, or float [zlm_linear_attention_segments(T, n_seqs)][H][D][V] of scratch, with which the step's T
// tokens run as segments side by side (three launches instead of one).  single_token: every sequence brings exactly
// one token (the state is updated in place, without chunks).
template <typename T>
static int la_launch(const T* proj, long row_stride, int q_off, int k_off, int v_off, int H, int D, int V, int act,
                     LaTurn turn, const float* pows, float* state, const int* slots, const int* cu_seqlens, int n_seqs,
                     int n_segments, bool single_token, float* seg_state, float* out, long out_stride, cudaStream_t stream) {
    const int Dp = (D + 3) / 4 * 4;
    const size_t smem = la_smem_floats(Dp) * sizeof(float);
    const int v_tiles = (V + LA_VT - 1) / LA_VT;
    cudaError_t e;
    if (single_token) {
        e = launch_pdl(la_decode_kernel<T>, dim3(n_seqs, H, v_tiles), dim3(LA_THREADS), 0, stream, proj, row_stride, q_off,
                       k_off, v_off, H, D, V, act, turn, pows, state, slots, cu_seqlens, out, out_stride);
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    if (sizeof(T) == 2 && D % 32 == 0 && D <= 128 && V % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
        row_stride % 8 == 0 && (uintptr_t)proj % 16 == 0) {
        const __nv_bfloat16* rows = reinterpret_cast<const __nv_bfloat16*>(proj);
        const size_t smem_full = la_fast_smem_floats(D, false) * sizeof(float), smem_local = la_fast_smem_floats(D, true) * sizeof(float);
        auto full = la_fast_kernel<false>;
        auto local = la_fast_kernel<true>;
        if ((e = cudaFuncSetAttribute(full, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_full)) != cudaSuccess) return (int)e;
        if (seg_state == nullptr) {
            e = launch_pdl(full, dim3(n_seqs, H, v_tiles), dim3(LA_THREADS), smem_full, stream, rows, row_stride, q_off, k_off,
                           v_off, H, D, V, act, turn, pows, state, slots, cu_seqlens, n_seqs, (float*)nullptr, out, out_stride);
            return e == cudaSuccess ? launch_status() : (int)e;
        }
        if ((e = cudaFuncSetAttribute(local, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_local)) != cudaSuccess) return (int)e;
        dim3 grid(n_segments, H, v_tiles);
        e = launch_pdl(local, grid, dim3(LA_THREADS), smem_local, stream, rows, row_stride, q_off, k_off, v_off, H, D, V, act,
                       turn, pows, state, slots, cu_seqlens, n_seqs, seg_state, out, out_stride);
        if (e != cudaSuccess) return (int)e;
        e = launch_pdl(la_segment_scan_kernel, dim3(n_seqs, H, (D * V + 255) / 256), dim3(256), 0, stream, pows,
                       (const float*)state, slots, cu_seqlens, n_seqs, H, D * V, seg_state);
        if (e != cudaSuccess) return (int)e;
        e = launch_pdl(full, grid, dim3(LA_THREADS), smem_full, stream, rows, row_stride, q_off, k_off, v_off, H, D, V, act, turn, pows,
                       state, slots, cu_seqlens, n_seqs, seg_state, out, out_stride);
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    auto full = decayed_linear_attention_kernel<T, false>;
    auto local = decayed_linear_attention_kernel<T, true>;
    if (smem > 48 * 1024) {
        if ((e = cudaFuncSetAttribute(full, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        if ((e = cudaFuncSetAttribute(local, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
    }
    if (seg_state == nullptr) {
        e = launch_pdl(full, dim3(n_seqs, H, v_tiles), dim3(LA_THREADS), smem, stream, proj, row_stride, q_off, k_off, v_off,
                       H, D, Dp, V, act, turn, pows, state, slots, cu_seqlens, n_seqs, (float*)nullptr, out, out_stride);
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    dim3 grid(n_segments, H, v_tiles);
    e = launch_pdl(local, grid, dim3(LA_THREADS), smem, stream, proj, row_stride, q_off, k_off, v_off, H, D, Dp, V, act,
                   turn, pows, state, slots, cu_seqlens, n_seqs, seg_state, out, out_stride);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(la_segment_scan_kernel, dim3(n_seqs, H, (D * V + 255) / 256), dim3(256), 0, stream, pows,
                   (const float*)state, slots, cu_seqlens, n_seqs, H, D * V, seg_state);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(full, grid, dim3(LA_THREADS), smem, stream, proj, row_stride, q_off, k_off, v_off, H, D, Dp, V, act, turn, pows,
                   state, slots, cu_seqlens, n_seqs, seg_state, out, out_stride);
    return e == cudaSuccess ? launch_status() : (int)e;
}

// An upper bound of the segments of a step of n_tokens tokens in n_seqs sequences: the entries ``seg_state`` needs.
ZLM_EXPORT int zlm_linear_attention_segments(int n_tokens, int n_seqs) { return n_tokens / LA_SEG + n_seqs; }
ZLM_EXPORT int zlm_linear_attention_segment() { return LA_SEG; }

// rot / inv_freq / positions / k_scale: rotary positions on q and k (the first rot dimensions of every head, halves
// paired; inv_freq float [rot/2], null: none; positions: one per token of the step) and a factor on k behind it.
ZLM_EXPORT int zlm_decayed_linear_attention(const void* proj, int dtype, long row_stride, int q_off, int k_off, int v_off,
                                            int H, int D, int V, int act, int rot, const float* inv_freq,
                                            const int* positions, float k_scale, const float* pows, float* state,
                                            const int* slots, const int* cu_seqlens, int n_seqs, int n_tokens,
                                            int single_token, float* seg_state, float* out, long out_stride,
                                            cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || (act != 0 && act != 1)) return ZLM_ERR_BAD_ARG;
    if (inv_freq != nullptr && (rot <= 0 || rot > D || (rot & 1) || positions == nullptr)) return ZLM_ERR_BAD_ARG;
    LaTurn turn;
    turn.inv_freq = inv_freq; turn.positions = positions; turn.rot = inv_freq != nullptr ? rot : 0; turn.k_scale = k_scale;
    if (D > LA_MAX_D || H > 65535 || (V + LA_VT - 1) / LA_VT > 65535 || n_seqs > 65535) return ZLM_ERR_UNSUPPORTED;
    const int n_segments = zlm_linear_attention_segments(n_tokens, n_seqs);
    if (dtype == ZLM_F32)
        return la_launch((const float*)proj, row_stride, q_off, k_off, v_off, H, D, V, act, turn, pows, state, slots, cu_seqlens,
                         n_seqs, n_segments, single_token != 0, seg_state, out, out_stride, stream);
    if (dtype == ZLM_BF16)
        return la_launch((const __nv_bfloat16*)proj, row_stride, q_off, k_off, v_off, H, D, V, act, turn, pows, state, slots,
                         cu_seqlens, n_seqs, n_segments, single_token != 0, seg_state, out, out_stride, stream);
    return ZLM_ERR_UNSUPPORTED;
}
