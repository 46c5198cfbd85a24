// Mixture of experts: routing, the grouping of (token, choice) pairs by expert, the experts' products over those
// groups, and the weighted sum of a token's expert outputs.
//
// Routing, per token, in float:
//   score_e  = sigmoid(z_e) or z_e's softmax                              (z: router logits)
//   (or, mode 2: the experts with the largest logits are chosen and weighted by the softmax over the chosen
//   logits alone)
//   choice_e = score_e + correction_e                                     (correction may be absent)
//   experts form n_groups equal groups of neighbours; a group's score is the sum of its group_best largest
//   choice scores; only experts of the keep_groups best groups can be chosen (the others count as -inf);
//   the `top` experts with the largest choice scores are chosen (ties: the lower index), and their weights are
//   score_e (without the correction), divided by their sum if `renormalize`, times `weight_scale`.
//   The last experts may be identity experts (n_real < E at the grouping and the products): they have no weights,
//   their output is the token's row itself, and the sum over a token's pairs takes it from there.
//
// Pair p = token * top + k.  The pairs are grouped by expert into `sorted` (offsets per expert in `offs`), and
// the rows of every expert are cut into tiles of GM rows (`tile_expert`, `tile_row`; `n_tiles[0]` tiles in all).
// The two products run over those tiles: gate/up with the activation (input rows gathered by token, output
// rows in sorted order) and down (output rows scattered to the pair's own row, float).  The sum over a token's
// pairs is taken by one thread in the order of k, so nothing depends on the step's other tokens.
#include "common.cuh"

namespace zlm {

constexpr int GM = 32, GN = 64, GK = 32;

// act(gate) * up of an expert: silu(g) u, or with a limit L > 0 the clamped swish
// min(g, L) sigmoid(slope min(g, L)) (clamp(u, -L, L) + 1)
__device__ __forceinline__ float expert_glu(float g, float u, float limit, float slope) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit) + 1.0f;
        return (g / (1.0f + expf(-slope * g))) * u;
    }
    return (g / (1.0f + expf(-g))) * u;
}

// ------------------------------------------------------------------- routing
// one block of RT_WARPS warps per token; shared: score[E], choice[E], group score[n_groups], and the token's
// row when the router's product is taken here.  z != null: the router logits were computed before.  Otherwise
// z_e = sum_i h[t, i] * w[e, i] is taken here, a warp per expert with the lanes walking the row in a fixed
// order (steps of few tokens: a product kernel of its own would cost more than the whole routing).
constexpr int RT_WARPS = 8;

template <typename TH>
__global__ void __launch_bounds__(RT_WARPS * 32)
route_kernel(const float* __restrict__ z, long z_stride, const TH* __restrict__ h, long h_stride, const TH* __restrict__ w,
             int d, const float* __restrict__ correction, int E, int top, int n_groups, int keep_groups, int group_best,
             int softmax_scores, int renormalize, float weight_scale, int n_extra, float* __restrict__ extra_out,
             int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float sm[];
    float* score = sm;                 // [E]
    float* choice = sm + E;            // [E]
    float* gscore = sm + 2 * E;        // [n_groups]
    float* logit = gscore + n_groups;  // [E]
    float* row = logit + E;            // [d] when the product is taken here
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (z != nullptr) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) logit[e] = z[(long)t * z_stride + e];
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) row[i] = to_float(h[(long)t * h_stride + i]);
        __syncthreads();
        constexpr int V = 16 / (int)sizeof(TH);
        const bool wide = d % V == 0 && (uintptr_t)w % 16 == 0;
        // the rows behind the experts' (n_extra of them) are further products of the same row: their sums go to extra_out
        for (int e = warp; e < E + n_extra; e += RT_WARPS) {
            const TH* we = w + (long)e * d;
            float acc = 0.f;
            if (wide) {
                // four vectors of the row are requested before the first is used: with a handful of blocks the
                // product is bound by the latency of its loads, not by their number
                for (int i0 = lane * V; i0 < d; i0 += 4 * 32 * V) {
                    uint4 raw[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + u * 32 * V;
                        raw[u] = i < d ? *reinterpret_cast<const uint4*>(we + i) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i = i0 + u * 32 * V;
                        if (i < d) {
                            const TH* wv = reinterpret_cast<const TH*>(&raw[u]);
#pragma unroll
                            for (int k = 0; k < V; ++k) acc = fmaf(row[i + k], to_float(wv[k]), acc);
                        }
                    }
                }
            } else {
                for (int i = lane; i < d; i += 32) acc = fmaf(row[i], to_float(we[i]), acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) {
                if (e < E) logit[e] = acc;
                else extra_out[(long)t * n_extra + (e - E)] = acc;
            }
        }
    }
    __syncthreads();
    if (warp != 0) return;
    const float* zr = logit;
    float zmax = -INFINITY, zsum = 0.f;
    if (softmax_scores == 1) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, zr[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(zr[e] - zmax);
        zsum = warp_sum(zsum);
    }
    for (int e = lane; e < E; e += 32) {
        // 2: the logit itself is the choice score; the weights are the softmax over the chosen logits (below)
        const float s = softmax_scores == 2 ? zr[e]
                        : (softmax_scores ? expf(zr[e] - zmax) / zsum : 1.0f / (1.0f + expf(-zr[e])));
        score[e] = s;
        choice[e] = correction ? s + correction[e] : s;
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
        const int size = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            // the sum of the group's group_best largest choice scores: take the largest that lies below the last taken
            float total = 0.f, last = INFINITY;
            int last_i = -1;
            for (int n = 0; n < group_best && n < size; ++n) {
                float best = -INFINITY;
                int best_i = -1;
                for (int i = 0; i < size; ++i) {
                    const float c = choice[g * size + i];
                    const bool below = c < last || (c == last && i > last_i);
                    if (below && (c > best || best_i < 0)) { best = c; best_i = i; }
                }
                total += best;
                last = best; last_i = best_i;
            }
            gscore[g] = total;
        }
        __syncwarp();
        for (int g = lane; g < n_groups; g += 32) {
            int ahead = 0;
            for (int o = 0; o < n_groups; ++o)
                ahead += (gscore[o] > gscore[g] || (gscore[o] == gscore[g] && o < g)) ? 1 : 0;
            if (ahead >= keep_groups)
                for (int i = 0; i < size; ++i) choice[g * size + i] = -INFINITY;
        }
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best || (c == best && e < best_e && c > -INFINITY)) { best = c; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;       // fewer finite candidates than `top`: cannot happen with a checked configuration
        if (lane == 0) {
            ids[(long)t * top + k] = best_e;
            weights[(long)t * top + k] = score[best_e];
            choice[best_e] = -INFINITY;
        }
        wsum += score[best_e];
        __syncwarp();
    }
    if (softmax_scores == 2) {
        if (lane == 0) {
            // the first chosen logit is the largest
            const float first = weights[(long)t * top];
            float total = 0.f;
            for (int k = 0; k < top; ++k) {
                const float w = expf(weights[(long)t * top + k] - first);
                weights[(long)t * top + k] = w;
                total += w;
            }
            for (int k = 0; k < top; ++k) weights[(long)t * top + k] /= total;
        }
        return;
    }
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) weights[(long)t * top + k] /= wsum;
    if (weight_scale != 1.0f && lane == 0)
        for (int k = 0; k < top; ++k) weights[(long)t * top + k] *= weight_scale;
}

// ------------------------------------------------------------------ grouping
// one block.  counts -> offsets -> sorted pairs and tiles.
__global__ void group_kernel(const int* __restrict__ ids, int P, int E, int n_real, int* __restrict__ offs,
                             int* __restrict__ sorted, int* __restrict__ place, int* __restrict__ tile_expert,
                             int* __restrict__ tile_row, int* __restrict__ n_tiles) {
    extern __shared__ int smi[];
    int* count = smi;             // [E]
    int* start = smi + E;         // [E + 1]
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            offs[e] = at;
            // an identity expert (e >= n_real) has no product: its pairs are grouped like the others and make no tile
            for (int r = 0; e < n_real && r < count[e]; r += GM) { tile_expert[tiles] = e; tile_row[tiles] = at + r; ++tiles; }
            at += count[e];
        }
        start[E] = at;
        offs[E] = at;
        n_tiles[0] = tiles;
    }
    __syncthreads();
    // pair p goes to the place its rank among its expert's pairs gives it: pairs in ascending order
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    if (P <= 1024) {
        // few pairs: a stable order (pairs of an expert in ascending order), so that a row's place does not depend
        // on the timing of the threads.  A pair's rank is the number of earlier pairs of its expert.
        int* cached = start + E + 1;          // [P]
        for (int p = threadIdx.x; p < P; p += blockDim.x) cached[p] = ids[p];
        __syncthreads();
        for (int p = threadIdx.x; p < P; p += blockDim.x) {
            const int e = cached[p];
            int rank = 0;
            for (int q = 0; q < p; ++q) rank += cached[q] == e ? 1 : 0;
            const int at = start[e] + rank;
            sorted[at] = p;
            place[p] = at;
        }
    } else {
        for (int p = threadIdx.x; p < P; p += blockDim.x) {
            const int e = ids[p];
            const int at = start[e] + atomicAdd(&count[e], 1);
            sorted[at] = p;
            place[p] = at;
        }
    }
}

// ----------------------------------------------------------- grouped products
// GLU: w is [E, 2N, K] (gate rows, then up rows); out[row, n] = silu(g) * u in the storage type, rows in sorted
//      order; the input row of sorted row s is token sorted[s] / top.
// else w is [E, N, K]; out[pair, n] = float, the input row is the sorted row itself.
template <typename TX, typename TW, bool GLU>
__global__ void __launch_bounds__(256)
grouped_kernel(const TX* __restrict__ x, long x_stride, const TW* __restrict__ w, void* __restrict__ out_, long out_stride,
               int N, int K, int top, int interleaved, float glu_limit, float glu_slope, const int* __restrict__ offs,
               const int* __restrict__ sorted, const int* __restrict__ tile_expert, const int* __restrict__ tile_row,
               const int* __restrict__ n_tiles) {
    __shared__ float xs[GK][GM + 1];
    __shared__ float ws[GLU ? 2 : 1][GK][GN + 1];
    __shared__ int row_in[GM], row_out[GM];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    if (tile >= n_tiles[0]) return;
    const int e = tile_expert[tile], r0 = tile_row[tile];
    const int rows = min(GM, offs[e + 1] - r0);
    const int n0 = blockIdx.x * GN;
    if (threadIdx.x < GM) {
        const int s = r0 + threadIdx.x;
        const int pair = threadIdx.x < rows ? sorted[s] : 0;
        row_in[threadIdx.x] = GLU ? pair / top : s;
        row_out[threadIdx.x] = GLU ? s : pair;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const TW* we = w + (long)e * (GLU ? 2 : 1) * N * K;
    float acc[GLU ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GM * GK; i += 256) {
            const int r = i / GK, k = i % GK;
            xs[k][r] = (r < rows && k0 + k < K) ? to_float(x[(long)row_in[r] * x_stride + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < GN * GK; i += 256) {
            const int r = i / GK, k = i % GK;
            const int n = n0 + r;
            const bool ok = n < N && k0 + k < K;
            // gate row n and up row n: rows (n, N + n), or (2n, 2n + 1) when the two alternate
            const long g_row = (GLU && interleaved) ? 2L * n : n, u_row = (GLU && interleaved) ? 2L * n + 1 : (long)N + n;
            ws[0][k][r] = ok ? to_float(we[g_row * K + k0 + k]) : 0.f;
            if (GLU) ws[1][k][r] = ok ? to_float(we[u_row * K + k0 + k]) : 0.f;
        }
        __syncthreads();
        const int kmax = min(GK, K - k0);
        for (int k = 0; k < kmax; ++k) {
            const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1];
#pragma unroll
            for (int m = 0; m < (GLU ? 2 : 1); ++m)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float wv = ws[m][k][tx * 4 + j];
                    acc[m][0][j] = fmaf(a0, wv, acc[m][0][j]);
                    acc[m][1][j] = fmaf(a1, wv, acc[m][1][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = ty * 2 + r;
        if (lr >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GLU) {
                const float g = round_to<TX>(acc[0][r][j]), u = round_to<TX>(acc[GLU ? 1 : 0][r][j]);
                ((TX*)out_)[(long)row_out[lr] * out_stride + n] = from_float<TX>(expert_glu(g, u, glu_limit, glu_slope));
            } else {
                ((float*)out_)[(long)row_out[lr] * out_stride + n] = acc[0][r][j];
            }
        }
    }
}

// The same products for steps of few tokens, where an expert has a handful of rows and the time is the time to
// read its weights once: a warp takes a weight row (gate and up rows together), its lanes walk K sixteen bytes at
// a time, and the row meets up to SK_ROWS input rows held in shared memory; a warp-wide sum ends each output.
constexpr int SK_ROWS = 8, SK_WARPS = 8, SK_PER_WARP = 4;      // a block: 32 weight rows (or pairs of them)

template <typename TW> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename TW> __device__ __forceinline__ void load16(const TW* p, float (&f)[Vec16<TW>::N]);
template <> __device__ __forceinline__ void load16<float>(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x; f[2 * i + 1] = v.y;
    }
}

template <typename TX, bool GLU>
__global__ void __launch_bounds__(SK_WARPS * 32)
grouped_skinny_kernel(const TX* __restrict__ x, long x_stride, const TX* __restrict__ w, void* __restrict__ out_,
                      long out_stride, int N, int K, int top, int interleaved, float glu_limit, float glu_slope,
                      const int* __restrict__ offs, const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                      const int* __restrict__ tile_row, const int* __restrict__ n_tiles) {
    extern __shared__ __align__(16) unsigned char sk_raw[];
    TX* xs = reinterpret_cast<TX*>(sk_raw);                     // [SK_ROWS][K]
    __shared__ int row_in[SK_ROWS], row_out[SK_ROWS];
    constexpr int V = Vec16<TX>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    if (tile >= n_tiles[0]) return;
    const int e = tile_expert[tile], r_first = tile_row[tile];
    const int rows_all = min(GM, offs[e + 1] - r_first);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TX* we = w + (long)e * (GLU ? 2 : 1) * N * K;
    for (int r0 = 0; r0 < rows_all; r0 += SK_ROWS) {
        const int rows = min(SK_ROWS, rows_all - r0);
        __syncthreads();                                        // the rows before are done with
        if (threadIdx.x < SK_ROWS) {
            const int s = r_first + r0 + threadIdx.x;
            const int pair = (int)threadIdx.x < rows ? sorted[s] : 0;
            row_in[threadIdx.x] = GLU ? pair / top : s;
            row_out[threadIdx.x] = GLU ? s : pair;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < SK_ROWS * (K / V); i += blockDim.x) {
            const int r = i / (K / V), k = (i % (K / V)) * V;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows) v = *reinterpret_cast<const uint4*>(x + (long)row_in[r] * x_stride + k);
            *reinterpret_cast<uint4*>(xs + (long)r * K + k) = v;
        }
        __syncthreads();
        for (int j = 0; j < SK_PER_WARP; ++j) {
            const int n = (blockIdx.x * SK_WARPS + warp) * SK_PER_WARP + j;
            if (n >= N) break;
            const long g_row = (GLU && interleaved) ? 2L * n : n, u_row = (GLU && interleaved) ? 2L * n + 1 : (long)N + n;
            float acc[GLU ? 2 : 1][SK_ROWS] = {};
            for (int k = lane * V; k < K; k += 32 * V) {
                float wg[V], wu[V];
                load16<TX>(we + g_row * K + k, wg);
                if (GLU) load16<TX>(we + u_row * K + k, wu);
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) {
                    if (r >= rows) break;               // the same for the whole block: a decode step's expert has a row or two
                    float xv[V];
                    load16<TX>(xs + (long)r * K + k, xv);
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        acc[0][r] = fmaf(xv[i], wg[i], acc[0][r]);
                        if (GLU) acc[GLU ? 1 : 0][r] = fmaf(xv[i], wu[i], acc[GLU ? 1 : 0][r]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < SK_ROWS; ++r) {
                if (r >= rows) break;
                const float g = warp_sum(acc[0][r]);
                const float u = GLU ? warp_sum(acc[GLU ? 1 : 0][r]) : 0.f;
                if (lane == 0) {
                    if (GLU) {
                        const float gr = round_to<TX>(g), ur = round_to<TX>(u);
                        ((TX*)out_)[(long)row_out[r] * out_stride + n] = from_float<TX>(expert_glu(gr, ur, glu_limit, glu_slope));
                    } else {
                        ((float*)out_)[(long)row_out[r] * out_stride + n] = g;
                    }
                }
            }
        }
    }
}

// rows[s, :] = x[sorted[s] / top, :]: the tokens' rows in grouped order, for products that want contiguous rows
template <typename T>
__global__ void gather_kernel(const T* __restrict__ x, long x_stride, const int* __restrict__ sorted, int top,
                              T* __restrict__ rows, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const long s = blockIdx.x;
    const T* src = x + (long)(sorted[s] / top) * x_stride;
    T* dst = rows + s * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
}

// out[t, :] (+)= sum_k weights[t, k] * y[row(t * top + k), :], row(p) = p, or place[p] when y is in grouped order.
// ids != null: a pair whose expert is an identity expert (ids[p] >= n_real) adds weights[p] * h[t, :] instead (its row
// of y was never written).  shared != null: float [T, d], the output of an expert that runs for every token, added
// times sigmoid(gate[t * gate_stride]) (gate == null: as it is).
template <typename TH>
__global__ void combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, const int* __restrict__ place,
                               const int* __restrict__ ids, int n_real, const TH* __restrict__ h, long h_stride,
                               const float* __restrict__ shared, const float* __restrict__ gate, long gate_stride,
                               float* __restrict__ out, long total, int d, int top, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / d;
    const int i = (int)(idx % d);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const long p = t * top + k;
        if (ids != nullptr && ids[p] >= n_real) acc = fmaf(weights[p], to_float(h[t * h_stride + i]), acc);
        else acc = fmaf(weights[p], y[(place ? (long)place[p] : p) * d + i], acc);
    }
    if (shared != nullptr) {
        const float g = gate ? 1.0f / (1.0f + expf(-gate[t * gate_stride])) : 1.0f;
        acc = fmaf(g, shared[idx], acc);
    }
    out[idx] = accumulate ? out[idx] + acc : acc;
}

// The same sum, four elements of a row a thread (d a multiple of 4, rows of y, shared and out on 16-byte boundaries):
// a pair's weight, expert and place are read once for the four.  Element by element the same arithmetic in the same order.
template <typename TH>
__global__ void combine_vec_kernel(const float* __restrict__ y, const float* __restrict__ weights, const int* __restrict__ place,
                                   const int* __restrict__ ids, int n_real, const TH* __restrict__ h, long h_stride,
                                   const float* __restrict__ shared, const float* __restrict__ gate, long gate_stride,
                                   float* __restrict__ out, long total4, int d, int top, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int d4 = d >> 2;
    const long t = idx / d4;
    const int i = (int)(idx % d4) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
        const long p = t * top + k;
        const float w = weights[p];
        if (ids != nullptr && ids[p] >= n_real) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(w, to_float(h[t * h_stride + i + e]), acc[e]);
        } else {
            const float4 v = *reinterpret_cast<const float4*>(y + (place ? (long)place[p] : p) * d + i);
            acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
            acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
        }
    }
    if (shared != nullptr) {
        const float g = gate ? 1.0f / (1.0f + expf(-gate[t * gate_stride])) : 1.0f;
        const float4 v = *reinterpret_cast<const float4*>(shared + t * d + i);
        acc[0] = fmaf(g, v.x, acc[0]); acc[1] = fmaf(g, v.y, acc[1]);
        acc[2] = fmaf(g, v.z, acc[2]); acc[3] = fmaf(g, v.w, acc[3]);
    }
    float4* o = reinterpret_cast<float4*>(out + t * d + i);
    if (accumulate) {
        const float4 v = *o;
        acc[0] = v.x + acc[0]; acc[1] = v.y + acc[1]; acc[2] = v.z + acc[2]; acc[3] = v.w + acc[3];
    }
    *o = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

}  // namespace zlm

using namespace zlm;

// z: float [T, E] router logits, or null: then h [T, d] (rows with a stride) and w [E, d] of one storage type are
// given and the logits are taken here; w then has n_extra more rows behind the experts', whose products with the
// token's row go to extra_out [T, n_extra] (float).  z_stride: elements between two rows of z (E, or more when the
// product had further columns).  The chosen scores are multiplied by weight_scale.
ZLM_EXPORT int zlm_moe_route(const float* z, long z_stride, const void* h, int h_dtype, long h_stride, const void* w, int d,
                             const float* correction, int T, int E, int top, int n_groups, int keep_groups,
                             int group_best, int softmax_scores, int renormalize, float weight_scale, int n_extra,
                             float* extra_out, int* ids, float* weights, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || n_groups <= 0 || E % n_groups || keep_groups <= 0 || keep_groups > n_groups ||
        group_best <= 0 || top > keep_groups * (E / n_groups) || (!z && (!h || !w || d <= 0)) || n_extra < 0 ||
        (z && z_stride < E) || (!z && n_extra > 0 && !extra_out))
        return ZLM_ERR_BAD_ARG;
    const size_t smem = (3 * (size_t)E + n_groups + (z ? 0 : d)) * sizeof(float);
    if (smem > 48 * 1024) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e;
    if (z || h_dtype == ZLM_F32)
        e = launch_pdl(route_kernel<float>, dim3(T), dim3(RT_WARPS * 32), smem, stream, z, z_stride, (const float*)h,
                       h_stride, (const float*)w, d, correction, E, top, n_groups, keep_groups, group_best, softmax_scores,
                       renormalize, weight_scale, n_extra, extra_out, ids, weights);
    else if (h_dtype == ZLM_BF16)
        e = launch_pdl(route_kernel<__nv_bfloat16>, dim3(T), dim3(RT_WARPS * 32), smem, stream, z, z_stride,
                       (const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)w, d, correction, E, top, n_groups,
                       keep_groups, group_best, softmax_scores, renormalize, weight_scale, n_extra, extra_out, ids, weights);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// The most tiles P pairs over E experts can make.
ZLM_EXPORT long zlm_moe_max_tiles_scratch(int P, int E) { return (long)(P + GM - 1) / GM + E; }

// place[p]: where pair p stands in ``sorted`` (the inverse of it).  The experts from n_real on are identity experts:
// their pairs are grouped and counted in offs, and get no tiles.
ZLM_EXPORT int zlm_moe_group(const int* ids, int P, int E, int n_real, int* offs, int* sorted, int* place, int* tile_expert,
                             int* tile_row, int* n_tiles, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0 || n_real < 0 || n_real > E) return ZLM_ERR_BAD_ARG;
    const size_t smem = (2 * (size_t)E + 1 + (P <= 1024 ? P : 0)) * sizeof(int);
    if (smem > 48 * 1024) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e = launch_pdl(group_kernel, dim3(1), dim3(1024), smem, stream, ids, P, E, n_real, offs, sorted, place,
                               tile_expert, tile_row, n_tiles);
    return e == cudaSuccess ? launch_status() : (int)e;
}

// glu != 0: x [T, K] (rows by token) -> out [P, N] storage type, sorted order, w [E, 2N, K]
// glu == 0: x [P, K] (sorted order)  -> out [P, N] float, pair order, w [E, N, K]
// interleaved (glu only): gate row n and up row n of an expert are rows 2n and 2n + 1 of its matrix.
// skinny: the step has few tokens; an expert's weights are streamed once against up to 8 rows at a time.
ZLM_EXPORT int zlm_moe_grouped(const void* x, int x_dtype, long x_stride, const void* w, int w_dtype, void* out,
                               long out_stride, int glu, int interleaved, int skinny, int P, int E, int N, int K, int top,
                               float glu_limit, float glu_slope, const int* offs, const int* sorted, const int* tile_expert, const int* tile_row,
                               const int* n_tiles, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0 || N <= 0 || K <= 0 || top <= 0) return ZLM_ERR_BAD_ARG;
    const long max_tiles = zlm_moe_max_tiles_scratch(P, E);
    if (max_tiles > 65535) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e;
    const int el = x_dtype == ZLM_F32 ? 4 : 2;
    const size_t sk_smem = (size_t)SK_ROWS * K * el;
    if (skinny && x_dtype == w_dtype && K % (16 / el) == 0 && x_stride % (16 / el) == 0 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)w % 16 == 0 && sk_smem <= 160 * 1024) {
        dim3 sgrid((N + SK_WARPS * SK_PER_WARP - 1) / (SK_WARPS * SK_PER_WARP), (unsigned)max_tiles);
#define ZLM_SK(TX, GLU)                                                                                              \
    do {                                                                                                             \
        static size_t allowed = 0;                                                                                   \
        if (sk_smem > 48 * 1024 && sk_smem > allowed) {                                                              \
            cudaError_t ea = cudaFuncSetAttribute(grouped_skinny_kernel<TX, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                  160 * 1024);                                                       \
            if (ea != cudaSuccess) return (int)ea;                                                                   \
            allowed = 160 * 1024;                                                                                    \
        }                                                                                                            \
        e = launch_pdl(grouped_skinny_kernel<TX, GLU>, sgrid, dim3(SK_WARPS * 32), sk_smem, stream, (const TX*)x, x_stride, \
                       (const TX*)w, out, out_stride, N, K, top, interleaved, glu_limit, glu_slope, offs, sorted, tile_expert,  \
                       tile_row, n_tiles);                                                                           \
    } while (0)
        if (x_dtype == ZLM_F32) { if (glu) ZLM_SK(float, true); else ZLM_SK(float, false); }
        else { if (glu) ZLM_SK(__nv_bfloat16, true); else ZLM_SK(__nv_bfloat16, false); }
#undef ZLM_SK
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    dim3 grid((N + GN - 1) / GN, (unsigned)max_tiles);
#define ZLM_GR(TX, TW, GLU)                                                                                         \
    e = launch_pdl(grouped_kernel<TX, TW, GLU>, grid, dim3(256), 0, stream, (const TX*)x, x_stride, (const TW*)w, out, \
                   out_stride, N, K, top, interleaved, glu_limit, glu_slope, offs, sorted, tile_expert, tile_row, n_tiles)
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32) { if (glu) ZLM_GR(float, float, true); else ZLM_GR(float, float, false); }
    else if (x_dtype == ZLM_BF16 && w_dtype == ZLM_BF16) { if (glu) ZLM_GR(__nv_bfloat16, __nv_bfloat16, true); else ZLM_GR(__nv_bfloat16, __nv_bfloat16, false); }
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_GR
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_moe_gather(const void* x, int dtype, long x_stride, const int* sorted, int top, void* rows, int P,
                              int d, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (d <= 0 || top <= 0) return ZLM_ERR_BAD_ARG;
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(gather_kernel<float>, dim3(P), dim3(256), 0, stream, (const float*)x, x_stride, sorted, top, (float*)rows, d);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(gather_kernel<__nv_bfloat16>, dim3(P), dim3(256), 0, stream, (const __nv_bfloat16*)x, x_stride, sorted,
                       top, (__nv_bfloat16*)rows, d);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// place: null when row p of y is pair p; else y is in grouped order and place[p] is pair p's row.  ids (with n_real,
// h, h_dtype, h_stride): the pairs of identity experts add the token's row of h.  shared / gate / gate_stride: an
// output for every token, added times the sigmoid of one number a token.
ZLM_EXPORT int zlm_moe_combine(const float* y, const float* weights, const int* place, const int* ids, int n_real,
                               const void* h, int h_dtype, long h_stride, const float* shared, const float* gate,
                               long gate_stride, float* out, int T, int d, int top, int accumulate, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || top <= 0 || (ids != nullptr && h == nullptr)) return ZLM_ERR_BAD_ARG;
    const long total = (long)T * d;
    cudaError_t e;
    if (d % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)shared % 16 == 0) {
        const long total4 = total / 4;
        const unsigned blocks = (unsigned)((total4 + 255) / 256);
        if (h_dtype == ZLM_BF16 && ids != nullptr)
            e = launch_pdl(combine_vec_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, y, weights, place, ids, n_real,
                           (const __nv_bfloat16*)h, h_stride, shared, gate, gate_stride, out, total4, d, top, accumulate);
        else
            e = launch_pdl(combine_vec_kernel<float>, dim3(blocks), dim3(256), 0, stream, y, weights, place, ids, n_real,
                           (const float*)h, h_stride, shared, gate, gate_stride, out, total4, d, top, accumulate);
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    if (h_dtype == ZLM_BF16 && ids != nullptr)
        e = launch_pdl(combine_kernel<__nv_bfloat16>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, y, weights,
                       place, ids, n_real, (const __nv_bfloat16*)h, h_stride, shared, gate, gate_stride, out, total, d, top,
                       accumulate);
    else
        e = launch_pdl(combine_kernel<float>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, y, weights, place,
                       ids, n_real, (const float*)h, h_stride, shared, gate, gate_stride, out, total, d, top, accumulate);
    return e == cudaSuccess ? launch_status() : (int)e;
}
