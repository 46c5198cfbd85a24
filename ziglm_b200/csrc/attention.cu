// Rotary positions, cache writes and attention over the paged cache: the plain
// kernels that take every head size (a multiple of 8), every number of heads
// and groups, both storage types, prompts, continued prompts and single decoded
// tokens alike.  They are the whole 32-bit path and the fallback of the bf16
// path for head sizes the tensor-core kernels do not cover.
//
// Formulas, as the reference computes them:
//   RoPE     pairs (i, i+rot/2) inside a head: theta = pos*inv_freq[i],
//            h[i]       = a*cos(theta) - b*sin(theta)
//            h[i+rot/2] = a*sin(theta) + b*cos(theta)
//            (src/model.zig:569-597,642-653; src/cuda_bridge.cu:2070-2108)
//            inv_freq comes from a table built once from the configuration (the
//            reference recomputes 1/powf(base, 2i/rot) per thread and ignores the
//            configured base, src/model.zig:405-413).
//   cache    keys are stored rotated (src/model.zig:655, src/kv_cache.zig:63-85)
//   scores   kvh = h / (n_heads/n_kv_heads); s_t = (q_h . K[t,kvh]) * scale
//            (src/model.zig:554,659-678)
//   mask     a token at position p sees keys [start, p], start = 0 or
//            p-window+1 (src/model.zig:660-661); nothing is materialised
//   softmax  m = max s, e = exp(s-m), p = e/sum e in float (src/math.zig:1088-1106)
//   values   o_h = sum_t p_t V[t,kvh,:] (src/model.zig:683-700)
//
// Cache layout: pages of `page_size` positions.  Page p of one layer holds
// [n_kv_heads][page_size][head_dim] for keys and the same for values.  A step
// gives each of its sequences a row of page numbers (`block_table`), so position
// t of sequence b lives in page block_table[b*bt_stride + t/page_size], row
// t%page_size.
#include "common.cuh"

namespace zlm {

// ------------------------------------------------------- rope + cache write
// One block per token.  The cosines and sines of the token's position are formed once in shared
// memory (float32 angles), then the threads walk the heads: q and k heads are rotated in place,
// k (rotated) and v heads are copied to the token's row of the cache pages.
// qkv row layout: [q: n_heads*hd | k: n_kv*hd | v: n_kv*hd]
constexpr int ROPE_MAX_HALF = 256;
constexpr int ATT_MAX_HD_ROPE = 512;     // the largest head the norming rotation takes

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
                                  const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                  int bt_stride, T* __restrict__ k_pages, T* __restrict__ v_pages, int page_size,
                                  long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot / 2;
    const bool have_table = inv_freq != nullptr && half > 0;
    if (have_table) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float theta = (float)pos * inv_freq[i];
            sincosf(theta, &sin_s[i], &cos_s[i]);
        }
    }
    __syncthreads();
    T* row0 = qkv + (long)t * row_stride;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;       // head h of the cache row lies h * page_size * hd further
        vdst = v_pages + off;
    }
    const long kv_head_stride = (long)page_size * hd;
    // this block's share of the heads, counted over q heads, k heads, v heads in that order
    const int total_heads = n_heads + n_kv + (v_pages != nullptr ? n_kv : 0);   // no value pages: the rows hold no value heads
    const int per = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per, h_hi = min(total_heads, h_lo + per);
    const int rot_hi = min(h_hi, n_heads + n_kv);            // heads below this one are rotated
    if (have_table && rot_hi > h_lo) {
        for (int idx = threadIdx.x; idx < (rot_hi - h_lo) * half; idx += blockDim.x) {
            const int head = h_lo + idx / half, i = idx % half;
            T* row = row0 + (long)head * hd;
            const float a = to_float(row[i]);
            const float b2 = to_float(row[i + half]);
            const float c = cos_s[i], sn = sin_s[i];
            const T lo = from_float<T>(a * c - b2 * sn);
            const T hi = from_float<T>(a * sn + b2 * c);
            row[i] = lo;
            row[i + half] = hi;
            if (kdst && head >= n_heads) {
                T* d = kdst + (long)(head - n_heads) * kv_head_stride;
                d[i] = lo;
                d[i + half] = hi;
            }
        }
    }
    if (kdst) {
        // what the rotation left alone of the k heads (everything when there is no table), and the v heads
        const int k_first = have_table ? rot : 0;
        const int k_rest = hd - k_first;
        const int k_lo = max(h_lo, n_heads), k_hi = rot_hi;
        for (int idx = threadIdx.x; idx < (k_hi - k_lo) * k_rest; idx += blockDim.x) {
            const int h = k_lo - n_heads + idx / k_rest, i = k_first + idx % k_rest;
            kdst[(long)h * kv_head_stride + i] = row0[(long)(n_heads + h) * hd + i];
        }
        const int v_lo = max(h_lo, n_heads + n_kv);
        for (int idx = threadIdx.x; idx < (h_hi - v_lo) * hd; idx += blockDim.x) {
            const int h = v_lo - n_heads - n_kv + idx / hd, i = idx % hd;
            vdst[(long)h * kv_head_stride + i] = row0[(long)(n_heads + n_kv + h) * hd + i];
        }
    }
}

// The same for bf16 rows whose heads, halves and strides are multiples of 8 elements: a thread moves
// 16 bytes at a time (8 pairs of the rotation, or 8 elements of a copy), which is what a prompt of
// thousands of tokens needs to run at memory speed.  Same arithmetic, element by element.
__global__ void rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd,
                                      int rot, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                      int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                                      __nv_bfloat16* __restrict__ v_pages, int page_size, long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];                       // positions, tables and frequencies are older than the step
    const int half = rot / 2;
    const bool have_table = inv_freq != nullptr && half > 0;
    if (have_table)
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;
        vdst = v_pages + off;
    }
    __syncthreads();
    pdl_wait();
    __nv_bfloat16* row0 = qkv + (long)t * row_stride;
    const long kv_head_stride = (long)page_size * hd;
    const int total_heads = n_heads + n_kv + (v_pages != nullptr ? n_kv : 0);   // no value pages: the rows hold no value heads
    const int per = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per, h_hi = min(total_heads, h_lo + per);
    const int rot_hi = min(h_hi, n_heads + n_kv);
    if (have_table && rot_hi > h_lo) {
        const int units = half / 8;
        for (int idx = threadIdx.x; idx < (rot_hi - h_lo) * units; idx += blockDim.x) {
            const int head = h_lo + idx / units, i0 = (idx % units) * 8;
            __nv_bfloat16* row = row0 + (long)head * hd;
            uint4 lo = *reinterpret_cast<const uint4*>(row + i0);
            uint4 hi = *reinterpret_cast<const uint4*>(row + i0 + half);
            __nv_bfloat162* lp = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x = __bfloat1622float2(lp[k]), y = __bfloat1622float2(hp[k]);
                const float c0 = cos_s[i0 + 2 * k], s0 = sin_s[i0 + 2 * k];
                const float c1 = cos_s[i0 + 2 * k + 1], s1 = sin_s[i0 + 2 * k + 1];
                lp[k] = __halves2bfloat162(__float2bfloat16_rn(x.x * c0 - y.x * s0), __float2bfloat16_rn(x.y * c1 - y.y * s1));
                hp[k] = __halves2bfloat162(__float2bfloat16_rn(x.x * s0 + y.x * c0), __float2bfloat16_rn(x.y * s1 + y.y * c1));
            }
            *reinterpret_cast<uint4*>(row + i0) = lo;
            *reinterpret_cast<uint4*>(row + i0 + half) = hi;
            if (kdst && head >= n_heads) {
                __nv_bfloat16* d = kdst + (long)(head - n_heads) * kv_head_stride;
                *reinterpret_cast<uint4*>(d + i0) = lo;
                *reinterpret_cast<uint4*>(d + i0 + half) = hi;
            }
        }
    }
    if (kdst) {
        const int k_first = have_table ? rot : 0;
        const int k_units = (hd - k_first) / 8;
        const int k_lo = max(h_lo, n_heads), k_hi = rot_hi;
        for (int idx = threadIdx.x; idx < (k_hi - k_lo) * k_units; idx += blockDim.x) {
            const int h = k_lo - n_heads + idx / k_units, i = k_first + (idx % k_units) * 8;
            *reinterpret_cast<uint4*>(kdst + (long)h * kv_head_stride + i) =
                *reinterpret_cast<const uint4*>(row0 + (long)(n_heads + h) * hd + i);
        }
        const int v_lo = max(h_lo, n_heads + n_kv), v_units = hd / 8;
        for (int idx = threadIdx.x; idx < (h_hi - v_lo) * v_units; idx += blockDim.x) {
            const int h = v_lo - n_heads - n_kv + idx / v_units, i = (idx % v_units) * 8;
            *reinterpret_cast<uint4*>(vdst + (long)h * kv_head_stride + i) =
                *reinterpret_cast<const uint4*>(row0 + (long)(n_heads + n_kv + h) * hd + i);
        }
    }
}

// Rotation with an amplitude, a unit RMS norm of every rotated query and key head, and the cache write.
// One warp per head at a time: the head is read into shared memory as floats, its first `rot` dimensions are
// turned (cosines and sines times `amplitude`), the head is divided by sqrt(mean over its first norm_dim
// dimensions of its squares + norm_eps) when norm_dim > 0, and written back (keys also to the cache).  Value
// heads are copied to the cache.  Everything between the read and the write is float.
constexpr int RNS_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(RNS_WARPS * 32)
rope_norm_store_kernel(T* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
                       const float* __restrict__ inv_freq, float amplitude, int norm_dim, float norm_eps,
                       int norm_first, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                       const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pages,
                       T* __restrict__ v_pages, int page_size, long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    __shared__ float head_s[RNS_WARPS][ATT_MAX_HD_ROPE];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot / 2;
    const bool turn = inv_freq != nullptr && half > 0;
    if (turn) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sin_s[i] = sn * amplitude;
            cos_s[i] = cs * amplitude;
        }
    }
    __syncthreads();
    T* row0 = qkv + (long)t * row_stride;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;
        vdst = v_pages + off;
    }
    const long kv_head_stride = (long)page_size * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total_heads = n_heads + 2 * n_kv;
    const int per = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per, h_hi = min(total_heads, h_lo + per);
    float* hs = head_s[warp];
    for (int head = h_lo + warp; head < h_hi; head += RNS_WARPS) {
        T* row = row0 + (long)head * hd;
        if (head >= n_heads + n_kv) {
            if (vdst) {
                T* d = vdst + (long)(head - n_heads - n_kv) * kv_head_stride;
                for (int i = lane; i < hd; i += 32) d[i] = row[i];
            }
            continue;
        }
        for (int i = lane; i < hd; i += 32) hs[i] = to_float(row[i]);
        __syncwarp();
        float ss = 0.f;
        if (norm_first && norm_dim > 0) {
            // the norm stands before the rotation and has a weight that all heads of a kind share
            for (int i = lane; i < norm_dim; i += 32) ss = fmaf(hs[i], hs[i], ss);
            ss = warp_sum(ss);
            const float inv0 = 1.0f / sqrtf(ss / (float)norm_dim + norm_eps);
            const float* w = head < n_heads ? q_weight : k_weight;
            for (int i = lane; i < norm_dim; i += 32) hs[i] = (hs[i] * inv0) * (w ? w[i] : 1.0f);
            __syncwarp();
            ss = 0.f;
        }
        float vals[ATT_MAX_HD_ROPE / 32];
#pragma unroll
        for (int r = 0; r < ATT_MAX_HD_ROPE / 32; ++r) {
            const int i = lane + 32 * r;
            float v = 0.f;
            if (i < hd) {
                v = hs[i];
                if (turn && i < half) v = v * cos_s[i] - hs[i + half] * sin_s[i];
                else if (turn && i < rot) v = v * cos_s[i - half] + hs[i - half] * sin_s[i - half];
                if (i < norm_dim) ss = fmaf(v, v, ss);
            }
            vals[r] = v;
        }
        float inv = 1.0f;
        if (norm_dim > 0 && !norm_first) {
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)norm_dim + norm_eps);
        }
        T* d = (kdst && head >= n_heads) ? kdst + (long)(head - n_heads) * kv_head_stride : nullptr;
#pragma unroll
        for (int r = 0; r < ATT_MAX_HD_ROPE / 32; ++r) {
            const int i = lane + 32 * r;
            if (i < hd) {
                const T o = from_float<T>(vals[r] * inv);
                row[i] = o;
                if (d) d[i] = o;
            }
        }
        __syncwarp();
    }
}

// The same for bf16 rows whose heads, rotated halves and strides are multiples of 8 elements: a thread moves 16
// bytes at a time.  A head is shared by LPH lanes of a warp (a power of two that covers its units: rot/16 units of
// 8 pairs of the rotation, then (hd - rot)/8 units of 8 elements that pass), so a warp works on 32/LPH heads at
// once and the sum of squares is folded over those lanes alone.  Same arithmetic, element by element.
__global__ void __launch_bounds__(RNS_WARPS * 32)
rope_norm_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
                           const float* __restrict__ inv_freq, float amplitude, int norm_dim, float norm_eps,
                           int norm_first, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                           const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                           __nv_bfloat16* __restrict__ v_pages, int page_size, long page_stride, int lph) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];                       // positions, tables and frequencies are older than the step
    const int half = rot / 2;
    const bool turn = inv_freq != nullptr && half > 0;
    if (turn) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sin_s[i] = sn * amplitude;
            cos_s[i] = cs * amplitude;
        }
    }
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;
        vdst = v_pages + off;
    }
    __syncthreads();
    pdl_wait();
    __nv_bfloat16* row0 = qkv + (long)t * row_stride;
    const long kv_head_stride = (long)page_size * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units_rot = turn ? rot / 16 : 0;
    const int first_tail = turn ? rot : 0;
    const int units = units_rot + (hd - first_tail) / 8;
    const int hpw = 32 / lph;                                   // heads a warp holds at once
    const int total_qk = n_heads + n_kv;
    const int sub = lane % lph;
    for (int head0 = (blockIdx.y * RNS_WARPS + warp) * hpw; head0 < total_qk; head0 += gridDim.y * RNS_WARPS * hpw) {
        const int head = head0 + lane / lph;
        const bool active = head < total_qk && sub < units;
        const bool pair = active && sub < units_rot;
        __nv_bfloat16* row = row0 + (long)head * hd;
        const int i0 = pair ? sub * 8 : first_tail + (sub - units_rot) * 8;
        float a[8], b[8];
        float ss = 0.f;
        if (active) {
            const uint4 lo = *reinterpret_cast<const uint4*>(row + i0);
            const __nv_bfloat162* lp = reinterpret_cast<const __nv_bfloat162*>(&lo);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x = __bfloat1622float2(lp[k]);
                a[2 * k] = x.x; a[2 * k + 1] = x.y;
            }
            if (pair) {
                const uint4 hi = *reinterpret_cast<const uint4*>(row + i0 + half);
                const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hi);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 y = __bfloat1622float2(hp[k]);
                    b[2 * k] = y.x; b[2 * k + 1] = y.y;
                }
            }
        }
        if (norm_first && norm_dim > 0) {
            // the norm stands before the rotation and has a weight that all heads of a kind share
            if (active) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (i0 + k < norm_dim) ss = fmaf(a[k], a[k], ss);
                    if (pair && i0 + half + k < norm_dim) ss = fmaf(b[k], b[k], ss);
                }
            }
            for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv0 = 1.0f / sqrtf(ss / (float)norm_dim + norm_eps);
            if (active) {
                const float* w = head < n_heads ? q_weight : k_weight;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (i0 + k < norm_dim) a[k] = (a[k] * inv0) * (w ? w[i0 + k] : 1.0f);
                    if (pair && i0 + half + k < norm_dim) b[k] = (b[k] * inv0) * (w ? w[i0 + half + k] : 1.0f);
                }
            }
            ss = 0.f;
        }
        if (active) {
            if (pair) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float c = cos_s[i0 + k], sn = sin_s[i0 + k];
                    const float u = a[k], v = b[k];
                    a[k] = u * c - v * sn;
                    b[k] = v * c + u * sn;
                    if (i0 + half + k < norm_dim) ss = fmaf(b[k], b[k], ss);
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (i0 + k < norm_dim) ss = fmaf(a[k], a[k], ss);
        }
        float inv = 1.0f;
        if (norm_dim > 0 && !norm_first) {
            for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            inv = 1.0f / sqrtf(ss / (float)norm_dim + norm_eps);
        }
        if (active) {
            __nv_bfloat16* d = (kdst && head >= n_heads) ? kdst + (long)(head - n_heads) * kv_head_stride : nullptr;
            uint4 lo;
            __nv_bfloat162* lp = reinterpret_cast<__nv_bfloat162*>(&lo);
#pragma unroll
            for (int k = 0; k < 4; ++k) lp[k] = __floats2bfloat162_rn(a[2 * k] * inv, a[2 * k + 1] * inv);
            *reinterpret_cast<uint4*>(row + i0) = lo;
            if (d) *reinterpret_cast<uint4*>(d + i0) = lo;
            if (pair) {
                uint4 hi;
                __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
                for (int k = 0; k < 4; ++k) hp[k] = __floats2bfloat162_rn(b[2 * k] * inv, b[2 * k + 1] * inv);
                *reinterpret_cast<uint4*>(row + i0 + half) = hi;
                if (d) *reinterpret_cast<uint4*>(d + i0 + half) = hi;
            }
        }
    }
    if (vdst) {
        const int v_units = hd / 8;
        const int n_threads = gridDim.y * blockDim.x;
        for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < n_kv * v_units; idx += n_threads) {
            const int h = idx / v_units, i = (idx % v_units) * 8;
            *reinterpret_cast<uint4*>(vdst + (long)h * kv_head_stride + i) =
                *reinterpret_cast<const uint4*>(row0 + (long)(total_qk + h) * hd + i);
        }
    }
}

// ------------------------------------------------------------ attention
// The keys a token sees, [start, pos], are cut into parts of ATT_PART = 256 consecutive keys counted from
// `start`.  Within a part warp w of a block takes the key blocks w and w + 4 of 32 keys: lane j scores key j of
// a block, then the lanes split the head's dimensions for the weighted sum of values; the four warps' partial
// results are merged in warp order into the part's (max, sum, weighted values).  The parts are then folded one
// after another, in ascending order, into the result.  A block works for G query heads that share a key/value
// head (the largest of 4, 2, 1 that divides the group), so a key or value row is read once for all of them.
//
// Two ways to run, with bit-for-bit the same result, because a part's result depends on (start, pos, part)
// alone and the fold is the same arithmetic in the same order:
//   whole   grid (T, n_heads / G, 1): a block computes and folds all parts of its token (prompts: the tokens
//           alone give enough blocks);
//   split   grid (T, n_heads / G, parts): a block computes one part and stores it in scratch memory, and
//           attention_fold_kernel folds a token's parts (steps of few tokens: the parts give the blocks).
constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 512;
constexpr int ATT_PART = ATT_WARPS * 2 * 32;

// k[d..d+VEC) of one key row as floats
template <typename T, int VEC> __device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&f)[VEC]);
template <> __device__ __forceinline__ void load_vec<float, 4>(const float* __restrict__ p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* __restrict__ p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x; f[2 * i + 1] = v.y;
    }
}

// Fold a part (mp, lp, op) into the running (m, l, o): every operation is one rounded multiply, add or fused
// multiply-add, written out so that both kernels that fold do exactly the same.
__device__ __forceinline__ void fold_weights(float m, float mp, float& m_new, float& a, float& b) {
    m_new = fmaxf(m, mp);
    a = expf(m - m_new);                 // exp(-inf) = 0 for the first part
    b = expf(mp - m_new);
}
__device__ __forceinline__ float fold_value(float o, float a, float op, float b) {
    return __fmaf_rn(op, b, __fmul_rn(o, a));
}

template <typename T, int VEC, int G, int NREG>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_general_kernel(const T* __restrict__ q, long q_row_stride, T* __restrict__ out, int n_heads, int n_kv,
                         int hd, float scale, float softcap, int window, int keep_first,
                         const float* __restrict__ sinks, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages, int page_size,
                         long page_stride, float* __restrict__ part_ml, float* __restrict__ part_o, int max_parts) {
    __shared__ float q_s[G][ATT_MAX_HD];
    __shared__ float acc_s[G][ATT_WARPS][NREG * 32];
    __shared__ float m_s[G][ATT_WARPS], l_s[G][ATT_WARPS];

    const int t = blockIdx.x, h0 = blockIdx.y * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int b = seq_of_token[t];
    const int kvh = h0 / (n_heads / n_kv);
    const int start = first_visible_key(pos, window);
    // the keys a token sees, counted through: the first tokens a window keeps (those before the window), then the window
    const int kept = min(keep_first, start);
    const int n_keys = kept + pos - start + 1;
    const int n_parts = (n_keys + ATT_PART - 1) / ATT_PART;
    const bool split = part_o != nullptr;
    const int p_lo = split ? (int)blockIdx.z : 0, p_hi = split ? min(n_parts, (int)blockIdx.z + 1) : n_parts;
    if (p_lo >= n_parts) return;
    const int* bt = block_table + (long)b * bt_stride;

    for (int i = threadIdx.x; i < G * hd; i += blockDim.x)
        q_s[i / hd][i % hd] = to_float(q[(long)t * q_row_stride + (long)(h0 + i / hd) * hd + i % hd]);
    __syncthreads();

    // the running result: thread x owns dimensions x, x + 128, ... of every head
    constexpr int NRUN = NREG / 4;
    float run_m[G], run_l[G], run_o[G][NRUN];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        run_m[g] = -INFINITY; run_l[g] = 0.f;
#pragma unroll
        for (int r = 0; r < NRUN; ++r) run_o[g][r] = 0.f;
    }

    for (int part = p_lo; part < p_hi; ++part) {
        float acc[G][NREG], m[G], l[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
            for (int i = 0; i < NREG; ++i) acc[g][i] = 0.f;
        }
        const int part_first = part * ATT_PART;
#pragma unroll 1
        for (int kb = warp; kb < 2 * ATT_WARPS; kb += ATT_WARPS) {
            const int first = part_first + kb * 32;
            if (first >= n_keys) break;                          // uniform per warp
            const bool valid = first + lane < n_keys;
            const int j = first + lane < kept ? first + lane : start + (first + lane - kept);
            float sc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) sc[g] = 0.f;
            long row_off = 0;
            if (valid) {
                const int page = bt[j / page_size];
                row_off = (long)page * page_stride + ((long)kvh * page_size + j % page_size) * hd;
                const T* krow = k_pages + row_off;
                // several 16-byte loads of the row in flight at once: the loop is bound by their latency
#pragma unroll 8
                for (int d = 0; d < hd; d += VEC) {
                    float kv[VEC];
                    load_vec<T, VEC>(krow + d, kv);
#pragma unroll
                    for (int g = 0; g < G; ++g)
#pragma unroll
                        for (int i = 0; i < VEC; ++i) sc[g] = fmaf(q_s[g][d + i], kv[i], sc[g]);
                }
            }
            float pr[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float sv = sc[g] * scale;
                if (softcap > 0.f) sv = softcap * tanhf(sv / softcap);       // a soft cap: scores stay inside (-cap, cap)
                if (!valid) sv = -INFINITY;
                const float m_new = fmaxf(m[g], warp_max(sv));   // lane 0 of the block is always valid
                const float corr = expf(m[g] - m_new);           // exp(-inf) = 0 on the first block
                pr[g] = valid ? expf(sv - m_new) : 0.f;
                l[g] = l[g] * corr + warp_sum(pr[g]);
                m[g] = m_new;
#pragma unroll
                for (int i = 0; i < NREG; ++i) acc[g][i] *= corr;
            }
            const int n_valid = min(32, n_keys - first);
#pragma unroll 4
            for (int jj = 0; jj < n_valid; ++jj) {
                const long voff = __shfl_sync(0xffffffffu, row_off, jj);
                const T* vrow = v_pages + voff;
                float pj[G];
#pragma unroll
                for (int g = 0; g < G; ++g) pj[g] = __shfl_sync(0xffffffffu, pr[g], jj);
#pragma unroll
                for (int i = 0; i < NREG; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) {
                        const float v = to_float(vrow[d]);
#pragma unroll
                        for (int g = 0; g < G; ++g) acc[g][i] = fmaf(pj[g], v, acc[g][i]);
                    }
                }
            }
        }
        __syncthreads();                                         // the part before has been folded
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (lane == 0) { m_s[g][warp] = m[g]; l_s[g][warp] = l[g]; }
#pragma unroll
            for (int i = 0; i < NREG; ++i) acc_s[g][warp][lane + 32 * i] = acc[g][i];
        }
        __syncthreads();
        // the four warps' results, merged in warp order: the part's (max, sum, weighted values)
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float big = -INFINITY;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) big = fmaxf(big, m_s[g][w]);
            float wgt[ATT_WARPS];
            float lp = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) {
                wgt[w] = m_s[g][w] == -INFINITY ? 0.f : expf(m_s[g][w] - big);
                lp = __fmaf_rn(l_s[g][w], wgt[w], lp);
            }
            float a, bb, m_new;
            fold_weights(run_m[g], big, m_new, a, bb);
#pragma unroll
            for (int r = 0; r < NRUN; ++r) {
                const int d = threadIdx.x + r * ATT_WARPS * 32;
                if (d < hd) {
                    float op = 0.f;
#pragma unroll
                    for (int w = 0; w < ATT_WARPS; ++w) op = __fmaf_rn(acc_s[g][w][d], wgt[w], op);
                    if (split) part_o[(((long)t * n_heads + h0 + g) * max_parts + part) * hd + d] = op;
                    else run_o[g][r] = fold_value(run_o[g][r], a, op, bb);
                }
            }
            if (split) {
                if (threadIdx.x == 0) {
                    float* ml = part_ml + (((long)t * n_heads + h0 + g) * max_parts + part) * 2;
                    ml[0] = big; ml[1] = lp;
                }
            } else {
                run_l[g] = fold_value(run_l[g], a, lp, bb);
                run_m[g] = m_new;
            }
        }
    }
    if (split) return;
    if (sinks != nullptr) {
        // a number in the softmax's denominator that belongs to no key: one more fold, with no values
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float a, bb, m_new;
            fold_weights(run_m[g], sinks[h0 + g], m_new, a, bb);
#pragma unroll
            for (int r = 0; r < NRUN; ++r) run_o[g][r] = fold_value(run_o[g][r], a, 0.f, bb);
            run_l[g] = fold_value(run_l[g], a, 1.0f, bb);
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int r = 0; r < NRUN; ++r) {
            const int d = threadIdx.x + r * ATT_WARPS * 32;
            if (d < hd) out[((long)t * n_heads + h0 + g) * hd + d] = from_float<T>(run_o[g][r] / run_l[g]);
        }
}

// grid (T, n_heads), 128 threads: folds the parts a split launch left in scratch memory, in ascending order.
template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_fold_kernel(T* __restrict__ out, int n_heads, int hd, int window, int keep_first,
                      const float* __restrict__ sinks, const int* __restrict__ positions,
                      const float* __restrict__ part_ml, const float* __restrict__ part_o, int max_parts) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int pos = positions[t];
    const int start = first_visible_key(pos, window);
    const int n_parts = (min(keep_first, start) + pos - start + 1 + ATT_PART - 1) / ATT_PART;
    const float* ml = part_ml + ((long)t * n_heads + h) * max_parts * 2;
    const float* po = part_o + ((long)t * n_heads + h) * max_parts * hd;
    constexpr int NRUN = ATT_MAX_HD / (ATT_WARPS * 32);
    float run_m = -INFINITY, run_l = 0.f, run_o[NRUN] = {};
    for (int part = 0; part < n_parts; ++part) {
        float a, bb, m_new;
        fold_weights(run_m, ml[2 * part], m_new, a, bb);
#pragma unroll
        for (int r = 0; r < NRUN; ++r) {
            const int d = threadIdx.x + r * ATT_WARPS * 32;
            if (d < hd) run_o[r] = fold_value(run_o[r], a, po[(long)part * hd + d], bb);
        }
        run_l = fold_value(run_l, a, ml[2 * part + 1], bb);
        run_m = m_new;
    }
    if (sinks != nullptr) {
        float a, bb, m_new;
        fold_weights(run_m, sinks[h], m_new, a, bb);
#pragma unroll
        for (int r = 0; r < NRUN; ++r) run_o[r] = fold_value(run_o[r], a, 0.f, bb);
        run_l = fold_value(run_l, a, 1.0f, bb);
    }
#pragma unroll
    for (int r = 0; r < NRUN; ++r) {
        const int d = threadIdx.x + r * ATT_WARPS * 32;
        if (d < hd) out[((long)t * n_heads + h) * hd + d] = from_float<T>(run_o[r] / run_l);
    }
}

template <typename T, int VEC, int G>
static int launch_attention(const void* q, long q_row_stride, void* out, int T_, int n_heads, int n_kv, int hd, float scale,
                            float softcap, int window, int keep_first, const float* sinks, const int* positions,
                            const int* seq_of_token, const int* block_table,
                            int bt_stride, const void* k_pages, const void* v_pages, int page_size, long page_stride,
                            float* part_ml, float* part_o, int max_parts, cudaStream_t stream) {
    dim3 grid(T_, n_heads / G, part_o ? max_parts : 1);
#define ZLM_ATT_GO(NREG)                                                                                              \
    attention_general_kernel<T, VEC, G, NREG><<<grid, ATT_WARPS * 32, 0, stream>>>(                                     \
        (const T*)q, q_row_stride, (T*)out, n_heads, n_kv, hd, scale, softcap, window, keep_first, sinks, positions, seq_of_token, block_table, \
        bt_stride, (const T*)k_pages, (const T*)v_pages, page_size, page_stride, part_ml, part_o, max_parts)
    if (hd <= 128) ZLM_ATT_GO(4);
    else if (hd <= 256) ZLM_ATT_GO(8);
    else ZLM_ATT_GO(16);
#undef ZLM_ATT_GO
    int rc = launch_status();
    if (rc || !part_o) return rc;
    attention_fold_kernel<T><<<dim3(T_, n_heads), ATT_WARPS * 32, 0, stream>>>((T*)out, n_heads, hd, window, keep_first, sinks,
                                                                           positions, part_ml, part_o, max_parts);
    return launch_status();
}

template <typename T, int VEC>
static int pick_group(int group, const void* q, long q_row_stride, void* out, int T_, int n_heads, int n_kv, int hd,
                      float scale, float softcap, int window, int keep_first, const float* sinks, const int* positions,
                      const int* seq_of_token, const int* block_table,
                      int bt_stride, const void* k_pages, const void* v_pages, int page_size, long page_stride,
                      float* part_ml, float* part_o, int max_parts, cudaStream_t stream) {
#define ZLM_ATT(GV)                                                                                                     \
    launch_attention<T, VEC, GV>(q, q_row_stride, out, T_, n_heads, n_kv, hd, scale, softcap, window, keep_first, sinks, positions, seq_of_token, \
                                 block_table, bt_stride, k_pages, v_pages, page_size, page_stride, part_ml, part_o,     \
                                 max_parts, stream)
    if (group % 4 == 0 && hd <= 256) return ZLM_ATT(4);
    if (group % 2 == 0) return ZLM_ATT(2);
    return ZLM_ATT(1);
#undef ZLM_ATT
}

// What stands between the q|k|v product and attention in a mixer whose q and k are normed as whole vectors: one
// block per token.  In order: (1) with norm weights, q (all heads as one vector) and k (likewise) are each divided by
// the root of (their mean square + eps) and multiplied by their weight, element by element; n_q / n_k are the counts
// the means are taken over (heads kept with zeros behind them have fewer true elements than hd a head); (2) the first
// `rot` dimensions of every q and k head are turned by the token's position, pairs (i, i + rot/2); (3) the values are
// mixed with those another layer left for the same tokens, v <- (1 - mix) v + mix v_other (mix_mode 2), or left there
// for later layers (mix_mode 1); (4) q, k, v are written back and k, v stored in the cache pages.  Everything between
// the read and the write is float.
// Rows: [q: n_heads*hd | k: n_kv*hd | v: n_kv*hd | anything else]; mix_buf: [T, n_kv*v_dim] contiguous, in the rows'
// type: the first v_dim elements of every value head (the rest of a head is zeros it is kept with).
template <typename T>
__global__ void __launch_bounds__(256)
qk_prep_kernel(T* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
               const float* __restrict__ inv_freq, const float* __restrict__ q_w, const float* __restrict__ k_w,
               int n_q, int n_k, float norm_eps, int mix_mode, float mix, T* __restrict__ mix_buf, int v_dim,
               const int* __restrict__ positions, const int* __restrict__ seq_of_token,
               const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
               int page_size, long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot / 2;
    const bool turn = inv_freq != nullptr && half > 0;
    if (turn)
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
    T* row0 = qkv + (long)t * row_stride;
    const int q_len = n_heads * hd, k_len = n_kv * hd;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_len; i += blockDim.x) { const float v = to_float(row0[i]); ss = fmaf(v, v, ss); }
        inv_q = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n_q + norm_eps);
    }
    if (k_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < k_len; i += blockDim.x) { const float v = to_float(row0[q_len + i]); ss = fmaf(v, v, ss); }
        inv_k = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n_k + norm_eps);
    }
    __syncthreads();
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;       // head h of the cache row lies h * page_size * hd further
        vdst = v_pages + off;
    }
    const long kv_head_stride = (long)page_size * hd;
    const int qk_heads = n_heads + n_kv;
    if (turn) {
        for (int idx = threadIdx.x; idx < qk_heads * half; idx += blockDim.x) {
            const int head = idx / half, i = idx - head * half;
            const bool is_k = head >= n_heads;
            const int at = head * hd + i;                   // q and k heads lie one behind the other
            float a = to_float(row0[at]), b2 = to_float(row0[at + half]);
            const float* w = is_k ? k_w : q_w;
            if (w != nullptr) {
                const int wi = at - (is_k ? q_len : 0);
                const float inv = is_k ? inv_k : inv_q;
                a = (a * inv) * w[wi];
                b2 = (b2 * inv) * w[wi + half];
            }
            const float c = cos_s[i], sn = sin_s[i];
            const T lo = from_float<T>(a * c - b2 * sn), hi = from_float<T>(b2 * c + a * sn);
            row0[at] = lo;
            row0[at + half] = hi;
            if (kdst && is_k) {
                T* d = kdst + (long)(head - n_heads) * kv_head_stride;
                d[i] = lo;
                d[i + half] = hi;
            }
        }
    }
    const int first_rest = turn ? rot : 0, rest = hd - first_rest;
    for (int idx = threadIdx.x; idx < qk_heads * rest; idx += blockDim.x) {
        const int head = idx / rest, i = first_rest + (idx - head * rest);
        const bool is_k = head >= n_heads;
        const float* w = is_k ? k_w : q_w;
        if (w == nullptr && !(kdst && is_k)) continue;      // nothing changes and nothing is stored
        const int at = head * hd + i;
        float a = to_float(row0[at]);
        if (w != nullptr) a = (a * (is_k ? inv_k : inv_q)) * w[at - (is_k ? q_len : 0)];
        const T o = from_float<T>(a);
        row0[at] = o;
        if (kdst && is_k) kdst[(long)(head - n_heads) * kv_head_stride + i] = o;
    }
    T* vrow = row0 + q_len + k_len;
    for (int idx = threadIdx.x; idx < k_len; idx += blockDim.x) {
        const int g = idx / hd, i = idx - g * hd;
        T o = vrow[idx];
        if (mix_mode != 0 && i < v_dim) {                    // what lies behind a head's v_dim values is zero and stays
            const long at = ((long)t * n_kv + g) * v_dim + i;
            if (mix_mode == 1) mix_buf[at] = o;
            else {
                o = from_float<T>((1.0f - mix) * to_float(o) + mix * to_float(mix_buf[at]));
                vrow[idx] = o;
            }
        }
        if (vdst) vdst[(long)g * kv_head_stride + i] = o;
    }
}


__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(p[k]);
        f[2 * k] = x.x;
        f[2 * k + 1] = x.y;
    }
}

__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __halves2bfloat162(__float2bfloat16_rn(f[2 * k]), __float2bfloat16_rn(f[2 * k + 1]));
    return v;
}

__device__ __forceinline__ void load_float8(const float* __restrict__ p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// The same for bf16 rows whose heads, halves, value sizes and strides are multiples of 8 elements: 16 bytes a thread
// and turn.  q and k of the token are read once, into shared memory (q_len + k_len elements), while their squares are
// summed; the second pass works from there.  Same arithmetic, element by element.
__global__ void __launch_bounds__(256)
qk_prep_vec_kernel(__nv_bfloat16* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
                   const float* __restrict__ inv_freq, const float* __restrict__ q_w, const float* __restrict__ k_w,
                   int n_q, int n_k, float norm_eps, int mix_mode, float mix, __nv_bfloat16* __restrict__ mix_buf,
                   int v_dim, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                   const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                   __nv_bfloat16* __restrict__ v_pages, int page_size, long page_stride) {
    extern __shared__ uint4 row_s[];
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];                       // positions, tables and frequencies are older than the step
    const int half = rot / 2;
    const bool turn = inv_freq != nullptr && half > 0;
    if (turn)
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;
        vdst = v_pages + off;
    }
    pdl_wait();
    __nv_bfloat16* row0 = qkv + (long)t * row_stride;
    const int q_len = n_heads * hd, k_len = n_kv * hd;
    const int q_units = q_len / 8, qk_units = (q_len + k_len) / 8;
    float ssq = 0.f, ssk = 0.f;
    for (int u = threadIdx.x; u < qk_units; u += blockDim.x) {
        const uint4 v = *reinterpret_cast<const uint4*>(row0 + (long)u * 8);
        row_s[u] = v;
        float f[8];
        bf16x8_to_float(v, f);
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(f[k], f[k], ss);
        if (u < q_units) ssq += ss; else ssk += ss;
    }
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_w != nullptr) inv_q = 1.0f / sqrtf(block_sum(ssq, scratch) / (float)n_q + norm_eps);
    if (k_w != nullptr) inv_k = 1.0f / sqrtf(block_sum(ssk, scratch) / (float)n_k + norm_eps);
    __syncthreads();
    const long kv_head_stride = (long)page_size * hd;
    const int qk_heads = n_heads + n_kv;
    if (turn) {
        const int units = half / 8;
        for (int idx = threadIdx.x; idx < qk_heads * units; idx += blockDim.x) {
            const int head = idx / units, i0 = (idx - head * units) * 8;
            const bool is_k = head >= n_heads;
            const int at = head * hd + i0;
            float a[8], b2[8];
            bf16x8_to_float(row_s[at / 8], a);
            bf16x8_to_float(row_s[(at + half) / 8], b2);
            const float* w = is_k ? k_w : q_w;
            if (w != nullptr) {
                const int wi = at - (is_k ? q_len : 0);
                const float inv = is_k ? inv_k : inv_q;
                float wa[8], wb[8];
                load_float8(w + wi, wa);
                load_float8(w + wi + half, wb);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    a[k] = (a[k] * inv) * wa[k];
                    b2[k] = (b2[k] * inv) * wb[k];
                }
            }
            float lo[8], hi[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float c = cos_s[i0 + k], sn = sin_s[i0 + k];
                lo[k] = a[k] * c - b2[k] * sn;
                hi[k] = b2[k] * c + a[k] * sn;
            }
            const uint4 lo_v = float_to_bf16x8(lo), hi_v = float_to_bf16x8(hi);
            *reinterpret_cast<uint4*>(row0 + at) = lo_v;
            *reinterpret_cast<uint4*>(row0 + at + half) = hi_v;
            if (kdst && is_k) {
                __nv_bfloat16* d = kdst + (long)(head - n_heads) * kv_head_stride;
                *reinterpret_cast<uint4*>(d + i0) = lo_v;
                *reinterpret_cast<uint4*>(d + i0 + half) = hi_v;
            }
        }
    }
    const int first_rest = turn ? rot : 0, rest_units = (hd - first_rest) / 8;
    for (int idx = threadIdx.x; idx < qk_heads * rest_units; idx += blockDim.x) {
        const int head = idx / rest_units, i0 = first_rest + (idx - head * rest_units) * 8;
        const bool is_k = head >= n_heads;
        const float* w = is_k ? k_w : q_w;
        if (w == nullptr && !(kdst && is_k)) continue;      // nothing changes and nothing is stored
        const int at = head * hd + i0;
        uint4 o = row_s[at / 8];
        if (w != nullptr) {
            const float inv = is_k ? inv_k : inv_q;
            float a[8], wa[8];
            bf16x8_to_float(o, a);
            load_float8(w + at - (is_k ? q_len : 0), wa);
#pragma unroll
            for (int k = 0; k < 8; ++k) a[k] = (a[k] * inv) * wa[k];
            o = float_to_bf16x8(a);
            *reinterpret_cast<uint4*>(row0 + at) = o;
        }
        if (kdst && is_k) *reinterpret_cast<uint4*>(kdst + (long)(head - n_heads) * kv_head_stride + i0) = o;
    }
    __nv_bfloat16* vrow = row0 + q_len + k_len;
    const int v_units = hd / 8;
    for (int idx = threadIdx.x; idx < n_kv * v_units; idx += blockDim.x) {
        const int g = idx / v_units, i0 = (idx - g * v_units) * 8;
        uint4 o = *reinterpret_cast<const uint4*>(vrow + g * hd + i0);
        if (mix_mode != 0 && i0 < v_dim) {                   // what lies behind a head's v_dim values is zero and stays
            __nv_bfloat16* other = mix_buf + ((long)t * n_kv + g) * v_dim + i0;
            if (mix_mode == 1) *reinterpret_cast<uint4*>(other) = o;
            else {
                float a[8], m[8];
                bf16x8_to_float(o, a);
                bf16x8_to_float(*reinterpret_cast<const uint4*>(other), m);
#pragma unroll
                for (int k = 0; k < 8; ++k) a[k] = (1.0f - mix) * a[k] + mix * m[k];
                o = float_to_bf16x8(a);
                *reinterpret_cast<uint4*>(vrow + g * hd + i0) = o;
            }
        }
        if (vdst) *reinterpret_cast<uint4*>(vdst + (long)g * kv_head_stride + i0) = o;
    }
}

}  // namespace zlm

using namespace zlm;

// Rotates q and k in place inside qkv and copies k (rotated) and v into the cache.
// inv_freq == nullptr: no rotation.  k_pages == nullptr: nothing is stored (a layer
// that reads another layer's cache).  v_pages == nullptr with k_pages: the rows are [q | k] and only the keys
// are stored (a latent that serves as key and value).
ZLM_EXPORT int zlm_rope_store(void* qkv, int dtype, long row_stride, int T, int n_heads, int n_kv, int hd, int rot,
                              const float* inv_freq, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, void* k_pages, void* v_pages, int page_size,
                              long page_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || rot < 0 || rot > hd || (rot & 1) || n_heads <= 0 || n_kv < 0 || page_size <= 0)
        return ZLM_ERR_BAD_ARG;
    if (rot / 2 > ROPE_MAX_HALF) return ZLM_ERR_UNSUPPORTED;
    // few tokens (a decode step): the heads of a token are shared out over several blocks
    const int total_heads = n_heads + n_kv + (v_pages != nullptr ? n_kv : 0);
    int parts = (296 + T - 1) / T;
    if (parts > total_heads) parts = total_heads;
    if (parts < 1) parts = 1;
    const int per = (total_heads + parts - 1) / parts;
    parts = (total_heads + per - 1) / per;
    const int work = per * (hd / 2);
    const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    dim3 grid(T, parts);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(rope_store_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, row_stride, n_heads, n_kv,
                       hd, rot, inv_freq, positions, seq_of_token, block_table, bt_stride, (float*)k_pages,
                       (float*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16 && hd % 8 == 0 && rot % 16 == 0 && row_stride % 8 == 0 && page_stride % 8 == 0 &&
             (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 && hd / 2 <= 2048)
        e = launch_pdl(rope_store_vec_kernel, grid, dim3(work >= 256 * 8 ? 256 : (work >= 128 * 8 ? 128 : 64)), 0, stream,
                       (__nv_bfloat16*)qkv, row_stride, n_heads, n_kv, hd, rot, inv_freq, positions, seq_of_token,
                       block_table, bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)qkv,
                       row_stride, n_heads, n_kv, hd, rot, inv_freq, positions, seq_of_token, block_table, bt_stride,
                       (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, page_stride);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// Like zlm_rope_store for rows [q heads | k heads | v heads | anything else] (row_stride elements a row), with the
// cosines and sines multiplied by `amplitude` and, when norm_dim > 0, every rotated q and k head divided by the
// root of (the mean of the squares of its first norm_dim dimensions + norm_eps) before it is written back and
// stored.  inv_freq == nullptr: no rotation.  k_pages == nullptr: nothing is stored.  norm_first != 0: the norm stands
// BEFORE the rotation instead, and q_weight / k_weight (float [hd], shared by all query / key heads; nullptr: none)
// multiply the normed heads.
ZLM_EXPORT int zlm_rope_norm_store(void* qkv, int dtype, long row_stride, int T, int n_heads, int n_kv, int hd, int rot,
                                   const float* inv_freq, float amplitude, int norm_dim, float norm_eps,
                                   int norm_first, const float* q_weight, const float* k_weight,
                                   const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                                   void* k_pages, void* v_pages, int page_size, long page_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || rot < 0 || rot > hd || (rot & 1) || n_heads <= 0 || n_kv < 0 || page_size <= 0 || norm_dim < 0 ||
        norm_dim > hd || (k_pages != nullptr && v_pages == nullptr))
        return ZLM_ERR_BAD_ARG;
    if (rot / 2 > ROPE_MAX_HALF || hd > ATT_MAX_HD_ROPE) return ZLM_ERR_UNSUPPORTED;
    const int total_heads = n_heads + 2 * n_kv;
    int parts = (296 + T - 1) / T;
    if (parts > (total_heads + RNS_WARPS - 1) / RNS_WARPS) parts = (total_heads + RNS_WARPS - 1) / RNS_WARPS;
    if (parts < 1) parts = 1;
    dim3 grid(T, parts);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(rope_norm_store_kernel<float>, grid, dim3(RNS_WARPS * 32), 0, stream, (float*)qkv, row_stride,
                       n_heads, n_kv, hd, rot, inv_freq, amplitude, norm_dim, norm_eps, norm_first, q_weight, k_weight,
                       positions, seq_of_token, block_table, bt_stride, (float*)k_pages, (float*)v_pages, page_size,
                       page_stride);
    else if (dtype == ZLM_BF16 && hd % 8 == 0 && (inv_freq == nullptr || rot % 16 == 0) && row_stride % 8 == 0 &&
             page_stride % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 &&
             (uintptr_t)v_pages % 16 == 0 && hd / 8 <= 32) {
        const int first_tail = (inv_freq != nullptr && rot > 0) ? rot : 0;
        const int units = first_tail / 16 + (hd - first_tail) / 8;
        int lph = 1;
        while (lph < units) lph <<= 1;
        const int per_block = RNS_WARPS * (32 / lph);
        int vparts = (296 + T - 1) / T;
        const int most = (n_heads + n_kv + per_block - 1) / per_block;
        if (vparts > most) vparts = most;
        if (vparts < 1) vparts = 1;
        e = launch_pdl(rope_norm_store_vec_kernel, dim3(T, vparts), dim3(RNS_WARPS * 32), 0, stream, (__nv_bfloat16*)qkv,
                       row_stride, n_heads, n_kv, hd, rot, inv_freq, amplitude, norm_dim, norm_eps, norm_first, q_weight,
                       k_weight, positions, seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pages,
                       (__nv_bfloat16*)v_pages, page_size, page_stride, lph);
    } else if (dtype == ZLM_BF16)
        e = launch_pdl(rope_norm_store_kernel<__nv_bfloat16>, grid, dim3(RNS_WARPS * 32), 0, stream, (__nv_bfloat16*)qkv,
                       row_stride, n_heads, n_kv, hd, rot, inv_freq, amplitude, norm_dim, norm_eps, norm_first, q_weight,
                       k_weight, positions, seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pages,
                       (__nv_bfloat16*)v_pages, page_size, page_stride);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// Floats of scratch memory that let zlm_attention_general spread a step of T tokens whose longest visible range
// is max_keys keys over more blocks (0: the step has enough tokens, or one part of keys).
ZLM_EXPORT long zlm_attention_general_scratch(int T, int n_heads, int n_kv, int hd, int max_keys) {
    if (T <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return 0;
    const int group = n_heads / n_kv, g = (group % 4 == 0 && hd <= 256) ? 4 : (group % 2 == 0 ? 2 : 1);
    const long parts = (max_keys + ATT_PART - 1) / ATT_PART;
    if (parts <= 1 || (long)T * (n_heads / g) >= 2 * 148) return 0;
    return (long)T * n_heads * parts * (hd + 2);
}

// keep_first (with a window): the first keep_first positions of a sequence stay visible behind the window.  sinks (float,
// one per query head; may be null): exp(sinks[h]) is added to the softmax's denominator of head h; it has no key and no
// value and is not scaled.
// max_keys: the most keys any token of the step sees.  scratch (float, scratch_floats elements; may be null):
// when it holds at least zlm_attention_general_scratch(...) floats and that is not 0, the parts of the keys are
// computed by blocks of their own and folded by a second kernel; the result is bit for bit the same.
ZLM_EXPORT int zlm_attention_general(const void* q, long q_row_stride, void* out, int dtype, int T, int n_heads,
                                     int n_kv, int hd, float scale, float softcap, int window, int keep_first,
                                     const float* sinks, const int* positions,
                                     const int* seq_of_token, const int* block_table, int bt_stride,
                                     const void* k_pages, const void* v_pages, int page_size, long page_stride,
                                     int max_keys, float* scratch, long scratch_floats, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0 || keep_first < 0) return ZLM_ERR_BAD_ARG;
    if (window <= 0) keep_first = 0;
    if (hd <= 0 || hd > ATT_MAX_HD || hd % 8) return ZLM_ERR_UNSUPPORTED;
    float *part_ml = nullptr, *part_o = nullptr;
    int max_parts = 1;
    const long need = zlm_attention_general_scratch(T, n_heads, n_kv, hd, max_keys);
    if (need > 0 && scratch != nullptr && scratch_floats >= need) {
        max_parts = (max_keys + ATT_PART - 1) / ATT_PART;
        if (max_parts > 65535) return ZLM_ERR_UNSUPPORTED;
        part_o = scratch;
        part_ml = scratch + (long)T * n_heads * max_parts * hd;
    }
    const int group = n_heads / n_kv;
    if (dtype == ZLM_F32)
        return pick_group<float, 4>(group, q, q_row_stride, out, T, n_heads, n_kv, hd, scale, softcap, window, keep_first, sinks,
                                    positions, seq_of_token, block_table, bt_stride, k_pages, v_pages, page_size, page_stride,
                                    part_ml, part_o, max_parts, stream);
    if (dtype == ZLM_BF16)
        return pick_group<__nv_bfloat16, 8>(group, q, q_row_stride, out, T, n_heads, n_kv, hd, scale, softcap, window, keep_first,
                                            sinks, positions, seq_of_token, block_table, bt_stride, k_pages, v_pages, page_size,
                                            page_stride, part_ml, part_o, max_parts, stream);
    return ZLM_ERR_UNSUPPORTED;
}

// See qk_prep_kernel.  q_w / k_w: float norm weights laid out like the q and the k heads of a row (null: that vector is
// not normed); n_q / n_k: the element counts of the means.  mix_mode 0: values as they are; 1: also left in mix_buf;
// 2: mixed with mix_buf ([T, n_kv * v_dim]: the true values of every head).  k_pages == nullptr: nothing is stored.
ZLM_EXPORT int zlm_qk_prep(void* qkv, int dtype, long row_stride, int T, int n_heads, int n_kv, int hd, int rot,
                           const float* inv_freq, const float* q_w, const float* k_w, int n_q, int n_k, float norm_eps,
                           int mix_mode, float mix, void* mix_buf, int v_dim, const int* positions, const int* seq_of_token,
                           const int* block_table, int bt_stride, void* k_pages, void* v_pages, int page_size,
                           long page_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || rot < 0 || rot > hd || (rot & 1) || n_heads <= 0 || n_kv <= 0 || page_size <= 0 || mix_mode < 0 ||
        mix_mode > 2 || (mix_mode != 0 && (mix_buf == nullptr || v_dim <= 0 || v_dim > hd)) || (k_pages != nullptr && v_pages == nullptr) ||
        (q_w != nullptr && n_q <= 0) || (k_w != nullptr && n_k <= 0))
        return ZLM_ERR_BAD_ARG;
    if (rot / 2 > ROPE_MAX_HALF) return ZLM_ERR_UNSUPPORTED;
    const int work = (n_heads + 2 * n_kv) * hd;
    const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(qk_prep_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)qkv, row_stride, n_heads, n_kv, hd,
                       rot, inv_freq, q_w, k_w, n_q, n_k, norm_eps, mix_mode, mix, (float*)mix_buf, v_dim, positions, seq_of_token,
                       block_table, bt_stride, (float*)k_pages, (float*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16 && hd % 8 == 0 && rot % 16 == 0 && row_stride % 8 == 0 && page_stride % 8 == 0 &&
             (mix_mode == 0 || v_dim % 8 == 0) && (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 &&
             (uintptr_t)v_pages % 16 == 0 && (uintptr_t)mix_buf % 16 == 0 && (uintptr_t)q_w % 16 == 0 &&
             (uintptr_t)k_w % 16 == 0 && (size_t)(n_heads + n_kv) * hd * 2 <= 40 * 1024)
        e = launch_pdl(qk_prep_vec_kernel, dim3(T), dim3(work >= 256 * 8 ? 256 : (work >= 128 * 8 ? 128 : 64)),
                       (size_t)(n_heads + n_kv) * hd * 2, stream, (__nv_bfloat16*)qkv, row_stride, n_heads, n_kv, hd, rot,
                       inv_freq, q_w, k_w, n_q, n_k, norm_eps, mix_mode, mix, (__nv_bfloat16*)mix_buf, v_dim, positions,
                       seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size,
                       page_stride);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(qk_prep_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)qkv, row_stride,
                       n_heads, n_kv, hd, rot, inv_freq, q_w, k_w, n_q, n_k, norm_eps, mix_mode, mix, (__nv_bfloat16*)mix_buf,
                       v_dim, positions, seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                       page_size, page_stride);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}
