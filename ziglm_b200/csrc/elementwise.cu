// Embedding gather, RMSNorm (with optional row gather) and the gated activation.
//
// Formulas follow the reference:
//   embedding  x = W_e[token] widened to float, times a scale that is 1 for this
//              architecture                      (src/model.zig:495-503)
//   RMSNorm    ss = sum x_i^2, inv = 1/sqrt(ss/n + eps), y_i = (x_i*inv)*w_i
//              (src/math.zig:850-945; GPU twin src/cuda_bridge.cu:1475-1534)
//   SwiGLU     act_j = silu(g_j)*u_j, silu(z) = z/(1+exp(-z))
//              (src/math.zig:1108-1117, src/cuda_bridge.cu:2271-2285)
// The residual stream is float in both precisions, so the norm always reads
// float and writes the storage type of the next matrix product.
#include "common.cuh"

namespace zlm {

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const long row = (long)tokens[t] * d;
    float* o = out + (long)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(table[row + i]) * scale;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  rows == nullptr: row r of the input; otherwise row
// rows[r] (this is how the final norm runs on the wanted positions only).
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}
template <typename TW> __device__ __forceinline__ void load4(const TW* p, float (&w)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&w)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&w)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
}

// VEC: the row length is a multiple of 4 and every pointer is 16-byte aligned, so a thread moves four
// elements at a time and keeps up to MAXV groups of its row in registers between the two passes.
template <typename TW, typename TO, bool VEC>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int d, float eps, float weight_offset) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long)(rows ? rows[r] : r) * d;
    TO* o = out + (long)r * d;
    if (VEC) {
        constexpr int MAXV = 8;
        float4 keep[MAXV];
        const int n4 = d >> 2;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                keep[k] = reinterpret_cast<const float4*>(xr)[i];
                ss = fmaf(keep[k].x, keep[k].x, ss); ss = fmaf(keep[k].y, keep[k].y, ss);
                ss = fmaf(keep[k].z, keep[k].z, ss); ss = fmaf(keep[k].w, keep[k].w, ss);
            }
        }
        for (int i = threadIdx.x + MAXV * blockDim.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                float ww[4];
                load4<TW>(w + 4 * i, ww);
                store4<TO>(o + 4 * i, (keep[k].x * inv) * (ww[0] + weight_offset), (keep[k].y * inv) * (ww[1] + weight_offset),
                           (keep[k].z * inv) * (ww[2] + weight_offset), (keep[k].w * inv) * (ww[3] + weight_offset));
            }
        }
        for (int i = threadIdx.x + MAXV * blockDim.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w + 4 * i, ww);
            store4<TO>(o + 4 * i, (v.x * inv) * (ww[0] + weight_offset), (v.y * inv) * (ww[1] + weight_offset),
                       (v.z * inv) * (ww[2] + weight_offset), (v.w * inv) * (ww[3] + weight_offset));
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = xr[i];
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            o[i] = from_float<TO>((xr[i] * inv) * (to_float(w[i]) + weight_offset));
    }
}

// --------------------------------------------------------- gated activation
// gu is [T, 2*I].  interleaved == 0: gate in columns [0, I), up in columns [I, 2I);
// interleaved != 0: gate j in column 2j, up j in column 2j+1.
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, long total, int I, int kind,
                                 int interleaved, float limit, float slope) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / I;
    const int j = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + (interleaved ? 2 * j : j)]);
    const float u = to_float(gu[t * 2 * I + (interleaved ? 2 * j + 1 : I + j)]);
    float a;
    if (kind == 2) {
        // clamped swish: g' = min(g, L), u' = clamp(u, -L, L); g' sigmoid(slope g') (u' + 1)
        const float gc = fminf(g, limit);
        const float uc = fminf(fmaxf(u, -limit), limit);
        out[idx] = from_float<T>((gc / (1.0f + expf(-slope * gc))) * (uc + 1.0f));
        return;
    }
    if (kind == 0) {
        a = g / (1.0f + expf(-g));                         // silu
    } else {
        const float c = 0.7978845608028654f;               // gelu (tanh form)
        a = 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
    }
    out[idx] = from_float<T>(a * u);
}

// A norm over a row that is a slice of a wider row (x and out with row strides of their own), and the same
// norm added into a float32 row (the norm behind a sublayer, summed into the residual stream in one pass):
//   out[r, i] (+)= x[r, i] / sqrt(mean_i x[r, i]^2 + eps) * (w[i] + weight_offset)
template <typename TW, typename TO, bool ADD, bool VEC>
__global__ void rmsnorm_strided_kernel(const float* __restrict__ x, long x_stride, const TW* __restrict__ w,
                                       TO* __restrict__ out, long out_stride, int d, float eps, float weight_offset) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + (long)blockIdx.x * x_stride;
    TO* o = out + (long)blockIdx.x * out_stride;
    float ss = 0.f;
    if constexpr (VEC) {
        // the row is a multiple of four long and every pointer and stride keeps sixteen bytes: four at a time
        const int n4 = d >> 2;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w + 4 * i, ww);
            float y0 = (v.x * inv) * (ww[0] + weight_offset), y1 = (v.y * inv) * (ww[1] + weight_offset);
            float y2 = (v.z * inv) * (ww[2] + weight_offset), y3 = (v.w * inv) * (ww[3] + weight_offset);
            if (ADD) {
                const float4 old = reinterpret_cast<const float4*>(o)[i];
                y0 += old.x; y1 += old.y; y2 += old.z; y3 += old.w;
            }
            store4<TO>(o + 4 * i, y0, y1, y2, y3);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = xr[i];
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float y = (xr[i] * inv) * (to_float(w[i]) + weight_offset);
            if (ADD) o[i] = from_float<TO>(to_float(o[i]) + y);
            else o[i] = from_float<TO>(y);
        }
    }
}

// The norm behind a sublayer, the residual sum and the norm before the next sublayer in one pass over a row:
//   x[r] += branch[r] / rms(branch[r]) * (w1 + off1);   h[r] = x[r] / rms(x[r]) * (w2 + off2)
// The new row of x stays in shared memory between the two norms (d floats of dynamic shared memory).
template <typename TW, typename TO, bool VEC>
__global__ void norm_add_norm_kernel(const float* __restrict__ branch, const TW* __restrict__ w1, float off1, float eps1,
                                     float* __restrict__ x, const TW* __restrict__ w2, float off2, float eps2,
                                     TO* __restrict__ h, int d) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* br = branch + (long)blockIdx.x * d;
    float* xr = x + (long)blockIdx.x * d;
    TO* hr = h + (long)blockIdx.x * d;
    if constexpr (VEC) {
        // d is a multiple of four and every pointer keeps sixteen bytes: four elements at a time
        const int n4 = d >> 2;
        float ss = 0.f;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(br)[i];
            reinterpret_cast<float4*>(row)[i] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv1 = 1.0f / sqrtf(ss / (float)d + eps1);
        float ss2 = 0.f;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 b4 = reinterpret_cast<const float4*>(row)[i];
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w1 + 4 * i, ww);
            v.x += (b4.x * inv1) * (ww[0] + off1); v.y += (b4.y * inv1) * (ww[1] + off1);
            v.z += (b4.z * inv1) * (ww[2] + off1); v.w += (b4.w * inv1) * (ww[3] + off1);
            reinterpret_cast<float4*>(xr)[i] = v;
            reinterpret_cast<float4*>(row)[i] = v;
            ss2 = fmaf(v.x, v.x, ss2); ss2 = fmaf(v.y, v.y, ss2); ss2 = fmaf(v.z, v.z, ss2); ss2 = fmaf(v.w, v.w, ss2);
        }
        ss2 = block_sum(ss2, scratch);
        const float inv2 = 1.0f / sqrtf(ss2 / (float)d + eps2);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(row)[i];
            float ww[4];
            load4<TW>(w2 + 4 * i, ww);
            store4<TO>(hr + 4 * i, (v.x * inv2) * (ww[0] + off2), (v.y * inv2) * (ww[1] + off2),
                       (v.z * inv2) * (ww[2] + off2), (v.w * inv2) * (ww[3] + off2));
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = br[i];
            row[i] = v;
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv1 = 1.0f / sqrtf(ss / (float)d + eps1);
        float ss2 = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = xr[i] + (row[i] * inv1) * (to_float(w1[i]) + off1);
            xr[i] = v;
            row[i] = v;
            ss2 = fmaf(v, v, ss2);
        }
        ss2 = block_sum(ss2, scratch);
        const float inv2 = 1.0f / sqrtf(ss2 / (float)d + eps2);
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            hr[i] = from_float<TO>((row[i] * inv2) * (to_float(w2[i]) + off2));
    }
}

// x[t, :] += table[row, :] for every row t of x (a learned vector added to the whole step)
// The norm behind a sublayer of an arrangement without norms before its sublayers, the residual sum with a
// multiplier, and the rows the next sublayer reads (the new residual in the step's storage type):
//   x[r] += mult * branch[r] / rms(branch[r]) * (w + off);   h[r] = x[r]      (h may be null)
template <typename TW, typename TO, bool VEC>
__global__ void norm_add_scaled_kernel(const float* __restrict__ branch, const TW* __restrict__ w, float off, float eps,
                                       float mult, float* __restrict__ x, TO* __restrict__ h, int d) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* br = branch + (long)blockIdx.x * d;
    float* xr = x + (long)blockIdx.x * d;
    float ss = 0.f;
    if constexpr (VEC) {
        // d is a multiple of four and every pointer keeps sixteen bytes: four elements at a time
        const int n4 = d >> 2;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(br)[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 b4 = reinterpret_cast<const float4*>(br)[i];
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w + 4 * i, ww);
            v.x += mult * ((b4.x * inv) * (ww[0] + off)); v.y += mult * ((b4.y * inv) * (ww[1] + off));
            v.z += mult * ((b4.z * inv) * (ww[2] + off)); v.w += mult * ((b4.w * inv) * (ww[3] + off));
            reinterpret_cast<float4*>(xr)[i] = v;
            if (h != nullptr) store4<TO>(h + (long)blockIdx.x * d + 4 * i, v.x, v.y, v.z, v.w);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = br[i];
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = xr[i] + mult * ((br[i] * inv) * (to_float(w[i]) + off));
            xr[i] = v;
            if (h != nullptr) h[(long)blockIdx.x * d + i] = from_float<TO>(v);
        }
    }
}

// The norm of a sum, in place: with s = alpha * x[r] + branch[r],
//   x[r] = s / sqrt(mean(s^2) + eps) * (w + off);   h[r] = x[r]      (h may be null)
// The residual stream of an arrangement whose norms stand behind the sums: the stream itself is normed.
template <typename TW, typename TO, bool VEC>
__global__ void sum_norm_kernel(const float* __restrict__ branch, const TW* __restrict__ w, float off, float eps,
                                float alpha, float* __restrict__ x, TO* __restrict__ h, int d) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* br = branch + (long)blockIdx.x * d;
    float* xr = x + (long)blockIdx.x * d;
    float ss = 0.f;
    if constexpr (VEC) {
        const int n4 = d >> 2;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 b4 = reinterpret_cast<const float4*>(br)[i];
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            const float s0 = fmaf(alpha, v.x, b4.x), s1 = fmaf(alpha, v.y, b4.y), s2 = fmaf(alpha, v.z, b4.z),
                        s3 = fmaf(alpha, v.w, b4.w);
            ss = fmaf(s0, s0, ss); ss = fmaf(s1, s1, ss); ss = fmaf(s2, s2, ss); ss = fmaf(s3, s3, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 b4 = reinterpret_cast<const float4*>(br)[i];
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w + 4 * i, ww);
            v.x = (fmaf(alpha, v.x, b4.x) * inv) * (ww[0] + off); v.y = (fmaf(alpha, v.y, b4.y) * inv) * (ww[1] + off);
            v.z = (fmaf(alpha, v.z, b4.z) * inv) * (ww[2] + off); v.w = (fmaf(alpha, v.w, b4.w) * inv) * (ww[3] + off);
            reinterpret_cast<float4*>(xr)[i] = v;
            if (h != nullptr) store4<TO>(h + (long)blockIdx.x * d + 4 * i, v.x, v.y, v.z, v.w);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float s = fmaf(alpha, xr[i], br[i]);
            ss = fmaf(s, s, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = (fmaf(alpha, xr[i], br[i]) * inv) * (to_float(w[i]) + off);
            xr[i] = v;
            if (h != nullptr) h[(long)blockIdx.x * d + i] = from_float<TO>(v);
        }
    }
}

// A norm of every head by itself, with a gate: row r of x (float) holds n_heads heads of hd elements;
//   out[r, h, i] = x[r, h, i] / sqrt(mean_i x[r, h, :]^2 + eps) * w[h * hd + i] * act(g[r, h * hd + i]) * mult
// w null: no weight.  gate_kind 0: no gate, 1: sigmoid(g), 2: silu(g) = g sigmoid(g).  One warp a head.
constexpr int HNG_WARPS = 4;
template <typename T>
__global__ void __launch_bounds__(HNG_WARPS * 32)
head_norm_gate_kernel(const float* __restrict__ x, long x_stride, const float* __restrict__ w, const T* __restrict__ g,
                      long g_stride, T* __restrict__ out, long out_stride, long n_pairs, int n_heads, int hd, float eps,
                      int gate_kind, float mult) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long pair = (long)blockIdx.x * HNG_WARPS + (threadIdx.x >> 5);
    if (pair >= n_pairs) return;
    const long r = pair / n_heads;
    const int h = (int)(pair % n_heads);
    const float* xr = x + r * x_stride + (long)h * hd;
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)hd + eps);
    for (int i = lane; i < hd; i += 32) {
        float y = xr[i] * inv;
        if (w != nullptr) y *= w[(long)h * hd + i];
        if (gate_kind != 0) {
            const float gv = to_float(g[r * g_stride + (long)h * hd + i]);
            const float sg = 1.0f / (1.0f + expf(-gv));
            y *= gate_kind == 2 ? gv * sg : sg;
        }
        out[r * out_stride + (long)h * hd + i] = from_float<T>(y * mult);
    }
}

// out[i] = act(x[i]); kind 0: the squared relu, max(x, 0)^2; kind 1: the exact gelu, x (1 + erf(x / sqrt 2)) / 2
template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, T* __restrict__ out, long n, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = to_float(x[i]);
    if (kind == 1) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    else { v = fmaxf(v, 0.f); v *= v; }
    out[i] = from_float<T>(v);
}

// out[t, i] = a[t, i] * sigmoid(g[t, i]) over rows with strides of their own (a gate on the heads' outputs)
template <typename T>
__global__ void sigmoid_mul_kernel(const T* __restrict__ a, long a_stride, const T* __restrict__ g, long g_stride,
                                   T* __restrict__ out, long out_stride, long total, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / n;
    const int i = (int)(idx - t * n);
    const float gv = to_float(g[t * g_stride + i]);
    out[t * out_stride + i] = from_float<T>(to_float(a[t * a_stride + i]) * (1.0f / (1.0f + expf(-gv))));
}

// The same for bf16 rows whose length, strides and addresses are multiples of 8 elements: 16 bytes a thread.
__global__ void sigmoid_mul_vec_kernel(const __nv_bfloat16* __restrict__ a, long a_stride, const __nv_bfloat16* __restrict__ g,
                                       long g_stride, __nv_bfloat16* __restrict__ out, long out_stride, long total8, int n8) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const long t = idx / n8;
    const int i = (int)(idx - t * n8) * 8;
    uint4 av = *reinterpret_cast<const uint4*>(a + t * a_stride + i);
    const uint4 gv = *reinterpret_cast<const uint4*>(g + t * g_stride + i);
    __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&av);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(ap[k]), y = __bfloat1622float2(gp[k]);
        ap[k] = __floats2bfloat162_rn(x.x * (1.0f / (1.0f + expf(-y.x))), x.y * (1.0f / (1.0f + expf(-y.y))));
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + i) = av;
}

// out[t, i] = in[t, i] over rows with strides of their own, from one storage type to another
template <typename TI, typename TO>
__global__ void convert_rows_kernel(const TI* __restrict__ in, long in_stride, TO* __restrict__ out, long out_stride,
                                    long total, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / n;
    const int i = (int)(idx - t * n);
    out[t * out_stride + i] = from_float<TO>(to_float(in[t * in_stride + i]));
}

// out[t, h * n + i] = a[t, h * n + i] * sigmoid(g[t, h]) * mult over rows with strides of their own: one gate a head.
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ a, long a_stride, const T* __restrict__ g, long g_stride,
                                  T* __restrict__ out, long out_stride, long total, int heads, int n, float mult) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int width = heads * n;
    const long t = idx / width;
    const int i = (int)(idx - t * width);
    const float gv = to_float(g[t * g_stride + i / n]);
    out[t * out_stride + i] = from_float<T>(to_float(a[t * a_stride + i]) * ((1.0f / (1.0f + expf(-gv))) * mult));
}

// The same for bf16 rows whose heads, strides and addresses are multiples of 8 elements: 16 bytes a thread.
__global__ void gate_heads_vec_kernel(const __nv_bfloat16* __restrict__ a, long a_stride, const __nv_bfloat16* __restrict__ g,
                                      long g_stride, __nv_bfloat16* __restrict__ out, long out_stride, long total8,
                                      int width8, int n8, float mult) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const long t = idx / width8;
    const int i8 = (int)(idx - t * width8);
    const float gv = to_float(g[t * g_stride + i8 / n8]);
    const float f = (1.0f / (1.0f + expf(-gv))) * mult;
    uint4 av = *reinterpret_cast<const uint4*>(a + t * a_stride + i8 * 8);
    __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&av);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(ap[k]);
        ap[k] = __floats2bfloat162_rn(x.x * f, x.y * f);
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + i8 * 8) = av;
}

// out[r, i] = x[r, i] / sqrt(mean_i x[r, i]^2 + eps) * w[i] * sigmoid(g[r, i]) * mult: the norm over the concatenated
// heads of a mixer and its output gate in one pass.  x float rows, g and out rows of the step's type, all with strides
// of their own.
template <typename T>
__global__ void norm_gate_kernel(const float* __restrict__ x, long x_stride, const float* __restrict__ w,
                                 const T* __restrict__ g, long g_stride, T* __restrict__ out, long out_stride, int d,
                                 float eps, float mult) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + (long)blockIdx.x * x_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float y = (xr[i] * inv) * w[i];
        if (g != nullptr) y *= 1.0f / (1.0f + expf(-to_float(g[(long)blockIdx.x * g_stride + i])));
        out[(long)blockIdx.x * out_stride + i] = from_float<T>(y * mult);
    }
}

// The same for a bf16 gate and result when the row length, the strides and the addresses are multiples of 4
// elements: 16 bytes of x, 8 of the gate and 8 of the result a thread and turn.
__global__ void norm_gate_vec_kernel(const float* __restrict__ x, long x_stride, const float* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ g, long g_stride, __nv_bfloat16* __restrict__ out,
                                     long out_stride, int d, float eps, float mult) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(x + (long)blockIdx.x * x_stride);
    const int d4 = d >> 2;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 v = xr[i];
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
    const float4* wr = reinterpret_cast<const float4*>(w);
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 v = xr[i], ww = wr[i];
        float y[4] = {(v.x * inv) * ww.x, (v.y * inv) * ww.y, (v.z * inv) * ww.z, (v.w * inv) * ww.w};
        if (g != nullptr) {
            const uint2 gv = *reinterpret_cast<const uint2*>(g + (long)blockIdx.x * g_stride + i * 4);
            const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.x));
            const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.y));
            y[0] *= 1.0f / (1.0f + expf(-g0.x)); y[1] *= 1.0f / (1.0f + expf(-g0.y));
            y[2] *= 1.0f / (1.0f + expf(-g1.x)); y[3] *= 1.0f / (1.0f + expf(-g1.y));
        }
        __nv_bfloat162 o0 = __floats2bfloat162_rn(y[0] * mult, y[1] * mult), o1 = __floats2bfloat162_rn(y[2] * mult, y[3] * mult);
        uint2 ov;
        ov.x = *reinterpret_cast<uint32_t*>(&o0);
        ov.y = *reinterpret_cast<uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(out + (long)blockIdx.x * out_stride + i * 4) = ov;
    }
}

// The same for rows of at most 8 elements a thread: x, the weight and the gate are requested together before the
// row's sum is formed, and x stays in registers.
__global__ void norm_gate_vec2_kernel(const float* __restrict__ x, long x_stride, const float* __restrict__ w,
                                      const __nv_bfloat16* __restrict__ g, long g_stride, __nv_bfloat16* __restrict__ out,
                                      long out_stride, int d, float eps, float mult) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(x + (long)blockIdx.x * x_stride);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const int d4 = d >> 2;
    float4 xv[2], wv[2];
    uint2 gv[2];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        xv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        wv[u] = xv[u];
        gv[u] = make_uint2(0u, 0u);
        if (i < d4) {
            xv[u] = xr[i];
            wv[u] = wr[i];
            if (g != nullptr) gv[u] = *reinterpret_cast<const uint2*>(g + (long)blockIdx.x * g_stride + i * 4);
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        ss = fmaf(xv[u].x, xv[u].x, ss); ss = fmaf(xv[u].y, xv[u].y, ss);
        ss = fmaf(xv[u].z, xv[u].z, ss); ss = fmaf(xv[u].w, xv[u].w, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i >= d4) continue;
        float y[4] = {(xv[u].x * inv) * wv[u].x, (xv[u].y * inv) * wv[u].y, (xv[u].z * inv) * wv[u].z, (xv[u].w * inv) * wv[u].w};
        if (g != nullptr) {
            const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv[u].x));
            const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv[u].y));
            y[0] *= 1.0f / (1.0f + expf(-g0.x)); y[1] *= 1.0f / (1.0f + expf(-g0.y));
            y[2] *= 1.0f / (1.0f + expf(-g1.x)); y[3] *= 1.0f / (1.0f + expf(-g1.y));
        }
        __nv_bfloat162 o0 = __floats2bfloat162_rn(y[0] * mult, y[1] * mult), o1 = __floats2bfloat162_rn(y[2] * mult, y[3] * mult);
        uint2 ov;
        ov.x = *reinterpret_cast<uint32_t*>(&o0);
        ov.y = *reinterpret_cast<uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(out + (long)blockIdx.x * out_stride + i * 4) = ov;
    }
}

template <typename TW>
__global__ void add_row_kernel(float* __restrict__ x, const TW* __restrict__ table_row, long total, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += to_float(table_row[i % d]);
}

__global__ void scale_kernel(float* __restrict__ x, long n, float factor) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= factor;
}

// y += x (float), used by parts that cannot fold their residual sum into a product
__global__ void add_kernel(float* __restrict__ y, const float* __restrict__ x, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += x[i];
}

template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(to_float(in[i]));
}

static int norm_threads(int d) {
    int t = 32;
    while (t < 512 && t * 4 < d) t <<= 1;
    return t;
}


// -------------------------------------------------------------- random weights
// Element i of a tensor with key k is a function of (k, i) alone:
//   h = mix64(k + i); a = top 24 bits of h, b = the 24 bits below them;
//   u1 = (a + 1) / 2^24 in (0, 1], angle = 2 pi b / 2^24;
//   z = sqrt(-2 ln u1) * cos(angle)                      (Box-Muller, one of its two values)
//   value = mean + std * z, rounded to the storage type.
// Every floating operation is a single IEEE-rounded +, *, / or sqrt in float (the _rn intrinsics keep
// the compiler from fusing them), and ln, sin and cos are the short polynomials below, so the same
// steps in NumPy give the same bits (ziglm_b200/weights/random_init.py: normal_values).  The
// reference fills its fixtures from one sequential generator (src/synthetic.zig:232-249); a counter
// lets any element be regenerated without the others, on the host or on the device.
__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float det_sin(float x) {          // x in [0, pi/4]
    const float x2 = __fmul_rn(x, x);
    float p = 2.75573192e-6f;                                 // 1/9!
    p = __fadd_rn(__fmul_rn(p, x2), -1.98412698e-4f);         // -1/7!
    p = __fadd_rn(__fmul_rn(p, x2), 8.33333333e-3f);          // 1/5!
    p = __fadd_rn(__fmul_rn(p, x2), -1.66666667e-1f);         // -1/3!
    p = __fadd_rn(__fmul_rn(p, x2), 1.0f);
    return __fmul_rn(x, p);
}

__device__ __forceinline__ float det_cos(float x) {          // x in [0, pi/4]
    const float x2 = __fmul_rn(x, x);
    float p = -2.75573192e-7f;                                // -1/10!
    p = __fadd_rn(__fmul_rn(p, x2), 2.48015873e-5f);          // 1/8!
    p = __fadd_rn(__fmul_rn(p, x2), -1.38888889e-3f);         // -1/6!
    p = __fadd_rn(__fmul_rn(p, x2), 4.16666667e-2f);          // 1/4!
    p = __fadd_rn(__fmul_rn(p, x2), -0.5f);
    return __fadd_rn(__fmul_rn(p, x2), 1.0f);
}

__device__ __forceinline__ float det_normal(uint64_t key, uint64_t index) {
    const uint64_t h = mix64(key + index);
    const uint32_t n = (uint32_t)(h >> 40) + 1u;              // 1 .. 2^24
    const uint32_t b = (uint32_t)(h >> 16) & 0xFFFFFFu;
    // ln(n / 2^24) = (e - 24) ln 2 + ln m with n = m 2^e, m in (sqrt(1/2), sqrt(2)]
    int e = 31 - __clz(n);
    float m = __fmul_rn((float)n, __int_as_float((127 - e) << 23));      // exact: n < 2^25, a power of two
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float p = 1.11111111e-1f;                                 // 1/9
    p = __fadd_rn(__fmul_rn(p, s2), 1.42857143e-1f);          // 1/7
    p = __fadd_rn(__fmul_rn(p, s2), 0.2f);
    p = __fadd_rn(__fmul_rn(p, s2), 3.33333333e-1f);
    p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
    const float ln_u = __fadd_rn(__fmul_rn((float)(e - 24), 0.693147182f), ln_m);
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));
    // cos(2 pi b / 2^24) by octants, the argument folded into [0, pi/4]
    const uint32_t oct = b >> 21, rem = b & 0x1FFFFFu;
    const float step = 3.74507039e-7f;                        // 2 pi / 2^24
    const float x = __fmul_rn((float)((oct & 1u) ? 0x200000u - rem : rem), step);
    float c;
    switch (oct) {
        case 0: c = det_cos(x); break;
        case 1: c = det_sin(x); break;
        case 2: c = -det_sin(x); break;
        case 3: c = -det_cos(x); break;
        case 4: c = -det_cos(x); break;
        case 5: c = -det_sin(x); break;
        case 6: c = det_sin(x); break;
        default: c = det_cos(x); break;
    }
    return __fmul_rn(r, c);
}

template <typename TO>
__global__ void fill_normal_kernel(TO* __restrict__ out, long n, uint64_t key, float mean, float std_dev) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        out[i] = from_float<TO>(__fadd_rn(mean, __fmul_rn(std_dev, det_normal(key, (uint64_t)i))));
}

}  // namespace zlm

using namespace zlm;

ZLM_EXPORT int zlm_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int d,
                         float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const int threads = d >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dtype == ZLM_F32)
        e = launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, tokens, out, d, scale);
    else if (table_dtype == ZLM_BF16)
        e = launch_pdl(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table,
                       tokens, out, d, scale);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype, const int* rows,
                           int n_rows, int d, float eps, float weight_offset, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const bool vec = d % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_NORM(TW, TO)                                                                                       \
    e = vec ? launch_pdl(rmsnorm_kernel<TW, TO, true>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w,  \
                         (TO*)out, rows, d, eps, weight_offset)                                                \
            : launch_pdl(rmsnorm_kernel<TW, TO, false>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w, \
                         (TO*)out, rows, d, eps, weight_offset)
    if (w_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_NORM(float, float);
    else if (w_dtype == ZLM_F32 && out_dtype == ZLM_BF16) ZLM_NORM(float, __nv_bfloat16);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_NORM(__nv_bfloat16, float);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_NORM(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_NORM
    return e == cudaSuccess ? launch_status() : (int)e;
}

// kind 0 silu, 1 gelu (tanh form), 2 clamped swish with (limit, slope); the two floats are read by kind 2 only
ZLM_EXPORT int zlm_gated_act(const void* gu, void* out, int dtype, int T, int I, int kind, int interleaved,
                             float limit, float slope, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0 || kind < 0 || kind > 2) return ZLM_ERR_BAD_ARG;
    const long total = (long)T * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(gated_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out,
                       total, I, kind, interleaved, limit, slope);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(gated_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, I, kind, interleaved, limit, slope);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// out rows (stride out_stride, storage out_dtype) = or += the RMS norm of x rows (float, stride x_stride).
ZLM_EXPORT int zlm_rmsnorm_strided(const float* x, long x_stride, const void* w, int w_dtype, void* out, int out_dtype,
                                   long out_stride, int add, int n_rows, int d, float eps, float weight_offset,
                                   cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0 || (add && out_dtype != ZLM_F32)) return ZLM_ERR_BAD_ARG;
    const int o_el = out_dtype == ZLM_F32 ? 4 : 2;
    const bool vec = d % 4 == 0 && x_stride % 4 == 0 && (out_stride * o_el) % 16 == 0 && (uintptr_t)x % 16 == 0 &&
                     (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_NORM_S(TW, TO, ADD)                                                                                      \
    e = vec ? launch_pdl(rmsnorm_strided_kernel<TW, TO, ADD, true>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, \
                         (const TW*)w, (TO*)out, out_stride, d, eps, weight_offset)                                  \
            : launch_pdl(rmsnorm_strided_kernel<TW, TO, ADD, false>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, \
                         (const TW*)w, (TO*)out, out_stride, d, eps, weight_offset)
    if (w_dtype == ZLM_F32 && out_dtype == ZLM_F32) { if (add) ZLM_NORM_S(float, float, true); else ZLM_NORM_S(float, float, false); }
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_F32) { if (add) ZLM_NORM_S(__nv_bfloat16, float, true); else ZLM_NORM_S(__nv_bfloat16, float, false); }
    else if (w_dtype == ZLM_F32 && out_dtype == ZLM_BF16) ZLM_NORM_S(float, __nv_bfloat16, false);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_NORM_S(__nv_bfloat16, __nv_bfloat16, false);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_NORM_S
    return e == cudaSuccess ? launch_status() : (int)e;
}

// branch, x: float [n_rows, d] contiguous; h: [n_rows, d] in out_dtype; w1, w2 of one type.
ZLM_EXPORT int zlm_norm_add_norm(const float* branch, const void* w1, float off1, float eps1, float* x, const void* w2,
                                 float off2, float eps2, int w_dtype, void* h, int out_dtype, int n_rows, int d,
                                 cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 40 * 1024) return ZLM_ERR_UNSUPPORTED;
    const bool vec = d % 4 == 0 && (uintptr_t)branch % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)h % 16 == 0 &&
                     (uintptr_t)w1 % 16 == 0 && (uintptr_t)w2 % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_NAN(TW, TO)                                                                                          \
    e = vec ? launch_pdl(norm_add_norm_kernel<TW, TO, true>, dim3(n_rows), dim3(threads), smem, stream, branch,    \
                         (const TW*)w1, off1, eps1, x, (const TW*)w2, off2, eps2, (TO*)h, d)                     \
            : launch_pdl(norm_add_norm_kernel<TW, TO, false>, dim3(n_rows), dim3(threads), smem, stream, branch,   \
                         (const TW*)w1, off1, eps1, x, (const TW*)w2, off2, eps2, (TO*)h, d)
    if (w_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_NAN(float, float);
    else if (w_dtype == ZLM_F32 && out_dtype == ZLM_BF16) ZLM_NAN(float, __nv_bfloat16);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_NAN(__nv_bfloat16, float);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_NAN(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_NAN
    return e == cudaSuccess ? launch_status() : (int)e;
}

// x rows (float, contiguous) += mult * RMS norm of branch rows (float, contiguous) with gain w + off; h (may be
// null): the new rows of x in h_dtype.
ZLM_EXPORT int zlm_norm_add_scaled(const float* branch, const void* w, int w_dtype, float off, float eps, float mult,
                                   float* x, void* h, int h_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const bool vec = d % 4 == 0 && (uintptr_t)branch % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                     (uintptr_t)h % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_NAS(TW, TO)                                                                                              \
    e = vec ? launch_pdl(norm_add_scaled_kernel<TW, TO, true>, dim3(n_rows), dim3(threads), 0, stream, branch,         \
                         (const TW*)w, off, eps, mult, x, (TO*)h, d)                                                 \
            : launch_pdl(norm_add_scaled_kernel<TW, TO, false>, dim3(n_rows), dim3(threads), 0, stream, branch,        \
                         (const TW*)w, off, eps, mult, x, (TO*)h, d)
    if (w_dtype == ZLM_F32 && (h == nullptr || h_dtype == ZLM_F32)) ZLM_NAS(float, float);
    else if (w_dtype == ZLM_F32 && h_dtype == ZLM_BF16) ZLM_NAS(float, __nv_bfloat16);
    else if (w_dtype == ZLM_BF16 && (h == nullptr || h_dtype == ZLM_F32)) ZLM_NAS(__nv_bfloat16, float);
    else if (w_dtype == ZLM_BF16 && h_dtype == ZLM_BF16) ZLM_NAS(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_NAS
    return e == cudaSuccess ? launch_status() : (int)e;
}

// x rows (float, contiguous) = RMS norm (gain w + off) of alpha * x + branch rows (float, contiguous); h (may be null):
// the new rows of x in h_dtype.
ZLM_EXPORT int zlm_sum_norm(const float* branch, const void* w, int w_dtype, float off, float eps, float alpha, float* x,
                            void* h, int h_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const bool vec = d % 4 == 0 && (uintptr_t)branch % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                     (uintptr_t)h % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_SN(TW, TO)                                                                                               \
    e = vec ? launch_pdl(sum_norm_kernel<TW, TO, true>, dim3(n_rows), dim3(threads), 0, stream, branch, (const TW*)w,  \
                         off, eps, alpha, x, (TO*)h, d)                                                              \
            : launch_pdl(sum_norm_kernel<TW, TO, false>, dim3(n_rows), dim3(threads), 0, stream, branch, (const TW*)w, \
                         off, eps, alpha, x, (TO*)h, d)
    if (w_dtype == ZLM_F32 && (h == nullptr || h_dtype == ZLM_F32)) ZLM_SN(float, float);
    else if (w_dtype == ZLM_F32 && h_dtype == ZLM_BF16) ZLM_SN(float, __nv_bfloat16);
    else if (w_dtype == ZLM_BF16 && (h == nullptr || h_dtype == ZLM_F32)) ZLM_SN(__nv_bfloat16, float);
    else if (w_dtype == ZLM_BF16 && h_dtype == ZLM_BF16) ZLM_SN(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_SN
    return e == cudaSuccess ? launch_status() : (int)e;
}

// kind 0: the squared relu, 1: the exact gelu.  out may be x.
ZLM_EXPORT int zlm_unary_act(const void* x, void* out, int dtype, long n, int kind, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind != 0 && kind != 1) return ZLM_ERR_BAD_ARG;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(unary_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, (float*)out, n, kind);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(unary_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x,
                       (__nv_bfloat16*)out, n, kind);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// out[t, i] = a[t, i] * sigmoid(g[t, i]), T rows of n elements, every operand with its own row stride.
ZLM_EXPORT int zlm_sigmoid_mul(const void* a, long a_stride, const void* g, long g_stride, void* out, long out_stride,
                               int dtype, int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const long total = (long)T * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(sigmoid_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, a_stride,
                       (const float*)g, g_stride, (float*)out, out_stride, total, n);
    else if (dtype == ZLM_BF16 && n % 8 == 0 && a_stride % 8 == 0 && g_stride % 8 == 0 && out_stride % 8 == 0 &&
             (uintptr_t)a % 16 == 0 && (uintptr_t)g % 16 == 0 && (uintptr_t)out % 16 == 0)
        e = launch_pdl(sigmoid_mul_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream,
                       (const __nv_bfloat16*)a, a_stride, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride,
                       total / 8, n / 8);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(sigmoid_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a,
                       a_stride, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, total, n);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// out rows = in rows, converted; T rows of n elements, each operand with its own row stride.
ZLM_EXPORT int zlm_convert_rows(const void* in, int in_dtype, long in_stride, void* out, int out_dtype, long out_stride,
                                int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const long total = (long)T * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
#define ZLM_CR(TI, TO)                                                                                              \
    e = launch_pdl(convert_rows_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)in, in_stride, (TO*)out, \
                   out_stride, total, n)
    if (in_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_CR(float, float);
    else if (in_dtype == ZLM_F32 && out_dtype == ZLM_BF16) ZLM_CR(float, __nv_bfloat16);
    else if (in_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_CR(__nv_bfloat16, float);
    else if (in_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_CR(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_CR
    return e == cudaSuccess ? launch_status() : (int)e;
}

// out[t, h * n + i] = a[t, h * n + i] * sigmoid(g[t, h]) * mult; T rows, every operand with its own row stride.
ZLM_EXPORT int zlm_gate_heads(const void* a, long a_stride, const void* g, long g_stride, void* out, long out_stride,
                              int dtype, int T, int heads, int n, float mult, cudaStream_t stream) {
    if (T <= 0 || heads <= 0 || n <= 0) return 0;
    const long total = (long)T * heads * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(gate_heads_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, a_stride,
                       (const float*)g, g_stride, (float*)out, out_stride, total, heads, n, mult);
    else if (dtype == ZLM_BF16 && n % 8 == 0 && a_stride % 8 == 0 && out_stride % 8 == 0 && (uintptr_t)a % 16 == 0 &&
             (uintptr_t)out % 16 == 0)
        e = launch_pdl(gate_heads_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream,
                       (const __nv_bfloat16*)a, a_stride, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride,
                       total / 8, heads * n / 8, n / 8, mult);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(gate_heads_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, a_stride,
                       (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, total, heads, n, mult);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// out rows = rmsnorm(x rows; w, eps) * sigmoid(g rows) * mult; g may be null (no gate).  x float, w float [d].
ZLM_EXPORT int zlm_norm_gate(const float* x, long x_stride, const float* w, const void* g, long g_stride, void* out,
                             long out_stride, int dtype, int n_rows, int d, float eps, float mult, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const int threads = norm_threads(d);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(norm_gate_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, w, (const float*)g,
                       g_stride, (float*)out, out_stride, d, eps, mult);
    else if (dtype == ZLM_BF16 && d % 4 == 0 && x_stride % 4 == 0 && g_stride % 4 == 0 && out_stride % 4 == 0 &&
             (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)g % 8 == 0 && (uintptr_t)out % 8 == 0)
        e = d <= 4096
                ? launch_pdl(norm_gate_vec2_kernel, dim3(n_rows), dim3(min(512, max(32, ((d / 4 + 1) / 2 + 31) / 32 * 32))), 0,
                             stream, x, x_stride, w, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, d, eps,
                             mult)
                : launch_pdl(norm_gate_vec_kernel, dim3(n_rows), dim3(256), 0, stream, x, x_stride, w,
                             (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, d, eps, mult);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(norm_gate_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, w,
                       (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, d, eps, mult);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

// x: float rows of n_heads * hd elements; every head is divided by its own root mean square; w (float, n_heads * hd,
// or null), g (rows of the output's type, or null with gate_kind 0), gate_kind 1 sigmoid, 2 silu; out in dtype.
ZLM_EXPORT int zlm_head_norm_gate(const float* x, long x_stride, const float* w, const void* g, long g_stride, void* out,
                                  long out_stride, int dtype, int n_rows, int n_heads, int hd, float eps, int gate_kind,
                                  float mult, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_heads <= 0 || hd <= 0 || gate_kind < 0 || gate_kind > 2 || (gate_kind != 0 && g == nullptr)) return ZLM_ERR_BAD_ARG;
    const long n_pairs = (long)n_rows * n_heads;
    const unsigned blocks = (unsigned)((n_pairs + HNG_WARPS - 1) / HNG_WARPS);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(HNG_WARPS * 32), 0, stream, x, x_stride, w,
                       (const float*)g, g_stride, (float*)out, out_stride, n_pairs, n_heads, hd, eps, gate_kind, mult);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(HNG_WARPS * 32), 0, stream, x, x_stride, w,
                       (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, out_stride, n_pairs, n_heads, hd, eps,
                       gate_kind, mult);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_add_row(float* x, const void* table_row, int dtype, int T, int d, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const long total = (long)T * d;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(add_row_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)table_row, total, d);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(add_row_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x,
                       (const __nv_bfloat16*)table_row, total, d);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_scale(float* x, long n, float factor, cudaStream_t stream) {
    if (n <= 0) return 0;
    cudaError_t e = launch_pdl(scale_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, factor);
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_add(float* y, const float* x, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(y, x, n);
    return launch_status();
}

ZLM_EXPORT int zlm_convert(const void* in, int in_dtype, void* out, int out_dtype, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == ZLM_F32 && out_dtype == ZLM_BF16)
        convert_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == ZLM_BF16 && out_dtype == ZLM_F32)
        convert_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    else
        return ZLM_ERR_UNSUPPORTED;
    return launch_status();
}

// out[i] = mean + std * z(key, i), i < n, z a standard normal value that depends on (key, i) only.
ZLM_EXPORT int zlm_fill_normal(void* out, int out_dtype, long n, unsigned long long key, float mean, float std_dev,
                               cudaStream_t stream) {
    if (n < 0 || (n > 0 && !out)) return ZLM_ERR_BAD_ARG;
    if (n == 0) return 0;
    long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == ZLM_BF16)
        fill_normal_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, mean, std_dev);
    else if (out_dtype == ZLM_F32)
        fill_normal_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, n, key, mean, std_dev);
    else
        return ZLM_ERR_UNSUPPORTED;
    return launch_status();
}
