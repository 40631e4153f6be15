// Row-wise kernels of decoders whose blocks are not the Llama shape: an embedding with
// sinusoidal positions, layer norm around a sublayer (the norm of a sublayer's output fused
// with the add into the stream and with the norm that the next sublayer reads), per-head
// norms of q, k and v fused with the write into cache pages, the gated per-head norm that
// closes a linear-attention mixer, element-wise activations and a weighted sum of two
// mixers.  All arithmetic is fp32 (angles fp64); storage is fp32 or bf16 by template.
#include "common.cuh"

namespace {

// ------------------------------------------------- embedding + sinusoidal positions
// out[t, 2i] = E[id, 2i] + sin(p f_i), out[t, 2i+1] = E[id, 2i+1] + cos(p f_i); the f_i come
// as doubles from the host and the angle is formed and reduced in double, so that the table
// entry is exact to fp32 rounding at any position.
template <typename TW>
__global__ void embed_sinusoid_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                      const TW* __restrict__ table, const double* __restrict__ freq,
                                      float* __restrict__ out, int d, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const double p = (double)positions[t];
    const bool ok = id >= 0 && id < vocab;           // ids are validated on the host; never read outside
    const TW* src = table + (size_t)(ok ? id : 0) * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const double ang = p * freq[i >> 1];
        const float pe = (float)((i & 1) ? cos(ang) : sin(ang));
        o[i] = (ok ? to_f32<TW>(src[i]) : 0.f) + pe;
    }
}

// ------------------------------------------------------------ layer norm around a sublayer
// For row r (src = rows ? rows[r] : r):
//   v = h[src] + (delta ? LN(delta[src]; post_w, post_b) : 0)     written back to h unless `rows`
//   out[r] = LN(v; next_w, next_b)                                  when `out` is given
// LN(x; w, b) = (x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations (two passes).
template <typename T>
__device__ __forceinline__ float wval(const T* w, int i, float dflt) { return w ? to_f32<T>(w[i]) : dflt; }

template <typename TA, typename TW>
__global__ void sandwich_norm_kernel(float* __restrict__ h, const TA* __restrict__ delta,
                                     const TW* __restrict__ post_w, const TW* __restrict__ post_b,
                                     const TW* __restrict__ next_w, const TW* __restrict__ next_b,
                                     TA* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hp = h + (size_t)src * d;
    const float inv_d = 1.0f / (float)d;
    if (delta) {
        const TA* dp = delta + (size_t)src * d;
        float s = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = to_f32<TA>(dp[i]);
            row[i] = v;
            s += v;
        }
        const float mean = block_sum(s, red) * inv_d;
        float q = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float c = row[i] - mean;
            q += c * c;
        }
        const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float y = (row[i] - mean) * inv * wval(post_w, i, 1.f) + wval(post_b, i, 0.f);
            const float v = hp[i] + y;
            if (!rows) hp[i] = v;
            row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) row[i] = hp[i];
    }
    if (!out) return;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) * inv_d;
    float q = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float c = row[i] - mean;
        q += c * c;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
    TA* op = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        op[i] = from_f32<TA>((row[i] - mean) * inv * wval(next_w, i, 1.f) + wval(next_b, i, 0.f));
}

// The same for bf16 activations and rows of a multiple of 8 up to 8 * 1024 elements: a thread keeps its 8
// elements in registers from the first load to the last store and moves 16 or 32 bytes per access.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}
template <typename TW>
__device__ __forceinline__ void weights8(const TW* w, int i0, float dflt, float (&f)[8]) {
    if (!w) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = dflt;
    } else if (sizeof(TW) == 2) {
        unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(w) + i0), f);
    } else {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i0);
        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i0 + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}
// mean and 1 / sqrt(variance + eps) of a row spread over the block, 8 elements a thread (two passes)
__device__ __forceinline__ void row_stats(const float (&v)[8], bool active, float inv_d, float eps, float* red,
                                          float& mean, float& inv) {
    float s = 0.f;
    if (active) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s += v[i];
    }
    mean = block_sum(s, red) * inv_d;
    float q = 0.f;
    if (active) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q += (v[i] - mean) * (v[i] - mean);
    }
    inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
}

template <typename TW>
__global__ void sandwich_norm_bf16x8_kernel(float* __restrict__ h, const bf16* __restrict__ delta,
                                            const TW* __restrict__ post_w, const TW* __restrict__ post_b,
                                            const TW* __restrict__ next_w, const TW* __restrict__ next_b,
                                            bf16* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const int i0 = threadIdx.x * 8;
    const bool active = i0 < d;
    const float inv_d = 1.0f / (float)d;
    float* hp = h + (size_t)src * d + i0;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (active) {
        const float4 a = *reinterpret_cast<const float4*>(hp);
        const float4 b = *reinterpret_cast<const float4*>(hp + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    if (delta) {
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = 0.f;
        if (active) unpack8(*reinterpret_cast<const uint4*>(delta + (size_t)src * d + i0), x);
        float mean, inv;
        row_stats(x, active, inv_d, eps, red, mean, inv);
        if (active) {
            float w[8], b[8];
            weights8(post_w, i0, 1.f, w);
            weights8(post_b, i0, 0.f, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] += (x[i] - mean) * inv * w[i] + b[i];
            if (!rows) {
                *reinterpret_cast<float4*>(hp) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(hp + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
    }
    if (!out) return;
    float mean, inv;
    row_stats(v, active, inv_d, eps, red, mean, inv);
    if (!active) return;
    float w[8], b[8], y[8];
    weights8(next_w, i0, 1.f, w);
    weights8(next_b, i0, 0.f, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = (v[i] - mean) * inv * w[i] + b[i];
    *reinterpret_cast<uint4*>(out + (size_t)r * d + i0) = pack8(y);
}

// ----------------------------------------- per-head norms of q, k, v + write into the pages
// qkv row: q heads [Hq][dk], k heads [Hkv][dk], v heads [Hkv][dv].  One warp per (token, head):
// q and k are divided by their root mean square over dk and multiplied by a weight of size dk
// shared by all heads (a null weight leaves them as they are); v is divided by its root mean
// square over dv when `v_norm` is set.  q is normed in place; k and v go to the token's slot of
// the cache (a page holds keys [Hkv][page][dk], then values [Hkv][page][dv]); slot < 0: no write.
template <typename TA, typename TW>
__global__ void head_norm_scatter_kernel(TA* __restrict__ qkv, int row_stride, const TW* __restrict__ q_w,
                                         const TW* __restrict__ k_w, int v_norm, float eps,
                                         const int* __restrict__ slot_of_token, TA* __restrict__ cache,
                                         int tokens, int Hq, int Hkv, int dk, int dv, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int heads = Hq + 2 * Hkv;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), hh = (int)(item % heads);
    TA* rowp = qkv + (size_t)t * row_stride;
    TA* x;
    int n;
    const TW* w = nullptr;
    bool norm;
    TA* dst = nullptr;
    const int slot = (cache && slot_of_token) ? slot_of_token[t] : -1;
    const size_t page_elems = (size_t)Hkv * page_size * (dk + dv);
    if (hh < Hq) {
        x = rowp + (size_t)hh * dk; n = dk; w = q_w; norm = q_w != nullptr;
    } else if (hh < Hq + Hkv) {
        const int g = hh - Hq;
        x = rowp + (size_t)Hq * dk + (size_t)g * dk; n = dk; w = k_w; norm = k_w != nullptr;
        if (slot >= 0)
            dst = cache + (size_t)(slot / page_size) * page_elems + ((size_t)g * page_size + slot % page_size) * dk;
    } else {
        const int g = hh - Hq - Hkv;
        x = rowp + (size_t)(Hq + Hkv) * dk + (size_t)g * dv; n = dv; norm = v_norm != 0;
        if (slot >= 0)
            dst = cache + (size_t)(slot / page_size) * page_elems + (size_t)Hkv * page_size * dk
                  + ((size_t)g * page_size + slot % page_size) * dv;
    }
    float inv = 1.f;
    if (norm) {
        float ss = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float v = to_f32<TA>(x[i]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)n + eps);
    }
    const bool in_place = hh < Hq;
    if (!in_place && !dst) return;
    if (in_place && !norm) return;
    for (int i = lane; i < n; i += 32) {
        float v = to_f32<TA>(x[i]);
        if (norm) v = v * inv * wval(w, i, 1.f);
        const TA y = from_f32<TA>(v);
        if (in_place) x[i] = y; else dst[i] = y;
    }
}

// --------------------------------------------------- gated per-head norm of a mixer's output
// o [T, H*dv] fp32 (what the recurrence returned).  One warp per (token, head):
//   out = o / sqrt(mean_head(o^2) + eps) * w * act(gate),  act = silu (0) or sigmoid (1);
// w has dv entries shared by the heads (w_per_head 0) or H*dv entries (1).
template <typename TA, typename TW>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const TA* __restrict__ gate, int gate_stride,
                                       const TW* __restrict__ w, int w_per_head, int act, float eps,
                                       TA* __restrict__ out, int tokens, int H, int dv) {
    pdl_trigger();
    pdl_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)tokens * H) return;
    const int t = (int)(item / H), hh = (int)(item % H);
    const float* x = o + ((size_t)t * H + hh) * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const TA* gp = gate + (size_t)t * gate_stride + (size_t)hh * dv;
    const TW* wp = w + (w_per_head ? (size_t)hh * dv : 0);
    TA* op = out + ((size_t)t * H + hh) * dv;
    for (int i = lane; i < dv; i += 32) {
        const float g = to_f32<TA>(gp[i]);
        const float sg = 1.0f / (1.0f + expf(-g));
        op[i] = from_f32<TA>(x[i] * inv * to_f32<TW>(wp[i]) * (act == 0 ? g * sg : sg));
    }
}

// --------------------------------------------------------------- element-wise activations
// kind 0: gelu with erf; 1: tanh; 2: gelu with tanh, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)));
// 3: the square of relu; 4: silu, z / (1 + exp(-z))
__device__ __forceinline__ float activate(float z, int kind) {
    if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    if (kind == 1) return tanhf(z);
    if (kind == 2) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    if (kind == 3) return z > 0.f ? z * z : 0.f;
    return z / (1.0f + expf(-z));
}

template <typename TA>
__global__ void activation_kernel(const TA* __restrict__ x, TA* __restrict__ out, long long n, int kind) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TA>(activate(to_f32<TA>(x[i]), kind));
}

// the first `cols` columns of every row of x [rows][stride], in place
template <typename TA>
__global__ void activation_cols_kernel(TA* __restrict__ x, int stride, long long total, int cols, int kind) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols;
        TA* p = x + r * stride + (i - r * cols);
        *p = from_f32<TA>(activate(to_f32<TA>(*p), kind));
    }
}

// out = sa * a + sb * b
template <typename TA>
__global__ void scaled_sum_kernel(const TA* __restrict__ a, const TA* __restrict__ b, float sa, float sb,
                                  TA* __restrict__ out, long long n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TA>(sa * to_f32<TA>(a[i]) + sb * to_f32<TA>(b[i]));
}

// ------------------------------------------------ what the linear-attention recurrences are fed
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// z [T, n] fp32, in place: z <- sigmoid(z + bias)^(1/tau), formed as exp(log_sigmoid(.) / tau) so that a
// decay close to one keeps its distance from one.
template <typename TW>
__global__ void gated_decay_kernel(float* __restrict__ z, const TW* __restrict__ bias, float inv_tau, long long total, int n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const float x = z[i] + (bias ? to_f32<TW>(bias[i % n]) : 0.f);
        z[i] = expf(log_sigmoid_f(x) * inv_tau);
    }
}

// One warp per (token, head) of a delta-rule mixer: from the key k [dk], the logits of the removal rate
// za [dk] and of the decay zw [dk] (fp32, in place) it makes
//   zw <- exp(-decay_rate * sigmoid(zw + zw_bias)),  u = k / sqrt(|k|^2 + unit_eps),  au = sigmoid(za + za_bias) * u.
template <typename TA, typename TW>
__global__ void delta_prepare_kernel(const TA* __restrict__ k, int k_stride, const TA* __restrict__ za, int za_stride,
                                     const TW* __restrict__ za_bias, float* __restrict__ zw, const TW* __restrict__ zw_bias,
                                     float decay_rate, float unit_eps, float* __restrict__ u, float* __restrict__ au,
                                     int tokens, int H, int dk) {
    pdl_trigger();
    pdl_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)tokens * H) return;
    const int t = (int)(item / H), hh = (int)(item % H);
    const TA* kp = k + (size_t)t * k_stride + (size_t)hh * dk;
    const TA* ap = za + (size_t)t * za_stride + (size_t)hh * dk;
    const size_t base = ((size_t)t * H + hh) * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) {
        const float x = to_f32<TA>(kp[i]);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + unit_eps);
    for (int i = lane; i < dk; i += 32) {
        const int c = hh * dk + i;
        const float unit = to_f32<TA>(kp[i]) * inv;
        u[base + i] = unit;
        au[base + i] = sigmoid_f(to_f32<TA>(ap[i]) + (za_bias ? to_f32<TW>(za_bias[c]) : 0.f)) * unit;
        zw[base + i] = expf(-decay_rate * sigmoid_f(zw[base + i] + (zw_bias ? to_f32<TW>(zw_bias[c]) : 0.f)));
    }
}

inline int ew_blocks(long long n) { return (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8); }
}  // namespace

RI_API int ri_embed_sinusoid(const int* ids, const int* positions, const void* table, int table_dtype,
                             const double* freq, float* out, int tokens, int d, int vocab, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == RI_BF16)
        RI_CHECKED(ri_launch(embed_sinusoid_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, ids, positions,
                             (const bf16*)table, freq, out, d, vocab));
    else
        RI_CHECKED(ri_launch(embed_sinusoid_kernel<float>, dim3(tokens), dim3(threads), 0, s, ids, positions,
                             (const float*)table, freq, out, d, vocab));
    return ri_launch_status();
}

template <typename TA, typename TW>
static int sandwich_norm_launch(float* h, const void* delta, const void* post_w, const void* post_b,
                                const void* next_w, const void* next_b, void* out, const int* rows,
                                int n_rows, int d, float eps, cudaStream_t s) {
    const size_t smem = (size_t)d * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(sandwich_norm_kernel<TA, TW>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int threads = d >= 2048 ? 512 : d >= 512 ? 256 : 128;
    RI_CHECKED(ri_launch(sandwich_norm_kernel<TA, TW>, dim3(n_rows), dim3(threads), smem, s, h, (const TA*)delta,
                         (const TW*)post_w, (const TW*)post_b, (const TW*)next_w, (const TW*)next_b, (TA*)out,
                         rows, d, eps));
    return ri_launch_status();
}

// act_dtype: of delta and out; w_dtype: of the four weight vectors (each may be null)
RI_API int ri_sandwich_norm(float* h, const void* delta, const void* post_w, const void* post_b,
                            const void* next_w, const void* next_b, void* out, int act_dtype, int w_dtype,
                            const int* rows, int n_rows, int d, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if ((size_t)d * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (act_dtype == RI_BF16 && d % 8 == 0 && d <= 8 * 1024 && aligned(h) && aligned(delta) && aligned(out) &&
        aligned(post_w) && aligned(post_b) && aligned(next_w) && aligned(next_b)) {
        const int threads = ((d / 8 + 31) / 32) * 32;
        if (w_dtype == RI_BF16)
            RI_CHECKED(ri_launch(sandwich_norm_bf16x8_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, h, (const bf16*)delta,
                                 (const bf16*)post_w, (const bf16*)post_b, (const bf16*)next_w, (const bf16*)next_b,
                                 (bf16*)out, rows, d, eps));
        else
            RI_CHECKED(ri_launch(sandwich_norm_bf16x8_kernel<float>, dim3(n_rows), dim3(threads), 0, s, h, (const bf16*)delta,
                                 (const float*)post_w, (const float*)post_b, (const float*)next_w, (const float*)next_b,
                                 (bf16*)out, rows, d, eps));
        return ri_launch_status();
    }
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16)
        return sandwich_norm_launch<bf16, bf16>(h, delta, post_w, post_b, next_w, next_b, out, rows, n_rows, d, eps, s);
    if (act_dtype == RI_BF16)
        return sandwich_norm_launch<bf16, float>(h, delta, post_w, post_b, next_w, next_b, out, rows, n_rows, d, eps, s);
    if (w_dtype == RI_BF16)
        return sandwich_norm_launch<float, bf16>(h, delta, post_w, post_b, next_w, next_b, out, rows, n_rows, d, eps, s);
    return sandwich_norm_launch<float, float>(h, delta, post_w, post_b, next_w, next_b, out, rows, n_rows, d, eps, s);
}

RI_API int ri_head_norm_scatter(void* qkv, int act_dtype, int row_stride, const void* q_w, const void* k_w,
                                int w_dtype, int v_norm, float eps, const int* slot_of_token, void* cache,
                                int tokens, int Hq, int Hkv, int dk, int dv, int page_size, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)tokens * (Hq + 2 * Hkv);
    const int warps = 4;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
#define RI_HNS(TA, TW) RI_CHECKED(ri_launch(head_norm_scatter_kernel<TA, TW>, grid, dim3(32 * warps), 0, s, (TA*)qkv, \
        row_stride, (const TW*)q_w, (const TW*)k_w, v_norm, eps, slot_of_token, (TA*)cache, tokens, Hq, Hkv, dk, dv, page_size))
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16) RI_HNS(bf16, bf16);
    else if (act_dtype == RI_BF16) RI_HNS(bf16, float);
    else if (w_dtype == RI_BF16) RI_HNS(float, bf16);
    else RI_HNS(float, float);
#undef RI_HNS
    return ri_launch_status();
}

RI_API int ri_gated_head_norm(const float* o, const void* gate, int gate_stride, const void* w, int w_dtype,
                              int w_per_head, int act, float eps, void* out, int act_dtype, int tokens, int H,
                              int dv, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)tokens * H;
    const int warps = 4;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
#define RI_GHN(TA, TW) RI_CHECKED(ri_launch(gated_head_norm_kernel<TA, TW>, grid, dim3(32 * warps), 0, s, o, \
        (const TA*)gate, gate_stride, (const TW*)w, w_per_head, act, eps, (TA*)out, tokens, H, dv))
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16) RI_GHN(bf16, bf16);
    else if (act_dtype == RI_BF16) RI_GHN(bf16, float);
    else if (w_dtype == RI_BF16) RI_GHN(float, bf16);
    else RI_GHN(float, float);
#undef RI_GHN
    return ri_launch_status();
}

RI_API int ri_activation(const void* x, void* out, int act_dtype, long long n, int kind, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == RI_BF16)
        RI_CHECKED(ri_launch(activation_kernel<bf16>, dim3(ew_blocks(n)), dim3(256), 0, s, (const bf16*)x, (bf16*)out, n, kind));
    else
        RI_CHECKED(ri_launch(activation_kernel<float>, dim3(ew_blocks(n)), dim3(256), 0, s, (const float*)x, (float*)out, n, kind));
    return ri_launch_status();
}

RI_API int ri_activation_cols(void* x, int act_dtype, int stride, int rows, int cols, int kind, void* stream) {
    const long long total = (long long)rows * cols;
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == RI_BF16)
        RI_CHECKED(ri_launch(activation_cols_kernel<bf16>, dim3(ew_blocks(total)), dim3(256), 0, s, (bf16*)x, stride, total, cols, kind));
    else
        RI_CHECKED(ri_launch(activation_cols_kernel<float>, dim3(ew_blocks(total)), dim3(256), 0, s, (float*)x, stride, total, cols, kind));
    return ri_launch_status();
}

RI_API int ri_scaled_sum(const void* a, const void* b, float sa, float sb, void* out, int act_dtype, long long n,
                         void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == RI_BF16)
        RI_CHECKED(ri_launch(scaled_sum_kernel<bf16>, dim3(ew_blocks(n)), dim3(256), 0, s, (const bf16*)a, (const bf16*)b,
                             sa, sb, (bf16*)out, n));
    else
        RI_CHECKED(ri_launch(scaled_sum_kernel<float>, dim3(ew_blocks(n)), dim3(256), 0, s, (const float*)a,
                             (const float*)b, sa, sb, (float*)out, n));
    return ri_launch_status();
}

RI_API int ri_gated_decay(float* z, const void* bias, int w_dtype, float inv_tau, int tokens, int n, void* stream) {
    const long long total = (long long)tokens * n;
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (w_dtype == RI_BF16)
        RI_CHECKED(ri_launch(gated_decay_kernel<bf16>, dim3(ew_blocks(total)), dim3(256), 0, s, z, (const bf16*)bias, inv_tau, total, n));
    else
        RI_CHECKED(ri_launch(gated_decay_kernel<float>, dim3(ew_blocks(total)), dim3(256), 0, s, z, (const float*)bias, inv_tau, total, n));
    return ri_launch_status();
}

RI_API int ri_delta_prepare(const void* k, int k_stride, const void* za, int za_stride, const void* za_bias, float* zw,
                            const void* zw_bias, int act_dtype, int w_dtype, float decay_rate, float unit_eps, float* u,
                            float* au, int tokens, int H, int dk, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)tokens * H;
    const int warps = 4;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
#define RI_DP(TA, TW) RI_CHECKED(ri_launch(delta_prepare_kernel<TA, TW>, grid, dim3(32 * warps), 0, s, (const TA*)k, k_stride, \
        (const TA*)za, za_stride, (const TW*)za_bias, zw, (const TW*)zw_bias, decay_rate, unit_eps, u, au, tokens, H, dk))
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16) RI_DP(bf16, bf16);
    else if (act_dtype == RI_BF16) RI_DP(bf16, float);
    else if (w_dtype == RI_BF16) RI_DP(float, bf16);
    else RI_DP(float, float);
#undef RI_DP
    return ri_launch_status();
}
