// Parts of decoders whose blocks norm AFTER the residual sum, and of the mixers such blocks use:
//
//   embedding times a scale                         h[t,:] = s * E[id_t,:]
//   rounding of the stream for the first sublayer   x = round(h)
//   scaled sum + RMS norm, in place                 h <- w * rms(alpha h + y (+ b));  x = round(h)
//   whole-row RMS norm with a sigmoid gate          out = w * rms(o) * sigmoid(g)
//   difference of two attention maps                out = (1 - c) * rms(a1 - lambda a2) * sigmoid(g)
//   queries, latent and rotated key of a latent attention, with the cache write
//   a bias on every row
//
// The stream, every sum of squares, every norm, gate and rotation are fp32; what is handed to a matrix
// product is rounded once, at the end.  The reference engine has only the pre-norm block
// (crates/infer-worker/src/components/decoder_block.rs:13-32); these stand beside its fused add + RMSNorm.
#include "common.cuh"

namespace {

template <typename TW>
__device__ __forceinline__ float wv(const TW* w, int i) { return w ? to_f32<TW>(w[i]) : 1.f; }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

inline int ew_blocks(long long n) { return (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8); }

template <typename TE>
__global__ void embed_scaled_kernel(const int* __restrict__ ids, const TE* __restrict__ table, float scale,
                                    float* __restrict__ out, int d, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const TE* row = table + (size_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)t * d + i] = to_f32<TE>(row[i]) * scale;
}

template <typename TO>
__global__ void round_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(x[i]);
}

// One CTA a row.  u = alpha h + y (+ b) is kept in shared memory between the sum of squares and the write.
template <typename TD, typename TW, typename TO>
__global__ void scale_add_norm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const TW* __restrict__ bias,
                                      float alpha, const TW* __restrict__ w, float eps, TO* __restrict__ act, int d) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    float* u = sm;
    float* red = sm + d;
    const size_t r = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = alpha * h[r * d + i];
        if (delta) v += to_f32<TD>(delta[r * d + i]);
        if (bias) v += to_f32<TW>(bias[i]);
        u[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float y = u[i] * inv * wv(w, i);
        h[r * d + i] = y;
        if (act) act[r * d + i] = from_f32<TO>(y);
    }
}

// out[t,:] = o[t,:] / sqrt(mean(o[t,:]^2) + eps) * w * sigmoid(gate[t,:]); one CTA a row, o read twice.
template <typename TG, typename TW, typename TO>
__global__ void row_norm_gate_kernel(const float* __restrict__ o, const TG* __restrict__ gate, int gate_stride,
                                     const TW* __restrict__ w, float eps, TO* __restrict__ out, int n) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* x = o + r * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = x[i] * inv * wv(w, i);
        if (gate) y *= sigmoid_f(to_f32<TG>(gate[r * gate_stride + i]));
        out[r * n + i] = from_f32<TO>(y);
    }
}

// a [T][H][2][vd] fp32 (the two maps of a head side by side); a warp a (token, head).
template <typename TG, typename TO>
__global__ void diff_combine_kernel(const float* __restrict__ a, float lambda, float out_scale, float eps,
                                    const TG* __restrict__ gate, int gate_stride, TO* __restrict__ out,
                                    int tokens, int H, int vd) {
    pdl_trigger();
    pdl_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)tokens * H) return;
    const int t = (int)(item / H), hh = (int)(item % H);
    const float* a1 = a + ((size_t)t * H + hh) * 2 * vd;
    const float* a2 = a1 + vd;
    float ss = 0.f;
    for (int i = lane; i < vd; i += 32) {
        const float o = a1[i] - lambda * a2[i];
        ss += o * o;
    }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)vd + eps);
    for (int i = lane; i < vd; i += 32) {
        float y = (a1[i] - lambda * a2[i]) * inv;
        if (gate) y *= sigmoid_f(to_f32<TG>(gate[(size_t)t * gate_stride + (size_t)hh * vd + i]));
        out[((size_t)t * H + hh) * vd + i] = from_f32<TO>(y);
    }
}

// proj [T][>= H*(d+r) + rank + r]: per head the plain part (d) and the part to rotate (r), then the
// low-rank vector (rank) and the shared key part to rotate (r).  One CTA a token:
//   q_plain [T][H*d]            the plain parts, rounded (one operand of the product with the keys' up-projection)
//   q_full  [T][H*(rank+r)]     only the last r channels of every head: the rotated parts
//   cache row [rank + r]        w * rms(low-rank vector), then the rotated shared key part
// Pairs (2i, 2i+1) turn by the angles of cos/sin [positions][r/2].
template <typename TI, typename TW, typename TA>
__global__ void latent_prepare_kernel(const TI* __restrict__ proj, int row_stride, const TW* __restrict__ c_w, float eps,
                                      const int* __restrict__ positions, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const int* __restrict__ slot_of_token,
                                      TA* __restrict__ cache, TA* __restrict__ q_plain, TA* __restrict__ q_full,
                                      int H, int d, int r, int rank, const TI* __restrict__ low_base, int low_stride,
                                      int interleaved) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
    const TI* row = proj + (size_t)t * row_stride;
    const int half = r >> 1;
    const int pos = positions[t];
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    for (int e = tid; e < H * d; e += nth) {
        const int hh = e / d, i = e - hh * d;
        q_plain[(size_t)t * H * d + e] = from_f32<TA>(to_f32<TI>(row[(size_t)hh * (d + r) + i]));
    }
    for (int e = tid; e < H * half; e += nth) {
        const int hh = e / half, i = e - hh * half;
        const TI* x = row + (size_t)hh * (d + r) + d;
        // the pair that turns together: channels (2i, 2i+1), or (i, i + r/2)
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32<TI>(x[ia]), v = to_f32<TI>(x[ib]), c = cr[i], s = sr[i];
        TA* o = q_full + ((size_t)t * H + hh) * (rank + r) + rank;
        o[ia] = from_f32<TA>(u * c - v * s);
        o[ib] = from_f32<TA>(v * c + u * s);
    }
    // the low-rank vector and the shared key part: behind the queries in the same row, or rows of their own
    const TI* low = low_base ? low_base + (size_t)t * low_stride : row + (size_t)H * (d + r);
    float ss = 0.f;
    for (int i = tid; i < rank; i += nth) {
        const float v = to_f32<TI>(low[i]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    if (!cache || !slot_of_token) return;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    TA* dst = cache + (size_t)slot * (rank + r);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = tid; i < rank; i += nth) dst[i] = from_f32<TA>(to_f32<TI>(low[i]) * inv * wv(c_w, i));
    for (int i = tid; i < half; i += nth) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32<TI>(low[rank + ia]), v = to_f32<TI>(low[rank + ib]), c = cr[i], s = sr[i];
        dst[rank + ia] = from_f32<TA>(u * c - v * s);
        dst[rank + ib] = from_f32<TA>(v * c + u * s);
    }
}

template <typename TX, typename TW>
__global__ void bias_rows_kernel(TX* __restrict__ x, const TW* __restrict__ bias, long long total, int n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f32<TX>(to_f32<TX>(x[i]) + to_f32<TW>(bias[i % n]));
}

}  // namespace

RI_API int ri_embed_scaled(const int* ids, const void* table, int table_dtype, float scale, float* out, int tokens,
                           int d, int vocab, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == RI_BF16)
        RI_CHECKED(ri_launch(embed_scaled_kernel<bf16>, dim3(tokens), dim3(256), 0, s, ids, (const bf16*)table, scale, out, d, vocab));
    else
        RI_CHECKED(ri_launch(embed_scaled_kernel<float>, dim3(tokens), dim3(256), 0, s, ids, (const float*)table, scale, out, d, vocab));
    return ri_launch_status();
}

RI_API int ri_round_rows(const float* x, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == RI_BF16)
        RI_CHECKED(ri_launch(round_rows_kernel<bf16>, dim3(ew_blocks(n)), dim3(256), 0, s, x, (bf16*)out, n));
    else
        RI_CHECKED(ri_launch(round_rows_kernel<float>, dim3(ew_blocks(n)), dim3(256), 0, s, x, (float*)out, n));
    return ri_launch_status();
}

// h fp32 [rows][d], in place: h <- w * rms(alpha h + delta + bias); act (may be null) gets h rounded.
// delta_dtype / w_dtype (of w and bias) / act_dtype: RI_F32 or RI_BF16.
RI_API int ri_scale_add_norm(float* h, const void* delta, int delta_dtype, const void* bias, float alpha, const void* w,
                             int w_dtype, float eps, void* act, int act_dtype, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(d + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define RI_SAN(TD, TW, TO) do { \
        static bool configured = false; \
        if (!configured && smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(scale_add_norm_kernel<TD, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; } \
        RI_CHECKED(ri_launch(scale_add_norm_kernel<TD, TW, TO>, dim3(rows), dim3(d >= 2048 ? 512 : 256), smem, s, h, \
            (const TD*)delta, (const TW*)bias, alpha, (const TW*)w, eps, (TO*)act, d)); } while (0)
#define RI_SAN2(TD, TW) do { if (act_dtype == RI_BF16) RI_SAN(TD, TW, bf16); else RI_SAN(TD, TW, float); } while (0)
    if (delta_dtype == RI_BF16 && w_dtype == RI_BF16) RI_SAN2(bf16, bf16);
    else if (delta_dtype == RI_BF16) RI_SAN2(bf16, float);
    else if (w_dtype == RI_BF16) RI_SAN2(float, bf16);
    else RI_SAN2(float, float);
#undef RI_SAN2
#undef RI_SAN
    return ri_launch_status();
}

RI_API int ri_row_norm_gate(const float* o, const void* gate, int gate_dtype, int gate_stride, const void* w, int w_dtype,
                            float eps, void* out, int out_dtype, int rows, int n, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_RNG(TG, TW, TO) RI_CHECKED(ri_launch(row_norm_gate_kernel<TG, TW, TO>, dim3(rows), dim3(n >= 2048 ? 512 : 256), 0, s, \
        o, (const TG*)gate, gate_stride, (const TW*)w, eps, (TO*)out, n))
#define RI_RNG2(TG, TW) do { if (out_dtype == RI_BF16) RI_RNG(TG, TW, bf16); else RI_RNG(TG, TW, float); } while (0)
    if (gate_dtype == RI_BF16 && w_dtype == RI_BF16) RI_RNG2(bf16, bf16);
    else if (gate_dtype == RI_BF16) RI_RNG2(bf16, float);
    else if (w_dtype == RI_BF16) RI_RNG2(float, bf16);
    else RI_RNG2(float, float);
#undef RI_RNG2
#undef RI_RNG
    return ri_launch_status();
}

RI_API int ri_diff_combine(const float* a, float lambda, float out_scale, float eps, const void* gate, int gate_dtype,
                           int gate_stride, void* out, int out_dtype, int tokens, int H, int vd, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)tokens * H;
    const int warps = 4;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
#define RI_DC(TG, TO) RI_CHECKED(ri_launch(diff_combine_kernel<TG, TO>, grid, dim3(32 * warps), 0, s, a, lambda, out_scale, eps, \
        (const TG*)gate, gate_stride, (TO*)out, tokens, H, vd))
    if (gate_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_DC(bf16, bf16); else RI_DC(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_DC(float, bf16); else RI_DC(float, float); }
#undef RI_DC
    return ri_launch_status();
}

// in_dtype: of proj (and low); act_dtype: of q_plain, q_full and the cache; w_dtype: of the low-rank vector's norm weight.
// low (may be null): rows [rank + r] of `low_stride` elements that hold the low-rank vector and the shared key part
// where they do not follow the queries in proj's rows.  interleaved: rotary pairs (2i, 2i+1), else (i, i + r/2).
// The cache of one layer is [pages][page][rank + r]: a token's row lies at slot_of_token[t] * (rank + r).
RI_API int ri_latent_prepare(const void* proj, int in_dtype, int row_stride, const void* c_w, int w_dtype, float eps,
                             const int* positions, const float* cos_t, const float* sin_t, const int* slot_of_token,
                             void* cache, void* q_plain, void* q_full, int act_dtype, int tokens, int H, int d, int r,
                             int rank, const void* low, int low_stride, int interleaved, void* stream) {
    if (tokens <= 0) return 0;
    if (r < 0 || (r & 1) || (r > 0 && (!cos_t || !sin_t || !positions))) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_LP(TI, TW, TA) RI_CHECKED(ri_launch(latent_prepare_kernel<TI, TW, TA>, dim3(tokens), dim3(256), 0, s, (const TI*)proj, \
        row_stride, (const TW*)c_w, eps, positions, cos_t, sin_t, slot_of_token, (TA*)cache, (TA*)q_plain, (TA*)q_full, H, d, r, rank, \
        (const TI*)low, low_stride, interleaved))
    if (act_dtype == RI_BF16) {
        if (in_dtype == RI_BF16) { if (w_dtype == RI_BF16) RI_LP(bf16, bf16, bf16); else RI_LP(bf16, float, bf16); }
        else { if (w_dtype == RI_BF16) RI_LP(float, bf16, bf16); else RI_LP(float, float, bf16); }
    } else {
        if (in_dtype != RI_F32) return (int)cudaErrorInvalidValue;
        if (w_dtype == RI_BF16) RI_LP(float, bf16, float); else RI_LP(float, float, float);
    }
#undef RI_LP
    return ri_launch_status();
}

RI_API int ri_bias_rows(void* x, int x_dtype, const void* bias, int w_dtype, int rows, int n, void* stream) {
    const long long total = (long long)rows * n;
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_BR(TX, TW) RI_CHECKED(ri_launch(bias_rows_kernel<TX, TW>, dim3(ew_blocks(total)), dim3(256), 0, s, (TX*)x, (const TW*)bias, total, n))
    if (x_dtype == RI_BF16) { if (w_dtype == RI_BF16) RI_BR(bf16, bf16); else RI_BR(bf16, float); }
    else { if (w_dtype == RI_BF16) RI_BR(float, bf16); else RI_BR(float, float); }
#undef RI_BR
    return ri_launch_status();
}
