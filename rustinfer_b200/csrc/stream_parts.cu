// Parts of decoders with several residual streams and with attention whose q, k, v need more than a
// rotation before they meet the cache: the normed embedding, the read / update of the streams fused
// with the RMS norm, and the kernel that turns a 32-bit q,k,v projection into rounded queries and cached
// keys and values.  All arithmetic is fp32; activations are fp32 or bf16 by the engine's dtype.
#include "common.cuh"

namespace {

template <typename TW>
__device__ __forceinline__ float wv(const TW* w, int i) { return w ? to_f32<TW>(w[i]) : 1.f; }

// ------------------------------------------------------------------ embedding + RMS norm
// out[t, :] (fp32) = E[ids[t], :] / sqrt(mean(E[ids[t], :]^2) + eps) * w.  One CTA a token.
template <typename TE, typename TW>
__global__ void embed_rmsnorm_kernel(const int* __restrict__ ids, const TE* __restrict__ table, const TW* __restrict__ w,
                                     float eps, float* __restrict__ out, int d, int vocab) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    float* row = sm;                       // [d]
    float* red = sm + d;                   // [33]
    const int t = blockIdx.x;
    int id = ids[t];
    id = min(max(id, 0), vocab - 1);
    const TE* src = table + (size_t)id * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = to_f32<TE>(src[i]);
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)t * d + i] = row[i] * inv * to_f32<TW>(w[i]);
}

// -------------------------------------------------- several streams: update, weighted sum, norm
// X [S][T][d] fp32 (with `fresh` only X[0] is written yet and stands for every stream).  For row r
// (token rows[r], or r):
//   if y:    X'_t = sum_s mix[s][t] X_s + write[t] y        (stored back unless `rows` is given)
//   u = sum_s read[s] X'_s                                  (read null: every weight 1)
//   out = w ? u / sqrt(mean(u^2) + eps) * w : u
// Sums run over s = 0, 1, .. in that order.
constexpr int MAX_STREAMS = 8;

// four consecutive elements at index i (a multiple of 4) of a row whose start is 16-byte aligned
__device__ __forceinline__ void load4(const float* p, int i, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p + i);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, int i, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p + i);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, int i, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, int i, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const unsigned*>(&a); t.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p + i) = t;
}

template <typename TY, typename TW, typename TO, int VEC>
__global__ void hyper_collect_kernel(float* __restrict__ X, int fresh, const TY* __restrict__ y,
                                     const float* __restrict__ mix, const float* __restrict__ write,
                                     const float* __restrict__ read, const TW* __restrict__ w, float eps,
                                     TO* __restrict__ out, const int* __restrict__ rows, int T, int d, int S) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    float* u = sm;                         // [d]
    float* red = sm + d;                   // [33]
    __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_write[MAX_STREAMS], s_read[MAX_STREAMS];
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_write[threadIdx.x] = y ? write[threadIdx.x] : 0.f;
        s_read[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
    }
    __syncthreads();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    const size_t plane = (size_t)T * d;
    float ss = 0.f;
    // VEC = 4: rows of a multiple of 4 elements, four at a time (16-byte loads of the streams)
    for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
        float xs[MAX_STREAMS][VEC];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) {
                const float* src = X + (fresh ? 0 : (size_t)s * plane) + (size_t)t * d;
                if (VEC == 4) load4(src, i, reinterpret_cast<float (&)[4]>(xs[s]));
                else xs[s][0] = src[i];
            }
        float acc[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
        if (y) {
            float yv[VEC];
            if (VEC == 4) load4(y + (size_t)t * d, i, reinterpret_cast<float (&)[4]>(yv));
            else yv[0] = to_f32<TY>(y[(size_t)t * d + i]);
#pragma unroll
            for (int to = 0; to < MAX_STREAMS; ++to)
                if (to < S) {
                    float n[VEC];
#pragma unroll
                    for (int v = 0; v < VEC; ++v) {
                        float a = 0.f;
#pragma unroll
                        for (int s = 0; s < MAX_STREAMS; ++s)
                            if (s < S) a = fmaf(s_mix[s * S + to], xs[s][v], a);
                        a = fmaf(s_write[to], yv[v], a);
                        n[v] = a;
                        acc[v] = fmaf(s_read[to], a, acc[v]);
                    }
                    if (!rows) {
                        float* dst = X + (size_t)to * plane + (size_t)t * d;
                        if (VEC == 4) store4(dst, i, reinterpret_cast<const float (&)[4]>(n));
                        else dst[i] = n[0];
                    }
                }
        } else {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) {
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[v] = fmaf(s_read[s], xs[s][v], acc[v]);
                }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            u[i + v] = acc[v];
            ss += acc[v] * acc[v];
        }
    }
    if (!out) return;
    if (!w) {
        __syncthreads();
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)r * d + i] = from_f32<TO>(u[i]);
        return;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float wv4[4], o[4];
            load4(w, i, wv4);
#pragma unroll
            for (int v = 0; v < 4; ++v) o[v] = u[i + v] * inv * wv4[v];
            store4(out + (size_t)r * d, i, o);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            out[(size_t)r * d + i] = from_f32<TO>(u[i] * inv * to_f32<TW>(w[i]));
    }
}

// ------------------------------------ q, k, v from the projection to the attention and the cache
// qkv [T][Hq*dk (+ Hkv*dk + Hkv*dv when has_kv)] fp32 or the activation dtype.  Per token: add the bias,
// norm q and k (mode 1: every head by its own root mean square, weights [dk] shared by the heads; mode 2:
// all of q by one root mean square and all of k by another, weights of the whole size), rotate the first
// `rot` channels of every head of q and k (pairs (2i, 2i+1) when interleaved, else (i, i + rot/2)) by the
// angles of cos/sin [positions][rot/2], store q rounded to the activation dtype and k, v into the pages of
// `cache` at slot_of_token[t] (page*page_size + offset; < 0 or no cache: not stored).  One CTA a token.
// Hv: heads of v where they are fewer than the heads of k (several attention maps, each with keys of
// its own, over one set of values); a page then holds Hkv heads of keys and Hv heads of values.
template <typename TI, typename TA, typename TW>
__global__ void qkv_prepare_kernel(const TI* __restrict__ qkv, int row_stride, const float* __restrict__ bias,
                                   const TW* __restrict__ q_w, const TW* __restrict__ k_w, int norm_mode, float eps,
                                   const int* __restrict__ positions, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int rot, int interleaved,
                                   const int* __restrict__ slot_of_token, TA* __restrict__ cache,
                                   TA* __restrict__ q_out, int Hq, int Hkv, int Hv, int dk, int dv, int has_kv, int page_size) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int nq = Hq * dk, nk = has_kv ? Hkv * dk : 0;
    float* qs = sm;                        // [nq]
    float* ks = qs + nq;                   // [nk]
    float* red = ks + nk;                  // [33]
    const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
    const TI* row = qkv + (size_t)t * row_stride;
    float ssq = 0.f, ssk = 0.f;
    for (int i = tid; i < nq + nk; i += nth) {
        float v = to_f32<TI>(row[i]);
        if (bias) v += bias[i];
        sm[i] = v;
        if (i < nq) ssq += v * v; else ssk += v * v;
    }
    if (norm_mode == 2) {
        ssq = block_sum(ssq, red);
        ssk = block_sum(ssk, red);
        const float iq = 1.0f / sqrtf(ssq / (float)nq + eps);
        const float ik = nk ? 1.0f / sqrtf(ssk / (float)nk + eps) : 0.f;
        for (int i = tid; i < nq; i += nth) qs[i] = qs[i] * iq * wv(q_w, i);
        for (int i = tid; i < nk; i += nth) ks[i] = ks[i] * ik * wv(k_w, i);
    } else if (norm_mode == 1) {
        __syncthreads();
        const int lane = tid & 31, warps = nth >> 5;
        const int heads = Hq + (has_kv ? Hkv : 0);
        for (int h = tid >> 5; h < heads; h += warps) {
            float* x = sm + (size_t)h * dk;
            const TW* w = h < Hq ? q_w : k_w;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss += x[i] * x[i];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)dk + eps);
            for (int i = lane; i < dk; i += 32) x[i] = x[i] * inv * wv(w, i);
        }
    }
    __syncthreads();
    if (rot > 0) {
        const int half = rot >> 1;
        const int heads = Hq + (has_kv ? Hkv : 0);
        const int pos = positions[t];
        const float* cr = cos_t + (size_t)pos * half;
        const float* sr = sin_t + (size_t)pos * half;
        for (int e = tid; e < heads * half; e += nth) {
            const int h = e / half, i = e - h * half;
            float* x = sm + (size_t)h * dk;
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = x[ia], b = x[ib], c = cr[i], s = sr[i];
            x[ia] = a * c - b * s;
            x[ib] = b * c + a * s;
        }
        __syncthreads();
    }
    for (int i = tid; i < nq; i += nth) q_out[(size_t)t * nq + i] = from_f32<TA>(qs[i]);
    if (!has_kv || !cache || !slot_of_token) return;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    const size_t page_elems = (size_t)page_size * ((size_t)Hkv * dk + (size_t)Hv * dv);
    TA* page = cache + (size_t)(slot / page_size) * page_elems;
    const int off = slot % page_size;
    for (int i = tid; i < nk; i += nth) {
        const int g = i / dk, c = i - g * dk;
        page[((size_t)g * page_size + off) * dk + c] = from_f32<TA>(ks[i]);
    }
    const int nv = Hv * dv;
    TA* vpage = page + (size_t)Hkv * page_size * dk;
    for (int i = tid; i < nv; i += nth) {
        const int g = i / dv, c = i - g * dv;
        float v = to_f32<TI>(row[nq + nk + i]);
        if (bias) v += bias[nq + nk + i];
        vpage[((size_t)g * page_size + off) * dv + c] = from_f32<TA>(v);
    }
}

}  // namespace

RI_API int ri_embed_rmsnorm(const int* ids, const void* table, int table_dtype, const void* w, int w_dtype, float eps,
                            float* out, int tokens, int d, int vocab, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(d + 33) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
#define RI_ER(TE, TW) RI_CHECKED(ri_launch(embed_rmsnorm_kernel<TE, TW>, dim3(tokens), dim3(256), smem, s, ids, \
        (const TE*)table, (const TW*)w, eps, out, d, vocab))
    if (table_dtype == RI_BF16 && w_dtype == RI_BF16) RI_ER(bf16, bf16);
    else if (table_dtype == RI_BF16) RI_ER(bf16, float);
    else if (w_dtype == RI_BF16) RI_ER(float, bf16);
    else RI_ER(float, float);
#undef RI_ER
    return ri_launch_status();
}

RI_API int ri_hyper_max_streams() { return MAX_STREAMS; }

// y_dtype / w_dtype / out_dtype: RI_F32 or RI_BF16 (of y, w and out; ignored for a null pointer).
RI_API int ri_hyper_collect(float* X, int fresh, const void* y, int y_dtype, const float* mix, const float* write,
                            const float* read, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                            const int* rows, int n_rows, int T, int d, int S, void* stream) {
    if (n_rows <= 0) return 0;
    if (S < 1 || S > MAX_STREAMS) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(d + 33) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const size_t ysz = y_dtype == RI_BF16 ? 2 : 4, wsz = w_dtype == RI_BF16 ? 2 : 4, osz = out_dtype == RI_BF16 ? 2 : 4;
    const bool vec = d % 4 == 0 && ((uintptr_t)X & 15) == 0 && (!y || ((uintptr_t)y % (4 * ysz)) == 0) &&
                     (!w || ((uintptr_t)w % (4 * wsz)) == 0) && (!out || ((uintptr_t)out % (4 * osz)) == 0);
#define RI_HC(TY, TW, TO) do { \
        if (vec) RI_CHECKED(ri_launch(hyper_collect_kernel<TY, TW, TO, 4>, dim3(n_rows), dim3(256), smem, s, X, fresh, \
            (const TY*)y, mix, write, read, (const TW*)w, eps, (TO*)out, rows, T, d, S)); \
        else RI_CHECKED(ri_launch(hyper_collect_kernel<TY, TW, TO, 1>, dim3(n_rows), dim3(256), smem, s, X, fresh, \
            (const TY*)y, mix, write, read, (const TW*)w, eps, (TO*)out, rows, T, d, S)); } while (0)
#define RI_HC2(TY, TW) do { if (out_dtype == RI_BF16) RI_HC(TY, TW, bf16); else RI_HC(TY, TW, float); } while (0)
    if (y_dtype == RI_BF16 && w_dtype == RI_BF16) RI_HC2(bf16, bf16);
    else if (y_dtype == RI_BF16) RI_HC2(bf16, float);
    else if (w_dtype == RI_BF16) RI_HC2(float, bf16);
    else RI_HC2(float, float);
#undef RI_HC2
#undef RI_HC
    return ri_launch_status();
}

// in_dtype: of qkv; act_dtype: of q_out and the cache; w_dtype: of the norm weights.  bias is fp32.
RI_API int ri_qkv_prepare(const void* qkv, int in_dtype, int row_stride, const float* bias, const void* q_w,
                          const void* k_w, int w_dtype, int norm_mode, float eps, const int* positions,
                          const float* cos_t, const float* sin_t, int rot, int interleaved, const int* slot_of_token,
                          void* cache, void* q_out, int act_dtype, int tokens, int Hq, int Hkv, int dk, int dv,
                          int has_kv, int page_size, int value_heads, void* stream) {
    if (tokens <= 0) return 0;
    const int Hv = value_heads > 0 ? value_heads : Hkv;
    if (rot < 0 || rot > dk || (rot & 1) || (rot > 0 && (!cos_t || !sin_t || !positions))) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(Hq * dk + (has_kv ? Hkv * dk : 0) + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define RI_QP(TI, TA, TW) do { \
        static bool configured = false; \
        if (!configured && smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(qkv_prepare_kernel<TI, TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; } \
        RI_CHECKED(ri_launch(qkv_prepare_kernel<TI, TA, TW>, dim3(tokens), dim3(256), smem, s, (const TI*)qkv, row_stride, bias, \
            (const TW*)q_w, (const TW*)k_w, norm_mode, eps, positions, cos_t, sin_t, rot, interleaved, slot_of_token, (TA*)cache, \
            (TA*)q_out, Hq, Hkv, Hv, dk, dv, has_kv, page_size)); } while (0)
    if (act_dtype == RI_BF16) {
        if (in_dtype == RI_BF16) { if (w_dtype == RI_BF16) RI_QP(bf16, bf16, bf16); else RI_QP(bf16, bf16, float); }
        else { if (w_dtype == RI_BF16) RI_QP(float, bf16, bf16); else RI_QP(float, bf16, float); }
    } else {
        if (in_dtype != RI_F32) return (int)cudaErrorInvalidValue;
        if (w_dtype == RI_BF16) RI_QP(float, float, bf16); else RI_QP(float, float, float);
    }
#undef RI_QP
    return ri_launch_status();
}
