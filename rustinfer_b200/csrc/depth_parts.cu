// Row and recurrence kernels of decoders that keep every layer's result (a weighted depth average hands the next
// layer its input), put a short causal convolution in front of a mixer, and run a gated linear recurrent unit
// beside attention.  The reference engine has none of these (its blocks are
// crates/infer-worker/src/components/decoder_block.rs:13-32); they stand beside the fused add + RMSNorm
// (elementwise.cu) and the layer norm around a sublayer (sequence_parts.cu).  All arithmetic is fp32; only the
// rounding of an output to the activation dtype is not.
#include "common.cuh"

namespace {

// --------------------------------------------------------------------- RMS norm around a sublayer, depth average
// One CTA a row.  With v the row of h_in:
//   delta:  v += rms(delta) * post_w         (the norm after a sublayer; post_w holds the residual's factor)
//   h_out:  h_out <- v                       (the stream after the sublayer; may be h_in itself)
//   dwa:    v <- sum_{j < n_prev} dwa[j] * hist[j] + dwa[n_prev] * v;   avg_out <- v   (the depth average)
//   out:    out <- rms(v) * next_w           (the norm before the next sublayer; next_w null: weight 1)
// rms(x) = x / sqrt(mean(x^2) + eps).  rows: only these rows are read, nothing but `out` is written.
template <typename TD, typename TO>
__global__ void rms_sandwich_kernel(const float* __restrict__ h_in, int in_stride, const TD* __restrict__ delta,
                                    int delta_stride, const float* __restrict__ post_w, float* __restrict__ h_out,
                                    const float* __restrict__ hist, long long layer_stride, int n_prev,
                                    const float* __restrict__ dwa, float* __restrict__ avg_out,
                                    const float* __restrict__ next_w, TO* __restrict__ out,
                                    const int* __restrict__ rows, int d, float eps) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float inv_d = 1.0f / (float)d;
    const float* hp = h_in + (size_t)src * in_stride;
    if (delta) {
        const TD* dp = delta + (size_t)src * delta_stride;
        float q = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = to_f32<TD>(dp[i]);
            row[i] = v;
            q += v * v;
        }
        const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x) row[i] = hp[i] + row[i] * inv * post_w[i];
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) row[i] = hp[i];
    }
    if (h_out && !rows && (delta || h_out != h_in))
        for (int i = threadIdx.x; i < d; i += blockDim.x) h_out[(size_t)src * d + i] = row[i];
    if (dwa) {
        const float w_last = dwa[n_prev];
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float a = 0.f;
            for (int j = 0; j < n_prev; ++j) a = fmaf(dwa[j], hist[(size_t)j * layer_stride + (size_t)src * d + i], a);
            a = fmaf(w_last, row[i], a);
            row[i] = a;
            if (avg_out && !rows) avg_out[(size_t)src * d + i] = a;
        }
    }
    if (!out) return;
    float q = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) q += row[i] * row[i];
    const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
    TO* op = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) op[i] = from_f32<TO>(row[i] * inv * (next_w ? next_w[i] : 1.f));
}

// ----------------------------------------------------------------------- short causal convolution with a state
// With x'[t][c] = x[t][c] + in_bias[c] (in_bias null: 0):
// y[t][c] = (residual ? x'[t][c] : 0) + bias[c] + sum_j w[c][j] * x'[t - taps + 1 + j][c] over the tokens of one
// entry; the taps - 1 inputs before the entry's first token come from state[slot] ([taps - 1][C], oldest first;
// zeros for a new request), and the entry's last taps - 1 inputs go back there.  A thread owns one channel of a
// chunk of CONV_CHUNK tokens of one entry; the thread of an entry's first chunk is the only one that reads or
// writes the channel's state.
constexpr int CONV_MAX_TAPS = 8, CONV_CHUNK = 32;

template <typename TI, typename TO>
__global__ void short_conv_kernel(const TI* __restrict__ x, int x_stride, const float* __restrict__ w,
                                  const float* __restrict__ bias, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                  TO* __restrict__ out, int out_stride, int C, int taps, int residual,
                                  const float* __restrict__ in_bias) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0;
    const int i0 = blockIdx.z * CONV_CHUNK;
    if (i0 >= q_len) return;
    const int back = taps - 1;
    float* st = state + ((size_t)state_slots[e] * back) * C + c;
    float wt[CONV_MAX_TAPS], win[CONV_MAX_TAPS - 1], old[CONV_MAX_TAPS - 1];
    const float ib = in_bias ? in_bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    // win[k]: the input k + 1 tokens back
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
        win[k] = 0.f;
        old[k] = 0.f;
        if (k < back) {
            if (i0 == 0) {
                old[k] = st[(size_t)(back - 1 - k) * C];
                win[k] = old[k];
            } else {
                const int idx = i0 - 1 - k;                  // >= 0: CONV_CHUNK >= taps - 1
                win[k] = to_f32<TI>(x[(size_t)(t0 + idx) * x_stride + c]) + ib;
            }
        }
    }
    const float b = bias ? bias[c] : 0.f;
    const int i1 = min(q_len, i0 + CONV_CHUNK);
    for (int i = i0; i < i1; ++i) {
        const float cur = to_f32<TI>(x[(size_t)(t0 + i) * x_stride + c]) + ib;
        float y = b + (residual ? cur : 0.f);
        y = fmaf(wt[back], cur, y);
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
            if (k < back) y = fmaf(wt[back - 1 - k], win[k], y);
        out[(size_t)(t0 + i) * out_stride + c] = from_f32<TO>(y);
#pragma unroll
        for (int k = CONV_MAX_TAPS - 2; k > 0; --k) win[k] = win[k - 1];
        win[0] = cur;
    }
    if (i0 != 0) return;
    // the inputs at q_len - back .. q_len - 1 (from the old state where that is before the entry's start)
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
        if (k >= back) continue;
        const int idx = q_len - 1 - k;                       // k tokens before the last
        float v;
        if (idx >= 0) v = to_f32<TI>(x[(size_t)(t0 + idx) * x_stride + c]) + ib;
        else {
            // -idx - 1 steps into the old state: old[j] is the input j + 1 before the start
            v = 0.f;
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
                if (j == -idx - 1) v = old[j];
        }
        st[(size_t)(back - 1 - k) * C] = v;
    }
}

// ------------------------------------------------------------------ gates of the real-gated linear recurrent unit
// u [T][C] fp32 in `blocks` equal parts of bs channels; wa, wi [blocks][bs][bs] ([out][in]), ba, bi [C]:
//   r = sigmoid(wa[b] u_b + ba),  i = sigmoid(wi[b] u_b + bi),  log a = -decay_scale * r * softplus(lam),
//   a_out = exp(log a),  x_out = sqrt(1 - a^2) * i * u          (1 - a^2 formed as -expm1(2 log a))
// A CTA of 256 threads owns GT tokens x GN channels of one part; every sum runs over k = 0, 1, .. in order with
// fp32 multiply-adds, so a value does not depend on which tokens share its tile.
constexpr int GT = 64, GN = 64, GK = 16;

template <typename TW>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const float* __restrict__ u, int u_stride, const TW* __restrict__ wa, const TW* __restrict__ wi,
                   const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ x_out, int T, int C, int bs) {
    pdl_trigger();
    pdl_wait();
    // tiles stored k-major, so that a thread's four tokens (or channels) of one k are one 16-byte load
    // (rows padded by four floats: the transposing stores of a warp then spread over eight banks)
    __shared__ __align__(16) float Us[GK][GT + 4];
    __shared__ __align__(16) float Wa[GK][GN + 4];
    __shared__ __align__(16) float Wi[GK][GN + 4];
    const int part = blockIdx.z;
    const int t0 = blockIdx.x * GT, n0 = blockIdx.y * GN;   // n0: first out channel within the part
    const int tid = threadIdx.x;
    const int tn = tid & 15, tt = tid >> 4;                  // channels 4 tn .. 4 tn + 3, tokens 4 tt .. 4 tt + 3
    float acc_a[4][4], acc_i[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc_a[i][j] = acc_i[i][j] = 0.f;
    const TW* wa_p = wa + (size_t)part * bs * bs;
    const TW* wi_p = wi + (size_t)part * bs * bs;
    for (int k0 = 0; k0 < bs; k0 += GK) {
        for (int e = tid; e < GT * GK; e += 256) {
            const int r = e / GK, k = e - r * GK;
            Us[k][r] = (t0 + r < T && k0 + k < bs) ? u[(size_t)(t0 + r) * u_stride + part * bs + k0 + k] : 0.f;
        }
        for (int e = tid; e < GN * GK; e += 256) {
            const int r = e / GK, k = e - r * GK;
            const bool ok = n0 + r < bs && k0 + k < bs;
            Wa[k][r] = ok ? to_f32<TW>(wa_p[(size_t)(n0 + r) * bs + k0 + k]) : 0.f;
            Wi[k][r] = ok ? to_f32<TW>(wi_p[(size_t)(n0 + r) * bs + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            const float4 uv = *reinterpret_cast<const float4*>(&Us[k][4 * tt]);
            const float4 va = *reinterpret_cast<const float4*>(&Wa[k][4 * tn]);
            const float4 vi = *reinterpret_cast<const float4*>(&Wi[k][4 * tn]);
            const float ur[4] = {uv.x, uv.y, uv.z, uv.w};
            const float ar[4] = {va.x, va.y, va.z, va.w};
            const float ir[4] = {vi.x, vi.y, vi.z, vi.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc_a[i][j] = fmaf(ur[i], ar[j], acc_a[i][j]);
                    acc_i[i][j] = fmaf(ur[i], ir[j], acc_i[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + 4 * tt + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + 4 * tn + j;
            if (n >= bs) continue;
            const int c = part * bs + n;
            const float r = 1.0f / (1.0f + expf(-(acc_a[i][j] + ba[c])));
            const float g = 1.0f / (1.0f + expf(-(acc_i[i][j] + bi[c])));
            const float l = lam[c];
            const float sp = l > 20.f ? l : log1pf(expf(l));
            const float log_a = -decay_scale * r * sp;
            a_out[(size_t)t * C + c] = expf(log_a);
            x_out[(size_t)t * C + c] = sqrtf(-expm1f(2.0f * log_a)) * g * u[(size_t)t * u_stride + c];
        }
    }
}

// ------------------------------------------------------------------------------------- the recurrence itself
// S_t = a_t * S_(t-1) + x_t per channel over the tokens of an entry, from state[slot] and back into it;
// out[t][c] = S_t * gelu_tanh(y[t][c] + y_bias[c]).  A thread a channel of an entry; the loads of sixteen tokens are
// in flight at once (none depends on the recurrence).
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TO>
__global__ void rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ x, const float* __restrict__ y,
                                  int y_stride, const float* __restrict__ y_bias, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                  TO* __restrict__ out, int C) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_q[e], t1 = cu_q[e + 1];
    if (t1 <= t0) return;
    float* sp = state + (size_t)state_slots[e] * C + c;
    float S = *sp;
    const float yb = y_bias ? y_bias[c] : 0.f;
    int t = t0;
    constexpr int AHEAD = 16;
    for (; t + AHEAD <= t1; t += AHEAD) {
        float av[AHEAD], xv[AHEAD], yv[AHEAD];
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            av[k] = a[(size_t)(t + k) * C + c];
            xv[k] = x[(size_t)(t + k) * C + c];
            yv[k] = y[(size_t)(t + k) * y_stride + c];
        }
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            S = fmaf(av[k], S, xv[k]);
            out[(size_t)(t + k) * C + c] = from_f32<TO>(S * gelu_tanh_f(yv[k] + yb));
        }
    }
    for (; t < t1; ++t) {
        S = fmaf(a[(size_t)t * C + c], S, x[(size_t)t * C + c]);
        out[(size_t)t * C + c] = from_f32<TO>(S * gelu_tanh_f(y[(size_t)t * y_stride + c] + yb));
    }
    *sp = S;
}

// ----------------------------------------------------------------------------------------- element-wise parts
// out[t][j] = o[t][j] * sigmoid(g[t][j / group]): group 1 a gate a channel, group = a head's width a gate a head
template <typename TI, typename TO>
__global__ void sigmoid_gate_kernel(const TI* __restrict__ o, int o_stride, const float* __restrict__ g, int g_stride,
                                    int group, TO* __restrict__ out, int T, int n) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), j = (int)(i - (long long)t * n);
        const float gv = g[(size_t)t * g_stride + j / group];
        out[i] = from_f32<TO>(to_f32<TI>(o[(size_t)t * o_stride + j]) / (1.0f + expf(-gv)));
    }
}

__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap) {
    pdl_trigger();
    pdl_wait();
    const float inv = 1.0f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

inline int ew_blocks(long long n) {
    const long long b = (n + 255) / 256;
    return (int)(b < 1 ? 1 : b > 148LL * 16 ? 148 * 16 : b);
}

}  // namespace

// h_in fp32 rows of in_stride; delta (may be null) rows of delta_stride, RI_F32 or RI_BF16; post_w, next_w, dwa
// fp32; h_out, avg_out fp32 [rows][d] (each may be null); hist: n_prev earlier results, layer_stride floats apart;
// out (may be null) [n_rows][d] of out_dtype; rows (may be null): gather, nothing but out is written.
RI_API int ri_rms_sandwich(const float* h_in, int in_stride, const void* delta, int delta_dtype, int delta_stride,
                           const float* post_w, float* h_out, const float* hist, long long layer_stride, int n_prev,
                           const float* dwa, float* avg_out, const float* next_w, void* out, int out_dtype,
                           const int* rows, int n_rows, int d, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024 || (delta && !post_w) || (dwa && n_prev > 0 && !hist)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 2048 ? 512 : d >= 512 ? 256 : 128;
#define RI_RS(TD, TO) do { \
        static size_t configured = 48 * 1024; \
        if (smem > configured) { \
            cudaError_t e = cudaFuncSetAttribute(rms_sandwich_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e; \
            configured = 200 * 1024; } \
        RI_CHECKED(ri_launch(rms_sandwich_kernel<TD, TO>, dim3(n_rows), dim3(threads), smem, s, h_in, in_stride, \
            (const TD*)delta, delta_stride, post_w, h_out, hist, layer_stride, n_prev, dwa, avg_out, next_w, (TO*)out, \
            rows, d, eps)); } while (0)
    if (delta_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_RS(bf16, bf16); else RI_RS(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_RS(float, bf16); else RI_RS(float, float); }
#undef RI_RS
    return ri_launch_status();
}

RI_API int ri_short_conv_max_taps() { return CONV_MAX_TAPS; }

// x rows of x_stride (RI_F32 or RI_BF16), w fp32 [C][taps], bias and in_bias fp32 [C] or null, state fp32 [slots][taps-1][C],
// out rows of out_stride of out_dtype.  max_q_len: an upper bound of the entries' token counts.
RI_API int ri_short_conv(const void* x, int x_dtype, int x_stride, const float* w, const float* bias, float* state,
                         const int* cu_q, const int* state_slots, void* out, int out_dtype, int out_stride,
                         int n_entries, int max_q_len, int C, int taps, int residual, const float* in_bias,
                         void* stream) {
    if (n_entries <= 0 || max_q_len <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((C + 127) / 128, n_entries, (max_q_len + CONV_CHUNK - 1) / CONV_CHUNK);
#define RI_SC(TI, TO) RI_CHECKED(ri_launch(short_conv_kernel<TI, TO>, grid, dim3(128), 0, s, (const TI*)x, x_stride, w, bias, \
        state, cu_q, state_slots, (TO*)out, out_stride, C, taps, residual, in_bias))
    if (x_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_SC(bf16, bf16); else RI_SC(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_SC(float, bf16); else RI_SC(float, float); }
#undef RI_SC
    return ri_launch_status();
}

// u fp32 rows of u_stride; wa, wi [blocks][bs][bs] of w_dtype; ba, bi, lam fp32 [C]; a_out, x_out fp32 [T][C]
RI_API int ri_rglru_gates(const float* u, int u_stride, const void* wa, const void* wi, int w_dtype, const float* ba,
                          const float* bi, const float* lam, float decay_scale, float* a_out, float* x_out, int T,
                          int C, int blocks, void* stream) {
    if (T <= 0) return 0;
    if (blocks <= 0 || C % blocks) return (int)cudaErrorInvalidValue;
    const int bs = C / blocks;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((T + GT - 1) / GT, (bs + GN - 1) / GN, blocks);
    if (w_dtype == RI_BF16)
        RI_CHECKED(ri_launch(rglru_gates_kernel<bf16>, grid, dim3(256), 0, s, u, u_stride, (const bf16*)wa, (const bf16*)wi,
                             ba, bi, lam, decay_scale, a_out, x_out, T, C, bs));
    else
        RI_CHECKED(ri_launch(rglru_gates_kernel<float>, grid, dim3(256), 0, s, u, u_stride, (const float*)wa,
                             (const float*)wi, ba, bi, lam, decay_scale, a_out, x_out, T, C, bs));
    return ri_launch_status();
}

// a, x fp32 [T][C]; y fp32 rows of y_stride; y_bias fp32 [C] or null; state fp32 [slots][C]; out [T][C] of out_dtype
RI_API int ri_rglru_scan(const float* a, const float* x, const float* y, int y_stride, const float* y_bias, float* state,
                         const int* cu_q, const int* state_slots, void* out, int out_dtype, int n_entries, int C,
                         void* stream) {
    if (n_entries <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = C >= 2048 ? 128 : 64;
    const dim3 grid((C + threads - 1) / threads, n_entries);
    if (out_dtype == RI_BF16)
        RI_CHECKED(ri_launch(rglru_scan_kernel<bf16>, grid, dim3(threads), 0, s, a, x, y, y_stride, y_bias, state, cu_q,
                             state_slots, (bf16*)out, C));
    else
        RI_CHECKED(ri_launch(rglru_scan_kernel<float>, grid, dim3(threads), 0, s, a, x, y, y_stride, y_bias, state, cu_q,
                             state_slots, (float*)out, C));
    return ri_launch_status();
}

// o rows of o_stride (RI_F32 or RI_BF16), g fp32 rows of g_stride, out [T][n] of out_dtype
RI_API int ri_sigmoid_gate(const void* o, int o_dtype, int o_stride, const float* g, int g_stride, int group, void* out,
                           int out_dtype, int T, int n, void* stream) {
    const long long total = (long long)T * n;
    if (total <= 0) return 0;
    if (group <= 0) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_SG(TI, TO) RI_CHECKED(ri_launch(sigmoid_gate_kernel<TI, TO>, dim3(ew_blocks(total)), dim3(256), 0, s, (const TI*)o, \
        o_stride, g, g_stride, group, (TO*)out, T, n))
    if (o_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_SG(bf16, bf16); else RI_SG(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_SG(float, bf16); else RI_SG(float, float); }
#undef RI_SG
    return ri_launch_status();
}

// x <- cap * tanh(x / cap), fp32, in place
RI_API int ri_softcap(float* x, long long total, float cap, void* stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    RI_CHECKED(ri_launch(softcap_kernel, dim3(ew_blocks(total)), dim3(256), 0, (cudaStream_t)stream, x, total, cap));
    return ri_launch_status();
}
