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
// four elements at a time where rows allow it (V = 4: d and the strides multiples of four, 16-byte aligned pointers)
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&lo);
    u.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// A short causal convolution on the normed output, for a step in which row r is the one token of entry r:
// out <- n + sum_j w[c][j] * n_(t - taps + 1 + j) with the earlier inputs from state[slots[r]] ([taps - 1][d], oldest
// first), which is shifted by the new input.  w null: none.
struct ConvTail {
    const float* w;              // [d][taps]
    float* state;                // [slots][taps - 1][d]
    const int* slots;
    int taps;
};

template <typename TO>
__device__ __forceinline__ float conv_tail(const ConvTail& ct, int r, int c, int d, float n) {
    const int back = ct.taps - 1;
    const float* wc = ct.w + (size_t)c * ct.taps;
    float* st = ct.state + (size_t)ct.slots[r] * back * d + c;
    float y = fmaf(wc[back], n, n);
    float prev = n;                                          // what row k is overwritten with, walking from the newest
    for (int k = back - 1; k >= 0; --k) {
        const float old = st[(size_t)k * d];
        y = fmaf(wc[k], old, y);
        st[(size_t)k * d] = prev;
        prev = old;
    }
    return y;
}

template <typename TD, typename TO, int V>
__global__ void rms_sandwich_kernel(const float* __restrict__ h_in, int in_stride, const TD* __restrict__ delta,
                                    int delta_stride, const float* __restrict__ post_w, float* __restrict__ h_out,
                                    const float* __restrict__ hist, long long layer_stride, int n_prev,
                                    const float* __restrict__ dwa, float* __restrict__ avg_out,
                                    const float* __restrict__ next_w, TO* __restrict__ out,
                                    const int* __restrict__ rows, int d, float eps, ConvTail ct) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row[];
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float inv_d = 1.0f / (float)d;
    const float* hp = h_in + (size_t)src * in_stride;
    const int step = blockDim.x * V, first = threadIdx.x * V;
    if (delta) {
        const TD* dp = delta + (size_t)src * delta_stride;
        float q = 0.f;
        for (int i = first; i < d; i += step) {
            if (V == 4) {
                const float4 v = load4<TD>(dp + i);
                *reinterpret_cast<float4*>(row + i) = v;
                q += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            } else {
                const float v = to_f32<TD>(dp[i]);
                row[i] = v;
                q += v * v;
            }
        }
        const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
        for (int i = first; i < d; i += step) {
            if (V == 4) {
                const float4 h = load4<float>(hp + i), w = load4<float>(post_w + i);
                float4 v = *reinterpret_cast<float4*>(row + i);
                v = make_float4(h.x + v.x * inv * w.x, h.y + v.y * inv * w.y, h.z + v.z * inv * w.z, h.w + v.w * inv * w.w);
                *reinterpret_cast<float4*>(row + i) = v;
            } else {
                row[i] = hp[i] + row[i] * inv * post_w[i];
            }
        }
    } else {
        for (int i = first; i < d; i += step) {
            if (V == 4) *reinterpret_cast<float4*>(row + i) = load4<float>(hp + i);
            else row[i] = hp[i];
        }
    }
    // (a thread reads back only what it wrote itself, so no barrier is needed between these loops)
    if (h_out && !rows && (delta || h_out != h_in))
        for (int i = first; i < d; i += step) {
            if (V == 4) store4<float>(h_out + (size_t)src * d + i, *reinterpret_cast<float4*>(row + i));
            else h_out[(size_t)src * d + i] = row[i];
        }
    if (dwa) {
        const float w_last = dwa[n_prev];
        for (int i = first; i < d; i += step) {
            if (V == 4) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int j = 0; j < n_prev; ++j) {
                    const float wj = dwa[j];
                    const float4 x = load4<float>(hist + (size_t)j * layer_stride + (size_t)src * d + i);
                    a = make_float4(fmaf(wj, x.x, a.x), fmaf(wj, x.y, a.y), fmaf(wj, x.z, a.z), fmaf(wj, x.w, a.w));
                }
                const float4 v = *reinterpret_cast<float4*>(row + i);
                a = make_float4(fmaf(w_last, v.x, a.x), fmaf(w_last, v.y, a.y), fmaf(w_last, v.z, a.z), fmaf(w_last, v.w, a.w));
                *reinterpret_cast<float4*>(row + i) = a;
                if (avg_out && !rows) store4<float>(avg_out + (size_t)src * d + i, a);
            } else {
                float a = 0.f;
                for (int j = 0; j < n_prev; ++j) a = fmaf(dwa[j], hist[(size_t)j * layer_stride + (size_t)src * d + i], a);
                a = fmaf(w_last, row[i], a);
                row[i] = a;
                if (avg_out && !rows) avg_out[(size_t)src * d + i] = a;
            }
        }
    }
    if (!out) return;
    float q = 0.f;
    for (int i = first; i < d; i += step) {
        if (V == 4) {
            const float4 v = *reinterpret_cast<float4*>(row + i);
            q += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        } else {
            q += row[i] * row[i];
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(q, red) * inv_d + eps);
    TO* op = out + (size_t)r * d;
    for (int i = first; i < d; i += step) {
        if (V == 4) {
            const float4 v = *reinterpret_cast<float4*>(row + i);
            const float4 w = next_w ? load4<float>(next_w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            float4 n = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w);
            if (ct.w)
                n = make_float4(conv_tail<TO>(ct, r, i, d, n.x), conv_tail<TO>(ct, r, i + 1, d, n.y),
                                conv_tail<TO>(ct, r, i + 2, d, n.z), conv_tail<TO>(ct, r, i + 3, d, n.w));
            store4<TO>(op + i, n);
        } else {
            float n = row[i] * inv * (next_w ? next_w[i] : 1.f);
            if (ct.w) n = conv_tail<TO>(ct, r, i, d, n);
            op[i] = from_f32<TO>(n);
        }
    }
}

// ----------------------------------------------------------------------- short causal convolution with a state
// With x'[t][c] = x[t][c] + in_bias[c] (in_bias null: 0):
// y[t][c] = (residual ? x'[t][c] : 0) + bias[c] + sum_j w[c][j] * x'[t - taps + 1 + j][c] over the tokens of one
// entry; the taps - 1 inputs before the entry's first token come from state[slot] ([taps - 1][C], oldest first;
// zeros for a new request), and the entry's last taps - 1 inputs go back there.  A thread owns one channel of a
// chunk of CONV_CHUNK tokens of one entry (their loads in flight at once); the thread of an entry's first chunk is the only one that reads or
// writes the channel's state.
constexpr int CONV_MAX_TAPS = 8, CONV_CHUNK = 8;

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
                const int idx = i0 - 1 - k;                  // >= 0: CONV_CHUNK >= CONV_MAX_TAPS - 1
                win[k] = to_f32<TI>(x[(size_t)(t0 + idx) * x_stride + c]) + ib;
            }
        }
    }
    const float b = bias ? bias[c] : 0.f;
    const int i1 = min(q_len, i0 + CONV_CHUNK);
    float in[CONV_CHUNK];
#pragma unroll
    for (int k = 0; k < CONV_CHUNK; ++k)
        in[k] = i0 + k < i1 ? to_f32<TI>(x[(size_t)(t0 + i0 + k) * x_stride + c]) + ib : 0.f;
#pragma unroll
    for (int kk = 0; kk < CONV_CHUNK; ++kk) {
        const int i = i0 + kk;
        if (i >= i1) break;
        const float cur = in[kk];
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
// Every sum runs over k = 0, 1, .. in order with fp32 multiply-adds, so a value does not depend on which tokens share
// its tile, nor on the tile's size.
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

constexpr int GK = 16;

// A CTA of 256 threads (16 x 16) owns 16 TM tokens x 16 TN channels of one part; a thread TM x TN outputs of both
// matrices.  <4, 4> for many tokens; <1, 2> for a step of few, so that the grid still has CTAs for the SMs.
// What a step of single tokens (token t is entry t) does right in the gates' epilogue instead of storing a and x:
// S = a * state[slot] + x back into the state, and out = S * gelu_tanh(y + y_bias).
template <typename TO>
struct StepTail {
    float* state;                // [slots][C]; null: store a_out and x_out
    const int* state_slots;
    const float* y;
    int y_stride;
    const float* y_bias;
    TO* out;                     // [T][C]
    float out_scale;             // a factor on out (a mixer that stands beside another one brings its weight)
};

template <typename TW, int TM, int TN, typename TO>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const float* __restrict__ u, int u_stride, const TW* __restrict__ wa, const TW* __restrict__ wi,
                   const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ lam,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ x_out, int T, int C, int bs,
                   StepTail<TO> tail) {
    pdl_trigger();
    pdl_wait();
    constexpr int GT = 16 * TM, GN = 16 * TN;
    // tiles stored k-major, so that a thread's tokens (or channels) of one k lie side by side
    // (rows padded by four floats: the transposing stores of a warp then spread over eight banks)
    __shared__ __align__(16) float Us[GK][GT + 4];
    __shared__ __align__(16) float Wa[GK][GN + 4];
    __shared__ __align__(16) float Wi[GK][GN + 4];
    const int part = blockIdx.z;
    const int t0 = blockIdx.x * GT, n0 = blockIdx.y * GN;   // n0: first out channel within the part
    const int tid = threadIdx.x;
    const int tn = tid & 15, tt = tid >> 4;                  // channels TN tn .., tokens TM tt ..
    float acc_a[TM][TN], acc_i[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc_a[i][j] = acc_i[i][j] = 0.f;
    const TW* wa_p = wa + (size_t)part * bs * bs;
    const TW* wi_p = wi + (size_t)part * bs * bs;
    // a tile's elements travel global -> registers -> shared memory; the next tile's loads are in flight while this
    // one is multiplied
    constexpr int UL = (GT * GK + 255) / 256, WL = (GN * GK + 255) / 256;
    float ureg[UL], areg[WL], ireg[WL];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int x = 0; x < UL; ++x) {
            const int e = tid + 256 * x, r = e / GK, k = e - r * GK;
            ureg[x] = (e < GT * GK && t0 + r < T && k0 + k < bs) ? u[(size_t)(t0 + r) * u_stride + part * bs + k0 + k] : 0.f;
        }
#pragma unroll
        for (int x = 0; x < WL; ++x) {
            const int e = tid + 256 * x, r = e / GK, k = e - r * GK;
            const bool ok = e < GN * GK && n0 + r < bs && k0 + k < bs;
            areg[x] = ok ? to_f32<TW>(wa_p[(size_t)(n0 + r) * bs + k0 + k]) : 0.f;
            ireg[x] = ok ? to_f32<TW>(wi_p[(size_t)(n0 + r) * bs + k0 + k]) : 0.f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < bs; k0 += GK) {
#pragma unroll
        for (int x = 0; x < UL; ++x) {
            const int e = tid + 256 * x, r = e / GK, k = e - r * GK;
            if (e < GT * GK) Us[k][r] = ureg[x];
        }
#pragma unroll
        for (int x = 0; x < WL; ++x) {
            const int e = tid + 256 * x, r = e / GK, k = e - r * GK;
            if (e < GN * GK) { Wa[k][r] = areg[x]; Wi[k][r] = ireg[x]; }
        }
        __syncthreads();
        if (k0 + GK < bs) fetch(k0 + GK);
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float ur[TM], ar[TN], ir[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ur[i] = Us[k][TM * tt + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                ar[j] = Wa[k][TN * tn + j];
                ir[j] = Wi[k][TN * tn + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc_a[i][j] = fmaf(ur[i], ar[j], acc_a[i][j]);
                    acc_i[i][j] = fmaf(ur[i], ir[j], acc_i[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int t = t0 + TM * tt + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + TN * tn + j;
            if (n >= bs) continue;
            const int c = part * bs + n;
            const float r = 1.0f / (1.0f + expf(-(acc_a[i][j] + ba[c])));
            const float g = 1.0f / (1.0f + expf(-(acc_i[i][j] + bi[c])));
            const float l = lam[c];
            const float sp = l > 20.f ? l : log1pf(expf(l));
            const float log_a = -decay_scale * r * sp;
            const float av = expf(log_a), xv = sqrtf(-expm1f(2.0f * log_a)) * g * u[(size_t)t * u_stride + c];
            if (tail.state) {
                float* sp_ = tail.state + (size_t)tail.state_slots[t] * C + c;
                const float S = fmaf(av, *sp_, xv);
                *sp_ = S;
                tail.out[(size_t)t * C + c] = from_f32<TO>(
                    tail.out_scale * S * gelu_tanh_f(tail.y[(size_t)t * tail.y_stride + c] + (tail.y_bias ? tail.y_bias[c] : 0.f)));
            } else {
                a_out[(size_t)t * C + c] = av;
                x_out[(size_t)t * C + c] = xv;
            }
        }
    }
}

// ------------------------------------------------------------------------------------- the recurrence itself
// S_t = a_t * S_(t-1) + x_t per channel over the tokens of an entry, from state[slot] and back into it;
// out[t][c] = S_t * gelu_tanh(y[t][c] + y_bias[c]).  A thread a channel of an entry.  The recurrence itself is one
// dependent multiply-add a token, so for entries of many tokens the walk does nothing else (the loads of 32 tokens
// in flight at once, S stored over x) and the gelu and the product run over all tokens at once in a second kernel.

template <typename TO, bool FUSED>
__global__ void rglru_scan_kernel(const float* __restrict__ a, float* __restrict__ x, const float* __restrict__ y,
                                  int y_stride, const float* __restrict__ y_bias, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                  TO* __restrict__ out, int C, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_q[e], t1 = cu_q[e + 1];
    if (t1 <= t0) return;
    float* sp = state + (size_t)state_slots[e] * C + c;
    float S = *sp;
    if (FUSED) {
        // few tokens an entry: S * gelu_tanh(y + b_y) written here
        const float yb = y_bias ? y_bias[c] : 0.f;
        for (int t = t0; t < t1; ++t) {
            S = fmaf(a[(size_t)t * C + c], S, x[(size_t)t * C + c]);
            out[(size_t)t * C + c] = from_f32<TO>(out_scale * S * gelu_tanh_f(y[(size_t)t * y_stride + c] + yb));
        }
    } else {
        // many tokens: the walk is one multiply-add a token and stores S over x; rglru_finish_kernel does the rest
        constexpr int AHEAD = 32;
        int t = t0;
        for (; t + AHEAD <= t1; t += AHEAD) {
            float av[AHEAD], xv[AHEAD];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                av[k] = a[(size_t)(t + k) * C + c];
                xv[k] = x[(size_t)(t + k) * C + c];
            }
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                S = fmaf(av[k], S, xv[k]);
                x[(size_t)(t + k) * C + c] = S;
            }
        }
        for (; t < t1; ++t) {
            S = fmaf(a[(size_t)t * C + c], S, x[(size_t)t * C + c]);
            x[(size_t)t * C + c] = S;
        }
    }
    *sp = S;
}

// out[t][c] = out_scale * S[t][c] * gelu_tanh(y[t][c] + y_bias[c])
template <typename TO>
__global__ void rglru_finish_kernel(const float* __restrict__ S, const float* __restrict__ y, int y_stride,
                                    const float* __restrict__ y_bias, TO* __restrict__ out, int T, int C, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)T * C;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / C), c = (int)(i - (long long)t * C);
        out[i] = from_f32<TO>(out_scale * S[i] * gelu_tanh_f(y[(size_t)t * y_stride + c] + (y_bias ? y_bias[c] : 0.f)));
    }
}

// ----------------------------------------------------------------------------------------- element-wise parts
// out[t][j] = scale * o[t][j] * sigmoid(g[t][j / group]): group 1 a gate a channel, group = a head's width a gate a head
template <typename TI, typename TO>
__global__ void sigmoid_gate_kernel(const TI* __restrict__ o, int o_stride, const float* __restrict__ g, int g_stride,
                                    int group, TO* __restrict__ out, int T, int n, float scale) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), j = (int)(i - (long long)t * n);
        const float gv = g[(size_t)t * g_stride + j / group];
        out[i] = from_f32<TO>(scale * to_f32<TI>(o[(size_t)t * o_stride + j]) / (1.0f + expf(-gv)));
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
// out (may be null) [n_rows][d] of out_dtype; rows (may be null): gather, nothing but out is written.  conv_w (may be
// null) fp32 [d][conv_taps] with conv_state fp32 [slots][conv_taps - 1][d] and conv_slots [n_rows]: see ConvTail.
RI_API int ri_rms_sandwich(const float* h_in, int in_stride, const void* delta, int delta_dtype, int delta_stride,
                           const float* post_w, float* h_out, const float* hist, long long layer_stride, int n_prev,
                           const float* dwa, float* avg_out, const float* next_w, void* out, int out_dtype,
                           const int* rows, int n_rows, int d, float eps, const float* conv_w, float* conv_state,
                           const int* conv_slots, int conv_taps, void* stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024 || (delta && !post_w) || (dwa && n_prev > 0 && !hist)) return (int)cudaErrorInvalidValue;
    if (conv_w && (rows || !out || !conv_slots || conv_taps < 1 || (conv_taps > 1 && !conv_state))) return (int)cudaErrorInvalidValue;
    const ConvTail ct{conv_w, conv_state, conv_slots, conv_taps};
    cudaStream_t s = (cudaStream_t)stream;
    const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = d % 4 == 0 && in_stride % 4 == 0 && delta_stride % 4 == 0 && layer_stride % 4 == 0 && al(h_in) && al(delta) &&
                     al(post_w) && al(h_out) && al(hist) && al(avg_out) && al(next_w) && al(out);
    const int lanes = vec ? d / 4 : d;
    const int threads = lanes >= 1024 ? 512 : lanes >= 256 ? 256 : lanes >= 128 ? 128 : 64;
#define RI_RS(TD, TO, V) do { \
        static size_t configured = 48 * 1024; \
        if (smem > configured) { \
            cudaError_t e = cudaFuncSetAttribute(rms_sandwich_kernel<TD, TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e; \
            configured = 200 * 1024; } \
        RI_CHECKED(ri_launch(rms_sandwich_kernel<TD, TO, V>, dim3(n_rows), dim3(threads), smem, s, h_in, in_stride, \
            (const TD*)delta, delta_stride, post_w, h_out, hist, layer_stride, n_prev, dwa, avg_out, next_w, (TO*)out, \
            rows, d, eps, ct)); } while (0)
#define RI_RS2(TD, TO) do { if (vec) RI_RS(TD, TO, 4); else RI_RS(TD, TO, 1); } while (0)
    if (delta_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_RS2(bf16, bf16); else RI_RS2(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_RS2(float, bf16); else RI_RS2(float, float); }
#undef RI_RS2
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
#define RI_GATES(TW, TM, TN) do { \
        const dim3 grid((T + 16 * TM - 1) / (16 * TM), (bs + 16 * TN - 1) / (16 * TN), blocks); \
        RI_CHECKED(ri_launch(rglru_gates_kernel<TW, TM, TN, float>, grid, dim3(256), 0, s, u, u_stride, (const TW*)wa, (const TW*)wi, \
                             ba, bi, lam, decay_scale, a_out, x_out, T, C, bs, StepTail<float>{})); } while (0)
    if (T > 128) { if (w_dtype == RI_BF16) RI_GATES(bf16, 4, 4); else RI_GATES(float, 4, 4); }
    else { if (w_dtype == RI_BF16) RI_GATES(bf16, 1, 2); else RI_GATES(float, 1, 2); }
#undef RI_GATES
    return ri_launch_status();
}

// A step in which every entry brings one token (token t is entry t, T entries): gates, decay, the recurrence's one
// step from state[state_slots[t]] and back, and out = S * gelu_tanh(y + y_bias), in one launch.
RI_API int ri_rglru_step(const float* u, int u_stride, const void* wa, const void* wi, int w_dtype, const float* ba,
                         const float* bi, const float* lam, float decay_scale, const float* y, int y_stride,
                         const float* y_bias, float* state, const int* state_slots, void* out, int out_dtype, int T, int C,
                         int blocks, float out_scale, void* stream) {
    if (T <= 0) return 0;
    if (blocks <= 0 || C % blocks || !state || !state_slots) return (int)cudaErrorInvalidValue;
    const int bs = C / blocks;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((T + 15) / 16, (bs + 31) / 32, blocks);
#define RI_STEP(TW, TO) RI_CHECKED(ri_launch(rglru_gates_kernel<TW, 1, 2, TO>, grid, dim3(256), 0, s, u, u_stride, (const TW*)wa, \
        (const TW*)wi, ba, bi, lam, decay_scale, (float*)nullptr, (float*)nullptr, T, C, bs, \
        StepTail<TO>{state, state_slots, y, y_stride, y_bias, (TO*)out, out_scale}))
    if (w_dtype == RI_BF16) { if (out_dtype == RI_BF16) RI_STEP(bf16, bf16); else RI_STEP(bf16, float); }
    else { if (out_dtype == RI_BF16) RI_STEP(float, bf16); else RI_STEP(float, float); }
#undef RI_STEP
    return ri_launch_status();
}

// a, x fp32 [T][C] (x is overwritten); y fp32 rows of y_stride; y_bias fp32 [C] or null; state fp32 [slots][C]; out [T][C]
// of out_dtype.  max_q_len: an upper bound of the entries' token counts (it picks the one-kernel or the two-kernel form).
RI_API int ri_rglru_scan(const float* a, float* x, const float* y, int y_stride, const float* y_bias, float* state,
                         const int* cu_q, const int* state_slots, void* out, int out_dtype, int n_entries, int C,
                         int T, int max_q_len, float out_scale, void* stream) {
    if (n_entries <= 0 || T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 64;
    const dim3 grid((C + threads - 1) / threads, n_entries);
    const bool fused = max_q_len <= 8;
#define RI_SCAN(TO, F) RI_CHECKED(ri_launch(rglru_scan_kernel<TO, F>, grid, dim3(threads), 0, s, a, x, y, y_stride, y_bias, \
        state, cu_q, state_slots, (TO*)out, C, out_scale))
    if (fused) { if (out_dtype == RI_BF16) RI_SCAN(bf16, true); else RI_SCAN(float, true); }
    else {
        if (out_dtype == RI_BF16) RI_SCAN(bf16, false); else RI_SCAN(float, false);
        const long long total = (long long)T * C;
        if (out_dtype == RI_BF16)
            RI_CHECKED(ri_launch(rglru_finish_kernel<bf16>, dim3(ew_blocks(total)), dim3(256), 0, s, (const float*)x, y, y_stride,
                                 y_bias, (bf16*)out, T, C, out_scale));
        else
            RI_CHECKED(ri_launch(rglru_finish_kernel<float>, dim3(ew_blocks(total)), dim3(256), 0, s, (const float*)x, y, y_stride,
                                 y_bias, (float*)out, T, C, out_scale));
    }
#undef RI_SCAN
    return ri_launch_status();
}

// o rows of o_stride (RI_F32 or RI_BF16), g fp32 rows of g_stride, out [T][n] of out_dtype
RI_API int ri_sigmoid_gate(const void* o, int o_dtype, int o_stride, const float* g, int g_stride, int group, void* out,
                           int out_dtype, int T, int n, float scale, void* stream) {
    const long long total = (long long)T * n;
    if (total <= 0) return 0;
    if (group <= 0) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_SG(TI, TO) RI_CHECKED(ri_launch(sigmoid_gate_kernel<TI, TO>, dim3(ew_blocks(total)), dim3(256), 0, s, (const TI*)o, \
        o_stride, g, g_stride, group, (TO*)out, T, n, scale))
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
