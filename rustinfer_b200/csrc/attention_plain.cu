// Paged causal GQA attention over the cache, any head size (compiled for one
// RI_HEAD_DIM and, where values have a size of their own, one RI_VALUE_DIM), storage fp32
// or bf16, all arithmetic fp32 on CUDA cores.  It is the attention of the true-32-bit path and the fallback of the bf16
// path; it serves whole prompts, portions of prompts and single decoded tokens alike.
//
// What it computes is RustInfer's paged attention
// (crates/infer-core/src/ports/fused_ops.rs:484-523): the query at position p of a
// request sees keys 0..p (with a window w: p-w+1..p), kv head = q head / (Hq/Hkv),
// scores (q.k)*scale, softmax with the maximum subtracted.  With a block size c the query
// at p sees only keys from floor(p/c)*c on (blocks are counted from position 0 of the
// request): a lower bound like the window's, and both may be given.  The reference has no fp32
// attention on the GPU (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_gqa.h:30).
//
// One CTA of 128 threads handles a tile of 16 consecutive query tokens of one request
// and one q head.  Keys are visited in chunks of KC that start at multiples of KC from
// key 0, with an online softmax; the order of every sum is therefore the same however
// the tokens were cut into steps or tiles, and so are the bits of the result.
#include "common.cuh"

#ifndef RI_HEAD_DIM
#error "compile with -DRI_HEAD_DIM=<head size>"
#endif

#ifndef RI_VALUE_DIM
#define RI_VALUE_DIM RI_HEAD_DIM
#endif

namespace {
constexpr int HD = RI_HEAD_DIM;                // size of a query and a key
constexpr int VD = RI_VALUE_DIM;               // size of a value and of a head's output
static_assert(HD >= 1 && HD <= 512 && VD >= 1 && VD <= 512, "head sizes up to 512");
constexpr int QT = 16;                         // query rows per CTA
constexpr int KC = HD <= 128 ? 64 : 32;        // keys per chunk
constexpr int THREADS = 128;
constexpr int NCOL = KC / 8;                   // score columns per thread
constexpr int NACC = (VD + 7) / 8;             // output dims per thread
constexpr int QS = HD + 1, KS = HD + 1, PS = KC + 1;
constexpr size_t SMEM_FLOATS = (size_t)QT * QS + (size_t)KC * KS + (size_t)KC * VD + (size_t)QT * PS;

// What mixers beyond plain grouped-query attention ask for.
//   softcap > 0      score <- softcap * tanh(score / softcap), after the scale
//   sink_values      with `sink`: the exponent of the term the denominator holds besides the keys', one per
//                    query head (null: 0 for every head)
//   maps >= 1        attention maps a head: the query heads come as [head][map], the key heads as
//                    [kv head][map], and the maps of a head share the values of kv head = head / (heads / kv heads).
//                    Hq counts query heads with their maps, Hkv the value heads; the cache holds Hkv * maps key heads.
//   value_in_key     the value of a key is its own first VD channels; the cache holds keys only
//   slopes           a linear distance bias: slopes[h] * (query position - key position) is taken off the score of
//                    query head h, after scale and cap (null: none)
struct Extra {
    float softcap;
    const float* sink_values;
    int maps;
    int value_in_key;
    const float* slopes;
};

// key head and value head of query head h
__device__ __forceinline__ void heads_of(int h, int Hq, int Hkv, int maps, int& key_head, int& value_head) {
    const int per = Hq / (Hkv * maps);                   // heads (each of `maps` maps) a kv head
    value_head = (h / maps) / per;
    key_head = value_head * maps + h % maps;
}

template <typename T, typename TO>
__global__ void __launch_bounds__(THREADS)
attention_plain_kernel(const T* __restrict__ q, int q_stride, TO* __restrict__ out, int out_stride,
                       const T* __restrict__ cache, const int* __restrict__ block_table,
                       int table_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                       const int* __restrict__ tile_entry, const int* __restrict__ tile_q0,
                       int Hq, int Hkv, int page_size, float scale, int window, int block, int sink, Extra ex) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* Qs = smem;
    float* Ks = Qs + QT * QS;
    float* Vs = Ks + KC * KS;
    float* Ps = Vs + KC * VD;

    const int tile = blockIdx.x, h = blockIdx.y;
    const int b = tile_entry[tile];
    if (b < 0) return;                                   // padding tile
    const int j0 = tile_q0[tile];
    const int q_begin = cu_q[b], q_len = cu_q[b + 1] - q_begin;
    const int kvl = kv_len[b];
    const int pos0 = kvl - q_len;                        // position of the entry's first token
    int kh, g;                                           // key head, value head
    heads_of(h, Hq, Hkv, ex.maps, kh, g);
    const int tid = threadIdx.x;
    const int row = tid >> 3, l8 = tid & 7;
    const int rows_here = min(QT, q_len - j0);
    if (rows_here <= 0) return;

    for (int e = tid; e < QT * HD; e += THREADS) {
        const int r = e / HD, d = e - r * HD;
        Qs[r * QS + d] = r < rows_here
            ? to_f32<T>(q[(size_t)(q_begin + j0 + r) * q_stride + (size_t)h * HD + d]) : 0.f;
    }

    const bool row_valid = row < rows_here;
    const int p_row = pos0 + j0 + row;                   // this row's position
    int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const int p_last = pos0 + j0 + rows_here - 1;        // last key any row of the tile sees
    int lo_tile = window > 0 ? max(0, pos0 + j0 - window + 1) : 0;   // first key its first row sees
    if (block > 0) {
        lo_row = max(lo_row, (p_row / block) * block);
        lo_tile = max(lo_tile, ((pos0 + j0) / block) * block);
    }

    // with a sink the sums start from a key of score 0 that has no value: maximum 0, sum exp(0 - 0) = 1
    // (with sink values: a term exp(sink_h) instead, so the maximum starts at sink_h)
    float m = sink ? (ex.sink_values ? ex.sink_values[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;
    const float slope = ex.slopes ? ex.slopes[h] : 0.f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

    const int* bt = block_table + (size_t)b * table_stride;
    // a page: keys [kv head][slot][HD], then values [kv head][slot][VD]
    const int Hk = Hkv * ex.maps;
    const size_t page_elems = (size_t)page_size * ((size_t)Hk * HD + (ex.value_in_key ? 0 : (size_t)Hkv * VD));
    const size_t k_base = (size_t)kh * page_size * HD;
    const size_t v_base = ex.value_in_key ? k_base : (size_t)Hk * page_size * HD + (size_t)g * page_size * VD;
    const int v_row = ex.value_in_key ? HD : VD;         // elements from one key's value to the next
    for (int kb = (lo_tile / KC) * KC; kb <= p_last; kb += KC) {
        __syncthreads();                                 // previous chunk's Vs/Ps reads are done
        // a warp a key: the page is looked up once per key and the lanes read along the head
        for (int kk = tid >> 5; kk < KC; kk += THREADS / 32) {
            const int key = kb + kk;
            const bool seen = key >= lo_tile && key <= p_last;
            const T* kp = cache;
            const T* vp = cache;
            if (seen) {
                const int blk = key / page_size;
                const size_t page = (size_t)bt[blk] * page_elems;
                const int off = key - blk * page_size;
                kp = cache + page + k_base + (size_t)off * HD;
                vp = cache + page + v_base + (size_t)off * v_row;
            }
            for (int d = tid & 31; d < HD; d += 32) Ks[kk * KS + d] = seen ? to_f32<T>(kp[d]) : 0.f;
            for (int d = tid & 31; d < VD; d += 32) Vs[kk * VD + d] = seen ? to_f32<T>(vp[d]) : 0.f;
        }
        __syncthreads();

        float s[NCOL];
        float cmax = -INFINITY;
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
            const int kk = l8 + 8 * c;
            const int key = kb + kk;
            float dot = 0.f;
            const float* qr = Qs + row * QS;
            const float* kr = Ks + kk * KS;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) dot = fmaf(qr[d], kr[d], dot);
            const bool seen = row_valid && key <= p_row && key >= lo_row;
            float sc = dot * scale;
            if (ex.softcap > 0.f) sc = ex.softcap * tanhf(sc / ex.softcap);
            if (ex.slopes) sc -= slope * (float)(p_row - key);
            s[c] = seen ? sc : -INFINITY;
            cmax = fmaxf(cmax, s[c]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
        const float m_new = fmaxf(m, cmax);
        float alpha = 1.f, psum = 0.f;
        if (m_new == -INFINITY) {
#pragma unroll
            for (int c = 0; c < NCOL; ++c) Ps[row * PS + l8 + 8 * c] = 0.f;
        } else {
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                const float p = (s[c] == -INFINITY) ? 0.f : expf(s[c] - m_new);
                Ps[row * PS + l8 + 8 * c] = p;
                psum += p;
            }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        __syncthreads();
        const float* pr = Ps + row * PS;
        for (int kk = 0; kk < KC; ++kk) {
            const float p = pr[kk];
            const float* vr = Vs + kk * VD + l8;
#pragma unroll
            for (int i = 0; i < NACC; ++i)
                if (VD % 8 == 0 || l8 + 8 * i < VD) acc[i] = fmaf(p, vr[8 * i], acc[i]);
        }
    }
    if (row_valid) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        TO* o = out + (size_t)(q_begin + j0 + row) * out_stride + (size_t)h * VD + l8;
#pragma unroll
        for (int i = 0; i < NACC; ++i)
            if (VD % 8 == 0 || l8 + 8 * i < VD) o[8 * i] = from_f32<TO>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------ entries of a single token
// One CTA per (kv head, entry that brings one token): the G query heads of the kv head share every
// key and value it reads.  Keys are taken in chunks of SK with a running maximum and sum per head
// (fp32 throughout): a thread a key for the scores (q in shared memory, a key element serves all G
// heads), a warp a head for the chunk's maximum and weights, a warp a key and a lane a value channel
// for the weighted sum, the warps' parts added at the end.  Same mask as above: keys lo .. p with
// lo the later of the window's and the block's start.  With gridDim.z > 1 the keys lo .. p are cut into that
// many ranges, a CTA each, which leave their maximum, sum and unnormalised weighted sum in `part`
// ([entry][head][range][VD + 2] fp32: the sums' VD values, then maximum and sum); the merge kernel below
// joins them (and adds the sink there).
constexpr int SK = 512;                        // keys per chunk
constexpr int SG = 16;                         // most query heads a kv head
constexpr int SV = (VD + 31) / 32;             // value channels a lane
// the parts of the weighted sum that meet in shared memory at the end: a warp's (old walk) or, in the wide walk,
// a thread's (up to 8 heads x 8 channels each)
constexpr size_t SINGLE_RED_FLOATS = (size_t)(THREADS / 32) * SG * VD > (size_t)THREADS * 64 ? (size_t)(THREADS / 32) * SG * VD
                                                                                             : (size_t)THREADS * 64;
constexpr size_t SINGLE_SMEM_FLOATS = (size_t)SG * HD + (size_t)SG * SK + 3 * SG + SINGLE_RED_FLOATS;

// GM: the most query heads a kv head this instantiation keeps sums for (4, 8 or 16).  With up to 8 heads, values
// whose rows are whole 16-byte pieces and a piece count that divides the CTA, the weighted sum runs "wide": a
// thread owns one 16-byte piece of the value row and every (THREADS / pieces)-th key, so that one load serves
// 8 (bf16) channels of all heads and 128 loads are in flight a CTA instead of 16; the threads' parts are added
// in a fixed order at the end.
template <typename T, typename TO, int GM>
__global__ void __launch_bounds__(THREADS)
attention_single_kernel(const T* __restrict__ q, int q_stride, TO* __restrict__ out, int out_stride,
                        const T* __restrict__ cache, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                        const int* __restrict__ entry_list, int Hq, int Hkv, int page_size, float scale,
                        int window, int block, int sink, float* __restrict__ part, Extra ex) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int Hk = Hkv * ex.maps;                        // key heads: a CTA each
    const int G = Hq / Hk;                               // query heads that read this CTA's key head
    float* qs = smem;                                    // [G][HD]
    float* sc = qs + SG * HD;                            // [G][SK]
    float* mrun = sc + SG * SK;                          // [G] running maximum
    float* lrun = mrun + SG;                             // [G] running sum
    float* arun = lrun + SG;                             // [G] what the chunk rescales the old sums by
    float* red = arun + SG;                              // [warps][G][VD]
    const int kh = blockIdx.x, kvh = kh / ex.maps, mp = kh - kvh * ex.maps;
    // the g-th of them is query head (kvh * G + g) * maps + mp
    const int head0 = kvh * G * ex.maps + mp, head_step = ex.maps;
    const int b = entry_list[blockIdx.y];
    if (b < 0) return;
    const int t = cu_q[b];
    if (cu_q[b + 1] - t != 1) return;
    int p = kv_len[b] - 1;
    const int p_query = p;                               // the token's own position (p becomes its range's end)
    int lo = window > 0 ? max(0, p - window + 1) : 0;
    if (block > 0) lo = max(lo, (p / block) * block);
    const int splits = gridDim.z;
    if (splits > 1) {
        // this CTA's range of the keys, a multiple of 64 long; it may be empty
        const int per = ((p - lo + 1 + splits - 1) / splits + 63) & ~63;
        lo += blockIdx.z * per;
        p = min(p, lo + per - 1);
        sink = 0;                                        // the merge adds it once
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int WARPS = THREADS / 32;
    for (int e = tid; e < G * HD; e += THREADS) {
        const int g = e / HD;
        qs[e] = to_f32<T>(q[(size_t)t * q_stride + (size_t)(head0 + g * head_step) * HD + (e - g * HD)]);
    }
    if (tid < G) {
        mrun[tid] = sink ? (ex.sink_values ? ex.sink_values[head0 + tid * head_step] : 0.f) : -INFINITY;
        lrun[tid] = sink ? 1.f : 0.f;
    }
    constexpr int VECW = 16 / (int)sizeof(T);               // elements of a 16-byte piece
    constexpr int PIECES = VD % VECW == 0 ? VD / VECW : 1;  // pieces of a value row
    constexpr bool WIDE_OK = GM <= 8 && VD % VECW == 0 && THREADS % PIECES == 0 && PIECES <= THREADS;
    constexpr int KG = WIDE_OK ? THREADS / PIECES : 1;      // keys a pass of the wide walk takes
    float acc[WIDE_OK ? 1 : GM][SV];
    float accw[WIDE_OK ? GM : 1][VECW];
#pragma unroll
    for (int g = 0; g < (WIDE_OK ? 1 : GM); ++g)
#pragma unroll
        for (int i = 0; i < SV; ++i) acc[g][i] = 0.f;
#pragma unroll
    for (int g = 0; g < (WIDE_OK ? GM : 1); ++g)
#pragma unroll
        for (int i = 0; i < VECW; ++i) accw[g][i] = 0.f;
    const int* bt = block_table + (size_t)b * table_stride;
    const size_t page_elems = (size_t)page_size * ((size_t)Hk * HD + (ex.value_in_key ? 0 : (size_t)Hkv * VD));
    const size_t k_base = (size_t)kh * page_size * HD;
    const size_t v_base = ex.value_in_key ? k_base : (size_t)Hk * page_size * HD + (size_t)kvh * page_size * VD;
    const int v_row = ex.value_in_key ? HD : VD;         // elements from one key's value to the next
    // value rows start on 16-byte boundaries (the cache itself does: the host checks)
    const bool wide = WIDE_OK && page_elems % VECW == 0 && v_base % VECW == 0 && v_row % VECW == 0;
    const int piece = tid % PIECES, kgroup = tid / PIECES;
    __syncthreads();
    for (int k0 = lo; k0 <= p; k0 += SK) {
        const int n = min(SK, p - k0 + 1);
        // scores of the chunk: a thread a key
        for (int kk = tid; kk < n; kk += THREADS) {
            const int key = k0 + kk, blk = key / page_size;
            const T* kp = cache + (size_t)bt[blk] * page_elems + k_base + (size_t)(key - blk * page_size) * HD;
            float s[SG];
#pragma unroll
            for (int g = 0; g < SG; ++g) s[g] = 0.f;
            constexpr int VEC = 16 / (int)sizeof(T);         // elements of a 16-byte load
            if (HD % VEC == 0 && page_elems % VEC == 0) {    // key rows start on 16-byte boundaries then
#pragma unroll 4
                for (int d0 = 0; d0 < HD; d0 += VEC) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kp + d0);
                    const T* e = reinterpret_cast<const T*>(&raw);
                    float kd[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) kd[i] = to_f32<T>(e[i]);
                    // a head's q comes four channels a shared-memory load (every thread the same address)
#pragma unroll
                    for (int g = 0; g < SG; ++g)
                        if (g < G) {
#pragma unroll
                            for (int i = 0; i < VEC; i += 4) {
                                const float4 q4 = *reinterpret_cast<const float4*>(qs + g * HD + d0 + i);
                                s[g] = fmaf(q4.x, kd[i], s[g]);
                                s[g] = fmaf(q4.y, kd[i + 1], s[g]);
                                s[g] = fmaf(q4.z, kd[i + 2], s[g]);
                                s[g] = fmaf(q4.w, kd[i + 3], s[g]);
                            }
                        }
                }
            } else {
                for (int d = 0; d < HD; ++d) {
                    const float kd = to_f32<T>(kp[d]);
#pragma unroll
                    for (int g = 0; g < SG; ++g)
                        if (g < G) s[g] = fmaf(qs[g * HD + d], kd, s[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < SG; ++g)
                if (g < G) {
                    float x = s[g] * scale;
                    if (ex.softcap > 0.f) x = ex.softcap * tanhf(x / ex.softcap);
                    if (ex.slopes) x -= ex.slopes[head0 + g * head_step] * (float)(p_query - key);
                    sc[g * SK + kk] = x;
                }
        }
        __syncthreads();
        // the chunk's maximum, the weights and their sum: a warp a head
        for (int g = warp; g < G; g += WARPS) {
            float mx = -INFINITY;
            for (int kk = lane; kk < n; kk += 32) mx = fmaxf(mx, sc[g * SK + kk]);
            mx = warp_max(mx);
            const float m_old = mrun[g], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int kk = lane; kk < n; kk += 32) {
                const float w = expf(sc[g * SK + kk] - m_new);
                sc[g * SK + kk] = w;
                sum += w;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float a = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                arun[g] = a;
                lrun[g] = lrun[g] * a + sum;
                mrun[g] = m_new;
            }
        }
        __syncthreads();
        if (WIDE_OK) {
#pragma unroll
            for (int g = 0; g < (WIDE_OK ? GM : 1); ++g)
                if (g < G) {
                    const float a = arun[g];
#pragma unroll
                    for (int i = 0; i < VECW; ++i) accw[g][i] *= a;
                }
        }
        if (WIDE_OK && wide) {
            // weighted sum of the values, wide: a thread a 16-byte piece of every KG-th key's row
#pragma unroll 4                                          // the loads of four keys in flight a thread
            for (int kk = kgroup; kk < n; kk += KG) {
                const int key = k0 + kk, blk = key / page_size;
                const T* vp = cache + (size_t)bt[blk] * page_elems + v_base + (size_t)(key - blk * page_size) * v_row + piece * VECW;
                const uint4 raw = *reinterpret_cast<const uint4*>(vp);
                const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int g = 0; g < (WIDE_OK ? GM : 1); ++g)
                    if (g < G) {
                        const float w = sc[g * SK + kk];
#pragma unroll
                        for (int i = 0; i < VECW; ++i) accw[g][i] = fmaf(w, to_f32<T>(e[i]), accw[g][i]);
                    }
            }
        } else {
            // weighted sum of the values: a warp a key, a lane a value channel
#pragma unroll
            for (int g = 0; g < (WIDE_OK ? 1 : GM); ++g)
                if (g < G) {
                    const float a = arun[g];
#pragma unroll
                    for (int i = 0; i < SV; ++i) acc[g][i] *= a;
                }
            if (!WIDE_OK) {
#pragma unroll 4                                          // the loads of four keys in flight
                for (int kk = warp; kk < n; kk += WARPS) {
                    const int key = k0 + kk, blk = key / page_size;
                    const T* vp = cache + (size_t)bt[blk] * page_elems + v_base + (size_t)(key - blk * page_size) * v_row;
                    float v[SV];
#pragma unroll
                    for (int i = 0; i < SV; ++i) v[i] = lane + 32 * i < VD ? to_f32<T>(vp[lane + 32 * i]) : 0.f;
#pragma unroll
                    for (int g = 0; g < (WIDE_OK ? 1 : GM); ++g)
                        if (g < G) {
                            const float w = sc[g * SK + kk];
#pragma unroll
                            for (int i = 0; i < SV; ++i) acc[g][i] = fmaf(w, v[i], acc[g][i]);
                        }
                }
            } else {
                // rows that are no whole 16-byte pieces at run time (an odd page or head count): a thread a
                // piece still, element by element
                for (int kk = kgroup; kk < n; kk += KG) {
                    const int key = k0 + kk, blk = key / page_size;
                    const T* vp = cache + (size_t)bt[blk] * page_elems + v_base + (size_t)(key - blk * page_size) * v_row + piece * VECW;
#pragma unroll
                    for (int g = 0; g < (WIDE_OK ? GM : 1); ++g)
                        if (g < G) {
                            const float w = sc[g * SK + kk];
#pragma unroll
                            for (int i = 0; i < VECW; ++i) accw[g][i] = fmaf(w, to_f32<T>(vp[i]), accw[g][i]);
                        }
                }
            }
        }
        __syncthreads();                                 // sc and arun are free for the next chunk
    }
    if (WIDE_OK) {
        // a thread's part: [key group][head][piece's channels]
#pragma unroll
        for (int g = 0; g < (WIDE_OK ? GM : 1); ++g)
            if (g < G) {
#pragma unroll
                for (int i = 0; i < VECW; ++i) red[((size_t)kgroup * GM + g) * VD + piece * VECW + i] = accw[g][i];
            }
    } else {
#pragma unroll
        for (int g = 0; g < (WIDE_OK ? 1 : GM); ++g)
            if (g < G) {
#pragma unroll
                for (int i = 0; i < SV; ++i)
                    if (lane + 32 * i < VD) red[((size_t)warp * SG + g) * VD + lane + 32 * i] = acc[g][i];
            }
    }
    __syncthreads();
    for (int e = tid; e < G * VD; e += THREADS) {
        const int g = e / VD, d = e - g * VD;
        float total = 0.f;
        if (WIDE_OK) {
            for (int w = 0; w < KG; ++w) total += red[((size_t)w * GM + g) * VD + d];
        } else {
            for (int w = 0; w < WARPS; ++w) total += red[((size_t)w * SG + g) * VD + d];
        }
        const float l = lrun[g];
        if (splits > 1) {
            float* dst = part + (((size_t)blockIdx.y * Hq + head0 + g * head_step) * splits + blockIdx.z) * (VD + 2);
            dst[d] = total;
            if (d == 0) { dst[VD] = mrun[g]; dst[VD + 1] = l; }
        } else {
            out[(size_t)t * out_stride + (size_t)(head0 + g * head_step) * VD + d] = from_f32<TO>(l > 0.f ? total / l : 0.f);
        }
    }
}

// Joins the ranges of one (entry, head), a warp each: M = the largest maximum (0 with the sink), L = sum
// l_z e^(m_z - M) (+ e^(-M) for the sink), out = sum acc_z e^(m_z - M) / L.  Lane z holds range z's weight (ranges
// beyond 32 in a second turn), so the ranges' numbers are loaded side by side rather than one after the other; the
// sums run over the ranges in their order, so the result is the same whatever else runs.
template <typename T>
__global__ void __launch_bounds__(32)
attention_single_merge_kernel(const float* __restrict__ part, T* __restrict__ out, int out_stride,
                              const int* __restrict__ cu_q, const int* __restrict__ entry_list,
                              int Hq, int splits, int sink, const float* __restrict__ sink_values) {
    pdl_trigger();
    pdl_wait();
    const int b = entry_list[blockIdx.y], h = blockIdx.x;
    if (b < 0) return;
    const int t = cu_q[b];
    if (cu_q[b + 1] - t != 1) return;
    constexpr int REC = VD + 2;
    const int lane = threadIdx.x;
    const float* src = part + ((size_t)blockIdx.y * Hq + h) * splits * REC;
    const float sv = sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY;    // the sink's exponent
    float mz[2], lz[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int z = lane + 32 * k;
        mz[k] = z < splits ? src[(size_t)z * REC + VD] : -INFINITY;
        lz[k] = z < splits ? src[(size_t)z * REC + VD + 1] : 0.f;
    }
    float M = fmaxf(sv, fmaxf(mz[0], mz[1]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float wz[2], L = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        wz[k] = mz[k] == -INFINITY ? 0.f : expf(mz[k] - M);
        L += lz[k] * wz[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (sink) L += expf(sv - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    constexpr int DPL = (VD + 31) / 32;                       // channels a lane
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
#pragma unroll 4
    for (int z = 0; z < splits; ++z) {
        const float w = __shfl_sync(0xffffffffu, wz[z >> 5], z & 31);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            // an empty range left its maximum at -inf and its sums unwritten: weight 0, and nothing read
            if (d < VD && w != 0.f) acc[i] = fmaf(src[(size_t)z * REC + d], w, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < VD) out[(size_t)t * out_stride + (size_t)h * VD + d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T, typename TO>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* cache,
           const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
           const int* tile_entry, const int* tile_q0, int n_tiles, int Hq, int Hkv, int page_size,
           float scale, int window, int block, int sink, Extra ex, cudaStream_t s) {
    static bool configured = false;
    const size_t smem = SMEM_FLOATS * sizeof(float);
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_plain_kernel<T, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, Hq);
    RI_CHECKED(ri_launch(attention_plain_kernel<T, TO>, dim3(grid), dim3(THREADS), smem, s,
        (const T*)q, q_stride, (TO*)out, out_stride, (const T*)cache, block_table, table_stride,
        cu_q, kv_len, tile_entry, tile_q0, Hq, Hkv, page_size, scale, window, block, sink, ex));
    return ri_launch_status();
}

bool extra_fits(int Hq, int Hkv, const Extra& ex) {
    return Hkv > 0 && ex.maps >= 1 && Hq % (Hkv * ex.maps) == 0 && (!ex.value_in_key || (VD <= HD && ex.maps == 1 && Hkv >= 1));
}
}  // namespace

RI_API int ri_attention_plain_head_dim() { return HD; }
RI_API int ri_attention_plain_value_dim() { return VD; }
RI_API int ri_attention_plain_tile_rows() { return QT; }

// q: rows of `q_stride` elements, head h at column h*HD; out rows of out_stride, head h at
// column h*VD.  cache: one layer, per page the keys [kv head][slot][HD] and then the values
// [kv head][slot][VD] ([page][K|V][kv head][slot][HD] when the two sizes are equal).  tile_entry[i] = batch entry of tile i
// (-1: skip), tile_q0[i] = its first query row within that entry.  sink: the softmax's denominator has one
// added, p_j = exp(s_j) / (1 + sum exp(s_j)): a key of score 0 that carries no value.
// The same with the options of `Extra` (see there) and, with out_f32, an fp32 `out` whatever the cache's dtype.
RI_API int ri_attention_plain_ex(const void* q, int q_stride, void* out, int out_stride,
                                 const void* cache, int dtype, const int* block_table, int table_stride,
                                 const int* cu_q, const int* kv_len, const int* tile_entry,
                                 const int* tile_q0, int n_tiles, int Hq, int Hkv, int page_size,
                                 float scale, int window, int block, int sink, float softcap,
                                 const float* sink_values, int maps, int value_in_key, int out_f32, const float* slopes,
                                 void* stream) {
    if (n_tiles <= 0) return 0;
    const Extra ex{softcap, sink_values, maps, value_in_key, slopes};
    if (!extra_fits(Hq, Hkv, ex)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RI_BF16 && out_f32)
        return launch<bf16, float>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q,
                                   kv_len, tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, block, sink, ex, s);
    if (dtype == RI_BF16)
        return launch<bf16, bf16>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q,
                                  kv_len, tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, block, sink, ex, s);
    return launch<float, float>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q,
                                kv_len, tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, block, sink, ex, s);
}

RI_API int ri_attention_plain(const void* q, int q_stride, void* out, int out_stride,
                              const void* cache, int dtype, const int* block_table, int table_stride,
                              const int* cu_q, const int* kv_len, const int* tile_entry,
                              const int* tile_q0, int n_tiles, int Hq, int Hkv, int page_size,
                              float scale, int window, int block, int sink, void* stream) {
    return ri_attention_plain_ex(q, q_stride, out, out_stride, cache, dtype, block_table, table_stride, cu_q, kv_len,
                                 tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, block, sink,
                                 0.f, nullptr, 1, 0, 0, nullptr, stream);
}

// Entries that bring a single token (entry_list[i], -1: skip): keys and values of a kv head are read once
// for its query heads.  splits > 1: every entry's keys in that many ranges (a CTA each) through `part`, fp32
// [n_entries][Hq][splits][VD + 2], and a second launch that joins them.  Returns cudaErrorNotSupported for more than 16 query heads a kv head or values
// wider than 128 (the caller then uses the tiled kernel above, which takes everything).
RI_API int ri_attention_single_ex(const void* q, int q_stride, void* out, int out_stride, const void* cache, int dtype,
                                  const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                  const int* entry_list, int n_entries, int Hq, int Hkv, int page_size, float scale,
                                  int window, int block, int sink, int splits, float* part, float softcap,
                                  const float* sink_values, int maps, int value_in_key, int out_f32,
                                  const float* slopes, void* stream) {
    if (n_entries <= 0) return 0;
    const Extra ex{softcap, sink_values, maps, value_in_key, slopes};
    if (!extra_fits(Hq, Hkv, ex)) return (int)cudaErrorInvalidValue;
    if (Hq / (Hkv * maps) > SG || SV > 4) return (int)cudaErrorNotSupported;
    if (splits < 1 || splits > 64 || (splits > 1 && !part)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(Hkv * maps, n_entries, splits);
#define RI_SINGLE(T, TO) do { const int G_ = Hq / (Hkv * maps); \
    if (G_ <= 4) RI_SINGLE_G(T, TO, 4); else if (G_ <= 8) RI_SINGLE_G(T, TO, 8); else RI_SINGLE_G(T, TO, 16); } while (0)
#define RI_SINGLE_G(T, TO, GM) do { static bool configured = false; \
    /* the parts' meeting place is as large as this many heads need: fewer heads, more CTAs an SM */ \
    const size_t wide_red = GM <= 8 ? (size_t)THREADS * GM * 8 : 0, old_red = (size_t)(THREADS / 32) * SG * VD; \
    const size_t smem = ((size_t)SG * HD + (size_t)SG * SK + 3 * SG + (wide_red > old_red ? wide_red : old_red)) * sizeof(float); \
    if (!configured) { \
        cudaError_t e = cudaFuncSetAttribute(attention_single_kernel<T, TO, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e; \
        configured = true; } \
    RI_CHECKED(ri_launch(attention_single_kernel<T, TO, GM>, dim3(grid), dim3(THREADS), smem, s, (const T*)q, q_stride, (TO*)out, \
        out_stride, (const T*)cache, block_table, table_stride, cu_q, kv_len, entry_list, Hq, Hkv, page_size, scale, \
        window, block, sink, part, ex)); \
    if (splits > 1) RI_CHECKED(ri_launch(attention_single_merge_kernel<TO>, dim3(Hq, n_entries), dim3(32), 0, s, \
        (const float*)part, (TO*)out, out_stride, cu_q, entry_list, Hq, splits, sink, sink_values)); } while (0)
    if (dtype == RI_BF16 && out_f32) RI_SINGLE(bf16, float);
    else if (dtype == RI_BF16) RI_SINGLE(bf16, bf16);
    else RI_SINGLE(float, float);
#undef RI_SINGLE
#undef RI_SINGLE_G
    return ri_launch_status();
}

RI_API int ri_attention_single(const void* q, int q_stride, void* out, int out_stride, const void* cache, int dtype,
                               const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                               const int* entry_list, int n_entries, int Hq, int Hkv, int page_size, float scale,
                               int window, int block, int sink, int splits, float* part, void* stream) {
    return ri_attention_single_ex(q, q_stride, out, out_stride, cache, dtype, block_table, table_stride, cu_q, kv_len,
                                  entry_list, n_entries, Hq, Hkv, page_size, scale, window, block, sink, splits, part,
                                  0.f, nullptr, 1, 0, 0, nullptr, stream);
}

RI_API int ri_attention_single_supports(int Hq, int Hkv) {
    return Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= SG && SV <= 4 &&
           SINGLE_SMEM_FLOATS * sizeof(float) <= 200 * 1024;
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
