// Paged attention on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulate) for mixers whose keys
// and values differ in size or in number of heads, compiled for one RI_HEAD_DIM (size of a query and a key) and
// one RI_VALUE_DIM (size of a value), both multiples of 16.  It is the bfloat16 engine's kernel for prompt portions
// of the attention with several maps a head and of the attention over one cached row a token, and for single
// tokens of geometries the one-CTA-a-key-head kernel does not take.
//
// Scores are fp32 sums of exact products of bf16 q and k; scale, cap (cap * tanh(s / cap)), mask and the online
// softmax are fp32; the softmax weights enter the product with the values unrounded: a weight is cut into three
// bf16 pieces (8 + 8 + 8 bits of its significand, their sum is the weight) and every piece is multiplied with the
// bf16 values on the tensor cores with fp32 accumulation, the small pieces first.
//
// A CTA of four warps takes 64 rows of one key head, a row being (query token, query head of that key head), so
// the heads that share a key head share every tile that is loaded; a warp owns 16 rows.  Keys come in tiles of KT
// that start at multiples of KT from key 0 (the sums' order does not depend on how a prompt was cut), gathered page
// by page with cp.async into a double buffer.  Options as in the fp32-arithmetic kernel: `maps` attention maps a
// head (query heads [head][map], key heads [kv head][map], one set of values), values that are the keys' own first
// channels, a window, a term exp(sink_h) in the denominator, fp32 or bf16 output.  With `splits` > 1 the key tiles of
// every CTA are cut into that many ranges, a CTA each (grid z), which leave their unnormalised sums, maximum and sum
// in a scratch; a second kernel joins them.  That is for steps of few tiles over many keys (single tokens of a long
// context), where one CTA a tile would leave most SMs idle.  The reference has one
// attention kernel pair for one head size (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_gqa.h:30).
#include "common.cuh"

#ifndef RI_HEAD_DIM
#error "compile with -DRI_HEAD_DIM=<key size> [-DRI_VALUE_DIM=<value size>]"
#endif
#ifndef RI_VALUE_DIM
#define RI_VALUE_DIM RI_HEAD_DIM
#endif

namespace {
constexpr int HD = RI_HEAD_DIM, VD = RI_VALUE_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 576, "key size: a multiple of 16, at most 576");
static_assert(VD % 16 == 0 && VD >= 16 && VD <= 256, "value size: a multiple of 16, at most 256");
constexpr int MT = 64;                         // rows a CTA
constexpr int THREADS = 128;
constexpr int KT = HD <= 128 ? 64 : 32;        // keys a tile
constexpr int KROW = HD + 8, VROW = VD + 8;    // padded rows: an odd count of 16-byte pieces, ldmatrix meets no conflict
constexpr int KCH = HD / 8, VCH = VD / 8;      // 16-byte pieces a row
constexpr int KS = HD / 16;                    // k-steps of q k^T
constexpr int NT = VD / 8;                     // n-tiles of the output
constexpr bool QREG = HD <= 128;               // the q fragments stay in registers
constexpr int PVG = 4;                         // value fragments (16 channels each) a group of the weights' products
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;              // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

struct Geometry {
    int Hq;                // query heads with their maps
    int Hkv;               // value heads
    int maps;              // maps a head
    int Gc;                // query heads of a key head a CTA takes
    int chunks;            // CTAs a key head's query heads are cut into
    int tpt;               // tokens a tile: MT / Gc
    int page_size;
    int window;            // 0: every earlier key
    int sink;              // the denominator holds exp(sink_values[h]) (null: exp(0)) besides the keys' terms
    int splits;            // ranges the key tiles of a CTA are cut into (grid z); > 1: results go through `part`
    float scale, softcap;  // softcap 0: scores are not capped
    const float* slopes;   // slopes[h] * (query position - key position) is taken off head h's scores (null: no such bias)
};

// keys k0 .. k0+KT-1 of key head `kh` (and, unless the values lie inside the keys, the values of value head `g`)
// into shared memory; keys outside [k_lo, k_hi) are zero-filled and their pages never looked up
template <bool VIK>
__device__ __forceinline__ void load_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ cache, const int* __restrict__ bt,
                                          int k0, int k_lo, int k_hi, size_t page_elems, size_t k_base, size_t v_base,
                                          int page_size) {
    constexpr int PIECES = KCH + (VIK ? 0 : VCH);
    for (int c = threadIdx.x; c < KT * PIECES; c += THREADS) {
        const int kk = c / PIECES, ch = c - kk * PIECES;
        const int key = k0 + kk;
        const bool ok = key >= k_lo && key < k_hi;
        const bf16* src = cache;
        if (ok) {
            const int blk = key / page_size, off = key - blk * page_size;
            const bf16* page = cache + (size_t)bt[blk] * page_elems;
            src = ch < KCH ? page + k_base + (size_t)off * HD + ch * 8 : page + v_base + (size_t)off * VD + (ch - KCH) * 8;
        }
        bf16* dst = ch < KCH ? Ks + kk * KROW + ch * 8 : Vs + kk * VROW + (ch - KCH) * 8;
        cp_async16(dst, src, ok);
    }
}

template <typename TO, bool VIK>
__global__ void __launch_bounds__(THREADS, VD <= 128 ? (VIK ? 4 : 3) : 1)      // values to 128 wide: three or four CTAs an SM
attention_rows_kernel(const bf16* __restrict__ q, int q_stride, TO* __restrict__ out, int out_stride,
                      const bf16* __restrict__ cache, const int* __restrict__ block_table, int table_stride,
                      const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                      const int* __restrict__ tile_entry, const int* __restrict__ tile_tok0,
                      const float* __restrict__ sink_values, float* __restrict__ part, Geometry gm) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [MT][KROW]
    bf16* KVs = Qs + MT * KROW;                              // [2 buffers][K: KT x KROW | V: KT x VROW]
    constexpr int BUF = KT * KROW + (VIK ? 0 : KT * VROW);

    const int b = tile_entry[blockIdx.x];
    if (b < 0) return;
    const int tok0 = tile_tok0[blockIdx.x];
    const int Hk = gm.Hkv * gm.maps;
    const int G = gm.Hq / Hk;                                // query heads a key head
    const int kh = blockIdx.y / gm.chunks, hc = blockIdx.y - kh * gm.chunks;
    const int kvh = kh / gm.maps, mp = kh - kvh * gm.maps;
    const int Gc = gm.Gc;
    const int g0 = hc * Gc, nheads = min(Gc, G - g0);        // heads g0 .. g0+nheads-1 of the key head's group
    const int q_begin = cu_q[b], q_len = cu_q[b + 1] - q_begin;
    const int pos0 = kv_len[b] - q_len;
    const int ntok = min(gm.tpt, q_len - tok0);
    if (ntok <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // query head of the group's g-th head: ((kvh * G + g) * maps + mp)
    auto head_of = [&](int hh) { return (kvh * G + g0 + hh) * gm.maps + mp; };

    for (int c = tid; c < MT * KCH; c += THREADS) {
        const int r = c / KCH, ch = c - r * KCH;
        const int jj = r / Gc, hh = r - jj * Gc;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (jj < ntok && hh < nheads)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(q_begin + tok0 + jj) * q_stride + (size_t)head_of(hh) * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * KROW + ch * 8) = v;
    }

    const int p_first = pos0 + tok0, p_last = p_first + ntok - 1;
    const int lo_tile = gm.window > 0 ? max(0, p_first - gm.window + 1) : 0;
    int t_begin = lo_tile / KT, t_end = p_last / KT + 1;
    if (gm.splits > 1) {
        // this CTA's range of the key tiles; it may be empty
        const int per = (t_end - t_begin + gm.splits - 1) / gm.splits;
        t_begin += blockIdx.z * per;
        t_end = min(t_end, t_begin + per);
    }
    const int* bt = block_table + (size_t)b * table_stride;
    const size_t page_elems = (size_t)gm.page_size * ((size_t)Hk * HD + (VIK ? 0 : (size_t)gm.Hkv * VD));
    const size_t k_base = (size_t)kh * gm.page_size * HD;
    const size_t v_base = (size_t)Hk * gm.page_size * HD + (size_t)kvh * gm.page_size * VD;

    if (t_begin < t_end)
        load_tile<VIK>(KVs, KVs + KT * KROW, cache, bt, t_begin * KT, lo_tile, p_last + 1, page_elems, k_base, v_base, gm.page_size);
    cp_async_commit();
    __syncthreads();                                          // Qs is written

    // this thread's two rows: 16 * warp + lane / 4 and that + 8
    int p_row[2], lo_row[2];
    bool ok_row[2];
    float m[2], l[2] = {0.f, 0.f}, slope[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        const int jj = r / Gc, hh = r - jj * Gc;
        ok_row[i] = jj < ntok && hh < nheads;
        if (gm.slopes && ok_row[i]) slope[i] = gm.slopes[head_of(hh)];
        p_row[i] = p_first + jj;
        lo_row[i] = gm.window > 0 ? max(0, p_row[i] - gm.window + 1) : 0;
        m[i] = -INFINITY;
        if (gm.sink && gm.splits == 1 && ok_row[i]) {           // with ranges, the join adds the term once
            // a term exp(sink_h) without a value: the maximum starts there and, in the one lane of four whose
            // partial sum stands for it, the sum at exp(sink_h - sink_h) = 1
            m[i] = (sink_values ? sink_values[head_of(hh)] : 0.f) * LOG2E;
            if ((lane & 3) == 0) l[i] = 1.f;
        }
    }
    const bool warp_active = (warp * 16) / Gc < ntok;        // rows beyond the tile's tokens: nothing to do

    unsigned qf[QREG ? KS : 1][4];
    if (QREG) {
#pragma unroll
        for (int ks = 0; ks < (QREG ? KS : 1); ++ks)
            ldmatrix_x4(qf[ks], Qs + (warp * 16 + (lane & 15)) * KROW + ks * 16 + (lane >> 4) * 8);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        bf16* Ks = KVs + buf * BUF;
        bf16* Vs = VIK ? Ks : Ks + KT * KROW;
        constexpr int VSTRIDE = VIK ? KROW : VROW;
        if (t + 1 < t_end) {
            bf16* Kn = KVs + (buf ^ 1) * BUF;
            load_tile<VIK>(Kn, Kn + KT * KROW, cache, bt, (t + 1) * KT, lo_tile, p_last + 1, page_elems, k_base, v_base, gm.page_size);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp_active) {
            float s[KT / 8][4];
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                unsigned qk[4];
                if (!QREG) ldmatrix_x4(qk, Qs + (warp * 16 + (lane & 15)) * KROW + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < KT / 16; ++np) {
                    unsigned kf[4];
                    ldmatrix_x4(kf, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * KROW + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * np], QREG ? qf[QREG ? ks : 0] : qk, kf[0], kf[1]);
                    mma_bf16(s[2 * np + 1], QREG ? qf[QREG ? ks : 0] : qk, kf[2], kf[3]);
                }
            }
            // scale, cap, mask; everything from here on in units of log2
            const int key0 = t * KT + (lane & 3) * 2;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + n * 8 + (e & 1);
                    const int i = e >> 1;
                    float sc = s[n][e] * gm.scale;
                    if (gm.softcap > 0.f) sc = gm.softcap * tanhf(sc / gm.softcap);
                    sc -= slope[i] * (float)(p_row[i] - key);
                    const bool seen = ok_row[i] && key <= p_row[i] && key >= lo_row[i];
                    s[n][e] = seen ? sc * LOG2E : -INFINITY;
                    mx[i] = fmaxf(mx[i], s[n][e]);
                }
            }
            float alpha[2], muse[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float mnew = fmaxf(m[i], mx[i]);
                muse[i] = mnew == -INFINITY ? 0.f : mnew;
                alpha[i] = exp2f(m[i] - muse[i]);
                m[i] = mnew;
                l[i] *= alpha[i];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[n][e] = exp2f(s[n][e] - muse[e >> 1]);
                    l[e >> 1] += s[n][e];
                }
            }
#pragma unroll
            for (int kk = 0; kk < KT / 16; ++kk) {
                unsigned pa[3][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a = s[2 * kk + (j >> 1)][(j & 1) * 2], c = s[2 * kk + (j >> 1)][(j & 1) * 2 + 1];
#pragma unroll
                    for (int piece = 0; piece < 3; ++piece) {
                        const unsigned packed = pack_bf16(a, c);
                        pa[piece][j] = packed;
                        a -= __uint_as_float(packed << 16);              // what the piece left out, exactly
                        c -= __uint_as_float(packed & 0xffff0000u);
                    }
                }
                // value fragments in groups of PVG: the products of one piece run over the whole group before the next
                // piece adds to the same accumulators, so consecutive products do not wait for one another
#pragma unroll
                for (int np0 = 0; np0 < NT / 2; np0 += PVG) {
                    unsigned vf[PVG][4];
#pragma unroll
                    for (int g = 0; g < PVG; ++g)
                        if (np0 + g < NT / 2)
                            ldmatrix_x4_trans(vf[g], Vs + (kk * 16 + (lane & 15)) * VSTRIDE + (np0 + g) * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int piece = 2; piece >= 0; --piece) {
#pragma unroll
                        for (int g = 0; g < PVG; ++g) {
                            if (np0 + g < NT / 2) {
                                mma_bf16(o[2 * (np0 + g)], pa[piece], vf[g][0], vf[g][1]);
                                mma_bf16(o[2 * (np0 + g) + 1], pa[piece], vf[g][2], vf[g][3]);
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();                                      // all warps are done with this buffer
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (!ok_row[i]) continue;
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        const int jj = r / Gc, hh = r - jj * Gc;
        if (gm.splits > 1) {
            float* dst = part + ((((size_t)blockIdx.x * gridDim.y + blockIdx.y) * MT + r) * gm.splits + blockIdx.z) * (VD + 2);
#pragma unroll
            for (int n = 0; n < NT; ++n)
                *reinterpret_cast<float2*>(dst + n * 8 + (lane & 3) * 2) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
            if ((lane & 3) == 0) { dst[VD] = m[i]; dst[VD + 1] = l[i]; }
            continue;
        }
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        TO* dst = out + (size_t)(q_begin + tok0 + jj) * out_stride + (size_t)head_of(hh) * VD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            } else {
                *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            }
        }
    }
}

// Joins the ranges of one row of a tile, a warp a row: M = the largest maximum (the sink's exponent among them),
// L = sum l_z 2^(m_z - M) (+ 2^(sink - M)), out = sum acc_z 2^(m_z - M) / L; maxima are in units of log2.  Lane z
// holds range z's weight 2^(m_z - M) (ranges beyond 32 in a second turn); the sums run over the ranges in their order.
constexpr int MERGE_WARPS = 4;
template <typename TO>
__global__ void __launch_bounds__(MERGE_WARPS * 32)
attention_rows_merge_kernel(const float* __restrict__ part, TO* __restrict__ out, int out_stride,
                            const int* __restrict__ cu_q, const int* __restrict__ tile_entry,
                            const int* __restrict__ tile_tok0, const float* __restrict__ sink_values, Geometry gm) {
    pdl_trigger();
    pdl_wait();
    const int b = tile_entry[blockIdx.x];
    if (b < 0) return;
    const int tok0 = tile_tok0[blockIdx.x];
    const int Hk = gm.Hkv * gm.maps, G = gm.Hq / Hk, Gc = gm.Gc;
    const int kh = blockIdx.y / gm.chunks, hc = blockIdx.y - kh * gm.chunks;
    const int kvh = kh / gm.maps, mp = kh - kvh * gm.maps;
    const int g0 = hc * Gc, nheads = min(Gc, G - g0);
    const int q_begin = cu_q[b], ntok = min(gm.tpt, cu_q[b + 1] - q_begin - tok0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z * MERGE_WARPS + warp;
    const int jj = r / Gc, hh = r - jj * Gc;
    if (r >= MT || jj >= ntok || hh >= nheads) return;
    const int head = (kvh * G + g0 + hh) * gm.maps + mp;
    constexpr int REC = VD + 2;
    const float* src = part + (((size_t)blockIdx.x * gridDim.y + blockIdx.y) * MT + r) * gm.splits * REC;
    const float sv = gm.sink ? (sink_values ? sink_values[head] : 0.f) * LOG2E : -INFINITY;
    // ranges lane and lane + 32 (splits <= 64)
    float mz[2], lz[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int z = lane + 32 * k;
        mz[k] = z < gm.splits ? src[(size_t)z * REC + VD] : -INFINITY;
        lz[k] = z < gm.splits ? src[(size_t)z * REC + VD + 1] : 0.f;
    }
    float M = fmaxf(sv, fmaxf(mz[0], mz[1]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float wz[2], L = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        wz[k] = mz[k] == -INFINITY ? 0.f : exp2f(mz[k] - M);
        L += lz[k] * wz[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (gm.sink) L += exp2f(sv - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    TO* dst = out + (size_t)(q_begin + tok0 + jj) * out_stride + (size_t)head * VD;
    constexpr int DPL = (VD + 31) / 32;                       // channels a lane
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    for (int z = 0; z < gm.splits; ++z) {
        const float w = __shfl_sync(0xffffffffu, wz[z >> 5], z & 31);
        if (w == 0.f) continue;                               // an empty range: its sums were never written
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < VD) acc[i] = fmaf(src[(size_t)z * REC + d], w, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d >= VD) continue;
        if constexpr (sizeof(TO) == 4) dst[d] = acc[i] * inv; else dst[d] = __float2bfloat16(acc[i] * inv);
    }
}

template <typename TO, bool VIK>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* cache, const int* block_table,
           int table_stride, const int* cu_q, const int* kv_len, const int* tile_entry, const int* tile_tok0,
           int n_tiles, const float* sink_values, float* part, const Geometry& gm, cudaStream_t s) {
    static bool configured = false;
    const size_t smem = ((size_t)MT * KROW + 2 * ((size_t)KT * KROW + (VIK ? 0 : (size_t)KT * VROW))) * sizeof(bf16);
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_rows_kernel<TO, VIK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, gm.Hkv * gm.maps * gm.chunks, gm.splits);
    RI_CHECKED(ri_launch(attention_rows_kernel<TO, VIK>, grid, dim3(THREADS), smem, s, (const bf16*)q, q_stride, (TO*)out,
                         out_stride, (const bf16*)cache, block_table, table_stride, cu_q, kv_len, tile_entry, tile_tok0,
                         sink_values, part, gm));
    if (gm.splits > 1)
        RI_CHECKED(ri_launch(attention_rows_merge_kernel<TO>, dim3(grid.x, grid.y, MT / MERGE_WARPS), dim3(MERGE_WARPS * 32), 0, s,
                             (const float*)part, (TO*)out, out_stride, cu_q, tile_entry, tile_tok0, sink_values, gm));
    return ri_launch_status();
}
}  // namespace

RI_API int ri_attention_rows_head_dim() { return HD; }
RI_API int ri_attention_rows_value_dim() { return VD; }

// Query heads of a key head one CTA takes: all of them up to 64 (then MT / that many tokens a tile), else 64.
RI_API int ri_attention_rows_heads_per_cta(int Hq, int Hkv, int maps) {
    if (Hkv <= 0 || maps <= 0 || Hq % (Hkv * maps)) return 0;
    const int G = Hq / (Hkv * maps);
    return G < MT ? G : MT;
}

// Tokens of one tile: tile_tok0 counts in these.
RI_API int ri_attention_rows_tokens_per_tile(int Hq, int Hkv, int maps) {
    const int gc = ri_attention_rows_heads_per_cta(Hq, Hkv, maps);
    return gc > 0 ? MT / gc : 0;
}

// CTAs of the attention kernel that fit an SM at once (0: the question failed), for the choice of the key ranges.
RI_API int ri_attention_rows_ctas_per_sm(int value_in_key, int out_f32) {
    int n = 0;
    cudaError_t e = cudaErrorInvalidValue;
#define RI_ROWS_OCC(TO, VIK) do { \
        const size_t smem = ((size_t)MT * KROW + 2 * ((size_t)KT * KROW + (VIK ? 0 : (size_t)KT * VROW))) * sizeof(bf16); \
        e = cudaFuncSetAttribute(attention_rows_kernel<TO, VIK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_rows_kernel<TO, VIK>, THREADS, smem); \
    } while (0)
    if (value_in_key) {
        if constexpr (VD <= HD) { if (out_f32) RI_ROWS_OCC(float, true); else RI_ROWS_OCC(bf16, true); }
    } else {
        if (out_f32) RI_ROWS_OCC(float, false); else RI_ROWS_OCC(bf16, false);
    }
#undef RI_ROWS_OCC
    return e == cudaSuccess ? n : 0;
}

// q [T][q_stride] bf16, head h at column h*HD; out rows of out_stride, head h at column h*VD, fp32 (out_f32) or bf16.
// cache: per page the keys [key head][slot][HD], then (unless value_in_key) the values [value head][slot][VD], bf16,
// every page starting on a 16-byte boundary.  tile_entry[i]: batch entry of tile i (-1: skip), tile_tok0[i] its first
// token within the entry; a tile holds ri_attention_rows_tokens_per_tile tokens.  splits > 1: the key tiles of every CTA
// in that many ranges through `part`, fp32 [n_tiles][key heads * chunks][64 rows][splits][VD + 2], and a second launch.
RI_API int ri_attention_rows(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                             const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                             const int* tile_entry, const int* tile_tok0, int n_tiles, int Hq, int Hkv, int page_size,
                             float scale, int window, int sink, float softcap, const float* sink_values, int maps,
                             int value_in_key, int out_f32, int splits, float* part, const float* slopes,
                             void* stream) {
    if (n_tiles <= 0) return 0;
    if (splits < 1 || splits > 64 || (splits > 1 && !part)) return (int)cudaErrorInvalidValue;
    const int gc = ri_attention_rows_heads_per_cta(Hq, Hkv, maps);
    if (gc <= 0 || (value_in_key && (maps != 1 || VD > HD)) || q_stride % 8) return (int)cudaErrorInvalidValue;
    const int G = Hq / (Hkv * maps);
    Geometry gm{Hq, Hkv, maps, gc, (G + gc - 1) / gc, MT / gc, page_size, window, sink, splits, scale, softcap, slopes};
    cudaStream_t s = (cudaStream_t)stream;
#define RI_ROWS_GO(TO, VIK) launch<TO, VIK>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q, kv_len, \
                                            tile_entry, tile_tok0, n_tiles, sink_values, part, gm, s)
    if (value_in_key) {
        if constexpr (VD <= HD) return out_f32 ? RI_ROWS_GO(float, true) : RI_ROWS_GO(bf16, true);
        return (int)cudaErrorInvalidValue;
    }
    return out_f32 ? RI_ROWS_GO(float, false) : RI_ROWS_GO(bf16, false);
#undef RI_ROWS_GO
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
