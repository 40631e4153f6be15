// A feed-forward of routed experts: the router's choice, the sort of (token, choice) pairs by expert,
// the experts' products over the sorted rows, and the weighted sum back per token.  Nothing here reads a
// count on the host: every launch has a grid that covers the worst case and finds its work in the offsets
// the sort left on the device, so a step of these kernels can be captured in a CUDA graph.
//
//   route    x [T][d], router matrix [E][d] fp32 -> logits z = W x in fp32 -> ids [T][top], weights [T][top] fp32,
//            counts[e] += 1 (or from given logits z [T][E])
//   sort     ids, counts -> offsets [E+1], order [T*top] (pairs in expert order, stable), place [T*top]
//   products rows of an expert times that expert's matrix (fp32 sums in a fixed order of k)
//   combine  y[t] = sum_j weight[t][j] * Y[place[t*top + j]] (+ shared[t]); counts put back to zero
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------- router
// One CTA a token.  Logit z_e = sum_i W[e][i] x[i] in fp32 (a lane every 32nd term, then a butterfly over the
// lanes: the same order whatever else is in the batch) unless the logits are given; then one warp chooses.  score s = sigmoid(z);
// choice c = s + correction.  With groups: the experts form
// n_groups equal groups of neighbours, a group's score is the sum of its two largest c, and only
// experts of the `keep` best groups can be chosen (the others count as -inf).  The `top` largest c are
// chosen, the lowest index among equals; their weights are the s (divided by their sum when renorm).
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

constexpr int ROUTE_WARPS = 4, ROUTE_CHUNK = 8;

template <typename TX>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_kernel(const float* __restrict__ z, const TX* __restrict__ x, const float* __restrict__ router,
                 int d, const float* __restrict__ correction, int T, int E,
                 int top, int n_groups, int keep, int renorm, int* __restrict__ ids,
                 float* __restrict__ weights, int* __restrict__ counts, int score) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    float* s = sm;                                         // [E] scores
    float* c = s + E;                                      // [E] choice scores
    float* gs = c + E;                                     // [n_groups] group scores
    if (x) {
        // the logits: the warps share the experts, eight at a time; a lane takes every 32nd term of all eight
        // sums (x is read once for them), then the lanes' parts meet in a butterfly
        const TX* xr = x + (size_t)t * d;
        for (int e0 = warp * ROUTE_CHUNK; e0 < E; e0 += ROUTE_WARPS * ROUTE_CHUNK) {
            float acc[ROUTE_CHUNK];
#pragma unroll
            for (int j = 0; j < ROUTE_CHUNK; ++j) acc[j] = 0.f;
#pragma unroll 4
            for (int i = lane; i < d; i += 32) {
                const float xv = to_f32<TX>(xr[i]);
#pragma unroll
                for (int j = 0; j < ROUTE_CHUNK; ++j)
                    if (e0 + j < E) acc[j] = fmaf(xv, router[(size_t)(e0 + j) * d + i], acc[j]);
            }
#pragma unroll
            for (int j = 0; j < ROUTE_CHUNK; ++j) {
                const float dot = warp_sum(acc[j]);
                if (lane == 0 && e0 + j < E) s[e0 + j] = dot;
            }
        }
        __syncthreads();
    }
    if (warp != 0) return;                                 // the choice is one warp's work
    for (int e = lane; e < E; e += 32) {
        // score 0: the sigmoid of the logit; 1: the logit itself, the chosen ones' weights their softmax
        const float zl = x ? s[e] : z[(size_t)t * E + e];
        const float sc = score == 1 ? zl : 1.0f / (1.0f + expf(-zl));
        s[e] = sc;
        c[e] = sc + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 0 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;            // the two largest
            for (int i = 0; i < per; ++i) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups get +inf as a mark, one by one
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && (v > best || bi == 0x7fffffff)) { best = v; bi = g; }
            }
            warp_argmax(best, bi);
            if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f, zmax = 0.f;
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (!isnan(v) && (v > best || (bi == 0x7fffffff && v > -INFINITY))) { best = v; bi = e; }
        }
        warp_argmax(best, bi);
        if (bi == 0x7fffffff) bi = 0;                      // nothing left to choose (the host rules this out)
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            weights[(size_t)t * top + r] = s[bi];
            atomicAdd(counts + bi, 1);
            c[bi] = NAN;                                   // taken
        }
        if (score == 1) {
            if (r == 0) zmax = s[bi];                      // the first choice has the largest logit
            wsum += expf(s[bi] - zmax);
        } else {
            wsum += s[bi];
        }
        __syncwarp();
    }
    if (score == 1) {
        if (lane < top) weights[(size_t)t * top + lane] = expf(weights[(size_t)t * top + lane] - zmax) / wsum;
    } else if (renorm && lane < top) {
        weights[(size_t)t * top + lane] /= wsum;
    }
}

// --------------------------------------------------------------------------------- sort
// CTA e: offset of expert e = counts of the experts before it; then the pairs that chose e, in their
// order of (token, choice), get the places offset, offset + 1, ...
__global__ void moe_sort_kernel(const int* __restrict__ ids, const int* __restrict__ counts, int N, int E,
                                int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ place) {
    pdl_trigger();
    pdl_wait();
    __shared__ int red[33];
    __shared__ int wtot[32];
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    int part = 0;
    for (int i = tid; i < e; i += blockDim.x) part += counts[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) red[warp] = part;
    __syncthreads();
    if (tid == 0) {
        int tot = 0;
        for (int w = 0; w < warps; ++w) tot += red[w];
        red[32] = tot;
        offsets[e] = tot;
        if (e == E - 1) offsets[E] = tot + counts[e];
    }
    __syncthreads();
    int at = red[32];
    for (int base = 0; base < N; base += blockDim.x) {
        const int i = base + tid;
        const bool mine = i < N && ids[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) wtot[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < warps; ++w) {
            if (w < warp) before += wtot[w];
            total += wtot[w];
        }
        if (mine) {
            const int p = at + before + __popc(ballot & ((1u << lane) - 1u));
            order[p] = i;
            place[i] = p;
        }
        at += total;
        __syncthreads();
    }
}

// ------------------------------------------------------------------------ experts' products
// Rows in expert order: row p of the product belongs to expert e with offsets[e] <= p < offsets[e+1].
// A [.., K]: row of place p is a[order[p] / top] when `gather`, else a[p].  W [E][Ntot][K].
//   GATED: Ntot = 2 N, the matrix's rows alternate gate_n, up_n: out[p][n] = silu(A.W[e][2n]) * (A.W[e][2n + 1])
//   else:  Ntot = N,   out[p][n] = A.W[e][n]
// Every sum runs over k = 0, 1, .. in that order with fp32 multiply-adds, so an output does not depend on
// which rows share its tile.  A CTA of 256 threads owns BM x BN outputs of one expert; the grid's x covers
// ceil(rows / BM) + E tiles (no expert's count is known to the host) and a CTA beyond the last tile returns.
constexpr int GBN = 64, GBK = 32;

// What a gated pair (gate g, up u) becomes.  kind 0: silu(g) * u.  kind 1: with g' = min(g, limit) and
// u' = clamp(u, -limit, limit): g' * sigmoid(alpha * g') * (u' + 1).
struct GluAct {
    int kind;
    float limit, alpha;
};
template <bool FAST>
__device__ __forceinline__ float glu_pair(float g, float u, const GluAct& act) {
    if (act.kind == 1) {
        g = fminf(g, act.limit);
        u = fminf(fmaxf(u, -act.limit), act.limit);
        const float e = FAST ? __expf(-act.alpha * g) : expf(-act.alpha * g);
        return g / (1.0f + e) * (u + 1.0f);
    }
    return g / (1.0f + (FAST ? __expf(-g) : expf(-g))) * u;
}

template <typename TA, typename TW, typename TO, int BM, bool GATED>
__global__ void __launch_bounds__(256)
moe_product_kernel(const TA* __restrict__ a, int a_stride, const TW* __restrict__ w, TO* __restrict__ out,
                   int out_stride, const int* __restrict__ offsets, const int* __restrict__ order, int top,
                   int gather, int E, int N, int K, GluAct act) {
    pdl_trigger();
    pdl_wait();
    constexpr int RM = BM / 16;                            // rows a thread: 16 thread rows
    constexpr int RN = GBN / 16;                           // columns a thread: 16 thread columns
    static_assert(RN == 4, "a thread's four columns are two adjacent pairs");
    __shared__ float As[BM][GBK + 1];
    __shared__ float Ws[GBN][GBK + 1];
    __shared__ int s_tile[3];                              // expert, first row, rows
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, row0 = 0, n_rows = 0;
        for (; e < E; ++e) {
            const int lo = offsets[e], cnt = offsets[e + 1] - lo;
            const int tiles = (cnt + BM - 1) / BM;
            if (tile < tiles) { row0 = lo + tile * BM; n_rows = min(BM, cnt - tile * BM); break; }
            tile -= tiles;
        }
        s_tile[0] = e; s_tile[1] = row0; s_tile[2] = n_rows;
    }
    __syncthreads();
    const int e = s_tile[0], row0 = s_tile[1], n_rows = s_tile[2];
    if (e >= E || n_rows <= 0) return;
    const int n0 = blockIdx.y * GBN;                       // first row of the matrix (of Ntot) this tile covers
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int Ntot = GATED ? 2 * N : N;
    const TW* we = w + (size_t)e * Ntot * K;
    // a thread's columns: the pairs (2 tx, 2 tx + 1) and (32 + 2 tx, 33 + 2 tx): a gate sits beside its up
    float acc[RM][RN];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RN; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GBK) {
        for (int idx = tid; idx < BM * GBK; idx += 256) {
            const int r = idx / GBK, kk = idx - r * GBK;
            float v = 0.f;
            if (r < n_rows && k0 + kk < K) {
                const int p = row0 + r;
                const int src = gather ? order[p] / top : p;
                v = to_f32<TA>(a[(size_t)src * a_stride + k0 + kk]);
            }
            As[r][kk] = v;
        }
        for (int idx = tid; idx < GBN * GBK; idx += 256) {
            const int c = idx / GBK, kk = idx - c * GBK;
            const bool ok = n0 + c < Ntot && k0 + kk < K;
            Ws[c][kk] = ok ? to_f32<TW>(we[(size_t)(n0 + c) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GBK; ++kk) {
            float av[RM];
#pragma unroll
            for (int i = 0; i < RM; ++i) av[i] = As[ty + 16 * i][kk];
#pragma unroll
            for (int j = 0; j < RN; ++j) {
                const float bv = Ws[2 * tx + (j & 1) + 32 * (j >> 1)][kk];
#pragma unroll
                for (int i = 0; i < RM; ++i) acc[i][j] = fmaf(av[i], bv, acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int r = ty + 16 * i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < RN; ++j) {
            const int n = n0 + 2 * tx + (j & 1) + 32 * (j >> 1);
            if (n >= Ntot) continue;
            float v = acc[i][j];
            if (GATED) {
                if (j & 1) continue;                                   // the pair's gate writes
                v = glu_pair<false>(v, acc[i][j + 1], act);
                out[(size_t)(row0 + r) * out_stride + (n >> 1)] = from_f32<TO>(v);
            } else {
                out[(size_t)(row0 + r) * out_stride + n] = from_f32<TO>(v);
            }
        }
    }
}

// The same products for bf16 rows and matrices on the tensor cores (mma.sync m16n8k16, fp32 accumulation):
// a CTA of four warps owns BM rows x 64 columns of one expert, a warp 16 of the columns; rows and matrix
// rows arrive by cp.async in 16-byte pieces through a ring of three stages of 64 k each (the rows gathered
// through `order`), fragments by ldmatrix from rows padded by 16 bytes.  K must be a multiple of 8 and the
// rows 16-byte aligned; other shapes take the kernel above.
constexpr int TBK = 64, TROW = TBK + 8, TSTAGES = 3;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;      // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int BM> constexpr size_t moe_mma_smem() {
    return (size_t)TSTAGES * (BM + GBN) * TROW * sizeof(bf16);
}

template <typename TO, int BM, bool GATED>
__global__ void __launch_bounds__(128)
moe_product_mma_kernel(const bf16* __restrict__ a, int a_stride, const bf16* __restrict__ w, TO* __restrict__ out,
                       int out_stride, const int* __restrict__ offsets, const int* __restrict__ order, int top,
                       int gather, int E, int N, int K, GluAct act) {
    pdl_trigger();
    pdl_wait();
    constexpr int MB = BM / 16;                            // 16-row blocks
    constexpr int STAGE = (BM + GBN) * TROW;               // elements a stage
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sm = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int s_tile[3];
    __shared__ int s_src[BM];                              // row of `a` behind every row of the tile (-1: none)
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, row0 = 0, n_rows = 0;
        for (; e < E; ++e) {
            const int lo = offsets[e], cnt = offsets[e + 1] - lo;
            const int tiles = (cnt + BM - 1) / BM;
            if (tile < tiles) { row0 = lo + tile * BM; n_rows = min(BM, cnt - tile * BM); break; }
            tile -= tiles;
        }
        s_tile[0] = e; s_tile[1] = row0; s_tile[2] = n_rows;
    }
    __syncthreads();
    const int e = s_tile[0], row0 = s_tile[1], n_rows = s_tile[2];
    if (e >= E || n_rows <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int r = tid; r < BM; r += 128) s_src[r] = r < n_rows ? (gather ? order[row0 + r] / top : row0 + r) : -1;
    __syncthreads();
    const int n0 = blockIdx.y * GBN;
    const int Ntot = GATED ? 2 * N : N;
    const bf16* we = w + (size_t)e * Ntot * K;
    const int kblocks = (K + TBK - 1) / TBK;

    auto load_stage = [&](int kb, int stage) {
        bf16* As = sm + (size_t)stage * STAGE;
        bf16* Ws = As + BM * TROW;
        const int k0 = kb * TBK;
        for (int c = tid; c < BM * (TBK / 8); c += 128) {
            const int r = c >> 3, ch = c & 7;
            const int src = s_src[r];
            const bool ok = src >= 0 && k0 + ch * 8 < K;
            cp_async16(As + r * TROW + ch * 8, ok ? a + (size_t)src * a_stride + k0 + ch * 8 : a, ok);
        }
        for (int c = tid; c < GBN * (TBK / 8); c += 128) {
            const int r = c >> 3, ch = c & 7;
            const bool ok = n0 + r < Ntot && k0 + ch * 8 < K;
            cp_async16(Ws + r * TROW + ch * 8, ok ? we + (size_t)(n0 + r) * K + k0 + ch * 8 : we, ok);
        }
    };

    float acc[MB][2][4];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;

#pragma unroll
    for (int st = 0; st < TSTAGES - 1; ++st) {
        if (st < kblocks) load_stage(st, st);
        cp_async_commit();
    }
    for (int kb = 0; kb < kblocks; ++kb) {
        cp_async_wait<TSTAGES - 2>();
        __syncthreads();                                   // stage kb has landed; stage kb-1 is free for all
        if (kb + TSTAGES - 1 < kblocks) load_stage(kb + TSTAGES - 1, (kb + TSTAGES - 1) % TSTAGES);
        cp_async_commit();
        const bf16* As = sm + (size_t)(kb % TSTAGES) * STAGE;
        const bf16* Ws = As + BM * TROW;
#pragma unroll
        for (int ks = 0; ks < TBK / 16; ++ks) {
            unsigned bfr[4];
            ldmatrix_x4(bfr, Ws + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * TROW + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                unsigned af[4];
                ldmatrix_x4(af, As + (m * 16 + (lane & 15)) * TROW + ks * 16 + (lane >> 4) * 8);
                mma_bf16(acc[m][0], af, bfr[0], bfr[1]);
                mma_bf16(acc[m][1], af, bfr[2], bfr[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = m * 16 + (lane >> 2) + 8 * half;
                if (r >= n_rows) continue;
                // a thread holds two neighbouring columns: of a gated matrix, a gate and its up
                const int n = n0 + warp * 16 + j * 8 + (lane & 3) * 2;
                const float v0 = acc[m][j][2 * half], v1 = acc[m][j][2 * half + 1];
                if (GATED) {
                    if (n + 1 < Ntot) out[(size_t)(row0 + r) * out_stride + (n >> 1)] = from_f32<TO>(glu_pair<true>(v0, v1, act));
                } else {
                    if (n < Ntot) out[(size_t)(row0 + r) * out_stride + n] = from_f32<TO>(v0);
                    if (n + 1 < Ntot) out[(size_t)(row0 + r) * out_stride + n + 1] = from_f32<TO>(v1);
                }
            }
}

// --------------------------------------------------------------------- gated pairs, alone
// in fp32 [rows][2 F], a row's columns alternating gate_n, up_n (what a product with a plain epilogue leaves):
// out[p][n] = glu_pair(in[p][2n], in[p][2n + 1]).
template <typename TO>
__global__ void glu_pairs_kernel(const float* __restrict__ in, TO* __restrict__ out, long long total, GluAct act) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const float2 p = reinterpret_cast<const float2*>(in)[i];
        out[i] = from_f32<TO>(glu_pair<false>(p.x, p.y, act));
    }
}

// ------------------------------------------------------------------------------- gather
// out[p][:] = x[order[p] / top][:]: the tokens' rows in expert order, for products that want their rows in one
// piece (16-byte copies; d a multiple of 8).
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ order, int top,
                                  bf16* __restrict__ out, int rows, int d) {
    pdl_trigger();
    pdl_wait();
    const int chunks = d >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * chunks;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / chunks), c = (int)(i - (long long)r * chunks);
        reinterpret_cast<uint4*>(out + (size_t)r * d)[c] = reinterpret_cast<const uint4*>(x + (size_t)(order[r] / top) * d)[c];
    }
}

// ------------------------------------------------------------------------------ combine
// out[t][c] = sum_j weights[t][j] * Y[place[t*top + j]][c] (+ shared[t][c]), j = 0, 1, .. in that order.
template <typename TS, typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ Y, const int* __restrict__ place,
                                   const float* __restrict__ weights, const TS* __restrict__ shared, TO* __restrict__ out,
                                   int top, int d, int* __restrict__ counts, int E) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (t == 0)
        for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;     // ready for the next step
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j)
            acc = fmaf(weights[(size_t)t * top + j], Y[(size_t)place[(size_t)t * top + j] * d + c], acc);
        if (shared) acc += to_f32<TS>(shared[(size_t)t * d + c]);
        out[(size_t)t * d + c] = from_f32<TO>(acc);
    }
}

}  // namespace

// Either z (fp32 [T][E]) or x ([T][d] of x_dtype) with router (fp32 [E][d]) is given.
RI_API int ri_moe_route(const float* z, const void* x, int x_dtype, const float* router, int d, const float* correction,
                        int T, int E, int top, int n_groups, int keep,
                        int renorm, int* ids, float* weights, int* counts, int score, void* stream) {
    if (T <= 0) return 0;
    if (score != 0 && score != 1) return (int)cudaErrorInvalidValue;
    if (E <= 0 || top <= 0 || top > E || top > 32 || (n_groups > 0 && (E % n_groups || keep <= 0 || keep > n_groups)))
        return (int)cudaErrorInvalidValue;
    const int warps = ROUTE_WARPS;
    const size_t smem = (size_t)(2 * E + (n_groups > 0 ? n_groups : 0)) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if ((z == nullptr) == (x == nullptr) || (x && !router)) return (int)cudaErrorInvalidValue;
    const dim3 grid(T);
    if (x && x_dtype == RI_BF16)
        RI_CHECKED(ri_launch(moe_route_kernel<bf16>, grid, dim3(32 * warps), smem, (cudaStream_t)stream, z, (const bf16*)x, router, d,
                             correction, T, E, top, n_groups > 0 ? n_groups : 0, keep, renorm, ids, weights, counts, score));
    else
        RI_CHECKED(ri_launch(moe_route_kernel<float>, grid, dim3(32 * warps), smem, (cudaStream_t)stream, z, (const float*)x, router, d,
                             correction, T, E, top, n_groups > 0 ? n_groups : 0, keep, renorm, ids, weights, counts, score));
    return ri_launch_status();
}

RI_API int ri_moe_sort(const int* ids, const int* counts, int N, int E, int* offsets, int* order, int* place, void* stream) {
    if (N <= 0) return 0;
    RI_CHECKED(ri_launch(moe_sort_kernel, dim3(E), dim3(256), 0, (cudaStream_t)stream, ids, counts, N, E, offsets, order, place));
    return ri_launch_status();
}

RI_API int ri_moe_product_rows(int rows, int E) { return rows / E >= 24 ? 64 : 16; }

// 1 (default): bf16 products on the tensor cores; 0: the fp32 multiply-add kernel for every dtype.
static int& ri_moe_tensor_cores() {
    static int on = 1;
    return on;
}
RI_API void ri_moe_set_tensor_cores(int on) { ri_moe_tensor_cores() = on ? 1 : 0; }

// a_dtype / w_dtype / out_dtype: RI_F32 or RI_BF16.  rows: T * top (the pairs).  gated: see the kernel;
// act_kind, act_limit, act_alpha: what a gated pair becomes (see GluAct).
RI_API int ri_moe_product(const void* a, int a_dtype, int a_stride, const void* w, int w_dtype, void* out, int out_dtype,
                          int out_stride, const int* offsets, const int* order, int top, int gather, int rows, int E,
                          int N, int K, int gated, int act_kind, float act_limit, float act_alpha, void* stream) {
    if (rows <= 0) return 0;
    if (act_kind != 0 && act_kind != 1) return (int)cudaErrorInvalidValue;
    const GluAct act{act_kind, act_limit, act_alpha};
    cudaStream_t s = (cudaStream_t)stream;
    const int bm = ri_moe_product_rows(rows, E);
    const dim3 grid((rows + bm - 1) / bm + E, ((gated ? 2 * N : N) + GBN - 1) / GBN);
#define RI_MP(TA, TW, TO, BM, G) RI_CHECKED(ri_launch(moe_product_kernel<TA, TW, TO, BM, G>, grid, dim3(256), 0, s, (const TA*)a, \
        a_stride, (const TW*)w, (TO*)out, out_stride, offsets, order, top, gather, E, N, K, act))
#define RI_MP_BM(TA, TW, TO, G) do { if (bm == 64) RI_MP(TA, TW, TO, 64, G); else RI_MP(TA, TW, TO, 16, G); } while (0)
    const bool tensor_cores = a_dtype == RI_BF16 && w_dtype == RI_BF16 && K % 8 == 0 && a_stride % 8 == 0 &&
                              ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ri_moe_tensor_cores();
    if (tensor_cores && ((gated && out_dtype == RI_BF16) || (!gated && out_dtype == RI_F32))) {
#define RI_MM(TO, BM, G) do { \
        static bool configured = false; \
        const size_t smem = moe_mma_smem<BM>(); \
        if (!configured) { \
            cudaError_t ce = cudaFuncSetAttribute(moe_product_mma_kernel<TO, BM, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (ce != cudaSuccess) return (int)ce; \
            configured = true; } \
        RI_CHECKED(ri_launch(moe_product_mma_kernel<TO, BM, G>, grid, dim3(128), smem, s, (const bf16*)a, a_stride, (const bf16*)w, \
            (TO*)out, out_stride, offsets, order, top, gather, E, N, K, act)); } while (0)
        if (gated) { if (bm == 64) RI_MM(bf16, 64, true); else RI_MM(bf16, 16, true); }
        else { if (bm == 64) RI_MM(float, 64, false); else RI_MM(float, 16, false); }
#undef RI_MM
        return ri_launch_status();
    }
    if (a_dtype == RI_BF16 && w_dtype == RI_BF16 && out_dtype == RI_BF16 && gated) RI_MP_BM(bf16, bf16, bf16, true);
    else if (a_dtype == RI_BF16 && w_dtype == RI_BF16 && out_dtype == RI_F32 && !gated) RI_MP_BM(bf16, bf16, float, false);
    else if (a_dtype == RI_F32 && w_dtype == RI_F32 && out_dtype == RI_F32 && gated) RI_MP_BM(float, float, float, true);
    else if (a_dtype == RI_F32 && w_dtype == RI_F32 && out_dtype == RI_F32 && !gated) RI_MP_BM(float, float, float, false);
    else return (int)cudaErrorInvalidValue;
#undef RI_MP_BM
#undef RI_MP
    return ri_launch_status();
}

// in fp32 [rows][2 F] (8-byte aligned), out [rows][F] of out_dtype
RI_API int ri_glu_pairs(const float* in, void* out, int out_dtype, long long total, int act_kind, float act_limit,
                        float act_alpha, void* stream) {
    if (total <= 0) return 0;
    if ((act_kind != 0 && act_kind != 1) || ((uintptr_t)in & 7)) return (int)cudaErrorInvalidValue;
    const GluAct act{act_kind, act_limit, act_alpha};
    const long long nb = (total + 255) / 256;
    const int blocks = (int)(nb < 8192 ? nb : 8192);
    if (out_dtype == RI_BF16)
        RI_CHECKED(ri_launch(glu_pairs_kernel<bf16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, in, (bf16*)out, total, act));
    else
        RI_CHECKED(ri_launch(glu_pairs_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, in, (float*)out, total, act));
    return ri_launch_status();
}

RI_API int ri_moe_gather(const void* x, const int* order, int top, void* out, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (d % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
    const long long items = (long long)rows * (d / 8);
    const int blocks = (int)((items + 255) / 256 < 8192 ? (items + 255) / 256 : 8192);
    RI_CHECKED(ri_launch(moe_gather_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, order, top,
                         (bf16*)out, rows, d));
    return ri_launch_status();
}

RI_API int ri_moe_combine(const float* Y, const int* place, const float* weights, const void* shared, int shared_dtype,
                          void* out, int out_dtype, int T, int top, int d, int* counts, int E, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
#define RI_MC(TS, TO) RI_CHECKED(ri_launch(moe_combine_kernel<TS, TO>, dim3(T), dim3(256), 0, s, Y, place, weights, \
        (const TS*)shared, (TO*)out, top, d, counts, E))
    if (shared_dtype == RI_BF16 && out_dtype == RI_BF16) RI_MC(bf16, bf16);
    else if (shared_dtype == RI_BF16) RI_MC(bf16, float);
    else if (out_dtype == RI_BF16) RI_MC(float, bf16);
    else RI_MC(float, float);
#undef RI_MC
    return ri_launch_status();
}
