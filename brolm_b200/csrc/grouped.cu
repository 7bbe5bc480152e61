// Routed and per-head products: a router that picks a few experts per token, the
// grouping of (token, expert) pairs by expert, and one grouped matrix product
//     Y[row, :] = W[g] * A[row, :]      (W[g] stored (N, K), row in group g)
// whose groups are either experts with the rows that chose them (row lists of
// any length, made on the device) or heads with the same rows each (a product
// per head over slices of a packed activation).  Nothing is read back to the
// host, so a step that uses these stays inside a captured CUDA graph.
//
// float operands run on CUDA cores, every output the fma sum over k in
// ascending order; bfloat16 operands run on the tensor cores (mma.sync
// m16n8k16, float accumulation; a pipelined kernel for operands whose rows
// start on 16-byte borders, a plain one for all others).  An output depends on its own row alone, so
// a token gives the same bits whatever else is in the batch.
#include "common.cuh"

namespace {

constexpr int GBM = 64, GBN = 64;

// ---------------------------------------------------------------------------
// Router: z = Wr x in float, the `top` largest z (ties: the lower index), weight
// f(z) with f = logistic function.  A block takes RT tokens (one when there are
// few, so that more SMs take part, with 32 warps so that many experts' rows are in
// flight at once; four when there are many, so that a row of Wr is fetched once for
// four tokens); a warp takes an expert at a time for all of the block's tokens.  A (token, expert) sum is the lanes' strided partial
// sums, added by one fixed tree: it does not depend on what else is in the block.
// ---------------------------------------------------------------------------
// A warp picks for token t from its scores zr [E] in shared memory (which it overwrites): the `top` largest,
// ties to the lower index, best first.
// mode ROUTE_LOGISTIC: the weight of a chosen expert is the logistic function of its score.
// mode ROUTE_SOFTMAX: s = softmax(z) over all experts; the choice goes by s + corr (a learned number per expert
// that takes no part in the weights); the weights are the chosen s over their sum (+ 1e-20).
// The softmax mode's further options (RouteOpts): the experts form `groups` equal groups of neighbours, a group's
// score is the largest s + corr in it, and only experts of the `keep` best groups (ties: the lower group) can be
// chosen; `renorm` 0 leaves the chosen s as they are instead of dividing by their sum; `wscale` multiplies the
// weights at the end.
enum : int { ROUTE_LOGISTIC = 0, ROUTE_SOFTMAX = 1 };

struct RouteOpts {
    int groups, keep, renorm;
    float wscale;
};

__device__ __forceinline__ void pick_top(float* zr, int E, int top, int t, int lane, int32_t* __restrict__ ids,
                                         float* __restrict__ wts, int mode, const float* __restrict__ corr,
                                         RouteOpts ro) {
    if (mode == ROUTE_SOFTMAX) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
        m = warp_max(m);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(zr[e] - m);
            zr[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) zr[e] *= inv;
        __syncwarp();
        if (ro.groups > 1 && ro.keep < ro.groups) {
            // groups - keep times: the group with the smallest score (ties: the higher group) leaves; a group that
            // has left holds -inf in every place, which no score of a group still in is
            const int size = E / ro.groups;
            for (int out = 0; out < ro.groups - ro.keep; ++out) {
                float worst = INFINITY;
                int at = -1;
                for (int g = lane; g < ro.groups; g += 32) {
                    float best = -INFINITY;
                    for (int j = 0; j < size; ++j) {
                        const int e = g * size + j;
                        if (zr[e] > -INFINITY) best = fmaxf(best, zr[e] + (corr ? corr[e] : 0.0f));
                    }
                    if (best > -INFINITY && (best < worst || (best == worst && g > at))) { worst = best; at = g; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ow = __shfl_xor_sync(0xffffffffu, worst, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (oa >= 0 && (at < 0 || ow < worst || (ow == worst && oa > at))) { worst = ow; at = oa; }
                }
                if (at < 0) break;
                for (int j = lane; j < size; j += 32) zr[at * size + j] = -INFINITY;
                __syncwarp();
            }
        }
        float total = 0.0f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float sc = zr[e];                  // a chosen expert's place holds -inf
                const float v = sc + (corr ? corr[e] : 0.0f);
                if (v > best || (v == best && e < at)) { best = v; at = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (at >= E) at = 0;
            if (lane == 0) {
                const float w = zr[at] > -INFINITY ? zr[at] : 0.0f;
                ids[(size_t)t * top + k] = at;
                wts[(size_t)t * top + k] = w;
                total += w;
                zr[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (lane == 0) {
            const float inv_total = (ro.renorm ? 1.0f / (total + 1e-20f) : 1.0f) * ro.wscale;
            for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= inv_total;
        }
        return;
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = zr[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = 0;                       // (every score was -inf or NaN)
        if (lane == 0) {
            ids[(size_t)t * top + k] = at;
            wts[(size_t)t * top + k] = 1.0f / (1.0f + expf(-best));
            zr[at] = -INFINITY;
        }
        __syncwarp();
    }
}

template <typename T, int RT>
__global__ void __launch_bounds__(RT == 1 ? 1024 : 256) route_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ wr,
                                                    int E, int D, int top, int tokens, int vec,
                                                    int32_t* __restrict__ ids, float* __restrict__ wts, int mode,
                                                    const float* __restrict__ corr, RouteOpts ro) {
    extern __shared__ float z[];                       // [RT][E]
    const int t0 = blockIdx.x * RT;
    const int nt = min(RT, tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        const T* w = wr + (size_t)e * D;
        float acc[RT];
#pragma unroll
        for (int r = 0; r < RT; ++r) acc[r] = 0.0f;
        if (vec) {
            // U chunks of the expert's row in flight per lane ahead of the first use
            constexpr int U = RT == 1 ? 8 : 2;
            for (int i0 = lane * 8; i0 < D; i0 += 256 * U) {
                if constexpr (sizeof(T) == 4) {             // float rows: a chunk of eight is two 16-byte loads
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int i = i0 + u * 256;
                        if (i < D) {
                            float wv[8];
                            load8(w + i, wv);
#pragma unroll
                            for (int r = 0; r < RT; ++r)
                                if (r < nt) {
                                    float xv[8];
                                    load8(x + (size_t)(t0 + r) * ldx + i, xv);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) acc[r] = fmaf(xv[j], wv[j], acc[r]);
                                }
                        }
                    }
                } else {
                uint4 wq[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    wq[u] = i0 + u * 256 < D ? *reinterpret_cast<const uint4*>(w + i0 + u * 256) : make_uint4(0u, 0u, 0u, 0u);
                uint4 xq[RT][U];
#pragma unroll
                for (int r = 0; r < RT; ++r)
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        xq[r][u] = (r < nt && i0 + u * 256 < D)
                                       ? *reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * ldx + i0 + u * 256)
                                       : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&wq[u]);
#pragma unroll
                    for (int r = 0; r < RT; ++r) {
                        const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&xq[r][u]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 a = __bfloat1622float2(hx[j]), b = __bfloat1622float2(hw[j]);
                            acc[r] = fmaf(a.x, b.x, acc[r]);
                            acc[r] = fmaf(a.y, b.y, acc[r]);
                        }
                    }
                }
                }
            }
        } else {
            for (int i = lane; i < D; i += 32) {
                const float wv = to_float(w[i]);
#pragma unroll
                for (int r = 0; r < RT; ++r)
                    if (r < nt) acc[r] = fmaf(to_float(x[(size_t)(t0 + r) * ldx + i]), wv, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            const float s = warp_sum(acc[r]);
            if (lane == 0) z[r * E + e] = s;
        }
    }
    __syncthreads();
    for (int r = warp; r < nt; r += nwarps) pick_top(z + r * E, E, top, t0 + r, lane, ids, wts, mode, corr, ro);
}

// The choice alone, for scores that a matrix product left in memory: z [tokens, E] float (ldz between rows).
// A block takes eight tokens, a warp one.
__global__ void __launch_bounds__(256) route_pick_kernel(const float* __restrict__ zs, long ldz, int E, int top, int tokens,
                                                         int32_t* __restrict__ ids, float* __restrict__ wts, int mode,
                                                         const float* __restrict__ corr, RouteOpts ro) {
    extern __shared__ float z[];                       // [8][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + warp;
    if (t >= tokens) return;
    float* zr = z + warp * E;
    for (int e = lane; e < E; e += 32) zr[e] = zs[(size_t)t * ldz + e];
    __syncwarp();
    pick_top(zr, E, top, t, lane, ids, wts, mode, corr, ro);
}

// ---------------------------------------------------------------------------
// Grouping: pairs p = token * top + choice, each with an expert id -> the pairs in
// expert order (perm), the experts' first rows (offsets) and the list of tiles of `tile_rows` rows.
// One block; the order of an expert's pairs among themselves is not fixed, and no
// result depends on it.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) group_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                     int32_t* __restrict__ perm, int32_t* __restrict__ offsets,
                                                     int32_t* __restrict__ tile_group, int32_t* __restrict__ tile_row0,
                                                     int max_tiles, int tile_rows) {
    extern __shared__ int sh[];                        // counts [E], starts [E]
    int* counts = sh;
    int* starts = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            starts[e] = row;
            offsets[e] = row;
            for (int r = 0; r < counts[e] && tile < max_tiles; r += tile_rows) {
                tile_group[tile] = e;
                tile_row0[tile] = row + r;
                ++tile;
            }
            row += counts[e];
        }
        offsets[E] = row;
        for (; tile < max_tiles; ++tile) tile_group[tile] = -1;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) perm[starts[e] + atomicAdd(&counts[e], 1)] = p;
    }
}

// ---------------------------------------------------------------------------
// The grouped product.
// ---------------------------------------------------------------------------
enum : int { MODE_HEADS = 0, MODE_UP = 1, MODE_DOWN = 2 };
enum : int { ACT_NONE = 0, ACT_RELU2 = 1 };

struct GroupedArgs {
    const void* a; long lda, a_goff;          // A rows; group g's slice starts a_goff * g further (heads)
    const void* w; long ldw, w_goff;          // W[g] = w + g * w_goff, rows of ldw
    void* out; long ldo, o_goff;
    int out_f32, act;
    int N, K;
    int mode;
    int rows;                                 // heads: rows of every group
    int tiles_per_group;                      // heads
    const int32_t* tile_group;                // experts: the tile list of group_kernel
    const int32_t* tile_row0;
    const int32_t* offsets;
    const int32_t* perm;
    const float* scale;                       // up: the weight of pair p multiplies its input row
    int top, tokens;
};

struct RowInfo {
    long a_off, o_off;
    float scale;
    int valid;
};

// What row r of tile `bt` is: returns the group, fills `info`.
__device__ __forceinline__ int tile_rows(const GroupedArgs& g, int bt, RowInfo* info) {
    int group, row0, end;
    if (g.mode == MODE_HEADS) {
        group = bt / g.tiles_per_group;
        row0 = (bt - group * g.tiles_per_group) * GBM;
        end = g.rows;
    } else {
        group = g.tile_group[bt];
        if (group < 0) return -1;
        row0 = g.tile_row0[bt];
        end = g.offsets[group + 1];
    }
    for (int r = threadIdx.x; r < GBM; r += blockDim.x) {
        RowInfo ri;
        const int s = row0 + r;
        ri.valid = s < end;
        ri.scale = 1.0f;
        ri.a_off = ri.o_off = 0;
        if (ri.valid) {
            if (g.mode == MODE_HEADS) {
                ri.a_off = (long)s * g.lda + (long)group * g.a_goff;
                ri.o_off = (long)s * g.ldo + (long)group * g.o_goff;
            } else {
                const int p = g.perm[s];
                const int tok = p / g.top, choice = p - tok * g.top;
                if (g.mode == MODE_UP) {
                    ri.a_off = (long)tok * g.lda;
                    ri.scale = g.scale ? g.scale[p] : 1.0f;
                    ri.o_off = (long)s * g.ldo;
                } else {
                    ri.a_off = (long)s * g.lda;
                    ri.o_off = ((long)choice * g.tokens + tok) * g.ldo;
                }
            }
        }
        info[r] = ri;
    }
    return group;
}

__device__ __forceinline__ float act_of(float v, int act) {
    if (act == ACT_RELU2) {
        v = fmaxf(v, 0.0f);
        return v * v;
    }
    return v;
}

// --- float: 16 x 16 threads, 4 x 4 outputs each, BK = 16 --------------------
__global__ void __launch_bounds__(256) grouped_f32_kernel(GroupedArgs g) {
    constexpr int BK = 16;
    __shared__ float As[BK][GBM + 4];
    __shared__ float Bs[BK][GBN + 4];
    __shared__ RowInfo info[GBM];
    const int group = tile_rows(g, blockIdx.y, info);
    if (group < 0) return;
    __syncthreads();
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * GBN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const float* A = (const float*)g.a;
    const float* W = (const float*)g.w + (size_t)group * g.w_goff;
    const RowInfo mine = info[lr];
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < g.K; k0 += BK) {
        float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
        const int k = k0 + lk;
        if (mine.valid) {
            const float* p = A + mine.a_off + k;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (k + i < g.K) a[i] = p[i] * mine.scale;
        }
        if (n0 + lr < g.N) {
            const float* p = W + (size_t)(n0 + lr) * g.ldw + k;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (k + i < g.K) b[i] = p[i];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = a[i];
            Bs[lk + i][lr] = b[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
    float* out = (float*)g.out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const RowInfo ri = info[ty * 4 + i];
        if (!ri.valid) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < g.N) out[ri.o_off + n] = act_of(acc[i][j], g.act);
        }
    }
}

// --- bfloat16: four warps, 32 x 32 outputs each, BK = 32, mma.sync ------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// eight consecutive elements of a row from k on, zeros beyond K; 16-byte load when `vec`
__device__ __forceinline__ uint4 load_chunk(const bf16* p, int k, int K, bool vec) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (vec && k + 8 <= K) return *reinterpret_cast<const uint4*>(p + k);
    bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (k + i < K) e[i] = p[k + i];
    return v;
}

__device__ __forceinline__ uint4 scale_chunk(uint4 v, float s) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        h[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
    }
    return v;
}

__global__ void __launch_bounds__(128) grouped_bf16_kernel(GroupedArgs g, int vec) {
    constexpr int BK = 32, LD = BK + 8;                 // rows of 80 bytes: ldmatrix phases hit all banks once
    __shared__ __align__(16) bf16 As[2][GBM][LD];
    __shared__ __align__(16) bf16 Bs[2][GBN][LD];
    __shared__ RowInfo info[GBM];
    const int group = tile_rows(g, blockIdx.y, info);
    if (group < 0) return;
    __syncthreads();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int n0 = blockIdx.x * GBN;
    const bf16* A = (const bf16*)g.a;
    const bf16* W = (const bf16*)g.w + (size_t)group * g.w_goff;
    // loader: chunks c = tid, tid + 128 of the 256 (row, 8 k) chunks of a tile
    const int r0 = tid >> 2, r1 = r0 + 32, kc = (tid & 3) * 8;
    const RowInfo i0 = info[r0], i1 = info[r1];
    const bool scaled = g.mode == MODE_UP;
    uint4 ra0, ra1, rb0, rb1;
    auto fetch = [&](int k0) {
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        ra0 = i0.valid ? load_chunk(A + i0.a_off, k0 + kc, g.K, vec) : zero;
        ra1 = i1.valid ? load_chunk(A + i1.a_off, k0 + kc, g.K, vec) : zero;
        rb0 = n0 + r0 < g.N ? load_chunk(W + (size_t)(n0 + r0) * g.ldw, k0 + kc, g.K, vec) : zero;
        rb1 = n0 + r1 < g.N ? load_chunk(W + (size_t)(n0 + r1) * g.ldw, k0 + kc, g.K, vec) : zero;
        if (scaled) {
            ra0 = scale_chunk(ra0, i0.scale);
            ra1 = scale_chunk(ra1, i1.scale);
        }
    };
    auto stash = [&](int buf) {
        *reinterpret_cast<uint4*>(&As[buf][r0][kc]) = ra0;
        *reinterpret_cast<uint4*>(&As[buf][r1][kc]) = ra1;
        *reinterpret_cast<uint4*>(&Bs[buf][r0][kc]) = rb0;
        *reinterpret_cast<uint4*>(&Bs[buf][r1][kc]) = rb1;
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f; }

    const int nk = (g.K + BK - 1) / BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kb = 0; kb < nk; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * BK);
#pragma unroll
        for (int ks = 0; ks < BK; ks += 16) {
            uint32_t af[2][4], bfr[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                ldsm_x4(smem_addr(&As[buf][wm + mt * 16 + (lane & 15)][ks + (lane >> 4) * 8]), af[mt][0], af[mt][1],
                        af[mt][2], af[mt][3]);
#pragma unroll
            for (int np = 0; np < 2; ++np)
                ldsm_x4(smem_addr(&Bs[buf][wn + np * 16 + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]),
                        bfr[np][0], bfr[np][1], bfr[np][2], bfr[np][3]);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    mma16816(acc[mt][2 * np], af[mt], bfr[np][0], bfr[np][1]);
                    mma16816(acc[mt][2 * np + 1], af[mt], bfr[np][2], bfr[np][3]);
                }
        }
        if (kb + 1 < nk) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const RowInfo ri = info[wm + mt * 16 + (lane >> 2) + 8 * half];
            if (!ri.valid) continue;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int n = n0 + wn + nt * 8 + (lane & 3) * 2;
                const float v0 = act_of(acc[mt][nt][2 * half], g.act), v1 = act_of(acc[mt][nt][2 * half + 1], g.act);
                if (g.out_f32) {
                    float* o = (float*)g.out + ri.o_off + n;
                    if (n < g.N) o[0] = v0;
                    if (n + 1 < g.N) o[1] = v1;
                } else {
                    bf16* o = (bf16*)g.out + ri.o_off + n;
                    if (n < g.N) o[0] = __float2bfloat16_rn(v0);
                    if (n + 1 < g.N) o[1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

// --- bfloat16, operands whose rows start on 16-byte borders: eight warps, 64 rows x FBN outputs a block, the tiles of A
// and W through a ring of cp.async stages; the gate of a pair is applied to the float sums ahead of the activation:
// act(g * (W x)), which is W (g x) without rounding g x to bfloat16 first.  Two shapes of the ring: four stages of
// 32 k (60 KB, three blocks to an SM) when the groups have many rows and the tensor cores set the pace; six stages of
// 64 k (162 KB, 80 KB of W in flight per block) when a group has a handful of rows (decoding) and the kernel is a
// stream of the matrices: with about one block per SM that is what it takes against the memory's latency.

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// (HEADS only tells the per-head products from the experts' in a profile: the code is the same)
template <int FBN, int BK, int STAGES, bool HEADS>
__global__ void __launch_bounds__(256) grouped_bf16_fast_kernel(GroupedArgs g) {
    constexpr int LD = BK + 8, CPR = BK / 8, WN = FBN / 4, NP = WN / 16;   // a warp: 32 rows x WN outputs
    extern __shared__ __align__(128) unsigned char fsm[];
    __shared__ RowInfo info[GBM];
    const int group = tile_rows(g, blockIdx.y, info);
    if (group < 0) return;
    __syncthreads();
    bf16* As = reinterpret_cast<bf16*>(fsm);                       // [STAGES][GBM][LD]
    bf16* Bs = As + STAGES * GBM * LD;                             // [STAGES][FBN][LD]
    const uint32_t as_base = smem_addr(As), bs_base = smem_addr(Bs);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 2) * 32, wn = (warp & 3) * WN;
    const int n0 = blockIdx.x * FBN;
    const bf16* A = (const bf16*)g.a;
    const bf16* W = (const bf16*)g.w + (size_t)group * g.w_goff;
    auto load_stage = [&](int stage, int kb) {                     // (K is a multiple of 8: a chunk is whole or absent)
#pragma unroll
        for (int i = 0; i < GBM * CPR / 256; ++i) {
            const int c = tid + i * 256, row = c / CPR, kc = (c % CPR) * 8, k = kb * BK + kc;
            const bool ok = info[row].valid && k < g.K;
            cp_async_16(as_base + (uint32_t)((stage * GBM + row) * LD + kc) * 2u, A + (ok ? info[row].a_off + k : 0),
                        ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < FBN * CPR / 256; ++i) {
            const int c = tid + i * 256, row = c / CPR, kc = (c % CPR) * 8, k = kb * BK + kc;
            const bool ok = n0 + row < g.N && k < g.K;
            cp_async_16(bs_base + (uint32_t)((stage * FBN + row) * LD + kc) * 2u,
                        W + (ok ? (size_t)(n0 + row) * g.ldw + k : 0), ok ? 16 : 0);
        }
    };
    float acc[2][2 * NP][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2 * NP; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f; }
    const int nk = (g.K + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    const uint32_t a_frag = as_base + (uint32_t)((wm + (lane & 15)) * LD + (lane >> 4) * 8) * 2u;
    const uint32_t b_frag = bs_base + (uint32_t)((wn + (lane & 7) + ((lane >> 4) << 3)) * LD + ((lane >> 3) & 1) * 8) * 2u;
    for (int kb = 0; kb < nk; ++kb) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                                   // stage kb has landed; everyone is done with stage kb - 1
        if (kb + STAGES - 1 < nk) load_stage((kb + STAGES - 1) % STAGES, kb + STAGES - 1);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const uint32_t sa = a_frag + (uint32_t)(kb % STAGES) * GBM * LD * 2u;
        const uint32_t sb = b_frag + (uint32_t)(kb % STAGES) * FBN * LD * 2u;
#pragma unroll
        for (int ks = 0; ks < BK; ks += 16) {
            uint32_t af[2][4], bfr[NP][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                ldsm_x4(sa + (uint32_t)(mt * 16 * LD + ks) * 2u, af[mt][0], af[mt][1], af[mt][2], af[mt][3]);
#pragma unroll
            for (int np = 0; np < NP; ++np)
                ldsm_x4(sb + (uint32_t)(np * 16 * LD + ks) * 2u, bfr[np][0], bfr[np][1], bfr[np][2], bfr[np][3]);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int np = 0; np < NP; ++np) {
                    mma16816(acc[mt][2 * np], af[mt], bfr[np][0], bfr[np][1]);
                    mma16816(acc[mt][2 * np + 1], af[mt], bfr[np][2], bfr[np][3]);
                }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const RowInfo ri = info[wm + mt * 16 + (lane >> 2) + 8 * half];
            if (!ri.valid) continue;
#pragma unroll
            for (int nt = 0; nt < 2 * NP; ++nt) {
                const int n = n0 + wn + nt * 8 + (lane & 3) * 2;
                const float v0 = act_of(acc[mt][nt][2 * half] * ri.scale, g.act);
                const float v1 = act_of(acc[mt][nt][2 * half + 1] * ri.scale, g.act);
                if (g.out_f32) {
                    float* o = (float*)g.out + ri.o_off + n;
                    if (n < g.N) o[0] = v0;
                    if (n + 1 < g.N) o[1] = v1;
                } else {
                    bf16* o = (bf16*)g.out + ri.o_off + n;
                    if (n < g.N) o[0] = __float2bfloat16_rn(v0);
                    if (n + 1 < g.N) o[1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

template <int FBN, int BK, int STAGES, bool HEADS>
int launch_fast(const GroupedArgs& g, int row_tiles, cudaStream_t stream) {
    constexpr int smem = STAGES * (GBM + FBN) * (BK + 8) * 2;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(grouped_bf16_fast_kernel<FBN, BK, STAGES, HEADS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    dim3 grid((g.N + FBN - 1) / FBN, row_tiles);
    grouped_bf16_fast_kernel<FBN, BK, STAGES, HEADS><<<grid, 256, smem, stream>>>(g);
    return launch_status();
}

// `few`: the groups have a handful of rows each (decoding), so the matrices are streamed rather than tiled
int launch_grouped(int dtype, GroupedArgs& g, int row_tiles, bool few, cudaStream_t stream) {
    if (g.N <= 0 || row_tiles <= 0) return BROLM_OK;
    if (g.K <= 0) return BROLM_ERR_BAD_SIZE;
    if (row_tiles > 65535) return BROLM_ERR_TOO_LARGE;
    dim3 grid((g.N + GBN - 1) / GBN, row_tiles);
    if (dtype == BROLM_F32) {
        if (!g.out_f32) return BROLM_ERR_BAD_DTYPE;
        grouped_f32_kernel<<<grid, 256, 0, stream>>>(g);
    } else if (dtype == BROLM_BF16) {
        const int vec = g.K % 8 == 0 && g.lda % 8 == 0 && g.a_goff % 8 == 0 && g.ldw % 8 == 0 && g.w_goff % 8 == 0 &&
                        ((uintptr_t)g.a & 15) == 0 && ((uintptr_t)g.w & 15) == 0;
        if (vec) {
            if (g.mode == MODE_HEADS)
                return few ? launch_fast<64, 64, 4, true>(g, row_tiles, stream)
                           : launch_fast<128, 32, 4, true>(g, row_tiles, stream);
            return few ? launch_fast<64, 64, 4, false>(g, row_tiles, stream)
                       : launch_fast<128, 32, 4, false>(g, row_tiles, stream);
        } else {
            grouped_bf16_kernel<<<grid, 128, 0, stream>>>(g, 0);
        }
    } else {
        return BROLM_ERR_BAD_DTYPE;
    }
    return launch_status();
}

}  // namespace

// ids [tokens, top] int32 and wts [tokens, top] float: the chosen experts of every token, best first.
// mode 0: the weights are the logistic function of the chosen scores; mode 1: softmax over all experts, the choice
// by softmax + corr (float [experts] or null), the weights the chosen softmax values over their sum.
// groups, keep, renorm, wscale: the softmax mode's options (see RouteOpts); 1, 1, 1, 1.0 are the plain router.
static inline bool route_opts_ok(int experts, int top, int groups, int keep) {
    return groups >= 1 && keep >= 1 && keep <= groups && experts % groups == 0 && top <= keep * (experts / groups);
}

BROLM_API int brolm_route_topk(int dtype, const void* x, long ldx, const void* wr, int tokens, int experts, int width,
                               int top, void* ids, void* wts, int mode, const void* corr, int groups, int keep,
                               int renorm, float wscale, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (experts <= 0 || top <= 0 || top > experts || width <= 0) return BROLM_ERR_BAD_SIZE;
    if (!route_opts_ok(experts, top, groups, keep)) return BROLM_ERR_BAD_SIZE;
    const RouteOpts ro = {groups, keep, renorm, wscale};
    if (experts > 8192) return BROLM_ERR_TOO_LARGE;
    const int vec = width % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)wr & 15) == 0;
    const bool many = tokens > 64 && experts <= 1024;      // (four rows of scores in the default shared memory)
    const int rt = many ? 4 : 1;
    const size_t smem = (size_t)rt * experts * sizeof(float);
    const int blocks = (tokens + rt - 1) / rt;
#define BROLM_ROUTE(T, RT)                                                                                        \
    route_kernel<T, RT><<<blocks, RT == 1 ? 1024 : 256, smem, stream>>>((const T*)x, ldx, (const T*)wr, experts, width, top, tokens, \
                                                       vec, (int32_t*)ids, (float*)wts, mode, (const float*)corr, ro)
    if (dtype == BROLM_F32) {
        if (many) BROLM_ROUTE(float, 4); else BROLM_ROUTE(float, 1);
    } else if (dtype == BROLM_BF16) {
        if (many) BROLM_ROUTE(bf16, 4); else BROLM_ROUTE(bf16, 1);
    } else {
        return BROLM_ERR_BAD_DTYPE;
    }
#undef BROLM_ROUTE
    return launch_status();
}

// The same choice from scores already in memory: z [tokens, experts] float, ldz floats between rows.
BROLM_API int brolm_route_pick(const void* z, long ldz, int tokens, int experts, int top, void* ids, void* wts,
                               int mode, const void* corr, int groups, int keep, int renorm, float wscale,
                               cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (experts <= 0 || top <= 0 || top > experts) return BROLM_ERR_BAD_SIZE;
    if (!route_opts_ok(experts, top, groups, keep)) return BROLM_ERR_BAD_SIZE;
    const RouteOpts ro = {groups, keep, renorm, wscale};
    if (experts > 1024) return BROLM_ERR_TOO_LARGE;          // (eight rows of scores in the default shared memory)
    route_pick_kernel<<<(tokens + 7) / 8, 256, (size_t)8 * experts * sizeof(float), stream>>>(
        (const float*)z, ldz, experts, top, tokens, (int32_t*)ids, (float*)wts, mode, (const float*)corr, ro);
    return launch_status();
}

// The tile list has room for max_tiles = ceil(pairs / tile_rows) + experts entries; tile_rows is 64 for the
// products of this file and 128 for the tcgen05 one.
BROLM_API int brolm_group_pairs(const void* ids, int pairs, int experts, void* perm, void* offsets, void* tile_group,
                                void* tile_row0, int max_tiles, int tile_rows, cudaStream_t stream) {
    if (pairs <= 0) return BROLM_OK;
    if (tile_rows != GBM && tile_rows != 2 * GBM) return BROLM_ERR_BAD_SIZE;
    if (experts <= 0 || experts > 4096) return BROLM_ERR_TOO_LARGE;
    group_kernel<<<1, 1024, 2 * (size_t)experts * sizeof(int), stream>>>((const int32_t*)ids, pairs, experts,
                                                                        (int32_t*)perm, (int32_t*)offsets,
                                                                        (int32_t*)tile_group, (int32_t*)tile_row0,
                                                                        max_tiles, tile_rows);
    return launch_status();
}

// Per-head product: out[r, g * o_goff + n] = sum_k w[g][n][k] * a[r, g * a_goff + k], for `rows` rows and
// `groups` heads.  Output float or the operands' type.
BROLM_API int brolm_heads_linear(int dtype, const void* a, long lda, long a_goff, const void* w, long ldw, long w_goff,
                                 void* out, long ldo, long o_goff, int out_f32, int rows, int groups, int N, int K,
                                 cudaStream_t stream) {
    if (rows <= 0 || groups <= 0) return BROLM_OK;
    GroupedArgs g = {};
    g.a = a; g.lda = lda; g.a_goff = a_goff; g.w = w; g.ldw = ldw; g.w_goff = w_goff;
    g.out = out; g.ldo = ldo; g.o_goff = o_goff; g.out_f32 = out_f32; g.act = ACT_NONE;
    g.N = N; g.K = K; g.mode = MODE_HEADS; g.rows = rows; g.tiles_per_group = (rows + GBM - 1) / GBM;
    const long long tiles = (long long)g.tiles_per_group * groups;
    if (tiles > 65535) return BROLM_ERR_TOO_LARGE;
    return launch_grouped(dtype, g, (int)tiles, rows <= 8, stream);
}

// Experts, first product: u[s, :] = act(W[e] (scale[p] * x[token of p, :])) for the s-th pair p of the expert
// order.  Second product (down != 0): out[choice of p][token of p][:] = W[e] u[s, :], float.
BROLM_API int brolm_experts_linear(int dtype, int down, const void* a, long lda, const void* w, long ldw, long w_goff,
                                   int groups, void* out, long ldo, int out_f32, int act, int N, int K, const void* tile_group,
                                   const void* tile_row0, const void* offsets, const void* perm, const void* scale,
                                   int top, int tokens, int max_tiles, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    GroupedArgs g = {};
    g.a = a; g.lda = lda; g.w = w; g.ldw = ldw; g.w_goff = w_goff; g.out = out; g.ldo = ldo;
    g.out_f32 = out_f32; g.act = act; g.N = N; g.K = K; g.mode = down ? MODE_DOWN : MODE_UP;
    g.tile_group = (const int32_t*)tile_group; g.tile_row0 = (const int32_t*)tile_row0;
    g.offsets = (const int32_t*)offsets; g.perm = (const int32_t*)perm; g.scale = (const float*)scale;
    g.top = top; g.tokens = tokens;
    return launch_grouped(dtype, g, max_tiles, (long)tokens * top <= 8L * groups, stream);
}
