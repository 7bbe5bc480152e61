// Causal grouped-query attention for bfloat16 on the tensor cores (mma.sync m16n8k16, float accumulation) with
// the head-wise options of the exact kernel (attn_simt.cu), for prompts and for decoding over the paged cache:
//
// * query/key rows of hd and value rows of vd elements, each a multiple of 16 up to 256;
// * a distance bias: slope[head] * (p - j) is taken off the scaled score of key j at query position p;
// * a soft cap cap * tanh(score / cap) on the scaled score, a learned bias by distance after it (a table
//   [query heads][dist_len] of which key j adds entry min(p - j, dist_len - 1)), and a sink, a number per query head
//   whose exponential joins the softmax's denominator (prompt kernel and the first decode kernel);
// * a window that keeps a sequence's first keys: key j is visible from p iff j <= p and
//   (p - j < window or j < keep_first); in the paged cache the first `ring_from` places are held for good and
//   the ring lies behind them;
// * every value head (`n_vh` = n_kv): block y = g * n_kv + c applies the weights of the query heads of kv head g
//   to the values of kv head c, and the output row of head h is [n_kv][vd].  This is what a mixing of the heads'
//   weights after the softmax needs: sum_j (sum_g' T[h,g'] w_g'(j)) v_c(j) = sum_g' T[h,g'] (sum_j w_g'(j) v_c(j)),
//   so a row-wise kernel mixes the float results afterwards.  With n_vh = 1 head h uses its own kv head.
//
// Scores, the mask, the softmax statistics and the output accumulator are float; the weights are rounded to
// bfloat16 for the second product.  The output is float (what the mixing reads) or bfloat16.
// Decoding has a second kernel for `n_vh` > 1, up to 8 query heads a kv head and n_kv * vd up to 512: one block per
// (split, kv head of the keys, sequence) keeps the value rows of every kv head beside the keys, computes the scores
// once and runs the second product transposed (see there).
// The tile machinery (64 keys a tile, four warps, cp.async staging, XOR-swizzled rows of whole 128-byte lines)
// is that of attn_mma.cuh.
#include "attn_mma.cuh"

namespace {

struct HmArgs {
    const bf16* q;          // rows of q_stride elements; head h at h * hd
    void* out;              // rows of out_stride elements; head h, value head c at (h * n_vh + c) * vd
    int q_stride, out_stride, out_f32;
    const int32_t* cu_q;    // [B+1]
    const int32_t* kv_len;  // [B] (decoding)
    const bf16* k;          // packed source: kv head g at g * hd of a row of kv_stride
    const bf16* v;          //                kv head c at c * vd of a row of v_stride
    int kv_stride, v_stride;
    const bf16* k_pages;    // [page][n_kv][KT][hd]
    const bf16* v_pages;    // [page][n_kv][KT][vd]
    const int32_t* page_table;
    int pt_stride, ring, ring_from;
    int n_kv, group, hd, vd, n_vh;
    float scale;
    int window, keep_first;
    const float* slopes;    // [n_kv * group] or null
    float cap;              // > 0: cap * tanh(scaled score / cap)
    const float* sink;      // [n_kv * group] or null
    const float* dist_bias; // [n_kv * group][dist_len] or null
    int dist_len;
    int sms;
    int n_splits;
    float* part_o;          // [B][n_q][n_vh][n_splits][vd]
    float* part_ml;         // [B][n_q][n_vh][n_splits][2]  (maximum in log2 units, sum)
};

__device__ unsigned g_headmix_tickets[MAX_TICKETS];     // one per (sequence, block row); zero between launches

// The score of key `dist` places back in log2 units: scale, cap, slope, the table's entry.  `masked` entries may
// carry any distance; the clamp keeps the table's read in range.
__device__ __forceinline__ float hm_score(float s, float scale, float cap, float inv_cap, float slope2, const float* db,
                                          int dist_len, int dist) {
    float v = s * scale;
    if (cap > 0.0f) v = cap * fast_tanh(v * inv_cap);
    v = v * LOG2E - slope2 * (float)dist;
    if (db) v = fmaf(db[min(max(dist, 0), dist_len - 1)], LOG2E, v);
    return v;
}

// ===========================================================================
// prompts that start at position 0
// ===========================================================================
// SCORED: the launch has a cap, a sink or a distance table (a kernel of its own, so that the others carry none of it).
template <int HD_MAX, int VD_MAX, bool SCORED = false>
__global__ void __launch_bounds__(NTHREADS) attn_headmix_prefill_kernel(HmArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hd = a.hd, vd = a.vd, hd16 = hd >> 4, vd16 = vd >> 4, cpr_k = hd >> 3, cpr_v = vd >> 3;
    const bool swz_k = (hd & 63) == 0, swz_v = (vd & 63) == 0;
    const uint32_t rowb_k = (uint32_t)hd * 2u, rowb_v = (uint32_t)vd * 2u;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + BM * hd;
    bf16* Vs = Ks + KT * hd;
    const uint32_t qs_base = smem_u32(Qs), ks_base = smem_u32(Ks), vs_base = smem_u32(Vs);

    // heaviest row tiles first, and the lightest beside them when every block is resident at once
    const int per_x = gridDim.y * gridDim.z, total = gridDim.x * per_x;
    const int n = blockIdx.x * per_x + blockIdx.z * gridDim.y + blockIdx.y;
    const int rank = (total <= 2 * a.sms && n >= a.sms) ? total - 1 - (n - a.sms) : n;
    const int xt = gridDim.x - 1 - rank / per_x;
    const int b = (rank % per_x) / gridDim.y, y = (rank % per_x) % gridDim.y;
    const int g = y / a.n_vh, c = a.n_vh > 1 ? y % a.n_vh : g;       // kv head of the keys, kv head of the values
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int n_rows = q_len * a.group;
    const int row0 = xt * BM;
    if (row0 >= n_rows) return;
    const int rows_here = min(BM, n_rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int keep = a.window > 0 ? a.keep_first : 0;
    const int tok_lo = row0 / a.group, tok_hi = (row0 + rows_here - 1) / a.group;
    const int key_lo = max(0, tok_lo - window + 1), key_hi = tok_hi;
    const int t_first = key_lo / KT, t_last = key_hi / KT;
    // tiles of the kept first keys that lie before the window's first tile
    const int n_kept = min((min(keep, key_lo) + KT - 1) / KT, t_first);
    const int n_tiles = n_kept + t_last - t_first + 1;
    auto tile_of = [&](int i) { return i < n_kept ? i : t_first + (i - n_kept); };

    for (int idx = threadIdx.x; idx < BM * cpr_k; idx += NTHREADS) {
        const int r = idx / cpr_k, cc = idx - r * cpr_k;
        const int row = row0 + r;
        const bool ok = r < rows_here;
        const int tok = ok ? row / a.group : 0, head = g * a.group + (ok ? row % a.group : 0);
        cp_async16(qs_base + tile_off(r, cc, hd, swz_k), a.q + (size_t)(q0 + tok) * a.q_stride + head * hd + cc * 8,
                   ok ? 16 : 0);
    }
    auto load_k = [&](int t) {
        for (int idx = threadIdx.x; idx < KT * cpr_k; idx += NTHREADS) {
            const int r = idx / cpr_k, cc = idx - r * cpr_k;
            const int kp = t * KT + r;
            const bool ok = kp <= key_hi;
            cp_async16(ks_base + tile_off(r, cc, hd, swz_k),
                       a.k + (size_t)(q0 + (ok ? kp : 0)) * a.kv_stride + g * hd + cc * 8, ok ? 16 : 0);
        }
    };
    auto load_v = [&](int t) {
        for (int idx = threadIdx.x; idx < KT * cpr_v; idx += NTHREADS) {
            const int r = idx / cpr_v, cc = idx - r * cpr_v;
            const int kp = t * KT + r;
            const bool ok = kp <= key_hi;
            cp_async16(vs_base + tile_off(r, cc, vd, swz_v),
                       a.v + (size_t)(q0 + (ok ? kp : 0)) * a.v_stride + c * vd + cc * 8, ok ? 16 : 0);
        }
    };
    load_k(tile_of(0));
    cp_async_commit();

    float o[VD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < VD_MAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    int rpos[2];
    float slope2[2];           // slope in log2 units
    const float* db[2];        // the head's row of the distance table
    float db_far[2];           // its last entry, in log2 units: what every key of a tile far enough back adds
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        rpos[i] = r < rows_here ? (row0 + r) / a.group : -1;
        const int head = g * a.group + (r < rows_here ? (row0 + r) % a.group : 0);
        slope2[i] = (a.slopes && r < rows_here) ? a.slopes[head] * LOG2E : 0.0f;
        db[i] = (SCORED && a.dist_bias) ? a.dist_bias + (size_t)head * a.dist_len : nullptr;
        db_far[i] = (SCORED && a.dist_bias) ? db[i][a.dist_len - 1] * LOG2E : 0.0f;
    }
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;
    const float scale2 = a.scale * LOG2E;

    const uint32_t x = lane & 7;
    const uint32_t xhi_k = swz_k ? (x & 6u) << 4 : 0u, xhi_v = swz_v ? (x & 6u) << 4 : 0u;
    const uint32_t jq = lane >> 4, jk = (lane >> 3) & 1, jv = lane >> 4;
    const uint32_t q_addr = qs_base + (warp * 16 + (lane & 15)) * rowb_k + ((swz_k ? (jq ^ (x & 1u)) : jq) << 4);
    const uint32_t k_addr = ks_base + ((lane & 7) + ((lane >> 4) << 3)) * rowb_k + ((swz_k ? (jk ^ (x & 1u)) : jk) << 4);
    const uint32_t v_addr = vs_base + ((lane & 7) + (((lane >> 3) & 1) << 3)) * rowb_v + ((swz_v ? (jv ^ (x & 1u)) : jv) << 4);
    const uint32_t kt_k = 16u * rowb_k, kt_v = 16u * rowb_v;

    for (int i = 0; i < n_tiles; ++i) {
        const int t = tile_of(i);
        load_v(t);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                       // queries and keys of this tile are in shared memory

        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < HD_MAX / 16; ++ks) {
            if (ks < hd16) {
                uint32_t af[4];
                const uint32_t coff = ((uint32_t)ks << 5) ^ xhi_k;
                ldmatrix_x4(q_addr + coff, af[0], af[1], af[2], af[3]);
#pragma unroll
                for (int kt = 0; kt < 4; ++kt) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(k_addr + kt * kt_k + coff, b0, b1, b2, b3);
                    mma_bf16(s[2 * kt], af, b0, b1);
                    mma_bf16(s[2 * kt + 1], af, b2, b3);
                }
            }
        }
        // scale, distance bias, mask
        const int tile_lo = t * KT, tile_hi = tile_lo + KT - 1;
        const bool edge = tile_hi > tok_lo || tile_lo < tok_hi - window + 1;
        const bool far_tile = SCORED && a.dist_bias && tok_lo - tile_hi >= a.dist_len - 1;   // no read of the table in this tile
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kp = tile_lo + nt * 8 + (lane & 3) * 2 + (e & 1);
                const int p = rpos[e >> 1];
                float v;
                if constexpr (SCORED) {
                    v = hm_score(s[nt][e], a.scale, a.cap, inv_cap, slope2[e >> 1], far_tile ? nullptr : db[e >> 1],
                                 a.dist_len, p - kp);
                    if (far_tile) v += db_far[e >> 1];
                } else {
                    v = s[nt][e] * scale2 - slope2[e >> 1] * (float)(p - kp);
                }
                if (edge && !(p >= 0 && kp <= p && (p - kp < window || kp < keep))) v = -INFINITY;
                s[nt][e] = v;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[r], mx);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = fast_exp2(m[r] - base);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float p0 = fast_exp2(s[nt][2 * r] - base), p1 = fast_exp2(s[nt][2 * r + 1] - base);
                s[nt][2 * r] = p0;
                s[nt][2 * r + 1] = p1;
                sum += p0 + p1;
            }
            l[r] = l[r] * corr + sum;
            m[r] = m_new;
#pragma unroll
            for (int d = 0; d < VD_MAX / 8; ++d) {
                o[d][2 * r] *= corr;
                o[d][2 * r + 1] *= corr;
            }
        }
        uint32_t pf[4][4];
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
            pf[kt][0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            pf[kt][1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            pf[kt][2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pf[kt][3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
        }
        cp_async_wait<0>();
        __syncthreads();                       // values are in; every warp is done with the keys
        if (i + 1 < n_tiles) load_k(tile_of(i + 1));
        cp_async_commit();
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
#pragma unroll
            for (int dp = 0; dp < VD_MAX / 16; ++dp) {
                if (dp < vd16) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_addr + kt * kt_v + (((uint32_t)dp << 5) ^ xhi_v), b0, b1, b2, b3);
                    mma_bf16(o[2 * dp], pf[kt], b0, b1);
                    mma_bf16(o[2 * dp + 1], pf[kt], b2, b3);
                }
            }
        }
        __syncthreads();                       // every warp is done with the values
    }
    cp_async_wait<0>();

    const int c_out = a.n_vh > 1 ? c : 0;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = l[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int rr = warp * 16 + (lane >> 2) + 8 * r;
        if (rr >= rows_here) continue;
        const int row = row0 + rr, tok = row / a.group, head = g * a.group + row % a.group;
        if constexpr (SCORED) {
            if (a.sink && m[r] > -INFINITY) sum += fast_exp2(a.sink[head] * LOG2E - m[r]);
        }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        const size_t at = (size_t)(q0 + tok) * a.out_stride + ((size_t)head * a.n_vh + c_out) * vd + (lane & 3) * 2;
#pragma unroll
        for (int d = 0; d < VD_MAX / 8; ++d) {
            if (d * 8 < vd) {
                if (a.out_f32)
                    *reinterpret_cast<float2*>((float*)a.out + at + d * 8) = make_float2(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
                else
                    *reinterpret_cast<__nv_bfloat162*>((bf16*)a.out + at + d * 8) =
                        __floats2bfloat162_rn(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
            }
        }
    }
}

// The end of a decode block.  At `stage0` lie the four warps' partial results as floats: wm[4][16] (maxima in log2
// units), wl[4][16] (sums) and wo[4][group][vd].  They are merged; with one split the result is written, else it
// goes to the scratch of this split and the block that finishes last among the splits of its (sequence, y) merges them.
// An output row of head h holds n_vh runs of vd elements, of which this block fills run c_out.
__device__ __forceinline__ void finish_decode(const HmArgs& a, float* stage0, int vd, int n_vh, int c_out, int b, int y,
                                              int g, int split, int q_row, int nthreads) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_q = a.n_kv * a.group;
    float* wm = stage0;
    float* wl = wm + 4 * 16;
    float* wo = wl + 4 * 16;
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.group * vd; idx += nthreads) {
        const int row = idx / vd, d = idx - row * vd;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, wm[w * 16 + row]);
        float sum = 0.0f, acc = 0.0f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(wm[w * 16 + row] - mx);
                sum += wl[w * 16 + row] * f;
                acc += wo[((size_t)w * a.group + row) * vd + d] * f;
            }
        }
        const int head = g * a.group + row;
        if (a.n_splits == 1) {
            if (a.sink && mx > -INFINITY) sum += fast_exp2(a.sink[head] * LOG2E - mx);
            const float res = sum > 0.0f ? acc / sum : 0.0f;
            const size_t at = (size_t)q_row * a.out_stride + ((size_t)head * n_vh + c_out) * vd + d;
            if (a.out_f32) ((float*)a.out)[at] = res;
            else ((bf16*)a.out)[at] = __float2bfloat16_rn(res);
        } else {
            const size_t slot = (((size_t)b * n_q + head) * n_vh + c_out) * a.n_splits + split;
            a.part_o[slot * vd + d] = acc;
            if (d == 0) {
                a.part_ml[slot * 2] = mx;
                a.part_ml[slot * 2 + 1] = sum;
            }
        }
    }
    if (a.n_splits == 1) return;

    // the block that finishes last among the splits of this (sequence, y) merges them
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ticket = &g_headmix_tickets[(size_t)b * gridDim.y + y];
        const unsigned prev = atomicAdd(ticket, 1u);
        is_last = prev == (unsigned)a.n_splits - 1u;
        if (is_last) *ticket = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float* factor = reinterpret_cast<float*>(stage0);    // [group][n_splits], then the sums [group]
    float* total = factor + a.group * a.n_splits;
    for (int row = warp; row < a.group; row += nthreads / 32) {
        const size_t slot0 = (((size_t)b * n_q + g * a.group + row) * n_vh + c_out) * a.n_splits;
        float2 ml0 = make_float2(-INFINITY, 0.0f), ml1 = ml0;
        if (lane < a.n_splits) ml0 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot0 + lane) * 2));
        if (lane + 32 < a.n_splits) ml1 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot0 + lane + 32) * 2));
        const float mx = warp_max(fmaxf(ml0.x, ml1.x));
        float sum = 0.0f;
        if (lane < a.n_splits) {
            const float f = (mx > -INFINITY && ml0.x > -INFINITY) ? fast_exp2(ml0.x - mx) : 0.0f;
            factor[row * a.n_splits + lane] = f;
            sum += ml0.y * f;
        }
        if (lane + 32 < a.n_splits) {
            const float f = (mx > -INFINITY && ml1.x > -INFINITY) ? fast_exp2(ml1.x - mx) : 0.0f;
            factor[row * a.n_splits + lane + 32] = f;
            sum += ml1.y * f;
        }
        sum = warp_sum(sum);
        if (a.sink && mx > -INFINITY) sum += fast_exp2(a.sink[g * a.group + row] * LOG2E - mx);
        if (lane == 0) total[row] = sum;
    }
    __syncthreads();
    const int q4 = vd >> 2;
    for (int idx = threadIdx.x; idx < a.group * q4; idx += nthreads) {
        const int row = idx / q4, d = (idx - row * q4) * 4;
        const int head = g * a.group + row;
        const size_t slot0 = (((size_t)b * n_q + head) * n_vh + c_out) * a.n_splits;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s0 = 0; s0 < a.n_splits; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s0 + s < a.n_splits) v[s] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (slot0 + s0 + s) * vd + d));
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s0 + s < a.n_splits) {
                    const float f = factor[row * a.n_splits + s0 + s];
                    acc.x += v[s].x * f; acc.y += v[s].y * f; acc.z += v[s].z * f; acc.w += v[s].w * f;
                }
        }
        const float sum = total[row];
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        const size_t at = (size_t)q_row * a.out_stride + ((size_t)head * n_vh + c_out) * vd + d;
        if (a.out_f32) {
            *reinterpret_cast<float4*>((float*)a.out + at) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else {
            bf16* dst = (bf16*)a.out + at;
            dst[0] = __float2bfloat16_rn(acc.x * inv);
            dst[1] = __float2bfloat16_rn(acc.y * inv);
            dst[2] = __float2bfloat16_rn(acc.z * inv);
            dst[3] = __float2bfloat16_rn(acc.w * inv);
        }
    }
}

// ===========================================================================
// decoding over the paged cache: one new token per sequence
// ===========================================================================
// Block (split, y, sequence).  The visible tiles of a sequence are the tiles of its kept first keys that lie
// before the window, then the window's tiles; they are dealt out to the splits in that order.  The four warps
// own 16 of a tile's 64 keys each; their partial results are merged in shared memory, and the block that is
// last among the splits of its (sequence, y) merges the splits from float scratch.
template <int HD_MAX, int VD_MAX>
__global__ void __launch_bounds__(NTHREADS) attn_headmix_decode_kernel(HmArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hd = a.hd, vd = a.vd, hd16 = hd >> 4, vd16 = vd >> 4, cpr_k = hd >> 3, cpr_v = vd >> 3;
    const bool swz_k = (hd & 63) == 0, swz_v = (vd & 63) == 0;
    const uint32_t rowb_k = (uint32_t)hd * 2u, rowb_v = (uint32_t)vd * 2u;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [16][hd]
    bf16* stage0 = Qs + 16 * hd;                             // STAGES x ([KT][hd] keys, [KT][vd] values)
    const uint32_t qs_base = smem_u32(Qs), st_base = smem_u32(stage0);
    const uint32_t stage_bytes = (uint32_t)KT * (rowb_k + rowb_v);

    const int split = blockIdx.x, y = blockIdx.y, b = blockIdx.z;
    const int g = y / a.n_vh, c = a.n_vh > 1 ? y % a.n_vh : g;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int pt_row[PT_ROW];
    for (int i = threadIdx.x; i < min(a.pt_stride, PT_ROW); i += NTHREADS) pt_row[i] = a.page_table[(size_t)b * a.pt_stride + i];
    const int kv_len = a.kv_len[b];
    const int q_row = a.cu_q[b];
    __syncthreads();
    pdl_wait();               // q and the newest key and value come from the kernels before this one
    const int pos = kv_len - 1;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int keep = a.window > 0 ? a.keep_first : 0;
    const int key_lo = max(0, pos - window + 1);
    int n_kept = 0, t_lo = 0, n_all = 0;
    if (kv_len > 0) {
        t_lo = key_lo / KT;
        n_kept = min((min(keep, key_lo) + KT - 1) / KT, t_lo);
        n_all = n_kept + pos / KT - t_lo + 1;
    }
    const int per = (n_all + a.n_splits - 1) / a.n_splits;
    const int i_begin = min(n_all, split * per), i_end = min(n_all, i_begin + per);
    const int n_tiles = i_end - i_begin;
    auto tile_of = [&](int i) { const int j = i_begin + i; return j < n_kept ? j : t_lo + (j - n_kept); };

    for (int idx = threadIdx.x; idx < 16 * cpr_k; idx += NTHREADS) {
        const int r = idx / cpr_k, cc = idx - r * cpr_k;
        const bool ok = r < a.group && kv_len > 0;
        cp_async16(qs_base + tile_off(r, cc, hd, swz_k),
                   a.q + (size_t)q_row * a.q_stride + (g * a.group + (ok ? r : 0)) * hd + cc * 8, ok ? 16 : 0);
    }
    auto page_of = [&](int i) -> int {                        // page that holds the i-th tile of the split
        const int p0 = tile_of(i) * KT;
        const int place = p0 < a.ring_from ? p0 : a.ring_from + (p0 - a.ring_from) % a.ring;
        const int entry = place / KT;
        return entry < PT_ROW ? pt_row[entry] : a.page_table[(size_t)b * a.pt_stride + entry];
    };
    auto load_tile = [&](int i, int page) {
        const int t = tile_of(i);
        const size_t ksrc = ((size_t)page * a.n_kv + g) * KT * hd, vsrc = ((size_t)page * a.n_kv + c) * KT * vd;
        const uint32_t kb = st_base + (i % STAGES) * stage_bytes, vb = kb + KT * rowb_k;
        for (int idx = threadIdx.x; idx < KT * cpr_k; idx += NTHREADS) {
            const int r = idx / cpr_k, cc = idx - r * cpr_k;
            const int kp = t * KT + r;
            const int bytes = (kp <= pos && (kp >= key_lo || kp < keep)) ? 16 : 0;   // other places read as zero
            cp_async16(kb + tile_off(r, cc, hd, swz_k), a.k_pages + ksrc + r * hd + cc * 8, bytes);
        }
        for (int idx = threadIdx.x; idx < KT * cpr_v; idx += NTHREADS) {
            const int r = idx / cpr_v, cc = idx - r * cpr_v;
            const int kp = t * KT + r;
            const int bytes = (kp <= pos && (kp >= key_lo || kp < keep)) ? 16 : 0;
            cp_async16(vb + tile_off(r, cc, vd, swz_v), a.v_pages + vsrc + r * vd + cc * 8, bytes);
        }
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < n_tiles) load_tile(i, page_of(i));
        cp_async_commit();
    }
    int page_next = (STAGES - 1 < n_tiles) ? page_of(STAGES - 1) : 0;

    const uint32_t x = lane & 7;
    const uint32_t xhi_k = swz_k ? (x & 6u) << 4 : 0u, xhi_v = swz_v ? (x & 6u) << 4 : 0u;
    const uint32_t jq = lane >> 4, jk = (lane >> 3) & 1, jv = lane >> 4;
    const uint32_t q_addr = qs_base + (lane & 15) * rowb_k + ((swz_k ? (jq ^ (x & 1u)) : jq) << 4);
    const uint32_t k_thr = (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * rowb_k + ((swz_k ? (jk ^ (x & 1u)) : jk) << 4);
    const uint32_t v_thr = KT * rowb_k + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * rowb_v +
                           ((swz_v ? (jv ^ (x & 1u)) : jv) << 4);

    float o[VD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < VD_MAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float slope2[2], db_far[2];
    const float* db[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        const int head = g * a.group + (row < a.group ? row : 0);
        slope2[r] = (a.slopes && row < a.group) ? a.slopes[head] * LOG2E : 0.0f;
        db[r] = a.dist_bias ? a.dist_bias + (size_t)head * a.dist_len : nullptr;
        db_far[r] = a.dist_bias ? db[r][a.dist_len - 1] * LOG2E : 0.0f;
    }
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;

    for (int i = 0; i < n_tiles; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                       // tile i has landed; everyone is done with tile i - 1
        if (i + STAGES - 1 < n_tiles) load_tile(i + STAGES - 1, page_next);
        cp_async_commit();
        if (i + STAGES < n_tiles) page_next = page_of(i + STAGES);
        const uint32_t sb = st_base + (i % STAGES) * stage_bytes;
        const int t = tile_of(i);

        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < HD_MAX / 16; ++ks) {
            if (ks < hd16) {
                uint32_t af[4], b0, b1, b2, b3;
                const uint32_t coff = ((uint32_t)ks << 5) ^ xhi_k;
                ldmatrix_x4(q_addr + coff, af[0], af[1], af[2], af[3]);
                ldmatrix_x4(sb + k_thr + coff, b0, b1, b2, b3);
                mma_bf16(s[0], af, b0, b1);
                mma_bf16(s[1], af, b2, b3);
            }
        }
        const int kbase = t * KT + warp * 16 + (lane & 3) * 2;
        const bool far_tile = a.dist_bias && pos - (t * KT + KT - 1) >= a.dist_len - 1;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kp = kbase + nt * 8 + (e & 1);
                float v = hm_score(s[nt][e], a.scale, a.cap, inv_cap, slope2[e >> 1], far_tile ? nullptr : db[e >> 1],
                                   a.dist_len, pos - kp);
                if (far_tile) v += db_far[e >> 1];
                s[nt][e] = (kp <= pos && (kp >= key_lo || kp < keep)) ? v : -INFINITY;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[r], mx);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = fast_exp2(m[r] - base);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float p0 = fast_exp2(s[nt][2 * r] - base), p1 = fast_exp2(s[nt][2 * r + 1] - base);
                s[nt][2 * r] = p0;
                s[nt][2 * r + 1] = p1;
                sum += p0 + p1;
            }
            l[r] = l[r] * corr + sum;
            m[r] = m_new;
#pragma unroll
            for (int d = 0; d < VD_MAX / 8; ++d) {
                o[d][2 * r] *= corr;
                o[d][2 * r + 1] *= corr;
            }
        }
        uint32_t pf[4];
        pf[0] = pack_bf16(s[0][0], s[0][1]);
        pf[1] = pack_bf16(s[0][2], s[0][3]);
        pf[2] = pack_bf16(s[1][0], s[1][1]);
        pf[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < VD_MAX / 16; ++dp) {
            if (dp < vd16) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(sb + v_thr + (((uint32_t)dp << 5) ^ xhi_v), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], pf, b0, b1);
                mma_bf16(o[2 * dp + 1], pf, b2, b3);
            }
        }
    }
    cp_async_wait<0>();
    pdl_trigger();
    __syncthreads();                           // the stages are free: they now hold the warps' partial results

    // merge the four warps: wm[4][16], wl[4][16], wo[4][group][vd] (float)
    float* wm = reinterpret_cast<float*>(stage0);
    float* wl = wm + 4 * 16;
    float* wo = wl + 4 * 16;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = l[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) {
            wm[warp * 16 + row] = m[r];
            wl[warp * 16 + row] = sum;
        }
        if (row < a.group) {
            float* dst = wo + ((size_t)warp * a.group + row) * vd + (lane & 3) * 2;
#pragma unroll
            for (int d = 0; d < VD_MAX / 8; ++d) {
                if (d * 8 < vd) {
                    dst[d * 8] = o[d][2 * r];
                    dst[d * 8 + 1] = o[d][2 * r + 1];
                }
            }
        }
    }
    finish_decode(a, reinterpret_cast<float*>(stage0), vd, a.n_vh, a.n_vh > 1 ? c : 0, b, y, g, split, q_row, NTHREADS);
}

// ===========================================================================
// decoding, every value head in one block
// ===========================================================================
// Block (split, kv head g, sequence): the scores of the group's heads (at most 8) are computed once a tile and
// meet the value rows of all n_kv kv heads, which lie in the stage beside the keys.  The second product runs
// transposed, O^T[dv x heads] = V^T[dv x keys] P^T[keys x heads]: the accumulator of the first product (row =
// head, columns = keys) is, element for element, the B fragment of P^T, so the weights never leave their
// registers, and an accumulator tile of 16 value elements x 8 heads costs four registers where the untransposed
// form pays for 16 rows of which a decode step fills `group`.  NT_MAX: tiles of 16 value elements over all value
// heads (n_kv * vd / 16).  A warp owns 16 of a tile's 64 keys, a thread one head's running maximum and sum.
constexpr int STAGES_ALL = 2;
constexpr int NT_LIMIT = 32;
constexpr int NTHREADS_ALL = 256;     // warps 0 to 3 take the first half of the value tiles, warps 4 to 7 the second

template <int HD_MAX, int NT_MAX>
__global__ void __launch_bounds__(NTHREADS_ALL) attn_headmix_decode_all_kernel(HmArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hd = a.hd, vd = a.vd, hd16 = hd >> 4, vd16 = vd >> 4, cpr_k = hd >> 3, cpr_v = vd >> 3;
    const int nt = a.n_kv * vd16;
    const bool swz_k = (hd & 63) == 0, swz_v = (vd & 63) == 0;
    const uint32_t rowb_k = (uint32_t)hd * 2u, rowb_v = (uint32_t)vd * 2u;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [16][hd]
    bf16* stage0 = Qs + 16 * hd;                             // STAGES_ALL x ([KT][hd] keys, [n_kv][KT][vd] values)
    const uint32_t qs_base = smem_u32(Qs), st_base = smem_u32(stage0);
    const uint32_t stage_bytes = (uint32_t)KT * (rowb_k + (uint32_t)a.n_kv * rowb_v);

    const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & 3, half = threadIdx.x >> 7;
    __shared__ int pt_row[PT_ROW];
    __shared__ uint32_t v_off[NT_LIMIT];                     // where tile idx of the values begins in a stage's values
    for (int i = threadIdx.x; i < min(a.pt_stride, PT_ROW); i += NTHREADS_ALL) pt_row[i] = a.page_table[(size_t)b * a.pt_stride + i];
    if (threadIdx.x < nt) v_off[threadIdx.x] = (uint32_t)(threadIdx.x / vd16) * KT * rowb_v + ((uint32_t)(threadIdx.x % vd16) << 5);
    const int kv_len = a.kv_len[b];
    const int q_row = a.cu_q[b];
    __syncthreads();
    pdl_wait();
    const int pos = kv_len - 1;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int keep = a.window > 0 ? a.keep_first : 0;
    const int key_lo = max(0, pos - window + 1);
    int n_kept = 0, t_lo = 0, n_all = 0;
    if (kv_len > 0) {
        t_lo = key_lo / KT;
        n_kept = min((min(keep, key_lo) + KT - 1) / KT, t_lo);
        n_all = n_kept + pos / KT - t_lo + 1;
    }
    const int per = (n_all + a.n_splits - 1) / a.n_splits;
    const int i_begin = min(n_all, split * per), i_end = min(n_all, i_begin + per);
    const int n_tiles = i_end - i_begin;
    auto tile_of = [&](int i) { const int j = i_begin + i; return j < n_kept ? j : t_lo + (j - n_kept); };

    for (int idx = threadIdx.x; idx < 16 * cpr_k; idx += NTHREADS_ALL) {
        const int r = idx / cpr_k, cc = idx - r * cpr_k;
        const bool ok = r < a.group && kv_len > 0;
        cp_async16(qs_base + tile_off(r, cc, hd, swz_k),
                   a.q + (size_t)q_row * a.q_stride + (g * a.group + (ok ? r : 0)) * hd + cc * 8, ok ? 16 : 0);
    }
    auto page_of = [&](int i) -> int {
        const int p0 = tile_of(i) * KT;
        const int place = p0 < a.ring_from ? p0 : a.ring_from + (p0 - a.ring_from) % a.ring;
        const int entry = place / KT;
        return entry < PT_ROW ? pt_row[entry] : a.page_table[(size_t)b * a.pt_stride + entry];
    };
    // a thread's part of a tile's copies: when the chunks of a row divide the block, its chunk of a row is fixed
    // and it walks down the rows (no division per copy)
    const bool even_k = NTHREADS_ALL % cpr_k == 0, even_v = NTHREADS_ALL % cpr_v == 0;
    const int k_r0 = threadIdx.x / cpr_k, k_cc = threadIdx.x % cpr_k, k_step = NTHREADS_ALL / cpr_k;
    const int v_r0 = threadIdx.x / cpr_v, v_cc = threadIdx.x % cpr_v, v_step = NTHREADS_ALL / cpr_v;
    auto load_tile = [&](int i, int page) {
        const int t = tile_of(i);
        const bf16* ksrc = a.k_pages + ((size_t)page * a.n_kv + g) * KT * hd;
        const bf16* vsrc = a.v_pages + (size_t)page * a.n_kv * KT * vd;      // [n_kv][KT][vd]: all kv heads' rows in a run
        const uint32_t kb = st_base + (i % STAGES_ALL) * stage_bytes, vb = kb + KT * rowb_k;
        auto seen = [&](int r) { const int kp = t * KT + r; return (kp <= pos && (kp >= key_lo || kp < keep)) ? 16 : 0; };
        if (even_k) {
            for (int r = k_r0; r < KT; r += k_step)
                cp_async16(kb + tile_off(r, k_cc, hd, swz_k), ksrc + r * hd + k_cc * 8, seen(r));    // other places read as zero
        } else {
            for (int idx = threadIdx.x; idx < KT * cpr_k; idx += NTHREADS_ALL) {
                const int r = idx / cpr_k, cc = idx - r * cpr_k;
                cp_async16(kb + tile_off(r, cc, hd, swz_k), ksrc + r * hd + cc * 8, seen(r));
            }
        }
        if (even_v) {
            for (int rr = v_r0; rr < a.n_kv * KT; rr += v_step) {
                const int c = rr / KT, r = rr - c * KT;
                cp_async16(vb + (uint32_t)c * KT * rowb_v + tile_off(r, v_cc, vd, swz_v), vsrc + (size_t)rr * vd + v_cc * 8, seen(r));
            }
        } else {
            for (int idx = threadIdx.x; idx < a.n_kv * KT * cpr_v; idx += NTHREADS_ALL) {
                const int rr = idx / cpr_v, cc = idx - rr * cpr_v;
                const int c = rr / KT, r = rr - c * KT;
                cp_async16(vb + (uint32_t)c * KT * rowb_v + tile_off(r, cc, vd, swz_v), vsrc + (size_t)rr * vd + cc * 8, seen(r));
            }
        }
    };
    if (n_tiles > 0) load_tile(0, page_of(0));
    cp_async_commit();
    int page_next = n_tiles > 1 ? page_of(1) : 0;

    const uint32_t x = lane & 7;
    const uint32_t xhi_k = swz_k ? (x & 6u) << 4 : 0u, xhi_v = swz_v ? (x & 6u) << 4 : 0u;
    const uint32_t jq = lane >> 4, jk = (lane >> 3) & 1;
    const uint32_t q_addr = qs_base + (lane & 15) * rowb_k + ((swz_k ? (jq ^ (x & 1u)) : jq) << 4);
    const uint32_t k_thr = (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * rowb_k + ((swz_k ? (jk ^ (x & 1u)) : jk) << 4);
    // V^T as the A operand: matrices (dims 0-7, keys 0-7), (dims 8-15, keys 0-7), (dims 0-7, keys 8-15), (dims 8-15, keys 8-15)
    const uint32_t v_thr = KT * rowb_k + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * rowb_v + ((swz_v ? (jk ^ (x & 1u)) : jk) << 4);

    constexpr int NT_HALF = NT_MAX / 2;
    const int idx0 = half * NT_HALF;                         // this warp's first value tile
    float o[NT_HALF][4];
#pragma unroll
    for (int i = 0; i < NT_HALF; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m = -INFINITY, l = 0.0f;
    const int hh = lane >> 2;                                 // the head whose statistics this thread keeps
    const float slope2 = (a.slopes && hh < a.group) ? a.slopes[g * a.group + hh] * LOG2E : 0.0f;
    const float scale2 = a.scale * LOG2E;
    const int src0 = ((lane & 3) * 2) * 4, src1 = src0 + 4;   // lanes that keep the heads of this thread's two columns

    for (int i = 0; i < n_tiles; ++i) {
        cp_async_wait<0>();
        __syncthreads();                       // tile i has landed; everyone is done with tile i - 1
        if (i + 1 < n_tiles) load_tile(i + 1, page_next);
        cp_async_commit();
        if (i + 2 < n_tiles) page_next = page_of(i + 2);
        const uint32_t sb = st_base + (i % STAGES_ALL) * stage_bytes;
        const int t = tile_of(i);

        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < HD_MAX / 16; ++ks) {
            if (ks < hd16) {
                uint32_t af[4], b0, b1, b2, b3;
                const uint32_t coff = ((uint32_t)ks << 5) ^ xhi_k;
                ldmatrix_x4(q_addr + coff, af[0], af[1], af[2], af[3]);
                ldmatrix_x4(sb + k_thr + coff, b0, b1, b2, b3);
                mma_bf16(s[0], af, b0, b1);
                mma_bf16(s[1], af, b2, b3);
            }
        }
        // rows 0 to 7 are the heads: s[.][0] and s[.][1] of head hh at keys kbase + 8 nt + {0, 1}
        const int kbase = t * KT + warp * 16 + (lane & 3) * 2;
        float w[2][2];
        float mx = -INFINITY;
#pragma unroll
        for (int n8 = 0; n8 < 2; ++n8) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kp = kbase + n8 * 8 + e;
                const float v = s[n8][e] * scale2 - slope2 * (float)(pos - kp);
                w[n8][e] = (kp <= pos && (kp >= key_lo || kp < keep)) ? v : -INFINITY;
                mx = fmaxf(mx, w[n8][e]);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);
        const float base = m_new == -INFINITY ? 0.0f : m_new;
        const float corr = fast_exp2(m - base);
        float sum = 0.0f;
#pragma unroll
        for (int n8 = 0; n8 < 2; ++n8) {
            w[n8][0] = fast_exp2(w[n8][0] - base);
            w[n8][1] = fast_exp2(w[n8][1] - base);
            sum += w[n8][0] + w[n8][1];
        }
        l = l * corr + sum;
        m = m_new;
        const uint32_t pb0 = pack_bf16(w[0][0], w[0][1]), pb1 = pack_bf16(w[1][0], w[1][1]);
        const float c0 = __shfl_sync(0xffffffffu, corr, src0), c1 = __shfl_sync(0xffffffffu, corr, src1);
#pragma unroll
        for (int j = 0; j < NT_HALF; ++j) {
            if (idx0 + j < nt) {
                o[j][0] *= c0; o[j][1] *= c1; o[j][2] *= c0; o[j][3] *= c1;
                uint32_t af[4];
                ldmatrix_x4_trans(sb + v_thr + (v_off[idx0 + j] ^ xhi_v), af[0], af[1], af[2], af[3]);
                mma_bf16(o[j], af, pb0, pb1);
            }
        }
    }
    cp_async_wait<0>();
    pdl_trigger();
    __syncthreads();                           // the stages are free: they now hold the warps' partial results

    const int vda = a.n_kv * vd;               // a head's output row: the value heads one after another
    float* wm = reinterpret_cast<float*>(stage0);
    float* wl = wm + 4 * 16;
    float* wo = wl + 4 * 16;                   // [4][group][vda]
    {
        float sum = l;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0 && half == 0) {
            wm[warp * 16 + hh] = m;
            wl[warp * 16 + hh] = sum;
        }
    }
    // o[idx]: elements idx * 16 + lane / 4 (+ 8) of the row, heads 2 (lane % 4) and 2 (lane % 4) + 1
    const int h0 = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < NT_HALF; ++j) {
        if (idx0 + j < nt) {
            const int e = (idx0 + j) * 16 + (lane >> 2);
            if (h0 < a.group) {
                float* dst = wo + ((size_t)warp * a.group + h0) * vda + e;
                dst[0] = o[j][0];
                dst[8] = o[j][2];
            }
            if (h0 + 1 < a.group) {
                float* dst = wo + ((size_t)warp * a.group + h0 + 1) * vda + e;
                dst[0] = o[j][1];
                dst[8] = o[j][3];
            }
        }
    }
    finish_decode(a, reinterpret_cast<float*>(stage0), vda, 1, 0, b, g, g, split, q_row, NTHREADS_ALL);
}

template <int HD_MAX, int VD_MAX, bool SCORED = false>
int launch_hm_prefill(const HmArgs& a, int batch, int max_q_len, cudaStream_t stream) {
    if constexpr (!SCORED) {
        if (a.cap > 0.0f || a.sink || a.dist_bias) return launch_hm_prefill<HD_MAX, VD_MAX, true>(a, batch, max_q_len, stream);
    }
    const size_t smem = ((size_t)(BM + KT) * a.hd + (size_t)KT * a.vd) * sizeof(bf16);
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(attn_headmix_prefill_kernel<HD_MAX, VD_MAX, SCORED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid((max_q_len * a.group + BM - 1) / BM, a.n_kv * a.n_vh, batch);
    attn_headmix_prefill_kernel<HD_MAX, VD_MAX, SCORED><<<grid, NTHREADS, smem, stream>>>(a);
    return launch_status();
}

template <int HD_MAX, int VD_MAX>
int launch_hm_decode(const HmArgs& a, int batch, cudaStream_t stream) {
    size_t smem = ((size_t)16 * a.hd + (size_t)STAGES * KT * (a.hd + a.vd)) * sizeof(bf16);
    const size_t merge = (size_t)(8 * 16 + 4 * a.group * a.vd) * sizeof(float) + 16 * a.hd * sizeof(bf16);
    if (merge > smem) smem = merge;
    const size_t last = (size_t)(a.group * a.n_splits + a.group) * sizeof(float) + 16 * a.hd * sizeof(bf16);
    if (last > smem) smem = last;
    if (smem > 227 * 1024) return BROLM_ERR_TOO_LARGE;
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(attn_headmix_decode_kernel<HD_MAX, VD_MAX>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid(a.n_splits, a.n_kv * a.n_vh, batch);
    return launch_pdl(attn_headmix_decode_kernel<HD_MAX, VD_MAX>, grid, dim3(NTHREADS), smem, stream, a);
}

// Whether the kernel that keeps every value head in one block takes these sizes, and its shared memory.
size_t decode_all_smem(int hd, int vd, int n_kv, int group, int n_splits) {
    if (group > 8 || n_kv * (vd / 16) > NT_LIMIT) return 0;
    size_t smem = ((size_t)16 * hd + (size_t)STAGES_ALL * KT * (hd + (size_t)n_kv * vd)) * sizeof(bf16);
    const size_t merge = (size_t)(8 * 16 + 4 * group * n_kv * vd) * sizeof(float) + 16 * hd * sizeof(bf16);
    if (merge > smem) smem = merge;
    const size_t last = (size_t)(group * n_splits + group) * sizeof(float) + 16 * hd * sizeof(bf16);
    if (last > smem) smem = last;
    return smem <= 227 * 1024 - 4096 ? smem : 0;
}

template <int HD_MAX, int NT_MAX>
int launch_hm_decode_all(const HmArgs& a, int batch, size_t smem, cudaStream_t stream) {
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(attn_headmix_decode_all_kernel<HD_MAX, NT_MAX>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid(a.n_splits, a.n_kv, batch);
    return launch_pdl(attn_headmix_decode_all_kernel<HD_MAX, NT_MAX>, grid, dim3(NTHREADS_ALL), smem, stream, a);
}

// The instantiated sizes: query/key rows up to 128 or 256, value rows up to 64, 128 or 256.
template <typename F128_64, typename F128_128, typename F128_256, typename F256_64, typename F256_128, typename F256_256>
int by_size(int hd, int vd, F128_64 a, F128_128 b, F128_256 c, F256_64 d, F256_128 e, F256_256 f) {
    if (hd <= 128) return vd <= 64 ? a() : vd <= 128 ? b() : c();
    return vd <= 64 ? d() : vd <= 128 ? e() : f();
}

int check_hm(int hd, int vd, int group, int n_kv, int q_stride, int out_stride, int batch, int all_values) {
    if (hd <= 0 || hd % 16 != 0 || vd <= 0 || vd % 16 != 0 || group <= 0 || n_kv <= 0) return BROLM_ERR_BAD_SIZE;
    if (hd > 256 || vd > 256) return BROLM_ERR_TOO_LARGE;
    if (q_stride % 8 != 0 || out_stride % 4 != 0) return BROLM_ERR_ALIGNMENT;
    if (batch > 65535 || (long long)n_kv * (all_values ? n_kv : 1) > 65535) return BROLM_ERR_TOO_LARGE;
    return BROLM_OK;
}

}  // namespace

// Prompts that start at position 0.  `out` is float (out_f32) or bfloat16, rows of out_stride elements;
// with all_values its row holds [head][n_kv][vd], else [head][vd].
BROLM_API int brolm_attn_headmix_prefill(const void* q, int q_stride, void* out, int out_stride, int out_f32,
                                         const void* cu_q, const void* k, int kv_stride, const void* v, int v_stride,
                                         int n_kv, int group, int hd, int vd, float scale, int window, int keep_first,
                                         const void* slopes, int all_values, int batch, int max_q_len, float cap,
                                         const void* sink, const void* dist_bias, int dist_len, cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    int st = check_hm(hd, vd, group, n_kv, q_stride, out_stride, batch, all_values);
    if (st) return st;
    if (kv_stride % 8 != 0 || v_stride % 8 != 0 || keep_first < 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)out & 15)) return BROLM_ERR_ALIGNMENT;
    HmArgs a = {};
    a.q = (const bf16*)q; a.out = out; a.q_stride = q_stride; a.out_stride = out_stride; a.out_f32 = out_f32 ? 1 : 0;
    a.cu_q = (const int32_t*)cu_q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.kv_stride = kv_stride; a.v_stride = v_stride;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.vd = vd; a.n_vh = all_values ? n_kv : 1;
    a.scale = scale; a.window = window; a.keep_first = keep_first; a.slopes = (const float*)slopes;
    if ((cap > 0.0f || sink || dist_bias) && all_values) return BROLM_ERR_BAD_SIZE;
    if (dist_bias && dist_len <= 0) return BROLM_ERR_BAD_SIZE;
    a.cap = cap; a.sink = (const float*)sink; a.dist_bias = (const float*)dist_bias; a.dist_len = dist_len;
    a.sms = device_sm_count(); a.n_splits = 1;
    return by_size(hd, vd,
                   [&] { return launch_hm_prefill<128, 64>(a, batch, max_q_len, stream); },
                   [&] { return launch_hm_prefill<128, 128>(a, batch, max_q_len, stream); },
                   [&] { return launch_hm_prefill<128, 256>(a, batch, max_q_len, stream); },
                   [&] { return launch_hm_prefill<256, 64>(a, batch, max_q_len, stream); },
                   [&] { return launch_hm_prefill<256, 128>(a, batch, max_q_len, stream); },
                   [&] { return launch_hm_prefill<256, 256>(a, batch, max_q_len, stream); });
}

// One query token per sequence (row cu_q[b] of q) over the paged cache; pages of 64 keys, group <= 16.
// ring_from: places held for good ahead of the ring (a multiple of the page size, at least keep_first).
// With n_splits > 1 (at most 64), part_o holds batch * heads * (all_values ? n_kv : 1) * n_splits * vd floats
// and part_ml that many pairs.
BROLM_API int brolm_attn_headmix_decode(const void* q, int q_stride, void* out, int out_stride, int out_f32,
                                        const void* cu_q, const void* kv_len, const void* k_pages, const void* v_pages,
                                        const void* page_table, int pt_stride, int ring, int ring_from, int page_size,
                                        int n_kv, int group, int hd, int vd, float scale, int window, int keep_first,
                                        const void* slopes, int all_values, int batch, int n_splits, void* part_o,
                                        void* part_ml, float cap, const void* sink, const void* dist_bias, int dist_len,
                                        cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    int st = check_hm(hd, vd, group, n_kv, q_stride, out_stride, batch, all_values);
    if (st) return st;
    if (group > 16) return BROLM_ERR_TOO_LARGE;
    if (page_size != KT || ring <= 0 || ring % KT != 0 || ring_from < 0 || ring_from % KT != 0) return BROLM_ERR_BAD_SIZE;
    if (keep_first < 0 || (window > 0 && ring_from < keep_first)) return BROLM_ERR_BAD_SIZE;
    if (n_splits < 1 || n_splits > MAX_MERGED_SPLITS) return BROLM_ERR_BAD_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml)) return BROLM_ERR_BAD_SIZE;
    if (n_splits > 1 && (long long)batch * n_kv * (all_values ? n_kv : 1) > MAX_TICKETS) return BROLM_ERR_TOO_LARGE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15)) return BROLM_ERR_ALIGNMENT;
    HmArgs a = {};
    a.q = (const bf16*)q; a.out = out; a.q_stride = q_stride; a.out_stride = out_stride; a.out_f32 = out_f32 ? 1 : 0;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len;
    a.k_pages = (const bf16*)k_pages; a.v_pages = (const bf16*)v_pages; a.page_table = (const int32_t*)page_table;
    a.pt_stride = pt_stride; a.ring = ring; a.ring_from = ring_from;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.vd = vd; a.n_vh = all_values ? n_kv : 1;
    a.scale = scale; a.window = window; a.keep_first = keep_first; a.slopes = (const float*)slopes;
    if ((cap > 0.0f || sink || dist_bias) && all_values) return BROLM_ERR_BAD_SIZE;
    if (dist_bias && dist_len <= 0) return BROLM_ERR_BAD_SIZE;
    a.cap = cap; a.sink = (const float*)sink; a.dist_bias = (const float*)dist_bias; a.dist_len = dist_len;
    a.sms = device_sm_count(); a.n_splits = n_splits; a.part_o = (float*)part_o; a.part_ml = (float*)part_ml;
    if (all_values && n_kv > 1) {
        if (const size_t smem = decode_all_smem(hd, vd, n_kv, group, n_splits)) {
            const int nt = n_kv * (vd / 16);
            if (hd <= 128) return nt <= 16 ? launch_hm_decode_all<128, 16>(a, batch, smem, stream)
                                           : launch_hm_decode_all<128, 32>(a, batch, smem, stream);
            return nt <= 16 ? launch_hm_decode_all<256, 16>(a, batch, smem, stream)
                            : launch_hm_decode_all<256, 32>(a, batch, smem, stream);
        }
    }
    return by_size(hd, vd,
                   [&] { return launch_hm_decode<128, 64>(a, batch, stream); },
                   [&] { return launch_hm_decode<128, 128>(a, batch, stream); },
                   [&] { return launch_hm_decode<128, 256>(a, batch, stream); },
                   [&] { return launch_hm_decode<256, 64>(a, batch, stream); },
                   [&] { return launch_hm_decode<256, 128>(a, batch, stream); },
                   [&] { return launch_hm_decode<256, 256>(a, batch, stream); });
}

// 1 when a decode step with these sizes keeps every value head in one block (its grid then has n_kv block rows a
// sequence instead of n_kv * n_kv), else 0.
BROLM_API int brolm_attn_headmix_decode_shares_keys(int hd, int vd, int n_kv, int group, int all_values, int n_splits) {
    return all_values && n_kv > 1 && hd % 16 == 0 && vd % 16 == 0 && decode_all_smem(hd, vd, n_kv, group, n_splits) ? 1 : 0;
}
