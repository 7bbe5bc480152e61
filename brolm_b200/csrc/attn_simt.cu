// Soft-capped, windowed, causal grouped-query attention on CUDA cores, for
// float and bfloat16 elements, with every product, score and sum in float.
//
// This is the exact path: the float model uses it for prompts and for
// decoding, and it is the reference the tensor-core kernels are checked
// against.  One block handles one (sequence, kv head) and a tile of 32
// "rows"; a row is a (query token, query head of the group) pair, so all
// query heads that share a kv head reuse the same staged keys and values.
//
// Keys come either from the packed projection output of this step
// (prompts: sequence b owns rows cu_q[b] .. cu_q[b+1]) or from the paged
// cache (decoding).  The key loop walks tiles of 32 keys anchored at
// multiples of 32 of the absolute position, and folds them in ascending
// order with one online-softmax update per tile.  The order of operations for
// one query therefore does not depend on how the tokens were cut into steps
// or on what else is in the batch: a prompt pass and a decode pass give the
// same bits for the same inputs.
//
// Scores follow wlejon/brolm src/gemma2.cpp:360-367: s = (q.k) * scale, then
// cap * tanh(s / cap), then the mask, then softmax.  Key j is visible from a
// query at position p iff 0 <= p - j < window (window <= 0: no window).
// With a sink, a learned number per query head, the softmax's denominator also
// holds exp(sink): a key that is always visible, is not scaled and has no value.
// With a chunk size C (chunk > 0) a key must also lie in the query's own chunk: j >= p - p % C, chunks
// counted from position 0 of the sequence.  Value rows may have a size of their own (vd), apart from
// the size of query and key rows (hd).
// Further options, each off by default.  A distance bias: slope[head] * (p - j) is taken off the scaled
// score.  Kept first keys: with a window, key j < keep_first stays visible however far back it lies; in the
// paged cache the first `ring_from` places are then held for good and the ring begins behind them (place of
// position p: p below ring_from, else ring_from + (p - ring_from) % ring).  Values of all kv heads
// (`v_all` > 0): a query head's weights are applied to the value rows of `v_all` kv heads from `v_from` on
// at once; the output row of a head is [n_kv][vd] and a call fills its kv heads' part of it (a caller
// whose n_kv * vd is beyond the kernel's row limit calls several times); what a mixing of the heads'
// weights after the softmax needs.  A float
// output whatever the element type of q, k and v (`out_f32`).  A learned bias by distance: a table
// [query heads][dist_len] of floats, of which key j adds entry min(p - j, dist_len - 1) of the head's row to its
// score after the scale and the cap (the caller lays the table out by distance, whatever rule maps a distance
// to a learned number).
#include "common.cuh"

namespace {

constexpr int ROWS = 32;         // rows per block
constexpr int KT = 32;           // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int RPW = ROWS / WARPS;  // rows per warp

struct AttnArgs {
    const void* q;            // [tokens, q_stride] elements; head h at h*hd
    void* out;                // [tokens, out_stride]
    int q_stride, out_stride;
    const int32_t* cu_q;      // [B+1] first packed row of each sequence
    const int32_t* kv_len;    // [B] keys of each sequence after this step
    // packed source
    const void* k;            // [tokens, kv_stride]; kv head g at g*hd
    const void* v;
    int kv_stride;            // of k
    int v_stride;             // of v
    // paged source
    const void* k_pages;      // [page][n_kv][page_size][hd]
    const void* v_pages;
    const int32_t* page_table;
    int pt_stride, ring, page_size;
    int n_kv, group, hd;
    int vd;                   // size of a value row (and of an output row)
    float scale, cap;
    int window;
    int chunk;                // > 0: keys before the start of the query's chunk are not visible
    int vec;                  // rows are read eight elements at a time (sizes and strides allow it); else one by one
    const float* sink;        // [n_kv * group] or null: exp(sink[head]) joins the softmax's denominator, with no value
    const float* slopes;      // [n_kv * group] or null: slopes[head] * (position - key) is taken off the score
    int keep_first;           // with a window: keys below this position stay visible
    int ring_from;            // paged: places held for good ahead of the ring
    int v_all;                // > 0: values of this many kv heads from v_from on; vd is then v_all * vd_head
    int v_from;
    int vd_head;              // a kv head's value size
    int out_f32;              // the output is float whatever T is
    const float* dist_bias;   // [n_kv * group][dist_len] or null: added to the capped score by min(p - j, dist_len - 1)
    int dist_len;
};

// Place of position p in a sequence's pages: the first `from` places are held for good, the ring lies behind them.
__device__ __forceinline__ int ring_place(int p, int from, int ring) { return p < from ? p : from + (p - from) % ring; }

// DPL: output dims per lane = ceil(vd / 32) rounded up to the instantiated size.
template <typename T, int DPL, bool PAGED>
__global__ void __launch_bounds__(WARPS * 32) attn_simt_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int hd = a.hd, vd = a.vd;
    const int hd4 = (hd + 3) & ~3;         // rows of q and k are padded with zeros to a multiple of four
    const int qs = hd4 + 4;                // padded stride of q and k rows (floats)
    float* Qs = smem;                      // [ROWS][qs]
    float* Ks = Qs + ROWS * qs;            // [KT][qs]
    float* Vs = Ks + KT * qs;              // [KT][vd]

    const int b = blockIdx.z, g = blockIdx.y;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int kv_len = a.kv_len[b];
    const int n_rows = q_len * a.group;
    const int row0 = blockIdx.x * ROWS;
    if (row0 >= n_rows || kv_len <= 0) return;
    const int rows_here = min(ROWS, n_rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int first_pos = kv_len - q_len;            // position of the sequence's first query
    const int window = a.window > 0 ? a.window : 0x3fffffff;

    // stage the queries of this tile as floats
    const T* qg = (const T*)a.q;
    if (!a.vec) {
        for (int idx = threadIdx.x; idx < ROWS * hd4; idx += blockDim.x) {
            const int r = idx / hd4, c = idx - r * hd4;
            float v = 0.0f;
            if (r < rows_here && c < hd) {
                const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
                v = to_float(qg[(size_t)(q0 + tok) * a.q_stride + head * hd + c]);
            }
            Qs[r * qs + c] = v;
        }
    }
    for (int idx = threadIdx.x; a.vec && idx < ROWS * (hd / 8); idx += blockDim.x) {
        const int r = idx / (hd / 8), c = (idx - r * (hd / 8)) * 8;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (r < rows_here) {
            const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
            load8(qg + (size_t)(q0 + tok) * a.q_stride + head * hd + c, v);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) Qs[r * qs + c + i] = v[i];
    }

    // key range of the whole tile
    const int tok_lo = row0 / a.group, tok_hi = (row0 + rows_here - 1) / a.group;
    const int pos_lo = first_pos + tok_lo, pos_hi = first_pos + tok_hi;
    int key_lo = max(0, pos_lo - window + 1);
    if (a.chunk > 0) key_lo = max(key_lo, pos_lo - pos_lo % a.chunk);
    const int key_hi = pos_hi;   // inclusive
    // keys below `kept` are read as well, whatever the window says (each row's own mask decides)
    const int kept = (a.keep_first > 0 && a.chunk <= 0) ? min(a.keep_first, key_lo) : 0;
    const int vdh = a.v_all ? a.vd_head : vd;          // row size of the value store
    const int out_head = a.v_all ? a.n_kv * vdh : vd;  // a head's row in the output, and where this call's part begins
    const int out_from = a.v_all ? a.v_from * vdh : 0;

    // per-row state of this warp
    int rpos[RPW];
    float m[RPW], l[RPW], acc[RPW][DPL], slope[RPW];
    const float* dbias[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        rpos[i] = r < rows_here ? first_pos + (row0 + r) / a.group : -1;
        dbias[i] = (a.dist_bias && r < rows_here) ? a.dist_bias + (size_t)(g * a.group + (row0 + r) % a.group) * a.dist_len : nullptr;
        slope[i] = (a.slopes && r < rows_here) ? a.slopes[g * a.group + (row0 + r) % a.group] : 0.0f;
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[i][d] = 0.0f;
    }

    for (int t0 = kept > 0 ? 0 : (key_lo / KT) * KT; t0 <= key_hi; t0 += KT) {
        if (t0 >= kept && t0 + KT <= key_lo) {        // between the kept first keys and the window: nothing to read
            t0 = (key_lo / KT) * KT - KT;
            continue;
        }
        __syncthreads();   // the tile before this one is consumed (and Qs is written, first time)
        // stage keys and values t0 .. t0+KT-1; places outside [key_lo, key_hi] read as zero
        if (!a.vec) {
            for (int idx = threadIdx.x; idx < KT * hd4; idx += blockDim.x) {
                const int j = idx / hd4, c = idx - j * hd4;
                const int kp = t0 + j;
                float v = 0.0f;
                if ((kp >= key_lo || kp < kept) && kp <= key_hi && c < hd) {
                    if (PAGED) {
                        const int ridx = ring_place(kp, a.ring_from, a.ring);
                        const int page = a.page_table[(size_t)b * a.pt_stride + ridx / a.page_size];
                        v = to_float(((const T*)a.k_pages)[(((size_t)page * a.n_kv + g) * a.page_size + ridx % a.page_size) * hd + c]);
                    } else {
                        v = to_float(((const T*)a.k)[(size_t)(q0 + kp) * a.kv_stride + g * hd + c]);
                    }
                }
                Ks[j * qs + c] = v;
            }
            for (int idx = threadIdx.x; idx < KT * vd; idx += blockDim.x) {
                const int j = idx / vd, c = idx - j * vd;
                const int kp = t0 + j;
                float v = 0.0f;
                if ((kp >= key_lo || kp < kept) && kp <= key_hi) {
                    const int vg = a.v_all ? a.v_from + c / vdh : g, vc = a.v_all ? c % vdh : c;
                    if (PAGED) {
                        const int ridx = ring_place(kp, a.ring_from, a.ring);
                        const int page = a.page_table[(size_t)b * a.pt_stride + ridx / a.page_size];
                        v = to_float(((const T*)a.v_pages)[(((size_t)page * a.n_kv + vg) * a.page_size + ridx % a.page_size) * vdh + vc]);
                    } else {
                        v = to_float(((const T*)a.v)[(size_t)(q0 + kp) * a.v_stride + vg * vdh + vc]);
                    }
                }
                Vs[j * vd + c] = v;
            }
        }
        for (int idx = threadIdx.x; a.vec && idx < KT * (hd / 8); idx += blockDim.x) {
            const int j = idx / (hd / 8), c = (idx - j * (hd / 8)) * 8;
            const int kp = t0 + j;
            float kv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if ((kp >= key_lo || kp < kept) && kp <= key_hi) {
                if (PAGED) {
                    const int ridx = ring_place(kp, a.ring_from, a.ring);
                    const int page = a.page_table[(size_t)b * a.pt_stride + ridx / a.page_size];
                    const size_t off = (((size_t)page * a.n_kv + g) * a.page_size + ridx % a.page_size) * hd + c;
                    load8((const T*)a.k_pages + off, kv);
                } else {
                    load8((const T*)a.k + (size_t)(q0 + kp) * a.kv_stride + g * hd + c, kv);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) Ks[j * qs + c + i] = kv[i];
        }
        for (int idx = threadIdx.x; a.vec && idx < KT * (vd / 8); idx += blockDim.x) {
            const int j = idx / (vd / 8), c = (idx - j * (vd / 8)) * 8;
            const int kp = t0 + j;
            float vv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if ((kp >= key_lo || kp < kept) && kp <= key_hi) {
                const int vg = a.v_all ? a.v_from + c / vdh : g, vc = a.v_all ? c % vdh : c;
                if (PAGED) {
                    const int ridx = ring_place(kp, a.ring_from, a.ring);
                    const int page = a.page_table[(size_t)b * a.pt_stride + ridx / a.page_size];
                    const size_t off = (((size_t)page * a.n_kv + vg) * a.page_size + ridx % a.page_size) * vdh + vc;
                    load8((const T*)a.v_pages + off, vv);
                } else {
                    load8((const T*)a.v + (size_t)(q0 + kp) * a.v_stride + vg * vdh + vc, vv);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) Vs[j * vd + c + i] = vv[i];
        }
        __syncthreads();

        // scores: lane j holds key t0 + j
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.0f;
        const float* kr = Ks + lane * qs;
        for (int c = 0; c < hd4; c += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(kr + c);
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(Qs + (warp * RPW + i) * qs + c);
                s[i] = fmaf(qq.x, kk.x, s[i]);
                s[i] = fmaf(qq.y, kk.y, s[i]);
                s[i] = fmaf(qq.z, kk.z, s[i]);
                s[i] = fmaf(qq.w, kk.w, s[i]);
            }
        }
        const int kp = t0 + lane;
        float p[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const bool visible = rpos[i] >= 0 && kp <= rpos[i] && (rpos[i] - kp < window || kp < a.keep_first) &&
                                 (a.chunk <= 0 || kp >= rpos[i] - rpos[i] % a.chunk);
            float sc = visible ? soft_cap(s[i] * a.scale, a.cap) : -INFINITY;
            if (visible && a.slopes) sc -= slope[i] * (float)(rpos[i] - kp);
            if (visible && dbias[i]) sc += dbias[i][min(rpos[i] - kp, a.dist_len - 1)];
            const float tile_max = warp_max(sc);
            const float m_new = fmaxf(m[i], tile_max);
            float corr = 1.0f;
            p[i] = 0.0f;
            if (m_new > -INFINITY) {
                corr = expf(m[i] - m_new);           // m[i] = -inf gives 0
                p[i] = visible ? expf(sc - m_new) : 0.0f;
            }
            l[i] = l[i] * corr + warp_sum(p[i]);
            m[i] = m_new;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[i][d] *= corr;
        }
        // acc[row][d] += sum_j p[row][j] * V[j][d], keys in ascending order
        for (int j = 0; j < KT; ++j) {
            float vj[DPL];
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                const int dim = lane + 32 * d;
                vj[d] = dim < vd ? Vs[j * vd + dim] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const float pj = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[i][d] = fmaf(pj, vj[d], acc[i][d]);
            }
        }
    }

    T* og = (T*)a.out;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        if (r >= rows_here) continue;
        const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
        float den = l[i];
        if (a.sink && m[i] > -INFINITY) den += expf(a.sink[head] - m[i]);
        const float inv = den > 0.0f ? 1.0f / den : 0.0f;
        if (a.out_f32) {
            float* dst = (float*)a.out + (size_t)(q0 + tok) * a.out_stride + (size_t)head * out_head + out_from;
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                const int dim = lane + 32 * d;
                if (dim < vd) dst[dim] = acc[i][d] * inv;
            }
            continue;
        }
        T* dst = og + (size_t)(q0 + tok) * a.out_stride + (size_t)head * out_head + out_from;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
            const int dim = lane + 32 * d;
            if (dim < vd) dst[dim] = from_float<T>(acc[i][d] * inv);
        }
    }
}

template <typename T, int DPL>
int launch(const AttnArgs& a, bool paged, int batch, int max_q_len, cudaStream_t stream) {
    const size_t smem = (size_t)((ROWS + KT) * (((a.hd + 3) & ~3) + 4) + KT * a.vd) * sizeof(float);
    if (smem > 227 * 1024) return BROLM_ERR_TOO_LARGE;
    dim3 grid((max_q_len * a.group + ROWS - 1) / ROWS, a.n_kv, batch);
    static size_t allowed[2] = {0, 0};        // raised once per size, not at every launch
    if (smem > allowed[paged]) {
        cudaError_t e = paged ? cudaFuncSetAttribute(attn_simt_kernel<T, DPL, true>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                              : cudaFuncSetAttribute(attn_simt_kernel<T, DPL, false>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed[paged] = smem;
    }
    if (paged)
        attn_simt_kernel<T, DPL, true><<<grid, WARPS * 32, smem, stream>>>(a);
    else
        attn_simt_kernel<T, DPL, false><<<grid, WARPS * 32, smem, stream>>>(a);
    return launch_status();
}

template <typename T>
int dispatch(const AttnArgs& a, bool paged, int batch, int max_q_len, cudaStream_t stream) {
    const int dpl = (a.vd + 31) / 32;
    if (dpl <= 1) return launch<T, 1>(a, paged, batch, max_q_len, stream);
    if (dpl <= 2) return launch<T, 2>(a, paged, batch, max_q_len, stream);
    if (dpl <= 4) return launch<T, 4>(a, paged, batch, max_q_len, stream);
    if (dpl <= 8) return launch<T, 8>(a, paged, batch, max_q_len, stream);
    if (dpl <= 16) return launch<T, 16>(a, paged, batch, max_q_len, stream);
    return BROLM_ERR_TOO_LARGE;
}

}  // namespace

// head_dim and the value size are at most 512.  Rows are read eight elements at a time when both are
// multiples of 8 and every stride is a multiple of 8 (8 elements then lie in one aligned 16-byte (bf16) or
// 32-byte (float) span); other sizes and strides are read one element at a time.
BROLM_API int brolm_attn_simt(int dtype, const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                              const void* kv_len, const void* k, const void* v, int kv_stride, const void* k_pages,
                              const void* v_pages, const void* page_table, int pt_stride, int ring, int page_size,
                              int n_kv, int group, int hd, float scale, float cap, int window, const void* sink,
                              int batch, int max_q_len, int vd, int v_stride, int chunk, const void* slopes,
                              int keep_first, int ring_from, int v_all, int v_from, int out_f32, const void* dist_bias,
                              int dist_len, cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    if (hd <= 0 || hd > 512 || group <= 0 || n_kv <= 0) return BROLM_ERR_BAD_SIZE;
    const int vd_head = vd;
    if (v_all < 0 || v_from < 0 || v_from + v_all > n_kv) return BROLM_ERR_BAD_SIZE;
    if (v_all) vd = vd * v_all;                        // a head's output row holds the values of several kv heads
    if (vd <= 0 || vd > 512) return BROLM_ERR_BAD_SIZE;
    if (keep_first < 0 || ring_from < 0 || (keep_first > 0 && chunk > 0)) return BROLM_ERR_BAD_SIZE;
    if (dist_bias && dist_len <= 0) return BROLM_ERR_BAD_SIZE;
    bool vec = hd % 8 == 0 && vd_head % 8 == 0 && q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0;
    if (batch > 65535 || n_kv > 65535) return BROLM_ERR_TOO_LARGE;
    const bool paged = k_pages != nullptr;
    if (paged) {
        if (ring <= 0 || page_size <= 0 || page_size % KT != 0 || ring % page_size != 0) return BROLM_ERR_BAD_SIZE;
        if (ring_from % page_size != 0 || ring_from < keep_first) return BROLM_ERR_BAD_SIZE;
    } else {
        if (!k || !v) return BROLM_ERR_ALIGNMENT;
        vec = vec && kv_stride % 8 == 0 && v_stride % 8 == 0 && ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0;
    }
    AttnArgs a;
    a.q = q; a.out = out; a.q_stride = q_stride; a.out_stride = out_stride;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len;
    a.k = k; a.v = v; a.kv_stride = kv_stride; a.v_stride = v_stride; a.vd = vd; a.chunk = chunk; a.vec = vec ? 1 : 0;
    a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = (const int32_t*)page_table;
    a.pt_stride = pt_stride; a.ring = ring; a.page_size = page_size;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window; a.sink = (const float*)sink;
    a.slopes = (const float*)slopes; a.keep_first = window > 0 ? keep_first : 0; a.ring_from = ring_from; a.v_all = v_all; a.v_from = v_from;
    a.vd_head = vd_head; a.out_f32 = out_f32 ? 1 : 0;
    a.dist_bias = (const float*)dist_bias; a.dist_len = dist_len;
    if (dtype == BROLM_F32) return dispatch<float>(a, paged, batch, max_q_len, stream);
    if (dtype == BROLM_BF16) return dispatch<bf16>(a, paged, batch, max_q_len, stream);
    return BROLM_ERR_BAD_DTYPE;
}
