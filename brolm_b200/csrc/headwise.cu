// Row-wise steps of an attention mixer between its products, one head at a time.
//
// qkv_finish: what lies between the q/k/v projection and the attention itself, in one pass over a token's row
//   [ q: n_q * hd | k: n_kv * hd | v: n_kv * vd ]:
//     * the projection may arrive as float partial sums of K slices, which are added in order, and a bias
//       (one number per column) is added to the sum;
//     * unit norm per head: every q and k head is divided by sqrt(mean(head^2) + eps); with `q_gain` / `k_gain`
//       (hd floats each, one row for all heads) the normed head is multiplied by it element by element;
//     * rotation of the first `rot` elements of every q and k head by pos * f_i, the angles' cos and sin from a
//       table [position][rot / 2][2]; the pair of f_i is (i, i + rot/2) ("half", pairing 0) or (2i, 2i + 1)
//       ("interleaved", pairing 1); the rest of the head passes unchanged;
//     * value mixing across layers: v <- (1 - lambda) v + lambda v_first, lambda a float on the device and v_first
//       float rows (tokens, n_kv * vd) that an earlier layer of the same step left (`v_keep` asks this layer to leave
//       its own values, as they are before any mixing, for the later ones);
//     * the result in the step's element type, rounded once, into the packed row and into the cache pages
//       (k rows of hd, value rows of vd; cache_rows[t] = page * page_size + place, negative: not kept).
//   A negative position marks a padding row, which is left untouched.
//
// heads_mix: what lies between an attention whose heads' weights are mixed after the softmax and the output product.
//   The attention left, for every query head g, its weights applied to the value rows of every kv head:
//   acc (tokens, H, n_kv, vd) float.  Head h's mixed weights are sum_g talk[h][g] * weights_g, and it applies them to
//   the values of its own kv head c(h) = h / (H / n_kv), so
//       out[t, h, :] = gate(t, h) * sum_g talk[h][g] * acc[t, g, c(h), :],   gate = sigmoid(gate_logit[t, h]) or 1.
//   Without a talk matrix acc is (tokens, H, vd), every head's own result, and only the gate is applied.
//
// Everything is float arithmetic; one block per token.
#include "common.cuh"

namespace {

struct FinishArgs {
    const void* proj;          // [parts][tokens][ldp]
    int n_parts;
    long long part_stride;
    long ldp;
    const float* bias;         // [cols] or null
    int n_q, n_kv, hd, vd;
    int head_norm;
    float eps;
    const float* q_gain;       // [hd] or null: a gain for every query head after its unit norm
    const float* k_gain;       // [hd] or null: the same for the key heads
    const int32_t* positions;
    const float* cos_sin;      // [positions][rot / 2][2] or null
    int rot, pairing;
    const float* lambda;       // device scalar or null
    const float* v_first;      // [tokens][ld_first] or null
    long ld_first;
    float* v_keep;             // [tokens][n_kv * vd] or null
    void* out;                 // [tokens][ldo]
    long ldo;
    void* k_pages;
    void* v_pages;
    const int32_t* cache_rows;
    int page_size;
};

__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename X, typename O>
__global__ void __launch_bounds__(256) qkv_finish_kernel(FinishArgs a) {
    extern __shared__ __align__(16) float row[];      // the token's q | k | v as floats
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int q_cols = a.n_q * a.hd, k_cols = a.n_kv * a.hd, v_cols = a.n_kv * a.vd;
    const int cols = q_cols + k_cols + v_cols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    pdl_wait();
    if (pos < 0) return;                               // a padding row
    const X* pr = (const X*)a.proj + (size_t)t * a.ldp;
    bool by_four = false;
    if constexpr (sizeof(X) == 4) {
        // float rows whose parts, bias and row all begin at multiples of 16 bytes: four numbers a load
        by_four = (cols & 3) == 0 && (a.ldp & 3) == 0 && (a.part_stride & 3) == 0 && ((uintptr_t)a.proj & 15) == 0 &&
                  ((uintptr_t)a.bias & 15) == 0;
        if (by_four) {
            const float* pf = reinterpret_cast<const float*>(pr);
            for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
                float4 v = *reinterpret_cast<const float4*>(pf + i);
                for (int p = 1; p < a.n_parts; ++p) {
                    const float4 u = *reinterpret_cast<const float4*>(pf + (size_t)p * a.part_stride + i);
                    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
                }
                if (a.bias) {
                    const float4 u = *reinterpret_cast<const float4*>(a.bias + i);
                    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
                }
                *reinterpret_cast<float4*>(row + i) = v;
            }
        }
    }
    if (!by_four) {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            float v = to_float(pr[i]);
            for (int p = 1; p < a.n_parts; ++p) v += to_float(pr[(size_t)p * a.part_stride + i]);
            if (a.bias) v += a.bias[i];
            row[i] = v;
        }
    }
    __syncthreads();
    // two neighbours a lane and one store for both, when every row they go to begins at an even element
    const bool pairs = (a.hd & 1) == 0 && (a.vd & 1) == 0 && (a.ldo & 1) == 0 && ((uintptr_t)a.out & 7) == 0 &&
                       ((uintptr_t)a.k_pages & 7) == 0 && ((uintptr_t)a.v_pages & 7) == 0 && ((uintptr_t)a.v_keep & 7) == 0;
    const int crow = a.k_pages ? a.cache_rows[t] : -1;
    const size_t page = crow >= 0 ? (size_t)(crow / a.page_size) : 0, place = crow >= 0 ? (size_t)(crow % a.page_size) : 0;
    O* orow = (O*)a.out + (size_t)t * a.ldo;
    const int hd = a.hd, half = a.rot / 2;
    const float* cs = a.cos_sin ? a.cos_sin + (size_t)pos * half * 2 : nullptr;
    // q and k heads, a warp per head
    for (int head = warp; head < a.n_q + a.n_kv; head += warps) {
        const float* x = row + (size_t)head * hd;
        float inv = 1.0f;
        if (a.head_norm) {
            float ss = 0.0f;
            for (int e = lane; e < hd; e += 32) ss += x[e] * x[e];
            ss = warp_sum(ss);
            inv = rsqrtf(ss / (float)hd + a.eps);
        }
        const bool is_k = head >= a.n_q;
        const float* gain = a.head_norm ? (is_k ? a.k_gain : a.q_gain) : nullptr;
        O* kdst = (is_k && crow >= 0) ? (O*)a.k_pages + ((page * a.n_kv + (head - a.n_q)) * a.page_size + place) * hd : nullptr;
        auto value = [&](int e) -> float {
            if (cs && e < a.rot) {
                int i, first;
                float u, w;
                if (a.pairing == 1) {
                    i = e >> 1;
                    first = (e & 1) == 0;
                    u = x[2 * i];
                    w = x[2 * i + 1];
                } else {
                    first = e < half;
                    i = first ? e : e - half;
                    u = x[i];
                    w = x[i + half];
                }
                u *= inv;
                w *= inv;
                if (gain) {
                    u *= a.pairing == 1 ? gain[2 * i] : gain[i];
                    w *= a.pairing == 1 ? gain[2 * i + 1] : gain[i + half];
                }
                const float c = cs[2 * i], s = cs[2 * i + 1];
                return first ? u * c - w * s : w * c + u * s;
            }
            return gain ? x[e] * inv * gain[e] : x[e] * inv;
        };
        if (pairs) {
            for (int e = 2 * lane; e < hd; e += 64) {
                const float v0 = value(e), v1 = value(e + 1);
                store_pair(orow + (size_t)head * hd + e, v0, v1);
                if (kdst) store_pair(kdst + e, v0, v1);
            }
        } else {
            for (int e = lane; e < hd; e += 32) {
                const O o = from_float<O>(value(e));
                orow[(size_t)head * hd + e] = o;
                if (kdst) kdst[e] = o;
            }
        }
    }
    // values
    const float lam = (a.lambda && a.v_first) ? *a.lambda : 0.0f;
    const float* vf = a.v_first ? a.v_first + (size_t)t * a.ld_first : nullptr;
    const int vd = a.vd;
    if (pairs) {
        for (int i = threadIdx.x * 2; i < v_cols; i += blockDim.x * 2) {
            float v0 = row[q_cols + k_cols + i], v1 = row[q_cols + k_cols + i + 1];
            if (a.v_keep) *reinterpret_cast<float2*>(a.v_keep + (size_t)t * v_cols + i) = make_float2(v0, v1);
            if (vf) {
                v0 = (1.0f - lam) * v0 + lam * vf[i];
                v1 = (1.0f - lam) * v1 + lam * vf[i + 1];
            }
            store_pair(orow + q_cols + k_cols + i, v0, v1);
            if (crow >= 0) {
                const int g = i / vd, d = i - g * vd;
                store_pair((O*)a.v_pages + ((page * a.n_kv + g) * a.page_size + place) * vd + d, v0, v1);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < v_cols; i += blockDim.x) {
        float v = row[q_cols + k_cols + i];
        if (a.v_keep) a.v_keep[(size_t)t * v_cols + i] = v;
        if (vf) v = (1.0f - lam) * v + lam * vf[i];
        const O o = from_float<O>(v);
        orow[q_cols + k_cols + i] = o;
        if (crow >= 0) {
            const int g = i / vd, d = i - g * vd;
            ((O*)a.v_pages)[((page * a.n_kv + g) * a.page_size + place) * vd + d] = o;
        }
    }
}

template <typename O>
__global__ void __launch_bounds__(256) heads_mix_kernel(const float* __restrict__ acc, long ld_acc, const float* __restrict__ talk,
                                                        const float* __restrict__ gate, long ld_gate, O* __restrict__ out,
                                                        long ldo, int heads, int n_kv, int vd) {
    extern __shared__ __align__(16) float tk[];        // talk [heads][heads]
    pdl_trigger();
    if (talk)
        for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) tk[i] = talk[i];
    pdl_wait();
    __syncthreads();
    const int t = blockIdx.x;
    const int group = heads / n_kv;
    const float* ar = acc + (size_t)t * ld_acc;
    // four neighbours of a head's row a thread when rows and addresses allow 16-byte steps (with a few tokens there
    // are threads to spare, and one number a thread is the shorter chain)
    if (gridDim.x >= 64 && (vd & 3) == 0 && (ld_acc & 3) == 0 && (ldo & 3) == 0 && ((uintptr_t)acc & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < heads * vd; i += gridDim.y * blockDim.x * 4) {
            const int h = i / vd, d = i - h * vd;
            const int c = h / group;
            float4 s4;
            if (talk) {
                s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int g = 0; g < heads; ++g) {
                    const float w = tk[h * heads + g];
                    const float4 v = *reinterpret_cast<const float4*>(ar + ((size_t)g * n_kv + c) * vd + d);
                    s4.x = fmaf(w, v.x, s4.x); s4.y = fmaf(w, v.y, s4.y); s4.z = fmaf(w, v.z, s4.z); s4.w = fmaf(w, v.w, s4.w);
                }
            } else {
                s4 = *reinterpret_cast<const float4*>(ar + i);
            }
            if (gate) {
                const float gt = 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate + h]));
                s4.x *= gt; s4.y *= gt; s4.z *= gt; s4.w *= gt;
            }
            O* dst = out + (size_t)t * ldo + i;
            store_pair(dst, s4.x, s4.y);
            store_pair(dst + 2, s4.z, s4.w);
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < heads * vd; i += gridDim.y * blockDim.x) {
        const int h = i / vd, d = i - h * vd;
        const int c = h / group;
        float s = 0.0f;
        if (talk) {
            for (int g = 0; g < heads; ++g) s = fmaf(tk[h * heads + g], ar[((size_t)g * n_kv + c) * vd + d], s);
        } else {
            s = ar[i];                                  // no mixing: acc is (tokens, heads * vd)
        }
        if (gate) s *= 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate + h]));
        out[(size_t)t * ldo + i] = from_float<O>(s);
    }
}

}  // namespace

BROLM_API int brolm_qkv_finish(const void* proj, int x_dtype, int n_parts, long long part_stride, long ldp, const void* bias,
                               int n_q, int n_kv, int hd, int vd, int head_norm, float eps, const void* positions,
                               const void* cos_sin, int rot, int pairing, const void* lambda, const void* v_first,
                               long ld_first, void* v_keep, void* out, int out_dtype, long ldo, void* k_pages, void* v_pages,
                               const void* cache_rows, int page_size, int tokens, const void* q_gain, const void* k_gain,
                               cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (n_q <= 0 || n_kv <= 0 || hd <= 0 || vd <= 0 || n_parts < 1) return BROLM_ERR_BAD_SIZE;
    if (cos_sin && (rot <= 0 || rot % 2 || rot > hd || pairing < 0 || pairing > 1)) return BROLM_ERR_BAD_SIZE;
    if (n_parts > 1 && x_dtype != BROLM_F32) return BROLM_ERR_BAD_DTYPE;
    const size_t smem = (size_t)((n_q + n_kv) * hd + n_kv * vd) * sizeof(float);
    if (smem > 200 * 1024) return BROLM_ERR_TOO_LARGE;
    FinishArgs a;
    a.proj = proj; a.n_parts = n_parts; a.part_stride = part_stride; a.ldp = ldp; a.bias = (const float*)bias;
    a.n_q = n_q; a.n_kv = n_kv; a.hd = hd; a.vd = vd; a.head_norm = head_norm; a.eps = eps;
    a.positions = (const int32_t*)positions; a.cos_sin = (const float*)cos_sin; a.rot = cos_sin ? rot : 0; a.pairing = pairing;
    a.lambda = (const float*)lambda; a.v_first = (const float*)v_first; a.ld_first = ld_first; a.v_keep = (float*)v_keep;
    a.out = out; a.ldo = ldo; a.k_pages = k_pages; a.v_pages = v_pages; a.cache_rows = (const int32_t*)cache_rows;
    a.page_size = page_size;
    a.q_gain = (const float*)q_gain; a.k_gain = (const float*)k_gain;
#define BROLM_QF(X, O)                                                                                             \
    do {                                                                                                           \
        static size_t allowed = 0;                                                                                 \
        if (smem > 48 * 1024 && smem > allowed) {                                                                  \
            cudaError_t e = cudaFuncSetAttribute(qkv_finish_kernel<X, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                       \
            if (e != cudaSuccess) return (int)e;                                                                   \
            allowed = smem;                                                                                        \
        }                                                                                                          \
        return launch_pdl(qkv_finish_kernel<X, O>, dim3(tokens), dim3(256), smem, stream, a);                      \
    } while (0)
    if (x_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_QF(float, float);
    if (x_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_QF(float, bf16);
    if (x_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_QF(bf16, bf16);
    if (x_dtype == BROLM_BF16 && out_dtype == BROLM_F32) BROLM_QF(bf16, float);
#undef BROLM_QF
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_heads_mix(const void* acc, long ld_acc, const void* talk, const void* gate, long ld_gate, void* out,
                              int out_dtype, long ldo, int heads, int n_kv, int vd, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (heads <= 0 || n_kv <= 0 || heads % n_kv || vd <= 0 || heads > 128) return BROLM_ERR_BAD_SIZE;
    const size_t smem = (size_t)heads * heads * sizeof(float);
    int by = (heads * vd + 255) / 256;
    if (by > 16) by = 16;
    dim3 grid(tokens, by);
    if (out_dtype == BROLM_F32)
        return launch_pdl(heads_mix_kernel<float>, grid, dim3(256), smem, stream, (const float*)acc, ld_acc, (const float*)talk,
                          (const float*)gate, ld_gate, (float*)out, ldo, heads, n_kv, vd);
    if (out_dtype == BROLM_BF16)
        return launch_pdl(heads_mix_kernel<bf16>, grid, dim3(256), smem, stream, (const float*)acc, ld_acc, (const float*)talk,
                          (const float*)gate, ld_gate, (bf16*)out, ldo, heads, n_kv, vd);
    return BROLM_ERR_BAD_DTYPE;
}
