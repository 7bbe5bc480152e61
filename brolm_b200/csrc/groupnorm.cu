// RMS norm in groups, alone and around the residual sum.
//
// A row of `hidden` elements is cut into `groups` equal consecutive parts; each part is divided by its own
// sqrt(mean(part^2) + eps) and the whole row is multiplied by a gain of `hidden` elements:
//     gnorm(x; w)[g*s + i] = x[g*s + i] * rsqrt(mean_i(x[g*s + .]^2) + eps) * (offset + w[g*s + i]),  s = hidden / groups.
// groups = 1 is the ordinary RMS norm.
//
//     group_rmsnorm:           out[r] = gnorm(x[rows[r] or r]; w)
//     residual_group_rmsnorm:  h += post ? gnorm(y; w_post) : y;   out = next ? gnorm(h; w_next) : h   (out optional)
//
// h is the float residual stream; y may come as partial sums [parts][rows][hidden] that are added in order.
// One block of 256 threads per row; a lane takes four elements at a time when the sizes and addresses allow.
// A row is cut into segments (a group, or an equal piece of a group when
// there are fewer groups than warps); a warp takes whole segments, sums their squares in lane order and leaves
// one partial sum per segment, and a group's statistic is the sum of its segments' partial sums in order: the
// order of every addition is fixed by the sizes alone, never by what else runs.  The row stays in shared
// memory between the passes, so y and h are read once and h is written once.  All arithmetic is float.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_SEGMENTS = 1024;

struct Segments {
    int groups, gs;      // groups and their size
    int sub, seg;        // pieces per group and the size of a piece (the last one of a group may be shorter)
    int n;               // groups * sub
};

__host__ __device__ inline Segments make_segments(int hidden, int groups) {
    Segments s;
    s.groups = groups;
    s.gs = hidden / groups;
    s.sub = groups >= WARPS ? 1 : WARPS / groups;
    if (s.sub > s.gs) s.sub = s.gs;
    s.seg = (s.gs + s.sub - 1) / s.sub;
    s.n = groups * s.sub;
    return s;
}

// 1 / sqrt(mean + eps) of group g from the partial sums of its segments
__device__ __forceinline__ float group_inv(const float* partial, const Segments& s, int g, float eps) {
    float t = 0.0f;
    for (int k = 0; k < s.sub; ++k) t += partial[g * s.sub + k];
    return rsqrtf(t / (float)s.gs + eps);
}


// V elements at once (V = 1, or 4 when every segment, the row and all addresses allow 16-byte steps)
template <int V> __device__ __forceinline__ void ld(const float* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
        v[0] = *p;
    }
}
template <int V> __device__ __forceinline__ void ld(const bf16* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
        v[0] = __bfloat162float(*p);
    }
}
template <int V> __device__ __forceinline__ void st(float* p, const float (&v)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <int V> __device__ __forceinline__ void st(bf16* p, const float (&v)[V]) {
    if constexpr (V == 4) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&a);
        u.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    } else {
        *p = __float2bfloat16_rn(v[0]);
    }
}

template <typename X, typename W, typename O, int V>
__global__ void __launch_bounds__(THREADS) group_rmsnorm_kernel(const X* __restrict__ x, const int32_t* __restrict__ rows,
                                                                const W* __restrict__ w, float eps, float offset,
                                                                O* __restrict__ out, int hidden, int groups) {
    extern __shared__ __align__(16) float smem[];
    const Segments s = make_segments(hidden, groups);
    float* row = smem;                 // [hidden]
    float* partial = smem + hidden;    // [s.n]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    const X* xr = x + r * hidden;
    for (int sg = warp; sg < s.n; sg += WARPS) {
        const int g = sg / s.sub, k = sg - g * s.sub;
        const int lo = g * s.gs + k * s.seg, hi = min(g * s.gs + s.gs, lo + s.seg);
        float ss = 0.0f;
        for (int i = lo + lane * V; i < hi; i += 32 * V) {
            float v[V];
            ld<V>(xr + i, v);
            st<V>(row + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) ss += v[e] * v[e];
        }
        ss = warp_sum(ss);
        if (lane == 0) partial[sg] = ss;
    }
    __syncthreads();
    O* orow = out + (size_t)blockIdx.x * hidden;
    for (int sg = warp; sg < s.n; sg += WARPS) {
        const int g = sg / s.sub, k = sg - g * s.sub;
        const int lo = g * s.gs + k * s.seg, hi = min(g * s.gs + s.gs, lo + s.seg);
        const float inv = group_inv(partial, s, g, eps);
        for (int i = lo + lane * V; i < hi; i += 32 * V) {
            float v[V], g_[V];
            ld<V>(row + i, v);
            ld<V>(w + i, g_);
#pragma unroll
            for (int e = 0; e < V; ++e) v[e] = v[e] * inv * (offset + g_[e]);
            st<V>(orow + i, v);
        }
    }
}

template <typename Y, typename W, typename O, int V>
__global__ void __launch_bounds__(THREADS) residual_group_rmsnorm_kernel(
    float* __restrict__ h, const Y* __restrict__ y, int n_parts, long long part_stride, const W* __restrict__ w_post,
    float eps_post, float off_post, const W* __restrict__ w_next, float eps_next, float off_next, O* __restrict__ out,
    int hidden, int groups) {
    extern __shared__ __align__(16) float smem[];
    const Segments s = make_segments(hidden, groups);
    float* row = smem;                 // [hidden]
    float* partial = smem + hidden;    // [2][s.n]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t base = (size_t)blockIdx.x * hidden;
    pdl_wait();
    // pass 1: y as the sum of its parts, and the squares of its groups
    for (int sg = warp; sg < s.n; sg += WARPS) {
        const int g = sg / s.sub, k = sg - g * s.sub;
        const int lo = g * s.gs + k * s.seg, hi = min(g * s.gs + s.gs, lo + s.seg);
        float ss = 0.0f;
        for (int i = lo + lane * V; i < hi; i += 32 * V) {
            float v[V];
            ld<V>(y + base + i, v);
            for (int p = 1; p < n_parts; ++p) {
                float t[V];
                ld<V>(y + (size_t)p * part_stride + base + i, t);
#pragma unroll
                for (int e = 0; e < V; ++e) v[e] += t[e];
            }
            st<V>(row + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) ss += v[e] * v[e];
        }
        ss = warp_sum(ss);
        if (lane == 0) partial[sg] = ss;
    }
    __syncthreads();
    // pass 2: the sum into the stream, and the squares of the new stream's groups
    for (int sg = warp; sg < s.n; sg += WARPS) {
        const int g = sg / s.sub, k = sg - g * s.sub;
        const int lo = g * s.gs + k * s.seg, hi = min(g * s.gs + s.gs, lo + s.seg);
        const float inv = w_post ? group_inv(partial, s, g, eps_post) : 1.0f;
        float ss = 0.0f;
        for (int i = lo + lane * V; i < hi; i += 32 * V) {
            float v[V], hn[V];
            ld<V>(row + i, v);
            if (w_post) {
                float g_[V];
                ld<V>(w_post + i, g_);
#pragma unroll
                for (int e = 0; e < V; ++e) v[e] = v[e] * inv * (off_post + g_[e]);
            }
            ld<V>(h + base + i, hn);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                hn[e] += v[e];
                ss += hn[e] * hn[e];
            }
            st<V>(h + base + i, hn);
            st<V>(row + i, hn);
        }
        ss = warp_sum(ss);
        if (lane == 0) partial[s.n + sg] = ss;
    }
    if (!out) return;
    __syncthreads();
    for (int sg = warp; sg < s.n; sg += WARPS) {
        const int g = sg / s.sub, k = sg - g * s.sub;
        const int lo = g * s.gs + k * s.seg, hi = min(g * s.gs + s.gs, lo + s.seg);
        const float inv = w_next ? group_inv(partial + s.n, s, g, eps_next) : 1.0f;
        for (int i = lo + lane * V; i < hi; i += 32 * V) {
            float v[V];
            ld<V>(row + i, v);
            if (w_next) {
                float g_[V];
                ld<V>(w_next + i, g_);
#pragma unroll
                for (int e = 0; e < V; ++e) v[e] = v[e] * inv * (off_next + g_[e]);
            }
            st<V>(out + base + i, v);
        }
    }
}

int check_sizes(int hidden, int groups, size_t* smem) {
    if (hidden <= 0 || groups <= 0 || hidden % groups) return BROLM_ERR_BAD_SIZE;
    const Segments s = make_segments(hidden, groups);
    if (s.n > MAX_SEGMENTS) return BROLM_ERR_TOO_LARGE;
    *smem = ((size_t)hidden + 2 * (size_t)s.n) * sizeof(float);
    if (*smem > 200 * 1024) return BROLM_ERR_TOO_LARGE;
    return BROLM_OK;
}

template <typename K>
int allow_smem(K kernel, size_t smem, size_t* allowed) {
    if (smem > 48 * 1024 && smem > *allowed) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        *allowed = smem;
    }
    return BROLM_OK;
}

// whether every segment begins and ends at a multiple of four elements
inline bool by_four(int hidden, int groups) {
    const Segments s = make_segments(hidden, groups);
    return hidden % 4 == 0 && s.gs % 4 == 0 && s.seg % 4 == 0;
}
template <typename... P> bool aligned16(P... p) { return (((uintptr_t)p | ...) & 15) == 0; }

template <typename X, typename W, typename O>
int launch_norm(const void* x, const void* rows, const void* w, float eps, float offset, void* out, int n, int hidden,
                int groups, size_t smem, cudaStream_t stream) {
    static size_t allowed[2] = {0, 0};
    if (by_four(hidden, groups) && aligned16(x, w, out)) {
        if (int e = allow_smem(group_rmsnorm_kernel<X, W, O, 4>, smem, &allowed[1])) return e;
        return launch_pdl(group_rmsnorm_kernel<X, W, O, 4>, dim3(n), dim3(THREADS), smem, stream, (const X*)x,
                          (const int32_t*)rows, (const W*)w, eps, offset, (O*)out, hidden, groups);
    }
    if (int e = allow_smem(group_rmsnorm_kernel<X, W, O, 1>, smem, &allowed[0])) return e;
    return launch_pdl(group_rmsnorm_kernel<X, W, O, 1>, dim3(n), dim3(THREADS), smem, stream, (const X*)x,
                      (const int32_t*)rows, (const W*)w, eps, offset, (O*)out, hidden, groups);
}

template <typename Y, typename W, typename O>
int launch_residual(void* h, const void* y, int n_parts, long long part_stride, const void* w_post, float eps_post,
                    float off_post, const void* w_next, float eps_next, float off_next, void* out, int n, int hidden,
                    int groups, size_t smem, cudaStream_t stream) {
    static size_t allowed[2] = {0, 0};
    if (by_four(hidden, groups) && part_stride % 4 == 0 && aligned16(h, y, w_post, w_next, out)) {
        if (int e = allow_smem(residual_group_rmsnorm_kernel<Y, W, O, 4>, smem, &allowed[1])) return e;
        return launch_pdl(residual_group_rmsnorm_kernel<Y, W, O, 4>, dim3(n), dim3(THREADS), smem, stream, (float*)h,
                          (const Y*)y, n_parts, part_stride, (const W*)w_post, eps_post, off_post, (const W*)w_next,
                          eps_next, off_next, (O*)out, hidden, groups);
    }
    if (int e = allow_smem(residual_group_rmsnorm_kernel<Y, W, O, 1>, smem, &allowed[0])) return e;
    return launch_pdl(residual_group_rmsnorm_kernel<Y, W, O, 1>, dim3(n), dim3(THREADS), smem, stream, (float*)h,
                      (const Y*)y, n_parts, part_stride, (const W*)w_post, eps_post, off_post, (const W*)w_next, eps_next,
                      off_next, (O*)out, hidden, groups);
}

}  // namespace

BROLM_API int brolm_group_rmsnorm(const void* x, int x_dtype, const void* rows, const void* w, int w_dtype, float eps,
                                  float offset, void* out, int out_dtype, int n, int hidden, int groups,
                                  cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    size_t smem = 0;
    if (int e = check_sizes(hidden, groups, &smem)) return e;
#define BROLM_GN(X, W, O) return launch_norm<X, W, O>(x, rows, w, eps, offset, out, n, hidden, groups, smem, stream)
#define BROLM_GN2(X, W)                               \
    do {                                              \
        if (out_dtype == BROLM_F32) BROLM_GN(X, W, float); \
        if (out_dtype == BROLM_BF16) BROLM_GN(X, W, bf16); \
        return BROLM_ERR_BAD_DTYPE;                   \
    } while (0)
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_F32) BROLM_GN2(float, float);
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_BF16) BROLM_GN2(float, bf16);
    if (x_dtype == BROLM_BF16 && w_dtype == BROLM_F32) BROLM_GN2(bf16, float);
    if (x_dtype == BROLM_BF16 && w_dtype == BROLM_BF16) BROLM_GN2(bf16, bf16);
#undef BROLM_GN2
#undef BROLM_GN
    return BROLM_ERR_BAD_DTYPE;
}

// w_post and w_next share one element type (w_dtype); either may be null.  out null: only the sum.
BROLM_API int brolm_residual_group_rmsnorm(void* h, const void* y, int y_dtype, int n_parts, long long part_stride,
                                           const void* w_post, float eps_post, float off_post, const void* w_next,
                                           float eps_next, float off_next, int w_dtype, void* out, int out_dtype, int n,
                                           int hidden, int groups, cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    if (n_parts < 1) return BROLM_ERR_BAD_SIZE;
    size_t smem = 0;
    if (int e = check_sizes(hidden, groups, &smem)) return e;
#define BROLM_RG(Y, W, O)                                                                                              \
    return launch_residual<Y, W, O>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, \
                                    out, n, hidden, groups, smem, stream)
#define BROLM_RG2(Y, W)                                             \
    do {                                                            \
        if (!out || out_dtype == BROLM_F32) BROLM_RG(Y, W, float);  \
        if (out_dtype == BROLM_BF16) BROLM_RG(Y, W, bf16);          \
        return BROLM_ERR_BAD_DTYPE;                                 \
    } while (0)
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_F32) BROLM_RG2(float, float);
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_BF16) BROLM_RG2(float, bf16);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_F32) BROLM_RG2(bf16, float);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_BF16) BROLM_RG2(bf16, bf16);
#undef BROLM_RG2
#undef BROLM_RG
    return BROLM_ERR_BAD_DTYPE;
}
