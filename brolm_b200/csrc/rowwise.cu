// Row-wise steps between the matrix products of a layer, all with float arithmetic:
//
//   cast            out = x in another element type
//   bias_act        out = act(sum of the parts of y + bias)
//   scaled_sum      out = sa * (sum of a's parts) + sb * (sum of b's parts)
//   qkv_norm_write  RMS norm of the whole query row and of the whole key row of a token (one
//                   statistic over all heads), and keys and values into the paged cache; the
//                   value rows may have a size of their own
//   gate_group_norm out = rmsnorm per group of (y * silu(z)) * gain
//   experts_combine out = sum over a token's choices of weight * (expert's result | the token's own
//                   row for an identity expert) + the shared expert's result, the latter times
//                   sigmoid(w . x) when a gate row w is given
//   norm_sigmoid_gate  out = (y / rms(y) * gain, or y itself without a gain) * sigmoid(z)
//
// Inputs are float or bfloat16, outputs as asked for.  One block per token (row); a row's result
// depends on that row alone.
#include "common.cuh"

namespace {

enum : int { RACT_NONE = 0, RACT_RELU2 = 1, RACT_GELU_TANH = 2, RACT_SILU = 3 };

__device__ __forceinline__ float row_act(float v, int act) {
    if (act == RACT_RELU2) {
        v = fmaxf(v, 0.0f);
        return v * v;
    }
    if (act == RACT_GELU_TANH) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    if (act == RACT_SILU) return v / (1.0f + expf(-v));
    return v;
}

template <typename X, typename O>
__global__ void __launch_bounds__(256) cast_kernel(const X* __restrict__ x, O* __restrict__ out, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = to_float(x[i + e]);
#pragma unroll
        for (int e = 0; e < 4; ++e) out[i + e] = from_float<O>(v[e]);
    } else {
        for (long long j = i; j < n; ++j) out[j] = from_float<O>(to_float(x[j]));
    }
}

template <typename Y, typename B, typename O>
__global__ void __launch_bounds__(256) bias_act_kernel(const Y* __restrict__ y, int n_parts, long long part_stride, long ldy,
                                                       const B* __restrict__ bias, int act, O* __restrict__ out, long ldo,
                                                       int cols) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const Y* yr = y + (size_t)r * ldy + c;
    float v = to_float(yr[0]);
    for (int s = 1; s < n_parts; ++s) v += to_float(yr[(size_t)s * part_stride]);
    if (bias) v += to_float(bias[c]);
    out[(size_t)r * ldo + c] = from_float<O>(row_act(v, act));
}

// The same over float sums, four neighbours a thread (every row and part begins at a multiple of 16 bytes).
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    uint2 packed;
    *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = packed;
}

template <typename B, typename O>
__global__ void __launch_bounds__(256) bias_act4_kernel(const float* y, int n_parts, long long part_stride, long ldy,
                                                        const B* __restrict__ bias, int act, O* out, long ldo, int cols) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= cols) return;
    const float* yr = y + (size_t)r * ldy + c;
    const float4 first = *reinterpret_cast<const float4*>(yr);
    float v[4] = {first.x, first.y, first.z, first.w};
    for (int s = 1; s < n_parts; ++s) {
        const float4 u = *reinterpret_cast<const float4*>(yr + (size_t)s * part_stride);
        v[0] += u.x; v[1] += u.y; v[2] += u.z; v[3] += u.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (bias) v[e] += to_float(bias[c + e]);
        v[e] = row_act(v[e], act);
    }
    store4(out + (size_t)r * ldo + c, v);              // (y and out may be the same rows: a thread reads what it writes first)
}

__global__ void __launch_bounds__(256) scaled_sum_kernel(const float* __restrict__ a, int a_parts, long long a_stride, float sa,
                                                         const float* __restrict__ b, int b_parts, long long b_stride, float sb,
                                                         float* __restrict__ out, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float va = a[i], vb = b[i];
    for (int s = 1; s < a_parts; ++s) va += a[(size_t)s * a_stride + i];
    for (int s = 1; s < b_parts; ++s) vb += b[(size_t)s * b_stride + i];
    out[i] = sa * va + sb * vb;
}

// proj row t: [ q: q_cols | k: k_cols | v: v_cols ] (float or bfloat16).  out row t takes the same layout in O.
// whole_norm: q <- q * rsqrt(mean(q^2) + eps) * wq over all q_cols at once, the same for k with wk.
// The cache of this layer is k_pages [page][n_kv][page_size][k_cols / n_kv], v_pages [...][v_cols / n_kv].
template <typename X, typename W, typename O>
__global__ void __launch_bounds__(256) qkv_norm_write_kernel(const X* __restrict__ proj, long ldp, int q_cols, int k_cols, int v_cols,
                                                             const W* __restrict__ wq, const W* __restrict__ wk, float eps,
                                                             int whole_norm, const int32_t* __restrict__ positions,
                                                             O* __restrict__ out, long ldo, O* __restrict__ k_pages,
                                                             O* __restrict__ v_pages, const int32_t* __restrict__ cache_rows,
                                                             int n_kv, int page_size) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    pdl_wait();
    if (pos < 0) return;                               // a padding row
    const X* pr = proj + (size_t)t * ldp;
    O* orow = out + (size_t)t * ldo;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (whole_norm) {
        float sq = 0.0f, sk = 0.0f;
        for (int i = threadIdx.x; i < q_cols; i += blockDim.x) {
            const float v = to_float(pr[i]);
            sq += v * v;
        }
        for (int i = threadIdx.x; i < k_cols; i += blockDim.x) {
            const float v = to_float(pr[q_cols + i]);
            sk += v * v;
        }
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        inv_q = rsqrtf(sq / (float)q_cols + eps);
        inv_k = rsqrtf(sk / (float)k_cols + eps);
    }
    const int crow = k_pages ? cache_rows[t] : -1;
    const int kd = k_cols / n_kv, vd = v_cols / n_kv;
    const size_t page = crow >= 0 ? (size_t)(crow / page_size) : 0, place = crow >= 0 ? (size_t)(crow % page_size) : 0;
    for (int i = threadIdx.x; i < q_cols; i += blockDim.x) {
        float v = to_float(pr[i]);
        if (whole_norm) v = v * inv_q * to_float(wq[i]);
        orow[i] = from_float<O>(v);
    }
    for (int i = threadIdx.x; i < k_cols; i += blockDim.x) {
        float v = to_float(pr[q_cols + i]);
        if (whole_norm) v = v * inv_k * to_float(wk[i]);
        const O o = from_float<O>(v);
        orow[q_cols + i] = o;
        if (crow >= 0) {
            const int g = i / kd, d = i - g * kd;
            k_pages[((page * n_kv + g) * page_size + place) * kd + d] = o;
        }
    }
    for (int i = threadIdx.x; i < v_cols; i += blockDim.x) {
        const O o = from_float<O>(to_float(pr[q_cols + k_cols + i]));
        orow[q_cols + k_cols + i] = o;
        if (crow >= 0) {
            const int g = i / vd, d = i - g * vd;
            v_pages[((page * n_kv + g) * page_size + place) * vd + d] = o;
        }
    }
}

// out[t, g*gs + i] = (y * silu(z))[.] * rsqrt(mean over the group + eps) * w[.]; one block per (group, token)
template <typename Z, typename W, typename O>
__global__ void __launch_bounds__(256) gate_group_norm_kernel(const float* __restrict__ y, long ldy, const Z* __restrict__ z, long ldz,
                                                              const W* __restrict__ w, float eps, int group_size,
                                                              O* __restrict__ out, long ldo) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y;
    const float* yr = y + (size_t)t * ldy + (size_t)g * group_size;
    const Z* zr = z + (size_t)t * ldz + (size_t)g * group_size;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < group_size; i += blockDim.x) {
        const float zz = to_float(zr[i]);
        const float v = yr[i] * (zz / (1.0f + expf(-zz)));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)group_size + eps);
    for (int i = threadIdx.x; i < group_size; i += blockDim.x) {
        const float zz = to_float(zr[i]);
        const float v = yr[i] * (zz / (1.0f + expf(-zz)));
        out[(size_t)t * ldo + (size_t)g * group_size + i] = from_float<O>(v * inv * to_float(w[(size_t)g * group_size + i]));
    }
}

// y [top][tokens][hidden] float (rows of choices that named an identity expert are never read), x the experts'
// input, shared [parts][tokens][hidden] float or null.  V: neighbours of a row a thread takes (four when hidden is a
// multiple of four and every row begins at a multiple of 16 bytes, else one).
template <typename X, int V>
__global__ void __launch_bounds__(256) experts_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ ids,
                                                              const float* __restrict__ wts, int top, int n_real,
                                                              const X* __restrict__ x, long ldx,
                                                              const float* __restrict__ shared, int shared_parts,
                                                              long long shared_stride, float* __restrict__ out, int tokens,
                                                              int hidden, const X* __restrict__ shared_gate, int gate_vec) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    float sg = 1.0f;
    if (shared_gate && shared_parts > 0) {
        // one number per token: the logistic function of the gate row's product with the token's input, summed
        // in float by a fixed tree (every block of the token computes the same)
        float dot = 0.0f;
        const X* xr = x + (size_t)t * ldx;
        if (gate_vec) {                                  // eight numbers a load
            for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
                float gv[8], xv[8];
                load8(shared_gate + i, gv);
                load8(xr + i, xv);
#pragma unroll
                for (int e = 0; e < 8; ++e) dot = fmaf(gv[e], xv[e], dot);
            }
        } else {
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) dot = fmaf(to_float(shared_gate[i]), to_float(xr[i]), dot);
        }
        dot = block_sum(dot, scratch);
        sg = 1.0f / (1.0f + expf(-dot));
    }
    if (c >= hidden) return;
    if constexpr (V == 4) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sh[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)t * top + k];
            const float w = wts[(size_t)t * top + k];
            float4 v;
            if (e < n_real) {
                v = *reinterpret_cast<const float4*>(y + ((size_t)k * tokens + t) * hidden + c);
            } else {
                const X* xr = x + (size_t)t * ldx + c;
                v = make_float4(to_float(xr[0]), to_float(xr[1]), to_float(xr[2]), to_float(xr[3]));
            }
            acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
            acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
        }
        for (int s = 0; s < shared_parts; ++s) {
            const float4 u = *reinterpret_cast<const float4*>(shared + (size_t)s * shared_stride + (size_t)t * hidden + c);
            sh[0] += u.x; sh[1] += u.y; sh[2] += u.z; sh[3] += u.w;
        }
        *reinterpret_cast<float4*>(out + (size_t)t * hidden + c) =
            make_float4(fmaf(sg, sh[0], acc[0]), fmaf(sg, sh[1], acc[1]), fmaf(sg, sh[2], acc[2]), fmaf(sg, sh[3], acc[3]));
        return;
    }
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
        const int e = ids[(size_t)t * top + k];
        const float w = wts[(size_t)t * top + k];
        const float v = e < n_real ? y[((size_t)k * tokens + t) * hidden + c] : to_float(x[(size_t)t * ldx + c]);
        acc = fmaf(w, v, acc);
    }
    float sh = 0.0f;
    for (int s = 0; s < shared_parts; ++s) sh += shared[(size_t)s * shared_stride + (size_t)t * hidden + c];
    out[(size_t)t * hidden + c] = fmaf(sg, sh, acc);
}

// out[t, i] = n(y)[t, i] * sigmoid(z[t, i]);  n(y) = y * rsqrt(mean(y^2) + eps) * w with a gain w, y itself
// without one.  One block per token.
template <typename Y, typename Z, typename W, typename O>
__global__ void __launch_bounds__(256) norm_sigmoid_gate_kernel(const Y* __restrict__ y, long ldy, const Z* __restrict__ z, long ldz,
                                                                const W* __restrict__ w, float eps, int cols,
                                                                O* __restrict__ out, long ldo) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const Y* yr = y + (size_t)t * ldy;
    const Z* zr = z + (size_t)t * ldz;
    float inv = 1.0f;
    if (w) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = to_float(yr[i]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        inv = rsqrtf(ss / (float)cols + eps);
    }
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = to_float(yr[i]);
        if (w) v = v * inv * to_float(w[i]);
        out[(size_t)t * ldo + i] = from_float<O>(v / (1.0f + expf(-to_float(zr[i]))));
    }
}

}  // namespace

BROLM_API int brolm_cast(const void* x, int x_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    const unsigned blocks = (unsigned)((n + 1023) / 1024);
#define BROLM_CAST(X, O) return launch_pdl(cast_kernel<X, O>, dim3(blocks), dim3(256), 0, stream, (const X*)x, (O*)out, n)
    if (x_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_CAST(float, bf16);
    if (x_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_CAST(float, float);
    if (x_dtype == BROLM_BF16 && out_dtype == BROLM_F32) BROLM_CAST(bf16, float);
    if (x_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_CAST(bf16, bf16);
#undef BROLM_CAST
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_bias_act(const void* y, int y_dtype, int n_parts, long long part_stride, long ldy, const void* bias,
                             int bias_dtype, int act, void* out, int out_dtype, long ldo, int rows, int cols,
                             cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return BROLM_OK;
    if (act < 0 || act > 3 || n_parts < 1) return BROLM_ERR_BAD_SIZE;
    if (y_dtype == BROLM_F32 && cols % 4 == 0 && ldy % 4 == 0 && part_stride % 4 == 0 && ldo % 4 == 0 &&
        ((uintptr_t)y & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        dim3 grid4(rows, (cols / 4 + 255) / 256);
#define BROLM_BA4(B, O) return launch_pdl(bias_act4_kernel<B, O>, grid4, dim3(256), 0, stream, (const float*)y, n_parts, \
                                          part_stride, ldy, (const B*)bias, act, (O*)out, ldo, cols)
        if (bias_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_BA4(float, float);
        if (bias_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_BA4(float, bf16);
        if (bias_dtype == BROLM_BF16 && out_dtype == BROLM_F32) BROLM_BA4(bf16, float);
        if (bias_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_BA4(bf16, bf16);
#undef BROLM_BA4
    }
    dim3 grid(rows, (cols + 255) / 256);
#define BROLM_BA(Y, B, O) return launch_pdl(bias_act_kernel<Y, B, O>, grid, dim3(256), 0, stream, (const Y*)y, n_parts, \
                                            part_stride, ldy, (const B*)bias, act, (O*)out, ldo, cols)
#define BROLM_BA2(Y, B)                                 \
    do {                                                \
        if (out_dtype == BROLM_F32) BROLM_BA(Y, B, float); \
        if (out_dtype == BROLM_BF16) BROLM_BA(Y, B, bf16); \
        return BROLM_ERR_BAD_DTYPE;                     \
    } while (0)
    if (y_dtype == BROLM_F32 && bias_dtype == BROLM_F32) BROLM_BA2(float, float);
    if (y_dtype == BROLM_F32 && bias_dtype == BROLM_BF16) BROLM_BA2(float, bf16);
    if (y_dtype == BROLM_BF16 && bias_dtype == BROLM_F32) BROLM_BA2(bf16, float);
    if (y_dtype == BROLM_BF16 && bias_dtype == BROLM_BF16) BROLM_BA2(bf16, bf16);
#undef BROLM_BA2
#undef BROLM_BA
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_scaled_sum(const void* a, int a_parts, long long a_stride, float sa, const void* b, int b_parts,
                               long long b_stride, float sb, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    if (a_parts < 1 || b_parts < 1) return BROLM_ERR_BAD_SIZE;
    return launch_pdl(scaled_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)a, a_parts,
                      a_stride, sa, (const float*)b, b_parts, b_stride, sb, (float*)out, n);
}

BROLM_API int brolm_qkv_norm_write(const void* proj, int x_dtype, long ldp, int q_cols, int k_cols, int v_cols,
                                   const void* wq, const void* wk, int w_dtype, float eps, int whole_norm,
                                   const void* positions, void* out, int out_dtype, long ldo, void* k_pages, void* v_pages,
                                   const void* cache_rows, int n_kv, int page_size, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (n_kv <= 0 || k_cols % n_kv || v_cols % n_kv || q_cols <= 0) return BROLM_ERR_BAD_SIZE;
    if (whole_norm && (!wq || !wk)) return BROLM_ERR_BAD_SIZE;
#define BROLM_QN(X, W, O) return launch_pdl(qkv_norm_write_kernel<X, W, O>, dim3(tokens), dim3(256), 0, stream, (const X*)proj, \
        ldp, q_cols, k_cols, v_cols, (const W*)wq, (const W*)wk, eps, whole_norm, (const int32_t*)positions, (O*)out, ldo,  \
        (O*)k_pages, (O*)v_pages, (const int32_t*)cache_rows, n_kv, page_size)
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_QN(float, float, float);
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_QN(float, bf16, bf16);
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_QN(float, float, bf16);
    if (x_dtype == BROLM_BF16 && w_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_QN(bf16, bf16, bf16);
#undef BROLM_QN
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_gate_group_norm(const void* y, long ldy, const void* z, int z_dtype, long ldz, const void* w, int w_dtype,
                                    float eps, int groups, int group_size, void* out, int out_dtype, long ldo, int tokens,
                                    cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (groups <= 0 || group_size <= 0) return BROLM_ERR_BAD_SIZE;
    if (groups > 65535) return BROLM_ERR_TOO_LARGE;
    dim3 grid(tokens, groups);
#define BROLM_GN(Z, W, O) return launch_pdl(gate_group_norm_kernel<Z, W, O>, grid, dim3(256), 0, stream, (const float*)y, ldy, \
                                            (const Z*)z, ldz, (const W*)w, eps, group_size, (O*)out, ldo)
    if (z_dtype == BROLM_F32 && w_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_GN(float, float, float);
    if (z_dtype == BROLM_F32 && w_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_GN(float, bf16, bf16);
    if (z_dtype == BROLM_F32 && w_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_GN(float, float, bf16);
    if (z_dtype == BROLM_BF16 && w_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_GN(bf16, bf16, bf16);
#undef BROLM_GN
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_experts_combine(const void* y, const void* ids, const void* wts, int top, int n_real, const void* x,
                                    int x_dtype, long ldx, const void* shared, int shared_parts, long long shared_stride,
                                    void* out, int tokens, int hidden, const void* shared_gate, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (!shared) shared_parts = 0;
    const int gate_vec = shared_gate && hidden % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 31) == 0 &&
                         ((uintptr_t)shared_gate & 31) == 0;
    const bool by_four = hidden % 4 == 0 && shared_stride % 4 == 0 && ((uintptr_t)y & 15) == 0 &&
                         ((uintptr_t)shared & 15) == 0 && ((uintptr_t)out & 15) == 0;
    dim3 grid(tokens, by_four ? (hidden / 4 + 255) / 256 : (hidden + 255) / 256);
#define BROLM_EC(X, V) return launch_pdl(experts_combine_kernel<X, V>, grid, dim3(256), 0, stream, (const float*)y,       \
                                         (const int32_t*)ids, (const float*)wts, top, n_real, (const X*)x, ldx,           \
                                         (const float*)shared, shared_parts, shared_stride, (float*)out, tokens, hidden, \
                                         (const X*)shared_gate, gate_vec)
    if (x_dtype == BROLM_F32) {
        if (by_four) BROLM_EC(float, 4);
        BROLM_EC(float, 1);
    }
    if (x_dtype == BROLM_BF16) {
        if (by_four) BROLM_EC(bf16, 4);
        BROLM_EC(bf16, 1);
    }
#undef BROLM_EC
    return BROLM_ERR_BAD_DTYPE;
}

// y, z and the gain w (null: no norm) are float or bfloat16 each; the result is float or bfloat16.
BROLM_API int brolm_norm_sigmoid_gate(const void* y, int y_dtype, long ldy, const void* z, int z_dtype, long ldz,
                                      const void* w, int w_dtype, float eps, int cols, void* out, int out_dtype, long ldo,
                                      int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (cols <= 0) return BROLM_ERR_BAD_SIZE;
    if (!w) w_dtype = BROLM_F32;
#define BROLM_NG(Y, Z, W, O) return launch_pdl(norm_sigmoid_gate_kernel<Y, Z, W, O>, dim3(tokens), dim3(256), 0, stream, \
                                               (const Y*)y, ldy, (const Z*)z, ldz, (const W*)w, eps, cols, (O*)out, ldo)
#define BROLM_NG2(Y, Z, W)                                    \
    do {                                                      \
        if (out_dtype == BROLM_F32) BROLM_NG(Y, Z, W, float); \
        if (out_dtype == BROLM_BF16) BROLM_NG(Y, Z, W, bf16); \
        return BROLM_ERR_BAD_DTYPE;                           \
    } while (0)
    if (y_dtype == BROLM_F32 && z_dtype == BROLM_F32 && w_dtype == BROLM_F32) BROLM_NG2(float, float, float);
    if (y_dtype == BROLM_F32 && z_dtype == BROLM_F32 && w_dtype == BROLM_BF16) BROLM_NG2(float, float, bf16);
    if (y_dtype == BROLM_F32 && z_dtype == BROLM_BF16 && w_dtype == BROLM_BF16) BROLM_NG2(float, bf16, bf16);
    if (y_dtype == BROLM_BF16 && z_dtype == BROLM_BF16 && w_dtype == BROLM_BF16) BROLM_NG2(bf16, bf16, bf16);
    if (y_dtype == BROLM_BF16 && z_dtype == BROLM_BF16 && w_dtype == BROLM_F32) BROLM_NG2(bf16, bf16, float);
    if (y_dtype == BROLM_BF16 && z_dtype == BROLM_F32 && w_dtype == BROLM_F32) BROLM_NG2(bf16, float, float);
    if (y_dtype == BROLM_BF16 && z_dtype == BROLM_F32 && w_dtype == BROLM_BF16) BROLM_NG2(bf16, float, bf16);
    if (y_dtype == BROLM_F32 && z_dtype == BROLM_BF16 && w_dtype == BROLM_F32) BROLM_NG2(float, bf16, float);
#undef BROLM_NG2
#undef BROLM_NG
    return BROLM_ERR_BAD_DTYPE;
}
