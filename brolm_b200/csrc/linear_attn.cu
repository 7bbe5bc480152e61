// Linear attention with a fixed decay per head, as a recurrence over the packed tokens of a step:
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        (S: d x dv floats per head and sequence)
//   o_t = S_t^T q_t
//
// q, k (d per head) and v (dv per head) are columns of one projection row per token, float or bfloat16; an
// activation (none, or silu) is applied to all three as they are read, in float.  The decay arrives as decay - 1
// (rounded from the host's double), and is applied as S + (decay - 1) S: a decay of 0.999 then keeps the digits
// that 0.999 itself loses when it is rounded to a float.  S lives in a float state row per sequence, laid out
// [head][value column][d padded to a multiple of four]; it is zero when the sequence starts, read at the start of
// the sequence's tokens of the step and written at their end.  One kernel serves a prompt and a step of single
// tokens.
//
// decay_scan_kernel: a block of 128 threads takes one (sequence, head) and 128 / DS value columns; the DS lanes of a
// column keep NJ float4 of the column's states each (d = 4 (j DS + ds) + e), so that q and k are read as float4 from
// shared memory and a column's state row is read and written in contiguous runs.  Tokens are staged sixteen at a
// time.  The sum over d of a column is folded across its DS lanes by shuffles.  Sequential in the tokens: the
// order of the additions of a token's result does not depend on how the sequence was cut into steps.
#include "common.cuh"

namespace {

struct ScanArgs {
    const void* qkv;          // [tokens][ld]; q of head h at q_off + h * d, k at k_off + h * d, v at v_off + h * dv
    long ld;
    int q_off, k_off, v_off;
    int heads, d, dv, dp;     // dp: d rounded up to a multiple of four
    int act;                  // 0: none, 1: silu
    const float* decay_m1;    // [heads] decay - 1
    const int32_t* cu_q;      // [B + 1]
    const int32_t* kv_len;    // [B]
    const int32_t* slots;     // [B]
    float* state;             // [slots][state_stride]
    long state_stride;
    float* out;               // [tokens][ldo] float; head h at h * dv
    long ldo;
    int ds;                   // lanes per value column (a power of two, at most 32)
};

constexpr int SCAN_TC = 16;

template <typename X>
__device__ __forceinline__ float read_act(const X* p, int act) {
    const float v = to_float(*p);
    return act == 1 ? v / (1.0f + expf(-v)) : v;
}

template <typename X, int NJ>
__global__ void __launch_bounds__(128) decay_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    const int DS = a.ds, VT = 128 / DS;
    const int dp = a.dp, dp4 = dp >> 2;
    float* sq = sm;                       // [TC][dp]
    float* sk = sq + SCAN_TC * dp;        // [TC][dp]
    float* sv = sk + SCAN_TC * dp;        // [TC][VT]
    const int b = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * VT;
    const int kv_len = a.kv_len[b];
    if (kv_len <= 0) return;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    if (q_len <= 0) return;
    const int ds = threadIdx.x % DS, vcol = threadIdx.x / DS, v = v0 + vcol;
    const bool live = v < a.dv;
    const float dm1 = a.decay_m1[h];
    float* st = a.state + (size_t)a.slots[b] * a.state_stride + ((size_t)h * a.dv + (live ? v : 0)) * dp;
    float S[NJ * 4];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int f = j * DS + ds;
        float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (live && f < dp4) s4 = *reinterpret_cast<const float4*>(st + 4 * f);
        S[4 * j] = s4.x; S[4 * j + 1] = s4.y; S[4 * j + 2] = s4.z; S[4 * j + 3] = s4.w;
    }
    pdl_wait();
    const X* base = (const X*)a.qkv;
    for (int t0 = 0; t0 < q_len; t0 += SCAN_TC) {
        const int n_tok = min(SCAN_TC, q_len - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_tok * dp; idx += 128) {
            const int tt = idx / dp, c = idx - tt * dp;
            const X* row = base + (size_t)(q0 + t0 + tt) * a.ld;
            sq[idx] = c < a.d ? read_act(row + a.q_off + h * a.d + c, a.act) : 0.0f;
            sk[idx] = c < a.d ? read_act(row + a.k_off + h * a.d + c, a.act) : 0.0f;
        }
        for (int idx = threadIdx.x; idx < n_tok * VT; idx += 128) {
            const int tt = idx / VT, c = idx - tt * VT;
            const X* row = base + (size_t)(q0 + t0 + tt) * a.ld;
            sv[idx] = v0 + c < a.dv ? read_act(row + a.v_off + h * a.dv + v0 + c, a.act) : 0.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < n_tok; ++tt) {
            const float vv = sv[tt * VT + vcol];
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * dp);
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * dp);
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int f = j * DS + ds;
                if (f < dp4) {
                    const float4 qq = q4[f], kk = k4[f];
                    S[4 * j] = fmaf(kk.x, vv, fmaf(dm1, S[4 * j], S[4 * j]));
                    S[4 * j + 1] = fmaf(kk.y, vv, fmaf(dm1, S[4 * j + 1], S[4 * j + 1]));
                    S[4 * j + 2] = fmaf(kk.z, vv, fmaf(dm1, S[4 * j + 2], S[4 * j + 2]));
                    S[4 * j + 3] = fmaf(kk.w, vv, fmaf(dm1, S[4 * j + 3], S[4 * j + 3]));
                    acc = fmaf(S[4 * j], qq.x, acc);
                    acc = fmaf(S[4 * j + 1], qq.y, acc);
                    acc = fmaf(S[4 * j + 2], qq.z, acc);
                    acc = fmaf(S[4 * j + 3], qq.w, acc);
                }
            }
            for (int o = DS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ds == 0 && live) a.out[(size_t)(q0 + t0 + tt) * a.ldo + (size_t)h * a.dv + v] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int f = j * DS + ds;
            if (f < dp4) *reinterpret_cast<float4*>(st + 4 * f) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
        }
    }
}

template <typename X>
int launch_scan(const ScanArgs& a0, int batch, cudaStream_t stream) {
    ScanArgs a = a0;
    const int dp4 = a.dp >> 2;
    int nj = 1;
    while (nj < 8 && nj * 4 < dp4) nj <<= 1;          // at most four lanes a column until a lane holds 32 states
    int ds = 1;
    while (ds * nj < dp4) ds <<= 1;
    if (ds > 32) return BROLM_ERR_TOO_LARGE;
    a.ds = ds;
    const int vt = 128 / ds;
    const size_t smem = (size_t)SCAN_TC * (2 * a.dp + vt) * sizeof(float);
    if (smem > 200 * 1024) return BROLM_ERR_TOO_LARGE;
    dim3 grid((a.dv + vt - 1) / vt, a.heads, batch);
#define BROLM_SCAN(NJ)                                                                                              \
    do {                                                                                                            \
        static size_t allowed = 0;                                                                                  \
        if (smem > 48 * 1024 && smem > allowed) {                                                                   \
            cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<X, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                        \
            if (e != cudaSuccess) return (int)e;                                                                    \
            allowed = smem;                                                                                         \
        }                                                                                                           \
        return launch_pdl(decay_scan_kernel<X, NJ>, grid, dim3(128), smem, stream, a);                              \
    } while (0)
    if (nj == 1) BROLM_SCAN(1);
    if (nj == 2) BROLM_SCAN(2);
    if (nj == 4) BROLM_SCAN(4);
    BROLM_SCAN(8);
#undef BROLM_SCAN
}

}  // namespace

// The state row of a sequence holds heads * dv * round_up(d, 4) floats for this mixer, from `state` on.
BROLM_API int brolm_decay_scan(const void* qkv, int x_dtype, long ld, int q_off, int k_off, int v_off, int heads, int d,
                               int dv, int act, const void* decay_m1, const void* cu_q, const void* kv_len,
                               const void* slots, void* state, long state_stride, void* out, long ldo, int batch,
                               cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || act < 0 || act > 1) return BROLM_ERR_BAD_SIZE;
    if (heads > 65535 || batch > 65535) return BROLM_ERR_TOO_LARGE;
    if (state_stride % 4 != 0 || ((uintptr_t)state & 15) != 0) return BROLM_ERR_ALIGNMENT;
    ScanArgs a;
    a.qkv = qkv; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.heads = heads; a.d = d; a.dv = dv; a.dp = (d + 3) & ~3; a.act = act;
    a.decay_m1 = (const float*)decay_m1;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len; a.slots = (const int32_t*)slots;
    a.state = (float*)state; a.state_stride = state_stride; a.out = (float*)out; a.ldo = ldo; a.ds = 1;
    if (x_dtype == BROLM_F32) return launch_scan<float>(a, batch, stream);
    if (x_dtype == BROLM_BF16) return launch_scan<bf16>(a, batch, stream);
    return BROLM_ERR_BAD_DTYPE;
}
