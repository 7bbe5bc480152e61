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
// time (float rows by cp.async through two buffers).  The sum over d of a column is four sums side by side in a lane,
// then folded across its DS lanes by shuffles, sixteen tokens at once.  Sequential in the tokens: the order of the
// additions of a token's result does not depend on how the sequence was cut into steps, only (through DS) on the
// launch's size.
#include <type_traits>

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
    int vec;                  // float rows: every run of q, k and v starts at a multiple of 16 bytes
    int early;                // a step of single tokens: takes part in programmatic launch
};

constexpr int SCAN_TC = 16;

template <typename X>
__device__ __forceinline__ float read_act(const X* p, int act) {
    const float v = to_float(*p);
    return act == 1 ? v / (1.0f + expf(-v)) : v;
}

__device__ __forceinline__ void scan_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Float rows are staged through two buffers filled by cp.async, the next sixteen tokens on their way while these are
// worked on, and the activation is applied in place once a buffer has landed; bfloat16 rows are converted as they
// are read, one buffer.
// DSC > 0: the lanes per column are known to the compiler and NJ * DSC float4 are exactly a row of d (no padding, no
// bounds in the inner loop, every offset a constant); DSC = 0: any d, lanes per column from the launch.
template <typename X, int NJ, int DSC>
__global__ void __launch_bounds__(128) decay_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    if (a.early) pdl_trigger();
    constexpr bool ASYNC = sizeof(X) == 4;
    constexpr bool EXACT = DSC > 0;
    const int DS = EXACT ? DSC : a.ds, VT = 128 / DS;
    const int dp = EXACT ? 4 * NJ * DSC : a.dp, dp4 = dp >> 2;
    const int stage = SCAN_TC * (2 * dp + VT);        // q [TC][dp], k [TC][dp], v [TC][VT]
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
    if (ASYNC) {
        // the padding of d to a multiple of four, and value columns beyond dv, stay zero in both buffers
        for (int i = threadIdx.x; i < 2 * stage; i += 128) sm[i] = 0.0f;
        __syncthreads();
    }
    pdl_wait();
    const X* base = (const X*)a.qkv;
    const int n_chunks = (q_len + SCAN_TC - 1) / SCAN_TC;
    const int vt_here = min(VT, a.dv - v0);

    auto issue = [&](int chunk) {                      // float rows only
        float* sq = sm + (chunk & 1) * stage;
        float* sk = sq + SCAN_TC * dp;
        float* sv = sk + SCAN_TC * dp;
        const int t0 = chunk * SCAN_TC, n_tok = min(SCAN_TC, q_len - t0);
        const float* fb = reinterpret_cast<const float*>(base);
        if (a.vec) {
            const int d4 = a.d >> 2, v4 = vt_here >> 2;
            for (int idx = threadIdx.x; idx < n_tok * d4; idx += 128) {
                const int tt = idx / d4, c = (idx - tt * d4) << 2;
                const float* row = fb + (size_t)(q0 + t0 + tt) * a.ld + h * a.d + c;
                scan_cp16(sq + tt * dp + c, row + a.q_off);
                scan_cp16(sk + tt * dp + c, row + a.k_off);
            }
            for (int idx = threadIdx.x; idx < n_tok * v4; idx += 128) {
                const int tt = idx / v4, c = (idx - tt * v4) << 2;
                scan_cp16(sv + tt * VT + c, fb + (size_t)(q0 + t0 + tt) * a.ld + a.v_off + h * a.dv + v0 + c);
            }
        } else {
            for (int idx = threadIdx.x; idx < n_tok * a.d; idx += 128) {
                const int tt = idx / a.d, c = idx - tt * a.d;
                const float* row = fb + (size_t)(q0 + t0 + tt) * a.ld + h * a.d + c;
                scan_cp4(sq + tt * dp + c, row + a.q_off);
                scan_cp4(sk + tt * dp + c, row + a.k_off);
            }
            for (int idx = threadIdx.x; idx < n_tok * vt_here; idx += 128) {
                const int tt = idx / vt_here, c = idx - tt * vt_here;
                scan_cp4(sv + tt * VT + c, fb + (size_t)(q0 + t0 + tt) * a.ld + a.v_off + h * a.dv + v0 + c);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (ASYNC) issue(0);
    for (int kc = 0; kc < n_chunks; ++kc) {
        const int t0 = kc * SCAN_TC, n_tok = min(SCAN_TC, q_len - t0);
        float* sq = sm + (ASYNC ? (kc & 1) * stage : 0);
        float* sk = sq + SCAN_TC * dp;
        float* sv = sk + SCAN_TC * dp;
        if (ASYNC) {
            if (kc + 1 < n_chunks) {
                issue(kc + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            if (a.act == 1) {
                for (int idx = threadIdx.x; idx < n_tok * (2 * dp + VT); idx += 128) {
                    // q and k rows lie back to back, the values behind them
                    const int at = idx < n_tok * dp ? idx
                                 : idx < 2 * n_tok * dp ? SCAN_TC * dp + (idx - n_tok * dp)
                                                        : 2 * SCAN_TC * dp + (idx - 2 * n_tok * dp);
                    const float x = sq[at];
                    sq[at] = x / (1.0f + expf(-x));
                }
                __syncthreads();
            }
        } else {
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
        }
        // A lane's part of every token's sum over d stays in a register of its own; only the two multiply-adds of a
        // state wait for the token before.
        float pv[SCAN_TC];
        const float4* q4 = reinterpret_cast<const float4*>(sq) + ds;
        const float4* k4 = reinterpret_cast<const float4*>(sk) + ds;
        auto tokens = [&](auto full) {
#pragma unroll
            for (int tt = 0; tt < SCAN_TC; ++tt) {
                pv[tt] = 0.0f;
                if (decltype(full)::value || tt < n_tok) {
                    const float vv = sv[tt * VT + vcol];
                    float ax = 0.0f, ay = 0.0f, az = 0.0f, aw = 0.0f;  // four sums side by side, joined in a fixed order
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        if (EXACT || j * DS + ds < dp4) {
                            const float4 qq = q4[tt * dp4 + j * DS], kk = k4[tt * dp4 + j * DS];
                            S[4 * j] = fmaf(kk.x, vv, fmaf(dm1, S[4 * j], S[4 * j]));
                            S[4 * j + 1] = fmaf(kk.y, vv, fmaf(dm1, S[4 * j + 1], S[4 * j + 1]));
                            S[4 * j + 2] = fmaf(kk.z, vv, fmaf(dm1, S[4 * j + 2], S[4 * j + 2]));
                            S[4 * j + 3] = fmaf(kk.w, vv, fmaf(dm1, S[4 * j + 3], S[4 * j + 3]));
                            ax = fmaf(S[4 * j], qq.x, ax);
                            ay = fmaf(S[4 * j + 1], qq.y, ay);
                            az = fmaf(S[4 * j + 2], qq.z, az);
                            aw = fmaf(S[4 * j + 3], qq.w, aw);
                        }
                    }
                    pv[tt] = (ax + ay) + (az + aw);
                }
            }
        };
        if (n_tok == SCAN_TC) tokens(std::true_type{});
        else tokens(std::false_type{});
        if (n_tok == 1) {                              // a single token: its sum alone crosses the lanes
            float acc = pv[0];
            for (int o = DS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ds == 0 && live) a.out[(size_t)(q0 + t0) * a.ldo + (size_t)h * a.dv + v] = acc;
            if (ASYNC) __syncthreads();
            continue;
        }
        // The sixteen sums over a column's DS lanes, all at once: at every step a lane hands half of what it holds to
        // the lane `o` away and adds what it gets to the half it keeps, so the lanes end with 16 / DS tokens each
        // (fifteen shuffles instead of four a token).  `first` is the first token a lane ends up with.
        int first = 0, held = SCAN_TC, o = DS >> 1;
#define BROLM_FOLD(H)                                                              \
        if (o > 0) {                                                               \
            const bool up = (ds & o) != 0;                                         \
            _Pragma("unroll") for (int i = 0; i < H; ++i) {                        \
                const float send = up ? pv[i] : pv[i + H];                         \
                const float keep = up ? pv[i + H] : pv[i];                         \
                pv[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);              \
            }                                                                      \
            if (up) first += H;                                                    \
            held = H;                                                              \
            o >>= 1;                                                               \
        }
        BROLM_FOLD(8)
        BROLM_FOLD(4)
        BROLM_FOLD(2)
        BROLM_FOLD(1)
#undef BROLM_FOLD
        bool writer = live;
        if (o > 0) {                                   // 32 lanes a column: two lanes hold halves of one token's sum
            pv[0] += __shfl_xor_sync(0xffffffffu, pv[0], o);
            writer = writer && (ds & 1) == 0;
        }
#pragma unroll
        float* orow = a.out + (size_t)(q0 + t0 + first) * a.ldo + (size_t)h * a.dv + v;
#pragma unroll
        for (int i = 0; i < SCAN_TC; ++i)
            if (writer && i < held && first + i < n_tok) orow[(size_t)i * a.ldo] = pv[i];
        if (ASYNC) __syncthreads();                    // the buffer is free for the chunk after the next
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int f = j * DS + ds;
            if (f < dp4) *reinterpret_cast<float4*>(st + 4 * f) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
        }
    }
}

template <typename X, int NJ, int DSC>
int launch_scan_as(const ScanArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    static size_t allowed = 0;
    if (smem > 48 * 1024 && smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<X, NJ, DSC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    // a prompt's scan runs long on few warps: plain stream order, so that its blocks spread evenly over the SMs
    if (!a.early) return launch_in_order(decay_scan_kernel<X, NJ, DSC>, grid, dim3(128), smem, stream, a);
    return launch_pdl(decay_scan_kernel<X, NJ, DSC>, grid, dim3(128), smem, stream, a);
}

template <typename X>
int launch_scan(const ScanArgs& a0, int batch, int max_q_len, cudaStream_t stream) {
    ScanArgs a = a0;
    const int dp4 = a.dp >> 2;
    const int sms = device_sm_count();
    // a lane keeps nj float4 of a column's states, ds lanes a column; fewer states a lane (more, smaller blocks)
    // while the grid would leave SMs without a block
    auto lanes = [&](int nj) { int ds = 1; while (ds * nj < dp4) ds <<= 1; return ds; };
    auto blocks = [&](int nj) { const int vt = 128 / lanes(nj); return (long long)((a.dv + vt - 1) / vt) * a.heads * batch; };
    int nj = 4;                                        // (eight would not leave the registers for sixteen tokens' sums)
    while (nj > 1 && lanes(nj) == 1 && nj / 2 >= dp4) nj >>= 1;                      // no more registers than states
    while (nj > 1 && lanes(nj / 2) <= 32 && blocks(nj) < sms) nj >>= 1;
    const int ds = lanes(nj);
    if (ds > 32) return BROLM_ERR_TOO_LARGE;
    a.ds = ds;
    a.early = max_q_len <= 1 ? 1 : 0;
    const int vt = 128 / ds;
    const bool async = sizeof(X) == 4;
    const size_t smem = (size_t)(async ? 2 : 1) * SCAN_TC * (2 * a.dp + vt) * sizeof(float);
    if (smem > 200 * 1024) return BROLM_ERR_TOO_LARGE;
    dim3 grid((a.dv + vt - 1) / vt, a.heads, batch);
    if constexpr (sizeof(X) == 4) {
        // the sizes of real layers (d = 32 .. 256 in whole lanes): everything about the row known to the compiler
        if (a.vec && nj * ds == dp4 && a.d == a.dp) {
            if (nj == 1 && ds == 8) return launch_scan_as<X, 1, 8>(a, grid, smem, stream);
            if (nj == 2 && ds == 8) return launch_scan_as<X, 2, 8>(a, grid, smem, stream);
            if (nj == 4 && ds == 8) return launch_scan_as<X, 4, 8>(a, grid, smem, stream);
            if (nj == 1 && ds == 16) return launch_scan_as<X, 1, 16>(a, grid, smem, stream);
            if (nj == 2 && ds == 16) return launch_scan_as<X, 2, 16>(a, grid, smem, stream);
            if (nj == 4 && ds == 16) return launch_scan_as<X, 4, 16>(a, grid, smem, stream);
        }
    }
    if (nj == 1) return launch_scan_as<X, 1, 0>(a, grid, smem, stream);
    if (nj == 2) return launch_scan_as<X, 2, 0>(a, grid, smem, stream);
    return launch_scan_as<X, 4, 0>(a, grid, smem, stream);
}

}  // namespace

// The state row of a sequence holds heads * dv * round_up(d, 4) floats for this mixer, from `state` on.
BROLM_API int brolm_decay_scan(const void* qkv, int x_dtype, long ld, int q_off, int k_off, int v_off, int heads, int d,
                               int dv, int act, const void* decay_m1, const void* cu_q, const void* kv_len,
                               const void* slots, void* state, long state_stride, void* out, long ldo, int batch,
                               int max_q_len, cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || act < 0 || act > 1) return BROLM_ERR_BAD_SIZE;
    if (heads > 65535 || batch > 65535) return BROLM_ERR_TOO_LARGE;
    if (state_stride % 4 != 0 || ((uintptr_t)state & 15) != 0) return BROLM_ERR_ALIGNMENT;
    ScanArgs a;
    a.qkv = qkv; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.heads = heads; a.d = d; a.dv = dv; a.dp = (d + 3) & ~3; a.act = act;
    a.decay_m1 = (const float*)decay_m1;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len; a.slots = (const int32_t*)slots;
    a.state = (float*)state; a.state_stride = state_stride; a.out = (float*)out; a.ldo = ldo; a.ds = 1; a.early = 0;
    a.vec = x_dtype == BROLM_F32 && d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 &&
            v_off % 4 == 0 && ((uintptr_t)qkv & 15) == 0;
    if (x_dtype == BROLM_F32) return launch_scan<float>(a, batch, max_q_len, stream);
    if (x_dtype == BROLM_BF16) return launch_scan<bf16>(a, batch, max_q_len, stream);
    return BROLM_ERR_BAD_DTYPE;
}
