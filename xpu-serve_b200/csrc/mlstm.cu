// The matrix-memory recurrence of xLSTM (mLSTM), one head at a time, in float32.
//
// Per head: a state S [D, Dv], a vector n [D] and a running maximum m (all zero at a sequence's start).
// For token t with query q (already times D^-1/2 here), key k, value v and the two gate pre-activations zi, zf:
//     i = cap tanh((zi + bi) / cap)                    log of the input gate
//     f = logsigmoid(cap tanh((zf + bf) / cap))        log of the forget gate
//     m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m')
//     S' = a S + b k v^T;  n' = a n + b k
//     o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
// The gates, the maximum, the state and every sum are float32 whatever the element type of q, k and v.
//
// One CTA walks the tokens of one (sequence, head) in order. Thread j keeps column j of S in registers, the thread behind the
// last column keeps n (the column that a value of 1 would make), so S'^T q and n' . q are the same loop. Heads of more than
// 224 value columns are cut over several CTAs, each with its own copy of n and m (the state has room for the copies). Tokens are staged in shared
// memory eight at a time; the first warp turns their pre-activations into (a, b, exp(-m')): the transcendental functions
// lane by lane, the maximum's recurrence by shuffles in order. The state is read from the sequence's slot before the
// first token and written back behind the last.
#include "common.cuh"

namespace {

constexpr int CH = 8;

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <typename TX, int DP>
__global__ void __launch_bounds__(256)
mlstm_scan_kernel(const TX* __restrict__ qkv, int64_t ld, int q_col, int k_col, int v_col, const float* __restrict__ gates,
                  int64_t ldg, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float* __restrict__ s_state,
                  float* __restrict__ nm_state, const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                  float* __restrict__ y, int H, int D, int Dv, int cols, float cap, float q_scale) {
    extern __shared__ float sm[];
    float* q_s = sm;                     // [CH, D]
    float* k_s = q_s + CH * D;           // [CH, D]
    float* v_s = k_s + CH * D;           // [CH, cols]
    float* a_s = v_s + CH * cols;          // [CH]
    float* b_s = a_s + CH;
    float* e_s = b_s + CH;               // exp(-m')
    float* nq_s = e_s + CH;              // n' . q
    __shared__ float m_last;
    // this CTA's value columns: col0 .. col0 + nv - 1 (thread j < nv), and its own copy of n (thread nv)
    const int seq = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int col0 = blockIdx.z * cols, nv = min(cols, Dv - col0), Z = gridDim.z;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    const int t_begin = cu_seqlens[seq], t_end = cu_seqlens[seq + 1];
    const int64_t slot = slots[seq];
    const float bi = i_bias[head], bf = f_bias[head];
    pdl_wait();
    if (t_end <= t_begin) return;
    float* s_mine = s_state + ((slot * H + head) * D) * (int64_t)Dv;
    float* nm_mine = nm_state + ((slot * H + head) * Z + blockIdx.z) * (int64_t)(D + 1);
    float S[DP];
#pragma unroll
    for (int d = 0; d < DP; ++d) S[d] = 0.0f;
    if (j < nv) {
#pragma unroll
        for (int d = 0; d < DP; ++d)
            if (d < D) S[d] = s_mine[(int64_t)d * Dv + col0 + j];
    } else if (j == nv) {
#pragma unroll
        for (int d = 0; d < DP; ++d)
            if (d < D) S[d] = nm_mine[d];
    }
    float m = nm_mine[D];            // (only the first warp follows it)
    const int HV = H * Dv;
    for (int c0 = t_begin; c0 < t_end; c0 += CH) {
        const int nc = min(CH, t_end - c0);
        for (int idx = threadIdx.x; idx < nc * D; idx += blockDim.x) {
            const int c = idx / D, d = idx - c * D;
            const TX* row = qkv + (int64_t)(c0 + c) * ld + head * D + d;
            q_s[idx] = to_f32(row[q_col]) * q_scale;
            k_s[idx] = to_f32(row[k_col]);
        }
        for (int idx = threadIdx.x; idx < nc * nv; idx += blockDim.x) {
            const int c = idx / nv, d = idx - c * nv;
            v_s[c * cols + d] = to_f32(qkv[(int64_t)(c0 + c) * ld + v_col + head * Dv + col0 + d]);
        }
        if (threadIdx.x < 32) {
            float gi = 0.0f, gf = 0.0f;
            if (lane < nc) {
                const float* g = gates + (int64_t)(c0 + lane) * ldg;
                gi = cap * tanhf((g[head] + bi) / cap);
                gf = log_sigmoid_f(cap * tanhf((g[H + head] + bf) / cap));
            }
            float m_before = 0.0f, m_after = 0.0f;
            for (int c = 0; c < nc; ++c) {
                const float fc = __shfl_sync(0xffffffffu, gf, c), ic = __shfl_sync(0xffffffffu, gi, c);
                const float mn = fmaxf(fc + m, ic);
                if (lane == c) {
                    m_before = m;
                    m_after = mn;
                }
                m = mn;
            }
            if (lane < nc) {
                a_s[lane] = expf(gf + m_before - m_after);
                b_s[lane] = expf(gi - m_after);
                e_s[lane] = expf(-m_after);
            }
            if (lane == 0) m_last = m;
        }
        __syncthreads();
        float acc[CH];
        const bool is_n = j == nv;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            acc[c] = 0.0f;
            if (c < nc) {
                const float a = a_s[c];
                const float bv = b_s[c] * (is_n ? 1.0f : (j < nv ? v_s[c * cols + j] : 0.0f));
                const float* kc = k_s + c * D;
                const float* qc = q_s + c * D;
                float sum = 0.0f;
#pragma unroll
                for (int d = 0; d < DP; ++d) {
                    if (d < D) {
                        S[d] = fmaf(a, S[d], bv * kc[d]);
                        sum = fmaf(S[d], qc[d], sum);
                    }
                }
                acc[c] = sum;
                if (is_n) nq_s[c] = sum;
            }
        }
        __syncthreads();
        if (j < nv) {
#pragma unroll
            for (int c = 0; c < CH; ++c)
                if (c < nc)
                    y[(int64_t)(c0 + c) * HV + head * Dv + col0 + j] = acc[c] / (fmaxf(fabsf(nq_s[c]), e_s[c]) + 1e-6f);
        }
        __syncthreads();      // the next tokens overwrite what was just read
    }
    if (j < nv) {
#pragma unroll
        for (int d = 0; d < DP; ++d)
            if (d < D) s_mine[(int64_t)d * Dv + col0 + j] = S[d];
    } else if (j == nv) {
#pragma unroll
        for (int d = 0; d < DP; ++d)
            if (d < D) nm_mine[d] = S[d];
        nm_mine[D] = m_last;
    }
}

}  // namespace

// qkv: [T, ld] rows in the activation type holding q at column q_col (H * D numbers), k at k_col and v at v_col (H * Dv).
// gates: [T, ldg] float32, the input gates' pre-activations in columns 0 .. H - 1 and the forget gates' in H .. 2 H - 1
// (without their biases). s_state: [slots, H, D, Dv] and nm_state: [slots, H, Z, D + 1] (n, then m; Z = xs_mlstm_copies(Dv))
// float32. y: [T, H * Dv] float32.
XS_API int xs_mlstm_copies(int Dv) { return (Dv + 223) / 224; }

XS_API int xs_mlstm_scan(const void* qkv, int64_t ld, int q_col, int k_col, int v_col, const float* gates, int64_t ldg,
                         const float* i_bias, const float* f_bias, float* s_state, float* nm_state, const int32_t* cu_seqlens,
                         const int32_t* slots, float* y, int n_seqs, int H, int D, int Dv, float cap, float q_scale, int dtype,
                         cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(n_seqs > 0 && H > 0 && D > 0 && Dv > 0 && cap > 0.0f, "mlstm: %d sequences, %d heads of %d and %d, cap %g", n_seqs, H,
               D, Dv, (double)cap);
    XS_REQUIRE(D <= 128, "mlstm: key size %d (at most 128)", D);
    const int Z = xs_mlstm_copies(Dv);
    const int cols = (Dv + Z - 1) / Z;
    XS_REQUIRE(H <= 65535 && Z <= 65535, "mlstm: %d heads, %d column blocks exceed the grid limit", H, Z);
    const int threads = ((cols + 1 + 31) / 32) * 32;
    const size_t smem = (size_t)(CH * (2 * D + cols) + 4 * CH) * sizeof(float);
    const dim3 grid(n_seqs, H, Z);
#define XS_GO(TT, DP)                                                                                                      \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(mlstm_scan_kernel<TT, DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        xs_launch(mlstm_scan_kernel<TT, DP>, grid, dim3(threads), smem, stream, (const TT*)qkv, ld, q_col, k_col, v_col,  \
                  gates, ldg, i_bias, f_bias, s_state, nm_state, cu_seqlens, slots, y, H, D, Dv, cols, cap, q_scale);      \
    } while (0)
#define XS_BY_D(TT)                      \
    do {                                 \
        if (D <= 16) XS_GO(TT, 16);      \
        else if (D <= 32) XS_GO(TT, 32); \
        else if (D <= 64) XS_GO(TT, 64); \
        else XS_GO(TT, 128);             \
    } while (0)
    XS_DISPATCH_DTYPE(dtype, TT, XS_BY_D(TT));
#undef XS_BY_D
#undef XS_GO
    XS_LAUNCH_CHECK("mlstm_scan");
    return 0;
}
