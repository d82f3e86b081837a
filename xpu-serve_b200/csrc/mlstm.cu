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
// One CTA walks the tokens of one (sequence, head, block of up to 64 value columns) in order, eight tokens at a time through
// two buffers in shared memory (four at a time for key sizes above 128). Its first warp is the producer: it stages the next eight tokens' q and k, turns their gate
// pre-activations into (a, b) (the transcendental functions lane by lane, the maximum's recurrence by shuffles in order),
// carries n (spread over its lanes: lane l keeps n[l], n[l + 32], ...) and leaves each token's denominator
// max(|n' . q|, exp(-m')) + 1e-6. The other warps are consumers. A tile of S (a quarter of its rows x 32 columns) belongs to
// one consumer warp, lane j keeping its rows of one column in registers (a few registers a lane, and four times the warps of
// a column a lane: the recurrence is a chain of dependent operations per state entry, so what fills the pipes is warps).
// While the producer works on the next tokens, a consumer runs S' = a S + b k v on its tile and leaves its quarter of
// S'^T q for each token in shared memory; the quarters are added, divided and stored one buffer later. Each CTA has its own
// copy of n and m (the state has room for one copy per block of columns), so that no CTA waits for another. The state is read
// from the sequence's slot before the first token and written back behind the last.
#include "common.cuh"

namespace {

// (tokens a buffer: eight; four for the widest heads, whose rows fill shared memory and registers)
constexpr int RG = 4;              // row groups: consumer warps that share a block of 32 columns
constexpr int MAX_CW = 2;          // blocks of 32 value columns a CTA
constexpr int COLS = 32 * MAX_CW;

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <typename TX, int DP, int CH>
__global__ void __launch_bounds__(32 * (MAX_CW * RG + 1), DP <= 64 ? 2 : 1)
mlstm_scan_kernel(const TX* __restrict__ qkv, int64_t ld, int q_col, int k_col, int v_col, const float* __restrict__ gates,
                  int64_t ldg, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float* __restrict__ s_state,
                  float* __restrict__ nm_state, const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                  float* __restrict__ y, int H, int D, int Dv, float cap, float q_scale, const int32_t* __restrict__ chunks,
                  int mode, float* __restrict__ s_chunk, float* __restrict__ nm_chunk) {
    constexpr int DR = DP / RG;                 // rows of S a consumer lane keeps
    constexpr int NR = (DP + 31) / 32;          // entries of n a producer lane keeps
    __shared__ __align__(16) float q_s[2][CH][DP];
    __shared__ __align__(16) float k_s[2][CH][DP];
    __shared__ float part_s[2][RG][CH][COLS];
    __shared__ float a_s[2][CH], b_s[2][CH], den_s[3][CH];
    // mode 0: blockIdx.x is a sequence, walked whole from its slot's state, which takes the end state.
    // mode 1: blockIdx.x is a chunk (sequence, first token, tokens), walked from the empty state (S = 0, n = 0, m = -inf,
    //         so that its first token's m is its own input gate); its end state and the sum of its log forget gates go
    //         to s_chunk / nm_chunk [chunk] (nm rows of D + 2: n, m, sum), nothing else is written.
    // mode 2: blockIdx.x is a chunk, walked from the state that s_chunk / nm_chunk [chunk] hold (what xs_mlstm_carry
    //         left there: the sequence's state before the chunk); only y is written.
    const int head = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seq = mode == 0 ? (int)blockIdx.x : chunks[3 * blockIdx.x];
    const bool producer = warp == 0;
    const int cw = (warp - 1) / RG, rg = (warp - 1) % RG;          // consumers: block of columns, row group
    const int n_consumers = (int)blockDim.x - 32;                   // consumer threads
    const int col0 = blockIdx.z * COLS, Z = gridDim.z;
    const int col = col0 + cw * 32 + lane;
    const bool has_col = !producer && col < Dv;
    const int row0 = rg * DR;
    pdl_launch_dependents();
    const int t_begin = mode == 0 ? cu_seqlens[seq] : chunks[3 * blockIdx.x + 1];
    const int t_end = mode == 0 ? cu_seqlens[seq + 1] : t_begin + chunks[3 * blockIdx.x + 2];
    const int64_t slot = slots[seq];
    const float bi = i_bias[head], bf = f_bias[head];
    pdl_wait();
    if (t_end <= t_begin) return;
    float* s_mine = mode == 0 ? s_state + ((slot * H + head) * D) * (int64_t)Dv
                              : s_chunk + (((int64_t)blockIdx.x * H + head) * D) * (int64_t)Dv;
    float* nm_mine = mode == 0 ? nm_state + ((slot * H + head) * Z + blockIdx.z) * (int64_t)(D + 1)
                               : nm_chunk + (((int64_t)blockIdx.x * H + head) * Z + blockIdx.z) * (int64_t)(D + 2);
    const bool from_empty = mode == 1, keep_state = mode != 2, write_y = mode != 1;
    const TX* v_mine = qkv + v_col + head * Dv + (has_col ? col : 0);
    const int HV = H * Dv;
    float S[DR], n[NR];
    TX vn[CH];
    float m = 0.0f, f_sum = 0.0f;
    if (producer) {
#pragma unroll
        for (int r = 0; r < NR; ++r) n[r] = (!from_empty && lane + 32 * r < D) ? nm_mine[lane + 32 * r] : 0.0f;
        m = from_empty ? -INFINITY : nm_mine[D];
        for (int idx = lane; idx < 2 * CH * DP; idx += 32) {        // the rows' padding stays zero from here on
            (&q_s[0][0][0])[idx] = 0.0f;
            (&k_s[0][0][0])[idx] = 0.0f;
        }
        __syncwarp();
    } else {
#pragma unroll
        for (int d = 0; d < DR; ++d)
            S[d] = (!from_empty && has_col && row0 + d < D) ? s_mine[(int64_t)(row0 + d) * Dv + col] : 0.0f;
    }

    // the producer's work on the tokens [c0, c0 + nc) into buffer `buf` (denominators into `dbuf`)
    // The producer's loads run one buffer ahead of its arithmetic: `fetch` asks for eight tokens' q, k and gate
    // pre-activations (every load issued before any is used), `stage` works on what the last fetch brought and then fetches
    // the tokens after, so that memory is waited for under the consumers' work and not in the producer's own chain.
    TX qr[CH][NR], kr[CH][NR];
    float zi = 0.0f, zf = 0.0f;
    auto fetch = [&](int c0, int nc) {
        if (lane < nc) {
            const float* g = gates + (int64_t)(c0 + lane) * ldg;
            zi = g[head];
            zf = g[H + head];
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int d = lane + 32 * r;
                if (c < nc && d < D) {
                    const TX* row = qkv + (int64_t)(c0 + c) * ld + head * D + d;
                    qr[c][r] = row[q_col];
                    kr[c][r] = row[k_col];
                }
            }
        }
    };
    auto stage = [&](int c0, int nc, int buf, int dbuf) {
        const float gi = cap * tanhf((zi + bi) / cap);
        const float gf = log_sigmoid_f(cap * tanhf((zf + bf) / cap));
        float m_before = 0.0f, m_after = 0.0f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const float fc = __shfl_sync(0xffffffffu, gf, c), ic = __shfl_sync(0xffffffffu, gi, c);
            if (c < nc) {
                const float mn = fmaxf(fc + m, ic);
                if (lane == c) {
                    m_before = m;
                    m_after = mn;
                }
                m = mn;
                f_sum += fc;
            }
        }
        const float a_mine = expf(gf + m_before - m_after), b_mine = expf(gi - m_after), e_mine = expf(-m_after);
        if (lane < nc) {
            a_s[buf][lane] = a_mine;
            b_s[buf][lane] = b_mine;
        }
        // n' = a n + b k and this lane's part of n' . q, token by token on the lane's own entries; the sums over the lanes after
        float part[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            part[c] = 0.0f;
            if (c < nc) {
                const float a = __shfl_sync(0xffffffffu, a_mine, c), b = __shfl_sync(0xffffffffu, b_mine, c);
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const int d = lane + 32 * r;
                    if (d < D) {
                        const float qd = to_f32(qr[c][r]) * q_scale, kd = to_f32(kr[c][r]);
                        q_s[buf][c][d] = qd;
                        k_s[buf][c][d] = kd;
                        n[r] = fmaf(a, n[r], b * kd);
                        part[c] = fmaf(n[r], qd, part[c]);
                    }
                }
            }
        }
        if (c0 + nc < t_end) fetch(c0 + nc, min(CH, t_end - c0 - nc));      // (nc is CH here: only a sequence's last tokens are fewer)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int c = 0; c < CH; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], o);
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const float e = __shfl_sync(0xffffffffu, e_mine, c);
            if (lane == 0 && c < nc) den_s[dbuf][c] = fmaxf(fabsf(part[c]), e) + 1e-6f;
        }
    };
    auto load_values = [&](int c0, int nc) {
#pragma unroll
        for (int c = 0; c < CH; ++c)
            if (has_col && c < nc) vn[c] = v_mine[(int64_t)(c0 + c) * ld];
    };
    // the consumers' last step for the tokens [c0, c0 + nc): the row groups' quarters added, divided, stored
    auto finish = [&](int c0, int nc, int buf, int dbuf) {
        const int cols_here = min(COLS, Dv - col0);
        for (int idx = (int)threadIdx.x - 32; idx < nc * cols_here; idx += n_consumers) {
            const int c = idx / cols_here, j = idx - c * cols_here;
            const float sum = (part_s[buf][0][c][j] + part_s[buf][1][c][j]) + (part_s[buf][2][c][j] + part_s[buf][3][c][j]);
            if (write_y) y[(int64_t)(c0 + c) * HV + head * Dv + col0 + j] = sum / den_s[dbuf][c];
        }
    };

    if (producer) {
        fetch(t_begin, min(CH, t_end - t_begin));
        stage(t_begin, min(CH, t_end - t_begin), 0, 0);
    } else load_values(t_begin, min(CH, t_end - t_begin));
    __syncthreads();
    int buf = 0, chunk = 0;
    for (int c0 = t_begin; c0 < t_end; c0 += CH, buf ^= 1, ++chunk) {
        const int nc = min(CH, t_end - c0), next = c0 + CH;
        if (producer) {
            if (next < t_end) stage(next, min(CH, t_end - next), buf ^ 1, (chunk + 1) % 3);
        } else {
            TX v[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) v[c] = vn[c];
            if (next < t_end) load_values(next, min(CH, t_end - next));
            if (chunk > 0) finish(c0 - CH, CH, buf ^ 1, (chunk + 2) % 3);      // the tokens before these (their denominators: chunk - 1)
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                if (c < nc) {
                    const float a = a_s[buf][c], bv = has_col ? b_s[buf][c] * to_f32(v[c]) : 0.0f;
                    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int d = 0; d < DR; d += 4) {
                        const float4 k4 = *reinterpret_cast<const float4*>(&k_s[buf][c][row0 + d]);
                        const float4 q4 = *reinterpret_cast<const float4*>(&q_s[buf][c][row0 + d]);
                        S[d] = fmaf(a, S[d], bv * k4.x);
                        S[d + 1] = fmaf(a, S[d + 1], bv * k4.y);
                        S[d + 2] = fmaf(a, S[d + 2], bv * k4.z);
                        S[d + 3] = fmaf(a, S[d + 3], bv * k4.w);
                        sum[0] = fmaf(S[d], q4.x, sum[0]);
                        sum[1] = fmaf(S[d + 1], q4.y, sum[1]);
                        sum[2] = fmaf(S[d + 2], q4.z, sum[2]);
                        sum[3] = fmaf(S[d + 3], q4.w, sum[3]);
                    }
                    part_s[buf][rg][c][cw * 32 + lane] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
                }
            }
        }
        __syncthreads();      // the next tokens are staged, and these are done with
    }
    if (!producer) {
        const int last = t_begin + (chunk - 1) * CH;
        finish(last, t_end - last, buf ^ 1, (chunk + 2) % 3);
    }
    if (!keep_state) return;
    if (producer) {
#pragma unroll
        for (int r = 0; r < NR; ++r)
            if (lane + 32 * r < D) nm_mine[lane + 32 * r] = n[r];
        if (lane == 0) {
            nm_mine[D] = m;
            if (mode == 1) nm_mine[D + 1] = f_sum;
        }
    } else if (has_col) {
#pragma unroll
        for (int d = 0; d < DR; ++d)
            if (row0 + d < D) s_mine[(int64_t)(row0 + d) * Dv + col] = S[d];
    }
}

// Between the two passes over chunks: for every (sequence, head), chunk by chunk in order, the chunk's entry of s_chunk /
// nm_chunk (its end state from the empty state: S_loc, n_loc, m_loc, and F, the sum of its log forget gates) is replaced by
// the sequence's state before the chunk, and the slot's state moves on over the chunk:
//     m' = max(m + F, m_loc);   S' = exp(m + F - m') S + exp(m_loc - m') S_loc;   n' likewise
// which is what the token-by-token recurrence gives (its maximum unrolls to exactly this). Afterwards the slot holds the
// state behind the step's last token.
__global__ void mlstm_carry_kernel(float* __restrict__ s_state, float* __restrict__ nm_state, float* __restrict__ s_chunk,
                                   float* __restrict__ nm_chunk, const int32_t* __restrict__ first_chunk,
                                   const int32_t* __restrict__ slots, int H, int D, int Dv, int Z) {
    pdl_launch_dependents();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int64_t slot = slots[seq];
    const int j0 = first_chunk[seq], j1 = first_chunk[seq + 1];
    pdl_wait();
    float* S = s_state + ((slot * H + head) * D) * (int64_t)Dv;
    float* nm = nm_state + (slot * H + head) * (int64_t)Z * (D + 1);
    const int n_s = D * Dv, n_n = Z * D;
    float m = nm[D];                                      // (every copy holds the same m)
    for (int j = j0; j < j1; ++j) {
        float* Sl = s_chunk + (((int64_t)j * H + head) * D) * (int64_t)Dv;
        float* nml = nm_chunk + ((int64_t)j * H + head) * (int64_t)Z * (D + 2);
        const float m_loc = nml[D], F = nml[D + 1];
        const float m_new = fmaxf(m + F, m_loc);
        const float ca = expf(m + F - m_new), cb = expf(m_loc - m_new);
        __syncthreads();                                  // every thread has read the chunk's m and F
        for (int e = threadIdx.x; e < n_s; e += blockDim.x) {
            const float loc = Sl[e], run = S[e];
            Sl[e] = run;
            S[e] = ca * run + cb * loc;
        }
        for (int e = threadIdx.x; e < n_n; e += blockDim.x) {
            const int z = e / D, d = e - z * D;
            const float loc = nml[z * (D + 2) + d], run = nm[z * (D + 1) + d];
            nml[z * (D + 2) + d] = run;
            nm[z * (D + 1) + d] = ca * run + cb * loc;
        }
        __syncthreads();
        if ((int)threadIdx.x < Z) nml[threadIdx.x * (D + 2) + D] = m;       // the chunk starts from this m
        m = m_new;
    }
    if ((int)threadIdx.x < Z) nm[threadIdx.x * (D + 1) + D] = m;
}

}  // namespace

// qkv: [T, ld] rows in the activation type holding q at column q_col (H * D numbers), k at k_col and v at v_col (H * Dv).
// gates: [T, ldg] float32, the input gates' pre-activations in columns 0 .. H - 1 and the forget gates' in H .. 2 H - 1
// (without their biases). s_state: [slots, H, D, Dv] and nm_state: [slots, H, Z, D + 1] (n, then m; Z = xs_mlstm_copies(Dv))
// float32. y: [T, H * Dv] float32.
XS_API int xs_mlstm_copies(int Dv) { return (Dv + COLS - 1) / COLS; }

// With a chunk list (chunks [n_chunks, 3]: sequence, first token, tokens; first_chunk [n_seqs + 1]; s_chunk [n_chunks, H, D, Dv]
// and nm_chunk [n_chunks, H, Z, D + 2] float32 scratch) the chunks run side by side: a pass from the empty state that leaves
// each chunk's end state, a carry over each sequence's chunks in order, and a pass from each chunk's true state that writes y
// (three launches, twice the recurrence's work, a sequence's tokens no longer one after another).
XS_API int xs_mlstm_scan(const void* qkv, int64_t ld, int q_col, int k_col, int v_col, const float* gates, int64_t ldg,
                         const float* i_bias, const float* f_bias, float* s_state, float* nm_state, const int32_t* cu_seqlens,
                         const int32_t* slots, float* y, int n_seqs, int H, int D, int Dv, float cap, float q_scale, int dtype,
                         const int32_t* chunks, const int32_t* first_chunk, int n_chunks, float* s_chunk, float* nm_chunk,
                         cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(n_seqs > 0 && H > 0 && D > 0 && Dv > 0 && cap > 0.0f, "mlstm: %d sequences, %d heads of %d and %d, cap %g", n_seqs, H,
               D, Dv, (double)cap);
    XS_REQUIRE(D <= 256, "mlstm: key size %d (at most 256)", D);
    const int Z = xs_mlstm_copies(Dv);
    XS_REQUIRE(H <= 65535 && Z <= 65535, "mlstm: %d heads, %d column blocks exceed the grid limit", H, Z);
    const bool chunked = chunks != nullptr;
    XS_REQUIRE(!chunked || (first_chunk != nullptr && n_chunks > 0 && s_chunk != nullptr && nm_chunk != nullptr),
               "mlstm: a chunk list needs its index and its scratch");
    dim3 grid(chunked ? n_chunks : n_seqs, H, Z);
    int mode = chunked ? 1 : 0;
    const int blocks = Dv >= COLS ? MAX_CW : (Dv + 31) / 32;      // blocks of 32 columns in a CTA (all CTAs alike)
    const int threads = 32 * (1 + blocks * RG);
#define XS_GO(TT, DP)                                                                                                  \
    xs_launch(mlstm_scan_kernel<TT, DP, (DP <= 128 ? 8 : 4)>, grid, dim3(threads), 0, stream, (const TT*)qkv, ld, q_col, k_col, v_col, gates,  \
              ldg, i_bias, f_bias, s_state, nm_state, cu_seqlens, slots, y, H, D, Dv, cap, q_scale, chunks, mode, s_chunk, nm_chunk)
#define XS_BY_D(TT)                      \
    do {                                 \
        if (D <= 16) XS_GO(TT, 16);      \
        else if (D <= 32) XS_GO(TT, 32); \
        else if (D <= 64) XS_GO(TT, 64); \
        else if (D <= 128) XS_GO(TT, 128); \
        else XS_GO(TT, 256);             \
    } while (0)
    XS_DISPATCH_DTYPE(dtype, TT, XS_BY_D(TT));
    XS_LAUNCH_CHECK("mlstm_scan");
    if (chunked) {
        xs_launch(mlstm_carry_kernel, dim3(n_seqs, H), dim3(256), 0, stream, s_state, nm_state, s_chunk, nm_chunk, first_chunk,
                  slots, H, D, Dv, Z);
        XS_LAUNCH_CHECK("mlstm_carry");
        mode = 2;
        XS_DISPATCH_DTYPE(dtype, TT, XS_BY_D(TT));
        XS_LAUNCH_CHECK("mlstm_scan (second pass)");
    }
#undef XS_BY_D
#undef XS_GO
    return 0;
}
