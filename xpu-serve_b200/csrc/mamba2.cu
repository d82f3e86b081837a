// Mamba-2: a causal depthwise convolution with silu over [x | B | C], then per head the recurrence
//
//   dt_t = softplus(dt_raw_t + dt_bias_h)                       a_t = exp(-exp(A_log_h) * dt_t)
//   S_t  = a_t * S_(t-1) + dt_t * B_t x_t^T                     S: [N, P] float32, zero at a sequence's start
//   y_t  = S_t^T C_t + D_h * x_t                                then y_t * silu(z_t) leaves this file's kernels
//
// in_proj's row of a token is [z: inner | x: inner | B: G N | C: G N | dt: heads] (inner = heads * P); head h reads the
// B and C of group h / (heads / G). Everything of the recurrence (dt, the decay, the state, the sums) is float32
// in both precision modes; the convolution reads and writes the activation type and sums in float32.
// A sequence keeps two things between steps: the convolution's last taps - 1 inputs, [taps - 1, channels] in the
// activation type, and the state, [heads, N, P] float32.
//
// The scan comes in two forms. One CTA per (sequence, head) walks the step's tokens in order (any number of tokens:
// single tokens, short pieces). For long pieces the tokens are cut into chunks that run side by side: every chunk
// first finds what it adds to the state and by how much it decays what came before (from a zero state), a second
// kernel carries the states from chunk to chunk, and the third walks every chunk again from its true starting state
// and writes the outputs.
#include <math.h>

#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// out[t, c] = silu(bias[c] + sum_k taps[c, k] * in(t - (taps - 1 - k), c)), where inputs before the step's first token
// come from the sequence's state. proj + col0 is the [x | B | C] part of in_proj's output.
template <typename T>
__global__ void mamba2_conv_kernel(const T* __restrict__ proj, int64_t ld, int col0, const float* __restrict__ taps_w,
                                   const float* __restrict__ bias, const T* __restrict__ state,
                                   const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ cu_seqlens,
                                   const int32_t* __restrict__ slots, T* __restrict__ out, int Tn, int C, int taps) {
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= C) return;
    float w[kMaxTaps];
    for (int k = 0; k < taps; ++k) w[k] = taps_w[(int64_t)c * taps + k];
    const float b = bias != nullptr ? bias[c] : 0.0f;
    const int seq = seq_of_token[t];
    const int local = t - cu_seqlens[seq];
    const int64_t slot = slots[seq];
    pdl_wait();
    float acc = b;
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;
        float v;
        if (local - back >= 0)
            v = to_f32(proj[(int64_t)(t - back) * ld + col0 + c]);
        else      // state row taps - 1 - j holds the input j positions before the step (j = back - local)
            v = to_f32(state[(slot * (taps - 1) + (taps - 1 - (back - local))) * C + c]);
        acc = fmaf(w[k], v, acc);
    }
    out[(int64_t)t * C + c] = from_f32<T>(silu_f(acc));
}

// The same for bfloat16 with 8 channels a thread (16-byte loads and stores): C, col0 and ld multiples of 8.
__global__ void mamba2_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ proj, int64_t ld, int col0,
                                          const float* __restrict__ taps_w, const float* __restrict__ bias,
                                          const __nv_bfloat16* __restrict__ state, const int32_t* __restrict__ seq_of_token,
                                          const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                                          __nv_bfloat16* __restrict__ out, int Tn, int C, int taps) {
    pdl_launch_dependents();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int t = blockIdx.x;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int local = t - cu_seqlens[seq];
    const int64_t slot = slots[seq];
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bias != nullptr ? bias[c + j] : 0.0f;
    float wv[32];                                   // the 8 channels' taps, contiguous in memory (taps <= 4 here)
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < 2 * taps) *reinterpret_cast<float4*>(wv + 4 * i) = *reinterpret_cast<const float4*>(taps_w + (int64_t)c * taps + 4 * i);
    pdl_wait();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (k >= taps) break;
        const int back = taps - 1 - k;
        const __nv_bfloat16* src = local - back >= 0 ? proj + (int64_t)(t - back) * ld + col0 + c
                                                      : state + (slot * (taps - 1) + (taps - 1 - (back - local))) * C + c;
        const uint4 raw = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(v2[j]);
            acc[2 * j] = fmaf(wv[(2 * j) * taps + k], f.x, acc[2 * j]);
            acc[2 * j + 1] = fmaf(wv[(2 * j + 1) * taps + k], f.y, acc[2 * j + 1]);
        }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(silu_f(acc[2 * j]), silu_f(acc[2 * j + 1]));
    *reinterpret_cast<uint4*>(out + (int64_t)t * C + c) = o;
}

// After the convolution: a sequence's state becomes its last taps - 1 inputs (the step's, and the old state's where the
// step brought fewer).
template <typename T>
__global__ void mamba2_conv_state_kernel(const T* __restrict__ proj, int64_t ld, int col0, T* __restrict__ state,
                                         const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots, int C,
                                         int taps) {
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int seq = blockIdx.x;
    if (c >= C) return;
    const int t0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - t0;
    const int64_t slot = slots[seq];
    pdl_wait();
    T* st = state + slot * (taps - 1) * C + c;
    T keep[kMaxTaps];
    for (int j = 0; j < taps - 1; ++j) {
        const int local = n - (taps - 1) + j;       // the input that row j holds after the step
        keep[j] = local >= 0 ? proj[(int64_t)(t0 + local) * ld + col0 + c] : st[(int64_t)(j + n) * C];
    }
    for (int j = 0; j < taps - 1; ++j) st[(int64_t)j * C] = keep[j];
}

// The recurrence, one CTA per (head, sequence or chunk); thread p owns column p of the state (NS rows at a time in
// registers, the rest in further rounds of NS).
//   MODE 0  whole sequences: state in, outputs, state out
//   MODE 1  a chunk from a zero state: writes its end state and its total decay to scratch, no outputs
//   MODE 2  a chunk from the state that the carry kernel left in scratch: outputs (the last chunk's end state was
//           written to the sequence's state by the carry kernel)
struct ScanArgs {
    const void* xbc;           // [T, C] after the convolution: x | B | C
    const void* proj;          // in_proj's output (z and dt_raw are read from it)
    int64_t ld;
    int dt_col;
    const float* dt_bias;
    const float* a_log;
    const float* d_skip;
    float* state;              // [slots + 1, heads, N, P]
    const int32_t* cu_seqlens;
    const int32_t* slots;
    float* y;                  // [T, inner] float32: y * silu(z)
    float* chunk_state;        // [chunks, heads, N, P]
    float* chunk_decay;        // [chunks, heads]
    const int32_t* chunk_seq;  // per chunk: sequence, first token, tokens  (3 words)
    int heads, P, N, G, C, chunk;
};

constexpr int kTok = 16;       // tokens whose B, C, dt and decay are staged in shared memory at a time

template <typename T, int NS, int MODE>
__global__ void mamba2_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];     // B[kTok][N], C[kTok][N], dt[kTok], decay[kTok]
    float* sB = sm;
    float* sC = sB + kTok * a.N;
    float* sdt = sC + kTok * a.N;
    float* sda = sdt + kTok;
    float* sX = sda + kTok;                         // x[kTok][threads]
    float* sY = sX + kTok * blockDim.x;             // y[kTok][threads]: a thread's own outputs until the chunk's tokens are done
    pdl_launch_dependents();
    const int h = blockIdx.x, unit = blockIdx.y;
    const int p = threadIdx.x;
    const bool live = p < a.P;
    int seq, t0, n;
    if (MODE == 0) {
        seq = unit;
        t0 = a.cu_seqlens[seq];
        n = a.cu_seqlens[seq + 1] - t0;
    } else {
        seq = a.chunk_seq[3 * unit];
        t0 = a.chunk_seq[3 * unit + 1];
        n = a.chunk_seq[3 * unit + 2];
    }
    const int g = h / (a.heads / a.G);
    const int inner = a.heads * a.P;
    const float bias = a.dt_bias[h], rate = -expf(a.a_log[h]), dskip = a.d_skip[h];
    const T* xbc = (const T*)a.xbc;
    const T* proj = (const T*)a.proj;
    pdl_wait();
    if (n <= 0) return;
    const int rounds = (a.N + NS - 1) / NS;
    const bool vec4 = (a.N & 3) == 0;
    // rows of B, C and x in whole 16-byte pieces (bfloat16)
    const bool vec8 = (a.N & 7) == 0 && (a.P & 7) == 0 && (a.C & 7) == 0 && (reinterpret_cast<uintptr_t>(a.xbc) & 15) == 0;
    float* st = MODE == 0 ? a.state + ((int64_t)a.slots[seq] * a.heads + h) * a.N * a.P
                          : a.chunk_state + ((int64_t)unit * a.heads + h) * a.N * a.P;
    // with more than one round of state rows the outputs are summed over the rounds in the output buffer
    for (int r = 0; r < rounds; ++r) {
        const int n_lo = r * NS;
        float S[NS];
#pragma unroll
        for (int k = 0; k < NS; ++k)
            S[k] = (MODE != 1 && live && n_lo + k < a.N) ? st[(int64_t)(n_lo + k) * a.P + p] : 0.0f;
        float total = 1.0f;
        for (int c0 = 0; c0 < n; c0 += kTok) {
            const int cnt = min(kTok, n - c0);
            __syncthreads();
            bool staged = false;
            if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                if (vec8) {
                    // 16-byte loads, four of B and four of C in flight a thread before anything is stored
                    const int per_row = a.N >> 3, total8 = cnt * per_row;
                    for (int base = 0; base < total8; base += 4 * blockDim.x) {
                        uint4 rb[4], rc[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int idx = base + u * blockDim.x + threadIdx.x;
                            if (idx < total8) {
                                const int tt = idx / per_row, kk = idx - tt * per_row;
                                const T* src = xbc + (int64_t)(t0 + c0 + tt) * a.C + inner + g * a.N + kk * 8;
                                rb[u] = *reinterpret_cast<const uint4*>(src);
                                rc[u] = *reinterpret_cast<const uint4*>(src + a.G * a.N);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int idx = base + u * blockDim.x + threadIdx.x;
                            if (idx < total8) {
                                const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&rb[u]);
                                const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&rc[u]);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    *reinterpret_cast<float2*>(sB + idx * 8 + 2 * j) = __bfloat1622float2(b2[j]);
                                    *reinterpret_cast<float2*>(sC + idx * 8 + 2 * j) = __bfloat1622float2(c2[j]);
                                }
                            }
                        }
                    }
                    const int per_x = a.P >> 3, total_x = cnt * per_x;
                    for (int idx = threadIdx.x; idx < total_x; idx += blockDim.x) {
                        const int tt = idx / per_x, pp = (idx - tt * per_x) * 8;
                        const uint4 raw = *reinterpret_cast<const uint4*>(xbc + (int64_t)(t0 + c0 + tt) * a.C + h * a.P + pp);
                        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<float2*>(sX + tt * blockDim.x + pp + 2 * j) = __bfloat1622float2(x2[j]);
                    }
                    staged = true;
                }
            }
            if (!staged) {
                for (int tt = 0; tt < cnt; ++tt) {
                    const int64_t row = (int64_t)(t0 + c0 + tt) * a.C;
                    for (int k = threadIdx.x; k < a.N; k += blockDim.x) {
                        sB[tt * a.N + k] = to_f32(xbc[row + inner + g * a.N + k]);
                        sC[tt * a.N + k] = to_f32(xbc[row + inner + (a.G + g) * a.N + k]);
                    }
                    for (int pp = threadIdx.x; pp < a.P; pp += blockDim.x) sX[tt * blockDim.x + pp] = to_f32(xbc[row + h * a.P + pp]);
                }
            }
            for (int tt = threadIdx.x; tt < cnt; tt += blockDim.x) {
                const float dt = softplus_f(to_f32(proj[(int64_t)(t0 + c0 + tt) * a.ld + a.dt_col + h]) + bias);
                sdt[tt] = dt;
                sda[tt] = expf(rate * dt);
            }
            __syncthreads();
            if (!live) continue;
            // the recurrence over the staged tokens reads shared memory only; outputs wait in sY
            for (int tt = 0; tt < cnt; ++tt) {
                const float x = sX[tt * blockDim.x + p];
                const float da = sda[tt], dtx = sdt[tt] * x;
                const float* Bt = sB + tt * a.N + n_lo;
                const float* Ct = sC + tt * a.N + n_lo;
                float y = 0.0f;
                if (vec4) {         // N a multiple of 4: B and C four at a time, four partial sums (a short dependency chain)
                    float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;
#pragma unroll
                    for (int k = 0; k < NS; k += 4) {
                        if (n_lo + k < a.N) {
                            const float4 b4 = *reinterpret_cast<const float4*>(Bt + k);
                            S[k] = fmaf(da, S[k], dtx * b4.x);
                            S[k + 1] = fmaf(da, S[k + 1], dtx * b4.y);
                            S[k + 2] = fmaf(da, S[k + 2], dtx * b4.z);
                            S[k + 3] = fmaf(da, S[k + 3], dtx * b4.w);
                            if (MODE != 1) {        // a chunk's first pass wants its end state only
                                const float4 c4 = *reinterpret_cast<const float4*>(Ct + k);
                                y0 = fmaf(S[k], c4.x, y0);
                                y1 = fmaf(S[k + 1], c4.y, y1);
                                y2 = fmaf(S[k + 2], c4.z, y2);
                                y3 = fmaf(S[k + 3], c4.w, y3);
                            }
                        }
                    }
                    y = (y0 + y1) + (y2 + y3);
                } else {
#pragma unroll
                    for (int k = 0; k < NS; ++k) {
                        if (n_lo + k < a.N) {
                            S[k] = fmaf(da, S[k], dtx * Bt[k]);
                            y = fmaf(S[k], Ct[k], y);
                        }
                    }
                }
                total *= da;
                sY[tt * blockDim.x + p] = y;
            }
            if (MODE != 1) {
                // the gate's loads of the staged tokens are independent of one another: four in flight at a time
                for (int t4 = 0; t4 < cnt; t4 += 4) {
                    float zv[4];
                    const bool last = rounds == 1 || r == rounds - 1;
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        zv[u] = (last && t4 + u < cnt) ? to_f32(proj[(int64_t)(t0 + c0 + t4 + u) * a.ld + h * a.P + p]) : 0.0f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int tt = t4 + u;
                        if (tt >= cnt) break;
                        const float x = sX[tt * blockDim.x + p], y = sY[tt * blockDim.x + p];
                        float* yo = a.y + (int64_t)(t0 + c0 + tt) * inner + h * a.P + p;
                        if (rounds == 1) *yo = fmaf(dskip, x, y) * silu_f(zv[u]);
                        else if (r == 0) *yo = y;
                        else if (!last) *yo += y;
                        else *yo = fmaf(dskip, x, *yo + y) * silu_f(zv[u]);
                    }
                }
            }
        }
        if (MODE != 2 && live) {
#pragma unroll
            for (int k = 0; k < NS; ++k)
                if (n_lo + k < a.N) st[(int64_t)(n_lo + k) * a.P + p] = S[k];
        }
        if (MODE == 1 && r == 0 && p == 0) a.chunk_decay[(int64_t)unit * a.heads + h] = total;
    }
}

// Carries the state from chunk to chunk: for each (sequence, head), S = the sequence's state; for its chunks in order,
// the chunk's scratch state is replaced by S (where the chunk starts) and S = decay * S + (what the chunk added). The
// final S is the sequence's state after the step. first_chunk: [n_seqs + 1].
__global__ void mamba2_carry_kernel(float* __restrict__ state, float* __restrict__ chunk_state,
                                    const float* __restrict__ chunk_decay, const int32_t* __restrict__ first_chunk,
                                    const int32_t* __restrict__ slots, int heads, int64_t NP) {
    pdl_launch_dependents();
    const int h = blockIdx.x, seq = blockIdx.y;
    const int c_lo = first_chunk[seq], c_hi = first_chunk[seq + 1];
    float* st = state + ((int64_t)slots[seq] * heads + h) * NP;
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.z * blockDim.x + threadIdx.x; i < NP; i += (int64_t)gridDim.z * blockDim.x) {
        float S = st[i];
        for (int c = c_lo; c < c_hi; ++c) {
            float* cs = chunk_state + ((int64_t)c * heads + h) * NP + i;
            const float added = *cs;
            *cs = S;
            S = fmaf(chunk_decay[(int64_t)c * heads + h], S, added);
        }
        st[i] = S;
    }
}

template <typename T, int MODE>
int launch_scan(const ScanArgs& a, int units, cudaStream_t stream) {
    const int threads = ((a.P + 31) / 32) * 32;
    const size_t smem = (size_t)(2 * kTok * a.N + 2 * kTok + 2 * kTok * threads) * sizeof(float);
    if (smem > 48 * 1024) {
        xs_set_error("mamba2_scan: a state of %d rows does not fit shared memory", a.N);
        return -1;
    }
    const dim3 grid(a.heads, units);
    if (a.N <= 16)
        return (int)xs_launch(mamba2_scan_kernel<T, 16, MODE>, grid, dim3(threads), smem, stream, a);
    if (a.N <= 32)
        return (int)xs_launch(mamba2_scan_kernel<T, 32, MODE>, grid, dim3(threads), smem, stream, a);
    if (a.N <= 64)
        return (int)xs_launch(mamba2_scan_kernel<T, 64, MODE>, grid, dim3(threads), smem, stream, a);
    return (int)xs_launch(mamba2_scan_kernel<T, 128, MODE>, grid, dim3(threads), smem, stream, a);
}

}  // namespace

XS_API int xs_mamba2_conv(const void* proj, int64_t ld, int col0, const float* taps_w, const float* bias, void* state,
                          const int32_t* seq_of_token, const int32_t* cu_seqlens, const int32_t* slots, void* out, int T,
                          int n_seqs, int C, int taps, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(C > 0 && taps >= 1 && taps <= kMaxTaps, "mamba2_conv: %d channels, %d taps (at most %d)", C, taps, kMaxTaps);
    XS_REQUIRE(n_seqs > 0 && C <= 65535 * 128, "mamba2_conv: %d tokens in %d sequences, %d channels", T, n_seqs, C);
    const int tiles = ceil_div_i(C, 128);
    if (dtype == XS_BF16 && taps <= 4 && (uintptr_t)taps_w % 16 == 0 && C % 8 == 0 && col0 % 8 == 0 && ld % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)state % 16 == 0 &&
        (uintptr_t)out % 16 == 0) {
        xs_launch(mamba2_conv_bf16x8_kernel, dim3(T, ceil_div_i(C / 8, 128)), dim3(128), 0, stream, (const __nv_bfloat16*)proj, ld,
                  col0, taps_w, bias, (const __nv_bfloat16*)state, seq_of_token, cu_seqlens, slots, (__nv_bfloat16*)out, T, C, taps);
    } else {
        XS_DISPATCH_DTYPE(dtype, TT,
                          xs_launch(mamba2_conv_kernel<TT>, dim3(T, tiles), dim3(128), 0, stream, (const TT*)proj, ld, col0,
                                    taps_w, bias, (const TT*)state, seq_of_token, cu_seqlens, slots, (TT*)out, T, C, taps));
    }
    XS_LAUNCH_CHECK("mamba2_conv");
    if (taps > 1) {
        XS_DISPATCH_DTYPE(dtype, TT,
                          xs_launch(mamba2_conv_state_kernel<TT>, dim3(n_seqs, tiles), dim3(128), 0, stream,
                                    (const TT*)proj, ld, col0, (TT*)state, cu_seqlens, slots, C, taps));
        XS_LAUNCH_CHECK("mamba2_conv_state");
    }
    return 0;
}

// Whole sequences, one CTA per (head, sequence).
XS_API int xs_mamba2_scan(const void* xbc, const void* proj, int64_t ld, int dt_col, const float* dt_bias,
                          const float* a_log, const float* d_skip, float* state, const int32_t* cu_seqlens,
                          const int32_t* slots, float* y, int n_seqs, int heads, int P, int N, int G, int dtype,
                          cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(heads > 0 && P > 0 && P <= 1024 && N > 0 && G > 0 && heads % G == 0, "mamba2_scan: %d heads of %d, state %d, %d groups",
               heads, P, N, G);
    XS_REQUIRE(n_seqs <= 65535, "mamba2_scan: %d sequences exceed the grid limit", n_seqs);
    ScanArgs a = {xbc, proj, ld, dt_col, dt_bias, a_log, d_skip, state, cu_seqlens, slots, y, nullptr, nullptr, nullptr,
                  heads, P, N, G, heads * P + 2 * G * N, 0};
    XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT, 0>(a, n_seqs, stream));
    XS_LAUNCH_CHECK("mamba2_scan");
    return 0;
}

// Long pieces in chunks: chunk_seq [chunks, 3] (sequence, first token, tokens) and first_chunk [n_seqs + 1] come
// from the host, which knows the step's lengths; chunk_state [chunks, heads, N, P] and chunk_decay [chunks, heads] are scratch.
XS_API int xs_mamba2_scan_chunked(const void* xbc, const void* proj, int64_t ld, int dt_col, const float* dt_bias,
                                  const float* a_log, const float* d_skip, float* state, const int32_t* cu_seqlens,
                                  const int32_t* slots, float* y, float* chunk_state, float* chunk_decay,
                                  const int32_t* chunk_seq, const int32_t* first_chunk, int chunks, int n_seqs, int heads,
                                  int P, int N, int G, int dtype, cudaStream_t stream) {
    if (n_seqs == 0 || chunks == 0) return 0;
    XS_REQUIRE(heads > 0 && P > 0 && P <= 1024 && N > 0 && G > 0 && heads % G == 0, "mamba2_scan: %d heads of %d, state %d, %d groups",
               heads, P, N, G);
    XS_REQUIRE(n_seqs <= 65535 && chunks <= 65535, "mamba2_scan: %d sequences in %d chunks exceed the grid limit", n_seqs, chunks);
    ScanArgs a = {xbc, proj, ld, dt_col, dt_bias, a_log, d_skip, state, cu_seqlens, slots, y, chunk_state, chunk_decay,
                  chunk_seq, heads, P, N, G, heads * P + 2 * G * N, 0};
    XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT, 1>(a, chunks, stream));
    XS_LAUNCH_CHECK("mamba2_scan (chunk states)");
    xs_launch(mamba2_carry_kernel, dim3(heads, n_seqs, ceil_div_i((int64_t)N * P, 256) < 64 ? ceil_div_i((int64_t)N * P, 256) : 64),
              dim3(256), 0, stream, state, chunk_state, chunk_decay, first_chunk, slots, heads, (int64_t)N * P);
    XS_LAUNCH_CHECK("mamba2_scan (carry)");
    XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT, 2>(a, chunks, stream));
    XS_LAUNCH_CHECK("mamba2_scan (outputs)");
    return 0;
}
