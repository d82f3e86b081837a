// Latent attention: every head's keys and values are products of ONE cached vector per position.
//
// A position's cache row is [c (R numbers: the down-projection's first R outputs, unit RMS times a weight) |
// k_rot (Dr numbers, rotated by position)], one row for all heads: [pages, 1, 1, page_size, R + Dr].
// Head h's key is [Wuk_h c | k_rot] and its value Wuv_h c. Because both are linear in c, the products with the
// per-head matrices move to the query's and the output's side:
//
//   score(i, j) = scale * ((Wuk_h^T q_h[:Dn]) . c_j + rot(q_h[Dn:]) . k_rot_j)          q~ = Wuk_h^T q_h[:Dn], R numbers
//   out_h(i)    = Wuv_h (sum_j p(i, j) c_j)                                             o~ = sum_j p c_j,     R numbers
//
// so attention itself runs over the cache rows alone, as multi-query attention with keys of R + Dr and values of R
// channels (the values ARE the keys' first R channels). The two small per-head products are batched matrix products
// outside this file. Visible keys: j <= i, and i - j < window when window > 0. With `sink` a learned number per
// head joins the softmax's denominator (exp(sink_h), once, with no key and no value). With `gate` a head's output is
// multiplied by sigmoid(gate[t, h]). Scores, the softmax and the sums are float32.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kMaxRank = 512;     // R of the generic kernel: 16 accumulators a lane

// One block per token: the latent's norm, the rotation of the shared key part and of every head's rotated query part,
// and the cache write. down: [T, R + Dr]; q: [T, H, Dn + Dr]; q_rot: [T, H, Dr]. The rotation couples channel i with
// i + dims/2 for i < dims/2 (dims <= Dr; channels from dims on pass); table: [positions, dims/2] (cos, sin).
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ down, int64_t ld_down, const T* __restrict__ q, int64_t ld_q,
                                      const float* __restrict__ norm_w, const float2* __restrict__ table,
                                      const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_of_token,
                                      const int32_t* __restrict__ page_table, int P, T* __restrict__ pool,
                                      T* __restrict__ q_rot, int H, int Dn, int Dr, int R, int dims, int page_size,
                                      float eps, int write_kv) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = dims / 2;
    const float2* cs = table != nullptr ? table + (int64_t)pos * half : nullptr;
    pdl_wait();
    if (write_kv) {
        const T* dr = down + (int64_t)t * ld_down;
        float ss = 0.0f;
        for (int c = threadIdx.x; c < R; c += blockDim.x) {
            const float v = to_f32(dr[c]);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
        const int page = page_table[(int64_t)seq_of_token[t] * P + pos / page_size];
        T* row = pool + ((int64_t)page * page_size + pos % page_size) * (R + Dr);
        for (int c = threadIdx.x; c < R; c += blockDim.x) row[c] = from_f32<T>(to_f32(dr[c]) * inv * norm_w[c]);
        for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
            float v = to_f32(dr[R + i]);
            if (cs != nullptr && i < dims) {
                const bool low = i < half;
                const float2 a = cs[low ? i : i - half];
                const float o = to_f32(dr[R + (low ? i + half : i - half)]);
                v = low ? v * a.x - o * a.y : v * a.x + o * a.y;
            }
            row[R + i] = from_f32<T>(v);
        }
    }
    for (int idx = threadIdx.x; idx < H * Dr; idx += blockDim.x) {
        const int h = idx / Dr, i = idx - h * Dr;
        const T* src = q + (int64_t)t * ld_q + (int64_t)h * (Dn + Dr) + Dn;
        float v = to_f32(src[i]);
        if (cs != nullptr && i < dims) {
            const bool low = i < half;
            const float2 a = cs[low ? i : i - half];
            const float o = to_f32(src[low ? i + half : i - half]);
            v = low ? v * a.x - o * a.y : v * a.x + o * a.y;
        }
        q_rot[((int64_t)t * H + h) * Dr + i] = from_f32<T>(v);
    }
}

// One warp per (token, head). Scores with lanes over keys, weighted sums with lanes over channels.
template <typename T>
__global__ void latent_attention_generic_kernel(const T* __restrict__ q_lat, int64_t qs_t, int64_t qs_h,
                                                const T* __restrict__ q_rot, const T* __restrict__ pool,
                                                const int32_t* __restrict__ page_table, int P,
                                                const int32_t* __restrict__ seq_of_token,
                                                const int32_t* __restrict__ positions, const T* __restrict__ gate,
                                                int64_t ld_gate, const float* __restrict__ sink, T* __restrict__ out,
                                                int64_t os_t, int64_t os_h, int Tn, int H, int R, int Dr, int page_size,
                                                float scale, int window) {
    extern __shared__ float q_sm[];   // [warps][R + Dr]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (int64_t)Tn * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int pos = positions[t];
    const int32_t* table = page_table + (int64_t)seq_of_token[t] * P;
    const int W = R + Dr;
    float* qs = q_sm + warp * W;
    const T* ql = q_lat + (int64_t)t * qs_t + (int64_t)h * qs_h;
    const T* qr = q_rot + ((int64_t)t * H + h) * Dr;
    for (int d = lane; d < R; d += 32) qs[d] = to_f32(ql[d]) * scale;
    for (int d = lane; d < Dr; d += 32) qs[R + d] = to_f32(qr[d]) * scale;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.0f;
    if (sink != nullptr) {      // the denominator starts with exp(sink - m) = 1 at m = sink
        m = sink[h];
        l = 1.0f;
    }
    float acc[kMaxRank / 32];
#pragma unroll
    for (int u = 0; u < kMaxRank / 32; ++u) acc[u] = 0.0f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = table[j / page_size];
            const T* kr = pool + ((int64_t)page * page_size + j % page_size) * W;
            float dot = 0.0f;
            for (int d = 0; d < W; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = j <= pos ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);   // 0 on the first block without a sink (m = -inf)
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int u = 0; u < kMaxRank / 32; ++u) acc[u] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int jk = j0 + jj;
            const int page = table[jk / page_size];
            const T* vr = pool + ((int64_t)page * page_size + jk % page_size) * W;
#pragma unroll
            for (int u = 0; u < kMaxRank / 32; ++u) {
                const int d = lane + 32 * u;
                if (d < R) acc[u] = fmaf(pj, to_f32(vr[d]), acc[u]);
            }
        }
    }
    float g = 1.0f;
    if (gate != nullptr) g = 1.0f / (1.0f + expf(-to_f32(gate[(int64_t)t * ld_gate + h])));
    const float norm = g / l;
    T* orow = out + (int64_t)t * os_t + (int64_t)h * os_h;
#pragma unroll
    for (int u = 0; u < kMaxRank / 32; ++u) {
        const int d = lane + 32 * u;
        if (d < R) orow[d] = from_f32<T>(acc[u] * norm);
    }
}

// out[b][M, N] = x[b][M, K] . w[b][N, K]^T for b < batch, every operand with a row stride and a batch stride: the
// per-head products on either side of the attention (CUDA-core FMAs, sums in an order that depends on K alone).
constexpr int BM = 64, BN = 64, BK = 32;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_batched_kernel(const T* __restrict__ x, int64_t ldx, int64_t sx, const T* __restrict__ w, int64_t ldw, int64_t sw,
                    T* __restrict__ out, int64_t ldo, int64_t so, int M, int N, int K) {
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z;
    x += (int64_t)b * sx;
    w += (int64_t)b * sw;
    out += (int64_t)b * so;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
            const int r = idx >> 5, k = idx & 31;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            xs[k][r] = (gm < M && gk < K) ? to_f32(x[(int64_t)gm * ldx + gk]) : 0.0f;
            ws[k][r] = (gn < N && gk < K) ? to_f32(w[(int64_t)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], bb[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) out[(int64_t)gm * ldo + gn] = from_f32<T>(acc[i][j]);
        }
    }
}

}  // namespace

XS_API int xs_latent_prepare(const void* down, int64_t ld_down, const void* q, int64_t ld_q, const float* norm_w,
                             const float* table, const int32_t* positions, const int32_t* seq_of_token,
                             const int32_t* page_table, int P, void* pool, void* q_rot, int T, int H, int Dn, int Dr, int R,
                             int dims, int page_size, float eps, int write_kv, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && Dn > 0 && Dr > 0 && R > 0, "latent_prepare: %d heads of %d + %d, rank %d", H, Dn, Dr, R);
    XS_REQUIRE(dims >= 0 && dims % 2 == 0 && dims <= Dr, "latent_prepare: %d rotated channels of %d", dims, Dr);
    XS_REQUIRE(!write_kv || (pool != nullptr && page_table != nullptr && P > 0), "latent_prepare: no cache to write to");
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(latent_prepare_kernel<TT>, dim3(T), dim3(128), 0, stream, (const TT*)down, ld_down,
                                (const TT*)q, ld_q, norm_w, (const float2*)table, positions, seq_of_token, page_table, P,
                                (TT*)pool, (TT*)q_rot, H, Dn, Dr, R, dims, page_size, eps, write_kv));
    XS_LAUNCH_CHECK("latent_prepare");
    return 0;
}

XS_API int xs_latent_attention_generic(const void* q_lat, int64_t qs_t, int64_t qs_h, const void* q_rot, const void* pool,
                                       const int32_t* page_table, int P, const int32_t* seq_of_token,
                                       const int32_t* positions, const void* gate, int64_t ld_gate, const float* sink,
                                       void* out, int64_t os_t, int64_t os_h, int T, int H, int R, int Dr, int page_size,
                                       float scale, int window, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && R > 0 && R <= kMaxRank && Dr > 0, "latent attention: %d heads, rank %d (at most %d), %d rotated", H, R,
               kMaxRank, Dr);
    XS_REQUIRE(window >= 0 && page_size > 0 && P > 0, "latent attention: window %d, page size %d, %d pages", window, page_size, P);
    const int warps = 4;
    const int blocks = ceil_div_i((int64_t)T * H, warps);
    const size_t smem = (size_t)warps * (R + Dr) * sizeof(float);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(latent_attention_generic_kernel<TT>, dim3(blocks), dim3(warps * 32), smem, stream,
                                (const TT*)q_lat, qs_t, qs_h, (const TT*)q_rot, (const TT*)pool, page_table, P, seq_of_token,
                                positions, (const TT*)gate, ld_gate, sink, (TT*)out, os_t, os_h, T, H, R, Dr, page_size,
                                scale, window));
    XS_LAUNCH_CHECK("latent_attention_generic");
    return 0;
}

XS_API int xs_gemm_batched(const void* x, int64_t ldx, int64_t sx, const void* w, int64_t ldw, int64_t sw, void* out,
                           int64_t ldo, int64_t so, int batch, int M, int N, int K, int dtype, cudaStream_t stream) {
    if (M == 0 || N == 0 || batch == 0) return 0;
    XS_REQUIRE(batch > 0 && batch <= 65535 && M > 0 && N > 0 && K > 0, "gemm_batched: %d x (%d x %d x %d)", batch, M, N, K);
    XS_REQUIRE(ldx >= K && ldw >= K && ldo >= N, "gemm_batched: a row stride is shorter than its row");
    const dim3 grid(ceil_div_i(N, BN), ceil_div_i(M, BM), batch);
    XS_REQUIRE(grid.y <= 65535, "gemm_batched: %d rows exceed the grid limit", M);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(gemm_batched_kernel<TT>, grid, dim3(256), 0, stream, (const TT*)x, ldx, sx, (const TT*)w,
                                ldw, sw, (TT*)out, ldo, so, M, N, K));
    XS_LAUNCH_CHECK("gemm_batched");
    return 0;
}
