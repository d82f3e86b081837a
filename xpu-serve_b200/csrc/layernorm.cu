// Residual add + layer norm without a bias, fused as the RMSNorm kernel of norm_embed.cu is:
//
//   LN(x, w, eps) = (x - mean(x)) * (mean((x - mean(x))^2) + eps)^(-1/2) * w        over the last dimension
//
// For each output row i (source row r = rows ? rows[i] : i):
//   v = h[r]                                   float32
//   if m:      b = m[r];  if post_w: b = LN(b, post_w, eps_post)
//              v = v + b;  h[r] = v            the residual sum stays float32
//   if w:      y[i] = LN(v, w, eps)            written in y's element type
// The mean is taken first and the variance from the deviations (two passes over a row that lives in
// shared memory), all in float32, whatever the element type of m and y.
#include "common.cuh"

namespace {

template <typename TM, typename TY>
__global__ void add_layernorm_kernel(float* __restrict__ h, const TM* __restrict__ m, const float* __restrict__ post_w,
                                     const float* __restrict__ w, TY* __restrict__ y, const int32_t* __restrict__ rows,
                                     int H, float eps_post, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* hr = h + r * H;
    const float inv_h = 1.0f / (float)H;
    if (m != nullptr) {
        const TM* mr = m + r * H;
        float s = 0.0f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float b = to_f32(mr[c]);
            row[c] = b;
            s += b;
        }
        if (post_w != nullptr) {
            const float mean = block_sum(s, scratch) * inv_h;
            float q = 0.0f;
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float d = row[c] - mean;
                q += d * d;
            }
            const float inv = 1.0f / sqrtf(block_sum(q, scratch) * inv_h + eps_post);
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + (row[c] - mean) * inv * post_w[c];
                row[c] = v;
                hr[c] = v;
            }
        } else {
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + row[c];
                row[c] = v;
                hr[c] = v;
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) row[c] = hr[c];
    }
    if (w == nullptr) return;
    float s = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) s += row[c];
    const float mean = block_sum(s, scratch) * inv_h;
    float q = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) * inv_h + eps);
    TY* yr = y + (int64_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) yr[c] = from_f32<TY>((row[c] - mean) * inv * w[c]);
}

// y[t, g, :] = x[t, g, :] / sqrt(mean(x[t, g, :]^2) + eps) * w[g, :]: a unit-RMS norm in `groups` equal parts of a
// row (x float32, y in the activation type). One block per (row, part).
template <typename TY>
__global__ void grouped_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TY* __restrict__ y,
                                       int width, int part, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t base = (int64_t)blockIdx.x * width + (int64_t)blockIdx.y * part;
    const float* xr = x + base;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < part; c += blockDim.x) ss += xr[c] * xr[c];
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
    const float* wr = w + (int64_t)blockIdx.y * part;
    for (int c = threadIdx.x; c < part; c += blockDim.x) y[base + c] = from_f32<TY>(xr[c] * inv * wr[c]);
}

}  // namespace

XS_API int xs_add_layernorm(float* h, const void* m, int m_dtype, const float* post_w, const float* w, void* y,
                            int y_dtype, const int32_t* rows, int n_rows, int H, float eps_post, float eps,
                            cudaStream_t stream) {
    if (n_rows == 0) return 0;
    XS_REQUIRE(n_rows > 0 && H > 0, "add_layernorm: %d rows of width %d", n_rows, H);
    XS_REQUIRE((size_t)H * 4 <= 200 * 1024, "add_layernorm: width %d does not fit shared memory (limit 51200)", H);
    XS_REQUIRE(w == nullptr || y != nullptr, "add_layernorm: a norm weight without an output");
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = H >= 4096 ? 512 : H >= 512 ? 256 : 128;
#define XS_GO(TM, TY)                                                                                          \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            cudaFuncSetAttribute(add_layernorm_kernel<TM, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 (int)smem);                                                                   \
        xs_launch(add_layernorm_kernel<TM, TY>, dim3(n_rows), dim3(threads), smem, stream, h, (const TM*)m,    \
                  post_w, w, (TY*)y, rows, H, eps_post, eps);                                                  \
    } while (0)
    XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_GO(TM, TY)));
#undef XS_GO
    XS_LAUNCH_CHECK("add_layernorm");
    return 0;
}

XS_API int xs_grouped_rmsnorm(const float* x, const float* w, void* y, int y_dtype, int rows, int width, int groups,
                              float eps, cudaStream_t stream) {
    if (rows == 0) return 0;
    XS_REQUIRE(rows > 0 && width > 0 && groups > 0 && width % groups == 0, "grouped_rmsnorm: %d rows of %d in %d parts",
               rows, width, groups);
    XS_REQUIRE(groups <= 65535, "grouped_rmsnorm: %d parts exceed the grid limit", groups);
    const int part = width / groups;
    const int threads = part >= 1024 ? 256 : 128;
    XS_DISPATCH_DTYPE(y_dtype, TY,
                      xs_launch(grouped_rmsnorm_kernel<TY>, dim3(rows, groups), dim3(threads), 0, stream, x, w, (TY*)y,
                                width, part, eps));
    XS_LAUNCH_CHECK("grouped_rmsnorm");
    return 0;
}
