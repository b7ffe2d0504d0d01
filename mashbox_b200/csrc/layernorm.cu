// Layer norm (mean and variance over a row, a weight and a bias per channel) on sublayer OUTPUTS and on the stream.
//
//   ln_add      x += ln(s1 y1 + s2 y2) w + b, row by row: x (N, D) is the float32 residual stream, y1 (and optionally y2)
//               what a sublayer returned, in the activation dtype.  The sublayers of such a block read the stream as
//               it is, so the kernel also leaves the new stream in the activation dtype (`copy`) for the next product.
//   layer_norm  out = ln(x[rows]) w + b in the activation dtype (the norm before the output head, on the wanted rows)
//   to_rows     out = x in the activation dtype (the stream as the embedding left it)
//
// mean = sum / D; variance = mean of the squared deviations from it (a second pass over the row, which sits in shared
// memory); eps inside the root.  All arithmetic float32; every reduction has a fixed shape, so a row's result does not
// depend on the batch.
#include "common.cuh"

template <typename T>
__global__ void ln_add_kernel(float* __restrict__ x, const T* __restrict__ y1, const T* __restrict__ y2, float s1, float s2,
                              const float* __restrict__ w, const float* __restrict__ b, float eps, T* __restrict__ copy,
                              int D) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float sum = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = s1 * mb_load(y1 + base + d);
        if (y2) v = fmaf(s2, mb_load(y2 + base + d), v);
        row[d] = v;
        sum += v;
    }
    const float mean = mb_block_sum(sum, scratch) / (float)D;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = row[d] - mean; ss = fmaf(c, c, ss); }
    const float r = 1.0f / sqrtf(mb_block_sum(ss, scratch) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = x[base + d] + ((row[d] - mean) * r * w[d] + b[d]);
        x[base + d] = v;
        if (copy) mb_store(copy + base + d, v);
    }
}

template <typename T>
__global__ void layer_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                  const float* __restrict__ b, float eps, T* __restrict__ out, int D) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t src = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * D, dst = (size_t)blockIdx.x * D;
    float sum = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = x[src + d]; row[d] = v; sum += v; }
    const float mean = mb_block_sum(sum, scratch) / (float)D;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = row[d] - mean; ss = fmaf(c, c, ss); }
    const float r = 1.0f / sqrtf(mb_block_sum(ss, scratch) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) mb_store(out + dst + d, (row[d] - mean) * r * w[d] + b[d]);
}

template <typename T>
__global__ void to_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) mb_store(out + i, x[i]);
}

static inline int ln_threads(int D) { return D >= 2048 ? 256 : D >= 512 ? 128 : 64; }

template <typename T>
static int ln_add_launch(float* x, const void* y1, const void* y2, float s1, float s2, const float* w, const float* b,
                         float eps, void* copy, int N, int D, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || D > 12000 || !y1) return -2;
    ln_add_kernel<T><<<N, ln_threads(D), (size_t)D * sizeof(float), st>>>(x, (const T*)y1, (const T*)y2, s1, s2, w, b, eps,
                                                                          (T*)copy, D);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int layer_norm_launch(const float* x, const int* rows, const float* w, const float* b, float eps, void* out, int N,
                             int D, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || D > 12000) return -2;
    layer_norm_kernel<T><<<N, ln_threads(D), (size_t)D * sizeof(float), st>>>(x, rows, w, b, eps, (T*)out, D);
    MB_LAUNCH_CHECK();
    return 0;
}

#define LN_ENTRY(SUF, T)                                                                                                  \
    MB_API int mb_ln_add_##SUF(float* x, const void* y1, const void* y2, float s1, float s2, const float* w, const float* b, \
                               float eps, void* copy, int N, int D, cudaStream_t st) {                                    \
        return ln_add_launch<T>(x, y1, y2, s1, s2, w, b, eps, copy, N, D, st);                                            \
    }                                                                                                                     \
    MB_API int mb_layer_norm_##SUF(const float* x, const int* rows, const float* w, const float* b, float eps, void* out,  \
                                   int N, int D, cudaStream_t st) {                                                       \
        return layer_norm_launch<T>(x, rows, w, b, eps, out, N, D, st);                                                   \
    }                                                                                                                     \
    MB_API int mb_to_rows_##SUF(const float* x, void* out, long long total, cudaStream_t st) {                            \
        if (total == 0) return 0;                                                                                         \
        to_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, (T*)out, total);                            \
        MB_LAUNCH_CHECK();                                                                                                \
        return 0;                                                                                                         \
    }
LN_ENTRY(f32, float)
LN_ENTRY(bf16, bf16)
