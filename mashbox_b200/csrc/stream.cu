// Kernels of the residual stream for blocks whose norm is Dynamic Tanh and whose layers hand on a weighted average of
// everything the stream has been so far.  All arithmetic is float32; T is the storage type of activations.
//
//   dyt             x[n] += delta[n] (+ delta2[n]);  out[n] = tanh(alpha x[n]) * w + b   (no mean, no variance)
//                   out is of the storage type, or float32 (the embedding's norm writes the stream itself)
//   depth_average   y = x + delta;  hist[idx + 1] = y;  x = sum_(j <= idx + 1) coef[j] hist[j];  optionally the norm that
//                   reads the stream next: normed = tanh(alpha x) * w + b
//   rms_pair_mean   out[n] = (a[n] / rms(a[n]) * wa + b[n] / rms(b[n]) * wb) / 2: two outputs that ran side by side, each
//                   normed over the whole row with a weight of its own
#include "common.cuh"

template <typename T, typename OUT>
__global__ void dyt_kernel(float* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ delta2, float alpha,
                           const float* __restrict__ w, const float* __restrict__ b, OUT* out, const int* __restrict__ rows,
                           int D, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / D;
    const int d = (int)(i - n * D);
    const long long src = (rows ? (long long)rows[n] : n) * D + d;
    float v = x[src];
    if (delta) {
        v += mb_load(delta + src);
        if (delta2) v += mb_load(delta2 + src);
        if (!rows) x[src] = v;
    }
    mb_store(out + i, tanhf(alpha * v) * w[d] + b[d]);
}

template <typename T>
__global__ void depth_average_kernel(float* __restrict__ x, const T* __restrict__ delta, float* __restrict__ hist,
                                     long long slot_stride, const float* __restrict__ coef, int idx, float nalpha,
                                     const float* __restrict__ nw, const float* __restrict__ nb, T* __restrict__ normed,
                                     int D, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = x[i];
    if (delta) v += mb_load(delta + i);
    hist[(size_t)(idx + 1) * slot_stride + i] = v;
    float acc = 0.0f;
    for (int j = 0; j <= idx; j++) acc = fmaf(coef[j], hist[(size_t)j * slot_stride + i], acc);
    acc = fmaf(coef[idx + 1], v, acc);
    x[i] = acc;
    if (normed) {
        const int d = (int)(i % D);
        mb_store(normed + i, tanhf(nalpha * acc) * nw[d] + nb[d]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
rms_pair_mean_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                     const float* __restrict__ wb, T* __restrict__ out, int D, float eps) {
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    float sa = 0.0f, sb = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float u = mb_load(a + n * D + d), v = mb_load(b + n * D + d);
        sa = fmaf(u, u, sa);
        sb = fmaf(v, v, sb);
    }
    sa = mb_block_sum(sa, scratch);
    sb = mb_block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)D + eps), rb = 1.0f / sqrtf(sb / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        mb_store(out + n * D + d, 0.5f * (mb_load(a + n * D + d) * ra * wa[d] + mb_load(b + n * D + d) * rb * wb[d]));
}

#define STREAM_API(SUF, T)                                                                                                 \
    MB_API int mb_dyt_##SUF(float* x, const void* delta, const void* delta2, float alpha, const float* w, const float* b,  \
                            void* out, int out_float, const int* rows, int N, int D, cudaStream_t st) {                    \
        if (N == 0) return 0;                                                                                              \
        const long long total = (long long)N * D;                                                                          \
        const unsigned blocks = (unsigned)((total + 255) / 256);                                                           \
        if (out_float)                                                                                                     \
            dyt_kernel<T, float><<<blocks, 256, 0, st>>>(x, (const T*)delta, (const T*)delta2, alpha, w, b, (float*)out,  \
                                                         rows, D, total);                                                  \
        else                                                                                                               \
            dyt_kernel<T, T><<<blocks, 256, 0, st>>>(x, (const T*)delta, (const T*)delta2, alpha, w, b, (T*)out, rows, D,  \
                                                     total);                                                               \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }                                                                                                                      \
    MB_API int mb_depth_average_##SUF(float* x, const void* delta, float* hist, long long slot_stride, const float* coef,  \
                                      int idx, float nalpha, const float* nw, const float* nb, void* normed, int N, int D, \
                                      cudaStream_t st) {                                                                   \
        if (N == 0) return 0;                                                                                              \
        if (idx < 0) return -2;                                                                                            \
        const long long total = (long long)N * D;                                                                          \
        depth_average_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, (const T*)delta, hist, slot_stride,    \
                                                                                 coef, idx, nalpha, nw, nb, (T*)normed, D, \
                                                                                 total);                                   \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }                                                                                                                      \
    MB_API int mb_rms_pair_mean_##SUF(const void* a, const void* b, const float* wa, const float* wb, void* out, int N,    \
                                      int D, float eps, cudaStream_t st) {                                                 \
        if (N == 0) return 0;                                                                                              \
        rms_pair_mean_kernel<T><<<N, 256, 0, st>>>((const T*)a, (const T*)b, wa, wb, (T*)out, D, eps);                     \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }

STREAM_API(f32, float)
STREAM_API(bf16, bf16)
