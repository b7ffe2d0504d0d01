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

__device__ __forceinline__ float4 ln_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ln_load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), c = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(c), __high2float(c));
}
__device__ __forceinline__ void ln_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ln_store4(bf16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// VEC: rows are read and written four values at a time (D a multiple of 4, every pointer on a 16-byte boundary).  The sums
// run in another order than in the plain form, so a model uses one form throughout: the choice depends on D and on the
// buffers' alignment, never on the batch.
template <typename T, bool VEC>
__global__ void ln_add_kernel(float* __restrict__ x, const T* __restrict__ y1, const T* __restrict__ y2, float s1, float s2,
                              const float* __restrict__ w, const float* __restrict__ b, float eps, T* __restrict__ copy,
                              int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float sum = 0.0f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
            const float4 a = ln_load4(y1 + base + d);
            float4 v = make_float4(s1 * a.x, s1 * a.y, s1 * a.z, s1 * a.w);
            if (y2) {
                const float4 c = ln_load4(y2 + base + d);
                v = make_float4(fmaf(s2, c.x, v.x), fmaf(s2, c.y, v.y), fmaf(s2, c.z, v.z), fmaf(s2, c.w, v.w));
            }
            ln_store4(row + d, v);
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float v = s1 * mb_load(y1 + base + d);
            if (y2) v = fmaf(s2, mb_load(y2 + base + d), v);
            row[d] = v;
            sum += v;
        }
    }
    const float mean = mb_block_sum(sum, scratch) / (float)D;
    float ss = 0.0f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {     // every thread reads back what it wrote itself
            const float4 v = ln_load4(row + d);
            const float c0 = v.x - mean, c1 = v.y - mean, c2 = v.z - mean, c3 = v.w - mean;
            ss = fmaf(c0, c0, ss); ss = fmaf(c1, c1, ss); ss = fmaf(c2, c2, ss); ss = fmaf(c3, c3, ss);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = row[d] - mean; ss = fmaf(c, c, ss); }
    }
    const float r = 1.0f / sqrtf(mb_block_sum(ss, scratch) / (float)D + eps);
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
            const float4 v = ln_load4(row + d), xv = ln_load4(x + base + d), wv = ln_load4(w + d), bv = ln_load4(b + d);
            const float4 o = make_float4(xv.x + ((v.x - mean) * r * wv.x + bv.x), xv.y + ((v.y - mean) * r * wv.y + bv.y),
                                         xv.z + ((v.z - mean) * r * wv.z + bv.z), xv.w + ((v.w - mean) * r * wv.w + bv.w));
            ln_store4(x + base + d, o);
            if (copy) ln_store4(copy + base + d, o);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float v = x[base + d] + ((row[d] - mean) * r * w[d] + b[d]);
            x[base + d] = v;
            if (copy) mb_store(copy + base + d, v);
        }
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
static inline bool ln_aligned(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr,
                              const void* e = nullptr, const void* f = nullptr) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(e) | reinterpret_cast<uintptr_t>(f)) & 15) == 0;
}

template <typename T>
static int ln_add_launch(float* x, const void* y1, const void* y2, float s1, float s2, const float* w, const float* b,
                         float eps, void* copy, int N, int D, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || D > 12000 || !y1) return -2;
    if (D % 4 == 0 && ln_aligned(x, y1, y2, w, b, copy))
        ln_add_kernel<T, true><<<N, D >= 2048 ? 256 : D >= 512 ? 128 : 64, (size_t)D * sizeof(float), st>>>(
            x, (const T*)y1, (const T*)y2, s1, s2, w, b, eps, (T*)copy, D);
    else
        ln_add_kernel<T, false><<<N, ln_threads(D), (size_t)D * sizeof(float), st>>>(x, (const T*)y1, (const T*)y2, s1, s2, w,
                                                                                     b, eps, (T*)copy, D);
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
