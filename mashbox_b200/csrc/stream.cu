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
#include <initializer_list>

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

// ---- the forms for rows whose width is a multiple of 4: a thread takes 4 neighbours of one row (grid: rows x pieces of
// 1,024 values), so nothing is divided and every access is 8 or 16 bytes wide
struct F4 { float v[4]; };
template <typename T> __device__ __forceinline__ F4 load4(const T* p);
template <> __device__ __forceinline__ F4 load4<float>(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    return F4{{a.x, a.y, a.z, a.w}};
}
template <> __device__ __forceinline__ F4 load4<bf16>(const bf16* p) {
    const uint2 a = *reinterpret_cast<const uint2*>(p);
    return F4{{__uint_as_float(a.x << 16), __uint_as_float(a.x & 0xffff0000u), __uint_as_float(a.y << 16),
               __uint_as_float(a.y & 0xffff0000u)}};
}
template <typename T> __device__ __forceinline__ void store4(T* p, const F4& a);
template <> __device__ __forceinline__ void store4<float>(float* p, const F4& a) {
    *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const F4& a) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(a.v[0], a.v[1]), pack_bf16(a.v[2], a.v[3]));
}

template <typename T, typename OUT>
__global__ void __launch_bounds__(256)
dyt4_kernel(float* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ delta2, float alpha,
            const float* __restrict__ w, const float* __restrict__ b, OUT* out, const int* __restrict__ rows, int D) {
    const int d = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (d >= D) return;
    const size_t n = blockIdx.x;
    const size_t src = (rows ? (size_t)rows[n] : n) * D + d;
    F4 v = load4<float>(x + src);
    if (delta) {
        const F4 a = load4<T>(delta + src);
#pragma unroll
        for (int e = 0; e < 4; e++) v.v[e] += a.v[e];
        if (delta2) {
            const F4 c = load4<T>(delta2 + src);
#pragma unroll
            for (int e = 0; e < 4; e++) v.v[e] += c.v[e];
        }
        if (!rows) store4<float>(x + src, v);
    }
    const F4 ww = load4<float>(w + d), bb = load4<float>(b + d);
#pragma unroll
    for (int e = 0; e < 4; e++) v.v[e] = tanhf(alpha * v.v[e]) * ww.v[e] + bb.v[e];
    store4<OUT>(out + n * D + d, v);
}

template <typename T>
__global__ void __launch_bounds__(256)
depth_average4_kernel(float* __restrict__ x, const T* __restrict__ delta, float* __restrict__ hist, long long slot_stride,
                      const float* __restrict__ coef, int idx, float nalpha, const float* __restrict__ nw,
                      const float* __restrict__ nb, T* __restrict__ normed, int D) {
    const int d = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (d >= D) return;
    const size_t i = (size_t)blockIdx.x * D + d;
    F4 v = load4<float>(x + i);
    if (delta) {
        const F4 a = load4<T>(delta + i);
#pragma unroll
        for (int e = 0; e < 4; e++) v.v[e] += a.v[e];
    }
    store4<float>(hist + (size_t)(idx + 1) * slot_stride + i, v);
    F4 acc = F4{{0.0f, 0.0f, 0.0f, 0.0f}};
    for (int j = 0; j <= idx; j++) {
        const float c = coef[j];
        const F4 h = load4<float>(hist + (size_t)j * slot_stride + i);
#pragma unroll
        for (int e = 0; e < 4; e++) acc.v[e] = fmaf(c, h.v[e], acc.v[e]);
    }
    const float c = coef[idx + 1];
#pragma unroll
    for (int e = 0; e < 4; e++) acc.v[e] = fmaf(c, v.v[e], acc.v[e]);
    store4<float>(x + i, acc);
    if (normed) {
        const F4 ww = load4<float>(nw + d), bb = load4<float>(nb + d);
#pragma unroll
        for (int e = 0; e < 4; e++) acc.v[e] = tanhf(nalpha * acc.v[e]) * ww.v[e] + bb.v[e];
        store4<T>(normed + i, acc);
    }
}

// every pointer on a 16-byte boundary, the width and the stride between history slots multiples of 4
static bool rows_of_four(int D, long long stride, std::initializer_list<const void*> ptrs) {
    if (D % 4 != 0 || stride % 4 != 0) return false;
    for (const void* p : ptrs) if (((uintptr_t)p & 15) != 0) return false;
    return true;
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

// The bf16 form for rows of up to 8,192 values, a multiple of 8: a thread brings its 16-byte pieces of both rows in at
// once and keeps them in registers between the sums of squares and the output, so every byte is read once.
template <int MAXV>                     // 16-byte pieces a thread: rows of up to 2,048 MAXV values
__global__ void __launch_bounds__(256)
rms_pair_mean_rows_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, const float* __restrict__ wa,
                          const float* __restrict__ wb, bf16* __restrict__ out, int D, float eps) {
    __shared__ float scratch[32];
    const size_t n = blockIdx.x;
    const int nv = D >> 3;
    const uint4* a4 = reinterpret_cast<const uint4*>(a + n * D);
    const uint4* b4 = reinterpret_cast<const uint4*>(b + n * D);
    uint4 ra4[MAXV], rb4[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int v = threadIdx.x + i * 256;
        ra4[i] = v < nv ? a4[v] : make_uint4(0u, 0u, 0u, 0u);
        rb4[i] = v < nv ? b4[v] : make_uint4(0u, 0u, 0u, 0u);
    }
    float sa = 0.0f, sb = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const uint32_t ua[4] = {ra4[i].x, ra4[i].y, ra4[i].z, ra4[i].w}, ub[4] = {rb4[i].x, rb4[i].y, rb4[i].z, rb4[i].w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float a0 = __uint_as_float(ua[e] << 16), a1 = __uint_as_float(ua[e] & 0xffff0000u);
            const float b0 = __uint_as_float(ub[e] << 16), b1 = __uint_as_float(ub[e] & 0xffff0000u);
            sa = fmaf(a0, a0, sa); sa = fmaf(a1, a1, sa);
            sb = fmaf(b0, b0, sb); sb = fmaf(b1, b1, sb);
        }
    }
    sa = mb_block_sum(sa, scratch);
    sb = mb_block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)D + eps), rb = 1.0f / sqrtf(sb / (float)D + eps);
    uint4* o4 = reinterpret_cast<uint4*>(out + n * D);
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int v = threadIdx.x + i * 256;
        if (v >= nv) continue;
        const uint32_t ua[4] = {ra4[i].x, ra4[i].y, ra4[i].z, ra4[i].w}, ub[4] = {rb4[i].x, rb4[i].y, rb4[i].z, rb4[i].w};
        const float4 wa0 = *reinterpret_cast<const float4*>(wa + v * 8), wa1 = *reinterpret_cast<const float4*>(wa + v * 8 + 4);
        const float4 wb0 = *reinterpret_cast<const float4*>(wb + v * 8), wb1 = *reinterpret_cast<const float4*>(wb + v * 8 + 4);
        const float fa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
        const float fb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float a0 = __uint_as_float(ua[e] << 16), a1 = __uint_as_float(ua[e] & 0xffff0000u);
            const float b0 = __uint_as_float(ub[e] << 16), b1 = __uint_as_float(ub[e] & 0xffff0000u);
            r[e] = pack_bf16(0.5f * (a0 * ra * fa[2 * e] + b0 * rb * fb[2 * e]), 0.5f * (a1 * ra * fa[2 * e + 1] + b1 * rb * fb[2 * e + 1]));
        }
        o4[v] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

template <typename T>
static bool pair_mean_rows(const void*, const void*, const float*, const float*, void*, int, int, float, cudaStream_t) { return false; }
template <>
bool pair_mean_rows<bf16>(const void* a, const void* b, const float* wa, const float* wb, void* out, int N, int D, float eps,
                          cudaStream_t st) {
    if (D % 8 != 0 || D > 8192) return false;
    if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)out | (uintptr_t)wa | (uintptr_t)wb) & 15) != 0) return false;
    if (D <= 2048)          // the fewer pieces a thread keeps, the more blocks a multiprocessor holds
        rms_pair_mean_rows_kernel<1><<<N, 256, 0, st>>>((const bf16*)a, (const bf16*)b, wa, wb, (bf16*)out, D, eps);
    else if (D <= 4096)
        rms_pair_mean_rows_kernel<2><<<N, 256, 0, st>>>((const bf16*)a, (const bf16*)b, wa, wb, (bf16*)out, D, eps);
    else
        rms_pair_mean_rows_kernel<4><<<N, 256, 0, st>>>((const bf16*)a, (const bf16*)b, wa, wb, (bf16*)out, D, eps);
    return true;
}

#define STREAM_API(SUF, T)                                                                                                 \
    MB_API int mb_dyt_##SUF(float* x, const void* delta, const void* delta2, float alpha, const float* w, const float* b,  \
                            void* out, int out_float, const int* rows, int N, int D, cudaStream_t st) {                    \
        if (N == 0) return 0;                                                                                              \
        const long long total = (long long)N * D;                                                                          \
        const unsigned blocks = (unsigned)((total + 255) / 256);                                                           \
        if (rows_of_four(D, 0, {x, delta, delta2, w, b, out})) {                                                           \
            const dim3 grid(N, (D / 4 + 255) / 256);                                                                       \
            if (out_float)                                                                                                 \
                dyt4_kernel<T, float><<<grid, 256, 0, st>>>(x, (const T*)delta, (const T*)delta2, alpha, w, b,            \
                                                            (float*)out, rows, D);                                         \
            else                                                                                                           \
                dyt4_kernel<T, T><<<grid, 256, 0, st>>>(x, (const T*)delta, (const T*)delta2, alpha, w, b, (T*)out, rows,  \
                                                        D);                                                                \
            MB_LAUNCH_CHECK();                                                                                             \
            return 0;                                                                                                      \
        }                                                                                                                  \
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
        if (rows_of_four(D, slot_stride, {x, delta, hist, nw, nb, normed})) {                                              \
            depth_average4_kernel<T><<<dim3(N, (D / 4 + 255) / 256), 256, 0, st>>>(x, (const T*)delta, hist, slot_stride,  \
                                                                                   coef, idx, nalpha, nw, nb, (T*)normed,  \
                                                                                   D);                                     \
            MB_LAUNCH_CHECK();                                                                                             \
            return 0;                                                                                                      \
        }                                                                                                                  \
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
        if (!pair_mean_rows<T>(a, b, wa, wb, out, N, D, eps, st))                                                          \
            rms_pair_mean_kernel<T><<<N, 256, 0, st>>>((const T*)a, (const T*)b, wa, wb, (T*)out, D, eps);                 \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }

STREAM_API(f32, float)
STREAM_API(bf16, bf16)
