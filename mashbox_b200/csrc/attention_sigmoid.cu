// Paged attention whose weights are not normalised over the keys: a visible key j weighs
//     sigmoid(scale q_i . k_j - slope_h (i - j) + bias_h)
// for the query at position i (causal: j <= i), with one slope and one bias per query head, and the output is the plain
// weighted sum of the values.  Keys and values have widths of their own (dim, vdim) and live in two pools,
// (pages, kv heads, page, width) each.  Scores, weights and sums are float32.
//
//   sigattn_prep     from the product's rows [q | k | v]: q and k divided by the root mean square of their WHOLE row
//                    (all heads at once) and multiplied by a weight per channel, q also by the position's temperature
//                    1 + coef ln(floor((p + 1) / every) + 1); every head's v divided by its own root mean square;
//                    q to a buffer, k and v into the pages of the token's position
//   sigattn_simple   one warp per (token, query head), keys in ascending position through the block table: the whole
//                    float32 path and every size the tensor-core form does not take
//   sigattn_mma      bf16 on mma.sync: 64 packed query rows of one (sequence, kv head) against key tiles of 64; a weight
//                    is split into two bf16 numbers (w = hi + lo, 16 bits of mantissa together) that both multiply the
//                    values, so the sum keeps float32's grade although the values are read as bf16
#include "common.cuh"

#define SA_WARPS 4

// grid (N), 256 threads
template <typename T>
__global__ void __launch_bounds__(256)
sigattn_prep_kernel(const T* __restrict__ rows, int stride, const float* __restrict__ qw, const float* __restrict__ kw,
                    const int* __restrict__ positions, const int* __restrict__ tok_row, const int* __restrict__ table,
                    int max_blocks, T* __restrict__ q_out, T* __restrict__ kpool, T* __restrict__ vpool, int H, int G, int dim,
                    int vdim, int page, int num_pages, float eps, float temp_coef, int temp_every, int* err) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, p = positions[n];
    const T* row = rows + (size_t)n * stride;
    const int QW = H * dim, KW = G * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < QW; i += blockDim.x) { const float a = mb_load(row + i); ss = fmaf(a, a, ss); }
    ss = mb_block_sum(ss, scratch);
    float r = 1.0f / sqrtf(ss / (float)QW + eps);
    const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((p + 1) / temp_every) + 1.0f) : 1.0f;
    for (int i = threadIdx.x; i < QW; i += blockDim.x)
        mb_store(q_out + (size_t)n * QW + i, mb_load(row + i) * r * qw[i] * temp);
    if (kpool == nullptr) return;
    const int pg = table[(size_t)tok_row[n] * max_blocks + p / page];
    if (pg < 0 || pg >= num_pages) {
        if (threadIdx.x == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
        return;
    }
    ss = 0.0f;
    for (int i = threadIdx.x; i < KW; i += blockDim.x) { const float a = mb_load(row + QW + i); ss = fmaf(a, a, ss); }
    ss = mb_block_sum(ss, scratch);
    r = 1.0f / sqrtf(ss / (float)KW + eps);
    const int slot = p % page;
    for (int i = threadIdx.x; i < KW; i += blockDim.x) {
        const int g = i / dim, d = i - g * dim;
        mb_store(kpool + (((size_t)pg * G + g) * page + slot) * dim + d, mb_load(row + QW + i) * r * kw[i]);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int g = warp; g < G; g += nwarp) {
        const T* vs = row + QW + KW + (size_t)g * vdim;
        float s2 = 0.0f;
        for (int c = lane; c < vdim; c += 32) { const float a = mb_load(vs + c); s2 = fmaf(a, a, s2); }
        s2 = mb_warp_sum(s2);
        const float rv = 1.0f / sqrtf(s2 / (float)vdim + eps);
        T* dst = vpool + (((size_t)pg * G + g) * page + slot) * vdim;
        for (int c = lane; c < vdim; c += 32) mb_store(dst + c, mb_load(vs + c) * rv);
    }
}

__device__ __forceinline__ float sa_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T, int MAXD>
__global__ void __launch_bounds__(SA_WARPS * 32)
sigattn_simple_kernel(const T* __restrict__ q, T* __restrict__ out, const int* __restrict__ positions,
                      const int* __restrict__ tok_row, const int* __restrict__ table, int max_blocks,
                      const T* __restrict__ kpool, const T* __restrict__ vpool, const float* __restrict__ slopes,
                      const float* __restrict__ bias, int N, int H, int G, int dim, int vdim, int page, int num_pages,
                      float scale, int* err) {
    __shared__ float qs[SA_WARPS][MAXD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * SA_WARPS + warp;
    if (item >= (long long)N * H) return;
    const int n = (int)(item / H), h = (int)(item % H);
    const int g = h / (H / G);
    const int pos = positions[n];
    const int* tb = table + (size_t)tok_row[n] * max_blocks;
    const T* qr = q + ((size_t)n * H + h) * dim;
    for (int d = lane; d < dim; d += 32) qs[warp][d] = mb_load(qr + d);
    __syncwarp();
    const float slope = slopes ? slopes[h] : 0.0f, b = bias ? bias[h] : 0.0f;
    float acc[MAXD / 32];
#pragma unroll
    for (int i = 0; i < MAXD / 32; i++) acc[i] = 0.0f;
    for (int base = 0; base <= pos; base += 32) {
        const int kp = base + lane;
        long long at = -1;
        float w = 0.0f;
        if (kp <= pos) {
            const int pg = tb[kp / page];
            if (pg < 0 || pg >= num_pages) {
                mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            } else {
                at = ((long long)pg * G + g) * page + (kp % page);
                const T* kr = kpool + at * dim;
                float a = 0.0f;
                for (int d = 0; d < dim; d++) a = fmaf(qs[warp][d], mb_load(kr + d), a);
                w = sa_sigmoid(a * scale - slope * (float)(pos - kp) + b);
            }
        }
        const int cnt = min(32, pos - base + 1);
        for (int j = 0; j < cnt; j++) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            const long long aj = __shfl_sync(0xffffffffu, at, j);
            if (aj < 0) continue;
            const T* vr = vpool + aj * vdim;
#pragma unroll
            for (int i = 0; i < MAXD / 32; i++) {
                const int d = lane + 32 * i;
                if (d < vdim) acc[i] = fmaf(wj, mb_load(vr + d), acc[i]);
            }
        }
    }
    T* o = out + ((size_t)n * H + h) * vdim;
#pragma unroll
    for (int i = 0; i < MAXD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < vdim) mb_store(o + d, acc[i]);
    }
}

template <typename T>
static int sigattn_prep_launch(const void* rows, int stride, const float* qw, const float* kw, const int* positions,
                               const int* tok_row, const int* table, int max_blocks, void* q_out, void* kpool, void* vpool,
                               int N, int H, int G, int dim, int vdim, int page, int num_pages, float eps, float temp_coef,
                               int temp_every, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (H < 1 || G < 1 || H % G || dim < 1 || vdim < 1 || page < 1) return -2;
    sigattn_prep_kernel<T><<<N, 256, 0, st>>>((const T*)rows, stride, qw, kw, positions, tok_row, table, max_blocks, (T*)q_out,
                                              (T*)kpool, (T*)vpool, H, G, dim, vdim, page, num_pages, eps, temp_coef,
                                              temp_every, err);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int sigattn_simple_launch(const void* q, void* out, const int* positions, const int* tok_row, const int* table,
                                 int max_blocks, const void* kpool, const void* vpool, const float* slopes,
                                 const float* bias, int N, int H, int G, int dim, int vdim, int page, int num_pages,
                                 float scale, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    const int W = dim > vdim ? dim : vdim;
    if (W > 512 || dim < 1 || vdim < 1 || G < 1 || H % G) return -2;
    const long long items = (long long)N * H;
    const unsigned blocks = (unsigned)((items + SA_WARPS - 1) / SA_WARPS);
    if (W <= 128)
        sigattn_simple_kernel<T, 128><<<blocks, SA_WARPS * 32, 0, st>>>(
            (const T*)q, (T*)out, positions, tok_row, table, max_blocks, (const T*)kpool, (const T*)vpool, slopes, bias, N, H, G,
            dim, vdim, page, num_pages, scale, err);
    else
        sigattn_simple_kernel<T, 512><<<blocks, SA_WARPS * 32, 0, st>>>(
            (const T*)q, (T*)out, positions, tok_row, table, max_blocks, (const T*)kpool, (const T*)vpool, slopes, bias, N, H, G,
            dim, vdim, page, num_pages, scale, err);
    MB_LAUNCH_CHECK();
    return 0;
}

#define SA_INSTANCES(SUF, T)                                                                                               \
    MB_API int mb_sigattn_prep_##SUF(const void* rows, int stride, const float* qw, const float* kw, const int* positions, \
                                     const int* tok_row, const int* table, int max_blocks, void* q_out, void* kpool,       \
                                     void* vpool, int N, int H, int G, int dim, int vdim, int page, int num_pages,         \
                                     float eps, float temp_coef, int temp_every, int* err, cudaStream_t st) {              \
        return sigattn_prep_launch<T>(rows, stride, qw, kw, positions, tok_row, table, max_blocks, q_out, kpool, vpool, N, \
                                      H, G, dim, vdim, page, num_pages, eps, temp_coef, temp_every, err, st);              \
    }                                                                                                                      \
    MB_API int mb_sigattn_simple_##SUF(const void* q, void* out, const int* positions, const int* tok_row,                 \
                                       const int* table, int max_blocks, const void* kpool, const void* vpool,             \
                                       const float* slopes, const float* bias, int N, int H, int G, int dim, int vdim,     \
                                       int page, int num_pages, float scale, int* err, cudaStream_t st) {                  \
        return sigattn_simple_launch<T>(q, out, positions, tok_row, table, max_blocks, kpool, vpool, slopes, bias, N, H,  \
                                        G, dim, vdim, page, num_pages, scale, err, st);                                    \
    }
SA_INSTANCES(f32, float)
SA_INSTANCES(bf16, bf16)
