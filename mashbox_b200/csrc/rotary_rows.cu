// What stands between a fused q/k/v product and attention when heads are normed before they are rotated, when keys and
// values differ in width, or when only a strip of a row is rotated.
//
//   norm_rope_kv_write   rows (N, stride) = [q: H heads of DK | k: KV heads of DK | v: KV heads of DV | ...].  Every q
//                        and k head is optionally divided by its root mean square and multiplied by a weight (DK values,
//                        shared by the heads), then its first RD values are rotated by the token's position; q is
//                        written back in place, k and v go into the page and slot of the position: kpool (pages, KV,
//                        page, DK), vpool (pages, KV, page, DV).
//   latent_rope          the rotated strips of latent attention: of every query head (H heads of q_head values, the
//                        strip at q_off) into the tail of that head's row of `qa` (H rows of qa_head values, the strip
//                        at qa_off), and of the token's shared key strip (kr_off in `rows`) into the tail of the
//                        position's cache row (pool (pages, 1, page, pool_row), the strip at pool_off).
//
// Rotation: pair i of RD/2 turns by position * freqs[i]; pairing 0 pairs value 2i with 2i + 1, pairing 1 value i with
// i + RD/2; cos and sin are multiplied by `gain` (1: a plain rotation).  Norms and angles are float32.
#include "common.cuh"

// v[0 .. W) in shared memory, the first RD values rotated in place by the threads of the block (a barrier before and after
// is the caller's)
__device__ __forceinline__ void rr_rotate(float* v, int RD, int pairing, const float* freqs, float pos, float gain) {
    for (int i = threadIdx.x; i < RD / 2; i += blockDim.x) {
        const int a = pairing ? i : 2 * i, b = pairing ? i + RD / 2 : 2 * i + 1;
        float sn, cs;
        sincosf(pos * freqs[i], &sn, &cs);
        sn *= gain;
        cs *= gain;
        const float u = v[a], w = v[b];
        v[a] = u * cs - w * sn;
        v[b] = w * cs + u * sn;
    }
}

// grid (N, ceil((H + KV) / NR_WARPS)): a block takes NR_WARPS of a token's H + KV heads, a warp a head; the token's cosines
// and sines are made once per block, by all its threads.  Shared memory: RD floats of cos and sin, then DK floats per warp.
#define NR_WARPS 8
template <typename T>
__global__ void __launch_bounds__(NR_WARPS * 32) norm_rope_kv_write_kernel(
    T* __restrict__ rows, int stride, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ freqs, int RD, int pairing, float gain, const int* __restrict__ positions,
    const int* __restrict__ tok_row, const int* __restrict__ table, int max_blocks, T* __restrict__ kpool,
    T* __restrict__ vpool, int H, int KV, int DK, int DV, int page, int num_pages, int* err) {
    extern __shared__ float smem[];
    float* cs = smem;                       // cos of the RD / 2 pairs, then sin
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = RD / 2;
    float* vals = smem + RD + warp * DK;
    const int pos = positions[n];
    if (freqs) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, c;
            sincosf((float)pos * freqs[i], &sn, &c);
            cs[i] = c * gain;
            cs[half + i] = sn * gain;
        }
    }
    __syncthreads();
    size_t slot = 0;
    bool have_page = false;
    if (kpool) {
        const int pg = table[(size_t)tok_row[n] * max_blocks + pos / page];
        if (pg < 0 || pg >= num_pages) {
            if (threadIdx.x == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
        } else {
            have_page = true;
            slot = (size_t)pg * KV * page + (pos % page);           // + kv head * page
        }
    }
    for (int b = blockIdx.y * NR_WARPS + warp; b < H + KV; b += gridDim.y * NR_WARPS) {
        const bool is_q = b < H;
        const int kvh = b - H;
        T* src = rows + (size_t)n * stride + (size_t)b * DK;       // the k heads follow the q heads
        const float* w = is_q ? qw : kw;
        float ss = 0.0f;
        for (int d = lane; d < DK; d += 32) { const float x = mb_load(src + d); vals[d] = x; ss = fmaf(x, x, ss); }
        if (w) {
            const float r = 1.0f / sqrtf(mb_warp_sum(ss) / (float)DK + eps);
            for (int d = lane; d < DK; d += 32) vals[d] = vals[d] * r * w[d];
        }
        __syncwarp();
        if (freqs) {
            for (int i = lane; i < half; i += 32) {
                const int a = pairing ? i : 2 * i, c = pairing ? i + half : 2 * i + 1;
                const float u = vals[a], v = vals[c];
                vals[a] = u * cs[i] - v * cs[half + i];
                vals[c] = v * cs[i] + u * cs[half + i];
            }
        }
        __syncwarp();
        if (is_q) {
            for (int d = lane; d < DK; d += 32) mb_store(src + d, vals[d]);
        } else if (have_page) {
            const size_t row = slot + (size_t)kvh * page;
            for (int d = lane; d < DK; d += 32) mb_store(kpool + row * DK + d, vals[d]);
            const T* vs = rows + (size_t)n * stride + (size_t)(H + KV) * DK + (size_t)kvh * DV;
            for (int d = lane; d < DV; d += 32) vpool[row * DV + d] = vs[d];
        }
        __syncwarp();
    }
}

template <typename T>
__global__ void latent_rope_kernel(const T* __restrict__ q, int q_stride, int q_head, int q_off, T* __restrict__ qa,
                                   int qa_head, int qa_off, const T* __restrict__ rows, int rows_stride, int kr_off,
                                   T* __restrict__ pool, int pool_row, int pool_off, const float* __restrict__ freqs, int RD,
                                   int W, int pairing, float gain, const int* __restrict__ positions,
                                   const int* __restrict__ tok_row, const int* __restrict__ table, int max_blocks, int H,
                                   int page, int num_pages, int* err) {
    extern __shared__ float vals[];
    const int n = blockIdx.x, h = blockIdx.y;
    const int pos = positions[n];
    const T* src = h < H ? q + (size_t)n * q_stride + (size_t)h * q_head + q_off : rows + (size_t)n * rows_stride + kr_off;
    for (int d = threadIdx.x; d < W; d += blockDim.x) vals[d] = mb_load(src + d);
    __syncthreads();
    if (freqs && RD > 0) rr_rotate(vals, RD, pairing, freqs, (float)pos, gain);
    __syncthreads();
    T* dst;
    if (h < H) {
        dst = qa + ((size_t)n * H + h) * qa_head + qa_off;
    } else {
        if (!pool) return;
        const int pg = table[(size_t)tok_row[n] * max_blocks + pos / page];
        if (pg < 0 || pg >= num_pages) {
            if (threadIdx.x == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            return;
        }
        dst = pool + ((size_t)pg * page + (pos % page)) * pool_row + pool_off;
    }
    for (int d = threadIdx.x; d < W; d += blockDim.x) mb_store(dst + d, vals[d]);
}

#define RR_ENTRIES(SUF, T)                                                                                                 \
    MB_API int mb_norm_rope_kv_write_##SUF(void* rows, int stride, const float* qw, const float* kw, float eps,            \
                                           const float* freqs, int RD, int pairing, float gain, const int* positions,     \
                                           const int* tok_row, const int* table, int max_blocks, void* kpool, void* vpool, \
                                           int N, int H, int KV, int DK, int DV, int page, int num_pages, int* err,       \
                                           cudaStream_t st) {                                                             \
        if (N == 0) return 0;                                                                                              \
        if (H < 1 || KV < 1 || H + KV > 65535 * NR_WARPS || DK < 1 || DV < 1 || DK > 1024 || RD < 0 || RD > DK || (RD & 1) ||                            \
            page < 1)                                                                                                      \
            return -2;                                                                                                     \
        norm_rope_kv_write_kernel<T><<<dim3(N, (H + KV + NR_WARPS - 1) / NR_WARPS), NR_WARPS * 32,                        \
                                       (size_t)(RD + NR_WARPS * DK) * sizeof(float), st>>>(                               \
            (T*)rows, stride, qw, kw, eps, freqs, RD, pairing, gain, positions, tok_row, table, max_blocks, (T*)kpool,     \
            (T*)vpool, H, KV, DK, DV, page, num_pages, err);                                                               \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }                                                                                                                      \
    MB_API int mb_latent_rope_##SUF(const void* q, int q_stride, int q_head, int q_off, void* qa, int qa_head, int qa_off, \
                                    const void* rows, int rows_stride, int kr_off, void* pool, int pool_row, int pool_off, \
                                    const float* freqs, int RD, int W, int pairing, float gain, const int* positions,     \
                                    const int* tok_row, const int* table, int max_blocks, int N, int H, int page,         \
                                    int num_pages, int* err, cudaStream_t st) {                                           \
        if (N == 0 || W == 0) return 0;                                                                                    \
        if (H < 1 || H + 1 > 65535 || W < 1 || W > 8192 || RD < 0 || RD > W || (RD & 1) || page < 1) return -2;            \
        latent_rope_kernel<T><<<dim3(N, H + 1), 32, (size_t)W * sizeof(float), st>>>(                                      \
            (const T*)q, q_stride, q_head, q_off, (T*)qa, qa_head, qa_off, (const T*)rows, rows_stride, kr_off, (T*)pool,  \
            pool_row, pool_off, freqs, RD, W, pairing, gain, positions, tok_row, table, max_blocks, H, page, num_pages,    \
            err);                                                                                                          \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }
RR_ENTRIES(f32, float)
RR_ENTRIES(bf16, bf16)
