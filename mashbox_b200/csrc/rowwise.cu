// Row-wise kernels of blocks that norm a sublayer's output before it joins the stream, of learned positions, of
// latents kept in pages and of per-head products.  All arithmetic is float32; T is the storage type of activations.
//
//   embed_pos        x[n] = table[token[n]] * scale + pos[position[n]]
//   post_norm_add    x[n] += delta[n] / sqrt(mean(delta[n]^2) + eps_p) * w_p;  optionally y[n] = x[n] / sqrt(mean(x[n]^2)
//                    + eps_n) * w_n (the norm that reads the stream next) and a copy of x[n] in the storage type
//   rms_segments     two stretches of columns of a product's rows, each RMS-normed with a weight of its own: the first
//                    goes to a buffer, the second into the cache page of the token's position (one vector per position)
//   gated_gather     g[n, j] = gelu_tanh(z[n, j]) * table[token[n], off + j]
//   sigmoid_mul      o[n, c] *= sigmoid(gate[n, c])
//   head_product     out[n, h, j] = sum_i in[n, h, i] * W[h, i, j], W given by three strides (a projection applied
//                    head by head from either side)
//   scale_rows       y *= s
#include "common.cuh"

#define MB_ERR_POSITION_RANGE 5     // a position outside the learned position table

template <typename T>
__global__ void embed_pos_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                 const T* __restrict__ table, const T* __restrict__ pos, float* __restrict__ x, int D, int V,
                                 int P, float scale, int* err) {
    const int n = blockIdx.x;
    int tok = tokens[n], p = positions[n];
    if (tok < 0 || tok >= V) { if (threadIdx.x == 0) mb_set_error(err, MB_ERR_TOKEN_RANGE); tok = 0; }
    if (p < 0 || p >= P) { if (threadIdx.x == 0) mb_set_error(err, MB_ERR_POSITION_RANGE); p = 0; }
    const T* e = table + (size_t)tok * D;
    const T* q = pos + (size_t)p * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) x[(size_t)n * D + d] = mb_load(e + d) * scale + mb_load(q + d);
}

// four values of a row at once (D a multiple of 4, 16-byte aligned rows)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                       __uint_as_float(r.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// VEC: rows are read and written four values at a time; the sums of squares run in the same order either way only
// within a form, so a model uses one form throughout (the choice depends on D alone).
template <typename T, bool VEC>
__global__ void post_norm_add_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ post_w,
                                     float post_eps, const float* __restrict__ next_w, float next_eps, T* __restrict__ normed,
                                     T* __restrict__ copy, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    float ss = 0.0f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
            const float4 v = load4(delta + (size_t)n * D + d);
            store4(row + d, v);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float v = mb_load(delta + (size_t)n * D + d);
            row[d] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = mb_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + post_eps);
    float s2 = 0.0f;
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
            const float4 xv = load4(x + (size_t)n * D + d), dv = load4(row + d), w = load4(post_w + d);
            const float4 v = make_float4(xv.x + dv.x * r * w.x, xv.y + dv.y * r * w.y, xv.z + dv.z * r * w.z, xv.w + dv.w * r * w.w);
            store4(x + (size_t)n * D + d, v);
            store4(row + d, v);
            s2 = fmaf(v.x, v.x, s2); s2 = fmaf(v.y, v.y, s2); s2 = fmaf(v.z, v.z, s2); s2 = fmaf(v.w, v.w, s2);
            if (copy) store4(copy + (size_t)n * D + d, v);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float v = x[(size_t)n * D + d] + row[d] * r * post_w[d];
            x[(size_t)n * D + d] = v;
            row[d] = v;
            s2 = fmaf(v, v, s2);
            if (copy) mb_store(copy + (size_t)n * D + d, v);
        }
    }
    if (!normed) return;
    s2 = mb_block_sum(s2, scratch);
    const float r2 = 1.0f / sqrtf(s2 / (float)D + next_eps);
    if (VEC) {
        for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
            const float4 v = load4(row + d), w = load4(next_w + d);
            store4(normed + (size_t)n * D + d, make_float4(v.x * r2 * w.x, v.y * r2 * w.y, v.z * r2 * w.z, v.w * r2 * w.w));
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) mb_store(normed + (size_t)n * D + d, row[d] * r2 * next_w[d]);
    }
}

template <typename T>
__global__ void rms_segments_kernel(const T* __restrict__ in, int stride, int off_a, int wa, const float* __restrict__ w_a,
                                    T* __restrict__ out_a, int off_b, int wb, const float* __restrict__ w_b, T* __restrict__ pool,
                                    const int* __restrict__ positions, const int* __restrict__ tok_row,
                                    const int* __restrict__ table, int max_blocks, int page, int num_pages, float eps,
                                    int* err, int pool_row) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, second = blockIdx.y;
    const int off = second ? off_b : off_a, W = second ? wb : wa;
    if (W <= 0) return;
    const float* w = second ? w_b : w_a;
    T* dst;
    if (!second) {
        dst = out_a + (size_t)n * wa;
    } else {
        const int p = positions[n];
        const int pg = table[(size_t)tok_row[n] * max_blocks + p / page];
        if (pg < 0 || pg >= num_pages) {
            if (threadIdx.x == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            return;
        }
        dst = pool + ((size_t)pg * page + p % page) * pool_row;       // a row may be wider than the stretch
    }
    const T* src = in + (size_t)n * stride + off;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < W; d += blockDim.x) { const float v = mb_load(src + d); ss = fmaf(v, v, ss); }
    ss = mb_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)W + eps);
    for (int d = threadIdx.x; d < W; d += blockDim.x) mb_store(dst + d, mb_load(src + d) * r * w[d]);
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gated_gather_kernel(const T* __restrict__ z, const int* __restrict__ tokens, const T* __restrict__ table,
                                    int table_stride, int off, T* __restrict__ out, int W, int V, int* err) {
    const int n = blockIdx.x;
    int tok = tokens[n];
    if (tok < 0 || tok >= V) { if (threadIdx.x == 0) mb_set_error(err, MB_ERR_TOKEN_RANGE); tok = 0; }
    for (int j = threadIdx.x; j < W; j += blockDim.x)
        mb_store(out + (size_t)n * W + j, gelu_tanh(mb_load(z + (size_t)n * W + j)) * mb_load(table + (size_t)tok * table_stride + off + j));
}

template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ o, const T* __restrict__ gate, int gate_stride, int C, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / C;
    const int c = (int)(i - n * C);
    const float g = mb_load(gate + (size_t)n * gate_stride + c);
    mb_store(o + i, mb_load(o + i) / (1.0f + expf(-g)));
}

// out[n, h, j] = sum_i in[n, h, i] W[h sh + i si + j sj].  COLS (sj == 1): a thread per j, i ascending.  Otherwise
// (si == 1): a warp per j, lanes over i, a fixed tree.  A block per (token, head); the input row sits in shared memory.
template <typename T, bool COLS>
__global__ void head_product_kernel(const T* __restrict__ in, const T* __restrict__ W, T* __restrict__ out, int H, int I, int J,
                                    long long sh, long long si, long long sj, int in_head, int out_head) {
    // in_head, out_head: the distance between two heads of a row (a head's values may be part of a longer stretch)
    extern __shared__ float xin[];
    const int n = blockIdx.x, h = blockIdx.y;
    for (int i = threadIdx.x; i < I; i += blockDim.x) xin[i] = mb_load(in + ((size_t)n * H + h) * in_head + i);
    __syncthreads();
    const T* Wh = W + (size_t)h * sh;
    T* o = out + ((size_t)n * H + h) * out_head;
    if (COLS) {
        for (int j = threadIdx.x; j < J; j += blockDim.x) {
            float acc = 0.0f;
            for (int i = 0; i < I; i++) acc = fmaf(xin[i], mb_load(Wh + (size_t)i * si + j), acc);
            mb_store(o + j, acc);
        }
    } else {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        for (int j = warp; j < J; j += nwarp) {
            float acc = 0.0f;
            for (int i = lane; i < I; i += 32) acc = fmaf(xin[i], mb_load(Wh + (size_t)j * sj + i), acc);
            acc = mb_warp_sum(acc);
            if (lane == 0) mb_store(o + j, acc);
        }
    }
}

__global__ void scale_rows_kernel(float* __restrict__ y, float s, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] *= s;
}

static inline int row_threads(int D) { return D >= 1024 ? 256 : D >= 256 ? 128 : 64; }

template <typename T>
static int embed_pos_launch(const int* tokens, const int* positions, const T* table, const T* pos, float* x, int N, int D,
                            int V, int P, float scale, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || V < 1 || P < 1) return -2;
    embed_pos_kernel<T><<<N, row_threads(D), 0, st>>>(tokens, positions, table, pos, x, D, V, P, scale, err);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int post_norm_add_launch(float* x, const T* delta, const float* post_w, float post_eps, const float* next_w,
                                float next_eps, T* normed, T* copy, int N, int D, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || D > 12000 || (normed && !next_w)) return -2;
    const bool vec = D % 4 == 0 && !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) |
                                     reinterpret_cast<uintptr_t>(post_w) | reinterpret_cast<uintptr_t>(next_w) |
                                     reinterpret_cast<uintptr_t>(normed) | reinterpret_cast<uintptr_t>(copy)) & 15);
    if (vec)
        post_norm_add_kernel<T, true><<<N, D >= 2048 ? 256 : D >= 512 ? 128 : 64, (size_t)D * sizeof(float), st>>>(
            x, delta, post_w, post_eps, next_w, next_eps, normed, copy, D);
    else
        post_norm_add_kernel<T, false><<<N, row_threads(D), (size_t)D * sizeof(float), st>>>(x, delta, post_w, post_eps, next_w,
                                                                                             next_eps, normed, copy, D);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int rms_segments_launch(const T* in, int stride, int off_a, int wa, const float* w_a, T* out_a, int off_b, int wb,
                               const float* w_b, T* pool, const int* positions, const int* tok_row, const int* table,
                               int max_blocks, int page, int num_pages, float eps, int N, int* err, cudaStream_t st,
                               int pool_row = 0) {
    if (N == 0) return 0;
    if (pool_row == 0) pool_row = wb;
    if (wa < 0 || wb < 0 || pool_row < wb || (wb > 0 && (!pool || !table || page < 1))) return -2;
    const int W = wa > wb ? wa : wb;
    if (W == 0) return 0;
    rms_segments_kernel<T><<<dim3(N, wb > 0 ? 2 : 1), row_threads(W), 0, st>>>(in, stride, off_a, wa, w_a, out_a, off_b, wb,
                                                                              w_b, pool, positions, tok_row, table,
                                                                              max_blocks, page, num_pages, eps, err, pool_row);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int gated_gather_launch(const T* z, const int* tokens, const T* table, int table_stride, int off, T* out, int N, int W,
                               int V, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (W < 1) return -2;
    gated_gather_kernel<T><<<N, row_threads(W), 0, st>>>(z, tokens, table, table_stride, off, out, W, V, err);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int sigmoid_mul_launch(T* o, const T* gate, int gate_stride, int N, int C, cudaStream_t st) {
    if (N == 0) return 0;
    const long long total = (long long)N * C;
    sigmoid_mul_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(o, gate, gate_stride, C, total);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int head_product_launch(const T* in, const T* W, T* out, int N, int H, int I, int J, long long sh, long long si,
                               long long sj, cudaStream_t st, int in_head = 0, int out_head = 0) {
    if (N == 0) return 0;
    if (in_head == 0) in_head = I;
    if (out_head == 0) out_head = J;
    if (H < 1 || H > 65535 || I < 1 || J < 1 || I > 12000 || (sj != 1 && si != 1) || in_head < I || out_head < J) return -2;
    const dim3 grid(N, H);
    if (sj == 1)
        head_product_kernel<T, true><<<grid, J >= 256 ? 256 : J >= 128 ? 128 : 64, (size_t)I * sizeof(float), st>>>(
            in, W, out, H, I, J, sh, si, sj, in_head, out_head);
    else
        head_product_kernel<T, false><<<grid, 256, (size_t)I * sizeof(float), st>>>(in, W, out, H, I, J, sh, si, sj,
                                                                                    in_head, out_head);
    MB_LAUNCH_CHECK();
    return 0;
}

#define ROWWISE_API(SUF, T)                                                                                               \
    MB_API int mb_embed_pos_##SUF(const int* tokens, const int* positions, const void* table, const void* pos, float* x,  \
                                  int N, int D, int V, int P, float scale, int* err, cudaStream_t st) {                   \
        return embed_pos_launch<T>(tokens, positions, (const T*)table, (const T*)pos, x, N, D, V, P, scale, err, st);      \
    }                                                                                                                     \
    MB_API int mb_post_norm_add_##SUF(float* x, const void* delta, const float* post_w, float post_eps,                  \
                                      const float* next_w, float next_eps, void* normed, void* copy, int N, int D,        \
                                      cudaStream_t st) {                                                                  \
        return post_norm_add_launch<T>(x, (const T*)delta, post_w, post_eps, next_w, next_eps, (T*)normed, (T*)copy, N,   \
                                       D, st);                                                                            \
    }                                                                                                                     \
    MB_API int mb_rms_segments_##SUF(const void* in, int stride, int off_a, int wa, const float* w_a, void* out_a,       \
                                     int off_b, int wb, const float* w_b, void* pool, const int* positions,               \
                                     const int* tok_row, const int* table, int max_blocks, int page, int num_pages,       \
                                     float eps, int N, int* err, cudaStream_t st) {                                       \
        return rms_segments_launch<T>((const T*)in, stride, off_a, wa, w_a, (T*)out_a, off_b, wb, w_b, (T*)pool,          \
                                      positions, tok_row, table, max_blocks, page, num_pages, eps, N, err, st);           \
    }                                                                                                                     \
    MB_API int mb_rms_segments_wide_##SUF(const void* in, int stride, int off_a, int wa, const float* w_a, void* out_a,  \
                                          int off_b, int wb, const float* w_b, void* pool, int pool_row,                  \
                                          const int* positions, const int* tok_row, const int* table, int max_blocks,     \
                                          int page, int num_pages, float eps, int N, int* err, cudaStream_t st) {         \
        return rms_segments_launch<T>((const T*)in, stride, off_a, wa, w_a, (T*)out_a, off_b, wb, w_b, (T*)pool,          \
                                      positions, tok_row, table, max_blocks, page, num_pages, eps, N, err, st, pool_row); \
    }                                                                                                                     \
    MB_API int mb_gated_gather_##SUF(const void* z, const int* tokens, const void* table, int table_stride, int off,     \
                                     void* out, int N, int W, int V, int* err, cudaStream_t st) {                         \
        return gated_gather_launch<T>((const T*)z, tokens, (const T*)table, table_stride, off, (T*)out, N, W, V, err,     \
                                      st);                                                                                \
    }                                                                                                                     \
    MB_API int mb_sigmoid_mul_##SUF(void* o, const void* gate, int gate_stride, int N, int C, cudaStream_t st) {         \
        return sigmoid_mul_launch<T>((T*)o, (const T*)gate, gate_stride, N, C, st);                                       \
    }                                                                                                                     \
    MB_API int mb_head_product_##SUF(const void* in, const void* W, void* out, int N, int H, int I, int J, long long sh,  \
                                     long long si, long long sj, cudaStream_t st) {                                       \
        return head_product_launch<T>((const T*)in, (const T*)W, (T*)out, N, H, I, J, sh, si, sj, st);                    \
    }                                                                                                                     \
    MB_API int mb_head_product_strided_##SUF(const void* in, int in_head, const void* W, void* out, int out_head, int N,  \
                                             int H, int I, int J, long long sh, long long si, long long sj,               \
                                             cudaStream_t st) {                                                           \
        return head_product_launch<T>((const T*)in, (const T*)W, (T*)out, N, H, I, J, sh, si, sj, st, in_head, out_head); \
    }

ROWWISE_API(f32, float)
ROWWISE_API(bf16, bf16)

MB_API int mb_scale_rows(float* y, float s, long long total, cudaStream_t st) {
    if (total == 0) return 0;
    scale_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(y, s, total);
    MB_LAUNCH_CHECK();
    return 0;
}
