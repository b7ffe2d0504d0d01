// Gated linear recurrences without a delta step -- S <- decay S + k v^T, o = S^T q, a matrix state per head in float32
// -- and what feeds them and reads them for two mixers:
//
//   gated linear attention: a decay per head and key channel, a = sigmoid(z)^(1/tau)
//     gla_gates   q times dim^-1/2, k, v widened to float32; a = exp(log_sigmoid(z + bias) / tau)
//   state-space duality (one decay per head and token, the state N x P per head; B is the key, C the query, dt x the value):
//     ssd_gates   x, B, C <- silu(convolved row + bias); dt = softplus(raw + dt_bias); v = dt x; k = B; q = C;
//                 decay = exp(-exp(A_log) dt)
//     ssd_out     y = o + D x;  y <- y silu(z);  each of `parts` equal stretches of a row divided by its own root mean
//                 square;  times a weight;  to the storage type
//   gated_scan    the recurrence itself (the kernel template shared with the delta rule; modes 1 and 2)
//
// Decays, their logarithms, softplus, dt, the state and the recurrence are float32 whatever the storage type.
#include "linear_scan.cuh"

__device__ __forceinline__ float gs_log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// grid (N, H).  rows (N, stride) = [q (H dim) | k (H dim) | v (H vdim) | ...]; z (N, H dim) float32.
template <typename T>
__global__ void gla_gates_kernel(const T* __restrict__ rows, int stride, const float* __restrict__ z,
                                 const float* __restrict__ zb, float inv_tau, float* __restrict__ q, float* __restrict__ k,
                                 float* __restrict__ v, float* __restrict__ g, int H, int dim, int vdim) {
    const int n = blockIdx.x, h = blockIdx.y;
    const T* row = rows + (size_t)n * stride;
    const float qs = 1.0f / sqrtf((float)dim);
    const size_t kd = ((size_t)n * H + h) * dim, vd = ((size_t)n * H + h) * vdim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        q[kd + i] = mb_load(row + (size_t)h * dim + i) * qs;
        k[kd + i] = mb_load(row + (size_t)(H + h) * dim + i);
        g[kd + i] = expf(gs_log_sigmoid(z[kd + i] + zb[(size_t)h * dim + i]) * inv_tau);
    }
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) v[vd + c] = mb_load(row + 2 * (size_t)H * dim + (size_t)h * vdim + c);
}

// grid (N, H + 2 G): blocks h < H make head h's values and decay, the others one group's B or C.
// xbc (N, H P + 2 G NS) = [x | B | C] after the convolution; dt (N, H) float32, raw.
template <typename T>
__global__ void ssd_gates_kernel(const T* __restrict__ xbc, const float* __restrict__ cb, const float* __restrict__ dt,
                                 const float* __restrict__ dt_bias, const float* __restrict__ A_log, float* __restrict__ q,
                                 float* __restrict__ k, float* __restrict__ v, float* __restrict__ g, int H, int G, int P,
                                 int NS) {
    const int n = blockIdx.x, b = blockIdx.y, C = H * P + 2 * G * NS;
    const T* row = xbc + (size_t)n * C;
    if (b < H) {
        const float step = dr_softplus(dt[(size_t)n * H + b] + dt_bias[b]);
        for (int c = threadIdx.x; c < P; c += blockDim.x) {
            const int ch = b * P + c;
            v[((size_t)n * H + b) * P + c] = step * dr_silu(mb_load(row + ch) + (cb ? cb[ch] : 0.0f));
        }
        if (threadIdx.x == 0) g[(size_t)n * H + b] = expf(-expf(A_log[b]) * step);
        return;
    }
    const int e = b - H, grp = e % G, off = H * P + (e < G ? 0 : G * NS) + grp * NS;
    float* dst = (e < G ? k : q) + ((size_t)n * G + grp) * NS;
    for (int i = threadIdx.x; i < NS; i += blockDim.x) dst[i] = dr_silu(mb_load(row + off + i) + (cb ? cb[off + i] : 0.0f));
}

// grid (N, parts): one stretch of inner / parts channels of a row.  o (N, H P) float32 from the recurrence; xbc as above
// (its first H P columns are x before bias and silu); z (N, z_stride), the gate's logits.
template <typename T>
__global__ void ssd_out_kernel(const float* __restrict__ o, const T* __restrict__ xbc, int xbc_stride,
                               const float* __restrict__ cb, const float* __restrict__ D, const T* __restrict__ z,
                               int z_stride, const float* __restrict__ w, T* __restrict__ out, int H, int P, int parts,
                               float eps) {
    extern __shared__ float vals[];
    __shared__ float scratch[32];
    const int n = blockIdx.x, part = blockIdx.y, inner = H * P, W = inner / parts, c0 = part * W;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const int c = c0 + i;
        const float x = dr_silu(mb_load(xbc + (size_t)n * xbc_stride + c) + (cb ? cb[c] : 0.0f));
        float y = fmaf(D[c / P], x, o[(size_t)n * inner + c]);
        y *= dr_silu(mb_load(z + (size_t)n * z_stride + c));
        vals[i] = y;
        ss = fmaf(y, y, ss);
    }
    const float r = 1.0f / sqrtf(mb_block_sum(ss, scratch) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) mb_store(out + (size_t)n * inner + c0 + i, vals[i] * r * w[c0 + i]);
}

#define GS_ENTRIES(SUF, T)                                                                                                 \
    MB_API int mb_gla_gates_##SUF(const void* rows, int stride, const float* z, const float* zb, float inv_tau, float* q,  \
                                  float* k, float* v, float* g, int N, int H, int dim, int vdim, cudaStream_t st) {        \
        if (N == 0) return 0;                                                                                              \
        if (H < 1 || H > 65535 || dim < 1 || vdim < 1) return -2;                                                          \
        gla_gates_kernel<T><<<dim3(N, H), (dim > vdim ? dim : vdim) > 64 ? 128 : 64, 0, st>>>(                             \
            (const T*)rows, stride, z, zb, inv_tau, q, k, v, g, H, dim, vdim);                                             \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }                                                                                                                      \
    MB_API int mb_ssd_gates_##SUF(const void* xbc, const float* cb, const float* dt, const float* dt_bias,                 \
                                  const float* A_log, float* q, float* k, float* v, float* g, int N, int H, int G, int P,  \
                                  int NS, cudaStream_t st) {                                                               \
        if (N == 0) return 0;                                                                                              \
        if (G < 1 || H % G || H + 2 * G > 65535 || P < 1 || NS < 1) return -2;                                             \
        ssd_gates_kernel<T><<<dim3(N, H + 2 * G), (P > NS ? P : NS) > 64 ? 128 : 64, 0, st>>>(                             \
            (const T*)xbc, cb, dt, dt_bias, A_log, q, k, v, g, H, G, P, NS);                                               \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }                                                                                                                      \
    MB_API int mb_ssd_out_##SUF(const float* o, const void* xbc, int xbc_stride, const float* cb, const float* D,          \
                                const void* z, int z_stride, const float* w, void* out, int N, int H, int P, int parts,    \
                                float eps, cudaStream_t st) {                                                              \
        if (N == 0) return 0;                                                                                              \
        if (H < 1 || P < 1 || parts < 1 || parts > 65535 || (H * P) % parts || H * P / parts > 12000) return -2;           \
        const int W = H * P / parts;                                                                                       \
        ssd_out_kernel<T><<<dim3(N, parts), W >= 1024 ? 256 : W >= 256 ? 128 : 64, (size_t)W * sizeof(float), st>>>(       \
            o, (const T*)xbc, xbc_stride, cb, D, (const T*)z, z_stride, w, (T*)out, H, P, parts, eps);                     \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }
GS_ENTRIES(f32, float)
GS_ENTRIES(bf16, bf16)

// per_head 0: g (N, H, dim); 1: g (N, H).  state (slots, ..): head h's matrix (dim, vdim) at h dim vdim.
MB_API int mb_gated_scan(const float* q, const float* k, const float* v, const float* g, float* o, float* state,
                         long long state_stride, const int* q_start, const int* q_len, const int* state_slot, int S, int H,
                         int G, int dim, int vdim, int per_head, int long_stretches, cudaStream_t st) {
    if (S == 0) return 0;
    if (G < 1 || H % G || H > 65535 || S > 65535 || dim < 1 || dim > 256 || vdim < 1) return -2;
#define GS_LAUNCH(LANES, R4, MODE)                                                                                         \
    {                                                                                                                      \
        const int cols = DR_THREADS / LANES * DR_CPT;                                                                      \
        const size_t smem = (size_t)DR_STAGES * DR_BATCH * (3 * 4 * R4 * LANES + cols + 1) * sizeof(float);                \
        static bool configured = false;                                                                                    \
        if (!configured && smem > 48 * 1024) {                                                                             \
            cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<LANES, R4, MODE>,                                       \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
            if (e != cudaSuccess) return (int)e;                                                                           \
            configured = true;                                                                                             \
        }                                                                                                                  \
        delta_rule_kernel<LANES, R4, MODE><<<dim3((vdim + cols - 1) / cols, H, S), DR_THREADS, smem, st>>>(                \
            q, k, v, g, nullptr, o, state, state_stride, q_start, q_len, state_slot, H, G, dim, vdim);                     \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }
#define GS_CASE(LANES, R4)                                                                                                 \
    if (dim <= 4 * R4 * LANES) {                                                                                           \
        if (per_head) GS_LAUNCH(LANES, R4, 2) else GS_LAUNCH(LANES, R4, 1)                                                 \
    }
    // Wide keys: more threads a column where sequences bring long stretches (a prompt gives few blocks, and the chain of one
    // token is shorter with fewer values a thread: 523 against 649 us on 2,048 tokens of 16 heads of 128 x 128), fewer where
    // every sequence brings a token or two (14.8 against 20.9 us on 8 sequences).
    GS_CASE(4, 1) GS_CASE(8, 1) GS_CASE(8, 2)
    if (long_stretches) { GS_CASE(16, 2) GS_CASE(32, 2) } else { GS_CASE(8, 4) GS_CASE(16, 4) }
#undef GS_CASE
#undef GS_LAUNCH
    return -2;
}
