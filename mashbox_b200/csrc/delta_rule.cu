// The gated delta rule with one decay per head and key channel, carried from token to token in a float32 state.
//
// Per head, with S (dim, vdim) the state, for every token in order:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// Column c of S (the dim values that belong to value channel c) never meets another column: S^T k and S^T q are dot
// products along a column, and the update adds k times the column's own u.  So a column is the unit of work: LANES
// threads hold it in registers, four values each (eight for the widest keys), the two dot products are partial sums
// (four chains a thread, added pairwise) met by shuffles, and a block of a few columns walks a sequence's tokens in
// order, reading the token's q, k, g (shared by all columns), v and beta from shared memory, BATCH tokens per barrier.  A prompt of any length, a
// portion and a single decoded token are the same loop; the state is read once and written once per step.  Every sum
// runs in a fixed order, so the result does not depend on how a prompt was cut into steps.
//
//   delta_gates   from the (convolved) q/k/v product and the small products: silu; q and k to unit vectors per head (q
//                 also times dim^-1/2); beta = sigmoid; g = exp(-exp(A) softplus(a + dt_bias)); all left in float32
//   delta_rule    the recurrence
//   gated_rms     o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) per head, to the storage type (w may be absent; the gate
//                 may be silu(gate) instead)
#include "common.cuh"

#include "linear_scan.cuh"

// grid (N, H): head h of token n.  qkv (N, 2 G dim + H vdim) = [q | k | v] after the convolution; low (N, low_stride)
// holds beta's logits in its first H columns; wide (N, H dim + H vdim) = [decay logits | gate logits].
template <typename T>
__global__ void delta_gates_kernel(const T* __restrict__ qkv, const T* __restrict__ low, int low_stride,
                                   const T* __restrict__ wide, const float* __restrict__ A_log,
                                   const float* __restrict__ dt_bias, float* __restrict__ q, float* __restrict__ k,
                                   float* __restrict__ v, float* __restrict__ g, float* __restrict__ beta, int H, int G,
                                   int dim, int vdim, float unit_eps) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, h = blockIdx.y, rep = H / G;
    const int C = 2 * G * dim + H * vdim;
    const T* row = qkv + (size_t)n * C;
    if (h % rep == 0) {
        const int j = h / rep;
        for (int which = 0; which < 2; which++) {
            const T* src = row + (size_t)which * G * dim + (size_t)j * dim;
            float ss = 0.0f;
            for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float a = dr_silu(mb_load(src + i)); ss = fmaf(a, a, ss); }
            ss = mb_block_sum(ss, scratch);
            const float r = (which == 0 ? 1.0f / sqrtf((float)dim) : 1.0f) / sqrtf(ss + unit_eps);
            float* dst = (which == 0 ? q : k) + ((size_t)n * G + j) * dim;
            for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = dr_silu(mb_load(src + i)) * r;
        }
    }
    for (int c = threadIdx.x; c < vdim; c += blockDim.x)
        v[((size_t)n * H + h) * vdim + c] = dr_silu(mb_load(row + 2 * (size_t)G * dim + (size_t)h * vdim + c));
    const float a = expf(A_log[h]);
    const T* w = wide + (size_t)n * ((size_t)H * dim + (size_t)H * vdim) + (size_t)h * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        g[((size_t)n * H + h) * dim + i] = expf(-a * dr_softplus(mb_load(w + i) + dt_bias[(size_t)h * dim + i]));
    if (threadIdx.x == 0) beta[(size_t)n * H + h] = dr_sigmoid(mb_load(low + (size_t)n * low_stride + h));
}

// grid (N, H): o (N, H vdim) float32 -> out in the storage type
template <typename T>
__global__ void gated_rms_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, int gate_off,
                                 const float* __restrict__ w, T* __restrict__ out, int H, int vdim, float eps, int silu) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, h = blockIdx.y;
    const float* src = o + ((size_t)n * H + h) * vdim;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
    ss = mb_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* gp = gate + (size_t)n * gate_stride + gate_off + (size_t)h * vdim;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        const float z = mb_load(gp + c);
        mb_store(out + ((size_t)n * H + h) * vdim + c, src[c] * r * (w ? w[c] : 1.0f) * (silu ? dr_silu(z) : dr_sigmoid(z)));
    }
}

template <typename T>
static int delta_gates_launch(const T* qkv, const T* low, int low_stride, const T* wide, const float* A_log,
                              const float* dt_bias, float* q, float* k, float* v, float* g, float* beta, int N, int H, int G,
                              int dim, int vdim, float unit_eps, cudaStream_t st) {
    if (N == 0) return 0;
    if (G < 1 || H % G || H > 65535 || dim < 1 || vdim < 1) return -2;
    const int W = dim > vdim ? dim : vdim;
    delta_gates_kernel<T><<<dim3(N, H), W > 64 ? 128 : 64, 0, st>>>(qkv, low, low_stride, wide, A_log, dt_bias, q, k, v, g,
                                                                    beta, H, G, dim, vdim, unit_eps);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_delta_gates_f32(const void* qkv, const void* low, int low_stride, const void* wide, const float* A_log,
                              const float* dt_bias, float* q, float* k, float* v, float* g, float* beta, int N, int H, int G,
                              int dim, int vdim, float unit_eps, cudaStream_t st) {
    return delta_gates_launch<float>((const float*)qkv, (const float*)low, low_stride, (const float*)wide, A_log, dt_bias, q,
                                     k, v, g, beta, N, H, G, dim, vdim, unit_eps, st);
}

MB_API int mb_delta_gates_bf16(const void* qkv, const void* low, int low_stride, const void* wide, const float* A_log,
                               const float* dt_bias, float* q, float* k, float* v, float* g, float* beta, int N, int H, int G,
                               int dim, int vdim, float unit_eps, cudaStream_t st) {
    return delta_gates_launch<bf16>((const bf16*)qkv, (const bf16*)low, low_stride, (const bf16*)wide, A_log, dt_bias, q, k,
                                    v, g, beta, N, H, G, dim, vdim, unit_eps, st);
}

// threads per column: 0 = as few as hold the keys at four values a thread; 8, 16 or 32 = that many (more values a thread)
static int dr_lanes = 0;
MB_API int mb_delta_rule_set_lanes(int lanes) { dr_lanes = lanes; return 0; }

MB_API int mb_delta_rule(const float* q, const float* k, const float* v, const float* g, const float* beta, float* o,
                         float* state, long long state_stride, const int* q_start, const int* q_len, const int* state_slot,
                         int S, int H, int G, int dim, int vdim, cudaStream_t st) {
    if (S == 0) return 0;
    if (G < 1 || H % G || H > 65535 || S > 65535 || dim < 1 || dim > 256 || vdim < 1) return -2;
#define DR_CASE(LANES, R4)                                                                                                 \
    if (dim <= 4 * R4 * LANES && (lanes == 0 || lanes == LANES)) {                                                         \
        const int cols = DR_THREADS / LANES * DR_CPT;                                                                      \
        const size_t smem = (size_t)DR_STAGES * DR_BATCH * (3 * 4 * R4 * LANES + cols + 1) * sizeof(float);                \
        static bool configured = false;                                                                                    \
        if (!configured && smem > 48 * 1024) {                                                                             \
            cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<LANES, R4, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                               \
            if (e != cudaSuccess) return (int)e;                                                                           \
            configured = true;                                                                                             \
        }                                                                                                                  \
        delta_rule_kernel<LANES, R4, 0><<<dim3((vdim + cols - 1) / cols, H, S), DR_THREADS, smem, st>>>(                      \
            q, k, v, g, beta, o, state, state_stride, q_start, q_len, state_slot, H, G, dim, vdim);                        \
        MB_LAUNCH_CHECK();                                                                                                 \
        return 0;                                                                                                          \
    }
    const int lanes = dr_lanes;
    DR_CASE(4, 1) DR_CASE(8, 1) DR_CASE(8, 2) DR_CASE(8, 4) DR_CASE(16, 1) DR_CASE(16, 2) DR_CASE(32, 1) DR_CASE(16, 4) DR_CASE(32, 2)
#undef DR_CASE
    return -2;
}

template <typename T>
static int gated_rms_launch(const float* o, const T* gate, int gate_stride, int gate_off, const float* w, T* out, int N,
                            int H, int vdim, float eps, int silu, cudaStream_t st) {
    if (N == 0) return 0;
    if (H < 1 || H > 65535 || vdim < 1) return -2;
    gated_rms_kernel<T><<<dim3(N, H), vdim > 64 ? 128 : vdim > 32 ? 64 : 32, 0, st>>>(o, gate, gate_stride, gate_off, w, out,
                                                                                     H, vdim, eps, silu);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_gated_rms_f32(const float* o, const void* gate, int gate_stride, int gate_off, const float* w, void* out, int N,
                            int H, int vdim, float eps, int silu, cudaStream_t st) {
    return gated_rms_launch<float>(o, (const float*)gate, gate_stride, gate_off, w, (float*)out, N, H, vdim, eps, silu, st);
}

MB_API int mb_gated_rms_bf16(const float* o, const void* gate, int gate_stride, int gate_off, const float* w, void* out, int N,
                             int H, int vdim, float eps, int silu, cudaStream_t st) {
    return gated_rms_launch<bf16>(o, (const bf16*)gate, gate_stride, gate_off, w, (bf16*)out, N, H, vdim, eps, silu, st);
}
