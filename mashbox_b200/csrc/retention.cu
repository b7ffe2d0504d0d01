// Retention: linear attention with one fixed decay per head, no softmax and no denominator, carried from token to token
// in a float32 state.
//
// Per head, with S (dim, vdim) the state, for every token in order:
//     S <- decay S + k v^T;   o = S^T q
// Column c of S (the dim values that belong to value channel c) never meets another column, so a column is the unit
// of work: RT_LANES threads hold it in registers, the dot product with q is met by shuffles, and a block of a few
// columns walks a sequence's tokens in order.  A prompt of any length, a portion and a single decoded token are the
// same loop; the state is read once and written once per step, and every sum runs in a fixed order.  The state is
// kept transposed, (heads, vdim, dim), so that a column is one contiguous stretch.
//
//   retention_prep   from the product's rows [q | k | v | ...] in the storage type: the first R dims of every head of q
//                    and k turn by position * freq_i (dim i with dim i + R/2), k times a constant after that; q, k, v
//                    left in float32
//   retention_scan   the recurrence, token by token (decode steps, short portions, the whole float32 path)
//   retention_chunk  the same recurrence for long stretches, a chunk of RC_T tokens at a time: inside a chunk
//                    o_t = decay^(t+1) S0^T q_t + sum_(s <= t) decay^(t-s) (q_t . k_s) v_s, and
//                    S <- decay^n S0 + sum_s decay^(n-1-s) k_s v_s^T, all in float32; the tokens of a chunk run side by
//                    side instead of one after the other
#include "common.cuh"

#define RT_THREADS 128
#define RT_LANES 8
#define RT_BATCH 16

// grid (N, H).  rows (N, stride) holds q at q_off, k at k_off (H dim each), v at v_off (H vdim).
template <typename T>
__global__ void retention_prep_kernel(const T* __restrict__ rows, int stride, int q_off, int k_off, int v_off,
                                      const int* __restrict__ positions, const float* __restrict__ freqs,
                                      float* __restrict__ q, float* __restrict__ k, float* __restrict__ v, int H, int dim,
                                      int vdim, int R, float k_scale) {
    const int n = blockIdx.x, h = blockIdx.y, half = R / 2;
    const float p = (float)positions[n];
    const T* row = rows + (size_t)n * stride;
    const T* qs = row + q_off + (size_t)h * dim;
    const T* ks = row + k_off + (size_t)h * dim;
    float* qd = q + ((size_t)n * H + h) * dim;
    float* kd = k + ((size_t)n * H + h) * dim;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(p * freqs[i], &s, &c);
        const float qa = mb_load(qs + i), qb = mb_load(qs + i + half);
        const float ka = mb_load(ks + i), kb = mb_load(ks + i + half);
        qd[i] = qa * c - qb * s;
        qd[i + half] = qb * c + qa * s;
        kd[i] = (ka * c - kb * s) * k_scale;
        kd[i + half] = (kb * c + ka * s) * k_scale;
    }
    for (int i = 2 * half + threadIdx.x; i < dim; i += blockDim.x) {
        qd[i] = mb_load(qs + i);
        kd[i] = mb_load(ks + i) * k_scale;
    }
    const T* vs = row + v_off + (size_t)h * vdim;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) v[((size_t)n * H + h) * vdim + c] = mb_load(vs + c);
}

// grid (column tiles, H, sequences), RT_THREADS threads: RT_THREADS / RT_LANES columns a block.  A thread holds R
// values of its column: channels r * RT_LANES + lane, so that the lanes of a column read one contiguous stretch of a
// token's q and k from shared memory and the columns of a warp read the same one.  dim <= R * RT_LANES.
template <int R>
__global__ void __launch_bounds__(RT_THREADS)
retention_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ decay, float* __restrict__ o, float* __restrict__ state,
                      long long state_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                      const int* __restrict__ state_slot, int H, int dim, int vdim) {
    constexpr int DP = R * RT_LANES, COLS = RT_THREADS / RT_LANES, BT = RT_BATCH;
    __shared__ __align__(16) float sq[BT][DP];
    __shared__ __align__(16) float sk[BT][DP];
    __shared__ float sv[BT][COLS];
    const int s = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * COLS;
    const int lane = threadIdx.x & (RT_LANES - 1), cg = threadIdx.x / RT_LANES, col = col0 + cg;
    const int a = q_start[s], len = q_len[s];
    const float dec = decay[h];
    const bool in = col < vdim;
    float* S = state + (size_t)state_slot[s] * state_stride + ((size_t)h * vdim + (in ? col : 0)) * dim;
    float st[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = r * RT_LANES + lane;
        st[r] = (in && i < dim) ? S[i] : 0.0f;
    }
    for (int t0 = 0; t0 < len; t0 += BT) {
        const int nb = min(BT, len - t0);
        for (int idx = threadIdx.x; idx < nb * DP; idx += RT_THREADS) {
            const int tt = idx / DP, i = idx - tt * DP;
            const size_t n = (size_t)(a + t0 + tt);
            sq[tt][i] = i < dim ? q[(n * H + h) * dim + i] : 0.0f;
            sk[tt][i] = i < dim ? k[(n * H + h) * dim + i] : 0.0f;
        }
        for (int idx = threadIdx.x; idx < nb * COLS; idx += RT_THREADS) {
            const int tt = idx / COLS, c = idx - tt * COLS;
            sv[tt][c] = col0 + c < vdim ? v[((size_t)(a + t0 + tt) * H + h) * vdim + col0 + c] : 0.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; tt++) {
            const float vv = sv[tt][cg];
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
            for (int r = 0; r < R; r += 2) {
                st[r] = fmaf(sk[tt][r * RT_LANES + lane], vv, dec * st[r]);
                acc0 = fmaf(st[r], sq[tt][r * RT_LANES + lane], acc0);
                if (r + 1 < R) {
                    st[r + 1] = fmaf(sk[tt][(r + 1) * RT_LANES + lane], vv, dec * st[r + 1]);
                    acc1 = fmaf(st[r + 1], sq[tt][(r + 1) * RT_LANES + lane], acc1);
                }
            }
            float acc = acc0 + acc1;
#pragma unroll
            for (int m = 1; m < RT_LANES; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (lane == 0 && in) o[((size_t)(a + t0 + tt) * H + h) * vdim + col] = acc;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = r * RT_LANES + lane;
        if (in && i < dim) S[i] = st[r];
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The chunk form.  grid (column tiles of RC_COLS, H, sequences), RC_THREADS threads.  A block keeps its RC_COLS columns
// of the state in shared memory (dim x RC_COLS) and walks the sequence in chunks of RC_T tokens:
//   A[t][s] = decay^(t-s) (q_t . k_s) for s <= t      (RC_T x RC_T, every block of the head computes it: dim FMAs each)
//   o[t][c] = decay^(t+1) sum_i q_t[i] S[i][c] + sum_(s <= t) A[t][s] v_s[c]
//   S[i][c] = decay^n S[i][c] + sum_s decay^(n-1-s) k_s[i] v_s[c]
// Powers of the decay come from a table made once per block (decay^0 .. decay^RC_T, by repeated multiplication).
#define RC_T 32
#define RC_COLS 32
#define RC_THREADS 256
#define RC_MAX_DIM 256

__global__ void __launch_bounds__(RC_THREADS)
retention_chunk_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ decay, float* __restrict__ o, float* __restrict__ state,
                       long long state_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                       const int* __restrict__ state_slot, int H, int dim, int vdim) {
    extern __shared__ __align__(16) float sm[];
    const int DPAD = dim + 1;                       // rows of q and k one float longer: t-major reads hit different banks
    float* sS = sm;                                 // [dim][RC_COLS]
    float* sq = sS + (size_t)dim * RC_COLS;         // [RC_T][DPAD]
    float* sk = sq + RC_T * DPAD;                   // [RC_T][DPAD]
    float* sv = sk + RC_T * DPAD;                   // [RC_T][RC_COLS]
    float* sA = sv + RC_T * RC_COLS;                // [RC_T][RC_T + 1]
    float* pw = sA + RC_T * (RC_T + 1);             // [RC_T + 1]
    const int s = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * RC_COLS, tid = threadIdx.x;
    const int a = q_start[s], len = q_len[s];
    const float dec = decay[h];
    float* S = state + (size_t)state_slot[s] * state_stride + (size_t)h * vdim * dim;
    if (tid == 0) {
        float p = 1.0f;
        for (int i = 0; i <= RC_T; i++) { pw[i] = p; p *= dec; }
    }
    for (int idx = tid; idx < dim * RC_COLS; idx += RC_THREADS) {
        const int c = idx / dim, i = idx - c * dim;             // the stored state is (vdim, dim): i runs fastest
        sS[i * RC_COLS + c] = col0 + c < vdim ? S[(size_t)(col0 + c) * dim + i] : 0.0f;
    }
    __syncthreads();
    for (int t0 = 0; t0 < len; t0 += RC_T) {
        const int nb = min(RC_T, len - t0);
        for (int idx = tid; idx < RC_T * dim; idx += RC_THREADS) {
            const int tt = idx / dim, i = idx - tt * dim;
            const size_t n = (size_t)(a + t0 + tt);
            const bool ok = tt < nb;
            sq[tt * DPAD + i] = ok ? q[(n * H + h) * dim + i] : 0.0f;
            sk[tt * DPAD + i] = ok ? k[(n * H + h) * dim + i] : 0.0f;
        }
        for (int idx = tid; idx < RC_T * RC_COLS; idx += RC_THREADS) {
            const int tt = idx / RC_COLS, c = idx - tt * RC_COLS;
            sv[idx] = (tt < nb && col0 + c < vdim) ? v[((size_t)(a + t0 + tt) * H + h) * vdim + col0 + c] : 0.0f;
        }
        __syncthreads();
        // A: RC_T * RC_T entries over RC_THREADS threads
        for (int idx = tid; idx < RC_T * RC_T; idx += RC_THREADS) {
            const int t = idx / RC_T, u = idx - t * RC_T;
            float acc = 0.0f;
            if (u <= t && t < nb) {
                const float* qr = sq + t * DPAD;
                const float* kr = sk + u * DPAD;
                for (int i = 0; i < dim; i++) acc = fmaf(qr[i], kr[i], acc);
                acc *= pw[t - u];
            }
            sA[t * (RC_T + 1) + u] = acc;
        }
        __syncthreads();
        // o: RC_T * RC_COLS outputs; thread -> (t, c) with c fastest (the state's and v's reads run along banks)
        for (int idx = tid; idx < RC_T * RC_COLS; idx += RC_THREADS) {
            const int t = idx / RC_COLS, c = idx - t * RC_COLS;
            if (t >= nb) continue;
            float carried = 0.0f;
            const float* qr = sq + t * DPAD;
            for (int i = 0; i < dim; i++) carried = fmaf(qr[i], sS[i * RC_COLS + c], carried);
            float acc = carried * pw[t + 1];
            const float* ar = sA + t * (RC_T + 1);
            for (int u = 0; u <= t; u++) acc = fmaf(ar[u], sv[u * RC_COLS + c], acc);
            if (col0 + c < vdim) o[((size_t)(a + t0 + t) * H + h) * vdim + col0 + c] = acc;
        }
        __syncthreads();
        // the state moves on by the chunk's nb tokens
        const float all = pw[nb];
        for (int idx = tid; idx < dim * RC_COLS; idx += RC_THREADS) {
            const int i = idx / RC_COLS, c = idx - i * RC_COLS;
            float acc = sS[idx] * all;
            for (int u = 0; u < nb; u++) acc = fmaf(sk[u * DPAD + i] * pw[nb - 1 - u], sv[u * RC_COLS + c], acc);
            sS[idx] = acc;
        }
        __syncthreads();
    }
    for (int idx = tid; idx < dim * RC_COLS; idx += RC_THREADS) {
        const int c = idx / dim, i = idx - c * dim;
        if (col0 + c < vdim) S[(size_t)(col0 + c) * dim + i] = sS[i * RC_COLS + c];
    }
}

template <typename T>
static int retention_prep_launch(const T* rows, int stride, int q_off, int k_off, int v_off, const int* positions,
                                 const float* freqs, float* q, float* k, float* v, int N, int H, int dim, int vdim, int R,
                                 float k_scale, cudaStream_t st) {
    if (N == 0) return 0;
    if (H < 1 || H > 65535 || dim < 1 || vdim < 1 || R < 0 || R > dim || (R & 1) || (R > 0 && !freqs)) return -2;
    const int W = dim > vdim ? dim : vdim;
    retention_prep_kernel<T><<<dim3(N, H), W > 64 ? 128 : 64, 0, st>>>(rows, stride, q_off, k_off, v_off, positions, freqs, q, k,
                                                                      v, H, dim, vdim, R, k_scale);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_retention_prep_f32(const void* rows, int stride, int q_off, int k_off, int v_off, const int* positions,
                                 const float* freqs, float* q, float* k, float* v, int N, int H, int dim, int vdim, int R,
                                 float k_scale, cudaStream_t st) {
    return retention_prep_launch<float>((const float*)rows, stride, q_off, k_off, v_off, positions, freqs, q, k, v, N, H, dim,
                                        vdim, R, k_scale, st);
}

MB_API int mb_retention_prep_bf16(const void* rows, int stride, int q_off, int k_off, int v_off, const int* positions,
                                  const float* freqs, float* q, float* k, float* v, int N, int H, int dim, int vdim, int R,
                                  float k_scale, cudaStream_t st) {
    return retention_prep_launch<bf16>((const bf16*)rows, stride, q_off, k_off, v_off, positions, freqs, q, k, v, N, H, dim,
                                       vdim, R, k_scale, st);
}

MB_API int mb_retention_scan(const float* q, const float* k, const float* v, const float* decay, float* o, float* state,
                             long long state_stride, const int* q_start, const int* q_len, const int* state_slot, int S,
                             int H, int dim, int vdim, cudaStream_t st) {
    if (S == 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || dim < 1 || dim > 256 || vdim < 1) return -2;
    const int cols = RT_THREADS / RT_LANES;
    const dim3 grid((vdim + cols - 1) / cols, H, S);
#define RT_CASE(R)                                                                                                   \
    if (dim <= R * RT_LANES) {                                                                                         \
        retention_scan_kernel<R><<<grid, RT_THREADS, 0, st>>>(q, k, v, decay, o, state, state_stride, q_start, q_len,  \
                                                              state_slot, H, dim, vdim);                               \
        MB_LAUNCH_CHECK();                                                                                             \
        return 0;                                                                                                      \
    }
    RT_CASE(2) RT_CASE(4) RT_CASE(8) RT_CASE(16) RT_CASE(32)
#undef RT_CASE
    return -2;
}

MB_API int mb_retention_chunk(const float* q, const float* k, const float* v, const float* decay, float* o, float* state,
                              long long state_stride, const int* q_start, const int* q_len, const int* state_slot, int S,
                              int H, int dim, int vdim, cudaStream_t st) {
    if (S == 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || dim < 1 || dim > RC_MAX_DIM || vdim < 1) return -2;
    const size_t smem = ((size_t)dim * RC_COLS + 2 * RC_T * (dim + 1) + RC_T * RC_COLS + RC_T * (RC_T + 1) + RC_T + 1) * sizeof(float);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    retention_chunk_kernel<<<dim3((vdim + RC_COLS - 1) / RC_COLS, H, S), RC_THREADS, smem, st>>>(
        q, k, v, decay, o, state, state_stride, q_start, q_len, state_slot, H, dim, vdim);
    MB_LAUNCH_CHECK();
    return 0;
}
