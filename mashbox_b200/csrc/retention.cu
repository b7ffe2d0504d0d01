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
//   the split form   the same recurrence for long stretches.  The decay is a constant of the head, so a sequence can be
//                    cut into segments that run side by side: every segment is scanned from a zero state (the first one
//                    from the sequence's own), which gives the part of every o that the segment's own tokens make and
//                    the state E_j the segment adds; a small kernel chains S0_(j+1) = decay^n S0_j + E_j; a second pass
//                    adds decay^(t+1) S0_j^T q_t to the t-th token of segment j.  All of it in float32.
#include "common.cuh"

#define RT_THREADS 128
#define RT_LANES 8
#define RT_BATCH 8
#define RT_STAGES 4

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

// two floats in one 64-bit register pair, and the fused multiply-add on such pairs (one issue slot, two results, each
// rounded as the single one is)
__device__ __forceinline__ uint64_t rt_pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void rt_unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t rt_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// global to shared memory without a register in between; size 0: the destination is set to zero
__device__ __forceinline__ void rt_cp16(float* smem, const float* gmem, int size) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(size));
}
__device__ __forceinline__ void rt_cp4(float* smem, const float* gmem, int size) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(size));
}

// The stretch of tokens a block walks.  Whole sequences: block z is sequence z.  Segments: a sequence of n tokens is cut
// into ceil(n / seg) segments, numbered through all sequences in order; block z finds its own by walking the lengths
// (there are few sequences in a step).  Returns false for a block beyond the last segment.
struct RtStretch {
    int s, j, first, len, z0;       // sequence, segment within it, first token, tokens, number of the sequence's segment 0
};
__device__ __forceinline__ bool rt_find(int z, int S, int seg, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                        RtStretch& r) {
    int base = 0;
    for (int s = 0; s < S; s++) {
        const int n = q_len[s], ns = (n + seg - 1) / seg;
        if (z < base + ns) {
            r.s = s; r.j = z - base; r.z0 = base;
            r.first = q_start[s] + r.j * seg;
            r.len = min(seg, n - r.j * seg);
            return true;
        }
        base += ns;
    }
    return false;
}

// grid (column tiles, H, sequences or segments), RT_THREADS threads: RT_THREADS / RT_LANES columns a block.  A thread
// holds 4 R4 values of its column, channels r4 * 4 RT_LANES + 4 lane + (0..3): the lanes of a column read one contiguous
// stretch of a token's q and k from shared memory, 16 bytes each, and the columns of a warp read the same one.
// dim <= 4 R4 RT_LANES.  The tokens' q, k, v come through a ring of RT_STAGES stages of RT_BATCH tokens, copied
// asynchronously: DRAM is a microsecond away and a stage is worked through in a fraction of that.
//   MODE 0  whole sequences: the state comes from the sequence's slot and goes back there
//   MODE 1  segments: segment 0 starts from the slot, the others from zero; the state a segment ends with goes to
//           carry[z]; o holds what the segment's own tokens (and for segment 0 the slot's state) give
//   MODE 2  the rest of o for the segments after the first: carry[z] now holds the state S0 the segment starts from,
//           and o_t += decay^(t+1) S0^T q_t for its t-th token; nothing is written but o
template <int R4, int MODE>
__global__ void __launch_bounds__(RT_THREADS)
retention_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ decay, float* __restrict__ o, float* __restrict__ state,
                      long long state_stride, int state_vec, float* __restrict__ carry, const int* __restrict__ q_start,
                      const int* __restrict__ q_len, const int* __restrict__ state_slot, int S, int seg, int H, int dim,
                      int vdim) {
    constexpr int DP = 4 * R4 * RT_LANES, COLS = RT_THREADS / RT_LANES, BT = RT_BATCH;
    extern __shared__ __align__(16) float ring[];
    typedef float (*RowsDP)[BT][DP];
    typedef float (*RowsC)[BT][COLS];
    RowsDP sq = reinterpret_cast<RowsDP>(ring), sk = sq + RT_STAGES;
    RowsC sv = reinterpret_cast<RowsC>(ring + 2 * RT_STAGES * BT * DP);
    const int h = blockIdx.y, col0 = blockIdx.x * COLS;
    const int lane = threadIdx.x & (RT_LANES - 1), cg = threadIdx.x / RT_LANES, col = col0 + cg;
    RtStretch w;
    if (MODE == 0) {
        w.s = blockIdx.z; w.j = 0; w.z0 = 0; w.first = q_start[w.s]; w.len = q_len[w.s];
    } else {
        if (!rt_find(blockIdx.z, S, seg, q_start, q_len, w)) return;
        if (MODE == 2 && w.j == 0) return;
    }
    const int a = w.first, len = w.len;
    const float dec = decay[h];
    const bool in = col < vdim;
    const size_t head_off = ((size_t)h * vdim + (in ? col : 0)) * dim;
    float* slot = state + (size_t)state_slot[w.s] * state_stride + head_off;
    float* mine = MODE == 0 ? slot : carry + (size_t)blockIdx.z * H * vdim * dim + head_off;
    const float* src = MODE == 2 ? mine : ((MODE == 0 || w.j == 0) ? slot : nullptr);
    const bool src_vec = (dim & 3) == 0 && (MODE == 2 || state_vec);
    float* dst = MODE == 2 ? nullptr : mine;
    const bool dst_vec = (dim & 3) == 0 && (MODE == 1 || state_vec);
    uint64_t st[2 * R4];            // the column in pairs: channels (i, i + 1)
#pragma unroll
    for (int r4 = 0; r4 < R4; r4++) {
        const int i = r4 * 4 * RT_LANES + lane * 4;
        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (src && in) {
            if (src_vec) {
                if (i < dim) x = *reinterpret_cast<const float4*>(src + i);
            } else {
                if (i < dim) x.x = src[i];
                if (i + 1 < dim) x.y = src[i + 1];
                if (i + 2 < dim) x.z = src[i + 2];
                if (i + 3 < dim) x.w = src[i + 3];
            }
        }
        st[2 * r4] = rt_pack2(x.x, x.y);
        st[2 * r4 + 1] = rt_pack2(x.z, x.w);
    }
    // 16 bytes a copy where every row starts on a 16-byte boundary (dim and vdim multiples of 4), else 4
    const bool vec = (dim & 3) == 0 && (vdim & 3) == 0;
    auto fetch = [&](int buf, int t0) {
        const int nb = min(BT, len - t0);
        if (vec) {
            for (int idx = threadIdx.x; idx < nb * (DP / 4); idx += RT_THREADS) {
                const int tt = idx / (DP / 4), i = (idx - tt * (DP / 4)) * 4;
                const size_t n = (size_t)(a + t0 + tt);
                const int sz = i < dim ? 16 : 0, ii = i < dim ? i : 0;
                rt_cp16(&sq[buf][tt][i], q + (n * H + h) * dim + ii, sz);
                if (MODE != 2) rt_cp16(&sk[buf][tt][i], k + (n * H + h) * dim + ii, sz);
            }
            if (MODE != 2)
                for (int idx = threadIdx.x; idx < nb * (COLS / 4); idx += RT_THREADS) {
                    const int tt = idx / (COLS / 4), c = (idx - tt * (COLS / 4)) * 4;
                    const bool ok = col0 + c < vdim;
                    rt_cp16(&sv[buf][tt][c], v + ((size_t)(a + t0 + tt) * H + h) * vdim + (ok ? col0 + c : 0), ok ? 16 : 0);
                }
        } else {
            for (int idx = threadIdx.x; idx < nb * DP; idx += RT_THREADS) {
                const int tt = idx / DP, i = idx - tt * DP;
                const size_t n = (size_t)(a + t0 + tt);
                const int sz = i < dim ? 4 : 0, ii = i < dim ? i : 0;
                rt_cp4(&sq[buf][tt][i], q + (n * H + h) * dim + ii, sz);
                if (MODE != 2) rt_cp4(&sk[buf][tt][i], k + (n * H + h) * dim + ii, sz);
            }
            if (MODE != 2)
                for (int idx = threadIdx.x; idx < nb * COLS; idx += RT_THREADS) {
                    const int tt = idx / COLS, c = idx - tt * COLS;
                    const bool ok = col0 + c < vdim;
                    rt_cp4(&sv[buf][tt][c], v + ((size_t)(a + t0 + tt) * H + h) * vdim + (ok ? col0 + c : 0), ok ? 4 : 0);
                }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // every iteration commits one group (an empty one beyond the end), so the group of the stage that is worked on next
    // is always the (RT_STAGES - 1)-th from the newest
    for (int p = 0; p < RT_STAGES - 1; p++) {
        if (p * BT < len) fetch(p, p * BT);
        else asm volatile("cp.async.commit_group;\n" ::);
    }
    const uint64_t zero2 = rt_pack2(0.0f, 0.0f), dec2 = rt_pack2(dec, dec);
    for (int t0 = 0, it = 0; t0 < len; t0 += BT, it++) {
        const int nb = min(BT, len - t0), buf = it % RT_STAGES;
        const int ahead = t0 + (RT_STAGES - 1) * BT;
        if (ahead < len) fetch((it + RT_STAGES - 1) % RT_STAGES, ahead);       // the stage worked on last iteration is free
        else asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(RT_STAGES - 1));
        __syncthreads();
        float pw = MODE == 2 ? powf(dec, (float)(t0 + 1)) : 0.0f;              // decay^(t + 1) at the stage's first token
#pragma unroll 2
        for (int tt = 0; tt < nb; tt++) {
            uint64_t asum0 = zero2, asum1 = zero2;
            if (MODE != 2) {
                const float vv = sv[buf][tt][cg];
                const uint64_t v2 = rt_pack2(vv, vv);
#pragma unroll
                for (int r4 = 0; r4 < R4; r4++) {
                    const float4 kk = *reinterpret_cast<const float4*>(&sk[buf][tt][r4 * 4 * RT_LANES + lane * 4]);
                    const float4 qq = *reinterpret_cast<const float4*>(&sq[buf][tt][r4 * 4 * RT_LANES + lane * 4]);
                    // the decayed value is a product rounded once; the new key and value are added by one fused step
                    st[2 * r4] = rt_fma2(rt_pack2(kk.x, kk.y), v2, rt_fma2(st[2 * r4], dec2, zero2));
                    st[2 * r4 + 1] = rt_fma2(rt_pack2(kk.z, kk.w), v2, rt_fma2(st[2 * r4 + 1], dec2, zero2));
                    asum0 = rt_fma2(st[2 * r4], rt_pack2(qq.x, qq.y), asum0);
                    asum1 = rt_fma2(st[2 * r4 + 1], rt_pack2(qq.z, qq.w), asum1);
                }
            } else {
#pragma unroll
                for (int r4 = 0; r4 < R4; r4++) {
                    const float4 qq = *reinterpret_cast<const float4*>(&sq[buf][tt][r4 * 4 * RT_LANES + lane * 4]);
                    asum0 = rt_fma2(st[2 * r4], rt_pack2(qq.x, qq.y), asum0);
                    asum1 = rt_fma2(st[2 * r4 + 1], rt_pack2(qq.z, qq.w), asum1);
                }
            }
            float a0, a1, a2, a3;
            rt_unpack2(asum0, a0, a1);
            rt_unpack2(asum1, a2, a3);
            float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int m = 1; m < RT_LANES; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (lane == 0 && in) {
                float* dsto = o + ((size_t)(a + t0 + tt) * H + h) * vdim + col;
                if (MODE == 2) *dsto = fmaf(pw, acc, *dsto);
                else *dsto = acc;
            }
            if (MODE == 2) pw *= dec;
        }
        __syncthreads();
    }
    if (dst && in) {
#pragma unroll
        for (int r4 = 0; r4 < R4; r4++) {
            const int i = r4 * 4 * RT_LANES + lane * 4;
            float4 x;
            rt_unpack2(st[2 * r4], x.x, x.y);
            rt_unpack2(st[2 * r4 + 1], x.z, x.w);
            if (dst_vec) {
                if (i < dim) *reinterpret_cast<float4*>(dst + i) = x;
            } else {
                if (i < dim) dst[i] = x.x;
                if (i + 1 < dim) dst[i + 1] = x.y;
                if (i + 2 < dim) dst[i + 2] = x.z;
                if (i + 3 < dim) dst[i + 3] = x.w;
            }
        }
    }
}

// Between the two passes over the segments: carry[z] comes in as the state segment z ends with when it starts from
// zero (segment 0: from the slot's state), E_j, and leaves as the state segment z starts from,
//     S0_0 = 0,   S0_(j+1) = decay^(n_j) S0_j + E_j        (n_j tokens in segment j)
// and what the last segment ends with goes to the sequence's slot.  grid (blocks over H vdim dim, sequences): a thread
// owns one value of the state and walks the sequence's segments in order.
__global__ void retention_carry_kernel(float* __restrict__ carry, const float* __restrict__ decay, float* __restrict__ state,
                                       long long state_stride, const int* __restrict__ q_len,
                                       const int* __restrict__ state_slot, int seg, int H, int dim, int vdim) {
    const int s = blockIdx.y;
    const size_t per = (size_t)H * vdim * dim, e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    int z0 = 0;
    for (int i = 0; i < s; i++) z0 += (q_len[i] + seg - 1) / seg;
    const int n = q_len[s], ns = (n + seg - 1) / seg;
    if (ns == 0) return;
    const float dec = decay[e / ((size_t)vdim * dim)], whole = powf(dec, (float)seg);
    float cur = 0.0f;
    for (int j = 0; j < ns; j++) {
        float* p = carry + (size_t)(z0 + j) * per + e;
        const float end = *p;
        *p = cur;
        const int nj = min(seg, n - j * seg);
        cur = fmaf(nj == seg ? whole : powf(dec, (float)nj), cur, end);
    }
    state[(size_t)state_slot[s] * state_stride + e] = cur;
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

static size_t rt_smem(int R4) {
    return (size_t)RT_STAGES * RT_BATCH * (2 * 4 * R4 * RT_LANES + RT_THREADS / RT_LANES) * sizeof(float);
}

template <int R4, int MODE>
static int rt_launch(dim3 grid, const float* q, const float* k, const float* v, const float* decay, float* o, float* state,
                     long long state_stride, float* carry, const int* q_start, const int* q_len, const int* state_slot,
                     int S, int seg, int H, int dim, int vdim, cudaStream_t st) {
    const size_t smem = rt_smem(R4);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(retention_scan_kernel<R4, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // 16-byte reads and writes of a slot's state need every column to start on such a boundary
    const int state_vec = ((uintptr_t)state & 15) == 0 && (state_stride & 3) == 0 && (dim & 3) == 0;
    retention_scan_kernel<R4, MODE><<<grid, RT_THREADS, smem, st>>>(q, k, v, decay, o, state, state_stride, state_vec, carry,
                                                                    q_start, q_len, state_slot, S, seg, H, dim, vdim);
    MB_LAUNCH_CHECK();
    return 0;
}

#define RT_DISPATCH(MODE, ...)                                           \
    (dim <= 32 ? rt_launch<1, MODE>(__VA_ARGS__)                         \
     : dim <= 64 ? rt_launch<2, MODE>(__VA_ARGS__)                       \
     : dim <= 128 ? rt_launch<4, MODE>(__VA_ARGS__) : rt_launch<8, MODE>(__VA_ARGS__))

MB_API int mb_retention_scan(const float* q, const float* k, const float* v, const float* decay, float* o, float* state,
                             long long state_stride, const int* q_start, const int* q_len, const int* state_slot, int S,
                             int H, int dim, int vdim, cudaStream_t st) {
    if (S == 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || dim < 1 || dim > 256 || vdim < 1) return -2;
    const int cols = RT_THREADS / RT_LANES;
    const dim3 grid((vdim + cols - 1) / cols, H, S);
    return RT_DISPATCH(0, grid, q, k, v, decay, o, state, state_stride, nullptr, q_start, q_len, state_slot, S, 0, H, dim, vdim,
                       st);
}

// N tokens in S sequences make at most N / seg + S segments; carry (carry_rows, H vdim dim) must hold as many rows.
MB_API int mb_retention_split(const float* q, const float* k, const float* v, const float* decay, float* o, float* state,
                              long long state_stride, const int* q_start, const int* q_len, const int* state_slot, int S,
                              int N, int H, int dim, int vdim, int seg, float* carry, int carry_rows, cudaStream_t st) {
    if (S == 0 || N == 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || dim < 1 || dim > 256 || vdim < 1 || seg < 1) return -2;
    const int most = N / seg + S;
    if (most > carry_rows || most > 65535 || ((uintptr_t)carry & 15)) return -2;
    const int cols = RT_THREADS / RT_LANES;
    const dim3 grid((vdim + cols - 1) / cols, H, most);
    int rc = RT_DISPATCH(1, grid, q, k, v, decay, o, state, state_stride, carry, q_start, q_len, state_slot, S, seg, H, dim,
                         vdim, st);
    if (rc) return rc;
    const size_t per = (size_t)H * vdim * dim;
    retention_carry_kernel<<<dim3((unsigned)((per + 255) / 256), S), 256, 0, st>>>(carry, decay, state, state_stride, q_len,
                                                                                  state_slot, seg, H, dim, vdim);
    MB_LAUNCH_CHECK();
    return RT_DISPATCH(2, grid, q, k, v, decay, o, state, state_stride, carry, q_start, q_len, state_slot, S, seg, H, dim,
                       vdim, st);
}
