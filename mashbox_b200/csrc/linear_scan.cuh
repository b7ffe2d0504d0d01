// The recurrence of a linear-attention layer whose state is a matrix per head, as one kernel template for its kinds:
//
//     MODE 0 (delta rule)       S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//     MODE 1 (gated, channels)  S <- diag(g) S + k v^T;  o = S^T q          g (N, H, dim): a decay per head and key channel
//     MODE 2 (gated, heads)     S <- g S + k v^T;  o = S^T q                g (N, H): one decay per head and token
//
// q and k come per group (G groups, head h reads group h / (H / G)), v per head; everything float32.  See the kernel's
// own comment for how the work is laid out.
#pragma once
#include "common.cuh"

#define DR_THREADS 128
#define DR_CPT 1            // columns a thread (more: what it reads of q, k, g from shared memory serves them all, but a
                            // sequence then gives fewer warps than the device has schedulers; 4 was slower at every size tried)
#define DR_BATCH 8
#define DR_STAGES 4

// two floats in one 64-bit register pair, and the fused multiply-add on such pairs
__device__ __forceinline__ uint64_t dr_pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void dr_unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t dr_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// 4 bytes from global to shared memory without a register in between; size 0: the destination is set to zero
__device__ __forceinline__ void dr_cp16(float* smem, const float* gmem, int size) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(size));
}
__device__ __forceinline__ void dr_cp4(float* smem, const float* gmem, int size) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(size));
}

__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// grid (column tiles, H, sequences), DR_THREADS threads: DR_THREADS / LANES groups of LANES threads, each group DR_CPT
// columns.  A thread holds 4 R4 values of each of its columns: channels r4 * 4 LANES + lane * 4 + c (r4 < R4, c < 4), so
// that its reads of a token's q, k, g are 16-byte loads, the lanes of a group read one contiguous stretch, and every
// value read serves DR_CPT columns; dim <= 4 R4 LANES = DP.  As many lanes as the key size allows (a whole warp from 128 on): a sequence gives
// heads x vdim x LANES threads, and one warp a scheduler cannot hide the latency of its own shared-memory reads and
// shuffles.  The next BT tokens are sent for (cp.async, zero fill beyond dim and vdim) while the current ones are
// worked on.
template <int LANES, int R4, int MODE>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ o,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ q_len, const int* __restrict__ state_slot, int H, int G, int dim, int vdim) {
    constexpr int DP = 4 * R4 * LANES, R = 4 * R4, CPT = DR_CPT, COLS = DR_THREADS / LANES * CPT, BT = DR_BATCH;
    // a ring of DR_STAGES stages of BT tokens: the inputs come from DRAM, a microsecond or two away, and a stage is worked
    // through in a fraction of that
    extern __shared__ __align__(16) float ring[];
    typedef float (*RowsDP)[BT][DP];
    typedef float (*RowsCP)[BT][COLS];
    typedef float (*RowsB)[BT];
    RowsDP sq = reinterpret_cast<RowsDP>(ring), sk = sq + DR_STAGES, sg = sk + DR_STAGES;
    RowsCP sv = reinterpret_cast<RowsCP>(ring + 3 * DR_STAGES * BT * DP);
    RowsB sb = reinterpret_cast<RowsB>(ring + 3 * DR_STAGES * BT * DP + DR_STAGES * BT * COLS);
    const int s = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * COLS;
    const int lane = threadIdx.x & (LANES - 1), cg = threadIdx.x / LANES, colA = col0 + cg * CPT;   // this thread's first column
    const int a = q_start[s], len = q_len[s], j = h / (H / G);
    float* S = state + (size_t)state_slot[s] * state_stride + (size_t)h * dim * vdim;
    uint64_t st[CPT][R / 2];                // the state values in pairs: channels (i, i + 1) of one column
#pragma unroll
    for (int c = 0; c < CPT; c++)
#pragma unroll
        for (int r4 = 0; r4 < R4; r4++)
#pragma unroll
            for (int x = 0; x < 4; x += 2) {
                const int i = r4 * 4 * LANES + lane * 4 + x;
                const bool in = colA + c < vdim;
                st[c][r4 * 2 + x / 2] = dr_pack2((in && i < dim) ? S[(size_t)i * vdim + colA + c] : 0.0f,
                                                 (in && i + 1 < dim) ? S[(size_t)(i + 1) * vdim + colA + c] : 0.0f);
            }
    // 16 bytes a copy where every row starts on a 16-byte boundary (dim and vdim multiples of 4), else 4
    const bool vec = (dim & 3) == 0 && (vdim & 3) == 0;
    auto fetch = [&](int buf, int t0) {
        const int nb = min(BT, len - t0);
        if (vec) {
            for (int idx = threadIdx.x; idx < nb * (DP / 4); idx += DR_THREADS) {
                const int tt = idx / (DP / 4), i = (idx - tt * (DP / 4)) * 4;
                const size_t n = (size_t)(a + t0 + tt);
                const int sz = i < dim ? 16 : 0;
                const int ii = i < dim ? i : 0;
                dr_cp16(&sq[buf][tt][i], q + (n * G + j) * dim + ii, sz);
                dr_cp16(&sk[buf][tt][i], k + (n * G + j) * dim + ii, sz);
                if (MODE != 2) dr_cp16(&sg[buf][tt][i], g + (n * H + h) * dim + ii, sz);
            }
            for (int idx = threadIdx.x; idx < nb * (COLS / 4); idx += DR_THREADS) {
                const int tt = idx / (COLS / 4), c = (idx - tt * (COLS / 4)) * 4;
                const bool in = col0 + c < vdim;
                dr_cp16(&sv[buf][tt][c], v + ((size_t)(a + t0 + tt) * H + h) * vdim + (in ? col0 + c : 0), in ? 16 : 0);
            }
        } else {
            for (int idx = threadIdx.x; idx < nb * DP; idx += DR_THREADS) {
                const int tt = idx / DP, i = idx - tt * DP;
                const size_t n = (size_t)(a + t0 + tt);
                const int sz = i < dim ? 4 : 0;
                const int ii = i < dim ? i : 0;
                dr_cp4(&sq[buf][tt][i], q + (n * G + j) * dim + ii, sz);
                dr_cp4(&sk[buf][tt][i], k + (n * G + j) * dim + ii, sz);
                if (MODE != 2) dr_cp4(&sg[buf][tt][i], g + (n * H + h) * dim + ii, sz);
            }
            for (int idx = threadIdx.x; idx < nb * COLS; idx += DR_THREADS) {
                const int tt = idx / COLS, c = idx - tt * COLS;
                const bool in = col0 + c < vdim;
                dr_cp4(&sv[buf][tt][c], v + ((size_t)(a + t0 + tt) * H + h) * vdim + (in ? col0 + c : 0), in ? 4 : 0);
            }
        }
        // one number per token and head: beta of the delta rule, or the head's decay
        if (MODE != 1 && threadIdx.x < nb)
            dr_cp4(&sb[buf][threadIdx.x], (MODE == 0 ? beta : g) + (size_t)(a + t0 + threadIdx.x) * H + h, 4);
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // every iteration commits one group (an empty one beyond the end), so the group of the stage that is worked on
    // next is always the (DR_STAGES - 1)-th from the newest
    for (int p = 0; p < DR_STAGES - 1; p++) {
        if (p * BT < len) fetch(p, p * BT);
        else asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int t0 = 0, it = 0; t0 < len; t0 += BT, it++) {
        const int nb = min(BT, len - t0), buf = it % DR_STAGES;
        const int ahead = t0 + (DR_STAGES - 1) * BT;
        if (ahead < len) fetch((it + DR_STAGES - 1) % DR_STAGES, ahead);      // the stage worked on last iteration is free
        else asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(DR_STAGES - 1));
        __syncthreads();
        if (MODE != 0) {
            // No delta step: nothing of a token's read-out feeds the next token, so the read-outs of a whole stage of tokens are met
            // together -- eight independent chains of shuffles in flight instead of one after every token.  The arithmetic
            // of a token is what it is in the other branch, in the same order.
            constexpr int TB = 8;
            for (int tt0 = 0; tt0 < nb; tt0 += TB) {
                float accs[TB][CPT];
#pragma unroll
                for (int j = 0; j < TB; j++) {
                    const int tt = tt0 + j;
#pragma unroll
                    for (int c = 0; c < CPT; c++) accs[j][c] = 0.0f;
                    if (tt < nb) {                      // the same for every thread of the block
                        uint64_t asum[CPT][2];
                        const uint64_t zero2 = dr_pack2(0.0f, 0.0f);
#pragma unroll
                        for (int c = 0; c < CPT; c++) asum[c][0] = asum[c][1] = zero2;
#pragma unroll
                        for (int r4 = 0; r4 < R4; r4++) {
                            float4 gg;
                            if (MODE == 2) gg.x = gg.y = gg.z = gg.w = sb[buf][tt];
                            else gg = *reinterpret_cast<const float4*>(&sg[buf][tt][r4 * 4 * LANES + lane * 4]);
                            const float4 kk = *reinterpret_cast<const float4*>(&sk[buf][tt][r4 * 4 * LANES + lane * 4]);
                            const float4 qq = *reinterpret_cast<const float4*>(&sq[buf][tt][r4 * 4 * LANES + lane * 4]);
                            const uint64_t g01 = dr_pack2(gg.x, gg.y), g23 = dr_pack2(gg.z, gg.w);
                            const uint64_t k01 = dr_pack2(kk.x, kk.y), k23 = dr_pack2(kk.z, kk.w);
                            const uint64_t q01 = dr_pack2(qq.x, qq.y), q23 = dr_pack2(qq.z, qq.w);
#pragma unroll
                            for (int c = 0; c < CPT; c++) {
                                const float uc = sv[buf][tt][cg * CPT + c];
                                const uint64_t u2 = dr_pack2(uc, uc);
                                st[c][r4 * 2] = dr_fma2(st[c][r4 * 2], g01, zero2);       // the decay: a product, rounded once
                                st[c][r4 * 2 + 1] = dr_fma2(st[c][r4 * 2 + 1], g23, zero2);
                                st[c][r4 * 2] = dr_fma2(k01, u2, st[c][r4 * 2]);
                                st[c][r4 * 2 + 1] = dr_fma2(k23, u2, st[c][r4 * 2 + 1]);
                                asum[c][0] = dr_fma2(st[c][r4 * 2], q01, asum[c][0]);
                                asum[c][1] = dr_fma2(st[c][r4 * 2 + 1], q23, asum[c][1]);
                            }
                        }
#pragma unroll
                        for (int c = 0; c < CPT; c++) {
                            float a0, a1, a2, a3;
                            dr_unpack2(asum[c][0], a0, a1);
                            dr_unpack2(asum[c][1], a2, a3);
                            accs[j][c] = (a0 + a1) + (a2 + a3);
                        }
                    }
                }
#pragma unroll
                for (int m = 1; m < LANES; m <<= 1)
#pragma unroll
                    for (int j = 0; j < TB; j++)
#pragma unroll
                        for (int c = 0; c < CPT; c++) accs[j][c] += __shfl_xor_sync(0xffffffffu, accs[j][c], m);
                if (lane == 0) {
#pragma unroll
                    for (int j = 0; j < TB; j++)
#pragma unroll
                        for (int c = 0; c < CPT; c++)
                            if (tt0 + j < nb && colA + c < vdim)
                                o[((size_t)(a + t0 + tt0 + j) * H + h) * vdim + colA + c] = accs[j][c];
                }
            }
        } else
#pragma unroll 2
        for (int tt = 0; tt < nb; tt++) {
            // a value of q, k, g read from shared memory serves the thread's CPT columns; the arithmetic runs on pairs
            // of floats (fma.rn.f32x2: one issue slot, two results, each rounded as the single one is)
            uint64_t dsum[CPT][2], asum[CPT][2], k2[R4][2];
            float dot[CPT], acc[CPT], u[CPT];
            const uint64_t zero2 = dr_pack2(0.0f, 0.0f);
#pragma unroll
            for (int c = 0; c < CPT; c++) dsum[c][0] = dsum[c][1] = asum[c][0] = asum[c][1] = zero2;
#pragma unroll
            for (int r4 = 0; r4 < R4; r4++) {
                float4 gg;
                if (MODE == 2) gg.x = gg.y = gg.z = gg.w = sb[buf][tt];
                else gg = *reinterpret_cast<const float4*>(&sg[buf][tt][r4 * 4 * LANES + lane * 4]);
                const float4 kk = *reinterpret_cast<const float4*>(&sk[buf][tt][r4 * 4 * LANES + lane * 4]);
                const uint64_t g01 = dr_pack2(gg.x, gg.y), g23 = dr_pack2(gg.z, gg.w);
                k2[r4][0] = dr_pack2(kk.x, kk.y);
                k2[r4][1] = dr_pack2(kk.z, kk.w);
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    st[c][r4 * 2] = dr_fma2(st[c][r4 * 2], g01, zero2);               // the decay: a product, rounded once
                    st[c][r4 * 2 + 1] = dr_fma2(st[c][r4 * 2 + 1], g23, zero2);
                    if (MODE == 0) {
                        dsum[c][0] = dr_fma2(st[c][r4 * 2], k2[r4][0], dsum[c][0]);
                        dsum[c][1] = dr_fma2(st[c][r4 * 2 + 1], k2[r4][1], dsum[c][1]);
                    }
                }
            }
            if (MODE == 0) {
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    float a0, a1, a2, a3;
                    dr_unpack2(dsum[c][0], a0, a1);
                    dr_unpack2(dsum[c][1], a2, a3);
                    dot[c] = (a0 + a1) + (a2 + a3);
                }
#pragma unroll
                for (int m = 1; m < LANES; m <<= 1)
#pragma unroll
                    for (int c = 0; c < CPT; c++) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], m);
                const float bt = sb[buf][tt];
#pragma unroll
                for (int c = 0; c < CPT; c++) u[c] = bt * (sv[buf][tt][cg * CPT + c] - dot[c]);
            } else {
#pragma unroll
                for (int c = 0; c < CPT; c++) { dot[c] = 0.0f; u[c] = sv[buf][tt][cg * CPT + c]; }
            }
#pragma unroll
            for (int r4 = 0; r4 < R4; r4++) {
                const float4 qq = *reinterpret_cast<const float4*>(&sq[buf][tt][r4 * 4 * LANES + lane * 4]);
                const uint64_t q01 = dr_pack2(qq.x, qq.y), q23 = dr_pack2(qq.z, qq.w);
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    const uint64_t u2 = dr_pack2(u[c], u[c]);
                    st[c][r4 * 2] = dr_fma2(k2[r4][0], u2, st[c][r4 * 2]);
                    st[c][r4 * 2 + 1] = dr_fma2(k2[r4][1], u2, st[c][r4 * 2 + 1]);
                    asum[c][0] = dr_fma2(st[c][r4 * 2], q01, asum[c][0]);
                    asum[c][1] = dr_fma2(st[c][r4 * 2 + 1], q23, asum[c][1]);
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; c++) {
                float a0, a1, a2, a3;
                dr_unpack2(asum[c][0], a0, a1);
                dr_unpack2(asum[c][1], a2, a3);
                acc[c] = (a0 + a1) + (a2 + a3);
            }
#pragma unroll
            for (int m = 1; m < LANES; m <<= 1)
#pragma unroll
                for (int c = 0; c < CPT; c++) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], m);
            if (lane == 0) {
#pragma unroll
                for (int c = 0; c < CPT; c++)
                    if (colA + c < vdim) o[((size_t)(a + t0 + tt) * H + h) * vdim + colA + c] = acc[c];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < CPT; c++)
#pragma unroll
        for (int r4 = 0; r4 < R4; r4++)
#pragma unroll
            for (int x = 0; x < 4; x += 2) {
                const int i = r4 * 4 * LANES + lane * 4 + x;
                float lo, hi;
                dr_unpack2(st[c][r4 * 2 + x / 2], lo, hi);
                if (colA + c < vdim && i < dim) S[(size_t)i * vdim + colA + c] = lo;
                if (colA + c < vdim && i + 1 < dim) S[(size_t)(i + 1) * vdim + colA + c] = hi;
            }
}

