// A feed-forward made of many small experts of which every token uses a few.
//
//   moe_select     router logits z (N, E) float32 -> per token its `top` experts and their weights.  score s = sigmoid(z);
//                  the choice is made on c = s + correction; the experts form `groups` equal runs of neighbours, a group
//                  is worth the sum of its two largest c, and only experts of the `keep` best groups can be chosen;
//                  the weight of a chosen expert is its s (not renormalised).  Ties go to the lower index.
//   moe_experts    for every (token, chosen expert): g = min(Wg h, L), u = clamp(Wu h, -L, L),
//                  y = Wd (g sigmoid(alpha g) (u + 1)), left in float32 per (token, place)
//   moe_combine    out[n] = sum over the places, in order, of weight * y
//
// moe_experts is the form for steps of few tokens (and of float32): blocks per (token, expert) stream that expert's
// three matrices, which is what a decode step has to read anyway.  Dot products run over lanes with 16-byte loads where
// rows allow.
#include "common.cuh"
#include <math.h>

// index of the largest of vals[0..n) (lowest index on ties) over a warp; every lane gets it
__device__ __forceinline__ int warp_argmax(const float* vals, int n, int lane) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
        const float c = vals[i];
        if (c > best || (c == best && i < at)) { best = c; at = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    return at;
}

// one warp per token; dynamic shared: s[E], c[E], gs[groups], kept[groups]
// softmax: the scores are softmax(z) over all experts instead of sigmoid(z); worth_max: a group is worth its largest c
// instead of the sum of its two largest; scale multiplies the weights; a row of z is z_stride floats long
__global__ void moe_select_kernel(const float* __restrict__ z, int z_stride, const float* __restrict__ correction,
                                  int* __restrict__ ids, float* __restrict__ wts, int E, int top, int groups, int keep,
                                  int softmax, int worth_max, float scale) {
    extern __shared__ float sm[];
    float* s = sm;
    float* c = sm + E;
    float* gs = sm + 2 * E;
    float* kept = gs + groups;
    const int n = blockIdx.x, lane = threadIdx.x;
    const float* zr = z + (size_t)n * z_stride;
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
        m = mb_warp_max(m);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) { const float v = expf(zr[e] - m); s[e] = v; sum += v; }
        sum = mb_warp_sum(sum);
        for (int e = lane; e < E; e += 32) {
            const float v = s[e] / sum;
            s[e] = v;
            c[e] = v + (correction ? correction[e] : 0.0f);
        }
    } else {
        for (int e = lane; e < E; e += 32) {
            const float v = 1.0f / (1.0f + expf(-zr[e]));
            s[e] = v;
            c[e] = v + (correction ? correction[e] : 0.0f);
        }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int gi = lane; gi < groups; gi += 32) {
            float a = -INFINITY, b = -INFINITY;                  // the two largest of the group
            for (int e = gi * per; e < (gi + 1) * per; e++) {
                const float v = c[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[gi] = (per > 1 && !worth_max) ? a + b : a;
            kept[gi] = 0.0f;
        }
        __syncwarp();
        for (int kk = 0; kk < keep; kk++) {
            const int at = warp_argmax(gs, groups, lane);
            __syncwarp();
            if (lane == 0) { gs[at] = -INFINITY; kept[at] = 1.0f; }
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (kept[e / per] == 0.0f) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int kk = 0; kk < top; kk++) {
        const int at = warp_argmax(c, E, lane);
        __syncwarp();
        if (lane == 0) {
            ids[(size_t)n * top + kk] = at;
            wts[(size_t)n * top + kk] = s[at] * scale;
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
}

// sum over k of w[k] x[k], lanes side by side, x in shared memory (float); 16-byte loads of bf16 rows that allow them
__device__ __forceinline__ float lane_dot(const float* w, const float* x, int K, int lane) {
    float acc = 0.0f;
    if ((K & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
        const float4* w4 = reinterpret_cast<const float4*>(w);
        for (int i = lane; i < K / 4; i += 32) {
            const float4 a = w4[i];
            acc = fmaf(a.x, x[4 * i], acc); acc = fmaf(a.y, x[4 * i + 1], acc);
            acc = fmaf(a.z, x[4 * i + 2], acc); acc = fmaf(a.w, x[4 * i + 3], acc);
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(w[i], x[i], acc);
    }
    return mb_warp_sum(acc);
}

__device__ __forceinline__ float lane_dot(const bf16* w, const float* x, int K, int lane) {
    float acc = 0.0f;
    if ((K & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
        const uint4* w8 = reinterpret_cast<const uint4*>(w);
        for (int i = lane; i < K / 8; i += 32) {
            const uint4 a = w8[i];
            const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int p = 0; p < 4; p++) {
                acc = fmaf(__uint_as_float(u[p] << 16), x[8 * i + 2 * p], acc);
                acc = fmaf(__uint_as_float(u[p] & 0xffff0000u), x[8 * i + 2 * p + 1], acc);
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(__bfloat162float(w[i]), x[i], acc);
    }
    return mb_warp_sum(acc);
}

// Steps of few tokens, two kernels, each with a block per (pair, stretch of MOE_ROWS output rows) so that a step of a
// handful of tokens still fills the device: gate and up with the activation, (pairs, F) float32; then down, into
// y (N, top, D) float32.  Dynamic shared: the input row (D or F floats).  wg, wu (E, F, D); wd (E, D, F).
#define MOE_ROWS 32

template <typename T>
__global__ void moe_experts_up_kernel(const T* __restrict__ h, const int* __restrict__ ids, const T* __restrict__ wg,
                                      const T* __restrict__ wu, long long gu_stride, float* __restrict__ act, int D, int F,
                                      int E, int top, float limit, float alpha, float shift) {
    extern __shared__ float hx[];
    const int pair = blockIdx.x, j0 = blockIdx.y * MOE_ROWS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int e = ids[pair];
    if (e < 0 || e >= E) e = 0;
    const T* row = h + (size_t)(pair / top) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) hx[d] = mb_load(row + d);
    __syncthreads();
    const T* g_rows = wg + (size_t)e * gu_stride;            // an expert's gate and up rows may lie in one tensor
    const T* u_rows = wu + (size_t)e * gu_stride;
    for (int j = j0 + warp; j < min(F, j0 + MOE_ROWS); j += nwarp) {
        float g = lane_dot(g_rows + (size_t)j * D, hx, D, lane);
        float u = lane_dot(u_rows + (size_t)j * D, hx, D, lane);
        if (lane == 0) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            act[(size_t)pair * F + j] = g / (1.0f + expf(-alpha * g)) * (u + shift);
        }
    }
}

template <typename T>
__global__ void moe_experts_down_kernel(const float* __restrict__ act, const int* __restrict__ ids, const T* __restrict__ wd,
                                        float* __restrict__ y, int D, int F, int E) {
    extern __shared__ float ax[];
    const int pair = blockIdx.x, d0 = blockIdx.y * MOE_ROWS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int e = ids[pair];
    if (e < 0 || e >= E) e = 0;
    for (int j = threadIdx.x; j < F; j += blockDim.x) ax[j] = act[(size_t)pair * F + j];
    __syncthreads();
    const T* d_rows = wd + (size_t)e * D * F;
    for (int d = d0 + warp; d < min(D, d0 + MOE_ROWS); d += nwarp) {
        const float v = lane_dot(d_rows + (size_t)d * F, ax, F, lane);
        if (lane == 0) y[(size_t)pair * D + d] = v;
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, T* __restrict__ out, int D,
                                   int top, long long total, const T* __restrict__ shared, const float* __restrict__ gate,
                                   int gate_stride) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / D;
    const int d = (int)(i - n * D);
    float acc = 0.0f;
    for (int kk = 0; kk < top; kk++) acc = fmaf(wts[n * top + kk], y[(n * top + kk) * D + d], acc);
    // an expert every token uses, times sigmoid of the token's gate logit (no gate: added as it is)
    if (shared) acc = fmaf(gate ? 1.0f / (1.0f + expf(-gate[n * gate_stride])) : 1.0f, mb_load(shared + i), acc);
    mb_store(out + i, acc);
}

MB_API int mb_moe_select(const float* z, int z_stride, const float* correction, int* ids, float* wts, int N, int E, int top,
                         int groups, int keep, int softmax, int worth_max, float scale, cudaStream_t st) {
    if (N == 0) return 0;
    if (E < 1 || top < 1 || top > E || groups < 1 || E % groups || keep < 1 || keep > groups || E > 8192 || z_stride < E) return -2;
    if ((long long)keep * (E / groups) < top) return -2;
    moe_select_kernel<<<N, 32, (size_t)(2 * E + 2 * groups) * sizeof(float), st>>>(z, z_stride, correction, ids, wts, E, top,
                                                                                   groups, keep, softmax, worth_max, scale);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int moe_experts_launch(const T* h, const int* ids, const T* wg, const T* wu, long long gu_stride, const T* wd, float* y,
                              float* act, int N, int D, int F, int E, int top, float limit, float alpha, float shift,
                              cudaStream_t st) {
    if (N == 0) return 0;
    const long long P = (long long)N * top;
    if (D < 1 || F < 1 || top < 1 || P > 0x7fffffff || D > 12000 || F > 12000 || (F + MOE_ROWS - 1) / MOE_ROWS > 65535 ||
        (D + MOE_ROWS - 1) / MOE_ROWS > 65535)
        return -2;
    moe_experts_up_kernel<T><<<dim3((unsigned)P, (F + MOE_ROWS - 1) / MOE_ROWS), 256, (size_t)D * sizeof(float), st>>>(
        h, ids, wg, wu, gu_stride, act, D, F, E, top, limit, alpha, shift);
    MB_LAUNCH_CHECK();
    moe_experts_down_kernel<T><<<dim3((unsigned)P, (D + MOE_ROWS - 1) / MOE_ROWS), 256, (size_t)F * sizeof(float), st>>>(
        act, ids, wd, y, D, F, E);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_moe_experts_f32(const void* h, const int* ids, const void* wg, const void* wu, long long gu_stride,
                              const void* wd, float* y, float* act, int N, int D, int F, int E, int top, float limit,
                              float alpha, float shift, cudaStream_t st) {
    return moe_experts_launch<float>((const float*)h, ids, (const float*)wg, (const float*)wu, gu_stride, (const float*)wd, y,
                                     act, N, D, F, E, top, limit, alpha, shift, st);
}

MB_API int mb_moe_experts_bf16(const void* h, const int* ids, const void* wg, const void* wu, long long gu_stride,
                               const void* wd, float* y, float* act, int N, int D, int F, int E, int top, float limit,
                               float alpha, float shift, cudaStream_t st) {
    return moe_experts_launch<bf16>((const bf16*)h, ids, (const bf16*)wg, (const bf16*)wu, gu_stride, (const bf16*)wd, y, act,
                                    N, D, F, E, top, limit, alpha, shift, st);
}

template <typename T>
static int moe_combine_launch(const float* y, const float* wts, T* out, int N, int D, int top, const T* shared,
                              const float* gate, int gate_stride, cudaStream_t st) {
    if (N == 0) return 0;
    const long long total = (long long)N * D;
    moe_combine_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(y, wts, out, D, top, total, shared, gate,
                                                                           gate_stride);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_moe_combine_f32(const float* y, const float* wts, void* out, int N, int D, int top, const void* shared,
                              const float* gate, int gate_stride, cudaStream_t st) {
    return moe_combine_launch<float>(y, wts, (float*)out, N, D, top, (const float*)shared, gate, gate_stride, st);
}

MB_API int mb_moe_combine_bf16(const float* y, const float* wts, void* out, int N, int D, int top, const void* shared,
                               const float* gate, int gate_stride, cudaStream_t st) {
    return moe_combine_launch<bf16>(y, wts, (bf16*)out, N, D, top, (const bf16*)shared, gate, gate_stride, st);
}

// ---------------------------------------------------------------------------------------------------------------------
// Steps of many tokens (bf16): the (token, place) pairs are sorted by expert on the device, and every expert's rows run
// through tensor-core tiles, so an expert's matrices are read once per 64 of its rows instead of once per row.
//
//   moe_sort        one block: counts per expert, offsets, the pairs in expert order (`sorted`), and the list of tiles
//                   (expert, first sorted row, rows <= 64); the launch sizes below depend on the number of pairs only,
//                   blocks beyond the tiles that exist leave at once
//   moe_grouped<0>  rows gathered from h by token, [Wg_e; Wu_e]: act = g sigmoid(alpha g) (u + 1) with the clamps, bf16,
//                   at the pair's sorted row
//   moe_grouped<1>  rows of act, Wd_e: float32 to the pair's own place in y (N, top, D), which moe_combine sums
//
// A tile is 64 rows x 64 output columns (of both matrices in mode 0), k in steps of 32 through two cp.async stages,
// four warps of 16 rows each, ldmatrix + mma.sync.m16n8k16 with float accumulation.  A row's result does not depend on
// where in its expert's run the sort put it.
#define GG_TM 64
#define GG_TN 64
#define GG_TK 32
#define GG_LD 40            // shared-memory row length in bf16: 80 bytes, so that 8 rows hit 8 different 16-byte columns

__global__ void moe_sort_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ offsets, int* __restrict__ sorted,
                                int* __restrict__ tiles /* 3 ints each */, int* __restrict__ n_tiles, int max_tiles) {
    extern __shared__ int sh[];
    int* cnt = sh;              // E
    int* start = sh + E;        // E + 1
    int* tstart = start + E + 1;  // E + 1
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        int e = ids[p];
        if (e < 0 || e >= E) e = 0;
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, t = 0;
        for (int e = 0; e < E; e++) {
            start[e] = a; tstart[e] = t;
            a += cnt[e];
            t += (cnt[e] + GG_TM - 1) / GG_TM;
        }
        start[E] = a; tstart[E] = t;
        *n_tiles = t < max_tiles ? t : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = start[e];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int nt = tstart[e + 1] - tstart[e];
        for (int i = 0; i < nt; i++) {
            const int t = tstart[e] + i;
            if (t >= max_tiles) break;
            tiles[3 * t] = e;
            tiles[3 * t + 1] = start[e] + i * GG_TM;
            tiles[3 * t + 2] = min(GG_TM, cnt[e] - i * GG_TM);
        }
        cnt[e] = start[e];                          // from here on: the next free sorted row of the expert
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        int e = ids[p];
        if (e < 0 || e >= E) e = 0;
        sorted[atomicAdd(&cnt[e], 1)] = p;
    }
}

__device__ __forceinline__ void gg_cp16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = smem_u32(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}

__device__ __forceinline__ void gg_ldsm4(uint32_t (&r)[4], const void* p) {
    const uint32_t s = smem_u32(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

__device__ __forceinline__ void gg_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MODE 0: A = h (rows by token = pair / top), B0 = wg, B1 = wu (E, Nout, K), out_act (pairs, Nout) bf16 by sorted row.
// MODE 1: A = act (rows by sorted row), B0 = wd (E, Nout, K), out_y (pairs, Nout) float32 by pair.
template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B0, const bf16* __restrict__ B1, long long b_stride,
                   const int* __restrict__ sorted, const int* __restrict__ tiles, const int* __restrict__ n_tiles, int top,
                   int Nout, int K, bf16* __restrict__ out_act, float* __restrict__ out_y, float limit, float alpha,
                   float shift) {
    constexpr int NB = MODE == 0 ? 2 : 1;
    __shared__ __align__(16) bf16 sA[2][GG_TM][GG_LD];
    __shared__ __align__(16) bf16 sB[2][NB][GG_TN][GG_LD];
    __shared__ int srow[GG_TM];                     // the pair of every row of the tile (-1: no row)
    const int t = blockIdx.x;
    if (t >= *n_tiles) return;
    const int e = tiles[3 * t], r0 = tiles[3 * t + 1], rows = tiles[3 * t + 2];
    const int n0 = blockIdx.y * GG_TN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < GG_TM) srow[tid] = tid < rows ? sorted[r0 + tid] : -1;
    __syncthreads();
    const bf16* Bp[NB];
    Bp[0] = B0 + (size_t)e * b_stride;
    if (MODE == 0) Bp[NB - 1] = B1 + (size_t)e * b_stride;
    // each thread copies chunks (row = c / 4, 8 k-values at (c % 4) * 8) c = tid and tid + 128 of every 64 x 32 tile
    auto load = [&](int stage, int k0) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int c = tid + i * 128, r = c >> 2, kk = k0 + (c & 3) * 8;
            const bool kin = kk < K;
            const int pair = srow[r];
            const size_t arow = MODE == 0 ? (size_t)(pair < 0 ? 0 : pair / top) : (size_t)(r0 + (r < rows ? r : 0));
            gg_cp16(&sA[stage][r][(c & 3) * 8], A + arow * K + (kin ? kk : 0), kin && pair >= 0);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int n = n0 + r;
                gg_cp16(&sB[stage][b][r][(c & 3) * 8], Bp[b] + (size_t)(n < Nout ? n : 0) * K + (kin ? kk : 0), kin && n < Nout);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    float acc[NB][8][4];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[b][j][x] = 0.0f;
    const int nk = (K + GG_TK - 1) / GG_TK;
    load(0, 0);
    for (int ks = 0; ks < nk; ks++) {
        if (ks + 1 < nk) {
            load((ks + 1) & 1, (ks + 1) * GG_TK);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const int st = ks & 1;
#pragma unroll
        for (int k16 = 0; k16 < GG_TK; k16 += 16) {
            uint32_t a[4];
            gg_ldsm4(a, &sA[st][warp * 16 + (lane & 15)][k16 + (lane >> 4) * 8]);
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    uint32_t w[4];          // two n-tiles of 8: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                    gg_ldsm4(w, &sB[st][b][j * 8 + (lane & 7) + (lane >> 4) * 8][k16 + ((lane >> 3) & 1) * 8]);
                    gg_mma(acc[b][j], a, w[0], w[1]);
                    gg_mma(acc[b][j + 1], a, w[2], w[3]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int pair = srow[r];
        if (pair < 0) continue;
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int x = 0; x < 2; x++) {
                const int n = n0 + j * 8 + (lane & 3) * 2 + x;
                if (n >= Nout) continue;
                if (MODE == 0) {
                    const float g = fminf(acc[0][j][half * 2 + x], limit);
                    const float u = fminf(fmaxf(acc[NB - 1][j][half * 2 + x], -limit), limit);
                    out_act[(size_t)(r0 + r) * Nout + n] = __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + shift));
                } else {
                    out_y[(size_t)pair * Nout + n] = acc[0][j][half * 2 + x];
                }
            }
    }
}

// ids (N, top); sorted, offsets, tiles, n_tiles: int scratch of P, E + 1, 3 max_tiles and 1 values; act (P, F) bf16
MB_API int mb_moe_grouped_bf16(const void* h, const int* ids, const void* wg, const void* wu, long long gu_stride,
                               const void* wd, float* y,
                               void* act, int* sorted, int* offsets, int* tiles, int* n_tiles, int N, int D, int F, int E,
                               int top, float limit, float alpha, float shift, cudaStream_t st) {
    if (N == 0) return 0;
    const long long P = (long long)N * top;
    if (D % 8 || F % 8 || D < 8 || F < 8 || E < 1 || E > 4096 || P > (1 << 24)) return -2;
    const int max_tiles = (int)(P / GG_TM) + E;
    moe_sort_kernel<<<1, 1024, (size_t)(3 * E + 2) * sizeof(int), st>>>(ids, (int)P, E, offsets, sorted, tiles, n_tiles, max_tiles);
    MB_LAUNCH_CHECK();
    moe_grouped_kernel<0><<<dim3(max_tiles, (F + GG_TN - 1) / GG_TN), 128, 0, st>>>(
        (const bf16*)h, (const bf16*)wg, (const bf16*)wu, gu_stride, sorted, tiles, n_tiles, top, F, D, (bf16*)act, nullptr,
        limit, alpha, shift);
    MB_LAUNCH_CHECK();
    moe_grouped_kernel<1><<<dim3(max_tiles, (D + GG_TN - 1) / GG_TN), 128, 0, st>>>(
        (const bf16*)act, (const bf16*)wd, nullptr, (long long)D * F, sorted, tiles, n_tiles, top, D, F, nullptr, y, limit,
        alpha, shift);
    MB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Steps of 128 tokens and more (bf16) hand the two products to the tcgen05 product in its grouped form, which wants the
// rows of every expert side by side, starting at a multiple of 128:
//   moe_sort_padded   one block: per pair its row in that layout (`place`), per tile of 128 rows its expert (-1: empty)
//   moe_gather_rows   h rows, by token, to their places
//   moe_combine_rows  out[n] = sum over the places, in order, of weight * y[place of (n, k)]
__global__ void moe_sort_padded_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ place,
                                       int* __restrict__ tile_expert, int max_tiles) {
    extern __shared__ int sh[];
    int* cnt = sh;              // E
    int* start = sh + E;        // E + 1, in tiles
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        int e = ids[p];
        if (e < 0 || e >= E) e = 0;
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; e++) { start[e] = t; t += (cnt[e] + 127) / 128; }
        start[E] = t;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (int t = start[e]; t < start[e + 1] && t < max_tiles; t++) tile_expert[t] = e;
        cnt[e] = start[e] * 128;                    // from here on: the next free row of the expert
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        int e = ids[p];
        if (e < 0 || e >= E) e = 0;
        place[p] = atomicAdd(&cnt[e], 1);
    }
}

__global__ void moe_gather_rows_kernel(const bf16* __restrict__ h, const int* __restrict__ place, bf16* __restrict__ rows, int D,
                                       int top) {
    const int p = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(p / top) * D);
    uint4* dst = reinterpret_cast<uint4*>(rows + (size_t)place[p] * D);
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void moe_combine_rows_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wts,
                                        bf16* __restrict__ out, int D, int top, const bf16* __restrict__ shared,
                                        const float* __restrict__ gate, int gate_stride) {
    const int n = blockIdx.x;
    const float sg = shared ? (gate ? 1.0f / (1.0f + expf(-gate[(size_t)n * gate_stride])) : 1.0f) : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int kk = 0; kk < top; kk++) acc = fmaf(wts[(size_t)n * top + kk], y[(size_t)place[(size_t)n * top + kk] * D + d], acc);
        if (shared) acc = fmaf(sg, __bfloat162float(shared[(size_t)n * D + d]), acc);
        out[(size_t)n * D + d] = __float2bfloat16_rn(acc);
    }
}

// place (N top), tile_expert (N top / 128 + E), rows ((N top / 128 + E) 128, D) bf16
MB_API int mb_moe_sort_gather(const void* h, const int* ids, int* place, int* tile_expert, void* rows, int N, int D, int E,
                              int top, cudaStream_t st) {
    if (N == 0) return 0;
    const long long P = (long long)N * top;
    if (D % 8 || D < 8 || E < 1 || E > 4096 || P > (1 << 24)) return -2;
    const int max_tiles = (int)(P / 128) + E;
    moe_sort_padded_kernel<<<1, 1024, (size_t)(2 * E + 1) * sizeof(int), st>>>(ids, (int)P, E, place, tile_expert, max_tiles);
    MB_LAUNCH_CHECK();
    moe_gather_rows_kernel<<<(unsigned)P, 128, 0, st>>>((const bf16*)h, place, (bf16*)rows, D, top);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_moe_combine_rows(const float* y, const int* place, const float* wts, void* out, int N, int D, int top,
                               const void* shared, const float* gate, int gate_stride, cudaStream_t st) {
    if (N == 0) return 0;
    moe_combine_rows_kernel<<<N, 256, 0, st>>>(y, place, wts, (bf16*)out, D, top, (const bf16*)shared, gate, gate_stride);
    MB_LAUNCH_CHECK();
    return 0;
}
