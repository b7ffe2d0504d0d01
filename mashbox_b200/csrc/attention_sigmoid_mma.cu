// Attention with sigmoid weights over the paged cache on tensor cores (bf16): prompt portions and decode tokens.
//
// A visible key j weighs  w = sigmoid(scale q_i . k_j - slope_h (i - j) + bias_h)  for the query at position i (j <= i);
// the output is the plain weighted sum of the values: no maximum, no denominator, nothing to rescale between key tiles.
// Keys (SIG_DIM wide) and values (SIG_VD wide) live in two pools, (pages, kv heads, page, width) each.
//
// The query rows of one sequence and one kv head are packed as (token, head-in-group): all query heads that read a kv
// head share every K/V tile that is loaded.  K and V tiles of 64 keys are gathered through the block table with
// cp.async into XOR-swizzled shared memory; scores and the weighted sum run on mma.sync.m16n8k16 with float
// accumulators.  A weight is computed in float32 and handed to the second product as two bf16 numbers, w = hi + lo (16
// bits of mantissa together), which both multiply the values: the weights of hundreds of keys add up with nothing to
// normalise them, and the sum keeps them at float32's grade although the values are read as bf16.
//   * prompt form: 64 rows per block, each of the 4 warps owns 16 rows and all 64 keys of a tile; two stages.
//     A work item is (sequence, tile of rows); the grid is (items, kv heads).
//   * decode form: at most 16 rows per block (one or a few tokens of one sequence), the 4 warps split the 64 keys of a
//     tile and meet through shared memory at the end; the keys of a sequence may be cut into splits that run side by
//     side (item: sequence, split, number of splits, slot), whose partial sums a second kernel adds in the order of the
//     splits.  Three stages.
//
// One library per pair of head sizes: compiled with -DSIG_DIM=<key dim> -DSIG_VD=<value dim>, multiples of 16.
#include "attention_common.cuh"

#ifndef SIG_DIM
#define SIG_DIM 64
#endif
#ifndef SIG_VD
#define SIG_VD 64
#endif

struct SigParams {
    const bf16* q; bf16* out;               // q[(n * H + h) * DIM + d], out[(n * H + h) * VD + d]
    const bf16* kpool; const bf16* vpool;   // [page][G][slot][DIM], [page][G][slot][VD]
    const void* items;
    const int* q_start; const int* q_len; const int* pos0; const int* seq_row;
    const int* table; int max_blocks;
    const float* slopes; const float* bias; // per query head, or null (0)
    float* part_o;                          // [slot][G][MAX_SPLITS][16 rows][VD]
    int H, G, group, page, num_pages;
    int page_shift;                         // log2(page) when the page size is a power of two, else -1
    float scale;
    int* err;
};

constexpr int BM = 64, BN = 64, THREADS = 128, STAGES = 2;
constexpr int DBM = 16, DSTAGES = 3, MAX_SPLITS = 16;
constexpr int KROW = tile_row<SIG_DIM>(), VROW = tile_row<SIG_VD>();
constexpr int STAGE_ELEMS = BN * KROW + BN * VROW;
constexpr size_t cmax(size_t a, size_t b) { return a > b ? a : b; }
constexpr size_t SMEM_BYTES = ((size_t)BM * KROW + (size_t)STAGES * STAGE_ELEMS) * sizeof(bf16);
// the stages of the decode form are also where its four warps meet at the end ([4 warps][16 rows][VD] floats)
constexpr size_t DSMEM_BYTES = (size_t)DBM * KROW * sizeof(bf16)
                               + cmax((size_t)DSTAGES * STAGE_ELEMS * sizeof(bf16), (size_t)4 * DBM * SIG_VD * sizeof(float));
static_assert(SIG_DIM % 16 == 0 && SIG_VD % 16 == 0 && SIG_DIM >= 16 && SIG_VD >= 16, "head sizes are multiples of 16");
static_assert(SIG_DIM <= 128 && SIG_VD <= 128, "head sizes up to 128");

// One tile of 64 keys and their values into a stage; rows at or beyond `hi` are filled with zeros.  Two threads share a
// row: its page, slot and addresses are worked out once, then the pair walks the row's 16-byte pieces side by side (a
// whole 32-byte sector per pair and instruction), the key's first, then the value's.
__device__ __forceinline__ void sig_load_tile(bf16* stage, const SigParams& P, const int* tb, int g, int kb, int hi, int tid) {
    constexpr int CK = SIG_DIM / 8, CV = SIG_VD / 8;
    static_assert(THREADS == 2 * BN, "two threads a row");
    const int row = tid >> 1, sub = tid & 1;
    const int kp = kb + row;
    const bf16* ksrc = P.kpool;
    const bf16* vsrc = P.vpool;
    int bytes = 0;
    if (kp < hi) {
        int block, slot;
        if (P.page_shift >= 0) { block = kp >> P.page_shift; slot = kp & (P.page - 1); }
        else { block = kp / P.page; slot = kp - block * P.page; }
        const int pg = tb[block];
        if (pg >= 0 && pg < P.num_pages) {
            const size_t r = ((size_t)pg * P.G + g) * P.page + slot;
            ksrc = P.kpool + r * SIG_DIM;
            vsrc = P.vpool + r * SIG_VD;
            bytes = 16;
        } else {
            mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
        }
    }
    bf16* vstage = stage + BN * KROW;
#pragma unroll
    for (int c = 0; c < CK; c += 2) cp_async16(stage + swz<SIG_DIM>(row, c + sub), ksrc + (bytes ? (c + sub) * 8 : 0), bytes);
#pragma unroll
    for (int c = 0; c < CV; c += 2) cp_async16(vstage + swz<SIG_VD>(row, c + sub), vsrc + (bytes ? (c + sub) * 8 : 0), bytes);
}

// sigmoid(z) = 1 / (1 + 2^(-z log2 e)) with the special-function unit's 2^x and reciprocal (a few ulp each, no slow
// path and no branch; 2^x = inf for a far negative z gives 0)
__device__ __forceinline__ float sig_unit(float z) {
    float e, w;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(z * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(w) : "f"(1.0f + e));
    return w;
}

// the weights of one 16 x 8 score tile: s holds q . k, rows gq (e = 0, 1) and gq + 8 (e = 2, 3), keys key0 + (e & 1)
__device__ __forceinline__ void sig_weights(float (&s)[4], int key0, const int (&rpos)[2], const float (&slope)[2],
                                            const float (&bias)[2], float scale) {
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int i = e >> 1, key = key0 + (e & 1);
        const float z = fmaf(s[e], scale, bias[i]) - slope[i] * (float)(rpos[i] - key);
        s[e] = key <= rpos[i] ? sig_unit(z) : 0.0f;
    }
}

// w = hi + lo as two bf16 pairs
__device__ __forceinline__ void sig_split(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
    hi = (uint32_t)__bfloat16_as_ushort(ha) | ((uint32_t)__bfloat16_as_ushort(hb) << 16);
    lo = pack_bf16(a - __bfloat162float(ha), b - __bfloat162float(hb));
}

__global__ void __launch_bounds__(THREADS) sigattn_mma_kernel(const SigParams P) {
    constexpr int DIM = SIG_DIM, VD = SIG_VD, CK = DIM / 8, KS = DIM / 16, DT = VD / 8, NT = 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + BM * KROW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tig = lane & 3;
    const int m0 = warp * 16;
    const int2 item = reinterpret_cast<const int2*>(P.items)[blockIdx.x];
    const int seq = item.x, m_tile = item.y, g = blockIdx.y;
    const int G = P.group, R = P.q_len[seq] * G, pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int row0 = m_tile * BM;
    if (row0 >= R) return;
    const int row_last = min(R, row0 + BM) - 1;
    const int hi = pos0 + row_last / G + 1;
    const int n_tiles = (hi + BN - 1) / BN;
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    for (int cid = tid; cid < BM * CK; cid += THREADS) {
        const int row = cid / CK, c = cid % CK, r = row0 + row;
        const bf16* src = P.q;
        int bytes = 0;
        if (r < R) {
            src = P.q + ((size_t)(tok0 + r / G) * P.H + (g * G + r % G)) * DIM + c * 8;
            bytes = 16;
        }
        cp_async16(qs + swz<DIM>(row, c), src, bytes);
    }
    cp_async_commit();
    sig_load_tile(kvs, P, tb, g, 0, hi, tid);
    cp_async_commit();

    int rpos[2];
    float slope[2], bias[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + m0 + gq + i * 8;
        const int h = g * G + r % G;
        rpos[i] = r < R ? pos0 + r / G : -1;
        slope[i] = P.slopes ? P.slopes[h] : 0.0f;
        bias[i] = P.bias ? P.bias[h] : 0.0f;
    }
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }

    cp_async_wait<1>();
    __syncthreads();
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldmatrix_x4(qf[ks], qs + swz<DIM>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
    const int warp_row = min(R - 1, row0 + m0 + 15);        // the warp's last row that exists
    const int warp_hi = warp_row >= row0 + m0 ? pos0 + warp_row / G : -1;

    for (int t = 0; t < n_tiles; t++) {
        cp_async_wait<0>();
        __syncthreads();                                    // tile t has landed; every warp is done with tile t - 1
        if (t + 1 < n_tiles) sig_load_tile(kvs + (size_t)((t + 1) % STAGES) * STAGE_ELEMS, P, tb, g, (t + 1) * BN, hi, tid);
        cp_async_commit();
        const bf16* kt = kvs + (size_t)(t % STAGES) * STAGE_ELEMS;
        const bf16* vt = kt + BN * KROW;
        const int kb = t * BN;
        if (kb > warp_hi) continue;                         // no row of this warp sees a key of the tile

        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + swz<DIM>(np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < NT; j++) sig_weights(s[j], kb + j * 8 + 2 * tig, rpos, slope, bias, P.scale);
#pragma unroll
        for (int kk = 0; kk < NT / 2; kk++) {
            uint32_t ah[4], al[4];
            sig_split(s[2 * kk][0], s[2 * kk][1], ah[0], al[0]);
            sig_split(s[2 * kk][2], s[2 * kk][3], ah[1], al[1]);
            sig_split(s[2 * kk + 1][0], s[2 * kk + 1][1], ah[2], al[2]);
            sig_split(s[2 * kk + 1][2], s[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
            for (int dp = 0; dp < VD / 16; dp++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + swz<VD>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
                mma_bf16(o[2 * dp], ah, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], ah, b[2], b[3]);
                mma_bf16(o[2 * dp], al, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], al, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + m0 + gq + i * 8;
        if (r >= R) continue;
        bf16* dst = P.out + ((size_t)(tok0 + r / G) * P.H + (g * G + r % G)) * VD + 2 * tig;
#pragma unroll
        for (int d = 0; d < DT; d++)
            *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2 * i], o[d][2 * i + 1]);
    }
}

// ------------------------------------------------------------------------------------------------ decode form
__global__ void __launch_bounds__(THREADS) sigattn_mma_decode_kernel(const SigParams P) {
    constexpr int DIM = SIG_DIM, VD = SIG_VD, CK = DIM / 8, KS = DIM / 16, DT = VD / 8, NT = 2, NC = VD / 32 + 1;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + DBM * KROW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tig = lane & 3;
    const int nbase = warp * 16;
    const int4 item = reinterpret_cast<const int4*>(P.items)[blockIdx.x];
    const int seq = item.x, split = item.y, n_splits = item.z, slot = item.w, g = blockIdx.y;
    const int G = P.group, R = min(DBM, P.q_len[seq] * G), pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int hi = pos0 + (R - 1) / G + 1;
    const int n_tiles = (hi + BN - 1) / BN;
    const int tps = (n_tiles + n_splits - 1) / n_splits;
    const int t_begin = split * tps, t_end = min(n_tiles, t_begin + tps);
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    for (int cid = tid; cid < DBM * CK; cid += THREADS) {
        const int row = cid / CK, c = cid % CK;
        const bf16* src = P.q;
        int bytes = 0;
        if (row < R) {
            src = P.q + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * DIM + c * 8;
            bytes = 16;
        }
        cp_async16(qs + swz<DIM>(row, c), src, bytes);
    }
    cp_async_commit();
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; s++) {
        if (t_begin + s < t_end) sig_load_tile(kvs + (size_t)s * STAGE_ELEMS, P, tb, g, (t_begin + s) * BN, hi, tid);
        cp_async_commit();
    }
    int rpos[2];
    float slope[2], bias[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = gq + i * 8;
        const int h = g * G + r % G;
        rpos[i] = r < R ? pos0 + r / G : -1;
        slope[i] = P.slopes ? P.slopes[h] : 0.0f;
        bias[i] = P.bias ? P.bias[h] : 0.0f;
    }
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }

    cp_async_wait<DSTAGES - 1>();
    __syncthreads();
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldmatrix_x4(qf[ks], qs + swz<DIM>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    for (int t = t_begin; t < t_end; t++) {
        cp_async_wait<DSTAGES - 2>();
        __syncthreads();
        {
            const int tn = t + DSTAGES - 1;
            if (tn < t_end) sig_load_tile(kvs + (size_t)((tn - t_begin) % DSTAGES) * STAGE_ELEMS, P, tb, g, tn * BN, hi, tid);
            cp_async_commit();
        }
        const bf16* kt = kvs + (size_t)((t - t_begin) % DSTAGES) * STAGE_ELEMS;
        const bf16* vt = kt + BN * KROW;
        const int kb = t * BN;
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t b[4];
            ldmatrix_x4(b, kt + swz<DIM>(nbase + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
#pragma unroll
        for (int j = 0; j < NT; j++) sig_weights(s[j], kb + nbase + j * 8 + 2 * tig, rpos, slope, bias, P.scale);
        uint32_t ah[4], al[4];
        sig_split(s[0][0], s[0][1], ah[0], al[0]);
        sig_split(s[0][2], s[0][3], ah[1], al[1]);
        sig_split(s[1][0], s[1][1], ah[2], al[2]);
        sig_split(s[1][2], s[1][3], ah[3], al[3]);
#pragma unroll
        for (int dp = 0; dp < VD / 16; dp++) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vt + swz<VD>(nbase + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
            mma_bf16(o[2 * dp], ah, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], ah, b[2], b[3]);
            mma_bf16(o[2 * dp], al, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], al, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                        // every warp is done with the K/V stages
    float* mo = reinterpret_cast<float*>(kvs);              // [4 warps][16 rows][VD]
#pragma unroll
    for (int i = 0; i < 2; i++) {
        float* dst = mo + (size_t)(warp * DBM + gq + i * 8) * VD + 2 * tig;
#pragma unroll
        for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
    }
    __syncthreads();
    // warp w finishes rows 4 w .. 4 w + 3: the four quarters of the keys in their order
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
        const int row = 4 * warp + rr;
        if (row >= R) continue;
        float acc[NC];
#pragma unroll
        for (int i = 0; i < NC; i++) {
            const int d = lane + 32 * i;
            acc[i] = 0.0f;
            if (d < VD) {
#pragma unroll
                for (int w = 0; w < 4; w++) acc[i] += mo[(size_t)(w * DBM + row) * VD + d];
            }
        }
        if (n_splits == 1) {
            bf16* dst = P.out + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * VD;
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int d = lane + 32 * i;
                if (d < VD) dst[d] = __float2bfloat16_rn(acc[i]);
            }
        } else {
            float* dst = P.part_o + ((((size_t)slot * P.G + g) * MAX_SPLITS + split) * DBM + row) * VD;
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int d = lane + 32 * i;
                if (d < VD) dst[d] = acc[i];
            }
        }
    }
}

// one block per (slot, kv head): the splits of every row are added in the order of the splits
__global__ void __launch_bounds__(THREADS) sigattn_merge_kernel(const SigParams P, const int2* slots) {
    constexpr int VD = SIG_VD, NC = VD / 32 + 1;
    const int slot = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = slots[slot].x, n_splits = slots[slot].y;
    const int G = P.group, R = min(DBM, P.q_len[seq] * G), tok0 = P.q_start[seq];
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
        const int row = 4 * warp + rr;
        if (row >= R) continue;
        const float* src = P.part_o + (((size_t)slot * P.G + g) * MAX_SPLITS * DBM + row) * VD;      // + split * DBM * VD
        float acc[NC];
#pragma unroll
        for (int i = 0; i < NC; i++) acc[i] = 0.0f;
        for (int s = 0; s < n_splits; s++) {
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int d = lane + 32 * i;
                if (d < VD) acc[i] += src[(size_t)s * DBM * VD + d];
            }
        }
        bf16* dst = P.out + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * VD;
#pragma unroll
        for (int i = 0; i < NC; i++) {
            const int d = lane + 32 * i;
            if (d < VD) dst[d] = __float2bfloat16_rn(acc[i]);
        }
    }
}

MB_API int mb_sigattn_mma_dims(int* dim, int* vd, int* rows) {
    *dim = SIG_DIM; *vd = SIG_VD; *rows = BM;
    return 0;
}

MB_API int mb_sigattn_mma_max_splits() { return MAX_SPLITS; }

static int sig_fill(SigParams& P, const void* q, void* out, const void* kpool, const void* vpool, const void* items,
                    const int* q_start, const int* q_len, const int* pos0, const int* seq_row, const int* table,
                    int max_blocks, const float* slopes, const float* bias, float* part_o, int H, int G, int page,
                    int num_pages, float scale, int* err) {
    if (G < 1 || H % G || page < 1 || G > 65535) return -2;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpool | (uintptr_t)vpool) & 15) != 0) return -2;
    P.q = (const bf16*)q; P.out = (bf16*)out; P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = items; P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks; P.slopes = slopes; P.bias = bias; P.part_o = part_o;
    P.H = H; P.G = G; P.group = H / G; P.page = page; P.num_pages = num_pages;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale = scale; P.err = err;
    return 0;
}

// the prompt form: n_items (sequence, tile of 64 packed rows) pairs
MB_API int mb_sigattn_mma(const void* q, void* out, const void* kpool, const void* vpool, const int* items, int n_items,
                          const int* q_start, const int* q_len, const int* pos0, const int* seq_row, const int* table,
                          int max_blocks, const float* slopes, const float* bias, int H, int G, int page, int num_pages,
                          float scale, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    SigParams P;
    if (sig_fill(P, q, out, kpool, vpool, items, q_start, q_len, pos0, seq_row, table, max_blocks, slopes, bias, nullptr, H,
                 G, page, num_pages, scale, err)) return -2;
    static bool ready = false;
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(sigattn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(sigattn_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ready = true;
    }
    sigattn_mma_kernel<<<dim3(n_items, G), THREADS, SMEM_BYTES, st>>>(P);
    MB_LAUNCH_CHECK();
    return 0;
}

// the decode form: n_items (sequence, split, n_splits, slot) items; n_slots (sequence, n_splits) entries for the kernel
// that adds the splits (0: no sequence is cut); part_o: n_slots * G * 16 splits * 16 rows * VD floats
MB_API int mb_sigattn_mma_decode(const void* q, void* out, const void* kpool, const void* vpool, const int* items,
                                 int n_items, const int* slots, int n_slots, float* part_o, const int* q_start,
                                 const int* q_len, const int* pos0, const int* seq_row, const int* table, int max_blocks,
                                 const float* slopes, const float* bias, int H, int G, int page, int num_pages, float scale,
                                 int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (n_slots > 0 && (!part_o || !slots)) return -2;
    SigParams P;
    if (sig_fill(P, q, out, kpool, vpool, items, q_start, q_len, pos0, seq_row, table, max_blocks, slopes, bias, part_o, H,
                 G, page, num_pages, scale, err)) return -2;
    static bool ready = false;
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(sigattn_mma_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DSMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(sigattn_mma_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ready = true;
    }
    sigattn_mma_decode_kernel<<<dim3(n_items, G), THREADS, DSMEM_BYTES, st>>>(P);
    MB_LAUNCH_CHECK();
    if (n_slots > 0) {
        sigattn_merge_kernel<<<dim3(n_slots, G), THREADS, 0, st>>>(P, (const int2*)slots);
        MB_LAUNCH_CHECK();
    }
    return 0;
}
