// Paged flash attention on tensor cores (bf16) in its GENERAL form: keys of GA_DK and values of GA_DV values (the
// library is compiled for one such pair, -DGA_DK=.. -DGA_DV=..; both multiples of 16 up to 256), pools whose rows may
// be wider than what is read of them (k_row, v_row: elements between two positions' rows; a pool whose row is key and
// value at once is handed in twice), and, each optional: capped scores s <- cap tanh(s / cap); a sink per query head,
// one more term exp(sink_h) in the softmax's denominator that has no value; a gate per token and query head, the
// head's result times sigmoid(gate).
//
// The query rows of one sequence and one KV head are packed as (token, head-in-group); a work item is (sequence, tile
// of rows, split of the keys); the grid is (items, KV heads).  K and V tiles of 64 keys are gathered page by page
// through the block table with cp.async into XOR-swizzled shared memory, scores and the weighted sum run on
// mma.sync.m16n8k16 with float accumulators, the softmax is online in float with exp2.
//   * PREFILL form: 64 rows per block, each of the 4 warps owns 16 rows and all 64 keys of a tile.
//   * DECODE form: at most 16 rows per block, the 4 warps split the 64 keys of a tile and meet in shared memory.
// With more than one split an item writes its unnormalised partial (o, m, l) to scratch memory and a second kernel
// merges the splits.  Sink and gate come in wherever a row is finished: at the end of an unsplit item, or in the merge.
#include "attention_common.cuh"

#ifndef GA_DK
#define GA_DK 64
#endif
#ifndef GA_DV
#define GA_DV 64
#endif

struct GenParams {
    AttnParams a;
    int k_row, v_row;                       // elements between the rows of two positions in the key and value pools
    float scale, softcap;                   // softcap 0: none
    const float* sinks;                     // one per query head, or null
    const bf16* gate; int gate_stride;      // gate[n * gate_stride + h], or null
};

// what a finished row is multiplied by and what its denominator gains: the sink joins after every key
__device__ __forceinline__ void ga_finish(const GenParams& P, int n, int h, float& m2, float& l, float& rescale, float& mult) {
    rescale = 1.0f;
    if (P.sinks) {
        const float sk = P.sinks[h] * 1.4426950408889634f, m_new = fmaxf(m2, sk);
        rescale = (m2 == -INFINITY) ? 0.0f : exp2f(m2 - m_new);
        l = l * rescale + exp2f(sk - m_new);
        m2 = m_new;
    }
    mult = l > 0.0f ? 1.0f / l : 0.0f;
    if (P.gate) mult /= 1.0f + expf(-__bfloat162float(P.gate[(size_t)n * P.gate_stride + h]));
}

template <int HD, int BN>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* pool, int row_elems, const AttnParams& P, const int* tb,
                                          int kvh, int kb, int lo, int hi, int tid) {
    constexpr int CH = HD / 8;
    const int shift = P.page_shift, mask = P.page - 1;
    int last_block = -1, pg = -1;
#pragma unroll
    for (int cid = tid; cid < BN * CH; cid += 128) {
        const int row = cid / CH, c = cid % CH;
        const int kp = kb + row;
        const bf16* src = pool;
        int bytes = 0;
        if (kp >= lo && kp < hi) {                       // below lo a window may have given the pages back
            int block, slot;
            if (shift >= 0) { block = kp >> shift; slot = kp & mask; }
            else { block = kp / P.page; slot = kp - block * P.page; }
            if (block != last_block) { pg = tb[block]; last_block = block; }
            if (pg >= 0 && pg < P.num_pages) {
                src += (((size_t)pg * P.KV + kvh) * P.page + slot) * row_elems + c * 8;
                bytes = 16;
            } else {
                mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            }
        }
        cp_async16(dst + swz<HD>(row, c), src, bytes);
    }
}

// SHARED: keys and values are one pool (a position's row is its key, the value that row's first DV values): the value
// product reads the key tile, nothing is fetched twice and a stage is a third to a half smaller.
template <int DK, int DV, bool DECODE, int STAGES, bool SHARED>
__global__ void __launch_bounds__(128) attn_general_kernel(const GenParams GP) {
    const AttnParams& P = GP.a;
    constexpr int BM = DECODE ? 16 : 64, BN = 64, CHQ = DK / 8;
    constexpr int NT = DECODE ? 2 : 8;      // 8-key tiles per warp per key tile
    constexpr int KS = DK / 16;             // k steps of q k^T
    constexpr int DT = DV / 8;              // 8-wide tiles of the output
    constexpr int ROWK = tile_row<DK>(), ROWV = tile_row<DV>();     // elements of a tile's row in shared memory
    constexpr int STAGE = BN * (ROWK + (SHARED ? 0 : ROWV));        // a stage: the key tile, then the value tile
    constexpr bool QREG = DK <= 128;        // the query fragments stay in registers (above: read again for every key tile)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + BM * ROWK;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int4 item = P.items[blockIdx.x];
    const int seq = item.x, m_tile = item.y, split = item.z, n_splits = item.w;
    const int kvh = blockIdx.y;
    const int G = P.G, R = P.q_len[seq] * G, pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int row0 = m_tile * BM;
    if (row0 >= R) return;
    const int row_last = min(R, row0 + BM) - 1;
    const int pos_min = pos0 + row0 / G, pos_max = pos0 + row_last / G;
    const int hi = pos_max + 1;
    const int lo = (P.window > 0 && pos_min - P.window + 1 > 0) ? pos_min - P.window + 1 : 0;
    const int lo_al = (lo / BN) * BN;
    const int n_tiles = (hi - lo_al + BN - 1) / BN;
    const int tps = (n_tiles + n_splits - 1) / n_splits;
    const int t_begin = split * tps, t_end = min(n_tiles, t_begin + tps);
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    for (int cid = tid; cid < BM * CHQ; cid += 128) {
        const int row = cid / CHQ, c = cid % CHQ, r = row0 + row;
        const bf16* src = P.q;
        int bytes = 0;
        if (r < R) {
            src = P.q + (size_t)(tok0 + r / G) * P.q_stride + (size_t)(kvh * G + r % G) * DK + c * 8;
            bytes = 16;
        }
        cp_async16(qs + swz<DK>(row, c), src, bytes);
    }
    cp_async_commit();
    auto fetch = [&](int t) {
        bf16* st = kvs + (size_t)((t - t_begin) % STAGES) * STAGE;
        load_tile<DK, BN>(st, P.kpool, GP.k_row, P, tb, kvh, lo_al + t * BN, lo, hi, tid);
        if (!SHARED) load_tile<DV, BN>(st + BN * ROWK, P.vpool, GP.v_row, P, tb, kvh, lo_al + t * BN, lo, hi, tid);
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (t_begin + s < t_end) fetch(t_begin + s);
        cp_async_commit();
    }

    const int m0 = DECODE ? 0 : warp * 16;
    const int nbase = DECODE ? warp * 16 : 0;
    int rpos[2], rlo[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + m0 + g + i * 8;
        if (r < R) {
            rpos[i] = pos0 + r / G;
            rlo[i] = (P.window > 0 && rpos[i] - P.window + 1 > 0) ? rpos[i] - P.window + 1 : 0;
        } else {
            rpos[i] = -1; rlo[i] = 0;
        }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }

    cp_async_wait<STAGES - 1>();
    __syncthreads();
    uint32_t qf[QREG ? KS : 1][4];
    if (QREG) {
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
            ldmatrix_x4(qf[QREG ? ks : 0], qs + swz<DK>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
    }
    const float LOG2E = 1.4426950408889634f;
    const float cap = GP.softcap, inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    for (int t = t_begin; t < t_end; t++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int tn = t + STAGES - 1;
            if (tn < t_end) fetch(tn);
            cp_async_commit();
        }
        const bf16* kt = kvs + (size_t)((t - t_begin) % STAGES) * STAGE;
        const bf16* vt = SHARED ? kt : kt + BN * ROWK;
        const int kb = lo_al + t * BN;

        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            if (!QREG) ldmatrix_x4(qf[0], qs + swz<DK>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + swz<DK>(nbase + np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[QREG ? ks : 0], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[QREG ? ks : 0], b[2], b[3]);
            }
        }
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = kb + nbase + j * 8 + 2 * tig + (e & 1);
                const bool ok = key <= rpos[i] && key >= rlo[i];
                float v = s[j][e] * GP.scale;
                // tanh(x) = 1 - 2 / (e^2x + 1) on the fast exponential and division (a few ulp; both ends saturate cleanly):
                // tanhf's own code was the longest chain of the tile (stalls on fixed-latency waits, tensor pipe 20 %)
                if (cap > 0.0f) v = cap * (1.0f - __fdividef(2.0f, __expf(2.0f * v * inv_cap) + 1.0f));
                v = ok ? v * LOG2E : -INFINITY;
                s[j][e] = v;
                tmax[i] = fmaxf(tmax[i], v);
            }
        }
        float corr[2], muse[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float m_new = fmaxf(m_run[i], tmax[i]);
            muse[i] = (m_new == -INFINITY) ? 0.0f : m_new;
            corr[i] = exp2f(m_run[i] - muse[i]);
            m_run[i] = m_new;
            l_run[i] *= corr[i];
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(s[j][e] - muse[e >> 1]);
                l_run[e >> 1] += p;
                s[j][e] = p;
            }
        }
#pragma unroll
        for (int d = 0; d < DT; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
#pragma unroll
        for (int kk = 0; kk < NT / 2; kk++) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DV / 16; dp++) {
                uint32_t b[4];
                const int vrow = nbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, vc = dp * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, vt + (SHARED ? swz<DK>(vrow, vc) : swz<DV>(vrow, vc)));
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    const int H = P.H;
    if (!DECODE) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = row0 + m0 + g + i * 8;
            if (r >= R) continue;
            const int tq = r / G, h = kvh * G + r % G;
            if (n_splits == 1) {
                float m2 = m_run[i], l = l_run[i], rescale, mult;
                ga_finish(GP, tok0 + tq, h, m2, l, rescale, mult);
                mult *= rescale;
                bf16* dst = P.out + ((size_t)(tok0 + tq) * H + h) * DV + 2 * tig;
#pragma unroll
                for (int d = 0; d < DT; d++)
                    *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2 * i] * mult, o[d][2 * i + 1] * mult);
            } else {
                const size_t base = ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits + split;
                float* dst = P.part_o + base * DV + 2 * tig;
#pragma unroll
                for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
                if (tig == 0) { P.part_ml[base * 2] = m_run[i]; P.part_ml[base * 2 + 1] = l_run[i]; }
            }
        }
    } else {
        __syncthreads();                                    // every warp is done with the K/V stages
        float* mo = reinterpret_cast<float*>(kvs);          // [4 warps][16 rows][DV]
        float* sm_m = mo + 4 * 16 * DV;                     // [4][16]
        float* sm_l = sm_m + 4 * 16;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int row = g + i * 8;
            float* dst = mo + ((size_t)(warp * 16 + row)) * DV + 2 * tig;
#pragma unroll
            for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
            if (tig == 0) { sm_m[warp * 16 + row] = m_run[i]; sm_l[warp * 16 + row] = l_run[i]; }
        }
        __syncthreads();
        for (int idx = tid; idx < 16 * DV; idx += 128) {
            const int row = idx / DV, d = idx % DV, r = row0 + row;
            if (r >= R) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w * 16 + row]);
            float acc = 0.0f, L = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float mw = sm_m[w * 16 + row];
                const float sc = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
                acc += mo[((size_t)(w * 16 + row)) * DV + d] * sc;
                L += sm_l[w * 16 + row] * sc;
            }
            const int tq = r / G, h = kvh * G + r % G;
            if (n_splits == 1) {
                float rescale, mult;
                ga_finish(GP, tok0 + tq, h, M, L, rescale, mult);
                P.out[((size_t)(tok0 + tq) * H + h) * DV + d] = __float2bfloat16_rn(acc * rescale * mult);
            } else {
                const size_t base = ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits + split;
                P.part_o[base * DV + d] = acc;
                if (d == 0) { P.part_ml[base * 2] = M; P.part_ml[base * 2 + 1] = L; }
            }
        }
    }
}

// Merges the splits of the tokens that were split: one block per (split token, head).
// part_tok[i] = (token index in the batch, number of splits of its sequence)
__global__ void attn_general_merge_kernel(const GenParams GP, const int2* __restrict__ part_tok, int DVr) {
    const AttnParams& P = GP.a;
    const int pt = blockIdx.x, h = blockIdx.y, H = P.H;
    const int n = part_tok[pt].x, ns = part_tok[pt].y;
    const size_t base = ((size_t)pt * H + h) * P.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < ns; s++) M = fmaxf(M, P.part_ml[(base + s) * 2]);
    float L = 0.0f;
    for (int s = 0; s < ns; s++) {
        const float ms = P.part_ml[(base + s) * 2];
        L += P.part_ml[(base + s) * 2 + 1] * ((ms == -INFINITY) ? 0.0f : exp2f(ms - M));
    }
    float M2 = M, rescale, mult;
    ga_finish(GP, n, h, M2, L, rescale, mult);
    for (int d = threadIdx.x; d < DVr; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < ns; s++) {
            const float ms = P.part_ml[(base + s) * 2];
            acc += P.part_o[(base + s) * DVr + d] * ((ms == -INFINITY) ? 0.0f : exp2f(ms - M));
        }
        P.out[((size_t)n * H + h) * DVr + d] = __float2bfloat16_rn(acc * rescale * mult);
    }
}

template <int DK, int DV, bool DECODE, int STAGES, bool SHARED>
static int launch_general(const GenParams& P, int n_items, cudaStream_t st) {
    constexpr int BM = DECODE ? 16 : 64;
    constexpr int ROWK = tile_row<DK>(), ROWV = SHARED ? 0 : tile_row<DV>();
    size_t smem = (size_t)BM * ROWK * 2 + (size_t)STAGES * 64 * (ROWK + ROWV) * 2;
    const size_t merge = (size_t)(4 * 16 * DV + 2 * 4 * 16) * 4 + (size_t)BM * ROWK * 2;
    if (DECODE && merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_general_kernel<DK, DV, DECODE, STAGES, SHARED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    attn_general_kernel<DK, DV, DECODE, STAGES, SHARED><<<dim3(n_items, P.a.KV), 128, smem, st>>>(P);
    MB_LAUNCH_CHECK();
    return 0;
}

static_assert(GA_DK % 16 == 0 && GA_DV % 16 == 0 && GA_DK >= 16 && GA_DV >= 16 && GA_DK <= 256 && GA_DV <= 256,
              "keys and values of the tensor-core form are multiples of 16 values, at most 256");

MB_API int mb_attn_general_dk() { return GA_DK; }
MB_API int mb_attn_general_dv() { return GA_DV; }

static void ga_fill(GenParams& GP, const void* q, int q_stride, void* out, const void* kpool, const void* vpool, int k_row,
                    int v_row, const int* q_start, const int* q_len, const int* pos0, const int* part_base,
                    const int* seq_row, const int* table, int max_blocks, float* part_o, float* part_ml, int max_splits,
                    int H, int KV, int page, int num_pages, int window, float scale, float softcap, const float* sinks,
                    const void* gate, int gate_stride, int* err) {
    AttnParams& P = GP.a;
    P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out;
    P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = nullptr;
    P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.part_base = part_base; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.part_o = part_o; P.part_ml = part_ml; P.max_splits = max_splits; P.counters = nullptr;
    P.H = H; P.KV = KV; P.G = H / KV; P.page = page; P.num_pages = num_pages; P.window = window;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    GP.k_row = k_row; GP.v_row = v_row; GP.scale = scale; GP.softcap = softcap; GP.sinks = sinks;
    GP.gate = (const bf16*)gate; GP.gate_stride = gate_stride;
}

// decode != 0: items are tiles of at most 16 rows; else tiles of 64 rows.
MB_API int mb_attn_general_bf16(const void* q, int q_stride, void* out, const void* kpool, const void* vpool, int k_row,
                                int v_row, const void* items, int n_items, int decode, const int* q_start,
                                const int* q_len, const int* pos0, const int* part_base, const int* seq_row,
                                const int* table, int max_blocks, float* part_o, float* part_ml, int max_splits, int H,
                                int KV, int DK, int DV, int page, int num_pages, int window, float scale, float softcap,
                                const float* sinks, const void* gate, int gate_stride, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (DK != GA_DK || DV != GA_DV || KV < 1 || H % KV || KV > 65535 || k_row < DK || v_row < DV || (k_row & 7) ||
        (v_row & 7) || (q_stride & 7))
        return -2;
    GenParams GP;
    ga_fill(GP, q, q_stride, out, kpool, vpool, k_row, v_row, q_start, q_len, pos0, part_base, seq_row, table, max_blocks,
            part_o, part_ml, max_splits, H, KV, page, num_pages, window, scale, softcap, sinks, gate, gate_stride, err);
    GP.a.items = (const int4*)items;
    constexpr int WIDE = (GA_DK > 128 || GA_DV > 128) ? 1 : 0;
    constexpr bool CAN_SHARE = GA_DV <= GA_DK;
    if (CAN_SHARE && kpool == vpool && k_row == v_row)
        return decode ? launch_general<GA_DK, GA_DV, true, 3, CAN_SHARE>(GP, n_items, st)
                      : launch_general<GA_DK, GA_DV, false, 2, CAN_SHARE>(GP, n_items, st);
    return decode ? launch_general<GA_DK, GA_DV, true, (WIDE ? 2 : 3), false>(GP, n_items, st)
                  : launch_general<GA_DK, GA_DV, false, 2, false>(GP, n_items, st);
}

MB_API int mb_attn_general_merge_bf16(float* part_o, float* part_ml, const void* part_tok, int n_part, void* out, int H,
                                      int DV, int max_splits, const float* sinks, const void* gate, int gate_stride,
                                      cudaStream_t st) {
    if (n_part == 0) return 0;
    GenParams GP;
    ga_fill(GP, nullptr, 0, out, nullptr, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, part_o,
            part_ml, max_splits, H, 1, 1, 0, 0, 1.0f, 0.0f, sinks, gate, gate_stride, nullptr);
    attn_general_merge_kernel<<<dim3(n_part, H), 128, 0, st>>>(GP, (const int2*)part_tok, DV);
    MB_LAUNCH_CHECK();
    return 0;
}
