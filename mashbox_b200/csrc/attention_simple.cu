// Paged attention, plain form: one warp per (token, query head), keys in ascending position through the block table.
// It serves the whole float32 path and, on the bf16 path, every head size the tensor-core kernel does not take.
// Scores, softmax and the weighted sum are float.  The order of every sum depends only on the query's position and
// the window, never on how tokens were cut into steps or which pages hold the keys.
//
// Keys and values may differ in width (HD values of a key row enter the score, HDV values of a value row the sum) and a
// row of either pool may be wider than what is read of it (k_row, v_row: the distance between two positions' rows; a
// pool whose rows are key and value at once is handed in twice).  Optional: a cap on the scores, s <- cap tanh(s / cap);
// a sink per query head, one more term exp(sink_h) in the softmax's denominator that has no value; a gate per token and
// query head, the head's result times sigmoid(gate).
#include "common.cuh"

#define SIMPLE_MAX_HD 1024         // the widest rows (three instantiations: up to 256, up to 512, and up to this)
#define WARPS 4

template <typename T, int MAXHD>
__global__ void __launch_bounds__(WARPS * 32) attn_simple_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, const int* __restrict__ positions,
    const int* __restrict__ tok_seq, const int* __restrict__ table, int max_blocks, const T* __restrict__ kpool,
    const T* __restrict__ vpool, int N, int H, int KV, int HD, int page, int num_pages, int window, float scale,
    int* err, int HDV, int k_row, int v_row, float softcap, const float* __restrict__ sinks,
    const T* __restrict__ gate, int gate_stride) {
    __shared__ float qs[WARPS][MAXHD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)N * H) return;
    const int n = (int)(item / H), h = (int)(item % H);
    const int kvh = h / (H / KV);
    const int pos = positions[n];
    const int* tb = table + (size_t)tok_seq[n] * max_blocks;
    const T* qr = q + (size_t)n * q_stride + (size_t)h * HD;
    for (int d = lane; d < HD; d += 32) qs[warp][d] = mb_load(qr + d);
    __syncwarp();
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[MAXHD / 32];
#pragma unroll
    for (int i = 0; i < MAXHD / 32; i++) acc[i] = 0.0f;
    for (int base = lo; base <= pos; base += 32) {
        const int kp = base + lane;
        const bool valid = kp <= pos;
        long long off = -1;        // the position's row among the rows of its kv head's pages (times k_row or v_row)
        float s = -INFINITY;
        if (valid) {
            const int pg = tb[kp / page];
            if (pg < 0 || pg >= num_pages) {
                mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            } else {
                off = ((long long)pg * KV + kvh) * page + (kp % page);
                const T* kr = kpool + off * k_row;
                float a = 0.0f;
                for (int d = 0; d < HD; d++) a = fmaf(qs[warp][d], mb_load(kr + d), a);
                s = a * scale;
                if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
            }
        }
        const float tmax = mb_warp_max(s);
        const float m_new = fmaxf(m, tmax);
        if (m_new == -INFINITY) continue;                      // only after a table error: nothing to add
        const float p = (off >= 0) ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + mb_warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAXHD / 32; i++) acc[i] *= corr;
        const int cnt = min(32, pos - base + 1);
        for (int j = 0; j < cnt; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            if (oj < 0) continue;
            const T* vr = vpool + oj * v_row;
#pragma unroll
            for (int i = 0; i < MAXHD / 32; i++) {
                const int d = lane + 32 * i;
                if (d < HDV) acc[i] = fmaf(pj, mb_load(vr + d), acc[i]);
            }
        }
        m = m_new;
    }
    if (sinks) {                                                // one more term in the denominator, after every key
        const float sk = sinks[h], m_new = fmaxf(m, sk), corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < MAXHD / 32; i++) acc[i] *= corr;
    }
    float inv = l > 0.0f ? 1.0f / l : 0.0f;
    if (gate) inv /= 1.0f + expf(-mb_load(gate + (size_t)n * gate_stride + h));
    T* o = out + (size_t)n * H * HDV + (size_t)h * HDV;
#pragma unroll
    for (int i = 0; i < MAXHD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < HDV) mb_store(o + d, acc[i] * inv);
    }
}

template <typename T>
static int attn_simple_launch(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                              const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                              int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                              cudaStream_t st, int HDV = 0, int k_row = 0, int v_row = 0, float softcap = 0.0f,
                              const float* sinks = nullptr, const void* gate_ = nullptr, int gate_stride = 0) {
    if (N == 0) return 0;
    if (HDV == 0) HDV = HD;
    if (k_row == 0) k_row = HD;
    if (v_row == 0) v_row = HDV;
    const T* gate = (const T*)gate_;
    const int widest = HD > HDV ? HD : HDV;
    if (widest > SIMPLE_MAX_HD || HD < 1 || HDV < 1 || KV < 1 || H % KV || k_row < HD || v_row < HDV) return -2;
    const long long items = (long long)N * H;
    if (widest <= 256)
        attn_simple_kernel<T, 256><<<(unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, st>>>(
            (const T*)q, q_stride, (T*)out, positions, tok_seq, table, max_blocks, (const T*)kpool, (const T*)vpool, N, H,
            KV, HD, page, num_pages, window, scale, err, HDV, k_row, v_row, softcap, sinks, gate, gate_stride);
    else if (widest <= 512)
        attn_simple_kernel<T, 512><<<(unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, st>>>(
            (const T*)q, q_stride, (T*)out, positions, tok_seq, table, max_blocks, (const T*)kpool, (const T*)vpool, N, H,
            KV, HD, page, num_pages, window, scale, err, HDV, k_row, v_row, softcap, sinks, gate, gate_stride);
    else
        attn_simple_kernel<T, SIMPLE_MAX_HD><<<(unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, st>>>(
            (const T*)q, q_stride, (T*)out, positions, tok_seq, table, max_blocks, (const T*)kpool, (const T*)vpool, N, H,
            KV, HD, page, num_pages, window, scale, err, HDV, k_row, v_row, softcap, sinks, gate, gate_stride);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_attn_simple_f32(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                              const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                              int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                              cudaStream_t st) {
    return attn_simple_launch<float>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N, H, KV,
                                     HD, page, num_pages, window, scale, err, st);
}
MB_API int mb_attn_simple_bf16(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                               const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                               int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                               cudaStream_t st) {
    return attn_simple_launch<__nv_bfloat16>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N,
                                             H, KV, HD, page, num_pages, window, scale, err, st);
}

// the general form: keys of HD and values of HDV, rows k_row and v_row apart, capped scores, sinks, a gate per head
MB_API int mb_attn_simple_ext_f32(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                                  const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                                  int KV, int HD, int HDV, int k_row, int v_row, int page, int num_pages, int window,
                                  float scale, float softcap, const float* sinks, const void* gate, int gate_stride,
                                  int* err, cudaStream_t st) {
    return attn_simple_launch<float>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N, H, KV,
                                     HD, page, num_pages, window, scale, err, st, HDV, k_row, v_row, softcap, sinks, gate,
                                     gate_stride);
}
MB_API int mb_attn_simple_ext_bf16(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                                   const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                                   int KV, int HD, int HDV, int k_row, int v_row, int page, int num_pages, int window,
                                   float scale, float softcap, const float* sinks, const void* gate, int gate_stride,
                                   int* err, cudaStream_t st) {
    return attn_simple_launch<__nv_bfloat16>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N,
                                             H, KV, HD, page, num_pages, window, scale, err, st, HDV, k_row, v_row, softcap,
                                             sinks, gate, gate_stride);
}
