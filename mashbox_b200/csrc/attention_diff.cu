// Differential attention over the paged cache, plain form: one warp per (token, query head).
//
// A head has two attention maps with queries and keys of their own and ONE set of values:
//     a_m = softmax(scale * q_m K_m^T) V  (m = 0, 1),   o = a_0 - lam * a_1,   out = o / sqrt(mean(o^2) + eps) * gain
// (the mean over the head's value dims).  A query row holds its head's two maps side by side, [q_0 | q_1], `dim` each;
// a key row of the cache likewise, kpool (pages, G, page, 2 dim); values vpool (pages, G, page, vdim).  Query head h
// reads kv head h / (H / G).  Which keys a query sees: those of its own block of `chunk` positions (blocks counted
// from position 0 of the sequence) up to its own position; chunk 0: every key up to its own position.  The step's
// own tokens are read from the cache like older ones.
//
// It serves the float32 path and, on the bf16 path, the sizes the tensor-core kernel does not take.  Scores, both
// softmaxes, the weighted sums, the difference and the norm are float.  Keys are taken in ascending position, 32 at a
// time from the block's start, so the order of every sum depends on the query's position only.
#include "common.cuh"

#define DIFF_MAX_DIM 256
#define DIFF_MAX_VDIM 256
#define DIFF_WARPS 4

template <typename T>
__global__ void __launch_bounds__(DIFF_WARPS * 32) attn_diff_simple_kernel(
    const T* __restrict__ q, T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ tok_row,
    const int* __restrict__ table, int max_blocks, const T* __restrict__ kpool, const T* __restrict__ vpool, int N,
    int H, int G, int dim, int vdim, int page, int num_pages, int chunk, float scale, float lam, float gain, float eps,
    int* err) {
    extern __shared__ float qs_all[];                              // per warp: 2 dim floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * DIFF_WARPS + warp;
    if (item >= (long long)N * H) return;
    float* qs = qs_all + (size_t)warp * 2 * dim;
    const int n = (int)(item / H), h = (int)(item % H);
    const int g = h / (H / G);
    const int pos = positions[n];
    const int* tb = table + (size_t)tok_row[n] * max_blocks;
    const T* qr = q + ((size_t)n * H + h) * 2 * dim;
    for (int d = lane; d < 2 * dim; d += 32) qs[d] = mb_load(qr + d);
    __syncwarp();
    const int lo = chunk > 0 ? pos / chunk * chunk : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    float acc0[DIFF_MAX_VDIM / 32], acc1[DIFF_MAX_VDIM / 32];
#pragma unroll
    for (int i = 0; i < DIFF_MAX_VDIM / 32; i++) acc0[i] = acc1[i] = 0.0f;
    for (int base = lo; base <= pos; base += 32) {
        const int kp = base + lane;
        long long row = -1;                                        // (page * G + g) * page_size + slot of this lane's key
        float s0 = -INFINITY, s1 = -INFINITY;
        if (kp <= pos) {
            const int pg = tb[kp / page];
            if (pg < 0 || pg >= num_pages) {
                mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            } else {
                row = ((long long)pg * G + g) * page + (kp % page);
                const T* kr = kpool + row * 2 * dim;
                float a = 0.0f, b = 0.0f;
                for (int d = 0; d < dim; d++) {
                    a = fmaf(qs[d], mb_load(kr + d), a);
                    b = fmaf(qs[dim + d], mb_load(kr + dim + d), b);
                }
                s0 = a * scale;
                s1 = b * scale;
            }
        }
        const float n0 = fmaxf(m0, mb_warp_max(s0)), n1 = fmaxf(m1, mb_warp_max(s1));
        if (n0 == -INFINITY) continue;                             // only after a table error: nothing to add
        const float p0 = row >= 0 ? expf(s0 - n0) : 0.0f, p1 = row >= 0 ? expf(s1 - n1) : 0.0f;
        const float c0 = expf(m0 - n0), c1 = expf(m1 - n1);
        l0 = l0 * c0 + mb_warp_sum(p0);
        l1 = l1 * c1 + mb_warp_sum(p1);
#pragma unroll
        for (int i = 0; i < DIFF_MAX_VDIM / 32; i++) { acc0[i] *= c0; acc1[i] *= c1; }
        const int cnt = min(32, pos - base + 1);
        for (int j = 0; j < cnt; j++) {
            const float w0 = __shfl_sync(0xffffffffu, p0, j), w1 = __shfl_sync(0xffffffffu, p1, j);
            const long long rj = __shfl_sync(0xffffffffu, row, j);
            if (rj < 0) continue;
            const T* vr = vpool + rj * vdim;
#pragma unroll
            for (int i = 0; i < DIFF_MAX_VDIM / 32; i++) {
                const int d = lane + 32 * i;
                if (d < vdim) {
                    const float v = mb_load(vr + d);
                    acc0[i] = fmaf(w0, v, acc0[i]);
                    acc1[i] = fmaf(w1, v, acc1[i]);
                }
            }
        }
        m0 = n0;
        m1 = n1;
    }
    const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_VDIM / 32; i++) {
        const int d = lane + 32 * i;
        const float o = d < vdim ? acc0[i] * i0 - lam * (acc1[i] * i1) : 0.0f;
        acc0[i] = o;
        ss = fmaf(o, o, ss);
    }
    ss = mb_warp_sum(ss);
    const float f = rsqrtf(ss / (float)vdim + eps) * gain;
    T* o = out + ((size_t)n * H + h) * vdim;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_VDIM / 32; i++) {
        const int d = lane + 32 * i;
        if (d < vdim) mb_store(o + d, acc0[i] * f);
    }
}

template <typename T>
static int attn_diff_simple_launch(const void* q, void* out, const int* positions, const int* tok_row, const int* table,
                                   int max_blocks, const void* kpool, const void* vpool, int N, int H, int G, int dim,
                                   int vdim, int page, int num_pages, int chunk, float scale, float lam, float gain,
                                   float eps, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (dim < 1 || dim > DIFF_MAX_DIM || vdim < 1 || vdim > DIFF_MAX_VDIM || G < 1 || H % G || chunk < 0) return -2;
    const long long items = (long long)N * H;
    const size_t smem = (size_t)DIFF_WARPS * 2 * dim * sizeof(float);
    attn_diff_simple_kernel<T><<<(unsigned)((items + DIFF_WARPS - 1) / DIFF_WARPS), DIFF_WARPS * 32, smem, st>>>(
        (const T*)q, (T*)out, positions, tok_row, table, max_blocks, (const T*)kpool, (const T*)vpool, N, H, G, dim,
        vdim, page, num_pages, chunk, scale, lam, gain, eps, err);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_attn_diff_simple_f32(const void* q, void* out, const int* positions, const int* tok_row, const int* table,
                                   int max_blocks, const void* kpool, const void* vpool, int N, int H, int G, int dim,
                                   int vdim, int page, int num_pages, int chunk, float scale, float lam, float gain,
                                   float eps, int* err, cudaStream_t st) {
    return attn_diff_simple_launch<float>(q, out, positions, tok_row, table, max_blocks, kpool, vpool, N, H, G, dim, vdim,
                                          page, num_pages, chunk, scale, lam, gain, eps, err, st);
}
MB_API int mb_attn_diff_simple_bf16(const void* q, void* out, const int* positions, const int* tok_row, const int* table,
                                    int max_blocks, const void* kpool, const void* vpool, int N, int H, int G, int dim,
                                    int vdim, int page, int num_pages, int chunk, float scale, float lam, float gain,
                                    float eps, int* err, cudaStream_t st) {
    return attn_diff_simple_launch<__nv_bfloat16>(q, out, positions, tok_row, table, max_blocks, kpool, vpool, N, H, G,
                                                  dim, vdim, page, num_pages, chunk, scale, lam, gain, eps, err, st);
}
