// Short causal convolutions over time, one filter per channel, that carry their last inputs from step to step.
//
//   y[t, c] = sum_{j < taps} w[c, j] * u[t - taps + 1 + j, c],   u = in (+ bias),   zeros before the sequence's start.
//
// A step brings each sequence's next tokens, laid end to end; what came before them is not in the step, so every
// sequence keeps its last taps - 1 inputs in a state slot: state[slot][j][c], j = 0 the oldest.  A token at least
// taps - 1 tokens into its sequence's stretch of the step reads only rows of the step.  The first tokens of a stretch
// need the state, and the state must be replaced by the stretch's last inputs: ONE thread per (sequence, channel) --
// the thread of the stretch's first token -- does both, first the outputs of the first min(len, taps - 1) tokens from
// the state in its registers, then the new state, so no thread reads a state another one writes.  The threads of the
// other early tokens have nothing to do.  Sums run from the oldest tap to the newest in both forms, so a token's
// output does not depend on where the prompt was cut.
//
// Two kernels: the convolution alone (optionally added to its input), and the one that follows a fused q/k/v
// product: bias, convolution, rotation of the rotated dims of q and k by the token's position, q to its own buffer,
// k and v into the cache pages of the token's position.
#include "common.cuh"

#define CONV_MAX_TAPS 8

struct ConvSeq {                       // what the kernels need to know of the step's sequences
    const int* tok_seq;                // per token: index of its sequence in the step
    const int* q_start;                // per sequence: its first token in the step
    const int* q_len;                  // per sequence: tokens it brings
    const int* state_slot;             // per sequence: its state slot
};

template <typename T>
__device__ __forceinline__ float conv_input(const T* in, size_t stride, const float* bias, int n, int c) {
    float u = mb_load(in + (size_t)n * stride + c);
    return bias ? u + bias[c] : u;
}

// output of token n, channel c, for a token at least taps - 1 tokens into its stretch
template <typename T>
__device__ __forceinline__ float conv_inner(const T* in, size_t stride, const float* bias, const float* w, int taps,
                                            int n, int c) {
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++)
        if (j < taps) acc = fmaf(w ? w[(size_t)c * taps + j] : 1.0f, conv_input(in, stride, bias, n - taps + 1 + j, c), acc);
    return acc;
}

// The first m = min(len, taps - 1) outputs of a stretch that starts at token a, channel c, into y[]; replaces the
// state (st points at state[slot][0][c], rows are `srow` floats apart).  -> m
template <typename T>
__device__ __forceinline__ int conv_head(const T* in, size_t stride, const float* bias, const float* w, int taps,
                                         float* st, size_t srow, int a, int len, int c, float (&y)[CONV_MAX_TAPS - 1]) {
    float hist[CONV_MAX_TAPS - 1], wt[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; j++) hist[j] = (j < taps - 1) ? st[(size_t)j * srow] : 0.0f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++) wt[j] = (j < taps) ? (w ? w[(size_t)c * taps + j] : 1.0f) : 0.0f;
    const int m = len < taps - 1 ? len : taps - 1;
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; i++) {
        if (i >= m) break;
        const float u = conv_input(in, stride, bias, a + i, c);
        float acc = 0.0f, newest = wt[0];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; j++)
            if (j < taps - 1) { acc = fmaf(wt[j], hist[j], acc); newest = wt[j + 1]; }
        y[i] = fmaf(newest, u, acc);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 2; j++) hist[j] = hist[j + 1];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; j++)
            if (j == taps - 2) hist[j] = u;
    }
    if (len > taps - 1) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; j++)
            if (j < taps - 1) hist[j] = conv_input(in, stride, bias, a + len - (taps - 1) + j, c);
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; j++)
        if (j < taps - 1) st[(size_t)j * srow] = hist[j];
    return m;
}

// ------------------------------------------------------------------------------------------------ the convolution alone
// out[n, c] = (residual ? in[n, c] : 0) + conv(in)[n, c].  Thread per (token, channel).
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ in, const float* __restrict__ w, float* __restrict__ state,
                                  size_t slot_stride, ConvSeq sq, T* __restrict__ out, int C, int taps, int residual) {
    const int n = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t >= taps - 1) {
        float y = conv_inner(in, C, nullptr, w, taps, n, c);
        if (residual) y += mb_load(in + (size_t)n * C + c);
        mb_store(out + (size_t)n * C + c, y);
        return;
    }
    if (t != 0) return;
    float y[CONV_MAX_TAPS - 1];
    float* st = state + (size_t)sq.state_slot[s] * slot_stride + c;
    const int m = conv_head(in, C, nullptr, w, taps, st, C, a, sq.q_len[s], c, y);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; i++) {
        if (i >= m) break;
        float v = y[i];
        if (residual) v += mb_load(in + (size_t)(a + i) * C + c);
        mb_store(out + (size_t)(a + i) * C + c, v);
    }
}

// ------------------------------------------------------------------------------------------------ after a q/k/v product
// A row of `in` holds [QU query units | KU key units | VH value heads]: units of `dim` channels (a head, or one map of
// a head with several maps), value heads of `vdim`.  The first RD dims of every unit are rotated, dim i with dim
// i + RD/2.  Query units go to q_out (N, QU * dim); `kper` consecutive key units make the key row of one kv head in
// the cache, kpool (pages, VH, page, kper * dim); vpool (pages, VH, page, vdim).  KU = 0: the row holds queries only.
struct ConvQkv {
    int QU, KU, VH, dim, vdim, kper, RD;
    const float* freqs;                 // RD / 2 angles per position step, or null: no rotation
    const int* positions; const int* tok_row; const int* table; int max_blocks, page, num_pages;
};

template <typename T>
__device__ __forceinline__ void qkv_emit(const ConvQkv& p, T* q_out, T* kpool, T* vpool, int n, int c, float y0, float y1,
                                         bool pair, int* err) {
    const int qk = (p.QU + p.KU) * p.dim;
    const int pos = p.positions[n];
    size_t slot = 0;
    if (c >= p.QU * p.dim) {
        const int pg = p.table[(size_t)p.tok_row[n] * p.max_blocks + pos / p.page];
        if (pg < 0 || pg >= p.num_pages) {
            mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            return;
        }
        slot = (size_t)pg * p.VH * p.page + (pos % p.page);        // + kv head * page, then * row width
    }
    if (c >= qk) {                                                  // a value
        const int e = c - qk, g = e / p.vdim;
        mb_store(vpool + (slot + (size_t)g * p.page) * p.vdim + e % p.vdim, y0);
        return;
    }
    if (pair) {
        float sn, cs;
        sincosf((float)pos * p.freqs[c % p.dim], &sn, &cs);
        const float r0 = y0 * cs - y1 * sn, r1 = y1 * cs + y0 * sn;
        y0 = r0; y1 = r1;
    }
    const int half = p.RD / 2;
    if (c < p.QU * p.dim) {
        T* o = q_out + (size_t)n * p.QU * p.dim + c;
        mb_store(o, y0);
        if (pair) mb_store(o + half, y1);
    } else {
        const int e = c - p.QU * p.dim, unit = e / p.dim, g = unit / p.kper;
        T* o = kpool + (slot + (size_t)g * p.page) * (p.kper * p.dim) + (unit % p.kper) * p.dim + e % p.dim;
        mb_store(o, y0);
        if (pair) mb_store(o + half, y1);
    }
}

template <typename T>
__global__ void conv_rope_kv_write_kernel(const T* __restrict__ in, const float* __restrict__ bias,
                                          const float* __restrict__ w, float* __restrict__ state, size_t slot_stride,
                                          ConvSeq sq, ConvQkv p, T* __restrict__ q_out, T* __restrict__ kpool,
                                          T* __restrict__ vpool, int taps, int* err) {
    const int C = (p.QU + p.KU) * p.dim + p.VH * p.vdim;
    const int n = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    bool pair = false;
    if (c < (p.QU + p.KU) * p.dim && p.freqs) {
        const int d = c % p.dim;
        if (d < p.RD / 2) pair = true;
        else if (d < p.RD) return;                                  // its partner's thread does both
    }
    const int c1 = c + p.RD / 2;
    const int s = sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t >= taps - 1) {
        const float y0 = conv_inner(in, C, bias, w, taps, n, c);
        const float y1 = pair ? conv_inner(in, C, bias, w, taps, n, c1) : 0.0f;
        qkv_emit(p, q_out, kpool, vpool, n, c, y0, y1, pair, err);
        return;
    }
    if (t != 0) return;
    float y0[CONV_MAX_TAPS - 1], y1[CONV_MAX_TAPS - 1];
    float* st = state + (size_t)sq.state_slot[s] * slot_stride;
    const int m = conv_head(in, C, bias, w, taps, st + c, C, a, sq.q_len[s], c, y0);
    if (pair) conv_head(in, C, bias, w, taps, st + c1, C, a, sq.q_len[s], c1, y1);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; i++) {
        if (i >= m) break;
        qkv_emit(p, q_out, kpool, vpool, a + i, c, y0[i], pair ? y1[i] : 0.0f, pair, err);
    }
}

// ------------------------------------------------------------------------------------------------ launches
template <typename T>
static int short_conv_launch(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                             const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int C,
                             int taps, int residual, cudaStream_t st) {
    if (N == 0 || C == 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || N > 0x7fffffff / 2 || in == out) return -2;
    ConvSeq sq{tok_seq, q_start, q_len, state_slot};
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    short_conv_kernel<T><<<dim3(N, (C + threads - 1) / threads), threads, 0, st>>>(
        (const T*)in, w, state, (size_t)slot_stride, sq, (T*)out, C, taps, residual);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_short_conv_f32(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                             const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int C,
                             int taps, int residual, cudaStream_t st) {
    return short_conv_launch<float>(in, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, out, N, C, taps,
                                    residual, st);
}
MB_API int mb_short_conv_bf16(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                              const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int C,
                              int taps, int residual, cudaStream_t st) {
    return short_conv_launch<__nv_bfloat16>(in, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, out, N, C,
                                            taps, residual, st);
}

template <typename T>
static int conv_qkv_launch(const void* in, const float* bias, const float* w, float* state, long long slot_stride,
                           const int* tok_seq, const int* q_start, const int* q_len, const int* state_slot,
                           const int* positions, const int* tok_row, const int* table, int max_blocks, void* q_out,
                           void* kpool, void* vpool, const float* freqs, int N, int QU, int KU, int VH, int dim,
                           int vdim, int kper, int RD, int page, int num_pages, int taps, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || dim < 1 || QU < 0 || KU < 0 || VH < 0 || (KU > 0 && (kper < 1 || KU != VH * kper)))
        return -2;
    if (freqs && (RD < 2 || RD % 2 || RD > dim)) return -2;
    if ((KU > 0 || VH > 0) && (!kpool || !vpool || !table)) return -2;
    const int C = (QU + KU) * dim + VH * vdim;
    ConvSeq sq{tok_seq, q_start, q_len, state_slot};
    ConvQkv p{QU, KU, VH, dim, vdim, kper, freqs ? RD : 0, freqs, positions, tok_row, table, max_blocks, page, num_pages};
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    conv_rope_kv_write_kernel<T><<<dim3(N, (C + threads - 1) / threads), threads, 0, st>>>(
        (const T*)in, bias, w, state, (size_t)slot_stride, sq, p, (T*)q_out, (T*)kpool, (T*)vpool, taps, err);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_conv_rope_kv_write_f32(const void* in, const float* bias, const float* w, float* state,
                                     long long slot_stride, const int* tok_seq, const int* q_start, const int* q_len,
                                     const int* state_slot, const int* positions, const int* tok_row, const int* table,
                                     int max_blocks, void* q_out, void* kpool, void* vpool, const float* freqs, int N,
                                     int QU, int KU, int VH, int dim, int vdim, int kper, int RD, int page,
                                     int num_pages, int taps, int* err, cudaStream_t st) {
    return conv_qkv_launch<float>(in, bias, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, positions,
                                  tok_row, table, max_blocks, q_out, kpool, vpool, freqs, N, QU, KU, VH, dim, vdim, kper,
                                  RD, page, num_pages, taps, err, st);
}
MB_API int mb_conv_rope_kv_write_bf16(const void* in, const float* bias, const float* w, float* state,
                                      long long slot_stride, const int* tok_seq, const int* q_start, const int* q_len,
                                      const int* state_slot, const int* positions, const int* tok_row, const int* table,
                                      int max_blocks, void* q_out, void* kpool, void* vpool, const float* freqs, int N,
                                      int QU, int KU, int VH, int dim, int vdim, int kper, int RD, int page,
                                      int num_pages, int taps, int* err, cudaStream_t st) {
    return conv_qkv_launch<__nv_bfloat16>(in, bias, w, state, slot_stride, tok_seq, q_start, q_len, state_slot,
                                          positions, tok_row, table, max_blocks, q_out, kpool, vpool, freqs, N, QU, KU,
                                          VH, dim, vdim, kper, RD, page, num_pages, taps, err, st);
}
