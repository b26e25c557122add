// Short causal convolutions over time, one filter per channel, that carry their last inputs from step to step.
//
//   y[t, c] = sum_{j < taps} w[j, c] * u[t - taps + 1 + j, c],   u = in (+ bias),   zeros before the sequence's start.
// The filters are held tap by tap, w (taps, channels), so that neighbouring threads read neighbouring weights.
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
        if (j < taps) acc = fmaf(w ? w[(size_t)j * stride + c] : 1.0f, conv_input(in, stride, bias, n - taps + 1 + j, c), acc);
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
    for (int j = 0; j < CONV_MAX_TAPS; j++) wt[j] = (j < taps) ? (w ? w[(size_t)j * stride + c] : 1.0f) : 0.0f;
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
                                  size_t slot_stride, ConvSeq sq, T* __restrict__ out, int C, int taps, int residual,
                                  int heads_only) {
    // heads_only: a block row per sequence, for the first tokens of its stretch and its state only
    const int n = heads_only ? sq.q_start[blockIdx.x] : blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = heads_only ? blockIdx.x : sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t >= taps - 1) {
        if (heads_only) return;
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
                                          T* __restrict__ vpool, int taps, int heads_only, int* err) {
    const int C = (p.QU + p.KU) * p.dim + p.VH * p.vdim;
    const int n = heads_only ? sq.q_start[blockIdx.x] : blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    bool pair = false;
    if (c < (p.QU + p.KU) * p.dim && p.freqs) {
        const int d = c % p.dim;
        if (d < p.RD / 2) pair = true;
        else if (d < p.RD) return;                                  // its partner's thread does both
    }
    const int c1 = c + p.RD / 2;
    const int s = heads_only ? blockIdx.x : sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t >= taps - 1) {
        if (heads_only) return;
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

// ------------------------------------------------------------------------------------------------ eight channels a thread
// The tokens that need no state (at least taps - 1 tokens into their stretch), with 128-bit accesses: a thread owns
// eight consecutive channels of a token (and, in a rotated stretch, the eight partner channels RD/2 further on).  These
// kernels take channel counts, unit sizes and value sizes that are multiples of 8 and rotations whose half is a
// multiple of 8; the heads of the stretches (and the state) are then left to the kernels above, launched over the
// sequences instead of the tokens (`heads_only`).  The sums are the same in the same order.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}

template <typename T>
__device__ __forceinline__ void conv_inner8(const T* in, size_t stride, const float* bias, const float* w, int taps, int n,
                                            int c, float (&y)[8]) {
    float b[8];
#pragma unroll
    for (int e = 0; e < 8; e++) { y[e] = 0.0f; b[e] = 0.0f; }
    if (bias) load8(bias + c, b);
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++) {
        if (j < taps) {
            float u[8], wt[8];
            load8(in + (size_t)(n - taps + 1 + j) * stride + c, u);
            if (w) load8(w + (size_t)j * stride + c, wt);           // the filters lie tap by tap: eight channels side by side
#pragma unroll
            for (int e = 0; e < 8; e++) y[e] = fmaf(w ? wt[e] : 1.0f, u[e] + b[e], y[e]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) short_conv_vec_kernel(const T* __restrict__ in, const float* __restrict__ w,
                                                            float* __restrict__ state, size_t slot_stride, ConvSeq sq,
                                                            T* __restrict__ out, int C, int taps, int residual) {
    const int n = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int s = sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t < taps - 1) return;                                       // a head of a stretch: the other kernel's
    float y[8];
    conv_inner8(in, C, nullptr, w, taps, n, c, y);
    if (residual) {
        float u[8];
        load8(in + (size_t)n * C + c, u);
#pragma unroll
        for (int e = 0; e < 8; e++) y[e] += u[e];
    }
    store8(out + (size_t)n * C + c, y);
}

// rotates (when pair; cs: the token's cosines and sines, one per rotated pair) and stores eight channels from c on (and
// their partners) of token n
template <typename T>
__device__ __forceinline__ void qkv_emit8(const ConvQkv& p, T* q_out, T* kpool, T* vpool, int n, int c, float (&y0)[8],
                                          float (&y1)[8], bool pair, const float2* cs, int* err) {
    const int qk = (p.QU + p.KU) * p.dim;
    const int pos = p.positions[n];
    size_t slot = 0;
    if (c >= p.QU * p.dim) {
        const int pg = p.table[(size_t)p.tok_row[n] * p.max_blocks + pos / p.page];
        if (pg < 0 || pg >= p.num_pages) {
            mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            return;
        }
        slot = (size_t)pg * p.VH * p.page + (pos % p.page);
    }
    if (c >= qk) {
        const int e = c - qk, g = e / p.vdim;
        store8(vpool + (slot + (size_t)g * p.page) * p.vdim + e % p.vdim, y0);
        return;
    }
    if (pair) {
        const int d = c % p.dim;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float2 t = cs[d + e];                             // (cos, sin) of the token's angle for this pair
            const float r0 = y0[e] * t.x - y1[e] * t.y, r1 = y1[e] * t.x + y0[e] * t.y;
            y0[e] = r0; y1[e] = r1;
        }
    }
    const int half = p.RD / 2;
    T* o;
    if (c < p.QU * p.dim) {
        o = q_out + (size_t)n * p.QU * p.dim + c;
    } else {
        const int e = c - p.QU * p.dim, unit = e / p.dim, g = unit / p.kper;
        o = kpool + (slot + (size_t)g * p.page) * (p.kper * p.dim) + (unit % p.kper) * p.dim + e % p.dim;
    }
    store8(o, y0);
    if (pair) store8(o + half, y1);
}

template <typename T>
__global__ void __launch_bounds__(128) conv_rope_kv_write_vec_kernel(const T* __restrict__ in, const float* __restrict__ bias,
                                                                    const float* __restrict__ w, float* __restrict__ state,
                                                                    size_t slot_stride, ConvSeq sq, ConvQkv p,
                                                                    T* __restrict__ q_out, T* __restrict__ kpool,
                                                                    T* __restrict__ vpool, int taps, int* err) {
    extern __shared__ float2 rope_cs[];                             // (cos, sin) of the token's RD / 2 pairs
    const int C = (p.QU + p.KU) * p.dim + p.VH * p.vdim;
    const int n = blockIdx.x;
    const int s = sq.tok_seq[n], a = sq.q_start[s], t = n - a;
    if (t < taps - 1) return;                                       // a head of a stretch: the other kernel's (whole block)
    if (p.freqs) {
        const float pos = (float)p.positions[n];
        for (int i = threadIdx.x; i < p.RD / 2; i += blockDim.x) {
            float sn, cs;
            sincosf(pos * p.freqs[i], &sn, &cs);
            rope_cs[i] = make_float2(cs, sn);
        }
        __syncthreads();
    }
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    bool pair = false;
    if (c < (p.QU + p.KU) * p.dim && p.freqs) {
        const int d = c % p.dim;
        if (d < p.RD / 2) pair = true;
        else if (d < p.RD) return;
    }
    const int c1 = c + p.RD / 2;
    float y0[8], y1[8];
    conv_inner8(in, C, bias, w, taps, n, c, y0);
    if (pair) conv_inner8(in, C, bias, w, taps, n, c1, y1);
    qkv_emit8(p, q_out, kpool, vpool, n, c, y0, y1, pair, rope_cs, err);
}

// ------------------------------------------------------------------------------------------------ launches
template <typename T>
static int short_conv_launch(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                             const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int S, int C,
                             int taps, int residual, cudaStream_t st) {
    if (N == 0 || C == 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || N > 0x7fffffff / 2 || in == out) return -2;
    ConvSeq sq{tok_seq, q_start, q_len, state_slot};
    if (C % 8 == 0 && slot_stride % 4 == 0 && (((uintptr_t)in | (uintptr_t)out | (uintptr_t)state) & 15) == 0) {
        const int groups = C / 8, threads = groups >= 128 ? 128 : ((groups + 31) / 32) * 32;
        if (N > S || taps == 1)                 // N == S: every stretch is one token, a head
            short_conv_vec_kernel<T><<<dim3(N, (groups + threads - 1) / threads), threads, 0, st>>>(
                (const T*)in, w, state, (size_t)slot_stride, sq, (T*)out, C, taps, residual);
        if (taps > 1) {
            const int th = C >= 256 ? 256 : ((C + 31) / 32) * 32;
            short_conv_kernel<T><<<dim3(S, (C + th - 1) / th), th, 0, st>>>(
                (const T*)in, w, state, (size_t)slot_stride, sq, (T*)out, C, taps, residual, 1);
        }
        MB_LAUNCH_CHECK();
        return 0;
    }
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    short_conv_kernel<T><<<dim3(N, (C + threads - 1) / threads), threads, 0, st>>>(
        (const T*)in, w, state, (size_t)slot_stride, sq, (T*)out, C, taps, residual, 0);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_short_conv_f32(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                             const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int S, int C,
                             int taps, int residual, cudaStream_t st) {
    return short_conv_launch<float>(in, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, out, N, S, C, taps,
                                    residual, st);
}
MB_API int mb_short_conv_bf16(const void* in, const float* w, float* state, long long slot_stride, const int* tok_seq,
                              const int* q_start, const int* q_len, const int* state_slot, void* out, int N, int S, int C,
                              int taps, int residual, cudaStream_t st) {
    return short_conv_launch<__nv_bfloat16>(in, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, out, N, S, C,
                                            taps, residual, st);
}

template <typename T>
static int conv_qkv_launch(const void* in, const float* bias, const float* w, float* state, long long slot_stride,
                           const int* tok_seq, const int* q_start, const int* q_len, const int* state_slot,
                           const int* positions, const int* tok_row, const int* table, int max_blocks, void* q_out,
                           void* kpool, void* vpool, const float* freqs, int N, int S, int QU, int KU, int VH,
                           int dim, int vdim, int kper, int RD, int page, int num_pages, int taps, int* err,
                           cudaStream_t st) {
    if (N == 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || dim < 1 || QU < 0 || KU < 0 || VH < 0 || (KU > 0 && (kper < 1 || KU != VH * kper)))
        return -2;
    if (freqs && (RD < 2 || RD % 2 || RD > dim)) return -2;
    if ((KU > 0 || VH > 0) && (!kpool || !vpool || !table)) return -2;
    const int C = (QU + KU) * dim + VH * vdim;
    ConvSeq sq{tok_seq, q_start, q_len, state_slot};
    ConvQkv p{QU, KU, VH, dim, vdim, kper, freqs ? RD : 0, freqs, positions, tok_row, table, max_blocks, page, num_pages};
    if (dim % 8 == 0 && (VH == 0 || vdim % 8 == 0) && (!freqs || RD % 16 == 0) && slot_stride % 4 == 0 &&
        (((uintptr_t)in | (uintptr_t)q_out | (uintptr_t)kpool | (uintptr_t)vpool | (uintptr_t)state | (uintptr_t)bias) & 15) == 0) {
        const int groups = C / 8, threads = groups >= 128 ? 128 : ((groups + 31) / 32) * 32;
        if (N > S || taps == 1)                 // N == S: every stretch is one token, a head
            conv_rope_kv_write_vec_kernel<T><<<dim3(N, (groups + threads - 1) / threads), threads,
                                               (freqs ? RD / 2 : 0) * sizeof(float2), st>>>(
                (const T*)in, bias, w, state, (size_t)slot_stride, sq, p, (T*)q_out, (T*)kpool, (T*)vpool, taps, err);
        if (taps > 1) {
            const int th = C >= 256 ? 256 : ((C + 31) / 32) * 32;
            conv_rope_kv_write_kernel<T><<<dim3(S, (C + th - 1) / th), th, 0, st>>>(
                (const T*)in, bias, w, state, (size_t)slot_stride, sq, p, (T*)q_out, (T*)kpool, (T*)vpool, taps, 1, err);
        }
        MB_LAUNCH_CHECK();
        return 0;
    }
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    conv_rope_kv_write_kernel<T><<<dim3(N, (C + threads - 1) / threads), threads, 0, st>>>(
        (const T*)in, bias, w, state, (size_t)slot_stride, sq, p, (T*)q_out, (T*)kpool, (T*)vpool, taps, 0, err);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_conv_rope_kv_write_f32(const void* in, const float* bias, const float* w, float* state,
                                     long long slot_stride, const int* tok_seq, const int* q_start, const int* q_len,
                                     const int* state_slot, const int* positions, const int* tok_row, const int* table,
                                     int max_blocks, void* q_out, void* kpool, void* vpool, const float* freqs, int N,
                                     int S, int QU, int KU, int VH, int dim, int vdim, int kper, int RD, int page,
                                     int num_pages, int taps, int* err, cudaStream_t st) {
    return conv_qkv_launch<float>(in, bias, w, state, slot_stride, tok_seq, q_start, q_len, state_slot, positions,
                                  tok_row, table, max_blocks, q_out, kpool, vpool, freqs, N, S, QU, KU, VH, dim, vdim, kper,
                                  RD, page, num_pages, taps, err, st);
}
MB_API int mb_conv_rope_kv_write_bf16(const void* in, const float* bias, const float* w, float* state,
                                      long long slot_stride, const int* tok_seq, const int* q_start, const int* q_len,
                                      const int* state_slot, const int* positions, const int* tok_row, const int* table,
                                      int max_blocks, void* q_out, void* kpool, void* vpool, const float* freqs, int N,
                                      int S, int QU, int KU, int VH, int dim, int vdim, int kper, int RD, int page,
                                      int num_pages, int taps, int* err, cudaStream_t st) {
    return conv_qkv_launch<__nv_bfloat16>(in, bias, w, state, slot_stride, tok_seq, q_start, q_len, state_slot,
                                          positions, tok_row, table, max_blocks, q_out, kpool, vpool, freqs, N, S, QU, KU,
                                          VH, dim, vdim, kper, RD, page, num_pages, taps, err, st);
}
