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
// moe_experts is the form for steps of few tokens: a block per (token, expert) streams that expert's three matrices once,
// which is what a decode step has to read anyway.  Dot products run over lanes with 16-byte loads where rows allow.
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
__global__ void moe_select_kernel(const float* __restrict__ z, const float* __restrict__ correction, int* __restrict__ ids,
                                  float* __restrict__ wts, int E, int top, int groups, int keep) {
    extern __shared__ float sm[];
    float* s = sm;
    float* c = sm + E;
    float* gs = sm + 2 * E;
    float* kept = gs + groups;
    const int n = blockIdx.x, lane = threadIdx.x;
    for (int e = lane; e < E; e += 32) {
        const float v = 1.0f / (1.0f + expf(-z[(size_t)n * E + e]));
        s[e] = v;
        c[e] = v + (correction ? correction[e] : 0.0f);
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
            gs[gi] = per > 1 ? a + b : a;
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
            wts[(size_t)n * top + kk] = s[at];
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

// grid (N, top); dynamic shared: h[D], act[F].  wg, wu (E, F, D); wd (E, D, F); y (N, top, D) float32
template <typename T>
__global__ void moe_experts_kernel(const T* __restrict__ h, const int* __restrict__ ids, const T* __restrict__ wg,
                                   const T* __restrict__ wu, const T* __restrict__ wd, float* __restrict__ y, int D, int F,
                                   int E, int top, float limit, float alpha) {
    extern __shared__ float sm[];
    float* hx = sm;
    float* act = sm + D;
    const int n = blockIdx.x, kk = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int e = ids[(size_t)n * top + kk];
    if (e < 0 || e >= E) e = 0;
    for (int d = threadIdx.x; d < D; d += blockDim.x) hx[d] = mb_load(h + (size_t)n * D + d);
    __syncthreads();
    const T* g_rows = wg + (size_t)e * F * D;
    const T* u_rows = wu + (size_t)e * F * D;
    for (int j = warp; j < F; j += nwarp) {
        float g = lane_dot(g_rows + (size_t)j * D, hx, D, lane);
        float u = lane_dot(u_rows + (size_t)j * D, hx, D, lane);
        if (lane == 0) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            act[j] = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
        }
    }
    __syncthreads();
    const T* d_rows = wd + (size_t)e * D * F;
    float* out = y + ((size_t)n * top + kk) * D;
    for (int d = warp; d < D; d += nwarp) {
        const float v = lane_dot(d_rows + (size_t)d * F, act, F, lane);
        if (lane == 0) out[d] = v;
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, T* __restrict__ out, int D,
                                   int top, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / D;
    const int d = (int)(i - n * D);
    float acc = 0.0f;
    for (int kk = 0; kk < top; kk++) acc = fmaf(wts[n * top + kk], y[(n * top + kk) * D + d], acc);
    mb_store(out + i, acc);
}

MB_API int mb_moe_select(const float* z, const float* correction, int* ids, float* wts, int N, int E, int top, int groups,
                         int keep, cudaStream_t st) {
    if (N == 0) return 0;
    if (E < 1 || top < 1 || top > E || groups < 1 || E % groups || keep < 1 || keep > groups || E > 8192) return -2;
    if ((long long)keep * (E / groups) < top) return -2;
    moe_select_kernel<<<N, 32, (size_t)(2 * E + 2 * groups) * sizeof(float), st>>>(z, correction, ids, wts, E, top, groups, keep);
    MB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int moe_experts_launch(const T* h, const int* ids, const T* wg, const T* wu, const T* wd, float* y, int N, int D, int F,
                              int E, int top, float limit, float alpha, cudaStream_t st) {
    if (N == 0) return 0;
    if (D < 1 || F < 1 || top < 1 || top > 65535 || (size_t)(D + F) * sizeof(float) > 96 * 1024) return -2;
    const size_t smem = (size_t)(D + F) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_experts_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    moe_experts_kernel<T><<<dim3(N, top), 256, smem, st>>>(h, ids, wg, wu, wd, y, D, F, E, top, limit, alpha);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_moe_experts_f32(const void* h, const int* ids, const void* wg, const void* wu, const void* wd, float* y, int N,
                              int D, int F, int E, int top, float limit, float alpha, cudaStream_t st) {
    return moe_experts_launch<float>((const float*)h, ids, (const float*)wg, (const float*)wu, (const float*)wd, y, N, D, F, E,
                                     top, limit, alpha, st);
}

MB_API int mb_moe_experts_bf16(const void* h, const int* ids, const void* wg, const void* wu, const void* wd, float* y, int N,
                               int D, int F, int E, int top, float limit, float alpha, cudaStream_t st) {
    return moe_experts_launch<bf16>((const bf16*)h, ids, (const bf16*)wg, (const bf16*)wu, (const bf16*)wd, y, N, D, F, E, top,
                                    limit, alpha, st);
}

template <typename T>
static int moe_combine_launch(const float* y, const float* wts, T* out, int N, int D, int top, cudaStream_t st) {
    if (N == 0) return 0;
    const long long total = (long long)N * D;
    moe_combine_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(y, wts, out, D, top, total);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_moe_combine_f32(const float* y, const float* wts, void* out, int N, int D, int top, cudaStream_t st) {
    return moe_combine_launch<float>(y, wts, (float*)out, N, D, top, st);
}

MB_API int mb_moe_combine_bf16(const float* y, const float* wts, void* out, int N, int D, int top, cudaStream_t st) {
    return moe_combine_launch<bf16>(y, wts, (bf16*)out, N, D, top, st);
}
