// Differential attention over the paged cache on tensor cores (bf16): prompt portions and decode tokens in one launch.
//
// A head has two attention maps (queries and keys of their own, DIFF_DIM each, side by side in a row) over one set of
// values (DIFF_VD):  a_m = softmax(scale q_m K_m^T) V,  out = rmsnorm_head(a_0 - lam a_1) * gain.  A query sees the keys
// of its own block of `chunk` positions (blocks counted from position 0 of the sequence; 0: no blocks) up to itself.
//
// The query rows of one sequence and one kv head are packed as (token, head-in-group), 64 rows per block: all query
// heads that read a kv head share every K/V tile that is loaded.  A work item is (sequence, tile of rows); the grid is
// (items, kv heads).  The block has 8 warps: warps 0-3 run map 0 and warps 4-7 map 1 of the same 64 rows, 16 rows per
// warp, so each warp is an ordinary flash attention with float accumulators (mma.sync.m16n8k16, online softmax with
// exp2) and both maps read ONE copy of the value tile.  K and V tiles of 64 keys are gathered through the block table
// with cp.async into XOR-swizzled shared memory, two stages.  At the end the warps of map 1 leave their normalised
// result in shared memory and the warps of map 0 form the difference, the head's norm and the output row.
//
// One library per pair of head sizes: compiled with -DDIFF_DIM=<dim of a map> -DDIFF_VD=<value dim>, multiples of 16.
#include "attention_common.cuh"

#ifndef DIFF_DIM
#define DIFF_DIM 64
#endif
#ifndef DIFF_VD
#define DIFF_VD 128
#endif

struct DiffParams {
    const bf16* q; bf16* out;               // q[(n * H + h) * 2 DIM + map * DIM + d], out[(n * H + h) * VD + d]
    const bf16* kpool; const bf16* vpool;   // [page][G][slot][2 DIM], [page][G][slot][VD]
    const int2* items;                      // (sequence, row tile)
    const int* q_start; const int* q_len; const int* pos0; const int* seq_row;
    const int* table; int max_blocks;
    int H, G, group, page, num_pages, chunk;
    float scale_log2, lam, gain, eps;
    int* err;
};

constexpr int BM = 64, BN = 64, THREADS = 256, STAGES = 2;
constexpr int KROW = tile_row<DIFF_DIM>(), VROW = tile_row<DIFF_VD>();
constexpr int STAGE_ELEMS = 2 * BN * KROW + BN * VROW;          // keys of map 0, keys of map 1, values
constexpr int Q_ELEMS = 2 * BM * KROW;
constexpr size_t SMEM_BYTES = (size_t)(Q_ELEMS + STAGES * STAGE_ELEMS) * sizeof(bf16);
static_assert(DIFF_DIM % 16 == 0 && DIFF_VD % 16 == 0 && DIFF_DIM >= 16 && DIFF_VD >= 16, "head sizes are multiples of 16");
static_assert(DIFF_DIM <= 128 && DIFF_VD <= 128, "head sizes up to 128");
static_assert((size_t)BM * (DIFF_VD + 4) * sizeof(float) <= (size_t)STAGES * STAGE_ELEMS * sizeof(bf16), "the meeting place fits");

__device__ __forceinline__ void load_kv_tile(bf16* stage, const DiffParams& P, const int* tb, int g, int kb, int lo,
                                             int hi, int tid) {
    constexpr int CK = DIFF_DIM / 8, CV = DIFF_VD / 8, CT = 2 * CK + CV;
    for (int cid = tid; cid < BN * CT; cid += THREADS) {
        const int row = cid / CT, c = cid % CT;
        const int kp = kb + row;
        const bf16* src = P.kpool;
        int bytes = 0;
        if (kp >= lo && kp < hi) {                          // below lo the pages may have been given back
            const int block = kp / P.page, slot = kp - block * P.page;
            const int pg = tb[block];
            if (pg >= 0 && pg < P.num_pages) {
                const size_t r = ((size_t)pg * P.G + g) * P.page + slot;
                src = c < 2 * CK ? P.kpool + r * (2 * DIFF_DIM) + c * 8 : P.vpool + r * DIFF_VD + (c - 2 * CK) * 8;
                bytes = 16;
            } else {
                mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            }
        }
        bf16* dst;
        if (c < CK) dst = stage + swz<DIFF_DIM>(row, c);
        else if (c < 2 * CK) dst = stage + BN * KROW + swz<DIFF_DIM>(row, c - CK);
        else dst = stage + 2 * BN * KROW + swz<DIFF_VD>(row, c - 2 * CK);
        cp_async16(dst, src, bytes);
    }
}

__global__ void __launch_bounds__(THREADS) attn_diff_mma_kernel(const DiffParams P) {
    constexpr int DIM = DIFF_DIM, VD = DIFF_VD;
    constexpr int CK = DIM / 8, KS = DIM / 16, DT = VD / 8, NT = 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + Q_ELEMS;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tig = lane & 3;
    const int map = warp >> 2, m0 = (warp & 3) * 16;
    const int2 item = P.items[blockIdx.x];
    const int seq = item.x, m_tile = item.y, g = blockIdx.y;
    const int G = P.group, R = P.q_len[seq] * G, pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int row0 = m_tile * BM;
    if (row0 >= R) return;
    const int row_last = min(R, row0 + BM) - 1;
    const int pos_min = pos0 + row0 / G, pos_max = pos0 + row_last / G;
    const int hi = pos_max + 1;
    const int lo = P.chunk > 0 ? pos_min / P.chunk * P.chunk : 0;
    const int lo_al = (lo / BN) * BN;
    const int n_tiles = (hi - lo_al + BN - 1) / BN;
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    for (int cid = tid; cid < BM * 2 * CK; cid += THREADS) {
        const int row = cid / (2 * CK), c = cid % (2 * CK), r = row0 + row;
        const bf16* src = P.q;
        int bytes = 0;
        if (r < R) {
            src = P.q + ((size_t)(tok0 + r / G) * P.H + (g * G + r % G)) * (2 * DIM) + c * 8;
            bytes = 16;
        }
        cp_async16(qs + (c < CK ? swz<DIM>(row, c) : BM * KROW + swz<DIM>(row, c - CK)), src, bytes);
    }
    cp_async_commit();
    load_kv_tile(kvs, P, tb, g, lo_al, lo, hi, tid);
    cp_async_commit();

    int rpos[2], rlo[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + m0 + gq + i * 8;
        if (r < R) {
            rpos[i] = pos0 + r / G;
            rlo[i] = P.chunk > 0 ? rpos[i] / P.chunk * P.chunk : 0;
        } else {
            rpos[i] = -1; rlo[i] = 0;
        }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }

    cp_async_wait<1>();
    __syncthreads();
    const bf16* qm = qs + map * BM * KROW;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldmatrix_x4(qf[ks], qm + swz<DIM>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    for (int t = 0; t < n_tiles; t++) {
        cp_async_wait<0>();
        __syncthreads();                                    // tile t has landed; every warp is done with tile t - 1
        if (t + 1 < n_tiles) load_kv_tile(kvs + (size_t)((t + 1) % STAGES) * STAGE_ELEMS, P, tb, g, lo_al + (t + 1) * BN, lo, hi, tid);
        cp_async_commit();
        const bf16* kt = kvs + (size_t)(t % STAGES) * STAGE_ELEMS + map * BN * KROW;
        const bf16* vt = kvs + (size_t)(t % STAGES) * STAGE_ELEMS + 2 * BN * KROW;
        const int kb = lo_al + t * BN;

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
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = kb + j * 8 + 2 * tig + (e & 1);
                const bool ok = key <= rpos[i] && key >= rlo[i];
                const float v = ok ? s[j][e] * P.scale_log2 : -INFINITY;
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
            for (int dp = 0; dp < VD / 16; dp++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + swz<VD>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
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
    // the two maps meet: map 1 leaves a_1 in shared memory, map 0 forms a_0 - lam a_1, the head's norm and the row
    __syncthreads();                                        // every warp is done with the K/V stages
    float* meet = reinterpret_cast<float*>(kvs);            // [64 rows][VD + 4]
    constexpr int MROW = VD + 4;
    if (map == 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
            float* dst = meet + (size_t)(m0 + gq + i * 8) * MROW + 2 * tig;
#pragma unroll
            for (int d = 0; d < DT; d++)
                *reinterpret_cast<float2*>(dst + d * 8) = make_float2(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
        }
    }
    __syncthreads();
    if (map == 0) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = row0 + m0 + gq + i * 8;
            const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
            const float* src = meet + (size_t)(m0 + gq + i * 8) * MROW + 2 * tig;
            float ss = 0.0f;
#pragma unroll
            for (int d = 0; d < DT; d++) {
                const float2 b = *reinterpret_cast<const float2*>(src + d * 8);
                const float x = o[d][2 * i] * inv - P.lam * b.x, y = o[d][2 * i + 1] * inv - P.lam * b.y;
                o[d][2 * i] = x; o[d][2 * i + 1] = y;
                ss = fmaf(x, x, fmaf(y, y, ss));
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (r >= R) continue;
            const float f = rsqrtf(ss / (float)VD + P.eps) * P.gain;
            bf16* dst = P.out + ((size_t)(tok0 + r / G) * P.H + (g * G + r % G)) * VD + 2 * tig;
#pragma unroll
            for (int d = 0; d < DT; d++)
                *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2 * i] * f, o[d][2 * i + 1] * f);
        }
    }
}

MB_API int mb_attn_diff_mma_dims(int* dim, int* vd, int* rows) {
    *dim = DIFF_DIM; *vd = DIFF_VD; *rows = BM;
    return 0;
}

MB_API int mb_attn_diff_mma(const void* q, void* out, const void* kpool, const void* vpool, const int* items, int n_items,
                            const int* q_start, const int* q_len, const int* pos0, const int* seq_row, const int* table,
                            int max_blocks, int H, int G, int page, int num_pages, int chunk, float scale, float lam,
                            float gain, float eps, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (G < 1 || H % G || page < 1 || chunk < 0) return -2;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpool | (uintptr_t)vpool) & 15) != 0) return -2;
    static bool ready = false;
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(attn_diff_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        ready = true;
    }
    DiffParams P;
    P.q = (const bf16*)q; P.out = (bf16*)out; P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = (const int2*)items; P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.H = H; P.G = G; P.group = H / G; P.page = page; P.num_pages = num_pages; P.chunk = chunk;
    P.scale_log2 = scale * 1.4426950408889634f; P.lam = lam; P.gain = gain; P.eps = eps; P.err = err;
    attn_diff_mma_kernel<<<dim3(n_items, G), THREADS, SMEM_BYTES, st>>>(P);
    MB_LAUNCH_CHECK();
    return 0;
}
