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
    int page_shift;                         // log2(page) when the page size is a power of two, else -1
    float scale_log2, lam, gain, eps;
    int* err;
};

constexpr int BM = 64, BN = 64, THREADS = 256, STAGES = 2;
constexpr int KROW = tile_row<DIFF_DIM>(), VROW = tile_row<DIFF_VD>();
constexpr int STAGE_ELEMS = 2 * BN * KROW + BN * VROW;          // keys of map 0, keys of map 1, values
constexpr int Q_ELEMS = 2 * BM * KROW;
constexpr size_t cmax(size_t a, size_t b) { return a > b ? a : b; }
// the stages are also where the two maps meet at the end ([64 rows][VD + 4] floats): room for the larger of the two
constexpr size_t SMEM_BYTES = Q_ELEMS * sizeof(bf16) + cmax((size_t)STAGES * STAGE_ELEMS * sizeof(bf16), (size_t)BM * (DIFF_VD + 4) * sizeof(float));
static_assert(DIFF_DIM % 16 == 0 && DIFF_VD % 16 == 0 && DIFF_DIM >= 16 && DIFF_VD >= 16, "head sizes are multiples of 16");
static_assert(DIFF_DIM <= 128 && DIFF_VD <= 128, "head sizes up to 128");

// One K/V tile of 64 keys into a stage.  Warp w fetches the eight key rows 8 w .. 8 w + 7; lane l copies 16-byte chunks l
// and l + 32 of a row's [map 0 | map 1 | values], so what a lane copies (which of the three sub-tiles, which chunk of
// its row) is the same for every row and tile.  With pages of a power of two of at least 8 positions the eight rows lie
// in one page, side by side (tiles start at multiples of 64): the table is read once per warp and tile and a row's
// address is the first row's plus a constant.  Other page sizes look every row up.
struct GatherLane {                         // what a lane copies, chunk l (j = 0) and chunk l + 32 (j = 1)
    bool on[2], is_v[2];
    int cc[2];                              // chunk within its sub-tile's row
    int sub[2];                             // element offset of the sub-tile in a stage
    int src[2];                             // element offset of the chunk in its source row
};
__device__ __forceinline__ GatherLane gather_lane(int lane) {
    constexpr int CK = DIFF_DIM / 8, CV = DIFF_VD / 8, CT = 2 * CK + CV;
    GatherLane L;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int c = lane + 32 * j;
        L.on[j] = c < CT;
        L.is_v[j] = c >= 2 * CK;
        L.cc[j] = c < CK ? c : (c < 2 * CK ? c - CK : c - 2 * CK);
        L.sub[j] = c < CK ? 0 : (c < 2 * CK ? BN * KROW : 2 * BN * KROW);
        L.src[j] = (c < 2 * CK ? c : c - 2 * CK) * 8;
    }
    return L;
}

__device__ __forceinline__ void load_kv_tile(bf16* stage, const DiffParams& P, const int* tb, int g, int kb, int lo,
                                             int hi, int tid) {
    constexpr int CT = 2 * (DIFF_DIM / 8) + DIFF_VD / 8, RW = BN / (THREADS / 32);
    const int warp = tid >> 5, lane = tid & 31;
    const GatherLane L = gather_lane(lane);
    const bool one_page = P.page_shift >= 3;
    const bf16 *k0 = P.kpool, *v0 = P.vpool;                // the warp's first row (one_page)
    bool have = false;
    if (one_page) {
        const int kp = kb + warp * RW;
        if (kp + RW > lo && kp < hi) {                      // rows outside [lo, hi) are not copied below
            const int pg = tb[kp >> P.page_shift];
            if (pg >= 0 && pg < P.num_pages) {
                const size_t r = ((size_t)pg * P.G + g) * P.page + (kp & (P.page - 1));
                k0 += r * (2 * DIFF_DIM);
                v0 += r * DIFF_VD;
                have = true;
            } else {
                mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RW; i++) {
        const int row = warp * RW + i, kp = kb + row;
        const bf16 *ksrc = k0 + i * (2 * DIFF_DIM), *vsrc = v0 + i * DIFF_VD;
        int bytes = (have && kp >= lo && kp < hi) ? 16 : 0; // below lo the pages may have been given back
        if (!one_page && kp >= lo && kp < hi) {
            const int block = kp / P.page, slot = kp - block * P.page;
            const int pg = tb[block];
            if (pg >= 0 && pg < P.num_pages) {
                const size_t r = ((size_t)pg * P.G + g) * P.page + slot;
                ksrc = P.kpool + r * (2 * DIFF_DIM);
                vsrc = P.vpool + r * DIFF_VD;
                bytes = 16;
            } else {
                mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            }
        }
        if (bytes == 0) { ksrc = P.kpool; vsrc = P.vpool; } // nothing is read, but the address must be a valid one
#pragma unroll
        for (int j = 0; j < (CT > 32 ? 2 : 1); j++) {
            if (!L.on[j]) continue;
            const int off = L.is_v[j] ? swz<DIFF_VD>(row, L.cc[j]) : swz<DIFF_DIM>(row, L.cc[j]);
            cp_async16(stage + L.sub[j] + off, (L.is_v[j] ? vsrc : ksrc) + L.src[j], bytes);
        }
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
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {       // no row of the warp moved its maximum: skip
#pragma unroll
            for (int d = 0; d < DT; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
        }
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

// ------------------------------------------------------------------------------------------------ decode form
// Sequences that bring at most 16 packed rows (one or a few tokens): a block has 16 rows, its 8 warps are (map, quarter
// of the 64 keys of a tile), so all of them work on every tile, and the keys of a sequence may be cut into `n_splits`
// blocks that run side by side.  Three stages of K/V tiles are in flight per block.  At the end the four quarters of
// each map meet in shared memory; with one split the block forms the difference, the head's norm and the output rows
// itself, with more it leaves each map's unnormalised sum, maximum and weight in global memory and the merge kernel
// below finishes the rows.  A work item is (sequence, split, n_splits, slot of the partial results).
constexpr int DBM = 16, DSTAGES = 3, MAX_SPLITS = 16;
constexpr int DQ_ELEMS = 2 * DBM * KROW;
// the stages are also where the quarters meet at the end ([8 warps][16 rows][VD] floats, maxima and weights)
constexpr size_t DSMEM_BYTES = DQ_ELEMS * sizeof(bf16) + cmax((size_t)DSTAGES * STAGE_ELEMS * sizeof(bf16),
                                                              (size_t)(8 * DBM * DIFF_VD + 2 * 8 * DBM) * sizeof(float));

struct DiffDecodeParams {
    DiffParams p;
    const int4* items;                      // (sequence, split, n_splits, slot)
    float* part_o;                          // [slot][G][MAX_SPLITS][2 maps][16 rows][VD]
    float* part_ml;                         // [slot][G][MAX_SPLITS][2 maps][16 rows][2]
};

// rows 2 warp, 2 warp + 1 of a block: the difference of the two maps (a[m][i]: this lane's columns lane + 32 i of map m,
// normalised), the head's norm, the output row
__device__ __forceinline__ void diff_finish_row(const DiffParams& P, float (&a0)[DIFF_VD / 32 + 1], float (&a1)[DIFF_VD / 32 + 1],
                                                int lane, bf16* dst) {
    constexpr int VD = DIFF_VD, NC = VD / 32 + 1;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int d = lane + 32 * i;
        const float o = d < VD ? a0[i] - P.lam * a1[i] : 0.0f;
        a0[i] = o;
        ss = fmaf(o, o, ss);
    }
    ss = mb_warp_sum(ss);
    const float f = rsqrtf(ss / (float)VD + P.eps) * P.gain;
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int d = lane + 32 * i;
        if (d < VD) dst[d] = __float2bfloat16_rn(a0[i] * f);
    }
}

__global__ void __launch_bounds__(THREADS, 2) attn_diff_mma_decode_kernel(const DiffDecodeParams DP) {
    constexpr int DIM = DIFF_DIM, VD = DIFF_VD;
    constexpr int CK = DIM / 8, KS = DIM / 16, DT = VD / 8, NT = 2, NC = VD / 32 + 1;
    const DiffParams& P = DP.p;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + DQ_ELEMS;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tig = lane & 3;
    const int map = warp >> 2, nbase = (warp & 3) * 16;
    const int4 item = DP.items[blockIdx.x];
    const int seq = item.x, split = item.y, n_splits = item.z, slot = item.w, g = blockIdx.y;
    const int G = P.group, R = min(DBM, P.q_len[seq] * G), pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int pos_max = pos0 + (R - 1) / G;
    const int hi = pos_max + 1;
    const int lo = P.chunk > 0 ? pos0 / P.chunk * P.chunk : 0;
    const int lo_al = (lo / BN) * BN;
    const int n_tiles = (hi - lo_al + BN - 1) / BN;
    const int tps = (n_tiles + n_splits - 1) / n_splits;
    const int t_begin = split * tps, t_end = min(n_tiles, t_begin + tps);
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    for (int cid = tid; cid < DBM * 2 * CK; cid += THREADS) {
        const int row = cid / (2 * CK), c = cid % (2 * CK);
        const bf16* src = P.q;
        int bytes = 0;
        if (row < R) {
            src = P.q + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * (2 * DIM) + c * 8;
            bytes = 16;
        }
        cp_async16(qs + (c < CK ? swz<DIM>(row, c) : DBM * KROW + swz<DIM>(row, c - CK)), src, bytes);
    }
    cp_async_commit();
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; s++) {
        if (t_begin + s < t_end) load_kv_tile(kvs + (size_t)s * STAGE_ELEMS, P, tb, g, lo_al + (t_begin + s) * BN, lo, hi, tid);
        cp_async_commit();
    }
    int rpos[2], rlo[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = gq + i * 8;
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

    cp_async_wait<DSTAGES - 1>();
    __syncthreads();
    const bf16* qm = qs + map * DBM * KROW;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldmatrix_x4(qf[ks], qm + swz<DIM>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    for (int t = t_begin; t < t_end; t++) {
        cp_async_wait<DSTAGES - 2>();
        __syncthreads();
        {
            const int tn = t + DSTAGES - 1;
            if (tn < t_end) load_kv_tile(kvs + (size_t)((tn - t_begin) % DSTAGES) * STAGE_ELEMS, P, tb, g, lo_al + tn * BN, lo, hi, tid);
            cp_async_commit();
        }
        const bf16* kt = kvs + (size_t)((t - t_begin) % DSTAGES) * STAGE_ELEMS + map * BN * KROW;
        const bf16* vt = kvs + (size_t)((t - t_begin) % DSTAGES) * STAGE_ELEMS + 2 * BN * KROW;
        const int kb = lo_al + t * BN;
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
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = kb + nbase + j * 8 + 2 * tig + (e & 1);
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
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {       // no row of the warp moved its maximum: skip
#pragma unroll
            for (int d = 0; d < DT; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
        }
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < VD / 16; dp++) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vt + swz<VD>(nbase + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
            mma_bf16(o[2 * dp], a, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    __syncthreads();                                        // every warp is done with the K/V stages
    float* mo = reinterpret_cast<float*>(kvs);              // [8 warps][16 rows][VD]
    float* sm_m = mo + 8 * DBM * VD;                        // [8][16]
    float* sm_l = sm_m + 8 * DBM;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int row = gq + i * 8;
        float* dst = mo + (size_t)(warp * DBM + row) * VD + 2 * tig;
#pragma unroll
        for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
        if (tig == 0) { sm_m[warp * DBM + row] = m_run[i]; sm_l[warp * DBM + row] = l_run[i]; }
    }
    __syncthreads();
    // warp w finishes rows 2 w and 2 w + 1: the four quarters of each map in the order of the quarters
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const int row = 2 * warp + rr;
        if (row >= R) continue;
        float acc[2][NC], M[2], L[2];
#pragma unroll
        for (int m = 0; m < 2; m++) {
            M[m] = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) M[m] = fmaxf(M[m], sm_m[(m * 4 + w) * DBM + row]);
            L[m] = 0.0f;
#pragma unroll
            for (int i = 0; i < NC; i++) acc[m][i] = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float mw = sm_m[(m * 4 + w) * DBM + row];
                const float f = mw == -INFINITY ? 0.0f : exp2f(mw - M[m]);
                L[m] = fmaf(sm_l[(m * 4 + w) * DBM + row], f, L[m]);
#pragma unroll
                for (int i = 0; i < NC; i++) {
                    const int d = lane + 32 * i;
                    if (d < VD) acc[m][i] = fmaf(mo[(size_t)((m * 4 + w) * DBM + row) * VD + d], f, acc[m][i]);
                }
            }
        }
        if (n_splits == 1) {
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const float inv = L[m] > 0.0f ? 1.0f / L[m] : 0.0f;
#pragma unroll
                for (int i = 0; i < NC; i++) acc[m][i] *= inv;
            }
            diff_finish_row(P, acc[0], acc[1], lane, P.out + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * VD);
        } else {
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const size_t base = ((((size_t)slot * P.G + g) * MAX_SPLITS + split) * 2 + m) * DBM + row;
#pragma unroll
                for (int i = 0; i < NC; i++) {
                    const int d = lane + 32 * i;
                    if (d < VD) DP.part_o[base * VD + d] = acc[m][i];
                }
                if (lane == 0) { DP.part_ml[base * 2] = M[m]; DP.part_ml[base * 2 + 1] = L[m]; }
            }
        }
    }
}

// one block per (slot, kv head): the splits of every row meet, in the order of the splits
__global__ void __launch_bounds__(THREADS) attn_diff_merge_kernel(const DiffParams P, const int2* slots, const float* part_o,
                                                                  const float* part_ml) {
    constexpr int VD = DIFF_VD, NC = VD / 32 + 1;
    const int slot = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = slots[slot].x, n_splits = slots[slot].y;
    const int G = P.group, R = min(DBM, P.q_len[seq] * G), tok0 = P.q_start[seq];
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const int row = 2 * warp + rr;
        if (row >= R) continue;
        float acc[2][NC];
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const size_t base0 = (((size_t)slot * P.G + g) * MAX_SPLITS * 2 + m) * DBM + row;     // + split * 2 * DBM
            // every split's maximum and weight first (loads that do not wait for one another), then the sums, four
            // splits' loads in flight at a time, added in the order of the splits
            float ms[MAX_SPLITS], ls[MAX_SPLITS];
            float M = -INFINITY, L = 0.0f;
#pragma unroll
            for (int s = 0; s < MAX_SPLITS; s++) {
                const float2 v = s < n_splits ? *reinterpret_cast<const float2*>(part_ml + (base0 + (size_t)s * 2 * DBM) * 2)
                                              : make_float2(-INFINITY, 0.0f);
                ms[s] = v.x; ls[s] = v.y;
                M = fmaxf(M, v.x);
            }
#pragma unroll
            for (int i = 0; i < NC; i++) acc[m][i] = 0.0f;
#pragma unroll
            for (int s0 = 0; s0 < MAX_SPLITS; s0 += 4) {
                if (s0 >= n_splits) break;
                float v[4][NC];
#pragma unroll
                for (int j = 0; j < 4; j++)
#pragma unroll
                    for (int i = 0; i < NC; i++) {
                        const int d = lane + 32 * i;
                        v[j][i] = (s0 + j < n_splits && d < VD) ? part_o[(base0 + (size_t)(s0 + j) * 2 * DBM) * VD + d] : 0.0f;
                    }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float f = ms[s0 + j] == -INFINITY ? 0.0f : exp2f(ms[s0 + j] - M);
                    L = fmaf(ls[s0 + j], f, L);
#pragma unroll
                    for (int i = 0; i < NC; i++) acc[m][i] = fmaf(v[j][i], f, acc[m][i]);
                }
            }
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
            for (int i = 0; i < NC; i++) acc[m][i] *= inv;
        }
        diff_finish_row(P, acc[0], acc[1], lane, P.out + ((size_t)(tok0 + row / G) * P.H + (g * G + row % G)) * VD);
    }
}

MB_API int mb_attn_diff_mma_dims(int* dim, int* vd, int* rows) {
    *dim = DIFF_DIM; *vd = DIFF_VD; *rows = BM;
    return 0;
}

static void fill_params(DiffParams& P, const void* q, void* out, const void* kpool, const void* vpool, const int* q_start,
                        const int* q_len, const int* pos0, const int* seq_row, const int* table, int max_blocks, int H,
                        int G, int page, int num_pages, int chunk, float scale, float lam, float gain, float eps, int* err) {
    P.q = (const bf16*)q; P.out = (bf16*)out; P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = nullptr; P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.H = H; P.G = G; P.group = H / G; P.page = page; P.num_pages = num_pages; P.chunk = chunk;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale_log2 = scale * 1.4426950408889634f; P.lam = lam; P.gain = gain; P.eps = eps; P.err = err;
}

// the decode form: n_items (sequence, split, n_splits, slot) items; n_slots (sequence, n_splits) entries for the merge
// kernel (0: no sequence is cut); part_o, part_ml: n_slots * G * 16 splits * 2 maps * 16 rows * (VD | 2) floats
MB_API int mb_attn_diff_mma_decode(const void* q, void* out, const void* kpool, const void* vpool, const int* items,
                                   int n_items, const int* slots, int n_slots, float* part_o, float* part_ml,
                                   const int* q_start, const int* q_len, const int* pos0, const int* seq_row,
                                   const int* table, int max_blocks, int H, int G, int page, int num_pages, int chunk,
                                   float scale, float lam, float gain, float eps, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (G < 1 || H % G || page < 1 || chunk < 0 || (n_slots > 0 && (!part_o || !part_ml || !slots))) return -2;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpool | (uintptr_t)vpool) & 15) != 0) return -2;
    static bool ready = false;
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(attn_diff_mma_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DSMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        // the largest shared-memory carve-out, so that two blocks share an SM where their stages fit
        cudaFuncSetAttribute(attn_diff_mma_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ready = true;
    }
    DiffDecodeParams DP;
    fill_params(DP.p, q, out, kpool, vpool, q_start, q_len, pos0, seq_row, table, max_blocks, H, G, page, num_pages, chunk,
                scale, lam, gain, eps, err);
    DP.items = (const int4*)items; DP.part_o = part_o; DP.part_ml = part_ml;
    attn_diff_mma_decode_kernel<<<dim3(n_items, G), THREADS, DSMEM_BYTES, st>>>(DP);
    MB_LAUNCH_CHECK();
    if (n_slots > 0) {
        attn_diff_merge_kernel<<<dim3(n_slots, G), THREADS, 0, st>>>(DP.p, (const int2*)slots, part_o, part_ml);
        MB_LAUNCH_CHECK();
    }
    return 0;
}

MB_API int mb_attn_diff_mma_max_splits() { return MAX_SPLITS; }

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
        cudaFuncSetAttribute(attn_diff_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ready = true;
    }
    DiffParams P;
    fill_params(P, q, out, kpool, vpool, q_start, q_len, pos0, seq_row, table, max_blocks, H, G, page, num_pages, chunk, scale,
                lam, gain, eps, err);
    P.items = (const int2*)items;
    attn_diff_mma_kernel<<<dim3(n_items, G), THREADS, SMEM_BYTES, st>>>(P);
    MB_LAUNCH_CHECK();
    return 0;
}
