// Paged attention on the tensor cores with TMA-fed K/V tiles, for steps that carry many rows: decode
// with eight or more sequences, and chunked prompt ingestion (several tokens of a sequence share the
// K/V tiles they attend to). Replaces, together with qkv_post_kernel, what the reference runs as
// rms_norm / rope_state / rms_norm_unit / cache_write_f32_state / gqa_decode_block_state for one row
// (crates/oxide-torch-models/src/gemma4_cuda/decode.rs:99-157; kernel_module.rs:1790-1894) and as
// cache_write_f32 / gqa_prefill_block for the rows of a prompt (decode.rs:176-325;
// kernel_module.rs:1896-1974). Attention scale is 1.0 as in the reference.
//
// Work. A *group* is up to 8 / G consecutive tokens of one sequence (G query heads per KV head); a
// *unit* is (group, kv head); its K/V positions [first visible, last token's position] are cut into
// tiles of 16 positions (aligned to 16 in position space; ring capacities and pages are multiples of
// 16, so a tile is 16 contiguous rows of one (page, kv head) slab). All tiles of all units form one
// sequence that is dealt to the consumer warps of the grid as equal contiguous ranges (whatever the
// raggedness of the batch, every warp streams the same number of bytes); a warp writes one
// un-normalised partial (m, l, sum p*v) per unit it touches, and attn_merge_kernel adds the partials of
// a unit in warp order, so results do not depend on scheduling.
//
// Data path. One producer warp per CTA: lane w feeds consumer warp w through its own ring of
// mbarrier-guarded stages; a stage is the K tile and the V tile, each loaded by cp.async.bulk.tensor.2d
// boxes of 64 elements x 16 rows with the 128-byte swizzle (bank-conflict-free ldmatrix). Tensor maps
// cover this GPU's own KV pool only; no multicast.
//
// Arithmetic. mma.sync.m16n8k16 BF16 with f32 accumulation. The 16 MMA rows hold the group's (token,
// head) rows twice: rows 0..7 the BF16 high part of q, rows 8..15 the BF16 low part (q = hi + lo to
// 2^-17), so that q . k is formed from the full f32 query at no extra MMA; the softmax weights p are
// split the same way for p . v. K and V are BF16 in the cache, so their products are exact in f32.
//
// HBM-bound: bytes per launch = 2 * visible positions * kv_heads * head_dim * 2 per sequence.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_gemm.cuh"

namespace oxg4 {

constexpr int kAmTile = 16;              // positions per tile
constexpr int kAmMaxGroups = 512;        // groups per launch
constexpr int kAmRows = 8;               // (token, head) rows per group: 8 hi + 8 lo = the 16 MMA rows

template <int D> struct AmGeom;
template <> struct AmGeom<256> { static constexpr int NCW = 3, NST = 4; };   // 3 x 4 x 16 KiB
template <> struct AmGeom<128> { static constexpr int NCW = 4, NST = 6; };   // 4 x 6 x 8 KiB
template <> struct AmGeom<64> { static constexpr int NCW = 4, NST = 8; };    // 4 x 8 x 4 KiB

struct AttnMmaArgs {
    const uint16_t* q_hl;        // [R][Nq][2][D] BF16: high part, then low part, of the normed and rotated query
    int Nq, Nkv, NG;
    const int32_t* grp_row0;     // [NG] first row of the group
    const int32_t* grp_n;        // [NG] tokens in the group (consecutive rows, consecutive positions); 0 = empty
    const int32_t* row_pos;      // [R] absolute position of the row's token
    const int32_t* row_seq;      // [R] sequence (page table / ring) of the row, or null: row r is sequence r
    const uint32_t* row_tok;     // [R] token ids or null; rows holding kInactiveToken sit the step out
    const int32_t* page_table;   // [B, pages_per_seq]
    int pages_per_seq, page_tokens;
    const int32_t* cap;          // [B] ring capacity of this layer kind
    int window;                  // a token sees the last `window` positions up to its own
    int part_rows;               // rows per partial slot (tokens per group * G <= 8)
    float* part;                 // [NG * Nkv + total consumer warps][part_rows][D + 2]
    int* err;                    // device flag, raised when a bounded wait ran out
    int* pre_out;                // [NG + 1] tile prefix of the groups, written by the attention kernel for the merge
    // merge only
    int total_warps;
    float* out;                  // [R, Nq * D]
    uint16_t* out_bf16;          // optional BF16 copy (input of the tcgen05 O projection)
};

// tiles of a group: positions [max(0, first + 1 - window), last] in tiles of 16
DEVINL int am_group_tiles(const AttnMmaArgs& a, int g, int& t0) {
    const int n = a.grp_n[g];
    t0 = 0;
    if (n <= 0) return 0;
    const int row0 = a.grp_row0[g];
    if (a.row_tok != nullptr && a.row_tok[row0] == kInactiveToken) return 0;
    const int first = a.row_pos[row0];
    const int lo = max(0, first + 1 - a.window);
    t0 = lo / kAmTile;
    return (first + n - 1) / kAmTile - t0 + 1;
}

// prefix[g] = tiles of the groups before g (per kv head); every thread of the CTA calls it
DEVINL void am_prefix(const AttnMmaArgs& a, int* pre) {
    for (int g = threadIdx.x; g < a.NG; g += blockDim.x) {
        int t0;
        pre[g + 1] = am_group_tiles(a, g, t0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        pre[0] = 0;
        for (int g = 0; g < a.NG; ++g) pre[g + 1] += pre[g];
    }
    __syncthreads();
}

// global tile t -> (group, kv head, tile inside the unit, tiles of the unit)
DEVINL void am_locate(const int* pre, int NG, int Nkv, int t, int& g, int& kvh, int& lt, int& nt) {
    int lo = 0, hi = NG;                       // largest g with pre[g] * Nkv <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)pre[mid] * Nkv <= t) lo = mid; else hi = mid;
    }
    g = lo;
    nt = pre[g + 1] - pre[g];
    const int off = t - pre[g] * Nkv;
    kvh = off / nt;
    lt = off - kvh * nt;
}

// contiguous range of the T tiles owned by warp w of W
DEVINL void am_range(int T, int W, int w, int& begin, int& len) {
    const int q = T / W, rem = T % W;
    begin = w * q + min(w, rem);
    len = q + (w < rem ? 1 : 0);
}
DEVINL int am_warp_of(int T, int W, int t) {
    const int q = T / W, rem = T % W;
    const int bnd = rem * (q + 1);
    return t < bnd ? t / (q + 1) : rem + (t - bnd) / q;
}

DEVINL void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
DEVINL void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
DEVINL void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (hi, lo) BF16 split of two f32 values, packed for an MMA operand (first value in the low half)
DEVINL void split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
    const uint32_t xh = f32_to_bf16_bits(x), yh = f32_to_bf16_bits(y);
    const float xr = x - __uint_as_float(xh << 16), yr = y - __uint_as_float(yh << 16);
    hi = xh | (yh << 16);
    lo = f32_to_bf16_bits(xr) | (f32_to_bf16_bits(yr) << 16);
}
DEVINL void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int D, int G>
__global__ void __launch_bounds__((AmGeom<D>::NCW + 1) * 32, 1)
attn_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                const AttnMmaArgs a) {
    constexpr int NCW = AmGeom<D>::NCW, NST = AmGeom<D>::NST;
    constexpr int BOXES = D / 64;                              // 64-element (128-byte) boxes per row
    constexpr uint32_t BOX_BYTES = kAmTile * 128;              // 2 KiB
    constexpr uint32_t KV_BYTES = BOXES * BOX_BYTES;           // one K (or V) tile
    constexpr uint32_t STAGE = 2 * KV_BYTES;
    constexpr int QS = D + 8;                                  // padded row of the query tile (elements)
    extern __shared__ unsigned char am_dyn[];
    unsigned char* stages = (unsigned char*)(((uintptr_t)am_dyn + 1023) & ~(uintptr_t)1023);
    uint16_t* qtiles = (uint16_t*)(stages + (size_t)NCW * NST * STAGE);          // [NCW][16][QS]
    __shared__ __align__(8) uint64_t full[NCW][NST], empty[NCW][NST];
    __shared__ int pre[kAmMaxGroups + 1];
    __shared__ int issued[NCW];
    __shared__ volatile int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int w = 0; w < NCW; ++w)
            for (int s = 0; s < NST; ++s) { mbar_init(&full[w][s], 1); mbar_init(&empty[w][s], 1); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < NCW) issued[tid] = 0;
    pdl_wait();
    pdl_launch();
    am_prefix(a, pre);                                         // contains the CTA-wide barriers
    const int T = pre[a.NG] * a.Nkv;
    const int W = (int)gridDim.x * NCW;
    if (blockIdx.x == 0)                                       // the merge kernel reads the prefix instead of redoing it
        for (int g = tid; g <= a.NG; g += (int)blockDim.x) a.pre_out[g] = pre[g];

    if (warp == NCW) {
        // ---- producer: lane w streams the tiles of consumer warp w ----
        if (lane < NCW) {
            int begin, len;
            am_range(T, W, (int)blockIdx.x * NCW + lane, begin, len);
            int t = begin, it = 0;
            const int end = begin + len;
            while (t < end && !failed) {
                int g, kvh, lt, nt;
                am_locate(pre, a.NG, a.Nkv, t, g, kvh, lt, nt);
                const int seg_end = min(end, t + (nt - lt));
                int t0;
                am_group_tiles(a, g, t0);
                const int row0 = a.grp_row0[g];
                const int seq = a.row_seq ? a.row_seq[row0] : row0;
                const int cap = a.cap[seq];
                const int32_t* pt = a.page_table + (size_t)seq * a.pages_per_seq;
                for (; t < seg_end; ++t, ++lt, ++it) {
                    const int s = it % NST;
                    if (it >= NST && !mbar_wait(&empty[lane][s], ((it / NST) & 1) ^ 1)) {
                        failed = 1;
                        atomicExch(a.err, 11);
                        break;
                    }
                    const int slot = ((t0 + lt) * kAmTile) % cap;
                    const int rowc = (pt[slot / a.page_tokens] * a.Nkv + kvh) * a.page_tokens + slot % a.page_tokens;
                    unsigned char* sk = stages + ((size_t)lane * NST + s) * STAGE;
                    mbar_expect_tx(&full[lane][s], STAGE);
#pragma unroll
                    for (int b = 0; b < BOXES; ++b) {
                        tma_load_2d(sk + b * BOX_BYTES, &map_k, b * 64, rowc, &full[lane][s]);
                        tma_load_2d(sk + KV_BYTES + b * BOX_BYTES, &map_v, b * 64, rowc, &full[lane][s]);
                    }
                }
                if (failed) break;
            }
            issued[lane] = it;
        }
    } else {
        // ---- consumer warp ----
        const int gw = (int)blockIdx.x * NCW + warp;
        int begin, len;
        am_range(T, W, gw, begin, len);
        uint16_t* qs = qtiles + (size_t)warp * 16 * QS;
        const uint32_t qs_addr = smem_u32(qs);
        const int mrow = lane >> 2;                             // MMA row of this lane's accumulators (0..7)
        const int mcol = (lane & 3) * 2;                        // first of its two columns inside an 8-wide tile
        // per-lane byte offsets of the ldmatrix row addresses
        const int lm_i = lane >> 3, lm_r = lane & 7;
        const uint32_t q_off = (uint32_t)((((lm_i & 1) * 8 + lm_r) * QS + (lm_i >> 1) * 8) * 2);
        int t = begin, it = 0;
        const int end = begin + len;
        while (t < end && !failed) {
            int g, kvh, lt, nt;
            am_locate(pre, a.NG, a.Nkv, t, g, kvh, lt, nt);
            const int seg_end = min(end, t + (nt - lt));
            int t0;
            am_group_tiles(a, g, t0);
            const int row0 = a.grp_row0[g], ntok = a.grp_n[g];
            const int first = a.row_pos[row0];
            const int nrows = ntok * G;
            // query tile: rows r < nrows hold the high parts, rows 8 + r the low parts, everything else zero
            __syncwarp();
            for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
                const int row = idx / (D / 8), ch = idx % (D / 8);
                const int r = row & 7;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (r < nrows) {
                    const int tok_i = r / G, h = r % G;
                    const uint16_t* src = a.q_hl + (((size_t)(row0 + tok_i) * a.Nq + kvh * G + h) * 2 + (row >> 3)) * D;
                    v = *reinterpret_cast<const uint4*>(src + ch * 8);
                }
                *reinterpret_cast<uint4*>(qs + (size_t)row * QS + ch * 8) = v;
            }
            __syncwarp();
            // this lane's logical row (token, head): its position and window
            const int my_tok = mrow / G;
            const bool row_ok = mrow < nrows;
            const int my_pos = first + my_tok;
            const int my_lo = max(0, my_pos + 1 - a.window);
            float m_run = -INFINITY, l_run = 0.0f;
            float o[D / 8][4];
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] = 0.0f; o[i][1] = 0.0f; o[i][2] = 0.0f; o[i][3] = 0.0f; }

            for (; t < seg_end; ++t, ++lt, ++it) {
                const int s = it % NST;
                if (!mbar_wait(&full[warp][s], (it / NST) & 1)) {
                    failed = 1;
                    if (lane == 0) atomicExch(a.err, 12);
                    break;
                }
                const uint32_t kb = smem_u32(stages + ((size_t)warp * NST + s) * STAGE);
                const uint32_t vb = kb + KV_BYTES;
                // ---- S = Q K^T for the 16 positions of the tile: two 8-wide column tiles ----
                float sc[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n) { sc[n][0] = 0.0f; sc[n][1] = 0.0f; sc[n][2] = 0.0f; sc[n][3] = 0.0f; }
#pragma unroll
                for (int kp = 0; kp < D / 32; ++kp) {              // pairs of 16-wide k-steps
                    uint32_t qa[4], qb[4];
                    ldmatrix_x4(qa, qs_addr + q_off + (uint32_t)(kp * 32) * 2);
                    ldmatrix_x4(qb, qs_addr + q_off + (uint32_t)(kp * 32 + 16) * 2);
#pragma unroll
                    for (int n = 0; n < 2; ++n) {
                        // matrices: (k-step a, dims 0..7), (a, 8..15), (b, 0..7), (b, 8..15) of positions n*8..n*8+7
                        const int c8 = kp * 4 + lm_i;              // 16-byte chunk (8 dims) inside the row
                        const int prow = n * 8 + lm_r;
                        uint32_t kf[4];
                        ldmatrix_x4(kf, kb + (uint32_t)((c8 >> 3) * BOX_BYTES + prow * 128 + (((c8 & 7) ^ (prow & 7)) << 4)));
                        mma_bf16_16816(sc[n], qa, kf[0], kf[1]);
                        mma_bf16_16816(sc[n], qb, kf[2], kf[3]);
                    }
                }
                // ---- online softmax over this lane's four scores (row mrow; hi row + lo row) ----
                const int pbase = (t0 + lt) * kAmTile;
                float sv[4];
                float tmax = -INFINITY;
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int p = pbase + n * 8 + mcol + j;
                        const float x = sc[n][j] + sc[n][j + 2];
                        const bool ok = row_ok && p <= my_pos && p >= my_lo;
                        sv[n * 2 + j] = ok ? x : -INFINITY;
                        tmax = fmaxf(tmax, sv[n * 2 + j]);
                    }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run, tmax);
                float pv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                float corr = 1.0f;
                if (m_new > -INFINITY) {
                    corr = expf(m_run - m_new);                    // exp(-inf) = 0 on the first tile with a visible position
#pragma unroll
                    for (int i = 0; i < 4; ++i) pv[i] = expf(sv[i] - m_new);
                }
                l_run = l_run * corr + ((pv[0] + pv[1]) + (pv[2] + pv[3]));
                if (__any_sync(0xffffffffu, m_new > m_run)) {
#pragma unroll
                    for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr; o[i][1] *= corr; o[i][2] *= corr; o[i][3] *= corr; }
                }
                m_run = m_new;
                // ---- O += P V : P split into high rows (0..7) and low rows (8..15) ----
                uint32_t pa[4];
                split_pack(pv[0], pv[1], pa[0], pa[1]);
                split_pack(pv[2], pv[3], pa[2], pa[3]);
#pragma unroll
                for (int np = 0; np < D / 16; ++np) {
                    // matrices: (positions 0..7, dims np*16 + 0..7), (8..15, same dims), (0..7, dims + 8), (8..15, dims + 8)
                    const int c8 = np * 2 + (lm_i >> 1);
                    const int prow = (lm_i & 1) * 8 + lm_r;
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vb + (uint32_t)((c8 >> 3) * BOX_BYTES + prow * 128 + (((c8 & 7) ^ (prow & 7)) << 4)));
                    mma_bf16_16816(o[2 * np], pa, vf[0], vf[1]);
                    mma_bf16_16816(o[2 * np + 1], pa, vf[2], vf[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[warp][s]);       // the stage may be refilled
            }
            if (failed) break;
            // ---- this warp's partial of the unit: slot (unit + warp), rows < nrows ----
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
            if (row_ok) {
                float* dst = a.part + ((size_t)(g * a.Nkv + kvh + gw) * a.part_rows + mrow) * (D + 2);
#pragma unroll
                for (int i = 0; i < D / 8; ++i)
                    *reinterpret_cast<float2*>(dst + i * 8 + mcol) = make_float2(o[i][0] + o[i][2], o[i][1] + o[i][3]);
                if ((lane & 3) == 0) { dst[D] = m_run; dst[D + 1] = l_run; }
            }
        }
        // after a failed wait: let this warp's copies in flight land (bounded) before the CTA's memory goes away
        if (failed) {
            __syncwarp();
            if (lane == 0)
                for (int w_it = it; w_it < issued[warp]; ++w_it) mbar_wait(&full[warp][w_it % NST], (w_it / NST) & 1);
        }
    }
}

template <int D>
inline size_t attn_mma_smem_bytes() {
    return (size_t)AmGeom<D>::NCW * AmGeom<D>::NST * (2 * (D / 64) * kAmTile * 128) + (size_t)AmGeom<D>::NCW * 16 * (D + 8) * 2 + 1024;
}

// One CTA per unit (group, kv head): adds the unit's partials in warp order and writes the normalised
// output rows. The partial slots of a unit are (unit + w) for the consumer warps w whose tile range
// meets the unit's.
template <int D, int G>
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnMmaArgs a) {
    constexpr int CH = 64;                                     // partials handled per round
    __shared__ float s_m[kAmRows][CH], s_e[kAmRows][CH], s_l[kAmRows][CH], s_L[kAmRows], s_M[kAmRows];
    pdl_wait();
    pdl_launch();
    const int u = blockIdx.x, g = u / a.Nkv, kvh = u % a.Nkv;
    // tile prefix of the groups as the attention kernel computed it (one round of loads instead of a CTA-wide scan)
    const int pre_g = __ldcg(a.pre_out + g), pre_g1 = __ldcg(a.pre_out + g + 1), pre_all = __ldcg(a.pre_out + a.NG);
    const int nt = pre_g1 - pre_g;
    if (nt == 0) return;
    const int T = pre_all * a.Nkv, W = a.total_warps;
    const int ub = pre_g * a.Nkv + kvh * nt;
    const int w0 = am_warp_of(T, W, ub), w1 = am_warp_of(T, W, ub + nt - 1);
    const int nrows = a.grp_n[g] * G, row0 = a.grp_row0[g];
    const int tid = threadIdx.x;
    const float* base = a.part + (size_t)(u + w0) * a.part_rows * (D + 2);
    const size_t slot = (size_t)a.part_rows * (D + 2);
    const int np = w1 - w0 + 1;
    if (np <= CH) {
        // the usual case: every (m, l) pair in one round of loads, scale factors from shared memory, one round of
        // loads for the weighted sums, normalised and written once
        for (int i = tid; i < nrows * np; i += blockDim.x) {
            const int r = i / np, w = i % np;
            const float* p = base + (size_t)w * slot + (size_t)r * (D + 2);
            s_m[r][w] = p[D];
            s_l[r][w] = p[D + 1];
        }
        __syncthreads();
        if (tid < nrows) {
            float M = -INFINITY;
            for (int w = 0; w < np; ++w) M = fmaxf(M, s_m[tid][w]);
            float L = 0.0f;
            for (int w = 0; w < np; ++w) {
                const float e = (s_m[tid][w] == -INFINITY) ? 0.0f : expf(s_m[tid][w] - M);
                s_e[tid][w] = e;
                L += e * s_l[tid][w];
            }
            s_L[tid] = L;
        }
        __syncthreads();
        for (int idx = tid; idx < nrows * D; idx += blockDim.x) {
            const int r = idx / D, d = idx % D;
            float acc = 0.0f;
            for (int w = 0; w < np; ++w) acc += s_e[r][w] * base[(size_t)w * slot + (size_t)r * (D + 2) + d];
            const size_t oi = (size_t)(row0 + r / G) * a.Nq * D + (size_t)(kvh * G + r % G) * D + d;
            const float ov = acc / s_L[r];
            a.out[oi] = ov;
            if (a.out_bf16) a.out_bf16[oi] = (uint16_t)f32_to_bf16_bits(ov);
        }
        return;
    }
    // many partials (one long sequence spread over most of the grid): running maximum and denominator first,
    // then the weighted sums CH partials at a time through the output buffer
    if (tid < nrows) {
        float M = -INFINITY;
        for (int w = 0; w < np; ++w) M = fmaxf(M, base[(size_t)w * slot + (size_t)tid * (D + 2) + D]);
        float L = 0.0f;
        for (int w = 0; w < np; ++w) {
            const float* p = base + (size_t)w * slot + (size_t)tid * (D + 2);
            const float e = (p[D] == -INFINITY) ? 0.0f : expf(p[D] - M);
            L += e * p[D + 1];
        }
        s_M[tid] = M;
        s_L[tid] = L;
    }
    __syncthreads();
    for (int c0 = 0; c0 < np; c0 += CH) {
        const int nc = min(CH, np - c0);
        __syncthreads();
        for (int i = tid; i < nrows * nc; i += blockDim.x) {
            const int r = i / nc, w = c0 + i % nc;
            const float mw = base[(size_t)w * slot + (size_t)r * (D + 2) + D];
            s_e[r][i % nc] = (mw == -INFINITY) ? 0.0f : expf(mw - s_M[r]);
        }
        __syncthreads();
        for (int idx = tid; idx < nrows * D; idx += blockDim.x) {
            const int r = idx / D, d = idx % D;
            float acc = 0.0f;
            for (int w = 0; w < nc; ++w) acc += s_e[r][w] * base[(size_t)(c0 + w) * slot + (size_t)r * (D + 2) + d];
            const size_t oi = (size_t)(row0 + r / G) * a.Nq * D + (size_t)(kvh * G + r % G) * D + d;
            if (c0 == 0) a.out[oi] = acc; else a.out[oi] += acc;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < nrows * D; idx += blockDim.x) {
        const int r = idx / D, d = idx % D;
        const size_t oi = (size_t)(row0 + r / G) * a.Nq * D + (size_t)(kvh * G + r % G) * D + d;
        const float ov = a.out[oi] / s_L[r];
        a.out[oi] = ov;
        if (a.out_bf16) a.out_bf16[oi] = (uint16_t)f32_to_bf16_bits(ov);
    }
}

// Per (row, head) warp: q/k RMS norm with weight + RoPE, v unit RMS norm (kernel_module.rs:1133-1246,
// 1510-1550), K/V append at slot position % capacity (kernel_module.rs:1423-1439), and the query written as
// BF16 high and low parts for attn_mma_kernel. With `q_hl` null only the K/V rows are produced (the
// SIMT attention kernel norms its own queries); with `write_kv` 0 only the queries (KV-shared layers).
struct QkvPostArgs {
    const float* qkv;            // [splits, R, qkv_n] projection output (K-split partials), columns q | k | v
    int qkv_n, splits, R, Nq, Nkv;
    const float* q_norm;
    const float* k_norm;
    const float* inv_freq;
    int rotary_half;
    float eps;
    const int32_t* row_pos;
    const int32_t* row_seq;
    const uint32_t* row_tok;
    void* kpool;
    void* vpool;
    const int32_t* page_table;
    int pages_per_seq, page_tokens;
    const int32_t* cap;
    uint16_t* q_hl;              // [R][Nq][2][D] or null
    int write_kv;                // 0: a KV-shared layer (its source layer has appended K/V; the projection holds q only)
};

// EPT (2, 4 or 8) consecutive f32 / 16-bit values per lane, moved with the widest aligned access
template <int EPT> DEVINL void ld_f32_vec(const float* p, float (&v)[EPT]) {
    if constexpr (EPT == 8) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else if constexpr (EPT == 4) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else {
        const float2 a = __ldcg(reinterpret_cast<const float2*>(p));
        v[0] = a.x; v[1] = a.y;
    }
}
template <int EPT> DEVINL void st_f32_vec(float* p, const float (&v)[EPT]) {
    if constexpr (EPT == 8) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else if constexpr (EPT == 4) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        reinterpret_cast<float2*>(p)[0] = make_float2(v[0], v[1]);
    }
}
template <int EPT> DEVINL void st_u16_vec(uint16_t* p, const uint32_t (&bits)[EPT]) {      // low 16 bits of every entry
    uint32_t w[EPT / 2];
#pragma unroll
    for (int i = 0; i < EPT / 2; ++i) w[i] = (bits[2 * i] & 0xffffu) | (bits[2 * i + 1] << 16);
    if constexpr (EPT == 8) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    else if constexpr (EPT == 4) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
    else *reinterpret_cast<uint32_t*>(p) = w[0];
}

template <typename KT, int D>
__global__ void __launch_bounds__(128) qkv_post_kernel(const QkvPostArgs a) {
    constexpr int EPT = D / 32;
    pdl_wait();
    pdl_launch();
    const int lane = threadIdx.x & 31;
    const int first_task = a.q_hl ? 0 : a.Nq;
    const int last_task = a.write_kv ? a.Nq + 2 * a.Nkv : a.Nq;      // tasks: q heads, then k heads, then v heads
    const int per_row = last_task - first_task;
    const int job = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (per_row <= 0 || job >= a.R * per_row) return;
    const int row = job / per_row, task = first_task + job % per_row;
    if (a.row_tok != nullptr && a.row_tok[row] == kInactiveToken) return;
    const int pos = a.row_pos[row];
    const int col = task * D;                                  // q heads, then k heads, then v heads
    float t[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) t[e] = 0.0f;
    for (int sp = 0; sp < a.splits; ++sp) {                    // K-split partials, in split order
        float v[EPT];
        ld_f32_vec<EPT>(a.qkv + ((size_t)sp * a.R + row) * a.qkv_n + col + lane * EPT, v);
#pragma unroll
        for (int e = 0; e < EPT; ++e) t[e] += v[e];
    }
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) ss += t[e] * t[e];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)D + a.eps);
    const bool is_v = task >= a.Nq + a.Nkv;
    float o[EPT];
    if (!is_v) {
        constexpr int half = D / 2;
        float w[EPT], fr[EPT];
        ld_f32_vec<EPT>((task < a.Nq ? a.q_norm : a.k_norm) + lane * EPT, w);
        ld_f32_vec<EPT>(a.inv_freq + (lane * EPT) % half, fr);               // a lane's elements lie in one half
#pragma unroll
        for (int e = 0; e < EPT; ++e) t[e] = t[e] * r * w[e];
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const int d = lane * EPT + e;
            const int fi = d % half;
            const float partner = __shfl_xor_sync(0xffffffffu, t[e], 16);      // element d +- D/2 lives 16 lanes away
            float v = t[e];
            if (fi < a.rotary_half) {
                float sn, cs;
                sincosf((float)pos * fr[e], &sn, &cs);
                const float rotated = d < half ? -partner : partner;
                v = v * cs + rotated * sn;
            }
            o[e] = v;
        }
    } else {
#pragma unroll
        for (int e = 0; e < EPT; ++e) o[e] = t[e] * r;
    }
    if (task < a.Nq) {
        uint16_t* dst = a.q_hl + ((size_t)row * a.Nq + task) * 2 * D + lane * EPT;
        uint32_t hi[EPT], lo[EPT];
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            hi[e] = f32_to_bf16_bits(o[e]);
            lo[e] = f32_to_bf16_bits(o[e] - __uint_as_float(hi[e] << 16));
        }
        st_u16_vec<EPT>(dst, hi);
        st_u16_vec<EPT>(dst + D, lo);
        return;
    }
    const int kvh = (task - a.Nq) % a.Nkv;
    const int seq = a.row_seq ? a.row_seq[row] : row;
    const int slot = pos % a.cap[seq];
    const size_t off = (((size_t)a.page_table[(size_t)seq * a.pages_per_seq + slot / a.page_tokens] * a.Nkv + kvh) *
                            a.page_tokens + slot % a.page_tokens) * (size_t)D + lane * EPT;
    KT* pool = (KT*)(is_v ? a.vpool : a.kpool);
    if constexpr (sizeof(KT) == 2) {
        uint32_t bits[EPT];
#pragma unroll
        for (int e = 0; e < EPT; ++e) bits[e] = f32_to_bf16_bits(o[e]);
        st_u16_vec<EPT>((uint16_t*)pool + off, bits);
    } else {
        st_f32_vec<EPT>((float*)pool + off, o);
    }
}

}  // namespace oxg4
