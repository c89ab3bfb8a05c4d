// Batched projection on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// out[b, n] = sum_k x[b, k] * W[n, k]   (the reference's cuBLAS contract, crates/oxide-torch-cuda/src/
// cublas.rs:101-153: BF16 operands, f32 accumulate, f32 output) for 1..256 activation rows (one block of 16 / 32 /
// 64 / 128 / 256 rows per weight tile), where the weight matrix is streamed from HBM exactly once.
//
// Roles are swapped with respect to a textbook GEMM because the batch is the small dimension: the
// 128-row weight tile is the MMA's M operand (A, K-major in shared memory), the activations are
// the N operand (B, K-major), the accumulator lives in TMEM as 128 lanes x N columns of f32. Two accumulators
// are allocated: the MMAs of a CTA's next work unit run while the epilogue warps drain the previous one.
//
//   warp 0, one lane : TMA producer  (cp.async.bulk.tensor.2d, 128-byte swizzle, NS-stage ring)
//   warp 1, one lane : MMA issuer    (tcgen05.mma.cta_group::1.kind::f16, 4 x K=16 per 64-wide stage)
//   warps 2..5       : epilogue      (tcgen05.ld 32x32b, one TMEM lane = one output row per thread;
//                                     a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31)
//
// A CTA walks the work units (tile, K-split, row block) u = blockIdx.x, blockIdx.x + gridDim.x, ... Rows past the end of the
// matrix and batch rows past B are zero-filled by TMA (tensor-map bounds) and masked at the store.
// Every mbarrier wait is bounded: when a wait runs out the kernel raises `*err`, stops issuing work,
// still frees its TMEM columns and returns, so a protocol bug cannot hang the GPU.
//
// HBM-bound: bytes per launch = N * K * 2 (+ B * K * 2 per tile from L2 for the activations).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace oxg4 {

constexpr int kTcThreads = 192;      // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue (one per TMEM lane quadrant)
constexpr int kTcTileM = 128;        // weight rows per tile (UMMA M)
constexpr int kTcTileK = 64;         // BF16 elements per stage row = 128 bytes = one swizzle atom row
// shared-memory stages of the TMA ring: 6 x 24 KiB for up to 64 activation rows per block, 4 x 48 KiB for 256
template <int BN> struct TcStages { static constexpr int value = BN <= 64 ? 6 : (BN <= 128 ? 5 : 4); };
constexpr uint32_t kTcSpinLimit = 2u * 1000u * 1000u;   // bounded mbarrier polling

struct TcGemmArgs {
    int N, K, B;             // rows of ONE weight matrix, columns, activation rows (cut into blocks of BN rows)
    int n_mats;              // 1, or 2 when gate and up are streamed by one launch (second tensor map)
    int S;                   // K-splits: a work unit is (128-row tile, split, row block); S partial outputs are added later
    int TB;                  // row blocks: ceil(B / BN). Units of one weight tile are adjacent, so that tile
                             // crosses HBM once and the other row blocks find it in L2 (prompt chunks: B up to 256)
    int kb_per_split;        // 64-column blocks per split
    float* out;              // [S, B, ld]; matrix m occupies columns col0 + m * N ..
    int ld, col0;            // row stride of `out` (>= n_mats * N) and first column written
    int* err;                // device flag, set non-zero if a bounded wait ran out
};

DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

DEVINL void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
DEVINL void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// returns false if the phase did not complete within the polling budget
DEVINL bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kTcSpinLimit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

DEVINL void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
DEVINL uint64_t umma_smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)1 << 16;                                   // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                   // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                   // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: BF16 x BF16 -> f32, both operands K-major, M x N tile
DEVINL uint32_t umma_idesc_bf16(int M, int N) {
    uint32_t d = 0;
    d |= 1u << 4;                       // D format f32
    d |= 1u << 7;                       // A format BF16
    d |= 1u << 10;                      // B format BF16
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}

template <int BN>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w1,
               const __grid_constant__ CUtensorMap map_x, const TcGemmArgs a) {
    static_assert(BN == 16 || BN == 32 || BN == 64 || BN == 128 || BN == 256, "activation rows per tile");
    constexpr int kTcStages = TcStages<BN>::value;
    constexpr uint32_t A_BYTES = kTcTileM * kTcTileK * 2;     // 16 KiB
    constexpr uint32_t B_BYTES = BN * kTcTileK * 2;
    constexpr uint32_t STAGE = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
    constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN;          // TMEM columns of one accumulator tile
    constexpr uint32_t TM_COLS = 2 * ACC_COLS;                // two accumulators (64..512 columns, a power of two): the
                                                              // MMAs of a unit run while the epilogue drains the previous one
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full[kTcStages], empty[kTcStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base;
    __shared__ volatile int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_per_mat = (a.N + kTcTileM - 1) / kTcTileM;
    const int n_tiles = tiles_per_mat * a.n_mats * a.S * a.TB;   // work units: (matrix, tile, split, row block)
    const int kblocks_all = (a.K + kTcTileK - 1) / kTcTileK;
    // unit u -> row block u % TB, split (u / TB) % S, tile index (over both matrices) u / (TB * S)
    auto kb_begin = [&](int u) { return ((u / a.TB) % a.S) * a.kb_per_split; };
    auto kb_end = [&](int u) { return min(kblocks_all, ((u / a.TB) % a.S + 1) * a.kb_per_split); };
    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 128); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        // The walk over this CTA's (unit, k-block) sequence. The weight tiles depend on nothing the preceding
        // kernel writes, so the first ring of them is requested BEFORE the dependency wait (the launch is
        // programmatic: this CTA may be resident while the preceding kernel still runs) and only the
        // activation tiles of those stages wait for it.
        // Everything that is constant over a unit (and needs an integer division) is computed once per unit: this
        // thread has to request a 16 KiB tile every ~350 ns for the CTA to get its share of the HBM bandwidth.
        // Every CTA starts its walk over a unit's k-blocks at a different block (jr), so that CTAs running in
        // step do not all ask L2 for the same activation tile at the same moment; the order of the f32 sums
        // inside a unit therefore depends on the CTA (fixed for a given launch geometry).
        int t = blockIdx.x;
        int k0 = 0, nk = 1, jr = 0, left = 0, trow = 0, xrow = 0;
        const CUtensorMap* wmap = &map_w;
        auto enter_unit = [&]() {
            const int sp = (t / a.TB) % a.S;
            k0 = sp * a.kb_per_split;
            nk = min(kblocks_all, k0 + a.kb_per_split) - k0;
            jr = (int)blockIdx.x % nk;
            left = nk;
            const int tg = t / (a.S * a.TB);
            const bool second = tg >= tiles_per_mat;
            wmap = second ? &map_w1 : &map_w;
            trow = (second ? tg - tiles_per_mat : tg) * kTcTileM;
            xrow = (t % a.TB) * BN;
        };
        auto advance = [&]() {
            if (++jr == nk) jr = 0;
            if (--left == 0) {
                t += gridDim.x;
                if (t < n_tiles) enter_unit();
            }
        };
        if (t < n_tiles) enter_unit();
        int pre_x[kTcStages], pre_row[kTcStages];
        int n_pre = 0;
        while (n_pre < kTcStages && t < n_tiles) {
            mbar_expect_tx(&full[n_pre], A_BYTES + B_BYTES);
            const int kx = (k0 + jr) * kTcTileK;
            tma_load_2d(tiles + (size_t)n_pre * STAGE, wmap, kx, trow, &full[n_pre]);
            pre_x[n_pre] = kx;
            pre_row[n_pre] = xrow;
            ++n_pre;
            advance();
        }
        pdl_wait();
        pdl_launch();
        for (int i = 0; i < n_pre; ++i) tma_load_2d(tiles + (size_t)i * STAGE + A_BYTES, &map_x, pre_x[i], pre_row[i], &full[i]);
        for (uint32_t it = (uint32_t)n_pre; t < n_tiles && !failed; ++it) {
            const int s = it % kTcStages;
            const uint32_t ph = (it / kTcStages) & 1;
            if (!mbar_wait(&empty[s], ph ^ 1)) { failed = 1; atomicExch(a.err, 1); break; }
            mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
            const int kx = (k0 + jr) * kTcTileK;
            tma_load_2d(tiles + (size_t)s * STAGE, wmap, kx, trow, &full[s]);
            tma_load_2d(tiles + (size_t)s * STAGE + A_BYTES, &map_x, kx, xrow, &full[s]);
            advance();
        }
    } else {
        pdl_wait();
        pdl_launch();
    }
    if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = umma_idesc_bf16(kTcTileM, BN);
        uint32_t it = 0, tile_i = 0;
        for (int t = blockIdx.x; t < n_tiles && !failed; t += gridDim.x, ++tile_i) {
            // accumulator tile_i % 2; its previous user (unit tile_i - 2) must have been drained by the epilogue
            const uint32_t ab = tile_i & 1, use = tile_i >> 1;
            if (use > 0 && !mbar_wait(&acc_empty[ab], (use - 1) & 1)) { failed = 1; atomicExch(a.err, 2); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + ab * ACC_COLS;
            const int nk = kb_end(t) - kb_begin(t);
            for (int j = 0; j < nk; ++j, ++it) {
                const int s = it % kTcStages;
                const uint32_t ph = (it / kTcStages) & 1;
                if (!mbar_wait(&full[s], ph)) { failed = 1; atomicExch(a.err, 3); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char* sa = tiles + (size_t)s * STAGE;
                const uint64_t da = umma_smem_desc(sa), db = umma_smem_desc(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < kTcTileK / 16; ++k) {
                    const uint32_t accumulate = (j > 0 || k > 0) ? 1u : 0u;
                    // advance 16 BF16 = 32 bytes inside the swizzle atom: +2 in units of 16 bytes
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(acc), "l"(da + (uint64_t)(2 * k)), "l"(db + (uint64_t)(2 * k)), "r"(idesc), "r"(accumulate)
                        : "memory");
                }
                // the stage may be refilled once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
            }
            if (failed) break;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&acc_full[ab])) : "memory");
        }
    }
    __syncwarp();

    // ---- epilogue: warps 2..5; thread = TMEM lane = output row of the tile ----
    if (warp >= 2) {
        const int quad = warp & 3;
        uint32_t tile_i = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++tile_i) {
            const uint32_t ab = tile_i & 1, use = tile_i >> 1;
            if (!mbar_wait(&acc_full[ab], use & 1)) { if (lane == 0) atomicExch(a.err, 4); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int tg = t / (a.S * a.TB), sp = (t / a.TB) % a.S, b0 = (t % a.TB) * BN;
            const bool second = tg >= tiles_per_mat;
            const int row = (second ? tg - tiles_per_mat : tg) * kTcTileM + quad * 32 + lane;
            float* dst = a.out + ((size_t)sp * a.B + b0) * a.ld + a.col0 + (second ? a.N : 0);
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + ab * ACC_COLS + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (b0 + c0 + j < a.B) dst[(size_t)(c0 + j) * a.ld + row] = __uint_as_float(v[j]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[ab])) : "memory");
        }
    }

    // ---- teardown: always reached, also after a failed wait ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TM_COLS));
    }
}

template <int BN>
inline size_t tc_gemm_smem_bytes() {
    const size_t a = (size_t)kTcTileM * kTcTileK * 2;
    const size_t b = (((size_t)BN * kTcTileK * 2 + 1023) / 1024) * 1024;
    return (a + b) * TcStages<BN>::value + 1024;
}

}  // namespace oxg4
