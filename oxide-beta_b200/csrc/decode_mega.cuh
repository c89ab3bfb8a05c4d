// Persistent decode kernel for one sequence with BF16 weights: ALL layers of a step in one cooperative
// launch, one CTA per SM.
//
// A decode step for one sequence streams every weight byte once and does almost no arithmetic, so the
// step time is (bytes / HBM bandwidth) plus whatever time the memory pipe sits idle. With one kernel per
// projection the pipe idles at every kernel boundary (drain, dependency wait, prologue, ramp-up). Here
// the weights never stop flowing: in every CTA one warp (the producer) walks the CTA's share of the
// whole step's weight stream — layer after layer, QKV, O, gate/up, down — and copies it piece by piece
// into a ring of shared-memory stages with bulk TMA copies (cp.async.bulk + mbarrier transaction
// counts), running as far ahead of the arithmetic as the ring allows. The other sixteen warps (the
// consumers) execute the step's dependency chain: prologue (residual update + RMS norms, the
// reference's rms_norm / add / mul_bf16_scalar / rms_norm_bf16 launches, crates/oxide-torch-models/src/
// gemma4_cuda/decode.rs:14-21,61-65,161-171), dot products of the activation vector with the weight
// rows found in the ring, epilogue (store / GeGLU), a grid-wide barrier, attention (attention.cuh,
// split over all CTAs), and so on. Barriers and prologues therefore cost arithmetic time but no memory
// time as long as they are shorter than the ring is deep.
//
// Work split: every CTA owns a contiguous block of rows of every weight matrix (for gate/up a block of
// (gate_i, up_i) pairs), so its share of a matrix is contiguous in memory. A piece is R whole rows
// (R a power of two <= 16) and is multiplied by ONE consumer warp on the tensor cores (mma.sync
// m16n8k16): the piece's rows, cut into 16 / R interleaved segments each, are the 16 rows of the A
// operand (read from the ring with ldmatrix), the matching segments of the activation vector are the
// columns of B. Pieces go to the warps round-robin, so as many pieces as the ring has stages are in
// work at once; every output row is summed by one warp in a fixed order.
//
// Every wait is bounded (mbarrier polls, grid barrier polls). When one runs out the CTA raises the
// abort word; every other wait in the grid sees it and gives up as well, the producers wait (bounded)
// for their copies in flight, and the kernel returns with a status the host turns into an error.
//
// HBM-bound: bytes per launch = all layers' projection weights + the visible K/V rows.
#pragma once
#include "attention.cuh"
#include "gemv.cuh"          // block_range
#include "gemv_mma.cuh"      // mma_bf16_16816
#include "tc_gemm.cuh"      // mbarrier helpers

namespace oxg4 {

constexpr int kMegaConsumerWarps = 16;
constexpr int kMegaConsumers = kMegaConsumerWarps * 32;      // 512: attention.cuh's BarFirst512 counts on it
constexpr int kMegaThreads = kMegaConsumers + 32;            // + the producer warp
constexpr int kMegaStages = kMegaConsumerWarps;             // one ring stage per consumer warp
constexpr int kMegaMaxJ = 11;                                 // hidden size <= 11 * 512
constexpr unsigned int kMegaSpinLimit = 1u << 21;             // polls (each up to ~2 us asleep) before a wait gives up

struct MegaLayer {            // per-layer model constants (device array)
    const void *wqkv, *wo, *wgate, *wup, *wdown;
    const float *input_ln, *post_attn_ln, *pre_ff_ln, *post_ff_ln, *q_norm, *k_norm, *inv_freq;
    float layer_scalar;
    int sliding, rotary_half;
};
struct MegaKv {               // per-layer cache pools (device array, per cache table)
    void *k, *v;
};
struct MegaSync {
    unsigned int arrived;     // grid barrier counter (zeroed before every launch)
    unsigned int abort;       // non-zero: a bounded wait ran out somewhere
    unsigned int first;       // which wait gave up first: 1 grid barrier, 2 producer (stage not released), 3 consumer (piece not delivered)
    unsigned int info[3];     // of that wait: CTA, piece or barrier number, warp
};
DEVINL void mega_fail(MegaSync* sy, int* status, unsigned int code, unsigned int cta, unsigned int n, unsigned int w) {
    if (atomicCAS(&sy->first, 0u, code) == 0u) {
        sy->info[0] = cta;
        sy->info[1] = n;
        sy->info[2] = w;
        *(volatile int*)status = (int)(code | (cta << 4) | (n << 12) | (w << 26));
    }
    atomicExch(&sy->abort, 1u);
}

struct MegaArgs {
    const MegaLayer* layers;
    const MegaKv* kv;
    int L, H, I, Nq, Nkv, qkv_n;
    int R[4], F[4];           // rows per piece and fractions per row: QKV, O, gate/up, down
    int stage_bytes;
    int pf_kb;                // KiB of the next matrix kind's share a CTA prefetches into L2 (0: off)
    int x_bytes;              // shared bytes of the activation / attention scratch region
    int slot_floats;          // shared floats for the partial sums
    const uint16_t* embed;
    const uint32_t* tokens;
    float embed_scale, eps;
    float *qkv_raw, *attn_out, *o_raw, *gu_raw, *down_raw, *h_out;
    // attention (AttnArgs fields that do not change with the layer)
    const int32_t* pos;
    const int32_t *pt_full, *pt_slide, *cap_full, *cap_slide;
    int pps_full, pps_slide, page_tokens, splits_full, splits_slide, min_split;
    float* part;
    unsigned int* ticket;
    MegaSync* sync;
    int* status;              // set non-zero when the kernel gave up
    unsigned long long* ts;   // optional timeline: CTA 0 stores 15 global-timer stamps per layer, or null
};

DEVINL unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
DEVINL unsigned int ld_relaxed_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
DEVINL void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16), completion on `bar`
DEVINL void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Bounded mbarrier wait that also gives up when the CTA (`dead`) or the grid (`abort`) has given up.
// The wait carries a suspend-time hint: a warp whose piece has not landed sleeps inside try_wait instead
// of re-issuing polls, which would take issue slots from the warps of its scheduler that are multiplying.
DEVINL bool mega_wait(uint64_t* bar, uint32_t parity, const volatile int* dead, const unsigned int* abort) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 1; i <= kMegaSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(2000u)
            : "memory");
        if (done) return true;
        if ((i & 7u) == 0u && (*dead || ld_relaxed_gpu(abort))) return false;
    }
    return false;
}
DEVINL void cons_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// sum over the 512 consumer threads, same total in every thread (warp order)
DEVINL float cons_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    cons_sync();
    if (lane == 0) red[warp] = v;
    cons_sync();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kMegaConsumerWarps; ++w) t += red[w];
    return t;
}

// Segments a weight row is cut into so that R rows fill the 16 rows of the mma A operand (8 at most:
// B has eight columns).
__host__ DEVINL int mega_nseg(int R) { return R >= 16 ? 1 : (16 / R > 8 ? 8 : 16 / R); }

// A CTA's share of one matrix kind. A piece is R whole rows, or (R == 1, F > 1) one of the F contiguous
// fractions of a row that is too long for a stage.
struct MegaShare {
    int r0, cnt;              // first row (pair for gate/up) and number of rows (pairs)
    int R, F, np;             // rows per piece, fractions per row, pieces (gate/up: gate and up row blocks alternate)
};
DEVINL MegaShare mega_share(int rows, int R, int F, bool pairs) {
    MegaShare s;
    block_range(rows, gridDim.x, blockIdx.x, s.r0, s.cnt);
    s.R = R;
    s.F = F;
    s.np = (s.cnt + R - 1) / R * F * (pairs ? 2 : 1);
    return s;
}

template <typename KT, int D, int G>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const MegaArgs a) {
    extern __shared__ __align__(128) unsigned char mega_smem[];
    __shared__ __align__(8) uint64_t full[kMegaStages], empty[kMegaStages];
    __shared__ float red[kMegaConsumerWarps];
    __shared__ float scratch[kMegaConsumerWarps * 16];
    __shared__ volatile int dead;              // a consumer of this CTA gave up (written only before a consumer barrier)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.H;
    constexpr int NS = kMegaStages;
    unsigned char* ring = mega_smem;                                         // [NS][stage_bytes]
    unsigned char* xreg = ring + (size_t)NS * a.stage_bytes;                 // activations (BF16) / attention scratch
    float* h_s = reinterpret_cast<float*>(xreg + a.x_bytes);                 // [H] residual stream
    float* slots = h_s + H;                                                   // partial sums
    uint16_t* xs = reinterpret_cast<uint16_t*>(xreg);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // matrix kinds: 0 QKV [qkv_n, H], 1 O [H, Nq*D], 2 gate/up [I, H] x 2, 3 down [H, I]
    const MegaShare sh0 = mega_share(a.qkv_n, a.R[0], a.F[0], false);
    const MegaShare sh1 = mega_share(H, a.R[1], a.F[1], false);
    const MegaShare sh2 = mega_share(a.I, a.R[2], a.F[2], true);
    const MegaShare sh3 = mega_share(H, a.R[3], a.F[3], false);

    if (warp == kMegaConsumerWarps) {
        // ================= producer: the CTA's share of the whole step's weight stream =================
        // One thread issues everything, so the work per piece is kept to a wait, an expect and one bulk copy
        // per row: all addressing is incremental.
        if (lane == 0) {
            unsigned int it = 0, st = 0, par = 0;
            bool ok = true;
            // `blocks` row blocks of `rows_left` rows in all, each block as s.F pieces (one per row fraction)
            auto stream = [&](const char* base, const MegaShare& s, const int K) {
                const uint32_t rowb = (uint32_t)K * 2u;
                const uint32_t fb = rowb / (uint32_t)s.F;                  // bytes of one row fraction
                const char* src = base + (size_t)s.r0 * rowb;
                for (int left = s.cnt; left > 0 && ok; left -= s.R, src += (size_t)s.R * rowb) {
                    const int nrows = min(s.R, left);
                    for (int f = 0; f < s.F; ++f) {
                        if (dead || !mega_wait(&empty[st], par ^ 1u, &dead, &a.sync->abort)) { ok = false; return; }
                        mbar_expect_tx(&full[st], (uint32_t)nrows * fb);
                        unsigned char* dst = ring + (size_t)st * a.stage_bytes;
                        const char* sp = src + (size_t)f * fb;
                        for (int r = 0; r < nrows; ++r, dst += fb + 16u, sp += rowb)   // rows land 16 bytes apart (see consume)
                            bulk_load(dst, sp, fb, &full[st]);
                        ++it;
                        if (++st == (unsigned)NS) { st = 0; par ^= 1u; }
                    }
                }
            };
            // gate and up row blocks alternate, so that a pair's two dot products finish close together
            auto stream2 = [&](const char* g0, const char* u0, const MegaShare& s, const int K) {
                const uint32_t rowb = (uint32_t)K * 2u;
                const uint32_t fb = rowb / (uint32_t)s.F;
                size_t off = (size_t)s.r0 * rowb;
                for (int left = s.cnt; left > 0 && ok; left -= s.R, off += (size_t)s.R * rowb) {
                    const int nrows = min(s.R, left);
                    for (int which = 0; which < 2; ++which) {
                        const char* src = (which ? u0 : g0) + off;
                        for (int f = 0; f < s.F; ++f) {
                            if (dead || !mega_wait(&empty[st], par ^ 1u, &dead, &a.sync->abort)) { ok = false; return; }
                            mbar_expect_tx(&full[st], (uint32_t)nrows * fb);
                            unsigned char* dst = ring + (size_t)st * a.stage_bytes;
                            const char* sp = src + (size_t)f * fb;
                            for (int r = 0; r < nrows; ++r, dst += fb + 16u, sp += rowb) bulk_load(dst, sp, fb, &full[st]);
                            ++it;
                            if (++st == (unsigned)NS) { st = 0; par ^= 1u; }
                        }
                    }
                }
            };
            // L2 prefetch of the start of a share (at most pf_kb KiB), issued one matrix kind ahead: while the
            // consumers sit in a barrier, a prologue or attention, HBM keeps working and the ring refills from L2
            auto warm = [&](const char* base, const MegaShare& s, const int K, size_t cap) {
                const size_t bytes = min((size_t)s.cnt * K * 2, cap);
                const char* p0 = base + (size_t)s.r0 * K * 2;
                for (size_t off = 0; off < bytes; off += 32768) prefetch_l2_bulk(p0 + off, min((size_t)32768, bytes - off));
            };
            const size_t cap = (size_t)a.pf_kb * 1024;
            for (int l = 0; l < a.L && ok; ++l) {
                const MegaLayer& ly = a.layers[l];
                if (cap) warm((const char*)ly.wo, sh1, a.Nq * D, cap);
                stream((const char*)ly.wqkv, sh0, H);
                if (cap) { warm((const char*)ly.wgate, sh2, H, cap / 2); warm((const char*)ly.wup, sh2, H, cap / 2); }
                stream((const char*)ly.wo, sh1, a.Nq * D);
                if (cap) warm((const char*)ly.wdown, sh3, a.I, cap);
                stream2((const char*)ly.wgate, (const char*)ly.wup, sh2, H);
                if (cap && l + 1 < a.L) warm((const char*)a.layers[l + 1].wqkv, sh0, H, cap);
                stream((const char*)ly.wdown, sh3, a.I);
            }
            if (!ok) {
                if (!dead && !ld_relaxed_gpu(&a.sync->abort)) mega_fail(a.sync, a.status, 2u, blockIdx.x, it, 16u);
                atomicExch(&a.sync->abort, 1u);
                // copies in flight land in this CTA's shared memory: wait (bounded) until they have
                const unsigned int issued = it;
                const unsigned int first = issued > (unsigned)NS ? issued - NS : 0u;
                for (unsigned int q = first; q < issued; ++q) mbar_wait(&full[q % NS], (q / NS) & 1u);
            }
        }
        return;
    }

    // ================= consumers =================
    unsigned int gen = 0;                 // grid barriers passed
    bool alive = true;                    // the same in all consumer threads: refreshed only right after a consumer barrier

    // all consumer threads call
    auto grid_barrier = [&]() {
        cons_sync();
        if (tid == 0) {
            ++gen;
            const unsigned int target = gen * gridDim.x;
            __threadfence();
            atomicAdd(&a.sync->arrived, 1u);
            unsigned int polls = 0;
            while (ld_acquire_gpu(&a.sync->arrived) < target) {
                __nanosleep(40);
                if (++polls > kMegaSpinLimit || ((polls & 255u) == 0u && ld_relaxed_gpu(&a.sync->abort))) {
                    dead = 1;
                    if (polls > kMegaSpinLimit) mega_fail(a.sync, a.status, 1u, blockIdx.x, gen, 0u);
                    break;
                }
            }
        } else {
            ++gen;
        }
        cons_sync();
        alive = !dead;
    };

    // dot products of xs[0..K) with this CTA's rows of one matrix kind on the tensor cores (mma.sync
    // m16n8k16). The ring has one stage per consumer warp: piece P of the step's stream lands in stage
    // P % 16 and is multiplied by warp P % 16, so sixteen pieces are in work at once and nothing is reduced
    // across warps. Each row (fraction) of a piece is cut into nseg = 16 / R interleaved segments (k-step
    // q of segment sg is k-step q * nseg + sg) and (row r, segment sg) is row r * nseg + sg of the 16-row A
    // operand, so all of A is real weight data; column n of B is segment n of the activation vector and
    // the useful outputs are C[r * nseg + sg][sg].
    unsigned int pcount = 0;              // pieces of the stream consumed so far (same in every consumer thread)
    long long dbg_wait = 0, dbg_work = 0; // cycles warp 0 spent waiting for the ring / computing (timeline runs only)
    const uint32_t my_stage = smem_u32(ring + (size_t)warp * a.stage_bytes);
    auto consume = [&](const int K, const MegaShare s, const bool gateup) {
        const int R = s.R, F = s.F;
        const int nseg = mega_nseg(R);
        const int Kf = K / F;                                // elements of one row (fraction) of a piece
        const int ksteps = (Kf >> 4) / nseg;                 // k-steps per segment
        const uint32_t rstride = (uint32_t)Kf * 2u + 16u;    // rows sit 16 bytes apart from back to back: conflict-free ldmatrix
        const int g = lane >> 2, t = lane & 3;
        // ldmatrix.x4: lane l addresses row (l & 7) of matrix (l >> 3): A rows 0-7 / 8-15, k 0-7 / 8-15
        int arow = (lane & 7) + 8 * ((lane >> 3) & 1);
        if (nseg * R <= 8) arow &= 7;                        // a single row per piece: A rows 8..15 are not used
        const int a_r = arow / nseg, a_sg = arow % nseg;     // A row i is (row i / nseg, segment i % nseg)
        const uint32_t kstep_bytes = (uint32_t)nseg * 32u;
        const uint32_t lane_off = (uint32_t)a_sg * 32u + (uint32_t)(lane >> 4) * 16u;
        // B operand: column g is segment g of the activations
        const bool bval = g < nseg;
        const uint32_t* xb = reinterpret_cast<const uint32_t*>(xs) + (bval ? g : 0) * 8 + t;
        const int xstep = nseg * 8;                          // 32-bit words per k-step
        // which accumulator element of this lane is a useful output, if any
        const int slo = g % nseg, shi = (g + 8) % nseg;
        const bool take_lo = (slo >> 1) == t;
        const bool take_hi = nseg * R > 8 && (shi >> 1) == t;
        float* scr = scratch + warp * 16;
        const unsigned int p0 = pcount;
        pcount += (unsigned)s.np;
        bool ok = alive;                  // this warp still follows the ring protocol
        int j = (int)((warp - (p0 & 15u)) & 15u);            // this warp's first piece of the phase
        for (; j < s.np; j += kMegaConsumerWarps) {
            const uint32_t par = ((p0 + (unsigned)j) >> 4) & 1u;      // the stage's fillings alternate parity
            const long long tw0 = a.ts ? clock64() : 0;
            if (ok && !mega_wait(&full[warp], par, &dead, &a.sync->abort)) {
                ok = false;
                dead = 1;
                if (!ld_relaxed_gpu(&a.sync->abort)) mega_fail(a.sync, a.status, 3u, blockIdx.x, p0 + (unsigned)j, (unsigned)warp);
            }
            const long long tw1 = a.ts ? clock64() : 0;
            if (!ok) continue;
            const int blk = j / F, f = j - blk * F;
            const int jr = gateup ? (blk >> 1) : blk;
            const int nrows = min(R, s.cnt - jr * R);
            float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t addr = my_stage + (uint32_t)min(a_r, nrows - 1) * rstride + lane_off;
            const uint32_t* xp = xb + f * (Kf >> 1);
            int ks = 0;
            for (; ks + 4 <= ksteps; ks += 4, addr += 4u * kstep_bytes, xp += 4 * xstep) {
                uint32_t w[4][4], b[4][2];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w[q][0]), "=r"(w[q][1]), "=r"(w[q][2]), "=r"(w[q][3])
                                 : "r"(addr + kstep_bytes * q));
                    b[q][0] = bval ? xp[q * xstep] : 0u;
                    b[q][1] = bval ? xp[q * xstep + 4] : 0u;
                }
                mma_bf16_16816(c0, w[0][0], w[0][1], w[0][2], w[0][3], b[0][0], b[0][1]);
                mma_bf16_16816(c1, w[1][0], w[1][1], w[1][2], w[1][3], b[1][0], b[1][1]);
                mma_bf16_16816(c0, w[2][0], w[2][1], w[2][2], w[2][3], b[2][0], b[2][1]);
                mma_bf16_16816(c1, w[3][0], w[3][1], w[3][2], w[3][3], b[3][0], b[3][1]);
            }
            for (; ks < ksteps; ++ks, addr += kstep_bytes, xp += xstep) {
                uint32_t w0, w1, w2, w3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                             : "r"(addr));
                const uint32_t b0 = bval ? xp[0] : 0u, b1 = bval ? xp[4] : 0u;
                mma_bf16_16816(c0, w0, w1, w2, w3, b0, b1);
            }
            // accumulator layout: [0] (row g, col 2t)  [1] (g, 2t+1)  [2] (g+8, 2t)  [3] (g+8, 2t+1)
            if (take_lo) scr[g] = (slo & 1) ? c0[1] + c1[1] : c0[0] + c1[0];
            if (take_hi) scr[g + 8] = (shi & 1) ? c0[3] + c1[3] : c0[2] + c1[2];
            __syncwarp();
            // the accumulators depend on every ldmatrix of the piece: the stage can go back now
            if (lane == 0) mbar_arrive(&empty[warp]);
            if (lane < nrows) {
                float tot = 0.0f;
                for (int sg = 0; sg < nseg; ++sg) tot += scr[lane * nseg + sg];
                const int rloc = jr * R + lane;
                slots[(gateup ? 2 * rloc + (blk & 1) : rloc) * F + f] = tot;
            }
            __syncwarp();
            if (a.ts) { dbg_wait += tw1 - tw0; dbg_work += clock64() - tw1; }
        }
        cons_sync();
        alive = !dead;
    };
    auto row_total = [&](int rc, int F) -> float {           // the fractions of a row, in order
        float tot = slots[rc * F];
        for (int f = 1; f < F; ++f) tot += slots[rc * F + f];
        return tot;
    };
    auto store_rows = [&](const MegaShare s, float* out) {
        for (int r = tid; r < s.cnt; r += kMegaConsumers) out[s.r0 + r] = row_total(r, s.F);
    };
    // xs = bf16(in[0..K))   (K a multiple of 4; `in` was written by other CTAs before the last grid barrier)
    auto load_plain = [&](const float* in, int K) {
        const float4* in4 = reinterpret_cast<const float4*>(in);
        uint2* x2 = reinterpret_cast<uint2*>(xs);
        const int n4 = K >> 2;
        for (int i0 = 0; i0 < n4; i0 += 4 * kMegaConsumers) {
            float4 v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int i = i0 + q * kMegaConsumers + tid;
                v[q] = (i < n4) ? __ldcg(in4 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int i = i0 + q * kMegaConsumers + tid;
                if (i < n4)
                    x2[i] = make_uint2(f32_to_bf16_bits(v[q].x) | (f32_to_bf16_bits(v[q].y) << 16),
                                       f32_to_bf16_bits(v[q].z) | (f32_to_bf16_bits(v[q].w) << 16));
            }
        }
        cons_sync();
    };
    // h = (h + rmsnorm(raw) * w_post) * scalar   (raw == null: h unchanged);  xs = bf16(rmsnorm(h) * w_norm)
    auto load_norm = [&](const float* raw, const float* w_post, float scalar, const float* w_norm) {
        float hv[kMegaMaxJ], wn[kMegaMaxJ];
        // model constants first: their (cold) loads overlap the loads of the projection output
#pragma unroll
        for (int j = 0; j < kMegaMaxJ; ++j) {
            const int i = tid + j * kMegaConsumers;
            wn[j] = (i < H) ? __ldg(w_norm + i) : 0.0f;
        }
        if (raw != nullptr) {
            float t[kMegaMaxJ], wp[kMegaMaxJ];
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < kMegaMaxJ; ++j) {
                const int i = tid + j * kMegaConsumers;
                wp[j] = (i < H) ? __ldg(w_post + i) : 0.0f;
                t[j] = (i < H) ? __ldcg(raw + i) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < kMegaMaxJ; ++j) ss += t[j] * t[j];
            ss = cons_sum(ss, red);
            const float r = 1.0f / sqrtf(ss / (float)H + a.eps);
#pragma unroll
            for (int j = 0; j < kMegaMaxJ; ++j) {
                const int i = tid + j * kMegaConsumers;
                hv[j] = (i < H) ? (h_s[i] + t[j] * r * wp[j]) * scalar : 0.0f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < kMegaMaxJ; ++j) {
                const int i = tid + j * kMegaConsumers;
                hv[j] = (i < H) ? h_s[i] : 0.0f;
            }
        }
        float ss2 = 0.0f;
#pragma unroll
        for (int j = 0; j < kMegaMaxJ; ++j) ss2 += hv[j] * hv[j];
        ss2 = cons_sum(ss2, red);
        const float r2 = 1.0f / sqrtf(ss2 / (float)H + a.eps);
#pragma unroll
        for (int j = 0; j < kMegaMaxJ; ++j) {
            const int i = tid + j * kMegaConsumers;
            if (i < H) {
                h_s[i] = hv[j];
                xs[i] = (uint16_t)f32_to_bf16_bits(hv[j] * r2 * wn[j]);
            }
        }
        cons_sync();
    };
    // pull the norm vectors of a coming prologue towards the SM while the current phase still runs
    auto warm = [&](const float* w) {
        if (w != nullptr)
            for (int i = tid * 32; i < H; i += kMegaConsumers * 32) prefetch_l2(w + i);
    };

    // the embedding row opens the residual stream (kernel_module.rs:1272-1285)
    {
        uint32_t tok = a.tokens[0];
        if (tok == kInactiveToken) tok = 0;
        for (int i = tid; i < H; i += kMegaConsumers)
            h_s[i] = __uint_as_float((uint32_t)a.embed[(size_t)tok * H + i] << 16) * a.embed_scale;
        cons_sync();
    }

    int n_stamp = 0;
    auto mark = [&]() {
        if (a.ts != nullptr && blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            a.ts[n_stamp] = t;
        }
        ++n_stamp;
    };

    AttnArgs at{};
    at.qkv = a.qkv_raw;
    at.qkv_n = a.qkv_n;
    at.qkv_splits = 1;
    at.B = 1;
    at.Nq = a.Nq;
    at.Nkv = a.Nkv;
    at.eps = a.eps;
    at.pos = a.pos;
    at.tokens = a.tokens;
    at.page_tokens = a.page_tokens;
    at.min_split = a.min_split;
    at.part = a.part;
    at.ticket = a.ticket;
    at.out = a.attn_out;

    for (int l = 0; l < a.L; ++l) {
        const MegaLayer& ly = a.layers[l];
        // ---- input norm + QKV (closes the previous layer's MLP block first) ----
        mark();
        if (l == 0) load_norm(nullptr, nullptr, 1.0f, ly.input_ln);
        else load_norm(a.down_raw, a.layers[l - 1].post_ff_ln, a.layers[l - 1].layer_scalar, ly.input_ln);
        mark();
        warm(ly.post_attn_ln);
        warm(ly.pre_ff_ln);
        consume(H, sh0, false);
        if (alive) store_rows(sh0, a.qkv_raw);
        mark();
        grid_barrier();
        mark();
        // ---- attention: (split, kv head) units dealt to the CTAs ----
        if (alive) {
            at.q_norm = ly.q_norm;
            at.k_norm = ly.k_norm;
            at.inv_freq = ly.inv_freq;
            at.rotary_half = ly.rotary_half;
            at.kpool = a.kv[l].k;
            at.vpool = a.kv[l].v;
            at.page_table = ly.sliding ? a.pt_slide : a.pt_full;
            at.pages_per_seq = ly.sliding ? a.pps_slide : a.pps_full;
            at.cap = ly.sliding ? a.cap_slide : a.cap_full;
            at.n_splits = ly.sliding ? a.splits_slide : a.splits_full;
            at.ts = a.ts ? a.ts + 15 * a.L + 2 + 4 * l : nullptr;
            at.ts_mid = nullptr;
            const int units = at.n_splits * a.Nkv;
            for (int u = blockIdx.x; u < units; u += gridDim.x) {
                attn_cta<KT, D, G, false, false, false>(at, reinterpret_cast<float*>(xreg), u % at.n_splits, u / at.n_splits, 0,
                                                 kMegaConsumers, BarFirst512{});
                cons_sync();
            }
        }
        mark();
        grid_barrier();
        mark();
        // ---- O projection ----
        load_plain(a.attn_out, a.Nq * D);
        mark();
        consume(a.Nq * D, sh1, false);
        if (alive) store_rows(sh1, a.o_raw);
        mark();
        grid_barrier();
        mark();
        // ---- post-attention norm + residual, pre-FF norm, gate/up + GeGLU ----
        load_norm(a.o_raw, ly.post_attn_ln, 1.0f, ly.pre_ff_ln);
        mark();
        consume(H, sh2, true);
        if (alive) {
            for (int r = tid; r < sh2.cnt; r += kMegaConsumers)
                a.gu_raw[sh2.r0 + r] = gelu_mul(row_total(2 * r, sh2.F), row_total(2 * r + 1, sh2.F));
        }
        mark();
        grid_barrier();
        mark();
        // ---- down projection ----
        load_plain(a.gu_raw, a.I);
        mark();
        warm(ly.post_ff_ln);
        if (l + 1 < a.L) warm(a.layers[l + 1].input_ln);
        consume(a.I, sh3, false);
        if (alive) store_rows(sh3, a.down_raw);
        mark();
        grid_barrier();
        mark();
    }
    if (a.ts != nullptr && blockIdx.x == 0 && tid == 0) {
        a.ts[15 * a.L] = (unsigned long long)dbg_wait;
        a.ts[15 * a.L + 1] = (unsigned long long)dbg_work;
    }
    // the LM head kernel applies the last pending update itself: it needs the residual stream as it stands
    if (blockIdx.x == 0 && alive)
        for (int i = tid; i < H; i += kMegaConsumers) a.h_out[i] = h_s[i];
}

}  // namespace oxg4
