// Weight-streaming projection kernel for BF16 weights, 1..16 activation rows per pass.
//
// Same prologues and epilogues as gemv.cuh (see there for the reference launches it replaces),
// but the contraction runs on the tensor cores so that the kernel stays HBM-bound instead of
// issue-bound: the BF16 -> f32 widening and the multiply-adds of the SIMT version cost about 30
// instructions per 16-byte weight load, this version 4.
//
// mma.sync.m16n8k16 (BF16 x BF16 -> f32) with the roles swapped: the activations are the 16-row A
// operand (batch rows; unused rows are zero registers), eight weight rows are the B operand. A
// lane (g = lane / 4, t = lane % 4) loads 16 contiguous bytes of weight row g at column
// 32 * chunk + 8 * t; the two halves of that load are the B fragments of two MMAs. The k positions
// inside a fragment are permuted, which is harmless because x is fetched with the same permutation.
// Products of BF16 values are exact in f32; accumulation is f32.
//
// Work split. Every CTA owns a contiguous block of output rows (EPI_GATEUP: (gate_i, up_i) pairs as
// 2*I virtual rows). The 16 warps split the COLUMNS: warp w takes the 32-column chunks w, w+16, ...
// and walks all rows of the block in groups of eight, 64 rows (eight groups) at a time, so every
// warp streams the same number of bytes whatever the block's height. The sixteen partial sums of a
// row meet in shared memory and are added in warp order (deterministic). Eight 16-byte loads per
// lane stay in flight: each weight register is refilled for the next chunk right after its MMAs.
//
// HBM-bound: bytes per launch = N * K * 2.
#pragma once
#include "gemv.cuh"

namespace oxg4 {

// rows of a CTA's block handled between two combines: 64 with up to 8 activation rows, 32 with up to
// 16 (twice the accumulators per row group, so half the groups to stay inside 128 registers)
__host__ __device__ constexpr int mma_rows_per_pass(int mb) { return mb == 16 ? 32 : 64; }

// Row stride (elements) of the activation rows in shared memory: K padded so that consecutive rows
// start 64 bytes apart modulo 128; the eight lanes of an LDS.128 phase (two batch rows x four column
// groups) then hit eight different 16-byte bank groups instead of colliding.
__host__ __device__ inline int mma_x_stride(int K) { return K + (((64 - (K * 2) % 128) + 128) % 128) / 2; }

DEVINL void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One pass over up to 64 rows (NG2 row groups of eight, NG2 a power of two) of a CTA's block for the
// 32-column chunks of one warp. The ring `w` always holds the next eight (chunk, group) loads: with
// fewer than eight row groups it reaches 8 / NG2 chunks ahead, so short blocks (few rows per CTA)
// keep as many bytes in flight as tall ones. Writes the warp's partial sums to `pc`.
template <int MB, int NG2>
DEVINL void mma_pass(const uint16_t* xs, int XS, int K, int nb, int nchunk, int warp, int g, int t,
                     const uint16_t* base, size_t gstride, int rows_left, uint4 (&w)[8], bool preloaded,
                     const uint16_t* next_base, int next_rows, bool preload_next, float* pc) {
    constexpr int CA = 8 / NG2;                       // chunks held in the ring
    constexpr int NW = kGemvWarps;
    const int nmy = warp < nchunk ? (nchunk - warp + NW - 1) / NW : 0;
    auto load_w = [&](const uint16_t* b, int gi, int rows, int col) -> uint4 {
        // rows at or beyond the end of the block, and columns at or beyond K, read as zero
        if (gi * 8 + g < rows && col < K) return ldg_stream16(b + (size_t)gi * gstride + col);
        return make_uint4(0u, 0u, 0u, 0u);
    };
    if (!preloaded) {
#pragma unroll
        for (int j = 0; j < CA; ++j)
#pragma unroll
            for (int gi = 0; gi < NG2; ++gi)
                w[j * NG2 + gi] = (j < nmy) ? load_w(base, gi, rows_left, (warp + NW * j) * 32 + t * 8)
                                            : make_uint4(0u, 0u, 0u, 0u);
    }
    float acc[NG2][4];
#pragma unroll
    for (int gi = 0; gi < NG2; ++gi) acc[gi][0] = acc[gi][1] = acc[gi][2] = acc[gi][3] = 0.0f;
    for (int ci = 0; ci < nmy; ci += CA) {
#pragma unroll
        for (int j = 0; j < CA; ++j) {
            const int i = ci + j;
            if (i < nmy) {
                const int col = (warp + NW * i) * 32 + t * 8;
                uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = make_uint4(0u, 0u, 0u, 0u);
                if (col < K) {
                    if (g < nb) xa = *reinterpret_cast<const uint4*>(xs + (size_t)g * XS + col);
                    if (MB == 16 && g + 8 < nb) xb = *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * XS + col);
                }
                const int in = i + CA;                 // the chunk that takes over this ring position
                const bool more = in < nmy;
                // with a full ring of groups (CA == 1) the first chunk of the next pass follows directly
                const bool cross = (CA == 1) && !more && preload_next;
                const int coln = (warp + NW * (more ? in : 0)) * 32 + t * 8;
                const uint16_t* nbase = more ? base : next_base;
                const int nrows = more ? rows_left : (cross ? next_rows : 0);
#pragma unroll
                for (int gi = 0; gi < NG2; ++gi) {
                    uint4& wr = w[j * NG2 + gi];
                    mma_bf16_16816(acc[gi], xa.x, xb.x, xa.y, xb.y, wr.x, wr.y);
                    mma_bf16_16816(acc[gi], xa.z, xb.z, xa.w, xb.w, wr.z, wr.w);
                    wr = load_w(nbase, gi, nrows, coln);
                }
            }
        }
    }
#pragma unroll
    for (int gi = 0; gi < NG2; ++gi) {
        const int rl = gi * 8 + 2 * t;
        if (g < nb) {
            pc[((size_t)rl * NW + warp) * nb + g] = acc[gi][0];
            pc[((size_t)(rl + 1) * NW + warp) * nb + g] = acc[gi][1];
        }
        if (MB == 16 && g + 8 < nb) {
            pc[((size_t)rl * NW + warp) * nb + g + 8] = acc[gi][2];
            pc[((size_t)(rl + 1) * NW + warp) * nb + g + 8] = acc[gi][3];
        }
    }
}

// MB = 8: up to 8 activation rows per pass (only the m < 8 half of the accumulator is kept);
// MB = 16: up to 16.
template <int MB, int PRO, int EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_mma_kernel(const GemvArgs a) {
    typedef uint16_t WT;
    constexpr int NW = kGemvWarps;
    constexpr int RP = mma_rows_per_pass(MB);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int b0 = blockIdx.y * a.bpp;
    const int nb = min(a.bpp, a.B - b0);              // <= MB
    const int XS = mma_x_stride(K);
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);                              // [nb][XS]
    float* red = reinterpret_cast<float*>(smem_raw + (((size_t)nb * XS * 2 + 15) & ~(size_t)15));   // [32]
    float* pieces = red + 32;                           // [2][64 rows][16 warps][nb]
    const size_t row_bytes = (size_t)K * 2;

    auto row_ptr = [&](int r) -> const WT* {
        if constexpr (EPI == EPI_GATEUP)
            return (const WT*)((r & 1) ? a.W1 : a.W0) + (size_t)(r >> 1) * K;
        else
            return (const WT*)a.W0 + (size_t)r * K;
    };

    int row_first = 0, rows_cta = 0;
    if constexpr (EPI == EPI_GATEUP) {
        block_range(a.N / 2, gridDim.x, blockIdx.x, row_first, rows_cta);
        row_first *= 2;
        rows_cta *= 2;
    } else {
        block_range(a.N, gridDim.x, blockIdx.x, row_first, rows_cta);
    }

    // ---- pre-dependency section: nothing here reads what the previous kernel wrote ----
    if (tid < 8 && rows_cta > 0) {
        constexpr size_t PIECE = 32 * 1024;
        const size_t cap = (size_t)a.pf_cap_kb * 1024;
        if constexpr (EPI == EPI_GATEUP) {
            const size_t slab = min((size_t)(rows_cta / 2) * row_bytes, cap / 2);
            const char* g0 = (const char*)a.W0 + (size_t)(row_first / 2) * row_bytes;
            const char* u0 = (const char*)a.W1 + (size_t)(row_first / 2) * row_bytes;
            for (size_t off = (size_t)(tid >> 1) * PIECE; off < slab; off += 4 * PIECE)
                prefetch_l2_bulk(((tid & 1) ? u0 : g0) + off, min(PIECE, slab - off));
        } else {
            const size_t slab = min((size_t)rows_cta * row_bytes, cap);
            const char* s0 = (const char*)a.W0 + (size_t)row_first * row_bytes;
            for (size_t off = (size_t)tid * PIECE; off < slab; off += 8 * PIECE)
                prefetch_l2_bulk(s0 + off, min(PIECE, slab - off));
        }
    }
    float wpost[kGemvMaxJ], wnorm[kGemvMaxJ];
    if constexpr (PRO == PRO_NORM) {
#pragma unroll
        for (int j = 0; j < kGemvMaxJ; ++j) {
            const int i = tid + j * kGemvThreads;
            wnorm[j] = (i < K) ? a.w_norm[i] : 0.0f;
            wpost[j] = (i < K && a.w_post) ? a.w_post[i] : 0.0f;
        }
    }
    stamp(a.ts, 0);
    pdl_wait();
    stamp(a.ts, 1);

    // ---- prologue: x[nb][K] (BF16) in shared memory ----
    if constexpr (PRO == PRO_PLAIN) {
        // four values per thread and step (K is a multiple of 8)
        const int k4 = K >> 2;
        for (int idx = tid; idx < nb * k4; idx += kGemvThreads) {
            const int b = idx / k4, i = (idx - b * k4) << 2;
            const float4 v = *reinterpret_cast<const float4*>(a.in + (size_t)(b0 + b) * K + i);
            uint2 pk;
            pk.x = f32_to_bf16_bits(v.x) | (f32_to_bf16_bits(v.y) << 16);
            pk.y = f32_to_bf16_bits(v.z) | (f32_to_bf16_bits(v.w) << 16);
            *reinterpret_cast<uint2*>(xs + (size_t)b * XS + i) = pk;
        }
    } else if (nb > 4) {
        // many activation rows: one warp per row, so no block-wide barrier is paid per row
        const bool writer = (blockIdx.x == 0);
        const int k4 = K >> 2;
        for (int b = warp; b < nb; b += NW) {
            const size_t ro = (size_t)(b0 + b) * K;
            uint32_t tok = 0;
            if (a.embed != nullptr) {
                tok = a.tokens[b0 + b];
                if (tok == kInactiveToken) tok = 0;
            }
            float r = 0.0f;
            if (a.embed == nullptr && a.raw != nullptr) {
                float ss = 0.0f;
                for (int i4 = lane; i4 < k4; i4 += 32) {
                    const float4 t4 = *reinterpret_cast<const float4*>(a.raw + ro + 4 * i4);
                    ss += t4.x * t4.x + t4.y * t4.y + t4.z * t4.z + t4.w * t4.w;
                }
                ss = warp_sum(ss);
                r = 1.0f / sqrtf(ss / (float)K + a.eps);
            }
            auto hidden4 = [&](int i4) -> float4 {
                float4 h;
                if (a.embed != nullptr) {
                    const uint2 e = *reinterpret_cast<const uint2*>((const uint16_t*)a.embed + (size_t)tok * K + 4 * i4);
                    h = make_float4(bf16lo(e.x) * a.embed_scale, bf16hi(e.x) * a.embed_scale,
                                    bf16lo(e.y) * a.embed_scale, bf16hi(e.y) * a.embed_scale);
                } else {
                    h = *reinterpret_cast<const float4*>(a.h_in + ro + 4 * i4);
                    if (a.raw != nullptr) {
                        const float4 t4 = *reinterpret_cast<const float4*>(a.raw + ro + 4 * i4);
                        const float4 w4 = *reinterpret_cast<const float4*>(a.w_post + 4 * i4);
                        h.x = (h.x + t4.x * r * w4.x) * a.scalar;
                        h.y = (h.y + t4.y * r * w4.y) * a.scalar;
                        h.z = (h.z + t4.z * r * w4.z) * a.scalar;
                        h.w = (h.w + t4.w * r * w4.w) * a.scalar;
                    }
                }
                return h;
            };
            float ss2 = 0.0f;
            for (int i4 = lane; i4 < k4; i4 += 32) {
                const float4 h = hidden4(i4);
                if (writer) *reinterpret_cast<float4*>(a.h_out + ro + 4 * i4) = h;
                ss2 += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
            }
            ss2 = warp_sum(ss2);
            const float r2 = 1.0f / sqrtf(ss2 / (float)K + a.eps);
            for (int i4 = lane; i4 < k4; i4 += 32) {
                const float4 h = hidden4(i4);
                const float4 w4 = *reinterpret_cast<const float4*>(a.w_norm + 4 * i4);
                uint2 pk;
                pk.x = f32_to_bf16_bits(h.x * r2 * w4.x) | (f32_to_bf16_bits(h.y * r2 * w4.y) << 16);
                pk.y = f32_to_bf16_bits(h.z * r2 * w4.z) | (f32_to_bf16_bits(h.w * r2 * w4.w) << 16);
                *reinterpret_cast<uint2*>(xs + (size_t)b * XS + 4 * i4) = pk;
            }
        }
    } else {
        const bool writer = (blockIdx.x == 0);
        for (int b = 0; b < nb; ++b) {
            float hv[kGemvMaxJ];
            float ss[1];
            if (a.embed != nullptr) {
                uint32_t tok = a.tokens[b0 + b];
                if (tok == kInactiveToken) tok = 0;
#pragma unroll
                for (int j = 0; j < kGemvMaxJ; ++j) {
                    const int i = tid + j * kGemvThreads;
                    hv[j] = (i < K) ? WTraits<uint16_t>::elem(a.embed, (size_t)tok * K + i) * a.embed_scale : 0.0f;
                }
            } else if (a.raw != nullptr) {
                float tv[kGemvMaxJ];
                ss[0] = 0.0f;
#pragma unroll
                for (int j = 0; j < kGemvMaxJ; ++j) {
                    const int i = tid + j * kGemvThreads;
                    tv[j] = (i < K) ? a.raw[(size_t)(b0 + b) * K + i] : 0.0f;
                    hv[j] = (i < K) ? a.h_in[(size_t)(b0 + b) * K + i] : 0.0f;
                    ss[0] += tv[j] * tv[j];
                }
                block_sum<1>(ss, red);
                const float r = 1.0f / sqrtf(ss[0] / (float)K + a.eps);
#pragma unroll
                for (int j = 0; j < kGemvMaxJ; ++j) hv[j] = (hv[j] + tv[j] * r * wpost[j]) * a.scalar;
            } else {
#pragma unroll
                for (int j = 0; j < kGemvMaxJ; ++j) {
                    const int i = tid + j * kGemvThreads;
                    hv[j] = (i < K) ? a.h_in[(size_t)(b0 + b) * K + i] : 0.0f;
                }
            }
            ss[0] = 0.0f;
#pragma unroll
            for (int j = 0; j < kGemvMaxJ; ++j) {
                const int i = tid + j * kGemvThreads;
                if (i < K) {
                    if (writer) a.h_out[(size_t)(b0 + b) * K + i] = hv[j];
                    ss[0] += hv[j] * hv[j];
                }
            }
            block_sum<1>(ss, red);
            const float r2 = 1.0f / sqrtf(ss[0] / (float)K + a.eps);
#pragma unroll
            for (int j = 0; j < kGemvMaxJ; ++j) {
                const int i = tid + j * kGemvThreads;
                if (i < K) xs[(size_t)b * XS + i] = (uint16_t)f32_to_bf16_bits(hv[j] * r2 * wnorm[j]);
            }
        }
    }
    __syncthreads();
    pdl_launch();
    stamp(a.ts, 2);

    // ---- body ----
    const int nchunk = (K + 31) >> 5;
    const size_t gstride = (size_t)((EPI == EPI_GATEUP) ? 4 : 8) * K;     // elements between row groups
    Cand best[2];
    best[0].s = best[1].s = -INFINITY;
    best[0].i = best[1].i = 0xffffffffu;

    uint4 w[8];
    int pass = 0;
    bool preloaded = false;
    const WT* base = (rows_cta > 0) ? row_ptr(row_first + g) : (const WT*)a.W0;
    for (int r0 = 0; r0 < rows_cta; r0 += RP, ++pass) {
        const int rows_left = rows_cta - r0;
        const int r1 = r0 + RP;
        const WT* next_base = (r1 < rows_cta) ? row_ptr(row_first + r1 + g) : base;
        const int next_rows = max(0, rows_cta - r1);
        const bool next_full = next_rows >= RP;
        float* pc = pieces + (size_t)(pass & 1) * RP * NW * nb;
        const int ng = (min(rows_left, RP) + 7) >> 3;
        if (RP == 64 && ng > 4) {
            mma_pass<MB, (RP == 64 ? 8 : 4)>(xs, XS, K, nb, nchunk, warp, g, t, base, gstride, rows_left, w, preloaded,
                                             next_base, next_rows, next_full, pc);
            preloaded = next_full;
        } else if (ng > 2) {
            mma_pass<MB, 4>(xs, XS, K, nb, nchunk, warp, g, t, base, gstride, rows_left, w, false, next_base, 0, false, pc);
        } else if (ng > 1) {
            mma_pass<MB, 2>(xs, XS, K, nb, nchunk, warp, g, t, base, gstride, rows_left, w, false, next_base, 0, false, pc);
        } else {
            mma_pass<MB, 1>(xs, XS, K, nb, nchunk, warp, g, t, base, gstride, rows_left, w, false, next_base, 0, false, pc);
        }
        base = next_base;
        // rows of the pass that no group produced must not be read by the combine: none are, it stops
        // at rows_here below
        __syncthreads();
        // combine in warp order and apply the epilogue
        const int rows_here = min(RP, rows_left);
        auto total = [&](int rl, int b) -> float {
            float s = 0.0f;
#pragma unroll
            for (int ww = 0; ww < NW; ++ww) s += pc[((size_t)rl * NW + ww) * nb + b];
            return s;
        };
        if constexpr (EPI == EPI_STORE) {
            for (int idx = tid; idx < rows_here * nb; idx += kGemvThreads) {
                const int rl = idx % rows_here, b = idx / rows_here;
                a.out[(size_t)(b0 + b) * a.N + row_first + r0 + rl] = total(rl, b);
            }
        } else if constexpr (EPI == EPI_GATEUP) {
            const int pairs = rows_here / 2;
            for (int idx = tid; idx < pairs * nb; idx += kGemvThreads) {
                const int pl = idx % pairs, b = idx / pairs;
                a.out[(size_t)(b0 + b) * (a.N / 2) + (row_first + r0) / 2 + pl] =
                    gelu_mul(total(2 * pl, b), total(2 * pl + 1, b));
            }
        } else {
            // thread -> (row tid % RP, batch rows tid / RP (+ 8 when RP == 64))
            constexpr int BH = kGemvThreads / RP;
            const int rl = tid & (RP - 1);
#pragma unroll
            for (int h = 0; h < 16 / BH; ++h) {
                const int b = tid / RP + BH * h;
                if (rl < rows_here && b < nb) {
                    const float v = total(rl, b);
                    const int vid = a.row_offset + row_first + r0 + rl;
                    const size_t gb = (size_t)(b0 + b) * a.n_total;
                    if (a.out) a.out[gb + vid] = v;
                    float s = v;      // kernel_module.rs:2008-2016
                    if (a.seen && a.penalty > 1.0f && a.seen[gb + vid]) s = s >= 0.0f ? s / a.penalty : s * a.penalty;
                    const Cand cnd{s, (uint32_t)vid};
                    if (s == s && s > -INFINITY && cand_better(cnd, best[h])) best[h] = cnd;
                }
            }
        }
        // no second barrier: the next pass writes the other half of `pieces`
    }

    if constexpr (EPI == EPI_LOGITS) {
        __shared__ unsigned int s_last;
        __syncthreads();
        Cand* wc = reinterpret_cast<Cand*>(pieces);        // [16 batch rows][RP]
        constexpr int BH = kGemvThreads / RP;
#pragma unroll
        for (int h = 0; h < 16 / BH; ++h) {
            const int b = tid / RP + BH * h;
            wc[b * RP + (tid & (RP - 1))] = best[h];
        }
        __syncthreads();
        if (warp < nb) {
            Cand c = wc[warp * RP + lane];
            if (RP == 64) {
                const Cand c2 = wc[warp * RP + 32 + lane];
                if (cand_better(c2, c)) c = c2;
            }
            c = warp_best(c);
            if (lane == 0) a.blk_best[(size_t)(b0 + warp) * gridDim.x + blockIdx.x] = c;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(&a.ticket[blockIdx.y], 1u) == gridDim.x - 1) ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int b = warp; b < nb; b += NW) {
                Cand c{-INFINITY, 0xffffffffu};
                for (int gi = lane; gi < (int)gridDim.x; gi += 32) {
                    const Cand* src = &a.blk_best[(size_t)(b0 + b) * gridDim.x + gi];
                    Cand o;
                    o.s = __ldcg(&src->s);
                    o.i = __ldcg(&src->i);
                    if (cand_better(o, c)) c = o;
                }
                c = warp_best(c);
                if (lane == 0) {
                    a.best_ids[b0 + b] = (c.i == 0xffffffffu) ? 0u : c.i;
                    a.best_scores[b0 + b] = c.s;
                }
            }
            if (tid == 0) a.ticket[blockIdx.y] = 0u;
        }
    }
    stamp(a.ts, 3);
}

}  // namespace oxg4
