// Weight-streaming projection kernel for small batches (1..4 activation rows per pass).
//
// One launch covers what the reference spreads over rms_norm[_bf16] + f32_to_bf16 + cublasGemmEx
// (+ slice / gelu_mul / add / mul_bf16_scalar) launches — crates/oxide-torch-models/src/
// gemma4_cuda/decode.rs:4-21,43-174 and tensor_ops.rs:61-157:
//   prologue  PRO_NORM : finish the previous block's residual update
//                        h = (h_in + rmsnorm(previous projection, w_post)) * layer_scalar
//                        (or h = embedding row * sqrt(H) for the first layer), store h once, then
//                        x = bf16(rmsnorm(h, w_norm))
//             PRO_PLAIN: x = bf16(in)
//   body      out[n] = sum_k x[k] * W[n,k], f32 accumulate, 16-byte coalesced streaming loads,
//             warp-shuffle reductions
//   epilogue  EPI_STORE : out[b, n]
//             EPI_GATEUP: out[b, i] = gelu_tanh(gate_i . x) * (up_i . x)
//             EPI_LOGITS: optional logits store + running arg-max with repetition penalty
//
// Work split (EPI_STORE / EPI_GATEUP). Every CTA owns a contiguous block of output rows (for
// EPI_GATEUP a block of (gate_i, up_i) pairs, streamed as 2*I virtual rows). The block is cut into
// 512-byte chunks (one 16-byte load per lane) and the chunks are dealt out as equal contiguous runs
// to the 16 warps, so all warps stream the same number of bytes whatever the matrix shape. A run
// that ends inside a row leaves a partial sum; the pieces of a row meet in shared memory and are
// added in a fixed order, which keeps the split-K reduction deterministic without atomics.
//
// The kernel is HBM-bound: bytes per launch = N * K * sizeof(weight).
#pragma once
#include "common.cuh"

namespace oxg4 {

enum { PRO_PLAIN = 0, PRO_NORM = 1 };
enum { EPI_STORE = 0, EPI_GATEUP = 1, EPI_LOGITS = 2 };

constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kSimtThreads = 1024;     // SIMT kernel: more warps, fewer registers, same bytes in flight per warp
constexpr int kSimtWarps = kSimtThreads / 32;
constexpr int kSimtMaxJ = 6;         // PRO_NORM keeps hidden/1024 values per thread: hidden <= 6144
constexpr int kGemvMaxJ = 11;        // PRO_NORM keeps hidden/512 values per thread: hidden <= 5632

struct GemvArgs {
    const void* W0;          // [N, K] row-major (EPI_GATEUP: gate)
    const void* W1;          // EPI_GATEUP: up projection
    int N, K;                // rows (EPI_GATEUP: virtual rows = 2 * intermediate), columns
    int cpr;                 // 512-byte chunks per row
    int slots;               // most pieces a row is cut into inside one CTA
    int B;                   // activation rows in the step
    int bpp;                 // activation rows per pass (tensor-core kernel: grid.y = ceil(B / bpp))
    // PRO_PLAIN
    const float* in;         // [B, K]
    // PRO_NORM (K == hidden size)
    const float* h_in;       // [B, K] residual stream before the pending update (unused with embed)
    float* h_out;            // [B, K] residual stream after it (written by block 0)
    const float* raw;        // [B, K] previous projection output still to be normed and added, or null
    const float* w_post;     // norm weight applied to `raw`
    float scalar;            // layer_scalar of the layer that just ended (1.0 otherwise)
    const float* w_norm;     // norm weight producing x
    const void* embed;       // embedding table [V, K] (same element type as W0), or null
    const uint32_t* tokens;  // [B]
    float embed_scale;
    float eps;
    // weights of later kernels to pull into L2 while this kernel runs (each CTA takes a slice)
    const void* pf_ptr[2];
    unsigned long long pf_bytes[2];
    int pf_cap_kb;           // bytes of its own weight block a CTA prefetches into L2 before the dependency wait (KiB)
    unsigned long long* ts;  // optional timeline slots of this launch (4 entries) or null
    // epilogue
    float* out;              // STORE: [B, N]; GATEUP: [B, N/2]; LOGITS: [B, n_total] or null
    const uint8_t* seen;     // LOGITS: [B, n_total] repetition bitmap or null
    float penalty;
    int row_offset;          // LOGITS: first vocabulary row of this rank's slice
    int n_total;             // LOGITS: full vocabulary (row stride of `out` and `seen`)
    Cand* blk_best;          // LOGITS: [B, gridDim.x]
    unsigned int* ticket;    // LOGITS: one counter per batch chunk (gridDim.y)
    uint32_t* best_ids;      // LOGITS: [B]
    float* best_scores;      // LOGITS: [B]
};

template <typename WT> struct WTraits;
template <> struct WTraits<float> {
    static constexpr int EPL = 4;                     // elements per 16-byte load
    typedef float XT;
    static DEVINL float elem(const void* base, size_t idx) { return ((const float*)base)[idx]; }
    static DEVINL void store_x(XT* p, float v) { *p = v; }          // f32 mode: no rounding
};
template <> struct WTraits<uint16_t> {
    static constexpr int EPL = 8;
    typedef uint16_t XT;
    static DEVINL float elem(const void* base, size_t idx) {
        return __uint_as_float((uint32_t)((const uint16_t*)base)[idx] << 16);
    }
    static DEVINL void store_x(XT* p, float v) { *p = (uint16_t)f32_to_bf16_bits(v); }
};

// acc[b] += dot(w (16 bytes of weights), x (matching activations of row b))
template <typename WT, int NB>
DEVINL void fma16(float (&acc)[NB], const uint4& w, const typename WTraits<WT>::XT* xs, int K, int k) {
    if constexpr (sizeof(WT) == 2) {
        const float w0 = bf16lo(w.x), w1 = bf16hi(w.x), w2 = bf16lo(w.y), w3 = bf16hi(w.y);
        const float w4 = bf16lo(w.z), w5 = bf16hi(w.z), w6 = bf16lo(w.w), w7 = bf16hi(w.w);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const uint4 x = *reinterpret_cast<const uint4*>(xs + (size_t)b * K + k);
            float a = acc[b];
            a = fmaf(w0, bf16lo(x.x), a); a = fmaf(w1, bf16hi(x.x), a);
            a = fmaf(w2, bf16lo(x.y), a); a = fmaf(w3, bf16hi(x.y), a);
            a = fmaf(w4, bf16lo(x.z), a); a = fmaf(w5, bf16hi(x.z), a);
            a = fmaf(w6, bf16lo(x.w), a); a = fmaf(w7, bf16hi(x.w), a);
            acc[b] = a;
        }
    } else {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const float4 x = *reinterpret_cast<const float4*>(xs + (size_t)b * K + k);
            float a = acc[b];
            a = fmaf(__uint_as_float(w.x), x.x, a); a = fmaf(__uint_as_float(w.y), x.y, a);
            a = fmaf(__uint_as_float(w.z), x.z, a); a = fmaf(__uint_as_float(w.w), x.w, a);
            acc[b] = a;
        }
    }
}

// rows [first, first + count) of `total` rows dealt to `parts` CTAs as evenly as possible
DEVINL void block_range(int total, int parts, int idx, int& first, int& count) {
    const int base = total / parts, rem = total % parts;
    first = idx * base + min(idx, rem);
    count = base + (idx < rem ? 1 : 0);
}

template <typename WT, int NB, int PRO, int EPI>
__global__ void __launch_bounds__(kSimtThreads, 1) gemv_kernel(const GemvArgs a) {
    typedef WTraits<WT> T;
    typedef typename T::XT XT;
    constexpr int EPL = T::EPL;
    constexpr int STEP = 32 * EPL;                     // elements per chunk
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.K;
    XT* xs = reinterpret_cast<XT*>(smem_raw);                                        // [NB][K]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)NB * K * sizeof(XT));   // [NB*32]
    float* pieces = red + NB * 32;                     // [rows_cta][slots][NB] / Cand scratch
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, a.B - b0);
    const size_t row_bytes = (size_t)K * sizeof(WT);

    auto row_ptr = [&](int r) -> const WT* {
        if constexpr (EPI == EPI_GATEUP)
            return (const WT*)((r & 1) ? a.W1 : a.W0) + (size_t)(r >> 1) * K;
        else
            return (const WT*)a.W0 + (size_t)r * K;
    };

    // this CTA's block of (virtual) rows
    int row_first = 0, rows_cta = 0;
    if constexpr (EPI == EPI_GATEUP) {
        block_range(a.N / 2, gridDim.x, blockIdx.x, row_first, rows_cta);
        row_first *= 2;
        rows_cta *= 2;
    } else if constexpr (EPI == EPI_STORE) {
        block_range(a.N, gridDim.x, blockIdx.x, row_first, rows_cta);
    }
    const int chunks_cta = rows_cta * a.cpr;
    const int lr = max(1, (chunks_cta + kSimtWarps - 1) / kSimtWarps);   // chunks per warp run

    // ---- pre-dependency section: nothing here reads what the previous kernel wrote ----
    // warm L2 with the start of what this CTA will stream
    if constexpr (EPI == EPI_LOGITS) {
        const int U = (a.N + 1) / 2;
        const int lines_per_row = (int)((row_bytes + 127) / 128);
        for (int j = 0; j < 2 * kSimtWarps; ++j) {
            const int u = blockIdx.x + gridDim.x * j;
            if (u >= U) break;
            const char* p0 = (const char*)row_ptr(u * 2);
            const int nl = (u * 2 + 1 < a.N) ? 2 * lines_per_row : lines_per_row;   // rows are adjacent
            for (int l = tid; l < nl; l += kSimtThreads) prefetch_l2(p0 + (size_t)l * 128);
        }
    } else {
        // this CTA's own block is contiguous in memory (two slabs for gate/up): bulk L2 prefetch
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
    }
    // slices of later kernels' weights: one 32 KiB bulk prefetch per thread at most
    if (tid >= 32) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const unsigned long long total = a.pf_bytes[which];
            if (total) {
                constexpr unsigned long long PIECE = 32 * 1024;
                const unsigned long long npieces = (total + PIECE - 1) / PIECE;
                for (unsigned long long pi = blockIdx.x + (unsigned long long)gridDim.x * (tid - 32); pi < npieces;
                     pi += (unsigned long long)gridDim.x * (kSimtThreads - 32)) {
                    const unsigned long long off = pi * PIECE;
                    prefetch_l2_bulk((const char*)a.pf_ptr[which] + off, (size_t)min(PIECE, total - off));
                }
            }
        }
    }
    // norm weights are model constants: fetch them before waiting on the previous kernel
    float wpost[kSimtMaxJ], wnorm[kSimtMaxJ];
    if constexpr (PRO == PRO_NORM) {
#pragma unroll
        for (int j = 0; j < kSimtMaxJ; ++j) {
            const int i = tid + j * kSimtThreads;
            wnorm[j] = (i < K) ? a.w_norm[i] : 0.0f;
            wpost[j] = (i < K && a.w_post) ? a.w_post[i] : 0.0f;
        }
    }
    stamp(a.ts, 0);
    pdl_wait();
    stamp(a.ts, 1);

    // ---- prologue: build x[nb][K] in shared memory ----
    if constexpr (PRO == PRO_PLAIN) {
        for (int b = 0; b < nb; ++b)
            for (int i = tid; i < K; i += kSimtThreads)
                T::store_x(xs + (size_t)b * K + i, a.in[(size_t)(b0 + b) * K + i]);
    } else {
        const bool writer = (blockIdx.x == 0);
        for (int b = 0; b < nb; ++b) {
            float hv[kSimtMaxJ];
            float ss[1];
            if (a.embed != nullptr) {
                // kernel_module.rs:1272-1285: embedding row widened to f32, times sqrt(hidden)
                uint32_t tok = a.tokens[b0 + b];
                if (tok == kInactiveToken) tok = 0;
#pragma unroll
                for (int j = 0; j < kSimtMaxJ; ++j) {
                    const int i = tid + j * kSimtThreads;
                    hv[j] = (i < K) ? T::elem(a.embed, (size_t)tok * K + i) * a.embed_scale : 0.0f;
                }
            } else if (a.raw == nullptr) {
                // nothing pending: h_in already is the layer's input (layer-wise tracing)
#pragma unroll
                for (int j = 0; j < kSimtMaxJ; ++j) {
                    const int i = tid + j * kSimtThreads;
                    hv[j] = (i < K) ? a.h_in[(size_t)(b0 + b) * K + i] : 0.0f;
                }
            } else {
                float t[kSimtMaxJ];
                ss[0] = 0.0f;
#pragma unroll
                for (int j = 0; j < kSimtMaxJ; ++j) {
                    const int i = tid + j * kSimtThreads;
                    t[j] = (i < K) ? a.raw[(size_t)(b0 + b) * K + i] : 0.0f;
                    hv[j] = (i < K) ? a.h_in[(size_t)(b0 + b) * K + i] : 0.0f;
                    ss[0] += t[j] * t[j];
                }
                block_sum<1>(ss, red);
                const float r = 1.0f / sqrtf(ss[0] / (float)K + a.eps);
#pragma unroll
                for (int j = 0; j < kSimtMaxJ; ++j) hv[j] = (hv[j] + t[j] * r * wpost[j]) * a.scalar;
            }
            ss[0] = 0.0f;
#pragma unroll
            for (int j = 0; j < kSimtMaxJ; ++j) {
                const int i = tid + j * kSimtThreads;
                if (i < K) {
                    if (writer) a.h_out[(size_t)(b0 + b) * K + i] = hv[j];
                    ss[0] += hv[j] * hv[j];
                }
            }
            block_sum<1>(ss, red);
            const float r2 = 1.0f / sqrtf(ss[0] / (float)K + a.eps);
#pragma unroll
            for (int j = 0; j < kSimtMaxJ; ++j) {
                const int i = tid + j * kSimtThreads;
                if (i < K) T::store_x(xs + (size_t)b * K + i, hv[j] * r2 * wnorm[j]);
            }
        }
    }
    // rows of a partial batch chunk that do not exist read zeros
    for (int b = nb; b < NB; ++b)
        for (int i = tid; i < K; i += kSimtThreads) xs[(size_t)b * K + i] = (XT)0;
    __syncthreads();
    pdl_launch();
    stamp(a.ts, 2);

    if constexpr (EPI != EPI_LOGITS) {
        // ---- body: this warp's contiguous run of the CTA's chunks, cut at row boundaries ----
        int c0 = warp * lr;
        const int c1 = min(chunks_cta, c0 + lr);
        const bool ragged = (K % STEP) != 0;          // the last chunk of a row is partly empty
        while (c0 < c1) {
            const int rl = c0 / a.cpr;                 // row inside the CTA's block
            const int rend = min(c1, (rl + 1) * a.cpr);
            const int cc = c0 - rl * a.cpr;
            const int ncs = rend - c0;
            const bool has_tail = ragged && (cc + ncs == a.cpr);
            const int nfull = has_tail ? ncs - 1 : ncs;
            const WT* p = row_ptr(row_first + rl) + (size_t)cc * STEP + lane * EPL;
            int k = cc * STEP + lane * EPL;
            float acc[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[b] = 0.0f;
            int j = 0;
            for (; j + 8 <= nfull; j += 8) {
                uint4 w[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) w[q] = ldg_stream16(p + q * STEP);
#pragma unroll
                for (int q = 0; q < 8; ++q) fma16<WT, NB>(acc, w[q], xs, K, k + q * STEP);
                p += 8 * STEP;
                k += 8 * STEP;
            }
            if (j + 4 <= nfull) {
                uint4 w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) w[q] = ldg_stream16(p + q * STEP);
#pragma unroll
                for (int q = 0; q < 4; ++q) fma16<WT, NB>(acc, w[q], xs, K, k + q * STEP);
                p += 4 * STEP;
                k += 4 * STEP;
                j += 4;
            }
            if (j + 2 <= nfull) {
                uint4 w0 = ldg_stream16(p), w1 = ldg_stream16(p + STEP);
                fma16<WT, NB>(acc, w0, xs, K, k);
                fma16<WT, NB>(acc, w1, xs, K, k + STEP);
                p += 2 * STEP;
                k += 2 * STEP;
                j += 2;
            }
            for (; j < ncs; ++j) {
                if (k < K) {
                    uint4 w0 = ldg_stream16(p);
                    fma16<WT, NB>(acc, w0, xs, K, k);
                }
                p += STEP;
                k += STEP;
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[b] = warp_sum(acc[b]);
            if (lane == 0) {
                const int slot = warp - (rl * a.cpr) / lr;
#pragma unroll
                for (int b = 0; b < NB; ++b) pieces[((size_t)rl * a.slots + slot) * NB + b] = acc[b];
            }
            c0 = rend;
        }
        __syncthreads();
        // ---- epilogue: add the pieces of each row in slot order ----
        auto row_total = [&](int rl, int b) -> float {
            const int first = (rl * a.cpr) / lr;
            const int last = ((rl + 1) * a.cpr - 1) / lr;
            float t = 0.0f;
            for (int s = 0; s <= last - first; ++s) t += pieces[((size_t)rl * a.slots + s) * NB + b];
            return t;
        };
        if constexpr (EPI == EPI_STORE) {
            for (int idx = tid; idx < rows_cta * nb; idx += kSimtThreads) {
                const int rl = idx % rows_cta, b = idx / rows_cta;
                a.out[(size_t)(b0 + b) * a.N + row_first + rl] = row_total(rl, b);
            }
        } else {
            const int pairs = rows_cta / 2;
            for (int idx = tid; idx < pairs * nb; idx += kSimtThreads) {
                const int pl = idx % pairs, b = idx / pairs;
                const float g = row_total(2 * pl, b), u = row_total(2 * pl + 1, b);
                a.out[(size_t)(b0 + b) * (a.N / 2) + row_first / 2 + pl] = gelu_mul(g, u);
            }
        }
    } else {
        // ---- body: one warp per row pair; logits + running arg-max ----
        Cand best[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) { best[b].s = -INFINITY; best[b].i = 0xffffffffu; }
        const int U = (a.N + 1) / 2;
        for (int u = blockIdx.x + gridDim.x * warp; u < U; u += gridDim.x * kSimtWarps) {
            const int r0 = u * 2;
            const bool has1 = (r0 + 1 < a.N);
            const WT* p0 = row_ptr(r0);
            const WT* p1 = has1 ? p0 + K : p0;
            float acc0[NB], acc1[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) { acc0[b] = 0.0f; acc1[b] = 0.0f; }
            int k = lane * EPL;
            for (; k + 3 * STEP < K; k += 4 * STEP) {
                uint4 wa[4], wb[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    wa[j] = ldg_stream16(p0 + k + j * STEP);
                    wb[j] = ldg_stream16(p1 + k + j * STEP);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    fma16<WT, NB>(acc0, wa[j], xs, K, k + j * STEP);
                    fma16<WT, NB>(acc1, wb[j], xs, K, k + j * STEP);
                }
            }
            for (; k < K; k += STEP) {
                uint4 wa = ldg_stream16(p0 + k);
                uint4 wb = ldg_stream16(p1 + k);
                fma16<WT, NB>(acc0, wa, xs, K, k);
                fma16<WT, NB>(acc1, wb, xs, K, k);
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) { acc0[b] = warp_sum(acc0[b]); acc1[b] = warp_sum(acc1[b]); }
            if (lane == 0) {
                const int v0 = a.row_offset + r0;                 // vocabulary id of row r0
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (b >= nb) continue;
                    const size_t base = (size_t)(b0 + b) * a.n_total;
                    if (a.out) {
                        a.out[base + v0] = acc0[b];
                        if (has1) a.out[base + v0 + 1] = acc1[b];
                    }
                    // kernel_module.rs:2008-2016: penalty on seen tokens, NaN skipped, strict '>'
                    float s0 = acc0[b], s1 = acc1[b];
                    if (a.seen && a.penalty > 1.0f) {
                        if (a.seen[base + v0]) s0 = s0 >= 0.0f ? s0 / a.penalty : s0 * a.penalty;
                        if (has1 && a.seen[base + v0 + 1]) s1 = s1 >= 0.0f ? s1 / a.penalty : s1 * a.penalty;
                    }
                    const Cand c0{s0, (uint32_t)v0}, c1{s1, (uint32_t)(v0 + 1)};
                    if (s0 == s0 && s0 > -INFINITY && cand_better(c0, best[b])) best[b] = c0;
                    if (has1 && s1 == s1 && s1 > -INFINITY && cand_better(c1, best[b])) best[b] = c1;
                }
            }
        }
        // block-level arg-max, then the last block to arrive merges all blocks
        Cand* wc = reinterpret_cast<Cand*>(pieces);
        __shared__ unsigned int s_last;
        if (lane == 0)
            for (int b = 0; b < NB; ++b) wc[b * kSimtWarps + warp] = best[b];
        __syncthreads();
        if (tid < nb) {
            Cand c = wc[tid * kSimtWarps];
            for (int w = 1; w < kSimtWarps; ++w)
                if (cand_better(wc[tid * kSimtWarps + w], c)) c = wc[tid * kSimtWarps + w];
            a.blk_best[(size_t)(b0 + tid) * gridDim.x + blockIdx.x] = c;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(&a.ticket[blockIdx.y], 1u) == gridDim.x - 1) ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int b = warp; b < nb; b += kSimtWarps) {
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
            if (tid == 0) a.ticket[blockIdx.y] = 0u;       // ready for the next launch / replay
        }
    }
    stamp(a.ts, 3);
}

}  // namespace oxg4
