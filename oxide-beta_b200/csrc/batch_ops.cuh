// Small per-row kernels around the tcgen05 batched projections (csrc/tc_gemm.cuh), used when a step
// carries eight or more sequences. The tensor-core kernel takes its activations from global memory
// through TMA, so the prologues that the small-batch kernels fuse (gemv.cuh) run here as tiny
// kernels of their own; at these batch sizes a step lasts milliseconds and three extra launches per
// layer are noise.
//
//   rows_norm_kernel  the reference's rms_norm + add + mul_bf16_scalar + rms_norm_bf16 chain
//                     (gemma4_cuda/decode.rs:14,19-20,61-65,161-171,362-367; kernel_module.rs:1133-1211):
//                     h = (h_in + rmsnorm(sum of the projection's K-split partials, w_post)) * layer_scalar
//                     (or h = embedding row * sqrt(H), or h = h_in), x = bf16(rmsnorm(h, w_norm))
//   geglu_rows_kernel gelu_mul_f32 + f32_to_bf16 (decode.rs:17, kernel_module.rs:1441-1458, 1338-1348)
#pragma once
#include "common.cuh"
#include "tc_gemm.cuh"

namespace oxg4 {

constexpr int kRowsThreads = 256;
constexpr int kMaxTp = 8;
constexpr unsigned int kPeerSpinLimit = 4u * 1000u * 1000u;     // bounded polling of a peer flag (a few ms)

// Tensor parallelism over peer memory: the all-reduce after a row-split projection is not a kernel of
// its own. Every rank PUSHES its partial [B, H] into slot `rank` of every rank's gather buffer (plain
// peer stores over NVLink: no round trip per element) and then raises a sequence number in every
// rank's flag array; the kernel that consumes the sum waits, with a bound, until its own flags carry
// the expected number from all ranks and adds the tp partials from LOCAL memory in rank order, so
// every rank computes the same bits. No multicast, no TMA from peer memory.
struct PeerExchange {
    int tp, rank;
    float* push[kMaxTp];             // push[r]: slot `rank` of rank r's gather buffer for this kind, as mapped on THIS GPU
    const float* gathered;           // local gather buffer [tp][B * H]
    unsigned int* flags[kMaxTp];     // flags[r]: rank r's flag array [kMaxTp] for this kind, as mapped on THIS GPU
    unsigned int* seq;               // local: number of exchanges of this kind completed by the local producer
    unsigned int* ticket;            // local: producer CTAs still to finish
    int* status;                     // local: set non-zero when a bounded wait ran out
};

DEVINL unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
DEVINL void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *flag >= want; false when the polling budget ran out.
DEVINL bool peer_flag_wait(const unsigned int* flag, unsigned int want, unsigned int limit = kPeerSpinLimit) {
    unsigned int it = 0;
    while (ld_acquire_sys(flag) < want && ++it < limit) {}
    return it < limit;
}

struct RowsNormArgs {
    int B, H;
    const float* h_in;       // [B, H] (unused with embed)
    float* h_out;            // [B, H]
    const float* raw;        // [raw_splits, B, H] partial outputs of the previous projection, or null
    int raw_splits;
    const float* w_post;
    float scalar;
    const float* w_norm;
    const uint16_t* embed;   // [V, H] BF16 embedding table, or null
    const uint32_t* tokens;  // [B]
    float embed_scale;
    float eps;
    uint16_t* x;             // [B, H] BF16 activations for the next projection
    PeerExchange px;         // px.tp > 1: `raw` is the local gather buffer; wait for every rank's push first
};

constexpr int kRowsMaxJ = 6;                  // float4 groups of a row held per thread: hidden <= 6 * 256 * 4 = 6144

// sum over the K-split partials of 4 consecutive elements, in split order; four splits' loads in flight at a time
DEVINL float4 sum_splits4(const float* base, size_t split_stride, int splits) {
    float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
        float4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)(s + q) * split_stride));
#pragma unroll
        for (int q = 0; q < 4; ++q) { t.x += v[q].x; t.y += v[q].y; t.z += v[q].z; t.w += v[q].w; }
    }
    for (; s < splits; ++s) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (size_t)s * split_stride));
        t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    return t;
}

// One CTA per row; hidden size a multiple of 4. The row is read once: the pending projection output (its
// K-split partials added in split order) and the residual stream stay in registers between the two reductions.
__global__ void __launch_bounds__(kRowsThreads) rows_norm_kernel(const RowsNormArgs a) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.x, tid = threadIdx.x, H = a.H, H4 = a.H >> 2;
    const size_t ro = (size_t)b * H;
    float4 hv[kRowsMaxJ];
    if (a.embed != nullptr) {
        uint32_t tok = a.tokens[b];
        if (tok == kInactiveToken) tok = 0;
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i4 = tid + j * kRowsThreads;
            hv[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (i4 < H4) {
                const uint2 e = *reinterpret_cast<const uint2*>(a.embed + (size_t)tok * H + 4 * i4);
                hv[j] = make_float4(bf16lo(e.x) * a.embed_scale, bf16hi(e.x) * a.embed_scale, bf16lo(e.y) * a.embed_scale,
                                    bf16hi(e.y) * a.embed_scale);
            }
        }
    } else if (a.raw == nullptr) {
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i4 = tid + j * kRowsThreads;
            hv[j] = i4 < H4 ? *reinterpret_cast<const float4*>(a.h_in + ro + 4 * i4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    } else {
        if (a.px.tp > 1) {
            // wait (bounded) until every rank has published this exchange
            if (tid < a.px.tp) {
                if (!peer_flag_wait(a.px.flags[a.px.rank] + tid, *a.px.seq)) atomicExch(a.px.status, 1);
            }
            __syncthreads();
        }
        float4 t[kRowsMaxJ];
        float ss[1] = {0.0f};
        const size_t split_stride = (size_t)a.B * H;
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i4 = tid + j * kRowsThreads;
            t[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            hv[j] = t[j];
            if (i4 < H4) {
                t[j] = sum_splits4(a.raw + ro + 4 * i4, split_stride, a.raw_splits);
                hv[j] = *reinterpret_cast<const float4*>(a.h_in + ro + 4 * i4);
            }
            ss[0] += t[j].x * t[j].x;
            ss[0] += t[j].y * t[j].y;
            ss[0] += t[j].z * t[j].z;
            ss[0] += t[j].w * t[j].w;
        }
        block_sum<1>(ss, red);
        const float r = 1.0f / sqrtf(ss[0] / (float)H + a.eps);
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i4 = tid + j * kRowsThreads;
            if (i4 < H4) {
                const float4 w = *reinterpret_cast<const float4*>(a.w_post + 4 * i4);
                hv[j].x = (hv[j].x + t[j].x * r * w.x) * a.scalar;
                hv[j].y = (hv[j].y + t[j].y * r * w.y) * a.scalar;
                hv[j].z = (hv[j].z + t[j].z * r * w.z) * a.scalar;
                hv[j].w = (hv[j].w + t[j].w * r * w.w) * a.scalar;
            }
        }
    }
    float ss2[1] = {0.0f};
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i4 = tid + j * kRowsThreads;
        if (i4 < H4) {
            *reinterpret_cast<float4*>(a.h_out + ro + 4 * i4) = hv[j];
            ss2[0] += hv[j].x * hv[j].x;
            ss2[0] += hv[j].y * hv[j].y;
            ss2[0] += hv[j].z * hv[j].z;
            ss2[0] += hv[j].w * hv[j].w;
        }
    }
    block_sum<1>(ss2, red);
    const float r2 = 1.0f / sqrtf(ss2[0] / (float)H + a.eps);
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i4 = tid + j * kRowsThreads;
        if (i4 < H4) {
            const float4 w = *reinterpret_cast<const float4*>(a.w_norm + 4 * i4);
            uint2 o;
            o.x = f32_to_bf16_bits(hv[j].x * r2 * w.x) | (f32_to_bf16_bits(hv[j].y * r2 * w.y) << 16);
            o.y = f32_to_bf16_bits(hv[j].z * r2 * w.z) | (f32_to_bf16_bits(hv[j].w * r2 * w.w) << 16);
            *reinterpret_cast<uint2*>(a.x + ro + 4 * i4) = o;
        }
    }
}

// out[i] = sum_s part[s][i] in split order (tensor parallelism: one compact buffer goes through the
// all-reduce instead of every K-split partial)
__global__ void __launch_bounds__(kRowsThreads)
sum_splits_kernel(const float* part, int splits, size_t n, float* out, const PeerExchange px) {
    __shared__ unsigned int s_last;
    pdl_wait();
    pdl_launch();
    const size_t i = ((size_t)blockIdx.x * kRowsThreads + threadIdx.x) * 4;      // n is a multiple of 4
    if (i < n) {
        const float4 t = sum_splits4(part + i, n, splits);
        if (px.tp > 1) {
            for (int r = 0; r < px.tp; ++r) *reinterpret_cast<float4*>(px.push[r] + i) = t;
        } else {
            *reinterpret_cast<float4*>(out + i) = t;
        }
    }
    if (px.tp > 1) {
        // the last CTA to finish publishes the exchange to every rank (its own flag array included); every thread
        // orders its own peer stores at system scope before its CTA reports in
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) s_last = (atomicAdd(px.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            __threadfence_system();
            if (threadIdx.x == 0) {
                *px.ticket = 0u;
                const unsigned int seq = *px.seq + 1u;
                *px.seq = seq;
                __threadfence_system();
                for (int r = 0; r < px.tp; ++r) st_release_sys(px.flags[r] + px.rank, seq);
            }
        }
    }
}

// ---- per-layer embeddings of the Gemma4-E models (crates/oxide-torch-models/src/gemma4_cuda/ple.rs) ---------
// out[r, :] = embedding row of the row's token widened to f32, times sqrt(hidden) (kernel_module.rs:1272-1285);
// the input of the context projection. grid (R), any block size.
template <typename WT>
__global__ void ple_embed_rows_kernel(int H, const WT* embed, const uint32_t* tokens, float scale, float* out) {
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.x;
    uint32_t tok = tokens[r];
    if (tok == kInactiveToken) tok = 0;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v;
        if constexpr (sizeof(WT) == 2) v = __uint_as_float((uint32_t)embed[(size_t)tok * H + i] << 16);
        else v = embed[(size_t)tok * H + i];
        out[(size_t)r * H + i] = v * scale;
    }
}

// packed_ple_state / packed_ple_rows (ple.rs:55-99, 100-150): one warp per (row, layer):
//   context = rmsnorm_P(ctx[r, l*P ..] * (1 / sqrt(hidden))) * w         (the norm runs over the layer's P values)
//   token   = table[token, l*P ..] widened to f32 * sqrt(P)
//   packed  = (context + token) * FRAC_1_SQRT_2
template <typename WT>
__global__ void __launch_bounds__(128)
ple_pack_kernel(int R, int L, int P, const float* ctx, const float* w, const WT* table, const uint32_t* tokens, float eps,
                float inv_sqrt_h, float sqrt_p, float* packed) {
    pdl_wait();
    pdl_launch();
    const int job = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (job >= R * L) return;
    const int r = job / L, l = job % L;
    uint32_t tok = tokens[r];
    if (tok == kInactiveToken) return;
    const size_t base = (size_t)r * L * P + (size_t)l * P;
    float ss = 0.0f;
    for (int i = lane; i < P; i += 32) {
        const float v = ctx[base + i] * inv_sqrt_h;
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)P + eps);
    for (int i = lane; i < P; i += 32) {
        const float c = ctx[base + i] * inv_sqrt_h * s * w[i];
        float t;
        if constexpr (sizeof(WT) == 2) t = __uint_as_float((uint32_t)table[(size_t)tok * L * P + (size_t)l * P + i] << 16);
        else t = table[(size_t)tok * L * P + (size_t)l * P + i];
        packed[base + i] = (c + t * sqrt_p) * 0.70710678118654752440f;
    }
}

// apply_ple, first half (ple.rs:151-170 with the closing adds of decode.rs:19-20): one CTA per row closes the MLP
// block's residual, h' = h_in + rmsnorm(raw, w_post) (no layer_scalar yet), and stores it; it is both the input of
// the gate projection and the residual the branch is added to. Hidden size a multiple of 4.
__global__ void __launch_bounds__(kRowsThreads)
ple_close_kernel(int H, const float* h_in, const float* raw, const float* w_post, float eps, float* h_out) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.x, tid = threadIdx.x, H4 = H >> 2;
    const size_t ro = (size_t)b * H;
    float4 t[kRowsMaxJ];
    float ss[1] = {0.0f};
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i4 = tid + j * kRowsThreads;
        t[j] = i4 < H4 ? *reinterpret_cast<const float4*>(raw + ro + 4 * i4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss[0] += t[j].x * t[j].x;
        ss[0] += t[j].y * t[j].y;
        ss[0] += t[j].z * t[j].z;
        ss[0] += t[j].w * t[j].w;
    }
    block_sum<1>(ss, red);
    const float r = 1.0f / sqrtf(ss[0] / (float)H + eps);
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i4 = tid + j * kRowsThreads;
        if (i4 < H4) {
            const float4 h = *reinterpret_cast<const float4*>(h_in + ro + 4 * i4);
            const float4 w = *reinterpret_cast<const float4*>(w_post + 4 * i4);
            *reinterpret_cast<float4*>(h_out + ro + 4 * i4) =
                make_float4(h.x + t[j].x * r * w.x, h.y + t[j].y * r * w.y, h.z + t[j].z * r * w.z, h.w + t[j].w * r * w.w);
        }
    }
}

// apply_ple, middle (ple.rs:171-172): act[r, i] = gelu(gate[r, i]) * packed[r, l*P + i]; grid (ceil(P / 256), R)
__global__ void __launch_bounds__(kRowsThreads)
ple_act_kernel(int P, int LP, int layer, const float* gate, const float* packed, float* act) {
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.y, i = blockIdx.x * kRowsThreads + threadIdx.x;
    if (i >= P) return;
    act[(size_t)r * P + i] = gelu_mul(gate[(size_t)r * P + i], packed[(size_t)r * LP + (size_t)layer * P + i]);
}

// Failure-path probe (one thread): the two kinds of bounded device-side wait this library uses, each on
// something that nobody will ever signal, with a small polling budget. The wait must run out, raise the
// status word and let the kernel return normally; nothing faults and the context stays usable.
//   kind 1: mbarrier phase that never completes (the wait of the TMA / tcgen05 / attention pipelines)
//   kind 2: peer flag that never reaches the expected sequence number (tensor-parallel exchange)
__global__ void wait_probe_kernel(int kind, unsigned int limit, const unsigned int* never_set, int* status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x != 0) return;
    if (kind == 1) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(&bar, 0, limit)) atomicExch(status, 21);
    } else {
        if (!peer_flag_wait(never_set, 1u, limit)) atomicExch(status, 22);
    }
}

// Measurement aid: fills a K/V pool with a fixed pseudo-random pattern (values in [-1, 1)), 16 bytes per thread and
// pass, so that decode steps at a long context can be timed without ingesting the prompts first.
template <typename KT>
__global__ void pool_fill_kernel(uint4* __restrict__ pool, size_t n16, uint32_t salt) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u ^ (uint32_t)(i >> 32) ^ salt;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h ^= h >> 15; h *= 0x2c1b3c6du; h ^= h >> 12; h *= 0x297a2d39u; h ^= h >> 15;
            if (sizeof(KT) == 2) {
                const float a = (float)(int)(h & 0xffu) * (1.0f / 128.0f) - 1.0f;
                const float b = (float)(int)((h >> 8) & 0xffu) * (1.0f / 128.0f) - 1.0f;
                w[j] = (uint32_t)f32_to_bf16_bits(a) | ((uint32_t)f32_to_bf16_bits(b) << 16);
            } else {
                w[j] = __float_as_uint((float)(int)(h & 0xffffu) * (1.0f / 32768.0f) - 1.0f);
            }
        }
        pool[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// x[b, i] = bf16(gelu_tanh(sum_s gu[s, b, i]) * sum_s gu[s, b, I + i]); grid (ceil(I / 256), B)
__global__ void __launch_bounds__(kRowsThreads)
geglu_rows_kernel(int B, int I, const float* gu, int splits, uint16_t* x) {
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.y, i = (blockIdx.x * kRowsThreads + threadIdx.x) * 4;          // I is a multiple of 4
    if (i >= I) return;
    const size_t split_stride = (size_t)B * 2 * (size_t)I;
    const float* row = gu + (size_t)b * (2 * (size_t)I);
    const float4 g = sum_splits4(row + i, split_stride, splits);
    const float4 u = sum_splits4(row + I + i, split_stride, splits);
    uint2 o;
    o.x = f32_to_bf16_bits(gelu_mul(g.x, u.x)) | (f32_to_bf16_bits(gelu_mul(g.y, u.y)) << 16);
    o.y = f32_to_bf16_bits(gelu_mul(g.z, u.z)) | (f32_to_bf16_bits(gelu_mul(g.w, u.w)) << 16);
    *reinterpret_cast<uint2*>(x + (size_t)b * I + i) = o;
}

}  // namespace oxg4
