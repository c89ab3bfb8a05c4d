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

constexpr int kRowsMaxJ = 24;                 // values of a row held per thread: hidden <= 24 * 256 = 6144

__global__ void __launch_bounds__(kRowsThreads) rows_norm_kernel(const RowsNormArgs a) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.x, tid = threadIdx.x, H = a.H;
    const size_t ro = (size_t)b * H;
    float hv[kRowsMaxJ];
    if (a.embed != nullptr) {
        uint32_t tok = a.tokens[b];
        if (tok == kInactiveToken) tok = 0;
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i = tid + j * kRowsThreads;
            hv[j] = i < H ? __uint_as_float((uint32_t)a.embed[(size_t)tok * H + i] << 16) * a.embed_scale : 0.0f;
        }
    } else if (a.raw == nullptr) {
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i = tid + j * kRowsThreads;
            hv[j] = i < H ? a.h_in[ro + i] : 0.0f;
        }
    } else {
        if (a.px.tp > 1) {
            // wait (bounded) until every rank has published this exchange
            if (tid < a.px.tp) {
                const unsigned int want = *a.px.seq;
                const unsigned int* f = a.px.flags[a.px.rank] + tid;
                unsigned int it = 0;
                while (ld_acquire_sys(f) < want && ++it < kPeerSpinLimit) {}
                if (it >= kPeerSpinLimit) atomicExch(a.px.status, 1);
            }
            __syncthreads();
        }
        // the row is read once: the pending projection output (its K-split partials added in split order) and the
        // residual stream stay in registers between the two reductions
        float t[kRowsMaxJ];
        float ss[1] = {0.0f};
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i = tid + j * kRowsThreads;
            float v = 0.0f;
            if (i < H) {
                for (int s = 0; s < a.raw_splits; ++s) v += __ldcg(a.raw + ((size_t)s * a.B + b) * H + i);
                hv[j] = a.h_in[ro + i];
            } else {
                hv[j] = 0.0f;
            }
            t[j] = v;
            ss[0] += v * v;
        }
        block_sum<1>(ss, red);
        const float r = 1.0f / sqrtf(ss[0] / (float)H + a.eps);
#pragma unroll
        for (int j = 0; j < kRowsMaxJ; ++j) {
            const int i = tid + j * kRowsThreads;
            if (i < H) hv[j] = (hv[j] + t[j] * r * a.w_post[i]) * a.scalar;
        }
    }
    float ss2[1] = {0.0f};
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i = tid + j * kRowsThreads;
        if (i < H) {
            a.h_out[ro + i] = hv[j];
            ss2[0] += hv[j] * hv[j];
        }
    }
    block_sum<1>(ss2, red);
    const float r2 = 1.0f / sqrtf(ss2[0] / (float)H + a.eps);
#pragma unroll
    for (int j = 0; j < kRowsMaxJ; ++j) {
        const int i = tid + j * kRowsThreads;
        if (i < H) a.x[ro + i] = (uint16_t)f32_to_bf16_bits(hv[j] * r2 * a.w_norm[i]);
    }
}

// out[i] = sum_s part[s][i] in split order (tensor parallelism: one compact buffer goes through the
// all-reduce instead of every K-split partial)
__global__ void __launch_bounds__(kRowsThreads)
sum_splits_kernel(const float* part, int splits, size_t n, float* out, const PeerExchange px) {
    __shared__ unsigned int s_last;
    pdl_wait();
    pdl_launch();
    const size_t i = (size_t)blockIdx.x * kRowsThreads + threadIdx.x;
    if (i < n) {
        float t = 0.0f;
        for (int s = 0; s < splits; ++s) t += part[(size_t)s * n + i];
        if (px.tp > 1) {
            for (int r = 0; r < px.tp; ++r) px.push[r][i] = t;
        } else {
            out[i] = t;
        }
    }
    if (px.tp > 1) {
        // the last CTA to finish publishes the exchange to every rank (its own flag array included)
        __threadfence();
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

// x[b, i] = bf16(gelu_tanh(sum_s gu[s, b, i]) * sum_s gu[s, b, I + i]); grid (ceil(I / 256), B)
__global__ void __launch_bounds__(kRowsThreads)
geglu_rows_kernel(int B, int I, const float* gu, int splits, uint16_t* x) {
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.y, i = blockIdx.x * kRowsThreads + threadIdx.x;
    if (i >= I) return;
    float g = 0.0f, u = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float* row = gu + ((size_t)s * B + b) * (2 * (size_t)I);
        g += row[i];
        u += row[I + i];
    }
    x[(size_t)b * I + i] = (uint16_t)f32_to_bf16_bits(gelu_mul(g, u));
}

}  // namespace oxg4
