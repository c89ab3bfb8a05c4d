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
};

__global__ void __launch_bounds__(kRowsThreads) rows_norm_kernel(const RowsNormArgs a) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.x, tid = threadIdx.x, H = a.H;
    const size_t ro = (size_t)b * H;
    float r = 0.0f;
    uint32_t tok = 0;
    if (a.embed != nullptr) {
        tok = a.tokens[b];
        if (tok == kInactiveToken) tok = 0;
    } else if (a.raw != nullptr) {
        float ss[1] = {0.0f};
        for (int i = tid; i < H; i += kRowsThreads) {
            float t = 0.0f;
            for (int s = 0; s < a.raw_splits; ++s) t += a.raw[((size_t)s * a.B + b) * H + i];
            ss[0] += t * t;
        }
        block_sum<1>(ss, red);
        r = 1.0f / sqrtf(ss[0] / (float)H + a.eps);
    }
    auto hidden = [&](int i) -> float {
        if (a.embed != nullptr) return __uint_as_float((uint32_t)a.embed[(size_t)tok * H + i] << 16) * a.embed_scale;
        float h = a.h_in[ro + i];
        if (a.raw != nullptr) {
            float t = 0.0f;
            for (int s = 0; s < a.raw_splits; ++s) t += a.raw[((size_t)s * a.B + b) * H + i];
            h = (h + t * r * a.w_post[i]) * a.scalar;
        }
        return h;
    };
    float ss2[1] = {0.0f};
    for (int i = tid; i < H; i += kRowsThreads) {
        const float h = hidden(i);
        a.h_out[ro + i] = h;
        ss2[0] += h * h;
    }
    block_sum<1>(ss2, red);
    const float r2 = 1.0f / sqrtf(ss2[0] / (float)H + a.eps);
    for (int i = tid; i < H; i += kRowsThreads)
        a.x[ro + i] = (uint16_t)f32_to_bf16_bits(a.h_out[ro + i] * r2 * a.w_norm[i]);
}

// out[i] = sum_s part[s][i] in split order (tensor parallelism: one compact buffer goes through the
// all-reduce instead of every K-split partial)
__global__ void __launch_bounds__(kRowsThreads) sum_splits_kernel(const float* part, int splits, size_t n, float* out) {
    pdl_wait();
    pdl_launch();
    const size_t i = (size_t)blockIdx.x * kRowsThreads + threadIdx.x;
    if (i >= n) return;
    float t = 0.0f;
    for (int s = 0; s < splits; ++s) t += part[(size_t)s * n + i];
    out[i] = t;
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
