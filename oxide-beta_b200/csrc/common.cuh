// Device-side helpers shared by every kernel of the Gemma4 decode step (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DEVINL __device__ __forceinline__

namespace oxg4 {

constexpr uint32_t kInactiveToken = 0xFFFFFFFFu;   // a batch row that sits out the current step

// BF16 <-> f32 exactly as the reference does it: widening is a 16-bit shift
// (kernel_module.rs:1163), narrowing is bits + 0x7fff + lsb, >> 16 (kernel_module.rs:1338-1348).
DEVINL float bf16lo(uint32_t packed) { return __uint_as_float(packed << 16); }
DEVINL float bf16hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
DEVINL uint32_t f32_to_bf16_bits(float f) {
    uint32_t b = __float_as_uint(f);
    return (b + 0x7fffu + ((b >> 16) & 1u)) >> 16;
}
DEVINL float round_bf16(float f) { return __uint_as_float(f32_to_bf16_bits(f) << 16); }

DEVINL float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
DEVINL float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch: `pdl_wait` blocks until the preceding kernel of the stream has
// completed and its writes are visible; `pdl_launch` lets the following kernel's CTAs start their
// own pre-wait section (weight prefetch) while this one is still running.
DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DEVINL void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming 16-byte load of data that is read once per step (weights): bypass L1.
DEVINL uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
DEVINL uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
DEVINL uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
DEVINL void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// Optional device timeline: block (0,0,0) thread 0 stores the global nanosecond timer.
DEVINL void stamp(unsigned long long* ts, int slot) {
    if (ts != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        ts[slot] = t;
    }
}
// Bulk L2 prefetch of a contiguous range (address and size multiples of 16 bytes).
DEVINL void prefetch_l2_bulk(const void* p, size_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"((uint32_t)bytes) : "memory");
}

// Deterministic block-wide sums of NV values at once. `red` holds NV * 32 floats of shared memory.
// Every thread returns the same totals (summed in warp order).
template <int NV>
DEVINL void block_sum(float (&v)[NV], float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
    __syncthreads();                       // protect `red` against the previous use
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) red[i * 32 + warp] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float t = 0.0f;
        for (int w = 0; w < nwarps; ++w) t += red[i * 32 + w];
        v[i] = t;
    }
}

// (score, index) candidates ordered the way the reference's top-k orders them: higher score
// first, and among equal scores the lower index (strict '>' in kernel_module.rs:2016,2055).
struct Cand {
    float s;
    uint32_t i;
};
DEVINL bool cand_better(const Cand& a, const Cand& b) {
    return a.s > b.s || (a.s == b.s && a.i < b.i);
}
DEVINL Cand warp_best(Cand c) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Cand other;
        other.s = __shfl_xor_sync(0xffffffffu, c.s, o);
        other.i = __shfl_xor_sync(0xffffffffu, c.i, o);
        if (cand_better(other, c)) c = other;
    }
    return c;
}

// kernel_module.rs:1441-1458 — tanh-GELU through expf, times the up projection.
DEVINL float gelu_mul(float x, float up) {
    float inner = 0.7978846f * (x + 0.044715f * x * x * x);
    float t;
    if (inner >= 0.0f) {
        float e = expf(-2.0f * inner);
        t = (1.0f - e) / (1.0f + e);
    } else {
        float e = expf(2.0f * inner);
        t = (e - 1.0f) / (e + 1.0f);
    }
    float gelu = 0.5f * x * (1.0f + t);
    return gelu * up;
}

}  // namespace oxg4
