// Step bookkeeping and top-k selection kernels.
//
// step_begin / step_end replace the reference's one-thread decode_state_update / mark_seen
// launches (crates/oxide-torch-cuda/src/kernel_module.rs:1287-1317,1981-1986): the token ids and
// positions of every sequence live on the device so that a captured step can be replayed for any
// position. topk_stage1 / topk_stage2 produce the same list as the reference's two-stage top-k
// (kernel_module.rs:1988-2075): descending score, lowest index first among equal scores,
// repetition penalty applied to seen tokens, NaN never selected, unused slots (-inf, 0).
#pragma once
#include "common.cuh"

namespace oxg4 {

struct StepCtl {              // device-resident control words, written by the host before a step
    int32_t mark_seen;        // 1: seen[b][token[b]] = 1 at step begin
    int32_t feed_back;        // 1: next token[b] = arg-max of this step (device-resident greedy loop)
    int32_t step;             // steps run since the loop started (index into `history`)
    int32_t history_cap;      // capacity of `history` in steps
    int32_t sample;           // 1: the token fed back is drawn from the step's top-k list (sample_candidates_kernel)
    float temperature, top_p;
};

__global__ void step_begin_kernel(int B, int V, const uint32_t* tokens, uint8_t* seen, const StepCtl* ctl) {
    pdl_wait();
    pdl_launch();
    if (!ctl->mark_seen) return;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {       // launched as a single block
        const uint32_t t = tokens[b];
        if (t != kInactiveToken && t < (uint32_t)V) seen[(size_t)b * V + t] = 1;
    }
}

__global__ void step_end_kernel(int B, uint32_t* tokens, int32_t* pos, const uint32_t* best_ids,
                                uint32_t* history, StepCtl* ctl) {
    pdl_wait();
    pdl_launch();
    const int fb = ctl->feed_back;
    const int step = ctl->step;
    const int hist_cap = ctl->history_cap;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {       // launched as a single block
        if (tokens[b] == kInactiveToken) continue;
        pos[b] += 1;
        if (fb) {
            const uint32_t nxt = best_ids[b];
            if (step < hist_cap) history[(size_t)step * B + b] = nxt;
            tokens[b] = nxt;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && fb) ctl->step = step + 1;
}

// f32::total_cmp key (the reference sorts candidates with it, sampling.rs:88-158)
DEVINL int32_t total_order_key_dev(float f) {
    int32_t b = __float_as_int(f);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return b;
}

// The reference's sample_topk_candidates (crates/oxide-torch-models/src/models/gemma4/sampling.rs:88-158) on
// the device, one thread per sequence over the step's (<= 64) top-k candidates: temperature, stable
// descending sort, softmax, top-p cut, xorshift64 (13, 7, 17), 24-bit uniform, cumulative pick. The same
// f32 operations in the same order as the host version (oxg4_sample_topk_candidates); the generator state
// lives on the device so that a sampled generation loop needs no per-token host round trip. The chosen
// token replaces best_ids[b], which step_end feeds back. `softcap` > 0 applies tanh(x / cap) * cap first.
__global__ void sample_candidates_kernel(int B, int k, float softcap, const uint32_t* tokens, const uint32_t* cand_ids,
                                         const float* cand_scores, const StepCtl* ctl, unsigned long long* rng,
                                         uint32_t* best_ids, float* best_scores) {
    pdl_wait();
    pdl_launch();
    if (!ctl->sample) return;
    const float temperature = ctl->temperature, top_p = ctl->top_p;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {       // launched as a single block
        if (tokens[b] == kInactiveToken) continue;
        uint32_t id[64];
        float v[64];
        int n = 0;
        for (int i = 0; i < k; ++i) {
            float s = cand_scores[(size_t)b * k + i];
            // final_logit_softcapping is applied to the candidate scores before they are sampled
            // (gemma4_cuda/mod.rs:573-579, decode.rs:644,746), as the host path does
            if (softcap > 0.0f) s = tanhf(s / softcap) * softcap;
            if (isfinite(s)) { id[n] = cand_ids[(size_t)b * k + i]; v[n] = s / temperature; ++n; }
        }
        if (n == 0) continue;                                  // keep the arg-max
        for (int i = 1; i < n; ++i) {                          // stable insertion sort, descending total order
            const float vi = v[i];
            const uint32_t ii = id[i];
            int j = i - 1;
            while (j >= 0 && total_order_key_dev(v[j]) < total_order_key_dev(vi)) { v[j + 1] = v[j]; id[j + 1] = id[j]; --j; }
            v[j + 1] = vi;
            id[j + 1] = ii;
        }
        const float maximum = v[0];
        float total = 0.0f;
        for (int i = 0; i < n; ++i) { v[i] = expf(v[i] - maximum); total += v[i]; }
        if (total == 0.0f || !isfinite(total)) continue;
        for (int i = 0; i < n; ++i) v[i] /= total;
        if (top_p < 1.0f) {
            float cumulative = 0.0f;
            int keep = 0;
            for (int i = 0; i < n; ++i) {
                cumulative += v[i];
                ++keep;
                if (cumulative >= top_p) break;
            }
            n = max(keep, 1);
            total = 0.0f;
            for (int i = 0; i < n; ++i) total += v[i];
        } else {
            total = 1.0f;
        }
        unsigned long long r = rng[b];
        if (r == 0) r = 0x4d595df4d0f33173ull;
        r ^= r << 13;
        r ^= r >> 7;
        r ^= r << 17;
        rng[b] = r;
        const float unit = __fdiv_rn((float)((uint32_t)(r >> 40)), 16777216.0f);
        float threshold = __fmul_rn(unit, total);
        int pick = n - 1;
        for (int i = 0; i < n; ++i) {
            if (threshold <= v[i]) { pick = i; break; }
            threshold = __fsub_rn(threshold, v[i]);
        }
        best_ids[b] = id[pick];
        best_scores[b] = v[pick];
    }
}

// Tensor parallelism: every rank holds the arg-max of its vocabulary slice; after an all-gather this
// picks the global winner (same tie-break as everywhere: higher score, then lower id).
__global__ void tp_pick_kernel(int B, int ranks, const float* all_scores, const uint32_t* all_ids,
                               uint32_t* ids, float* scores) {
    pdl_wait();
    pdl_launch();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        Cand best{all_scores[b], all_ids[b]};
        for (int r = 1; r < ranks; ++r) {
            const Cand c{all_scores[(size_t)r * B + b], all_ids[(size_t)r * B + b]};
            if (cand_better(c, best)) best = c;
        }
        ids[b] = best.i;
        scores[b] = best.s;
    }
}

constexpr int kTopkThreads = 256;
constexpr int kTopkChunk = 2048;

// k rounds of block-wide arg-max with removal over `n` candidates held in shared memory.
DEVINL void topk_rounds(float* sc, uint32_t* id, int n, int top_k, Cand* wbest, Cand* out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int r = 0; r < top_k; ++r) {
        Cand c{-INFINITY, 0xffffffffu};
        int where = -1;
        for (int i = tid; i < n; i += kTopkThreads) {
            Cand o{sc[i], id[i]};
            if (o.s > -INFINITY && cand_better(o, c)) { c = o; where = i; }
        }
        Cand w = warp_best(c);
        if (lane == 0) wbest[warp] = w;
        __syncthreads();
        Cand best = wbest[0];
        for (int j = 1; j < kTopkThreads / 32; ++j)
            if (cand_better(wbest[j], best)) best = wbest[j];
        if (where >= 0 && c.s == best.s && c.i == best.i) sc[where] = -INFINITY;   // unique index
        if (tid == 0) {
            out[r].s = best.s;
            out[r].i = best.i == 0xffffffffu ? 0u : best.i;
        }
        __syncthreads();
    }
}

// grid (chunks, B): per-chunk sorted top-k over columns [col0, col0 + n_cols) of the [B, ld] logits (a
// tensor-parallel rank scans its own vocabulary slice); candidate ids are vocabulary ids
__global__ void __launch_bounds__(kTopkThreads)
topk_stage1_kernel(const float* logits, int ld, int col0, int n_cols, const uint8_t* seen, float penalty, int top_k,
                   Cand* stage) {
    __shared__ float sc[kTopkChunk];
    __shared__ uint32_t id[kTopkChunk];
    __shared__ Cand wbest[kTopkThreads / 32];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.y;
    const int start = blockIdx.x * kTopkChunk;
    const int n = min(kTopkChunk, n_cols - start);
    const size_t base = (size_t)b * ld + col0 + start;
    for (int i = threadIdx.x; i < n; i += kTopkThreads) {
        float s = logits[base + i];
        if (seen != nullptr && penalty > 1.0f && seen[base + i] != 0) s = s >= 0.0f ? s / penalty : s * penalty;
        sc[i] = (s == s) ? s : -INFINITY;         // NaN is never selected
        id[i] = (uint32_t)(col0 + start + i);
    }
    __syncthreads();
    topk_rounds(sc, id, n, top_k, wbest, stage + ((size_t)b * gridDim.x + blockIdx.x) * top_k);
}

// Tensor parallelism: every rank holds the sorted top-k of its vocabulary slice; after an all-gather
// ([ranks][B][k] scores and ids) one block per sequence merges the ranks * k candidates into the global
// top-k (descending score, lower id first among equal scores, as everywhere).
__global__ void __launch_bounds__(kTopkThreads)
tp_topk_merge_kernel(int B, int ranks, int k, const float* all_scores, const uint32_t* all_ids, uint32_t* ids,
                     float* scores) {
    __shared__ float sc[8 * 64];
    __shared__ uint32_t id[8 * 64];
    __shared__ Cand wbest[kTopkThreads / 32];
    __shared__ Cand outc[64];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.x, n = ranks * k;
    for (int i = threadIdx.x; i < n; i += kTopkThreads) {
        const int r = i / k, j = i % k;
        sc[i] = all_scores[((size_t)r * B + b) * k + j];
        id[i] = all_ids[((size_t)r * B + b) * k + j];
    }
    __syncthreads();
    topk_rounds(sc, id, n, k, wbest, outc);
    __syncthreads();
    for (int r = threadIdx.x; r < k; r += kTopkThreads) {
        ids[(size_t)b * k + r] = outc[r].i;
        scores[(size_t)b * k + r] = outc[r].s;
    }
}

// grid (1, B): merge of chunks * top_k candidates; dynamic shared memory = n * 8 bytes
__global__ void __launch_bounds__(kTopkThreads)
topk_stage2_kernel(const Cand* stage, int n, int top_k, uint32_t* ids, float* scores) {
    extern __shared__ __align__(16) unsigned char sm2[];
    float* sc = reinterpret_cast<float*>(sm2);
    uint32_t* id = reinterpret_cast<uint32_t*>(sm2) + n;
    __shared__ Cand wbest[kTopkThreads / 32];
    __shared__ Cand outc[64];
    pdl_wait();
    pdl_launch();
    const int b = blockIdx.y;
    for (int i = threadIdx.x; i < n; i += kTopkThreads) {
        const Cand c = stage[(size_t)b * n + i];
        sc[i] = c.s;
        id[i] = c.i;
    }
    __syncthreads();
    topk_rounds(sc, id, n, top_k, wbest, outc);
    __syncthreads();
    for (int r = threadIdx.x; r < top_k; r += kTopkThreads) {
        ids[(size_t)b * top_k + r] = outc[r].i;
        scores[(size_t)b * top_k + r] = outc[r].s;
    }
}

}  // namespace oxg4
