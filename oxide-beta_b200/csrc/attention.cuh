// Decode attention over a paged KV cache: one launch per layer does what the reference spreads
// over slice_rows x3, rms_norm (q), rope_state (q), rms_norm (k), rope_state (k), rms_norm_unit
// (v), cache_write_f32_state x2 and gqa_decode_block_state
// (crates/oxide-torch-models/src/gemma4_cuda/decode.rs:82-157; device math in
// crates/oxide-torch-cuda/src/kernel_module.rs:1133-1246,1423-1439,1510-1550,1790-1894).
//
// Grid (split, kv_head, sequence). The visible positions of a sequence are partitioned into up
// to `n_splits` contiguous ranges; each CTA streams its range of K and V rows once (split-KV
// "flash decoding" with an online softmax per warp), writes an un-normalised partial, and the
// last CTA of a (sequence, kv_head) to finish merges the partials in split order, so the result
// does not depend on scheduling. Attention scale is 1.0 as in the reference (no 1/sqrt(d)).
//
// Cache layout: pool[page][kv_head][token_in_page][head_dim]; a sequence's slot -> page mapping
// comes from its page table. Ring semantics follow the reference: slot = position % capacity,
// capacity = min(window, max_seq) on sliding layers (kernel_module.rs:1811-1831), so the ring
// itself implements the window.
//
// HBM-bound: bytes per launch = 2 * visible_positions * kv_heads * head_dim * sizeof(KV element).
#pragma once
#include <cooperative_groups.h>
#include <type_traits>

#include "common.cuh"

namespace oxg4 {

constexpr int kAttnThreads = 512;
constexpr int kAttnWarps = kAttnThreads / 32;

struct AttnArgs {
    const float* qkv;        // [qkv_splits, B, qkv_n] QKV projection output (K-split partials), columns q | k | v
    int qkv_n;
    int qkv_splits;          // partials to add (1 for the small-batch kernels)
    uint16_t* out_bf16;      // optional BF16 copy of the output, [B, Nq * D] (input of the tcgen05 O projection)
    int B, Nq, Nkv;
    const float* q_norm;     // [D]
    const float* k_norm;     // [D]
    const float* inv_freq;   // [D/2]: theta^(-2i/D) / factor
    int rotary_half;         // rotary_dim / 2; frequency lanes at or above it pass through
    float eps;
    const int32_t* pos;      // [B] absolute position of the token being processed
    const uint32_t* tokens;  // [B] (kInactiveToken rows are skipped)
    void* kpool;
    void* vpool;
    const int32_t* page_table;   // [B, pages_per_seq]
    int pages_per_seq, page_tokens;
    const int32_t* cap;      // [B] ring capacity of this layer kind for each sequence
    int window;              // a token sees the last `window` positions up to its own (sliding layers), INT_MAX otherwise
    const int32_t* row_seq;  // [B] sequence (page table, ring) of every row, or null: row b is sequence b
    int n_splits, min_split;
    float* part;             // [B, Nkv, n_splits, G, D + 2]
    unsigned int* ticket;    // [B, Nkv]
    float* out;              // [B, Nq * D]
    // weights of a later kernel to pull into L2 while this kernel runs (each CTA takes a slice)
    const void* pf_ptr;
    unsigned long long pf_bytes;
    unsigned long long* ts;  // optional timeline slots of this launch (4 entries) or null
    unsigned long long* ts_mid;  // optional: one more stamp, taken when the CTA's own partial is complete
};

template <typename KT, int EPT> struct KVec;
template <> struct KVec<uint16_t, 8> {
    static DEVINL void load(const uint16_t* p, float (&o)[8]) {
        uint4 v = ldg_stream16(p);
        o[0] = bf16lo(v.x); o[1] = bf16hi(v.x); o[2] = bf16lo(v.y); o[3] = bf16hi(v.y);
        o[4] = bf16lo(v.z); o[5] = bf16hi(v.z); o[6] = bf16lo(v.w); o[7] = bf16hi(v.w);
    }
};
template <> struct KVec<uint16_t, 4> {
    static DEVINL void load(const uint16_t* p, float (&o)[4]) {
        uint2 v = ldg_stream8(p);
        o[0] = bf16lo(v.x); o[1] = bf16hi(v.x); o[2] = bf16lo(v.y); o[3] = bf16hi(v.y);
    }
};
template <> struct KVec<uint16_t, 2> {
    static DEVINL void load(const uint16_t* p, float (&o)[2]) {
        uint32_t v = ldg_stream4(p);
        o[0] = bf16lo(v); o[1] = bf16hi(v);
    }
};
template <> struct KVec<float, 8> {
    static DEVINL void load(const float* p, float (&o)[8]) {
        uint4 a = ldg_stream16(p), b = ldg_stream16(p + 4);
        o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y); o[2] = __uint_as_float(a.z);
        o[3] = __uint_as_float(a.w); o[4] = __uint_as_float(b.x); o[5] = __uint_as_float(b.y);
        o[6] = __uint_as_float(b.z); o[7] = __uint_as_float(b.w);
    }
};
template <> struct KVec<float, 4> {
    static DEVINL void load(const float* p, float (&o)[4]) {
        uint4 a = ldg_stream16(p);
        o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y); o[2] = __uint_as_float(a.z);
        o[3] = __uint_as_float(a.w);
    }
};
template <> struct KVec<float, 2> {
    static DEVINL void load(const float* p, float (&o)[2]) {
        uint2 a = ldg_stream8(p);
        o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y);
    }
};

// A lane's slice of one K or V row as loaded (packed), converted only when it is consumed, so that
// the next positions' loads can be in flight in few registers.
template <typename KT, int EPT> struct KRaw {
    static constexpr int NWORDS = EPT * (int)sizeof(KT) / 4;
    uint32_t w[NWORDS];
};
template <typename KT, int EPT> DEVINL void kraw_load(const KT* p, KRaw<KT, EPT>& r) {
    constexpr int NWD = KRaw<KT, EPT>::NWORDS;
    if constexpr (NWD == 8) {
        const uint4 x = ldg_stream16(p), y = ldg_stream16((const char*)p + 16);
        r.w[0] = x.x; r.w[1] = x.y; r.w[2] = x.z; r.w[3] = x.w; r.w[4] = y.x; r.w[5] = y.y; r.w[6] = y.z; r.w[7] = y.w;
    } else if constexpr (NWD == 4) {
        const uint4 x = ldg_stream16(p);
        r.w[0] = x.x; r.w[1] = x.y; r.w[2] = x.z; r.w[3] = x.w;
    } else if constexpr (NWD == 2) {
        const uint2 x = ldg_stream8(p);
        r.w[0] = x.x; r.w[1] = x.y;
    } else {
        r.w[0] = ldg_stream4(p);
    }
}
template <typename KT, int EPT> DEVINL void kraw_cvt(const KRaw<KT, EPT>& r, float (&o)[EPT]) {
    if constexpr (sizeof(KT) == 2) {
#pragma unroll
        for (int i = 0; i < EPT / 2; ++i) { o[2 * i] = bf16lo(r.w[i]); o[2 * i + 1] = bf16hi(r.w[i]); }
    } else {
#pragma unroll
        for (int i = 0; i < EPT; ++i) o[i] = __uint_as_float(r.w[i]);
    }
}

template <typename KT> DEVINL KT kv_store_cvt(float v);
template <> DEVINL float kv_store_cvt<float>(float v) { return v; }
template <> DEVINL uint16_t kv_store_cvt<uint16_t>(float v) { return (uint16_t)f32_to_bf16_bits(v); }
template <typename KT> DEVINL float kv_widen(KT v);
template <> DEVINL float kv_widen<float>(float v) { return v; }
template <> DEVINL float kv_widen<uint16_t>(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }

struct BarCta {
    DEVINL void operator()() const { __syncthreads(); }
};

// One CTA's share of a launch: split `s` of kv head `kvh` of sequence `b`, computed by the `nthreads`
// threads that call it (tid = threadIdx.x < nthreads). `sm` is attn_smem_floats() floats of shared memory.
// PDL: wait for the preceding kernel after the constant loads (stand-alone kernel only).
template <typename KT, int D, int G, bool CL, bool PDL, bool DEEP, typename BAR>
DEVINL void attn_cta(const AttnArgs& a, float* sm, const int s, const int kvh, const int b, const int nthreads,
                     const BAR bar) {
    constexpr int EPT = D / 32;
    const int NW = nthreads >> 5;            // 16 warps when few CTAs exist (latency), 4 when many (occupancy)
    float* qs = sm;                          // [G][D]
    float* kcur = qs + G * D;                // [D]
    float* vcur = kcur + D;                  // [D]
    float* wm = vcur + D;                    // [NW][G]
    float* wl = wm + NW * G;                 // [NW][G]
    float* wacc = wl + NW * G;               // [NW][G][D]
    float* cpart = wacc + NW * G * D;        // [G][D + 2] this CTA's partial (cluster variant)
    float* rope = cpart + G * (D + 2);       // [D] cos (first half) and sin (second half) of pos * inv_freq
    __shared__ unsigned int s_last;
    __shared__ float s_scale[16 * 8], s_l[16 * 8], s_M[8];   // merge scratch: up to 16 warps or cluster splits x 8 heads

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = D / 2;

    if (a.pf_bytes) {
        // one 32 KiB bulk prefetch per thread at most (a single thread issuing dozens of them would sit on the
        // CTA's critical path for microseconds)
        constexpr unsigned long long PIECE = 32 * 1024;
        const unsigned long long npieces = (a.pf_bytes + PIECE - 1) / PIECE;
        const unsigned long long ncta = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
        const unsigned long long me = ((unsigned long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        for (unsigned long long pi = me + ncta * tid; pi < npieces; pi += ncta * nthreads) {
            const unsigned long long off = pi * PIECE;
            prefetch_l2_bulk((const char*)a.pf_ptr + off, (size_t)min(PIECE, a.pf_bytes - off));
        }
    }
    // model constants for this lane's slice of a head: fetched before the dependency wait
    float wq[EPT], wk[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int d = lane * EPT + e;
        wq[e] = a.q_norm[d];
        wk[e] = a.k_norm[d];
    }
    // Step state (token, position, ring capacity, page table) is written by the step's first kernel or the
    // previous step's last one. Every kernel of the step waits for its predecessor BEFORE it lets its
    // successor start, so when this code runs, everything but the immediately preceding kernel (the QKV
    // projection) has completed: the step state may be read, and the rotation factors computed, ahead
    // of the dependency wait.
    const bool active = a.tokens[b] != kInactiveToken;
    const int pos = a.pos[b];
    const int sb = a.row_seq ? a.row_seq[b] : b;
    const int cap = a.cap[sb];
    const int lo = max(0, pos + 1 - min(cap, a.window));
    // The variant that merges through global memory (CL = false) serves the rows of a prompt chunk: K and V of
    // every row, the current position included, are already in the cache (qkv_post_kernel appended the whole
    // chunk first), so the CTA only norms its queries.
    constexpr bool ext = !CL;
    const int n = pos - lo + 1;
    const int n_eff = min(a.n_splits, (n + a.min_split - 1) / a.min_split);
    const bool has_work = active && s < n_eff;
    float* part = a.part + (((size_t)b * a.Nkv + kvh) * a.n_splits) * (size_t)(G * (D + 2));
    size_t cur_off = 0;
    // this CTA's range of positions, and the loads of its first step: K/V rows of earlier positions were
    // written by earlier steps, so they can be in flight while the QKV projection finishes and while the
    // prologue below runs
    const int begin = has_work ? lo + (int)(((long long)n * s) / n_eff) : 0;
    const int end = has_work ? lo + (int)(((long long)n * (s + 1)) / n_eff) : 0;
    constexpr int PD = DEEP ? 4 : 2;
    typedef KRaw<KT, EPT> Raw;
    const KT* kpool = (const KT*)a.kpool;
    const KT* vpool = (const KT*)a.vpool;
    const int32_t* pt = a.page_table + (size_t)sb * a.pages_per_seq;
    auto row_offset = [&](int p) -> size_t {
        const int slot = p % cap;
        return (((size_t)pt[slot / a.page_tokens] * a.Nkv + kvh) * a.page_tokens +
                (slot % a.page_tokens)) * (size_t)D + lane * EPT;
    };
    auto issue = [&](int p, Raw& kr, Raw& vr) {            // loads only; the current token comes from shared memory
        if (p < end && (p != pos || ext)) {
            const size_t off = row_offset(p);
            kraw_load<KT, EPT>(kpool + off, kr);
            kraw_load<KT, EPT>(vpool + off, vr);
        }
    };
    Raw kr[PD], vr[PD];
    if (has_work && !ext) {
#pragma unroll
        for (int q = 0; q < PD; ++q) issue(begin + warp + q * NW, kr[q], vr[q]);
    }
    if (has_work) {
        const int slot_cur = pos % cap;
        cur_off = (((size_t)pt[slot_cur / a.page_tokens] * a.Nkv + kvh) *
                       a.page_tokens + (slot_cur % a.page_tokens)) * (size_t)D;
        // rotation factors of this position, one cosf or sinf per thread instead of 2 * D / 32 per lane
        for (int i = tid; i < D; i += nthreads) {
            const int fi = i % half;
            if (fi < a.rotary_half) {
                const float angle = (float)pos * a.inv_freq[fi];
                rope[i] = i < half ? cosf(angle) : sinf(angle);
            }
        }
    }
    stamp(a.ts, 0);
    if constexpr (PDL) {
        pdl_wait();
        pdl_launch();
    }
    stamp(a.ts, 1);
    if (has_work && ext) {
        // rows of a prompt chunk: the K/V rows of this very chunk were appended by the preceding kernel, so
        // nothing may be read from the cache before the dependency wait
#pragma unroll
        for (int q = 0; q < PD; ++q) issue(begin + warp + q * NW, kr[q], vr[q]);
    }

    if (has_work) {
        const bool owner = (s == n_eff - 1);        // the range that contains `pos`
        bar();                                      // the rotation factors are in shared memory
        // tasks 0..G-1: query heads (norm + rope); task G: key (norm + rope + append);
        // task G+1: value (unit norm + append). One warp per task.
        const int n_tasks = (owner && !ext) ? G + 2 : G;
        for (int task = warp; task < n_tasks; task += NW) {
            int col;
            if (task < G) col = (kvh * G + task) * D;
            else if (task == G) col = a.Nq * D + kvh * D;
            else col = (a.Nq + a.Nkv) * D + kvh * D;
            float t[EPT];
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < EPT; ++e) {
                float v = 0.0f;
                for (int sp = 0; sp < a.qkv_splits; ++sp)
                    v += __ldcg(a.qkv + ((size_t)sp * a.B + b) * a.qkv_n + col + lane * EPT + e);
                t[e] = v;
                ss += v * v;
            }
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)D + a.eps);
            float* dst = task < G ? qs + task * D : (task == G ? kcur : vcur);
            if (task <= G) {
#pragma unroll
                for (int e = 0; e < EPT; ++e) dst[lane * EPT + e] = t[e] * r * (task < G ? wq[e] : wk[e]);
                __syncwarp();
                float o[EPT];
#pragma unroll
                for (int e = 0; e < EPT; ++e) {
                    const int d = lane * EPT + e;
                    const int fi = d % half;
                    float v = dst[d];
                    if (fi < a.rotary_half) {
                        const float pv = dst[d < half ? d + half : d - half];
                        const float rotated = d < half ? -pv : pv;
                        v = v * rope[fi] + rotated * rope[half + fi];
                    }
                    o[e] = v;
                }
                __syncwarp();
#pragma unroll
                for (int e = 0; e < EPT; ++e) dst[lane * EPT + e] = o[e];
            } else {
#pragma unroll
                for (int e = 0; e < EPT; ++e) dst[lane * EPT + e] = t[e] * r;
            }
            if (task >= G) {
                // append to the cache; keep the stored (possibly BF16-rounded) value for this step
                KT* pool = (KT*)(task == G ? a.kpool : a.vpool);
                __syncwarp();
#pragma unroll
                for (int e = 0; e < EPT; ++e) {
                    const int d = lane * EPT + e;
                    const KT stored = kv_store_cvt<KT>(dst[d]);
                    pool[cur_off + d] = stored;
                    dst[d] = kv_widen<KT>(stored);
                }
            }
        }
        bar();
        stamp(a.ts, 2);

        float q_[G][EPT];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < EPT; ++e) q_[g][e] = qs[g * D + lane * EPT + e];
        float m[G], l[G], acc[G][EPT];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.0f;
#pragma unroll
            for (int e = 0; e < EPT; ++e) acc[g][e] = 0.0f;
        }
        // The PD positions of a step: all PD * G dot products first, their butterfly reductions interleaved
        // (PD * G independent shuffles per level instead of one dependent chain per score), then the
        // updates in position order.
        auto use_step = [&](int p0, const Raw* kr, const Raw* vr, auto pd_tag) {
            constexpr int NP = decltype(pd_tag)::value;
            float sc[NP][G];
#pragma unroll
            for (int q = 0; q < NP; ++q) {
                const int pq = p0 + q * NW;
                float kf[EPT];
                if (pq == pos && !ext) {
#pragma unroll
                    for (int e = 0; e < EPT; ++e) kf[e] = kcur[lane * EPT + e];
                } else {
                    kraw_cvt<KT, EPT>(kr[q], kf);          // rows past `end` were never loaded: their scores are not used
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float t = 0.0f;
#pragma unroll
                    for (int e = 0; e < EPT; ++e) t = fmaf(q_[g][e], kf[e], t);
                    sc[q][g] = t;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int q = 0; q < NP; ++q)
#pragma unroll
                    for (int g = 0; g < G; ++g) sc[q][g] += __shfl_xor_sync(0xffffffffu, sc[q][g], o);
            // one online-softmax step for the NP positions together: a single rescale of the running sums
            float pe[NP][G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float mn = m[g];
#pragma unroll
                for (int q = 0; q < NP; ++q)
                    if (p0 + q * NW < end) mn = fmaxf(mn, sc[q][g]);
                const float corr = expf(m[g] - mn);       // exp(-inf) = 0 on the first step
                float ls = l[g] * corr;
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    pe[q][g] = (p0 + q * NW < end) ? expf(sc[q][g] - mn) : 0.0f;
                    ls += pe[q][g];
                }
                l[g] = ls;
                m[g] = mn;
#pragma unroll
                for (int e = 0; e < EPT; ++e) acc[g][e] *= corr;
            }
#pragma unroll
            for (int q = 0; q < NP; ++q) {
                const int pq = p0 + q * NW;
                if (pq >= end) break;
                float vf[EPT];
                if (pq == pos && !ext) {
#pragma unroll
                    for (int e = 0; e < EPT; ++e) vf[e] = vcur[lane * EPT + e];
                } else {
                    kraw_cvt<KT, EPT>(vr[q], vf);
                }
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int e = 0; e < EPT; ++e) acc[g][e] = fmaf(pe[q][g], vf[e], acc[g][e]);
            }
        };
        // PD positions per step, the next step's loads issued before this step's arithmetic: 2 * PD rows of
        // K and of V in flight per warp (PD = 4 when one sequence has the whole GPU and latency is all that counts)
        for (int p = begin + warp; p < end; p += PD * NW) {
            Raw nk[PD], nv[PD];
#pragma unroll
            for (int q = 0; q < PD; ++q) issue(p + (PD + q) * NW, nk[q], nv[q]);
            use_step(p, kr, vr, std::integral_constant<int, PD>{});
#pragma unroll
            for (int q = 0; q < PD; ++q) { kr[q] = nk[q]; vr[q] = nv[q]; }
        }

        stamp(a.ts_mid, 1);
        // merge the warps of this CTA (fixed warp order)
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (lane == 0) { wm[warp * G + g] = m[g]; wl[warp * G + g] = l[g]; }
#pragma unroll
            for (int e = 0; e < EPT; ++e) wacc[((size_t)warp * G + g) * D + lane * EPT + e] = acc[g][e];
        }
        bar();
        // one scale factor exp(m_w - M) per (warp, head), computed once instead of once per output element
        if (tid < NW * G) {
            const int g = tid % G;
            float M = -INFINITY;
            for (int w = 0; w < NW; ++w) M = fmaxf(M, wm[w * G + g]);
            const float mw = wm[tid];
            s_scale[tid] = (mw == -INFINITY) ? 0.0f : expf(mw - M);
            if (tid < G) s_M[g] = M;
        }
        bar();
        float* my = CL ? cpart : part + (size_t)s * (G * (D + 2));
        for (int idx = tid; idx < G * D; idx += nthreads) {
            const int g = idx / D, d = idx % D;
            float A = 0.0f, L = 0.0f;
            for (int w = 0; w < NW; ++w) {
                const float e = s_scale[w * G + g];
                A += e * wacc[((size_t)w * G + g) * D + d];
                L += e * wl[w * G + g];
            }
            my[g * (D + 2) + d] = A;
            if (d == 0) { my[g * (D + 2) + D] = s_M[g]; my[g * (D + 2) + D + 1] = L; }
        }
    }

    if constexpr (CL) {
        // ---- cluster merge: every CTA finishes a slice of the outputs from its peers' shared memory ----
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        stamp(a.ts_mid, 2);
        cluster.sync();                                    // every CTA of the cluster arrives, with or without work
        stamp(a.ts_mid, 3);
        if (active) {
            // (m, l) of every split -> this CTA's shared memory in one round of remote loads, then one scale
            // factor per (split, head); the weighted sums below are independent remote loads
            if (tid < n_eff * G) {
                const int sp = tid / G, g = tid % G;
                const float* ps = cluster.map_shared_rank(cpart, sp) + g * (D + 2);
                s_scale[tid] = ps[D];
                s_l[tid] = ps[D + 1];
            }
            bar();
            if (tid < G) {
                const int g = tid;
                float M = -INFINITY;
                for (int sp = 0; sp < n_eff; ++sp) M = fmaxf(M, s_scale[sp * G + g]);
                float L = 0.0f;
                for (int sp = 0; sp < n_eff; ++sp) {
                    const float ms = s_scale[sp * G + g];
                    const float e = (ms == -INFINITY) ? 0.0f : expf(ms - M);
                    s_scale[sp * G + g] = e;
                    L += e * s_l[sp * G + g];
                }
                s_M[g] = L;
            }
            bar();
            const int cs = (int)gridDim.x;
            const int per = (G * D + cs - 1) / cs;
            const int hi = min(G * D, (s + 1) * per);
            for (int idx = s * per + tid; idx < hi; idx += nthreads) {
                const int g = idx / D, d = idx % D;
                float A = 0.0f;
                for (int sp = 0; sp < n_eff; ++sp)
                    A += s_scale[sp * G + g] * cluster.map_shared_rank(cpart, sp)[g * (D + 2) + d];
                {
                    const size_t oi = (size_t)b * a.Nq * D + (size_t)(kvh * G + g) * D + d;
                    const float ov = A / s_M[g];
                    a.out[oi] = ov;
                    if (a.out_bf16) a.out_bf16[oi] = (uint16_t)f32_to_bf16_bits(ov);
                }
            }
        }
        cluster.sync();                                    // no CTA leaves while a peer may still read its partial
        stamp(a.ts, 3);
        return;
    }
    // ---- last CTA of this (sequence, kv head) merges the split partials in split order ----
    stamp(a.ts_mid, 0);
    __threadfence();
    bar();
    if (tid == 0)
        s_last = (atomicAdd(&a.ticket[b * a.Nkv + kvh], 1u) == (unsigned)a.n_splits - 1u) ? 1u : 0u;
    bar();
    if (s_last) {
        __threadfence();
        if (active) {
            // (m, l) of every split -> shared memory, one scale factor per (split, head), then the
            // weighted sum over splits with independent loads (fixed split order)
            constexpr int PS = G * (D + 2);
            float* sf = wacc;                         // [n_eff][G] m, then exp(m - M)
            float* sl = wacc + a.n_splits * G;        // [n_eff][G] l
            float* sL = sl + a.n_splits * G;          // [G]
            for (int idx = tid; idx < n_eff * G; idx += nthreads) {
                const int sp = idx / G, g = idx % G;
                sf[idx] = __ldcg(part + (size_t)sp * PS + g * (D + 2) + D);
                sl[idx] = __ldcg(part + (size_t)sp * PS + g * (D + 2) + D + 1);
            }
            bar();
            if (warp < G) {
                const int g = warp;
                float M = -INFINITY;
                for (int sp = lane; sp < n_eff; sp += 32) M = fmaxf(M, sf[sp * G + g]);
                M = warp_max(M);
                float L = 0.0f;
                for (int sp = lane; sp < n_eff; sp += 32) {
                    const float ms = sf[sp * G + g];
                    const float e = (ms == -INFINITY) ? 0.0f : expf(ms - M);
                    sf[sp * G + g] = e;
                    L += e * sl[sp * G + g];
                }
                L = warp_sum(L);
                if (lane == 0) sL[g] = L;
            }
            bar();
            for (int idx = tid; idx < G * D; idx += nthreads) {
                const int g = idx / D, d = idx % D;
                const float* ps = part + g * (D + 2) + d;
                float A = 0.0f;
                // sixteen independent loads in flight per round trip to L2
                for (int s0 = 0; s0 < n_eff; s0 += 16) {
                    float v[16];
#pragma unroll
                    for (int q = 0; q < 16; ++q) v[q] = (s0 + q < n_eff) ? __ldcg(ps + (size_t)(s0 + q) * PS) : 0.0f;
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        if (s0 + q < n_eff) A += sf[(s0 + q) * G + g] * v[q];
                }
                {
                    const size_t oi = (size_t)b * a.Nq * D + (size_t)(kvh * G + g) * D + d;
                    const float ov = A / sL[g];
                    a.out[oi] = ov;
                    if (a.out_bf16) a.out_bf16[oi] = (uint16_t)f32_to_bf16_bits(ov);
                }
            }
        }
        if (tid == 0) a.ticket[b * a.Nkv + kvh] = 0u;
    }
    stamp(a.ts, 3);
}

// CL = true (decode steps): the splits of one (sequence, kv head) form a thread-block cluster (gridDim.x <= 16
// CTAs); partials stay in shared memory and are merged through distributed shared memory after one cluster
// barrier; the CTA that owns the current position also norms, rotates and appends its K and V.
// CL = false (rows of a prompt chunk): K/V are in the cache already, partials go through global memory and the
// last CTA to arrive (atomic ticket) merges them.
template <typename KT, int D, int G, bool CL, bool DEEP = false>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnArgs a) {
    extern __shared__ __align__(16) float attn_sm[];
    attn_cta<KT, D, G, CL, true, DEEP>(a, attn_sm, blockIdx.x, blockIdx.y, blockIdx.z, blockDim.x, BarCta{});
}

template <int D, int G>
inline size_t attn_smem_bytes() {
    return sizeof(float) * (size_t)(G * D + 2 * D + 2 * kAttnWarps * G + kAttnWarps * G * D + G * (D + 2) + D);   // + page table
}

}  // namespace oxg4
