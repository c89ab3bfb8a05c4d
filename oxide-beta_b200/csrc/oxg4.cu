// Host runtime and C ABI of the B200-native Gemma4 token-generation path (see include/oxg4.h).
//
// Stands in for the reference's Gemma4 CUDA executor — crates/oxide-torch-models/src/gemma4_cuda/
// {mod,decode,attention,cache,tensor_ops}.rs — and the pieces of crates/oxide-torch-cuda it drives
// (kernel module, cuBLAS GEMM wrapper, CUDA-graph wrapper). Where the reference issues about 27
// launches per layer (decode.rs:4-21,43-174) with a separate f32 buffer between each, this runtime
// issues five: QKV projection, attention, O projection, gate/up projection, down projection; the
// norms, casts, residual adds, RoPE, KV append and GeGLU live in their prologues and epilogues.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/oxg4.h"
#include "attention.cuh"
#include "attention_mma.cuh"
#include "gemv.cuh"
#include "gemv_mma.cuh"
#include "sampling.cuh"
#include "batch_ops.cuh"
#include "tc_gemm.cuh"
#include "tp.h"

using namespace oxg4;

// ------------------------------------------------------------------------------------------------
// errors
// ------------------------------------------------------------------------------------------------
static thread_local std::string g_err;

static int32_t fail(int32_t code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CK(expr)                                                                                 \
    do {                                                                                         \
        cudaError_t e__ = (expr);                                                                \
        if (e__ != cudaSuccess)                                                                  \
            return fail(e__ == cudaErrorMemoryAllocation ? OXG4_OOM : OXG4_CUDA,                 \
                        "Gemma 4 CUDA error: %s (%s) at %s:%d", cudaGetErrorString(e__), #expr,  \
                        __FILE__, __LINE__);                                                     \
    } while (0)
#define TRY(expr)                        \
    do {                                 \
        int32_t s__ = (expr);            \
        if (s__ != OXG4_OK) return s__;  \
    } while (0)

extern "C" const char* oxg4_last_error(void) { return g_err.c_str(); }

// ------------------------------------------------------------------------------------------------
// model
// ------------------------------------------------------------------------------------------------
struct Tensor {
    void* d = nullptr;
    int dtype = OXG4_F32;     // element type on the device
    std::vector<int64_t> shape;
    size_t bytes = 0;
};

struct GemvPlan {             // how a projection is cut into CTA row blocks and warp runs
    int N = 0, K = 0, cpr = 0, grid = 0, slots = 1, rows_max = 0;
};

struct LayerPlan {            // Gemma4DecodeLayerPlan (gemma4_cuda/mod.rs:65-93)
    bool sliding = false;
    // head geometry of this layer (local to the tensor-parallel rank): sliding layers use head_dim and
    // num_key_value_heads, global layers global_head_dim and, with attention_k_eq_v, num_global_key_value_heads
    // (mod.rs:391-395, cache.rs:63-68)
    int D = 0, Nkv = 0, G = 1;
    int qkv_n = 0, qw = 0;    // rows of the fused projection ((Nq + 2 Nkv) D, or Nq D for a KV-shared layer), Nq * D
    int source = 0;           // the layer whose K/V cache this layer reads: itself, or for the last
    bool shared = false;      // num_kv_shared_layers layers the last earlier layer of the same type (cache.rs:43-86)
    GemvPlan p_qkv, p_o;
    // per-layer embeddings (ple.rs:151-185), null when hidden_size_per_layer_input == 0
    const void *w_ple_gate = nullptr, *w_ple_proj = nullptr;
    const float* ple_norm = nullptr;
    int rotary_dim = 0;
    float theta = 0, factor = 1, layer_scalar = 1;
    const void *wqkv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr, *wdown = nullptr;
    const float *input_ln = nullptr, *post_attn_ln = nullptr, *pre_ff_ln = nullptr,
                *post_ff_ln = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    float* inv_freq = nullptr;
};

struct ProfileSlot {
    double ms = 0;
    int count = 0;
};

struct oxg4_model {
    oxg4_config cfg{};
    std::vector<int32_t> layer_sliding, rotary_dim;
    std::vector<float> rope_theta, rope_factor;
    int device = 0;
    cudaStream_t stream = nullptr;
    int num_sms = 148;
    bool use_pdl = true;
    int far_prefetch = 0;         // bit mask: which kernels pull a LATER kernel's weights into L2 (1 qkv, 2 attention, 4 gate/up, 8 down)
    int far_prefetch_mb = 64;     // most MiB one kernel prefetches that way
    int pf_cap_kb = 128;          // KiB of its own weight block a CTA pulls into L2 before the dependency wait
    int pf_cap_gu_kb = -1, pf_cap_down_kb = -1;   // overrides for the gate/up and down projections (-1: pf_cap_kb)
    bool timeline = false;        // OXG4_TIMELINE: kernels stamp the global timer into the cache's buffer     // pull later kernels' weights into L2 during latency-bound kernels
    bool finalized = false;
    std::map<std::string, Tensor> tensors;
    // upload path: two pinned staging slots; the host copy into one overlaps the DMA out of the other
    void* stage[2] = {nullptr, nullptr};
    cudaEvent_t stage_ev[2] = {nullptr, nullptr};
    int stage_next = 0;
    std::vector<LayerPlan> layers;
    const void* embed = nullptr;
    const float* final_norm = nullptr;
    // local (per tensor-parallel rank) sizes
    int H = 0, Nq = 0, I = 0, V = 0, Vloc = 0, v0 = 0;
    int Dmax = 0, qkv_n_max = 0, qw_max = 0, kvw_max = 0;   // largest head_dim / fused rows / Nq*D / Nkv*D over the layers
    int P = 0;                // hidden_size_per_layer_input (0: no per-layer embeddings)
    const void *ple_embed = nullptr, *ple_model_proj = nullptr;
    const float* ple_proj_norm = nullptr;
    GemvPlan p_ple_ctx, p_ple_gate, p_ple_proj;
    int es = 2;               // bytes per weight element
    GemvPlan p_gateup, p_down, p_lm;
    int p_lm_simt_grid = 1;    // the SIMT logits kernel deals row pairs to warps across the grid
    long long launches = 0;
    int tp = 1, tp_rank = 0;
    void* comm = nullptr;         // ncclComm_t once oxg4_model_tp_init has run
    std::vector<struct oxg4_cache*> caches;     // live cache tables: destroyed with the model if the caller has not
    std::map<std::string, ProfileSlot> profile;
    bool profiling = false;
    std::vector<std::pair<std::string, std::pair<cudaEvent_t, cudaEvent_t>>> prof_events;
};

static int32_t bind_device(const oxg4_model* m) {
    CK(cudaSetDevice(m->device));
    return OXG4_OK;
}

static std::string canonical(const char* name) {
    std::string n(name);
    const std::string p = "model.language_model.";
    if (n.rfind(p, 0) == 0) n = n.substr(p.size());
    return n;
}

static inline uint16_t host_f32_to_bf16(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
static inline float host_bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    memcpy(&f, &b, 4);
    return f;
}

// full-model head geometry of layer l (before tensor-parallel sharding)
static int layer_head_dim(const oxg4_config& c, const int32_t* sliding, int l) {
    return sliding[l] ? c.head_dim : c.global_head_dim;
}
static int layer_kv_heads(const oxg4_config& c, const int32_t* sliding, int l) {
    if (!sliding[l] && c.attention_k_eq_v && c.num_global_key_value_heads > 0) return c.num_global_key_value_heads;
    return c.num_key_value_heads;
}
// layer index of a canonical tensor name "layers.N....", or -1
static int layer_of_name(const std::string& n) {
    if (n.rfind("layers.", 0) != 0) return -1;
    return atoi(n.c_str() + 7);
}

static GemvPlan make_plan(int N, int K, int es, int num_sms, int group /*rows that stay in one CTA*/) {
    GemvPlan p;
    p.N = N;
    p.K = K;
    const int step = 32 * (16 / es);
    p.cpr = (K + step - 1) / step;
    const int groups = N / group;
    p.grid = std::max(1, std::min(num_sms, groups));
    const int rows_min = (groups / p.grid) * group;
    p.rows_max = ((groups + p.grid - 1) / p.grid) * group;
    const int lr_min = std::max(1, (rows_min * p.cpr + kSimtWarps - 1) / kSimtWarps);
    p.slots = std::min(kSimtWarps, (p.cpr - 1) / lr_min + 2);
    return p;
}

extern "C" int32_t oxg4_model_create(const oxg4_config* c, int32_t device, oxg4_model** out) {
    if (!c || !out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (c->num_attention_heads <= 0 || c->num_key_value_heads <= 0 ||
        c->num_attention_heads % c->num_key_value_heads != 0 || c->hidden_size <= 0 ||
        c->num_hidden_layers <= 0)
        return fail(OXG4_INVALID_SHAPE, "invalid Gemma 4 attention configuration");   // config.rs:151-161
    if (!c->layer_is_sliding || !c->rotary_dim || !c->rope_theta || !c->rope_factor)
        return fail(OXG4_INVALID_ARGUMENT, "per-layer plan arrays are missing");
    if (c->weight_dtype != OXG4_F32 && c->weight_dtype != OXG4_BF16)
        return fail(OXG4_INVALID_ARGUMENT, "weight_dtype must be OXG4_F32 or OXG4_BF16");
    const int tp = c->tp_size <= 0 ? 1 : c->tp_size;
    if (tp != 1 && tp != 2 && tp != 4 && tp != 8) return fail(OXG4_INVALID_ARGUMENT, "tp_size must be 1, 2, 4 or 8");
    if (c->tp_rank < 0 || c->tp_rank >= tp) return fail(OXG4_INVALID_ARGUMENT, "tp_rank out of range");
    if (c->intermediate_size % tp != 0 || c->vocab_size % tp != 0)
        return fail(OXG4_INVALID_SHAPE, "tp_size must divide kv heads, intermediate size and vocabulary");
    if (c->num_kv_shared_layers < 0 || c->num_kv_shared_layers >= c->num_hidden_layers)
        return fail(OXG4_INVALID_SHAPE, "num_kv_shared_layers must leave at least one layer with its own cache");
    if (c->hidden_size_per_layer_input < 0 || (c->hidden_size_per_layer_input > 0 && c->vocab_size_per_layer_input <= 0))
        return fail(OXG4_INVALID_SHAPE, "per-layer embeddings need vocab_size_per_layer_input");
    for (int l = 0; l < c->num_hidden_layers; ++l) {           // head geometry of both layer kinds
        const int d = layer_head_dim(*c, c->layer_is_sliding, l), kvh = layer_kv_heads(*c, c->layer_is_sliding, l);
        if (d != 64 && d != 128 && d != 256)
            return fail(OXG4_UNSUPPORTED, "head_dim / global_head_dim must be 64, 128 or 256");
        if (kvh <= 0 || c->num_attention_heads % kvh != 0)
            return fail(OXG4_INVALID_SHAPE, "invalid Gemma 4 attention configuration");
        if (kvh % tp != 0 || c->num_attention_heads % tp != 0)
            return fail(OXG4_INVALID_SHAPE, "tp_size must divide kv heads, intermediate size and vocabulary");
        const int g = c->num_attention_heads / kvh;
        if (g != 1 && g != 2 && g != 4 && g != 8)
            return fail(OXG4_UNSUPPORTED, "query heads per KV head must be 1, 2, 4 or 8");
    }
    const int esz = c->weight_dtype == OXG4_BF16 ? 2 : 4;
    if ((c->hidden_size * esz) % 16 || (c->intermediate_size / tp * esz) % 16)
        return fail(OXG4_INVALID_SHAPE, "hidden and intermediate sizes must be multiples of 16 bytes");
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return fail(OXG4_CUDA, "Gemma 4 CUDA error: no CUDA device (%s); this library has no CPU path",
                    cudaGetErrorString(e));
    if (device < 0 || device >= ndev) return fail(OXG4_INVALID_ARGUMENT, "device ordinal %d out of range", device);
    oxg4_model* m = new oxg4_model();
    m->cfg = *c;
    const int L = c->num_hidden_layers;
    m->layer_sliding.assign(c->layer_is_sliding, c->layer_is_sliding + L);
    m->rotary_dim.assign(c->rotary_dim, c->rotary_dim + L);
    m->rope_theta.assign(c->rope_theta, c->rope_theta + L);
    m->rope_factor.assign(c->rope_factor, c->rope_factor + L);
    m->cfg.layer_is_sliding = m->layer_sliding.data();
    m->cfg.rotary_dim = m->rotary_dim.data();
    m->cfg.rope_theta = m->rope_theta.data();
    m->cfg.rope_factor = m->rope_factor.data();
    m->cfg.tp_size = tp;
    m->device = device;
    m->H = c->hidden_size;
    m->Nq = c->num_attention_heads / tp;
    m->P = c->hidden_size_per_layer_input;
    m->I = c->intermediate_size / tp;
    m->V = c->vocab_size;
    m->Vloc = c->vocab_size / tp;
    m->v0 = m->Vloc * c->tp_rank;
    m->es = esz;
    m->tp = tp;
    m->tp_rank = c->tp_rank;
    m->use_pdl = getenv("OXG4_DISABLE_PDL") == nullptr;
    m->timeline = getenv("OXG4_TIMELINE") != nullptr;
    if (const char* e = getenv("OXG4_PREFETCH_KB")) m->pf_cap_kb = std::max(0, atoi(e));
    if (const char* e = getenv("OXG4_PREFETCH_KB_GATEUP")) m->pf_cap_gu_kb = std::max(0, atoi(e));
    if (const char* e = getenv("OXG4_PREFETCH_KB_DOWN")) m->pf_cap_down_kb = std::max(0, atoi(e));
    if (const char* e = getenv("OXG4_FAR_PREFETCH")) m->far_prefetch = atoi(e);
    if (const char* e = getenv("OXG4_FAR_PREFETCH_MB")) m->far_prefetch_mb = std::max(1, atoi(e));
    if (cudaSetDevice(device) != cudaSuccess) { delete m; return fail(OXG4_CUDA, "Gemma 4 CUDA error: cudaSetDevice"); }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) m->num_sms = prop.multiProcessorCount;
    // a dedicated non-blocking stream: the legacy default stream cannot be captured (mod.rs:223-226)
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete m;
        return fail(OXG4_CUDA, "Gemma 4 CUDA error: stream creation failed");
    }
    *out = m;
    return OXG4_OK;
}

extern "C" void oxg4_cache_destroy(oxg4_cache* c);

extern "C" void oxg4_model_destroy(oxg4_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    cudaStreamSynchronize(m->stream);
    while (!m->caches.empty()) oxg4_cache_destroy(m->caches.back());   // a table points into its model: it goes first
    for (auto& kv : m->tensors) cudaFree(kv.second.d);
    for (auto& l : m->layers) cudaFree(l.inv_freq);
    for (int i = 0; i < 2; ++i) {
        if (m->stage[i]) cudaFreeHost(m->stage[i]);
        if (m->stage_ev[i]) cudaEventDestroy(m->stage_ev[i]);
    }
    if (m->comm) nccl().CommDestroy(m->comm);
    cudaStreamDestroy(m->stream);
    delete m;
}

// which slice of a checkpoint tensor a tensor-parallel rank keeps
constexpr size_t kStageBytes = 32u << 20;      // one pinned staging slot of the upload path

extern "C" int32_t oxg4_model_upload(oxg4_model* m, const char* name, int32_t dtype, const int64_t* shape,
                                     int32_t rank, const void* data, size_t bytes) {
    if (!m || !name || !shape || !data) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (m->finalized) return fail(OXG4_INVALID_ARGUMENT, "model is already finalized");
    if (dtype != OXG4_F32 && dtype != OXG4_BF16) return fail(OXG4_INVALID_ARGUMENT, "unsupported tensor dtype");
    TRY(bind_device(m));
    const std::string n = canonical(name);
    int64_t count = 1;
    for (int i = 0; i < rank; ++i) count *= shape[i];
    const size_t src_es = dtype == OXG4_BF16 ? 2 : 4;
    if (bytes != (size_t)count * src_es) return fail(OXG4_INVALID_SHAPE, "tensor `%s`: byte count does not match shape", n.c_str());
    // the reference's loader accepts BF16 only (mod.rs:247-251); the f32 mode is this build's extension
    if (m->cfg.weight_dtype == OXG4_BF16 && dtype != OXG4_BF16)
        return fail(OXG4_INVALID_ARGUMENT, "tensor `%s`: BF16 models take BF16 tensors", n.c_str());
    const bool is_matrix = rank == 2;
    Tensor t;
    t.shape.assign(shape, shape + rank);
    if (!is_matrix) {
        // norm weights and layer_scalar: widened to f32 once (exact); +1 folded in if requested
        std::vector<float> f((size_t)count);
        for (int64_t i = 0; i < count; ++i) {
            float v = dtype == OXG4_BF16 ? host_bf16_to_f32(((const uint16_t*)data)[i]) : ((const float*)data)[i];
            if (m->cfg.norm_weight_offset && n.find("layer_scalar") == std::string::npos) v += 1.0f;
            f[i] = v;
        }
        t.dtype = OXG4_F32;
        t.bytes = (size_t)count * 4;
        CK(cudaMalloc(&t.d, t.bytes));
        CK(cudaMemcpy(t.d, f.data(), t.bytes, cudaMemcpyHostToDevice));
    } else {
        // matrices keep the model's weight type
        const int dst_dtype = m->cfg.weight_dtype;
        const size_t dst_es = dst_dtype == OXG4_BF16 ? 2 : 4;
        const void* src = data;
        std::vector<uint8_t> conv;
        if ((int)dtype != dst_dtype) {      // only BF16 checkpoint into an f32 model
            conv.resize((size_t)count * 4);
            float* f = (float*)conv.data();
            for (int64_t i = 0; i < count; ++i) f[i] = host_bf16_to_f32(((const uint16_t*)data)[i]);
            src = conv.data();
        }
        t.dtype = dst_dtype;
        // tensor parallelism: keep only this rank's rows / columns (csrc/tp.h)
        const int ln_ = layer_of_name(n);
        const bool has_layer = ln_ >= 0 && ln_ < m->cfg.num_hidden_layers;
        const ShardSpec sh = shard_of(n, shape[0], shape[1], m->tp_rank, m->tp, m->cfg.num_attention_heads,
                                      has_layer ? layer_kv_heads(m->cfg, m->cfg.layer_is_sliding, ln_) : m->cfg.num_key_value_heads,
                                      has_layer ? layer_head_dim(m->cfg, m->cfg.layer_is_sliding, ln_) : m->cfg.head_dim,
                                      m->cfg.intermediate_size);
        t.shape = {sh.nrows, sh.ncols};
        t.bytes = (size_t)sh.nrows * sh.ncols * dst_es;
        CK(cudaMalloc(&t.d, t.bytes));
        // Loader fast path (stands in for the synchronous per-tensor copies of gemma4_cuda/mod.rs:236-279): the
        // caller's bytes (an mmap view of the checkpoint, pageable) are copied block by block into one of two
        // pinned slots and leave it by asynchronous DMA, so the host copy of block i + 1 overlaps the transfer of
        // block i. The SOURCE is no longer needed once the call returns (every byte is in pinned memory or on
        // the device), which is what SafeTensorLoader::with_view requires; the device is synchronised once, in
        // oxg4_model_finalize.
        const size_t row_b = (size_t)sh.ncols * dst_es, src_row_b = (size_t)shape[1] * dst_es;
        const size_t rows_per_block = std::max<size_t>(1, kStageBytes / row_b);
        if (row_b > kStageBytes) {
            // a single row wider than a slot: plain synchronous copy
            const char* s0 = (const char*)src + ((size_t)sh.row0 * shape[1] + sh.col0) * dst_es;
            CK(cudaMemcpy2D(t.d, row_b, s0, src_row_b, row_b, (size_t)sh.nrows, cudaMemcpyHostToDevice));
        } else {
            for (size_t r0 = 0; r0 < (size_t)sh.nrows; r0 += rows_per_block) {
                const size_t nr = std::min(rows_per_block, (size_t)sh.nrows - r0);
                const int slot = m->stage_next;
                m->stage_next ^= 1;
                if (!m->stage[slot]) {
                    CK(cudaMallocHost(&m->stage[slot], kStageBytes));
                    CK(cudaEventCreateWithFlags(&m->stage_ev[slot], cudaEventDisableTiming));
                } else {
                    CK(cudaEventSynchronize(m->stage_ev[slot]));      // the slot's previous DMA has drained
                }
                const char* s0 = (const char*)src + ((size_t)(sh.row0 + r0) * shape[1] + sh.col0) * dst_es;
                if (row_b == src_row_b) {
                    memcpy(m->stage[slot], s0, nr * row_b);
                } else {
                    for (size_t r = 0; r < nr; ++r) memcpy((char*)m->stage[slot] + r * row_b, s0 + r * src_row_b, row_b);
                }
                CK(cudaMemcpyAsync((char*)t.d + r0 * row_b, m->stage[slot], nr * row_b, cudaMemcpyHostToDevice, m->stream));
                CK(cudaEventRecord(m->stage_ev[slot], m->stream));
            }
        }
    }
    auto it = m->tensors.find(n);
    if (it != m->tensors.end()) { cudaFree(it->second.d); m->tensors.erase(it); }
    m->tensors[n] = t;
    return OXG4_OK;
}

static int32_t need(oxg4_model* m, const std::string& name, std::vector<int64_t> shape, const Tensor** out) {
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return fail(OXG4_INVALID_ARGUMENT, "missing CUDA weight `%s`", name.c_str());   // mod.rs:359-364
    if (!shape.empty() && it->second.shape != shape) {
        int64_t a = 1, b = 1;
        for (auto v : shape) a *= v;
        for (auto v : it->second.shape) b *= v;
        if (a != b) return fail(OXG4_INVALID_SHAPE, "weight `%s` has an unexpected shape", name.c_str());
    }
    *out = &it->second;
    return OXG4_OK;
}

// opt a kernel in to the full 227 KiB of shared memory (static + dynamic) of an sm_100 CTA
template <typename F>
static int32_t allow_big_smem(F* kernel) {
    cudaFuncAttributes fa;
    CK(cudaFuncGetAttributes(&fa, (const void*)kernel));
    const int big = 227 * 1024 - (int)fa.sharedSizeBytes;
    CK(cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    return OXG4_OK;
}

template <typename WT, int NB>
static int32_t set_gemv_attrs() {
#define SETA(PRO, EPI) TRY(allow_big_smem(gemv_kernel<WT, NB, PRO, EPI>))
    SETA(PRO_NORM, EPI_STORE);
    SETA(PRO_PLAIN, EPI_STORE);
    SETA(PRO_NORM, EPI_GATEUP);
    SETA(PRO_NORM, EPI_LOGITS);
#undef SETA
    return OXG4_OK;
}

template <int MB>
static int32_t set_mma_attrs() {
    TRY(allow_big_smem(gemv_mma_kernel<MB, PRO_NORM, EPI_STORE>));
    TRY(allow_big_smem(gemv_mma_kernel<MB, PRO_PLAIN, EPI_STORE>));
    TRY(allow_big_smem(gemv_mma_kernel<MB, PRO_NORM, EPI_GATEUP>));
    TRY(allow_big_smem(gemv_mma_kernel<MB, PRO_NORM, EPI_LOGITS>));
    return OXG4_OK;
}

template <typename KT, int D>
static int32_t set_attn_attrs() {
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 1, false>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 2, false>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 4, false>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 8, false>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 1, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 2, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 4, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 8, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 1, true, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 2, true, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 4, true, true>));
    TRY(allow_big_smem(attn_decode_kernel<KT, D, 8, true, true>));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 1, true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 2, true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 4, true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 8, true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 1, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 2, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 4, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CK(cudaFuncSetAttribute(attn_decode_kernel<KT, D, 8, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    return OXG4_OK;
}

extern "C" int32_t oxg4_model_finalize(oxg4_model* m) {
    if (!m) return fail(OXG4_INVALID_ARGUMENT, "null model");
    if (m->finalized) return OXG4_OK;
    TRY(bind_device(m));
    CK(cudaStreamSynchronize(m->stream));          // every staged upload has landed
    for (int i = 0; i < 2; ++i) {
        if (m->stage[i]) { cudaFreeHost(m->stage[i]); m->stage[i] = nullptr; }
        if (m->stage_ev[i]) { cudaEventDestroy(m->stage_ev[i]); m->stage_ev[i] = nullptr; }
    }
    const oxg4_config& c = m->cfg;
    const int L = c.num_hidden_layers, H = m->H;
    const Tensor* t = nullptr;
    TRY(need(m, "embed_tokens.weight", {c.vocab_size, H}, &t));
    m->embed = t->d;
    TRY(need(m, "norm.weight", {H}, &t));
    m->final_norm = (const float*)t->d;
    if (m->P > 0) {
        // per-layer embeddings (ple.rs:14-21,41-48): token table [V_ple, L * P], context projection [L * P, H], norm [P]
        TRY(need(m, "embed_tokens_per_layer.weight", {c.vocab_size_per_layer_input, (int64_t)L * m->P}, &t));
        m->ple_embed = t->d;
        TRY(need(m, "per_layer_model_projection.weight", {(int64_t)L * m->P, H}, &t));
        m->ple_model_proj = t->d;
        TRY(need(m, "per_layer_projection_norm.weight", {m->P}, &t));
        m->ple_proj_norm = (const float*)t->d;
        m->p_ple_ctx = make_plan(L * m->P, H, m->es, m->num_sms, 1);
        m->p_ple_gate = make_plan(m->P, H, m->es, m->num_sms, 1);
        m->p_ple_proj = make_plan(H, m->P, m->es, m->num_sms, 1);
    }
    m->layers.resize(L);
    const int first_shared = L - c.num_kv_shared_layers;       // cache.rs:43-45
    int last_sliding = -1, last_full = -1;
    m->Dmax = m->qkv_n_max = m->qw_max = m->kvw_max = 0;
    for (int l = 0; l < L; ++l) {
        LayerPlan& p = m->layers[l];
        const std::string pre = "layers." + std::to_string(l) + ".";
        p.sliding = m->layer_sliding[l] != 0;
        p.D = layer_head_dim(c, m->layer_sliding.data(), l);
        p.Nkv = layer_kv_heads(c, m->layer_sliding.data(), l) / m->tp;
        p.G = m->Nq / p.Nkv;
        p.qw = m->Nq * p.D;
        p.shared = l >= first_shared;
        if (!p.shared) {
            p.source = l;
            (p.sliding ? last_sliding : last_full) = l;
        } else {
            p.source = p.sliding ? last_sliding : last_full;
            if (p.source < 0)
                return fail(OXG4_INVALID_ARGUMENT, "shared layer %d has no preceding %s KV source", l,
                            p.sliding ? "sliding_attention" : "full_attention");       // cache.rs:76-80
        }
        const int D = p.D;
        const int64_t QW = p.qw, KW = (int64_t)p.Nkv * D;
        p.rotary_dim = m->rotary_dim[l];
        p.theta = m->rope_theta[l];
        p.factor = m->rope_factor[l];
        if (p.rotary_dim < 0 || p.rotary_dim > D) return fail(OXG4_INVALID_SHAPE, "layer %d: rotary_dim out of range", l);
        if (p.shared) {
            // a KV-shared layer keeps its q projection only (mod.rs:287, 420-424)
            const Tensor* q;
            TRY(need(m, pre + "self_attn.q_proj.weight", {QW, H}, &q));
            p.wqkv = q->d;
            p.qkv_n = (int)QW;
        } else {
            // fuse q/k/v rows into one [q;k;v, H] matrix (mod.rs:283-350)
            const Tensor *q, *k, *v;
            TRY(need(m, pre + "self_attn.q_proj.weight", {QW, H}, &q));
            TRY(need(m, pre + "self_attn.k_proj.weight", {KW, H}, &k));
            TRY(need(m, pre + "self_attn.v_proj.weight", {KW, H}, &v));
            Tensor f;
            f.dtype = q->dtype;
            f.shape = {QW + 2 * KW, H};
            f.bytes = q->bytes + k->bytes + v->bytes;
            CK(cudaMalloc(&f.d, f.bytes));
            CK(cudaMemcpy(f.d, q->d, q->bytes, cudaMemcpyDeviceToDevice));
            CK(cudaMemcpy((char*)f.d + q->bytes, k->d, k->bytes, cudaMemcpyDeviceToDevice));
            CK(cudaMemcpy((char*)f.d + q->bytes + k->bytes, v->d, v->bytes, cudaMemcpyDeviceToDevice));
            for (const char* nm : {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"}) {
                auto it = m->tensors.find(pre + nm);
                cudaFree(it->second.d);
                m->tensors.erase(it);
            }
            m->tensors[pre + "self_attn.qkv_proj.weight"] = f;
            p.wqkv = f.d;
            p.qkv_n = (int)(QW + 2 * KW);
            TRY(need(m, pre + "self_attn.k_norm.weight", {D}, &t)); p.k_norm = (const float*)t->d;
        }
        TRY(need(m, pre + "self_attn.o_proj.weight", {H, QW}, &t)); p.wo = t->d;
        TRY(need(m, pre + "mlp.gate_proj.weight", {m->I, H}, &t)); p.wgate = t->d;
        TRY(need(m, pre + "mlp.up_proj.weight", {m->I, H}, &t)); p.wup = t->d;
        TRY(need(m, pre + "mlp.down_proj.weight", {H, m->I}, &t)); p.wdown = t->d;
        TRY(need(m, pre + "input_layernorm.weight", {H}, &t)); p.input_ln = (const float*)t->d;
        TRY(need(m, pre + "post_attention_layernorm.weight", {H}, &t)); p.post_attn_ln = (const float*)t->d;
        TRY(need(m, pre + "pre_feedforward_layernorm.weight", {H}, &t)); p.pre_ff_ln = (const float*)t->d;
        TRY(need(m, pre + "post_feedforward_layernorm.weight", {H}, &t)); p.post_ff_ln = (const float*)t->d;
        TRY(need(m, pre + "self_attn.q_norm.weight", {D}, &t)); p.q_norm = (const float*)t->d;
        if (m->P > 0) {
            TRY(need(m, pre + "per_layer_input_gate.weight", {m->P, H}, &t)); p.w_ple_gate = t->d;
            TRY(need(m, pre + "per_layer_projection.weight", {H, m->P}, &t)); p.w_ple_proj = t->d;
            TRY(need(m, pre + "post_per_layer_input_norm.weight", {H}, &t)); p.ple_norm = (const float*)t->d;
        }
        TRY(need(m, pre + "layer_scalar", {1}, &t));          // mandatory, mod.rs:447
        CK(cudaMemcpy(&p.layer_scalar, t->d, 4, cudaMemcpyDeviceToHost));
        // kernel_module.rs:1539-1540: frequency = powf(theta, -(2 i)/head_dim) / factor, in f32
        std::vector<float> inv(D / 2);
        for (int i = 0; i < D / 2; ++i) {
            const float exponent = -((float)(2 * i)) / (float)D;
            inv[i] = powf(p.theta, exponent) / p.factor;
        }
        CK(cudaMalloc(&p.inv_freq, sizeof(float) * (D / 2)));
        CK(cudaMemcpy(p.inv_freq, inv.data(), sizeof(float) * (D / 2), cudaMemcpyHostToDevice));
        p.p_qkv = make_plan(p.qkv_n, H, m->es, m->num_sms, 1);
        p.p_o = make_plan(H, (int)QW, m->es, m->num_sms, 1);
        m->Dmax = std::max(m->Dmax, D);
        m->qkv_n_max = std::max(m->qkv_n_max, p.qkv_n);
        m->qw_max = std::max(m->qw_max, p.qw);
        m->kvw_max = std::max(m->kvw_max, p.Nkv * D);
    }
    m->p_gateup = make_plan(2 * m->I, H, m->es, m->num_sms, 2);
    m->p_down = make_plan(H, m->I, m->es, m->num_sms, 1);
    m->p_lm = make_plan(m->Vloc, H, m->es, m->num_sms, 1);
    m->p_lm_simt_grid = std::min(m->num_sms, std::max(1, (m->Vloc + 2 * kSimtWarps - 1) / (2 * kSimtWarps)));
    if (m->es == 2) {
        TRY((set_gemv_attrs<uint16_t, 1>()));
        TRY((set_mma_attrs<8>()));
        TRY((set_mma_attrs<16>()));
    } else {
        TRY((set_gemv_attrs<float, 1>())); TRY((set_gemv_attrs<float, 2>())); TRY((set_gemv_attrs<float, 4>()));
    }
    TRY((set_attn_attrs<uint16_t, 64>())); TRY((set_attn_attrs<uint16_t, 128>())); TRY((set_attn_attrs<uint16_t, 256>()));
    TRY((set_attn_attrs<float, 64>())); TRY((set_attn_attrs<float, 128>())); TRY((set_attn_attrs<float, 256>()));
    TRY(allow_big_smem(topk_stage2_kernel));
    CK(cudaDeviceSynchronize());
    m->finalized = true;
    return OXG4_OK;
}

extern "C" int64_t oxg4_weight_count(const oxg4_model* m) { return m ? (int64_t)m->tensors.size() : 0; }
extern "C" int64_t oxg4_weight_bytes(const oxg4_model* m) {
    int64_t b = 0;
    if (m) for (auto& kv : m->tensors) b += (int64_t)kv.second.bytes;
    return b;
}
extern "C" int32_t oxg4_synchronize(oxg4_model* m) {
    if (!m) return fail(OXG4_INVALID_ARGUMENT, "null model");
    TRY(bind_device(m));
    CK(cudaStreamSynchronize(m->stream));
    return OXG4_OK;
}
extern "C" int64_t oxg4_kernel_launches(const oxg4_model* m) { return m ? m->launches : 0; }

extern "C" int32_t oxg4_tp_shard(const char* name, int64_t rows, int64_t cols, int32_t tp_rank, int32_t tp_size,
                                 int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t intermediate,
                                 int64_t* out4) {
    if (!name || !out4) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(OXG4_INVALID_ARGUMENT, "tp_rank out of range");
    const ShardSpec s = shard_of(canonical(name), rows, cols, tp_rank, tp_size, heads, kv_heads, head_dim, intermediate);
    out4[0] = s.row0; out4[1] = s.nrows; out4[2] = s.col0; out4[3] = s.ncols;
    return OXG4_OK;
}

extern "C" int32_t oxg4_tp_unique_id(void* out) {
    if (!out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (!nccl().load()) return fail(OXG4_NCCL, "NCCL: %s", nccl().error.c_str());
    NcclApi::UniqueId id;
    const int rc = nccl().GetUniqueId(&id);
    if (rc != 0) return fail(OXG4_NCCL, "NCCL: ncclGetUniqueId: %s", nccl().GetErrorString(rc));
    memcpy(out, &id, sizeof id);
    return OXG4_OK;
}

extern "C" int32_t oxg4_model_tp_init(oxg4_model* m, const void* unique_id) {
    if (!m || !unique_id) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (m->tp == 1) return OXG4_OK;
    if (m->comm) return fail(OXG4_INVALID_ARGUMENT, "tensor-parallel communicator already initialised");
    TRY(bind_device(m));
    if (!nccl().load()) return fail(OXG4_NCCL, "NCCL: %s", nccl().error.c_str());
    NcclApi::UniqueId id;
    memcpy(&id, unique_id, sizeof id);
    NcclApi::Comm comm = nullptr;
    const int rc = nccl().CommInitRank(&comm, m->tp, id, m->tp_rank);
    if (rc != 0) return fail(OXG4_NCCL, "NCCL: ncclCommInitRank: %s", nccl().GetErrorString(rc));
    m->comm = comm;
    return OXG4_OK;
}

// ------------------------------------------------------------------------------------------------
// cache table + per-batch workspace
// ------------------------------------------------------------------------------------------------
struct GraphEntry {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int kernels = 0;
};

enum StepKind { STEP_TOPK = 0, STEP_LOGITS = 1, STEP_PREFILL = 2 };

struct oxg4_cache {
    oxg4_model* m = nullptr;
    int B = 0, PT = 256, kv_dtype = OXG4_BF16;
    std::vector<int32_t> max_seq, pos_host;
    int pps_full = 0, pps_slide = 0;
    int min_split = 32;
    std::vector<int> attn_splits;             // per layer: split-KV CTAs per (sequence, kv head) of the one-row attention kernel
    std::vector<int> ls_qkv, ls_o, lps_qkv, lps_o;   // per layer: K-splits of the tcgen05 QKV / O projections (decode, prompt chunk)
    int physical_caches = 0;
    bool attn_cluster = true;     // merge split-KV partials through a thread-block cluster's shared memory
    std::vector<void*> kpool, vpool;          // per layer
    std::vector<size_t> pool_bytes;           // per layer, 0 for a KV-shared layer
    int64_t kv_bytes = 0;
    int32_t *pt_full = nullptr, *pt_slide = nullptr, *cap_full = nullptr, *cap_slide = nullptr;
    uint32_t* tokens = nullptr;
    int32_t* pos = nullptr;
    uint8_t* seen = nullptr;
    StepCtl* ctl = nullptr;
    uint32_t* history = nullptr;
    int history_cap = 0;
    // workspace
    float *hA = nullptr, *hB = nullptr, *qkv_raw = nullptr, *attn_out = nullptr, *o_raw = nullptr,
          *gu_raw = nullptr, *down_raw = nullptr, *logits = nullptr, *attn_part = nullptr;
    unsigned int *attn_ticket = nullptr, *lm_ticket = nullptr;
    Cand *blk_best = nullptr, *topk_stage = nullptr;
    uint32_t *best_ids = nullptr, *topk_ids = nullptr, *tp_ids = nullptr, *loc_ids = nullptr, *tpk_ids = nullptr;
    float *tp_scores = nullptr, *loc_scores = nullptr, *tpk_scores = nullptr;   // tensor-parallel top-k exchange
    float *best_scores = nullptr, *topk_scores = nullptr;
    // pinned staging
    uint32_t* h_tokens = nullptr;
    StepCtl* h_ctl = nullptr;
    unsigned long long* rng = nullptr;        // [B] xorshift64 state of the device-side sampler
    int want_sample = 0;                      // copied into the step's control words by stage_inputs
    float sample_temperature = 1.0f, sample_top_p = 1.0f;
    uint32_t* h_ids = nullptr;
    float* h_scores = nullptr;
    std::map<std::string, GraphEntry> graphs;
    std::vector<void*> owned;                 // every device allocation, for destroy
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    unsigned long long* ts_buf = nullptr;     // [kMaxTimeline][4] optional device timeline
    // rows a pass over the layers may carry: the batch for a decode step, up to kPrefillRows prompt tokens for a chunk
    int rows_cap = 0;
    // prompt chunks: per-row metadata (token, position, sequence) and the attention groups, device + pinned host
    uint32_t *pf_tok = nullptr, *h_pf_tok = nullptr;
    int32_t *pf_pos = nullptr, *pf_seq = nullptr, *h_pf_meta = nullptr;
    int32_t *pf_grp_row0[2] = {nullptr, nullptr}, *pf_grp_n[2] = {nullptr, nullptr};   // attention groups of a chunk, per layer kind (sliding, global)
    // per-layer embeddings: embedding rows (f32 + BF16), context projection output, packed per-layer inputs, scratch
    float *ple_emb = nullptr, *ple_ctx = nullptr, *ple_packed = nullptr, *ple_h = nullptr, *ple_gate = nullptr, *ple_act = nullptr,
          *ple_raw = nullptr;

    int32_t *dec_grp_row0 = nullptr, *dec_grp_n = nullptr;      // decode: one group per sequence
    float *last_h = nullptr, *last_raw = nullptr;               // [B, H] residual stream / pending update of every sequence's last prompt token
    uint16_t* last_x = nullptr;                                 // [B, H] tcgen05 path: its normed BF16 activations
    // tensor-core attention (BF16 KV pages): query hi/lo tiles, per-warp partials, one tensor map per layer and pool
    bool mma_attn = false;
    uint16_t* q_hl = nullptr;
    float* am_part = nullptr;
    int* am_pre = nullptr;                    // tile prefix of the attention groups, attention kernel -> merge kernel
    std::vector<CUtensorMap> kmap, vmap;
    // tcgen05 path (decode with eight or more sequences, and every prompt chunk of a BF16 model): BF16
    // activations, K-split partial outputs, error flag
    bool use_tc = false, tc_ok = false;
    int s_gu = 1, s_down = 1;                                  // K-splits for a decode step (B rows)
    int ps_gu = 1, ps_down = 1;                                // K-splits for a full prompt chunk
    uint16_t *x_h = nullptr, *x_a = nullptr, *x_i = nullptr;
    float *qkv_part = nullptr, *o_part = nullptr, *gu_part = nullptr, *down_part = nullptr;
    int* tc_err = nullptr;
    // peer-memory exchange for tensor parallelism (two kinds: after O, after down)
    void* px_block = nullptr;                 // [2][tp][B*H] floats + [2][kMaxTp] flags, shared with the peers through CUDA IPC
    void* px_peer_base[kMaxTp] = {};          // peers' blocks as mapped here (own entry = px_block)
    unsigned int* px_local = nullptr;         // seq[2], ticket[2], status
    bool peer_ready = false;
    PeerExchange px[2];
};
constexpr int kMaxTimeline = 1024;

// Test hook: the n-th device allocation of a cache table from now on reports out-of-memory (0 = off).
static int g_fail_alloc_after = 0;

extern "C" void oxg4_debug_fail_alloc_after(int32_t n) { g_fail_alloc_after = n; }

template <typename T>
static int32_t dalloc(oxg4_cache* c, T** p, size_t count, bool zero = true) {
    void* d = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    if (g_fail_alloc_after > 0 && --g_fail_alloc_after == 0)
        return fail(OXG4_OOM, "Gemma 4 CUDA error: out of memory (injected by oxg4_debug_fail_alloc_after)");
    CK(cudaMalloc(&d, bytes));
    if (zero) CK(cudaMemset(d, 0, bytes));
    c->owned.push_back(d);
    *p = (T*)d;
    return OXG4_OK;
}

constexpr int kPrefillRows = 256;             // most prompt tokens one pass over the layers carries

static int32_t tc_gemm_setup();
static int32_t attn_mma_setup();
static int tc_pick_splits(int tiles, int kblocks, int grid, int B, int n_total, int K, double max_extra = 0.3);
static int32_t encode_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

static int32_t cache_build(oxg4_cache* c) {
    oxg4_model* m = c->m;
    const int B = c->B, L = m->cfg.num_hidden_layers, H = m->H, PT = c->PT;
    const size_t kes = c->kv_dtype == OXG4_BF16 ? 2 : 4;
    // Ring capacities. The reference keeps min(window, max_seq) rows on sliding layers and max_seq on global
    // ones (cache.rs:58-62) and lets the ring itself implement the window. Here a sliding ring keeps
    // kPrefillRows - 1 more rows, because a prompt chunk appends all its K/V rows before any of its tokens
    // attends (the earliest token of the chunk still needs the rows that the latest one would overwrite), and
    // every capacity is rounded up to the 16-position tile of the tensor-core attention; the window is
    // applied by the kernels (a token sees positions (pos - window, pos]), so the visible set is the reference's.
    auto round_up = [](int v, int q) { return (v + q - 1) / q * q; };
    std::vector<int32_t> capf(B), caps(B);
    int maxf = 0, maxs = 0, vis_s = 0;
    for (int b = 0; b < B; ++b) {
        capf[b] = round_up(c->max_seq[b], kAmTile);
        caps[b] = round_up(std::min(m->cfg.sliding_window + kPrefillRows - 1, c->max_seq[b]), kAmTile);
        maxf = std::max(maxf, capf[b]);
        maxs = std::max(maxs, caps[b]);
        vis_s = std::max(vis_s, std::min(m->cfg.sliding_window, c->max_seq[b]));
    }
    c->pps_full = (maxf + PT - 1) / PT;
    c->pps_slide = (maxs + PT - 1) / PT;
    std::vector<int32_t> ptf((size_t)B * c->pps_full, 0), pts((size_t)B * c->pps_slide, 0);
    int pages_full = 0, pages_slide = 0;
    for (int b = 0; b < B; ++b) {
        for (int i = 0; i < (capf[b] + PT - 1) / PT; ++i) ptf[(size_t)b * c->pps_full + i] = pages_full++;
        for (int i = 0; i < (caps[b] + PT - 1) / PT; ++i) pts[(size_t)b * c->pps_slide + i] = pages_slide++;
    }
    TRY(dalloc(c, &c->pt_full, ptf.size()));
    TRY(dalloc(c, &c->pt_slide, pts.size()));
    TRY(dalloc(c, &c->cap_full, B));
    TRY(dalloc(c, &c->cap_slide, B));
    CK(cudaMemcpy(c->pt_full, ptf.data(), ptf.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->pt_slide, pts.data(), pts.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->cap_full, capf.data(), B * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->cap_slide, caps.data(), B * 4, cudaMemcpyHostToDevice));
    c->mma_attn = c->kv_dtype == OXG4_BF16 && PT % kAmTile == 0 && getenv("OXG4_DISABLE_MMA_ATTN") == nullptr;
    c->kpool.assign(L, nullptr);
    c->vpool.assign(L, nullptr);
    c->pool_bytes.assign(L, 0);
    c->kmap.resize(L);
    c->vmap.resize(L);
    c->attn_splits.assign(L, 1);
    c->min_split = 16;
    c->attn_cluster = true;
    int smax = 1, part_floats = 1, ticket_n = 1;
    for (int l = 0; l < L; ++l) {
        const LayerPlan& p = m->layers[l];
        if (p.shared) {
            // a KV-shared layer reads the pools of its source layer (cache.rs:70-84)
            c->kpool[l] = c->kpool[p.source];
            c->vpool[l] = c->vpool[p.source];
            c->kmap[l] = c->kmap[p.source];
            c->vmap[l] = c->vmap[p.source];
        } else {
            const int pages = p.sliding ? pages_slide : pages_full;
            const size_t bytes = (size_t)pages * p.Nkv * PT * p.D * kes;
            uint8_t *k, *v;
            TRY(dalloc(c, &k, bytes));      // zeroed like the reference's DeviceBuffer::zeroed
            TRY(dalloc(c, &v, bytes));
            c->kpool[l] = k;
            c->vpool[l] = v;
            c->pool_bytes[l] = bytes;
            c->kv_bytes += 2 * (int64_t)bytes;
            ++c->physical_caches;
            if (c->mma_attn) {
                // the pool as a [pages * kv_heads * page_tokens, head_dim] BF16 matrix; boxes of 64 elements x 16 rows
                TRY(encode_bf16_2d(&c->kmap[l], k, (uint64_t)pages * p.Nkv * PT, (uint64_t)p.D, kAmTile));
                TRY(encode_bf16_2d(&c->vmap[l], v, (uint64_t)pages * p.Nkv * PT, (uint64_t)p.D, kAmTile));
            }
        }
        // split-KV geometry of the one-row attention kernel: enough CTAs to fill the GPU a few times over at the longest context
        const int pairs = std::max(1, p.Nkv * B);
        const int want = std::max(1, (8 * m->num_sms + pairs - 1) / pairs);
        // clusters of 16 CTAs (non-portable size) only while one CTA per SM is enough for the whole step
        int cluster_max = 16;
        if (const char* e = getenv("OXG4_ATTN_CLUSTER_MAX")) cluster_max = std::max(1, std::min(16, atoi(e)));
        const int cap_splits = pairs * 16 <= m->num_sms ? cluster_max : std::min(cluster_max, 8);
        auto pow2_floor = [](int v) { int q = 1; while (q * 2 <= v) q *= 2; return q; };
        const int vis = p.sliding ? vis_s : maxf;
        c->attn_splits[l] = pow2_floor(std::max(1, std::min({want, cap_splits, (vis + c->min_split - 1) / c->min_split})));
        smax = std::max(smax, c->attn_splits[l]);
        part_floats = std::max(part_floats, p.Nkv * c->attn_splits[l] * p.G * (p.D + 2));
        ticket_n = std::max(ticket_n, p.Nkv);
    }
    const int R = c->rows_cap = std::max(B, kPrefillRows);
    const int qw = m->qw_max;
    TRY(dalloc(c, &c->tokens, B));
    TRY(dalloc(c, &c->pos, B));
    TRY(dalloc(c, &c->seen, (size_t)B * m->V));
    TRY(dalloc(c, &c->ctl, 1));
    TRY(dalloc(c, &c->rng, B));
    TRY(dalloc(c, &c->hA, (size_t)R * H));
    TRY(dalloc(c, &c->hB, (size_t)R * H));
    TRY(dalloc(c, &c->qkv_raw, (size_t)R * m->qkv_n_max));
    TRY(dalloc(c, &c->attn_out, (size_t)R * qw));
    TRY(dalloc(c, &c->o_raw, (size_t)R * H));
    TRY(dalloc(c, &c->gu_raw, (size_t)R * m->I));
    TRY(dalloc(c, &c->down_raw, (size_t)R * H));
    TRY(dalloc(c, &c->logits, (size_t)B * m->V));
    TRY(dalloc(c, &c->attn_part, (size_t)R * part_floats));
    TRY(dalloc(c, &c->attn_ticket, (size_t)R * ticket_n));
    TRY(dalloc(c, &c->lm_ticket, (size_t)B + 1));
    TRY(dalloc(c, &c->blk_best, (size_t)B * m->num_sms));
    const int chunks = (m->V + kTopkChunk - 1) / kTopkChunk;
    TRY(dalloc(c, &c->topk_stage, (size_t)B * chunks * 64));
    TRY(dalloc(c, &c->tp_ids, (size_t)B * m->tp));
    TRY(dalloc(c, &c->tp_scores, (size_t)B * m->tp));
    TRY(dalloc(c, &c->loc_ids, (size_t)B * 64));
    TRY(dalloc(c, &c->loc_scores, (size_t)B * 64));
    TRY(dalloc(c, &c->tpk_ids, (size_t)B * 64 * m->tp));
    TRY(dalloc(c, &c->tpk_scores, (size_t)B * 64 * m->tp));
    TRY(dalloc(c, &c->best_ids, B));
    TRY(dalloc(c, &c->best_scores, B));
    TRY(dalloc(c, &c->topk_ids, (size_t)B * 64));
    TRY(dalloc(c, &c->topk_scores, (size_t)B * 64));
    if (m->timeline) TRY(dalloc(c, &c->ts_buf, (size_t)kMaxTimeline * 4));
    // prompt chunks
    TRY(dalloc(c, &c->pf_tok, kPrefillRows));
    TRY(dalloc(c, &c->pf_pos, kPrefillRows));
    TRY(dalloc(c, &c->pf_seq, kPrefillRows));
    for (int k = 0; k < 2; ++k) {
        TRY(dalloc(c, &c->pf_grp_row0[k], kAmMaxGroups));
        TRY(dalloc(c, &c->pf_grp_n[k], kAmMaxGroups));
    }
    TRY(dalloc(c, &c->last_h, (size_t)B * H));
    TRY(dalloc(c, &c->last_raw, (size_t)B * H));
    TRY(dalloc(c, &c->last_x, (size_t)B * H));
    CK(cudaMallocHost(&c->h_pf_tok, sizeof(uint32_t) * kPrefillRows));
    CK(cudaMallocHost(&c->h_pf_meta, sizeof(int32_t) * (2 * kPrefillRows + 4 * kAmMaxGroups)));
    {
        std::vector<int32_t> r0(B), ones(B, 1);
        for (int b = 0; b < B; ++b) r0[b] = b;
        TRY(dalloc(c, &c->dec_grp_row0, B));
        TRY(dalloc(c, &c->dec_grp_n, B));
        CK(cudaMemcpy(c->dec_grp_row0, r0.data(), B * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(c->dec_grp_n, ones.data(), B * 4, cudaMemcpyHostToDevice));
    }
    TRY(dalloc(c, &c->tc_err, 1));
    if (c->mma_attn) {
        TRY(attn_mma_setup());
        int kvh_max = 1;
        for (auto& p : m->layers) kvh_max = std::max(kvh_max, p.Nkv);
        TRY(dalloc(c, &c->q_hl, (size_t)R * 2 * m->qw_max));
        const int warps = m->num_sms * 4;                       // upper bound of the consumer warps of a launch
        TRY(dalloc(c, &c->am_part, ((size_t)std::min(R, kAmMaxGroups) * kvh_max + warps) * kAmRows * (m->Dmax + 2)));
        TRY(dalloc(c, &c->am_pre, (size_t)kAmMaxGroups + 1));
    }
    // models with per-layer embeddings run through the small-batch kernels only (the extra projections per layer
    // are tiny and have no tcgen05 variant)
    c->tc_ok = m->es == 2 && m->P == 0 && getenv("OXG4_DISABLE_TCGEN05") == nullptr;
    c->use_tc = c->tc_ok && B >= 8 && B <= kPrefillRows;       // up to 256 sequences: row blocks of 128 / 256 (UMMA N)
    c->ls_qkv.assign(L, 1);
    c->ls_o.assign(L, 1);
    c->lps_qkv.assign(L, 1);
    c->lps_o.assign(L, 1);
    if (m->P > 0) {
        const size_t lp = (size_t)L * m->P;
        TRY(dalloc(c, &c->ple_emb, (size_t)R * H));
        TRY(dalloc(c, &c->ple_ctx, (size_t)R * lp));
        TRY(dalloc(c, &c->ple_packed, (size_t)R * lp));
        TRY(dalloc(c, &c->ple_h, (size_t)R * H));
        TRY(dalloc(c, &c->ple_gate, (size_t)R * m->P));
        TRY(dalloc(c, &c->ple_act, (size_t)R * m->P));
        TRY(dalloc(c, &c->ple_raw, (size_t)R * H));
    }
    if (c->tc_ok) {
        TRY(tc_gemm_setup());
        const int sms = m->num_sms;
        auto tiles = [](int n) { return (n + kTcTileM - 1) / kTcTileM; };
        auto kbs = [](int k) { return (k + kTcTileK - 1) / kTcTileK; };
        const int Bd = std::min(B, kPrefillRows);
        size_t qkv_part_n = 1, o_part_n = 1;
        auto rows_splits = [&](int sd, int sp) { return (size_t)std::max(sd * B, sp * kPrefillRows); };
        for (int l = 0; l < L; ++l) {
            const LayerPlan& p = m->layers[l];
            c->ls_qkv[l] = tc_pick_splits(tiles(p.qkv_n), kbs(H), sms, Bd, p.qkv_n, H);
            c->ls_o[l] = tc_pick_splits(tiles(H), kbs(p.qw), sms, Bd, H, p.qw);
            // a full chunk is one 256-row block per weight tile (UMMA N = 256): K-splits fill the SMs where a projection
            // has few tiles; their partial outputs are cheap next to the tensor-core work of 256 rows
            c->lps_qkv[l] = tc_pick_splits(tiles(p.qkv_n), kbs(H), sms, kPrefillRows, p.qkv_n, H, 1.0);
            c->lps_o[l] = tc_pick_splits(tiles(H), kbs(p.qw), sms, kPrefillRows, H, p.qw, 1.0);
            qkv_part_n = std::max(qkv_part_n, rows_splits(c->ls_qkv[l], c->lps_qkv[l]) * p.qkv_n);
            o_part_n = std::max(o_part_n, rows_splits(c->ls_o[l], c->lps_o[l]) * H);
        }
        c->s_gu = tc_pick_splits(2 * tiles(m->I), kbs(H), sms, Bd, 2 * m->I, H);
        c->s_down = tc_pick_splits(tiles(H), kbs(m->I), sms, Bd, H, m->I);
        c->ps_gu = tc_pick_splits(2 * tiles(m->I), kbs(H), sms, kPrefillRows, 2 * m->I, H, 1.0);
        c->ps_down = tc_pick_splits(tiles(H), kbs(m->I), sms, kPrefillRows, H, m->I, 1.0);
        TRY(dalloc(c, &c->x_h, (size_t)R * H));
        TRY(dalloc(c, &c->x_a, (size_t)R * qw));
        TRY(dalloc(c, &c->x_i, (size_t)R * m->I));
        TRY(dalloc(c, &c->qkv_part, qkv_part_n));
        TRY(dalloc(c, &c->o_part, o_part_n));
        TRY(dalloc(c, &c->gu_part, rows_splits(c->s_gu, c->ps_gu) * 2 * m->I));
        TRY(dalloc(c, &c->down_part, rows_splits(c->s_down, c->ps_down) * H));
        if (m->tp > 1 && c->use_tc && B <= 64) {
            const size_t bytes = sizeof(float) * 2 * (size_t)m->tp * B * H + sizeof(unsigned int) * 2 * kMaxTp;
            CK(cudaMalloc(&c->px_block, bytes));          // own allocation: its IPC handle is exported
            CK(cudaMemset(c->px_block, 0, bytes));
            TRY(dalloc(c, &c->px_local, 8));
        }
    }
    CK(cudaMallocHost(&c->h_tokens, sizeof(uint32_t) * B));
    CK(cudaMallocHost(&c->h_ctl, sizeof(StepCtl)));
    CK(cudaMallocHost(&c->h_ids, sizeof(uint32_t) * B * 64));
    CK(cudaMallocHost(&c->h_scores, sizeof(float) * B * 64));
    CK(cudaEventCreate(&c->ev0));
    CK(cudaEventCreate(&c->ev1));
    CK(cudaDeviceSynchronize());
    return OXG4_OK;
}

extern "C" void oxg4_cache_destroy(oxg4_cache* c) {
    if (!c) return;
    {
        auto& live = c->m->caches;
        live.erase(std::remove(live.begin(), live.end(), c), live.end());
    }
    cudaSetDevice(c->m->device);
    cudaStreamSynchronize(c->m->stream);
    for (auto& g : c->graphs) {
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
        if (g.second.graph) cudaGraphDestroy(g.second.graph);
    }
    for (int r = 0; r < kMaxTp; ++r)
        if (c->px_peer_base[r] && c->px_peer_base[r] != c->px_block) cudaIpcCloseMemHandle(c->px_peer_base[r]);
    if (c->px_block) cudaFree(c->px_block);
    for (void* p : c->owned) cudaFree(p);
    if (c->h_tokens) cudaFreeHost(c->h_tokens);
    if (c->h_pf_tok) cudaFreeHost(c->h_pf_tok);
    if (c->h_pf_meta) cudaFreeHost(c->h_pf_meta);
    if (c->h_ctl) cudaFreeHost(c->h_ctl);
    if (c->h_ids) cudaFreeHost(c->h_ids);
    if (c->h_scores) cudaFreeHost(c->h_scores);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    delete c;
}

extern "C" int32_t oxg4_cache_create(oxg4_model* m, int32_t batch, const int32_t* max_seq, int32_t page_tokens,
                                     int32_t kv_dtype, oxg4_cache** out) {
    if (!m || !max_seq || !out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (!m->finalized) return fail(OXG4_INVALID_ARGUMENT, "model is not finalized");
    if (batch <= 0) return fail(OXG4_INVALID_SHAPE, "batch must be positive");
    for (int b = 0; b < batch; ++b)
        if (max_seq[b] <= 0) return fail(OXG4_INVALID_SHAPE, "zero max_sequence");     // cache.rs:36-38
    if (page_tokens <= 0) return fail(OXG4_INVALID_SHAPE, "page_tokens must be positive");
    if (kv_dtype != OXG4_F32 && kv_dtype != OXG4_BF16) return fail(OXG4_INVALID_ARGUMENT, "kv_dtype must be OXG4_F32 or OXG4_BF16");
    TRY(bind_device(m));
    oxg4_cache* c = new oxg4_cache();
    c->m = m;
    c->B = batch;
    c->PT = page_tokens;
    c->kv_dtype = kv_dtype;
    c->max_seq.assign(max_seq, max_seq + batch);
    c->pos_host.assign(batch, 0);
    m->caches.push_back(c);
    int32_t s = cache_build(c);
    if (s != OXG4_OK) {
        std::string keep = g_err;
        oxg4_cache_destroy(c);
        g_err = keep;
        return s;
    }
    *out = c;
    return OXG4_OK;
}

extern "C" int32_t oxg4_cache_tp_export(oxg4_cache* c, void* handle_out_64) {
    if (!c || !handle_out_64) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (!c->px_block) return fail(OXG4_UNSUPPORTED, "this cache table has no peer exchange buffer (needs tp_size > 1 and 8..64 sequences)");
    TRY(bind_device(c->m));
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, c->px_block));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle_out_64, &h, 64);
    return OXG4_OK;
}

extern "C" int32_t oxg4_cache_tp_connect(oxg4_cache* c, const void* handles) {
    if (!c || !handles) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (!c->px_block) return fail(OXG4_UNSUPPORTED, "this cache table has no peer exchange buffer");
    if (c->peer_ready) return OXG4_OK;
    oxg4_model* m = c->m;
    TRY(bind_device(m));
    for (int r = 0; r < m->tp; ++r) {
        if (r == m->tp_rank) { c->px_peer_base[r] = c->px_block; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * 64, 64);
        void* p = nullptr;
        CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->px_peer_base[r] = p;
    }
    const size_t bh = (size_t)c->B * m->H;
    for (int kind = 0; kind < 2; ++kind) {
        PeerExchange& x = c->px[kind];
        x.tp = m->tp;
        x.rank = m->tp_rank;
        for (int r = 0; r < m->tp; ++r) {
            char* base = (char*)c->px_peer_base[r];
            x.push[r] = (float*)base + ((size_t)kind * m->tp + m->tp_rank) * bh;
            x.flags[r] = (unsigned int*)(base + sizeof(float) * 2 * m->tp * bh) + (size_t)kind * kMaxTp;
        }
        x.gathered = (const float*)c->px_block + (size_t)kind * m->tp * bh;
        x.seq = c->px_local + kind;
        x.ticket = c->px_local + 2 + kind;
        x.status = (int*)(c->px_local + 4);
    }
    c->peer_ready = getenv("OXG4_TP_NCCL") == nullptr;
    // graphs captured before the connection used the NCCL path
    for (auto& g : c->graphs) {
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
        if (g.second.graph) cudaGraphDestroy(g.second.graph);
    }
    c->graphs.clear();
    return OXG4_OK;
}

extern "C" int32_t oxg4_cache_info_get(const oxg4_cache* c, oxg4_cache_info* o) {
    if (!c || !o) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    o->batch = c->B;
    o->layer_count = c->m->cfg.num_hidden_layers;
    o->physical_cache_count = c->physical_caches;
    o->shared_layer_count = c->m->cfg.num_hidden_layers - c->physical_caches;
    o->page_tokens = c->PT;
    o->kv_dtype = c->kv_dtype;
    o->kv_bytes = c->kv_bytes;
    return OXG4_OK;
}

extern "C" int32_t oxg4_cache_position(const oxg4_cache* c, int32_t b) {
    if (!c || b < 0 || b >= c->B) return -1;
    return c->pos_host[b];
}

extern "C" int32_t oxg4_cache_reset(oxg4_cache* c) {
    if (!c) return fail(OXG4_INVALID_ARGUMENT, "null cache");
    TRY(bind_device(c->m));
    cudaStream_t st = c->m->stream;
    CK(cudaMemsetAsync(c->pos, 0, sizeof(int32_t) * c->B, st));
    CK(cudaMemsetAsync(c->seen, 0, (size_t)c->B * c->m->V, st));
    CK(cudaStreamSynchronize(st));
    std::fill(c->pos_host.begin(), c->pos_host.end(), 0);
    return OXG4_OK;
}

// ------------------------------------------------------------------------------------------------
// tcgen05 projection: tensor maps, split choice, launch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int32_t encode_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) return fail(OXG4_CUDA, "Gemma 4 CUDA error: cuTensorMapEncodeTiled is unavailable");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcTileK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(OXG4_CUDA, "Gemma 4 CUDA error: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return OXG4_OK;
}

// out[B, N] = x[B, K] . W[N, K]^T on device pointers (BF16 in, f32 out), B <= 64, K a multiple of 8.
// K-splits for a tcgen05 projection: work units = tiles * S should fill the grid in whole rounds;
// the S partial outputs cost S * B * n * 8 bytes of extra traffic, kept under ~30 % of the weights.
static int tc_pick_splits(int tiles, int kblocks, int grid, int B, int n_total, int K, double max_extra) {
    int best = 1;
    double best_score = -1.0;
    for (int S = 1; S <= 16 && S <= kblocks / 2 + (kblocks < 2 ? 1 : 0); ++S) {
        const double units = (double)tiles * S;
        const double rounds = std::ceil(units / grid);
        const double eff = units / (rounds * grid);
        const double extra = S == 1 ? 0.0 : (double)S * B * n_total * 8.0 / ((double)n_total * K * 2.0);
        if (extra > max_extra) break;
        const double score = eff / (1.0 + extra);
        if (score > best_score + 1e-9) { best_score = score; best = S; }
    }
    // no split may be empty: an empty unit would hand stale accumulator columns to the epilogue
    const int kbps = (kblocks + best - 1) / best;
    return (kblocks + kbps - 1) / kbps;
}

// out[S, B, n_mats * N] = per-split partials of x[B, K] . W_m[N, K]^T on device pointers (BF16 in, f32 out).
static int32_t tc_gemm_launch(const void* w_dev, const void* w1_dev, const void* x_dev, int N, int K, int B, int S,
                              float* out_dev, int ld, int col0, int* err_dev, int num_sms, cudaStream_t st, bool pdl) {
    if (B < 1 || B > kPrefillRows || K % 8 != 0)
        return fail(OXG4_INVALID_SHAPE, "tcgen05 projection: 1..%d rows and K %% 8 == 0 required", kPrefillRows);
    const int bn = B <= 16 ? 16 : (B <= 32 ? 32 : (B <= 64 ? 64 : (B <= 128 ? 128 : 256)));
    CUtensorMap mw, mw1, mx;
    TRY(encode_bf16_2d(&mw, w_dev, (uint64_t)N, (uint64_t)K, kTcTileM));
    TRY(encode_bf16_2d(&mw1, w1_dev ? w1_dev : w_dev, (uint64_t)N, (uint64_t)K, kTcTileM));
    TRY(encode_bf16_2d(&mx, x_dev, (uint64_t)B, (uint64_t)K, (uint32_t)bn));
    const int kblocks = (K + kTcTileK - 1) / kTcTileK;
    TcGemmArgs a{};
    a.N = N; a.K = K; a.B = B;
    a.n_mats = w1_dev ? 2 : 1;
    a.S = S;
    a.TB = (B + bn - 1) / bn;
    a.kb_per_split = (kblocks + S - 1) / S;
    a.out = out_dev;
    a.ld = ld;
    a.col0 = col0;
    a.err = err_dev;
    const int units = ((N + kTcTileM - 1) / kTcTileM) * a.n_mats * S * a.TB;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(units, num_sms));
    cfg.blockDim = dim3(kTcThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    if (bn == 16) {
        cfg.dynamicSmemBytes = tc_gemm_smem_bytes<16>();
        e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<16>, mw, mw1, mx, a);
    } else if (bn == 32) {
        cfg.dynamicSmemBytes = tc_gemm_smem_bytes<32>();
        e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<32>, mw, mw1, mx, a);
    } else if (bn == 64) {
        cfg.dynamicSmemBytes = tc_gemm_smem_bytes<64>();
        e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<64>, mw, mw1, mx, a);
    } else if (bn == 128) {
        cfg.dynamicSmemBytes = tc_gemm_smem_bytes<128>();
        e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<128>, mw, mw1, mx, a);
    } else {
        cfg.dynamicSmemBytes = tc_gemm_smem_bytes<256>();
        e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<256>, mw, mw1, mx, a);
    }
    CK(e);
    return OXG4_OK;
}

static int32_t tc_gemm_setup() {
    TRY(allow_big_smem(tc_gemm_kernel<16>));
    TRY(allow_big_smem(tc_gemm_kernel<32>));
    TRY(allow_big_smem(tc_gemm_kernel<64>));
    TRY(allow_big_smem(tc_gemm_kernel<128>));
    TRY(allow_big_smem(tc_gemm_kernel<256>));
    return OXG4_OK;
}


// ------------------------------------------------------------------------------------------------
// one decode step
// ------------------------------------------------------------------------------------------------
struct Launcher {
    oxg4_model* m;
    unsigned long long* ts_base = nullptr;
    int cluster_x = 0;            // > 0: launch the next kernel with thread-block clusters of this many CTAs along x
    bool coop = false;            // launch the next kernel cooperatively (all CTAs resident at once), without PDL
    int kernels = 0;
    unsigned long long* ts() const { return (ts_base && kernels < kMaxTimeline) ? ts_base + (size_t)kernels * 4 : nullptr; }
    int32_t status = OXG4_OK;

    template <typename... KArgs, typename... Args>
    void go(const char* kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
        if (status != OXG4_OK) return;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if (m->profiling) {
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            cudaEventRecord(e0, m->stream);
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = m->stream;
        cudaLaunchAttribute attr[2];
        int na = 0;
        if (coop) {
            attr[na].id = cudaLaunchAttributeCooperative;
            attr[na].val.cooperative = 1;
            ++na;
        } else if (m->use_pdl && !m->profiling) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        }
        if (cluster_x > 0) {
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = cluster_x;
            attr[na].val.clusterDim.y = 1;
            attr[na].val.clusterDim.z = 1;
            ++na;
        }
        cfg.attrs = attr;
        cfg.numAttrs = na;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
        if (e != cudaSuccess) {
            status = fail(OXG4_CUDA, "Gemma 4 CUDA error: launch of %s failed: %s", kind, cudaGetErrorString(e));
            return;
        }
        if (m->profiling) {
            cudaEventRecord(e1, m->stream);
            m->prof_events.push_back({kind, {e0, e1}});
        }
        ++kernels;
    }

    // tcgen05 batched projection (csrc/tc_gemm.cuh): partials [S, B, ld] of x . W^T
    void tc(const char* kind, oxg4_cache* c, int rows, const void* w0, const void* w1, const uint16_t* x, int N, int K,
            int S, float* out, int ld, int col0) {
        if (status != OXG4_OK) return;
        cudaEvent_t e0, e1;
        prof_begin(e0, e1);
        status = tc_gemm_launch(w0, w1, x, N, K, rows, S, out, ld, col0, c->tc_err, m->num_sms, m->stream,
                                m->use_pdl && !m->profiling);
        if (status != OXG4_OK) return;
        prof_end(kind, e0, e1);
        ++kernels;
    }

    // profiling steps bracket every launch (collectives included) with a pair of events on the model's stream
    void prof_begin(cudaEvent_t& e0, cudaEvent_t& e1) {
        e0 = e1 = nullptr;
        if (!m->profiling) return;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, m->stream);
    }
    void prof_end(const char* kind, cudaEvent_t e0, cudaEvent_t e1) {
        if (!m->profiling) return;
        cudaEventRecord(e1, m->stream);
        m->prof_events.push_back({kind, {e0, e1}});
    }

    // in-place sum over the tensor-parallel ranks (one NCCL all-reduce on the model's stream)
    void allreduce(float* buf, size_t count) {
        if (status != OXG4_OK || m->tp == 1) return;
        if (!m->comm) { status = fail(OXG4_NCCL, "tensor-parallel model used before oxg4_model_tp_init"); return; }
        cudaEvent_t e0, e1;
        prof_begin(e0, e1);
        const int rc = nccl().AllReduce(buf, buf, count, NcclApi::kFloat32, NcclApi::kSum, m->comm, m->stream);
        if (rc != 0) { status = fail(OXG4_NCCL, "NCCL: ncclAllReduce: %s", nccl().GetErrorString(rc)); return; }
        prof_end("allreduce", e0, e1);
        ++kernels;
    }
    void allgather(const void* src, void* dst, size_t bytes_per_rank) {
        if (status != OXG4_OK || m->tp == 1) return;
        if (!m->comm) { status = fail(OXG4_NCCL, "tensor-parallel model used before oxg4_model_tp_init"); return; }
        cudaEvent_t e0, e1;
        prof_begin(e0, e1);
        const int rc = nccl().AllGather(src, dst, bytes_per_rank, NcclApi::kUint8, m->comm, m->stream);
        if (rc != 0) { status = fail(OXG4_NCCL, "NCCL: ncclAllGather: %s", nccl().GetErrorString(rc)); return; }
        prof_end("allgather", e0, e1);
        ++kernels;
    }
};

template <typename WT>
static void (*pick_gemv(int nb, int pro, int epi))(const GemvArgs) {
#define PICK(NB)                                                                              \
    if (pro == PRO_NORM && epi == EPI_STORE) return gemv_kernel<WT, NB, PRO_NORM, EPI_STORE>;       \
    if (pro == PRO_PLAIN && epi == EPI_STORE) return gemv_kernel<WT, NB, PRO_PLAIN, EPI_STORE>;     \
    if (pro == PRO_NORM && epi == EPI_GATEUP) return gemv_kernel<WT, NB, PRO_NORM, EPI_GATEUP>;     \
    if (pro == PRO_NORM && epi == EPI_LOGITS) return gemv_kernel<WT, NB, PRO_NORM, EPI_LOGITS>;
    if (nb == 1) { PICK(1) }
    if constexpr (sizeof(WT) == 4) {      // BF16 weights with more than one row use the tensor-core kernel
        if (nb == 2) { PICK(2) }
        if (nb == 4) { PICK(4) }
    }
#undef PICK
    return nullptr;
}

template <int MB>
static void (*pick_mma(int pro, int epi))(const GemvArgs) {
    if (pro == PRO_NORM && epi == EPI_STORE) return gemv_mma_kernel<MB, PRO_NORM, EPI_STORE>;
    if (pro == PRO_PLAIN && epi == EPI_STORE) return gemv_mma_kernel<MB, PRO_PLAIN, EPI_STORE>;
    if (pro == PRO_NORM && epi == EPI_GATEUP) return gemv_mma_kernel<MB, PRO_NORM, EPI_GATEUP>;
    if (pro == PRO_NORM && epi == EPI_LOGITS) return gemv_mma_kernel<MB, PRO_NORM, EPI_LOGITS>;
    return nullptr;
}

static void launch_gemv(Launcher& ln, const char* kind, oxg4_cache* c, int rows, GemvArgs a, const GemvPlan& p, int pro,
                        int epi) {
    oxg4_model* m = c->m;
    const int B = rows;
    a.N = p.N;
    a.K = p.K;
    a.cpr = p.cpr;
    a.slots = p.slots;
    a.B = B;
    a.eps = m->cfg.rms_norm_eps;
    a.ts = ln.ts();
    a.pf_cap_kb = m->pf_cap_kb;
    if (epi == EPI_GATEUP && m->pf_cap_gu_kb >= 0) a.pf_cap_kb = m->pf_cap_gu_kb;
    if (!strcmp(kind, "down") && m->pf_cap_down_kb >= 0) a.pf_cap_kb = m->pf_cap_down_kb;
    if (pro == PRO_NORM && p.K > std::min(kGemvMaxJ * kGemvThreads, kSimtMaxJ * kSimtThreads)) {
        ln.status = fail(OXG4_UNSUPPORTED, "hidden size above %d is not supported",
                         std::min(kGemvMaxJ * kGemvThreads, kSimtMaxJ * kSimtThreads));
        return;
    }
    const size_t limit = 226 * 1024;
    if (m->es == 2 && B > 1) {
        // tensor-core kernel: as many activation rows per pass as shared memory allows (at most 16)
        auto need = [&](int nb) { return (((size_t)nb * mma_x_stride(p.K) * 2 + 15) & ~(size_t)15) + 128 + (size_t)2 * mma_rows_per_pass(nb > 8 ? 16 : 8) * kGemvWarps * nb * 4; };
        int bpp = std::min(B, 16);
        while (bpp > 1 && need(bpp) > limit) --bpp;
        if (need(bpp) > limit) {
            ln.status = fail(OXG4_UNSUPPORTED, "projection %s needs %zu bytes of shared memory", kind, need(bpp));
            return;
        }
        a.bpp = bpp;
        auto fn = bpp <= 8 ? pick_mma<8>(pro, epi) : pick_mma<16>(pro, epi);
        dim3 grid(p.grid, (B + bpp - 1) / bpp, 1);
        ln.go(kind, fn, grid, dim3(kGemvThreads), need(bpp), a);
        return;
    }
    // one activation row with BF16 weights, or f32 weights: SIMT kernel
    const int nb = B >= 3 ? 4 : B;
    a.bpp = nb;
    size_t smem = (size_t)nb * p.K * m->es + (size_t)nb * 32 * 4;
    size_t extra = (size_t)p.rows_max * p.slots * nb * 4;
    extra = std::max(extra, (size_t)nb * kSimtWarps * sizeof(Cand));
    smem += extra;
    if (smem > limit) {
        ln.status = fail(OXG4_UNSUPPORTED, "projection %s needs %zu bytes of shared memory", kind, smem);
        return;
    }
    auto fn = m->es == 2 ? pick_gemv<uint16_t>(nb, pro, epi) : pick_gemv<float>(nb, pro, epi);
    dim3 grid(epi == EPI_LOGITS ? m->p_lm_simt_grid : p.grid, (B + nb - 1) / nb, 1);
    ln.go(kind, fn, grid, dim3(kSimtThreads), smem, a);
}

template <typename KT>
static void (*pick_attn(int D, int G, bool cl, bool deep))(const AttnArgs) {
#define PA1(DD, GG)                                                                       \
    if (D == DD && G == GG) {                                                             \
        if (cl && deep) return attn_decode_kernel<KT, DD, GG, true, true>;                \
        return cl ? attn_decode_kernel<KT, DD, GG, true> : attn_decode_kernel<KT, DD, GG, false>; \
    }
#define PA(DD) PA1(DD, 1) PA1(DD, 2) PA1(DD, 4) PA1(DD, 8)
    PA(64) PA(128) PA(256)
#undef PA
#undef PA1
    return nullptr;
}

typedef void (*AttnMmaFn)(const CUtensorMap, const CUtensorMap, const AttnMmaArgs);
typedef void (*AttnMergeFn)(const AttnMmaArgs);
static void pick_attn_mma(int D, int G, AttnMmaFn* fn, AttnMergeFn* merge, size_t* smem, int* ncw) {
    *fn = nullptr;
#define PM1(DD, GG)                                            \
    if (D == DD && G == GG) {                                  \
        *fn = attn_mma_kernel<DD, GG>;                         \
        *merge = attn_merge_kernel<DD, GG>;                    \
        *smem = attn_mma_smem_bytes<DD>();                     \
        *ncw = AmGeom<DD>::NCW;                                \
    }
#define PM(DD) PM1(DD, 1) PM1(DD, 2) PM1(DD, 4) PM1(DD, 8)
    PM(64) PM(128) PM(256)
#undef PM
#undef PM1
}

static int32_t attn_mma_setup() {
#define SM1(DD, GG) TRY(allow_big_smem(attn_mma_kernel<DD, GG>));
#define SM(DD) SM1(DD, 1) SM1(DD, 2) SM1(DD, 4) SM1(DD, 8)
    SM(64) SM(128) SM(256)
#undef SM
#undef SM1
    return OXG4_OK;
}

// The rows one pass over the layers carries: the sequences of a decode step, or up to kPrefillRows prompt
// tokens (a chunk), each with its token id, absolute position and, for a chunk, the sequence it belongs to.
struct RowSet {
    int R = 0;
    const uint32_t* tok = nullptr;       // device [R]; kInactiveToken rows sit a decode step out
    const int32_t* pos = nullptr;        // device [R]
    const int32_t* seq = nullptr;        // device [R], or null: row r is sequence r
    bool chunk = false;                  // prompt chunk: all K/V rows are appended before any token attends
    // attention groups (consecutive tokens of one sequence), per layer kind (0 sliding, 1 global): a group holds
    // up to 8 / G tokens and G (query heads per KV head) may differ between the kinds
    const int32_t* grp_row0[2] = {nullptr, nullptr};
    const int32_t* grp_n[2] = {nullptr, nullptr};
    int NG[2] = {0, 0};
};

// Launches every kernel of one step on the model's stream (eagerly or under stream capture).
struct TraceCtx {
    const float* inject_dev;   // [L][B][H] layer inputs to force, or null
    float* trace_dev;          // [L+1][B][H] receives every layer's input and the final hidden state
};

// q/k norm + RoPE + v norm + KV append + attention of layer l for the rows of `rs` (decode.rs:99-157,
// 176-325). qkv: [qkv_splits, R, qkv_n] projection output; the result goes to c->attn_out (+ BF16 copy).
static void launch_attention(Launcher& ln, oxg4_cache* c, const RowSet& rs, int l, const float* qkv, int qkv_splits,
                             uint16_t* out_bf16, bool many_rows) {
    oxg4_model* m = c->m;
    const LayerPlan& p = m->layers[l];
    const int D = p.D, R = rs.R, kind = p.sliding ? 0 : 1;
    const int32_t* page_table = p.sliding ? c->pt_slide : c->pt_full;
    const int pps = p.sliding ? c->pps_slide : c->pps_full;
    const int32_t* cap = p.sliding ? c->cap_slide : c->cap_full;
    const int window = p.sliding ? m->cfg.sliding_window : 0x7fffffff;
    const bool use_mma = c->mma_attn && (many_rows || rs.chunk);
    // K and V of the rows are in the cache before the attention kernel starts: rows of a prompt chunk (appended by
    // qkv_post_kernel), and every row of a KV-shared layer (its source layer appended them earlier in the step)
    const bool kv_in_cache = rs.chunk || p.shared;
    if (use_mma || (rs.chunk && !p.shared)) {
        // norms, RoPE and the K/V append of every row first (a chunk's later tokens are visible to none of its earlier ones
        // only through the causal mask, so all rows may be in the cache before attention starts)
        QkvPostArgs q{};
        q.qkv = qkv; q.qkv_n = p.qkv_n; q.splits = qkv_splits; q.R = R; q.Nq = m->Nq; q.Nkv = p.Nkv;
        q.q_norm = p.q_norm; q.k_norm = p.k_norm; q.inv_freq = p.inv_freq; q.rotary_half = p.rotary_dim / 2;
        q.eps = m->cfg.rms_norm_eps;
        q.row_pos = rs.pos; q.row_seq = rs.seq; q.row_tok = rs.tok;
        q.kpool = c->kpool[l]; q.vpool = c->vpool[l];
        q.page_table = page_table; q.pages_per_seq = pps; q.page_tokens = c->PT; q.cap = cap;
        q.q_hl = use_mma ? c->q_hl : nullptr;
        q.write_kv = p.shared ? 0 : 1;
        const int per_row = (use_mma ? m->Nq : 0) + (p.shared ? 0 : 2 * p.Nkv);
        void (*fn)(const QkvPostArgs) = nullptr;
        if (c->kv_dtype == OXG4_BF16) fn = D == 64 ? qkv_post_kernel<uint16_t, 64> : D == 128 ? qkv_post_kernel<uint16_t, 128> : qkv_post_kernel<uint16_t, 256>;
        else fn = D == 64 ? qkv_post_kernel<float, 64> : D == 128 ? qkv_post_kernel<float, 128> : qkv_post_kernel<float, 256>;
        ln.go("qkv_post", fn, dim3((R * per_row + 3) / 4), dim3(128), 0, q);
    }
    if (use_mma) {
        AttnMmaArgs a{};
        a.q_hl = c->q_hl; a.Nq = m->Nq; a.Nkv = p.Nkv; a.NG = rs.NG[kind];
        a.grp_row0 = rs.grp_row0[kind]; a.grp_n = rs.grp_n[kind];
        a.row_pos = rs.pos; a.row_seq = rs.seq; a.row_tok = rs.tok;
        a.page_table = page_table; a.pages_per_seq = pps; a.page_tokens = c->PT; a.cap = cap;
        a.window = window;
        a.part_rows = rs.chunk ? kAmRows : p.G;
        a.part = c->am_part;
        a.pre_out = c->am_pre;
        a.err = c->tc_err;
        a.out = c->attn_out;
        a.out_bf16 = out_bf16;
        AttnMmaFn fn;
        AttnMergeFn merge;
        size_t smem;
        int ncw;
        pick_attn_mma(D, p.G, &fn, &merge, &smem, &ncw);
        a.total_warps = m->num_sms * ncw;
        ln.go("attn", fn, dim3(m->num_sms), dim3((ncw + 1) * 32), smem, c->kmap[l], c->vmap[l], a);
        ln.go("attn_merge", merge, dim3(rs.NG[kind] * p.Nkv), dim3(128), 0, a);
        return;
    }
    AttnArgs a{};
    a.qkv = qkv;
    a.qkv_splits = qkv_splits;
    a.out_bf16 = out_bf16;
    a.qkv_n = p.qkv_n;
    a.B = R;
    a.Nq = m->Nq;
    a.Nkv = p.Nkv;
    a.q_norm = p.q_norm;
    a.k_norm = p.k_norm;
    a.inv_freq = p.inv_freq;
    a.rotary_half = p.rotary_dim / 2;
    a.eps = m->cfg.rms_norm_eps;
    a.pos = rs.pos;
    a.tokens = rs.tok;
    a.row_seq = rs.seq;
    a.window = window;
    a.kpool = c->kpool[l];
    a.vpool = c->vpool[l];
    a.page_table = page_table;
    a.pages_per_seq = pps;
    a.page_tokens = c->PT;
    a.cap = cap;
    a.n_splits = c->attn_splits[l];
    a.min_split = c->min_split;
    a.part = c->attn_part;
    a.ticket = c->attn_ticket;
    a.out = c->attn_out;
    if ((m->far_prefetch & 2) && !rs.chunk) {
        // the attention kernel of a one-sequence step moves almost no bytes: HBM is idle, so it pulls the up
        // projection's weights (or as much as the cap allows) into L2 for the kernel after next
        a.pf_ptr = p.wup;
        a.pf_bytes = std::min<unsigned long long>((unsigned long long)m->I * m->H * m->es, (unsigned long long)m->far_prefetch_mb << 20);
    }
    a.ts = ln.ts();
    a.ts_mid = ln.ts_base ? ln.ts_base + 4 * (size_t)(kMaxTimeline - 1 - l) : nullptr;   // extra stamps, from the end of the buffer
    const bool cl = !kv_in_cache;                // decode: cluster merge; K/V already in the cache: ticket merge
    // few CTAs (one sequence): 16 warps each to cut latency; many CTAs: 4 warps each so that several
    // fit on an SM (the kernel needs ~90 registers per thread)
    const int aw = (a.n_splits * p.Nkv * R <= m->num_sms) ? kAttnWarps : 4;
    // more K/V rows in flight per warp when latency is all that counts (with more than two query heads
    // per kv head the extra rows would spill registers)
    const bool deep = cl && aw == kAttnWarps && p.G <= 2;
    auto fn = c->kv_dtype == OXG4_BF16 ? pick_attn<uint16_t>(D, p.G, cl, deep) : pick_attn<float>(D, p.G, cl, deep);
    const size_t smem = sizeof(float) * (size_t)(p.G * D + 2 * D + 2 * aw * p.G + aw * p.G * D + p.G * (D + 2) + D);
    ln.cluster_x = cl ? a.n_splits : 0;
    ln.go("attn", fn, dim3(a.n_splits, p.Nkv, R), dim3(aw * 32), smem, a);
    ln.cluster_x = 0;
}

// Per-layer embeddings (Gemma4-E; ple.rs). Once per pass: the packed per-layer inputs of every row.
static void ple_prepare(oxg4_cache* c, Launcher& ln, const RowSet& rs) {
    oxg4_model* m = c->m;
    const int R = rs.R, H = m->H, L = m->cfg.num_hidden_layers, P = m->P;
    const float scale = sqrtf((float)H);
    if (m->es == 2)
        ln.go("ple", ple_embed_rows_kernel<uint16_t>, dim3(R), dim3(256), 0, H, (const uint16_t*)m->embed, rs.tok, scale, c->ple_emb);
    else
        ln.go("ple", ple_embed_rows_kernel<float>, dim3(R), dim3(256), 0, H, (const float*)m->embed, rs.tok, scale, c->ple_emb);
    GemvArgs a{};                       // context = bf16(embedding) . per_layer_model_projection^T (ple.rs:85)
    a.W0 = m->ple_model_proj;
    a.in = c->ple_emb;
    a.out = c->ple_ctx;
    launch_gemv(ln, "ple", c, R, a, m->p_ple_ctx, PRO_PLAIN, EPI_STORE);
    const float inv_sqrt_h = 1.0f / sqrtf((float)H), sqrt_p = sqrtf((float)P);
    const dim3 grid((R * L + 3) / 4);
    if (m->es == 2)
        ln.go("ple", ple_pack_kernel<uint16_t>, grid, dim3(128), 0, R, L, P, (const float*)c->ple_ctx, m->ple_proj_norm,
              (const uint16_t*)m->ple_embed, rs.tok, m->cfg.rms_norm_eps, inv_sqrt_h, sqrt_p, c->ple_packed);
    else
        ln.go("ple", ple_pack_kernel<float>, grid, dim3(128), 0, R, L, P, (const float*)c->ple_ctx, m->ple_proj_norm,
              (const float*)m->ple_embed, rs.tok, m->cfg.rms_norm_eps, inv_sqrt_h, sqrt_p, c->ple_packed);
}

// apply_ple of layer l (ple.rs:151-185) after the MLP block: h' = h + rmsnorm(down) is closed here, the branch
// gate -> gelu * per-layer input -> projection is left pending in c->ple_raw; the next kernel's prologue adds
// rmsnorm(branch, post_per_layer_input_norm) and applies layer_scalar.
static void ple_layer(oxg4_cache* c, Launcher& ln, const RowSet& rs, int l) {
    oxg4_model* m = c->m;
    const LayerPlan& p = m->layers[l];
    const int R = rs.R, H = m->H, P = m->P;
    ln.go("ple", ple_close_kernel, dim3(R), dim3(kRowsThreads), 0, H, (const float*)c->hA, (const float*)c->down_raw,
          p.post_ff_ln, m->cfg.rms_norm_eps, c->ple_h);
    {
        GemvArgs a{};
        a.W0 = p.w_ple_gate;
        a.in = c->ple_h;
        a.out = c->ple_gate;
        launch_gemv(ln, "ple", c, R, a, m->p_ple_gate, PRO_PLAIN, EPI_STORE);
    }
    ln.go("ple", ple_act_kernel, dim3((P + kRowsThreads - 1) / kRowsThreads, R), dim3(kRowsThreads), 0, P,
          m->cfg.num_hidden_layers * P, l, (const float*)c->ple_gate, (const float*)c->ple_packed, c->ple_act);
    {
        GemvArgs a{};
        a.W0 = p.w_ple_proj;
        a.in = c->ple_act;
        a.out = c->ple_raw;
        launch_gemv(ln, "ple", c, R, a, m->p_ple_proj, PRO_PLAIN, EPI_STORE);
    }
}

// All layers for the rows of `rs`. On return the last layer's residual update is still pending:
// tcgen05 path: c->hA (+ the partials of the down projection), small-batch path: c->hA + c->down_raw.
static void run_layers(oxg4_cache* c, Launcher& ln, const RowSet& rs, bool use_tc, bool peer, bool last_layer_prefetch,
                       const TraceCtx* tr) {
    oxg4_model* m = c->m;
    const int R = rs.R, L = m->cfg.num_hidden_layers, H = m->H;
    const int s_gu = rs.chunk ? c->ps_gu : c->s_gu, s_down = rs.chunk ? c->ps_down : c->s_down;
    if (m->P > 0) ple_prepare(c, ln, rs);
    for (int l = 0; l < L; ++l) {
        const LayerPlan& p = m->layers[l];
        const int s_qkv = rs.chunk ? c->lps_qkv[l] : c->ls_qkv[l], s_o = rs.chunk ? c->lps_o[l] : c->ls_o[l];
        if (use_tc) {
            // ---- many rows: tcgen05 projections fed by TMA, per-row kernels around them ----
            const int nqkv = p.qkv_n, qw = p.qw;
            auto copy_trace_tc = [&]() {
                if (tr && ln.status == OXG4_OK &&
                    cudaMemcpyAsync(tr->trace_dev + (size_t)l * R * H, c->hB, sizeof(float) * R * H,
                                    cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess)
                    ln.status = fail(OXG4_CUDA, "Gemma 4 CUDA error: trace copy failed");
            };
            RowsNormArgs n{};
            n.B = R; n.H = H;
            n.h_in = c->hA; n.h_out = c->hB;
            n.w_norm = p.input_ln;
            n.scalar = 1.0f;
            n.eps = m->cfg.rms_norm_eps;
            n.x = c->x_h;
            if (l == 0) {
                n.embed = (const uint16_t*)m->embed;
                n.tokens = rs.tok;
                n.embed_scale = sqrtf((float)H);
            } else {
                n.raw = m->tp > 1 ? (peer ? c->px[1].gathered : c->down_raw) : c->down_part;
                n.raw_splits = m->tp > 1 ? (peer ? m->tp : 1) : s_down;
                if (m->tp > 1 && peer) n.px = c->px[1];
                n.w_post = m->layers[l - 1].post_ff_ln;
                n.scalar = m->layers[l - 1].layer_scalar;
            }
            ln.go("norm", rows_norm_kernel, dim3(R), dim3(kRowsThreads), 0, n);
            copy_trace_tc();
            if (tr && tr->inject_dev) {
                RowsNormArgs f = n;                      // layer-wise teacher forcing: forced input, nothing pending
                f.embed = nullptr; f.raw = nullptr; f.w_post = nullptr; f.scalar = 1.0f;
                f.h_in = tr->inject_dev + (size_t)l * R * H;
                ln.go("norm", rows_norm_kernel, dim3(R), dim3(kRowsThreads), 0, f);
            }
            ln.tc("qkv", c, R, p.wqkv, nullptr, c->x_h, nqkv, H, s_qkv, c->qkv_part, nqkv, 0);
            launch_attention(ln, c, rs, l, c->qkv_part, s_qkv, c->x_a, true);
            // row-split projection under tensor parallelism: without K-splits the kernel writes the rank's partial
            // sum straight into the buffer that is all-reduced (one launch less); with the peer-memory exchange
            // the summation kernel is what pushes it to the peers
            const bool direct = m->tp > 1 && !peer && s_o == 1;
            ln.tc("o", c, R, p.wo, nullptr, c->x_a, H, qw, s_o, direct ? c->o_raw : c->o_part, H, 0);
            const size_t bh = (size_t)R * H;
            const dim3 sum_grid((unsigned)((bh / 4 + kRowsThreads - 1) / kRowsThreads));
            PeerExchange none{};
            none.tp = 1;
            const float* xo = peer ? c->px[0].gathered : c->o_raw;        // what the next norm reads
            const int xs = peer ? m->tp : 1;                              // partials to add there
            if (m->tp > 1) {      // add the K-splits locally, then the ranks
                if (!direct)
                    ln.go("sum", sum_splits_kernel, sum_grid, dim3(kRowsThreads), 0, (const float*)c->o_part, s_o, bh,
                          c->o_raw, peer ? c->px[0] : none);
                if (!peer) ln.allreduce(c->o_raw, bh);
            }
            RowsNormArgs n2{};
            n2.B = R; n2.H = H;
            n2.h_in = c->hB; n2.h_out = c->hA;
            n2.raw = m->tp > 1 ? xo : c->o_part;
            n2.raw_splits = m->tp > 1 ? xs : s_o;
            n2.px = (m->tp > 1 && peer) ? c->px[0] : none;
            n2.w_post = p.post_attn_ln;
            n2.scalar = 1.0f;
            n2.w_norm = p.pre_ff_ln;
            n2.eps = m->cfg.rms_norm_eps;
            n2.x = c->x_h;
            ln.go("norm", rows_norm_kernel, dim3(R), dim3(kRowsThreads), 0, n2);
            ln.tc("gateup", c, R, p.wgate, p.wup, c->x_h, m->I, H, s_gu, c->gu_part, 2 * m->I, 0);
            ln.go("geglu", geglu_rows_kernel, dim3((m->I / 4 + kRowsThreads - 1) / kRowsThreads, R), dim3(kRowsThreads), 0, R,
                  m->I, (const float*)c->gu_part, s_gu, c->x_i);
            const bool direct_d = m->tp > 1 && !peer && s_down == 1;
            ln.tc("down", c, R, p.wdown, nullptr, c->x_i, H, m->I, s_down, direct_d ? c->down_raw : c->down_part, H, 0);
            if (m->tp > 1) {
                if (!direct_d)
                    ln.go("sum", sum_splits_kernel, sum_grid, dim3(kRowsThreads), 0, (const float*)c->down_part, s_down, bh,
                          c->down_raw, peer ? c->px[1] : none);
                if (!peer) ln.allreduce(c->down_raw, bh);
            }
            continue;
        }
        {   // input norm + QKV projection (decode.rs:61-98); also closes the previous layer
            GemvArgs a{};
            a.W0 = p.wqkv;
            a.h_in = c->hA;
            a.h_out = c->hB;
            a.w_norm = p.input_ln;
            a.scalar = 1.0f;
            if (l == 0) {
                a.embed = m->embed;
                a.tokens = rs.tok;
                a.embed_scale = sqrtf((float)H);
            } else if (m->P > 0) {
                // the previous layer ended with its per-layer-embedding branch: h = (h' + rmsnorm(branch)) * scalar
                a.h_in = c->ple_h;
                a.raw = c->ple_raw;
                a.w_post = m->layers[l - 1].ple_norm;
                a.scalar = m->layers[l - 1].layer_scalar;
            } else {
                a.raw = c->down_raw;
                a.w_post = m->layers[l - 1].post_ff_ln;
                a.scalar = m->layers[l - 1].layer_scalar;
            }
            a.out = c->qkv_raw;
            if (m->far_prefetch & 1) {
                a.pf_ptr[0] = p.wo;
                a.pf_bytes[0] = (unsigned long long)p.p_o.N * p.p_o.K * m->es;
            }
            auto copy_trace = [&]() {
                if (tr && ln.status == OXG4_OK &&
                    cudaMemcpyAsync(tr->trace_dev + (size_t)l * R * H, c->hB, sizeof(float) * R * H,
                                    cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess)
                    ln.status = fail(OXG4_CUDA, "Gemma 4 CUDA error: trace copy failed");
            };
            launch_gemv(ln, "qkv", c, R, a, p.p_qkv, PRO_NORM, EPI_STORE);
            copy_trace();          // the layer's input as this library computed it
            if (tr && tr->inject_dev) {
                // layer-wise teacher forcing: redo the projection from the forced input, nothing pending
                a.embed = nullptr;
                a.raw = nullptr;
                a.w_post = nullptr;
                a.scalar = 1.0f;
                a.h_in = tr->inject_dev + (size_t)l * R * H;
                launch_gemv(ln, "qkv", c, R, a, p.p_qkv, PRO_NORM, EPI_STORE);
            }
        }
        launch_attention(ln, c, rs, l, c->qkv_raw, 1, nullptr, false);
        {   // O projection (decode.rs:159)
            GemvArgs a{};
            a.W0 = p.wo;
            a.in = c->attn_out;
            a.out = c->o_raw;
            launch_gemv(ln, "o", c, R, a, p.p_o, PRO_PLAIN, EPI_STORE);
            ln.allreduce(c->o_raw, (size_t)R * H);        // row-split projection: sum the ranks' partial outputs
        }
        {   // post-attention norm + residual, pre-FF norm, gate and up projections (decode.rs:161-171, 14-16)
            GemvArgs a{};
            a.W0 = p.wgate;
            a.W1 = p.wup;
            a.h_in = c->hB;
            a.h_out = c->hA;
            a.raw = c->o_raw;
            a.w_post = p.post_attn_ln;
            a.scalar = 1.0f;
            a.w_norm = p.pre_ff_ln;
            a.out = c->gu_raw;
            if (m->far_prefetch & 4) {
                a.pf_ptr[0] = p.wdown;
                a.pf_bytes[0] = std::min<unsigned long long>((unsigned long long)m->p_down.N * m->p_down.K * m->es, (unsigned long long)m->far_prefetch_mb << 20);
            }
            launch_gemv(ln, "gateup", c, R, a, m->p_gateup, PRO_NORM, EPI_GATEUP);
        }
        {   // GeGLU + down projection (decode.rs:17-18)
            GemvArgs a{};
            a.W0 = p.wdown;
            a.in = c->gu_raw;
            a.out = c->down_raw;
            if (m->far_prefetch & 8) {
                if (l + 1 < L) {
                    a.pf_ptr[0] = m->layers[l + 1].wqkv;
                    a.pf_bytes[0] = (unsigned long long)m->layers[l + 1].p_qkv.N * m->layers[l + 1].p_qkv.K * m->es;
                } else if (last_layer_prefetch) {
                    a.pf_ptr[0] = (const char*)m->embed + (size_t)m->v0 * H * m->es;
                    a.pf_bytes[0] = std::min<unsigned long long>((unsigned long long)m->Vloc * H * m->es, 64ull << 20);
                }
            }
            launch_gemv(ln, "down", c, R, a, m->p_down, PRO_PLAIN, EPI_STORE);
            ln.allreduce(c->down_raw, (size_t)R * H);
        }
        if (m->P > 0) ple_layer(c, ln, rs, l);
    }
}

// tcgen05 path: the last layer's pending update + final norm for `rows` rows: h -> c->hB, x -> c->x_h
static void closing_norm_tc(oxg4_cache* c, Launcher& ln, int rows, bool chunk, bool peer) {
    oxg4_model* m = c->m;
    const int L = m->cfg.num_hidden_layers;
    RowsNormArgs n{};
    n.B = rows; n.H = m->H;
    n.h_in = c->hA; n.h_out = c->hB;
    n.raw = m->tp > 1 ? (peer ? c->px[1].gathered : c->down_raw) : c->down_part;
    n.raw_splits = m->tp > 1 ? (peer ? m->tp : 1) : (chunk ? c->ps_down : c->s_down);
    if (m->tp > 1 && peer) n.px = c->px[1];
    n.w_post = m->layers[L - 1].post_ff_ln;
    n.scalar = m->layers[L - 1].layer_scalar;
    n.w_norm = m->final_norm;
    n.eps = m->cfg.rms_norm_eps;
    n.x = c->x_h;
    ln.go("norm", rows_norm_kernel, dim3(rows), dim3(kRowsThreads), 0, n);
}

// Tied LM head over B rows + arg-max / top-k (decode.rs:495-508, kernel_module.rs:1988-2075).
// tcgen05 path: x [B, H] BF16 normed activations. Small-batch path: the pending update (h_in + raw) is closed by
// the kernel's prologue.
static void lm_head(oxg4_cache* c, Launcher& ln, int kind, int top_k, float penalty, bool use_tc, const uint16_t* x,
                    const float* h_in, const float* raw, const TraceCtx* tr) {
    oxg4_model* m = c->m;
    const int B = c->B, L = m->cfg.num_hidden_layers, H = m->H;
    auto trace_final = [&]() {
        if (tr && ln.status == OXG4_OK &&
            cudaMemcpyAsync(tr->trace_dev + (size_t)L * B * H, c->hB, sizeof(float) * B * H, cudaMemcpyDeviceToDevice,
                            m->stream) != cudaSuccess)
            ln.status = fail(OXG4_CUDA, "Gemma 4 CUDA error: trace copy failed");
    };
    if (use_tc) {
        trace_final();
        const int k = (kind == STEP_TOPK) ? top_k : 1;
        uint32_t* out_ids = k == 1 ? c->best_ids : c->topk_ids;
        float* out_scores = k == 1 ? c->best_scores : c->topk_scores;
        if (m->tp > 1 && kind == STEP_TOPK) {
            // every rank ranks its own vocabulary slice; N * k (score, id) pairs per sequence cross the links
            // instead of the [B, V] logits
            ln.tc("lmhead", c, B, (const char*)m->embed + (size_t)m->v0 * H * m->es, nullptr, x, m->Vloc, H, 1,
                  c->logits, m->V, m->v0);
            const int chunks = (m->Vloc + kTopkChunk - 1) / kTopkChunk;
            ln.go("topk1", topk_stage1_kernel, dim3(chunks, B), dim3(kTopkThreads), 0, (const float*)c->logits, m->V,
                  m->v0, m->Vloc, (const uint8_t*)c->seen, penalty, k, c->topk_stage);
            ln.go("topk2", topk_stage2_kernel, dim3(1, B), dim3(kTopkThreads), (size_t)chunks * k * 8,
                  (const Cand*)c->topk_stage, chunks * k, k, c->loc_ids, c->loc_scores);
            ln.allgather(c->loc_scores, c->tpk_scores, sizeof(float) * B * k);
            ln.allgather(c->loc_ids, c->tpk_ids, sizeof(uint32_t) * B * k);
            ln.go("tp_pick", tp_topk_merge_kernel, dim3(B), dim3(kTopkThreads), 0, B, m->tp, k,
                  (const float*)c->tpk_scores, (const uint32_t*)c->tpk_ids, out_ids, out_scores);
            return;
        }
        // full logits wanted on the host: every rank fills its vocabulary columns, the sum assembles the rows
        if (m->tp > 1 && cudaMemsetAsync(c->logits, 0, sizeof(float) * (size_t)B * m->V, m->stream) != cudaSuccess)
            ln.status = fail(OXG4_CUDA, "Gemma 4 CUDA error: cudaMemsetAsync failed");
        ln.tc("lmhead", c, B, (const char*)m->embed + (size_t)m->v0 * H * m->es, nullptr, x, m->Vloc, H, 1, c->logits,
              m->V, m->v0);
        ln.allreduce(c->logits, (size_t)B * m->V);
        // top-k over the full logits (k = 1 is the arg-max the greedy loop feeds back)
        const int chunks = (m->V + kTopkChunk - 1) / kTopkChunk;
        ln.go("topk1", topk_stage1_kernel, dim3(chunks, B), dim3(kTopkThreads), 0, (const float*)c->logits, m->V, 0,
              m->V, (const uint8_t*)c->seen, penalty, k, c->topk_stage);
        ln.go("topk2", topk_stage2_kernel, dim3(1, B), dim3(kTopkThreads), (size_t)chunks * k * 8,
              (const Cand*)c->topk_stage, chunks * k, k, out_ids, out_scores);
        return;
    }
    // post-FF norm + residual + layer_scalar of the last layer, final norm, tied LM head with fused arg-max
    GemvArgs a{};
    a.W0 = (const char*)m->embed + (size_t)m->v0 * H * m->es;
    a.h_in = h_in;
    a.h_out = c->hB;
    a.raw = raw;
    a.w_post = m->P > 0 ? m->layers[L - 1].ple_norm : m->layers[L - 1].post_ff_ln;
    a.scalar = m->layers[L - 1].layer_scalar;
    a.w_norm = m->final_norm;
    const bool want_logits = (kind == STEP_LOGITS) || top_k > 1;
    a.out = want_logits ? c->logits : nullptr;
    a.seen = c->seen;
    a.penalty = penalty;
    a.row_offset = m->v0;
    a.n_total = m->V;
    a.blk_best = c->blk_best;
    a.ticket = c->lm_ticket;
    a.best_ids = c->best_ids;
    a.best_scores = c->best_scores;
    if (m->tp > 1 && want_logits) {
        // every rank fills its vocabulary columns; the others stay zero and the sum assembles the row
        if (cudaMemsetAsync(c->logits, 0, sizeof(float) * (size_t)B * m->V, m->stream) != cudaSuccess)
            ln.status = fail(OXG4_CUDA, "Gemma 4 CUDA error: cudaMemsetAsync failed");
    }
    launch_gemv(ln, "lmhead", c, B, a, m->p_lm, PRO_NORM, EPI_LOGITS);
    if (m->tp > 1) {
        if (want_logits) ln.allreduce(c->logits, (size_t)B * m->V);
        ln.allgather(c->best_scores, c->tp_scores, sizeof(float) * B);
        ln.allgather(c->best_ids, c->tp_ids, sizeof(uint32_t) * B);
        ln.go("tp_pick", tp_pick_kernel, dim3(1), dim3(128), 0, B, m->tp, (const float*)c->tp_scores,
              (const uint32_t*)c->tp_ids, c->best_ids, c->best_scores);
    }
    trace_final();
    if (kind == STEP_TOPK && top_k > 1) {
        const int chunks = (m->V + kTopkChunk - 1) / kTopkChunk;
        ln.go("topk1", topk_stage1_kernel, dim3(chunks, B), dim3(kTopkThreads), 0, (const float*)c->logits,
              m->V, 0, m->V, (const uint8_t*)c->seen, penalty, top_k, c->topk_stage);
        ln.go("topk2", topk_stage2_kernel, dim3(1, B), dim3(kTopkThreads), (size_t)chunks * top_k * 8,
              (const Cand*)c->topk_stage, chunks * top_k, top_k, c->topk_ids, c->topk_scores);
    }
}

static int32_t run_step(oxg4_cache* c, int kind, int top_k, float penalty, int* n_kernels,
                        const TraceCtx* tr = nullptr) {
    oxg4_model* m = c->m;
    Launcher ln{m};
    ln.ts_base = c->ts_buf;
    const int B = c->B;
    // Sums over peer memory only in steps whose last exchange is consumed (the closing norm before the
    // LM head): a prompt-ingestion step skips that norm, so it takes the NCCL all-reduce instead and the
    // single exchange buffer per kind is never pushed into while a peer may still read it.
    const bool peer = c->peer_ready && kind != STEP_PREFILL;
    ln.go("step_begin", step_begin_kernel, dim3(1), dim3(128), 0, B, m->V,
          (const uint32_t*)c->tokens, c->seen, (const StepCtl*)c->ctl);
    RowSet rs;
    rs.R = B;
    rs.tok = c->tokens;
    rs.pos = c->pos;
    for (int k = 0; k < 2; ++k) {        // decode: one token per group, whatever the layer kind
        rs.grp_row0[k] = c->dec_grp_row0;
        rs.grp_n[k] = c->dec_grp_n;
        rs.NG[k] = B;
    }
    run_layers(c, ln, rs, c->use_tc, peer, kind != STEP_PREFILL, tr);
    if (kind != STEP_PREFILL) {
        if (c->use_tc) closing_norm_tc(c, ln, B, false, peer);
        const bool ple = m->P > 0;       // the last layer's pending update is then its per-layer-embedding branch
        lm_head(c, ln, kind, top_k, penalty, c->use_tc, c->x_h, ple ? c->ple_h : c->hA, ple ? c->ple_raw : c->down_raw, tr);
    }
    if (kind == STEP_TOPK && top_k > 1)      // a no-op unless the step's control words ask for a sampled token
        ln.go("sample", sample_candidates_kernel, dim3(1), dim3(64), 0, B, top_k, m->cfg.final_logit_softcapping,
              (const uint32_t*)c->tokens,
              (const uint32_t*)c->topk_ids, (const float*)c->topk_scores, (const StepCtl*)c->ctl, c->rng, c->best_ids,
              c->best_scores);
    ln.go("step_end", step_end_kernel, dim3(1), dim3(128), 0, B, c->tokens, c->pos,
          (const uint32_t*)c->best_ids, c->history, c->ctl);
    if (n_kernels) *n_kernels = ln.kernels;
    return ln.status;
}

static bool graphs_disabled() { return getenv("GEMMA4_DISABLE_CUDA_GRAPH") != nullptr; }

// Replays (capturing on first use) the step graph keyed on (kind, top_k, penalty bits), as the
// reference keys its captured graph (decode.rs:689-699). The graph lives in the cache table.
static int32_t launch_step(oxg4_cache* c, int kind, int top_k, float penalty) {
    oxg4_model* m = c->m;
    if (graphs_disabled() || m->profiling) {
        int n = 0;
        TRY(run_step(c, kind, top_k, penalty, &n));
        m->launches += n;
        return OXG4_OK;
    }
    uint32_t pbits;
    memcpy(&pbits, &penalty, 4);
    char key[64];
    snprintf(key, sizeof key, "%d:%d:%08x", kind, top_k, pbits);
    auto it = c->graphs.find(key);
    if (it == c->graphs.end()) {
        GraphEntry g;
        CK(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        int n = 0;
        int32_t s = run_step(c, kind, top_k, penalty, &n);
        cudaError_t e = cudaStreamEndCapture(m->stream, &g.graph);   // always end the capture (cuda_graph.rs:84-97)
        if (s != OXG4_OK) {
            if (g.graph) cudaGraphDestroy(g.graph);
            return s;
        }
        CK(e);
        CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
        g.kernels = n;
        if (getenv("GEMMA4_PROFILE")) fprintf(stderr, "Gemma4 CUDA Graph: captured step kind %d (%d kernels)\n", kind, n);
        it = c->graphs.emplace(key, g).first;
    }
    CK(cudaGraphLaunch(it->second.exec, m->stream));
    m->launches += it->second.kernels;
    return OXG4_OK;
}

static int32_t check_tokens(oxg4_cache* c, const uint32_t* tokens, bool allow_inactive) {
    for (int b = 0; b < c->B; ++b) {
        if (tokens[b] == kInactiveToken) {
            if (!allow_inactive) return fail(OXG4_INVALID_ARGUMENT, "token id exceeds CUDA decode vocabulary");
            continue;
        }
        if (tokens[b] >= (uint32_t)c->m->V)
            return fail(OXG4_INVALID_ARGUMENT, "token id exceeds CUDA decode vocabulary");     // decode.rs:675-679
        if (c->m->P > 0 && tokens[b] >= (uint32_t)c->m->cfg.vocab_size_per_layer_input)
            return fail(OXG4_INVALID_SHAPE, "invalid batched PLE input");                       // ple.rs:113-119
        if (c->pos_host[b] >= c->max_seq[b])
            return fail(OXG4_INVALID_SHAPE, "sequence %d is longer than the cache table's max_sequence", b);
    }
    return OXG4_OK;
}

static int32_t stage_inputs(oxg4_cache* c, const uint32_t* tokens, int mark_seen, int feed_back) {
    cudaStream_t st = c->m->stream;
    memcpy(c->h_tokens, tokens, sizeof(uint32_t) * c->B);
    c->h_ctl->mark_seen = mark_seen;
    c->h_ctl->feed_back = feed_back;
    c->h_ctl->step = 0;
    c->h_ctl->history_cap = c->history_cap;
    c->h_ctl->sample = c->want_sample;
    c->h_ctl->temperature = c->sample_temperature;
    c->h_ctl->top_p = c->sample_top_p;
    CK(cudaMemcpyAsync(c->tokens, c->h_tokens, sizeof(uint32_t) * c->B, cudaMemcpyHostToDevice, st));
    CK(cudaMemcpyAsync(c->ctl, c->h_ctl, sizeof(StepCtl), cudaMemcpyHostToDevice, st));
    return OXG4_OK;
}

static void advance_host(oxg4_cache* c, const uint32_t* tokens, int steps = 1) {
    for (int b = 0; b < c->B; ++b)
        if (tokens[b] != kInactiveToken) c->pos_host[b] += steps;
}

// the tcgen05 kernels raise a device flag instead of hanging when one of their bounded waits runs out
static int32_t check_tc(oxg4_cache* c) {
    if (!c->tc_ok && !c->mma_attn) return OXG4_OK;
    int err = 0;
    CK(cudaMemcpy(&err, c->tc_err, sizeof err, cudaMemcpyDeviceToHost));
    if (err) {
        cudaMemset(c->tc_err, 0, sizeof err);
        return fail(OXG4_TIMEOUT, "%s: a bounded barrier wait ran out (code %d)",
                    err >= 10 ? "tensor-core attention" : "tcgen05 projection", err);
    }
    if (c->peer_ready) {
        CK(cudaMemcpy(&err, c->px_local + 4, sizeof err, cudaMemcpyDeviceToHost));
        if (err) {
            cudaMemset(c->px_local + 4, 0, sizeof err);
            return fail(OXG4_TIMEOUT, "tensor-parallel exchange: a peer did not publish its partial sums in time");
        }
    }
    return OXG4_OK;
}

static void softcap(float* v, size_t n, float cap) {     // mod.rs:573-579
    if (cap > 0.0f)
        for (size_t i = 0; i < n; ++i) v[i] = tanhf(v[i] / cap) * cap;
}

extern "C" int32_t oxg4_prefill_token(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens) {
    if (!m || !c || !tokens || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(bind_device(m));
    TRY(check_tokens(c, tokens, true));
    TRY(stage_inputs(c, tokens, 0, 0));
    TRY(launch_step(c, STEP_PREFILL, 0, 1.0f));
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    advance_host(c, tokens);
    return OXG4_OK;
}

extern "C" int32_t oxg4_decode_logits(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens, float* logits) {
    if (!m || !c || !tokens || !logits || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(bind_device(m));
    TRY(check_tokens(c, tokens, true));
    TRY(stage_inputs(c, tokens, 0, 0));
    TRY(launch_step(c, STEP_LOGITS, 1, 1.0f));
    CK(cudaMemcpyAsync(logits, c->logits, sizeof(float) * (size_t)c->B * m->V, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    softcap(logits, (size_t)c->B * m->V, m->cfg.final_logit_softcapping);
    advance_host(c, tokens);
    return OXG4_OK;
}

extern "C" int32_t oxg4_decode_topk(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens, int32_t top_k,
                                    float penalty, int32_t mark_seen, uint32_t* ids, float* scores) {
    if (!m || !c || !tokens || !ids || !scores || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(bind_device(m));
    TRY(check_tokens(c, tokens, true));
    top_k = std::min(std::max(top_k, 1), 64);                 // decode.rs:680
    top_k = std::min(top_k, m->V);
    TRY(stage_inputs(c, tokens, mark_seen ? 1 : 0, 0));
    TRY(launch_step(c, STEP_TOPK, top_k, penalty));
    const uint32_t* src_i = top_k == 1 ? c->best_ids : c->topk_ids;
    const float* src_s = top_k == 1 ? c->best_scores : c->topk_scores;
    CK(cudaMemcpyAsync(c->h_ids, src_i, sizeof(uint32_t) * c->B * top_k, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaMemcpyAsync(c->h_scores, src_s, sizeof(float) * c->B * top_k, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    memcpy(ids, c->h_ids, sizeof(uint32_t) * c->B * top_k);
    memcpy(scores, c->h_scores, sizeof(float) * c->B * top_k);
    softcap(scores, (size_t)c->B * top_k, m->cfg.final_logit_softcapping);
    advance_host(c, tokens);
    return OXG4_OK;
}

extern "C" int32_t oxg4_decode_greedy(oxg4_model* m, oxg4_cache* c, const uint32_t* first_tokens, int32_t steps,
                                      uint32_t* out_ids, float* ms_per_step) {
    if (!m || !c || !first_tokens || !out_ids || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    if (steps <= 0) return fail(OXG4_INVALID_ARGUMENT, "steps must be positive");
    TRY(bind_device(m));
    TRY(check_tokens(c, first_tokens, true));
    for (int b = 0; b < c->B; ++b)
        if (first_tokens[b] != kInactiveToken && c->pos_host[b] + steps > c->max_seq[b])
            return fail(OXG4_INVALID_SHAPE, "sequence %d would outgrow the cache table's max_sequence", b);
    if (c->history_cap < steps) {
        uint32_t* h = nullptr;
        TRY(dalloc(c, &h, (size_t)steps * c->B));
        c->history = h;
        c->history_cap = steps;
        // the history pointer is a kernel argument: graphs captured with the old one are stale
        for (auto& g : c->graphs) {
            if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
            if (g.second.graph) cudaGraphDestroy(g.second.graph);
        }
        c->graphs.clear();
    }
    TRY(stage_inputs(c, first_tokens, 0, 1));
    // capture (if needed) before the timed region
    if (!graphs_disabled()) {
        uint32_t pbits;
        float one = 1.0f;
        memcpy(&pbits, &one, 4);
        char key[64];
        snprintf(key, sizeof key, "%d:%d:%08x", (int)STEP_TOPK, 1, pbits);
        if (c->graphs.find(key) == c->graphs.end()) {
            // one warm step outside the timed loop would change the state; capture does not execute
            GraphEntry g;
            CK(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
            int n = 0;
            int32_t s = run_step(c, STEP_TOPK, 1, 1.0f, &n);
            cudaError_t e = cudaStreamEndCapture(m->stream, &g.graph);
            if (s != OXG4_OK) { if (g.graph) cudaGraphDestroy(g.graph); return s; }
            CK(e);
            CK(cudaGraphInstantiate(&g.exec, g.graph, 0));
            g.kernels = n;
            c->graphs.emplace(key, g);
        }
    }
    CK(cudaEventRecord(c->ev0, m->stream));
    for (int s = 0; s < steps; ++s) TRY(launch_step(c, STEP_TOPK, 1, 1.0f));
    CK(cudaEventRecord(c->ev1, m->stream));
    CK(cudaMemcpyAsync(out_ids, c->history, sizeof(uint32_t) * (size_t)steps * c->B, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    if (ms_per_step) *ms_per_step = ms / steps;
    advance_host(c, first_tokens, steps);
    return OXG4_OK;
}

// Device-resident sampled generation: `steps` tokens per sequence drawn from the top-k list of every step
// by sample_candidates_kernel, fed back on the device; one synchronisation at the end. `seeds` holds one
// xorshift64 state per sequence and receives the state after the last draw, so that a host loop calling
// oxg4_sample_topk_candidates with the same state continues identically.
extern "C" int32_t oxg4_decode_sampled(oxg4_model* m, oxg4_cache* c, const uint32_t* first_tokens, int32_t steps,
                                       int32_t top_k, float temperature, float top_p, float penalty,
                                       uint64_t* seeds, uint32_t* out_ids, float* ms_per_step) {
    if (!m || !c || !first_tokens || !seeds || !out_ids || c->m != m)
        return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    if (steps <= 0) return fail(OXG4_INVALID_ARGUMENT, "steps must be positive");
    if (!std::isfinite(temperature) || temperature <= 0.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation temperature must be finite and greater than zero");
    if (!std::isfinite(top_p) || top_p < 0.0f || top_p > 1.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation top_p must be finite and between zero and one");
    if (!std::isfinite(penalty) || penalty < 1.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation repetition_penalty must be finite and at least one");
    top_k = std::min(std::min(std::max(top_k, 1), 64), m->V);
    if (top_k < 2) return fail(OXG4_INVALID_ARGUMENT, "sampling needs at least two candidates; use oxg4_decode_greedy for top_k = 1");
    if (m->tp > 1) return fail(OXG4_UNSUPPORTED, "device-side sampling is not available with tensor parallelism");
    TRY(bind_device(m));
    TRY(check_tokens(c, first_tokens, true));
    for (int b = 0; b < c->B; ++b)
        if (first_tokens[b] != kInactiveToken && c->pos_host[b] + steps > c->max_seq[b])
            return fail(OXG4_INVALID_SHAPE, "sequence %d would outgrow the cache table's max_sequence", b);
    if (c->history_cap < steps) {
        uint32_t* h = nullptr;
        TRY(dalloc(c, &h, (size_t)steps * c->B));
        c->history = h;
        c->history_cap = steps;
        for (auto& g : c->graphs) {                       // the history pointer is a kernel argument
            if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
            if (g.second.graph) cudaGraphDestroy(g.second.graph);
        }
        c->graphs.clear();
    }
    CK(cudaMemcpyAsync(c->rng, seeds, sizeof(uint64_t) * c->B, cudaMemcpyHostToDevice, m->stream));
    c->want_sample = 1;
    c->sample_temperature = temperature;
    c->sample_top_p = top_p;
    int32_t s = stage_inputs(c, first_tokens, 1, 1);
    c->want_sample = 0;
    if (s != OXG4_OK) return s;
    CK(cudaEventRecord(c->ev0, m->stream));
    for (int i = 0; i < steps; ++i) TRY(launch_step(c, STEP_TOPK, top_k, penalty));
    CK(cudaEventRecord(c->ev1, m->stream));
    CK(cudaMemcpyAsync(out_ids, c->history, sizeof(uint32_t) * (size_t)steps * c->B, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaMemcpyAsync(seeds, c->rng, sizeof(uint64_t) * c->B, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    if (ms_per_step) *ms_per_step = ms / steps;
    advance_host(c, first_tokens, steps);
    return OXG4_OK;
}

extern "C" int32_t oxg4_profile_step(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens) {
    if (!m || !c || !tokens || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(bind_device(m));
    TRY(check_tokens(c, tokens, true));
    TRY(stage_inputs(c, tokens, 0, 0));
    m->profiling = true;
    m->prof_events.clear();
    int32_t s = launch_step(c, STEP_TOPK, 1, 1.0f);
    m->profiling = false;
    if (s != OXG4_OK) return s;
    CK(cudaStreamSynchronize(m->stream));
    TRY(check_tc(c));
    m->profile.clear();
    for (auto& pe : m->prof_events) {
        float ms = 0;
        cudaEventElapsedTime(&ms, pe.second.first, pe.second.second);
        ProfileSlot& ps = m->profile[pe.first];
        ps.ms += ms;
        ps.count += 1;
        cudaEventDestroy(pe.second.first);
        cudaEventDestroy(pe.second.second);
    }
    m->prof_events.clear();
    advance_host(c, tokens);
    return OXG4_OK;
}

extern "C" int32_t oxg4_decode_trace(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens, const float* inject,
                                     float* trace, float* logits) {
    if (!m || !c || !tokens || !trace || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(bind_device(m));
    TRY(check_tokens(c, tokens, true));
    const int L = m->cfg.num_hidden_layers;
    const size_t per = (size_t)c->B * m->H;
    float *d_inject = nullptr, *d_trace = nullptr;
    CK(cudaMalloc(&d_trace, sizeof(float) * per * (L + 1)));
    if (inject) {
        if (cudaMalloc(&d_inject, sizeof(float) * per * L) != cudaSuccess) { cudaFree(d_trace); return fail(OXG4_OOM, "out of device memory"); }
        // ordered on the model's stream: a blocking copy from pageable memory may return before its DMA has
        // landed, and the model's non-blocking stream does not wait for the default stream
        cudaMemcpyAsync(d_inject, inject, sizeof(float) * per * L, cudaMemcpyHostToDevice, m->stream);
    }
    int32_t s = stage_inputs(c, tokens, 0, 0);
    TraceCtx tr{d_inject, d_trace};
    int n = 0;
    if (s == OXG4_OK) s = run_step(c, STEP_LOGITS, 1, 1.0f, &n, &tr);      // eager launches, no graph
    if (s == OXG4_OK && cudaStreamSynchronize(m->stream) != cudaSuccess) s = fail(OXG4_CUDA, "Gemma 4 CUDA error: trace step failed");
    if (s == OXG4_OK) {
        m->launches += n;
        cudaMemcpy(trace, d_trace, sizeof(float) * per * (L + 1), cudaMemcpyDeviceToHost);
        if (logits) {
            cudaMemcpy(logits, c->logits, sizeof(float) * (size_t)c->B * m->V, cudaMemcpyDeviceToHost);
            softcap(logits, (size_t)c->B * m->V, m->cfg.final_logit_softcapping);
        }
        advance_host(c, tokens);
    }
    cudaFree(d_trace);
    cudaFree(d_inject);
    return s;
}

// ------------------------------------------------------------------------------------------------
// Diagnostic entry points: the counterparts of the reference's smoke functions (gemma4_cuda/smoke.rs:8-204), one
// token through one block of one layer, built from the kernels of the one-sequence decode step. Single-GPU models.
// ------------------------------------------------------------------------------------------------
struct ScratchTable {      // a one-sequence cache table for entry points that take none (workspace + a 16-token ring)
    oxg4_cache* c = nullptr;
    ~ScratchTable() { if (c) oxg4_cache_destroy(c); }
    int32_t open(oxg4_model* m) {
        const int32_t max_seq = 16;
        return oxg4_cache_create(m, 1, &max_seq, 16, OXG4_F32, &c);
    }
};

static int32_t smoke_check(oxg4_model* m, uint32_t token, int32_t layer, bool need_layer, bool own_kv) {
    if (!m) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (!m->finalized) return fail(OXG4_INVALID_ARGUMENT, "model is not finalized");
    if (m->tp > 1) return fail(OXG4_UNSUPPORTED, "the diagnostic entry points run on a single-GPU model");
    if (token >= (uint32_t)m->V) return fail(OXG4_INVALID_ARGUMENT, "token id exceeds CUDA embedding table");   // attention.rs:13-17
    if (need_layer && (layer < 0 || layer >= m->cfg.num_hidden_layers)) return fail(OXG4_INVALID_ARGUMENT, "layer out of range");
    if (own_kv && m->layers[layer].shared) return fail(OXG4_UNSUPPORTED, "layer %d shares the K/V of layer %d", layer, m->layers[layer].source);
    return OXG4_OK;
}

static int32_t smoke_stage(oxg4_cache* c, uint32_t token) {
    c->h_tokens[0] = token;
    CK(cudaMemcpyAsync(c->tokens, c->h_tokens, sizeof(uint32_t), cudaMemcpyHostToDevice, c->m->stream));
    return OXG4_OK;
}

static int32_t smoke_finish(oxg4_cache* c, Launcher& ln, const float* dev, float* host, size_t n) {
    oxg4_model* m = c->m;
    TRY(ln.status);
    m->launches += ln.kernels;
    CK(cudaMemcpyAsync(host, dev, sizeof(float) * n, cudaMemcpyDeviceToHost, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    return OXG4_OK;
}

// input norm + fused QKV projection of `layer` on the embedding of the staged token: layer input -> c->hB, qkv -> c->qkv_raw
static void smoke_qkv(oxg4_cache* c, Launcher& ln, int layer) {
    oxg4_model* m = c->m;
    const LayerPlan& p = m->layers[layer];
    GemvArgs a{};
    a.W0 = p.wqkv;
    a.embed = m->embed;
    a.tokens = c->tokens;
    a.embed_scale = sqrtf((float)m->H);
    a.h_out = c->hB;
    a.w_norm = p.input_ln;
    a.scalar = 1.0f;
    a.out = c->qkv_raw;
    launch_gemv(ln, "qkv", c, 1, a, p.p_qkv, PRO_NORM, EPI_STORE);
}

static RowSet smoke_rows(oxg4_cache* c) {
    RowSet rs;
    rs.R = 1;
    rs.tok = c->tokens;
    rs.pos = c->pos;
    for (int k = 0; k < 2; ++k) {
        rs.grp_row0[k] = c->dec_grp_row0;
        rs.grp_n[k] = c->dec_grp_n;
        rs.NG[k] = 1;
    }
    return rs;
}

// embedding_logits (smoke.rs:8-30): embedding row * sqrt(hidden) -> BF16 -> tied LM head; no final norm, no soft cap
extern "C" int32_t oxg4_smoke_embedding_logits(oxg4_model* m, uint32_t token, float* logits) {
    if (!logits) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    TRY(smoke_check(m, token, 0, false, false));
    TRY(bind_device(m));
    ScratchTable t;
    TRY(t.open(m));
    oxg4_cache* c = t.c;
    TRY(smoke_stage(c, token));
    Launcher ln{m};
    if (m->es == 2)
        ln.go("embed", ple_embed_rows_kernel<uint16_t>, dim3(1), dim3(256), 0, m->H, (const uint16_t*)m->embed,
              (const uint32_t*)c->tokens, sqrtf((float)m->H), c->hA);
    else
        ln.go("embed", ple_embed_rows_kernel<float>, dim3(1), dim3(256), 0, m->H, (const float*)m->embed,
              (const uint32_t*)c->tokens, sqrtf((float)m->H), c->hA);
    GemvArgs a{};
    a.W0 = m->embed;
    a.in = c->hA;
    a.out = c->logits;
    launch_gemv(ln, "lmhead", c, 1, a, m->p_lm, PRO_PLAIN, EPI_STORE);
    return smoke_finish(c, ln, c->logits, logits, (size_t)m->V);
}

// decoder_mlp_smoke (smoke.rs:32-59): hidden + rmsnorm(down(gelu(gate x) * up x), post_ff_ln), x = rmsnorm(hidden, pre_ff_ln)
extern "C" int32_t oxg4_smoke_decoder_mlp(oxg4_model* m, uint32_t token, int32_t layer, float* out) {
    if (!out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    TRY(smoke_check(m, token, layer, true, false));
    TRY(bind_device(m));
    ScratchTable t;
    TRY(t.open(m));
    oxg4_cache* c = t.c;
    TRY(smoke_stage(c, token));
    const LayerPlan& p = m->layers[layer];
    Launcher ln{m};
    {
        GemvArgs a{};
        a.W0 = p.wgate;
        a.W1 = p.wup;
        a.embed = m->embed;
        a.tokens = c->tokens;
        a.embed_scale = sqrtf((float)m->H);
        a.h_out = c->hA;
        a.w_norm = p.pre_ff_ln;
        a.scalar = 1.0f;
        a.out = c->gu_raw;
        launch_gemv(ln, "gateup", c, 1, a, m->p_gateup, PRO_NORM, EPI_GATEUP);
    }
    {
        GemvArgs a{};
        a.W0 = p.wdown;
        a.in = c->gu_raw;
        a.out = c->down_raw;
        launch_gemv(ln, "down", c, 1, a, m->p_down, PRO_PLAIN, EPI_STORE);
    }
    {   // the residual update is the prologue of the projection that would follow: hB = hA + rmsnorm(down, post_ff_ln)
        GemvArgs a{};
        a.W0 = p.wqkv;
        a.h_in = c->hA;
        a.h_out = c->hB;
        a.raw = c->down_raw;
        a.w_post = p.post_ff_ln;
        a.scalar = 1.0f;
        a.w_norm = p.input_ln;
        a.out = c->qkv_raw;
        launch_gemv(ln, "qkv", c, 1, a, p.p_qkv, PRO_NORM, EPI_STORE);
    }
    return smoke_finish(c, ln, c->hB, out, (size_t)m->H);
}

// decoder_attention_smoke (smoke.rs:61-126): the attention residual branch of one layer for one token at position 0
// (a single position attends to itself; the rotation at position 0 is the identity for any theta)
extern "C" int32_t oxg4_smoke_decoder_attention(oxg4_model* m, uint32_t token, int32_t layer, float* out) {
    if (!out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    TRY(smoke_check(m, token, layer, true, true));
    TRY(bind_device(m));
    ScratchTable t;
    TRY(t.open(m));
    oxg4_cache* c = t.c;
    TRY(smoke_stage(c, token));
    const LayerPlan& p = m->layers[layer];
    Launcher ln{m};
    smoke_qkv(c, ln, layer);
    launch_attention(ln, c, smoke_rows(c), layer, c->qkv_raw, 1, nullptr, false);
    {
        GemvArgs a{};
        a.W0 = p.wo;
        a.in = c->attn_out;
        a.out = c->o_raw;
        launch_gemv(ln, "o", c, 1, a, p.p_o, PRO_PLAIN, EPI_STORE);
    }
    {   // hA = hB + rmsnorm(o, post_attn_ln): the prologue of the gate/up projection
        GemvArgs a{};
        a.W0 = p.wgate;
        a.W1 = p.wup;
        a.h_in = c->hB;
        a.h_out = c->hA;
        a.raw = c->o_raw;
        a.w_post = p.post_attn_ln;
        a.scalar = 1.0f;
        a.w_norm = p.pre_ff_ln;
        a.out = c->gu_raw;
        launch_gemv(ln, "gateup", c, 1, a, m->p_gateup, PRO_NORM, EPI_GATEUP);
    }
    return smoke_finish(c, ln, c->hA, out, (size_t)m->H);
}

// cached_attention_smoke (smoke.rs:128-204): one token appended to the layer's K/V ring of a one-sequence cache
// table (the counterpart of new_kv_cache, cache.rs:5-29) and attended against it; returns [heads * head_dim] and
// advances the table's position. The layer's own RoPE parameters are used (the reference passes theta 10000,
// factor 1, full rotary: the sliding layers' values). Use such a table for nothing but these calls.
extern "C" int32_t oxg4_smoke_cached_attention(oxg4_model* m, oxg4_cache* c, uint32_t token, int32_t layer, float* attended) {
    if (!c || !attended || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    TRY(smoke_check(m, token, layer, true, true));
    if (c->B != 1) return fail(OXG4_INVALID_SHAPE, "cached attention smoke takes a one-sequence cache table");
    TRY(bind_device(m));
    TRY(check_tokens(c, &token, false));
    TRY(smoke_stage(c, token));
    Launcher ln{m};
    smoke_qkv(c, ln, layer);
    launch_attention(ln, c, smoke_rows(c), layer, c->qkv_raw, 1, nullptr, false);
    TRY(smoke_finish(c, ln, c->attn_out, attended, (size_t)m->layers[layer].qw));
    c->pos_host[0] += 1;
    CK(cudaMemcpyAsync(c->pos, c->pos_host.data(), sizeof(int32_t), cudaMemcpyHostToDevice, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    return OXG4_OK;
}

extern "C" int32_t oxg4_debug_timeline(oxg4_cache* c, unsigned long long* out, int32_t max_entries) {
    if (!c || !out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (!c->ts_buf) return fail(OXG4_UNSUPPORTED, "timeline recording is off (set OXG4_TIMELINE before creating the model)");
    TRY(bind_device(c->m));
    const int n = std::min(max_entries, kMaxTimeline * 4);
    CK(cudaMemcpy(out, c->ts_buf, sizeof(unsigned long long) * n, cudaMemcpyDeviceToHost));
    return OXG4_OK;
}

extern "C" float oxg4_profile_ms(const oxg4_model* m, const char* kind) {
    if (!m || !kind) return -1.0f;
    auto it = m->profile.find(kind);
    if (it == m->profile.end() || it->second.count == 0) return -1.0f;
    return (float)(it->second.ms / it->second.count);
}

extern "C" int32_t oxg4_profile_count(const oxg4_model* m, const char* kind) {
    if (!m || !kind) return 0;
    auto it = m->profile.find(kind);
    return it == m->profile.end() ? 0 : it->second.count;
}

// prefill_prompt (decode.rs:386-459): the prompts of all sequences go through the layers in chunks of up to
// kPrefillRows tokens, each chunk one pass with matrix-shaped projections (tcgen05 for BF16 weights) and causal /
// sliding paged attention over the chunk; a chunk may hold the tail of one sequence and the head of the next.
// Unlike the reference there is no 4096-token limit and no requirement that the prompt fits the sliding ring.
extern "C" int32_t oxg4_prefill(oxg4_model* m, oxg4_cache* c, const uint32_t* tokens, const int32_t* lens,
                                float* last_logits) {
    if (!m || !c || !tokens || !lens || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    const int B = c->B, H = m->H;
    std::vector<int64_t> off(B + 1, 0);
    for (int b = 0; b < B; ++b) {
        if (lens[b] <= 0) return fail(OXG4_INVALID_ARGUMENT, "batched prefill requires at least one token per sequence");
        if (c->pos_host[b] != 0) return fail(OXG4_INVALID_ARGUMENT, "batched prefill requires an empty cache table");   // decode.rs:392-396
        if (lens[b] > c->max_seq[b]) return fail(OXG4_INVALID_SHAPE, "prompt does not fit the cache table");
        off[b + 1] = off[b] + lens[b];
    }
    for (int64_t i = 0; i < off[B]; ++i) {
        if (tokens[i] >= (uint32_t)m->V) return fail(OXG4_INVALID_ARGUMENT, "token id exceeds CUDA decode vocabulary");
        if (m->P > 0 && tokens[i] >= (uint32_t)m->cfg.vocab_size_per_layer_input)
            return fail(OXG4_INVALID_SHAPE, "invalid batched PLE input");                       // ple.rs:113-119
    }
    TRY(bind_device(m));
    if (getenv("OXG4_PREFILL_BY_TOKEN")) {
        // the reference's sequential alternative (prefill_token, decode.rs:464-472): one token per sequence and step
        int maxlen = 0;
        for (int b = 0; b < B; ++b) maxlen = std::max(maxlen, lens[b]);
        std::vector<uint32_t> step_tokens(B);
        for (int t = 0; t + 1 < maxlen; ++t) {
            for (int b = 0; b < B; ++b) step_tokens[b] = (t + 1 < lens[b]) ? tokens[off[b] + t] : kInactiveToken;
            TRY(oxg4_prefill_token(m, c, step_tokens.data()));
        }
        for (int b = 0; b < B; ++b) step_tokens[b] = tokens[off[b] + lens[b] - 1];
        if (last_logits) return oxg4_decode_logits(m, c, step_tokens.data(), last_logits);
        return oxg4_prefill_token(m, c, step_tokens.data());
    }
    const bool use_tc = c->tc_ok;
    // tokens per attention group, per layer kind (0 sliding, 1 global): 8 / (query heads per KV head)
    int tg[2] = {1, 1};
    for (auto& lp : m->layers) tg[lp.sliding ? 0 : 1] = std::max(1, kAmRows / lp.G);
    int32_t* h_pos = c->h_pf_meta;
    int32_t* h_seq = h_pos + kPrefillRows;
    int32_t* h_g0[2] = {h_seq + kPrefillRows, h_seq + kPrefillRows + 2 * kAmMaxGroups};
    int32_t* h_gn[2] = {h_g0[0] + kAmMaxGroups, h_g0[1] + kAmMaxGroups};
    int b = 0, p = 0;                                          // next token to place: sequence b, position p
    while (b < B) {
        int R = 0, NG[2] = {0, 0};
        std::vector<std::pair<int, int>> finishing;            // (sequence, row) of every last prompt token in this chunk
        while (b < B && R < kPrefillRows) {
            const int take = std::min(kPrefillRows - R, lens[b] - p);
            for (int i = 0; i < take; ++i) {
                c->h_pf_tok[R + i] = tokens[off[b] + p + i];
                h_pos[R + i] = p + i;
                h_seq[R + i] = b;
            }
            for (int k = 0; k < 2; ++k)
                for (int i = 0; i < take; i += tg[k]) {
                    h_g0[k][NG[k]] = R + i;
                    h_gn[k][NG[k]] = std::min(tg[k], take - i);
                    ++NG[k];
                }
            R += take;
            p += take;
            if (p == lens[b]) { finishing.push_back({b, R - 1}); ++b; p = 0; }
        }
        cudaStream_t st = m->stream;
        CK(cudaMemcpyAsync(c->pf_tok, c->h_pf_tok, sizeof(uint32_t) * R, cudaMemcpyHostToDevice, st));
        CK(cudaMemcpyAsync(c->pf_pos, h_pos, sizeof(int32_t) * R, cudaMemcpyHostToDevice, st));
        CK(cudaMemcpyAsync(c->pf_seq, h_seq, sizeof(int32_t) * R, cudaMemcpyHostToDevice, st));
        for (int k = 0; k < 2; ++k) {
            CK(cudaMemcpyAsync(c->pf_grp_row0[k], h_g0[k], sizeof(int32_t) * NG[k], cudaMemcpyHostToDevice, st));
            CK(cudaMemcpyAsync(c->pf_grp_n[k], h_gn[k], sizeof(int32_t) * NG[k], cudaMemcpyHostToDevice, st));
        }
        const bool prof = getenv("GEMMA4_PROFILE") != nullptr && getenv("OXG4_PROFILE_PREFILL") != nullptr;
        m->profiling = prof;           // events around every launch of the chunk (a measurement aid, like the reference's GEMMA4_PROFILE)
        Launcher ln{m};
        RowSet rs;
        rs.R = R;
        rs.tok = c->pf_tok;
        rs.pos = c->pf_pos;
        rs.seq = c->pf_seq;
        rs.chunk = true;
        for (int k = 0; k < 2; ++k) {
            rs.grp_row0[k] = c->pf_grp_row0[k];
            rs.grp_n[k] = c->pf_grp_n[k];
            rs.NG[k] = NG[k];
        }
        run_layers(c, ln, rs, use_tc, false, false, nullptr);
        if (last_logits && !finishing.empty() && ln.status == OXG4_OK) {
            // keep what the LM head will need of every sequence that ends in this chunk
            if (use_tc) closing_norm_tc(c, ln, R, true, false);
            for (auto& f : finishing) {
                if (use_tc) {
                    CK(cudaMemcpyAsync(c->last_x + (size_t)f.first * H, c->x_h + (size_t)f.second * H, sizeof(uint16_t) * H,
                                       cudaMemcpyDeviceToDevice, st));
                } else {
                    // the last layer's pending update: the MLP block's output, or with per-layer embeddings that branch
                    const float* h_src = m->P > 0 ? c->ple_h : c->hA;
                    const float* raw_src = m->P > 0 ? c->ple_raw : c->down_raw;
                    CK(cudaMemcpyAsync(c->last_h + (size_t)f.first * H, h_src + (size_t)f.second * H, sizeof(float) * H,
                                       cudaMemcpyDeviceToDevice, st));
                    CK(cudaMemcpyAsync(c->last_raw + (size_t)f.first * H, raw_src + (size_t)f.second * H,
                                       sizeof(float) * H, cudaMemcpyDeviceToDevice, st));
                }
            }
        }
        m->profiling = false;
        TRY(ln.status);
        m->launches += ln.kernels;
        CK(cudaStreamSynchronize(st));                         // the pinned staging is reused by the next chunk
        if (prof) {
            std::map<std::string, double> sum;
            for (auto& pe : m->prof_events) {
                float ms = 0;
                cudaEventElapsedTime(&ms, pe.second.first, pe.second.second);
                sum[pe.first] += ms;
                cudaEventDestroy(pe.second.first);
                cudaEventDestroy(pe.second.second);
            }
            m->prof_events.clear();
            fprintf(stderr, "Gemma4 prefill chunk (%d rows):", R);
            for (auto& kv : sum) fprintf(stderr, " %s %.3f ms", kv.first.c_str(), kv.second);
            fprintf(stderr, "\n");
        }
        TRY(check_tc(c));
    }
    // device step state: every sequence continues at position lens[b]
    std::vector<int32_t> np(lens, lens + B);
    CK(cudaMemcpyAsync(c->pos, np.data(), sizeof(int32_t) * B, cudaMemcpyHostToDevice, m->stream));
    CK(cudaStreamSynchronize(m->stream));      // np leaves scope; later steps read c->pos in stream order
    for (int i = 0; i < B; ++i) c->pos_host[i] = lens[i];
    if (last_logits) {
        Launcher ln{m};
        lm_head(c, ln, STEP_LOGITS, 1, 1.0f, use_tc, c->last_x, c->last_h, c->last_raw, nullptr);
        TRY(ln.status);
        m->launches += ln.kernels;
        CK(cudaMemcpyAsync(last_logits, c->logits, sizeof(float) * (size_t)B * m->V, cudaMemcpyDeviceToHost, m->stream));
        CK(cudaStreamSynchronize(m->stream));
        TRY(check_tc(c));
        softcap(last_logits, (size_t)B * m->V, m->cfg.final_logit_softcapping);
    }
    return OXG4_OK;
}

// ------------------------------------------------------------------------------------------------
// host mirror of the generation loop (models/gemma4/generation.rs, sampling.rs)
// ------------------------------------------------------------------------------------------------
static inline int32_t total_order_key(float f) {      // f32::total_cmp
    int32_t b;
    memcpy(&b, &f, 4);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return b;
}

struct Scored {
    int64_t id;
    float v;
};

static int64_t draw(std::vector<Scored>& cand, float top_p, uint64_t* random) {
    const float maximum = cand[0].v;
    float total = 0.0f;
    for (auto& s : cand) { s.v = expf(s.v - maximum); total += s.v; }
    if (total == 0.0f || !std::isfinite(total)) return -1;
    for (auto& s : cand) s.v /= total;
    if (top_p < 1.0f) {
        float cumulative = 0.0f;
        size_t keep = 0;
        for (auto& s : cand) {
            cumulative += s.v;
            ++keep;
            if (cumulative >= top_p) break;
        }
        cand.resize(std::max<size_t>(keep, 1));
        total = 0.0f;
        for (auto& s : cand) total += s.v;
    } else {
        total = 1.0f;
    }
    uint64_t r = *random;
    if (r == 0) r = 0x4d595df4d0f33173ull;
    r ^= r << 13;
    r ^= r >> 7;
    r ^= r << 17;
    *random = r;
    const float unit = (float)((uint32_t)(r >> 40)) / 16777216.0f;
    float threshold = unit * total;
    for (auto& s : cand) {
        if (threshold <= s.v) return s.id;
        threshold -= s.v;
    }
    return cand.back().id;
}

extern "C" int64_t oxg4_sample_token(const float* logits, int64_t n, float temperature, int64_t top_k, float top_p,
                                     uint64_t* random) {
    if (!logits || !random || n <= 0 || !(temperature > 0.0f) || !(top_p >= 0.0f && top_p <= 1.0f)) return -1;
    std::vector<Scored> cand;
    cand.reserve((size_t)n);
    for (int64_t i = 0; i < n; ++i)
        if (std::isfinite(logits[i])) cand.push_back({i, logits[i] / temperature});
    if (cand.empty()) return -1;
    auto desc = [](const Scored& a, const Scored& b) { return total_order_key(a.v) > total_order_key(b.v); };
    const size_t keep = (size_t)std::min<int64_t>(std::max<int64_t>(top_k, 1), (int64_t)cand.size());
    if (keep < cand.size()) {
        std::partial_sort(cand.begin(), cand.begin() + keep, cand.end(), desc);
        cand.resize(keep);
    } else {
        std::sort(cand.begin(), cand.end(), desc);
    }
    return draw(cand, top_p, random);
}

extern "C" int64_t oxg4_sample_topk_candidates(const uint32_t* ids, const float* scores, int64_t n, float temperature,
                                               float top_p, uint64_t* random) {
    if (!ids || !scores || !random || n <= 0 || !(temperature > 0.0f) || !(top_p >= 0.0f && top_p <= 1.0f)) return -1;
    std::vector<Scored> cand;
    for (int64_t i = 0; i < n; ++i)
        if (std::isfinite(scores[i])) cand.push_back({(int64_t)ids[i], scores[i] / temperature});
    if (cand.empty()) return -1;
    std::stable_sort(cand.begin(), cand.end(),
                     [](const Scored& a, const Scored& b) { return total_order_key(a.v) > total_order_key(b.v); });
    return draw(cand, top_p, random);
}

extern "C" int32_t oxg4_generate(oxg4_model* m, const uint32_t* prompt, int64_t n_prompt,
                                 const oxg4_generation_config* g, int32_t kv_dtype, oxg4_token_callback on_token,
                                 void* user, uint32_t* out_ids, int64_t* n_out) {
    if (!m || !g || !out_ids || !n_out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    // GenerationConfig::validate (generation.rs:6-33)
    if (!std::isfinite(g->temperature) || g->temperature <= 0.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation temperature must be finite and greater than zero");
    if (!std::isfinite(g->top_p) || g->top_p < 0.0f || g->top_p > 1.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation top_p must be finite and between zero and one");
    if (g->top_k == 0) return fail(OXG4_INVALID_ARGUMENT, "generation top_k must be greater than zero");
    if (!std::isfinite(g->repetition_penalty) || g->repetition_penalty < 1.0f)
        return fail(OXG4_INVALID_ARGUMENT, "generation repetition_penalty must be finite and at least one");
    for (int64_t i = 0; i < g->n_stop_sequences; ++i)
        if (g->stop_sequence_lens[i] == 0)
            return fail(OXG4_INVALID_ARGUMENT, "generation stop-token sequences cannot be empty");
    if (!prompt || n_prompt <= 0)
        return fail(OXG4_INVALID_ARGUMENT, "Gemma 4 generation requires at least one input token");
    if (g->max_new_tokens < 0 || n_prompt + g->max_new_tokens > 0x7fffffff)
        return fail(OXG4_INVALID_ARGUMENT, "Gemma 4 sequence length overflow");
    const int32_t max_seq = (int32_t)(n_prompt + g->max_new_tokens);
    oxg4_cache* cache = nullptr;
    TRY(oxg4_cache_create(m, 1, &max_seq, 256, kv_dtype, &cache));
    std::vector<float> logits((size_t)m->V);
    const int32_t len = (int32_t)n_prompt;
    int32_t s = oxg4_prefill(m, cache, prompt, &len, logits.data());
    if (s != OXG4_OK) { oxg4_cache_destroy(cache); return s; }
    uint64_t random = g->seed;
    std::vector<uint32_t> generated;
    uint32_t ids[64];
    float scores[64];
    int n_cand = 0;
    bool have_cand = false;
    for (int64_t it = 0; it < g->max_new_tokens; ++it) {
        if (!have_cand && g->repetition_penalty > 1.0f) {
            // apply_repetition_penalty over the tokens generated so far (generation.rs:143-157)
            std::vector<uint32_t> uniq(generated);
            std::sort(uniq.begin(), uniq.end());
            uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
            for (uint32_t t : uniq)
                if (t < (uint32_t)m->V) logits[t] = logits[t] >= 0.0f ? logits[t] / g->repetition_penalty : logits[t] * g->repetition_penalty;
        }
        const int64_t next = have_cand
                                 ? oxg4_sample_topk_candidates(ids, scores, n_cand, g->temperature, g->top_p, &random)
                                 : oxg4_sample_token(logits.data(), m->V, g->temperature, g->top_k, g->top_p, &random);
        if (next < 0) { oxg4_cache_destroy(cache); return fail(OXG4_INVALID_ARGUMENT, "invalid sampling input"); }
        generated.push_back((uint32_t)next);
        if (on_token && on_token((uint32_t)next, user) != 0) {
            oxg4_cache_destroy(cache);
            return fail(OXG4_INVALID_ARGUMENT, "token callback returned an error");
        }
        bool stop = false;
        for (int64_t e = 0; e < g->n_eos; ++e) stop |= g->eos_token_ids[e] == (uint32_t)next;
        int64_t so = 0;
        for (int64_t q = 0; q < g->n_stop_sequences && !stop; ++q) {
            const int64_t sl = g->stop_sequence_lens[q];
            if ((int64_t)generated.size() >= sl &&
                std::equal(g->stop_sequences + so, g->stop_sequences + so + sl, generated.end() - sl))
                stop = true;
            so += sl;
        }
        if (stop) break;
        const uint32_t tok = (uint32_t)next;
        n_cand = (int)std::min<int64_t>(std::max<int64_t>(g->top_k, 1), 64);
        n_cand = std::min(n_cand, m->V);
        s = oxg4_decode_topk(m, cache, &tok, n_cand, g->repetition_penalty, 1, ids, scores);
        if (s != OXG4_OK) { oxg4_cache_destroy(cache); return s; }
        have_cand = true;
    }
    oxg4_cache_destroy(cache);
    memcpy(out_ids, prompt, sizeof(uint32_t) * (size_t)n_prompt);
    memcpy(out_ids + n_prompt, generated.data(), sizeof(uint32_t) * generated.size());
    *n_out = n_prompt + (int64_t)generated.size();
    return OXG4_OK;
}

// Failure-path probe: runs a bounded device-side wait that nothing will ever satisfy, with a polling budget
// of `spin_limit`, then reports through the same status word and check as every step does.
// Measurement aid (no counterpart in the reference): an empty cache table is marked as holding lens[b] positions of
// every sequence and its K/V pools are filled with a fixed pseudo-random pattern, so that decode steps at a long
// context can be timed without ingesting the prompts. The contents are not the K/V of any prompt.
extern "C" int32_t oxg4_debug_fill_cache(oxg4_model* m, oxg4_cache* c, const int32_t* lens) {
    if (!m || !c || !lens || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    for (int b = 0; b < c->B; ++b) {
        if (c->pos_host[b] != 0) return fail(OXG4_INVALID_ARGUMENT, "synthetic fill requires an empty cache table");
        if (lens[b] <= 0 || lens[b] > c->max_seq[b]) return fail(OXG4_INVALID_SHAPE, "length does not fit the cache table");
    }
    TRY(bind_device(m));
    const int L = m->cfg.num_hidden_layers;
    for (int l = 0; l < L; ++l) {
        const size_t n16 = c->pool_bytes[l] / 16;
        if (n16 == 0) continue;
        const int grid = (int)std::min<size_t>((n16 + 255) / 256, (size_t)m->num_sms * 16);
        if (c->kv_dtype == OXG4_BF16) {
            pool_fill_kernel<uint16_t><<<grid, 256, 0, m->stream>>>((uint4*)c->kpool[l], n16, 2u * l + 1u);
            pool_fill_kernel<uint16_t><<<grid, 256, 0, m->stream>>>((uint4*)c->vpool[l], n16, 2u * l + 2u);
        } else {
            pool_fill_kernel<float><<<grid, 256, 0, m->stream>>>((uint4*)c->kpool[l], n16, 2u * l + 1u);
            pool_fill_kernel<float><<<grid, 256, 0, m->stream>>>((uint4*)c->vpool[l], n16, 2u * l + 2u);
        }
    }
    CK(cudaGetLastError());
    CK(cudaMemcpyAsync(c->pos, lens, sizeof(int32_t) * c->B, cudaMemcpyHostToDevice, m->stream));
    CK(cudaStreamSynchronize(m->stream));
    for (int b = 0; b < c->B; ++b) c->pos_host[b] = lens[b];
    return OXG4_OK;
}

extern "C" int32_t oxg4_debug_wait_timeout(oxg4_model* m, oxg4_cache* c, int32_t kind, uint32_t spin_limit) {
    if (!m || !c || c->m != m) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    if (kind != 1 && kind != 2) return fail(OXG4_INVALID_ARGUMENT, "kind must be 1 (mbarrier) or 2 (peer flag)");
    if (spin_limit == 0 || spin_limit > 1000000u) return fail(OXG4_INVALID_ARGUMENT, "spin_limit must be 1..1000000");
    TRY(bind_device(m));
    // the flag that is waited on is the (zero) attention ticket array: nothing writes it during the probe
    wait_probe_kernel<<<1, 32, 0, m->stream>>>(kind, spin_limit, c->attn_ticket, c->tc_err);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(m->stream));
    int err = 0;
    CK(cudaMemcpy(&err, c->tc_err, sizeof err, cudaMemcpyDeviceToHost));
    if (err) {
        CK(cudaMemset(c->tc_err, 0, sizeof err));
        return fail(OXG4_TIMEOUT, "%s: a bounded wait ran out (code %d)", err == 21 ? "mbarrier wait" : "peer flag wait", err);
    }
    return OXG4_OK;
}

// ------------------------------------------------------------------------------------------------
// top-k without any allocation
// ------------------------------------------------------------------------------------------------
// Scratch of oxg4_topk_noalloc: the per-chunk candidate lists that the first top-k stage hands to the
// second. It is part of the library image, so every GPU that loads the library holds these 512 KiB
// until the process exits. All calls on a device share it.
constexpr int kNoAllocMaxRows = 4;
constexpr int kNoAllocMaxVocab = 524288;
constexpr int kNoAllocMaxChunks = kNoAllocMaxVocab / kTopkChunk;
static __device__ __align__(256) Cand g_noalloc_topk_scratch[kNoAllocMaxRows * kNoAllocMaxChunks * 64];

// g_noalloc_topk_scratch is a host-side stand-in in host code, not a device address; the device address
// is looked up once per device with that device current.
static Cand* g_noalloc_scratch_addr[64] = {};

extern "C" int32_t oxg4_topk_noalloc(const float* logits_dev, int32_t rows, int32_t vocab,
                                     const uint8_t* seen_dev, float repetition_penalty, int32_t top_k,
                                     uint32_t* ids_dev, float* scores_dev, void* cuda_stream) {
    if (!logits_dev || !ids_dev || !scores_dev) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    if (rows < 1 || rows > kNoAllocMaxRows)
        return fail(OXG4_INVALID_SHAPE, "oxg4_topk_noalloc handles 1..%d rows per call, got %d", kNoAllocMaxRows, rows);
    if (vocab < 1 || vocab > kNoAllocMaxVocab)
        return fail(OXG4_INVALID_SHAPE, "oxg4_topk_noalloc handles a vocabulary of at most %d, got %d", kNoAllocMaxVocab, vocab);
    top_k = std::min(std::max(top_k, 1), 64);
    top_k = std::min(top_k, vocab);
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(OXG4_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (g_noalloc_scratch_addr[dev] == nullptr) {
        // first call on this device: resolve the array's device address and opt the merge kernel in to
        // its shared-memory size. Neither call allocates; both should happen outside stream capture.
        Cand* p = nullptr;
        CK(cudaGetSymbolAddress((void**)&p, g_noalloc_topk_scratch));
        TRY(allow_big_smem(topk_stage2_kernel));
        g_noalloc_scratch_addr[dev] = p;
    }
    Cand* scratch = g_noalloc_scratch_addr[dev];
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const int chunks = (vocab + kTopkChunk - 1) / kTopkChunk;
    // every scratch entry the merge reads is written by the first stage of the same call, so nothing
    // has to be cleared between calls
    topk_stage1_kernel<<<dim3(chunks, rows), kTopkThreads, 0, st>>>(logits_dev, vocab, 0, vocab, seen_dev,
                                                                    repetition_penalty, top_k, scratch);
    CK(cudaGetLastError());
    topk_stage2_kernel<<<dim3(1, rows), kTopkThreads, (size_t)chunks * top_k * 8, st>>>(scratch, chunks * top_k, top_k,
                                                                                        ids_dev, scores_dev);
    CK(cudaGetLastError());
    return OXG4_OK;
}

// ------------------------------------------------------------------------------------------------
// tcgen05 projection: stand-alone entry used by the parity tests of csrc/tc_gemm.cuh
// ------------------------------------------------------------------------------------------------
constexpr int kDebugReps = 10;
extern "C" int32_t oxg4_debug_tc_gemm(const uint16_t* w_host, const uint16_t* x_host, int32_t N, int32_t K, int32_t B,
                                      float* out_host, float* ms_or_null) {
    if (!w_host || !x_host || !out_host) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    TRY(tc_gemm_setup());
    void *w = nullptr, *x = nullptr;
    float* o = nullptr;
    int* e = nullptr;
    cudaDeviceProp prop;
    int dev = 0;
    CK(cudaGetDevice(&dev));
    CK(cudaGetDeviceProperties(&prop, dev));
    const int sms = prop.multiProcessorCount;
    const int S = tc_pick_splits((N + kTcTileM - 1) / kTcTileM, (K + kTcTileK - 1) / kTcTileK, sms, B, N, K);
    CK(cudaMalloc(&w, (size_t)N * K * 2));
    CK(cudaMalloc(&x, (size_t)B * K * 2));
    CK(cudaMalloc(&o, (size_t)S * B * N * 4));
    CK(cudaMalloc(&e, 4));
    CK(cudaMemcpy(w, w_host, (size_t)N * K * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(x, x_host, (size_t)B * K * 2, cudaMemcpyHostToDevice));
    CK(cudaMemset(o, 0xff, (size_t)S * B * N * 4));
    CK(cudaMemset(e, 0, 4));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int32_t s = tc_gemm_launch(w, nullptr, x, N, K, B, S, o, N, 0, e, sms, 0, false);       // warm-up + result
    if (s == OXG4_OK) {
        cudaEventRecord(e0, 0);
        for (int rep = 0; rep < kDebugReps && s == OXG4_OK; ++rep) s = tc_gemm_launch(w, nullptr, x, N, K, B, S, o, N, 0, e, sms, 0, false);
        cudaEventRecord(e1, 0);
    }
    int err = 0;
    if (s == OXG4_OK && cudaDeviceSynchronize() != cudaSuccess) s = fail(OXG4_CUDA, "Gemma 4 CUDA error: tcgen05 projection failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (s == OXG4_OK) {
        cudaMemcpy(&err, e, 4, cudaMemcpyDeviceToHost);
        if (err) s = fail(OXG4_TIMEOUT, "tcgen05 projection: a bounded barrier wait ran out (code %d)", err);
    }
    if (s == OXG4_OK) {
        std::vector<float> part((size_t)S * B * N);
        cudaMemcpy(part.data(), o, part.size() * 4, cudaMemcpyDeviceToHost);
        for (size_t i2 = 0; i2 < (size_t)B * N; ++i2) {
            float t = 0.0f;
            for (int sp = 0; sp < S; ++sp) t += part[(size_t)sp * B * N + i2];      // split order, as the consumers do
            out_host[i2] = t;
        }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms_or_null) *ms_or_null = ms / kDebugReps;        // mean of back-to-back launches
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(w); cudaFree(x); cudaFree(o); cudaFree(e);
    return s;
}

#include "tp_group.inl"
