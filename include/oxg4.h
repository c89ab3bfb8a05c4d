/* oxg4.h — C ABI of the B200-native Gemma4 token-generation path.
 *
 * This library replaces, for Gemma4 decode only, what the reference project (tuna2134/oxide-beta)
 * implements in crates/oxide-torch-cuda (kernel module, cuBLAS and CUDA-graph wrappers) and in
 * crates/oxide-torch-models/src/gemma4_cuda (the Gemma4 CUDA executor). The reference's Rust
 * types become owners of the opaque handles declared here; their public signatures do not change.
 * Each entry point cites the reference interface it stands in for (paths inside the reference).
 *
 * Conventions
 *   - every function returns an oxg4_status; 0 is success; no exception crosses the boundary
 *   - a failing call leaves a message retrievable with oxg4_last_error()
 *   - all pointers are HOST pointers; device memory never crosses the boundary
 *   - handles are not thread-safe; calls on one model/cache are serialised by the caller
 *     (the reference state is Rc<RefCell<..>>, i.e. !Send + !Sync)
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails
 */
#ifndef OXG4_H
#define OXG4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct oxg4_model oxg4_model;   /* Gemma4CudaState        (gemma4_cuda/mod.rs:161-175)   */
typedef struct oxg4_cache oxg4_cache;   /* Gemma4CudaCacheTable   (gemma4_cuda/mod.rs:119-159)   */

typedef enum {
    OXG4_OK = 0,
    OXG4_INVALID_SHAPE = 1,     /* oxide_torch::Error::InvalidShape                               */
    OXG4_INVALID_ARGUMENT = 2,  /* oxide_torch::Error::Execution for bad input                    */
    OXG4_CUDA = 3,              /* Error::Execution("Gemma 4 CUDA error: ...") mod.rs:581-583     */
    OXG4_NCCL = 4,
    OXG4_OOM = 5,
    OXG4_TIMEOUT = 6,
    OXG4_UNSUPPORTED = 7
} oxg4_status;

typedef enum { OXG4_F32 = 0, OXG4_BF16 = 1 } oxg4_dtype;

/* Subset of Gemma4TextConfig the decode path reads (models/gemma4/config.rs:103-148) plus the
 * per-layer plan fields of Gemma4DecodeLayerPlan (gemma4_cuda/mod.rs:65-93, 365-413). */
typedef struct {
    int32_t vocab_size;
    int32_t hidden_size;
    int32_t num_hidden_layers;
    int32_t num_attention_heads;
    int32_t num_key_value_heads;
    int32_t head_dim;
    int32_t global_head_dim;          /* head_dim of the global (full_attention) layers (mod.rs:391-395) */
    int32_t intermediate_size;
    int32_t sliding_window;
    float rms_norm_eps;
    float final_logit_softcapping;    /* 0 = none; applied on the host to returned scores/logits   */
    int32_t weight_dtype;             /* OXG4_BF16: the reference's recipe (BF16 weights, BF16-
                                         rounded GEMM inputs, f32 accumulate and activations).
                                         OXG4_F32: f32 weights, no rounding (tiny CPU-checkable case) */
    int32_t norm_weight_offset;       /* 0: x*s*w as the reference; 1: x*s*(1+w)                   */
    const int32_t* layer_is_sliding;  /* [num_hidden_layers] 1 = sliding_attention                 */
    const int32_t* rotary_dim;        /* [num_hidden_layers] (partial_rotary_factor * head_dim)     */
    const float* rope_theta;          /* [num_hidden_layers]                                        */
    const float* rope_factor;         /* [num_hidden_layers]                                        */
    int32_t tp_rank;                  /* tensor-parallel rank of this process (0 when tp_size = 1)  */
    int32_t tp_size;                  /* 1, 2, 4 or 8; must divide the KV-head count               */
    /* Gemma4-E fields (config.rs:116-139); zero = the feature is off */
    int32_t num_global_key_value_heads; /* KV heads of the global layers when attention_k_eq_v is set
                                           (cache.rs:63-68); 0 = num_key_value_heads                 */
    int32_t attention_k_eq_v;
    int32_t num_kv_shared_layers;     /* the last n layers read the K/V cache of the last earlier layer of
                                         their own type and have a q projection only (cache.rs:43-86)  */
    int32_t hidden_size_per_layer_input; /* width P of the per-layer embeddings (ple.rs); 0 = none      */
    int32_t vocab_size_per_layer_input;  /* rows of embed_tokens_per_layer.weight                        */
} oxg4_config;

typedef struct {
    int32_t batch;
    int32_t layer_count;              /* Gemma4CudaCacheTable::layer_count                          */
    int32_t physical_cache_count;     /* ::physical_cache_count                                     */
    int32_t shared_layer_count;       /* ::shared_layer_count (layers that read another layer's cache) */
    int32_t page_tokens;
    int32_t kv_dtype;
    int64_t kv_bytes;                 /* device bytes held by K and V pools                         */
} oxg4_cache_info;

/* Message of the most recent failing call on this thread. */
const char* oxg4_last_error(void);

/* ---- model: Gemma4CudaState::load (gemma4_cuda/mod.rs:221-466) split into three steps ---------- */

/* CudaContext::new(n) + stream creation (mod.rs:221-232). `device` is the ordinal of Device::Cuda(n). */
int32_t oxg4_model_create(const oxg4_config* config, int32_t device, oxg4_model** out);

/* Upload of one checkpoint tensor (mod.rs:236-279). `name` is the checkpoint name with or without
 * the "model.language_model." prefix. The copy has completed when the call returns, so it may be
 * made from inside SafeTensorLoader::with_view (crates/oxide-torch/src/safetensors.rs:182-189).
 * With tp_size > 1 the full tensor is passed and only this rank's shard is kept. */
int32_t oxg4_model_upload(oxg4_model* model, const char* name, int32_t dtype, const int64_t* shape,
                          int32_t rank, const void* data, size_t bytes);

/* QKV fusion + decode-plan construction (mod.rs:283-449). */
int32_t oxg4_model_finalize(oxg4_model* model);

void oxg4_model_destroy(oxg4_model* model);

/* Gemma4CudaState::weight_count / weight_bytes (mod.rs:468-476). */
int64_t oxg4_weight_count(const oxg4_model* model);
int64_t oxg4_weight_bytes(const oxg4_model* model);

/* Gemma4CudaState::synchronize (mod.rs:478-480). */
int32_t oxg4_synchronize(oxg4_model* model);

/* Tensor parallelism (no counterpart in the reference, which is single-GPU): every rank creates
 * its model with the same tp_size and its own tp_rank; rank 0 obtains an id, the host program
 * distributes the 128 bytes to the other ranks, and all ranks call oxg4_model_tp_init. */
int32_t oxg4_tp_unique_id(void* out_128_bytes);
/* The sub-matrix of checkpoint tensor `name` ([rows, cols]) that rank tp_rank of tp_size keeps:
 * out4 = {first row, rows kept, first column, columns kept}. Pure host arithmetic. q/k/v, gate and up
 * are split by rows (whole heads / intermediate columns), o and down by columns, the rest replicated. */
int32_t oxg4_tp_shard(const char* name, int64_t rows, int64_t cols, int32_t tp_rank, int32_t tp_size,
                      int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t intermediate, int64_t* out4);
int32_t oxg4_model_tp_init(oxg4_model* model, const void* unique_id_128_bytes);

/* Tensor parallelism driven by one host thread (no counterpart in the reference). The reference's surface is
 * single-threaded (Gemma4ForCausalLM::generate owns an Rc<RefCell<Gemma4CudaState>>, models/gemma4/
 * generation.rs:70-140), so a multi-GPU state behind it cannot need one process or thread per rank from its
 * caller: the group handle below owns one model per device in `device_ordinals` and one internal worker
 * thread + stream per rank, and every call fans out to the ranks and waits. Semantics, arguments and
 * results are those of the single-GPU entry points of the same name; uploads take the FULL tensor (every
 * rank keeps its shard); NCCL is set up inside oxg4_tp_model_finalize. Handles are not thread-safe. */
typedef struct oxg4_tp_model oxg4_tp_model;
typedef struct oxg4_tp_cache oxg4_tp_cache;
int32_t oxg4_tp_model_create(const oxg4_config* config, const int32_t* device_ordinals, int32_t tp, oxg4_tp_model** out);
int32_t oxg4_tp_model_upload(oxg4_tp_model* model, const char* name, int32_t dtype, const int64_t* shape,
                             int32_t rank, const void* data, size_t bytes);
int32_t oxg4_tp_model_finalize(oxg4_tp_model* model);
void oxg4_tp_model_destroy(oxg4_tp_model* model);
int64_t oxg4_tp_weight_bytes(const oxg4_tp_model* model);
int32_t oxg4_tp_cache_create(oxg4_tp_model* model, int32_t batch, const int32_t* max_seq, int32_t page_tokens,
                             int32_t kv_dtype, oxg4_tp_cache** out);
void oxg4_tp_cache_destroy(oxg4_tp_cache* cache);
int32_t oxg4_tp_cache_position(const oxg4_tp_cache* cache, int32_t b);
int32_t oxg4_tp_prefill(oxg4_tp_model* model, oxg4_tp_cache* cache, const uint32_t* tokens, const int32_t* lens,
                        float* last_logits);
int32_t oxg4_tp_decode_logits(oxg4_tp_model* model, oxg4_tp_cache* cache, const uint32_t* tokens, float* logits);
int32_t oxg4_tp_decode_topk(oxg4_tp_model* model, oxg4_tp_cache* cache, const uint32_t* tokens, int32_t top_k,
                            float repetition_penalty, int32_t mark_seen, uint32_t* ids, float* scores);
int32_t oxg4_tp_decode_greedy(oxg4_tp_model* model, oxg4_tp_cache* cache, const uint32_t* first_tokens, int32_t steps,
                              uint32_t* out_ids, float* ms_per_step);

/* Peer-memory exchange for tensor parallelism (no counterpart in the reference). With tp_size > 1 and
 * 8..64 sequences the sums after the O and down projections can travel through buffers that the
 * ranks map into each other with CUDA IPC instead of NCCL calls: every rank exports the handle of its
 * cache table's exchange block, the host program gathers the tp_size handles (64 bytes each, in rank
 * order) and every rank connects. Until connected (or with OXG4_TP_NCCL set) the NCCL path is used. All
 * ranks must make the same sequence of step calls. */
int32_t oxg4_cache_tp_export(oxg4_cache* cache, void* handle_out_64_bytes);
int32_t oxg4_cache_tp_connect(oxg4_cache* cache, const void* handles_tp_size_x_64_bytes);

/* ---- KV cache: new_cache_table (gemma4_cuda/cache.rs:31-95) -------------------------------------- */

/* `max_seq[b]` is the longest sequence (prompt + generated) sequence b may reach. Sliding layers
 * get a ring of min(sliding_window, max_seq[b]) positions, global layers max_seq[b] positions, in
 * pages of `page_tokens` tokens. kv_dtype OXG4_F32 is the reference's cache; OXG4_BF16 halves it. */
int32_t oxg4_cache_create(oxg4_model* model, int32_t batch, const int32_t* max_seq,
                          int32_t page_tokens, int32_t kv_dtype, oxg4_cache** out);
void oxg4_cache_destroy(oxg4_cache* cache);
int32_t oxg4_cache_info_get(const oxg4_cache* cache, oxg4_cache_info* out);
/* Tokens processed so far for sequence b (Gemma4CudaKvCache::len semantics on a global layer). */
int32_t oxg4_cache_position(const oxg4_cache* cache, int32_t b);
/* Empties the cache and the seen-token bitmap so the table can serve a new generation
 * (reset_generation_state, mod.rs:178-180, plus a fresh table). */
int32_t oxg4_cache_reset(oxg4_cache* cache);

/* ---- steps ------------------------------------------------------------------------------------------ */

/* prefill_prompt (gemma4_cuda/decode.rs:431-459). `tokens` holds the prompts back to back,
 * `lens[b]` tokens for sequence b. last_logits (may be NULL) receives [batch, vocab] f32 logits
 * of each prompt's final token. The cache must be empty. */
int32_t oxg4_prefill(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens,
                     const int32_t* lens, float* last_logits);

/* prefill_token (decode.rs:464-472): one token per sequence, no LM head.
 * A token id of 0xFFFFFFFF leaves that sequence untouched in this step. */
int32_t oxg4_prefill_token(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens);

/* decode_token (decode.rs:476-486): one token per sequence, logits [batch, vocab] to the host. */
int32_t oxg4_decode_logits(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens, float* logits);

/* decode_topk (decode.rs:666-783): one token per sequence; returns for each sequence the top_k
 * (clamped to 1..=64) candidates in descending order, repetition penalty applied on the device
 * to tokens marked seen. ids/scores are [batch, top_k]. The step is captured as a CUDA graph on
 * first use for a (top_k, penalty) pair and replayed afterwards. */
int32_t oxg4_decode_topk(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens, int32_t top_k,
                         float repetition_penalty, int32_t mark_seen, uint32_t* ids, float* scores);

/* Device-resident greedy loop (no counterpart in the reference, whose host samples every token):
 * runs `steps` decode steps feeding each step's arg-max back as the next token without leaving
 * the GPU, then returns the generated ids [steps, batch] and the mean device time per step.
 * Equivalent to calling oxg4_decode_topk(top_k = 1, penalty = 1) `steps` times. */
int32_t oxg4_decode_greedy(oxg4_model* model, oxg4_cache* cache, const uint32_t* first_tokens,
                           int32_t steps, uint32_t* out_ids, float* ms_per_step);

/* Device-resident sampled generation (no counterpart in the reference, whose host draws every token
 * in sample_topk_candidates, sampling.rs:88-158): runs `steps` decode steps; after each one a kernel
 * draws the next token from the step's top_k (2..=64) candidates with the reference's arithmetic
 * (temperature, softmax, top-p, xorshift64 13/7/17, 24-bit uniform) and feeds it back without leaving
 * the GPU. Tokens fed in are marked seen, the repetition penalty applies as in oxg4_decode_topk.
 * seeds: [batch] generator states, updated in place, so that oxg4_sample_topk_candidates continues the
 * same stream on the host. out_ids: [steps, batch]. Not available with tensor parallelism. */
int32_t oxg4_decode_sampled(oxg4_model* model, oxg4_cache* cache, const uint32_t* first_tokens, int32_t steps,
                            int32_t top_k, float temperature, float top_p, float repetition_penalty,
                            uint64_t* seeds, uint32_t* out_ids, float* ms_per_step);

/* Number of kernels launched by this library since the model was created (graph replays count
 * the kernels inside the graph). */
int64_t oxg4_kernel_launches(const oxg4_model* model);

/* Mean device time in milliseconds, measured with CUDA events on the model's stream, of the
 * launches of the kind `kind` ("qkv", "attn", "o", "gateup", "down", "lmhead", "norm", "geglu", "sum",
 * "topk1", "topk2", "allreduce", "allgather", ...) during the most recent oxg4_profile_step call, and
 * how many launches of that kind the step made; that call runs one eager decode step with events
 * around every kernel and every tensor-parallel collective. Measurement aid in the role of the
 * reference's GEMMA4_PROFILE hook (crates/oxide-torch-models/examples/gemma4_load.rs:277-284). */
int32_t oxg4_profile_step(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens);
float oxg4_profile_ms(const oxg4_model* model, const char* kind);
int32_t oxg4_profile_count(const oxg4_model* model, const char* kind);

/* Diagnostic entry points: the reference's smoke functions (crates/oxide-torch-models/src/gemma4_cuda/smoke.rs),
 * one token through one block of one layer, on a single-GPU model.
 *   oxg4_smoke_embedding_logits   embedding_logits (smoke.rs:8-30): embedding row * sqrt(hidden) -> BF16 -> tied LM
 *                                 head; logits[vocab_size], no final norm, no soft cap
 *   oxg4_smoke_decoder_mlp        decoder_mlp_smoke (smoke.rs:32-59): out[hidden_size]
 *   oxg4_smoke_decoder_attention  decoder_attention_smoke (smoke.rs:61-126), one token at position 0: out[hidden_size]
 *   oxg4_smoke_cached_attention   cached_attention_smoke (smoke.rs:128-204): appends the token to `layer`'s K/V ring of
 *                                 a ONE-sequence cache table and returns the attention output
 *                                 attended[num_attention_heads * head_dim of the layer]; the table's position
 *                                 advances by one. A one-sequence table created with oxg4_cache_create stands in
 *                                 for new_kv_cache (cache.rs:5-29); use it for nothing but these calls.
 * hidden_size / heads / epsilon / window, which the reference takes as arguments, come from the model's config.
 * The layer's own RoPE parameters are used where the reference passes theta 10000, factor 1 and the full head
 * (the sliding layers' values; identical at position 0). KV-shared layers are refused by the attention calls. */
int32_t oxg4_smoke_embedding_logits(oxg4_model* model, uint32_t token, float* logits);
int32_t oxg4_smoke_decoder_mlp(oxg4_model* model, uint32_t token, int32_t layer, float* out);
int32_t oxg4_smoke_decoder_attention(oxg4_model* model, uint32_t token, int32_t layer, float* out);
int32_t oxg4_smoke_cached_attention(oxg4_model* model, oxg4_cache* cache, uint32_t token, int32_t layer, float* attended);

/* Failure-path test hooks (no counterpart in the reference, whose errors are Result values and whose
 * capture always ends, crates/oxide-torch-cuda/src/cuda_graph.rs:84-97). Neither faults or hangs a GPU.
 * oxg4_debug_wait_timeout runs one of the library's bounded device-side waits (kind 1: mbarrier phase,
 * kind 2: tensor-parallel peer flag) on something nobody signals, with a polling budget of `spin_limit`:
 * the kernel returns, the status word is raised and the call returns OXG4_TIMEOUT; later calls work.
 * oxg4_debug_fail_alloc_after makes the n-th device allocation of the next oxg4_cache_create report
 * OXG4_OOM (0 switches it off); the failed create must release everything it had allocated. */
int32_t oxg4_debug_wait_timeout(oxg4_model* model, oxg4_cache* cache, int32_t kind, uint32_t spin_limit);
void oxg4_debug_fail_alloc_after(int32_t n);

/* Measurement aid (no counterpart in the reference): marks lens[b] positions of every sequence of an EMPTY cache
 * table as cached and fills the K/V pools with a fixed pseudo-random pattern, so that decode steps at a long
 * context can be timed without ingesting the prompts first. The pool contents are not the K/V of any prompt:
 * only timing, never parity, may be taken from a table filled this way. */
int32_t oxg4_debug_fill_cache(oxg4_model* model, oxg4_cache* cache, const int32_t* lens);

/* Top-k selection that allocates nothing (no counterpart in the reference). It is meant for callers
 * that are not allowed to allocate device memory at the moment they need a top-k: code running
 * between cudaStreamBeginCapture and cudaStreamEndCapture on a stream, where cudaMalloc is illegal;
 * serving loops with a fixed memory budget that forbid allocation after start-up; and hosts that own
 * every byte of device memory through their own arena. The usual path (oxg4_decode_topk) keeps its
 * candidate lists in buffers that oxg4_cache_create allocates; this variant runs the same two
 * kernels with the candidate lists in a fixed 512 KiB array inside the library image, so it calls
 * no cudaMalloc, cudaFree or any other allocating routine.
 *   logits_dev  [rows, vocab] f32, DEVICE pointer        seen_dev  [rows, vocab] bytes or NULL (DEVICE)
 *   ids_dev     [rows, top_k] u32, DEVICE pointer        scores_dev [rows, top_k] f32, DEVICE pointer
 *   cuda_stream a cudaStream_t (NULL = the default stream); the call only enqueues work on it.
 * Limits: rows <= 4 and vocab <= 524288 per call (larger sizes are rejected with
 * OXG4_INVALID_SHAPE); top_k is clamped to 1..=64 as in oxg4_decode_topk. Result order, tie-break,
 * penalty and NaN handling are those of oxg4_decode_topk.
 * The array is shared by every call on a device and keeps the previous call's contents. Nothing in
 * it has to start at zero (each call overwrites every entry it later reads), but two calls whose
 * kernels overlap on the GPU (different streams, no ordering between them) race on it: order them.
 * The first call on each device looks up the array's device address and configures the merge
 * kernel; make that first call before any stream capture begins. */
int32_t oxg4_topk_noalloc(const float* logits_dev, int32_t rows, int32_t vocab, const uint8_t* seen_dev,
                          float repetition_penalty, int32_t top_k, uint32_t* ids_dev, float* scores_dev,
                          void* cuda_stream);

/* Layer-wise trace of one decode step, the counterpart of the reference's GEMMA4_TRACE_LAYERS
 * fingerprints (gemma4_cuda/mod.rs:182-199, decode.rs:351-369), returning the tensors themselves.
 * `trace` receives [layers + 1, batch, hidden] f32: the input of every layer as this library
 * computed it (entry l > 0 = output of layer l - 1) and the final hidden state. `inject` (may be
 * NULL) holds [layers, batch, hidden] f32 values that REPLACE the input of every layer after it
 * has been recorded (layer-wise teacher forcing for parity tests); `logits` (may be NULL) receives
 * [batch, vocab]. Runs eagerly (no graph) and advances the cache like oxg4_decode_logits. */
int32_t oxg4_decode_trace(oxg4_model* model, oxg4_cache* cache, const uint32_t* tokens, const float* inject,
                          float* trace, float* logits);

/* Stand-alone run of the tcgen05/TMEM batched projection kernel (csrc/tc_gemm.cuh) for its parity
 * tests: out[B, N] = x[B, K] . W[N, K]^T with BF16 inputs given as bit patterns, f32 output, the
 * contract of Cublas::linear_bf16_f32 (crates/oxide-torch-cuda/src/cublas.rs:101-153). 1 <= B <= 256,
 * K a multiple of 8. ms (may be NULL) receives the mean device time of ten back-to-back launches. Returns OXG4_TIMEOUT
 * if one of the kernel's bounded barrier waits ran out. */
int32_t oxg4_debug_tc_gemm(const uint16_t* w_host, const uint16_t* x_host, int32_t N, int32_t K, int32_t B,
                           float* out_host, float* ms);

/* Diagnostics (no counterpart in the reference): when the environment variable OXG4_TIMELINE is
 * set before oxg4_model_create, every kernel of a step stamps the GPU's nanosecond timer at entry,
 * after its dependency wait, after its prologue and at exit. Copies the stamps of the most recent
 * step, four per kernel in launch order, to `out`. */
int32_t oxg4_debug_timeline(oxg4_cache* cache, unsigned long long* out, int32_t max_entries);

/* ---- host-side mirror of the generation loop -------------------------------------------------------- */

/* GenerationConfig (models/gemma4/config.rs:7-33). */
typedef struct {
    int64_t max_new_tokens;
    float temperature;
    int64_t top_k;
    float top_p;
    float repetition_penalty;
    uint64_t seed;
    const uint32_t* eos_token_ids;
    int64_t n_eos;
    const uint32_t* stop_sequences;       /* flattened */
    const int64_t* stop_sequence_lens;
    int64_t n_stop_sequences;
} oxg4_generation_config;

typedef int32_t (*oxg4_token_callback)(uint32_t token, void* user);

/* Gemma4ForCausalLM::generate / generate_stream (models/gemma4/generation.rs:47-140) for one
 * sequence: validate, new cache table, prefill, sample, callback, EOS / stop check, decode_topk.
 * out_ids must hold n_prompt + max_new_tokens entries; *n_out receives the length written
 * (prompt followed by the generated ids). A non-zero callback return aborts with
 * OXG4_INVALID_ARGUMENT, mirroring an Err from on_token. */
int32_t oxg4_generate(oxg4_model* model, const uint32_t* prompt, int64_t n_prompt,
                      const oxg4_generation_config* generation, int32_t kv_dtype,
                      oxg4_token_callback on_token, void* user, uint32_t* out_ids, int64_t* n_out);

/* sample_token / sample_topk_candidates (models/gemma4/sampling.rs:9-158). Return the token id or
 * -1 for the inputs the reference rejects. `random` is the xorshift64 state, updated in place. */
int64_t oxg4_sample_token(const float* logits, int64_t n, float temperature, int64_t top_k,
                          float top_p, uint64_t* random);
int64_t oxg4_sample_topk_candidates(const uint32_t* ids, const float* scores, int64_t n,
                                    float temperature, float top_p, uint64_t* random);

#ifdef __cplusplus
}
#endif
#endif /* OXG4_H */
