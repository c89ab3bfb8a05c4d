/* A plain C caller of the library's C ABI (include/oxg4.h), compiled by tests/test_c_driver.py.
 *
 * It walks the calls that the reference's Rust side would make through a `-sys` crate:
 * oxg4_model_create -> oxg4_model_upload (every tensor) -> oxg4_model_finalize -> oxg4_cache_create ->
 * oxg4_prefill -> host arg-max -> oxg4_decode_topk (greedy loop) -> destroy, i.e. Gemma4CudaState::load,
 * new_cache_table, prefill_prompt and decode_topk as generate_with_callback drives them
 * (crates/oxide-torch-models/src/models/gemma4/generation.rs:92-133).
 *
 * Input: one binary file written by the test (configuration, prompt, tensors). Output on stdout:
 * "TOKENS: t0 t1 ..." or, when no CUDA device exists, "NO_DEVICE: <message>" with exit code 3.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "oxg4.h"

static void die(const char* what) {
    fprintf(stderr, "c_driver: %s: %s\n", what, oxg4_last_error());
    exit(1);
}

static void rd(void* dst, size_t n, FILE* f) {
    if (fread(dst, 1, n, f) != n) {
        fprintf(stderr, "c_driver: short read\n");
        exit(2);
    }
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 2;
    char magic[8];
    rd(magic, 8, f);
    if (memcmp(magic, "OXG4TEST", 8) != 0) return 2;
    int32_t ci[10];           /* vocab, hidden, layers, heads, kv_heads, head_dim, intermediate, window, weight dtype, kv dtype */
    float eps;
    rd(ci, sizeof ci, f);
    rd(&eps, 4, f);
    const int L = ci[2];
    int32_t* sliding = malloc(sizeof(int32_t) * L);
    int32_t* rotary = malloc(sizeof(int32_t) * L);
    float* theta = malloc(sizeof(float) * L);
    float* factor = malloc(sizeof(float) * L);
    rd(sliding, sizeof(int32_t) * L, f);
    rd(rotary, sizeof(int32_t) * L, f);
    rd(theta, sizeof(float) * L, f);
    rd(factor, sizeof(float) * L, f);
    uint32_t n_prompt, n_decode, n_tensors;
    rd(&n_prompt, 4, f);
    uint32_t* prompt = malloc(4 * n_prompt);
    rd(prompt, 4 * n_prompt, f);
    rd(&n_decode, 4, f);
    rd(&n_tensors, 4, f);

    oxg4_config cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.vocab_size = ci[0]; cfg.hidden_size = ci[1]; cfg.num_hidden_layers = L; cfg.num_attention_heads = ci[3];
    cfg.num_key_value_heads = ci[4]; cfg.head_dim = ci[5]; cfg.global_head_dim = ci[5]; cfg.intermediate_size = ci[6];
    cfg.sliding_window = ci[7]; cfg.rms_norm_eps = eps; cfg.final_logit_softcapping = 0.0f; cfg.weight_dtype = ci[8];
    cfg.layer_is_sliding = sliding; cfg.rotary_dim = rotary; cfg.rope_theta = theta; cfg.rope_factor = factor;
    cfg.tp_rank = 0; cfg.tp_size = 1;

    oxg4_model* model = NULL;
    int32_t st = oxg4_model_create(&cfg, 0, &model);
    if (st == OXG4_CUDA) {
        printf("NO_DEVICE: %s\n", oxg4_last_error());
        return 3;
    }
    if (st != OXG4_OK) die("oxg4_model_create");
    for (uint32_t t = 0; t < n_tensors; ++t) {
        uint32_t name_len, dtype, rank;
        char name[256];
        int64_t shape[4];
        uint64_t nbytes;
        rd(&name_len, 4, f);
        if (name_len >= sizeof name) return 2;
        rd(name, name_len, f);
        name[name_len] = 0;
        rd(&dtype, 4, f);
        rd(&rank, 4, f);
        rd(shape, 8 * rank, f);
        rd(&nbytes, 8, f);
        void* data = malloc(nbytes);
        rd(data, nbytes, f);
        if (oxg4_model_upload(model, name, (int32_t)dtype, shape, (int32_t)rank, data, nbytes) != OXG4_OK) die(name);
        free(data);                                 /* the copy has completed when the call returns */
    }
    fclose(f);
    if (oxg4_model_finalize(model) != OXG4_OK) die("oxg4_model_finalize");
    if (oxg4_weight_count(model) <= 0 || oxg4_weight_bytes(model) <= 0) die("weight accounting");

    oxg4_cache* cache = NULL;
    const int32_t max_seq = (int32_t)(n_prompt + n_decode);
    if (oxg4_cache_create(model, 1, &max_seq, 256, ci[9], &cache) != OXG4_OK) die("oxg4_cache_create");
    float* logits = malloc(sizeof(float) * cfg.vocab_size);
    const int32_t len = (int32_t)n_prompt;
    if (oxg4_prefill(model, cache, prompt, &len, logits) != OXG4_OK) die("oxg4_prefill");
    uint32_t tok = 0;
    for (int32_t i = 1; i < cfg.vocab_size; ++i)
        if (logits[i] > logits[tok]) tok = (uint32_t)i;      /* greedy: first maximum */
    printf("TOKENS:");
    for (uint32_t s = 0; s < n_decode; ++s) {
        printf(" %u", tok);
        if (s + 1 == n_decode) break;
        uint32_t id;
        float score;
        if (oxg4_decode_topk(model, cache, &tok, 1, 1.0f, 1, &id, &score) != OXG4_OK) die("oxg4_decode_topk");
        tok = id;
    }
    printf("\n");
    if (oxg4_cache_position(cache, 0) != (int32_t)(n_prompt + n_decode - 1)) die("cache position");
    oxg4_cache_destroy(cache);
    oxg4_model_destroy(model);
    free(logits); free(prompt); free(sliding); free(rotary); free(theta); free(factor);
    return 0;
}
