// Tensor parallelism driven by ONE host thread: a group handle owns one model per GPU and one worker thread
// per rank, so that the reference's single-threaded surface (Gemma4ForCausalLM::generate holds an
// Rc<RefCell<Gemma4CudaState>>, crates/oxide-torch-models/src/models/gemma4/generation.rs:70-140) can drive
// N GPUs without a launcher: every call below hands the same per-rank call to all workers and waits for
// them. The per-rank calls are the ordinary entry points (oxg4_model_upload keeps the rank's shard, the step
// functions issue their NCCL collectives on the rank's own stream). Included at the end of oxg4.cu.
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

namespace {

class RankWorkers {
public:
    explicit RankWorkers(int n) : n_(n), status_(n, OXG4_OK), message_(n) {
        for (int r = 0; r < n; ++r) threads_.emplace_back([this, r] { loop(r); });
    }
    ~RankWorkers() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            quit_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (auto& t : threads_) t.join();
    }
    // runs fn(rank) on every worker; returns the first non-OK status and leaves its message for oxg4_last_error
    int32_t run(const std::function<int32_t(int)>& fn) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &fn;
            pending_ = n_;
            ++generation_;
        }
        cv_.notify_all();
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [this] { return pending_ == 0; });
        for (int r = 0; r < n_; ++r)
            if (status_[r] != OXG4_OK) {
                g_err = "rank " + std::to_string(r) + ": " + message_[r];
                return status_[r];
            }
        return OXG4_OK;
    }

private:
    void loop(int r) {
        unsigned long long seen = 0;
        for (;;) {
            const std::function<int32_t(int)>* fn = nullptr;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (quit_) return;
                fn = fn_;
            }
            const int32_t s = (*fn)(r);
            std::lock_guard<std::mutex> lk(mu_);
            status_[r] = s;
            message_[r] = s == OXG4_OK ? std::string() : g_err;     // g_err is the worker thread's own
            if (--pending_ == 0) done_.notify_all();
        }
    }
    int n_;
    std::vector<std::thread> threads_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    const std::function<int32_t(int)>* fn_ = nullptr;
    unsigned long long generation_ = 0;
    int pending_ = 0;
    bool quit_ = false;
    std::vector<int32_t> status_;
    std::vector<std::string> message_;
};

}  // namespace

struct oxg4_tp_cache;

struct oxg4_tp_model {
    int tp = 1;
    std::vector<oxg4_model*> rank;
    RankWorkers* workers = nullptr;
    std::vector<oxg4_tp_cache*> caches;           // live tables: destroyed with the group if the caller has not
};

struct oxg4_tp_cache {
    oxg4_tp_model* g = nullptr;
    std::vector<oxg4_cache*> rank;
    std::vector<std::vector<float>> scratch_f;        // results of the ranks other than 0 (identical copies)
    std::vector<std::vector<uint32_t>> scratch_u;
};

extern "C" void oxg4_tp_cache_destroy(oxg4_tp_cache* c);

extern "C" void oxg4_tp_model_destroy(oxg4_tp_model* g) {
    if (!g) return;
    while (!g->caches.empty()) oxg4_tp_cache_destroy(g->caches.back());
    if (g->workers) {
        g->workers->run([&](int r) {
            if (g->rank[r]) oxg4_model_destroy(g->rank[r]);
            return OXG4_OK;
        });
        delete g->workers;
    }
    delete g;
}

extern "C" int32_t oxg4_tp_model_create(const oxg4_config* c, const int32_t* device_ordinals, int32_t tp,
                                        oxg4_tp_model** out) {
    if (!c || !device_ordinals || !out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (tp != 1 && tp != 2 && tp != 4 && tp != 8) return fail(OXG4_INVALID_ARGUMENT, "tp must be 1, 2, 4 or 8");
    for (int a = 0; a < tp; ++a)
        for (int b = a + 1; b < tp; ++b)
            if (device_ordinals[a] == device_ordinals[b])
                return fail(OXG4_INVALID_ARGUMENT, "every tensor-parallel rank needs its own device");
    oxg4_tp_model* g = new oxg4_tp_model();
    g->tp = tp;
    g->rank.assign(tp, nullptr);
    g->workers = new RankWorkers(tp);
    const int32_t s = g->workers->run([&](int r) {
        oxg4_config rc = *c;
        rc.tp_rank = r;
        rc.tp_size = tp;
        return oxg4_model_create(&rc, device_ordinals[r], &g->rank[r]);
    });
    if (s != OXG4_OK) {
        const std::string keep = g_err;
        oxg4_tp_model_destroy(g);
        g_err = keep;
        return s;
    }
    *out = g;
    return OXG4_OK;
}

extern "C" int32_t oxg4_tp_model_upload(oxg4_tp_model* g, const char* name, int32_t dtype, const int64_t* shape,
                                        int32_t rank, const void* data, size_t bytes) {
    if (!g) return fail(OXG4_INVALID_ARGUMENT, "null model");
    return g->workers->run([&](int r) { return oxg4_model_upload(g->rank[r], name, dtype, shape, rank, data, bytes); });
}

extern "C" int32_t oxg4_tp_model_finalize(oxg4_tp_model* g) {
    if (!g) return fail(OXG4_INVALID_ARGUMENT, "null model");
    TRY(g->workers->run([&](int r) { return oxg4_model_finalize(g->rank[r]); }));
    if (g->tp == 1 || g->rank[0]->comm) return OXG4_OK;
    unsigned char id[128];
    TRY(oxg4_tp_unique_id(id));
    return g->workers->run([&](int r) { return oxg4_model_tp_init(g->rank[r], id); });
}

extern "C" int64_t oxg4_tp_weight_bytes(const oxg4_tp_model* g) {
    int64_t b = 0;
    if (g) for (auto* m : g->rank) b += oxg4_weight_bytes(m);
    return b;
}

extern "C" void oxg4_tp_cache_destroy(oxg4_tp_cache* c) {
    if (!c) return;
    {
        auto& live = c->g->caches;
        live.erase(std::remove(live.begin(), live.end(), c), live.end());
    }
    c->g->workers->run([&](int r) {
        if (c->rank[r]) oxg4_cache_destroy(c->rank[r]);
        return OXG4_OK;
    });
    delete c;
}

extern "C" int32_t oxg4_tp_cache_create(oxg4_tp_model* g, int32_t batch, const int32_t* max_seq, int32_t page_tokens,
                                        int32_t kv_dtype, oxg4_tp_cache** out) {
    if (!g || !out) return fail(OXG4_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    oxg4_tp_cache* c = new oxg4_tp_cache();
    c->g = g;
    c->rank.assign(g->tp, nullptr);
    c->scratch_f.resize(g->tp);
    c->scratch_u.resize(g->tp);
    const int32_t s = g->workers->run(
        [&](int r) { return oxg4_cache_create(g->rank[r], batch, max_seq, page_tokens, kv_dtype, &c->rank[r]); });
    if (s != OXG4_OK) {
        const std::string keep = g_err;
        oxg4_tp_cache_destroy(c);
        g_err = keep;
        return s;
    }
    g->caches.push_back(c);
    *out = c;
    return OXG4_OK;
}

extern "C" int32_t oxg4_tp_cache_position(const oxg4_tp_cache* c, int32_t b) {
    return c ? oxg4_cache_position(c->rank[0], b) : -1;
}

// every rank computes the same results; rank 0 writes into the caller's buffers, the others into scratch
extern "C" int32_t oxg4_tp_prefill(oxg4_tp_model* g, oxg4_tp_cache* c, const uint32_t* tokens, const int32_t* lens,
                                   float* last_logits) {
    if (!g || !c || c->g != g) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    const size_t n = (size_t)c->rank[0]->B * g->rank[0]->V;
    return g->workers->run([&](int r) {
        float* dst = last_logits;
        if (last_logits && r > 0) {
            c->scratch_f[r].resize(n);
            dst = c->scratch_f[r].data();
        }
        return oxg4_prefill(g->rank[r], c->rank[r], tokens, lens, dst);
    });
}

extern "C" int32_t oxg4_tp_decode_logits(oxg4_tp_model* g, oxg4_tp_cache* c, const uint32_t* tokens, float* logits) {
    if (!g || !c || !logits || c->g != g) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    const size_t n = (size_t)c->rank[0]->B * g->rank[0]->V;
    return g->workers->run([&](int r) {
        float* dst = logits;
        if (r > 0) {
            c->scratch_f[r].resize(n);
            dst = c->scratch_f[r].data();
        }
        return oxg4_decode_logits(g->rank[r], c->rank[r], tokens, dst);
    });
}

extern "C" int32_t oxg4_tp_decode_topk(oxg4_tp_model* g, oxg4_tp_cache* c, const uint32_t* tokens, int32_t top_k,
                                       float penalty, int32_t mark_seen, uint32_t* ids, float* scores) {
    if (!g || !c || !ids || !scores || c->g != g) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    const size_t n = (size_t)c->rank[0]->B * 64;
    return g->workers->run([&](int r) {
        uint32_t* di = ids;
        float* ds = scores;
        if (r > 0) {
            c->scratch_u[r].resize(n);
            c->scratch_f[r].resize(std::max(c->scratch_f[r].size(), n));
            di = c->scratch_u[r].data();
            ds = c->scratch_f[r].data();
        }
        return oxg4_decode_topk(g->rank[r], c->rank[r], tokens, top_k, penalty, mark_seen, di, ds);
    });
}

extern "C" int32_t oxg4_tp_decode_greedy(oxg4_tp_model* g, oxg4_tp_cache* c, const uint32_t* first_tokens, int32_t steps,
                                         uint32_t* out_ids, float* ms_per_step) {
    if (!g || !c || !out_ids || c->g != g) return fail(OXG4_INVALID_ARGUMENT, "null or mismatched handle");
    if (steps <= 0) return fail(OXG4_INVALID_ARGUMENT, "steps must be positive");
    const size_t n = (size_t)c->rank[0]->B * steps;
    std::vector<float> ms(g->tp, 0.0f);
    TRY(g->workers->run([&](int r) {
        uint32_t* dst = out_ids;
        if (r > 0) {
            c->scratch_u[r].resize(n);
            dst = c->scratch_u[r].data();
        }
        return oxg4_decode_greedy(g->rank[r], c->rank[r], first_tokens, steps, dst, &ms[r]);
    }));
    if (ms_per_step) *ms_per_step = *std::max_element(ms.begin(), ms.end());
    return OXG4_OK;
}
