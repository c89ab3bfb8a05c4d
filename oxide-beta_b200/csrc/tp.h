// Tensor-parallel plumbing (host side): which slice of each checkpoint tensor a rank keeps, and a
// minimal run-time binding of NCCL (the library is looked up with dlopen, so liboxg4.so has no
// link-time dependency on it and single-GPU users never load it).
//
// The reference is single-GPU (no collective anywhere in it); the split is the standard one for a
// decoder block: q/k/v, gate and up are split by output rows (whole heads / intermediate columns),
// o and down by input columns, norms and scalars are replicated, the tied embedding table is
// replicated for the lookup and split by vocabulary rows for the LM head.
#pragma once
#include <dlfcn.h>
#include <stdint.h>

#include <string>

namespace oxg4 {

struct ShardSpec {
    // kept sub-matrix of a [rows, cols] tensor: rows [row0, row0 + nrows), columns [col0, col0 + ncols)
    int64_t row0 = 0, nrows = 0, col0 = 0, ncols = 0;
    bool replicated = true;
};

// `name` is the canonical tensor name (no checkpoint prefix). heads/kv_heads/head_dim/intermediate
// are the FULL model's sizes.
inline ShardSpec shard_of(const std::string& name, int64_t rows, int64_t cols, int tp_rank, int tp_size,
                          int heads, int kv_heads, int head_dim, int intermediate) {
    ShardSpec s;
    s.nrows = rows;
    s.ncols = cols;
    if (tp_size <= 1) return s;
    auto ends_with = [&](const char* suf) {
        const std::string t(suf);
        return name.size() >= t.size() && name.compare(name.size() - t.size(), t.size(), t) == 0;
    };
    const int64_t qw = (int64_t)heads / tp_size * head_dim;        // query columns per rank
    const int64_t kw = (int64_t)kv_heads / tp_size * head_dim;     // key/value columns per rank
    const int64_t iw = (int64_t)intermediate / tp_size;
    if (ends_with("self_attn.q_proj.weight")) { s.replicated = false; s.row0 = qw * tp_rank; s.nrows = qw; }
    else if (ends_with("self_attn.k_proj.weight") || ends_with("self_attn.v_proj.weight")) {
        s.replicated = false; s.row0 = kw * tp_rank; s.nrows = kw;
    } else if (ends_with("self_attn.o_proj.weight")) { s.replicated = false; s.col0 = qw * tp_rank; s.ncols = qw; }
    else if (ends_with("mlp.gate_proj.weight") || ends_with("mlp.up_proj.weight")) {
        s.replicated = false; s.row0 = iw * tp_rank; s.nrows = iw;
    } else if (ends_with("mlp.down_proj.weight")) { s.replicated = false; s.col0 = iw * tp_rank; s.ncols = iw; }
    return s;
}

// ---- NCCL through dlopen ---------------------------------------------------------------------------
struct NcclApi {
    typedef struct { char internal[128]; } UniqueId;
    typedef void* Comm;
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, Comm, void*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, Comm, void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    void* handle = nullptr;
    std::string error;
    static constexpr int kFloat32 = 7, kUint8 = 1, kSum = 0;      // ncclFloat32, ncclUint8, ncclSum

    bool load() {
        if (handle) return true;
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (handle) break;
        }
        if (!handle) { error = "libnccl.so.2 not found"; return false; }
        GetUniqueId = (int (*)(UniqueId*))dlsym(handle, "ncclGetUniqueId");
        CommInitRank = (int (*)(Comm*, int, UniqueId, int))dlsym(handle, "ncclCommInitRank");
        CommDestroy = (int (*)(Comm))dlsym(handle, "ncclCommDestroy");
        AllReduce = (int (*)(const void*, void*, size_t, int, int, Comm, void*))dlsym(handle, "ncclAllReduce");
        AllGather = (int (*)(const void*, void*, size_t, int, Comm, void*))dlsym(handle, "ncclAllGather");
        GetErrorString = (const char* (*)(int))dlsym(handle, "ncclGetErrorString");
        if (!GetUniqueId || !CommInitRank || !CommDestroy || !AllReduce || !AllGather || !GetErrorString) {
            error = "libnccl.so.2 lacks an expected symbol";
            return false;
        }
        return true;
    }
};

inline NcclApi& nccl() {
    static NcclApi api;
    return api;
}

}  // namespace oxg4
