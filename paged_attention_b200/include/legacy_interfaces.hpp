#pragma once
// The reference's older host-fp32, single-head interfaces, kept as API surface so that callers
// written against them still compile: AttentionBackend (include/attention_backend.hpp:3-8),
// KVPool (include/kv_pool.hpp:3-13), Sequence (include/sequence.hpp:3-12), the device-side
// accessors ContiguousKV / PagedKV (include/kv_layout.hpp:4-30), ContiguousKVStore
// (include/kv_store.hpp:6-27), CUDA_CHECK (include/cuda_check.hpp:9-17) and the seeded input
// helpers (include/attention_utils.hpp:13-35).  The fp32 kernels that used to sit behind them are
// not rebuilt; paged_decode_backend.hpp puts the B200 decode engine behind the two abstract classes.

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

// Evaluates the call once; on failure prints the CUDA error with its location and aborts,
// which is how the legacy code paths report CUDA failures.
#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                                                         \
    do {                                                                                         \
        const cudaError_t pd_legacy_err_ = (call);                                               \
        if (pd_legacy_err_ != cudaSuccess) {                                                     \
            std::fprintf(stderr, "CUDA error %s at %s:%d: %s\n", cudaGetErrorName(pd_legacy_err_), \
                         __FILE__, __LINE__, cudaGetErrorString(pd_legacy_err_));                \
            std::abort();                                                                        \
        }                                                                                        \
    } while (0)
#endif

// One attention call on host buffers: q[d], K[T][d], V[T][d] -> out[d].
class AttentionBackend {
public:
    virtual ~AttentionBackend() = default;
    virtual void run(const float* q, const float* K, const float* V, float* out, int T, int d) = 0;
    virtual const char* name() const = 0;
};

// A pool of sequence slots holding K/V on the device; slot ids are small non-negative ints,
// admit() answers -1 when nothing is free.
class KVPool {
public:
    virtual ~KVPool() = default;
    virtual int  admit(const float* h_K, const float* h_V, int actual_len) = 0;
    virtual void release(int slot) = 0;
    virtual void append_token(int slot, int actual_len, const float* h_k, const float* h_v) = 0;
    virtual void decode(int slot, const float* h_q, float* h_out) = 0;
    virtual int  actual_len(int slot) const = 0;
    virtual bool is_occupied(int slot) const = 0;
};

// Buffers of one sequence in the legacy batch runner.
struct Sequence {
    float* d_q;
    float* d_K;
    float* d_V;
    float* d_scores;
    float* d_out;
    float* h_out;
    int    T;
    int    d;
};

#ifdef __CUDACC__
#define PD_LEGACY_DEVICE __forceinline__ __device__
#else
#define PD_LEGACY_DEVICE inline
#endif

// Element accessors over fp32 K/V: contiguous [T][d], or paged [page][slot][d] through a block table.
struct ContiguousKV {
    const float* K;
    const float* V;
    PD_LEGACY_DEVICE float key(int token, int dim, int d) const { return K[token * d + dim]; }
    PD_LEGACY_DEVICE float val(int token, int dim, int d) const { return V[token * d + dim]; }
};

struct PagedKV {
    const float* K_pool;
    const float* V_pool;
    const int*   block_table;
    int          page_size;
    PD_LEGACY_DEVICE size_t at(int token, int dim, int d) const {
        return (static_cast<size_t>(block_table[token / page_size]) * page_size + token % page_size) * d + dim;
    }
    PD_LEGACY_DEVICE float key(int token, int dim, int d) const { return K_pool[at(token, dim, d)]; }
    PD_LEGACY_DEVICE float val(int token, int dim, int d) const { return V_pool[at(token, dim, d)]; }
};

// Device copy of one sequence's fp32 K/V, freed with the object.
struct ContiguousKVStore {
    float* d_K = nullptr;
    float* d_V = nullptr;

    ContiguousKVStore(const float* h_K, const float* h_V, int T, int d) {
        const size_t bytes = sizeof(float) * static_cast<size_t>(T) * d;
        CUDA_CHECK(cudaMalloc(&d_K, bytes));
        CUDA_CHECK(cudaMalloc(&d_V, bytes));
        CUDA_CHECK(cudaMemcpy(d_K, h_K, bytes, cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(d_V, h_V, bytes, cudaMemcpyHostToDevice));
    }
    ~ContiguousKVStore() { cudaFree(d_K); cudaFree(d_V); }
    ContiguousKVStore(const ContiguousKVStore&)            = delete;
    ContiguousKVStore& operator=(const ContiguousKVStore&) = delete;

    ContiguousKV accessor() const { return ContiguousKV{d_K, d_V}; }
};

// Seeded uniform(-1, 1) inputs and the comparison helper of the legacy tests.
struct AttnInputs {
    std::vector<float> q, K, V;
};

inline void fill_random(float* data, int len, uint32_t seed) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::generate(data, data + len, [&] { return dist(rng); });
}

inline float max_abs_diff(const float* a, const float* b, int len) {
    float worst = 0.0f;
    for (int i = 0; i < len; i++) worst = std::max(worst, std::fabs(a[i] - b[i]));
    return worst;
}

inline AttnInputs make_attention_inputs(int d, int T, uint32_t seed) {
    AttnInputs in;
    in.q.resize(d);
    in.K.resize(static_cast<size_t>(d) * T);
    in.V.resize(static_cast<size_t>(d) * T);
    fill_random(in.q.data(), d, seed);
    fill_random(in.K.data(), d * T, seed + 1);
    fill_random(in.V.data(), d * T, seed + 2);
    return in;
}
