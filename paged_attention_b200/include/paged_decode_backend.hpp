#pragma once
// The B200 decode engine behind the reference's two legacy abstract classes:
//   PagedDecodeAttention : AttentionBackend   one (q, K, V) -> out call on host fp32 buffers
//   PagedDecodePool      : KVPool             admit / append_token / decode / release on host fp32
// Both store K/V as fp16 in a decode::PagedKVCache with one kv head and head_dim 128 (the only
// head_dim the engine supports; other sizes throw std::invalid_argument), so results differ from
// an fp32 kernel by fp16 storage rounding (about 1e-3 on uniform(-1,1) inputs).

#include "decode/paged_kv_cache.hpp"
#include "legacy_interfaces.hpp"

#include <cuda_fp16.h>

#include <memory>
#include <stdexcept>
#include <vector>

namespace pd_legacy {

inline std::vector<half> to_half(const float* x, size_t n) {
    std::vector<half> h(n);
    for (size_t i = 0; i < n; i++) h[i] = __float2half(x[i]);
    return h;
}

// RAII device buffer of halves filled from host floats.
class HalfBuffer {
public:
    HalfBuffer(const float* x, size_t n) : n_(n) {
        const std::vector<half> h = to_half(x, n);
        CUDA_CHECK(cudaMalloc(&d_, sizeof(half) * std::max<size_t>(n, 1)));
        CUDA_CHECK(cudaMemcpy(d_, h.data(), sizeof(half) * n, cudaMemcpyHostToDevice));
    }
    explicit HalfBuffer(size_t n) : n_(n) { CUDA_CHECK(cudaMalloc(&d_, sizeof(half) * std::max<size_t>(n, 1))); }
    ~HalfBuffer() { cudaFree(d_); }
    HalfBuffer(const HalfBuffer&)            = delete;
    HalfBuffer& operator=(const HalfBuffer&) = delete;
    half* get() const { return d_; }
    void to_host(float* out) const {
        std::vector<half> h(n_);
        CUDA_CHECK(cudaMemcpy(h.data(), d_, sizeof(half) * n_, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n_; i++) out[i] = __half2float(h[i]);
    }
private:
    half*  d_ = nullptr;
    size_t n_;
};

}  // namespace pd_legacy

class PagedDecodePool : public KVPool {
public:
    static constexpr int kPageSize = 16;

    PagedDecodePool(int num_pages, int max_slots, int max_pages_per_slot, int d) : d_(d) {
        decode::PagedKVCache::Config cfg{};
        cfg.num_pages = num_pages; cfg.page_size = kPageSize; cfg.num_kv_heads = 1; cfg.head_dim = d;
        cfg.max_slots = max_slots; cfg.max_pages_per_slot = max_pages_per_slot;
        cache_ = std::make_unique<decode::PagedKVCache>(cfg);   // throws std::invalid_argument unless d == 128
    }

    // Claims a slot and loads actual_len tokens; -1 (and nothing claimed) if no slot or not enough pages.
    int admit(const float* h_K, const float* h_V, int actual_len) override {
        const int slot = cache_->admit();
        if (slot < 0) return -1;
        if (actual_len > 0) {
            pd_legacy::HalfBuffer k(h_K, static_cast<size_t>(actual_len) * d_), v(h_V, static_cast<size_t>(actual_len) * d_);
            if (!cache_->append(slot, k.get(), v.get(), actual_len)) {
                cache_->release(slot);
                return -1;
            }
        }
        return slot;
    }
    void release(int slot) override { cache_->release(slot); }
    // actual_len is the length before this token, as in the legacy interface; it must match the pool's.
    void append_token(int slot, int actual_len, const float* h_k, const float* h_v) override {
        if (actual_len != cache_->seq_len(slot)) throw std::invalid_argument("append_token: actual_len does not match the slot");
        pd_legacy::HalfBuffer k(h_k, d_), v(h_v, d_);
        if (!cache_->append(slot, k.get(), v.get(), 1)) throw std::length_error("append_token: out of pages");
    }
    void decode(int slot, const float* h_q, float* h_out) override {
        pd_legacy::HalfBuffer q(h_q, d_), out(static_cast<size_t>(d_));
        cache_->plan({slot}, 1);
        cache_->run(q.get(), out.get());
        CUDA_CHECK(cudaDeviceSynchronize());
        out.to_host(h_out);
    }
    int  actual_len(int slot) const override { return cache_->seq_len(slot); }
    bool is_occupied(int slot) const override { return cache_->occupied(slot); }
    int  free_page_count() const { return cache_->free_pages(); }

private:
    int d_;
    std::unique_ptr<decode::PagedKVCache> cache_;
};

class PagedDecodeAttention : public AttentionBackend {
public:
    void run(const float* q, const float* K, const float* V, float* out, int T, int d) override {
        const int pages = (T + PagedDecodePool::kPageSize - 1) / PagedDecodePool::kPageSize;
        PagedDecodePool pool(std::max(pages, 1), 1, std::max(pages, 1), d);
        const int slot = pool.admit(K, V, T);
        if (slot < 0) throw std::runtime_error("PagedDecodeAttention: pool setup failed");
        pool.decode(slot, q, out);
    }
    const char* name() const override { return "paged_decode_b200"; }
};
