#pragma once
// decode::PagedKVCache (src/decode/paged_kv_cache.hpp:17-93) as a handle on the library's cache
// object.  Pool, free list, block table, append + FP8 quantiser and the plan/run driver all live
// behind pd_cache_*; this class only keeps the reference's member names and error behaviour.

#include "decode.hpp"

#include <cstddef>
#include <vector>

namespace decode {

class PagedKVCache {
public:
    struct Config {
        int     num_pages;
        int     page_size;
        int     num_kv_heads;
        int     head_dim;
        int     max_slots;
        int     max_pages_per_slot;
        KVDtype dtype   = KVDtype::FP16;
        float   k_scale = 1.0f;   // stored = value / scale (FP8 only)
        float   v_scale = 1.0f;
    };

    explicit PagedKVCache(const Config& cfg) : cfg_(cfg) {
        const pd_cache_config c = to_c(cfg);
        check(pd_cache_create(&c, &h_));
    }
    ~PagedKVCache() { pd_cache_destroy(h_); }
    PagedKVCache(const PagedKVCache&)            = delete;
    PagedKVCache& operator=(const PagedKVCache&) = delete;

    static size_t bytes_per_page(const Config& cfg) { const pd_cache_config c = to_c(cfg); return pd_cache_bytes_per_page(&c); }
    static int pages_for_budget(const Config& cfg, size_t budget_bytes) {
        const pd_cache_config c = to_c(cfg);
        return pd_cache_pages_for_budget(&c, budget_bytes);
    }

    int admit() { return pd_cache_admit(h_); }
    bool append(int slot, const half* d_k, const half* d_v, int n, cudaStream_t stream = 0) {
        const int rc = pd_cache_append(h_, slot, d_k, d_v, n, stream);
        if (rc == PD_OUT_OF_PAGES) return false;
        check(rc);
        return true;
    }
    void release(int slot) { check(pd_cache_release(h_, slot)); }
    // Not in the reference: one fp8 scale per kv head (num_kv_heads positive floats each) instead of the
    // per-tensor scales of the config; only while the cache holds no tokens.
    void set_head_scales(const std::vector<float>& k_scales, const std::vector<float>& v_scales) {
        if (k_scales.size() != v_scales.size()) throw std::invalid_argument("set_head_scales: sizes differ");
        check(pd_cache_set_head_scales(h_, k_scales.empty() ? nullptr : k_scales.data(),
                                       v_scales.empty() ? nullptr : v_scales.data()));
    }
    void shuffle_free_pages(unsigned seed) { pd_cache_shuffle_free_pages(h_, seed); }

    void plan(const std::vector<int>& slots, int num_q_heads, int num_ctas = 0, cudaStream_t stream = 0) {
        check(pd_cache_plan(h_, slots.data(), static_cast<int>(slots.size()), num_q_heads, num_ctas, stream));
        plan_ = detail::to_plan(pd_cache_last_plan(h_));
    }
    // Not in the reference: plan() cut on the device from the cache's device-side lengths (slots
    // 0..batch-1, or the device array d_slot_ids).  last_plan() is empty afterwards.
    void plan_device(int batch, int num_q_heads, int num_ctas = 0, const int* d_slot_ids = nullptr, cudaStream_t stream = 0) {
        check(pd_cache_plan_device(h_, d_slot_ids, batch, num_q_heads, num_ctas, stream));
        plan_ = DecodePlan{};
    }
    void run(const half* d_q, half* d_out, cudaStream_t stream = 0) { check(pd_cache_run(h_, d_q, d_out, stream)); }
    void decode(const half* d_q, half* d_out, int batch, int num_q_heads, int num_ctas = 0, cudaStream_t stream = 0) {
        check(pd_cache_decode(h_, d_q, d_out, batch, num_q_heads, num_ctas, stream));
        plan_ = detail::to_plan(pd_cache_last_plan(h_));
    }
    const DecodePlan& last_plan() const { return plan_; }

    DecodeParams params() const {
        DecodeParams p{};
        check(pd_cache_params(h_, as_pd(p)));
        return p;
    }

    int    seq_len(int slot)  const { return pd_cache_seq_len(h_, slot); }
    bool   occupied(int slot) const { return pd_cache_occupied(h_, slot) != 0; }
    int    free_pages()       const { return pd_cache_free_pages(h_); }
    int    max_seq_len()      const { return pd_cache_max_seq_len(h_); }
    size_t total_bytes()      const { return pd_cache_total_bytes(h_); }
    const Config& config()    const { return cfg_; }
    std::vector<int> block_table(int slot) const {
        std::vector<int> t(cfg_.max_pages_per_slot);
        t.resize(pd_cache_block_table(h_, slot, t.data(), static_cast<int>(t.size())));
        return t;
    }

private:
    static pd_cache_config to_c(const Config& c) {
        return pd_cache_config{c.num_pages, c.page_size, c.num_kv_heads, c.head_dim, c.max_slots,
                               c.max_pages_per_slot, static_cast<int>(c.dtype), c.k_scale, c.v_scale};
    }
    Config     cfg_;
    pd_cache*  h_ = nullptr;
    DecodePlan plan_;
};

}  // namespace decode
