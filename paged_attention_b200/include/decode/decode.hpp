#pragma once
// The reference's decode:: host interface (src/decode/decode.hpp) as a header-only forwarder
// into libpd_b200.so.  Same names, arguments, defaults and exceptions.

#include "decode_types.hpp"

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace decode {

// Status of a C-ABI call -> the exception the reference throws for the same mistake
// (std::invalid_argument, std::length_error); CUDA failures, on which the reference aborts
// the process, become std::runtime_error.
inline void check(int rc) {
    switch (rc) {
        case PD_OK: return;
        case PD_INVALID_ARGUMENT: throw std::invalid_argument(pd_last_error());
        case PD_LENGTH_ERROR: throw std::length_error(pd_last_error());
        default: throw std::runtime_error(std::string("pd_b200: ") + pd_last_error());
    }
}

// One decode step's schedule (src/decode/decode.hpp:21-27): CTA c runs segments
// [cta_seg_begin[c], cta_seg_begin[c+1]); item_seg_begin indexes the segments of each (row, kv head).
struct DecodePlan {
    int num_ctas = 0;
    int tile     = 0;
    std::vector<int4> segments;
    std::vector<int>  cta_seg_begin;
    std::vector<int>  item_seg_begin;
};

inline int tile_tokens(KVDtype dtype, int head_dim, int group) {
    int v = 0;
    check(pd_tile_tokens(static_cast<int>(dtype), head_dim, group, &v));
    return v;
}
inline int wave_ctas(KVDtype dtype, int head_dim, int group) {
    int v = 0;
    check(pd_wave_ctas(static_cast<int>(dtype), head_dim, group, &v));
    return v;
}
inline int default_ctas(KVDtype dtype, int head_dim, int group) {
    int v = 0;
    check(pd_default_ctas(static_cast<int>(dtype), head_dim, group, &v));
    return v;
}

namespace detail {
inline DecodePlan to_plan(const pd_plan* p) {
    DecodePlan out;
    out.num_ctas = pd_plan_num_ctas(p);
    out.tile     = pd_plan_tile(p);
    const int n  = pd_plan_num_segments(p);
    const int* s = pd_plan_segments(p);
    out.segments.resize(n);
    for (int i = 0; i < n; i++) out.segments[i] = make_int4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
    out.cta_seg_begin.assign(pd_plan_cta_seg_begin(p), pd_plan_cta_seg_begin(p) + out.num_ctas + 1);
    out.item_seg_begin.assign(pd_plan_item_seg_begin(p), pd_plan_item_seg_begin(p) + pd_plan_num_items(p) + 1);
    return out;
}
}  // namespace detail

inline DecodePlan make_plan(KVDtype dtype, const std::vector<int>& seq_lens, int num_q_heads,
                            int num_kv_heads, int head_dim, int num_ctas = 0) {
    pd_plan* p = nullptr;
    check(pd_make_plan(static_cast<int>(dtype), seq_lens.data(), static_cast<int>(seq_lens.size()), num_q_heads,
                       num_kv_heads, head_dim, num_ctas, &p));
    DecodePlan out = detail::to_plan(p);
    pd_plan_free(p);
    return out;
}

// Device copy of a plan plus the workspace for rows split across CTAs (src/decode/decode.hpp:44-62).
class DevicePlan {
public:
    DevicePlan() { check(pd_device_plan_create(&h_)); }
    ~DevicePlan() { pd_device_plan_destroy(h_); }
    DevicePlan(const DevicePlan&)            = delete;
    DevicePlan& operator=(const DevicePlan&) = delete;

    void upload(const DecodePlan& plan, int group, int head_dim, cudaStream_t stream = 0) {
        // the C ABI uploads from its own plan object: rebuild one that holds exactly this schedule
        pd_plan* p = nullptr;
        check(pd_plan_from_arrays(plan.num_ctas, plan.tile, reinterpret_cast<const int*>(plan.segments.data()),
                                  static_cast<int>(plan.segments.size()), plan.cta_seg_begin.data(),
                                  plan.item_seg_begin.data(), static_cast<int>(plan.item_seg_begin.size()) - 1, &p));
        const int rc = pd_device_plan_upload(h_, p, group, head_dim, stream);
        pd_plan_free(p);
        check(rc);
    }
    void bind(DecodeParams& p) const { check(pd_device_plan_bind(h_, as_pd(p))); }

    // Not in the reference: the same plan cut on the device from device-resident lengths (row b has
    // d_seq_lens[d_slot_ids ? d_slot_ids[b] : b]).  No host copy, no wait; allocation-free once the buffers
    // have grown to the largest batch, so it can be captured into a CUDA graph with the decode after it.
    void build(KVDtype dtype, const int* d_seq_lens, int batch, int num_q_heads, int num_kv_heads, int head_dim,
               int num_ctas = 0, const int* d_slot_ids = nullptr, cudaStream_t stream = 0) {
        check(pd_device_plan_build(h_, static_cast<int>(dtype), d_seq_lens, d_slot_ids, batch, num_q_heads, num_kv_heads,
                                   head_dim, num_ctas, stream));
    }

private:
    pd_device_plan* h_ = nullptr;
};

inline void paged_decode(KVDtype dtype, const DecodeParams& p, cudaStream_t stream = 0) {
    check(pd_paged_decode(static_cast<int>(dtype), as_pd(p), stream));
}

}  // namespace decode
