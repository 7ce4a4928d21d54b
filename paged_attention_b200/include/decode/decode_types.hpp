#pragma once
// decode::KVDtype and decode::DecodeParams with the reference's names and field order
// (src/decode/decode_types.hpp:8-45), defined on top of the C ABI's pd_params so that a
// DecodeParams can be handed to libpd_b200.so unchanged.

#include "pd_b200.h"

#include <cuda_fp16.h>
#include <vector_types.h>

#include <cstddef>
#include <type_traits>

namespace decode {

enum class KVDtype { FP16 = PD_FP16, FP8_E4M3 = PD_FP8_E4M3 };

inline int kv_dtype_bytes(KVDtype t) { return pd_kv_dtype_bytes(static_cast<int>(t)); }
inline const char* kv_dtype_name(KVDtype t) { return pd_kv_dtype_name(static_cast<int>(t)); }

// Non-owning view of everything one decode launch reads; all pointers are device pointers.
// Typed twin of pd_params: same offsets, so reinterpret_cast between the two is the contract.
struct DecodeParams {
    const half* q;                 // [batch][num_q_heads][head_dim]
    half*       out;               // [batch][num_q_heads][head_dim]
    const void* k_cache;           // [num_pages][num_kv_heads][page_size][head_dim], fp16 or e4m3 bytes
    const void* v_cache;
    const int*  block_table;       // [num_slots][block_table_stride]
    const int*  seq_lens;          // [num_slots]
    const int*  slot_ids;          // [batch] or nullptr (row i reads slot i)
    int         block_table_stride;
    int         batch;
    int         num_q_heads;
    int         num_kv_heads;
    int         head_dim;
    int         page_size;
    float       sm_scale;
    float       k_scale;
    float       v_scale;
    const int4* segments;          // (row, kv head, token begin, token end)
    const int*  cta_seg_begin;     // [num_ctas + 1]
    const int*  item_seg_begin;    // [batch * num_kv_heads + 1]
    int         num_ctas;
    int         needs_merge;
    float*      partial_out;       // [num_segments][group][head_dim]
    float*      partial_lse;       // [num_segments][group]
};

static_assert(std::is_standard_layout<DecodeParams>::value, "DecodeParams crosses a C ABI");
static_assert(sizeof(DecodeParams) == sizeof(pd_params), "DecodeParams must mirror pd_params");
static_assert(offsetof(DecodeParams, segments) == offsetof(pd_params, segments) &&
              offsetof(DecodeParams, partial_lse) == offsetof(pd_params, partial_lse) &&
              offsetof(DecodeParams, sm_scale) == offsetof(pd_params, sm_scale),
              "DecodeParams must mirror pd_params");

inline const pd_params* as_pd(const DecodeParams& p) { return reinterpret_cast<const pd_params*>(&p); }
inline pd_params* as_pd(DecodeParams& p) { return reinterpret_cast<pd_params*>(&p); }

}  // namespace decode
