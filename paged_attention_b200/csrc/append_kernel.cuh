#pragma once
// Append-time scatter of new tokens into the paged pools, with the FP8 E4M3
// quantiser.  Stands in for append_kernel<KV> of the reference
// (src/decode/paged_kv_cache.cu:25-39) and produces the same bytes:
//   dst = ((page * num_kv_heads + h) * page_size + pos % page_size) * head_dim + d
//   fp16: copy;  fp8: e4m3(rn, satfinite)(float(x) * (1/scale)).
// One thread moves 8 consecutive head-dim elements of K and of V (16-byte loads,
// 16- or 8-byte stores) instead of one element.

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace pdk {

__device__ __forceinline__ uint32_t quant4_e4m3(uint32_t h01, uint32_t h23, float inv) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h01));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&h23));
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// One source of tokens: n tokens for one slot, starting at position start_pos.
struct AppendJob {
    const __half* k;          // [n][num_kv_heads][head_dim]
    const __half* v;
    const int*    table_row;  // the slot's block-table row (device)
    int           start_pos;
    int           n;
    int           first_unit; // prefix sum of units over jobs (batched launch)
};

// Optional per-kv-head quantisation scales (device arrays of num_kv_heads floats, or null: the per-tensor
// factors apply).  The stored byte is e4m3(x * (1 / scale[h])) with the reciprocal correctly rounded, the
// same arithmetic as the per-tensor path.  The reference has one scale per tensor only.
struct AppendHeadScales {
    const float* k;
    const float* v;
};

template<bool FP8>
__device__ __forceinline__ void append_unit(const AppendJob& job, int unit, void* k_cache, void* v_cache,
                                            int num_kv_heads, int page_size, float inv_k, float inv_v,
                                            const AppendHeadScales& hs = AppendHeadScales{nullptr, nullptr})
{
    constexpr int D = 128, VEC = 8, PER_ROW = D / VEC;   // 16 threads per (token, head) row
    const int c = unit % PER_ROW;
    const int h = (unit / PER_ROW) % num_kv_heads;
    const int i = unit / (PER_ROW * num_kv_heads);
    const int pos  = job.start_pos + i;
    const int page = __ldg(job.table_row + pos / page_size);
    const size_t dst = ((static_cast<size_t>(page) * num_kv_heads + h) * page_size + pos % page_size) * D + c * VEC;
    const size_t src = (static_cast<size_t>(i) * num_kv_heads + h) * D + c * VEC;
    const uint4 kx = *reinterpret_cast<const uint4*>(job.k + src);
    const uint4 vx = *reinterpret_cast<const uint4*>(job.v + src);
    if constexpr (FP8) {
        if (hs.k) inv_k = __frcp_rn(__ldg(hs.k + h));
        if (hs.v) inv_v = __frcp_rn(__ldg(hs.v + h));
        uint2 kq, vq;
        kq.x = quant4_e4m3(kx.x, kx.y, inv_k); kq.y = quant4_e4m3(kx.z, kx.w, inv_k);
        vq.x = quant4_e4m3(vx.x, vx.y, inv_v); vq.y = quant4_e4m3(vx.z, vx.w, inv_v);
        *reinterpret_cast<uint2*>(static_cast<unsigned char*>(k_cache) + dst) = kq;
        *reinterpret_cast<uint2*>(static_cast<unsigned char*>(v_cache) + dst) = vq;
    } else {
        *reinterpret_cast<uint4*>(static_cast<__half*>(k_cache) + dst) = kx;
        *reinterpret_cast<uint4*>(static_cast<__half*>(v_cache) + dst) = vx;
    }
}

template<bool FP8>
__global__ void __launch_bounds__(256)
append_kernel(AppendJob job, void* k_cache, void* v_cache, int num_kv_heads, int page_size,
              float inv_k, float inv_v, AppendHeadScales hs)
{
    const int units = job.n * num_kv_heads * 16;
    for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < units; u += gridDim.x * blockDim.x)
        append_unit<FP8>(job, u, k_cache, v_cache, num_kv_heads, page_size, inv_k, inv_v, hs);
}

// Many slots in one launch: jobs[] lives in device memory, first_unit is the
// running sum of units; each thread finds its job by binary search.
template<bool FP8>
__global__ void __launch_bounds__(256)
append_batch_kernel(const AppendJob* __restrict__ jobs, int num_jobs, int total_units, void* k_cache,
                    void* v_cache, int num_kv_heads, int page_size, float inv_k, float inv_v, AppendHeadScales hs)
{
    for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < total_units; u += gridDim.x * blockDim.x) {
        int lo = 0, hi = num_jobs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (jobs[mid].first_unit <= u) lo = mid; else hi = mid - 1;
        }
        const AppendJob job = jobs[lo];
        append_unit<FP8>(job, u - job.first_unit, k_cache, v_cache, num_kv_heads, page_size, inv_k, inv_v, hs);
    }
}

// Applies a step's block-table and length updates: (slot, index, page) triples, then (slot, length) pairs.
__global__ void __launch_bounds__(256)
apply_updates_kernel(const int* __restrict__ table_updates, int num_table, const int* __restrict__ len_updates,
                     int num_len, int* block_table, int table_stride, int* seq_lens)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < num_table) {
        const int slot = table_updates[3 * i], index = table_updates[3 * i + 1], page = table_updates[3 * i + 2];
        block_table[static_cast<size_t>(slot) * table_stride + index] = page;
    } else if (i < num_table + num_len) {
        const int j = i - num_table;
        seq_lens[len_updates[2 * j]] = len_updates[2 * j + 1];
    }
}

}  // namespace pdk
