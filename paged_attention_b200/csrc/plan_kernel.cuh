// Device-side planner: the cut of decode::make_plan (src/decode/decode.cu:65-108 of the reference)
// computed on the GPU from the sequence lengths that already live there, so that a decode step needs
// no host knowledge of the lengths, no host-to-device copy of a plan, and can sit inside a CUDA graph.
// The reference always plans on the host; the arrays this kernel writes are bit-identical to what the
// host planner produces for the same lengths, tile and grid.
//
// The flat list of (row, kv head, tile) work units is cut into runs of `per = ceil(total / grid)`
// units; CTA c owns units [c * per, (c + 1) * per).  Item i = (row, kv head) owns units
// [P_i, P_i + tiles_i), so it is cut at every multiple of `per` strictly inside that range, and the
// piece that starts at c * per is the first segment of CTA c.  Two block-wide prefix sums (tiles per
// row, pieces per item) are all the communication the cut needs; one CTA of 1024 threads does it.
//
// With cumulative shares from the host's adaptive cut (PlanJob::shares, active once the host has seen
// usable rates) the cut points become B_c = round(total * share_c) instead of c * per: the cut of the host's
// weighted planner, bit for bit.  Only for grids up to PLAN_MAX_WEIGHTED CTAs and at least 8 units per CTA,
// so that no CTA's share is empty; otherwise the equal cut stands.
#pragma once

#include <cuda_runtime.h>

namespace pdk {

constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_WEIGHTED = 1024;

// Slots of the `info` array the planner leaves behind for the host (diagnostics, tests).
constexpr int PLAN_INFO_CTAS     = 0;   // CTAs that received work (the rest of the grid idles)
constexpr int PLAN_INFO_SEGMENTS = 1;
constexpr int PLAN_INFO_WIDEST   = 2;   // most pieces any (row, kv head) was cut in
constexpr int PLAN_INFO_BAD_ROW  = 3;   // 1 + first row whose length was <= 0 (0: none); such rows get no work
constexpr int PLAN_INFO_INTS     = 4;

struct PlanJob {
    const int* seq_lens;       // [slots], device
    const int* slot_ids;       // [batch] or null = identity
    int batch, num_kv_heads, tile, grid;
    int lse_per_segment;       // LSE slots per segment: the GQA group, or all query heads for head-fused row plans
    int num_counters;          // arrival counters to clear: one per (row, kv head) of the layer
    int4* segments;            // capacity batch * num_kv_heads + grid
    int*  cta_seg_begin;       // [grid + 1]
    int*  item_seg_begin;      // [batch * num_kv_heads + 1]
    int*  row_tile_begin;      // [batch + 1] scratch: tiles of one kv head before each row
    int*  info;                // [PLAN_INFO_INTS]
    float* partial_lse;        // the arrival counters of the in-kernel merge follow segments * group LSEs
    const double* shares;      // null, or [0] = active flag, [1 + c] = cumulative share before CTA c, c = 0..grid
};

// Exclusive prefix sum of value(0..n-1) into out[0..n] (out[n] = total), all threads of the block.
template<typename F>
__device__ int block_exclusive_scan(int n, F value, int* out, int* warp_sums, int* carry)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) *carry = 0;
    __syncthreads();
    for (int base = 0; base < n; base += PLAN_THREADS) {
        const int i = base + tid;
        const int v = i < n ? value(i) : 0;
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (lane == 31) warp_sums[warp] = x;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += y;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int before = *carry + (warp ? warp_sums[warp - 1] : 0);
        if (i < n) out[i] = before + x - v;
        __syncthreads();
        if (tid == PLAN_THREADS - 1) *carry = before + x;
        __syncthreads();
    }
    if (tid == 0) out[n] = *carry;
    __syncthreads();
    return *carry;
}

__global__ void __launch_bounds__(PLAN_THREADS)
plan_kernel(const PlanJob j)
{
    __shared__ int warp_sums[32];
    __shared__ int carry;
    __shared__ int widest, bad_row;
    __shared__ int bound[PLAN_MAX_WEIGHTED + 1];   // weighted cut: first unit of every CTA
    const int tid = threadIdx.x;
    if (tid == 0) { widest = 0; bad_row = 0; }
    __syncthreads();

    auto row_len = [&](int b) { return j.seq_lens[j.slot_ids ? j.slot_ids[b] : b]; };
    auto row_tiles = [&](int b) {
        const int len = row_len(b);
        if (len <= 0) { atomicCAS(&bad_row, 0, b + 1); return 0; }
        return (len + j.tile - 1) / j.tile;
    };
    const int row_total = block_exclusive_scan(j.batch, row_tiles, j.row_tile_begin, warp_sums, &carry);
    const long long total = static_cast<long long>(row_total) * j.num_kv_heads;
    const int items = j.batch * j.num_kv_heads;
    const long long per = total > 0 ? (total + j.grid - 1) / j.grid : 1;
    const bool weighted = j.shares != nullptr && j.grid <= PLAN_MAX_WEIGHTED && total >= 8LL * j.grid &&
                          total < (1LL << 31) && j.shares[0] != 0.0;
    const int ctas = total > 0 ? (weighted ? j.grid : static_cast<int>((total + per - 1) / per)) : 0;
    if (weighted) {
        for (int c = tid; c <= j.grid; c += PLAN_THREADS) {
            long long b = llround(static_cast<double>(total) * j.shares[1 + c]);
            if (b > total) b = total;
            bound[c] = static_cast<int>(c == j.grid ? total : b);
        }
        __syncthreads();
    }
    // weighted cut: the CTA that owns unit t, i.e. the largest c with bound[c] <= t
    auto cta_of = [&](long long t) {
        int lo = 0, hi = j.grid - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (bound[mid] <= t) lo = mid; else hi = mid - 1;
        }
        return lo;
    };

    // units before item i, and its own
    auto item_begin = [&](int i) {
        const int b = i / j.num_kv_heads, h = i % j.num_kv_heads;
        const int t = j.row_tile_begin[b + 1] - j.row_tile_begin[b];
        return static_cast<long long>(j.row_tile_begin[b]) * j.num_kv_heads + static_cast<long long>(h) * t;
    };
    auto item_pieces = [&](int i) {
        const int b = i / j.num_kv_heads;
        const int t = j.row_tile_begin[b + 1] - j.row_tile_begin[b];
        if (t == 0) return 0;
        const long long p0 = item_begin(i);
        const int n = weighted ? cta_of(p0 + t - 1) - cta_of(p0) + 1
                               : static_cast<int>((p0 + t - 1) / per - p0 / per) + 1;
        atomicMax(&widest, n);
        return n;
    };
    const int nseg = block_exclusive_scan(items, item_pieces, j.item_seg_begin, warp_sums, &carry);

    for (int i = tid; i < items; i += PLAN_THREADS) {
        const int b = i / j.num_kv_heads, h = i % j.num_kv_heads;
        const int t = j.row_tile_begin[b + 1] - j.row_tile_begin[b];
        if (t == 0) continue;
        const int len = row_len(b);
        const long long p0 = item_begin(i), p1 = p0 + t;
        int idx = j.item_seg_begin[i];
        if (weighted) {
            for (int c = cta_of(p0); c < j.grid && bound[c] < p1; c++, idx++) {
                const long long from = bound[c] > p0 ? bound[c] : p0;
                const long long to   = bound[c + 1] < p1 ? bound[c + 1] : p1;
                const int tok_end = static_cast<int>(to - p0) * j.tile;
                j.segments[idx] = make_int4(b, h, static_cast<int>(from - p0) * j.tile, tok_end < len ? tok_end : len);
                if (from == bound[c]) j.cta_seg_begin[c] = idx;
            }
            continue;
        }
        for (long long c = p0 / per; c * per < p1; c++, idx++) {
            const long long from = c * per > p0 ? c * per : p0;
            const long long to   = (c + 1) * per < p1 ? (c + 1) * per : p1;
            const int tok_end = static_cast<int>(to - p0) * j.tile;
            j.segments[idx] = make_int4(b, h, static_cast<int>(from - p0) * j.tile, tok_end < len ? tok_end : len);
            if (from == c * per) j.cta_seg_begin[c] = idx;
        }
    }
    for (int c = ctas + tid; c <= j.grid; c += PLAN_THREADS) j.cta_seg_begin[c] = nseg;   // idle CTAs: empty ranges
    int* counters = reinterpret_cast<int*>(j.partial_lse + static_cast<size_t>(nseg) * j.lse_per_segment);
    for (int i = tid; i < j.num_counters; i += PLAN_THREADS) counters[i] = 0;
    __syncthreads();
    if (tid == 0) {
        j.info[PLAN_INFO_CTAS] = ctas;
        j.info[PLAN_INFO_SEGMENTS] = nseg;
        j.info[PLAN_INFO_WIDEST] = widest;
        j.info[PLAN_INFO_BAD_ROW] = bad_row;
    }
}

}  // namespace pdk
