#pragma once
// Read-only streaming probe: the attainable HBM read rate that the decode kernel is
// compared with.  Same role as read_kernel of the reference's benchmark
// (bench/bench_decode.cu:69-78, "copy" mode :224-240): 16 bytes per thread per step,
// XOR-folded so the loads stay live.

#include <cstdint>
#include <cuda_runtime.h>

namespace pdk {

__global__ void __launch_bounds__(512)
stream_read_kernel(const uint4* __restrict__ x, size_t n, unsigned* sink)
{
    uint32_t acc = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * stride < n; i += 4 * stride) {
        const uint4 a = __ldcs(x + i), b = __ldcs(x + i + stride), c = __ldcs(x + i + 2 * stride), d = __ldcs(x + i + 3 * stride);
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < n; i += stride) {
        const uint4 a = __ldcs(x + i);
        acc ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x12345678u) *sink = acc;
}

// Diagnostic access patterns for the same read: every block streams its OWN contiguous
// slice of the buffer (pattern 1), or visits the 4 KB chunks of its slice in a scrambled
// order (pattern 2, what scattered 16-token fp16 pages look like to DRAM), 2 KB chunks (3).
__global__ void __launch_bounds__(512)
stream_read_pattern_kernel(const uint4* __restrict__ x, size_t n, int pattern, unsigned* sink)
{
    uint32_t acc = 0;
    if (pattern >= 100) {
        // teams of T = pattern - 100 consecutive blocks share one contiguous slice and take its
        // 32 KB chunks round-robin: fewer, denser streams than one slice per block
        const int T = pattern - 100;
        const size_t teams = gridDim.x / T, team = blockIdx.x / T, member = blockIdx.x % T;
        const size_t per_team = n / teams;
        const uint4* tbase = x + per_team * team;
        constexpr size_t CH = 2048;                      // uint4 per 32 KB chunk = 512 threads x 4 loads
        for (size_t c = member; (c + 1) * CH <= per_team; c += T) {
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; k++) v[k] = __ldcs(tbase + c * CH + k * 512 + threadIdx.x);
#pragma unroll
            for (int k = 0; k < 4; k++) acc ^= v[k].x ^ v[k].y ^ v[k].z ^ v[k].w;
        }
        if (acc == 0x12345678u) *sink = acc;
        return;
    }
    const size_t per_block = n / gridDim.x;              // uint4 per block
    const uint4* base = x + per_block * blockIdx.x;
    const int chunk = pattern == 3 ? 128 : 256;          // uint4 per chunk: 2 KB or 4 KB
    const size_t nchunks = per_block / chunk;            // scrambled with an odd multiplier when a power of two
    const int per_iter = 512 * 4 / chunk;                // chunks covered per iteration by the block (4 loads/thread)
    for (size_t c0 = 0; c0 + per_iter <= nchunks; c0 += per_iter) {
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const size_t lin = c0 * chunk + k * 512 + threadIdx.x;   // position inside this iteration's window
            size_t ci = lin / chunk;
            const size_t off = lin % chunk;
            if (pattern >= 2) ci = (ci * 2654435761ull + 12345) % nchunks;
            v[k] = __ldcs(base + ci * chunk + off);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) acc ^= v[k].x ^ v[k].y ^ v[k].z ^ v[k].w;
    }
    if (acc == 0x12345678u) *sink = acc;
}

}  // namespace pdk
