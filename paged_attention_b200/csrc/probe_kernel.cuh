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

}  // namespace pdk
