// libpd_b200.so: host side of the engine and its C ABI (include/pd_b200.h).
//
// Host logic here is new code written against the reference's observable
// behaviour (src/decode/decode.cu, src/decode/paged_kv_cache.cu): same plan for
// the same (tile, num_ctas), same allocator decisions, same cache bytes.

#include "pd_b200.h"

#include "append_kernel.cuh"
#include "decode_kernel.cuh"
#include "plan_kernel.cuh"
#include "probe_kernel.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <numeric>
#include <random>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

// ---- errors -----------------------------------------------------------------------

thread_local std::string g_last_error;

int set_error(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define PD_CUDA(expr)                                                                      \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess)                                                             \
            return set_error(PD_CUDA_ERROR, "CUDA error %s at %s:%d: %s", cudaGetErrorName(e_), \
                             __FILE__, __LINE__, cudaGetErrorString(e_));                  \
    } while (0)

// ---- kernel shapes --------------------------------------------------------------------
// CTA shape and pipeline depth per cache dtype: Config<consumer warps, 16-token groups per warp per tile,
// stages, CTAs per SM>, plus one producer warp per CTA.  fp16: 4 warps, 64-token tiles, 3 stages of 32 KB, two
// CTAs per SM.  e4m3: 4 warps of two groups (a warp's unit is 32 tokens), 128-token tiles, 3 stages of 32 KB,
// two CTAs per SM.  The two macros let a tuning build try other shapes (python -m paged_attention_b200.build
// takes extra compiler flags from the environment variable PD_B200_NVCC_FLAGS).
#ifndef PD_B200_FP16_SHAPE
#define PD_B200_FP16_SHAPE 4132
#endif
#ifndef PD_B200_FP8_SHAPE
#define PD_B200_FP8_SHAPE 4232
#endif
// a shape is written as four decimal digits: warps, groups per warp, stages, CTAs per SM
template<int DIGITS> using ShapeOf = pdk::Config<DIGITS / 1000, DIGITS / 100 % 10, DIGITS / 10 % 10, DIGITS % 10>;
template<typename KV> struct DefaultConfig;
template<> struct DefaultConfig<__half>        { using type = ShapeOf<PD_B200_FP16_SHAPE>; };
template<> struct DefaultConfig<__nv_fp8_e4m3> { using type = ShapeOf<PD_B200_FP8_SHAPE>; };

struct KernelInfo {
    const void* fn;
    int tile, threads, smem, per_sm, stages;
    void (*launch)(const pd_params&, const CUtensorMap&, const CUtensorMap&, int, int, int, unsigned*, const pdk::GatherOut&,
                   const pdk::HeadScales&, const pdk::CtaStats&, cudaStream_t);
    void (*merge)(const pd_params&, int, cudaStream_t);
};

template<typename KV, int GROUP, typename C>
void launch_decode(const pd_params& p, const CUtensorMap& km, const CUtensorMap& vm, int btl, int row_gather, int seg_limit,
                   unsigned* status, const pdk::GatherOut& gather, const pdk::HeadScales& scales, const pdk::CtaStats& stats,
                   cudaStream_t stream) {
    using S = pdk::Shape<KV, GROUP, C>;
    pdk::paged_decode_kernel<KV, GROUP, C><<<p.num_ctas, S::THREADS, S::SMEM_BYTES, stream>>>(p, km, vm, btl, row_gather, seg_limit, status, gather, scales, stats);
}
// The merge kernel is launched as a programmatic dependent of the decode kernel before it: its CTAs are
// placed while the decode grid drains and wait inside the kernel (griddepcontrol.wait) until that grid is
// complete, which takes the launch latency out of the gap between the two kernels.
constexpr int MERGE_GRID_CAP = 148 * 8;
template<typename Kernel>
void launch_dependent(Kernel kernel, int blocks, const pd_params& p, int seg_limit, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, p, seg_limit);
}
template<int GROUP>
void launch_merge(const pd_params& p, int seg_limit, cudaStream_t stream) {
    const int pairs = p.batch * p.num_q_heads;
    if (pairs > MERGE_GRID_CAP) launch_dependent(pdk::merge_segments_kernel<GROUP, false, true>, MERGE_GRID_CAP, p, seg_limit, stream);
    else                        launch_dependent(pdk::merge_segments_kernel<GROUP, false, false>, pairs, p, seg_limit, stream);
}

template<typename KV, int GROUP>
KernelInfo make_info() {
    using C = typename DefaultConfig<KV>::type;
    using S = pdk::Shape<KV, GROUP, C>;
    return KernelInfo{reinterpret_cast<const void*>(&pdk::paged_decode_kernel<KV, GROUP, C>), S::TILE, S::THREADS,
                      S::SMEM_BYTES, C::MIN_CTAS, C::STAGES, &launch_decode<KV, GROUP, C>, &launch_merge<GROUP>};
}

template<typename KV>
const KernelInfo* info_by_group(int group) {
    static const KernelInfo t[4] = {make_info<KV, 1>(), make_info<KV, 2>(), make_info<KV, 4>(), make_info<KV, 8>()};
    switch (group) {
        case 1: return &t[0];
        case 2: return &t[1];
        case 4: return &t[2];
        case 8: return &t[3];
    }
    return nullptr;
}

// Head-fused tiles (all 8 kv heads of one token unit per tile, one consumer warp per kv head); used for
// plans made by pd_make_plan when the layer has exactly 8 kv heads, for both cache types: 3 stages of
// 64 KB, one CTA per SM.  Measured on the batch 64 x 8192 fp16 layer: 314 us against 320 us for the
// (row, kv head) schedule, and 0.9 % instead of 2.6 % over one contiguous page per sequence; on the
// same layer with the e4m3 cache 164.8 us against 168.7 us.
template<typename KV> struct FusedConfig;
template<> struct FusedConfig<__half> { using type = pdk::Config<8, 1, 3, 1, 8>; };
// e4m3: a warp's unit is 32 tokens, so a tile is 32 tokens of all 8 kv heads: two 16 KB boxes per pool and tile
// with 16-token pages, the same 64 KB per stage as the fp16 shape.
template<> struct FusedConfig<__nv_fp8_e4m3> { using type = pdk::Config<8, 2, 3, 1, 8>; };

template<int GROUP>
void launch_merge_rows(const pd_params& p, int seg_limit, cudaStream_t stream) {
    const int pairs = p.batch * p.num_q_heads;
    if (pairs > MERGE_GRID_CAP) launch_dependent(pdk::merge_segments_kernel<GROUP, true, true>, MERGE_GRID_CAP, p, seg_limit, stream);
    else                        launch_dependent(pdk::merge_segments_kernel<GROUP, true, false>, pairs, p, seg_limit, stream);
}

template<typename KV, int GROUP>
KernelInfo make_fused_info() {
    using C = typename FusedConfig<KV>::type;
    using S = pdk::Shape<KV, GROUP, C>;
    return KernelInfo{reinterpret_cast<const void*>(&pdk::paged_decode_kernel<KV, GROUP, C>), S::TILE, S::THREADS,
                      S::SMEM_BYTES, C::MIN_CTAS, C::STAGES, &launch_decode<KV, GROUP, C>, &launch_merge_rows<GROUP>};
}

template<typename KV>
const KernelInfo* fused_info_of(int group) {
    static const KernelInfo t[4] = {make_fused_info<KV, 1>(), make_fused_info<KV, 2>(), make_fused_info<KV, 4>(),
                                    make_fused_info<KV, 8>()};
    switch (group) {
        case 1: return &t[0];
        case 2: return &t[1];
        case 4: return &t[2];
        case 8: return &t[3];
    }
    return nullptr;
}
// The head-fused kernel of a cache dtype (its tile is 16 tokens for fp16, 32 for e4m3); null for other dtypes.
const KernelInfo* fused_info(int dtype, int group) {
    if (dtype == PD_FP16) return fused_info_of<__half>(group);
    if (dtype == PD_FP8_E4M3) return fused_info_of<__nv_fp8_e4m3>(group);
    return nullptr;
}
constexpr int FUSED_HEADS = 8;
int g_head_fused = std::getenv("PD_B200_NO_HEAD_FUSED") == nullptr ? 1 : 0;   // 0 never, 1 where it wins, 2 always

}  // namespace
#include "adaptive_cut.hpp"
namespace {

// Same argument checks, in the same order, as the reference's dispatch
// (src/decode/decode.cu:18-39): head_dim first, then the group size.
int find_kernel(int dtype, int head_dim, int group, const KernelInfo** out) {
    if (dtype != PD_FP16 && dtype != PD_FP8_E4M3) return set_error(PD_INVALID_ARGUMENT, "unsupported KV dtype %d", dtype);
    if (head_dim != 128) return set_error(PD_INVALID_ARGUMENT, "unsupported head_dim %d", head_dim);
    const KernelInfo* k = dtype == PD_FP16 ? info_by_group<__half>(group) : info_by_group<__nv_fp8_e4m3>(group);
    if (!k) return set_error(PD_INVALID_ARGUMENT, "unsupported GQA group size %d", group);
    *out = k;
    return PD_OK;
}

// cudaFuncSetAttribute once per (kernel, device).
std::mutex g_cfg_mutex;
std::vector<std::pair<const void*, int>> g_configured;
int configure(const KernelInfo* k) {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_cfg_mutex);
    for (auto& c : g_configured) if (c.first == k->fn && c.second == dev) return PD_OK;
    PD_CUDA(cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k->smem));
    g_configured.emplace_back(k->fn, dev);
    return PD_OK;
}

// ---- per-device status word -----------------------------------------------------------

constexpr int MAX_DEVICES = 64;
unsigned* g_status[MAX_DEVICES] = {};
std::mutex g_status_mutex;
int status_word(unsigned** out) {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return set_error(PD_INTERNAL, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status[dev]) {
        PD_CUDA(cudaMalloc(&g_status[dev], sizeof(unsigned)));
        PD_CUDA(cudaMemset(g_status[dev], 0, sizeof(unsigned)));
    }
    *out = g_status[dev];
    return PD_OK;
}

// ---- TMA descriptors --------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;
int encode_fn(EncodeTiledFn* out) {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    });
    if (!g_encode) return set_error(PD_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    *out = g_encode;
    return PD_OK;
}

unsigned gcd_u(unsigned a, unsigned b) { while (b) { const unsigned t = a % b; a = b; b = t; } return a; }

// Tensor map over one pool [page][kv head][token][dim].
//   fp16: 5-D  (64 dims, token, panel, kv head, page), box (64, 2^btl, 2, 1, 1)
//   fp8 : 4-D  (128 dims, token, kv head, page),       box (128, 2^btl, 1, 1)
// so a box lands in shared memory as [panel][token][128 bytes] under the 128-byte swizzle.
//   row_gather (pages of fewer than 4 tokens): 2-D (row bytes, pool rows = page x kv head x token), box
//   (128 bytes, 1 row) for cp.async.bulk.tensor ... tile::gather4, which fetches four such rows per copy.
int make_tensor_map(CUtensorMap* map, int dtype, const void* pool, int num_pages, int num_kv_heads,
                    int page_size, int btl, int box_heads = 1, bool row_gather = false) {
    EncodeTiledFn enc;
    if (int rc = encode_fn(&enc)) return rc;
    if (reinterpret_cast<uintptr_t>(pool) % 16 != 0)
        return set_error(PD_INVALID_ARGUMENT, "KV pool pointer must be 16-byte aligned");
    const cuuint64_t pages = num_pages > 0 ? static_cast<cuuint64_t>(num_pages) : (1ull << 31);
    const cuuint64_t row = dtype == PD_FP16 ? 256 : 128;
    const CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    CUresult r;
    if (row_gather) {
        const cuuint64_t rows = std::min<cuuint64_t>(pages * num_kv_heads * page_size, 1ull << 31);
        const cuuint64_t dims[2]    = {128, rows};
        const cuuint64_t strides[1] = {row};
        const cuuint32_t box[2]     = {dtype == PD_FP16 ? 64u : 128u, 1};
        const cuuint32_t estr[2]    = {1, 1};
        r = enc(map, dtype == PD_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (dtype == PD_FP16) {
        const cuuint64_t dims[5]    = {64, static_cast<cuuint64_t>(page_size), 2, static_cast<cuuint64_t>(num_kv_heads), pages};
        const cuuint64_t strides[4] = {row, 128, row * page_size, row * page_size * num_kv_heads};
        const cuuint32_t box[5]     = {64, 1u << btl, 2, static_cast<cuuint32_t>(box_heads), 1};
        const cuuint32_t estr[5]    = {1, 1, 1, 1, 1};
        r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(pool), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[4]    = {128, static_cast<cuuint64_t>(page_size), static_cast<cuuint64_t>(num_kv_heads), pages};
        const cuuint64_t strides[3] = {row, row * page_size, row * page_size * num_kv_heads};
        const cuuint32_t box[4]     = {128, 1u << btl, static_cast<cuuint32_t>(box_heads), 1};
        const cuuint32_t estr[4]    = {1, 1, 1, 1};
        r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(pool), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return set_error(PD_CUDA_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return PD_OK;
}

}  // namespace
#include "host_plan.hpp"

// ---- DevicePlan ---------------------------------------------------------------------------------

struct pd_device_plan {
    int device = -1;
    void*  arena = nullptr;      // segments | cta_seg_begin | item_seg_begin, one allocation
    size_t arena_cap = 0;
    void*  staging = nullptr;    // pinned host mirror of the arena
    size_t staging_cap = 0;
    cudaEvent_t staged = nullptr;   // completion of the last upload out of `staging`
    float* partial = nullptr;
    size_t partial_cap = 0;      // floats
    // views into the arena
    const void* segments = nullptr;
    const int*  cta_seg_begin = nullptr;
    const int*  item_seg_begin = nullptr;
    float* partial_out = nullptr;
    float* partial_lse = nullptr;
    int    num_ctas = 0;
    int    needs_merge = 0;
    int    num_segments = 0;
    int    num_items = 0;
    // set by pd_device_plan_build (plan cut on the device): scratch and result slots inside the arena
    bool   built_on_device = false;
    int    tile = 0;
    int*   row_tile_begin = nullptr;
    int*   info = nullptr;
    struct Fused {                 // the same step cut into head-fused row segments (valid: exactly 8 kv heads)
        bool valid = false;
        int dtype = -1, group = 0, batch = 0, num_ctas = 0, num_segments = 0, needs_merge = 0;
        size_t rows = 0;           // segments * num_q_heads
        const void* segments = nullptr;
        const int* cta_seg_begin = nullptr;
        const int* row_seg_begin = nullptr;
        float* partial_out = nullptr;
        unsigned long long* stats = nullptr;   // per-CTA record of the launches of this schedule (adaptive cut)
    } fused,
      weighted;                    // the caller's (row, kv head) schedule cut in unequal shares (adaptive cut)
    unsigned long long* stats = nullptr;       // record of launches that run the caller's plan as it is
    // Per schedule region: the LSE array and the arrival counters of the in-kernel merge behind it (what
    // pd_device_plan_reset clears; the counters' exact start follows the plan's real segment count, which for
    // plans cut on the device only the device knows, so the whole tail of the region is cleared).
    struct Tail { void* ptr = nullptr; size_t bytes = 0; } tails[3];
};

namespace {
// Launch-time lookup: standard segment array (what pd_params carries) -> head-fused schedule.
std::mutex g_fused_mutex;
struct AltSchedules { pd_device_plan::Fused fused, weighted; unsigned long long* stats = nullptr; };
std::unordered_map<const void*, AltSchedules> g_fused_registry;
}  // namespace

// ---- cache -----------------------------------------------------------------------------------------

struct pd_cache {
    pd_cache_config cfg{};
    void* d_k = nullptr;
    void* d_v = nullptr;
    int*  d_block_table = nullptr;
    int*  d_seq_lens = nullptr;
    int*  d_slot_ids = nullptr;
    size_t slot_ids_cap = 0;
    pd_plan* plan = nullptr;
    pd_device_plan* device_plan = nullptr;
    int plan_batch = 0, plan_num_q_heads = 0;
    bool plan_identity = false;
    float* d_head_scales = nullptr;       // optional per-kv-head scales: k[num_kv_heads] then v[num_kv_heads]
    bool plan_on_device = false;          // the current plan was cut by pd_cache_plan_device
    const int* plan_slot_ids = nullptr;   // ... for these rows (device pointer of the caller, or null)
    std::vector<int> free_pages;
    std::vector<std::vector<int>> tables;
    std::vector<int> seq_lens;
    std::vector<char> occupied;
    // batched append: pinned staging + device copy of the step's job list, grow-only
    void*  batch_staging = nullptr;
    void*  batch_device = nullptr;
    size_t batch_cap = 0;
    cudaEvent_t batch_staged = nullptr;
    cudaEvent_t batch_done = nullptr;     // the last batched append's kernels (release waits for them)
    bool batch_pending = false;
};

extern "C" {

const char* pd_last_error(void) { return g_last_error.c_str(); }
const char* pd_version(void) { return "pd_b200 0.1 (sm_100a)"; }

int pd_kv_dtype_bytes(int dtype) { return dtype == PD_FP16 ? 2 : 1; }
const char* pd_kv_dtype_name(int dtype) { return dtype == PD_FP16 ? "fp16" : "fp8_e4m3"; }

int pd_set_head_fused(int mode) {
    if (mode < 0 || mode > 2) return set_error(PD_INVALID_ARGUMENT, "set_head_fused: mode must be 0, 1 or 2");
    g_head_fused = mode;
    return PD_OK;
}
int pd_head_fused(void) { return g_head_fused; }

int pd_set_adaptive_cut(int on) {
    g_adaptive = on != 0;
    return PD_OK;
}
int pd_adaptive_cut(void) { return g_adaptive ? 1 : 0; }
// Introspection: the i-th rate table (in no particular order): its grid, weights and latest record.
// Returns the grid size, 0 when there is no such table.
int pd_adaptive_cut_table(int index, float* weights, unsigned long long* record, int cap) {
    std::lock_guard<std::mutex> lock(g_rate_mutex);
    int i = 0;
    for (auto& kv : g_rates) {
        if (i++ != index) continue;
        const RateTable& t = kv.second;
        for (int c = 0; c < t.grid && c < cap; c++) {
            if (weights) weights[c] = t.weights.empty() ? 1.f : t.weights[c];
            if (record) { record[2 * c] = t.host[2 * c]; record[2 * c + 1] = t.host[2 * c + 1]; }
        }
        if (record && t.grid <= cap) record[2 * t.grid] = t.host[2 * t.grid];
        return t.grid;
    }
    return 0;
}
int pd_adaptive_cut_refresh(void* stream_) {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    std::vector<RateTable*> tables;
    {
        std::lock_guard<std::mutex> lock(g_rate_mutex);
        for (auto& kv : g_rates)
            if (kv.first.device == dev) tables.push_back(&kv.second);
    }
    if (g_adaptive)
        for (RateTable* t : tables) update_weights(t, static_cast<cudaStream_t>(stream_));
    return PD_OK;
}
int pd_adaptive_cut_reset(void) {
    std::lock_guard<std::mutex> lock(g_rate_mutex);
    for (auto& kv : g_rates) {
        kv.second.weights.clear();
        kv.second.updates = 0;
        if (kv.second.shares) cudaMemset(kv.second.shares, 0, sizeof(double));   // device plans go back to equal shares
        if (kv.second.copy_queued) cudaEventSynchronize(kv.second.copied);
        kv.second.copy_queued = false;
        kv.second.resync = true;   // launches issued since the last copy are not in `host` yet: the next copy only re-bases
        if (kv.second.host) kv.second.seen.assign(kv.second.host, kv.second.host + 2 * static_cast<size_t>(kv.second.grid) + 1);
    }
    return PD_OK;
}

int pd_tile_tokens(int dtype, int head_dim, int group, int* out) {
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, head_dim, group, &k)) return rc;
    *out = k->tile;
    return PD_OK;
}

int pd_wave_ctas(int dtype, int head_dim, int group, int* out) {
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, head_dim, group, &k)) return rc;
    if (int rc = configure(k)) return rc;
    int dev = 0, sms = 0, resident = 0;
    PD_CUDA(cudaGetDevice(&dev));
    PD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    PD_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, k->fn, k->threads, k->smem));
    *out = sms * resident;
    return PD_OK;
}

// One wave at the residency the kernel was shaped for (never more than fits).
int pd_default_ctas(int dtype, int head_dim, int group, int* out) {
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, head_dim, group, &k)) return rc;
    int wave = 0;
    if (int rc = pd_wave_ctas(dtype, head_dim, group, &wave)) return rc;
    int dev = 0, sms = 0;
    PD_CUDA(cudaGetDevice(&dev));
    PD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    *out = std::min(wave, sms * k->per_sm);
    if (*out <= 0) return set_error(PD_CUDA_ERROR, "decode kernel does not fit on this device");
    return PD_OK;
}

int pd_make_plan_tiled(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                       int num_ctas, pd_plan** out) {
    if (!out || (batch > 0 && !seq_lens)) return set_error(PD_INVALID_ARGUMENT, "make_plan: null argument");
    return build_plan(tile, seq_lens, batch, num_q_heads, num_kv_heads, num_ctas, out);
}

int pd_make_plan(int dtype, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                 int head_dim, int num_ctas, pd_plan** out) {
    if (!out || (batch > 0 && !seq_lens)) return set_error(PD_INVALID_ARGUMENT, "make_plan: null argument");
    if (num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    const int group = num_q_heads / num_kv_heads;
    int tile = 0;
    if (int rc = pd_tile_tokens(dtype, head_dim, group, &tile)) return rc;
    const int forced = num_ctas > 0 ? num_ctas : 0;
    if (num_ctas <= 0)
        if (int rc = pd_default_ctas(dtype, head_dim, group, &num_ctas)) return rc;
    if (int rc = build_plan(tile, seq_lens, batch, num_q_heads, num_kv_heads, num_ctas, out)) return rc;
    pd_plan* plan = *out;
    plan->dtype = dtype; plan->batch = batch; plan->num_q_heads = num_q_heads; plan->num_kv_heads = num_kv_heads;
    plan->forced_ctas = forced;
    plan->seq_lens.assign(seq_lens, seq_lens + batch);
    return PD_OK;
}

int pd_make_plan_weighted(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads,
                          const float* weights, int num_ctas, pd_plan** out) {
    if (!out || !weights || (batch > 0 && !seq_lens)) return set_error(PD_INVALID_ARGUMENT, "make_plan_weighted: null argument");
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    if (num_ctas <= 0 || batch <= 0) return set_error(PD_INVALID_ARGUMENT, "make_plan_weighted: batch and num_ctas must be positive");
    double sum = 0.0;
    for (int c = 0; c < num_ctas; c++) {
        if (!(weights[c] >= 0.f)) return set_error(PD_INVALID_ARGUMENT, "make_plan_weighted: weights must not be negative");
        sum += weights[c];
    }
    if (!(sum > 0.0)) return set_error(PD_INVALID_ARGUMENT, "make_plan_weighted: some weight must be positive");
    return build_plan_weighted(tile, seq_lens, batch, num_kv_heads, std::vector<float>(weights, weights + num_ctas), out);
}

int pd_plan_from_arrays(int num_ctas, int tile, const int* segments, int num_segments, const int* cta_seg_begin,
                        const int* item_seg_begin, int num_items, pd_plan** out) {
    if (!out || num_ctas < 0 || tile <= 0 || num_segments < 0 || num_items < 0 || !cta_seg_begin || !item_seg_begin ||
        (num_segments > 0 && !segments))
        return set_error(PD_INVALID_ARGUMENT, "plan_from_arrays: bad argument");
    // the tables must index the segment array consistently: the kernels trust them
    if (cta_seg_begin[0] != 0 || cta_seg_begin[num_ctas] != num_segments || item_seg_begin[0] != 0 ||
        item_seg_begin[num_items] != num_segments)
        return set_error(PD_INVALID_ARGUMENT, "plan_from_arrays: tables do not cover the segments");
    for (int c = 0; c < num_ctas; c++)
        if (cta_seg_begin[c] > cta_seg_begin[c + 1]) return set_error(PD_INVALID_ARGUMENT, "plan_from_arrays: cta_seg_begin is not monotone");
    for (int i = 0; i < num_items; i++)
        if (item_seg_begin[i] > item_seg_begin[i + 1]) return set_error(PD_INVALID_ARGUMENT, "plan_from_arrays: item_seg_begin is not monotone");
    for (int s = 0; s < num_segments; s++) {
        const int* g = segments + 4 * s;
        if (g[0] < 0 || g[1] < 0 || g[2] < 0 || g[2] >= g[3] || g[2] % tile != 0)
            return set_error(PD_INVALID_ARGUMENT, "plan_from_arrays: segment %d is malformed", s);
    }
    pd_plan* plan = new pd_plan();
    plan->num_ctas = num_ctas;
    plan->tile = tile;
    plan->num_items = num_items;
    plan->segments.assign(segments, segments + 4 * static_cast<size_t>(num_segments));
    plan->cta_seg_begin.assign(cta_seg_begin, cta_seg_begin + num_ctas + 1);
    plan->item_seg_begin.assign(item_seg_begin, item_seg_begin + num_items + 1);
    // If the arrays describe a regular layer (items in (row, kv head) order, every item covering its
    // row's tokens from 0 without gaps, the same length for all heads of a row), remember the layer so
    // that the device plan can also carry the head-fused schedule; the KV dtype stays unknown (-2).
    if (num_segments > 0) {
        int rows = 0, heads = 0;
        for (int s = 0; s < num_segments; s++) {
            rows = std::max(rows, segments[4 * s] + 1);
            heads = std::max(heads, segments[4 * s + 1] + 1);
        }
        bool regular = static_cast<long long>(rows) * heads == num_items;
        std::vector<int> lens(regular ? rows : 0, 0);
        for (int i = 0; regular && i < num_items; i++) {
            const int b = i / heads, h = i % heads;
            int at = 0;
            for (int s = item_seg_begin[i]; regular && s < item_seg_begin[i + 1]; s++) {
                const int* g = segments + 4 * s;
                regular = g[0] == b && g[1] == h && g[2] == at;
                at = g[3];
            }
            if (regular && h == 0) lens[b] = at;
            regular = regular && at > 0 && at == lens[b];
        }
        if (regular) {
            plan->dtype = -2;
            plan->batch = rows;
            plan->num_kv_heads = heads;
            plan->seq_lens = std::move(lens);
        }
    }
    *out = plan;
    return PD_OK;
}

void pd_plan_free(pd_plan* plan) { delete plan; }
int pd_plan_num_ctas(const pd_plan* p) { return p->num_ctas; }
int pd_plan_tile(const pd_plan* p) { return p->tile; }
int pd_plan_num_segments(const pd_plan* p) { return static_cast<int>(p->segments.size() / 4); }
int pd_plan_num_items(const pd_plan* p) { return p->num_items; }
const int* pd_plan_segments(const pd_plan* p) { return p->segments.data(); }
const int* pd_plan_cta_seg_begin(const pd_plan* p) { return p->cta_seg_begin.data(); }
const int* pd_plan_item_seg_begin(const pd_plan* p) { return p->item_seg_begin.data(); }

// ---- DevicePlan -------------------------------------------------------------------------------------

int pd_device_plan_create(pd_device_plan** out) {
    if (!out) return set_error(PD_INVALID_ARGUMENT, "device_plan_create: null argument");
    *out = new pd_device_plan();
    return PD_OK;
}

void pd_device_plan_destroy(pd_device_plan* dp) {
    if (!dp) return;
    if (dp->segments) {
        std::lock_guard<std::mutex> lock(g_fused_mutex);
        g_fused_registry.erase(dp->segments);
    }
    if (dp->staged) { cudaEventSynchronize(dp->staged); cudaEventDestroy(dp->staged); }
    cudaFree(dp->arena);
    cudaFree(dp->partial);
    cudaFreeHost(dp->staging);
    delete dp;
}

}  // extern "C"
namespace {
// One wave of the head-fused kernel: SMs x CTAs per SM (one, by shared memory).
int fused_wave(const KernelInfo* fk) {
    int dev = 0, sms = 0, resident = 0;
    if (fk && configure(fk) == PD_OK && cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fk->fn, fk->threads, fk->smem) == cudaSuccess)
        return sms * std::min(resident, fk->per_sm);
    cudaGetLastError();
    return 0;
}
}  // namespace
extern "C" {

int pd_device_plan_upload(pd_device_plan* dp, const pd_plan* plan, int group, int head_dim, void* stream_) {
    if (!dp || !plan) return set_error(PD_INVALID_ARGUMENT, "device_plan_upload: null argument");
    if (group <= 0 || head_dim <= 0) return set_error(PD_INVALID_ARGUMENT, "device_plan_upload: group and head_dim must be positive");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t nseg = plan->segments.size() / 4;
    auto round16 = [](size_t x) { return (x + 15) & ~static_cast<size_t>(15); };

    // The same step as head-fused row segments, when the plan says enough about the layer (made by
    // pd_make_plan) and the layer has exactly 8 kv heads: rows are the work items, 16 tokens the unit.
    pd_plan* rows_plan = nullptr;
    const KernelInfo* fk = nullptr;
    // -2: rebuilt from arrays, the dtype is only known at decode; such plans get the fp16 kernel's row cut, which
    // a decode with another dtype ignores (its tile differs)
    const bool layer_known = plan->dtype == PD_FP16 || plan->dtype == PD_FP8_E4M3 || plan->dtype == -2;
    const int fused_dtype = plan->dtype == -2 ? PD_FP16 : plan->dtype;
    if (layer_known && plan->num_kv_heads == FUSED_HEADS && plan->batch > 0 &&
        (plan->num_q_heads == 0 || plan->num_q_heads / plan->num_kv_heads == group) && head_dim == 128) {
        fk = fused_info(fused_dtype, group);
        int grid = plan->forced_ctas;
        if (fk && grid <= 0) grid = fused_wave(fk);
        // a plan rebuilt from a caller's arrays does not say whether its grid was asked for; a grid smaller
        // than one CTA per SM is taken as asked for (sharing the GPU, a sweep) and kept
        if (fk && plan->dtype == -2 && plan->num_ctas > 0 && plan->num_ctas < grid) grid = plan->num_ctas;
        if (!fk || grid <= 0 ||
            build_plan(fk->tile, plan->seq_lens.data(), plan->batch, 1, 1, grid, &rows_plan) != PD_OK)
            rows_plan = nullptr;
    }
    // Adaptive cut: the schedule that will run (head-fused where it wins, else the caller's) is cut again in
    // shares proportional to the rates its CTAs showed in earlier launches, once such a record exists.
    pd_plan* weighted_plan = nullptr;
    unsigned long long* stats_fused = nullptr;
    unsigned long long* stats_std = nullptr;
    const bool fused_runs = rows_plan && g_head_fused != 0 &&
                            (g_head_fused == 2 || plan_merge_mode(*rows_plan) != pdk::MERGE_SEPARATE);
    if (g_adaptive && plan->batch > 0 && static_cast<int>(plan->seq_lens.size()) == plan->batch) {
        if (fused_runs) {
            RateTable* t = rate_table(fk->fn, rows_plan->num_ctas);
            const std::vector<float> weights = update_weights(t, stream);
            if (t) stats_fused = t->slots;
            if (t && !weights.empty()) {
                pd_plan* w = nullptr;
                if (build_plan_weighted(fk->tile, plan->seq_lens.data(), plan->batch, 1, weights, &w) == PD_OK) {
                    delete rows_plan;
                    rows_plan = w;
                }
            }
        } else if (plan->dtype == PD_FP16 || plan->dtype == PD_FP8_E4M3) {
            const KernelInfo* sk = nullptr;
            if (find_kernel(plan->dtype, head_dim, group, &sk) == PD_OK && sk->tile == plan->tile && plan->num_ctas > 0 &&
                plan->num_kv_heads > 0 && plan->num_q_heads / plan->num_kv_heads == group) {
                RateTable* t = rate_table(sk->fn, plan->num_ctas);
                const std::vector<float> weights = update_weights(t, stream);
                if (t) stats_std = t->slots;
                if (t && !weights.empty() &&
                    build_plan_weighted(plan->tile, plan->seq_lens.data(), plan->batch, plan->num_kv_heads, weights,
                                        &weighted_plan) != PD_OK)
                    weighted_plan = nullptr;
            }
        }
    }
    struct PlanGuard { pd_plan*& p; ~PlanGuard() { delete p; } } guard{rows_plan}, guard_w{weighted_plan};

    const size_t seg_bytes  = round16(sizeof(int) * plan->segments.size());
    const size_t cta_bytes  = round16(sizeof(int) * plan->cta_seg_begin.size());
    const size_t item_bytes = round16(sizeof(int) * plan->item_seg_begin.size());
    const size_t std_bytes  = seg_bytes + cta_bytes + item_bytes;
    const size_t fseg_bytes = rows_plan ? round16(sizeof(int) * rows_plan->segments.size()) : 0;
    const size_t fcta_bytes = rows_plan ? round16(sizeof(int) * rows_plan->cta_seg_begin.size()) : 0;
    const size_t frow_bytes = rows_plan ? round16(sizeof(int) * rows_plan->item_seg_begin.size()) : 0;
    const size_t alt_bytes  = std_bytes + fseg_bytes + fcta_bytes + frow_bytes;
    const size_t wseg_bytes = weighted_plan ? round16(sizeof(int) * weighted_plan->segments.size()) : 0;
    const size_t wcta_bytes = weighted_plan ? round16(sizeof(int) * weighted_plan->cta_seg_begin.size()) : 0;
    const size_t witm_bytes = weighted_plan ? round16(sizeof(int) * weighted_plan->item_seg_begin.size()) : 0;
    const size_t total = alt_bytes + wseg_bytes + wcta_bytes + witm_bytes;
    const void* old_key = dp->segments;
    if (total > dp->arena_cap) {
        PD_CUDA(cudaFree(dp->arena));
        dp->arena = nullptr; dp->arena_cap = 0;
        PD_CUDA(cudaMalloc(&dp->arena, total));
        dp->arena_cap = total;
    }
    if (!dp->staged) PD_CUDA(cudaEventCreateWithFlags(&dp->staged, cudaEventDisableTiming));
    else PD_CUDA(cudaEventSynchronize(dp->staged));   // the previous upload still reads `staging`
    if (total > dp->staging_cap) {
        PD_CUDA(cudaFreeHost(dp->staging));
        dp->staging = nullptr; dp->staging_cap = 0;
        PD_CUDA(cudaMallocHost(&dp->staging, total));
        dp->staging_cap = total;
    }
    char* h = static_cast<char*>(dp->staging);
    std::memcpy(h, plan->segments.data(), sizeof(int) * plan->segments.size());
    std::memcpy(h + seg_bytes, plan->cta_seg_begin.data(), sizeof(int) * plan->cta_seg_begin.size());
    std::memcpy(h + seg_bytes + cta_bytes, plan->item_seg_begin.data(), sizeof(int) * plan->item_seg_begin.size());
    if (rows_plan) {
        std::memcpy(h + std_bytes, rows_plan->segments.data(), sizeof(int) * rows_plan->segments.size());
        std::memcpy(h + std_bytes + fseg_bytes, rows_plan->cta_seg_begin.data(), sizeof(int) * rows_plan->cta_seg_begin.size());
        std::memcpy(h + std_bytes + fseg_bytes + fcta_bytes, rows_plan->item_seg_begin.data(),
                    sizeof(int) * rows_plan->item_seg_begin.size());
    }
    if (weighted_plan) {
        std::memcpy(h + alt_bytes, weighted_plan->segments.data(), sizeof(int) * weighted_plan->segments.size());
        std::memcpy(h + alt_bytes + wseg_bytes, weighted_plan->cta_seg_begin.data(), sizeof(int) * weighted_plan->cta_seg_begin.size());
        std::memcpy(h + alt_bytes + wseg_bytes + wcta_bytes, weighted_plan->item_seg_begin.data(),
                    sizeof(int) * weighted_plan->item_seg_begin.size());
    }
    if (total) PD_CUDA(cudaMemcpyAsync(dp->arena, dp->staging, total, cudaMemcpyHostToDevice, stream));
    PD_CUDA(cudaEventRecord(dp->staged, stream));

    // Workspace for split rows, one region per schedule: [segments][heads][head_dim] outputs,
    // [segments][heads] LSEs, then one arrival counter per (row, kv head) for the in-kernel merge (zero
    // between launches: the merging warp re-arms its counter).
    const size_t rows = nseg * group;
    // every region starts on a 16-byte boundary: the merges read partial rows as float4
    auto round4 = [](size_t floats) { return (floats + 3) & ~static_cast<size_t>(3); };
    const size_t std_need = round4(rows * (head_dim + 1) + plan->num_items);
    const size_t frows = rows_plan ? (rows_plan->segments.size() / 4) * static_cast<size_t>(group) * FUSED_HEADS : 0;
    const size_t f_need = rows_plan ? round4(frows * (head_dim + 1) + plan->num_items) : 0;
    const size_t wrows = weighted_plan ? (weighted_plan->segments.size() / 4) * static_cast<size_t>(group) : 0;
    const size_t w_need = weighted_plan ? round4(wrows * (head_dim + 1) + plan->num_items) : 0;
    const size_t need = std_need + f_need + w_need;
    if (need > dp->partial_cap) {
        PD_CUDA(cudaFree(dp->partial));
        dp->partial = nullptr; dp->partial_cap = 0;
        PD_CUDA(cudaMalloc(&dp->partial, sizeof(float) * need));
        dp->partial_cap = need;
    }
    char* a = static_cast<char*>(dp->arena);
    dp->segments       = a;
    dp->cta_seg_begin  = reinterpret_cast<const int*>(a + seg_bytes);
    dp->item_seg_begin = reinterpret_cast<const int*>(a + seg_bytes + cta_bytes);
    dp->partial_out    = dp->partial;
    dp->partial_lse    = dp->partial ? dp->partial + rows * head_dim : nullptr;
    dp->built_on_device = false;
    dp->num_ctas       = plan->num_ctas;
    dp->num_segments   = static_cast<int>(nseg);
    dp->num_items      = plan->num_items;
    // Where rows are cut in a few pieces (a long batch: 2-3 segments per row) the decode kernel merges
    // them itself (one warp per split row); a row cut in dozens of pieces (one long sequence spread over
    // the whole grid) merges faster in the separate kernel, which puts a warp on every (row, query head).
    dp->needs_merge = plan_merge_mode(*plan);
    for (auto& t : dp->tails) t = pd_device_plan::Tail{};
    if (plan->num_items) {
        dp->tails[0] = {dp->partial + rows * head_dim, sizeof(float) * (rows + plan->num_items)};
        PD_CUDA(cudaMemsetAsync(dp->partial + rows * (head_dim + 1), 0, sizeof(int) * plan->num_items, stream));
    }

    dp->fused = pd_device_plan::Fused{};
    if (rows_plan) {
        auto& f = dp->fused;
        f.valid = true;
        f.dtype = plan->dtype; f.group = group; f.batch = plan->batch;
        f.num_ctas = rows_plan->num_ctas;
        f.num_segments = static_cast<int>(rows_plan->segments.size() / 4);
        f.needs_merge = plan_merge_mode(*rows_plan);
        f.stats = stats_fused;
        f.rows = frows;
        f.segments = a + std_bytes;
        f.cta_seg_begin = reinterpret_cast<const int*>(a + std_bytes + fseg_bytes);
        f.row_seg_begin = reinterpret_cast<const int*>(a + std_bytes + fseg_bytes + fcta_bytes);
        f.partial_out = dp->partial + std_need;
        dp->tails[1] = {f.partial_out + frows * head_dim, sizeof(float) * (frows + plan->num_items)};
        PD_CUDA(cudaMemsetAsync(f.partial_out + frows * (head_dim + 1), 0, sizeof(int) * plan->num_items, stream));
    }
    dp->weighted = pd_device_plan::Fused{};
    dp->stats = stats_std;
    if (weighted_plan) {
        auto& f = dp->weighted;
        f.valid = true;
        f.dtype = plan->dtype; f.group = group; f.batch = plan->batch;
        f.num_ctas = weighted_plan->num_ctas;
        f.num_segments = static_cast<int>(weighted_plan->segments.size() / 4);
        f.needs_merge = plan_merge_mode(*weighted_plan);
        f.rows = wrows;
        f.segments = a + alt_bytes;
        f.cta_seg_begin = reinterpret_cast<const int*>(a + alt_bytes + wseg_bytes);
        f.row_seg_begin = reinterpret_cast<const int*>(a + alt_bytes + wseg_bytes + wcta_bytes);   // (row, kv head) items
        f.partial_out = dp->partial + std_need + f_need;
        f.stats = stats_std;
        dp->tails[2] = {f.partial_out + wrows * head_dim, sizeof(float) * (wrows + plan->num_items)};
        PD_CUDA(cudaMemsetAsync(f.partial_out + wrows * (head_dim + 1), 0, sizeof(int) * plan->num_items, stream));
    }
    {
        std::lock_guard<std::mutex> lock(g_fused_mutex);
        if (old_key) g_fused_registry.erase(old_key);
        if (dp->fused.valid || dp->weighted.valid || dp->stats)
            g_fused_registry[dp->segments] = AltSchedules{dp->fused, dp->weighted, dp->stats};
        else g_fused_registry.erase(dp->segments);
    }
    return PD_OK;
}

// The plan of a step cut by plan_kernel from lengths that live on the device.  Nothing here waits for
// the device or copies from the host; buffers only grow, so after a first call with the largest batch
// later calls allocate nothing and the call can be captured into a CUDA graph together with the decode.
int pd_device_plan_build(pd_device_plan* dp, int dtype, const int* d_seq_lens, const int* d_slot_ids, int batch,
                         int num_q_heads, int num_kv_heads, int head_dim, int num_ctas, void* stream_) {
    if (!dp || (batch > 0 && !d_seq_lens)) return set_error(PD_INVALID_ARGUMENT, "device_plan_build: null argument");
    if (batch < 0) return set_error(PD_INVALID_ARGUMENT, "device_plan_build: negative batch");
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    const int group = num_q_heads / num_kv_heads;
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, head_dim, group, &k)) return rc;
    int grid = num_ctas;
    if (grid <= 0)
        if (int rc = pd_default_ctas(dtype, head_dim, group, &grid)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    auto round16 = [](size_t x) { return (x + 15) & ~static_cast<size_t>(15); };
    const size_t items = static_cast<size_t>(batch) * num_kv_heads;
    const size_t cap_seg = items + grid;                       // every cut adds one segment: at most grid - 1 cuts
    const size_t seg_bytes  = round16(sizeof(int4) * cap_seg);
    const size_t cta_bytes  = round16(sizeof(int) * (grid + 1));
    const size_t item_bytes = round16(sizeof(int) * (items + 1));
    const size_t row_bytes  = round16(sizeof(int) * (batch + 1));
    const size_t info_bytes = round16(sizeof(int) * pdk::PLAN_INFO_INTS);
    // The head-fused schedule of the same step, where the layer allows it and the batch is wide enough for
    // rows to be cut in few pieces (how they are really cut is only known on the device: each row decides
    // by its own piece count who merges it, see MERGE_HYBRID).
    const KernelInfo* fk = nullptr;
    int fgrid = 0;
    if (num_kv_heads == FUSED_HEADS && head_dim == 128 && g_head_fused != 0) {
        fk = fused_info(dtype, group);
        fgrid = num_ctas > 0 ? num_ctas : fused_wave(fk);
        if (!fk || fgrid <= 0 || (g_head_fused == 1 && batch * 3 < fgrid)) { fk = nullptr; fgrid = 0; }
    }
    const size_t fcap_seg   = fk ? static_cast<size_t>(batch) + fgrid : 0;
    const size_t fseg_bytes = fk ? round16(sizeof(int4) * fcap_seg) : 0;
    const size_t fcta_bytes = fk ? round16(sizeof(int) * (fgrid + 1)) : 0;
    const size_t frow_bytes = fk ? round16(sizeof(int) * (batch + 1)) : 0;
    const size_t std_bytes  = seg_bytes + cta_bytes + item_bytes + row_bytes + info_bytes;
    const size_t total = std_bytes + fseg_bytes + fcta_bytes + 2 * frow_bytes + (fk ? info_bytes : 0);
    const void* old_key = dp->segments;
    if (total > dp->arena_cap) {
        PD_CUDA(cudaFree(dp->arena));
        dp->arena = nullptr; dp->arena_cap = 0;
        PD_CUDA(cudaMalloc(&dp->arena, total));
        dp->arena_cap = total;
    }
    const size_t rows = cap_seg * group;
    const size_t std_need = (rows * (head_dim + 1) + items + 3) & ~static_cast<size_t>(3);   // float4 reads of the next region
    const size_t frows = fcap_seg * num_q_heads;
    const size_t need = std_need + (fk ? frows * (head_dim + 1) + items : 0);
    if (need > dp->partial_cap) {
        PD_CUDA(cudaFree(dp->partial));
        dp->partial = nullptr; dp->partial_cap = 0;
        PD_CUDA(cudaMalloc(&dp->partial, sizeof(float) * need));
        dp->partial_cap = need;
    }
    char* a = static_cast<char*>(dp->arena);
    dp->segments        = a;
    dp->cta_seg_begin   = reinterpret_cast<const int*>(a + seg_bytes);
    dp->item_seg_begin  = reinterpret_cast<const int*>(a + seg_bytes + cta_bytes);
    dp->row_tile_begin  = reinterpret_cast<int*>(a + seg_bytes + cta_bytes + item_bytes);
    dp->info            = reinterpret_cast<int*>(a + seg_bytes + cta_bytes + item_bytes + row_bytes);
    dp->partial_out     = dp->partial;
    dp->partial_lse     = dp->partial + rows * head_dim;
    dp->num_ctas        = grid;                  // the launch grid; CTAs past the cut's own count idle
    dp->num_segments    = static_cast<int>(cap_seg);
    dp->num_items       = static_cast<int>(items);
    dp->needs_merge     = pdk::MERGE_HYBRID;     // how rows were cut is only known on the device
    dp->built_on_device = true;
    dp->tile            = k->tile;
    dp->fused           = pd_device_plan::Fused{};
    dp->weighted        = pd_device_plan::Fused{};
    dp->stats           = nullptr;
    for (auto& t : dp->tails) t = pd_device_plan::Tail{};
    dp->tails[0] = {dp->partial_lse, sizeof(float) * (rows + items)};
    pdk::PlanJob job{};
    job.seq_lens = d_seq_lens; job.slot_ids = d_slot_ids;
    job.batch = batch; job.num_kv_heads = num_kv_heads; job.tile = k->tile; job.grid = grid;
    job.lse_per_segment = group; job.num_counters = static_cast<int>(items);
    job.segments = reinterpret_cast<int4*>(a);
    job.cta_seg_begin = const_cast<int*>(dp->cta_seg_begin);
    job.item_seg_begin = const_cast<int*>(dp->item_seg_begin);
    job.row_tile_begin = dp->row_tile_begin;
    job.info = dp->info;
    job.partial_lse = dp->partial_lse;
    // Adaptive cut: the planner reads the shares the host derived from earlier launches (device memory
    // with a stable address, so a captured plan keeps following them), and the decode launches of this plan
    // add to the same record.  The host folds new readings in here unless the stream is being captured;
    // callers that replay a captured step call pd_adaptive_cut_refresh between replays instead.
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) { cudaGetLastError(); capture = cudaStreamCaptureStatusActive; }
    const bool capturing = capture != cudaStreamCaptureStatusNone;
    if (g_adaptive && batch > 0) {
        if (RateTable* t = rate_table(k->fn, grid, !capturing)) {
            if (!capturing) update_weights(t, stream);
            job.shares = t->shares;
            dp->stats = t->slots;
        }
    }
    pdk::plan_kernel<<<1, pdk::PLAN_THREADS, 0, stream>>>(job);
    PD_CUDA(cudaGetLastError());
    if (fk) {
        char* fa = a + std_bytes;
        auto& f = dp->fused;
        f.valid = true;
        f.dtype = dtype; f.group = group; f.batch = batch;
        f.num_ctas = fgrid;
        f.num_segments = static_cast<int>(fcap_seg);
        f.needs_merge = pdk::MERGE_HYBRID;
        f.rows = frows;
        f.segments = fa;
        f.cta_seg_begin = reinterpret_cast<const int*>(fa + fseg_bytes);
        f.row_seg_begin = reinterpret_cast<const int*>(fa + fseg_bytes + fcta_bytes);
        f.partial_out = dp->partial + std_need;
        pdk::PlanJob fj{};
        fj.seq_lens = d_seq_lens; fj.slot_ids = d_slot_ids;
        fj.batch = batch; fj.num_kv_heads = 1; fj.tile = fk->tile; fj.grid = fgrid;   // work items are rows
        fj.lse_per_segment = num_q_heads; fj.num_counters = static_cast<int>(items);
        fj.segments = reinterpret_cast<int4*>(fa);
        fj.cta_seg_begin = const_cast<int*>(f.cta_seg_begin);
        fj.item_seg_begin = const_cast<int*>(f.row_seg_begin);
        fj.row_tile_begin = reinterpret_cast<int*>(fa + fseg_bytes + fcta_bytes + frow_bytes);
        fj.info = reinterpret_cast<int*>(fa + fseg_bytes + fcta_bytes + 2 * frow_bytes);
        fj.partial_lse = f.partial_out + frows * head_dim;
        dp->tails[1] = {f.partial_out + frows * head_dim, sizeof(float) * (frows + items)};
        if (g_adaptive && batch > 0) {
            if (RateTable* t = rate_table(fk->fn, fgrid, !capturing)) {
                if (!capturing) update_weights(t, stream);
                fj.shares = t->shares;
                f.stats = t->slots;
            }
        }
        pdk::plan_kernel<<<1, pdk::PLAN_THREADS, 0, stream>>>(fj);
        PD_CUDA(cudaGetLastError());
    }
    {
        std::lock_guard<std::mutex> lock(g_fused_mutex);
        if (old_key) g_fused_registry.erase(old_key);
        if (dp->fused.valid || dp->stats) g_fused_registry[dp->segments] = AltSchedules{dp->fused, dp->weighted, dp->stats};
        else g_fused_registry.erase(dp->segments);
    }
    return PD_OK;
}

int pd_device_plan_info(const pd_device_plan* dp, int* out, void* stream_) {
    if (!dp || !out) return set_error(PD_INVALID_ARGUMENT, "device_plan_info: null argument");
    if (!dp->built_on_device) return set_error(PD_INVALID_ARGUMENT, "device_plan_info: the plan was not built on the device");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PD_CUDA(cudaMemcpyAsync(out, dp->info, sizeof(int) * pdk::PLAN_INFO_INTS, cudaMemcpyDeviceToHost, stream));
    PD_CUDA(cudaStreamSynchronize(stream));
    return PD_OK;
}

int pd_device_plan_fetch(const pd_device_plan* dp, pd_plan** out, void* stream_) {
    if (!dp || !out) return set_error(PD_INVALID_ARGUMENT, "device_plan_fetch: null argument");
    int info[pdk::PLAN_INFO_INTS];
    if (int rc = pd_device_plan_info(dp, info, stream_)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    pd_plan* plan = new pd_plan();
    plan->num_ctas = info[pdk::PLAN_INFO_CTAS];
    plan->tile = dp->tile;
    plan->num_items = dp->num_items;
    plan->segments.resize(4 * static_cast<size_t>(info[pdk::PLAN_INFO_SEGMENTS]));
    plan->cta_seg_begin.resize(plan->num_ctas + 1);
    plan->item_seg_begin.resize(plan->num_items + 1);
    cudaError_t e = cudaSuccess;
    if (!plan->segments.empty())
        e = cudaMemcpyAsync(plan->segments.data(), dp->segments, sizeof(int) * plan->segments.size(), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(plan->cta_seg_begin.data(), dp->cta_seg_begin, sizeof(int) * plan->cta_seg_begin.size(), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(plan->item_seg_begin.data(), dp->item_seg_begin, sizeof(int) * plan->item_seg_begin.size(), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { delete plan; return set_error(PD_CUDA_ERROR, "device_plan_fetch: %s", cudaGetErrorString(e)); }
    *out = plan;
    return PD_OK;
}

int pd_device_plan_bind(const pd_device_plan* dp, pd_params* p) {
    if (!dp || !p) return set_error(PD_INVALID_ARGUMENT, "device_plan_bind: null argument");
    p->segments       = dp->segments;
    p->cta_seg_begin  = dp->cta_seg_begin;
    p->item_seg_begin = dp->item_seg_begin;
    p->num_ctas       = dp->num_ctas;
    p->needs_merge    = dp->needs_merge;
    p->partial_out    = dp->partial_out;
    p->partial_lse    = dp->partial_lse;
    return PD_OK;
}

// After a PD_KERNEL_TIMEOUT: a CTA that gave up on a bounded wait skipped its arrivals, so the counters of
// the in-kernel merge may hold partial counts that the next launch of the same plan would trip over.
int pd_device_plan_reset(pd_device_plan* dp, void* stream_) {
    if (!dp) return set_error(PD_INVALID_ARGUMENT, "device_plan_reset: null argument");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    for (const auto& t : dp->tails)
        if (t.ptr && t.bytes) PD_CUDA(cudaMemsetAsync(t.ptr, 0, t.bytes, stream));
    return PD_OK;
}

// ---- decode -----------------------------------------------------------------------------------------------

}  // extern "C"

namespace {
// Which schedule a decode of these params runs.  The plan they were bound to (pd_device_plan_bind) may carry,
// next to the caller's (row, kv head) cut, the same step cut by rows for the head-fused kernel (fp16, 8 kv
// heads, plan made by pd_make_plan) and the caller's cut in unequal shares (adaptive cut); they are found
// through the address of the bound segment array.  Params that point at arrays of the caller's own run as
// they are.
struct Selection {
    const pd_params* params;
    const KernelInfo* kernel;
    int box_heads;                 // kv heads per TMA box: 1, or 8 for the head-fused kernel
    int schedule;                  // 0 the caller's plan, 1 head-fused rows, 2 the caller's plan in unequal shares
    unsigned long long* stats;
};
Selection select_schedule(int dtype, const pd_params* p, const KernelInfo* k, bool gathered, pd_params* scratch) {
    Selection sel{p, k, 1, 0, nullptr};
    AltSchedules alt;
    {
        std::lock_guard<std::mutex> lock(g_fused_mutex);
        auto it = g_fused_registry.find(p->segments);
        if (it == g_fused_registry.end()) return sel;
        alt = it->second;
    }
    const int group = p->num_q_heads / p->num_kv_heads;
    auto matches = [&](const pd_device_plan::Fused& f) {
        return f.valid && (f.dtype == dtype || (f.dtype == -2 && dtype == PD_FP16)) && f.batch == p->batch && f.group == group;
    };
    const KernelInfo* fk = p->num_kv_heads == FUSED_HEADS ? fused_info(dtype, group) : nullptr;
    // Head-fused, mode 1: not where rows would be spread over more than 4 CTAs each.
    const bool use_fused = fk && g_head_fused && matches(alt.fused) &&
                           (g_head_fused == 2 || alt.fused.needs_merge != pdk::MERGE_SEPARATE);
    const bool use_weighted = !use_fused && g_adaptive && matches(alt.weighted);
    if (g_adaptive && !use_fused && !use_weighted) sel.stats = alt.stats;
    if (use_fused || use_weighted) {
        const pd_device_plan::Fused& f = use_fused ? alt.fused : alt.weighted;
        *scratch = *p;
        scratch->segments = f.segments;
        scratch->cta_seg_begin = f.cta_seg_begin;
        scratch->item_seg_begin = f.row_seg_begin;       // work items: rows (head-fused) or (row, kv head)
        scratch->num_ctas = f.num_ctas;
        scratch->needs_merge = f.needs_merge;            // this schedule has its own splits
        if (gathered && scratch->needs_merge) scratch->needs_merge = pdk::MERGE_IN_KERNEL;   // gathered rows are written by the decode kernel
        scratch->partial_out = f.partial_out;
        scratch->partial_lse = f.partial_out + f.rows * p->head_dim;
        sel.params = scratch;
        sel.schedule = use_fused ? 1 : 2;
        if (use_fused) { sel.kernel = fk; sel.box_heads = FUSED_HEADS; }
        if (g_adaptive) sel.stats = f.stats;
    }
    return sel;
}

int decode_impl(int dtype, const pd_params* p, int num_pages, const pdk::GatherOut& gather, void* stream_,
                const pdk::HeadScales& scales = pdk::HeadScales{nullptr, nullptr}) {
    if (!p) return set_error(PD_INVALID_ARGUMENT, "paged_decode: null params");
    if (p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, p->head_dim, p->num_q_heads / p->num_kv_heads, &k)) return rc;
    if (p->page_size <= 0) return set_error(PD_INVALID_ARGUMENT, "page_size must be positive");
    if (p->num_ctas <= 0 || p->batch <= 0) return PD_OK;   // empty plan: nothing to do
    if (!p->q || (!p->out && !gather.world) || !p->k_cache || !p->v_cache || !p->block_table || !p->segments ||
        !p->cta_seg_begin || !p->item_seg_begin)
        return set_error(PD_INVALID_ARGUMENT, "paged_decode: null device pointer");
    if (p->needs_merge && (!p->partial_out || !p->partial_lse))
        return set_error(PD_INVALID_ARGUMENT, "paged_decode: split rows need the partial workspace");
    if (reinterpret_cast<uintptr_t>(p->q) % 16 != 0 || reinterpret_cast<uintptr_t>(p->out) % 16 != 0)
        return set_error(PD_INVALID_ARGUMENT, "paged_decode: q and out must be 16-byte aligned");
    pd_params alt_params;
    Selection sel = select_schedule(dtype, p, k, gather.world != 0, &alt_params);
    p = sel.params;
    k = sel.kernel;
    const int box_heads = sel.box_heads;
    unsigned long long* stats_slots = sel.stats;
    if (int rc = configure(k)) return rc;
    unsigned* status = nullptr;
    if (int rc = status_word(&status)) return rc;

    // A box is the largest run of tokens that never straddles a page or a tile.  Where that is fewer than four
    // tokens (pages of 1, 2, 3, 5, ... tokens) the (row, kv head) kernel gathers four rows per copy instead:
    // one TMA operation per token would leave the copy engine, not DRAM, as the limit.
    const unsigned box_tokens = gcd_u(static_cast<unsigned>(p->page_size), static_cast<unsigned>(k->tile));
    int btl = 0;
    while ((1u << (btl + 1)) <= box_tokens) btl++;
    const bool row_gather = box_heads == 1 && btl < 2;
    if (row_gather) btl = 2;
    CUtensorMap k_map, v_map;
    if (int rc = make_tensor_map(&k_map, dtype, p->k_cache, num_pages, p->num_kv_heads, p->page_size, btl, box_heads, row_gather)) return rc;
    if (int rc = make_tensor_map(&v_map, dtype, p->v_cache, num_pages, p->num_kv_heads, p->page_size, btl, box_heads, row_gather)) return rc;

    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    k->launch(*p, k_map, v_map, btl, row_gather ? 1 : 0, 0, status, gather, scales, pdk::CtaStats{stats_slots}, stream);
    PD_CUDA(cudaGetLastError());
    if (p->needs_merge && p->needs_merge != pdk::MERGE_IN_KERNEL) {
        k->merge(*p, 0, stream);
        PD_CUDA(cudaGetLastError());
    }
    return PD_OK;
}
}  // namespace

extern "C" {

int pd_paged_decode_bounded(int dtype, const pd_params* p, int num_pages, void* stream) {
    return decode_impl(dtype, p, num_pages, pdk::GatherOut{}, stream);
}

int pd_paged_decode(int dtype, const pd_params* p, void* stream) {
    return pd_paged_decode_bounded(dtype, p, 0, stream);
}

int pd_paged_decode_scaled(int dtype, const pd_params* p, int num_pages, const float* d_k_scales, const float* d_v_scales,
                           void* stream) {
    return decode_impl(dtype, p, num_pages, pdk::GatherOut{}, stream, pdk::HeadScales{d_k_scales, d_v_scales});
}

int pd_describe_launch(int dtype, const pd_params* p, int* out) {
    if (!p || !out) return set_error(PD_INVALID_ARGUMENT, "describe_launch: null argument");
    if (p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, p->head_dim, p->num_q_heads / p->num_kv_heads, &k)) return rc;
    pd_params scratch;
    const Selection sel = select_schedule(dtype, p, k, false, &scratch);
    out[0] = sel.schedule;
    out[1] = sel.params->num_ctas;
    out[2] = sel.kernel->tile;
    out[3] = sel.box_heads;
    out[4] = sel.kernel->threads / 32 - 1;
    out[5] = sel.kernel->stages;
    out[6] = sel.kernel->per_sm;
    out[7] = sel.params->needs_merge;
    return PD_OK;
}

// ---- decode without any allocation -------------------------------------------------------------------------
//
// For callers that must not let this library allocate device memory.  Two kinds exist in
// practice: a serving process that gave every free byte of HBM to its KV pool when it started,
// so a workspace cudaMalloc at step time fails (or lands wherever the pool left a hole); and a
// latency-critical step loop that bans cudaMalloc/cudaFree outright because both stall the
// whole device while they run.  The ordinary path sizes the split-row workspace
// (partial_out | partial_lse) with cudaMalloc in pd_device_plan_upload and keeps its status word
// in a small cudaMalloc'd cell; this entry point takes both from arrays that are part of the
// loaded library image instead.
//
// The arrays below are ordinary device globals.  Their names are usable directly in device
// code; in host code a name is only a handle for the runtime, never a device address, so the
// address handed to the kernels comes from cudaGetSymbolAddress, once per device.

namespace {

constexpr size_t STATIC_SCRATCH_FLOATS = size_t(2) << 20;   // 8 MiB per GPU that loads the library

static __device__ __align__(256) float    g_static_partials[STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned g_static_status[64];   // [0] is the status word

struct StaticScratch {
    float*    partials = nullptr;
    unsigned* status   = nullptr;
    bool      ready    = false;
};
StaticScratch g_static_scratch[MAX_DEVICES];
std::mutex    g_static_scratch_mutex;

// One-time set-up for the current device: resolve the device addresses of the two arrays.
int static_scratch(const StaticScratch** out) {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return set_error(PD_INTERNAL, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    StaticScratch& s = g_static_scratch[dev];
    if (!s.ready) {
        float* partials = nullptr;
        unsigned* status = nullptr;
        PD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&partials), g_static_partials));
        PD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_static_status));
        s.partials = partials;
        s.status   = status;
        s.ready    = true;
    }
    *out = &s;
    return PD_OK;
}

}  // namespace

int pd_paged_decode_static(int dtype, const pd_params* p, int num_segments, int num_pages,
                           unsigned* d_status, void* stream_) {
    if (!p) return set_error(PD_INVALID_ARGUMENT, "paged_decode_static: null params");
    if (p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    const int group = p->num_q_heads / p->num_kv_heads;
    const KernelInfo* k;
    if (int rc = find_kernel(dtype, p->head_dim, group, &k)) return rc;
    if (p->page_size <= 0) return set_error(PD_INVALID_ARGUMENT, "page_size must be positive");
    if (num_segments < 0) return set_error(PD_INVALID_ARGUMENT, "paged_decode_static: num_segments must not be negative");
    const size_t rows = static_cast<size_t>(num_segments) * group;
    const size_t need = rows * (p->head_dim + 1);
    if (need > STATIC_SCRATCH_FLOATS)
        return set_error(PD_INVALID_ARGUMENT,
                         "paged_decode_static: %d segments x group %d need %zu bytes of split-row workspace, "
                         "the built-in workspace holds %zu bytes; plan with fewer CTAs or use pd_paged_decode",
                         num_segments, group, need * sizeof(float), STATIC_SCRATCH_FLOATS * sizeof(float));
    if (p->num_ctas <= 0 || p->batch <= 0) return PD_OK;
    if (!p->q || !p->out || !p->k_cache || !p->v_cache || !p->block_table || !p->segments || !p->cta_seg_begin ||
        !p->item_seg_begin)
        return set_error(PD_INVALID_ARGUMENT, "paged_decode_static: null device pointer");
    if (int rc = configure(k)) return rc;
    const StaticScratch* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;

    if (reinterpret_cast<uintptr_t>(p->q) % 16 != 0 || reinterpret_cast<uintptr_t>(p->out) % 16 != 0)
        return set_error(PD_INVALID_ARGUMENT, "paged_decode_static: q and out must be 16-byte aligned");
    pd_params local = *p;                       // same launch, workspace redirected to the built-in array
    local.partial_out = scratch->partials;
    local.partial_lse = scratch->partials + rows * p->head_dim;
    local.needs_merge = p->needs_merge ? pdk::MERGE_SEPARATE : 0;   // the built-in array carries no arrival counters

    const unsigned box_tokens = gcd_u(static_cast<unsigned>(p->page_size), static_cast<unsigned>(k->tile));
    int btl = 0;
    while ((1u << (btl + 1)) <= box_tokens) btl++;
    const bool row_gather = btl < 2;
    if (row_gather) btl = 2;
    CUtensorMap k_map, v_map;
    if (int rc = make_tensor_map(&k_map, dtype, p->k_cache, num_pages, p->num_kv_heads, p->page_size, btl, 1, row_gather)) return rc;
    if (int rc = make_tensor_map(&v_map, dtype, p->v_cache, num_pages, p->num_kv_heads, p->page_size, btl, 1, row_gather)) return rc;

    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // The kernels compare the declared count with the plan they walk (cta_seg_begin on the device): a CTA
    // whose segments lie beyond it stores nothing and reports ST_WORKSPACE instead of writing past the array.
    const int seg_limit = std::max(num_segments, 1);
    k->launch(local, k_map, v_map, btl, row_gather ? 1 : 0, seg_limit, d_status ? d_status : scratch->status, pdk::GatherOut{},
              pdk::HeadScales{nullptr, nullptr}, pdk::CtaStats{nullptr}, stream);
    PD_CUDA(cudaGetLastError());
    if (local.needs_merge) {
        k->merge(local, seg_limit, stream);
        PD_CUDA(cudaGetLastError());
    }
    return PD_OK;
}

int pd_kernel_status(void* stream, unsigned* out) {
    if (!out) return set_error(PD_INVALID_ARGUMENT, "kernel_status: null argument");
    unsigned* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    PD_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    PD_CUDA(cudaMemcpy(out, status, sizeof(unsigned), cudaMemcpyDeviceToHost));
    if (*out) {
        PD_CUDA(cudaMemset(status, 0, sizeof(unsigned)));
        if ((*out >> 24) == pdk::ST_WORKSPACE)
            return set_error(PD_KERNEL_TIMEOUT, "decode kernel: the plan has more segments than the workspace holds (CTA %u gave up)",
                             *out & 0xffffffu);
        return set_error(PD_KERNEL_TIMEOUT, "decode kernel: bounded wait %u expired in CTA %u", *out >> 24, *out & 0xffffffu);
    }
    return PD_OK;
}

// ---- bandwidth probe ---------------------------------------------------------------------------------------

int pd_stream_read(const void* d_buf, size_t bytes, int blocks, void* stream_) {
    if (!d_buf || bytes < 16 || blocks <= 0 || reinterpret_cast<uintptr_t>(d_buf) % 16 != 0)
        return set_error(PD_INVALID_ARGUMENT, "stream_read: bad argument");
    unsigned* sink = nullptr;
    if (int rc = status_word(&sink)) return rc;   // never written: the fold value cannot match
    pdk::stream_read_kernel<<<blocks, 512, 0, static_cast<cudaStream_t>(stream_)>>>(
        static_cast<const uint4*>(d_buf), bytes / 16, sink);
    PD_CUDA(cudaGetLastError());
    return PD_OK;
}

// ---- append ------------------------------------------------------------------------------------------------

int pd_append_tokens_scaled(int dtype, const void* d_k, const void* d_v, void* k_cache, void* v_cache,
                            const int* d_block_table_row, int start_pos, int n, int num_kv_heads, int head_dim,
                            int page_size, float k_scale, float v_scale, const float* d_k_scales, const float* d_v_scales,
                            void* stream_) {
    if (dtype != PD_FP16 && dtype != PD_FP8_E4M3) return set_error(PD_INVALID_ARGUMENT, "unsupported KV dtype %d", dtype);
    if (head_dim != 128) return set_error(PD_INVALID_ARGUMENT, "append: head_dim must be 128");
    if (n <= 0) return PD_OK;
    if (!d_k || !d_v || !k_cache || !v_cache || !d_block_table_row || num_kv_heads <= 0 || page_size <= 0 || start_pos < 0)
        return set_error(PD_INVALID_ARGUMENT, "append: bad argument");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v) | reinterpret_cast<uintptr_t>(k_cache) |
         reinterpret_cast<uintptr_t>(v_cache)) % 16 != 0)
        return set_error(PD_INVALID_ARGUMENT, "append: K/V buffers must be 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    pdk::AppendJob job{static_cast<const __half*>(d_k), static_cast<const __half*>(d_v), d_block_table_row, start_pos, n, 0};
    const long long units = static_cast<long long>(n) * num_kv_heads * 16;
    const int blocks = static_cast<int>(std::min<long long>((units + 255) / 256, 148 * 16));
    if (dtype == PD_FP16)
        pdk::append_kernel<false><<<blocks, 256, 0, stream>>>(job, k_cache, v_cache, num_kv_heads, page_size, 1.f, 1.f,
                                                              pdk::AppendHeadScales{nullptr, nullptr});
    else
        pdk::append_kernel<true><<<blocks, 256, 0, stream>>>(job, k_cache, v_cache, num_kv_heads, page_size,
                                                             1.f / k_scale, 1.f / v_scale,
                                                             pdk::AppendHeadScales{d_k_scales, d_v_scales});
    PD_CUDA(cudaGetLastError());
    return PD_OK;
}

int pd_append_tokens(int dtype, const void* d_k, const void* d_v, void* k_cache, void* v_cache,
                     const int* d_block_table_row, int start_pos, int n, int num_kv_heads, int head_dim,
                     int page_size, float k_scale, float v_scale, void* stream) {
    return pd_append_tokens_scaled(dtype, d_k, d_v, k_cache, v_cache, d_block_table_row, start_pos, n, num_kv_heads,
                                   head_dim, page_size, k_scale, v_scale, nullptr, nullptr, stream);
}

// ---- outputs gathered over the GPUs of a node by peer stores ---------------------------------------------------
//
// One process per GPU.  Each rank allocates one block: GATHER_BUFFERS gathered-output buffers used in
// rotation (step e fills buffer e mod 4), one flag per peer, one CTA counter.  Blocks are exchanged as
// CUDA IPC handles; after pd_gather_connect every rank can store into every peer's block.
// Why four buffers: a rank may run step e+1's decode before it waits for step e's rows (the wait then
// overlaps the next decode).  Its stream order is d(e+1), w(e), use(e), d(e+2), w(e+1), ...; a peer's
// d(e+4) overwrites buffer e mod 4 and is ordered after that peer's w(e+2), i.e. after this rank's d(e+2)
// has finished, which in this rank's stream comes after use(e).  With the wait directly behind every
// decode two buffers would do.

} // extern "C"

constexpr unsigned GATHER_BUFFERS = 4;
struct pd_gather_group {
    int world = 0, rank = 0;
    size_t out_bytes = 0, block_bytes = 0;
    unsigned epoch = 0;
    char* block[pdk::MAX_GATHER] = {};      // block[rank] is the local allocation, the rest are IPC mappings
    bool connected = false;
    size_t flags_offset() const { return GATHER_BUFFERS * out_bytes; }
};

extern "C" {

int pd_gather_create(int world, int rank, size_t out_bytes, pd_gather_group** out) {
    if (!out || world < 1 || world > pdk::MAX_GATHER || rank < 0 || rank >= world || out_bytes == 0)
        return set_error(PD_INVALID_ARGUMENT, "gather_create: world must be 1..%d, rank inside it, out_bytes positive", pdk::MAX_GATHER);
    pd_gather_group* g = new pd_gather_group();
    g->world = world; g->rank = rank;
    g->out_bytes = (out_bytes + 255) & ~static_cast<size_t>(255);
    g->block_bytes = GATHER_BUFFERS * g->out_bytes + 256;
    void* b = nullptr;
    cudaError_t e = cudaMalloc(&b, g->block_bytes);
    if (e == cudaSuccess) e = cudaMemset(b, 0, g->block_bytes);
    if (e != cudaSuccess) {
        cudaFree(b);
        delete g;
        return set_error(PD_CUDA_ERROR, "gather_create: %s", cudaGetErrorString(e));
    }
    g->block[rank] = static_cast<char*>(b);
    g->connected = world == 1;
    *out = g;
    return PD_OK;
}

void pd_gather_destroy(pd_gather_group* g) {
    if (!g) return;
    for (int r = 0; r < g->world; r++) {
        if (!g->block[r]) continue;
        if (r == g->rank) cudaFree(g->block[r]);
        else cudaIpcCloseMemHandle(g->block[r]);
    }
    delete g;
}

int pd_gather_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

int pd_gather_export(const pd_gather_group* g, unsigned char* handle) {
    if (!g || !handle) return set_error(PD_INVALID_ARGUMENT, "gather_export: null argument");
    cudaIpcMemHandle_t h;
    PD_CUDA(cudaIpcGetMemHandle(&h, g->block[g->rank]));
    std::memcpy(handle, &h, sizeof h);
    return PD_OK;
}

int pd_gather_connect(pd_gather_group* g, const unsigned char* all_handles) {
    if (!g || !all_handles) return set_error(PD_INVALID_ARGUMENT, "gather_connect: null argument");
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank || g->block[r]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, all_handles + static_cast<size_t>(r) * sizeof h, sizeof h);
        void* ptr = nullptr;
        PD_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        g->block[r] = static_cast<char*>(ptr);
    }
    g->connected = true;
    return PD_OK;
}

void* pd_gather_buffer(const pd_gather_group* g, int which) {
    if (!g) return nullptr;
    const unsigned index = which < 0 ? g->epoch % GATHER_BUFFERS : static_cast<unsigned>(which) % GATHER_BUFFERS;
    return g->block[g->rank] + index * g->out_bytes;
}

unsigned pd_gather_epoch(const pd_gather_group* g) { return g ? g->epoch : 0; }

}  // extern "C"
namespace {
int decode_gather_impl(int dtype, const pd_params* p, int num_pages, pd_gather_group* g, int row_stride_heads,
                       int head_offset, int row_offset, bool wait, void* stream) {
    if (!g || !p) return set_error(PD_INVALID_ARGUMENT, "decode_gather: null argument");
    if (!g->connected) return set_error(PD_INVALID_ARGUMENT, "decode_gather: call pd_gather_connect first");
    if (row_stride_heads < p->num_q_heads + head_offset || head_offset < 0 || row_offset < 0)
        return set_error(PD_INVALID_ARGUMENT, "decode_gather: this rank's slice does not fit the gathered row");
    const size_t last = (static_cast<size_t>(p->batch + row_offset) * row_stride_heads) * 128 * sizeof(__half);
    if (last > g->out_bytes) return set_error(PD_INVALID_ARGUMENT, "decode_gather: gathered layout exceeds the buffer");
    if (p->num_ctas <= 0 || p->batch <= 0) return set_error(PD_INVALID_ARGUMENT, "decode_gather: empty plan");
    g->epoch++;
    pdk::GatherOut go{};
    pdk::GatherFlags gf{};
    go.world = g->world; go.rank = g->rank;
    go.row_stride = row_stride_heads; go.head_offset = head_offset; go.row_offset = row_offset;
    for (int r = 0; r < g->world; r++) {
        go.out[r]   = reinterpret_cast<__half*>(g->block[r] + (g->epoch % GATHER_BUFFERS) * g->out_bytes);
        gf.flags[r] = reinterpret_cast<unsigned*>(g->block[r] + g->flags_offset());
    }
    // Gathered rows are written by the decode kernel itself, so split rows are merged in-kernel here
    // even where the plan preferred the separate merge kernel; workspaces bound by
    // pd_device_plan_bind always carry the arrival counters that needs.
    pd_params local = *p;
    if (local.needs_merge) local.needs_merge = pdk::MERGE_IN_KERNEL;
    const int rc = decode_impl(dtype, &local, num_pages, go, stream);
    if (rc != PD_OK) { g->epoch--; return rc; }
    // the announcement: one warp, launched as a programmatic dependent of the decode kernel
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const unsigned* wait_flags = wait ? reinterpret_cast<const unsigned*>(g->block[g->rank] + g->flags_offset()) : nullptr;
    unsigned* status = nullptr;
    if (int rc2 = status_word(&status)) return rc2;
    PD_CUDA(cudaLaunchKernelEx(&cfg, pdk::gather_signal_kernel, gf, g->world, g->rank, g->epoch, wait_flags, status));
    return PD_OK;
}
}  // namespace
extern "C" {

int pd_paged_decode_gather(int dtype, const pd_params* p, int num_pages, pd_gather_group* g, int row_stride_heads,
                           int head_offset, int row_offset, void* stream) {
    return decode_gather_impl(dtype, p, num_pages, g, row_stride_heads, head_offset, row_offset, false, stream);
}

int pd_paged_decode_gather_sync(int dtype, const pd_params* p, int num_pages, pd_gather_group* g, int row_stride_heads,
                                int head_offset, int row_offset, void* stream) {
    return decode_gather_impl(dtype, p, num_pages, g, row_stride_heads, head_offset, row_offset, true, stream);
}

int pd_gather_wait_epoch(pd_gather_group* g, unsigned epoch, void* stream) {
    if (!g) return set_error(PD_INVALID_ARGUMENT, "gather_wait: null argument");
    unsigned* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    PD_CUDA(cudaLaunchKernelEx(&cfg, pdk::gather_wait_kernel,
                               reinterpret_cast<const unsigned*>(g->block[g->rank] + g->flags_offset()), g->world, epoch, status));
    return PD_OK;
}

int pd_gather_wait(pd_gather_group* g, void* stream) {
    if (!g) return set_error(PD_INVALID_ARGUMENT, "gather_wait: null argument");
    return pd_gather_wait_epoch(g, g->epoch, stream);
}

// ---- PagedKVCache ---------------------------------------------------------------------------------------------

size_t pd_cache_bytes_per_page(const pd_cache_config* cfg) {
    return 2ull * cfg->num_kv_heads * cfg->page_size * cfg->head_dim * pd_kv_dtype_bytes(cfg->dtype);
}

int pd_cache_pages_for_budget(const pd_cache_config* cfg, size_t budget_bytes) {
    return static_cast<int>(budget_bytes / pd_cache_bytes_per_page(cfg));
}

void pd_cache_destroy(pd_cache* c) {
    if (!c) return;
    cudaFree(c->d_k);
    cudaFree(c->d_v);
    cudaFree(c->d_block_table);
    cudaFree(c->d_seq_lens);
    cudaFree(c->d_slot_ids);
    cudaFree(c->d_head_scales);
    if (c->batch_staged) { cudaEventSynchronize(c->batch_staged); cudaEventDestroy(c->batch_staged); }
    if (c->batch_done) { cudaEventSynchronize(c->batch_done); cudaEventDestroy(c->batch_done); }
    cudaFreeHost(c->batch_staging);
    cudaFree(c->batch_device);
    pd_plan_free(c->plan);
    pd_device_plan_destroy(c->device_plan);
    delete c;
}

int pd_cache_create(const pd_cache_config* cfg, pd_cache** out) {
    if (!cfg || !out) return set_error(PD_INVALID_ARGUMENT, "PagedKVCache: null argument");
    if (cfg->num_pages <= 0 || cfg->page_size <= 0 || cfg->num_kv_heads <= 0 || cfg->max_slots <= 0 ||
        cfg->max_pages_per_slot <= 0)
        return set_error(PD_INVALID_ARGUMENT, "PagedKVCache: all sizes must be positive");
    if (cfg->head_dim != 128) return set_error(PD_INVALID_ARGUMENT, "PagedKVCache: head_dim must be 128");
    if (cfg->dtype != PD_FP16 && cfg->dtype != PD_FP8_E4M3) return set_error(PD_INVALID_ARGUMENT, "PagedKVCache: unsupported KV dtype");
    pd_cache* c = new pd_cache();
    c->cfg = *cfg;
    c->tables.resize(cfg->max_slots);
    c->seq_lens.assign(cfg->max_slots, 0);
    c->occupied.assign(cfg->max_slots, 0);
    auto fail = [&](int rc) { pd_cache_destroy(c); return rc; };
#define PD_CACHE_CUDA(expr)                                                                           \
    do {                                                                                              \
        cudaError_t e_ = (expr);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return fail(set_error(PD_CUDA_ERROR, "CUDA error %s at %s:%d: %s", cudaGetErrorName(e_),  \
                                  __FILE__, __LINE__, cudaGetErrorString(e_)));                       \
    } while (0)
    const size_t half_bytes = pd_cache_bytes_per_page(cfg) / 2 * cfg->num_pages;
    const size_t table_bytes = sizeof(int) * static_cast<size_t>(cfg->max_slots) * cfg->max_pages_per_slot;
    PD_CACHE_CUDA(cudaMalloc(&c->d_k, half_bytes));
    PD_CACHE_CUDA(cudaMalloc(&c->d_v, half_bytes));
    // Pools start as zeros: the decode kernel copies whole pages, and bytes a sequence
    // never wrote must not decode to NaN.
    PD_CACHE_CUDA(cudaMemset(c->d_k, 0, half_bytes));
    PD_CACHE_CUDA(cudaMemset(c->d_v, 0, half_bytes));
    PD_CACHE_CUDA(cudaMalloc(&c->d_block_table, table_bytes));
    PD_CACHE_CUDA(cudaMalloc(&c->d_seq_lens, sizeof(int) * cfg->max_slots));
    PD_CACHE_CUDA(cudaMemset(c->d_block_table, 0, table_bytes));
    PD_CACHE_CUDA(cudaMemset(c->d_seq_lens, 0, sizeof(int) * cfg->max_slots));
#undef PD_CACHE_CUDA
    if (int rc = pd_device_plan_create(&c->device_plan)) return fail(rc);
    // Pages are taken from the back of the list; page 0 goes out first.
    c->free_pages.resize(cfg->num_pages);
    for (int i = 0; i < cfg->num_pages; i++) c->free_pages[i] = cfg->num_pages - 1 - i;
    *out = c;
    return PD_OK;
}

int pd_cache_admit(pd_cache* c) {
    for (int s = 0; s < c->cfg.max_slots; s++)
        if (!c->occupied[s]) {
            c->occupied[s] = 1;
            c->seq_lens[s] = 0;
            return s;
        }
    return -1;
}

int pd_cache_append(pd_cache* c, int slot, const void* d_k, const void* d_v, int n, void* stream_) {
    if (!c || slot < 0 || slot >= c->cfg.max_slots || !c->occupied[slot])
        return set_error(PD_INVALID_ARGUMENT, "append: slot is not admitted");
    if (n <= 0) return PD_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int ps = c->cfg.page_size;
    const int old_len = c->seq_lens[slot];
    const int new_len = old_len + n;
    const int have = static_cast<int>(c->tables[slot].size());
    const int need = (new_len + ps - 1) / ps;
    if (need > c->cfg.max_pages_per_slot) return set_error(PD_LENGTH_ERROR, "append: sequence exceeds max_pages_per_slot");
    if (need - have > static_cast<int>(c->free_pages.size()))
        return set_error(PD_OUT_OF_PAGES, "append: out of pages");
    for (int i = have; i < need; i++) {
        c->tables[slot].push_back(c->free_pages.back());
        c->free_pages.pop_back();
    }
    int* row = c->d_block_table + static_cast<size_t>(slot) * c->cfg.max_pages_per_slot;
    // Pageable-source copies are staged by the driver before they return.
    if (need > have)
        PD_CUDA(cudaMemcpyAsync(row + have, c->tables[slot].data() + have, sizeof(int) * (need - have),
                                cudaMemcpyHostToDevice, stream));
    c->seq_lens[slot] = new_len;
    PD_CUDA(cudaMemcpyAsync(c->d_seq_lens + slot, &c->seq_lens[slot], sizeof(int), cudaMemcpyHostToDevice, stream));
    if (int rc = pd_append_tokens_scaled(c->cfg.dtype, d_k, d_v, c->d_k, c->d_v, row, old_len, n, c->cfg.num_kv_heads,
                                         c->cfg.head_dim, ps, c->cfg.k_scale, c->cfg.v_scale, c->d_head_scales,
                                         c->d_head_scales ? c->d_head_scales + c->cfg.num_kv_heads : nullptr, stream))
        return rc;
    // As in the reference (src/decode/paged_kv_cache.cu:133-134) the call returns with the tokens in place.
    PD_CUDA(cudaStreamSynchronize(stream));
    return PD_OK;
}

// One decode step's appends for many slots: the allocator runs for every slot in the order given
// (so block tables come out exactly as from the same pd_cache_append calls in that order), then
// ONE packed host->device copy carries the job list, the new block-table entries and the new
// lengths, and two launches apply them: table/length updates, then the token scatter for all
// slots at once.  All-or-nothing: if the pool cannot hold every slot's tokens nothing changes.
// Stream-ordered: returns without waiting; the K/V sources must stay valid until the stream
// has run the scatter.
int pd_cache_append_batch(pd_cache* c, int count, const int* slots, const void* const* d_k, const void* const* d_v,
                          const int* n, void* stream_) {
    if (!c || count < 0 || (count > 0 && (!slots || !d_k || !d_v || !n)))
        return set_error(PD_INVALID_ARGUMENT, "append_batch: bad argument");
    if (count == 0) return PD_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int ps = c->cfg.page_size;
    // ---- validate everything before touching the allocator
    long long new_pages = 0, total_units = 0;
    std::vector<char> seen(c->cfg.max_slots, 0);
    for (int i = 0; i < count; i++) {
        const int slot = slots[i];
        if (slot < 0 || slot >= c->cfg.max_slots || !c->occupied[slot])
            return set_error(PD_INVALID_ARGUMENT, "append_batch: slot is not admitted");
        if (seen[slot]) return set_error(PD_INVALID_ARGUMENT, "append_batch: slot %d appears twice", slot);
        seen[slot] = 1;
        if (n[i] < 0) return set_error(PD_INVALID_ARGUMENT, "append_batch: negative token count");
        if (n[i] == 0) continue;
        if (!d_k[i] || !d_v[i] || (reinterpret_cast<uintptr_t>(d_k[i]) | reinterpret_cast<uintptr_t>(d_v[i])) % 16 != 0)
            return set_error(PD_INVALID_ARGUMENT, "append_batch: K/V sources must be non-null and 16-byte aligned");
        const int need = (c->seq_lens[slot] + n[i] + ps - 1) / ps;
        if (need > c->cfg.max_pages_per_slot) return set_error(PD_LENGTH_ERROR, "append: sequence exceeds max_pages_per_slot");
        new_pages += need - static_cast<int>(c->tables[slot].size());
        total_units += static_cast<long long>(n[i]) * c->cfg.num_kv_heads * 16;
    }
    if (total_units > 0x7fffffffLL) return set_error(PD_LENGTH_ERROR, "append_batch: too many tokens in one batch");
    if (new_pages > static_cast<long long>(c->free_pages.size())) return set_error(PD_OUT_OF_PAGES, "append: out of pages");

    // ---- packed buffer: jobs | (slot, index, page) table updates | (slot, length) updates
    struct TableUpdate { int slot, index, page; };
    struct LenUpdate { int slot, len; };
    auto round16 = [](size_t x) { return (x + 15) & ~static_cast<size_t>(15); };
    const size_t jobs_bytes = round16(sizeof(pdk::AppendJob) * count);
    const size_t tab_bytes  = round16(sizeof(TableUpdate) * static_cast<size_t>(new_pages));
    const size_t len_bytes  = round16(sizeof(LenUpdate) * count);
    const size_t total = jobs_bytes + tab_bytes + len_bytes;
    if (!c->batch_staged) PD_CUDA(cudaEventCreateWithFlags(&c->batch_staged, cudaEventDisableTiming));
    else PD_CUDA(cudaEventSynchronize(c->batch_staged));      // the previous batch still reads the staging buffer
    if (total > c->batch_cap) {
        PD_CUDA(cudaFreeHost(c->batch_staging));
        PD_CUDA(cudaFree(c->batch_device));
        c->batch_staging = c->batch_device = nullptr; c->batch_cap = 0;
        const size_t cap = std::max<size_t>(total * 2, 4096);
        PD_CUDA(cudaMallocHost(&c->batch_staging, cap));
        PD_CUDA(cudaMalloc(&c->batch_device, cap));
        c->batch_cap = cap;
    }
    char* h = static_cast<char*>(c->batch_staging);
    auto* jobs = reinterpret_cast<pdk::AppendJob*>(h);
    auto* tabs = reinterpret_cast<TableUpdate*>(h + jobs_bytes);
    auto* lens = reinterpret_cast<LenUpdate*>(h + jobs_bytes + tab_bytes);
    long long units = 0;
    int t = 0, live = 0;
    for (int i = 0; i < count; i++) {
        const int slot = slots[i];
        const int old_len = c->seq_lens[slot];
        const int have = static_cast<int>(c->tables[slot].size());
        const int need = (old_len + n[i] + ps - 1) / ps;
        for (int j = have; j < need; j++) {
            const int page = c->free_pages.back();
            c->free_pages.pop_back();
            c->tables[slot].push_back(page);
            tabs[t++] = TableUpdate{slot, j, page};
        }
        c->seq_lens[slot] = old_len + n[i];
        lens[i] = LenUpdate{slot, c->seq_lens[slot]};
        if (n[i] == 0) continue;
        jobs[live++] = pdk::AppendJob{static_cast<const __half*>(d_k[i]), static_cast<const __half*>(d_v[i]),
                                      c->d_block_table + static_cast<size_t>(slot) * c->cfg.max_pages_per_slot,
                                      old_len, n[i], static_cast<int>(units)};
        units += static_cast<long long>(n[i]) * c->cfg.num_kv_heads * 16;
    }
    PD_CUDA(cudaMemcpyAsync(c->batch_device, c->batch_staging, total, cudaMemcpyHostToDevice, stream));
    PD_CUDA(cudaEventRecord(c->batch_staged, stream));
    char* d = static_cast<char*>(c->batch_device);
    pdk::apply_updates_kernel<<<(t + count + 255) / 256, 256, 0, stream>>>(
        reinterpret_cast<const int*>(d + jobs_bytes), t, reinterpret_cast<const int*>(d + jobs_bytes + tab_bytes), count,
        c->d_block_table, c->cfg.max_pages_per_slot, c->d_seq_lens);
    PD_CUDA(cudaGetLastError());
    if (live > 0) {
        const int blocks = static_cast<int>(std::min<long long>((units + 255) / 256, 148 * 16));
        const bool fp8 = c->cfg.dtype == PD_FP8_E4M3;
        const float ik = fp8 ? 1.f / c->cfg.k_scale : 1.f, iv = fp8 ? 1.f / c->cfg.v_scale : 1.f;
        const pdk::AppendHeadScales hs{c->d_head_scales, c->d_head_scales ? c->d_head_scales + c->cfg.num_kv_heads : nullptr};
        if (fp8)
            pdk::append_batch_kernel<true><<<blocks, 256, 0, stream>>>(reinterpret_cast<const pdk::AppendJob*>(d), live,
                static_cast<int>(units), c->d_k, c->d_v, c->cfg.num_kv_heads, ps, ik, iv, hs);
        else
            pdk::append_batch_kernel<false><<<blocks, 256, 0, stream>>>(reinterpret_cast<const pdk::AppendJob*>(d), live,
                static_cast<int>(units), c->d_k, c->d_v, c->cfg.num_kv_heads, ps, ik, iv, hs);
        PD_CUDA(cudaGetLastError());
    }
    if (!c->batch_done) PD_CUDA(cudaEventCreateWithFlags(&c->batch_done, cudaEventDisableTiming));
    PD_CUDA(cudaEventRecord(c->batch_done, stream));
    c->batch_pending = true;
    return PD_OK;
}

int pd_cache_release(pd_cache* c, int slot) {
    if (!c || slot < 0 || slot >= c->cfg.max_slots || !c->occupied[slot])
        return set_error(PD_INVALID_ARGUMENT, "release: slot is not admitted");
    // A batched append is stream-ordered and may still be on its way (table updates, token scatter) on a
    // stream the memset below is not ordered with; the slot's pages must not go back to the free list, nor its
    // device-side length to zero, before that append has landed.
    if (c->batch_pending) {
        PD_CUDA(cudaEventSynchronize(c->batch_done));
        c->batch_pending = false;
    }
    for (int page : c->tables[slot]) c->free_pages.push_back(page);   // in table order
    c->tables[slot].clear();
    c->seq_lens[slot] = 0;
    c->occupied[slot] = 0;
    PD_CUDA(cudaMemset(c->d_seq_lens + slot, 0, sizeof(int)));
    return PD_OK;
}

void pd_cache_shuffle_free_pages(pd_cache* c, unsigned seed) {
    std::mt19937 rng(seed);
    std::shuffle(c->free_pages.begin(), c->free_pages.end(), rng);
}

int pd_cache_params(const pd_cache* c, pd_params* p) {
    if (!c || !p) return set_error(PD_INVALID_ARGUMENT, "params: null argument");
    std::memset(p, 0, sizeof *p);
    const bool fp8 = c->cfg.dtype == PD_FP8_E4M3;
    p->k_cache            = c->d_k;
    p->v_cache            = c->d_v;
    p->block_table        = c->d_block_table;
    p->seq_lens           = c->d_seq_lens;
    p->block_table_stride = c->cfg.max_pages_per_slot;
    p->num_kv_heads       = c->cfg.num_kv_heads;
    p->head_dim           = c->cfg.head_dim;
    p->page_size          = c->cfg.page_size;
    p->sm_scale           = 1.0f / std::sqrt(static_cast<float>(c->cfg.head_dim));
    p->k_scale            = fp8 ? c->cfg.k_scale : 1.0f;
    p->v_scale            = fp8 ? c->cfg.v_scale : 1.0f;
    return PD_OK;
}

int pd_cache_plan(pd_cache* c, const int* slots, int num_slots, int num_q_heads, int num_ctas, void* stream_) {
    if (!c || (num_slots > 0 && !slots)) return set_error(PD_INVALID_ARGUMENT, "plan: null argument");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::vector<int> lens(num_slots);
    for (int i = 0; i < num_slots; i++) {
        if (slots[i] < 0 || slots[i] >= c->cfg.max_slots || !c->occupied[slots[i]])
            return set_error(PD_INVALID_ARGUMENT, "plan: slot is not admitted");
        lens[i] = c->seq_lens[slots[i]];
    }
    pd_plan* plan = nullptr;
    if (int rc = pd_make_plan(c->cfg.dtype, lens.data(), num_slots, num_q_heads, c->cfg.num_kv_heads, c->cfg.head_dim,
                              num_ctas, &plan))
        return rc;
    if (int rc = validate_plan(*plan, lens.data(), num_slots, c->cfg.num_kv_heads)) { pd_plan_free(plan); return rc; }
    pd_plan_free(c->plan);
    c->plan = plan;
    if (int rc = pd_device_plan_upload(c->device_plan, plan, num_q_heads / c->cfg.num_kv_heads, c->cfg.head_dim, stream))
        return rc;
    if (static_cast<size_t>(num_slots) > c->slot_ids_cap) {
        PD_CUDA(cudaFree(c->d_slot_ids));
        c->d_slot_ids = nullptr; c->slot_ids_cap = 0;
        PD_CUDA(cudaMalloc(&c->d_slot_ids, sizeof(int) * num_slots));
        c->slot_ids_cap = num_slots;
    }
    if (num_slots)
        PD_CUDA(cudaMemcpyAsync(c->d_slot_ids, slots, sizeof(int) * num_slots, cudaMemcpyHostToDevice, stream));
    c->plan_batch = num_slots;
    c->plan_num_q_heads = num_q_heads;
    c->plan_identity = true;
    c->plan_on_device = false;
    for (int i = 0; i < num_slots; i++) c->plan_identity = c->plan_identity && slots[i] == i;
    return PD_OK;
}

int pd_cache_plan_device(pd_cache* c, const int* d_slot_ids, int batch, int num_q_heads, int num_ctas, void* stream) {
    if (!c) return set_error(PD_INVALID_ARGUMENT, "plan_device: null cache");
    if (batch < 0 || (!d_slot_ids && batch > c->cfg.max_slots))
        return set_error(PD_INVALID_ARGUMENT, "plan_device: batch exceeds the cache's slots");
    if (int rc = pd_device_plan_build(c->device_plan, c->cfg.dtype, c->d_seq_lens, d_slot_ids, batch, num_q_heads,
                                      c->cfg.num_kv_heads, c->cfg.head_dim, num_ctas, stream))
        return rc;
    pd_plan_free(c->plan);
    c->plan = nullptr;
    c->plan_batch = batch;
    c->plan_num_q_heads = num_q_heads;
    c->plan_identity = d_slot_ids == nullptr;
    c->plan_on_device = true;
    c->plan_slot_ids = d_slot_ids;
    return PD_OK;
}

int pd_cache_run(pd_cache* c, const void* d_q, void* d_out, void* stream) {
    if (!c) return set_error(PD_INVALID_ARGUMENT, "run: null cache");
    if (!c->plan && !c->plan_on_device) return set_error(PD_INVALID_ARGUMENT, "run: no plan; call plan() first");
    pd_params p;
    pd_cache_params(c, &p);
    p.q = d_q;
    p.out = d_out;
    p.slot_ids = c->plan_identity ? nullptr : c->plan_on_device ? c->plan_slot_ids : c->d_slot_ids;   // row i reads slot i: skip the indirection
    p.batch = c->plan_batch;
    p.num_q_heads = c->plan_num_q_heads;
    pd_device_plan_bind(c->device_plan, &p);
    return pd_paged_decode_scaled(c->cfg.dtype, &p, c->cfg.num_pages, c->d_head_scales,
                                  c->d_head_scales ? c->d_head_scales + c->cfg.num_kv_heads : nullptr, stream);
}

int pd_cache_describe_launch(const pd_cache* c, int* out) {
    if (!c || !out) return set_error(PD_INVALID_ARGUMENT, "describe_launch: null argument");
    if (!c->plan && !c->plan_on_device) return set_error(PD_INVALID_ARGUMENT, "describe_launch: no plan; call plan() first");
    pd_params p;
    pd_cache_params(c, &p);
    p.batch = c->plan_batch;
    p.num_q_heads = c->plan_num_q_heads;
    pd_device_plan_bind(c->device_plan, &p);
    return pd_describe_launch(c->cfg.dtype, &p, out);
}

int pd_cache_set_head_scales(pd_cache* c, const float* k_scales, const float* v_scales) {
    if (!c) return set_error(PD_INVALID_ARGUMENT, "set_head_scales: null cache");
    if (c->cfg.dtype != PD_FP8_E4M3) return set_error(PD_INVALID_ARGUMENT, "set_head_scales: only an fp8 cache is quantised");
    if ((k_scales == nullptr) != (v_scales == nullptr))
        return set_error(PD_INVALID_ARGUMENT, "set_head_scales: give both arrays or neither");
    for (int len : c->seq_lens)
        if (len > 0) return set_error(PD_INVALID_ARGUMENT, "set_head_scales: the cache already holds tokens quantised with the old scales");
    if (!k_scales) {
        PD_CUDA(cudaFree(c->d_head_scales));
        c->d_head_scales = nullptr;
        return PD_OK;
    }
    const int n = c->cfg.num_kv_heads;
    for (int h = 0; h < n; h++)
        if (!(k_scales[h] > 0.f) || !(v_scales[h] > 0.f)) return set_error(PD_INVALID_ARGUMENT, "set_head_scales: scales must be positive");
    if (!c->d_head_scales) PD_CUDA(cudaMalloc(&c->d_head_scales, sizeof(float) * 2 * n));
    PD_CUDA(cudaMemcpy(c->d_head_scales, k_scales, sizeof(float) * n, cudaMemcpyHostToDevice));
    PD_CUDA(cudaMemcpy(c->d_head_scales + n, v_scales, sizeof(float) * n, cudaMemcpyHostToDevice));
    return PD_OK;
}

int pd_cache_decode(pd_cache* c, const void* d_q, void* d_out, int batch, int num_q_heads, int num_ctas, void* stream) {
    if (!c || batch < 0) return set_error(PD_INVALID_ARGUMENT, "decode: bad argument");
    std::vector<int> slots(batch);
    std::iota(slots.begin(), slots.end(), 0);
    if (int rc = pd_cache_plan(c, slots.data(), batch, num_q_heads, num_ctas, stream)) return rc;
    return pd_cache_run(c, d_q, d_out, stream);
}

const pd_plan* pd_cache_last_plan(const pd_cache* c) { return c->plan; }
int pd_cache_seq_len(const pd_cache* c, int slot) { return c->seq_lens[slot]; }
int pd_cache_occupied(const pd_cache* c, int slot) { return c->occupied[slot]; }
int pd_cache_free_pages(const pd_cache* c) { return static_cast<int>(c->free_pages.size()); }
int pd_cache_max_seq_len(const pd_cache* c) { return *std::max_element(c->seq_lens.begin(), c->seq_lens.end()); }
size_t pd_cache_total_bytes(const pd_cache* c) { return pd_cache_bytes_per_page(&c->cfg) * c->cfg.num_pages; }
int pd_cache_config_of(const pd_cache* c, pd_cache_config* out) { *out = c->cfg; return PD_OK; }
int pd_cache_block_table(const pd_cache* c, int slot, int* out, int cap) {
    const auto& t = c->tables[slot];
    for (int i = 0; i < cap && i < static_cast<int>(t.size()); i++) out[i] = t[i];
    return static_cast<int>(t.size());
}
int pd_cache_free_list(const pd_cache* c, int* out, int cap) {
    for (int i = 0; i < cap && i < static_cast<int>(c->free_pages.size()); i++) out[i] = c->free_pages[i];
    return static_cast<int>(c->free_pages.size());
}

}  // extern "C"
