// C entry points around the UNMODIFIED reference sources, which are compiled
// where they lie (see oracle/Makefile: REF=<checkout of emaanh/paged-attention>).
// TEST INFRASTRUCTURE ONLY: the result, oracle/_ref/libpd_ref.so, pins the CPU
// oracle, generates the golden vectors under tests/golden/, serves as the
// reference arm of the benchmark and lets GPU parity tests run the reference's
// own kernels next to the engine on identical bytes.  The shipped library never
// loads it.
//
// Everything below is glue; the algorithms come from the reference's
//   src/attention/cpu/attention.cpp   (cpu_attention)
//   src/decode/decode.cu              (make_plan, tile_tokens, DevicePlan, paged_decode)
//   src/decode/paged_kv_cache.cu      (PagedKVCache)

#include "decode/paged_kv_cache.hpp"
#include "cpu/attention.hpp"

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <exception>
#include <stdexcept>
#include <string>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

using decode::KVDtype;
using decode::PagedKVCache;

namespace {
thread_local std::string g_err;
KVDtype to_dtype(int d) { return d == 0 ? KVDtype::FP16 : KVDtype::FP8_E4M3; }

template<typename F>
int guarded(F&& f) {
    try { f(); return 0; }
    catch (const std::invalid_argument& e) { g_err = e.what(); return 1; }
    catch (const std::length_error& e) { g_err = e.what(); return 2; }
    catch (const std::exception& e) { g_err = e.what(); return 3; }
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// ---- scalar conversions through the CUDA headers' host paths --------------------
uint8_t ref_e4m3_from_float(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
float ref_e4m3_to_float(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(__half(h));
}
float ref_half_to_float(uint16_t bits) {
    __half_raw r; r.x = bits;
    return __half2float(__half(r));
}
uint16_t ref_float_to_half(float f) {
    const __half h = __float2half(f);
    return static_cast<__half_raw>(h).x;
}
// The storage round trip of the reference's decode test (tests/test_paged_decode.cu:28-31).
void ref_quantize_e4m3(const uint16_t* half_in, long n, float scale, uint8_t* out) {
    const float inv = 1.f / scale;
    for (long i = 0; i < n; i++)
        out[i] = ref_e4m3_from_float(ref_half_to_float(half_in[i]) * inv);
}

// ---- CPU attention ---------------------------------------------------------------
void ref_cpu_attention(const float* q, const float* K, const float* V, float* out, int T, int d) {
    cpu_attention(q, K, V, out, T, d);
}

// Drives cpu_attention over a paged multi-head cache: gathers each (row, kv head)
// into contiguous fp32 [T][d], then calls cpu_attention for each query head of the
// group.  `rows` lists the batch rows to compute (a bounded sample of the batch).
// Returns the wall time of the attention calls alone in *attn_seconds (gather
// excluded), using `threads` OpenMP threads over (row, q head) pairs.
int ref_paged_cpu_decode(int dtype, const uint16_t* q, const void* k_cache, const void* v_cache,
                         const int* block_table, int block_table_stride, const int* seq_lens,
                         const int* rows, int num_rows, int num_q_heads, int num_kv_heads,
                         int head_dim, int page_size, float k_scale, float v_scale,
                         float* out /* [num_rows][hq][d] */, int threads, double* attn_seconds) {
    const int D = head_dim, group = num_q_heads / num_kv_heads;
    std::vector<std::vector<float>> Ks(static_cast<size_t>(num_rows) * num_kv_heads), Vs(Ks.size());
    std::vector<float> qf(static_cast<size_t>(num_rows) * num_q_heads * D);
#if defined(_OPENMP)
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
    for (int item = 0; item < num_rows * num_kv_heads; item++) {
        const int r = item / num_kv_heads, h = item % num_kv_heads, b = rows[r];
        const int T = seq_lens[b];
        const int* bt = block_table + static_cast<size_t>(b) * block_table_stride;
        auto& K = Ks[item]; auto& V = Vs[item];
        K.resize(static_cast<size_t>(T) * D); V.resize(K.size());
        for (int t = 0; t < T; t++) {
            const size_t base = ((static_cast<size_t>(bt[t / page_size]) * num_kv_heads + h) * page_size + t % page_size) * D;
            for (int d = 0; d < D; d++) {
                if (dtype == 0) {
                    K[static_cast<size_t>(t) * D + d] = ref_half_to_float(static_cast<const uint16_t*>(k_cache)[base + d]);
                    V[static_cast<size_t>(t) * D + d] = ref_half_to_float(static_cast<const uint16_t*>(v_cache)[base + d]);
                } else {
                    K[static_cast<size_t>(t) * D + d] = ref_e4m3_to_float(static_cast<const uint8_t*>(k_cache)[base + d]) * k_scale;
                    V[static_cast<size_t>(t) * D + d] = ref_e4m3_to_float(static_cast<const uint8_t*>(v_cache)[base + d]) * v_scale;
                }
            }
        }
        for (int g = 0; g < group; g++)
            for (int d = 0; d < D; d++)
                qf[(static_cast<size_t>(r) * num_q_heads + h * group + g) * D + d] =
                    ref_half_to_float(q[(static_cast<size_t>(b) * num_q_heads + h * group + g) * D + d]);
    }
    const auto t0 = std::chrono::steady_clock::now();
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < num_rows * num_q_heads; i++) {
        const int r = i / num_q_heads, hq = i % num_q_heads, h = hq / group, b = rows[r];
        cpu_attention(&qf[static_cast<size_t>(i) * D], Ks[r * num_kv_heads + h].data(),
                      Vs[r * num_kv_heads + h].data(), out + static_cast<size_t>(i) * D, seq_lens[b], D);
    }
    const auto t1 = std::chrono::steady_clock::now();
    if (attn_seconds) *attn_seconds = std::chrono::duration<double>(t1 - t0).count();
    return 0;
}

int ref_omp_max_threads() {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---- planner -----------------------------------------------------------------------
// tile_tokens makes no CUDA call; make_plan makes none when num_ctas > 0.
int ref_tile_tokens(int dtype, int head_dim, int group, int* out) {
    return guarded([&] { *out = decode::tile_tokens(to_dtype(dtype), head_dim, group); });
}
int ref_default_ctas(int dtype, int head_dim, int group, int* out) {
    return guarded([&] { *out = decode::default_ctas(to_dtype(dtype), head_dim, group); });
}
int ref_make_plan(int dtype, const int* seq_lens, int batch, int hq, int hkv, int head_dim, int num_ctas,
                  int* out_num_ctas, int* out_tile, int* segments, int seg_cap, int* out_num_segments,
                  int* cta_seg_begin, int cta_cap, int* item_seg_begin) {
    return guarded([&] {
        const std::vector<int> lens(seq_lens, seq_lens + batch);
        const decode::DecodePlan p = decode::make_plan(to_dtype(dtype), lens, hq, hkv, head_dim, num_ctas);
        if (static_cast<int>(p.segments.size()) > seg_cap || static_cast<int>(p.cta_seg_begin.size()) > cta_cap)
            throw std::runtime_error("ref_make_plan: output capacity too small");
        *out_num_ctas = p.num_ctas;
        *out_tile = p.tile;
        *out_num_segments = static_cast<int>(p.segments.size());
        std::memcpy(segments, p.segments.data(), sizeof(int4) * p.segments.size());
        std::memcpy(cta_seg_begin, p.cta_seg_begin.data(), sizeof(int) * p.cta_seg_begin.size());
        std::memcpy(item_seg_begin, p.item_seg_begin.data(), sizeof(int) * p.item_seg_begin.size());
    });
}

// ---- the reference's PagedKVCache (needs a GPU) ---------------------------------------
void* ref_cache_create(int num_pages, int page_size, int num_kv_heads, int head_dim, int max_slots,
                       int max_pages_per_slot, int dtype, float k_scale, float v_scale) {
    PagedKVCache* c = nullptr;
    guarded([&] {
        PagedKVCache::Config cfg{};
        cfg.num_pages = num_pages; cfg.page_size = page_size; cfg.num_kv_heads = num_kv_heads;
        cfg.head_dim = head_dim; cfg.max_slots = max_slots; cfg.max_pages_per_slot = max_pages_per_slot;
        cfg.dtype = to_dtype(dtype); cfg.k_scale = k_scale; cfg.v_scale = v_scale;
        c = new PagedKVCache(cfg);
    });
    return c;
}
void ref_cache_destroy(void* c) { delete static_cast<PagedKVCache*>(c); }
int ref_cache_admit(void* c) { return static_cast<PagedKVCache*>(c)->admit(); }
// 1 appended, 0 out of pages, -1 invalid_argument, -2 length_error
int ref_cache_append(void* c, int slot, const void* d_k, const void* d_v, int n) {
    bool ok = false;
    const int rc = guarded([&] {
        ok = static_cast<PagedKVCache*>(c)->append(slot, static_cast<const half*>(d_k), static_cast<const half*>(d_v), n);
    });
    return rc == 0 ? (ok ? 1 : 0) : -rc;
}
int ref_cache_release(void* c, int slot) { return -guarded([&] { static_cast<PagedKVCache*>(c)->release(slot); }); }
void ref_cache_shuffle(void* c, unsigned seed) { static_cast<PagedKVCache*>(c)->shuffle_free_pages(seed); }
int ref_cache_free_pages(void* c) { return static_cast<PagedKVCache*>(c)->free_pages(); }
int ref_cache_seq_len(void* c, int slot) { return static_cast<PagedKVCache*>(c)->seq_len(slot); }
int ref_cache_table(void* c, int slot, int* out, int cap) {
    const auto& t = static_cast<PagedKVCache*>(c)->block_table(slot);
    for (int i = 0; i < cap && i < static_cast<int>(t.size()); i++) out[i] = t[i];
    return static_cast<int>(t.size());
}
void ref_cache_pointers(void* c, const void** k, const void** v, const int** block_table, const int** seq_lens) {
    const decode::DecodeParams p = static_cast<PagedKVCache*>(c)->params();
    *k = p.k_cache; *v = p.v_cache; *block_table = p.block_table; *seq_lens = p.seq_lens;
}
int ref_cache_plan(void* c, const int* slots, int n, int hq, int num_ctas) {
    return guarded([&] { static_cast<PagedKVCache*>(c)->plan(std::vector<int>(slots, slots + n), hq, num_ctas); });
}
int ref_cache_run(void* c, const void* d_q, void* d_out) {
    return guarded([&] { static_cast<PagedKVCache*>(c)->run(static_cast<const half*>(d_q), static_cast<half*>(d_out)); });
}
int ref_cache_decode(void* c, const void* d_q, void* d_out, int batch, int hq, int num_ctas) {
    return guarded([&] {
        static_cast<PagedKVCache*>(c)->decode(static_cast<const half*>(d_q), static_cast<half*>(d_out), batch, hq, num_ctas);
    });
}
void ref_cache_plan_info(void* c, int* num_ctas, int* tile, int* num_segments) {
    const auto& p = static_cast<PagedKVCache*>(c)->last_plan();
    *num_ctas = p.num_ctas; *tile = p.tile; *num_segments = static_cast<int>(p.segments.size());
}

// The reference's decode on caller-owned buffers, as its torch binding drives it
// (bindings/torch_decode.cu:21-59): plan from host lengths, then paged_decode.
struct RefDecoder {
    decode::DecodePlan plan;
    decode::DevicePlan device_plan;
};
void* ref_decoder_create() { return new RefDecoder(); }
void ref_decoder_destroy(void* d) { delete static_cast<RefDecoder*>(d); }
int ref_decoder_plan(void* d, int dtype, const int* seq_lens_host, int batch, int hq, int hkv, int head_dim, int num_ctas) {
    return guarded([&] {
        auto* r = static_cast<RefDecoder*>(d);
        r->plan = decode::make_plan(to_dtype(dtype), std::vector<int>(seq_lens_host, seq_lens_host + batch), hq, hkv, head_dim, num_ctas);
        r->device_plan.upload(r->plan, hq / hkv, head_dim, 0);
    });
}
int ref_decoder_run(void* d, int dtype, const void* q, void* out, const void* k_cache, const void* v_cache,
                    const int* block_table, int block_table_stride, const int* seq_lens_dev, int batch,
                    int hq, int hkv, int head_dim, int page_size, float k_scale, float v_scale, void* stream) {
    return guarded([&] {
        auto* r = static_cast<RefDecoder*>(d);
        decode::DecodeParams p{};
        p.q = static_cast<const half*>(q); p.out = static_cast<half*>(out);
        p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.seq_lens = seq_lens_dev;
        p.slot_ids = nullptr; p.block_table_stride = block_table_stride;
        p.batch = batch; p.num_q_heads = hq; p.num_kv_heads = hkv; p.head_dim = head_dim; p.page_size = page_size;
        p.sm_scale = 1.0f / std::sqrt(static_cast<float>(head_dim)); p.k_scale = k_scale; p.v_scale = v_scale;
        r->device_plan.bind(p);
        decode::paged_decode(to_dtype(dtype), p, static_cast<cudaStream_t>(stream));
    });
}
void ref_decoder_info(void* d, int* num_ctas, int* num_segments) {
    auto* r = static_cast<RefDecoder*>(d);
    *num_ctas = r->plan.num_ctas; *num_segments = static_cast<int>(r->plan.segments.size());
}

}  // extern "C"
