// C++ caller of the decode:: headers shipped with the engine (paged_attention_b200/include),
// written the way the reference's own hot-path tests call its library
// (tests/test_paged_decode.cu:50-151, 206-221): seeded inputs, PagedKVCache::admit/append/decode,
// an inline double-precision attention over the values as stored, exceptions on misuse.
// Plain main(), no test framework: prints one line per check and returns nonzero on failure.

#include "decode/paged_kv_cache.hpp"
#include "paged_decode_backend.hpp"
#include "attention_backend.hpp"
#include "attention_utils.hpp"
#include "kv_pool.hpp"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <random>
#include <stdexcept>
#include <vector>

using decode::KVDtype;
using decode::PagedKVCache;

namespace {

int g_failed = 0;
#define CHECK(cond)                                                                  \
    do {                                                                             \
        if (!(cond)) { std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); g_failed++; } \
    } while (0)

half* upload(const std::vector<half>& h) {
    half* d = nullptr;
    cudaMalloc(&d, sizeof(half) * h.size());
    cudaMemcpy(d, h.data(), sizeof(half) * h.size(), cudaMemcpyHostToDevice);
    return d;
}

// fp16 cache only here (the fp8 byte-level checks live in the Python suite against the oracle).
float run_case(int hq, int hkv, int page, const std::vector<int>& lens, int num_ctas, int chunk) {
    const int B = static_cast<int>(lens.size()), D = 128, G = hq / hkv;
    std::mt19937 rng(1234);
    std::normal_distribution<float> normal(0.f, 1.f);
    std::vector<std::vector<half>> K(B), V(B);
    int max_pages = 0, total_pages = 0;
    for (int b = 0; b < B; b++) {
        K[b].resize(static_cast<size_t>(lens[b]) * hkv * D);
        V[b].resize(K[b].size());
        for (auto& x : K[b]) x = __float2half(normal(rng));
        for (auto& x : V[b]) x = __float2half(normal(rng));
        const int pages = (lens[b] + page - 1) / page;
        max_pages = std::max(max_pages, pages);
        total_pages += pages;
    }
    std::vector<half> q(static_cast<size_t>(B) * hq * D);
    for (auto& x : q) x = __float2half(normal(rng));

    PagedKVCache::Config cfg{};
    cfg.num_pages = total_pages + 3; cfg.page_size = page; cfg.num_kv_heads = hkv; cfg.head_dim = D;
    cfg.max_slots = B; cfg.max_pages_per_slot = max_pages; cfg.dtype = KVDtype::FP16;
    PagedKVCache cache(cfg);
    std::vector<half*> dK(B), dV(B);
    for (int b = 0; b < B; b++) {
        CHECK(cache.admit() == b);
        dK[b] = upload(K[b]);
        dV[b] = upload(V[b]);
    }
    const size_t row = static_cast<size_t>(hkv) * D;
    std::vector<int> done(B, 0);
    for (bool progress = true; progress;) {
        progress = false;
        for (int b = 0; b < B; b++) {
            const int n = std::min(chunk > 0 ? chunk : lens[b], lens[b] - done[b]);
            if (n <= 0) continue;
            CHECK(cache.append(b, dK[b] + done[b] * row, dV[b] + done[b] * row, n));
            done[b] += n;
            progress = true;
        }
    }
    half* dq = upload(q);
    half* dout = nullptr;
    cudaMalloc(&dout, sizeof(half) * q.size());
    cache.decode(dq, dout, B, hq, num_ctas);
    cudaDeviceSynchronize();
    std::vector<half> out(q.size());
    cudaMemcpy(out.data(), dout, sizeof(half) * out.size(), cudaMemcpyDeviceToHost);
    CHECK(cache.last_plan().num_ctas > 0 && cache.last_plan().tile > 0);

    float max_err = 0.f;
    const double scale = 1.0 / std::sqrt(static_cast<double>(D));
    for (int b = 0; b < B; b++)
        for (int h = 0; h < hq; h++) {
            const int kv = h / G, T = lens[b];
            std::vector<double> s(T);
            double mx = -INFINITY, sum = 0;
            for (int t = 0; t < T; t++) {
                double dot = 0;
                for (int d = 0; d < D; d++)
                    dot += double(__half2float(q[(size_t(b) * hq + h) * D + d])) * __half2float(K[b][(size_t(t) * hkv + kv) * D + d]);
                s[t] = dot * scale;
                mx = std::max(mx, s[t]);
            }
            for (int t = 0; t < T; t++) { s[t] = std::exp(s[t] - mx); sum += s[t]; }
            for (int d = 0; d < D; d++) {
                double o = 0;
                for (int t = 0; t < T; t++) o += s[t] * __half2float(V[b][(size_t(t) * hkv + kv) * D + d]);
                const float got = __half2float(out[(size_t(b) * hq + h) * D + d]);
                CHECK(std::isfinite(got));
                max_err = std::max(max_err, static_cast<float>(std::fabs(got - o / sum)));
            }
        }
    for (int b = 0; b < B; b++) { cudaFree(dK[b]); cudaFree(dV[b]); }
    cudaFree(dq);
    cudaFree(dout);
    return max_err;
}

template<typename E, typename F>
bool throws(F&& f) {
    try { f(); } catch (const E&) { return true; } catch (...) { return false; }
    return false;
}

}  // namespace

int main() {
    constexpr float TOL = 2e-3f;
    struct { const char* name; int hq, hkv, page; std::vector<int> lens; int ctas, chunk; } cases[] = {
        {"single token", 32, 8, 16, {1}, 0, 0},
        {"mixed lengths", 32, 8, 16, {1, 15, 16, 17, 129, 1000, 4099}, 0, 0},
        {"gqa group 8", 8, 1, 16, {777}, 0, 0},
        {"page size 8", 16, 4, 8, {300, 2500}, 0, 0},
        {"forced 7 ctas", 32, 8, 16, {5000, 90, 1, 700}, 7, 0},
        {"forced 1000 ctas", 32, 8, 16, {5000, 90, 1, 700}, 1000, 0},
        {"scattered pages", 32, 8, 16, {400, 333, 612}, 0, 5},
    };
    for (auto& c : cases) {
        const float err = run_case(c.hq, c.hkv, c.page, c.lens, c.ctas, c.chunk);
        std::printf("%-18s max abs err %.3e %s\n", c.name, err, err < TOL ? "ok" : "FAIL");
        CHECK(err < TOL);
    }

    // OutOfPagesRejectsAppend (tests/test_paged_decode.cu:206-221 of the reference)
    {
        PagedKVCache::Config cfg{};
        cfg.num_pages = 2; cfg.page_size = 16; cfg.num_kv_heads = 1; cfg.head_dim = 128;
        cfg.max_slots = 2; cfg.max_pages_per_slot = 4;
        PagedKVCache cache(cfg);
        half* d = upload(std::vector<half>(64 * 64, __float2half(0.f)));
        const int s = cache.admit();
        CHECK(cache.append(s, d, d, 32));
        CHECK(cache.free_pages() == 0);
        CHECK(!cache.append(s, d, d, 1));
        CHECK(cache.seq_len(s) == 32);
        CHECK(cache.block_table(s) == std::vector<int>({0, 1}));
        CHECK(throws<std::length_error>([&] { cache.append(s, d, d, 64); }));
        CHECK(throws<std::invalid_argument>([&] { cache.append(1, d, d, 1); }));
        CHECK(throws<std::invalid_argument>([&] { cache.plan({1}, 4); }));
        cache.release(s);
        CHECK(cache.free_pages() == 2);
        CHECK(throws<std::invalid_argument>([&] { cache.release(s); }));
        cudaFree(d);
    }
    // argument errors of the free functions
    CHECK(throws<std::invalid_argument>([] { decode::make_plan(KVDtype::FP16, {5, 0}, 8, 8, 128, 4); }));
    CHECK(throws<std::invalid_argument>([] { decode::make_plan(KVDtype::FP16, {5}, 7, 4, 128, 4); }));
    CHECK(throws<std::invalid_argument>([] { decode::tile_tokens(KVDtype::FP16, 64, 4); }));
    CHECK(throws<std::invalid_argument>([] { decode::tile_tokens(KVDtype::FP8_E4M3, 128, 3); }));
    CHECK(throws<std::invalid_argument>([] {
        PagedKVCache::Config cfg{};
        cfg.num_pages = 2; cfg.page_size = 16; cfg.num_kv_heads = 1; cfg.head_dim = 64; cfg.max_slots = 1; cfg.max_pages_per_slot = 1;
        PagedKVCache c(cfg);
    }));
    CHECK(decode::default_ctas(KVDtype::FP16, 128, 4) > 0 && decode::wave_ctas(KVDtype::FP8_E4M3, 128, 8) > 0);

    // driving the kernel directly with DecodePlan / DevicePlan / DecodeParams, as the reference's
    // torch binding does (bindings/torch_decode.cu:21-59)
    {
        const int B = 2, hq = 8, hkv = 2, D = 128, page = 16, L = 300;
        PagedKVCache::Config cfg{};
        cfg.num_pages = 2 * 19; cfg.page_size = page; cfg.num_kv_heads = hkv; cfg.head_dim = D; cfg.max_slots = B; cfg.max_pages_per_slot = 19;
        PagedKVCache cache(cfg);
        std::vector<half> kv(static_cast<size_t>(L) * hkv * D, __float2half(0.25f));
        half* d = upload(kv);
        for (int b = 0; b < B; b++) CHECK(cache.append(cache.admit(), d, d, L));
        std::vector<half> q(static_cast<size_t>(B) * hq * D, __float2half(0.5f));
        half* dq = upload(q);
        half* dout = nullptr;
        cudaMalloc(&dout, sizeof(half) * q.size());
        decode::DecodePlan plan = decode::make_plan(KVDtype::FP16, {L, L}, hq, hkv, D, 9);
        decode::DevicePlan dp;
        dp.upload(plan, hq / hkv, D);
        decode::DecodeParams p = cache.params();
        p.q = dq; p.out = dout; p.batch = B; p.num_q_heads = hq;
        dp.bind(p);
        decode::paged_decode(KVDtype::FP16, p);
        cudaDeviceSynchronize();
        std::vector<half> out(q.size());
        cudaMemcpy(out.data(), dout, sizeof(half) * out.size(), cudaMemcpyDeviceToHost);
        for (half x : out) CHECK(std::fabs(__half2float(x) - 0.25f) < 1e-3f);   // all values equal -> output is that value
        cudaFree(d); cudaFree(dq); cudaFree(dout);
    }
    // A caller that asks for a small grid (to share the GPU with another stream, or to sweep CTA counts) gets
    // no more CTAs than it asked for, also where the library swaps in its own schedule of the same step
    // (fp16 layers with 8 kv heads run a row-wise schedule on a grid of their own).
    {
        const int B = 3, hq = 32, hkv = 8, D = 128, page = 16, L = 2000;
        PagedKVCache::Config cfg{};
        cfg.num_pages = B * 125; cfg.page_size = page; cfg.num_kv_heads = hkv; cfg.head_dim = D; cfg.max_slots = B; cfg.max_pages_per_slot = 125;
        PagedKVCache cache(cfg);
        std::vector<half> kv(static_cast<size_t>(L) * hkv * D, __float2half(-0.75f));
        half* d = upload(kv);
        for (int b = 0; b < B; b++) CHECK(cache.append(cache.admit(), d, d, L));
        std::vector<half> q(static_cast<size_t>(B) * hq * D, __float2half(0.125f));
        half* dq = upload(q);
        half* dout = nullptr;
        cudaMalloc(&dout, sizeof(half) * q.size());
        for (int asked : {9, 40}) {
            decode::DecodePlan plan = decode::make_plan(KVDtype::FP16, {L, L, L}, hq, hkv, D, asked);
            decode::DevicePlan dp;
            dp.upload(plan, hq / hkv, D);
            decode::DecodeParams p = cache.params();
            p.q = dq; p.out = dout; p.batch = B; p.num_q_heads = hq;
            dp.bind(p);
            int info[8] = {};
            CHECK(pd_describe_launch(PD_FP16, decode::as_pd(p), info) == PD_OK);
            CHECK(info[1] > 0 && info[1] <= asked);
            decode::paged_decode(KVDtype::FP16, p);
            cudaDeviceSynchronize();
            std::vector<half> out(q.size());
            cudaMemcpy(out.data(), dout, sizeof(half) * out.size(), cudaMemcpyDeviceToHost);
            for (half x : out) CHECK(std::fabs(__half2float(x) + 0.75f) < 1e-3f);
        }
        cudaFree(d); cudaFree(dq); cudaFree(dout);
    }
    // The legacy interfaces with the engine behind them: backend-vs-CPU parity on seeded uniform(-1,1)
    // inputs (tests/test_helpers.hpp:10-19 of the reference, at fp16-storage tolerance) and the pool
    // semantics its pool tests pin (tests/test_paged_pool.cpp:25-77,135-156; tests/test_contiguous_pool.cpp:34-65).
    {
        PagedDecodeAttention backend;
        AttentionBackend& b = backend;
        for (int T : {1, 17, 1000, 5000}) {
            const AttnInputs in = make_attention_inputs(128, T, 7 + T);
            std::vector<float> got(128), want(128);
            b.run(in.q.data(), in.K.data(), in.V.data(), got.data(), T, 128);
            std::vector<double> s(T);
            double mx = -INFINITY, sum = 0;
            for (int t = 0; t < T; t++) {
                double dot = 0;
                for (int d = 0; d < 128; d++) dot += double(in.q[d]) * in.K[size_t(t) * 128 + d];
                s[t] = dot / std::sqrt(128.0);
                mx = std::max(mx, s[t]);
            }
            for (int t = 0; t < T; t++) { s[t] = std::exp(s[t] - mx); sum += s[t]; }
            for (int d = 0; d < 128; d++) {
                double o = 0;
                for (int t = 0; t < T; t++) o += s[t] * in.V[size_t(t) * 128 + d];
                want[d] = float(o / sum);
            }
            const float err = max_abs_diff(got.data(), want.data(), 128);
            std::printf("legacy backend T=%-5d max abs err %.3e %s\n", T, err, err < TOL ? "ok" : "FAIL");
            CHECK(err < TOL);
        }
        CHECK(throws<std::invalid_argument>([&] { float x[7] = {}; b.run(x, x, x, x, 1, 7); }));   // head_dim 128 only

        const int d = 128, T = 32;
        std::vector<float> K(size_t(T) * d, 0.f), V(size_t(T) * d, 0.f);
        {   // admit / release / slot reuse
            PagedDecodePool pool(8, 4, 4, d);
            KVPool& p = pool;
            const int s0 = p.admit(K.data(), V.data(), T), s1 = p.admit(K.data(), V.data(), T);
            CHECK(s0 >= 0 && s1 >= 0 && s0 != s1);
            CHECK(p.is_occupied(s0) && p.actual_len(s0) == T);
            const int free_before = pool.free_page_count();
            p.release(s0);
            CHECK(!p.is_occupied(s0) && pool.free_page_count() > free_before);
            CHECK(p.admit(K.data(), V.data(), T) == s0);
        }
        {   // -1 when the pages run out, pages recycled after release
            PagedDecodePool pool(2, 4, 4, d);
            CHECK(pool.admit(K.data(), V.data(), 16) >= 0);
            const int s1 = pool.admit(K.data(), V.data(), 16);
            CHECK(s1 >= 0);
            CHECK(pool.admit(K.data(), V.data(), 16) == -1);
            CHECK(pool.free_page_count() == 0);
            pool.release(s1);
            CHECK(pool.free_page_count() == 1);
            CHECK(pool.admit(K.data(), V.data(), 16) >= 0);
        }
        {   // appending across a page boundary takes one more page: 3 -> 3 -> 2
            PagedDecodePool pool(4, 2, 4, d);
            const int s = pool.admit(K.data(), V.data(), 15);
            CHECK(pool.free_page_count() == 3);
            pool.append_token(s, 15, K.data(), V.data());
            CHECK(pool.free_page_count() == 3 && pool.actual_len(s) == 16);
            pool.append_token(s, 16, K.data(), V.data());
            CHECK(pool.free_page_count() == 2 && pool.actual_len(s) == 17);
            std::vector<float> q(d, 0.5f), out(d, -1.f);
            pool.decode(s, q.data(), out.data());
            for (float x : out) CHECK(x == 0.f);   // zero values give a zero output
        }
    }
    std::printf(g_failed ? "FAILED (%d checks)\n" : "all checks passed\n", g_failed);
    return g_failed ? 1 : 0;
}
