// CPU oracle for the paged split-KV decode path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain scalar C++, the algorithms of the reference
// project (emaanh/paged-attention) that the CUDA engine must reproduce.  It is
// the checker used by the test-suite, by the smoke test and by the benchmark's
// CPU-baseline leg.  Nothing in the shipped library links, loads or calls it.
//
// Parity status: PINNED.  Every function here is checked (tests/test_oracle_pin.py)
// against outputs of the reference's own code compiled from its sources
// (oracle/_ref, see oracle/Makefile) and against the known answers stored in
// tests/golden/ that were generated from that build.
//
// Each function cites the reference file:line it follows.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <random>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

// ---- storage types ---------------------------------------------------------

// IEEE binary16 -> binary32.
float half_to_float(uint16_t h) {
    const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
    const uint32_t exp  = (h >> 10) & 0x1fu;
    const uint32_t man  = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {   // subnormal: value = man * 2^-24
            const float v = std::ldexp(static_cast<float>(man), -24);
            std::memcpy(&bits, &v, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// binary32 -> binary16, round to nearest even (what __float2half does).
uint16_t float_to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint16_t sign = static_cast<uint16_t>((x >> 16) & 0x8000u);
    const uint32_t ax   = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u);
    const double a = std::fabs(static_cast<double>(f));
    if (a >= 65520.0) return sign | 0x7c00u;
    if (a < std::ldexp(1.0, -14)) {   // subnormal half: units of 2^-24
        return sign | static_cast<uint16_t>(std::nearbyint(std::ldexp(a, 24)));
    }
    int e;
    const double m = std::frexp(a, &e);   // a = m * 2^e, m in [0.5, 1)
    int q = static_cast<int>(std::nearbyint(std::ldexp(m, 11)));   // 1024..2048
    int ee = e - 1;
    if (q == 2048) { q = 1024; ee++; }
    return sign | static_cast<uint16_t>(((ee + 15) << 10) | (q - 1024));
}

// float -> FP8 E4M3 byte: round to nearest even, saturate to +-448, NaN -> 0x7f.
// Follows __nv_fp8_e4m3(float) as used by the append path's quantize<>
// (src/decode/paged_kv_cache.cu:20-22).
uint8_t e4m3_from_float(float x) {
    if (std::isnan(x)) return 0x7f;
    const uint8_t sign = std::signbit(x) ? 0x80 : 0x00;
    const double a = std::fabs(static_cast<double>(x));
    if (a >= 448.0) return sign | 0x7e;
    if (a < std::ldexp(1.0, -6)) {   // subnormal: units of 2^-9 (8 -> smallest normal)
        return sign | static_cast<uint8_t>(std::nearbyint(std::ldexp(a, 9)));
    }
    int e;
    const double m = std::frexp(a, &e);   // m in [0.5, 1)
    int q = static_cast<int>(std::nearbyint(std::ldexp(m, 4)));   // 8..16
    int ee = e - 1;
    if (q == 16) { q = 8; ee++; }
    int bits = ((ee + 7) << 3) | (q - 8);
    if (bits > 0x7e) bits = 0x7e;
    return sign | static_cast<uint8_t>(bits);
}

float e4m3_to_float(uint8_t b) {
    const int e = (b >> 3) & 0xf, m = b & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = std::ldexp(static_cast<float>(m), -9);
    else v = std::ldexp(1.0f + m / 8.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

// Allocator model: the host half of PagedKVCache
// (src/decode/paged_kv_cache.cu:43-82 ctor, 84-93 admit, 95-112 append,
//  138-146 release, 148-151 shuffle).
struct Pool {
    int num_pages, page_size, max_slots, max_pages_per_slot;
    std::vector<int>              free_pages;
    std::vector<std::vector<int>> tables;
    std::vector<int>              seq_lens;
    std::vector<char>             occupied;
};

}  // namespace

extern "C" {

float    orc_half_to_float(uint16_t h)  { return half_to_float(h); }
uint16_t orc_float_to_half(float f)     { return float_to_half(f); }
uint8_t  orc_e4m3_from_float(float x)   { return e4m3_from_float(x); }
float    orc_e4m3_to_float(uint8_t b)   { return e4m3_to_float(b); }

// What one cache element holds after an append: the kernel multiplies by the
// reciprocal of the scale (src/decode/paged_kv_cache.cu:20-22,130), it does not divide.
void orc_quantize_e4m3(const uint16_t* half_in, long n, float scale, uint8_t* out) {
    const float inv = 1.f / scale;
    for (long i = 0; i < n; i++) out[i] = e4m3_from_float(half_to_float(half_in[i]) * inv);
}

// ---- planner: decode::make_plan (src/decode/decode.cu:65-108) -----------------
// `tile` and `num_ctas` are inputs here (the reference derives them from the
// kernel configuration and the device).  segments is int[4*seg_cap] of
// (row, kv head, token begin, token end).  Returns 0 ok, 1 invalid argument,
// 2 capacity too small.
int orc_make_plan(int tile, int num_ctas, const int* seq_lens, int batch, int num_q_heads,
                  int num_kv_heads, int* out_num_ctas, int* segments, int seg_cap,
                  int* out_num_segments, int* cta_seg_begin, int cta_cap, int* item_seg_begin) {
    if (num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0 || tile <= 0 || num_ctas <= 0) return 1;
    const int items = batch * num_kv_heads;
    std::vector<int> item_tiles(items);
    long total = 0;
    for (int b = 0; b < batch; b++) {
        if (seq_lens[b] <= 0) return 1;
        for (int h = 0; h < num_kv_heads; h++) {
            item_tiles[b * num_kv_heads + h] = (seq_lens[b] + tile - 1) / tile;
            total += item_tiles[b * num_kv_heads + h];
        }
    }
    for (int i = 0; i <= items; i++) item_seg_begin[i] = 0;
    if (total == 0) { *out_num_ctas = 0; *out_num_segments = 0; cta_seg_begin[0] = 0; return 0; }
    const long per = (total + num_ctas - 1) / num_ctas;
    const int ctas = static_cast<int>((total + per - 1) / per);
    if (ctas + 1 > cta_cap) return 2;
    int nseg = 0, item = 0, in_item = 0;
    for (int c = 0; c < ctas; c++) {
        cta_seg_begin[c] = nseg;
        long left = per;
        while (left > 0 && item < items) {
            const int take = static_cast<int>(std::min<long>(left, item_tiles[item] - in_item));
            const int b = item / num_kv_heads, h = item % num_kv_heads;
            if (nseg >= seg_cap) return 2;
            segments[4 * nseg + 0] = b;
            segments[4 * nseg + 1] = h;
            segments[4 * nseg + 2] = in_item * tile;
            segments[4 * nseg + 3] = std::min((in_item + take) * tile, seq_lens[b]);
            nseg++;
            item_seg_begin[item + 1]++;
            in_item += take;
            left -= take;
            if (in_item == item_tiles[item]) { item++; in_item = 0; }
        }
    }
    cta_seg_begin[ctas] = nseg;
    for (int i = 0; i < items; i++) item_seg_begin[i + 1] += item_seg_begin[i];
    *out_num_ctas = ctas;
    *out_num_segments = nseg;
    return 0;
}

// ---- allocator ------------------------------------------------------------------

void* orc_pool_create(int num_pages, int page_size, int max_slots, int max_pages_per_slot) {
    if (num_pages <= 0 || page_size <= 0 || max_slots <= 0 || max_pages_per_slot <= 0) return nullptr;
    Pool* p = new Pool{num_pages, page_size, max_slots, max_pages_per_slot, {}, {}, {}, {}};
    p->tables.resize(max_slots);
    p->seq_lens.assign(max_slots, 0);
    p->occupied.assign(max_slots, 0);
    p->free_pages.resize(num_pages);
    // popped from the back, so page 0 is handed out first (:71-73)
    std::iota(p->free_pages.rbegin(), p->free_pages.rend(), 0);
    return p;
}
void orc_pool_destroy(void* h) { delete static_cast<Pool*>(h); }

int orc_pool_admit(void* h) {
    Pool* p = static_cast<Pool*>(h);
    for (int s = 0; s < p->max_slots; s++)
        if (!p->occupied[s]) { p->occupied[s] = 1; p->seq_lens[s] = 0; return s; }
    return -1;
}

// 1 = appended, 0 = out of pages (nothing changed), -1 = slot not admitted
// (std::invalid_argument in the reference), -2 = longer than max_pages_per_slot
// (std::length_error).  On success new_pages_begin receives the index of the
// first newly mapped block-table entry.
int orc_pool_append(void* h, int slot, int n, int* new_pages_begin) {
    Pool* p = static_cast<Pool*>(h);
    if (slot < 0 || slot >= p->max_slots || !p->occupied[slot]) return -1;
    const int have = static_cast<int>(p->tables[slot].size());
    if (new_pages_begin) *new_pages_begin = have;
    if (n <= 0) return 1;
    const int new_len = p->seq_lens[slot] + n;
    const int need = (new_len + p->page_size - 1) / p->page_size;
    if (need > p->max_pages_per_slot) return -2;
    if (need - have > static_cast<int>(p->free_pages.size())) return 0;
    for (int i = have; i < need; i++) {
        p->tables[slot].push_back(p->free_pages.back());
        p->free_pages.pop_back();
    }
    p->seq_lens[slot] = new_len;
    return 1;
}

int orc_pool_release(void* h, int slot) {
    Pool* p = static_cast<Pool*>(h);
    if (slot < 0 || slot >= p->max_slots || !p->occupied[slot]) return -1;
    for (int page : p->tables[slot]) p->free_pages.push_back(page);   // table order (:141)
    p->tables[slot].clear();
    p->seq_lens[slot] = 0;
    p->occupied[slot] = 0;
    return 0;
}

void orc_pool_shuffle(void* h, unsigned seed) {
    Pool* p = static_cast<Pool*>(h);
    std::mt19937 rng(seed);
    std::shuffle(p->free_pages.begin(), p->free_pages.end(), rng);
}

int orc_pool_free_pages(void* h) { return static_cast<int>(static_cast<Pool*>(h)->free_pages.size()); }
int orc_pool_seq_len(void* h, int slot) { return static_cast<Pool*>(h)->seq_lens[slot]; }
int orc_pool_occupied(void* h, int slot) { return static_cast<Pool*>(h)->occupied[slot]; }
int orc_pool_table(void* h, int slot, int* out, int cap) {
    const auto& t = static_cast<Pool*>(h)->tables[slot];
    const int n = std::min<int>(cap, static_cast<int>(t.size()));
    for (int i = 0; i < n; i++) out[i] = t[i];
    return static_cast<int>(t.size());
}
int orc_pool_free_list(void* h, int* out, int cap) {
    const auto& f = static_cast<Pool*>(h)->free_pages;
    const int n = std::min<int>(cap, static_cast<int>(f.size()));
    for (int i = 0; i < n; i++) out[i] = f[i];
    return static_cast<int>(f.size());
}

// ---- append: append_kernel<KV> (src/decode/paged_kv_cache.cu:25-39) -------------
// k, v: fp16 bits [n][num_kv_heads][head_dim].  Caches: [page][kv head][slot][dim],
// 2 bytes (dtype 0) or 1 byte (dtype 1) per element.  block_table_row is the
// slot's row of page ids.
void orc_append(int dtype, const uint16_t* k, const uint16_t* v, int n, void* k_cache, void* v_cache,
                const int* block_table_row, int start_pos, int num_kv_heads, int head_dim,
                int page_size, float k_scale, float v_scale) {
    const float inv_k = 1.f / k_scale, inv_v = 1.f / v_scale;
    for (int i = 0; i < n; i++) {
        const int pos  = start_pos + i;
        const int page = block_table_row[pos / page_size];
        for (int h = 0; h < num_kv_heads; h++)
            for (int d = 0; d < head_dim; d++) {
                const size_t dst = ((static_cast<size_t>(page) * num_kv_heads + h) * page_size + pos % page_size) * head_dim + d;
                const size_t src = (static_cast<size_t>(i) * num_kv_heads + h) * head_dim + d;
                if (dtype == 0) {
                    static_cast<uint16_t*>(k_cache)[dst] = float_to_half(half_to_float(k[src]));
                    static_cast<uint16_t*>(v_cache)[dst] = float_to_half(half_to_float(v[src]));
                } else {
                    static_cast<uint8_t*>(k_cache)[dst] = e4m3_from_float(half_to_float(k[src]) * inv_k);
                    static_cast<uint8_t*>(v_cache)[dst] = e4m3_from_float(half_to_float(v[src]) * inv_v);
                }
            }
    }
}

// ---- attention ------------------------------------------------------------------

// cpu_attention (src/attention/cpu/attention.cpp:5-34): fp32, one head,
// contiguous K/V [T][d]; scores -> max -> exp / sum / normalise -> weighted sum.
void orc_cpu_attention(const float* q, const float* K, const float* V, float* out, int T, int d) {
    std::vector<float> scores(T);
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    float max_score = -INFINITY;
    for (int i = 0; i < T; i++) {
        float dot = 0.0f;
        for (int j = 0; j < d; j++) dot += q[j] * K[i * d + j];
        scores[i] = dot * scale;
        if (scores[i] > max_score) max_score = scores[i];
    }
    float sum = 0.0f;
    for (float& x : scores) { x = std::exp(x - max_score); sum += x; }
    for (float& x : scores) x /= sum;
    for (int j = 0; j < d; j++) {
        float acc = 0.0f;
        for (int i = 0; i < T; i++) acc += scores[i] * V[i * d + j];
        out[j] = acc;
    }
}

static inline float cache_value(int dtype, const void* cache, size_t idx, float scale) {
    if (dtype == 0) return half_to_float(static_cast<const uint16_t*>(cache)[idx]);
    return e4m3_to_float(static_cast<const uint8_t*>(cache)[idx]) * scale;
}

// Multi-head GQA paged decode over the cache bytes as stored.  For every
// (batch row, query head) the row's K/V of kv head hq/group are gathered through
// the block table into contiguous fp32 [T][d] and handed to orc_cpu_attention;
// this is how the single-head reference CPU backend is driven for this path.
// precision 0: fp32 via orc_cpu_attention.  precision 1: the double-precision
// loop of the reference's decode test (tests/test_paged_decode.cu:111-145) with
// an explicit sm_scale.  q: fp16 bits [batch][hq][d]; out: float [batch][hq][d].
void orc_paged_decode(int precision, int dtype, const uint16_t* q, const void* k_cache,
                      const void* v_cache, const int* block_table, int block_table_stride,
                      const int* seq_lens, const int* slot_ids, int batch, int num_q_heads,
                      int num_kv_heads, int head_dim, int page_size, float sm_scale,
                      float k_scale, float v_scale, float* out, int threads) {
    const int group = num_q_heads / num_kv_heads;
    const int D = head_dim;
#if defined(_OPENMP)
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(dynamic, 1)
    for (int item = 0; item < batch * num_kv_heads; item++) {
        const int b = item / num_kv_heads, h = item % num_kv_heads;
        const int slot = slot_ids ? slot_ids[b] : b;
        const int T = seq_lens[slot];
        const int* bt = block_table + static_cast<size_t>(slot) * block_table_stride;
        std::vector<float> K(static_cast<size_t>(T) * D), V(static_cast<size_t>(T) * D);
        for (int t = 0; t < T; t++) {
            const size_t base = ((static_cast<size_t>(bt[t / page_size]) * num_kv_heads + h) * page_size + t % page_size) * D;
            for (int d = 0; d < D; d++) {
                K[static_cast<size_t>(t) * D + d] = cache_value(dtype, k_cache, base + d, k_scale);
                V[static_cast<size_t>(t) * D + d] = cache_value(dtype, v_cache, base + d, v_scale);
            }
        }
        for (int g = 0; g < group; g++) {
            const int hq = h * group + g;
            const size_t qo = (static_cast<size_t>(b) * num_q_heads + hq) * D;
            std::vector<float> qf(D);
            for (int d = 0; d < D; d++) qf[d] = half_to_float(q[qo + d]);
            if (precision == 0) {
                orc_cpu_attention(qf.data(), K.data(), V.data(), out + qo, T, D);
            } else {
                std::vector<double> s(T);
                double mx = -INFINITY;
                for (int t = 0; t < T; t++) {
                    double dot = 0;
                    for (int d = 0; d < D; d++) dot += double(qf[d]) * K[static_cast<size_t>(t) * D + d];
                    s[t] = dot * sm_scale;
                    mx = std::max(mx, s[t]);
                }
                double sum = 0;
                for (int t = 0; t < T; t++) { s[t] = std::exp(s[t] - mx); sum += s[t]; }
                for (int d = 0; d < D; d++) {
                    double o = 0;
                    for (int t = 0; t < T; t++) o += s[t] * V[static_cast<size_t>(t) * D + d];
                    out[qo + d] = static_cast<float>(o / sum);
                }
            }
        }
    }
}

// LSE merge of normalised split partials (merge_segments_kernel,
// src/decode/decode_kernels.cuh:409-432): out = sum 2^(lse_s-max) o_s / sum 2^(lse_s-max).
void orc_merge(const float* partial_out, const float* partial_lse, int num_parts, int dim, float* out) {
    float lse_max = -INFINITY;
    for (int s = 0; s < num_parts; s++) lse_max = std::max(lse_max, partial_lse[s]);
    for (int d = 0; d < dim; d++) {
        float num = 0.f, den = 0.f;
        for (int s = 0; s < num_parts; s++) {
            const float w = std::exp2(partial_lse[s] - lse_max);
            num = std::fma(w, partial_out[static_cast<size_t>(s) * dim + d], num);
            den += w;
        }
        out[d] = num / den;
    }
}

}  // extern "C"
