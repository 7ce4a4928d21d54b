#pragma once
// Paged split-KV flash-decoding for sm_100a: TMA + mbarrier pipeline, warp-specialised.
//
// Stands in for paged_decode_kernel / merge_segments_kernel of the reference
// (src/decode/decode_kernels.cuh:123-403, 409-432) and keeps their contract: a
// persistent grid of num_ctas CTAs, CTA c streams segments
// [cta_seg_begin[c], cta_seg_begin[c+1]) of the host-built plan; a (row, kv head)
// covered by one segment is written to `out` directly, otherwise each segment
// leaves a normalised fp32 partial + base-2 LSE for the merge kernel.
//
// What is different from the reference, and why:
//  * K/V pages are brought in by TMA (cp.async.bulk.tensor) from one tensor map
//    over the whole pool [page][kv head][token][dim]; the block-table entry is the
//    page coordinate.  One producer warp issues the copies (each lane owns one box
//    and prefetches its page ids a chunk ahead), WARPS consumer warps do the math.
//    The two sides meet only through full/empty mbarriers, so loads run ahead of
//    the math across tile and segment boundaries by STAGES-1 tiles.
//  * Tokens are the M dimension of mma.m16n8k16 and the (<= 8) query heads of the
//    GQA group the N dimension: S^T = K Q^T and O^T = V^T P^T.  No MMA row is
//    padding, which halves the tensor instruction count of the reference's
//    heads-as-M layout.  P^T reaches its B-fragment layout with two movmatrix.
//  * Shared memory uses the TMA 128-byte swizzle; fp16 rows are split in two
//    64-element panels so a box lands as [panel][token][128 B].  ldmatrix
//    (fp16) and 16-byte loads (fp8) are conflict-free for page sizes >= 8.
//  * Every wait is bounded; on expiry the CTA records a code in a status word,
//    raises a CTA-wide abort flag and drains its copies.  Nothing traps.
//  * A second tile shape (Config::HEADS = 8) takes 16 tokens of all 8 kv heads per tile, one consumer
//    warp per kv head, with rows (not (row, kv head) pairs) as the plan's work items: a page's K (or V)
//    block is then one contiguous 32 KB copy.
//  * Rows cut in a few pieces are merged by the decode kernel itself (the last piece to arrive does it);
//    the merge kernel, launched as a programmatic dependent, handles rows cut in many pieces.
//  * Optional extras behind null pointers: per-kv-head scales, outputs stored into the gathered buffers
//    of peer GPUs, a per-CTA record of busy time and tiles for the host's adaptive cut.

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "pd_b200.h"

namespace pdk {

constexpr int HEAD_DIM = 128;
constexpr int OSTRIDE  = HEAD_DIM + 4;   // padded row of the cross-warp merge scratch (floats)

// pd_params::needs_merge: 0 = no row is split, 1 = run merge_segments_kernel after the decode
// kernel (any workspace of [segments][group][129] floats will do), 2 = the decode kernel merges
// itself; the workspace then carries one zeroed int per (row, kv head) after the LSE array.
constexpr int MERGE_SEPARATE  = 1;
constexpr int MERGE_IN_KERNEL = 2;
// Plans cut on the device: the host cannot know how rows were cut, so each (row, kv head) decides for
// itself.  Cut in at most HYBRID_MAX_PIECES pieces: merged by the decode kernel's last arriver; in more:
// left to merge_segments_kernel, which is always launched in this mode and skips everything else.
constexpr int MERGE_HYBRID = 3;
constexpr int HYBRID_MAX_PIECES = 4;

// status word codes (code << 24 | blockIdx)
constexpr unsigned ST_FULL_TIMEOUT  = 1;   // consumer gave up waiting for a tile
constexpr unsigned ST_EMPTY_TIMEOUT = 2;   // producer gave up waiting for a free stage
constexpr unsigned ST_DRAIN_TIMEOUT = 3;   // producer gave up draining copies after an abort
constexpr unsigned ST_SYNC_TIMEOUT  = 4;   // a consumer warp gave up waiting for its siblings
constexpr unsigned ST_GATHER_TIMEOUT = 5;  // a peer's "slice has landed" flag never arrived
constexpr unsigned ST_WORKSPACE      = 6;  // the plan has more segments than the split-row workspace was sized for

// Where outputs go.  world == 0: to pd_params::out, [batch][num_q_heads][128].  world > 0: this
// GPU's rows are one slice of a layout gathered over `world` GPUs of the node, and every output
// is stored straight into the gathered buffer of every peer (plain 16-byte peer stores over NVLink; the
// local buffer is out[rank]).  The kernel itself neither fences nor signals: gather_signal_kernel, a
// programmatic dependent launched right behind it, raises this rank's flag on every peer once this grid
// has completed (all its stores performed), and gather_wait_kernel waits for the peers' flags.
// Optional per-kv-head dequantisation scales (device arrays of num_kv_heads floats, or null: the
// per-tensor pd_params::k_scale / v_scale apply).  The reference has one scale per tensor only.
struct HeadScales {
    const float* k;
    const float* v;
};

// Optional per-CTA record for the host's adaptive cut: every launch adds the CTA's busy nanoseconds to
// slots[2 * cta] and the tiles it processed to slots[2 * cta + 1], and CTA 0 counts the launch in
// slots[2 * grid]; the host works with differences between two readings.  Null switches the record off.
struct CtaStats {
    unsigned long long* slots;
};
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr int MAX_GATHER = 8;
struct GatherOut {
    int       world;
    int       rank;
    int       row_stride;    // query heads per row of the gathered layout
    int       head_offset;   // first head of this rank's slice within a row (kv-head sharding)
    int       row_offset;    // first row of this rank's slice (batch sharding)
    __half*   out[MAX_GATHER];
};
struct GatherFlags {
    unsigned* flags[MAX_GATHER];   // flags[r]: the flag array in rank r's memory, one word per sender
};

__device__ __forceinline__ size_t out_index(const pd_params& p, const GatherOut& gp, int row, int head) {
    return gp.world ? (static_cast<size_t>(row + gp.row_offset) * gp.row_stride + head + gp.head_offset) * 128
                    : (static_cast<size_t>(row) * p.num_q_heads + head) * 128;
}
template<typename T>
__device__ __forceinline__ void store_out(const pd_params& p, const GatherOut& gp, size_t index, T value) {
    if (gp.world == 0) {
        *reinterpret_cast<T*>(static_cast<__half*>(p.out) + index) = value;
    } else {
        for (int r = 0; r < gp.world; r++) *reinterpret_cast<T*>(gp.out[r] + index) = value;
    }
}

// HEADS = 1: a tile is TILE tokens of ONE kv head, the consumer warps split the tile's tokens and
// merge their softmax states at a segment's end (the reference's (row, kv head) work items).
// HEADS = 8 ("head-fused"): a tile is 16 tokens of ALL 8 kv heads of a row, fetched as one box per
// page and pool (32 KB of contiguous DRAM for fp16 instead of eight separate 4 KB pieces read at
// different times by different CTAs), consumer warp w owns kv head w outright, so nothing is merged
// across warps and a segment ends without any CTA-wide synchronisation.  Work items are rows.
template<int WARPS_, int GROUPS_PER_WARP_, int STAGES_, int MIN_CTAS_, int HEADS_ = 1>
struct Config {
    static constexpr int WARPS           = WARPS_;             // consumer warps (one more warp produces)
    static constexpr int GROUPS_PER_WARP = GROUPS_PER_WARP_;   // 16-token groups per warp per tile
    static constexpr int STAGES          = STAGES_;
    static constexpr int MIN_CTAS        = MIN_CTAS_;
    static constexpr int HEADS           = HEADS_;             // kv heads per tile
    static_assert(HEADS_ == 1 || (HEADS_ == WARPS_ && GROUPS_PER_WARP_ <= 2), "head-fused: one warp per kv head, one unit per tile");
};

template<typename KV, int GROUP, typename C>
struct Shape {
    static constexpr int THREADS     = (C::WARPS + 1) * 32;
    static constexpr int CONSUMERS   = C::WARPS * 32;
    static constexpr int HEADS       = C::HEADS;
    static constexpr int TILE        = C::WARPS * C::GROUPS_PER_WARP * 16 / HEADS;   // tokens per tile
    static constexpr int ROW_BYTES   = HEAD_DIM * static_cast<int>(sizeof(KV));
    static constexpr int TILE_BYTES  = TILE * ROW_BYTES * HEADS;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int PIPE_BYTES  = C::STAGES * STAGE_BYTES;
    // The cross-warp merge runs over at most 4 heads at a time (two passes for a
    // group of 8), which keeps two CTAs of the fp16 configuration on one SM.
    static constexpr int GROUP_PAD   = GROUP < 2 ? 2 : (GROUP > 4 ? 4 : GROUP);
    static constexpr int PASSES      = GROUP > 4 ? 2 : 1;
    static constexpr int MERGE_BYTES = HEADS > 1 ? 0 : (C::WARPS * GROUP_PAD * OSTRIDE + 2 * C::WARPS * 8) * 4;
    static constexpr int BAR_BYTES   = 2 * C::STAGES * 8 + 16;
    // One slot of query rows per stage: the producer copies a segment's [GROUP][128] fp16 rows
    // along with the segment's first tile, so consumers never wait on a global load of Q.
    // (Head-fused tiles would need all query heads of a row per slot; there the consumer warps load
    // their own rows from global memory at a segment's start instead.)
    static constexpr int Q_SLOT_BYTES = HEADS > 1 ? 0 : GROUP * HEAD_DIM * 2;
    static constexpr int Q_BYTES      = C::STAGES * Q_SLOT_BYTES;
    // Head-fused: [GROUP][128] fp16 staging rows per consumer warp, from which finished rows leave as 16-byte stores.
    static constexpr int OUT_STAGE_OFFSET = PIPE_BYTES + Q_BYTES + MERGE_BYTES + ((BAR_BYTES + 15) & ~15);
    static constexpr int OUT_STAGE_BYTES  = HEADS > 1 ? C::WARPS * GROUP * HEAD_DIM * 2 : 0;
    // +1024: the pipeline is aligned to the 128B-swizzle period by hand
    static constexpr int SMEM_BYTES  = 1024 + OUT_STAGE_OFFSET + OUT_STAGE_BYTES;
    static_assert(sizeof(KV) == 2 ? (HEADS == 1 || C::GROUPS_PER_WARP == 1) : C::GROUPS_PER_WARP % 2 == 0,
                  "a warp works on 16-token units of an fp16 cache, 32-token units of an e4m3 cache");
    static_assert(GROUP >= 1 && GROUP <= 8, "a KV group fills the 8 columns of one MMA");
};

// ---- PTX wrappers -------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after about 2^31 SM cycles (~1 s).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) return false;
    }
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// One box of a 4-D (fp8) or 5-D (fp16) tensor map into shared memory.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(pol) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4, uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
                 " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(pol) : "memory");
}
// Four rows of a 2-D tensor map (box: `cols` x 1 row), gathered into four consecutive 128-byte rows of shared
// memory: one copy instruction for four tokens whose rows lie anywhere in the pool (pages of 1 or 2 tokens).
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col,
                                            int r0, int r1, int r2, int r3, uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.L2::cache_hint"
                 " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "l"(pol) : "memory");
}
// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128_zero(uint32_t addr) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" :: "r"(addr), "r"(0u) : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// D(16x8) += A(16x16, row) * B(16x8, col), fp16 in, fp32 accumulate.
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// Byte offset, inside one K or V tile, of the 128-byte shared-memory row that
// holds token `t` (0..TILE-1), panel `h` (fp16: dims 64h..64h+63; fp8: h = 0).
// A tile is a run of boxes of 2^btl tokens; a box is [panel][token][128 B].
// With HEADS kv heads per box the box is [kv head][panel][token][128 B].
template<typename KV, int HEADS = 1>
__device__ __forceinline__ uint32_t row_offset(int t, int h, int btl, int head = 0) {
    constexpr int PANELS = sizeof(KV);   // 2 for fp16, 1 for fp8
    const int box = t >> btl, r = t & ((1 << btl) - 1);
    return static_cast<uint32_t>((((box * HEADS + head) * PANELS + h) << btl) + r) << 7;
}
// Address of 16-byte chunk c of a 128-byte row under the TMA 128B swizzle
// (chunk index XOR row index mod 8; the tile base is 1024-byte aligned).
__device__ __forceinline__ uint32_t swz(uint32_t row_off, int c) {
    return row_off + (((c ^ (row_off >> 7)) & 7) << 4);
}

// ---- fp16 cache, one 16-token group: S^T = K Q^T, online softmax, O^T += V^T P^T -------------------
//
// `rows(t, panel)` gives the byte offset, from the tile base, of the 128-byte shared-memory row
// that holds token t of the group's (row, kv head), panel = dims 64*panel...
// grp_row is the first token of the group inside the tile; grp_valid (1..16+) how many of its tokens exist.
// Returns true if it wrote to shared memory (dead V rows cleared), so the caller fences before
// handing the stage back to the copy engine.
template<typename Rows>
__device__ __forceinline__ bool process_group_f16(const uint32_t k_tile, const uint32_t v_tile, const Rows rows,
                                                  const int grp_row, const int grp_valid, const uint32_t (&qb)[8][2],
                                                  float (&acc)[8][4], float (&m_run)[2], float (&l_run)[2],
                                                  const float qk_scale, const int lane)
{
    const int g = lane >> 2;
    bool wrote = false;
    if (grp_valid < 16) {
        // Rows past the end hold whatever the page or the stage held before; a NaN
        // there would survive P = 0 in the PV product, so clear V's dead rows.
        constexpr int CH = HEAD_DIM * 2 / 16;
        for (int idx = lane; idx < 16 * CH; idx += 32) {
            const int r = idx / CH, c = idx % CH;
            if (r >= grp_valid)
                sts128_zero(v_tile + rows(grp_row + r, c >> 3) + ((c & 7) << 4));
        }
        wrote = true;
        __syncwarp();
    }

    // ---- 1. S^T = K Q^T : 16 tokens x 8 heads, two interleaved accumulators.
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
        const int t = grp_row + (lane & 7) + ((lane >> 3) & 1) * 8;
        const uint32_t r0 = rows(t, 0), r1 = rows(t, 1);
        const int hi = lane >> 4;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            uint32_t a[4];
            ldmatrix_x4(a, k_tile + swz(ks < 4 ? r0 : r1, (ks & 3) * 2 + hi));
            if (ks & 1) mma_16816(s1, a, qb[ks][0], qb[ks][1]);
            else        mma_16816(s0, a, qb[ks][0], qb[ks][1]);
        }
    }

    // ---- 2. online softmax. This lane: tokens g, g+8 of the group, heads 2qd, 2qd+1.
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; i++) x[i] = (s0[i] + s1[i]) * qk_scale;
    if (grp_valid < 16) {
        if (g >= grp_valid)     { x[0] = -INFINITY; x[1] = -INFINITY; }
        if (g + 8 >= grp_valid) { x[2] = -INFINITY; x[3] = -INFINITY; }
    }
    float mx[2] = {fmaxf(x[0], x[2]), fmaxf(x[1], x[3])};
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float m_new = fmaxf(m_run[h], mx[h]);
        alpha[h] = exp2f(m_run[h] - m_new);
        m_run[h] = m_new;
    }
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; i++) pr[i] = exp2f(x[i] - m_run[i & 1]);
    l_run[0] = l_run[0] * alpha[0] + (pr[0] + pr[2]);
    l_run[1] = l_run[1] * alpha[1] + (pr[1] + pr[3]);
#pragma unroll
    for (int mt = 0; mt < 8; mt++) {
        acc[mt][0] *= alpha[0]; acc[mt][1] *= alpha[1];
        acc[mt][2] *= alpha[0]; acc[mt][3] *= alpha[1];
    }

    // ---- 3. O^T += V^T P^T.  P^T's B fragment = transposed 8x8 blocks of the scores.
    const uint32_t pb0 = movmatrix_trans(pack_half2(pr[0], pr[1]));   // tokens 0..7
    const uint32_t pb1 = movmatrix_trans(pack_half2(pr[2], pr[3]));   // tokens 8..15
    {
        const int t = grp_row + (lane & 7) + ((lane >> 4) & 1) * 8;
        const uint32_t r0 = rows(t, 0), r1 = rows(t, 1);
        const int hi = (lane >> 3) & 1;
#pragma unroll
        for (int mt = 0; mt < 8; mt++) {
            uint32_t a[4];
            ldmatrix_x4_trans(a, v_tile + swz(mt < 4 ? r0 : r1, (mt & 3) * 2 + hi));
            mma_16816(acc[mt], a, pb0, pb1);
        }
    }
    return wrote;
}

// ---- e4m3 cache, one 32-token group ------------------------------------------------------------------
//
// The cache bytes are widened to fp16 in registers (cvt.f16x2.e4m3x2, exact) and meet the fp16 query rows
// and the fp16-rounded softmax weights in the same mma.m16n8k16 as the fp16 cache.  (mma.sync on e4m3
// operands is not a tensor-core instruction of sm_100a: it compiles, but ncu counts 18 issued instructions
// per mma - widening of both operands, two fp16 MMAs, four adds - so feeding the bytes to it directly, with
// queries and weights split into three e4m3 terms each, cost 870 instructions per 32 tokens and was slower.)
// What keeps the instruction count per byte down, since an fp8 layer has half the bytes per token and the
// same work per token as an fp16 one:
//  * a warp's unit is 32 tokens: one round of maxima, shuffles and exponentials per 32 tokens;
//  * K as the A operand: lane (g, qd) reads the 16-byte chunks 2qd, 2qd+1 of its token rows; each 4-byte word
//    widens into the two halves of a k-step's fragment (dims d, d+1 | d+2, d+3; the query fragments are loaded
//    in the same dim order, which a dot product does not see);
//  * V as the A operand of O^T += V^T P^T: ldmatrix.m16n16.x2.trans.b8 over chunk `mt` of the 32 token rows
//    delivers, per lane, dim g (and g + 8) of four tokens per half as one register each; widened, they are
//    the fragments of that dim tile for both 16-token halves, with no byte shuffling at all;
//  * the accumulators are rescaled only when some running maximum moved (rare after the first tiles).
// MMA row r of a 16-token half holds token tau16(r): any assignment would do, this one makes the 16 rows that
// one transposed ldmatrix touches fall into different bank groups under the 128-byte swizzle.
__device__ __forceinline__ int tau16(int r) { return r < 8 ? r : 8 + ((r + 4) & 7); }

__device__ __forceinline__ uint32_t widen_lo(uint32_t w) {      // bytes 0, 1 -> f16x2
    uint32_t r;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t widen_hi(uint32_t w) {      // bytes 2, 3 -> f16x2
    uint32_t r;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(r) : "r"(w));
    return r;
}
// 16 dims x 32 tokens of a byte tile, transposed: lanes 0..15 give the addresses of the 16-byte chunks of
// matrix rows (tokens) 0..15, lanes 16..31 of rows 16..31.  Lane (g, qd) receives r0: dim g of rows 4qd..4qd+3,
// r1: dim g + 8 of the same rows, r2, r3: the same for rows 16 + 4qd...
__device__ __forceinline__ void ldmatrix_b8_x2_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// grp_row: first token of the group inside the tile; grp_valid (1..32+): how many of its tokens exist.
template<typename Rows>
__device__ __forceinline__ bool process_group_e4m3(const uint32_t k_tile, const uint32_t v_tile, const Rows rows,
                                                   const int grp_row, const int grp_valid, const uint32_t (&qb)[8][2],
                                                   float (&acc)[8][4], float (&m_run)[2], float (&l_run)[2],
                                                   const float qk_scale, const int lane)
{
    const int g = lane >> 2, qd = lane & 3;
    bool wrote = false;
    if (grp_valid < 32) {
        // dead V rows: a NaN byte there would survive a zero weight in the PV product
        for (int idx = lane; idx < 32 * 8; idx += 32) {
            const int r = idx >> 3, c = idx & 7;
            if (r >= grp_valid) sts128_zero(v_tile + rows(grp_row + r, 0) + (c << 4));
        }
        wrote = true;
        __syncwarp();
    }

    // ---- 1. S^T = K Q^T for both 16-token halves, two interleaved accumulators each.
    const int tok_lo = g, tok_hi = tau16(g + 8);      // tokens of MMA rows g, g + 8 within a half
    float x[2][4];
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const uint32_t r0 = rows(grp_row + 16 * hh + tok_lo, 0), r1 = rows(grp_row + 16 * hh + tok_hi, 0);
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint4 lo = lds128(k_tile + swz(r0, 2 * qd + j));
            const uint4 hi = lds128(k_tile + swz(r1, 2 * qd + j));
            const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint32_t a[4] = {widen_lo(wl[m]), widen_lo(wh[m]), widen_hi(wl[m]), widen_hi(wh[m])};
                const int ks = 4 * j + m;
                if (m & 1) mma_16816(s1, a, qb[ks][0], qb[ks][1]);
                else       mma_16816(s0, a, qb[ks][0], qb[ks][1]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) x[hh][i] = (s0[i] + s1[i]) * qk_scale;
        if (grp_valid < 32) {
            if (16 * hh + tok_lo >= grp_valid) { x[hh][0] = -INFINITY; x[hh][1] = -INFINITY; }
            if (16 * hh + tok_hi >= grp_valid) { x[hh][2] = -INFINITY; x[hh][3] = -INFINITY; }
        }
    }

    // ---- 2. online softmax over the 32 tokens.  This lane: 4 tokens, heads 2qd, 2qd+1.
    float mx[2] = {fmaxf(fmaxf(x[0][0], x[0][2]), fmaxf(x[1][0], x[1][2])),
                   fmaxf(fmaxf(x[0][1], x[0][3]), fmaxf(x[1][1], x[1][3]))};
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float m_new = fmaxf(m_run[h], mx[h]);
        alpha[h] = exp2f(m_run[h] - m_new);
        m_run[h] = m_new;
    }
    float pr[2][4];
#pragma unroll
    for (int hh = 0; hh < 2; hh++)
#pragma unroll
        for (int i = 0; i < 4; i++) pr[hh][i] = exp2f(x[hh][i] - m_run[i & 1]);
    l_run[0] = l_run[0] * alpha[0] + ((pr[0][0] + pr[0][2]) + (pr[1][0] + pr[1][2]));
    l_run[1] = l_run[1] * alpha[1] + ((pr[0][1] + pr[0][3]) + (pr[1][1] + pr[1][3]));
    // the accumulators only change scale when some maximum moved, which after the first tiles is rare
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int mt = 0; mt < 8; mt++) {
            acc[mt][0] *= alpha[0]; acc[mt][1] *= alpha[1];
            acc[mt][2] *= alpha[0]; acc[mt][3] *= alpha[1];
        }
    }

    // ---- 3. O^T += V^T P^T.  P^T's B fragments = transposed 8x8 blocks of the weights (MMA rows 0..7, 8..15).
    uint32_t pb[2][2];
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        pb[hh][0] = movmatrix_trans(pack_half2(pr[hh][0], pr[hh][1]));
        pb[hh][1] = movmatrix_trans(pack_half2(pr[hh][2], pr[hh][3]));
    }
    {
        // matrix row i of a half = MMA row (k index) 2(i >> 2) + (i & 1) + 8(i >> 1 & 1): the widened low half of a
        // register is then k = 2qd, 2qd+1 (a0 / a1), the high half k = 2qd+8, 2qd+9 (a2 / a3)
        const int i = lane & 15;
        const int t = grp_row + 16 * (lane >> 4) + tau16(2 * (i >> 2) + (i & 1) + 8 * ((i >> 1) & 1));
        const uint32_t r = rows(t, 0);
#pragma unroll
        for (int mt = 0; mt < 8; mt++) {
            uint32_t v[4];
            ldmatrix_b8_x2_trans(v, v_tile + swz(r, mt));
            const uint32_t a0[4] = {widen_lo(v[0]), widen_lo(v[1]), widen_hi(v[0]), widen_hi(v[1])};
            const uint32_t a1[4] = {widen_lo(v[2]), widen_lo(v[3]), widen_hi(v[2]), widen_hi(v[3])};
            mma_16816(acc[mt], a0, pb[0][0], pb[0][1]);
            mma_16816(acc[mt], a1, pb[1][0], pb[1][1]);
        }
    }
    return wrote;
}

// LSE-weighted mean of the normalised partials of one (row, query head), by one warp:
//   out = sum_s 2^(lse_s - max) o_s / sum_s 2^(lse_s - max)      (base-2 LSE)
// Partials are read past L1 (.cg): another SM wrote them.
template<int GROUP>
// Partial (segment s, this head) lives at index s * stride + gq: stride = GROUP, gq = hq % GROUP for
// (row, kv head) work items; stride = num_q_heads, gq = hq for head-fused rows.
__device__ __forceinline__ void merge_one_head(const pd_params& p, const GatherOut& gp, int b, int hq, int s0, int s1,
                                               int lane, int stride, int gq)
{
    float lse_max = -INFINITY;
    for (int s = s0 + lane; s < s1; s += 32) lse_max = fmaxf(lse_max, __ldcg(p.partial_lse + s * stride + gq));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lse_max = fmaxf(lse_max, __shfl_xor_sync(0xffffffffu, lse_max, o));

    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (int base = s0; base < s1; base += 32) {
        const int s = base + lane;
        const float w_mine = s < s1 ? exp2f(__ldcg(p.partial_lse + s * stride + gq) - lse_max) : 0.f;
        const int n = min(32, s1 - base);
        for (int j = 0; j < n; j++) {
            const float w = __shfl_sync(0xffffffffu, w_mine, j);
            const float4 o = __ldcg(reinterpret_cast<const float4*>(
                p.partial_out + (static_cast<size_t>(base + j) * stride + gq) * HEAD_DIM + lane * 4));
            num.x = fmaf(w, o.x, num.x); num.y = fmaf(w, o.y, num.y);
            num.z = fmaf(w, o.z, num.z); num.w = fmaf(w, o.w, num.w);
            den += w;
        }
    }
    const __half2 lo = __floats2half2_rn(num.x / den, num.y / den);
    const __half2 hi = __floats2half2_rn(num.z / den, num.w / den);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    store_out(p, gp, out_index(p, gp, b, hq) + lane * 4, packed);
}

// All GROUP query heads of one (row, kv head) by one warp, with the loads of the heads in flight
// together: used by the decode kernel's own merge, where the merging warp holds up its CTA's
// pipeline until it is done.  Up to 32 segments per row in the fast path.
template<int GROUP>
__device__ __forceinline__ void merge_item(const pd_params& p, const GatherOut& gp, int b, int kv_head, int s0, int s1,
                                           int lane, int stride = GROUP, int first = 0)
{
    const int n = s1 - s0;
    if (n > 32) {
        for (int hd = 0; hd < GROUP; hd++) merge_one_head<GROUP>(p, gp, b, kv_head * GROUP + hd, s0, s1, lane, stride, first + hd);
        return;
    }
    float w[GROUP], den[GROUP];
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++)
        w[hd] = lane < n ? __ldcg(p.partial_lse + (s0 + lane) * stride + first + hd) : -INFINITY;   // LSE of segment s0 + lane
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) {
        float mx = w[hd];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        w[hd] = exp2f(w[hd] - mx);                                                         // 0 for lanes >= n
        den[hd] = 0.f;
    }
    float4 num[GROUP];
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) num[hd] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
    for (int j = 0; j < n; j++) {
        float4 o[GROUP];
#pragma unroll
        for (int hd = 0; hd < GROUP; hd++)
            o[hd] = __ldcg(reinterpret_cast<const float4*>(
                p.partial_out + (static_cast<size_t>(s0 + j) * stride + first + hd) * HEAD_DIM + lane * 4));
#pragma unroll
        for (int hd = 0; hd < GROUP; hd++) {
            const float wj = __shfl_sync(0xffffffffu, w[hd], j);
            num[hd].x = fmaf(wj, o[hd].x, num[hd].x); num[hd].y = fmaf(wj, o[hd].y, num[hd].y);
            num[hd].z = fmaf(wj, o[hd].z, num[hd].z); num[hd].w = fmaf(wj, o[hd].w, num[hd].w);
            den[hd] += wj;   // same order of additions as merge_one_head: both merges give the same bits
        }
    }
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) {
        const __half2 lo = __floats2half2_rn(num[hd].x / den[hd], num[hd].y / den[hd]);
        const __half2 hi = __floats2half2_rn(num[hd].z / den[hd], num[hd].w / den[hd]);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        store_out(p, gp, out_index(p, gp, b, kv_head * GROUP + hd) + lane * 4, packed);
    }
}

// ---- decode kernel ---------------------------------------------------------------

template<typename KV, int GROUP, typename C>
__global__ void __launch_bounds__((C::WARPS + 1) * 32, C::MIN_CTAS)
paged_decode_kernel(const __grid_constant__ pd_params p, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const int btl /* log2(tokens per box) */,
                    const int row_gather /* boxes are four rows gathered one by one: the maps are 2-D [pool row][dims] */,
                    const int seg_limit /* segments the split-row workspace holds; 0 = sized by the plan's owner */,
                    unsigned* __restrict__ status, const __grid_constant__ GatherOut gp,
                    const __grid_constant__ HeadScales hs, const __grid_constant__ CtaStats st)
{
    const unsigned long long t_entry = (st.slots && threadIdx.x == 0) ? global_ns() : 0ull;
#ifdef PD_B200_LOAD_ONLY
    constexpr bool no_math = true;    // diagnostic build: stream the tiles, skip the arithmetic
#else
    constexpr bool no_math = false;
#endif
    constexpr int nst = C::STAGES;
    using S = Shape<KV, GROUP, C>;
    constexpr bool FP8 = sizeof(KV) == 1;
    constexpr int STAGES = C::STAGES;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t pipe = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (pipe - smem_u32(smem_raw));   // generic view of the aligned base
    const uint32_t q_slots = pipe + S::PIPE_BYTES;                              // [STAGES][GROUP][128] halves
    float* w_o = reinterpret_cast<float*>(gen + S::PIPE_BYTES + S::Q_BYTES);
    float* w_m = w_o + C::WARPS * S::GROUP_PAD * OSTRIDE;
    float* w_l = w_m + C::WARPS * 8;
    const uint32_t bars = pipe + S::PIPE_BYTES + S::Q_BYTES + S::MERGE_BYTES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + S::PIPE_BYTES + S::Q_BYTES + S::MERGE_BYTES + 2 * STAGES * 8 + 8);
    auto full_bar  = [&](int s) { return bars + s * 8; };
    auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
    const uint32_t sync_bar = bars + 2 * STAGES * 8;   // consumer-warp rendezvous (bounded, unlike bar.sync)

    // Let a dependent launch (the merge kernel) be scheduled as soon as SMs have room; it waits for this
    // whole grid before it reads anything this grid writes.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int seg_begin = p.cta_seg_begin[blockIdx.x];
    const int seg_end   = p.cta_seg_begin[blockIdx.x + 1];
    if (seg_begin >= seg_end) return;
    if (seg_limit > 0 && seg_end > seg_limit) {
        // A workspace of fixed size (the built-in one) and a plan with more segments than the caller
        // declared: this CTA's partial rows would land outside it.  Nothing is stored; the status word says so.
        if (threadIdx.x == 0) atomicCAS(status, 0u, (ST_WORKSPACE << 24) | (blockIdx.x & 0xffffffu));
        return;
    }

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == C::WARPS * 32) {   // producer lane 0: have the descriptors on their way before the first copy needs them
        asm volatile("prefetch.tensormap [%0];" :: "l"(&k_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&v_map) : "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), C::WARPS); }
        mbar_init(sync_bar, C::WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int4* segments = static_cast<const int4*>(p.segments);
    auto fail = [&](unsigned code) {
        atomicCAS(status, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
        *abort_flag = 1;
    };

    if (warp == C::WARPS) {
        // ================= producer warp =================
        const int bt_tokens = 1 << btl;                 // tokens per box
        const int bpt       = S::TILE >> btl;           // boxes per tile
        const uint32_t box_bytes = static_cast<uint32_t>(bt_tokens) * S::ROW_BYTES * S::HEADS;
        const uint64_t pol = l2_evict_first_policy();
        const int ps = p.page_size;
        int issued = 0;                                 // tiles issued so far
        int p_stage = 0;                                // stage of the next tile and the parity of its round
        uint32_t p_phase = 0;
        bool ok = true;

        auto table_of = [&](int b) {
            const int slot = p.slot_ids ? __ldg(p.slot_ids + b) : b;
            return p.block_table + static_cast<size_t>(slot) * p.block_table_stride;
        };
        // Issue the copies of one tile: lanes [lane0, lane0 + nb) own one box each when
        // the tile has <= 32 boxes, otherwise every lane walks boxes lane, lane+32, ...
        auto issue_tile = [&](const int4& sg, int tile_tok, int4 my_page, int lane0, const int* bt) -> bool {
            const int stage = p_stage;
            if (!mbar_wait(empty_bar(stage), p_phase ^ 1)) { if (lane == 0) fail(ST_EMPTY_TIMEOUT); return false; }
            if (*abort_flag) return false;
            const int valid = min(S::TILE, sg.w - tile_tok);
            const int nb = (valid + bt_tokens - 1) >> btl;
            const bool first_tile = S::HEADS == 1 && tile_tok == sg.z;   // the segment's query rows ride along
            if (lane == 0) {
                mbar_expect_tx(full_bar(stage), 2u * nb * box_bytes + (first_tile ? S::Q_SLOT_BYTES : 0));
                if (first_tile)
                    bulk_load(q_slots + stage * S::Q_SLOT_BYTES,
                              static_cast<const __half*>(p.q) + (static_cast<size_t>(sg.x) * p.num_q_heads + sg.y * GROUP) * HEAD_DIM,
                              S::Q_SLOT_BYTES, full_bar(stage));
            }
            __syncwarp();
            const uint32_t k_dst = pipe + stage * S::STAGE_BYTES;
            const uint32_t v_dst = k_dst + S::TILE_BYTES;
            const int head_coord = S::HEADS == 1 ? sg.y : 0;   // a head-fused box spans kv heads 0..7
            auto copy_box = [&](int j, int4 page4) {
                const int page = page4.x;
                if (S::HEADS == 1 && row_gather) {
                    // pages smaller than four tokens: the box's four tokens are four rows of the pool, looked up
                    // one by one (tokens past the segment's end repeat its last token; their rows are masked)
                    const int t0 = tile_tok + 4 * j, last = sg.w - 1;
                    const int pg[4] = {page4.x, page4.y, page4.z, page4.w};
                    int r[4];
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        r[i] = (pg[i] * p.num_kv_heads + head_coord) * ps + min(t0 + i, last) % ps;
                    constexpr int PANELS = sizeof(KV);
#pragma unroll
                    for (int h = 0; h < PANELS; h++) {
                        tma_gather4(k_dst + j * box_bytes + h * 512, &k_map, full_bar(stage), 64 * h, r[0], r[1], r[2], r[3], pol);
                        tma_gather4(v_dst + j * box_bytes + h * 512, &v_map, full_bar(stage), 64 * h, r[0], r[1], r[2], r[3], pol);
                    }
                    return;
                }
                const int tok_in_page = (tile_tok + (j << btl)) % ps;
                if constexpr (FP8) {
                    tma_load_4d(k_dst + j * box_bytes, &k_map, full_bar(stage), 0, tok_in_page, head_coord, page, pol);
                    tma_load_4d(v_dst + j * box_bytes, &v_map, full_bar(stage), 0, tok_in_page, head_coord, page, pol);
                } else {
                    tma_load_5d(k_dst + j * box_bytes, &k_map, full_bar(stage), 0, tok_in_page, 0, head_coord, page, pol);
                    tma_load_5d(v_dst + j * box_bytes, &v_map, full_bar(stage), 0, tok_in_page, 0, head_coord, page, pol);
                }
            };
            if (bpt <= 32) {
                const int j = lane - lane0;
                if (j >= 0 && j < nb) copy_box(j, my_page);
            } else {
                for (int j = lane; j < nb; j += 32)
                    copy_box(j, make_int4(__ldg(bt + (tile_tok + (j << btl)) / ps), 0, 0, 0));
            }
            issued++;
            if (++p_stage == nst) { p_stage = 0; p_phase ^= 1; }
            return true;
        };

        // A chunk is up to 32 boxes of one segment: lane l owns box l of the chunk.
        const int chunk_tiles  = bpt <= 32 ? 32 / bpt : 1;
        const int chunk_tokens = chunk_tiles * S::TILE;
        int  seg = seg_begin;
        int4 sg  = __ldg(segments + seg);
        const int* bt = table_of(sg.x);
        int  tok = sg.z;
        // the page id of this lane's box (row_gather: of each of its four tokens)
        auto page_of = [&](const int4& s, const int* table, int chunk_tok) {
            const int t = chunk_tok + (lane << btl);
            int4 pg = make_int4(0, 0, 0, 0);
            if (bpt <= 32 && t < s.w) {
                pg.x = __ldg(table + t / ps);
                if (S::HEADS == 1 && row_gather) {
                    const int last = s.w - 1;
                    pg.y = __ldg(table + min(t + 1, last) / ps);
                    pg.z = __ldg(table + min(t + 2, last) / ps);
                    pg.w = __ldg(table + min(t + 3, last) / ps);
                }
            }
            return pg;
        };
        int4 page = page_of(sg, bt, tok);
        while (ok && seg < seg_end) {
            // Look one chunk ahead (possibly into the next segment) so its page ids are
            // in flight while this chunk's copies are issued.
            int  n_seg = seg, n_tok = tok + chunk_tokens;
            int4 n_sg = sg;
            const int* n_bt = bt;
            if (n_tok >= sg.w) {
                n_seg = seg + 1;
                if (n_seg < seg_end) { n_sg = __ldg(segments + n_seg); n_bt = table_of(n_sg.x); n_tok = n_sg.z; }
            }
            const int4 n_page = n_seg < seg_end ? page_of(n_sg, n_bt, n_tok) : make_int4(0, 0, 0, 0);
            for (int ti = 0; ti < chunk_tiles; ti++) {
                const int tile_tok = tok + ti * S::TILE;
                if (tile_tok >= sg.w) break;
                if (!issue_tile(sg, tile_tok, page, ti * bpt, bt)) { ok = false; break; }
            }
            seg = n_seg; sg = n_sg; bt = n_bt; tok = n_tok; page = n_page;
        }
        if (!ok || *abort_flag) {
            // Drain: no copy may still be in flight towards this CTA's shared memory at exit.
            for (int i = 0; i < min(issued, nst); i++) {
                int s = p_stage - 1 - i;                 // walk back over the most recent issues
                uint32_t par = p_phase;
                if (s < 0) { s += nst; par ^= 1; }
                if (!mbar_wait(full_bar(s), par)) { if (lane == 0) fail(ST_DRAIN_TIMEOUT); break; }
            }
        }
        return;
    }

    // ================= consumer warps =================
    const int g  = lane >> 2;   // fragment row
    const int qd = lane & 3;    // fragment column pair: this lane owns heads 2qd, 2qd+1
    // softmax runs in base 2; with per-head scales the factor belongs to the segment's kv head
    float qk_scale = p.sm_scale * p.k_scale * 1.4426950408889634f;
    float v_scale  = p.v_scale;
    if constexpr (S::HEADS > 1) {
        if (hs.k) qk_scale = p.sm_scale * __ldg(hs.k + warp) * 1.4426950408889634f;
        if (hs.v) v_scale = __ldg(hs.v + warp);
    }

    float acc[8][4];
    float m_run[2], l_run[2];
    uint32_t qb[8][2];          // Q^T B-fragments for the 8 k-steps

    unsigned tiles_done = 0;
    int c_stage = 0;            // stage of the next tile to consume and the parity of its round
    uint32_t c_phase = 0;
    bool alive = true;
    uint32_t sync_phase = 0;
    // All consumer warps meet here; gives up (and aborts the CTA) instead of hanging
    // if a warp that bailed out never arrives.
    auto consumer_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(sync_bar);
        const bool ok = mbar_wait(sync_bar, sync_phase);
        sync_phase ^= 1;
        if (!ok) { if (lane == 0) fail(ST_SYNC_TIMEOUT); alive = false; }
        return ok;
    };

    for (int seg = seg_begin; alive && seg < seg_end; seg++) {
        const int4 sg = __ldg(segments + seg);
        bool need_q = true;   // Q^T fragments are read from the slot of the segment's first tile
        if constexpr (S::HEADS == 1) {
            if (hs.k) qk_scale = p.sm_scale * __ldg(hs.k + sg.y) * 1.4426950408889634f;
            if (hs.v) v_scale = __ldg(hs.v + sg.y);
        }
        if constexpr (S::HEADS > 1) {
            // head-fused: this warp's kv head is `warp`; its query rows come straight from global memory
            const bool live = g < GROUP;
            const __half* qrow = static_cast<const __half*>(p.q)
                + (static_cast<size_t>(sg.x) * p.num_q_heads + warp * GROUP + (live ? g : 0)) * HEAD_DIM;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                if constexpr (FP8) {
                    const int db = (2 * qd + (ks >> 2)) * 16 + (ks & 3) * 4;
                    const uint2 v = __ldg(reinterpret_cast<const uint2*>(qrow + db));
                    qb[ks][0] = live ? v.x : 0u;
                    qb[ks][1] = live ? v.y : 0u;
                } else {
                    const uint32_t lo = __ldg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * qd));
                    const uint32_t hi = __ldg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * qd));
                    qb[ks][0] = live ? lo : 0u;
                    qb[ks][1] = live ? hi : 0u;
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < 8; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
        m_run[0] = m_run[1] = -INFINITY;
        l_run[0] = l_run[1] = 0.f;

        for (int tok = sg.z; tok < sg.w; tok += S::TILE) {
            const int stage = c_stage;
            if (!mbar_wait(full_bar(stage), c_phase)) { if (lane == 0) fail(ST_FULL_TIMEOUT); alive = false; break; }
            if (*abort_flag) { alive = false; break; }
            if (need_q && S::HEADS == 1) {
                // column n = g is query head g of the group (zero when g >= GROUP)
                need_q = false;
                const bool live = g < GROUP;
                const uint32_t qrow = q_slots + stage * S::Q_SLOT_BYTES + (live ? g : 0) * (HEAD_DIM * 2);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    if constexpr (FP8) {
                        // k-slots {2qd, 2qd+1 | 2qd+8, 2qd+9} of k-step ks are dims db..db+3: one 4-byte word of K
                        const int db = (2 * qd + (ks >> 2)) * 16 + (ks & 3) * 4;
                        const uint2 v = lds64(qrow + db * 2);
                        qb[ks][0] = live ? v.x : 0u;
                        qb[ks][1] = live ? v.y : 0u;
                    } else {
                        const uint32_t lo = lds32(qrow + (ks * 16 + 2 * qd) * 2);
                        const uint32_t hi = lds32(qrow + (ks * 16 + 8 + 2 * qd) * 2);
                        qb[ks][0] = live ? lo : 0u;
                        qb[ks][1] = live ? hi : 0u;
                    }
                }
            }
            const uint32_t k_tile = pipe + stage * S::STAGE_BYTES;
            const uint32_t v_tile = k_tile + S::TILE_BYTES;
            const int valid = sg.w - tok;   // tokens of this tile that exist (may exceed TILE)
            bool wrote = false;

            // a warp's unit of work: 16 tokens (fp16 cache) or 32 tokens (e4m3 cache, one k-step of its MMA)
            constexpr int UNIT = FP8 ? 2 : 1;
#pragma unroll
            for (int gi = 0; gi < C::GROUPS_PER_WARP; gi += UNIT) {
                const int grp_row = S::HEADS > 1 ? 0 : (warp * C::GROUPS_PER_WARP + gi) * 16;
                if (grp_row >= valid || no_math) break;           // warp-uniform
                const int grp_valid = valid - grp_row;            // >= 1; short only in a sequence's last group
                const int box_head = S::HEADS > 1 ? warp : 0;
                auto rows = [&](int t, int panel) { return row_offset<KV, S::HEADS>(t, panel, btl, box_head); };
                if constexpr (FP8)
                    wrote |= process_group_e4m3(k_tile, v_tile, rows, grp_row, grp_valid, qb, acc, m_run, l_run, qk_scale, lane);
                else
                    wrote |= process_group_f16(k_tile, v_tile, rows, grp_row, grp_valid, qb, acc, m_run, l_run, qk_scale, lane);
            }

            // Release the stage to the producer.
            if (wrote) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(stage));
            if (++c_stage == nst) { c_stage = 0; c_phase ^= 1; }
            tiles_done++;
        }
        if (!alive) break;

        // ---- segment end: merge the warps' softmax states and write the result.
        // Accumulator mt of a lane: dims 16mt + g (values 0, 1) and 16mt + g + 8 (values 2, 3), heads 2qd, 2qd+1.
        {
            float l[2] = {l_run[0], l_run[1]};
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                l[0] += __shfl_xor_sync(0xffffffffu, l[0], o);
                l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
            }
            if constexpr (S::HEADS > 1) {
                // Head-fused: this warp owns kv head `warp` of row sg.x outright.  Work items are rows:
                // item_seg_begin is indexed by row, partials by (segment, query head).  Nothing is exchanged
                // between warps.  A whole row goes through the warp's staging rows in shared memory so that it
                // leaves as 16-byte stores, 512 contiguous bytes per instruction (to every peer's buffer when
                // the output is gathered); a piece of a split row is stored as fp32 partials from the fragments.
                const int s0 = p.item_seg_begin[sg.x], s1 = p.item_seg_begin[sg.x + 1];
                const bool whole_row = s1 - s0 == 1;
                __half* stage_rows = reinterpret_cast<__half*>(gen + S::OUT_STAGE_OFFSET) + warp * (GROUP * HEAD_DIM);
                if (whole_row) __syncwarp();   // the previous row's chunks have been read
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int hd = 2 * qd + h;
                    if (hd < GROUP) {
                        const int hq = warp * GROUP + hd;
                        const float inv = v_scale / l[h];
                        const size_t prow = (static_cast<size_t>(seg) * p.num_q_heads + hq) * HEAD_DIM;
#pragma unroll
                        for (int mt = 0; mt < 8; mt++) {
                            const int d0 = 16 * mt + g, d1 = d0 + 8;
                            const float o0 = acc[mt][h] * inv, o1 = acc[mt][2 + h] * inv;
                            if (whole_row) {
                                stage_rows[hd * HEAD_DIM + d0] = __float2half(o0);
                                stage_rows[hd * HEAD_DIM + d1] = __float2half(o1);
                            } else {
                                p.partial_out[prow + d0] = o0;
                                p.partial_out[prow + d1] = o1;
                            }
                        }
                        if (!whole_row && g == 0)
                            p.partial_lse[static_cast<size_t>(seg) * p.num_q_heads + hq] = m_run[h] + log2f(l[h]);
                    }
                }
                if (whole_row) {
                    __syncwarp();
                    const size_t orow = out_index(p, gp, sg.x, warp * GROUP);   // the group's heads are consecutive rows of 128
                    for (int c = lane; c < GROUP * 16; c += 32)
                        store_out(p, gp, orow + c * 8, *reinterpret_cast<const uint4*>(stage_rows + c * 8));
                }
                if (!whole_row && (p.needs_merge == MERGE_IN_KERNEL ||
                                   (p.needs_merge == MERGE_HYBRID && s1 - s0 <= HYBRID_MAX_PIECES))) {
                    // one arrival counter per (row, kv head); the warp that completes it merges the head's group
                    int* counter = reinterpret_cast<int*>(p.partial_lse + static_cast<size_t>(p.cta_seg_begin[p.num_ctas]) * p.num_q_heads)
                                   + sg.x * S::HEADS + warp;
                    __threadfence();
                    __syncwarp();
                    int seen = 0;
                    if (lane == 0) seen = atomicAdd(counter, 1);
                    seen = __shfl_sync(0xffffffffu, seen, 0);
                    if (seen == s1 - s0 - 1) {
                        __threadfence();
                        merge_item<GROUP>(p, gp, sg.x, warp, s0, s1, lane, p.num_q_heads, warp * GROUP);
                        if (lane == 0) *counter = 0;
                    }
                }
                continue;
            }
            const int item = sg.x * p.num_kv_heads + sg.y;
            const bool whole = p.item_seg_begin[item + 1] - p.item_seg_begin[item] == 1;
#pragma unroll
            for (int pass = 0; pass < S::PASSES; pass++) {
                const int head0 = pass * 4;   // heads [head0, head0 + GROUP_PAD) in this pass
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int head = 2 * qd + h;
                    if (head < GROUP && head >= head0 && head < head0 + S::GROUP_PAD) {
                        float* row = w_o + (warp * S::GROUP_PAD + (head - head0)) * OSTRIDE;
#pragma unroll
                        for (int mt = 0; mt < 8; mt++) {
                            row[16 * mt + g]     = acc[mt][h];
                            row[16 * mt + g + 8] = acc[mt][2 + h];
                        }
                        if (g == 0) { w_m[warp * 8 + head] = m_run[h]; w_l[warp * 8 + head] = l[h]; }
                    }
                }
                if (!consumer_sync()) break;
                // every thread combines four consecutive dims of one head over the warps: the outputs leave as
                // 8-byte (fp16 row) or 16-byte (fp32 partial) stores, 256 or 512 contiguous bytes per warp
                constexpr int HEADS = GROUP < S::GROUP_PAD ? GROUP : S::GROUP_PAD;
                for (int i = tid; i < HEADS * (HEAD_DIM / 4); i += S::CONSUMERS) {
                    const int hl = i / (HEAD_DIM / 4), d = (i % (HEAD_DIM / 4)) * 4, hd = head0 + hl;
                    float m_all = -INFINITY;
#pragma unroll
                    for (int w = 0; w < C::WARPS; w++) m_all = fmaxf(m_all, w_m[w * 8 + hd]);
                    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
                    float den = 0.f;
#pragma unroll
                    for (int w = 0; w < C::WARPS; w++) {
                        const float wt = exp2f(w_m[w * 8 + hd] - m_all);   // 0 for warps that saw no tokens
                        const float4 o = *reinterpret_cast<const float4*>(w_o + (w * S::GROUP_PAD + hl) * OSTRIDE + d);
                        num.x = fmaf(wt, o.x, num.x); num.y = fmaf(wt, o.y, num.y);
                        num.z = fmaf(wt, o.z, num.z); num.w = fmaf(wt, o.w, num.w);
                        den = fmaf(wt, w_l[w * 8 + hd], den);
                    }
                    const float4 o = make_float4(num.x / den * v_scale, num.y / den * v_scale, num.z / den * v_scale, num.w / den * v_scale);
                    if (whole) {
                        const __half2 lo = __floats2half2_rn(o.x, o.y), hi = __floats2half2_rn(o.z, o.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                        store_out(p, gp, out_index(p, gp, sg.x, sg.y * GROUP + hd) + d, packed);
                    } else {
                        const size_t row = static_cast<size_t>(seg) * GROUP + hd;
                        *reinterpret_cast<float4*>(p.partial_out + row * HEAD_DIM + d) = o;
                        if (d == 0) p.partial_lse[row] = m_all + log2f(den);
                    }
                }
                if (!consumer_sync()) break;   // scratch is rewritten by the next pass / segment
            }
            const int s0 = p.item_seg_begin[item], s1 = p.item_seg_begin[item + 1];
            if (alive && !whole && (p.needs_merge == MERGE_IN_KERNEL ||
                                    (p.needs_merge == MERGE_HYBRID && s1 - s0 <= HYBRID_MAX_PIECES))) {
                // Last one in merges: every consumer warp of every segment of this (row, kv head)
                // publishes its partial stores and counts itself; the warp that completes the count
                // finds all partials visible and combines them, then re-arms the counter.
                int* counter = reinterpret_cast<int*>(p.partial_lse + static_cast<size_t>(p.cta_seg_begin[p.num_ctas]) * GROUP) + item;
                __threadfence();
                __syncwarp();
                int seen = 0;
                if (lane == 0) seen = atomicAdd(counter, 1);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen == (s1 - s0) * C::WARPS - 1) {
                    __threadfence();
                    merge_item<GROUP>(p, gp, sg.x, sg.y, s0, s1, lane);
                    if (lane == 0) *counter = 0;
                }
            }
        }
    }
    if (st.slots && tid == 0) {
        // results unused: these compile to reductions the thread does not wait for
        atomicAdd(st.slots + 2 * blockIdx.x, global_ns() - t_entry);
        atomicAdd(st.slots + 2 * blockIdx.x + 1, static_cast<unsigned long long>(tiles_done));
        if (blockIdx.x == 0) atomicAdd(st.slots + 2 * gridDim.x, 1ull);
    }
}

// ---- merge kernel -------------------------------------------------------------------
// One CTA of four warps per (row, query head) whose (row, kv head) was split.
// Up to MERGE_WIDE_MIN pieces: warp 0 alone, lanes first over the segments (max and sum of the base-2
// LSE weights by butterfly shuffles), then over the head dimension, four floats per lane, with each
// segment's weight broadcast by shuffle: the arithmetic of merge_segments_kernel
// (src/decode/decode_kernels.cuh:409-432), in the order the decode kernel's own merge uses, so both give
// the same bits.  More pieces (one long sequence spread over the whole grid: dozens per row): the four
// warps take every fourth piece each, four loads in flight per warp, and add up through shared memory;
// with one warp per (row, head) such a merge was a third of a single-sequence decode step.
// ROW_ITEMS = true: the plan's work items are rows (head-fused tiles).
constexpr int MERGE_WIDE_MIN = 8;
// One (row, query head) pair by the four warps of a CTA; s0, s1: the pair's segment range.
template<int GROUP, bool ROW_ITEMS>
__device__ __forceinline__ void merge_pair(const pd_params& p, int idx, int s0, int s1, int seg_limit, float4 (*part_num)[32], float* part_den)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = idx / p.num_q_heads, hq = idx % p.num_q_heads;
    if (s1 - s0 <= 1) return;   // written directly by the decode kernel
    if (seg_limit > 0 && s1 > seg_limit) return;   // beyond a fixed-size workspace: the decode kernel has reported it
    if (p.needs_merge == MERGE_HYBRID && s1 - s0 <= HYBRID_MAX_PIECES) return;   // merged by the decode kernel
    GatherOut local{};   // world = 0: plain output
    const int stride = ROW_ITEMS ? p.num_q_heads : GROUP;
    const int gq     = ROW_ITEMS ? hq : hq % GROUP;
    if (s1 - s0 <= MERGE_WIDE_MIN) {
        if (warp == 0) merge_one_head<GROUP>(p, local, b, hq, s0, s1, lane, stride, gq);
        return;
    }
    float lse_max = -INFINITY;
    for (int s = s0 + lane; s < s1; s += 32) lse_max = fmaxf(lse_max, __ldcg(p.partial_lse + s * stride + gq));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lse_max = fmaxf(lse_max, __shfl_xor_sync(0xffffffffu, lse_max, o));
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (int base = s0 + warp; base < s1; base += 16) {
        float  w[4];
        float4 o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = base + 4 * j;
            const bool live = s < s1;
            w[j] = live ? exp2f(__ldcg(p.partial_lse + s * stride + gq) - lse_max) : 0.f;
            o[j] = live ? __ldcg(reinterpret_cast<const float4*>(
                              p.partial_out + (static_cast<size_t>(s) * stride + gq) * HEAD_DIM + lane * 4))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            num.x = fmaf(w[j], o[j].x, num.x); num.y = fmaf(w[j], o[j].y, num.y);
            num.z = fmaf(w[j], o[j].z, num.z); num.w = fmaf(w[j], o[j].w, num.w);
            den += w[j];
        }
    }
    part_num[warp][lane] = num;
    if (lane == 0) part_den[warp] = den;
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int w = 1; w < 4; w++) {
        const float4 other = part_num[w][lane];
        num.x += other.x; num.y += other.y; num.z += other.z; num.w += other.w;
        den += part_den[w];
    }
    const __half2 lo = __floats2half2_rn(num.x / den, num.y / den);
    const __half2 hi = __floats2half2_rn(num.z / den, num.w / den);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    store_out(p, local, out_index(p, local, b, hq) + lane * 4, packed);
}

// WALK = false: one CTA per pair (grid = pairs).  WALK = true: a capped grid whose CTAs walk their pairs;
// used when there are thousands of pairs, which is where this kernel is launched although almost every
// pair is done after reading two integers (plans cut on the device).
template<int GROUP, bool ROW_ITEMS = false, bool WALK = false>
__global__ void __launch_bounds__(128)
merge_segments_kernel(const __grid_constant__ pd_params p, const int seg_limit)
{
    __shared__ float4 part_num[4][32];
    __shared__ float  part_den[4];
    const int pairs = p.batch * p.num_q_heads;
    auto item_of = [&](int idx) {
        const int b = idx / p.num_q_heads, hq = idx % p.num_q_heads;
        return ROW_ITEMS ? b : b * p.num_kv_heads + hq / GROUP;
    };
    // Launched as a programmatic dependent of the decode kernel: the CTAs may already be resident while
    // the decode kernel drains.  The plan arrays were written before that kernel started, so the first
    // pair's bounds are fetched ahead of the wait; everything else read below is that kernel's output.
    int s0 = 0, s1 = 0;
    if (static_cast<int>(blockIdx.x) < pairs) {
        s0 = p.item_seg_begin[item_of(blockIdx.x)];
        s1 = p.item_seg_begin[item_of(blockIdx.x) + 1];
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (static_cast<int>(blockIdx.x) >= pairs) return;
    merge_pair<GROUP, ROW_ITEMS>(p, blockIdx.x, s0, s1, seg_limit, part_num, part_den);
    if constexpr (WALK) {
        for (int idx = blockIdx.x + gridDim.x; idx < pairs; idx += gridDim.x) {
            __syncthreads();   // the scratch is reused
            merge_pair<GROUP, ROW_ITEMS>(p, idx, p.item_seg_begin[item_of(idx)], p.item_seg_begin[item_of(idx) + 1],
                                         seg_limit, part_num, part_den);
        }
    }
}

// Waits (bounded) until every peer's flag has reached `epoch`: their slices are in this GPU's
// gathered buffer.  One warp, lane r watches peer r.  Gives up after about a second and records
// ST_GATHER_TIMEOUT << 24 | peer in the status word; the context stays usable.
// Raises flags[r][rank] = epoch on every rank r.  Launched as a programmatic dependent right behind the decode
// kernel whose rows it announces: its warp may be resident early, but it does nothing until that grid has
// completed and its stores, the ones into the peers' buffers included, have been performed
// (griddepcontrol.wait); the system-scope fence then orders them before the flags for whoever polls them.
// wait_flags != null: the same warp then waits (bounded) until every rank's flag in this GPU's own array has
// reached the epoch, i.e. the whole gathered layer is here - one dependent launch instead of two for callers
// that want the step complete before anything else runs.
__global__ void gather_signal_kernel(const __grid_constant__ GatherFlags gf, int world, int rank, unsigned epoch,
                                     const unsigned* wait_flags, unsigned* status)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();
    volatile unsigned* f = gf.flags[r] + rank;
    *f = epoch;
    if (wait_flags) {
        const volatile unsigned* w = wait_flags + r;
        const long long t0 = clock64();
        while (static_cast<int>(*w - epoch) < 0) {
            if (clock64() - t0 > (1ll << 31)) {
                atomicCAS(status, 0u, (ST_GATHER_TIMEOUT << 24) | static_cast<unsigned>(r));
                break;
            }
            __nanosleep(100);
        }
        __threadfence_system();
    }
}

// Launched as a programmatic dependent of the kernel before it in the stream (the decode whose rows it waits
// for, or any other): its one warp may be resident and polling while that kernel drains, which takes the
// launch latency out of the path; it returns only after that kernel has completed as well
// (griddepcontrol.wait), so whatever follows in the stream sees both the local and the peers' rows.
__global__ void gather_wait_kernel(const unsigned* flags, int world, unsigned epoch, unsigned* status)
{
    const int r = threadIdx.x;
    if (r < world) {
        const volatile unsigned* f = flags + r;
        const long long t0 = clock64();
        while (static_cast<int>(*f - epoch) < 0) {
            if (clock64() - t0 > (1ll << 31)) {
                atomicCAS(status, 0u, (ST_GATHER_TIMEOUT << 24) | static_cast<unsigned>(r));
                break;
            }
            __nanosleep(200);
        }
        __threadfence_system();
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace pdk
