#pragma once
// Head-fused paged decode in which CTAs that run out of work take work from CTAs that still have some.
//
// The plan (src/decode/decode.cu:65-108 of the reference) cuts a step into equal shares before the launch.
// SMs do not stream at the same rate and the rate of one SM moves from launch to launch, so the CTAs of one
// launch finish several percent apart, and while the last ones finish, DRAM is no longer kept busy.  Here a
// CTA's producer warp publishes, in one 64-bit word per CTA, which tiles of its current segment it has not
// issued yet.  A CTA whose own segments are all issued looks for the CTA with the most tiles left, cuts the
// back half off with one compare-and-swap, and streams that half as a piece of its own: same row, its own
// slot in the split-row workspace, merged with the row's other pieces by whichever piece finishes last.
//
// Nothing waits on another CTA: the word is read, swapped or added to, never spun on, and the arrival
// count of a row is an atomic add whose result says who is last.  The kernel is the head-fused shape of
// paged_decode_kernel (one consumer warp per kv head, rows as work items) with two changes:
//  * consumers do not walk the plan; every pipeline stage carries a tag written by the producer (first tile
//    of a piece, plain tile, end of piece, exit), because only the producer knows where a piece ends;
//  * a row's arrival counter counts weights: a segment of the plan adds 65536 minus the pieces taken from
//    it, a taken piece adds 1, and the row is complete at 65536 x (segments of the row).  A segment's own
//    count of taken pieces is final when its owner's claim fails, which is before the owner arrives, so no
//    sum short of the total can be mistaken for it.

#include "decode_kernel.cuh"

namespace pdk {

constexpr int STEALS_PER_SEG  = 15;   // pieces that may be cut off one segment (4 bits of the word)
constexpr int STEALS_PER_CTA  = 4;    // pieces one CTA may take per launch (each has its own workspace slot)
#ifndef PD_B200_STEAL_MIN_TILES
#define PD_B200_STEAL_MIN_TILES 4
#endif
constexpr int STEAL_MIN_TILES = PD_B200_STEAL_MIN_TILES;   // unissued tiles below which a segment is left alone
constexpr int PIECE_TAKEN     = 1 << 30;   // piece id: a slot of the taken-piece workspace, not a plan segment

struct StealArgs {
    unsigned long long* words;       // [grid]: segment ordinal | pieces taken | next tile to issue | end tile
    int*   seg_nsteal;               // [segments]: pieces taken from a segment, written by its owner when it ends
    int*   seg_slots;                // [segments][STEALS_PER_SEG]: workspace slots of those pieces
    float* out;                      // [grid * STEALS_PER_CTA][num_q_heads][128] partial rows of taken pieces
    float* lse;                      // [grid * STEALS_PER_CTA][num_q_heads]
    unsigned long long* count;       // pieces taken since the process started (may be null)
};

// word: [63:52] ordinal of the segment within its CTA, [51:48] pieces taken, [47:24] next tile the owner
// will claim, [23:0] end tile; tiles are counted from the segment's first token.
__device__ __forceinline__ unsigned long long sw_pack(int ord, int taken, int front, int end) {
    return (static_cast<unsigned long long>(ord) << 52) | (static_cast<unsigned long long>(taken) << 48) |
           (static_cast<unsigned long long>(front) << 24) | static_cast<unsigned long long>(end);
}
__device__ __forceinline__ int sw_ord(unsigned long long w)   { return static_cast<int>(w >> 52); }
__device__ __forceinline__ int sw_taken(unsigned long long w) { return static_cast<int>(w >> 48) & 15; }
__device__ __forceinline__ int sw_front(unsigned long long w) { return static_cast<int>(w >> 24) & 0xffffff; }
__device__ __forceinline__ int sw_end(unsigned long long w)   { return static_cast<int>(w) & 0xffffff; }
constexpr unsigned long long SW_FRONT_ONE = 1ull << 24;
constexpr int SW_MAX_ORD   = 4095;
constexpr int SW_MAX_TILES = (1 << 24) - 2;

// stage tags
constexpr int TAG_TILE  = 0;
constexpr int TAG_FIRST = 1;   // first tile of a piece: y = row, w = piece id
constexpr int TAG_END   = 2;   // no data; y = pieces taken from the piece that ends
constexpr int TAG_EXIT  = 3;

template<typename KV, int GROUP, typename C>
struct StealShape {
    using S = Shape<KV, GROUP, C>;
    static constexpr int TAG_OFFSET = S::OUT_STAGE_OFFSET + S::OUT_STAGE_BYTES;
    static constexpr int SMEM_BYTES = S::SMEM_BYTES + 16 * C::STAGES + 16;
};

// Merge of one (row, kv head) whose pieces are the row's plan segments [s0, s1) and whatever was taken
// from them: at most 32 pieces (the taker's rule).  Same arithmetic as merge_item.
template<int GROUP>
__device__ __forceinline__ void merge_row_pieces(const pd_params& p, const GatherOut& gp, const StealArgs& sa, int b,
                                                 int kv_head, int s0, int s1, int lane)
{
    const int stat = s1 - s0;
    const int mine = lane < stat ? 1 + __ldcg(sa.seg_nsteal + s0 + lane) : 0;   // pieces of segment s0 + lane
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    const int n = min(32, __shfl_sync(0xffffffffu, incl, 31));
    const int excl = incl - mine;
    int j = 0;                                  // segment of piece `lane`: the first one whose running count exceeds it
    for (int i = 0; i < stat; i++) {
        const int e = __shfl_sync(0xffffffffu, incl, i);
        if (lane >= e) j = i + 1;
    }
    const int base = __shfl_sync(0xffffffffu, excl, j & 31);
    int id = 0;
    if (lane < n) {
        const int k = lane - base;
        id = k == 0 ? s0 + j : (PIECE_TAKEN | __ldcg(sa.seg_slots + (s0 + j) * STEALS_PER_SEG + k - 1));
    }
    const int hq_n = p.num_q_heads, first = kv_head * GROUP;
    auto lse_of = [&](int piece) {
        return (piece & PIECE_TAKEN) ? sa.lse + static_cast<size_t>(piece & (PIECE_TAKEN - 1)) * hq_n
                                     : p.partial_lse + static_cast<size_t>(piece) * hq_n;
    };
    auto out_of = [&](int piece) {
        return (piece & PIECE_TAKEN) ? sa.out + static_cast<size_t>(piece & (PIECE_TAKEN - 1)) * hq_n * HEAD_DIM
                                     : p.partial_out + static_cast<size_t>(piece) * hq_n * HEAD_DIM;
    };
    float w[GROUP], den[GROUP];
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) w[hd] = lane < n ? __ldcg(lse_of(id) + first + hd) : -INFINITY;
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) {
        float mx = w[hd];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        w[hd] = exp2f(w[hd] - mx);
        den[hd] = 0.f;
    }
    float4 num[GROUP];
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) num[hd] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
    for (int q = 0; q < n; q++) {
        const float* rows = out_of(__shfl_sync(0xffffffffu, id, q)) + static_cast<size_t>(first) * HEAD_DIM + lane * 4;
        float4 o[GROUP];
#pragma unroll
        for (int hd = 0; hd < GROUP; hd++) o[hd] = __ldcg(reinterpret_cast<const float4*>(rows + hd * HEAD_DIM));
#pragma unroll
        for (int hd = 0; hd < GROUP; hd++) {
            const float wq = __shfl_sync(0xffffffffu, w[hd], q);
            num[hd].x = fmaf(wq, o[hd].x, num[hd].x); num[hd].y = fmaf(wq, o[hd].y, num[hd].y);
            num[hd].z = fmaf(wq, o[hd].z, num[hd].z); num[hd].w = fmaf(wq, o[hd].w, num[hd].w);
            den[hd] += wq;
        }
    }
#pragma unroll
    for (int hd = 0; hd < GROUP; hd++) {
        const __half2 lo = __floats2half2_rn(num[hd].x / den[hd], num[hd].y / den[hd]);
        const __half2 hi = __floats2half2_rn(num[hd].z / den[hd], num[hd].w / den[hd]);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        store_out(p, gp, out_index(p, gp, b, first + hd) + lane * 4, packed);
    }
}

template<typename KV, int GROUP, typename C>
__global__ void __launch_bounds__((C::WARPS + 1) * 32, 1)
paged_decode_steal_kernel(const __grid_constant__ pd_params p, const __grid_constant__ CUtensorMap k_map,
                          const __grid_constant__ CUtensorMap v_map, const int btl /* log2(tokens per box) */,
                          unsigned* __restrict__ status, const __grid_constant__ GatherOut gp,
                          const __grid_constant__ HeadScales hs, const __grid_constant__ CtaStats st,
                          const __grid_constant__ StealArgs sa)
{
    static_assert(C::HEADS > 1, "rows as work items: the head-fused tile shape only");
    const unsigned long long t_entry = (st.slots && threadIdx.x == 0) ? global_ns() : 0ull;
    using S = Shape<KV, GROUP, C>;
    using SS = StealShape<KV, GROUP, C>;
    constexpr bool FP8 = sizeof(KV) == 1;
    constexpr int STAGES = C::STAGES;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t pipe = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (pipe - smem_u32(smem_raw));
    const uint32_t bars = pipe + S::PIPE_BYTES + S::Q_BYTES + S::MERGE_BYTES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + S::PIPE_BYTES + S::Q_BYTES + S::MERGE_BYTES + 2 * STAGES * 8 + 8);
    const uint32_t tags = pipe + SS::TAG_OFFSET;
    auto full_bar  = [&](int s) { return bars + s * 8; };
    auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int seg_begin = p.cta_seg_begin[blockIdx.x];
    const int seg_end   = p.cta_seg_begin[blockIdx.x + 1];
    if (seg_begin >= seg_end) return;

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == C::WARPS * 32) {
        asm volatile("prefetch.tensormap [%0];" :: "l"(&k_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&v_map) : "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), C::WARPS); }
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
        const int bt_tokens = 1 << btl;
        const int bpt       = S::TILE >> btl;                 // boxes per tile, <= 32
        const uint32_t box_bytes = static_cast<uint32_t>(bt_tokens) * S::ROW_BYTES * S::HEADS;
        const uint64_t pol = l2_evict_first_policy();
        const int ps = p.page_size;
        const int chunk_tiles = 32 / bpt;                     // lane l owns box l of a chunk
        int issued = 0, p_stage = 0;
        uint32_t p_phase = 0;

        auto acquire = [&]() -> bool {
            if (!mbar_wait(empty_bar(p_stage), p_phase ^ 1)) { if (lane == 0) fail(ST_EMPTY_TIMEOUT); return false; }
            return *abort_flag == 0;
        };
        auto advance = [&]() { issued++; if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1; } };
        auto write_tag = [&](int x, int y, int z, int w) {
            asm volatile("st.shared.v4.s32 [%0], {%1, %2, %3, %4};" :: "r"(tags + p_stage * 16), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
        };
        // a stage without data: the end of a piece, or the end of the CTA's work
        auto post = [&](int kind, int y) -> bool {
            if (!acquire()) return false;
            if (lane == 0) { write_tag(kind, y, 0, 0); mbar_arrive(full_bar(p_stage)); }
            __syncwarp();
            advance();
            return true;
        };
        auto table_of = [&](int b) {
            const int slot = p.slot_ids ? __ldg(p.slot_ids + b) : b;
            return p.block_table + static_cast<size_t>(slot) * p.block_table_stride;
        };

        // Tiles [first, last) of the segment sg, tile t being tokens sg.z + t * TILE onwards.  on_offer: the piece
        // is this CTA's own segment number ord, and the tiles it has not claimed yet can be taken by others, so
        // every tile beyond the first few is claimed (one atomic add, sent one tile early) before it is issued.
        // Returns how many pieces others took from it, or -1 after a failure.
        auto run_piece = [&](const int4 sg, const int* bt, int first, int last, bool on_offer, int ord, int piece_id) -> int {
            int claimed = last;
            if (on_offer) {
                claimed = min(last, first + STAGES);
                if (lane == 0) atomicExch(sa.words + blockIdx.x, sw_pack(ord, 0, claimed, last));
            }
            unsigned long long pending = 0;
            int taken = 0;
            bool done = false;
            auto page_at = [&](int tile0) {
                const int t = sg.z + tile0 * S::TILE + (lane << btl);
                return t < sg.w ? __ldg(bt + t / ps) : 0;
            };
            int tc = first;
            int page = page_at(tc);
            while (!done) {
                const int n_page = page_at(tc + chunk_tiles);   // in flight while this chunk is issued
                for (int ti = 0; ti < chunk_tiles; ti++) {
                    const int t = tc + ti;
                    if (t >= claimed) {
                        if (t >= last) { done = true; break; }              // every tile was ours: nothing was taken
                        const unsigned long long r = __shfl_sync(0xffffffffu, pending, 0);
                        if (sw_front(r) >= sw_end(r)) { taken = sw_taken(r); done = true; break; }   // the rest went to others
                        claimed = sw_front(r) + 1;
                    }
                    if (!acquire()) return -1;
                    const int tile_tok = sg.z + t * S::TILE;
                    const int valid = sg.w - tile_tok;            // may exceed TILE
                    const int nb = (min(valid, S::TILE) + bt_tokens - 1) >> btl;
                    if (lane == 0) {
                        write_tag(t == first ? TAG_FIRST : TAG_TILE, sg.x, valid, piece_id);
                        mbar_expect_tx(full_bar(p_stage), 2u * nb * box_bytes);
                    }
                    __syncwarp();
                    const int j = lane - ti * bpt;
                    if (j >= 0 && j < nb) {
                        const uint32_t k_dst = pipe + p_stage * S::STAGE_BYTES + j * box_bytes;
                        const uint32_t v_dst = k_dst + S::TILE_BYTES;
                        const int tok_in_page = (tile_tok + (j << btl)) % ps;
                        if constexpr (FP8) {
                            tma_load_4d(k_dst, &k_map, full_bar(p_stage), 0, tok_in_page, 0, page, pol);
                            tma_load_4d(v_dst, &v_map, full_bar(p_stage), 0, tok_in_page, 0, page, pol);
                        } else {
                            tma_load_5d(k_dst, &k_map, full_bar(p_stage), 0, tok_in_page, 0, 0, page, pol);
                            tma_load_5d(v_dst, &v_map, full_bar(p_stage), 0, tok_in_page, 0, 0, page, pol);
                        }
                    }
                    advance();
                    if (on_offer && t + 1 == claimed && claimed < last && lane == 0)
                        pending = atomicAdd(sa.words + blockIdx.x, SW_FRONT_ONE);
                }
                tc += chunk_tiles;
                page = n_page;
            }
            return post(TAG_END, taken) ? taken : -1;
        };

        bool ok = true;
        // the CTA's own segments
        int4 sg = __ldg(segments + seg_begin);
        const int* bt = table_of(sg.x);
        for (int seg = seg_begin; ok && seg < seg_end; seg++) {
            int4 n_sg = sg;
            const int* n_bt = bt;
            if (seg + 1 < seg_end) { n_sg = __ldg(segments + seg + 1); n_bt = table_of(n_sg.x); }
            const int ntiles = (sg.w - sg.z + S::TILE - 1) / S::TILE;
            const int ord = seg - seg_begin;
            ok = run_piece(sg, bt, 0, ntiles, ord <= SW_MAX_ORD && ntiles <= SW_MAX_TILES, ord, seg) >= 0;
            sg = n_sg; bt = n_bt;
        }
        // then pieces of other CTAs' segments
        for (int k = 0; ok && k < STEALS_PER_CTA; k++) {
            bool got = false;
            int v_seg = 0, v_first = 0, v_last = 0, v_nth = 0;
            int4 v_sg = make_int4(0, 0, 0, 0);
            for (int attempt = 0; attempt < 3 && !got; attempt++) {
                unsigned long long best_key = 0, best_w = 0;
                for (int c = lane; c < p.num_ctas; c += 32) {
                    const unsigned long long w = *reinterpret_cast<volatile unsigned long long*>(sa.words + c);
                    const int rem = sw_end(w) - sw_front(w);
                    if (c != static_cast<int>(blockIdx.x) && rem >= STEAL_MIN_TILES && sw_taken(w) < STEALS_PER_SEG) {
                        const unsigned long long key = (static_cast<unsigned long long>(rem) << 32) | static_cast<unsigned>(c);
                        if (key > best_key) { best_key = key; best_w = w; }
                    }
                }
                unsigned long long top = best_key;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, top, o);
                    top = other > top ? other : top;
                }
                if (top == 0) break;                                      // nobody has enough left
                const int src = __ffs(__ballot_sync(0xffffffffu, best_key == top)) - 1;
                unsigned long long w = __shfl_sync(0xffffffffu, best_w, src);
                const int v = static_cast<int>(top & 0xffffffffu);
                const int ord = sw_ord(w);
                v_seg = __ldg(p.cta_seg_begin + v) + ord;
                v_sg = __ldg(segments + v_seg);
                const int pieces = __ldg(p.item_seg_begin + v_sg.x + 1) - __ldg(p.item_seg_begin + v_sg.x);
                const int allowed = min(STEALS_PER_SEG, 32 / max(pieces, 1) - 1);   // a row stays within 32 pieces
                int won = 0, f = 0, e = 0, s = 0;
                if (lane == 0) {
                    for (int tries = 0; tries < 4; tries++) {
                        f = sw_front(w); e = sw_end(w); s = sw_taken(w);
                        if (sw_ord(w) != ord || e - f < STEAL_MIN_TILES || s >= allowed) break;
                        const int ne = e - (e - f) / 2;
                        const unsigned long long old = atomicCAS(sa.words + v, w, sw_pack(ord, s + 1, f, ne));
                        if (old == w) { won = 1; f = ne; break; }
                        w = old;
                    }
                }
                got = __shfl_sync(0xffffffffu, won, 0) != 0;
                v_first = __shfl_sync(0xffffffffu, f, 0);
                v_last  = __shfl_sync(0xffffffffu, e, 0);
                v_nth   = __shfl_sync(0xffffffffu, s, 0);
            }
            if (!got) break;
            const int slot = blockIdx.x * STEALS_PER_CTA + k;
            if (lane == 0) {
                sa.seg_slots[v_seg * STEALS_PER_SEG + v_nth] = slot;
                __threadfence();
                if (sa.count) atomicAdd(sa.count, 1ull);
            }
            ok = run_piece(v_sg, table_of(v_sg.x), v_first, v_last, false, 0, PIECE_TAKEN | slot) >= 0;
        }
        if (ok) ok = post(TAG_EXIT, 0);
        if (!ok || *abort_flag) {
            for (int i = 0; i < min(issued, STAGES); i++) {
                int s = p_stage - 1 - i;
                uint32_t par = p_phase;
                if (s < 0) { s += STAGES; par ^= 1; }
                if (!mbar_wait(full_bar(s), par)) { if (lane == 0) fail(ST_DRAIN_TIMEOUT); break; }
            }
        }
        return;
    }

    // ================= consumer warps: warp w owns kv head w =================
    const int g  = lane >> 2;
    const int qd = lane & 3;
    float qk_scale = p.sm_scale * p.k_scale * 1.4426950408889634f;
    float v_scale  = p.v_scale;
    if (hs.k) qk_scale = p.sm_scale * __ldg(hs.k + warp) * 1.4426950408889634f;
    if (hs.v) v_scale = __ldg(hs.v + warp);

    float acc[8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qb[8][2];
    unsigned tiles_done = 0;
    int c_stage = 0;
    uint32_t c_phase = 0;
    int row = 0, piece = 0;
    const int total_segments = p.cta_seg_begin[p.num_ctas];

    for (;;) {
        const int stage = c_stage;
        if (!mbar_wait(full_bar(stage), c_phase)) { if (lane == 0) fail(ST_FULL_TIMEOUT); break; }
        if (*abort_flag) break;
        if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1; }
        const uint4 tag = lds128(tags + stage * 16);
        const int kind = static_cast<int>(tag.x);

        if (kind >= TAG_END) {
            __syncwarp();                                    // every lane has its copy of the tag
            if (lane == 0) mbar_arrive(empty_bar(stage));
            if (kind == TAG_EXIT) break;
            // ---- end of a piece.  Accumulator mt of a lane: dims 16mt + g (values 0, 1) and 16mt + g + 8
            // (values 2, 3), heads 2qd, 2qd + 1.
            const int taken_from_it = static_cast<int>(tag.y);
            float l[2] = {l_run[0], l_run[1]};
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                l[0] += __shfl_xor_sync(0xffffffffu, l[0], o);
                l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
            }
            const bool is_taken = (piece & PIECE_TAKEN) != 0;
            const int slot = piece & (PIECE_TAKEN - 1);
            const int s0 = p.item_seg_begin[row], s1 = p.item_seg_begin[row + 1];
            const bool whole_row = !is_taken && s1 - s0 == 1 && taken_from_it == 0;
            float* part_out = (is_taken ? sa.out : p.partial_out) + static_cast<size_t>(slot) * p.num_q_heads * HEAD_DIM;
            float* part_lse = (is_taken ? sa.lse : p.partial_lse) + static_cast<size_t>(slot) * p.num_q_heads;
            __half* stage_rows = reinterpret_cast<__half*>(gen + S::OUT_STAGE_OFFSET) + warp * (GROUP * HEAD_DIM);
            if (whole_row) __syncwarp();
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int hd = 2 * qd + h;
                if (hd < GROUP) {
                    const int hq = warp * GROUP + hd;
                    const float inv = v_scale / l[h];
#pragma unroll
                    for (int mt = 0; mt < 8; mt++) {
                        const int d0 = 16 * mt + g, d1 = d0 + 8;
                        const float o0 = acc[mt][h] * inv, o1 = acc[mt][2 + h] * inv;
                        if (whole_row) {
                            stage_rows[hd * HEAD_DIM + d0] = __float2half(o0);
                            stage_rows[hd * HEAD_DIM + d1] = __float2half(o1);
                        } else {
                            part_out[hq * HEAD_DIM + d0] = o0;
                            part_out[hq * HEAD_DIM + d1] = o1;
                        }
                    }
                    if (!whole_row && g == 0) part_lse[hq] = m_run[h] + log2f(l[h]);
                }
            }
            if (whole_row) {
                __syncwarp();
                const size_t orow = out_index(p, gp, row, warp * GROUP);
                for (int c = lane; c < GROUP * 16; c += 32)
                    store_out(p, gp, orow + c * 8, *reinterpret_cast<const uint4*>(stage_rows + c * 8));
            } else {
                // every warp leaves the segment's count before its own arrival: the warp that merges this kv
                // head may run before the other warps of this CTA get here
                if (!is_taken && lane == 0) sa.seg_nsteal[slot] = taken_from_it;
                int* counter = reinterpret_cast<int*>(p.partial_lse + static_cast<size_t>(total_segments) * p.num_q_heads)
                               + row * S::HEADS + warp;
                const int weight = is_taken ? 1 : (1 << 16) - taken_from_it;
                __threadfence();
                __syncwarp();
                int seen = 0;
                if (lane == 0) seen = atomicAdd(counter, weight);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen + weight == (s1 - s0) << 16) {
                    __threadfence();
                    merge_row_pieces<GROUP>(p, gp, sa, row, warp, s0, s1, lane);
                    if (lane == 0) *counter = 0;
                }
            }
            continue;
        }

        if (kind == TAG_FIRST) {
            row = static_cast<int>(tag.y);
            piece = static_cast<int>(tag.w);
            const bool live = g < GROUP;
            const __half* qrow = static_cast<const __half*>(p.q)
                + (static_cast<size_t>(row) * p.num_q_heads + warp * GROUP + (live ? g : 0)) * HEAD_DIM;
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
#pragma unroll
            for (int mt = 0; mt < 8; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.f;
        }

        const uint32_t k_tile = pipe + stage * S::STAGE_BYTES;
        const uint32_t v_tile = k_tile + S::TILE_BYTES;
        const int valid = static_cast<int>(tag.z);
        auto rows = [&](int t, int panel) { return row_offset<KV, S::HEADS>(t, panel, btl, warp); };
        bool wrote;
        if constexpr (FP8) wrote = process_group_e4m3(k_tile, v_tile, rows, 0, valid, qb, acc, m_run, l_run, qk_scale, lane);
        else               wrote = process_group_f16(k_tile, v_tile, rows, 0, valid, qb, acc, m_run, l_run, qk_scale, lane);
        if (wrote) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
        tiles_done++;
    }
    if (st.slots && tid == 0) {
        atomicAdd(st.slots + 2 * blockIdx.x, global_ns() - t_entry);
        atomicAdd(st.slots + 2 * blockIdx.x + 1, static_cast<unsigned long long>(tiles_done));
        if (blockIdx.x == 0) atomicAdd(st.slots + 2 * gridDim.x, 1ull);
    }
}

}  // namespace pdk
