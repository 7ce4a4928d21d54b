// Host planner: decode::make_plan (src/decode/decode.cu:65-108 of the reference), its cut with unequal
// shares, and the checks every plan passes before the kernels see it.
// Part of pd_abi.cu (included there, after the error helpers); not a stand-alone header.
#pragma once

namespace {

// ---- planner ------------------------------------------------------------------------------

// The flat list of (row, kv head, tile) work units is cut into num_ctas contiguous
// runs of `per` units; each maximal run of one (row, head) inside a CTA's share is a
// segment.  Produces exactly the plan of decode::make_plan (src/decode/decode.cu:65-108)
// for the same tile and num_ctas.
int build_plan(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads, int num_ctas,
               pd_plan** out);

}  // namespace

struct pd_plan {
    int num_ctas = 0;
    int tile     = 0;
    int num_items = 0;
    std::vector<int> segments;        // 4 ints each
    std::vector<int> cta_seg_begin;
    std::vector<int> item_seg_begin;
    // what pd_make_plan knew when it cut the plan (dtype < 0: unknown, e.g. built from arrays); lets the
    // device plan also carry the head-fused schedule of the same step
    int dtype = -1, batch = 0, num_q_heads = 0, num_kv_heads = 0, forced_ctas = 0;
    std::vector<int> seq_lens;
};

namespace {

int build_plan(int tile, const int* seq_lens, int batch, int num_q_heads, int num_kv_heads, int num_ctas,
               pd_plan** out) {
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads != 0)
        return set_error(PD_INVALID_ARGUMENT, "num_q_heads must be a multiple of num_kv_heads");
    if (tile <= 0 || num_ctas <= 0 || batch < 0) return set_error(PD_INVALID_ARGUMENT, "make_plan: tile, num_ctas must be positive");
    long long total = 0;
    for (int b = 0; b < batch; b++) {
        if (seq_lens[b] <= 0) return set_error(PD_INVALID_ARGUMENT, "make_plan: every sequence needs at least one token");
        total += static_cast<long long>((seq_lens[b] + tile - 1) / tile) * num_kv_heads;
    }
    pd_plan* plan = new pd_plan();
    plan->tile = tile;
    plan->num_items = batch * num_kv_heads;
    plan->item_seg_begin.assign(plan->num_items + 1, 0);
    if (total == 0) {   // empty batch: nothing to launch
        plan->cta_seg_begin.assign(1, 0);
        *out = plan;
        return PD_OK;
    }
    const long long per = (total + num_ctas - 1) / num_ctas;   // work units per CTA
    plan->num_ctas = static_cast<int>((total + per - 1) / per);
    plan->cta_seg_begin.reserve(plan->num_ctas + 1);
    plan->cta_seg_begin.push_back(0);
    long long room = per;                                      // units the current CTA can still take
    for (int item = 0; item < plan->num_items; item++) {
        const int b = item / num_kv_heads, h = item % num_kv_heads;
        const int len = seq_lens[b];
        const int tiles = (len + tile - 1) / tile;
        int first = 0;
        while (first < tiles) {
            if (room == 0) {
                plan->cta_seg_begin.push_back(static_cast<int>(plan->segments.size() / 4));
                room = per;
            }
            const int take = static_cast<int>(std::min<long long>(room, tiles - first));
            const int seg[4] = {b, h, first * tile, std::min((first + take) * tile, len)};
            plan->segments.insert(plan->segments.end(), seg, seg + 4);
            plan->item_seg_begin[item + 1] = plan->item_seg_begin[item + 1] + 1;
            first += take;
            room -= take;
        }
    }
    plan->cta_seg_begin.push_back(static_cast<int>(plan->segments.size() / 4));
    for (int i = 0; i < plan->num_items; i++) plan->item_seg_begin[i + 1] += plan->item_seg_begin[i];
    if (static_cast<int>(plan->cta_seg_begin.size()) != plan->num_ctas + 1) {
        delete plan;
        return set_error(PD_INTERNAL, "planner produced an inconsistent CTA table");
    }
    *out = plan;
    return PD_OK;
}

// Where rows are cut in a few pieces (a long batch: 2-3 segments per row) the decode kernel merges
// them itself (one warp per split row); a row cut in dozens of pieces (one long sequence spread over
// the whole grid) merges faster in the separate kernel, which puts a warp on every (row, query head).
int plan_merge_mode(const pd_plan& pl) {
    const int items = static_cast<int>(pl.item_seg_begin.size()) - 1;
    if (static_cast<int>(pl.segments.size() / 4) <= items) return 0;
    int widest = 0;
    for (int i = 0; i < items; i++) widest = std::max(widest, pl.item_seg_begin[i + 1] - pl.item_seg_begin[i]);
    return widest > pdk::HYBRID_MAX_PIECES ? pdk::MERGE_SEPARATE : pdk::MERGE_IN_KERNEL;
}

// The planner's cut with unequal shares: CTA c owns the work units [B_c, B_{c+1}) with
// B_c = round(total * (w_0 + ... + w_{c-1}) / (w_0 + ... + w_{n-1})).  Same segment rules as build_plan.
int build_plan_weighted(int tile, const int* seq_lens, int batch, int heads, const std::vector<float>& weights, pd_plan** out) {
    const int grid = static_cast<int>(weights.size());
    if (tile <= 0 || batch <= 0 || heads <= 0 || grid <= 0) return set_error(PD_INVALID_ARGUMENT, "weighted plan: bad argument");
    long long total = 0;
    for (int b = 0; b < batch; b++) {
        if (seq_lens[b] <= 0) return set_error(PD_INVALID_ARGUMENT, "make_plan: every sequence needs at least one token");
        total += static_cast<long long>((seq_lens[b] + tile - 1) / tile) * heads;
    }
    double wsum = 0.0;
    for (float w : weights) wsum += w;
    std::vector<long long> bound(grid + 1, 0);
    double acc = 0.0;
    for (int c = 0; c < grid; c++) {
        acc += weights[c];
        bound[c + 1] = std::max(bound[c], std::min<long long>(total, std::llround(total * (acc / wsum))));
    }
    bound[grid] = total;
    pd_plan* plan = new pd_plan();
    plan->tile = tile;
    plan->num_items = batch * heads;
    plan->num_ctas = grid;
    plan->item_seg_begin.assign(plan->num_items + 1, 0);
    plan->cta_seg_begin.assign(grid + 1, 0);
    int cta = 0;
    long long at = 0;                                           // work units before the current item
    for (int item = 0; item < plan->num_items; item++) {
        const int b = item / heads, h = item % heads, len = seq_lens[b];
        const int tiles = (len + tile - 1) / tile;
        int first = 0;
        while (first < tiles) {
            while (bound[cta + 1] <= at + first) {              // this CTA's share is used up: the next one starts here
                cta++;
                plan->cta_seg_begin[cta] = static_cast<int>(plan->segments.size() / 4);
            }
            const int take = static_cast<int>(std::min<long long>(bound[cta + 1] - (at + first), tiles - first));
            const int seg[4] = {b, h, first * tile, std::min((first + take) * tile, len)};
            plan->segments.insert(plan->segments.end(), seg, seg + 4);
            plan->item_seg_begin[item + 1]++;
            first += take;
        }
        at += tiles;
    }
    for (int c = cta + 1; c <= grid; c++) plan->cta_seg_begin[c] = static_cast<int>(plan->segments.size() / 4);
    for (int i = 0; i < plan->num_items; i++) plan->item_seg_begin[i + 1] += plan->item_seg_begin[i];
    *out = plan;
    return PD_OK;
}

// Host-side validation of a plan against the lengths it was made for; every index
// the kernels will dereference is checked here so the device never reads out of range.
int validate_plan(const pd_plan& plan, const int* seq_lens, int batch, int num_kv_heads) {
    const int nseg = static_cast<int>(plan.segments.size() / 4);
    if (static_cast<int>(plan.cta_seg_begin.size()) != plan.num_ctas + 1) return set_error(PD_INTERNAL, "plan: cta table size");
    for (int c = 0; c < plan.num_ctas; c++)
        if (plan.cta_seg_begin[c] > plan.cta_seg_begin[c + 1]) return set_error(PD_INTERNAL, "plan: cta table not monotone");
    if (plan.cta_seg_begin.front() != 0 || plan.cta_seg_begin.back() != nseg) return set_error(PD_INTERNAL, "plan: cta table ends");
    for (int s = 0; s < nseg; s++) {
        const int* g = &plan.segments[4 * s];
        if (g[0] < 0 || g[0] >= batch || g[1] < 0 || g[1] >= num_kv_heads || g[2] < 0 || g[2] >= g[3] ||
            g[3] > seq_lens[g[0]] || g[2] % plan.tile != 0)
            return set_error(PD_INTERNAL, "plan: segment %d out of range", s);
    }
    return PD_OK;
}

}  // namespace
