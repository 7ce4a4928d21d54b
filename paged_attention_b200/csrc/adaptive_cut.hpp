// Adaptive cut: per-CTA streaming rates recorded by the decode kernel, and the weights derived from them.
// Part of pd_abi.cu (included there, after the error helpers); not a stand-alone header.
#pragma once

namespace {

// Adaptive cut.  SMs do not stream at the same rate (on B200 groups of SMs are 5-10 % slower than others,
// stable from launch to launch, and CTA c of a grid always lands on the same SM), so with equal shares the
// slow SMs finish 20-30 us after the fast ones on a 300 us layer and the tail runs at a fraction of the
// bandwidth.  Every launch therefore leaves (busy time, tiles) per CTA in a small device table;
// pd_device_plan_upload queues a copy of it to pinned host memory behind the launches so far, and the
// upload after that turns the copy into relative rates and cuts the step in shares proportional to them.
// The caller-visible plan is never changed; the weighted cut is a second schedule inside the device plan.
bool g_adaptive = std::getenv("PD_B200_NO_ADAPTIVE") == nullptr;
struct RateTable {
    int grid = 0;
    unsigned long long* slots = nullptr;     // device: per CTA running totals (busy ns, tiles), advanced by every launch
    unsigned long long* host = nullptr;      // pinned copy of an earlier state of `slots`
    std::vector<unsigned long long> seen;    // the totals the weights already account for
    cudaEvent_t copied = nullptr;            // completion of the copy into `host`
    bool copy_queued = false;
    std::vector<float> weights;              // mean 1; empty until the first usable record
    int updates = 0;
    bool resync = false;                     // after a reset: the next copy only re-bases `seen` (launches from before the reset say nothing new)
    // For the device-side planner: shares[0] = 1.0 once weights exist (0.0: cut in equal shares), then
    // shares[1 + c] = (w_0 + .. + w_c-1) / sum(w) for c = 0..grid.  Device memory with a stable address, so a
    // captured plan kernel picks up whatever the host wrote last.
    double* shares = nullptr;
};
struct RateKey {
    int device; const void* fn; int grid;
    bool operator==(const RateKey& o) const { return device == o.device && fn == o.fn && grid == o.grid; }
};
struct RateKeyHash {
    size_t operator()(const RateKey& k) const {
        return std::hash<const void*>()(k.fn) ^ (static_cast<size_t>(k.grid) * 0x9e3779b97f4a7c15ull) ^ static_cast<size_t>(k.device);
    }
};
std::mutex g_rate_mutex;
std::unordered_map<RateKey, RateTable, RateKeyHash> g_rates;

// The table of (this device, kernel, grid); created on first use.  Pointers into the map stay valid.
// create = false (a stream capture is under way: nothing may be allocated): only an existing table.
RateTable* rate_table(const void* fn, int grid, bool create = true) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || grid <= 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_rate_mutex);
    if (!create) {
        auto it = g_rates.find(RateKey{dev, fn, grid});
        return it == g_rates.end() || !it->second.slots ? nullptr : &it->second;
    }
    RateTable& t = g_rates[RateKey{dev, fn, grid}];
    if (!t.slots) {
        const size_t bytes = sizeof(unsigned long long) * (2 * grid + 1);   // + launches so far
        const size_t share_bytes = sizeof(double) * (grid + 2);
        void* dev_mem = nullptr;
        void* host = nullptr;
        void* share_mem = nullptr;
        if (cudaMalloc(&dev_mem, bytes) != cudaSuccess || cudaMemset(dev_mem, 0, bytes) != cudaSuccess ||
            cudaMalloc(&share_mem, share_bytes) != cudaSuccess || cudaMemset(share_mem, 0, share_bytes) != cudaSuccess ||
            cudaMallocHost(&host, bytes) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.copied, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(dev_mem);
            cudaFree(share_mem);
            cudaFreeHost(host);
            g_rates.erase(RateKey{dev, fn, grid});
            return nullptr;
        }
        std::memset(host, 0, bytes);
        t.slots = static_cast<unsigned long long*>(dev_mem);
        t.host = static_cast<unsigned long long*>(host);
        t.shares = static_cast<double*>(share_mem);
        t.seen.assign(2 * static_cast<size_t>(grid) + 1, 0);
        t.grid = grid;
    }
    return &t;
}

// Folds the latest record into the weights.  Only records of launches long enough that the fixed cost of
// a CTA (a few microseconds) does not matter are used.  Returns a copy of the weights taken under the lock
// (empty while there are none): another host thread planning for the same (device, kernel, grid) may
// rewrite the table's own vector at any time.
void fold_readings(RateTable* t, cudaStream_t stream);
std::vector<float> update_weights(RateTable* t, cudaStream_t stream) {
    if (!t) return {};
    std::lock_guard<std::mutex> lock(g_rate_mutex);
    fold_readings(t, stream);
    return t->weights;
}
void fold_readings(RateTable* t, cudaStream_t stream) {
    // Use the copy queued by an earlier upload if it has landed, then queue the next one behind the
    // launches issued so far.  Nothing here waits for the device.
    const bool have_copy = t->copy_queued && cudaEventQuery(t->copied) == cudaSuccess;
    cudaGetLastError();   // cudaErrorNotReady is expected
    struct Requeue {
        RateTable* t; cudaStream_t s; bool go;
        ~Requeue() {
            if (!go) return;
            if (cudaMemcpyAsync(t->host, t->slots, sizeof(unsigned long long) * (2 * t->grid + 1), cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                cudaEventRecord(t->copied, s) == cudaSuccess)
                t->copy_queued = true;
            else
                cudaGetLastError();
        }
    } requeue{t, stream, have_copy || !t->copy_queued};
    if (!have_copy) return;
    const int n = t->grid;
    std::vector<double> rate(n, 0.0);
    double sum = 0.0, busy_total = 0.0;
    int valid = 0;
    const unsigned long long launches = t->host[2 * n] - t->seen[2 * n];
    for (int c = 0; c < n; c++) {
        const double ns = static_cast<double>(t->host[2 * c] - t->seen[2 * c]);
        const double tiles = static_cast<double>(t->host[2 * c + 1] - t->seen[2 * c + 1]);
        busy_total += ns;
        if (ns <= 0.0 || tiles <= 0.0) continue;
        rate[c] = tiles / ns;
        sum += rate[c];
        valid++;
    }
    if (launches == 0) return;                             // nothing ran since the last reading
    t->seen.assign(t->host, t->host + 2 * static_cast<size_t>(n) + 1);
    if (t->resync) { t->resync = false; return; }
    // Only launches in which every CTA worked, and for long enough (120 us on average) that its few
    // microseconds of ramp-up and epilogue do not matter, say something about streaming rates.
    // (The equal cut can leave the last CTA or two of a grid without work; they keep their weight.)
    if (valid < n - std::max(2, n / 64) || busy_total / static_cast<double>(launches) / valid < 120000.0) return;
    const double mean = sum / valid;
    // SMs of one GPU differ by 10 % or so; a reading that spreads over more than 1.5x saw something else
    // (another stream's kernels sharing the SMs, a preempted context) and says nothing about the SMs.
    double lo = mean, hi = mean;
    for (int c = 0; c < n; c++)
        if (rate[c] > 0.0) { lo = std::min(lo, rate[c]); hi = std::max(hi, rate[c]); }
    if (hi > 1.5 * lo) return;
    if (t->weights.empty()) t->weights.assign(n, 1.0f);
#ifndef PD_B200_CUT_GAIN_EARLY
#define PD_B200_CUT_GAIN_EARLY 0.5
#endif
#ifndef PD_B200_CUT_GAIN
#define PD_B200_CUT_GAIN 0.3
#endif
    const double gain = t->updates < 4 ? PD_B200_CUT_GAIN_EARLY : PD_B200_CUT_GAIN;
    double wsum = 0.0;
    for (int c = 0; c < n; c++) {
        if (!(rate[c] > 0.0)) { wsum += t->weights[c]; continue; }
        const double target = std::min(1.3, std::max(0.7, rate[c] / mean));
        t->weights[c] = static_cast<float>((1.0 - gain) * t->weights[c] + gain * target);
        wsum += t->weights[c];
    }
    for (int c = 0; c < n; c++) t->weights[c] = static_cast<float>(t->weights[c] * n / wsum);
    t->updates++;
    // the same cumulative shares build_plan_weighted computes, for the device-side planner
    std::vector<double> shares(n + 2, 0.0);
    double total = 0.0, acc = 0.0;
    for (float w : t->weights) total += w;
    shares[0] = 1.0;
    for (int c = 0; c < n; c++) {
        acc += t->weights[c];
        shares[2 + c] = acc / total;
    }
    if (cudaMemcpyAsync(t->shares, shares.data(), sizeof(double) * (n + 2), cudaMemcpyHostToDevice, stream) != cudaSuccess)
        cudaGetLastError();   // pageable source: the call returns once the bytes are staged
}

}  // namespace
