// The rank-sliced row loader in stream order: a little-endian u32 token file, mapped read-only, rows of
// seq_len + 1 tokens, rank k reading slots [start.row + k*B, +B) of each global batch of B*world rows
// (src/data/source.rs:7-12,204-230, src/data/positioning.rs:44-68, src/data/rows.rs:150-165). The rows a rank draws
// are consecutive in the file, so one step is one pinned staging copy, one host-to-device copy and one kernel that
// widens the ids to i64 and writes inputs [B,S] and targets [B,S] (src/data/batch.rs:51-71).
// The shuffled order depends on rand 0.10.3's StdRng and is not offered.
// With a target mask (TargetMask::PrefixLm, src/data/mask.rs:36-47) or the document mask (src/data/host_masks.rs:49-77,
// src/data/segments.rs:62-101) on, the same stream also yields the [B,S] f32 loss mask, the count of scored positions,
// the [B,S] i32 segment ids and the cumulative segment offsets, built on the device from the staged window.
// TargetMask::SpeechAudio needs boostr's SpeechLayout, which is not vendored, and is not offered.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>

#include "oxz_internal.h"

// One source: a token file mapped read-only. It keeps its own whole rows and drops its own tail, so no row spans two
// sources; global row r counts rows from the start of source 0 (src/data/source.rs:1-6, 96-118).
struct Part {
    int fd = -1;
    const uint32_t* tokens = nullptr;
    size_t map_bytes = 0;
    uint64_t n_tokens = 0, rows = 0, first_row = 0;
};

// Ascending, disjoint global row ranges; row r of the set is the r-th row across them (src/data/row_ranges.rs).
struct Ranges {
    std::vector<uint64_t> start, end, before;
    uint64_t len = 0;
    void push(uint64_t a, uint64_t b) {
        start.push_back(a);
        end.push_back(b);
        before.push_back(len);
        len += b - a;
    }
    uint64_t global_row(uint64_t row) const {
        size_t i = before.size();
        while (i > 1 && before[i - 1] > row) i--;
        return i ? start[i - 1] + (row - before[i - 1]) : row;
    }
};

// A weighted mixture of the sources as a virtual row order, stream order (src/data/mixture/state.rs:1-8): an epoch is
// rows_per_epoch slots; source i fills quota[i] of them in smooth weighted round-robin order, the same every epoch;
// the p-th slot of source i in epoch e is its draw e * quota[i] + p, and draw k reads the source's row k % n_i.
struct Mixture {
    static constexpr uint64_t BLOCK = 4096;
    std::vector<double> weights;
    bool requested = false;  // rows_per_epoch was given rather than derived
    uint64_t rows_per_epoch = 0;
    std::vector<uint64_t> quotas;
    std::vector<Ranges> sources;     // each source's training rows
    std::vector<uint16_t> schedule;  // source of every slot
    std::vector<uint32_t> prefix;    // per BLOCK slots: how many slots of each source came before
    uint64_t cur_slot = 0;
    std::vector<uint32_t> cur_counts;

    // EpochSchedule::locate (src/data/mixture/schedule.rs:74-99): the slot's source and how many of its slots came before
    bool locate(uint64_t slot, uint32_t* source, uint64_t* before_out) {
        if (slot >= schedule.size()) return false;
        const size_t width = quotas.size();
        if (cur_counts.size() != width || cur_slot > slot || slot - cur_slot >= BLOCK) {
            const uint64_t block = slot / BLOCK;
            cur_slot = block * BLOCK;
            cur_counts.assign(prefix.begin() + block * width, prefix.begin() + (block + 1) * width);
        }
        for (uint64_t i = cur_slot; i < slot; i++) cur_counts[schedule[i]]++;
        *source = schedule[slot];
        *before_out = cur_counts[*source];
        cur_counts[*source]++;
        cur_slot = slot + 1;
        return true;
    }
};

// A host thread that keeps the next batches' rows copied into pinned buffers while the device works on the current one
// (PrefetchDataLoader, src/data/prefetch.rs:37-61): it draws batches in order from the loader's position, so the batch
// sequence is the unprefetched loader's.
struct Prefetch {
    struct Slot {
        uint32_t* host = nullptr;       // pinned, one batch of rows
        cudaEvent_t copied = nullptr;   // the host-to-device copy that last read `host`
        std::vector<uint64_t> rows;
        oxz_data_position next{0, 0};
        int32_t status = 0;
        std::string error;
    };
    std::vector<Slot> slots;
    std::deque<int> ready, idle;
    std::mutex mu;
    std::condition_variable cv;
    bool stop = false;
    std::thread worker;
};

struct oxz_loader {
    std::vector<Part> parts;
    std::unique_ptr<Mixture> mix;
    // RowOrder::Shuffled with the permutations supplied by the caller: (epoch, permutation of the loader's rows), at
    // most two epochs at a time so that a prefetch thread can cross into the next one. Empty: stream order.
    std::vector<std::pair<uint64_t, std::vector<uint32_t>>> orders;
    std::unique_ptr<Prefetch> pre;
    uint32_t prefetch_depth = 0;
    uint64_t total_rows = 0, seq_len = 0;
    Ranges ranges;  // the global rows this loader reads
    oxz_row_layout layout{};
    uint64_t rank = 0;
    oxz_data_position pos{0, 0};
    int device = 0;
    // two sets of buffers, so the batch handed out last stays valid while the next one is drawn
    uint32_t* h_stage[2] = {nullptr, nullptr};
    uint32_t* d_stage[2] = {nullptr, nullptr};
    int64_t* d_inputs[2] = {nullptr, nullptr};
    int64_t* d_targets[2] = {nullptr, nullptr};
    cudaEvent_t staged[2] = {nullptr, nullptr};
    int slot = 0;
    // masks
    bool target_mask = false, document_mask = false;
    uint32_t target_base = 0, n_always = 0, separator = 0;
    uint32_t always[OXZ_MAX_ALWAYS_SCORE] = {};
    float* d_loss_mask[2] = {nullptr, nullptr};
    int32_t* d_seg_ids[2] = {nullptr, nullptr};
    int32_t* d_cu[2] = {nullptr, nullptr};        // B*S + 1 offsets at most
    uint32_t* d_row_base[2] = {nullptr, nullptr};  // B + 1
    unsigned long long* d_counts[2] = {nullptr, nullptr};  // {scored, segments}
    unsigned long long* h_counts[2] = {nullptr, nullptr};  // pinned
    int last = -1;  // slot of the batch handed out last
};

namespace {

// One thread per (row, position): inputs take tokens [0, S), targets tokens [1, S + 1) of each row.
__global__ void __launch_bounds__(256) k_split_rows(const uint32_t* __restrict__ window, uint64_t rows, uint64_t seq_len,
                                                    int64_t* __restrict__ inputs, int64_t* __restrict__ targets) {
    const uint64_t n = rows * seq_len;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t r = i / seq_len, s = i - r * seq_len;
        const uint32_t* row = window + r * (seq_len + 1);
        inputs[i] = static_cast<int64_t>(row[s]);
        targets[i] = static_cast<int64_t>(row[s + 1]);
    }
}

struct MaskRule {
    uint32_t target_base, n_always, separator;
    int32_t has_target, has_document;
    uint32_t always[OXZ_MAX_ALWAYS_SCORE];
};

// k_split_rows plus the loss mask: a position scores iff its TARGET id passes the rule and its INPUT is not the
// document separator. The scored positions are counted with integer atomics (one per block), so the count is exact.
__global__ void __launch_bounds__(256) k_split_rows_masked(const uint32_t* __restrict__ window, uint64_t rows, uint64_t seq_len,
                                                           MaskRule rule, int64_t* __restrict__ inputs,
                                                           int64_t* __restrict__ targets, float* __restrict__ loss_mask,
                                                           unsigned long long* __restrict__ counts) {
    const uint64_t n = rows * seq_len;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    uint32_t mine = 0;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t r = i / seq_len, s = i - r * seq_len;
        const uint32_t* row = window + r * (seq_len + 1);
        const uint32_t in = row[s], tg = row[s + 1];
        inputs[i] = static_cast<int64_t>(in);
        targets[i] = static_cast<int64_t>(tg);
        bool scored = true;
        if (rule.has_target) {
            scored = tg >= rule.target_base;
            for (uint32_t k = 0; k < rule.n_always; k++) scored |= tg == rule.always[k];
        }
        if (rule.has_document && in == rule.separator) scored = false;
        loss_mask[i] = scored ? 1.0f : 0.0f;
        mine += scored ? 1u : 0u;
    }
    __shared__ uint32_t sh[8];
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_down_sync(0xffffffffu, mine, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t t = 0;
        for (int w = 0; w < 8; w++) t += sh[w];
        if (t) atomicAdd(&counts[0], static_cast<unsigned long long>(t));
    }
}

// Segments, step 1: one warp per row counts the segments the row closes: one per separator among its inputs, and
// one more for the row end unless the last input is itself a separator (src/data/segments.rs:84-99).
__global__ void __launch_bounds__(256) k_row_closings(const uint32_t* __restrict__ window, uint32_t rows, uint32_t seq_len,
                                                      uint32_t separator, uint32_t* __restrict__ row_base) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const uint32_t* row = window + static_cast<uint64_t>(warp) * (seq_len + 1);
    uint32_t c = 0;
    for (uint32_t s = lane; s < seq_len; s += 32) c += row[s] == separator ? 1u : 0u;
    for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
    if (lane == 0) row_base[warp] = c + (row[seq_len - 1] != separator ? 1u : 0u);
}

// Step 2: one block turns the per-row counts into exclusive prefix sums in place; row_base[rows] and counts[1]
// receive the number of segments, and the first offset is 0.
__global__ void __launch_bounds__(256) k_scan_rows(uint32_t* __restrict__ row_base, uint32_t rows, int32_t* __restrict__ cu,
                                                   unsigned long long* __restrict__ counts) {
    __shared__ uint32_t sh[256];
    __shared__ uint32_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (uint32_t base = 0; base < rows; base += 256) {
        const uint32_t i = base + threadIdx.x;
        const uint32_t v = i < rows ? row_base[i] : 0u;
        sh[threadIdx.x] = v;
        __syncthreads();
        for (int o = 1; o < 256; o <<= 1) {  // inclusive scan
            const uint32_t add = threadIdx.x >= static_cast<uint32_t>(o) ? sh[threadIdx.x - o] : 0u;
            __syncthreads();
            sh[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < rows) row_base[i] = carry + sh[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == 255) carry += sh[255];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        row_base[rows] = carry;
        counts[1] = carry;
        cu[0] = 0;
    }
}

// Step 3: one block per row walks the row in chunks of 256 positions with a running count of the separators seen:
// a token's segment is the row's first segment plus the separators before it; a separator at s closes its segment
// at flat offset b*S + s + 1, the row end closes the last one unless a separator already did.
__global__ void __launch_bounds__(256) k_fill_segments(const uint32_t* __restrict__ window, uint32_t seq_len, uint32_t separator,
                                                       const uint32_t* __restrict__ row_base, int32_t* __restrict__ seg_ids,
                                                       int32_t* __restrict__ cu) {
    const uint32_t b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t* row = window + static_cast<uint64_t>(b) * (seq_len + 1);
    const uint32_t first = row_base[b];
    __shared__ uint32_t warp_sum[8];
    __shared__ uint32_t seen;  // separators in the chunks before this one
    if (threadIdx.x == 0) seen = 0;
    __syncthreads();
    for (uint32_t base = 0; base < seq_len; base += 256) {
        const uint32_t s = base + threadIdx.x;
        const bool live = s < seq_len;
        const uint32_t flag = live && row[s] == separator ? 1u : 0u;
        const uint32_t ballot = __ballot_sync(0xffffffffu, flag);
        const uint32_t before_in_warp = __popc(ballot & ((1u << lane) - 1u));
        if (lane == 0) warp_sum[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = seen + before_in_warp;
        for (uint32_t w = 0; w < warp; w++) before += warp_sum[w];
        if (live) {
            const uint64_t flat = static_cast<uint64_t>(b) * seq_len + s;
            seg_ids[flat] = static_cast<int32_t>(first + before);
            if (flag) cu[first + before + 1] = static_cast<int32_t>(flat + 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t t = 0;
            for (int w = 0; w < 8; w++) t += warp_sum[w];
            seen += t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && row[seq_len - 1] != separator)
        cu[first + seen + 1] = static_cast<int32_t>((static_cast<uint64_t>(b) + 1) * seq_len);
}

void stop_prefetch(oxz_loader* l) {
    if (!l->pre) return;
    {
        std::lock_guard<std::mutex> g(l->pre->mu);
        l->pre->stop = true;
    }
    l->pre->cv.notify_all();
    if (l->pre->worker.joinable()) l->pre->worker.join();
    cudaSetDevice(l->device);
    for (auto& slot : l->pre->slots) {
        if (slot.copied) {
            cudaEventSynchronize(slot.copied);
            cudaEventDestroy(slot.copied);
        }
        if (slot.host) cudaFreeHost(slot.host);
    }
    l->pre.reset();
}

void release(oxz_loader* l) {
    if (!l) return;
    stop_prefetch(l);
    if (l->d_stage[0] || l->h_stage[0]) cudaSetDevice(l->device);
    for (int i = 0; i < 2; i++) {
        if (l->h_stage[i]) cudaFreeHost(l->h_stage[i]);
        if (l->d_stage[i]) cudaFree(l->d_stage[i]);
        if (l->d_inputs[i]) cudaFree(l->d_inputs[i]);
        if (l->d_targets[i]) cudaFree(l->d_targets[i]);
        if (l->staged[i]) cudaEventDestroy(l->staged[i]);
        if (l->d_loss_mask[i]) cudaFree(l->d_loss_mask[i]);
        if (l->d_seg_ids[i]) cudaFree(l->d_seg_ids[i]);
        if (l->d_cu[i]) cudaFree(l->d_cu[i]);
        if (l->d_row_base[i]) cudaFree(l->d_row_base[i]);
        if (l->d_counts[i]) cudaFree(l->d_counts[i]);
        if (l->h_counts[i]) cudaFreeHost(l->h_counts[i]);
    }
    for (Part& p : l->parts) {
        if (p.tokens) munmap(const_cast<uint32_t*>(p.tokens), p.map_bytes);
        if (p.fd >= 0) close(p.fd);
    }
    delete l;
}

// RowRanges::global_row (src/data/row_ranges.rs:100-106)
uint64_t global_row(const oxz_loader* l, uint64_t row) { return l->ranges.global_row(row); }

// RowStore::row (src/data/source.rs:140-158): where global row r starts, or null past the last whole row.
const uint32_t* row_tokens(const oxz_loader* l, uint64_t r) {
    for (const Part& p : l->parts)
        if (r < p.first_row + p.rows) return r >= p.first_row ? p.tokens + (r - p.first_row) * (l->seq_len + 1) : nullptr;
    return nullptr;
}

}  // namespace

using namespace oxz;

extern "C" {

// Maps the files in order. `what` words the errors of an unusable range for the one-file entry point.
static int32_t start_prefetch(oxz_loader* l, uint32_t depth);

static int32_t open_parts(oxz_loader* l, const char* const* paths, uint32_t n_paths, uint64_t seq_len) {
    using namespace oxz;
    if (n_paths == 0) return fail(OXZ_ERR_DATA, "no data files given. Pass -d <file.bin>, or set trainer.data.sources.");
    for (uint32_t i = 0; i < n_paths; i++) {
        const char* path = paths[i];
        if (!path) return fail(OXZ_ERR_INVALID, "oxz_loader_open: path %u is null", i);
        l->parts.emplace_back();
        Part& p = l->parts.back();
        p.fd = open(path, O_RDONLY);
        if (p.fd < 0) return fail(OXZ_ERR_DATA, "failed to open data file %s: %s", path, strerror(errno));
        struct stat st;
        if (fstat(p.fd, &st) != 0) return fail(OXZ_ERR_DATA, "failed to stat data file %s: %s", path, strerror(errno));
        if (st.st_size % 4 != 0)
            return fail(OXZ_ERR_DATA, "data file %s is %lld bytes, not a multiple of 4: it is not a u32 token array. Rebuild it as raw u32 tokens.",
                        path, (long long)st.st_size);
        p.n_tokens = (uint64_t)st.st_size / 4;
        if (st.st_size > 0) {
            void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, p.fd, 0);
            if (m == MAP_FAILED) return fail(OXZ_ERR_DATA, "failed to mmap data file %s: %s", path, strerror(errno));
            p.tokens = static_cast<const uint32_t*>(m);
            p.map_bytes = (size_t)st.st_size;
        }
        p.rows = p.n_tokens / (seq_len + 1);  // the tail shorter than a row is never read
        p.first_row = l->total_rows;
        l->total_rows += p.rows;
    }
    return OXZ_OK;
}

static int32_t finish_open(oxz_loader* l, uint64_t seq_len, uint64_t rank_batch_size, uint64_t rank, uint64_t world, int32_t device) {
    using namespace oxz;
    l->seq_len = seq_len;
    l->layout = oxz_row_layout{l->ranges.len, rank_batch_size, world};
    l->rank = rank;
    l->device = device;
    OXZ_TRY(oxz_rows_check(&l->layout));
    if (rank >= world)
        return fail(OXZ_ERR_DATA, "rank %llu is not below world size %llu. Pass a rank in [0, %llu).", (unsigned long long)rank,
                    (unsigned long long)world, (unsigned long long)world);
    return OXZ_OK;
}

int32_t oxz_loader_open(const char* path, uint64_t seq_len, uint64_t rank_batch_size, uint64_t rank, uint64_t world,
                        uint64_t first_row, uint64_t end_row, int32_t device, oxz_loader** out) {
    return oxz::guarded("oxz_loader_open", [&]() -> int32_t {
        if (!path || !out) return fail(OXZ_ERR_INVALID, "oxz_loader_open: null argument");
        *out = nullptr;
        if (seq_len == 0) return fail(OXZ_ERR_DATA, "model.max_seq_len is 0: a row needs at least one input and one target token");
        oxz_loader* l = new oxz_loader();
        int32_t s = open_parts(l, &path, 1, seq_len);
        if (s == OXZ_OK) {
            if (end_row == 0) end_row = l->total_rows;
            if (first_row >= end_row || end_row > l->total_rows)
                s = fail(OXZ_ERR_DATA, "row range [%llu, %llu) does not fit the data's %llu whole rows", (unsigned long long)first_row,
                         (unsigned long long)end_row, (unsigned long long)l->total_rows);
        }
        if (s == OXZ_OK) {
            l->ranges.push(first_row, end_row);
            s = finish_open(l, seq_len, rank_batch_size, rank, world, device);
        }
        if (s != OXZ_OK) {
            release(l);
            return s;
        }
        *out = l;
        return OXZ_OK;
    });
}

int32_t oxz_loader_open_files(const char* const* paths, uint32_t n_paths, uint64_t seq_len, uint64_t rank_batch_size,
                              uint64_t rank, uint64_t world, const uint64_t* spans, uint32_t n_spans, int32_t device,
                              oxz_loader** out) {
    return oxz::guarded("oxz_loader_open_files", [&]() -> int32_t {
        if (!out || (n_paths && !paths) || (n_spans && !spans)) return fail(OXZ_ERR_INVALID, "oxz_loader_open_files: null argument");
        *out = nullptr;
        if (seq_len == 0) return fail(OXZ_ERR_DATA, "model.max_seq_len is 0: a row needs at least one input and one target token");
        oxz_loader* l = new oxz_loader();
        int32_t s = open_parts(l, paths, n_paths, seq_len);
        const uint64_t total = l->total_rows;
        if (s == OXZ_OK && n_spans == 0) {  // RowRanges::whole
            if (total) l->ranges.push(0, total);
        }
        // RowRanges::new (src/data/row_ranges.rs:40-76)
        uint64_t prev_end = 0;
        for (uint32_t i = 0; s == OXZ_OK && i < n_spans; i++) {
            const uint64_t a = spans[2 * i], b = spans[2 * i + 1];
            if (a >= b || b > total)
                s = fail(OXZ_ERR_DATA, "row range [%llu, %llu) is not a non-empty range inside the %llu whole rows of this data. Pick a range inside [0, %llu).",
                         (unsigned long long)a, (unsigned long long)b, (unsigned long long)total, (unsigned long long)total);
            else if (i > 0 && a < prev_end)
                s = fail(OXZ_ERR_DATA, "row range [%llu, %llu) starts before row %llu, the end of the range before it. Pass ranges in ascending order without overlap.",
                         (unsigned long long)a, (unsigned long long)b, (unsigned long long)prev_end);
            else {
                l->ranges.push(a, b);
                prev_end = b;
            }
        }
        if (s == OXZ_OK) s = finish_open(l, seq_len, rank_batch_size, rank, world, device);
        if (s != OXZ_OK) {
            release(l);
            return s;
        }
        *out = l;
        return OXZ_OK;
    });
}

// quotas (src/data/mixture/quota.rs:22-57): floor of each share, the rows left over one each by largest remainder,
// lower index first on a tie; rounding error the other way takes rows back from the smallest remainders.
static void mixture_quotas(const double* weights, uint32_t n, uint64_t rows, std::vector<uint64_t>& counts) {
    double total = 0.0;
    for (uint32_t i = 0; i < n; i++) total += weights[i];
    std::vector<double> shares(n), rem(n);
    counts.assign(n, 0);
    uint64_t assigned = 0;
    for (uint32_t i = 0; i < n; i++) {
        shares[i] = weights[i] / total * (double)rows;
        const double fl = std::floor(shares[i]);
        rem[i] = shares[i] - fl;
        counts[i] = fl >= (double)rows ? rows : (uint64_t)fl;
        assigned += counts[i];
    }
    std::vector<uint32_t> order(n);
    for (uint32_t i = 0; i < n; i++) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return rem[a] > rem[b]; });
    if (assigned <= rows) {
        for (uint64_t k = 0; k < rows - assigned; k++) counts[order[k % n]]++;
    } else {
        uint64_t excess = assigned - rows;
        for (uint64_t k = 0; excess; k++) {
            const uint32_t i = order[n - 1 - (k % n)];
            if (counts[i] > 0) {
                counts[i]--;
                excess--;
            }
        }
    }
}

int32_t oxz_mixture_quotas(const double* weights, uint32_t n_weights, uint64_t rows, uint64_t* quotas) {
    return oxz::guarded("oxz_mixture_quotas", [&]() -> int32_t {
        if (!weights || !quotas || n_weights == 0) return fail(OXZ_ERR_INVALID, "oxz_mixture_quotas: null argument");
        for (uint32_t i = 0; i < n_weights; i++)
            if (!(std::isfinite(weights[i]) && weights[i] > 0.0))
                return fail(OXZ_ERR_DATA, "trainer.data.sources[%u].weight is %g: a weight must be a finite number above 0. Set it to the source's share, for example 1.0.", i, weights[i]);
        std::vector<uint64_t> q;
        mixture_quotas(weights, n_weights, rows, q);
        for (uint32_t i = 0; i < n_weights; i++) quotas[i] = q[i];
        return OXZ_OK;
    });
}

int32_t oxz_loader_set_mixture(oxz_loader* l, const double* weights, uint32_t n_weights, int32_t has_rows_per_epoch,
                               uint64_t rows_per_epoch) {
    return oxz::guarded("oxz_loader_set_mixture", [&]() -> int32_t {
        if (!l || (n_weights && !weights)) return fail(OXZ_ERR_INVALID, "oxz_loader_set_mixture: null argument");
        if (!l->orders.empty())
            return fail(OXZ_ERR_UNSUPPORTED, "oxz_loader_set_mixture: the loader reads a caller-supplied row order; a mixture draws its sources' rows in passes of their own. Clear the row order first");
        const uint64_t MAX_ROWS = 1ull << 28;
        if (n_weights != l->parts.size())
            return fail(OXZ_ERR_DATA, "trainer.data.sources sets %u weight(s), and the loader reads %zu source(s). Set one weight per source in trainer.data.sources, and remove the -d flags.",
                        n_weights, l->parts.size());
        if (n_weights > 65536)
            return fail(OXZ_ERR_DATA, "trainer.data.sources lists %u weighted sources, more than the 65536 a mixture can index. Merge some sources into one file.", n_weights);
        std::unique_ptr<Mixture> m(new Mixture());
        // the training rows of each source: the loader's ranges cut at the source's bounds (src/data/mixture/loader.rs:60-84)
        for (uint32_t i = 0; i < n_weights; i++) {
            const Part& part = l->parts[i];
            Ranges r;
            for (size_t k = 0; k < l->ranges.start.size(); k++) {
                const uint64_t a = std::max(l->ranges.start[k], part.first_row), b = std::min(l->ranges.end[k], part.first_row + part.rows);
                if (a < b) r.push(a, b);
            }
            if (!(std::isfinite(weights[i]) && weights[i] > 0.0))
                return fail(OXZ_ERR_DATA, "trainer.data.sources[%u].weight is %g: a weight must be a finite number above 0. Set it to the source's share, for example 1.0.", i, weights[i]);
            if (r.len == 0)
                return fail(OXZ_ERR_DATA, "trainer.data.sources[%u] holds no training rows, and its weight %g asks for rows. Remove the source, or use a file of at least one row of model.max_seq_len + 1 tokens outside the holdout.", i, weights[i]);
            if (r.len > 0xffffffffull)
                return fail(OXZ_ERR_DATA, "trainer.data.sources[%u] holds %llu training rows, more than the 4294967295 a row order can index. Split the file.", i, (unsigned long long)r.len);
            m->sources.push_back(std::move(r));
        }
        uint64_t total = 0;
        for (const Ranges& r : m->sources) total += r.len;
        const uint64_t rows = has_rows_per_epoch ? rows_per_epoch : total;
        if (rows == 0 || rows > MAX_ROWS)
            return fail(OXZ_ERR_DATA, "trainer.data.rows_per_epoch is %llu: an epoch needs at least 1 row and at most %llu rows, because the schedule keeps 2 bytes per row. Set trainer.data.rows_per_epoch inside that range.",
                        (unsigned long long)rows, (unsigned long long)MAX_ROWS);
        m->weights.assign(weights, weights + n_weights);
        m->requested = has_rows_per_epoch != 0;
        m->rows_per_epoch = rows;
        mixture_quotas(weights, n_weights, rows, m->quotas);
        // smooth weighted round-robin over the quotas (src/data/mixture/schedule.rs:103-122)
        {
            std::vector<int64_t> credit(n_weights, 0);
            m->schedule.reserve(rows);
            for (uint64_t k = 0; k < rows; k++) {
                uint32_t pick = 0;
                for (uint32_t i = 0; i < n_weights; i++) {
                    credit[i] += (int64_t)m->quotas[i];
                    if (credit[i] > credit[pick]) pick = i;
                }
                credit[pick] -= (int64_t)rows;
                m->schedule.push_back((uint16_t)pick);
            }
            std::vector<uint32_t> counts(n_weights, 0);
            for (uint64_t k = 0; k < rows; k++) {
                if (k % Mixture::BLOCK == 0) m->prefix.insert(m->prefix.end(), counts.begin(), counts.end());
                counts[m->schedule[k]]++;
            }
        }
        // the layout counts rows per epoch; the position resets to the start (src/data/mixture/loader.rs:28-33)
        oxz_row_layout layout = l->layout;
        layout.num_rows = rows;
        OXZ_TRY(oxz_rows_check(&layout));
        const uint32_t depth = l->pre ? l->prefetch_depth : 0;
        stop_prefetch(l);
        l->layout = layout;
        l->pos = oxz_data_position{0, 0};
        l->mix = std::move(m);
        return depth ? start_prefetch(l, depth) : (int32_t)OXZ_OK;
    });
}

int32_t oxz_loader_mixture_sources(const oxz_loader* l, oxz_mixture_source* out, uint32_t cap, uint32_t* n_sources) {
    return oxz::guarded("oxz_loader_mixture_sources", [&]() -> int32_t {
        if (!l || !n_sources) return fail(OXZ_ERR_INVALID, "oxz_loader_mixture_sources: null argument");
        *n_sources = l->mix ? (uint32_t)l->mix->weights.size() : 0;
        for (uint32_t i = 0; out && i < cap && i < *n_sources; i++)
            out[i] = oxz_mixture_source{l->mix->weights[i], l->mix->quotas[i], l->mix->sources[i].len};
        return OXZ_OK;
    });
}

int32_t oxz_loader_source_rows(const oxz_loader* l, uint64_t* rows, uint32_t cap, uint32_t* n_sources) {
    return oxz::guarded("oxz_loader_source_rows", [&]() -> int32_t {
        if (!l || !n_sources) return fail(OXZ_ERR_INVALID, "oxz_loader_source_rows: null argument");
        *n_sources = (uint32_t)l->parts.size();
        for (uint32_t i = 0; rows && i < cap && i < l->parts.size(); i++) rows[i] = l->parts[i].rows;
        return OXZ_OK;
    });
}

int32_t oxz_loader_close(oxz_loader* l) {
    return oxz::guarded("oxz_loader_close", [&]() -> int32_t {
        release(l);
        return OXZ_OK;
    });
}

int32_t oxz_loader_num_rows(const oxz_loader* l, uint64_t* rows) {
    return oxz::guarded("oxz_loader_num_rows", [&]() -> int32_t {
        if (!l || !rows) return fail(OXZ_ERR_INVALID, "oxz_loader_num_rows: null argument");
        *rows = l->layout.num_rows;
        return OXZ_OK;
    });
}

int32_t oxz_loader_position(const oxz_loader* l, oxz_data_position* pos) {
    return oxz::guarded("oxz_loader_position", [&]() -> int32_t {
        if (!l || !pos) return fail(OXZ_ERR_INVALID, "oxz_loader_position: null argument");
        *pos = l->pos;
        return OXZ_OK;
    });
}

int32_t oxz_loader_seek(oxz_loader* l, oxz_data_position pos) {
    return oxz::guarded("oxz_loader_seek", [&]() -> int32_t {
        if (!l) return fail(OXZ_ERR_INVALID, "oxz_loader_seek: null loader");
        if (pos.row > l->layout.num_rows)
            return fail(OXZ_ERR_DATA,
                        "data position epoch %llu row %llu is past this shard's %llu rows: the checkpoint was saved over "
                        "different data or a different model.max_seq_len. Resume with the original data and config, or "
                        "start a fresh run.",
                        (unsigned long long)pos.epoch, (unsigned long long)pos.row, (unsigned long long)l->layout.num_rows);
        // a prefetch thread has drawn ahead from the old position: it starts over from the new one
        const uint32_t depth = l->pre ? l->prefetch_depth : 0;
        stop_prefetch(l);
        l->pos = pos;
        return depth ? start_prefetch(l, depth) : (int32_t)OXZ_OK;
    });
}

int32_t oxz_loader_set_row_order(oxz_loader* l, uint64_t epoch, const uint32_t* perm, uint64_t n) {
    return oxz::guarded("oxz_loader_set_row_order", [&]() -> int32_t {
        if (!l) return fail(OXZ_ERR_INVALID, "oxz_loader_set_row_order: null loader");
        if (perm && l->mix)
            return fail(OXZ_ERR_UNSUPPORTED, "oxz_loader_set_row_order: a mixture draws its sources' rows in passes of their own (src/data/mixture/draw.rs:44-62); a caller-supplied row order serves a loader without weights");
        if (perm) {
            if (n != l->layout.num_rows)
                return fail(OXZ_ERR_DATA, "the row order holds %llu rows and the loader %llu: pass the permutation of the loader's rows",
                            (unsigned long long)n, (unsigned long long)l->layout.num_rows);
            OXZ_TRY(oxz_rows_check_permutation(perm, n));
        }
        // a prefetch thread reads the orders: it stops, and starts over from the loader's position with the new ones
        const uint32_t depth = l->pre ? l->prefetch_depth : 0;
        stop_prefetch(l);
        if (!perm) {
            l->orders.clear();
        } else {
            bool replaced = false;
            for (auto& o : l->orders)
                if (o.first == epoch) {
                    o.second.assign(perm, perm + n);
                    replaced = true;
                }
            if (!replaced) {
                if (l->orders.size() >= 2) {  // keep the newest two: drop the lowest epoch
                    size_t drop = l->orders[0].first < l->orders[1].first ? 0 : 1;
                    l->orders.erase(l->orders.begin() + drop);
                }
                l->orders.emplace_back(epoch, std::vector<uint32_t>(perm, perm + n));
            }
        }
        return depth ? start_prefetch(l, depth) : (int32_t)OXZ_OK;
    });
}

// The global rows of this rank's part of the next global batch, where each starts in its file, and the position after
// the batch. Does not move the loader.
static int32_t draw_rows(oxz_loader* l, oxz_data_position from, std::vector<uint64_t>& row_ids, std::vector<const uint32_t*>& src,
                         oxz_data_position* next_out) {
    using namespace oxz;
    const uint64_t B = l->layout.rank_batch_size, S = l->seq_len;
    oxz_data_position next;
    OXZ_TRY(oxz_rows_next_window(&l->layout, from, l->rank, S, 0, nullptr, 0, row_ids.data(), nullptr, nullptr, &next));
    for (uint64_t b = 0; b < B; b++) {
        if (l->mix) {
            // the slot's source, that source's draw over the whole run, the draw's row (src/data/mixture/state.rs:150-178)
            uint32_t source = 0;
            uint64_t before = 0;
            const uint64_t slot = row_ids[b];
            if (!l->mix->locate(slot, &source, &before))
                return fail(OXZ_ERR_DATA, "mixture slot %llu of epoch %llu is past the %llu rows of an epoch. This is a loader bug: report it with the data and config.",
                            (unsigned long long)slot, (unsigned long long)next.epoch, (unsigned long long)l->mix->rows_per_epoch);
            const Ranges& src_rows = l->mix->sources[source];
            const unsigned __int128 draw = (unsigned __int128)next.epoch * l->mix->quotas[source] + before;
            row_ids[b] = src_rows.global_row((uint64_t)(draw % src_rows.len));
        } else {
            uint64_t loader_row = row_ids[b];  // stream order: the row at slot i is row i
            if (!l->orders.empty()) {
                // EpochOrder::row (src/data/rows.rs:240-256) with the epoch's permutation as the caller made it
                const std::vector<uint32_t>* perm = nullptr;
                for (const auto& o : l->orders)
                    if (o.first == next.epoch) perm = &o.second;
                if (!perm)
                    return fail(OXZ_ERR_DATA, "the next batch reads epoch %llu and the loader holds no row order for it: call oxz_loader_set_row_order with epoch_permutation(num_rows, seed, %llu)",
                                (unsigned long long)next.epoch, (unsigned long long)next.epoch);
                loader_row = (*perm)[loader_row];
            }
            row_ids[b] = global_row(l, loader_row);  // loader row -> global row across the ranges
        }
        src[b] = row_tokens(l, row_ids[b]);
        if (!src[b])
            return fail(OXZ_ERR_DATA, "row %llu is past the %llu whole rows of this data. This is a loader bug: report it with the data and config.",
                        (unsigned long long)row_ids[b], (unsigned long long)l->total_rows);
    }
    *next_out = next;
    return OXZ_OK;
}

// a rank's slots are consecutive loader rows: runs that are also consecutive in one file move as one copy
static void copy_rows(const oxz_loader* l, const std::vector<const uint32_t*>& src, uint32_t* dst) {
    const uint64_t B = l->layout.rank_batch_size, width = l->seq_len + 1;
    for (uint64_t b = 0; b < B;) {
        uint64_t e = b + 1;
        while (e < B && src[e] == src[e - 1] + width) e++;
        memcpy(dst + b * width, src[b], (e - b) * width * 4);
        b = e;
    }
}

static void prefetch_loop(oxz_loader* l, oxz_data_position pos) {
    Prefetch& q = *l->pre;
    cudaSetDevice(l->device);
    const uint64_t B = l->layout.rank_batch_size;
    std::vector<const uint32_t*> src(B);
    for (;;) {
        int i;
        {
            std::unique_lock<std::mutex> g(q.mu);
            q.cv.wait(g, [&] { return q.stop || !q.idle.empty(); });
            if (q.stop) return;
            i = q.idle.front();
            q.idle.pop_front();
        }
        Prefetch::Slot& slot = q.slots[i];
        cudaEventSynchronize(slot.copied);  // the copy that last read this buffer must be over
        slot.rows.assign(B, 0);
        slot.status = draw_rows(l, pos, slot.rows, src, &slot.next);
        if (slot.status == OXZ_OK) {
            copy_rows(l, src, slot.host);
            pos = slot.next;
        } else {
            slot.error = oxz_last_error();  // the text crosses the thread boundary with the slot
        }
        const bool failed = slot.status != OXZ_OK;
        {
            std::lock_guard<std::mutex> g(q.mu);
            q.ready.push_back(i);
        }
        q.cv.notify_all();
        if (failed) return;
    }
}

static int32_t start_prefetch(oxz_loader* l, uint32_t depth) {
    using namespace oxz;
    const uint64_t B = l->layout.rank_batch_size, width = l->seq_len + 1;
    OXZ_CUDA(cudaSetDevice(l->device));
    l->pre.reset(new Prefetch());
    // `depth` batches kept ready, plus one being filled and one being copied to the device
    l->pre->slots.resize(depth + 2);
    for (size_t i = 0; i < l->pre->slots.size(); i++) {
        cudaError_t e = cudaMallocHost((void**)&l->pre->slots[i].host, B * width * 4);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&l->pre->slots[i].copied, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            stop_prefetch(l);
            return fail(OXZ_ERR_CUDA, "oxz_loader_set_prefetch: %s", cudaGetErrorString(e));
        }
        l->pre->idle.push_back((int)i);
    }
    l->pre->worker = std::thread(prefetch_loop, l, l->pos);
    return OXZ_OK;
}

int32_t oxz_loader_set_prefetch(oxz_loader* l, uint32_t depth) {
    return oxz::guarded("oxz_loader_set_prefetch", [&]() -> int32_t {
        if (!l) return fail(OXZ_ERR_INVALID, "oxz_loader_set_prefetch: null loader");
        if (depth > 64) return fail(OXZ_ERR_INVALID, "oxz_loader_set_prefetch: %u batches ahead, at most 64", depth);
        stop_prefetch(l);
        l->prefetch_depth = depth;
        return depth ? start_prefetch(l, depth) : (int32_t)OXZ_OK;
    });
}

int32_t oxz_loader_next_rows(oxz_loader* l, uint64_t* rows) {
    return oxz::guarded("oxz_loader_next_rows", [&]() -> int32_t {
        if (!l || !rows) return fail(OXZ_ERR_INVALID, "oxz_loader_next_rows: null argument");
        if (l->pre) return fail(OXZ_ERR_STATE, "oxz_loader_next_rows: the prefetch thread draws this loader's rows. Turn prefetching off first");
        const uint64_t B = l->layout.rank_batch_size;
        std::vector<uint64_t> row_ids(B);
        std::vector<const uint32_t*> src(B);
        oxz_data_position next;
        OXZ_TRY(draw_rows(l, l->pos, row_ids, src, &next));
        memcpy(rows, row_ids.data(), B * 8);
        l->pos = next;
        return OXZ_OK;
    });
}

int32_t oxz_loader_next_batch_async(oxz_loader* l, void* stream, int64_t** inputs, int64_t** targets, uint64_t* rows) {
    return oxz::guarded("oxz_loader_next_batch_async", [&]() -> int32_t {
        if (!l || !inputs || !targets) return fail(OXZ_ERR_INVALID, "oxz_loader_next_batch_async: null argument");
        const uint64_t B = l->layout.rank_batch_size, S = l->seq_len, width = S + 1;
        OXZ_CUDA(cudaSetDevice(l->device));
        if (!l->d_stage[0]) {
            for (int i = 0; i < 2; i++) {
                OXZ_CUDA(cudaMallocHost((void**)&l->h_stage[i], B * width * 4));
                OXZ_CUDA(cudaMalloc((void**)&l->d_stage[i], B * width * 4));
                OXZ_CUDA(cudaMalloc((void**)&l->d_inputs[i], B * S * 8));
                OXZ_CUDA(cudaMalloc((void**)&l->d_targets[i], B * S * 8));
                OXZ_CUDA(cudaEventCreateWithFlags(&l->staged[i], cudaEventDisableTiming));
            }
        }
        oxz_data_position next;
        std::vector<uint64_t> row_ids(B);
        const int k = l->slot;
        cudaStream_t s = (cudaStream_t)stream;
        // the pinned buffers of this slot (tokens in, counts out) may still be in use by the batch issued two batches ago
        OXZ_CUDA(cudaEventSynchronize(l->staged[k]));
        if (l->pre) {
            // the worker has the rows in a pinned buffer already, or is about to
            Prefetch& q = *l->pre;
            int i;
            {
                std::unique_lock<std::mutex> g(q.mu);
                q.cv.wait(g, [&] { return !q.ready.empty(); });
                i = q.ready.front();
                q.ready.pop_front();
            }
            Prefetch::Slot& slot = q.slots[i];
            if (slot.status != OXZ_OK) {
                const int32_t st = slot.status;
                const std::string text = slot.error;
                stop_prefetch(l);  // the worker has left; a seek or a new set_prefetch starts another
                oxz_set_last_error(text.c_str());
                return st;
            }
            row_ids = slot.rows;
            next = slot.next;
            OXZ_CUDA(cudaMemcpyAsync(l->d_stage[k], slot.host, B * width * 4, cudaMemcpyHostToDevice, s));
            OXZ_CUDA(cudaEventRecord(slot.copied, s));
            {
                std::lock_guard<std::mutex> g(q.mu);
                q.idle.push_back(i);
            }
            q.cv.notify_all();
        } else {
            std::vector<const uint32_t*> src(B);
            OXZ_TRY(draw_rows(l, l->pos, row_ids, src, &next));
            copy_rows(l, src, l->h_stage[k]);
            OXZ_CUDA(cudaMemcpyAsync(l->d_stage[k], l->h_stage[k], B * width * 4, cudaMemcpyHostToDevice, s));
        }
        const uint64_t n = B * S;
        const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
        const bool masked = l->target_mask || l->document_mask;
        if (!l->h_counts[0])
            for (int i = 0; i < 2; i++) OXZ_CUDA(cudaMallocHost((void**)&l->h_counts[i], 16));
        if (masked && !l->d_loss_mask[0]) {
            for (int i = 0; i < 2; i++) {
                OXZ_CUDA(cudaMalloc((void**)&l->d_loss_mask[i], n * 4));
                OXZ_CUDA(cudaMalloc((void**)&l->d_counts[i], 16));
            }
        }
        if (l->document_mask && !l->d_seg_ids[0]) {
            for (int i = 0; i < 2; i++) {
                OXZ_CUDA(cudaMalloc((void**)&l->d_seg_ids[i], n * 4));
                OXZ_CUDA(cudaMalloc((void**)&l->d_cu[i], (n + 1) * 4));
                OXZ_CUDA(cudaMalloc((void**)&l->d_row_base[i], (B + 1) * 4));
            }
        }
        if (!masked) {
            k_split_rows<<<blocks ? blocks : 1, 256, 0, s>>>(l->d_stage[k], B, S, l->d_inputs[k], l->d_targets[k]);
            l->h_counts[k][0] = n;  // an unmasked batch scores every position (src/data/host_masks.rs:56-57)
            l->h_counts[k][1] = 0;
        } else {
            MaskRule rule{};
            rule.has_target = l->target_mask ? 1 : 0;
            rule.has_document = l->document_mask ? 1 : 0;
            rule.target_base = l->target_base;
            rule.n_always = l->n_always;
            rule.separator = l->separator;
            for (uint32_t i = 0; i < l->n_always; i++) rule.always[i] = l->always[i];
            OXZ_CUDA(cudaMemsetAsync(l->d_counts[k], 0, 16, s));
            k_split_rows_masked<<<blocks ? blocks : 1, 256, 0, s>>>(l->d_stage[k], B, S, rule, l->d_inputs[k], l->d_targets[k],
                                                                   l->d_loss_mask[k], l->d_counts[k]);
            if (l->document_mask) {
                k_row_closings<<<(unsigned)((B * 32 + 255) / 256), 256, 0, s>>>(l->d_stage[k], (uint32_t)B, (uint32_t)S, l->separator, l->d_row_base[k]);
                k_scan_rows<<<1, 256, 0, s>>>(l->d_row_base[k], (uint32_t)B, l->d_cu[k], l->d_counts[k]);
                k_fill_segments<<<(unsigned)B, 256, 0, s>>>(l->d_stage[k], (uint32_t)S, l->separator, l->d_row_base[k], l->d_seg_ids[k], l->d_cu[k]);
            }
            OXZ_CUDA(cudaMemcpyAsync(l->h_counts[k], l->d_counts[k], 16, cudaMemcpyDeviceToHost, s));
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "launch of the batch kernels failed: %s", cudaGetErrorString(e));
        // marks the point after which this slot's pinned buffers (tokens in, counts out) may be touched again
        OXZ_CUDA(cudaEventRecord(l->staged[k], s));
        l->last = k;
        *inputs = l->d_inputs[k];
        *targets = l->d_targets[k];
        if (rows) memcpy(rows, row_ids.data(), B * 8);
        l->pos = next;
        l->slot ^= 1;
        return OXZ_OK;
    });
}

int32_t oxz_loader_set_target_mask(oxz_loader* l, int32_t on, uint32_t target_base, const uint32_t* always_score, uint32_t n_always) {
    return oxz::guarded("oxz_loader_set_target_mask", [&]() -> int32_t {
        if (!l || (on && n_always && !always_score)) return fail(OXZ_ERR_INVALID, "oxz_loader_set_target_mask: null argument");
        if (on && n_always > OXZ_MAX_ALWAYS_SCORE)
            return fail(OXZ_ERR_INVALID, "oxz_loader_set_target_mask: %u always-scored ids, at most %u", n_always, OXZ_MAX_ALWAYS_SCORE);
        l->target_mask = on != 0;
        l->target_base = target_base;
        l->n_always = on ? n_always : 0;
        for (uint32_t i = 0; i < l->n_always; i++) l->always[i] = always_score[i];
        return OXZ_OK;
    });
}

int32_t oxz_loader_set_document_mask(oxz_loader* l, int32_t on, uint32_t separator_id) {
    return oxz::guarded("oxz_loader_set_document_mask", [&]() -> int32_t {
        if (!l) return fail(OXZ_ERR_INVALID, "oxz_loader_set_document_mask: null loader");
        if (on && l->layout.rank_batch_size * l->seq_len > 0x7fffffffull)
            return fail(OXZ_ERR_DATA,
                        "a batch of %llu x %llu tokens overflows the i32 segment offsets. Lower trainer.batch_size or "
                        "model.max_seq_len.", (unsigned long long)l->layout.rank_batch_size, (unsigned long long)l->seq_len);
        l->document_mask = on != 0;
        l->separator = separator_id;
        return OXZ_OK;
    });
}

int32_t oxz_loader_batch_masks(const oxz_loader* l, oxz_batch_masks* out) {
    return oxz::guarded("oxz_loader_batch_masks", [&]() -> int32_t {
        if (!l || !out) return fail(OXZ_ERR_INVALID, "oxz_loader_batch_masks: null argument");
        if (l->last < 0) return fail(OXZ_ERR_STATE, "oxz_loader_batch_masks: no batch has been drawn yet");
        const int k = l->last;
        const bool masked = l->d_loss_mask[k] && (l->target_mask || l->document_mask);
        const bool segs = l->d_seg_ids[k] && l->document_mask;
        out->loss_mask = masked ? l->d_loss_mask[k] : nullptr;
        out->segment_ids = segs ? l->d_seg_ids[k] : nullptr;
        out->cu_seqlens = segs ? l->d_cu[k] : nullptr;
        out->scored = reinterpret_cast<const uint64_t*>(&l->h_counts[k][0]);
        out->n_segments = reinterpret_cast<const uint64_t*>(&l->h_counts[k][1]);
        return OXZ_OK;
    });
}

}  // extern "C"
