// The rank-sliced row loader in stream order: a little-endian u32 token file, mapped read-only, rows of
// seq_len + 1 tokens, rank k reading slots [start.row + k*B, +B) of each global batch of B*world rows
// (src/data/source.rs:7-12,204-230, src/data/positioning.rs:44-68, src/data/rows.rs:150-165). The rows a rank draws
// are consecutive in the file, so one step is one pinned staging copy, one host-to-device copy and one kernel that
// widens the ids to i64 and writes inputs [B,S] and targets [B,S] (src/data/batch.rs:51-71).
// The shuffled order depends on rand 0.10.3's StdRng and is not offered.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

#include "oxz_internal.h"

struct oxz_loader {
    int fd = -1;
    const uint32_t* tokens = nullptr;
    size_t map_bytes = 0;
    uint64_t n_tokens = 0, seq_len = 0, first_row = 0;
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

void release(oxz_loader* l) {
    if (!l) return;
    if (l->d_stage[0] || l->h_stage[0]) cudaSetDevice(l->device);
    for (int i = 0; i < 2; i++) {
        if (l->h_stage[i]) cudaFreeHost(l->h_stage[i]);
        if (l->d_stage[i]) cudaFree(l->d_stage[i]);
        if (l->d_inputs[i]) cudaFree(l->d_inputs[i]);
        if (l->d_targets[i]) cudaFree(l->d_targets[i]);
        if (l->staged[i]) cudaEventDestroy(l->staged[i]);
    }
    if (l->tokens) munmap(const_cast<uint32_t*>(l->tokens), l->map_bytes);
    if (l->fd >= 0) close(l->fd);
    delete l;
}

}  // namespace

using namespace oxz;

extern "C" {

int32_t oxz_loader_open(const char* path, uint64_t seq_len, uint64_t rank_batch_size, uint64_t rank, uint64_t world,
                        uint64_t first_row, uint64_t end_row, int32_t device, oxz_loader** out) {
    if (!path || !out) return fail(OXZ_ERR_INVALID, "oxz_loader_open: null argument");
    *out = nullptr;
    if (seq_len == 0) return fail(OXZ_ERR_DATA, "model.max_seq_len is 0: a row needs at least one input and one target token");
    oxz_loader* l = new oxz_loader();
    l->fd = open(path, O_RDONLY);
    if (l->fd < 0) {
        int32_t s = fail(OXZ_ERR_DATA, "failed to open data file %s: %s", path, strerror(errno));
        release(l);
        return s;
    }
    struct stat st;
    if (fstat(l->fd, &st) != 0) {
        int32_t s = fail(OXZ_ERR_DATA, "failed to stat data file %s: %s", path, strerror(errno));
        release(l);
        return s;
    }
    if (st.st_size % 4 != 0) {
        int32_t s = fail(OXZ_ERR_DATA, "data file %s is %lld bytes, not a multiple of 4: it is not a u32 token file", path, (long long)st.st_size);
        release(l);
        return s;
    }
    l->n_tokens = (uint64_t)st.st_size / 4;
    if (st.st_size > 0) {
        void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, l->fd, 0);
        if (m == MAP_FAILED) {
            int32_t s = fail(OXZ_ERR_DATA, "failed to mmap data file %s: %s", path, strerror(errno));
            release(l);
            return s;
        }
        l->tokens = static_cast<const uint32_t*>(m);
        l->map_bytes = (size_t)st.st_size;
    }
    const uint64_t total_rows = l->n_tokens / (seq_len + 1);  // the tail shorter than a row is never read
    if (end_row == 0) end_row = total_rows;
    if (first_row >= end_row || end_row > total_rows) {
        int32_t s = fail(OXZ_ERR_DATA, "row range [%llu, %llu) does not fit the data's %llu whole rows", (unsigned long long)first_row,
                         (unsigned long long)end_row, (unsigned long long)total_rows);
        release(l);
        return s;
    }
    l->seq_len = seq_len;
    l->first_row = first_row;
    l->layout = oxz_row_layout{end_row - first_row, rank_batch_size, world};
    l->rank = rank;
    l->device = device;
    int32_t s = oxz_rows_check(&l->layout);
    if (s == OXZ_OK && rank >= world)
        s = fail(OXZ_ERR_DATA, "rank %llu is not below world size %llu. Pass a rank in [0, %llu).", (unsigned long long)rank,
                 (unsigned long long)world, (unsigned long long)world);
    if (s != OXZ_OK) {
        release(l);
        return s;
    }
    *out = l;
    return OXZ_OK;
}

int32_t oxz_loader_close(oxz_loader* l) {
    release(l);
    return OXZ_OK;
}

int32_t oxz_loader_num_rows(const oxz_loader* l, uint64_t* rows) {
    if (!l || !rows) return fail(OXZ_ERR_INVALID, "oxz_loader_num_rows: null argument");
    *rows = l->layout.num_rows;
    return OXZ_OK;
}

int32_t oxz_loader_position(const oxz_loader* l, oxz_data_position* pos) {
    if (!l || !pos) return fail(OXZ_ERR_INVALID, "oxz_loader_position: null argument");
    *pos = l->pos;
    return OXZ_OK;
}

int32_t oxz_loader_seek(oxz_loader* l, oxz_data_position pos) {
    if (!l) return fail(OXZ_ERR_INVALID, "oxz_loader_seek: null loader");
    if (pos.row > l->layout.num_rows)
        return fail(OXZ_ERR_DATA,
                    "data position epoch %llu row %llu is past this shard's %llu rows: the checkpoint was saved over "
                    "different data or a different model.max_seq_len. Resume with the original data and config, or "
                    "start a fresh run.",
                    (unsigned long long)pos.epoch, (unsigned long long)pos.row, (unsigned long long)l->layout.num_rows);
    l->pos = pos;
    return OXZ_OK;
}

int32_t oxz_loader_next_batch_async(oxz_loader* l, void* stream, int64_t** inputs, int64_t** targets, uint64_t* rows) {
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
    OXZ_TRY(oxz_rows_next_window(&l->layout, l->pos, l->rank, S, l->first_row, nullptr, 0, row_ids.data(), nullptr, nullptr, &next));
    if ((row_ids[B - 1] + 1) * width > l->n_tokens)
        return fail(OXZ_ERR_DATA, "row %llu is past the %llu whole rows of this data. This is a loader bug: report it with the data and config.",
                    (unsigned long long)row_ids[B - 1], (unsigned long long)(l->n_tokens / width));
    const int k = l->slot;
    // the pinned buffer of this slot may still feed the copy issued two batches ago
    OXZ_CUDA(cudaEventSynchronize(l->staged[k]));
    // a rank's slots are consecutive rows in stream order: one contiguous span of the file
    memcpy(l->h_stage[k], l->tokens + row_ids[0] * width, B * width * 4);
    cudaStream_t s = (cudaStream_t)stream;
    OXZ_CUDA(cudaMemcpyAsync(l->d_stage[k], l->h_stage[k], B * width * 4, cudaMemcpyHostToDevice, s));
    OXZ_CUDA(cudaEventRecord(l->staged[k], s));
    const uint64_t n = B * S;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    k_split_rows<<<blocks ? blocks : 1, 256, 0, s>>>(l->d_stage[k], B, S, l->d_inputs[k], l->d_targets[k]);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "launch of k_split_rows failed: %s", cudaGetErrorString(e));
    *inputs = l->d_inputs[k];
    *targets = l->d_targets[k];
    if (rows) memcpy(rows, row_ids.data(), B * 8);
    l->pos = next;
    l->slot ^= 1;
    return OXZ_OK;
}

}  // extern "C"
