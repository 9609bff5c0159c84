// The flat layout of the trainable parameters: tile-aligned tensor starts, buckets, per-rank shards and the
// AdamW groups. Pure host code: a plan is built and queried without a GPU.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "oxz_internal.h"

namespace oxz {

static thread_local std::string g_last_error;

int32_t fail(int32_t status, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

void clear_error() { g_last_error.clear(); }

}  // namespace oxz

using namespace oxz;

extern "C" {

uint32_t oxz_abi_version(void) { return OXZ_ABI_VERSION; }

const char* oxz_last_error(void) { return g_last_error.c_str(); }

const char* oxz_status_name(int32_t status) {
    switch (status) {
        case OXZ_OK: return "OXZ_OK";
        case OXZ_ERR_INVALID: return "OXZ_ERR_INVALID";
        case OXZ_ERR_CUDA: return "OXZ_ERR_CUDA";
        case OXZ_ERR_NCCL: return "OXZ_ERR_NCCL";
        case OXZ_ERR_STATE: return "OXZ_ERR_STATE";
        case OXZ_ERR_ABORTED: return "OXZ_ERR_ABORTED";
        case OXZ_ERR_UNSUPPORTED: return "OXZ_ERR_UNSUPPORTED";
        case OXZ_ERR_DATA: return "OXZ_ERR_DATA";
        case OXZ_ERR_TIMEOUT: return "OXZ_ERR_TIMEOUT";
        default: return "OXZ_ERR_UNKNOWN";
    }
}

int32_t oxz_plan_create(const oxz_plan_desc* d, oxz_plan** out) {
    return oxz::guarded("oxz_plan_create", [&]() -> int32_t {
        if (!d || !out) return fail(OXZ_ERR_INVALID, "oxz_plan_create: null argument");
        *out = nullptr;
        if (d->n_tensors > 0 && !d->numel) return fail(OXZ_ERR_INVALID, "oxz_plan_create: numel is null");
        if (d->n_tensors >= (1u << 24))
            return fail(OXZ_ERR_INVALID, "oxz_plan_create: %llu tensors, at most %u fit a tile entry",
                        (unsigned long long)d->n_tensors, (1u << 24) - 1);
        for (int32_t dt : {d->grad_dtype, d->param_dtype})
            if (dt != OXZ_F32 && dt != OXZ_BF16 && dt != OXZ_F16)
                return fail(OXZ_ERR_INVALID, "oxz_plan_create: dtype %d is none of f32, bf16, f16", dt);
        if (d->world < 1 || d->world > (int32_t)MAX_PEERS)
            return fail(OXZ_ERR_INVALID, "oxz_plan_create: world size %d is outside [1, %u]", d->world, MAX_PEERS);
        if (d->rank < 0 || d->rank >= d->world)
            return fail(OXZ_ERR_INVALID, "rank %d is not below world size %d. Pass a rank in [0, %d).", d->rank,
                        d->world, d->world);
        if (d->sync_mode < OXZ_SYNC_SINGLE || d->sync_mode > OXZ_SYNC_REPLICATED)
            return fail(OXZ_ERR_INVALID, "oxz_plan_create: unknown sync mode %d", d->sync_mode);
        if ((d->sync_mode == OXZ_SYNC_SINGLE) != (d->world == 1))
            return fail(OXZ_ERR_INVALID,
                        "oxz_plan_create: sync mode %d with world size %d. World 1 runs no collective and takes "
                        "OXZ_SYNC_SINGLE; more ranks need OXZ_SYNC_P2P, OXZ_SYNC_COPY, OXZ_SYNC_NCCL or OXZ_SYNC_REPLICATED",
                        d->sync_mode, d->world);

        oxz_plan* p = new oxz_plan();
        p->T = d->n_tensors;
        p->gdt = d->grad_dtype;
        p->pdt = d->param_dtype;
        p->cw = d->world;
        p->cr = d->rank;
        // full replicas: the layout of a single rank, the communicator's size only for the gradient sum
        p->world = d->sync_mode == OXZ_SYNC_REPLICATED ? 1 : d->world;
        p->rank = d->sync_mode == OXZ_SYNC_REPLICATED ? 0 : d->rank;
        p->mode = d->sync_mode;
        p->device = d->device;
        p->numel.assign(d->numel, d->numel + d->n_tensors);
        p->offset.resize(p->T);
        p->group_of.resize(p->T);

        // groups: distinct (lr_scale, no_decay) pairs in first-seen order
        for (uint64_t i = 0; i < p->T; i++) {
            const float ls = d->lr_scale ? d->lr_scale[i] : 1.0f;
            const uint8_t nd = d->no_decay ? (d->no_decay[i] ? 1 : 0) : 0;
            if (!(std::isfinite(ls) && ls >= 0.0f)) {
                delete p;
                return fail(OXZ_ERR_INVALID, "oxz_plan_create: lr_scale[%llu] is %g: it must be finite and not negative",
                            (unsigned long long)i, (double)ls);
            }
            size_t gi = 0;
            for (; gi < p->group_lr_scale.size(); gi++)
                if (p->group_lr_scale[gi] == ls && p->group_no_decay[gi] == nd) break;
            if (gi == p->group_lr_scale.size()) {
                if (gi == MAX_GROUPS) {
                    delete p;
                    return fail(OXZ_ERR_INVALID, "oxz_plan_create: more than %u distinct (lr_scale, decay) groups", MAX_GROUPS);
                }
                p->group_lr_scale.push_back(ls);
                p->group_no_decay.push_back(nd);
            }
            p->group_of[i] = (uint8_t)gi;
        }
        if (p->group_lr_scale.empty()) {
            p->group_lr_scale.push_back(1.0f);
            p->group_no_decay.push_back(0);
        }

        // tile-aligned tensor starts
        uint64_t tiles = 0;
        for (uint64_t i = 0; i < p->T; i++) {
            p->offset[i] = tiles * TILE;
            tiles += (p->numel[i] + TILE - 1) / TILE;
            p->numel_total += p->numel[i];
        }
        const uint64_t W = (uint64_t)p->world;
        uint64_t total = ((tiles + W - 1) / W) * W;
        if (total == 0) total = W;
        if (total >= 0xFFFFFFFFull) {
            delete p;
            return fail(OXZ_ERR_INVALID, "oxz_plan_create: %llu tiles do not fit 32-bit tile indices",
                        (unsigned long long)total);
        }
        p->total_tiles = total;

        const uint64_t bucket_bytes = d->bucket_bytes ? d->bucket_bytes : (64ull << 20);
        uint64_t bt = bucket_bytes / (TILE * dtype_size(p->gdt));
        bt = (bt / W) * W;
        if (bt < W) bt = W;
        if (bt > total) bt = total;
        p->bucket_tiles = bt;
        p->n_buckets = (total + bt - 1) / bt;
        p->last_bucket_tiles = total - (p->n_buckets - 1) * bt;
        p->local_tiles = total / W;

        p->tile_meta.assign(total, PAD_TILE);
        for (uint64_t i = 0; i < p->T; i++) {
            const uint64_t first = p->offset[i] / TILE, n = (p->numel[i] + TILE - 1) / TILE;
            const uint32_t meta = (uint32_t)i | ((uint32_t)p->group_of[i] << 24);
            for (uint64_t t = 0; t < n; t++) p->tile_meta[first + t] = meta;
        }
        *out = p;
        return OXZ_OK;
    });
}

int32_t oxz_plan_query(const oxz_plan* p, oxz_plan_info* info) {
    return oxz::guarded("oxz_plan_query", [&]() -> int32_t {
        if (!p || !info) return fail(OXZ_ERR_INVALID, "oxz_plan_query: null argument");
        info->n_tensors = p->T;
        info->numel_total = p->numel_total;
        info->padded_total = p->total_tiles * TILE;
        info->tile_elems = TILE;
        info->n_buckets = p->n_buckets;
        info->bucket_elems = p->bucket_tiles * TILE;
        info->local_elems = p->local_tiles * TILE;
        info->n_groups = p->group_lr_scale.size();
        return OXZ_OK;
    });
}

int32_t oxz_plan_tensor_offsets(const oxz_plan* p, uint64_t* offsets) {
    return oxz::guarded("oxz_plan_tensor_offsets", [&]() -> int32_t {
        if (!p || (!offsets && p->T)) return fail(OXZ_ERR_INVALID, "oxz_plan_tensor_offsets: null argument");
        for (uint64_t i = 0; i < p->T; i++) offsets[i] = p->offset[i];
        return OXZ_OK;
    });
}

int32_t oxz_plan_bucket(const oxz_plan* p, uint64_t b, int32_t rank, uint64_t* start, uint64_t* len,
                        uint64_t* shard_start, uint64_t* shard_len) {
    return oxz::guarded("oxz_plan_bucket", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_plan_bucket: null plan");
        if (b >= p->n_buckets)
            return fail(OXZ_ERR_INVALID, "oxz_plan_bucket: bucket %llu of %llu", (unsigned long long)b,
                        (unsigned long long)p->n_buckets);
        if (rank < 0 || rank >= p->cw)
            return fail(OXZ_ERR_INVALID, "rank %d is not below world size %d. Pass a rank in [0, %d).", rank, p->cw,
                        p->cw);
        if (p->mode == OXZ_SYNC_REPLICATED) rank = 0;  // every rank owns everything
        const uint64_t tiles = (b == p->n_buckets - 1) ? p->last_bucket_tiles : p->bucket_tiles;
        const uint64_t shard = tiles / (uint64_t)p->world;
        const uint64_t s = b * p->bucket_tiles;
        if (start) *start = s * TILE;
        if (len) *len = tiles * TILE;
        if (shard_start) *shard_start = (s + (uint64_t)rank * shard) * TILE;
        if (shard_len) *shard_len = shard * TILE;
        return OXZ_OK;
    });
}

int32_t oxz_plan_local_index(const oxz_plan* p, int32_t rank, uint64_t flat_index, uint64_t* local_index) {
    return oxz::guarded("oxz_plan_local_index", [&]() -> int32_t {
        if (!p || !local_index) return fail(OXZ_ERR_INVALID, "oxz_plan_local_index: null argument");
        if (rank < 0 || rank >= p->cw)
            return fail(OXZ_ERR_INVALID, "rank %d is not below world size %d. Pass a rank in [0, %d).", rank, p->cw,
                        p->cw);
        if (p->mode == OXZ_SYNC_REPLICATED) rank = 0;  // every rank owns everything
        if (flat_index >= p->total_tiles * TILE)
            return fail(OXZ_ERR_INVALID, "oxz_plan_local_index: element %llu is past the flat space of %llu",
                        (unsigned long long)flat_index, (unsigned long long)(p->total_tiles * TILE));
        const uint64_t ft = flat_index / TILE;
        const uint64_t b = ft / p->bucket_tiles;
        const uint64_t tiles = (b == p->n_buckets - 1) ? p->last_bucket_tiles : p->bucket_tiles;
        const uint64_t shard = tiles / (uint64_t)p->world;
        const uint64_t within = ft - b * p->bucket_tiles;
        if (within / shard != (uint64_t)rank) {
            *local_index = UINT64_MAX;
            return OXZ_OK;
        }
        const uint64_t full_shard = p->bucket_tiles / (uint64_t)p->world;
        const uint64_t lt = b * full_shard + (within - (uint64_t)rank * shard);
        *local_index = lt * TILE + flat_index % TILE;
        return OXZ_OK;
    });
}

}  // extern "C"
