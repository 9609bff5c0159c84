// Optimizer-state file in the reference's layout (src/checkpoint_set/optimizer_io.rs:1-5): a SafeTensors file keyed
// `<name>.exp_avg`, `<name>.exp_avg_sq`, `<name>.master` (parameters narrower than f32 only) and `__step` (F64),
// with the metadata {"format": "oxidizr-optimizer", "optimizer": "adamw"} (optimizer_io.rs:20, 66-74).
// With several ranks each owns a slice of the state: the slices are merged bit for bit before rank 0 writes, and
// every rank reads the whole file and keeps what it owns.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>

#include "oxz_internal.h"
#include "oxz_json.h"
#include "oxz_nccl.h"

using namespace oxz;

namespace {

struct Entry {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;
};

bool parse_header(const std::string& text, std::map<std::string, Entry>& out) {
    JsonReader j{text.data(), text.data() + text.size()};
    j.object([&](const std::string& name) {
        if (name == "__metadata__") { j.skip(); return; }
        Entry en;
        j.object([&](const std::string& key) {
            if (key == "dtype") en.dtype = j.str();
            else if (key == "shape" || key == "data_offsets") {
                std::vector<uint64_t> v;
                if (!j.eat('[')) { j.ok = false; return; }
                if (!j.eat(']')) {
                    do { uint64_t x = 0; j.u64(&x); v.push_back(x); } while (j.ok && j.eat(','));
                    if (!j.eat(']')) j.ok = false;
                }
                if (key == "shape") en.shape = v;
                else if (v.size() == 2) { en.begin = v[0]; en.end = v[1]; }
                else j.ok = false;
            } else j.skip();
        });
        if (j.ok) out[name] = en;
    });
    j.ws();
    return j.ok && j.p == j.e;
}

std::string json_escape(const char* s) {
    std::string out;
    for (; *s; s++) {
        if (*s == '"' || *s == '\\') { out += '\\'; out += *s; }
        else if ((unsigned char)*s < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", *s); out += b; }
        else out += *s;
    }
    return out;
}

int32_t io_fail(const char* path, const char* what, const char* next) {
    return fail(OXZ_ERR_INVALID, "optimizer state file '%s': %s: %s. %s", path, what, strerror(errno), next);
}

uint64_t shape_numel(const uint64_t* dims, uint32_t nd) {
    uint64_t n = 1;
    for (uint32_t i = 0; i < nd; i++) n *= dims[i];
    return n;
}

float* array_of(oxz_plan* p, int kind) {
    return kind == OXZ_STATE_MASTER ? p->master : kind == OXZ_STATE_EXP_AVG ? p->exp_avg : p->exp_avg_sq;
}

// The whole of one tensor's state on the host: this rank's slices, merged with the other ranks' through a sum of the
// raw 32-bit patterns (exactly one rank contributes non-zero bits per element, so every bit survives, -0.0 included).
// `d` is device scratch of at least n words that every rank allocated (and agreed on) before the first gather, so no
// rank can drop out of a collective here for want of memory.
int32_t gather_tensor(oxz_plan* p, oxz_comm* comm, int kind, uint64_t t, std::vector<uint32_t>& host, uint32_t* d) {
    const uint64_t n = p->numel[t];
    host.assign(n, 0u);
    if (n == 0) return OXZ_OK;
    if (p->world == 1) return oxz_state_export(p, kind, t, host.data());
    OXZ_CUDA(cudaMemsetAsync(d, 0, n * 4, p->stream));
    const float* arr = array_of(p, kind);
    const uint64_t lo = p->offset[t], hi = lo + n, be = p->bucket_tiles * TILE, full = be / (uint64_t)p->world;
    for (uint64_t b = lo / be; b < p->n_buckets && b * be < hi; b++) {
        const uint64_t tiles = (b == p->n_buckets - 1) ? p->last_bucket_tiles : p->bucket_tiles;
        const uint64_t shard = tiles * TILE / (uint64_t)p->world;
        const uint64_t s0 = b * be + (uint64_t)p->rank * shard, s1 = s0 + shard;
        const uint64_t a = lo > s0 ? lo : s0, z = hi < s1 ? hi : s1;
        if (a < z)
            OXZ_CUDA(cudaMemcpyAsync(d + (a - lo), arr + b * full + (a - s0), (z - a) * 4, cudaMemcpyDeviceToDevice, p->stream));
    }
    int32_t st = comm_stream_allreduce_u32(comm, d, n, p->stream);
    if (st == OXZ_OK) {
        cudaError_t e = cudaMemcpyAsync(host.data(), d, n * 4, cudaMemcpyDeviceToHost, p->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(p->stream);
        if (e != cudaSuccess) st = fail(OXZ_ERR_CUDA, "oxz_optimizer_save: %s", cudaGetErrorString(e));
    }
    return st;
}

// Every rank hands in whether it failed; all leave knowing whether any did. One word through the communicator.
int32_t agree_on_failure(oxz_plan* p, oxz_comm* comm, bool failed, bool* any_failed) {
    *any_failed = failed;
    if (p->world == 1) return OXZ_OK;
    uint32_t* d_flag = reinterpret_cast<uint32_t*>(static_cast<char*>(comm->d_small) + 128);
    const uint32_t mine = failed ? 1u : 0u;
    uint32_t all = 0;
    OXZ_CUDA(cudaMemcpyAsync(d_flag, &mine, 4, cudaMemcpyHostToDevice, p->stream));
    OXZ_TRY(comm_stream_allreduce_u32(comm, d_flag, 1, p->stream));
    OXZ_CUDA(cudaMemcpyAsync(&all, d_flag, 4, cudaMemcpyDeviceToHost, p->stream));
    OXZ_CUDA(cudaStreamSynchronize(p->stream));
    *any_failed = all != 0;
    return OXZ_OK;
}

int32_t check_call(oxz_plan* p, oxz_comm* comm, const char* path, const char* const* names, const uint32_t* ndim,
                   const uint64_t* dims, const char* who) {
    if (!p || !path || (p->T && (!names || !ndim || !dims))) return fail(OXZ_ERR_INVALID, "%s: null argument", who);
    if (!p->allocated) return fail(OXZ_ERR_STATE, "%s: the plan has no device state. Call oxz_state_alloc first", who);
    if (p->inflight) return fail(OXZ_ERR_STATE, "%s: a step is in flight. Call oxz_step_wait first", who);
    if (p->world > 1) {
        OXZ_TRY(comm_check(comm, who));
        if (comm != p->comm) return fail(OXZ_ERR_INVALID, "%s: this is not the communicator the state was allocated with", who);
    }
    const uint64_t* d = dims;
    for (uint64_t i = 0; i < p->T; i++) {
        if (!names[i]) return fail(OXZ_ERR_INVALID, "%s: tensor %llu has no checkpoint name", who, (unsigned long long)i);
        if (shape_numel(d, ndim[i]) != p->numel[i])
            return fail(OXZ_ERR_INVALID, "%s: the shape of '%s' holds %llu elements, the plan %llu", who, names[i],
                        (unsigned long long)shape_numel(d, ndim[i]), (unsigned long long)p->numel[i]);
        d += ndim[i];
    }
    return OXZ_OK;
}

}  // namespace

extern "C" {

int32_t oxz_optimizer_save(oxz_plan* p, oxz_comm* comm, const char* path, const char* const* names,
                           const uint32_t* ndim, const uint64_t* dims) {
    return oxz::guarded("oxz_optimizer_save", [&]() -> int32_t {
        OXZ_TRY(check_call(p, comm, path, names, ndim, dims, "oxz_optimizer_save"));
        OXZ_CUDA(cudaSetDevice(p->device));
        const bool has_master = p->pdt != OXZ_F32;
        const bool writer = p->cr == 0;  // with full replicas every rank holds everything and rank 0 alone writes
        const char* next = "Check that the checkpoint directory is writable and has free space.";

        // header: entries in the order the data is written
        std::string header = "{\"__metadata__\":{\"format\":\"oxidizr-optimizer\",\"optimizer\":\"adamw\"}";
        uint64_t off = 0;
        const int kinds[3] = {OXZ_STATE_EXP_AVG, OXZ_STATE_EXP_AVG_SQ, OXZ_STATE_MASTER};
        const char* suffix[3] = {".exp_avg", ".exp_avg_sq", ".master"};
        {
            const uint64_t* d = dims;
            for (uint64_t i = 0; i < p->T; i++) {
                std::string shape = "[";
                for (uint32_t k = 0; k < ndim[i]; k++) shape += (k ? "," : "") + std::to_string(d[k]);
                shape += "]";
                for (int k = 0; k < (has_master ? 3 : 2); k++) {
                    header += ",\"" + json_escape(names[i]) + suffix[k] + "\":{\"dtype\":\"F32\",\"shape\":" + shape +
                              ",\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + p->numel[i] * 4) + "]}";
                    off += p->numel[i] * 4;
                }
                d += ndim[i];
            }
            header += ",\"__step\":{\"dtype\":\"F64\",\"shape\":[1],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + 8) + "]}}";
            while (header.size() % 8) header += ' ';
        }

        std::string tmp = std::string(path) + ".tmp";
        FILE* f = nullptr;
        // A file error on the writing rank must not leave the other ranks waiting in the gathers below: the writer
        // remembers it, keeps taking part in every collective, and reports it at the end.
        int32_t io = OXZ_OK;
        std::string io_text;
        auto io_failed = [&]() {
            if (io == OXZ_OK) {
                io = io_fail(path, "write failed", next);
                io_text = oxz_last_error();
            }
            if (f) { fclose(f); f = nullptr; }
        };
        if (writer) {
            f = fopen(tmp.c_str(), "wb");
            const uint64_t hl = header.size();
            if (!f || fwrite(&hl, 8, 1, f) != 1 || fwrite(header.data(), 1, hl, f) != hl) io_failed();
        }
        std::vector<uint32_t> host;
        int32_t st = OXZ_OK;
        // the merge scratch, sized for the largest tensor: allocated by every rank, and agreed on, before any gather
        uint32_t* d_merge = nullptr;
        if (p->world > 1) {
            uint64_t widest = 1;
            for (uint64_t i = 0; i < p->T; i++) widest = p->numel[i] > widest ? p->numel[i] : widest;
            const cudaError_t e = cudaMalloc((void**)&d_merge, widest * 4);
            if (e != cudaSuccess) cudaGetLastError();
            bool any = false;
            st = agree_on_failure(p, comm, e != cudaSuccess, &any);
            if (st == OXZ_OK && any)
                st = e != cudaSuccess ? fail(OXZ_ERR_CUDA, "oxz_optimizer_save: no device memory for the merge of %llu elements: %s", (unsigned long long)widest, cudaGetErrorString(e))
                                      : fail(OXZ_ERR_STATE, "oxz_optimizer_save: another rank has no device memory for the merge; nothing was written");
        }
        for (uint64_t i = 0; i < p->T && st == OXZ_OK; i++) {
            for (int k = 0; k < (has_master ? 3 : 2) && st == OXZ_OK; k++) {
                st = gather_tensor(p, comm, kinds[k], i, host, d_merge);
                if (st == OXZ_OK && f && !host.empty() && fwrite(host.data(), 4, host.size(), f) != host.size()) io_failed();
            }
        }
        if (d_merge) cudaFree(d_merge);
        if (writer) {
            const double step = (double)p->timestep;
            if (st == OXZ_OK && f && fwrite(&step, 8, 1, f) != 1) io_failed();
            if (f && fclose(f) != 0) { f = nullptr; io_failed(); }
            f = nullptr;
            // atomic: an error leaves an existing file unchanged (optimizer_io.rs:62-64)
            if (st == OXZ_OK && io == OXZ_OK && rename(tmp.c_str(), path) != 0) io_failed();
            if (st != OXZ_OK || io != OXZ_OK) remove(tmp.c_str());
            if (st == OXZ_OK && io != OXZ_OK) {
                oxz_set_last_error(io_text.c_str());
                st = io;
            }
        }
        // Only the writing rank sees a file error. Every rank must leave with the same answer, or the others would
        // take a checkpoint that does not exist for written: one more word crosses the ranks (when the collectives
        // themselves still work).
        if (p->world > 1 && (st == OXZ_OK || (writer && st == io && io != OXZ_OK))) {
            const std::string mine = st != OXZ_OK ? std::string(oxz_last_error()) : std::string();
            bool any = false;
            const int32_t agreed = agree_on_failure(p, comm, st != OXZ_OK, &any);
            if (agreed != OXZ_OK) return agreed;
            if (st != OXZ_OK) oxz_set_last_error(mine.c_str());
            else if (any) st = fail(OXZ_ERR_INVALID, "optimizer state file '%s': the writing rank could not write it (its own error text says why); nothing was saved", path);
        }
        return st;
    });
}

int32_t oxz_optimizer_load(oxz_plan* p, const char* path, const char* const* names, const uint32_t* ndim,
                           const uint64_t* dims) {
    return oxz::guarded("oxz_optimizer_load", [&]() -> int32_t {
        OXZ_TRY(check_call(p, p ? p->comm : nullptr, path, names, ndim, dims, "oxz_optimizer_load"));
        OXZ_CUDA(cudaSetDevice(p->device));
        const char* next = "Restore the file from the run that wrote it.";
        const char* mismatch = "The file does not match this model's trainable parameters. Resume with the config that wrote this checkpoint.";
        FILE* f = fopen(path, "rb");
        if (!f) return io_fail(path, "open failed", next);
        uint64_t hl = 0;
        if (fread(&hl, 8, 1, f) != 1 || hl == 0 || hl > (1ull << 30)) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': open failed: not a SafeTensors file. %s", path, next); }
        std::string text(hl, '\0');
        if (fread(&text[0], 1, hl, f) != hl) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': open failed: truncated header. %s", path, next); }
        std::map<std::string, Entry> entries;
        if (!parse_header(text, entries)) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': open failed: the header is not valid JSON. %s", path, next); }
        const uint64_t data0 = 8 + hl;

        // strict and atomic (optimizer_io.rs:113-116): every check runs before anything is loaded
        const bool has_master = p->pdt != OXZ_F32;
        const char* suffix[3] = {".exp_avg", ".exp_avg_sq", ".master"};
        const int kinds[3] = {OXZ_STATE_EXP_AVG, OXZ_STATE_EXP_AVG_SQ, OXZ_STATE_MASTER};
        size_t expected = 1;
        {
            const uint64_t* d = dims;
            for (uint64_t i = 0; i < p->T; i++) {
                for (int k = 0; k < (has_master ? 3 : 2); k++) {
                    const std::string key = std::string(names[i]) + suffix[k];
                    auto it = entries.find(key);
                    if (it == entries.end()) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': load failed: missing key '%s'. %s", path, key.c_str(), mismatch); }
                    const Entry& en = it->second;
                    bool same = en.shape.size() == ndim[i];
                    for (uint32_t q = 0; same && q < ndim[i]; q++) same = en.shape[q] == d[q];
                    if (!same) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': load failed: shape mismatch for '%s'. %s", path, key.c_str(), mismatch); }
                    if (en.dtype != "F32" || en.end - en.begin != p->numel[i] * 4) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': load failed: dtype mismatch for '%s' (%s). %s", path, key.c_str(), en.dtype.c_str(), mismatch); }
                    expected++;
                }
                d += ndim[i];
            }
        }
        auto st_it = entries.find("__step");
        if (st_it == entries.end() || st_it->second.dtype != "F64" || st_it->second.end - st_it->second.begin != 8) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': load failed: missing key '__step' (F64). %s", path, mismatch); }
        if (entries.size() != expected) {
            for (const auto& kv : entries) {
                bool known = kv.first == "__step";
                for (uint64_t i = 0; !known && i < p->T; i++)
                    for (int k = 0; !known && k < (has_master ? 3 : 2); k++) known = kv.first == std::string(names[i]) + suffix[k];
                if (!known) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': load failed: unknown name '%s'. %s", path, kv.first.c_str(), mismatch); }
            }
        }
        {
            uint64_t need = 0;
            for (const auto& kv : entries) need = kv.second.end > need ? kv.second.end : need;
            if (fseek(f, 0, SEEK_END) != 0 || (uint64_t)ftell(f) < data0 + need) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': open failed: the data is shorter than the header says. %s", path, next); }
        }
        double step = 0.0;
        if (fseek(f, (long)(data0 + st_it->second.begin), SEEK_SET) != 0 || fread(&step, 8, 1, f) != 1 || !(step >= 0.0) || step != std::floor(step)) { fclose(f); return fail(OXZ_ERR_INVALID, "optimizer state file '%s': read of '__step' failed. %s", path, next); }

        std::vector<float> host;
        int32_t st = OXZ_OK;
        for (uint64_t i = 0; i < p->T && st == OXZ_OK; i++) {
            if (p->numel[i] == 0) continue;
            for (int k = 0; k < (has_master ? 3 : 2) && st == OXZ_OK; k++) {
                const Entry& en = entries[std::string(names[i]) + suffix[k]];
                host.resize(p->numel[i]);
                if (fseek(f, (long)(data0 + en.begin), SEEK_SET) != 0 || fread(host.data(), 4, host.size(), f) != host.size())
                    st = fail(OXZ_ERR_INVALID, "optimizer state file '%s': read of '%s%s' failed: truncated data. %s", path, names[i], suffix[k], next);
                else st = oxz_state_import(p, kinds[k], i, host.data());
            }
        }
        fclose(f);
        if (st == OXZ_OK) p->timestep = (uint64_t)step;
        return st;
    });
}

}  // extern "C"
