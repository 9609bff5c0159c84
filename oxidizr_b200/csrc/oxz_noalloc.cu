// oxz_grad_norm_static: the global gradient norm for callers that must not allocate.
//
// oxz_grad_norm keeps its per-cluster partial sums, the three reduced doubles and the result record in device
// memory that it obtains with cudaMalloc on its first call per device. Some hosts of this library cannot afford
// that: a trainer whose caching allocator already owns all of the device's memory (a late cudaMalloc fails or
// evicts its pool), a serving process with a fixed memory budget checked at start-up, or a step loop that must not
// hit the device-wide synchronisation that cudaMalloc and cudaFree imply. For them this file keeps the same
// scratch in one file-scope __device__ array that is part of the library image: every GPU that loads the library
// holds these few KiB until the process exits, and no call here allocates or frees anything, on the device or in
// pinned host memory.
#include <cmath>
#include <mutex>

#include "oxz_internal.h"

namespace {

constexpr uint32_t MAX_CLUSTERS = OXZ_STATIC_NORM_MAX_CLUSTERS;  // partial-sum slots the array holds
constexpr size_t PARTIALS_BYTES = size_t(MAX_CLUSTERS) * 3 * sizeof(double);
constexpr size_t ACC_OFFSET = PARTIALS_BYTES;                    // the reducer's four doubles
constexpr size_t SCALARS_OFFSET = ACC_OFFSET + 256;              // one oxz::DevScalars
constexpr size_t SCRATCH_BYTES = SCALARS_OFFSET + 256;
constexpr int MAX_DEVICES = 64;

// In host code this name is only a handle for the runtime, not an address a kernel can use: the device address is
// asked for once per device with cudaGetSymbolAddress (below) and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_norm_scratch[SCRATCH_BYTES];

struct DeviceSetup {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_norm_scratch on this device
    int resident_clusters = 0;         // clusters of 4 blocks the device holds at once
};

std::mutex g_mu;
DeviceSetup g_setup[MAX_DEVICES];

}  // namespace

extern "C" int32_t oxz_grad_norm_static(const void* device_grads, int32_t dtype, uint64_t n, double loss_scale,
                                        double max_grad_value, uint32_t clusters, void* stream, double* norm) {
    using namespace oxz;
    // like every other entry point: whatever C++ throws inside (the mutex, the error text) becomes a status
    return guarded("oxz_grad_norm_static", [&]() -> int32_t {
    if (!norm || (!device_grads && n)) return fail(OXZ_ERR_INVALID, "oxz_grad_norm_static: null argument");
    if (dtype != OXZ_F32 && dtype != OXZ_BF16 && dtype != OXZ_F16)
        return fail(OXZ_ERR_INVALID, "oxz_grad_norm_static: dtype %d is none of f32, bf16, f16", dtype);
    if ((uintptr_t)device_grads & 15) return fail(OXZ_ERR_INVALID, "oxz_grad_norm_static: the gradients are not 16-byte aligned");
    if (!std::isnan(max_grad_value) && !(std::isfinite(max_grad_value) && max_grad_value > 0.0))
        return fail(OXZ_ERR_INVALID, "trainer.max_grad_value is %g: it must be a finite positive number. Set a positive value, or remove the key to disable per-element clipping.", max_grad_value);
    if (clusters > MAX_CLUSTERS)
        return fail(OXZ_ERR_INVALID,
                    "oxz_grad_norm_static: %u clusters asked for, but the static scratch holds the partial sums of at "
                    "most %u. Ask for fewer (0 = as many as the device holds at once, capped at that maximum), or "
                    "use oxz_grad_norm, which sizes its scratch to the device",
                    clusters, MAX_CLUSTERS);
    int dev = 0;
    OXZ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(OXZ_ERR_UNSUPPORTED, "oxz_grad_norm_static: device ordinal %d is past %d", dev, MAX_DEVICES);
    DeviceSetup setup;
    {
        // Set-up happens in the first call on each device, with that device current: the symbol's device address
        // and the launch geometry are looked up once and kept. Make that first call outside any stream capture.
        std::lock_guard<std::mutex> lock(g_mu);
        DeviceSetup& d = g_setup[dev];
        if (!d.ready) {
            void* ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&ptr, g_norm_scratch);
            if (e != cudaSuccess || ptr == nullptr)
                return fail(OXZ_ERR_CUDA, "oxz_grad_norm_static: cudaGetSymbolAddress on device %d failed: %s", dev, cudaGetErrorString(e));
            LaunchGeom g;
            OXZ_TRY(query_geom(dev, &g));
            d.scratch = static_cast<unsigned char*>(ptr);
            d.resident_clusters = (int)norm_partial_slots(g);
            d.ready = true;
        }
        setup = d;
    }
    uint32_t use = clusters ? clusters : (uint32_t)setup.resident_clusters;
    if (use > MAX_CLUSTERS) use = MAX_CLUSTERS;
    if (use > (uint32_t)setup.resident_clusters) use = (uint32_t)setup.resident_clusters;  // one wave, always
    if (use == 0) use = 1;

    double* partials = reinterpret_cast<double*>(setup.scratch);
    double* acc = reinterpret_cast<double*>(setup.scratch + ACC_OFFSET);
    DevScalars* scalars = reinterpret_cast<DevScalars*>(setup.scratch + SCALARS_OFFSET);
    cudaStream_t s = (cudaStream_t)stream;
    const bool scaled = !std::isnan(loss_scale) && loss_scale != 0.0;
    const int clamp_on = std::isnan(max_grad_value) ? 0 : 1;
    // Nothing in the scratch has to start at zero: each stage overwrites exactly what the next one reads (every
    // cluster stores its slot, the reducer reads `use` slots and stores all four of its doubles, the last kernel stores the
    // whole record), so what an earlier call left behind is never read.
    OXZ_TRY(launch_sumsq_plain(s, (int)use * 4, device_grads, dtype, n, scaled ? (float)(1.0 / loss_scale) : 1.0f,
                               clamp_on ? (float)max_grad_value : 0.f, clamp_on, partials));
    OXZ_TRY(launch_reduce_partials(s, partials, use, acc, nullptr));
    FinalizeParams fp{};
    fp.max_grad_norm = 1.7976931348623157e308;  // a pure measurement: nothing is rescaled
    OXZ_TRY(launch_finalize(s, acc, fp, scalars));
    // The result goes straight into the caller's double; the runtime stages a copy to pageable memory itself.
    OXZ_CUDA(cudaMemcpyAsync(norm, &scalars->norm, sizeof(double), cudaMemcpyDeviceToHost, s));
    OXZ_CUDA(cudaStreamSynchronize(s));
    return OXZ_OK;
    });
}
