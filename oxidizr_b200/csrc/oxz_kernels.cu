// Hand-written sm_100a kernels of the data-parallel optimizer step.
//
// All of them are HBM- or NVLink-bound streaming kernels: no tensor cores, 128- and 256-bit coalesced accesses, grids sized in
// multiples of the SM count, one 8-element vector per lane and one 256-element tile per warp. A tile never
// straddles two tensors (tensor starts are tile-aligned), so the group scalars are warp-uniform.
//
//   k_sumsq        unscale + non-finite detection + sum of squares; warp shuffle, then a thread-block-cluster
//                  reduction through distributed shared memory, one partial per cluster.
//   k_pull_sumsq   the same fused with the gradient sum over ranks: every rank pulls its tiles from all peers'
//                  buffers over NVLink with plain 128-bit loads and adds them in f32 in rank order.
//   k_pull_bulk    the same pull with 1-D bulk asynchronous copies into shared memory (16-bit gradients, 2/4/8 ranks);
//                  chunks of tensors no rank has a gradient for are not fetched.
//   k_reduce_partials / k_finalize   partials -> norm, overflow, clip coefficients, all on the device.
//   k_gate / k_decide   the ranks' barriers and their one small sum through mailboxes in peer memory (ranks on
//                  distinct GPUs): bounded waits, sums in rank order, the decision fused with the exchange.
//   k_adamw        clip-scale + bias-corrected AdamW + decoupled decay by group + f32 master and narrow working
//                  weights; with peers it stores the working weights into every rank's buffer (the all-gather).
//   k_adamw_wide   the same on two tiles per warp with 256-bit stores of the 16-bit weights (two ranks).
//   k_adamw_staged the same with its inputs staged through shared memory (kept for the measured comparison).
//   k_sumsq_tensors   per-tensor sums of squares for the report after a skipped step.
//   k_flatten      per-tensor gradients -> flat buffer.
//
// The update uses explicit round-to-nearest intrinsics so that no multiply-add is contracted: every f32
// operation rounds once, and the result is bit-identical to a plain C restatement compiled without contraction.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "oxz_internal.h"

namespace cg = cooperative_groups;

namespace oxz {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int CLUSTER = 4;
constexpr uint32_t FLAG_INF = 1u, FLAG_NAN = 2u;

// ---------------------------------------------------------------- vector access

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }

// 8 consecutive elements of dtype DT starting at element index `e` (a multiple of 8) as f32, from a buffer the
// library allocated (256-byte aligned base, so an f32 vector is 32-byte aligned).
template <int DT>
__device__ __forceinline__ void load8(const void* base, uint64_t e, float (&x)[8]) {
    if constexpr (DT == OXZ_F32) {
        // one 256-bit access per lane (sm_100): a warp covers 1 KiB contiguously with a single instruction
        const float* p = static_cast<const float*>(base) + e;
        asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3]), "=f"(x[4]), "=f"(x[5]), "=f"(x[6]), "=f"(x[7])
                     : "l"(p));
    } else {
        uint4 r = ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + e));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if constexpr (DT == OXZ_BF16) {
                x[2 * i] = __uint_as_float(w[i] << 16);
                x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            } else {
                __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
                float2 f = __half22float2(h);
                x[2 * i] = f.x;
                x[2 * i + 1] = f.y;
            }
        }
    }
}

// The same for memory the caller owns, which is only promised to be 16-byte aligned: f32 goes as two 128-bit loads.
template <int DT>
__device__ __forceinline__ void load8_user(const void* base, uint64_t e, float (&x)[8]) {
    if constexpr (DT == OXZ_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + e);
        float4 a = ld_stream(p), b = ld_stream(p + 1);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else {
        load8<DT>(base, e, x);
    }
}

template <int DT>
__device__ __forceinline__ void store8(void* base, uint64_t e, const float (&x)[8]) {
    if constexpr (DT == OXZ_F32) {
        float* p = static_cast<float*>(base) + e;
        asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(x[0]), "f"(x[1]), "f"(x[2]),
                     "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7])
                     : "memory");
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if constexpr (DT == OXZ_BF16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        st_stream(reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + e), make_uint4(w[0], w[1], w[2], w[3]));
    }
}

__device__ __forceinline__ uint32_t flat_tile(const TileMap& m, uint32_t lt) {
    uint32_t b = lt / m.tiles_per_shard;
    uint32_t within = lt - b * m.tiles_per_shard;
    uint32_t shard = (b == m.n_buckets - 1) ? m.last_shard_tiles : m.tiles_per_shard;
    return b * m.tiles_per_bucket + m.rank * shard + within;
}

__device__ __forceinline__ bool finite_f32(float x) { return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u; }

// ---------------------------------------------------------------- sum of squares

struct NormAcc {
    double sum = 0.0;
    uint32_t flags = 0;
};

// Adds the squares of 8 gradients (already widened to f32) to `a`.
// The overflow decision must not depend on the summation order: a step overflows exactly when some element's
// f32 square is not finite. The fast path sums the 8 squares in f32; only when that sum is not finite does the
// slow path look at each square, so a partial sum that overflows by itself is never mistaken for an overflow.
__device__ __forceinline__ void acc8(const float (&g)[8], float inv_scale, float clamp_hi, bool clamp_on, NormAcc& a) {
    float x[8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        x[i] = __fmul_rn(g[i], inv_scale);
        s = fmaf(x[i], x[i], s);
    }
    if (finite_f32(s)) {
        if (clamp_on) {
            float sc = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float c = fminf(fmaxf(x[i], -clamp_hi), clamp_hi);
                sc = fmaf(c, c, sc);
            }
            a.sum += static_cast<double>(sc);
        } else {
            a.sum += static_cast<double>(s);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float q = __fmul_rn(x[i], x[i]);
        if (!finite_f32(q)) {
            a.flags |= (q != q) ? FLAG_NAN : FLAG_INF;
        } else {
            float c = clamp_on ? fminf(fmaxf(x[i], -clamp_hi), clamp_hi) : x[i];
            a.sum += static_cast<double>(__fmul_rn(c, c));
        }
    }
}

// Warp shuffle -> shared memory -> distributed shared memory of the cluster's first block -> one partial per cluster.
// partials[cluster][0] = sum, [1] = 1 if an infinity was seen, [2] = 1 if a NaN was seen. No atomics: the order
// of every addition is fixed, so the norm is reproducible from run to run.
__device__ __forceinline__ void cluster_reduce_store(NormAcc a, double* partials) {
    __shared__ double s_sum[WARPS];
    __shared__ uint32_t s_flag[WARPS];
    __shared__ double c_sum[CLUSTER];
    __shared__ uint32_t c_flag[CLUSTER];
    cg::cluster_group cluster = cg::this_cluster();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a.sum += __shfl_down_sync(0xffffffffu, a.sum, o);
        a.flags |= __shfl_down_sync(0xffffffffu, a.flags, o);
    }
    if (lane == 0) {
        s_sum[warp] = a.sum;
        s_flag[warp] = a.flags;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        uint32_t f = 0;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            t += s_sum[w];
            f |= s_flag[w];
        }
        const unsigned r = cluster.block_rank();
        double* dst_sum = cluster.map_shared_rank(c_sum, 0);
        uint32_t* dst_flag = cluster.map_shared_rank(c_flag, 0);
        dst_sum[r] = t;
        dst_flag[r] = f;
    }
    cluster.sync();
    if (cluster.block_rank() == 0 && threadIdx.x == 0) {
        double t = 0.0;
        uint32_t f = 0;
#pragma unroll
        for (int r = 0; r < CLUSTER; r++) {
            t += c_sum[r];
            f |= c_flag[r];
        }
        const uint32_t cid = blockIdx.x / CLUSTER;
        partials[3 * cid + 0] = t;
        partials[3 * cid + 1] = (f & FLAG_INF) ? 1.0 : 0.0;
        partials[3 * cid + 2] = (f & FLAG_NAN) ? 1.0 : 0.0;
    }
}

// CHECK = false is the common step: every tensor has a gradient. Padding holds zeros, so no tile needs its
// metadata and the pass is a pure stream. CHECK = true looks up each tile's tensor to leave absent ones out.
// All loads of an iteration are issued before anything depends on them.
template <int DT, int ILP, bool CHECK>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(THREADS)
    k_sumsq(const void* __restrict__ grads, TileMap map, const uint32_t* __restrict__ tile_meta,
            const uint8_t* __restrict__ present, float inv_scale, float clamp_hi, int clamp_on,
            double* __restrict__ partials) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    NormAcc a;
    const uint32_t per_iter = gridDim.x * WARPS * ILP;
    for (uint32_t base = map.first_tile + (blockIdx.x * WARPS + warp) * ILP; base < map.n_local_tiles; base += per_iter) {
        float g[ILP][8];
        bool on[ILP];
        uint32_t meta[ILP];
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            const uint32_t lt = base + j;
            on[j] = lt < map.n_local_tiles;
            if (on[j]) {
                load8<DT>(grads, static_cast<uint64_t>(lt) * TILE + lane * 8, g[j]);
                if constexpr (CHECK) meta[j] = tile_meta[flat_tile(map, lt)];
            }
        }
        if constexpr (CHECK) {
#pragma unroll
            for (int j = 0; j < ILP; j++)
                if (on[j]) on[j] = meta[j] != PAD_TILE && present[meta[j] & 0xffffffu];
        }
#pragma unroll
        for (int j = 0; j < ILP; j++)
            if (on[j]) acc8(g[j], inv_scale, clamp_hi, clamp_on != 0, a);
    }
    cluster_reduce_store(a, partials);
}

// Every tensor present, 16-bit gradients: the shard is one contiguous stream, read 256 bits per lane (16 elements),
// VEC such loads in flight per thread. Library-owned memory, so 32-byte alignment holds.
// CHECK: some tensor has no gradient this step; every vector (16 lanes share a tile) looks its tile's tensor up and
// leaves the vector out when that tensor is absent or the tile is padding. The lookups are issued with the loads.
template <int DT, int VEC, bool CHECK>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(THREADS)
    k_sumsq_stream16(const uint16_t* __restrict__ grads, uint64_t first, uint64_t end, float inv_scale, float clamp_hi,
                     int clamp_on, double* __restrict__ partials, TileMap map, const uint32_t* __restrict__ tile_meta,
                     const uint8_t* __restrict__ present) {
    static_assert(DT == OXZ_BF16 || DT == OXZ_F16, "16-bit gradients only");
    NormAcc a;
    const uint64_t nvec = (end - first) / 16;  // the range is a whole number of 256-element tiles
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * THREADS;
    const uint16_t* base = grads + first;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * THREADS + threadIdx.x; i < nvec; i += stride * VEC) {
        uint32_t w[VEC][8];
        bool on[VEC];
        uint32_t meta[VEC];
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            const uint64_t v = i + static_cast<uint64_t>(j) * stride;
            on[j] = v < nvec;
            if (on[j]) {
                asm volatile("ld.global.cs.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                             : "=r"(w[j][0]), "=r"(w[j][1]), "=r"(w[j][2]), "=r"(w[j][3]), "=r"(w[j][4]), "=r"(w[j][5]),
                               "=r"(w[j][6]), "=r"(w[j][7])
                             : "l"(base + v * 16));
                if constexpr (CHECK) meta[j] = __ldg(&tile_meta[flat_tile(map, static_cast<uint32_t>((first + v * 16) / TILE))]);
            }
        }
        if constexpr (CHECK) {
#pragma unroll
            for (int j = 0; j < VEC; j++)
                if (on[j]) on[j] = meta[j] != PAD_TILE && __ldg(&present[meta[j] & 0xffffffu]) != 0;
        }
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            if (!on[j]) continue;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float x[8];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t u = w[j][4 * h + q];
                    if constexpr (DT == OXZ_BF16) {
                        x[2 * q] = __uint_as_float(u << 16);
                        x[2 * q + 1] = __uint_as_float(u & 0xffff0000u);
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
                        x[2 * q] = f.x;
                        x[2 * q + 1] = f.y;
                    }
                }
                acc8(x, inv_scale, clamp_hi, clamp_on != 0, a);
            }
        }
    }
    cluster_reduce_store(a, partials);
}

// The standalone measurement over a plain array: n elements, any n; the tail is read element by element.
template <int DT>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(THREADS)
    k_sumsq_plain(const void* __restrict__ grads, uint64_t n, float inv_scale, float clamp_hi, int clamp_on,
                  double* __restrict__ partials) {
    NormAcc a;
    const uint64_t nvec = n / 8;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * THREADS;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * THREADS + threadIdx.x; i < nvec; i += stride) {
        float g[8];
        load8_user<DT>(grads, i * 8, g);
        acc8(g, inv_scale, clamp_hi, clamp_on != 0, a);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && (n & 7)) {
        float g[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint64_t e = nvec * 8 + k;
            float v = 0.f;
            if (e < n) {
                if constexpr (DT == OXZ_F32) v = static_cast<const float*>(grads)[e];
                else if constexpr (DT == OXZ_BF16) v = __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t*>(grads)[e]) << 16);
                else v = __half2float(static_cast<const __half*>(grads)[e]);
            }
            g[k] = v;
        }
        acc8(g, inv_scale, clamp_hi, clamp_on != 0, a);
    }
    cluster_reduce_store(a, partials);
}

// Per-tensor sums of squares over this rank's tiles: out[3 * t + {0, 1, 2}] += {sum, infinities seen, NaNs seen} of
// tensor t. A warp walks its tiles in order and keeps a running sum while the tensor stays the same, so the atomic
// adds number a few per warp and tensor, not one per tile. Off the step's path: a diagnostic after a skipped step.
template <int DT>
__global__ void __launch_bounds__(THREADS)
    k_sumsq_tensors(const void* __restrict__ grads, TileMap map, const uint32_t* __restrict__ tile_meta,
                    const uint8_t* __restrict__ present, float inv_scale, float clamp_hi, int clamp_on,
                    double* __restrict__ out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per_iter = gridDim.x * WARPS;
    uint32_t cur = PAD_TILE;
    NormAcc a;
    auto flush = [&]() {
        if (cur == PAD_TILE) return;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a.sum += __shfl_down_sync(0xffffffffu, a.sum, o);
            a.flags |= __shfl_down_sync(0xffffffffu, a.flags, o);
        }
        if (lane == 0) {
            atomicAdd(&out[3 * static_cast<size_t>(cur) + 0], a.sum);
            if (a.flags & FLAG_INF) atomicAdd(&out[3 * static_cast<size_t>(cur) + 1], 1.0);
            if (a.flags & FLAG_NAN) atomicAdd(&out[3 * static_cast<size_t>(cur) + 2], 1.0);
        }
        a = NormAcc();
    };
    for (uint32_t lt = map.first_tile + blockIdx.x * WARPS + warp; lt < map.n_local_tiles; lt += per_iter) {
        const uint32_t meta = tile_meta[flat_tile(map, lt)];
        if (meta == PAD_TILE) continue;
        const uint32_t t = meta & 0xffffffu;
        if (!present[t]) continue;
        if (t != cur) {
            flush();
            cur = t;
        }
        float g[8];
        load8<DT>(grads, static_cast<uint64_t>(lt) * TILE + lane * 8, g);
        acc8(g, inv_scale, clamp_hi, clamp_on != 0, a);
    }
    flush();
}

// A vector of 8 elements as it sits in memory: 16-bit types stay packed (4 registers) until they are needed, so a
// lane can keep eight remote loads in flight without eight times the registers.
template <int DT>
struct RawVec {
    uint4 v;
};
template <>
struct RawVec<OXZ_F32> {
    float x[8];
};

template <int DT>
__device__ __forceinline__ void load_raw(const void* base, uint64_t e, RawVec<DT>& r) {
    if constexpr (DT == OXZ_F32) load8<OXZ_F32>(base, e, r.x);
    else r.v = ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + e));
}

template <int DT>
__device__ __forceinline__ void widen_raw(const RawVec<DT>& r, float (&x)[8]) {
    if constexpr (DT == OXZ_F32) {
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = r.x[i];
    } else {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if constexpr (DT == OXZ_BF16) {
                x[2 * i] = __uint_as_float(w[i] << 16);
                x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                x[2 * i] = f.x;
                x[2 * i + 1] = f.y;
            }
        }
    }
}

// WORLD > 0: the rank count is known at compile time (2, 4 or 8). Every lane then issues all of an iteration's
// loads at once - WORLD sources x ILP tiles = 8 vectors of 16 bytes - which is what it takes to cover NVLink's
// latency at its bandwidth; the additions still run in rank order. WORLD == 0 is the general form.
template <int DT, bool CHECK, int WORLD>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(THREADS)
    k_pull_sumsq(PeerTable peers, int world, int staged, TileMap map, const uint32_t* __restrict__ tile_meta,
                 const uint8_t* __restrict__ present, float inv_scale, float clamp_hi, int clamp_on,
                 float* __restrict__ reduced, double* __restrict__ partials) {
    // staged != 0: the other ranks' gradients were copied into local staging buffers laid out like this rank's
    // state (indexed by local element); this rank's own gradients are read in place (indexed by flat element).
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    NormAcc a;
    if constexpr (WORLD > 0) {
        constexpr int ILP = 8 / WORLD;
        const uint32_t per_iter = gridDim.x * WARPS * ILP;
        for (uint32_t base = map.first_tile + (blockIdx.x * WARPS + warp) * ILP; base < map.n_local_tiles; base += per_iter) {
            RawVec<DT> raw[ILP][WORLD];
            bool on[ILP];
            uint32_t meta[ILP];
#pragma unroll
            for (int j = 0; j < ILP; j++) {
                const uint32_t lt = base + j;
                on[j] = lt < map.n_local_tiles;
                if (on[j]) {
                    const uint32_t ft = flat_tile(map, lt);
                    const uint64_t fe = static_cast<uint64_t>(ft) * TILE + lane * 8;
                    const uint64_t le = static_cast<uint64_t>(lt) * TILE + lane * 8;
#pragma unroll
                    for (int r = 0; r < WORLD; r++)
                        load_raw<DT>(peers.grads[r], (staged && r != static_cast<int>(map.rank)) ? le : fe, raw[j][r]);
                    if constexpr (CHECK) meta[j] = tile_meta[ft];
                }
            }
#pragma unroll
            for (int j = 0; j < ILP; j++) {
                if (!on[j]) continue;
                if constexpr (CHECK) {
                    if (meta[j] == PAD_TILE || !present[meta[j] & 0xffffffu]) continue;
                }
                float s[8];
                widen_raw<DT>(raw[j][0], s);
#pragma unroll
                for (int r = 1; r < WORLD; r++) {
                    float p[8];
                    widen_raw<DT>(raw[j][r], p);
#pragma unroll
                    for (int i = 0; i < 8; i++) s[i] = __fadd_rn(s[i], p[i]);
                }
                store8<OXZ_F32>(reduced, static_cast<uint64_t>(base + j) * TILE + lane * 8, s);
                acc8(s, inv_scale, clamp_hi, clamp_on != 0, a);
            }
        }
    } else {
        const uint32_t per_iter = gridDim.x * WARPS;
        for (uint32_t lt = map.first_tile + blockIdx.x * WARPS + warp; lt < map.n_local_tiles; lt += per_iter) {
            const uint32_t ft = flat_tile(map, lt);
            uint32_t meta = 0;
            if constexpr (CHECK) meta = tile_meta[ft];
            const uint64_t fe = static_cast<uint64_t>(ft) * TILE + lane * 8;
            const uint64_t le = static_cast<uint64_t>(lt) * TILE + lane * 8;
            const int me = static_cast<int>(map.rank);
            float s[8];
            load8<DT>(peers.grads[0], (staged && me != 0) ? le : fe, s);
            int r = 1;
            for (; r + 1 < world; r += 2) {
                float p0[8], p1[8];
                load8<DT>(peers.grads[r], (staged && r != me) ? le : fe, p0);
                load8<DT>(peers.grads[r + 1], (staged && r + 1 != me) ? le : fe, p1);
#pragma unroll
                for (int i = 0; i < 8; i++) s[i] = __fadd_rn(__fadd_rn(s[i], p0[i]), p1[i]);
            }
            for (; r < world; r++) {
                float p0[8];
                load8<DT>(peers.grads[r], (staged && r != me) ? le : fe, p0);
#pragma unroll
                for (int i = 0; i < 8; i++) s[i] = __fadd_rn(s[i], p0[i]);
            }
            if constexpr (CHECK) {
                if (meta == PAD_TILE || !present[meta & 0xffffffu]) continue;
            }
            store8<OXZ_F32>(reduced, static_cast<uint64_t>(lt) * TILE + lane * 8, s);
            acc8(s, inv_scale, clamp_hi, clamp_on != 0, a);
        }
    }
    cluster_reduce_store(a, partials);
}

// ---------------------------------------------------------------- pull-reduce with bulk asynchronous copies
//
// The same work as k_pull_sumsq for the common shape (16-bit gradients, 2, 4 or 8 ranks), with
// the peers' tiles brought into shared memory by 1-D bulk asynchronous copies (cp.async.bulk + mbarrier) instead of
// per-lane loads: one elected thread issues WORLD copies of 4 KiB (8 tiles) per stage, STAGES stages deep, so the
// NVLink requests are large and independent of the warps' progress. Measured on two B200 with both directions
// loaded: 669 GB/s per direction for bulk reads against 635 GB/s for 128-bit loads. No load is shared across the cluster:
// every block fetches what it needs itself. Every wait on an mbarrier is bounded; when a bound runs out the block
// records it in scalars->wait_expired, waits once more (bounded) for its copies in flight, and returns.
constexpr int BULK_TILES = 8;                       // tiles per chunk: one per warp
constexpr uint32_t BULK_BYTES = BULK_TILES * TILE * 2;  // 4 KiB per source and chunk
constexpr uint32_t BULK_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t spins = 0; spins < limit; spins++) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

template <int DT, int WORLD, int STAGES>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(THREADS)
    k_pull_bulk(PeerTable peers, TileMap map, const uint32_t* __restrict__ tile_meta, const uint8_t* __restrict__ present,
                int check, float inv_scale, float clamp_hi, int clamp_on, float* __restrict__ reduced,
                double* __restrict__ partials, DevScalars* __restrict__ scalars, uint32_t wait_limit) {
    static_assert(DT == OXZ_BF16 || DT == OXZ_F16, "16-bit gradients only");
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    __shared__ __align__(8) uint64_t bar[STAGES];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t STAGE_BYTES = BULK_BYTES * WORLD;
    const uint32_t n_chunks = (map.n_local_tiles - map.first_tile) / BULK_TILES;
    NormAcc a;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bar[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](uint32_t chunk, int stage) {  // one thread: expect the bytes, then one copy per rank
        const uint32_t lt0 = map.first_tile + chunk * BULK_TILES;
        const uint64_t byte0 = static_cast<uint64_t>(flat_tile(map, lt0)) * TILE * 2;
        const uint32_t b = smem_addr(&bar[stage]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(STAGE_BYTES) : "memory");
#pragma unroll
        for (int r = 0; r < WORLD; r++)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_addr(bulk_smem + stage * STAGE_BYTES + r * BULK_BYTES)),
                           "l"(static_cast<const unsigned char*>(peers.grads[r]) + byte0), "r"(BULK_BYTES), "r"(b) : "memory");
    };
    // With absent tensors (check): a chunk none of whose tiles takes part is not fetched at all - an expert no rank
    // routed to is millions of elements that need not cross NVLink. Its first and last tile decide: both left out and
    // of one tensor (or both padding) means every tile between them is too; anything else is fetched and sorted out
    // tile by tile below. Every thread evaluates it alike, so the block agrees without talking.
    auto chunk_live = [&](uint32_t chunk) -> bool {
        if (!check) return true;
        const uint32_t ft0 = flat_tile(map, map.first_tile + chunk * BULK_TILES);
        const uint32_t m0 = __ldg(&tile_meta[ft0]), m7 = __ldg(&tile_meta[ft0 + BULK_TILES - 1]);
        const bool out0 = m0 == PAD_TILE || !__ldg(&present[m0 & 0xffffffu]);
        const bool out7 = m7 == PAD_TILE || !__ldg(&present[m7 & 0xffffffu]);
        return !(out0 && out7 && m0 == m7);
    };
    // Every thread keeps the same books: which stages have copies in flight, and the phase each stage completes next.
    uint32_t pending = 0, phase = 0;
    for (int s = 0; s < STAGES; s++) {
        const uint32_t c = blockIdx.x + static_cast<uint32_t>(s) * gridDim.x;
        if (c < n_chunks && chunk_live(c)) {
            if (threadIdx.x == 0) issue(c, s);
            pending |= 1u << s;
        }
    }
    int stage = 0;
    bool ok = true;
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        if (!(pending & (1u << stage))) {
            // nothing was fetched for this chunk: nothing to sum; the stage takes the chunk STAGES rounds ahead
            const uint32_t ahead = c + static_cast<uint32_t>(STAGES) * gridDim.x;
            if (ahead < n_chunks && chunk_live(ahead)) {
                if (threadIdx.x == 0) issue(ahead, stage);
                pending |= 1u << stage;
            }
            if (++stage == STAGES) stage = 0;
            continue;
        }
        // wait_limit is BULK_SPIN_LIMIT in production; a test lowers it to see the run-out path without any fault
        // the verdict must be the block's, not the thread's: a thread that saw the copies land on its last poll must
        // not go on to a barrier its neighbours never reach
        const int landed = mbar_wait_bounded(smem_addr(&bar[stage]), (phase >> stage) & 1u, wait_limit) ? 1 : 0;
        if (!__syncthreads_and(landed)) {
            ok = false;
            break;
        }
        pending &= ~(1u << stage);
        phase ^= 1u << stage;
        const unsigned char* st = bulk_smem + stage * STAGE_BYTES + warp * (TILE * 2) + lane * 16;
        float s8[8];
        {
            RawVec<DT> v;
            v.v = *reinterpret_cast<const uint4*>(st);
            widen_raw<DT>(v, s8);
        }
#pragma unroll
        for (int r = 1; r < WORLD; r++) {
            RawVec<DT> v;
            v.v = *reinterpret_cast<const uint4*>(st + r * BULK_BYTES);
            float p8[8];
            widen_raw<DT>(v, p8);
#pragma unroll
            for (int i = 0; i < 8; i++) s8[i] = __fadd_rn(s8[i], p8[i]);
        }
        const uint32_t lt = map.first_tile + c * BULK_TILES + warp;
        bool keep = true;
        if (check) {  // some tensor has no gradient this step: its tiles, and padding, stay out of the sum and the norm
            const uint32_t meta = tile_meta[flat_tile(map, lt)];
            keep = meta != PAD_TILE && present[meta & 0xffffffu];
        }
        if (keep) {
            store8<OXZ_F32>(reduced, static_cast<uint64_t>(lt) * TILE + lane * 8, s8);
            acc8(s8, inv_scale, clamp_hi, clamp_on != 0, a);
        }
        __syncthreads();  // every warp has read this stage: it may be refilled
        const uint32_t nc = c + static_cast<uint32_t>(STAGES) * gridDim.x;
        if (nc < n_chunks && chunk_live(nc)) {
            if (threadIdx.x == 0) issue(nc, stage);
            pending |= 1u << stage;
        }
        if (++stage == STAGES) stage = 0;
    }
    if (!ok) {
        // A wait ran out: say so, then give the copies still in flight into this block's shared memory one more
        // bounded chance (the full limit) to land before the block ends, stage by stage. The partial sums of this
        // block are incomplete; the host reports the step as failed.
        if (threadIdx.x == 0) atomicExch(&scalars->wait_expired, 1);
        for (int s = 0; s < STAGES; s++)
            if (pending & (1u << s)) mbar_wait_bounded(smem_addr(&bar[s]), (phase >> s) & 1u, BULK_SPIN_LIMIT);
        // This block's tiles were not summed. Poison the norm (a NaN seen), so that after the all-reduce every rank
        // takes the step for an overflow and leaves its state untouched; this rank also reports the time-out.
        a.flags |= FLAG_NAN;
    }
    // the tiles past the last whole chunk (fewer than BULK_TILES, at the end of the last bucket's shard): plain loads
    const uint32_t tail0 = map.first_tile + n_chunks * BULK_TILES;
    if (blockIdx.x == gridDim.x - 1 && tail0 + warp < map.n_local_tiles) {
        const uint32_t lt = tail0 + warp;
        const uint32_t ft = flat_tile(map, lt);
        const uint64_t fe = static_cast<uint64_t>(ft) * TILE + lane * 8;
        bool keep = true;
        if (check) {
            const uint32_t meta = tile_meta[ft];
            keep = meta != PAD_TILE && present[meta & 0xffffffu];
        }
        float s8[8];
        load8<DT>(peers.grads[0], fe, s8);
#pragma unroll
        for (int r = 1; r < WORLD; r++) {
            float p8[8];
            load8<DT>(peers.grads[r], fe, p8);
#pragma unroll
            for (int i = 0; i < 8; i++) s8[i] = __fadd_rn(s8[i], p8[i]);
        }
        if (keep) {
            store8<OXZ_F32>(reduced, static_cast<uint64_t>(lt) * TILE + lane * 8, s8);
            acc8(s8, inv_scale, clamp_hi, clamp_on != 0, a);
        }
    }
    cluster_reduce_store(a, partials);
}

// Adds the per-cluster partials in index order; the block's threads leave {sum, inf, NaN} in t_out[0..3) (shared).
__device__ __forceinline__ void block_sum_partials(const double* __restrict__ partials, uint32_t slots, double (&sh)[3][THREADS],
                                                   double (&t_out)[3]) {
    double t[3] = {0.0, 0.0, 0.0};
    // contiguous chunks per thread keep the order fixed
    const uint32_t per = (slots + THREADS - 1) / THREADS;
    const uint32_t lo = threadIdx.x * per, hi = min(slots, lo + per);
    for (uint32_t i = lo; i < hi; i++)
        for (int k = 0; k < 3; k++) t[k] += partials[3 * i + k];
    for (int k = 0; k < 3; k++) sh[k][threadIdx.x] = t[k];
    __syncthreads();
    if (threadIdx.x < 3) {
        double r = 0.0;
        for (int i = 0; i < THREADS; i++) r += sh[threadIdx.x][i];
        t_out[threadIdx.x] = r;
    }
    __syncthreads();
}

// One block. acc[ACC_EXPIRED] tells the other ranks (it rides on the same all-reduce) that a bounded wait of this
// rank's pull ran out, so that every rank reports the step failed and none takes it for an overflow.
__global__ void __launch_bounds__(THREADS) k_reduce_partials(const double* __restrict__ partials, uint32_t slots,
                                                             double* __restrict__ acc, const DevScalars* __restrict__ scalars) {
    __shared__ double sh[3][THREADS];
    __shared__ double t[3];
    block_sum_partials(partials, slots, sh, t);
    if (threadIdx.x < 3) acc[threadIdx.x] = t[threadIdx.x];
    if (threadIdx.x == 3) acc[ACC_EXPIRED] = (scalars != nullptr && scalars->wait_expired) ? 1.0 : 0.0;
}

// acc = {sum of squares, infinities seen, NaNs seen, waits run out} summed over every rank.
// norm, the overflow decision and the clip coefficients follow src/grad_clip.rs:36-56 and src/trainer.rs:619-645.
__device__ __forceinline__ void finalize_scalars(const double* acc, const FinalizeParams& fp, DevScalars* out) {
    const double sum = acc[0];
    double norm;
    if (acc[2] > 0.0) norm = __longlong_as_double(0x7ff8000000000000ll);
    else if (acc[1] > 0.0) norm = __longlong_as_double(0x7ff0000000000000ll);
    else norm = sqrt(sum);
    const bool overflow = !isfinite(norm);
    float c1 = 1.f, c2 = 1.f;
    if (!overflow && norm > fp.max_grad_norm) c1 = static_cast<float>(fp.max_grad_norm / (norm + fp.clip_eps));
    if (!overflow && !fp.spike_skip && fp.has_target) {
        const double eff = norm < fp.max_grad_norm ? norm : fp.max_grad_norm;
        if (eff > fp.target_grad_norm && eff > 1e-8) {
            // The reference calls the norm clip a second time with the target as its limit (src/trainer.rs:635-645):
            // it measures the gradients again, as the first clip left them. Each of them is then fl(g * c1), so that
            // second norm is c1 * norm within 2^-24 relative (exactly norm when the first clip did not fire), and no
            // second pass over the gradients is needed. It is a little under max_grad_norm, not max_grad_norm itself.
            const double again = static_cast<double>(c1) * norm;
            if (again > fp.target_grad_norm) c2 = static_cast<float>(fp.target_grad_norm / (again + fp.clip_eps));
        }
    }
    // a wait that ran out anywhere: some rank's sum is incomplete, the step must change nothing on any rank
    // (this rank's own flag is part of that sum: nothing of `out` is read here)
    const bool expired = acc[ACC_EXPIRED] > 0.0;
    out->norm = norm;
    out->sumsq = sum;
    out->c1 = c1;
    out->c2 = c2;
    out->overflow = overflow ? 1 : 0;
    out->skip = (overflow || fp.spike_skip || expired) ? 1 : 0;
    if (expired) atomicMax(&out->wait_expired, 1);
}

__global__ void k_finalize(const double* __restrict__ acc, FinalizeParams fp, DevScalars* __restrict__ out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    finalize_scalars(acc, fp, out);
}

// ---------------------------------------------------------------- exchanges between ranks through peer memory
//
// Ranks on distinct GPUs, one kernel per rank and exchange, each in its own stream. Nothing here may run with two
// ranks on one GPU: their kernels would wait on one another with no promise of running at the same time.

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Waits until `slot` carries exchange number `seq` or later. 0: it does; 1: limit_ns went by; 2: the host raised the
// abort flag (oxz_comm_abort). Never unbounded.
__device__ __forceinline__ int mail_wait(const MailSlot* slot, unsigned long long seq, unsigned long long limit_ns,
                                         const int32_t* abort_flag) {
    const unsigned long long t0 = global_ns();
    // the clock decides; the poll count is a second bound should the clock ever stand still (a poll with its share of
    // the sleeps takes well over 10 ns)
    const unsigned long long max_polls = limit_ns / 10ull + 4096ull;
    for (unsigned long long polls = 0; polls < max_polls; polls++) {
        if (ld_acquire_sys(&slot->seq) >= seq) return 0;
        if ((polls & 63ull) == 63ull) {
            if (abort_flag != nullptr && *reinterpret_cast<const volatile int32_t*>(abort_flag) != 0) return 2;
            if (global_ns() - t0 > limit_ns) return 1;
            __nanosleep(200);
        }
    }
    return 1;
}

// Posts this rank's arrival at exchange `seq` in every rank's mailbox (its own included) and waits for every rank's.
// The payload bytes were written by the block before; the fence makes them, and whatever this rank's earlier kernels
// stored into peer memory, visible before the number that announces them. Returns the block's verdict: 0 = every
// rank arrived, else the worst wait result. Thread r serves rank r.
__device__ __forceinline__ int mail_arrive_and_wait(const MailPeers& mail, int world, int rank, unsigned long long seq,
                                                    unsigned long long limit_ns, const int32_t* abort_flag) {
    __shared__ int verdict;
    const int par = static_cast<int>(seq & 1ull);
    if (threadIdx.x == 0) verdict = 0;
    __threadfence_system();
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {
        st_release_sys(&mail.box[threadIdx.x]->slot[par][rank].seq, seq);
        const int w = mail_wait(&mail.box[rank]->slot[par][threadIdx.x], seq, limit_ns, abort_flag);
        if (w) atomicMax(&verdict, w);
    }
    __syncthreads();
    return verdict;
}

__global__ void __launch_bounds__(THREADS) k_gate(MailPeers mail, int world, int rank, unsigned long long seq,
                                                  const uint8_t* __restrict__ present_in, uint8_t* __restrict__ present_out,
                                                  uint32_t T, DevScalars* __restrict__ scalars, unsigned long long limit_ns,
                                                  const int32_t* __restrict__ abort_flag) {
    const int par = static_cast<int>(seq & 1ull);
    for (int r = 0; r < world; r++) {
        unsigned char* dst = mail.box[r]->slot[par][rank].payload;
        for (uint32_t i = threadIdx.x; i < T; i += THREADS) dst[i] = present_in[i];
    }
    const int v = mail_arrive_and_wait(mail, world, rank, seq, limit_ns, abort_flag);
    if (v) {
        // some rank never arrived: record it; the kernels after this one still run on whatever the peers hold, the
        // decision kernel turns the step into a reported failure that changes nothing
        if (threadIdx.x == 0) atomicMax(&scalars->wait_expired, v);
        return;
    }
    const MailBox* mine = mail.box[rank];
    for (uint32_t i = threadIdx.x; i < T; i += THREADS) {
        unsigned char any = 0;
        for (int r = 0; r < world; r++) any |= mine->slot[par][r].payload[i];
        present_out[i] = any ? 1 : 0;
    }
}

__global__ void __launch_bounds__(THREADS) k_decide(MailPeers mail, int world, int rank, unsigned long long seq,
                                                    const double* __restrict__ partials, uint32_t slots, double* __restrict__ acc,
                                                    uint32_t n_extras, int sum_norm, FinalizeParams fp, DevScalars* __restrict__ scalars,
                                                    unsigned long long limit_ns, const int32_t* __restrict__ abort_flag) {
    __shared__ double sh[3][THREADS];
    __shared__ double t[3];
    block_sum_partials(partials, slots, sh, t);
    const int par = static_cast<int>(seq & 1ull);
    const uint32_t n = ACC_EXTRAS + n_extras;
    // this rank's contribution: its three norm terms, whether one of its waits ran out, its extras (already in acc)
    if (threadIdx.x < n) {
        double v;
        if (threadIdx.x < 3) v = t[threadIdx.x];
        else if (threadIdx.x == ACC_EXPIRED) v = scalars->wait_expired ? 1.0 : 0.0;
        else v = acc[threadIdx.x];
        for (int r = 0; r < world; r++) reinterpret_cast<double*>(mail.box[r]->slot[par][rank].payload)[threadIdx.x] = v;
    }
    const int verdict = mail_arrive_and_wait(mail, world, rank, seq, limit_ns, abort_flag);
    if (verdict) {
        if (threadIdx.x == 0) {
            atomicMax(&scalars->wait_expired, verdict);
            scalars->norm = __longlong_as_double(0x7ff8000000000000ll);
            scalars->c1 = scalars->c2 = 1.f;
            scalars->overflow = 0;
            scalars->skip = 1;
        }
        return;
    }
    // every rank adds the contributions in rank order: the same bits everywhere
    if (threadIdx.x < n) {
        const MailBox* mine = mail.box[rank];
        double total = 0.0;
        for (int r = 0; r < world; r++) total += reinterpret_cast<const double*>(mine->slot[par][r].payload)[threadIdx.x];
        acc[threadIdx.x] = (threadIdx.x < 3 && !sum_norm) ? t[threadIdx.x] : total;
    }
    __syncthreads();
    if (threadIdx.x == 0) finalize_scalars(acc, fp, scalars);
}

// ---------------------------------------------------------------- AdamW

__device__ __forceinline__ void adam1(float& p, float& m, float& v, float g, const AdamParams& k, float step,
                                      float decay) {
    if (!k.decay_after) p = __fmul_rn(p, decay);
    m = __fadd_rn(__fmul_rn(k.beta1, m), __fmul_rn(k.one_minus_beta1, g));
    const float gg = __fmul_rn(g, g);
    v = __fadd_rn(__fmul_rn(k.beta2, v), __fmul_rn(k.one_minus_beta2, gg));
    const float root = __fsqrt_rn(v);
    const float denom = k.eps_mode == 0 ? __fadd_rn(__fdiv_rn(root, k.bias2_sqrt), k.eps) : __fadd_rn(root, k.eps);
    const float q = __fdiv_rn(m, denom);
    p = __fsub_rn(p, __fmul_rn(step, q));
    if (k.decay_after) p = __fmul_rn(p, decay);
}

template <int PDT>
__device__ __forceinline__ void pack8(const float (&x)[8], uint32_t (&w)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if constexpr (PDT == OXZ_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
}

template <int GDT, int PDT, int ILP, int MINB, bool CHECK>
__global__ void __launch_bounds__(THREADS, MINB)
    k_adamw(const void* __restrict__ gsrc, float* __restrict__ master, float* __restrict__ exp_avg,
            float* __restrict__ exp_avg_sq, PeerTable peers, int n_work, TileMap map,
            const uint32_t* __restrict__ tile_meta, const uint8_t* __restrict__ present,
            const DevScalars* __restrict__ scalars, AdamParams k) {
    // The skip decision was taken on the device by the norm pass: an overflow or a spike veto changes nothing.
    if (scalars->skip) return;
    const float c1 = scalars->c1, c2 = scalars->c2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per_iter = gridDim.x * WARPS * ILP;
    for (uint32_t base = map.first_tile + (blockIdx.x * WARPS + warp) * ILP; base < map.n_local_tiles; base += per_iter) {
        float g[ILP][8], p[ILP][8], m[ILP][8], v[ILP][8];
        bool on[ILP];
        uint32_t ftile[ILP], meta[ILP];
        // every load of the iteration is issued here, none depends on another
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            const uint32_t lt = base + j;
            on[j] = lt < map.n_local_tiles;
            if (on[j]) {
                const uint64_t le = static_cast<uint64_t>(lt) * TILE + lane * 8;
                load8<GDT>(gsrc, le, g[j]);
                load8<OXZ_F32>(master, le, p[j]);
                load8<OXZ_F32>(exp_avg, le, m[j]);
                load8<OXZ_F32>(exp_avg_sq, le, v[j]);
                ftile[j] = flat_tile(map, lt);
                meta[j] = tile_meta[ftile[j]];
            }
        }
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            if (!on[j] || meta[j] == PAD_TILE) continue;
            if constexpr (CHECK) {
                if (!present[meta[j] & 0xffffffu]) continue;
            }
            const uint32_t grp = meta[j] >> 24;
            const float step = k.step_size[grp], decay = k.decay_mul[grp];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float x = __fmul_rn(g[j][i], k.inv_scale);
                if (k.clamp_on) {
                    x = x > k.clamp_hi ? k.clamp_hi : x;
                    x = x < -k.clamp_hi ? -k.clamp_hi : x;
                }
                x = __fmul_rn(__fmul_rn(x, c1), c2);
                adam1(p[j][i], m[j][i], v[j][i], x, k, step, decay);
            }
            const uint64_t le = static_cast<uint64_t>(base + j) * TILE + lane * 8;
            store8<OXZ_F32>(master, le, p[j]);
            store8<OXZ_F32>(exp_avg, le, m[j]);
            store8<OXZ_F32>(exp_avg_sq, le, v[j]);
            const uint64_t fe = static_cast<uint64_t>(ftile[j]) * TILE + lane * 8;
            if (k.push_hint == 0 || PDT == OXZ_F32) {
                for (int r = 0; r < n_work; r++) store8<PDT>(peers.work[r], fe, p[j]);
            } else if constexpr (PDT != OXZ_F32) {
                uint32_t w[4];
                pack8<PDT>(p[j], w);
                for (int r = 0; r < n_work; r++)
                    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(peers.work[r]) + fe) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
}

// One element's share of the update as k_adamw does it: unscale, clamp, both clip coefficients, AdamW.
__device__ __forceinline__ void adam_tile8(float (&p)[8], float (&m)[8], float (&v)[8], const float (&g)[8], const AdamParams& k,
                                           float c1, float c2, float step, float decay) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float x = __fmul_rn(g[i], k.inv_scale);
        if (k.clamp_on) {
            x = x > k.clamp_hi ? k.clamp_hi : x;
            x = x < -k.clamp_hi ? -k.clamp_hi : x;
        }
        x = __fmul_rn(__fmul_rn(x, c1), c2);
        adam1(p[i], m[i], v[i], x, k, step, decay);
    }
}


// The update with the push of 16-bit working weights as 256-bit peer stores. A warp takes two neighbouring tiles per
// round (the f32 state still moves one 256-bit access per lane and array); the two tiles' packed weights, 16 bytes per
// lane each, are exchanged by shuffles so that lanes 0-15 hold tile A and lanes 16-31 tile B in 32-byte pieces, and
// every rank's buffer receives ONE 32-byte store per lane for the pair: half the peer-store instructions of k_adamw
// and 1 KiB per warp and peer. Where the two tiles are not neighbours in the flat space (a shard's odd end) or one of
// them is left out, each goes the 128-bit way. Same arithmetic, same bits as k_adamw.
template <int GDT, int PDT, bool CHECK>
__global__ void __launch_bounds__(THREADS, 2)
    k_adamw_wide(const void* __restrict__ gsrc, float* __restrict__ master, float* __restrict__ exp_avg,
                 float* __restrict__ exp_avg_sq, PeerTable peers, int n_work, TileMap map,
                 const uint32_t* __restrict__ tile_meta, const uint8_t* __restrict__ present,
                 const DevScalars* __restrict__ scalars, AdamParams k) {
    static_assert(PDT == OXZ_BF16 || PDT == OXZ_F16, "16-bit working weights only");
    if (scalars->skip) return;
    const float c1 = scalars->c1, c2 = scalars->c2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per_iter = gridDim.x * WARPS * 2;
    for (uint32_t base = map.first_tile + (blockIdx.x * WARPS + warp) * 2; base < map.n_local_tiles; base += per_iter) {
        float g[2][8], p[2][8], m[2][8], v[2][8];
        bool on[2];
        uint32_t ftile[2], meta[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t lt = base + j;
            on[j] = lt < map.n_local_tiles;
            ftile[j] = 0;
            meta[j] = PAD_TILE;
            if (on[j]) {
                const uint64_t le = static_cast<uint64_t>(lt) * TILE + lane * 8;
                load8<GDT>(gsrc, le, g[j]);
                load8<OXZ_F32>(master, le, p[j]);
                load8<OXZ_F32>(exp_avg, le, m[j]);
                load8<OXZ_F32>(exp_avg_sq, le, v[j]);
                ftile[j] = flat_tile(map, lt);
                meta[j] = tile_meta[ftile[j]];
            }
        }
        uint32_t w[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            on[j] = on[j] && meta[j] != PAD_TILE;
            if constexpr (CHECK) on[j] = on[j] && present[meta[j] & 0xffffffu];
            if (!on[j]) continue;
            const uint32_t grp = meta[j] >> 24;
            adam_tile8(p[j], m[j], v[j], g[j], k, c1, c2, k.step_size[grp], k.decay_mul[grp]);
            const uint64_t le = static_cast<uint64_t>(base + j) * TILE + lane * 8;
            store8<OXZ_F32>(master, le, p[j]);
            store8<OXZ_F32>(exp_avg, le, m[j]);
            store8<OXZ_F32>(exp_avg_sq, le, v[j]);
            pack8<PDT>(p[j], w[j]);
        }
        if (on[0] && on[1] && ftile[1] == ftile[0] + 1) {  // warp-uniform: tiles and their flags are
            const int src = 2 * (lane & 15);
            uint32_t out[8];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t a_lo = __shfl_sync(0xffffffffu, w[0][q], src), b_lo = __shfl_sync(0xffffffffu, w[1][q], src);
                const uint32_t a_hi = __shfl_sync(0xffffffffu, w[0][q], src + 1), b_hi = __shfl_sync(0xffffffffu, w[1][q], src + 1);
                out[q] = lane < 16 ? a_lo : b_lo;
                out[4 + q] = lane < 16 ? a_hi : b_hi;
            }
            const uint64_t fe = static_cast<uint64_t>(ftile[0]) * TILE + (lane < 16 ? 0 : TILE) + (lane & 15) * 16;
            for (int r = 0; r < n_work; r++) {
                uint16_t* dst = static_cast<uint16_t*>(peers.work[r]) + fe;
                asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(out[0]), "r"(out[1]), "r"(out[2]),
                             "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7])
                             : "memory");
            }
        } else {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                if (!on[j]) continue;
                const uint64_t fe = static_cast<uint64_t>(ftile[j]) * TILE + lane * 8;
                for (int r = 0; r < n_work; r++)
                    st_stream(reinterpret_cast<uint4*>(static_cast<uint16_t*>(peers.work[r]) + fe), make_uint4(w[j][0], w[j][1], w[j][2], w[j][3]));
            }
        }
    }
}

// The update with its four input streams staged through shared memory by 1-D bulk asynchronous copies (cp.async.bulk
// + mbarrier, each block fetching for itself), for one rank with every tensor present: STAGES stages of 8 tiles, one elected thread
// issues the four copies of a stage (gradients, master, exp_avg, exp_avg_sq), each warp updates one tile of the stage
// from shared memory and stores its results straight to global memory. It exists to measure staging against the
// direct 256-bit loads of k_adamw on the same work; same arithmetic, same bits. Every wait is bounded.
template <int GDT, int PDT, int STAGES>
__global__ void __launch_bounds__(THREADS)
    k_adamw_staged(const void* __restrict__ gsrc, float* __restrict__ master, float* __restrict__ exp_avg,
                   float* __restrict__ exp_avg_sq, void* __restrict__ work, uint32_t n_tiles,
                   const uint32_t* __restrict__ tile_meta, DevScalars* __restrict__ scalars, AdamParams k) {
    extern __shared__ __align__(128) unsigned char stage_smem[];
    __shared__ __align__(8) uint64_t bar[STAGES];
    if (scalars->skip) return;
    constexpr uint32_t GS = GDT == OXZ_F32 ? 4 : 2;
    constexpr uint32_t G_BYTES = BULK_TILES * TILE * GS, F_BYTES = BULK_TILES * TILE * 4;
    constexpr uint32_t STAGE_BYTES = G_BYTES + 3 * F_BYTES;
    const float c1 = scalars->c1, c2 = scalars->c2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_chunks = n_tiles / BULK_TILES;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bar[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](uint32_t chunk, int stage) {
        const uint64_t e0 = static_cast<uint64_t>(chunk) * BULK_TILES * TILE;
        const uint32_t b = smem_addr(&bar[stage]);
        unsigned char* dst = stage_smem + static_cast<size_t>(stage) * STAGE_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(STAGE_BYTES) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_addr(dst)), "l"(static_cast<const unsigned char*>(gsrc) + e0 * GS), "r"(G_BYTES), "r"(b) : "memory");
#pragma unroll
        for (int a = 0; a < 3; a++) {
            const float* src = a == 0 ? master : a == 1 ? exp_avg : exp_avg_sq;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_addr(dst + G_BYTES + a * F_BYTES)), "l"(src + e0), "r"(F_BYTES), "r"(b) : "memory");
        }
    };
    uint32_t pending = 0, phase = 0;
    for (int s = 0; s < STAGES; s++) {
        const uint32_t c = blockIdx.x + static_cast<uint32_t>(s) * gridDim.x;
        if (c < n_chunks) {
            if (threadIdx.x == 0) issue(c, s);
            pending |= 1u << s;
        }
    }
    int stage = 0;
    bool ok = true;
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const int landed = mbar_wait_bounded(smem_addr(&bar[stage]), (phase >> stage) & 1u, BULK_SPIN_LIMIT) ? 1 : 0;
        if (!__syncthreads_and(landed)) {
            ok = false;
            break;
        }
        pending &= ~(1u << stage);
        phase ^= 1u << stage;
        const unsigned char* st = stage_smem + static_cast<size_t>(stage) * STAGE_BYTES;
        const uint32_t tile = c * BULK_TILES + warp;
        const uint32_t meta = tile_meta[tile];
        float g[8], pmv[3][8];  // master, exp_avg, exp_avg_sq
        if constexpr (GDT == OXZ_F32) {
            const float4* q = reinterpret_cast<const float4*>(st + warp * (TILE * 4) + lane * 32);
            const float4 a = q[0], b2 = q[1];
            g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b2.x; g[5] = b2.y; g[6] = b2.z; g[7] = b2.w;
        } else {
            RawVec<GDT> r;
            r.v = *reinterpret_cast<const uint4*>(st + warp * (TILE * 2) + lane * 16);
            widen_raw<GDT>(r, g);
        }
#pragma unroll
        for (int a = 0; a < 3; a++) {
            const float4* q = reinterpret_cast<const float4*>(st + G_BYTES + a * F_BYTES + warp * (TILE * 4) + lane * 32);
            const float4 lo = q[0], hi = q[1];
            pmv[a][0] = lo.x; pmv[a][1] = lo.y; pmv[a][2] = lo.z; pmv[a][3] = lo.w;
            pmv[a][4] = hi.x; pmv[a][5] = hi.y; pmv[a][6] = hi.z; pmv[a][7] = hi.w;
        }
        // The barrier that frees the stage takes a predicate formed from EVERY value just loaded from shared memory, so
        // those loads have returned when a thread reaches it. A plain barrier does not wait for them: with the memory
        // pipe backed up by the kernel's own stores a shared-memory load can still be queued when the refill's bytes
        // land, and then reads the next chunk's data (seen as a few stale lanes per 10^8 elements).
        uint32_t seen = 0;
#pragma unroll
        for (int i = 0; i < 8; i++)
            seen ^= __float_as_uint(g[i]) ^ __float_as_uint(pmv[0][i]) ^ __float_as_uint(pmv[1][i]) ^ __float_as_uint(pmv[2][i]);
        (void)__syncthreads_or(seen == 0x7fc01234u);  // the outcome is of no interest: it may be refilled now
        const uint32_t nc = c + static_cast<uint32_t>(STAGES) * gridDim.x;
        if (nc < n_chunks) {
            if (threadIdx.x == 0) issue(nc, stage);
            pending |= 1u << stage;
        }
        if (++stage == STAGES) stage = 0;
        if (meta == PAD_TILE) continue;
        const uint32_t grp = meta >> 24;
        adam_tile8(pmv[0], pmv[1], pmv[2], g, k, c1, c2, k.step_size[grp], k.decay_mul[grp]);
        const uint64_t e = static_cast<uint64_t>(tile) * TILE + lane * 8;
        store8<OXZ_F32>(master, e, pmv[0]);
        store8<OXZ_F32>(exp_avg, e, pmv[1]);
        store8<OXZ_F32>(exp_avg_sq, e, pmv[2]);
        if (work != nullptr) store8<PDT>(work, e, pmv[0]);
    }
    if (!ok) {
        // a copy of this block never landed: say so, give the copies in flight their bounded chance, and leave; the
        // tiles this block had not reached keep their old state and the host reports the step failed
        if (threadIdx.x == 0) atomicMax(&scalars->wait_expired, 1);
        for (int s = 0; s < STAGES; s++)
            if (pending & (1u << s)) mbar_wait_bounded(smem_addr(&bar[s]), (phase >> s) & 1u, BULK_SPIN_LIMIT);
        return;
    }
    // the tiles past the last whole chunk: the direct way, by the last block
    const uint32_t tail0 = n_chunks * BULK_TILES;
    if (blockIdx.x == gridDim.x - 1 && tail0 + warp < n_tiles) {
        const uint32_t tile = tail0 + warp;
        const uint32_t meta = tile_meta[tile];
        if (meta != PAD_TILE) {
            const uint64_t e = static_cast<uint64_t>(tile) * TILE + lane * 8;
            float g[8], p[8], m[8], v[8];
            load8<GDT>(gsrc, e, g);
            load8<OXZ_F32>(master, e, p);
            load8<OXZ_F32>(exp_avg, e, m);
            load8<OXZ_F32>(exp_avg_sq, e, v);
            const uint32_t grp = meta >> 24;
            adam_tile8(p, m, v, g, k, c1, c2, k.step_size[grp], k.decay_mul[grp]);
            store8<OXZ_F32>(master, e, p);
            store8<OXZ_F32>(exp_avg, e, m);
            store8<OXZ_F32>(exp_avg_sq, e, v);
            if (work != nullptr) store8<PDT>(work, e, p);
        }
    }
}

// ---------------------------------------------------------------- flatten

// Each warp takes several tiles per round and walks them in phases (tile entries, then the per-tensor lookups, then
// every data load, then the stores), so that the dependent lookups of one tile overlap those of the others and enough
// bytes are in flight per SM to fill HBM. 16-bit vectors stay packed in registers; only an accumulation widens them.
template <int DT>
__global__ void __launch_bounds__(THREADS, 3)
    k_flatten(void* __restrict__ flat, uint32_t n_tiles, const uint32_t* __restrict__ tile_meta,
              const uint64_t* __restrict__ offsets, const uint64_t* __restrict__ numel,
              const void* const* __restrict__ src, int accumulate) {
    constexpr int ILP = DT == OXZ_F32 ? 2 : 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per_iter = gridDim.x * WARPS * ILP;
    for (uint32_t base = (blockIdx.x * WARPS + warp) * ILP; base < n_tiles; base += per_iter) {
        uint32_t meta[ILP];
#pragma unroll
        for (int j = 0; j < ILP; j++) meta[j] = base + j < n_tiles ? tile_meta[base + j] : PAD_TILE;
        const void* s[ILP];
        uint64_t te[ILP], n[ILP];  // element within the tensor, the tensor's length
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            s[j] = nullptr;
            te[j] = n[j] = 0;
            if (meta[j] != PAD_TILE) {
                const uint32_t t = meta[j] & 0xffffffu;
                s[j] = src[t];
                te[j] = static_cast<uint64_t>(base + j) * TILE + lane * 8 - offsets[t];
                n[j] = numel[t];
            }
        }
        RawVec<DT> x[ILP], old[ILP];
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            if constexpr (DT == OXZ_F32) {
#pragma unroll
                for (int i = 0; i < 8; i++) x[j].x[i] = 0.f;
            } else {
                x[j].v = make_uint4(0u, 0u, 0u, 0u);
            }
            if (s[j] != nullptr && te[j] + 8 <= n[j]) {
                // the caller's memory is promised 16-byte aligned only
                if constexpr (DT == OXZ_F32) load8_user<OXZ_F32>(s[j], te[j], x[j].x);
                else x[j].v = ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(s[j]) + te[j]));
            }
        }
        if (accumulate) {
#pragma unroll
            for (int j = 0; j < ILP; j++)
                if (s[j] != nullptr) load_raw<DT>(flat, static_cast<uint64_t>(base + j) * TILE + lane * 8, old[j]);
        }
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            if (base + j >= n_tiles) continue;
            const uint64_t fe = static_cast<uint64_t>(base + j) * TILE + lane * 8;
            const bool ragged = s[j] != nullptr && te[j] + 8 > n[j];  // the tensor ends inside this vector
            if (!ragged && !(accumulate && s[j] != nullptr)) {
                if (accumulate && s[j] == nullptr && meta[j] != PAD_TILE) continue;  // nothing to add
                // a plain copy (or zeros for padding and for a tensor without a gradient)
                if constexpr (DT == OXZ_F32) store8<OXZ_F32>(flat, fe, x[j].x);
                else st_stream(reinterpret_cast<uint4*>(static_cast<uint16_t*>(flat) + fe), x[j].v);
                continue;
            }
            float f[8];
            widen_raw<DT>(x[j], f);
            if (ragged) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    f[i] = 0.f;
                    if (te[j] + i < n[j]) {
                        if constexpr (DT == OXZ_F32) f[i] = static_cast<const float*>(s[j])[te[j] + i];
                        else if constexpr (DT == OXZ_BF16)
                            f[i] = __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t*>(s[j])[te[j] + i]) << 16);
                        else f[i] = __half2float(static_cast<const __half*>(s[j])[te[j] + i]);
                    }
                }
            }
            if (accumulate) {
                float o[8];
                widen_raw<DT>(old[j], o);
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = __fadd_rn(o[i], f[i]);
            }
            store8<DT>(flat, fe, f);
        }
    }
}

// ---------------------------------------------------------------- launchers

static int adam_variant() {  // read at every launch, so that a test can compare the forms within one process; -1: not set
    const char* e = getenv("OXZ_ADAM_VARIANT");
    return e ? atoi(e) : -1;
}

static thread_local int32_t g_last_update_kernel = 0;
int32_t last_update_kernel() { return g_last_update_kernel; }

static int adam_blocks_per_sm(int variant) { return variant == 1 ? 4 : variant == 2 ? 2 : 3; }

// Clusters of CLUSTER blocks of `func` that can be resident on the device at once.
static int max_cluster_blocks(const void* func, int fallback) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CLUSTER * 1024);
    cfg.blockDim = dim3(THREADS);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = CLUSTER;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, func, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fallback;
    }
    return n * CLUSTER;
}

int32_t query_geom(int device, LaunchGeom* g) {
    cudaDeviceProp prop;
    OXZ_CUDA(cudaGetDeviceProperties(&prop, device));
    g->sm_count = prop.multiProcessorCount;
    // The reduction kernels are persistent: every block takes an equal share, so the grid must be resident in
    // one wave. Size it by the clusters the device can hold at once, the smallest over the variants.
    int nb = g->sm_count * 4;
    nb -= nb % CLUSTER;
    const void* funcs[] = {
        (const void*)k_sumsq<OXZ_F32, 4, false>,  (const void*)k_sumsq<OXZ_BF16, 4, false>, (const void*)k_sumsq<OXZ_F16, 4, false>,
        (const void*)k_sumsq<OXZ_F32, 4, true>,   (const void*)k_sumsq<OXZ_BF16, 4, true>,  (const void*)k_sumsq<OXZ_F16, 4, true>,
        (const void*)k_sumsq_plain<OXZ_F32>, (const void*)k_sumsq_plain<OXZ_BF16>, (const void*)k_sumsq_plain<OXZ_F16>,
        (const void*)k_sumsq_stream16<OXZ_BF16, 2, false>, (const void*)k_sumsq_stream16<OXZ_F16, 2, false>,
        (const void*)k_sumsq_stream16<OXZ_BF16, 2, true>, (const void*)k_sumsq_stream16<OXZ_F16, 2, true>};
    for (const void* f : funcs) {
        const int m = max_cluster_blocks(f, nb);
        if (m < nb) nb = m;
    }
    // the pull kernels hold up to eight vectors per lane; their register use, and so their grid, depends on the dtype
    const void* pulls[3][8] = {
        {(const void*)k_pull_sumsq<OXZ_F32, false, 0>, (const void*)k_pull_sumsq<OXZ_F32, true, 0>, (const void*)k_pull_sumsq<OXZ_F32, false, 2>, (const void*)k_pull_sumsq<OXZ_F32, true, 2>,
         (const void*)k_pull_sumsq<OXZ_F32, false, 4>, (const void*)k_pull_sumsq<OXZ_F32, true, 4>, (const void*)k_pull_sumsq<OXZ_F32, false, 8>, (const void*)k_pull_sumsq<OXZ_F32, true, 8>},
        {(const void*)k_pull_sumsq<OXZ_BF16, false, 0>, (const void*)k_pull_sumsq<OXZ_BF16, true, 0>, (const void*)k_pull_sumsq<OXZ_BF16, false, 2>, (const void*)k_pull_sumsq<OXZ_BF16, true, 2>,
         (const void*)k_pull_sumsq<OXZ_BF16, false, 4>, (const void*)k_pull_sumsq<OXZ_BF16, true, 4>, (const void*)k_pull_sumsq<OXZ_BF16, false, 8>, (const void*)k_pull_sumsq<OXZ_BF16, true, 8>},
        {(const void*)k_pull_sumsq<OXZ_F16, false, 0>, (const void*)k_pull_sumsq<OXZ_F16, true, 0>, (const void*)k_pull_sumsq<OXZ_F16, false, 2>, (const void*)k_pull_sumsq<OXZ_F16, true, 2>,
         (const void*)k_pull_sumsq<OXZ_F16, false, 4>, (const void*)k_pull_sumsq<OXZ_F16, true, 4>, (const void*)k_pull_sumsq<OXZ_F16, false, 8>, (const void*)k_pull_sumsq<OXZ_F16, true, 8>}};
    for (int dt = 0; dt < 3; dt++) {
        int pb = nb;
        for (const void* f : pulls[dt]) {
            const int m = max_cluster_blocks(f, pb);
            if (m < pb) pb = m;
        }
        g->pull_blocks[dt] = pb > 0 ? pb : CLUSTER;
        if (const char* e = getenv("OXZ_PULL_BLOCKS")) {  // tuning aid
            int want = atoi(e) / CLUSTER * CLUSTER;
            if (want >= CLUSTER && want < g->pull_blocks[dt]) g->pull_blocks[dt] = want;
        }
    }
    g->norm_blocks = nb > 0 ? nb : CLUSTER;
    for (int i = 0; i < 3; i++) {
        int bb = g->sm_count * 2;
        bb -= bb % CLUSTER;
        g->bulk_blocks[i] = bb < g->norm_blocks ? bb : g->norm_blocks;
    }
    g->adam_blocks = g->sm_count * adam_blocks_per_sm(adam_variant());
    return OXZ_OK;
}

uint32_t norm_partial_slots(const LaunchGeom& g) { return static_cast<uint32_t>(g.norm_blocks / CLUSTER); }
uint32_t pull_partial_slots(const LaunchGeom& g, int32_t dt) {
    return static_cast<uint32_t>(g.pull_blocks[dt == OXZ_F32 ? 0 : dt == OXZ_BF16 ? 1 : 2] / CLUSTER);
}

static int32_t check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return OXZ_OK;
}

template <bool CHECK>
static int32_t launch_sumsq_c(cudaStream_t s, const LaunchGeom& g, const void* grads, int32_t dt, const TileMap& map,
                              const uint32_t* tile_meta, const uint8_t* present, float inv_scale, float clamp_hi,
                              int32_t clamp_on, double* partials) {
    constexpr int ILP = 4;
    dim3 grid(g.norm_blocks), block(THREADS);
    // measured on B200 (2.47 GB of bf16): 0.383 ms with two 256-bit loads in flight per thread, 0.397 ms with
    // four, 0.420 ms for the tile-wise 128-bit form (0.63 ms when that form also looks the tensors' flags up)
    if (dt != OXZ_F32) {
        const uint64_t first = static_cast<uint64_t>(map.first_tile) * TILE, end = static_cast<uint64_t>(map.n_local_tiles) * TILE;
        const uint16_t* g16 = static_cast<const uint16_t*>(grads);
        if (dt == OXZ_BF16) k_sumsq_stream16<OXZ_BF16, 2, CHECK><<<grid, block, 0, s>>>(g16, first, end, inv_scale, clamp_hi, clamp_on, partials, map, tile_meta, present);
        else k_sumsq_stream16<OXZ_F16, 2, CHECK><<<grid, block, 0, s>>>(g16, first, end, inv_scale, clamp_hi, clamp_on, partials, map, tile_meta, present);
        return check_launch("k_sumsq_stream16");
    }
    switch (dt) {
        case OXZ_F32: k_sumsq<OXZ_F32, ILP, CHECK><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, partials); break;
        case OXZ_BF16: k_sumsq<OXZ_BF16, ILP, CHECK><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, partials); break;
        case OXZ_F16: k_sumsq<OXZ_F16, ILP, CHECK><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, partials); break;
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", dt);
    }
    return check_launch("k_sumsq");
}

int32_t launch_sumsq(cudaStream_t s, const LaunchGeom& g, const void* grads, int32_t dt, const TileMap& map,
                     const uint32_t* tile_meta, const uint8_t* present, bool check_present, float inv_scale,
                     float clamp_hi, int32_t clamp_on, double* partials) {
    return check_present ? launch_sumsq_c<true>(s, g, grads, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, partials)
                         : launch_sumsq_c<false>(s, g, grads, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, partials);
}

int32_t launch_sumsq_plain(cudaStream_t s, int blocks, const void* grads, int32_t dt, uint64_t n, float inv_scale,
                           float clamp_hi, int32_t clamp_on, double* partials) {
    dim3 grid(blocks), block(THREADS);
    switch (dt) {
        case OXZ_F32: k_sumsq_plain<OXZ_F32><<<grid, block, 0, s>>>(grads, n, inv_scale, clamp_hi, clamp_on, partials); break;
        case OXZ_BF16: k_sumsq_plain<OXZ_BF16><<<grid, block, 0, s>>>(grads, n, inv_scale, clamp_hi, clamp_on, partials); break;
        case OXZ_F16: k_sumsq_plain<OXZ_F16><<<grid, block, 0, s>>>(grads, n, inv_scale, clamp_hi, clamp_on, partials); break;
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", dt);
    }
    return check_launch("k_sumsq_plain");
}

int32_t launch_sumsq_tensors(cudaStream_t s, const LaunchGeom& g, const void* grads, int32_t dt, const TileMap& map,
                             const uint32_t* tile_meta, const uint8_t* present, float inv_scale, float clamp_hi,
                             int32_t clamp_on, double* out) {
    dim3 grid(g.sm_count * 4), block(THREADS);
    switch (dt) {
        case OXZ_F32: k_sumsq_tensors<OXZ_F32><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, out); break;
        case OXZ_BF16: k_sumsq_tensors<OXZ_BF16><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, out); break;
        case OXZ_F16: k_sumsq_tensors<OXZ_F16><<<grid, block, 0, s>>>(grads, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, out); break;
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", dt);
    }
    return check_launch("k_sumsq_tensors");
}

template <bool CHECK, int WORLD>
static int32_t launch_pull_w(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int staged, int32_t dt,
                             const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, float inv_scale,
                             float clamp_hi, int32_t clamp_on, float* reduced, double* partials) {
    dim3 grid(g.pull_blocks[dt == OXZ_F32 ? 0 : dt == OXZ_BF16 ? 1 : 2]), block(THREADS);
    switch (dt) {
        case OXZ_F32: k_pull_sumsq<OXZ_F32, CHECK, WORLD><<<grid, block, 0, s>>>(peers, world, staged, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials); break;
        case OXZ_BF16: k_pull_sumsq<OXZ_BF16, CHECK, WORLD><<<grid, block, 0, s>>>(peers, world, staged, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials); break;
        case OXZ_F16: k_pull_sumsq<OXZ_F16, CHECK, WORLD><<<grid, block, 0, s>>>(peers, world, staged, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials); break;
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", dt);
    }
    return check_launch("k_pull_sumsq");
}

template <bool CHECK>
static int32_t launch_pull_c(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int staged, int32_t dt,
                             const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, float inv_scale,
                             float clamp_hi, int32_t clamp_on, float* reduced, double* partials) {
    switch (world) {
        case 2: return launch_pull_w<CHECK, 2>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials);
        case 4: return launch_pull_w<CHECK, 4>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials);
        case 8: return launch_pull_w<CHECK, 8>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials);
        default: return launch_pull_w<CHECK, 0>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials);
    }
}

int32_t launch_pull_sumsq(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int staged, int32_t dt,
                          const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, bool check_present,
                          float inv_scale, float clamp_hi, int32_t clamp_on, float* reduced, double* partials) {
    return check_present ? launch_pull_c<true>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials)
                         : launch_pull_c<false>(s, g, peers, world, staged, dt, map, tile_meta, present, inv_scale, clamp_hi, clamp_on, reduced, partials);
}

template <int DT, int WORLD, int STAGES>
static int32_t launch_pull_bulk_t(cudaStream_t s, int blocks, const PeerTable& peers, const TileMap& map,
                                  const uint32_t* tile_meta, const uint8_t* present, bool check_present, float inv_scale,
                                  float clamp_hi, int32_t clamp_on, float* reduced, double* partials, DevScalars* scalars) {
    const size_t smem = static_cast<size_t>(BULK_BYTES) * WORLD * STAGES;
    // Per instantiation and device: allow the dynamic shared memory, then size the grid to the clusters that are
    // resident at once with it (a persistent grid must be one wave). Idempotent: a race only repeats the calls.
    static int resident[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(OXZ_ERR_UNSUPPORTED, "device ordinal %d is past 64", dev);
    if (resident[dev] == 0) {
        cudaError_t e = cudaFuncSetAttribute(k_pull_bulk<DT, WORLD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "cudaFuncSetAttribute(k_pull_bulk): %s", cudaGetErrorString(e));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CLUSTER * 1024);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = CLUSTER;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, k_pull_bulk<DT, WORLD, STAGES>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = blocks / CLUSTER / 2;
        }
        resident[dev] = n * CLUSTER > 0 ? n * CLUSTER : CLUSTER;
    }
    if (blocks > resident[dev]) blocks = resident[dev];
    // OXZ_PULL_WAIT_LIMIT lowers the bound of the main-loop waits (0: the first wait gives up at once) so that a test can
    // see the run-out path: the kernel records it, still collects its copies in flight and ends normally.
    // "N@R" lowers it on rank R alone: the other ranks then learn of the run-out through the step's exchange.
    const char* lim = getenv("OXZ_PULL_WAIT_LIMIT");
    uint32_t wait_limit = BULK_SPIN_LIMIT;
    if (lim) {
        const char* at = strchr(lim, '@');
        if (!at || static_cast<uint32_t>(strtoul(at + 1, nullptr, 10)) == map.rank) wait_limit = static_cast<uint32_t>(strtoul(lim, nullptr, 10));
    }
    k_pull_bulk<DT, WORLD, STAGES><<<dim3(blocks), dim3(THREADS), smem, s>>>(peers, map, tile_meta, present, check_present ? 1 : 0, inv_scale, clamp_hi, clamp_on, reduced, partials, scalars, wait_limit);
    return check_launch("k_pull_bulk");
}

bool pull_bulk_fits(const TileMap& map, int32_t world, int32_t dt) {
    if (dt == OXZ_F32 || (world != 2 && world != 4 && world != 8)) return false;
    // a chunk must not straddle two buckets' shards; a ragged end of the last shard is handled by plain loads
    if (map.tiles_per_shard % BULK_TILES || map.first_tile % BULK_TILES) return false;
    return true;
}

int32_t launch_pull_bulk(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int32_t dt,
                         const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, bool check_present,
                         float inv_scale, float clamp_hi, int32_t clamp_on, float* reduced, double* partials,
                         uint32_t slots, DevScalars* scalars) {
    int blocks = g.bulk_blocks[world == 2 ? 0 : world == 4 ? 1 : 2];
    if (const char* e = getenv("OXZ_BULK_BLOCKS")) {  // tuning aid: another grid size, still a whole number of clusters
        const int want = atoi(e) / CLUSTER * CLUSTER;
        if (want >= CLUSTER) blocks = want;
    }
    if (static_cast<uint32_t>(blocks / CLUSTER) > slots) blocks = static_cast<int>(slots) * CLUSTER;  // one partial slot per cluster
    if (blocks < CLUSTER) return fail(OXZ_ERR_INVALID, "launch_pull_bulk: no partial slot to write to");
#define OXZ_BULK(DT) \
    switch (world) { \
        case 2: return launch_pull_bulk_t<DT, 2, 4>(s, blocks, peers, map, tile_meta, present, check_present, inv_scale, clamp_hi, clamp_on, reduced, partials, scalars); \
        case 4: return launch_pull_bulk_t<DT, 4, 4>(s, blocks, peers, map, tile_meta, present, check_present, inv_scale, clamp_hi, clamp_on, reduced, partials, scalars); \
        default: return launch_pull_bulk_t<DT, 8, 3>(s, blocks, peers, map, tile_meta, present, check_present, inv_scale, clamp_hi, clamp_on, reduced, partials, scalars); \
    }
    if (dt == OXZ_BF16) { OXZ_BULK(OXZ_BF16) }
    OXZ_BULK(OXZ_F16)
#undef OXZ_BULK
}

int32_t launch_reduce_partials(cudaStream_t s, const double* partials, uint32_t slots, double* acc, const DevScalars* scalars) {
    k_reduce_partials<<<1, THREADS, 0, s>>>(partials, slots, acc, scalars);
    return check_launch("k_reduce_partials");
}

int32_t launch_gate(cudaStream_t s, const MailPeers& mail, int32_t world, int32_t rank, uint64_t seq, const uint8_t* present_in,
                    uint8_t* present_out, uint32_t T, DevScalars* scalars, uint64_t limit_ns, const int32_t* abort_flag) {
    if (T > MAIL_PAYLOAD) return fail(OXZ_ERR_INVALID, "launch_gate: %u flags do not fit a mailbox slot", T);
    k_gate<<<1, THREADS, 0, s>>>(mail, world, rank, seq, present_in, present_out, T, scalars, limit_ns, abort_flag);
    return check_launch("k_gate");
}

int32_t launch_decide(cudaStream_t s, const MailPeers& mail, int32_t world, int32_t rank, uint64_t seq, const double* partials,
                      uint32_t slots, double* acc, uint32_t n_extras, int32_t sum_norm, const FinalizeParams& fp,
                      DevScalars* scalars, uint64_t limit_ns, const int32_t* abort_flag) {
    k_decide<<<1, THREADS, 0, s>>>(mail, world, rank, seq, partials, slots, acc, n_extras, sum_norm, fp, scalars, limit_ns, abort_flag);
    return check_launch("k_decide");
}

int32_t launch_finalize(cudaStream_t s, const double* acc, const FinalizeParams& fp, DevScalars* scalars) {
    k_finalize<<<1, 32, 0, s>>>(acc, fp, scalars);
    return check_launch("k_finalize");
}

// The update kernel's shape: tiles per warp per iteration (ILP) and the resident blocks per SM its register budget
// is held to. Measured on B200 on the 1.24 B-parameter set (28 B/param): ILP 1 x 3 blocks/SM streams 6.4 TB/s,
// ILP 2 x 2 blocks/SM 5.4 TB/s, ILP 1 x 4 blocks/SM 5.7 TB/s. OXZ_ADAM_VARIANT=1|2 selects the other two for tuning.
template <int GDT, int PDT, bool CHECK>
static void launch_adamw_v(int variant, dim3 grid, cudaStream_t s, const void* gsrc, float* master, float* m, float* v,
                           const PeerTable& peers, int32_t n_work, const TileMap& map, const uint32_t* tile_meta,
                           const uint8_t* present, const DevScalars* scalars, const AdamParams& ap) {
    dim3 block(THREADS);
#define OXZ_ADAM(ILP, MINB) k_adamw<GDT, PDT, ILP, MINB, CHECK><<<grid, block, 0, s>>>(gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap)
    switch (variant) {
        case 1: OXZ_ADAM(1, 4); break;
        case 2: OXZ_ADAM(2, 2); break;
        default: OXZ_ADAM(1, 3); break;
    }
#undef OXZ_ADAM
}

// The staged form: grid = the blocks resident at once with its shared memory (a persistent grid is one wave).
template <int GDT, int PDT, int STAGES>
static int32_t launch_adamw_staged(cudaStream_t s, const LaunchGeom& g, const void* gsrc, float* master, float* m, float* v,
                                   void* work, uint32_t n_tiles, const uint32_t* tile_meta, const DevScalars* scalars,
                                   const AdamParams& ap) {
    constexpr size_t smem = static_cast<size_t>(STAGES) * BULK_TILES * TILE * ((GDT == OXZ_F32 ? 4 : 2) + 12);
    static int per_sm[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(OXZ_ERR_UNSUPPORTED, "device ordinal %d is past 64", dev);
    if (per_sm[dev] == 0) {
        cudaError_t e = cudaFuncSetAttribute(k_adamw_staged<GDT, PDT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "cudaFuncSetAttribute(k_adamw_staged): %s", cudaGetErrorString(e));
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_adamw_staged<GDT, PDT, STAGES>, THREADS, smem);
        if (e != cudaSuccess || n <= 0) return fail(OXZ_ERR_CUDA, "k_adamw_staged does not fit an SM with %zu bytes of shared memory", smem);
        per_sm[dev] = n;
    }
    k_adamw_staged<GDT, PDT, STAGES><<<dim3(g.sm_count * per_sm[dev]), dim3(THREADS), smem, s>>>(
        gsrc, master, m, v, work, n_tiles, tile_meta, const_cast<DevScalars*>(scalars), ap);
    return check_launch("k_adamw_staged");
}

template <int GDT, bool CHECK>
static int32_t launch_adamw_g(cudaStream_t s, const LaunchGeom& g, const void* gsrc, float* master, float* m, float* v,
                              const PeerTable& peers, int32_t n_work, int32_t pdt, const TileMap& map,
                              const uint32_t* tile_meta, const uint8_t* present, const DevScalars* scalars,
                              const AdamParams& ap) {
    int variant = adam_variant();
    // Not set: with two ranks and 16-bit weights the wide-store form (its update is HBM-bound with the push riding along,
    // and two tiles per warp at two blocks per SM stream it 4 % faster: 3.05 against 3.19 ms on the 1.24 B set); the
    // one-tile form everywhere else (one rank: 5.40 against 6.45 ms; four ranks, wire-bound: 2.93 against 2.97 ms).
    if (variant < 0) variant = (n_work == 2 && pdt != OXZ_F32) ? 3 : 0;
    // OXZ_ADAM_VARIANT=4: the shared-memory-staged form, where it applies (one rank, every tensor present, the whole
    // range: local and flat tiles coincide). Measured against the direct loads, not the default.
    // (5: the same with four stages instead of three.)
    if ((variant == 4 || variant == 5) && !CHECK && n_work <= 1 && map.first_tile == 0 && map.tiles_per_shard == map.tiles_per_bucket && map.rank == 0) {
        void* work = n_work ? peers.work[0] : nullptr;
        g_last_update_kernel = OXZ_UPDATE_KERNEL_STAGED;
#define OXZ_STAGED(PDT) \
        (variant == 4 ? launch_adamw_staged<GDT, PDT, 3>(s, g, gsrc, master, m, v, work, map.n_local_tiles, tile_meta, scalars, ap) \
                      : launch_adamw_staged<GDT, PDT, 4>(s, g, gsrc, master, m, v, work, map.n_local_tiles, tile_meta, scalars, ap))
        switch (pdt) {
            case OXZ_F32: return OXZ_STAGED(OXZ_F32);
            case OXZ_BF16: return OXZ_STAGED(OXZ_BF16);
            case OXZ_F16: return OXZ_STAGED(OXZ_F16);
            default: return fail(OXZ_ERR_INVALID, "unknown parameter dtype %d", pdt);
        }
#undef OXZ_STAGED
    }
    // OXZ_ADAM_VARIANT=3: 256-bit stores of the 16-bit working weights (two tiles per warp)
    if (variant == 3 && pdt != OXZ_F32 && n_work >= 1) {
        dim3 grid2(g.sm_count * 2), block(THREADS);
        g_last_update_kernel = OXZ_UPDATE_KERNEL_WIDE;
        if (pdt == OXZ_BF16) k_adamw_wide<GDT, OXZ_BF16, CHECK><<<grid2, block, 0, s>>>(gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap);
        else k_adamw_wide<GDT, OXZ_F16, CHECK><<<grid2, block, 0, s>>>(gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap);
        return check_launch("k_adamw_wide");
    }
    dim3 grid(g.adam_blocks);
    if (const char* e = getenv("OXZ_ADAM_BLOCKS")) {  // tuning aid: another grid size
        const int want = atoi(e);
        if (want > 0) grid = dim3(want);
    }
    g_last_update_kernel = OXZ_UPDATE_KERNEL_TILE;
    switch (pdt) {
        case OXZ_F32: launch_adamw_v<GDT, OXZ_F32, CHECK>(variant, grid, s, gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap); break;
        case OXZ_BF16: launch_adamw_v<GDT, OXZ_BF16, CHECK>(variant, grid, s, gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap); break;
        case OXZ_F16: launch_adamw_v<GDT, OXZ_F16, CHECK>(variant, grid, s, gsrc, master, m, v, peers, n_work, map, tile_meta, present, scalars, ap); break;
        default: return fail(OXZ_ERR_INVALID, "unknown parameter dtype %d", pdt);
    }
    return check_launch("k_adamw");
}

template <bool CHECK>
static int32_t launch_adamw_c(cudaStream_t s, const LaunchGeom& g, const void* gsrc, int32_t gdt, float* master, float* m,
                              float* v, const PeerTable& peers, int32_t n_work, int32_t pdt, const TileMap& map,
                              const uint32_t* tile_meta, const uint8_t* present, const DevScalars* scalars,
                              const AdamParams& ap) {
    switch (gdt) {
        case OXZ_F32: return launch_adamw_g<OXZ_F32, CHECK>(s, g, gsrc, master, m, v, peers, n_work, pdt, map, tile_meta, present, scalars, ap);
        case OXZ_BF16: return launch_adamw_g<OXZ_BF16, CHECK>(s, g, gsrc, master, m, v, peers, n_work, pdt, map, tile_meta, present, scalars, ap);
        case OXZ_F16: return launch_adamw_g<OXZ_F16, CHECK>(s, g, gsrc, master, m, v, peers, n_work, pdt, map, tile_meta, present, scalars, ap);
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", gdt);
    }
}

int32_t launch_adamw(cudaStream_t s, const LaunchGeom& g, const void* gsrc, int32_t gdt, float* master, float* m,
                     float* v, const PeerTable& peers, int32_t n_work, int32_t pdt, const TileMap& map,
                     const uint32_t* tile_meta, const uint8_t* present, bool check_present, const DevScalars* scalars,
                     const AdamParams& ap) {
    return check_present ? launch_adamw_c<true>(s, g, gsrc, gdt, master, m, v, peers, n_work, pdt, map, tile_meta, present, scalars, ap)
                         : launch_adamw_c<false>(s, g, gsrc, gdt, master, m, v, peers, n_work, pdt, map, tile_meta, present, scalars, ap);
}

int32_t launch_flatten(cudaStream_t s, const LaunchGeom& g, void* flat, int32_t dt, uint32_t n_tiles,
                       const uint32_t* tile_meta, const uint64_t* d_offsets, const uint64_t* d_numel,
                       const void* const* d_src, int32_t accumulate) {
    dim3 grid(g.sm_count * 3), block(THREADS);
    switch (dt) {
        case OXZ_F32: k_flatten<OXZ_F32><<<grid, block, 0, s>>>(flat, n_tiles, tile_meta, d_offsets, d_numel, d_src, accumulate); break;
        case OXZ_BF16: k_flatten<OXZ_BF16><<<grid, block, 0, s>>>(flat, n_tiles, tile_meta, d_offsets, d_numel, d_src, accumulate); break;
        case OXZ_F16: k_flatten<OXZ_F16><<<grid, block, 0, s>>>(flat, n_tiles, tile_meta, d_offsets, d_numel, d_src, accumulate); break;
        default: return fail(OXZ_ERR_INVALID, "unknown gradient dtype %d", dt);
    }
    return check_launch("k_flatten");
}

}  // namespace oxz
