// Lattice kernels for one pos_dim (compile with -DPERMUTO_DIM=2..7), sm_100a.
//
// Work decomposition shared by all kernels: one thread owns one point and LPT consecutive
// levels.  blockIdx.x walks point tiles, blockIdx.y walks level groups, and blocks are
// dispatched x-fastest, so the whole grid sweeps the points once per level group: the
// slices of the value table (and of its gradient) that are live at any time are the LPT
// slices of one group, which stay L2-resident.  With LPT = 4 and two features per level a
// thread produces / consumes 8 consecutive floats of a feature row = one 32-byte sector,
// moved with a single 256-bit access (ld/st.global.v8.f32, new on sm_100), directly in the
// final [N, 2L] layout -- no transposed intermediate.
//
// What each kernel replaces in the reference (paths relative to its root):
//   forward_kernel          kernels/permutohedral_encoding/EncodingGPU.cuh:68-256
//   backward_kernel         EncodingGPU.cuh:259-414 (table) and :530-769 (positions), fused
//   double_backward_kernel  EncodingGPU.cuh:1016-1257 and :1260-1493, fused
#include "permuto_geometry.cuh"
#include "permuto_internal.h"

#ifndef PERMUTO_DIM
#error "compile with -DPERMUTO_DIM=<2..7>"
#endif

namespace permuto {
namespace {

constexpr int D = PERMUTO_DIM;
#ifndef PERMUTO_THREADS
#define PERMUTO_THREADS 256
#endif
// Resident blocks per SM the register allocator must leave room for.  Measured on B200: the
// gather+scatter kernels ran at 64-71 registers (36-46 % of the warps an SM can hold) and gain a
// few per cent when capped at 64; the gather-only position-gradient kernel gains 10 % at 51.
#ifndef PERMUTO_MIN_BLOCKS
#define PERMUTO_MIN_BLOCKS 4
#endif
#ifndef PERMUTO_MIN_BLOCKS_GATHER_ONLY
#define PERMUTO_MIN_BLOCKS_GATHER_ONLY (PERMUTO_DIM <= 4 ? 5 : 4)  // 5 spills and loses from pos_dim 5 up
#endif
constexpr int kThreads = PERMUTO_THREADS;
constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ void load_pos(const Problem& p, int64_t n, float (&pos)[D]) {
    const float* src = p.positions + n * p.pos_stride_n;
#pragma unroll
    for (int i = 0; i < D; ++i) pos[i] = __ldg(src + i * p.pos_stride_d);
}

// unsigned modulo by the capacity (EncodingGPU.cuh:34-36); a mask when it is a power of two
__device__ __forceinline__ void to_slots(const Problem& p, const Simplex<D>& s, uint32_t (&slot)[D + 1]) {
    if (p.cap_is_pow2) {
#pragma unroll
        for (int r = 0; r <= D; ++r) slot[r] = s.hash[r] & (p.capacity - 1u);
    } else {
#pragma unroll
        for (int r = 0; r <= D; ++r) slot[r] = s.hash[r] % p.capacity;
    }
}

// 8 consecutive floats of a feature row, 32-byte aligned
__device__ __forceinline__ void load8(const float* src, float (&v)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(src));
}
__device__ __forceinline__ void store8(float* dst, const float (&v)[8]) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "f"(v[0]), "f"(v[1]),
                 "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
}

// Row segment [2*l0, 2*(l0+LPT)) of point n: vector path when the whole group is inside the
// level range and rows are 32-byte aligned, else per-level float2 accesses.
template <int LPT>
__device__ __forceinline__ void load_row_segment(const Problem& p, const float* rows, int64_t n, int l0,
                                                 float (&v)[2 * LPT]) {
    const float* src = rows + n * p.width + 2 * l0;
    if (LPT == 4 && p.rows_vec8_ok && l0 + LPT <= p.level_end) {
        float t[8];
        load8(src, t);
#pragma unroll
        for (int i = 0; i < 2 * LPT; ++i) v[i] = t[i % 8];
    } else {
#pragma unroll
        for (int k = 0; k < LPT; ++k) {
            float2 g = make_float2(0.f, 0.f);
            if (l0 + k < p.level_end) g = __ldg(reinterpret_cast<const float2*>(src) + k);
            v[2 * k] = g.x;
            v[2 * k + 1] = g.y;
        }
    }
}
template <int LPT>
__device__ __forceinline__ void store_row_segment(const Problem& p, float* rows, int64_t n, int l0,
                                                  const float (&v)[2 * LPT]) {
    float* dst = rows + n * p.width + 2 * l0;
    if (LPT == 4 && p.rows_vec8_ok && l0 + LPT <= p.level_end) {
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = v[i % (2 * LPT)];
        store8(dst, t);
    } else {
#pragma unroll
        for (int k = 0; k < LPT; ++k)
            if (l0 + k < p.level_end) reinterpret_cast<float2*>(dst)[k] = make_float2(v[2 * k], v[2 * k + 1]);
    }
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
template <int LPT>
__global__ void __launch_bounds__(kThreads, PERMUTO_MIN_BLOCKS) forward_kernel(const ForwardArgs a) {
    const Problem& p = a.p;
    const int64_t n = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (n >= p.n_points) return;
    const int pass_begin = p.level_begin + (int)blockIdx.y * p.levels_per_pass;
    const int pass_end = min(pass_begin + p.levels_per_pass, p.level_end);

    float pos[D];
    load_pos(p, n, pos);

#pragma unroll 1
    for (int l0 = pass_begin; l0 < pass_end; l0 += LPT) {
    float out[2 * LPT];
#pragma unroll
    for (int k = 0; k < LPT; ++k) {
        const int l = l0 + k;
        float ax = 0.f, ay = 0.f;
        if (l < pass_end) {  // uniform over the block
            const float w_lvl = __ldg(p.anneal + l);
            if (w_lvl != 0.0f) {  // a closed coarse-to-fine window contributes exact zeros
                Simplex<D> s;
                locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
                uint32_t slot[D + 1];
                to_slots(p, s, slot);
                const float* base = p.table + (size_t)l * p.capacity * 2u;
                float2 v[D + 1];
#pragma unroll
                for (int r = 0; r <= D; ++r) v[r] = gather2(base, slot[r]);
#pragma unroll
                for (int r = 0; r <= D; ++r) {
                    const float w = s.bary[r] * w_lvl;  // EncodingGPU.cuh:234
                    ax = fmaf(v[r].x, w, ax);
                    ay = fmaf(v[r].y, w, ay);
                }
            }
        }
        out[2 * k] = ax;
        out[2 * k + 1] = ay;
    }
    store_row_segment<LPT>(p, a.features, n, l0, out);
    }

    // raw points appended after the lattice levels (EncodingGPU.cuh:105-121)
    if (p.extra_levels > 0 && blockIdx.y == 0 && p.level_begin == 0) {
        float* dst = a.features + n * p.width + 2 * p.nr_levels;
        for (int c = 0; c < 2 * p.extra_levels; ++c) {
            float v = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) v = (c == i) ? pos[i] * p.points_scaling : v;
            dst[c] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------
// scatter-add of the d+1 table-gradient entries of one level, colliding lanes merged first
// ------------------------------------------------------------------------------------------
// On coarse levels the 32 points of a warp hit a handful of slots; sending 32 same-address
// reductions to L2 serialises there (2.0-3.6 ms per backward instead of 0.47 on the training
// shape).  match.any groups the lanes by slot, a pointer-jumping suffix sum over each group's
// lanes (log2 of the largest group rounds) leaves the group total in its lowest lane, and only
// that lane issues the vector reduction.  The summation order is fixed by the lane order, so a
// warp's contribution is deterministic.
__device__ __forceinline__ void merge_and_red(float* level_base, uint32_t slot, float x, float y, bool active,
                                              unsigned lane, unsigned group) {
    const int largest = __reduce_max_sync(kFullMask, __popc(group));
    const unsigned above = group & (0xfffffffeu << lane);
    int next = above ? (__ffs(above) - 1) : -1;
    for (int span = 1; span < largest; span <<= 1) {  // warp-uniform trip count
        const int src = next >= 0 ? next : (int)lane;
        const float x2 = __shfl_sync(kFullMask, x, src);
        const float y2 = __shfl_sync(kFullMask, y, src);
        const int n2 = __shfl_sync(kFullMask, next, src);
        if (next >= 0) {
            x += x2;
            y += y2;
            next = n2;
        }
    }
    const bool leader = (group & ((1u << lane) - 1u)) == 0u;
    if (leader && active) red_add2(level_base, slot, x, y);
}

// Merging pays only while a warp's 32 points share slots: per warp and vertex the number of
// distinct slots on the training shape is 6, 7, 9, 15, 22, 38, 63, 96, 116, 124 of 128 for levels
// 0..9 and 128 from level 11 on, and match.any itself is slowest when all keys differ.  The
// match of vertex 0 doubles as the probe: when it finds more than kMergeBelow distinct slots the
// level is scattered directly and -- collisions only get rarer towards finer levels -- the warp
// stops probing for the rest of its pass (`probe` is warp-uniform state owned by the caller).
#ifndef PERMUTO_MERGE_BELOW
#define PERMUTO_MERGE_BELOW 24
#endif
constexpr int kMergeBelow = PERMUTO_MERGE_BELOW;

__device__ __forceinline__ void scatter_level(float* level_base, const uint32_t (&slot)[D + 1], const float (&ax)[D + 1],
                                              const float (&ay)[D + 1], bool active, unsigned lane, bool& probe) {
    if (probe) {
        const uint32_t idle = 0xffffffffu - lane;  // idle lanes match nobody
        const unsigned group0 = __match_any_sync(kFullMask, active ? slot[0] : idle);
        const bool leader0 = (group0 & ((1u << lane) - 1u)) == 0u;
        const int distinct = __popc(__ballot_sync(kFullMask, leader0));
        if (distinct <= kMergeBelow) {
            merge_and_red(level_base, slot[0], ax[0], ay[0], active, lane, group0);
#pragma unroll
            for (int r = 1; r <= D; ++r) {
                const unsigned group = __match_any_sync(kFullMask, active ? slot[r] : idle);
                merge_and_red(level_base, slot[r], ax[r], ay[r], active, lane, group);
            }
            return;
        }
        probe = false;
    }
    if (active) {
#pragma unroll
        for (int r = 0; r <= D; ++r) red_add2(level_base, slot[r], ax[r], ay[r]);
    }
}

// ------------------------------------------------------------------------------------------
// first-order backward: table gradient (scatter) and/or position gradient (gather)
// ------------------------------------------------------------------------------------------
template <int LPT, bool TABLE, bool POS>
__global__ void __launch_bounds__(kThreads, (TABLE ? PERMUTO_MIN_BLOCKS : PERMUTO_MIN_BLOCKS_GATHER_ONLY)) backward_kernel(const BackwardArgs a) {
    const Problem& p = a.p;
    const int64_t n_raw = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = n_raw < p.n_points;
    const int64_t n = active ? n_raw : p.n_points - 1;  // idle lanes shadow the last point
    const int pass_begin = p.level_begin + (int)blockIdx.y * p.levels_per_pass;
    const int pass_end = min(pass_begin + p.levels_per_pass, p.level_end);
    const unsigned lane = threadIdx.x & 31u;
    constexpr float kInv = 1.0f / (D + 1);

    float pos[D];
    load_pos(p, n, pos);

    float dpos[D];
#pragma unroll
    for (int i = 0; i < D; ++i) dpos[i] = 0.f;
    bool probe = a.aggregate != 0;

    // the next group's 32 bytes of the gradient row are requested before this group is worked on
    float g_next[2 * LPT];
    load_row_segment<LPT>(p, a.grad_features, n, pass_begin, g_next);
#pragma unroll 1
    for (int l0 = pass_begin; l0 < pass_end; l0 += LPT) {
    float g[2 * LPT];
#pragma unroll
    for (int i = 0; i < 2 * LPT; ++i) g[i] = g_next[i];
    if (l0 + LPT < pass_end) load_row_segment<LPT>(p, a.grad_features, n, l0 + LPT, g_next);
#pragma unroll
    for (int k = 0; k < LPT; ++k) {
        const int l = l0 + k;
        if (l >= pass_end) continue;  // uniform
        const float w_lvl = __ldg(p.anneal + l);
        if (w_lvl == 0.0f) continue;  // every addend of this level is an exact zero
        Simplex<D> s;
        locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
        uint32_t slot[D + 1];
        to_slots(p, s, slot);
        const float gx = g[2 * k], gy = g[2 * k + 1];

        if (POS) {
            // EncodingGPU.cuh:671-749
            const float* base = p.table + (size_t)l * p.capacity * 2u;
            float dBs[D + 2];
            const float gxs = gx * w_lvl * kInv, gys = gy * w_lvl * kInv;  // level weight and 1/(d+1) folded in
#pragma unroll
            for (int r = 0; r <= D; ++r) {
                const float2 v = gather2(base, slot[r]);
                dBs[r] = fmaf(v.y, gys, v.x * gxs);
            }
            dBs[D + 1] = dBs[0];
            float T[D + 1];  // dE of the coordinate whose rank is k
#pragma unroll
            for (int kk = 0; kk <= D; ++kk) T[kk] = dBs[D - kk] - dBs[D + 1 - kk];
            float dE[D + 1];
#pragma unroll
            for (int i = 0; i <= D; ++i) {
                float v = 0.f;
#pragma unroll
                for (int kk = 0; kk <= D; ++kk) v = (s.rank[i] == kk) ? T[kk] : v;
                dE[i] = v;
            }
            float run = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) {
                run += dE[i];
                const float sc = __ldg(p.scale + l * D + i);
                dpos[i] += sc * (run - (float)(i + 1) * dE[i + 1]);
            }
        }

        if (TABLE) {
            float* gbase = a.lattice_grad + (size_t)l * p.capacity * 2u;
            float ax[D + 1], ay[D + 1];
            const float gxw = gx * w_lvl, gyw = gy * w_lvl;  // EncodingGPU.cuh:405-410
#pragma unroll
            for (int r = 0; r <= D; ++r) {
                ax[r] = s.bary[r] * gxw;
                ay[r] = s.bary[r] * gyw;
            }
            scatter_level(gbase, slot, ax, ay, active, lane, probe);
        }
    }
    }
    if (POS && active) {
        float* dst = a.positions_grad + n * D;
#pragma unroll
        for (int i = 0; i < D; ++i) red_add1(dst + i, dpos[i]);  // accumulates across level groups
    }
}

// ------------------------------------------------------------------------------------------
// double backward of the position gradient
// ------------------------------------------------------------------------------------------
template <int LPT, bool TABLE, bool GGF>
__global__ void __launch_bounds__(kThreads, PERMUTO_MIN_BLOCKS) double_backward_kernel(const DoubleBackwardArgs a) {
    const Problem& p = a.p;
    const int64_t n_raw = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = n_raw < p.n_points;
    const int64_t n = active ? n_raw : p.n_points - 1;
    const int pass_begin = p.level_begin + (int)blockIdx.y * p.levels_per_pass;
    const int pass_end = min(pass_begin + p.levels_per_pass, p.level_end);
    const unsigned lane = threadIdx.x & 31u;
    constexpr float kInv = 1.0f / (D + 1);

    float pos[D], dpg[D];
    load_pos(p, n, pos);
#pragma unroll
    for (int i = 0; i < D; ++i) dpg[i] = __ldg(a.double_positions_grad + n * D + i);
    bool probe = a.aggregate != 0;  // as in backward_kernel

    float g_next[2 * LPT];  // as in backward_kernel: the next group's gradient segment is requested early
    if (TABLE) load_row_segment<LPT>(p, a.grad_features, n, pass_begin, g_next);
#pragma unroll 1
    for (int l0 = pass_begin; l0 < pass_end; l0 += LPT) {
    float g[2 * LPT];
    if (TABLE) {
#pragma unroll
        for (int i = 0; i < 2 * LPT; ++i) g[i] = g_next[i];
        if (l0 + LPT < pass_end) load_row_segment<LPT>(p, a.grad_features, n, l0 + LPT, g_next);
    }
    float out[2 * LPT];
#pragma unroll
    for (int k = 0; k < LPT; ++k) {
        const int l = l0 + k;
        float ox = 0.f, oy = 0.f;
        if (l < pass_end) {
            const float w_lvl = __ldg(p.anneal + l);
            if (w_lvl != 0.0f) {
                Simplex<D> s;
                locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
                uint32_t slot[D + 1];
                to_slots(p, s, slot);

                // d loss / d elevated (EncodingGPU.cuh:1187-1199)
                float gs[D], dE[D + 1];
#pragma unroll
                for (int i = 0; i < D; ++i) gs[i] = dpg[i] * __ldg(p.scale + l * D + i);
#pragma unroll
                for (int j = 0; j <= D; ++j) dE[j] = 0.f;
#pragma unroll
                for (int i = 0; i < D; ++i) {
#pragma unroll
                    for (int j = 0; j <= i; ++j) dE[j] += gs[i];
                }
#pragma unroll
                for (int i = 0; i < D; ++i) dE[i + 1] -= gs[i] * (float)(i + 1);
                // d loss / d barycentric (EncodingGPU.cuh:1213-1218), via the rank-sorted vector
                float sdE[D + 1];
#pragma unroll
                for (int kk = 0; kk <= D; ++kk) {
                    float v = 0.f;
#pragma unroll
                    for (int i = 0; i <= D; ++i) v = (s.rank[i] == kk) ? dE[i] * kInv : v;
                    sdE[kk] = v;
                }
                float dB[D + 1];
#pragma unroll
                for (int m = 1; m <= D; ++m) dB[m] = sdE[D - m] - sdE[D + 1 - m];
                dB[0] = sdE[D] - sdE[0];

                if (GGF) {
                    const float* base = p.table + (size_t)l * p.capacity * 2u;
#pragma unroll
                    for (int r = 0; r <= D; ++r) {
                        const float2 v = gather2(base, slot[r]);
                        const float c = dB[r] * w_lvl;  // EncodingGPU.cuh:1484-1485
                        ox = fmaf(c, v.x, ox);
                        oy = fmaf(c, v.y, oy);
                    }
                }
                if (TABLE) {
                    float* gbase = a.lattice_grad + (size_t)l * p.capacity * 2u;
                    const float gx = g[2 * k], gy = g[2 * k + 1];
                    float ax[D + 1], ay[D + 1];
#pragma unroll
                    for (int r = 0; r <= D; ++r) {
                        const float c = dB[r] * w_lvl;  // EncodingGPU.cuh:1244-1245
                        ax[r] = c * gx;
                        ay[r] = c * gy;
                    }
                    scatter_level(gbase, slot, ax, ay, active, lane, probe);
                }
            }
        }
        out[2 * k] = ox;
        out[2 * k + 1] = oy;
    }
    if (GGF && active) store_row_segment<LPT>(p, a.grad_grad_features, n, l0, out);
    }
    if (GGF && active && p.extra_levels > 0 && blockIdx.y == 0 && p.level_begin == 0) {  // EncodingGPU.cuh:1290-1295
        float* dst = a.grad_grad_features + n * p.width + 2 * p.nr_levels;
        for (int c = 0; c < 2 * p.extra_levels; ++c) dst[c] = 0.f;
    }
}

// ------------------------------------------------------------------------------------------
// debug view: one thread per (point, level)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) debug_kernel(const DebugArgs a) {
    const Problem& p = a.p;
    const int64_t n = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (n >= p.n_points) return;
    const int l = blockIdx.y;
    float pos[D];
    load_pos(p, n, pos);
    Simplex<D> s;
    locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
    uint32_t slot[D + 1];
    to_slots(p, s, slot);
    const int64_t base = (n * p.nr_levels + l) * (D + 1);
#pragma unroll
    for (int r = 0; r <= D; ++r) {
        if (a.keys) {
            int key[D];
            vertex_key<D>(s, r, key);
#pragma unroll
            for (int i = 0; i < D; ++i) a.keys[(base + r) * D + i] = key[i];
        }
        if (a.slots) a.slots[base + r] = (int32_t)slot[r];
        if (a.bary) a.bary[base + r] = s.bary[r];
        if (a.rank) a.rank[base + r] = s.rank[r];
    }
}

// Levels handled by one thread in one sweep over the points.  A multiple of 4 (one 32-byte row
// segment per inner step).  More levels per pass means fewer sweeps -- each sweep re-reads the
// positions and touches only its own 32-byte pieces of every 128-byte line of the feature rows,
// which costs a 4x DRAM over-fetch on the gradient reads with one group per sweep -- but a larger
// set of table slices is live in L2 at once: capacity * 8 bytes per level for the values and as
// much again for their gradient.  Measured on B200 (pos_dim 3 and 4, capacities 2^18..2^20):
// scatter-only kernels are fastest with every level in one sweep even when the gradient table
// exceeds L2; gather kernels want about 96 MB live, gather+scatter kernels about 64 MB.
enum class Traffic { Gather, Scatter, Both };

inline int pick_levels_per_pass(const Problem& p, int requested, Traffic t) {
    const int levels = p.level_end - p.level_begin;
    int lpp = requested;
    if (lpp <= 0) {
        const double slice = 8.0 * p.capacity;
        const double mb = 1024.0 * 1024.0;
        if (t == Traffic::Scatter)
            lpp = levels;
        else if (t == Traffic::Gather)
            lpp = (int)(96.0 * mb / slice);
        else
            lpp = (int)(64.0 * mb / (2.0 * slice));
    }
    lpp = (lpp / 4) * 4;
    if (lpp < 4) lpp = 4;
    if (lpp > levels) lpp = ((levels + 3) / 4) * 4;
    return lpp;
}

inline dim3 grid_for(const Problem& p) {
    const unsigned gx = (unsigned)((p.n_points + kThreads - 1) / kThreads);
    const unsigned gy = (unsigned)((p.level_end - p.level_begin + p.levels_per_pass - 1) / p.levels_per_pass);
    return dim3(gx, gy, 1);
}

// small problems get one level per thread so that the grid still covers the machine
inline bool use_single_level(const Problem& p) {
    const int64_t groups4 = (p.level_end - p.level_begin + 3) / 4;
    const int64_t blocks4 = ((p.n_points + kThreads - 1) / kThreads) * groups4;
    return blocks4 < 2 * 148;
}

template <class Args>
inline Args with_schedule(const Args& in, bool single, Traffic t) {
    Args a = in;
    a.p.levels_per_pass = single ? 1 : pick_levels_per_pass(a.p, a.p.levels_per_pass, t);
    return a;
}

}  // namespace

#define PERMUTO_CAT_(a, b) a##b
#define PERMUTO_CAT(a, b) PERMUTO_CAT_(a, b)

cudaError_t PERMUTO_CAT(launch_forward_dim, PERMUTO_DIM)(const ForwardArgs& a0, cudaStream_t st) {
    const bool single = use_single_level(a0.p);
    const ForwardArgs a = with_schedule(a0, single, Traffic::Gather);
    if (single)
        forward_kernel<1><<<grid_for(a.p), kThreads, 0, st>>>(a);
    else
        forward_kernel<4><<<grid_for(a.p), kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

template <int LPT>
static cudaError_t launch_backward_lpt(const BackwardArgs& a0, cudaStream_t st) {
    const BackwardArgs a = with_schedule(
        a0, LPT == 1, (a0.lattice_grad && a0.positions_grad) ? Traffic::Both : (a0.lattice_grad ? Traffic::Scatter : Traffic::Gather));
    const dim3 g = grid_for(a.p);
    if (a.lattice_grad && a.positions_grad)
        backward_kernel<LPT, true, true><<<g, kThreads, 0, st>>>(a);
    else if (a.lattice_grad)
        backward_kernel<LPT, true, false><<<g, kThreads, 0, st>>>(a);
    else if (a.positions_grad)
        backward_kernel<LPT, false, true><<<g, kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t PERMUTO_CAT(launch_backward_dim, PERMUTO_DIM)(const BackwardArgs& a, cudaStream_t st) {
    return use_single_level(a.p) ? launch_backward_lpt<1>(a, st) : launch_backward_lpt<4>(a, st);
}

template <int LPT>
static cudaError_t launch_double_lpt(const DoubleBackwardArgs& a0, cudaStream_t st) {
    const DoubleBackwardArgs a = with_schedule(
        a0, LPT == 1,
        (a0.lattice_grad && a0.grad_grad_features) ? Traffic::Both : (a0.lattice_grad ? Traffic::Scatter : Traffic::Gather));
    const dim3 g = grid_for(a.p);
    if (a.lattice_grad && a.grad_grad_features)
        double_backward_kernel<LPT, true, true><<<g, kThreads, 0, st>>>(a);
    else if (a.lattice_grad)
        double_backward_kernel<LPT, true, false><<<g, kThreads, 0, st>>>(a);
    else if (a.grad_grad_features)
        double_backward_kernel<LPT, false, true><<<g, kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t PERMUTO_CAT(launch_double_backward_dim, PERMUTO_DIM)(const DoubleBackwardArgs& a, cudaStream_t st) {
    return use_single_level(a.p) ? launch_double_lpt<1>(a, st) : launch_double_lpt<4>(a, st);
}

cudaError_t PERMUTO_CAT(launch_debug_dim, PERMUTO_DIM)(const DebugArgs& a, cudaStream_t st) {
    const dim3 g((unsigned)((a.p.n_points + kThreads - 1) / kThreads), (unsigned)a.p.nr_levels, 1);
    debug_kernel<<<g, kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace permuto
