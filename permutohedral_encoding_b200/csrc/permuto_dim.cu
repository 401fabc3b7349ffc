// Lattice kernels for one pos_dim (compile with -DPERMUTO_DIM=2..7), sm_100a.
//
// Work decomposition shared by all kernels: one thread owns one point and walks levels in steps
// of LPS levels.  blockIdx.x walks point tiles, blockIdx.y walks passes of `levels_per_pass`
// levels, and blocks are dispatched x-fastest, so the whole grid sweeps the points once per
// pass: the slices of the value table (and of its gradient) that are live at any time are those
// of one pass, which stay L2-resident.  A step covers LPS = 8 / F levels of F features each,
// i.e. 8 consecutive floats of a feature row = one 32-byte sector, moved with a single 256-bit
// access (ld/st.global.v8.f32, new on sm_100), directly in the final [N, F*L] layout -- no
// transposed intermediate.  F = 2 is the reference's only supported width; F = 4 and 8 (which
// the reference lists as not yet implemented, Encoding.cuh:140-143) make every table access a
// 16- or 32-byte one, i.e. half or all of the sector the memory system moves anyway (measured on
// B200 over an L2-resident region: 16-byte random gathers run at three quarters of the rate of
// 8-byte ones, 16-byte vector reductions at the same rate as 8-byte ones; a 32-byte access is two
// 16-byte ones).
//
// What each kernel replaces in the reference (paths relative to its root):
//   forward_kernel          kernels/permutohedral_encoding/EncodingGPU.cuh:68-256
//   backward_kernel         EncodingGPU.cuh:259-414 (table) and :530-769 (positions), fused
//   double_backward_kernel  EncodingGPU.cuh:1016-1257 and :1260-1493, fused
#include <cuda_fp16.h>

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
// The forward kernel is bound by the LSU pipe, not by instruction-level parallelism: at 60
// registers (what a cap of 64 invites) it runs 4 % slower than at 32 with twice the resident warps.
#ifndef PERMUTO_MIN_BLOCKS_FORWARD
#define PERMUTO_MIN_BLOCKS_FORWARD (PERMUTO_DIM <= 3 ? 8 : (PERMUTO_DIM == 4 ? 6 : 4))
#endif
constexpr int kThreads = PERMUTO_THREADS;
// wider table entries keep more addends live per vertex: leave them more registers
constexpr int min_blocks(int feats, bool gather_only) {
    return feats == 8 ? 2
                      : (feats == 4 || D >= 6) ? 3
                                               : (gather_only ? PERMUTO_MIN_BLOCKS_GATHER_ONLY : PERMUTO_MIN_BLOCKS);
}
constexpr unsigned kFullMask = 0xffffffffu;

// A point's coordinates.  Rows of 2 or 4 contiguous floats on an aligned base are one 8- or
// 16-byte load (consecutive threads then read consecutive vectors); every other case -- odd
// pos_dim, strided or transposed positions -- takes one 4-byte load per coordinate, which for
// contiguous rows still touches each 128-byte line from a single warp instruction group.
__device__ __forceinline__ void load_pos(const Problem& p, int64_t n, float (&pos)[D]) {
    if ((D == 2 || D == 4) && p.pos_vec_ok) {
        if (D == 2) {
            const float2 t = __ldg(reinterpret_cast<const float2*>(p.positions) + n);
            pos[0] = t.x;
            pos[D - 1] = t.y;
        } else {
            const float4 t = __ldg(reinterpret_cast<const float4*>(p.positions) + n);
            pos[0] = t.x;
            pos[1 % D] = t.y;
            pos[2 % D] = t.z;
            pos[3 % D] = t.w;
        }
        return;
    }
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

// ---- F consecutive floats (one table entry, or one level of a feature row) ------------------
template <int F>
__device__ __forceinline__ void load_feats(const float* __restrict__ src, float (&v)[F]) {
    if (F == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(src));
        v[0] = t.x;
        v[1] = t.y;
    } else {
#pragma unroll
        for (int q = 0; q < F / 4; ++q) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(src) + q);
            v[4 * q + 0] = t.x;
            v[4 * q + 1] = t.y;
            v[4 * q + 2] = t.z;
            v[4 * q + 3] = t.w;
        }
    }
}
template <int F>
__device__ __forceinline__ void store_feats(float* dst, const float (&v)[F]) {
    if (F == 2) {
        *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1]);
    } else {
#pragma unroll
        for (int q = 0; q < F / 4; ++q)
            reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
}

// 8 consecutive floats of a feature row (or one 8-feature table entry), 32-byte aligned
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

// Aligned gather of one table entry (all F features) through the read-only path.  HALF: the
// table is stored as fp16 (storage only -- every product and sum below stays fp32), so an entry is
// 2F bytes: one 4-, 8- or 16-byte load.  Random accesses are bound by operations per second, not
// bytes, so a 4-feature fp16 entry (8 bytes) costs what a 2-feature fp32 entry costs, and the
// table takes half the room in L2.
template <int F, bool HALF>
__device__ __forceinline__ void gather(const void* __restrict__ table, int level, uint32_t capacity, uint32_t slot,
                                       float (&v)[F]) {
    const size_t entry = (size_t)level * capacity + slot;
    if (HALF) {
        const __half2* src = reinterpret_cast<const __half2*>(table) + entry * (F / 2);
        if (F == 2) {
            const unsigned raw = __ldg(reinterpret_cast<const unsigned*>(src));
            const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&raw));
            v[0] = t.x;
            v[1] = t.y;
        } else if (F == 4) {
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            v[0] = a.x;
            v[1] = a.y;
            v[2 % F] = b.x;
            v[3 % F] = b.y;
        } else {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
            const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                v[(2 * q) % F] = t.x;
                v[(2 * q + 1) % F] = t.y;
            }
        }
    } else {
        const float* src = reinterpret_cast<const float*>(table) + entry * F;
        if (F == 8) {
            asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=f"(v[0]), "=f"(v[1]), "=f"(v[2 % F]), "=f"(v[3 % F]), "=f"(v[4 % F]), "=f"(v[5 % F]),
                           "=f"(v[6 % F]), "=f"(v[7 % F])
                         : "l"(src));
        } else {
            load_feats<F>(src, v);
        }
    }
}

// vector reduction of one table-gradient entry: 8 bytes (F = 2) or 16 bytes (F = 4) per L2
// atomic -- both run at the same operation rate -- and two 16-byte ones for F = 8
template <int F>
__device__ __forceinline__ void red_add(float* level_base, uint32_t slot, const float (&x)[F]) {
    float* p = level_base + (size_t)slot * F;
    if (F == 2) {
        asm volatile("red.relaxed.gpu.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(x[0]), "f"(x[1]) : "memory");
    } else {
#pragma unroll
        for (int q = 0; q < F / 4; ++q)
            asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4 * q), "f"(x[4 * q]),
                         "f"(x[4 * q + 1]), "f"(x[4 * q + 2]), "f"(x[4 * q + 3])
                         : "memory");
    }
}

// Row segment of point n starting at level l0: LPS levels of F floats.  One 32-byte vector access
// when the segment is a whole, aligned 8-float group; else per-level accesses.
template <int F, int LPS>
__device__ __forceinline__ void load_row_segment(const Problem& p, const float* rows, int64_t n, int l0,
                                                 float (&v)[F * LPS]) {
    const float* src = rows + n * p.width + F * l0;
    if (F * LPS == 8 && p.rows_vec8_ok && l0 + LPS <= p.level_end) {
        load8(src, reinterpret_cast<float(&)[8]>(v));
    } else {
#pragma unroll
        for (int k = 0; k < LPS; ++k) {
            float t[F];
#pragma unroll
            for (int f = 0; f < F; ++f) t[f] = 0.f;
            if (l0 + k < p.level_end) load_feats<F>(src + F * k, t);
#pragma unroll
            for (int f = 0; f < F; ++f) v[F * k + f] = t[f];
        }
    }
}
template <int F, int LPS>
__device__ __forceinline__ void store_row_segment(const Problem& p, float* rows, int64_t n, int l0,
                                                  const float (&v)[F * LPS]) {
    float* dst = rows + n * p.width + F * l0;
    if (F * LPS == 8 && p.rows_vec8_ok && l0 + LPS <= p.level_end) {
        store8(dst, reinterpret_cast<const float(&)[8]>(v));
    } else {
#pragma unroll
        for (int k = 0; k < LPS; ++k) {
            if (l0 + k < p.level_end) {
                float t[F];
#pragma unroll
                for (int f = 0; f < F; ++f) t[f] = v[F * k + f];
                store_feats<F>(dst + F * k, t);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
// One step of a point's feature row: LPS levels of F features (8 floats) starting at level l0;
// levels at or beyond `end` give zeros (EncodingGPU.cuh:130-254 for one level).
template <int F, int LPS, bool HALF>
__device__ __forceinline__ void encode_step(const Problem& p, const float (&pos)[D], int l0, int end,
                                            float (&out)[F * LPS]) {
#pragma unroll
    for (int k = 0; k < LPS; ++k) {
        const int l = l0 + k;
        float acc[F];
#pragma unroll
        for (int f = 0; f < F; ++f) acc[f] = 0.f;
        if (l < end) {  // uniform over the block
            const float w_lvl = __ldg(p.anneal + l);
            if (w_lvl != 0.0f) {  // a closed coarse-to-fine window contributes exact zeros
                Simplex<D> s;
                locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
                uint32_t slot[D + 1];
                to_slots(p, s, slot);
                float v[D + 1][F];
#pragma unroll
                for (int r = 0; r <= D; ++r) gather<F, HALF>(p.table, l, p.capacity, slot[r], v[r]);
#pragma unroll
                for (int r = 0; r <= D; ++r) {
                    const float w = s.bary[r] * w_lvl;  // EncodingGPU.cuh:234
#pragma unroll
                    for (int f = 0; f < F; ++f) acc[f] = fmaf(v[r][f], w, acc[f]);
                }
            }
        }
#pragma unroll
        for (int f = 0; f < F; ++f) out[F * k + f] = acc[f];
    }
}

template <int F, int LPS, bool HALF>
__global__ void __launch_bounds__(kThreads, (F == 2 ? PERMUTO_MIN_BLOCKS_FORWARD : min_blocks(F, false))) forward_kernel(const ForwardArgs a) {
    const Problem& p = a.p;
    const int64_t n = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (n >= p.n_points) return;
    const int pass_begin = p.level_begin + (int)blockIdx.y * p.levels_per_pass;
    const int pass_end = min(pass_begin + p.levels_per_pass, p.level_end);

    float pos[D];
    load_pos(p, n, pos);

#pragma unroll 1
    for (int l0 = pass_begin; l0 < pass_end; l0 += LPS) {
        float out[F * LPS];
        encode_step<F, LPS, HALF>(p, pos, l0, pass_end, out);
        store_row_segment<F, LPS>(p, a.features, n, l0, out);
    }

    // raw points appended after the lattice levels (EncodingGPU.cuh:105-121)
    if (p.extra_levels > 0 && blockIdx.y == 0 && p.level_begin == 0) {
        float* dst = a.features + n * p.width + F * p.nr_levels;
        for (int c = 0; c < F * p.extra_levels; ++c) {
            float v = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) v = (c == i) ? pos[i] * p.points_scaling : v;
            dst[c] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------
// forward fused with the consumer's first linear layer (tcgen05 + TMEM)
// ------------------------------------------------------------------------------------------
// The users of the encoding feed the [N, F*L] feature row straight into a small MLP (reference:
// examples/train_toy_example.py:18-26, README.md:39-40).  Here a block of 128 threads encodes 128
// points, passes the 128 x K feature tile (K = F*(L+extra), rounded to tf32) through shared memory
// 8 columns at a time and multiplies it by the layer's weight [H, K] on the tensor cores: K/8
// tcgen05.mma of shape 128 x H x 8 (kind::tf32, fp32 accumulate) issued by one thread, accumulator
// in tensor memory, read back with tcgen05.ld (thread t holds row t) and written as [N, H] with
// the bias added.  The 192 B/point feature row and the separate GEMM's read of it never touch HBM.
//
// Shared-memory operand layout (K-major, no swizzle -- the canonical layout of the tcgen05
// matrix descriptor): 8 rows x 16 bytes form a contiguous 128-byte core matrix; the core
// matrices of consecutive 4-column groups follow each other (leading byte offset 128) and those
// of consecutive 8-row groups are a fixed number of bytes apart (stride byte offset).
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 64-bit shared-memory matrix descriptor: start address, leading / stride byte offsets (all in
// units of 16 bytes), descriptor version 1 (Blackwell), no swizzle
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(leading_bytes >> 4) << 16) |
           ((uint64_t)(stride_bytes >> 4) << 32) | (1ull << 46);
}

// 32-bit instruction descriptor for kind::tf32: D = fp32 (bits 4-5 = 1), A and B = tf32 (bits 7-9
// and 10-12 = 2), both K-major (bits 15, 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24
__device__ __forceinline__ uint32_t instr_desc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}

// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread is done
__device__ __forceinline__ void commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}

// Bounded wait for phase `parity` of an mbarrier: false when the limit ran out (the caller then
// reports it and skips its output instead of spinning for ever).
__device__ __forceinline__ bool wait_bounded(uint32_t mbar, uint32_t parity) {
    for (int it = 0; it < (1 << 20); ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

}  // namespace umma

constexpr int kTileRows = 128;  // points per block = rows of one tcgen05.mma
#ifndef PERMUTO_FUSED_RING
#define PERMUTO_FUSED_RING 2
#endif
constexpr int kRing = PERMUTO_FUSED_RING;  // 128 x 8 slices in flight between the threads and the tensor core
constexpr uint32_t kSliceBytes = kTileRows * 8 * 4;  // one slice: 128 rows x 8 tf32 = 4 KB

// The A operand of every product is never whole in shared memory: 8 columns of the 128-row tile
// (a K = 8 slice of the product) are written into a ring of kRing slices and consumed by one
// tcgen05.mma right away, accumulating in tensor memory.  That keeps a block at 8 KB + the
// weights instead of 128 x K x 4 bytes, so that shared memory neither limits the resident blocks
// nor eats the L1 capacity the coarse levels' gathers live on.
struct SliceRing {
    unsigned char* base;   // kRing slices
    uint64_t* free_bar;    // one mbarrier per slice: arrives when the MMA that read it is done
    uint32_t base_addr;
    uint32_t row_off;      // this thread's row inside a slice
    int pushed;            // slices written so far (all layers)
    bool ok;               // no bounded wait has run out

    // Write this thread's 8 values of the next slice; when the whole block has, thread 0 issues
    // D[128 x n] (+)= slice[128 x 8] * B[n x 8]^T and commits to the slice's barrier.
    // Block-uniform control flow: every thread of the block calls it.
    __device__ __forceinline__ void push(const float (&v)[8], uint32_t tmem_d, uint32_t b_addr, uint32_t b_stride,
                                         uint32_t idesc, bool accumulate) {
        const int slot = pushed % kRing;
        // the MMA that read this slice kRing pushes ago must be done before it is overwritten
        if (pushed >= kRing) ok = umma::wait_bounded(umma::smem_u32(&free_bar[slot]), (uint32_t)((pushed / kRing - 1) & 1)) && ok;
        unsigned char* dst = base + (size_t)slot * kSliceBytes + row_off;
        *reinterpret_cast<float4*>(dst) =
            make_float4(umma::to_tf32(v[0]), umma::to_tf32(v[1]), umma::to_tf32(v[2]), umma::to_tf32(v[3]));
        *reinterpret_cast<float4*>(dst + 128) =
            make_float4(umma::to_tf32(v[4]), umma::to_tf32(v[5]), umma::to_tf32(v[6]), umma::to_tf32(v[7]));
        // the block's writes -> visible to the tensor core (async proxy); then one thread issues the slice's MMA
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            umma::mma_tf32(tmem_d, umma::smem_desc(base_addr + (uint32_t)slot * kSliceBytes, 128u, 256u),
                           umma::smem_desc(b_addr, 128u, b_stride), idesc, accumulate);
            umma::commit(umma::smem_u32(&free_bar[slot]));  // covers every MMA issued so far
        }
        ++pushed;
    }

    // Wait until every MMA issued so far is done (the last commit covers them all); the result is
    // made block-uniform, because tcgen05.ld afterwards must be executed by whole warps.
    __device__ __forceinline__ bool drain() {
        const int last = pushed - 1;
        ok = umma::wait_bounded(umma::smem_u32(&free_bar[last % kRing]), (uint32_t)((last / kRing) & 1)) && ok;
        ok = __syncthreads_and(ok) != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        return ok;
    }
};

// weight [rows, cols] row-major in global memory -> shared memory in the K-major operand layout
// with `chunks` 16-byte column groups per row, rounded to tf32; columns beyond `cols` are zero
__device__ __forceinline__ void stage_weight(unsigned char* tile, const float* __restrict__ weight, int rows, int cols,
                                             int chunks) {
    const uint32_t stride = (uint32_t)chunks * 128u;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(weight) & 15u) == 0);
    for (int e = threadIdx.x; e < rows * chunks; e += kTileRows) {
        const int n = e / chunks, kc = e - n * chunks;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = weight + (size_t)n * cols + 4 * kc;
        if (vec && 4 * kc + 3 < cols) {
            w = __ldg(reinterpret_cast<const float4*>(src));
        } else {
            if (4 * kc + 0 < cols) w.x = __ldg(src + 0);
            if (4 * kc + 1 < cols) w.y = __ldg(src + 1);
            if (4 * kc + 2 < cols) w.z = __ldg(src + 2);
            if (4 * kc + 3 < cols) w.w = __ldg(src + 3);
        }
        *reinterpret_cast<float4*>(tile + (size_t)(n >> 3) * stride + (size_t)kc * 128 + (n & 7) * 16) =
            make_float4(umma::to_tf32(w.x), umma::to_tf32(w.y), umma::to_tf32(w.z), umma::to_tf32(w.w));
    }
}

// 16 consecutive accumulator columns of this thread's row (tensor-memory lane = row)
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));  // all 32 lanes of the warp take part
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// erf to 1.5e-7 absolute (Abramowitz & Stegun 7.1.26) in about 15 instructions: the hidden
// activations are rounded to tf32 (5e-4 relative) right afterwards, and erff() itself would be
// most of the instructions of a hidden layer
__device__ __forceinline__ float erf_fast(float x) {
    const float ax = fabsf(x);
    const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.0f));
    const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
    return copysignf(1.0f - poly * __expf(-ax * ax), x);
}

__device__ __forceinline__ float activate(float x, int kind) {
    if (kind == PERMUTO_ACT_RELU) return fmaxf(x, 0.f);
    if (kind == PERMUTO_ACT_GELU) return 0.5f * x * (1.0f + erf_fast(x * 0.70710678118654752f));  // torch.nn.GELU()
    return x;
}

#ifndef PERMUTO_FUSED_MIN_BLOCKS
#define PERMUTO_FUSED_MIN_BLOCKS 8
#endif
// HMAX = 0: the encoding followed by ONE linear layer (out = features @ W^T + b).
// HMAX = 32 / 64: a whole small MLP behind the encoding; hidden widths are multiples of 16 up to
// HMAX (a thread holds its row of hidden activations in registers between two layers).
template <int F, int LPS, bool HALF, int HMAX>
__global__ void __launch_bounds__(kTileRows, (F == 2 && HMAX <= 32 ? PERMUTO_FUSED_MIN_BLOCKS : 4))
forward_mlp_kernel(const ForwardLinearArgs a) {
    const Problem& p = a.p;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t slice_free[kRing];
    __shared__ uint32_t tmem_base;

    const int t = threadIdx.x;
    const int warp = t >> 5;
    const int H0 = a.layer[0].out_features;
    const uint32_t tmem_cols = (uint32_t)a.tmem_cols;  // a power of two >= 32 (host-computed)

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(umma::smem_u32(&tmem_base)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (t == 0) {
#pragma unroll
        for (int i = 0; i < kRing; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(umma::smem_u32(&slice_free[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    // shared memory: the slice ring, then the weight of every layer that runs on the tensor core
    unsigned char* tile_w = smem_raw + kRing * kSliceBytes;
    const int chunks0 = a.k_pad / 4;
    stage_weight(tile_w, a.layer[0].weight, H0, p.width, chunks0);
    if (HMAX > 0) {
        unsigned char* next = tile_w + (size_t)H0 * a.k_pad * 4;
        for (int i = 1; i < a.nr_layers; ++i) {
            const MlpLayer& ly = a.layer[i];
            if (ly.out_features % 16 != 0) break;  // a narrow last layer is evaluated in registers
            stage_weight(next, ly.weight, ly.out_features, ly.in_features, ly.in_features / 4);
            next += (size_t)ly.out_features * ly.in_features * 4;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base;

    SliceRing ring;
    ring.base = smem_raw;
    ring.free_bar = slice_free;
    ring.base_addr = umma::smem_u32(smem_raw);
    ring.row_off = (uint32_t)(t >> 3) * 256u + (uint32_t)(t & 7) * 16u;  // 8-row groups 256 bytes apart
    ring.pushed = 0;
    ring.ok = true;

    // ---- layer 0: this thread's point -> row t of every slice ----------------------------------
    const int64_t n_raw = (int64_t)blockIdx.x * kTileRows + t;
    const bool active = n_raw < p.n_points;
    const int64_t n = active ? n_raw : p.n_points - 1;  // idle rows shadow the last point and are not stored
    {
        float pos[D];
        load_pos(p, n, pos);
        const int lattice_cols = F * p.nr_levels;
        // a column past the lattice levels: a concatenated raw coordinate (EncodingGPU.cuh:105-121) or padding
        auto tail_value = [&](int c) -> float {
            float v = 0.f;
            const int i = c - lattice_cols;
#pragma unroll
            for (int j = 0; j < D; ++j) v = (i == j && c < p.width) ? pos[j] * p.points_scaling : v;
            return v;
        };
        const int nsteps = (p.nr_levels + LPS - 1) / LPS;  // steps that hold lattice levels
        const int ksteps = a.k_pad / 8;                    // all steps: one tcgen05.mma each
        const uint32_t idesc = umma::instr_desc_tf32(kTileRows, H0);
        const uint32_t addr_w = umma::smem_u32(tile_w);
#pragma unroll 1
        for (int s = 0; s < ksteps; ++s) {
            float out[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = 0.f;
            if (s < nsteps) encode_step<F, LPS, HALF>(p, pos, s * LPS, p.nr_levels, out);
            if (8 * s + 8 > lattice_cols) {  // block-uniform: only the last step(s) reach past the lattice levels
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int c = 8 * s + i;
                    out[i] = (c >= lattice_cols) ? tail_value(c) : out[i];
                }
            }
            ring.push(out, tmem, addr_w + (uint32_t)s * 256u, (uint32_t)chunks0 * 128u, idesc, s > 0);
        }
    }

    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);  // tensor-memory lane = 32*warp + lane = row t
    bool ok = true;
    int last = 0;          // layer whose accumulators are in tensor memory
    uint32_t col = 0;      // ... starting at this column

    // ---- hidden layers: accumulators -> registers (+bias, activation) -> slices -> next product ----
    if (HMAX > 0) {
        constexpr int HM = HMAX > 0 ? HMAX : 16;
        uint32_t w_addr = umma::smem_u32(tile_w) + (uint32_t)H0 * (uint32_t)a.k_pad * 4u;
        for (int i = 1; i < a.nr_layers; ++i) {
            const MlpLayer& ly = a.layer[i];
            const int width = ly.in_features;  // = out_features of layer i-1, a multiple of 16 up to HMAX
            ok = ring.drain() && ok;
            float h[HM];
            const float* bias = a.layer[i - 1].bias;
            const int kind = a.activation;
#pragma unroll
            for (int c = 0; c < HM / 16; ++c) {
                if (16 * c < width) {
                    float v[16];
                    tmem_load16(lane_base + col + 16u * c, v);
                    if (bias) {  // 64-byte aligned groups of a tensor allocated by the caller: vector loads when possible
#pragma unroll
                        for (int k = 0; k < 16; ++k) v[k] += __ldg(bias + 16 * c + k);
                    }
                    // one uniform branch per group, not one per element
                    if (kind == PERMUTO_ACT_GELU) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) h[16 * c + k] = activate(v[k], PERMUTO_ACT_GELU);
                    } else if (kind == PERMUTO_ACT_RELU) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) h[16 * c + k] = fmaxf(v[k], 0.f);
                    } else {
#pragma unroll
                        for (int k = 0; k < 16; ++k) h[16 * c + k] = v[k];
                    }
                }
            }
            if (ly.out_features % 16 != 0) {
                // narrow last layer (e.g. one output): plain fp32 dot products in registers
                if (active && ok) {
                    for (int o = 0; o < ly.out_features; ++o) {
                        float acc = ly.bias ? __ldg(ly.bias + o) : 0.f;
                        const float* w = ly.weight + (size_t)o * width;
#pragma unroll
                        for (int k = 0; k < HM; ++k)
                            if (k < width) acc = fmaf(h[k], __ldg(w + k), acc);
                        a.out[n_raw * ly.out_features + o] = acc;
                    }
                }
                last = -1;  // everything is written
                break;
            }
            const uint32_t dst_col = col ^ (uint32_t)a.tmem_half;  // ping-pong between the two halves
            const uint32_t idesc = umma::instr_desc_tf32(kTileRows, ly.out_features);
#pragma unroll
            for (int j = 0; j < HM / 8; ++j) {
                if (8 * j < width) {
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = h[8 * j + k];
                    ring.push(v, tmem + dst_col, w_addr + (uint32_t)j * 256u, (uint32_t)(width / 4) * 128u, idesc, j > 0);
                }
            }
            w_addr += (uint32_t)ly.out_features * (uint32_t)width * 4u;
            col = dst_col;
            last = i;
        }
    }

    // ---- last tensor-core layer: accumulators + bias -> out[N, out_features] -------------------------
    if (last >= 0) {
        ok = ring.drain() && ok;
        const int H = a.layer[last].out_features;
        const float* bias = a.layer[last].bias;
        if (ok) {
            float* dst = a.out + n_raw * H;
            for (int c = 0; c < H; c += 16) {
                float v[16];
                tmem_load16(lane_base + col + (uint32_t)c, v);
                if (active) {
#pragma unroll
                    for (int h8 = 0; h8 < 2; ++h8) {
                        float o[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) o[k] = v[8 * h8 + k] + (bias ? __ldg(bias + c + 8 * h8 + k) : 0.f);
                        if (a.out_vec8_ok) {
                            store8(dst + c + 8 * h8, o);
                        } else {
                            reinterpret_cast<float4*>(dst + c + 8 * h8)[0] = make_float4(o[0], o[1], o[2], o[3]);
                            reinterpret_cast<float4*>(dst + c + 8 * h8)[1] = make_float4(o[4], o[5], o[6], o[7]);
                        }
                    }
                }
            }
        }
    }
    if (!ok && a.status && t == 0) atomicExch(a.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
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
//
// The d+1 vertices are merged together, round by round, not one after the other: a round is a
// chain match/shuffle -> add -> shuffle whose latency nothing else in the warp can hide, and the
// d+1 chains are independent of each other.  (With the vertices merged one after the other the
// coarse half of the levels took as long as the fine half, although it sends a quarter of the
// reductions to L2.)
//
// Merging pays only while a warp's 32 points share slots: per warp and vertex the number of
// distinct slots on the training shape is 6, 7, 9, 15, 22, 38, 63, 96, 116, 124 of 128 for levels
// 0..9 and 128 from level 11 on, and match.any itself is slowest when all keys differ.  The
// match of vertex 0 doubles as the probe: when it finds more than kMergeBelow distinct slots the
// level is scattered directly and -- collisions only get rarer towards finer levels -- the warp
// stops probing until its walk over the levels restarts at the coarsest one.
//
// Blocks start their walk over the steps of a pass at different steps (block index modulo the
// number of steps), so that at any moment the blocks in flight work on different levels instead
// of all sending their reductions to the few hot slots of the same coarse level (2-4 % on the
// scatter kernels).
#ifndef PERMUTO_MERGE_BELOW
#define PERMUTO_MERGE_BELOW 24
#endif
#ifndef PERMUTO_STAGGER
#define PERMUTO_STAGGER 1
#endif
constexpr int kMergeBelow = PERMUTO_MERGE_BELOW;
constexpr bool kStagger = PERMUTO_STAGGER != 0;

// per-thread state of the scatter of one warp
struct Scatter {
    unsigned lane;
    bool active;  // this lane owns a point
    bool probe;   // warp-uniform: keep testing levels for mergeable collisions
};

// Vertices merged side by side: all of them up to pos_dim 4; beyond that half at a time, which
// keeps the d+1 partial sums, group masks and chain pointers within the register budget.
#ifndef PERMUTO_MERGE_CHUNK
#define PERMUTO_MERGE_CHUNK (PERMUTO_DIM <= 4 ? PERMUTO_DIM + 1 : (PERMUTO_DIM + 2) / 2)
#endif
constexpr int kMergeChunk = PERMUTO_MERGE_CHUNK;

// vertices [R0, R0 + CNT) of one level: segmented suffix sums over the lanes of every group,
// then one reduction per group from its lowest lane.  group[0] is passed in when R0 == 0.
template <int F, int R0, int CNT>
__device__ __forceinline__ void merge_vertices(const Scatter& sc, float* level_base, const uint32_t (&slot)[D + 1],
                                               float (&add)[D + 1][F], unsigned group0) {
    const unsigned lane = sc.lane;
    const uint32_t idle = 0xffffffffu - lane;  // idle lanes match nobody
    const unsigned below = (1u << lane) - 1u;
    unsigned group[CNT];
    int next[CNT];  // next higher lane of the same group, -1 at the end of the chain
    int largest = 0;
#pragma unroll
    for (int c = 0; c < CNT; ++c) {
        group[c] = (R0 == 0 && c == 0) ? group0 : __match_any_sync(kFullMask, sc.active ? slot[R0 + c] : idle);
        largest = max(largest, __popc(group[c]));
        const unsigned above = group[c] & (0xfffffffeu << lane);
        next[c] = above ? (__ffs(above) - 1) : -1;
    }
    largest = __reduce_max_sync(kFullMask, largest);
    for (int span = 1; span < largest; span <<= 1) {  // warp-uniform trip count
#pragma unroll
        for (int c = 0; c < CNT; ++c) {
            const int src = next[c] >= 0 ? next[c] : (int)lane;
            float x2[F];
#pragma unroll
            for (int f = 0; f < F; ++f) x2[f] = __shfl_sync(kFullMask, add[R0 + c][f], src);
            const int n2 = __shfl_sync(kFullMask, next[c], src);
            if (next[c] >= 0) {
#pragma unroll
                for (int f = 0; f < F; ++f) add[R0 + c][f] += x2[f];
                next[c] = n2;
            }
        }
    }
    if (sc.active) {
#pragma unroll
        for (int c = 0; c < CNT; ++c)
            if ((group[c] & below) == 0u) red_add<F>(level_base, slot[R0 + c], add[R0 + c]);
    }
}

template <int F, int R0>
__device__ __forceinline__ void merge_from(const Scatter& sc, float* level_base, const uint32_t (&slot)[D + 1],
                                           float (&add)[D + 1][F], unsigned group0) {
    if constexpr (R0 <= D) {
        constexpr int CNT = (D + 1 - R0) < kMergeChunk ? (D + 1 - R0) : kMergeChunk;
        merge_vertices<F, R0, CNT>(sc, level_base, slot, add, group0);
        merge_from<F, R0 + CNT>(sc, level_base, slot, add, group0);
    }
}

template <int F>
__device__ __forceinline__ void scatter_level(Scatter& sc, float* level_base, const uint32_t (&slot)[D + 1],
                                              float (&add)[D + 1][F]) {
    if (sc.probe) {
        const unsigned lane = sc.lane;
        const unsigned group0 = __match_any_sync(kFullMask, sc.active ? slot[0] : 0xffffffffu - lane);
        const int distinct = __popc(__ballot_sync(kFullMask, (group0 & ((1u << lane) - 1u)) == 0u));
        if (distinct <= kMergeBelow) {
            merge_from<F, 0>(sc, level_base, slot, add, group0);
            return;
        }
        sc.probe = false;
    }
    if (sc.active) {
#pragma unroll
        for (int r = 0; r <= D; ++r) red_add<F>(level_base, slot[r], add[r]);
    }
}

// ------------------------------------------------------------------------------------------
// first-order backward: table gradient (scatter) and/or position gradient (gather)
// ------------------------------------------------------------------------------------------
template <int F, int LPS, bool TABLE, bool POS, bool HALF>
__global__ void __launch_bounds__(kThreads, min_blocks(F, !TABLE))
backward_kernel(const BackwardArgs a) {
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
    Scatter sc{lane, active, a.aggregate != 0};

    // steps of the pass are walked cyclically from a block-dependent start (see PERMUTO_STAGGER)
    const int nsteps = (pass_end - pass_begin + LPS - 1) / LPS;
    int step = (TABLE && kStagger) ? (int)(blockIdx.x % (unsigned)nsteps) : 0;

    // the next step's 32 bytes of the gradient row are requested before this step is worked on
    float g_next[F * LPS];
    load_row_segment<F, LPS>(p, a.grad_features, n, pass_begin + step * LPS, g_next);
#pragma unroll 1
    for (int it = 0; it < nsteps; ++it) {
        const int l0 = pass_begin + step * LPS;
        step = (step + 1 == nsteps) ? 0 : step + 1;
        if (TABLE && l0 == pass_begin) sc.probe = a.aggregate != 0;
        float g[F * LPS];
#pragma unroll
        for (int i = 0; i < F * LPS; ++i) g[i] = g_next[i];
        if (it + 1 < nsteps) load_row_segment<F, LPS>(p, a.grad_features, n, pass_begin + step * LPS, g_next);
#pragma unroll
        for (int k = 0; k < LPS; ++k) {
            const int l = l0 + k;
            if (l >= pass_end) continue;  // uniform
            const float w_lvl = __ldg(p.anneal + l);
            if (w_lvl == 0.0f) continue;  // every addend of this level is an exact zero
            Simplex<D> s;
            locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
            uint32_t slot[D + 1];
            to_slots(p, s, slot);

            if (POS) {
                // EncodingGPU.cuh:671-749
                float gs[F];  // upstream gradient with the level weight and 1/(d+1) folded in
#pragma unroll
                for (int f = 0; f < F; ++f) gs[f] = g[F * k + f] * w_lvl * kInv;
                float dBs[D + 2];
#pragma unroll
                for (int r = 0; r <= D; ++r) {
                    float v[F];
                    gather<F, HALF>(p.table, l, p.capacity, slot[r], v);
                    float t = v[0] * gs[0];
#pragma unroll
                    for (int f = 1; f < F; ++f) t = fmaf(v[f], gs[f], t);
                    dBs[r] = t;
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
                float* gbase = a.lattice_grad + (size_t)l * p.capacity * F;
                float gw[F];  // EncodingGPU.cuh:405-410
#pragma unroll
                for (int f = 0; f < F; ++f) gw[f] = g[F * k + f] * w_lvl;
                float add[D + 1][F];
#pragma unroll
                for (int r = 0; r <= D; ++r) {
#pragma unroll
                    for (int f = 0; f < F; ++f) add[r][f] = s.bary[r] * gw[f];
                }
                scatter_level<F>(sc, gbase, slot, add);
            }
        }
    }
    // Optional: the concatenated raw coordinates are outputs too, d out[F*L + i] / d pos[i] =
    // points_scaling.  The reference leaves this term out (its backward grids exclude the extra
    // levels, src/Encoding.cu:129-134,161), so it is added only on request.
    if (POS && a.concat_grad && p.extra_levels > 0 && blockIdx.y == 0 && p.level_begin == 0) {
        const float* g = a.grad_features + n * p.width + F * p.nr_levels;
#pragma unroll
        for (int i = 0; i < D; ++i) dpos[i] = fmaf(__ldg(g + i), p.points_scaling, dpos[i]);
    }
    if (POS && active) {
        float* dst = a.positions_grad + n * D;
#pragma unroll
        for (int i = 0; i < D; ++i) red_add1(dst + i, dpos[i]);  // accumulates across passes
    }
}

// ------------------------------------------------------------------------------------------
// double backward of the position gradient
// ------------------------------------------------------------------------------------------
template <int F, int LPS, bool TABLE, bool GGF, bool HALF>
__global__ void __launch_bounds__(kThreads, min_blocks(F, false)) double_backward_kernel(const DoubleBackwardArgs a) {
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
    Scatter sc{lane, active, a.aggregate != 0};  // as in backward_kernel
    const int nsteps = (pass_end - pass_begin + LPS - 1) / LPS;
    int step = (TABLE && kStagger) ? (int)(blockIdx.x % (unsigned)nsteps) : 0;

    float g_next[F * LPS];  // as in backward_kernel: the next step's gradient segment is requested early
    if (TABLE) load_row_segment<F, LPS>(p, a.grad_features, n, pass_begin + step * LPS, g_next);
#pragma unroll 1
    for (int it = 0; it < nsteps; ++it) {
        const int l0 = pass_begin + step * LPS;
        step = (step + 1 == nsteps) ? 0 : step + 1;
        if (TABLE && l0 == pass_begin) sc.probe = a.aggregate != 0;
        float g[F * LPS];
        if (TABLE) {
#pragma unroll
            for (int i = 0; i < F * LPS; ++i) g[i] = g_next[i];
            if (it + 1 < nsteps) load_row_segment<F, LPS>(p, a.grad_features, n, pass_begin + step * LPS, g_next);
        }
        float out[F * LPS];
#pragma unroll
        for (int k = 0; k < LPS; ++k) {
            const int l = l0 + k;
            float o[F];
#pragma unroll
            for (int f = 0; f < F; ++f) o[f] = 0.f;
            if (l < pass_end) {
                const float w_lvl = __ldg(p.anneal + l);
                if (w_lvl != 0.0f) {
                    Simplex<D> s;
                    locate_simplex<D>(pos, p.shift + l * D, p.scale + l * D, s);
                    uint32_t slot[D + 1];
                    to_slots(p, s, slot);

                    // d loss / d elevated (EncodingGPU.cuh:1187-1199)
                    float gsd[D], dE[D + 1];
#pragma unroll
                    for (int i = 0; i < D; ++i) gsd[i] = dpg[i] * __ldg(p.scale + l * D + i);
#pragma unroll
                    for (int j = 0; j <= D; ++j) dE[j] = 0.f;
#pragma unroll
                    for (int i = 0; i < D; ++i) {
#pragma unroll
                        for (int j = 0; j <= i; ++j) dE[j] += gsd[i];
                    }
#pragma unroll
                    for (int i = 0; i < D; ++i) dE[i + 1] -= gsd[i] * (float)(i + 1);
                    // d loss / d barycentric (EncodingGPU.cuh:1213-1218), via the rank-sorted vector
                    float sdE[D + 1];
#pragma unroll
                    for (int kk = 0; kk <= D; ++kk) {
                        float v = 0.f;
#pragma unroll
                        for (int i = 0; i <= D; ++i) v = (s.rank[i] == kk) ? dE[i] * kInv : v;
                        sdE[kk] = v;
                    }
                    float dBw[D + 1];  // dB * level weight
#pragma unroll
                    for (int m = 1; m <= D; ++m) dBw[m] = (sdE[D - m] - sdE[D + 1 - m]) * w_lvl;
                    dBw[0] = (sdE[D] - sdE[0]) * w_lvl;

                    if (GGF) {
#pragma unroll
                        for (int r = 0; r <= D; ++r) {
                            float v[F];
                            gather<F, HALF>(p.table, l, p.capacity, slot[r], v);  // EncodingGPU.cuh:1484-1485
#pragma unroll
                            for (int f = 0; f < F; ++f) o[f] = fmaf(dBw[r], v[f], o[f]);
                        }
                    }
                    if (TABLE) {
                        float* gbase = a.lattice_grad + (size_t)l * p.capacity * F;
                        float add[D + 1][F];
#pragma unroll
                        for (int r = 0; r <= D; ++r) {
#pragma unroll
                            for (int f = 0; f < F; ++f) add[r][f] = dBw[r] * g[F * k + f];  // EncodingGPU.cuh:1244-1245
                        }
                        scatter_level<F>(sc, gbase, slot, add);
                    }
                }
            }
#pragma unroll
            for (int f = 0; f < F; ++f) out[F * k + f] = o[f];
        }
        if (GGF && active) store_row_segment<F, LPS>(p, a.grad_grad_features, n, l0, out);
    }
    if (GGF && active && p.extra_levels > 0 && blockIdx.y == 0 && p.level_begin == 0) {  // EncodingGPU.cuh:1290-1295
        float* dst = a.grad_grad_features + n * p.width + F * p.nr_levels;
        for (int c = 0; c < F * p.extra_levels; ++c) dst[c] = 0.f;
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

// Levels handled by one thread in one sweep over the points.  A multiple of the levels per step
// (one 32-byte row segment per step).  More levels per pass means fewer sweeps -- each sweep
// re-reads the positions and touches only its own 32-byte pieces of every 128-byte line of the
// feature rows, which costs a 4x DRAM over-fetch on the gradient reads with one step per sweep
// -- but a larger set of table slices is live in L2 at once: capacity * 4F bytes per level for
// the values and as much again for their gradient.  Measured on B200 (pos_dim 3, 4 and 6,
// capacities 2^18..2^20, F = 2): scatter-only kernels are fastest with every level in one sweep
// up to a gradient table of about 100 MB; gather kernels, and scatter kernels beyond that, with
// two sweeps, the finest third of the levels in the second; gather+scatter kernels with about
// 64 MB live.
enum class Traffic { Gather, Scatter, Both };

inline int pick_levels_per_pass(const Problem& p, int requested, Traffic t, int lps) {
    const int levels = p.level_end - p.level_begin;
    int lpp = requested;
    if (lpp <= 0) {
        const double slice = (p.table_half ? 2.0 : 4.0) * p.nr_feat * p.capacity;
        const double mb = 1024.0 * 1024.0;
        if (t == Traffic::Scatter) {
            // one sweep while the fp32 gradient table is within reach of L2 (measured up to the
            // 100.7 MB of capacity 2^19 x 24 levels); beyond that the same two sweeps as the gather
            // kernels (capacity 2^20 x 24 levels, 201 MB: 1.05 ms against 1.84 in one sweep)
            const double gslice = 4.0 * p.nr_feat * p.capacity;
            if (gslice * levels <= 128.0 * mb) {
                lpp = levels;
            } else {
                lpp = ((2 * levels + 2) / 3 + lps - 1) / lps * lps;
                const int cap = (int)(128.0 * mb / gslice);
                if (lpp > cap) lpp = cap;
            }
        }
        else if (t == Traffic::Gather) {
            // Coarse levels touch few slots whatever the capacity; what must fit in L2 together
            // is the saturated, fine levels of a pass.  Two passes with the finest third of the
            // levels in the second one measured best from capacity 2^18 to 2^20 (forward at 2^20 and
            // 24 levels: 0.70 ms against 0.91 with two equal passes and 0.93 with one); tables of a
            // few MB stay in one pass, very large slices are capped at 128 MB per pass.
            if (slice * levels <= 32.0 * mb) {
                lpp = levels;
            } else {
                lpp = ((2 * levels + 2) / 3 + lps - 1) / lps * lps;
                const int cap = (int)(128.0 * mb / slice);
                if (lpp > cap) lpp = cap;
            }
        }
        else
            lpp = (int)(64.0 * mb / (slice + 4.0 * p.nr_feat * p.capacity));  // values + their fp32 gradient
    }
    lpp = (lpp / lps) * lps;
    if (lpp < lps) lpp = lps;
    if (lpp > levels) lpp = ((levels + lps - 1) / lps) * lps;
    return lpp;
}

inline dim3 grid_for(const Problem& p) {
    const unsigned gx = (unsigned)((p.n_points + kThreads - 1) / kThreads);
    const unsigned gy = (unsigned)((p.level_end - p.level_begin + p.levels_per_pass - 1) / p.levels_per_pass);
    return dim3(gx, gy, 1);
}

// small problems get one level per thread and pass so that the grid still covers the machine
inline bool use_single_level(const Problem& p) {
    const int lps = 8 / p.nr_feat;
    const int64_t steps = (p.level_end - p.level_begin + lps - 1) / lps;
    const int64_t blocks = ((p.n_points + kThreads - 1) / kThreads) * steps;
    const int sms = sm_count();
    return lps > 1 && blocks < 2 * (sms > 0 ? sms : 148);
}

template <class Args>
inline Args with_schedule(const Args& in, bool single, Traffic t) {
    Args a = in;
    a.p.levels_per_pass = single ? 1 : pick_levels_per_pass(a.p, a.p.levels_per_pass, t, 8 / a.p.nr_feat);
    return a;
}

template <int F, int LPS>
cudaError_t launch_forward(const ForwardArgs& a, cudaStream_t st) {
    if (a.p.table_half)
        forward_kernel<F, LPS, true><<<grid_for(a.p), kThreads, 0, st>>>(a);
    else
        forward_kernel<F, LPS, false><<<grid_for(a.p), kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

template <int F, int LPS>
cudaError_t launch_forward_linear(const ForwardLinearArgs& a, cudaStream_t st) {
    size_t smem = (size_t)kRing * kSliceBytes + (size_t)a.layer[0].out_features * a.k_pad * sizeof(float);
    int hmax = 0;  // widest hidden layer
    for (int i = 1; i < a.nr_layers; ++i) {
        if (a.layer[i].in_features > hmax) hmax = a.layer[i].in_features;
        if (a.layer[i].out_features % 16 == 0) smem += (size_t)a.layer[i].out_features * a.layer[i].in_features * sizeof(float);
    }
    const dim3 g((unsigned)((a.p.n_points + kTileRows - 1) / kTileRows));
    auto launch = [&](auto kernel) -> cudaError_t {
        if (smem + 1024 > 48 * 1024) {  // the kernel's few static shared words count against the default limit
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        kernel<<<g, kTileRows, smem, st>>>(a);
        return cudaGetLastError();
    };
    const bool h = a.p.table_half != 0;
    if (a.nr_layers == 1) return h ? launch(forward_mlp_kernel<F, LPS, true, 0>) : launch(forward_mlp_kernel<F, LPS, false, 0>);
    if (hmax <= 32) return h ? launch(forward_mlp_kernel<F, LPS, true, 32>) : launch(forward_mlp_kernel<F, LPS, false, 32>);
    return h ? launch(forward_mlp_kernel<F, LPS, true, 64>) : launch(forward_mlp_kernel<F, LPS, false, 64>);
}

// The table is only read where something is gathered (position gradient, grad-grad features):
// the scatter-only kernels have no fp16 variant.
template <int F, int LPS>
cudaError_t launch_backward(const BackwardArgs& a, cudaStream_t st) {
    const dim3 g = grid_for(a.p);
    const bool h = a.p.table_half != 0;
    if (a.lattice_grad && a.positions_grad) {
        if (h) backward_kernel<F, LPS, true, true, true><<<g, kThreads, 0, st>>>(a);
        else backward_kernel<F, LPS, true, true, false><<<g, kThreads, 0, st>>>(a);
    } else if (a.lattice_grad) {
        backward_kernel<F, LPS, true, false, false><<<g, kThreads, 0, st>>>(a);
    } else if (a.positions_grad) {
        if (h) backward_kernel<F, LPS, false, true, true><<<g, kThreads, 0, st>>>(a);
        else backward_kernel<F, LPS, false, true, false><<<g, kThreads, 0, st>>>(a);
    }
    return cudaGetLastError();
}

template <int F, int LPS>
cudaError_t launch_double(const DoubleBackwardArgs& a, cudaStream_t st) {
    const dim3 g = grid_for(a.p);
    const bool h = a.p.table_half != 0;
    if (a.lattice_grad && a.grad_grad_features) {
        if (h) double_backward_kernel<F, LPS, true, true, true><<<g, kThreads, 0, st>>>(a);
        else double_backward_kernel<F, LPS, true, true, false><<<g, kThreads, 0, st>>>(a);
    } else if (a.lattice_grad) {
        double_backward_kernel<F, LPS, true, false, false><<<g, kThreads, 0, st>>>(a);
    } else if (a.grad_grad_features) {
        if (h) double_backward_kernel<F, LPS, false, true, true><<<g, kThreads, 0, st>>>(a);
        else double_backward_kernel<F, LPS, false, true, false><<<g, kThreads, 0, st>>>(a);
    }
    return cudaGetLastError();
}

// feature width and step size are compile-time: pick the instantiation
#define PERMUTO_BY_WIDTH(fn, a, single, st)                                              \
    switch ((a).p.nr_feat) {                                                             \
        case 2: return (single) ? fn<2, 1>(a, st) : fn<2, 4>(a, st);                     \
        case 4: return (single) ? fn<4, 1>(a, st) : fn<4, 2>(a, st);                     \
        case 8: return fn<8, 1>(a, st);                                                  \
        default: return cudaErrorInvalidValue;                                           \
    }

}  // namespace

#define PERMUTO_CAT_(a, b) a##b
#define PERMUTO_CAT(a, b) PERMUTO_CAT_(a, b)

cudaError_t PERMUTO_CAT(launch_forward_dim, PERMUTO_DIM)(const ForwardArgs& a0, cudaStream_t st) {
    const bool single = use_single_level(a0.p);
    const ForwardArgs a = with_schedule(a0, single, Traffic::Gather);
    PERMUTO_BY_WIDTH(launch_forward, a, single, st)
}

cudaError_t PERMUTO_CAT(launch_forward_linear_dim, PERMUTO_DIM)(const ForwardLinearArgs& a, cudaStream_t st) {
    switch (a.p.nr_feat) {  // always whole 8-float steps: the tile is padded, not the level loop
        case 2: return launch_forward_linear<2, 4>(a, st);
        case 4: return launch_forward_linear<4, 2>(a, st);
        case 8: return launch_forward_linear<8, 1>(a, st);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t PERMUTO_CAT(launch_backward_dim, PERMUTO_DIM)(const BackwardArgs& a0, cudaStream_t st) {
    const bool single = use_single_level(a0.p);
    const Traffic t = (a0.lattice_grad && a0.positions_grad) ? Traffic::Both
                                                             : (a0.lattice_grad ? Traffic::Scatter : Traffic::Gather);
    const BackwardArgs a = with_schedule(a0, single, t);
    PERMUTO_BY_WIDTH(launch_backward, a, single, st)
}

cudaError_t PERMUTO_CAT(launch_double_backward_dim, PERMUTO_DIM)(const DoubleBackwardArgs& a0, cudaStream_t st) {
    const bool single = use_single_level(a0.p);
    const Traffic t = (a0.lattice_grad && a0.grad_grad_features)
                          ? Traffic::Both
                          : (a0.lattice_grad ? Traffic::Scatter : Traffic::Gather);
    const DoubleBackwardArgs a = with_schedule(a0, single, t);
    PERMUTO_BY_WIDTH(launch_double, a, single, st)
}

cudaError_t PERMUTO_CAT(launch_debug_dim, PERMUTO_DIM)(const DebugArgs& a, cudaStream_t st) {
    const dim3 g((unsigned)((a.p.n_points + kThreads - 1) / kThreads), (unsigned)a.p.nr_levels, 1);
    debug_kernel<<<g, kThreads, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace permuto
