// Per-(point, level) geometry of the permutohedral lattice: elevate, find the enclosing
// simplex, barycentric weights, hash the d+1 vertex keys.
//
// Behaviour follows kernels/permutohedral_encoding/EncodingGPU.cuh:130-223 and :22-45 of the
// reference (paths relative to its project root): the integer results (remainder-0 point,
// ranks, keys, slots) are bit-identical to it, and the barycentric weights too.  The code is
// organised differently: ranks are turned into a "sorted residual" vector with selects so
// that nothing is indexed dynamically (no local memory), and the d+1 hashes are derived from
// one base hash because the hash is linear over Z/2^32.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace permuto {

constexpr uint32_t kHashMul = 2531011u;  // EncodingGPU.cuh:29

// M^e mod 2^32
__host__ __device__ constexpr uint32_t hash_pow(int e) {
    uint32_t r = 1u;
    for (int i = 0; i < e; ++i) r *= kHashMul;
    return r;
}

template <int D>
struct Simplex {
    int rem0[D + 1];    // remainder-0 lattice point after the rank wrap (multiples of D+1)
    int rank[D + 1];    // permutation of 0..D
    float bary[D + 1];  // barycentric weight of the vertex with remainder r
    float sorted_res[D + 1];  // residual/(D+1) of the coordinate whose rank is k
};

// pos: D floats.  shift, scale: this level's rows.  Rounding of every operation of the elevate
// step is explicit, because simplex selection at fine levels hinges on single ulps of the
// elevated coordinates (they reach 1e5..1e6).  The sequence below is what nvcc's default
// -fmad=true makes of the reference source (.cuh:130-138), established by comparing against the
// reference's own outputs for every pos_dim (cf_i = t_i*scale_i, t_i = pos_i + shift_i):
//   i = D      : e[D] = -(D*cf_D), sm = cf_D
//   2 <= i < D : e[i] = fma(-i, cf_i, sm), sm = sm + cf_i       (cf_i rounded, it feeds i*cf_i)
//   i = 1      : e[1] = fma(-t_1, scale_1, sm), e[0] = fma(t_1, scale_1, sm)
template <int D>
__device__ __forceinline__ void locate_simplex(const float (&pos)[D], const float* __restrict__ shift,
                                               const float* __restrict__ scale, Simplex<D>& s) {
    constexpr float kInv = 1.0f / (D + 1);
    constexpr float kDp1 = (float)(D + 1);
    float e[D + 1];
    float sm = 0.0f;
#pragma unroll
    for (int i = D; i > 0; --i) {
        const float t = __fadd_rn(pos[i - 1], __ldg(shift + i - 1));
        const float sc = __ldg(scale + i - 1);
        if (i == 1) {
            e[1] = __fmaf_rn(-t, sc, sm);
            sm = __fmaf_rn(t, sc, sm);
        } else {
            const float cf = __fmul_rn(t, sc);
            if (i == D) {
                e[i] = -__fmul_rn((float)i, cf);
                sm = cf;
            } else {
                e[i] = __fmaf_rn(-(float)i, cf, sm);
                sm = __fadd_rn(sm, cf);
            }
        }
    }
    e[0] = sm;

    // nearest remainder-0 point, ties towards the lower multiple (.cuh:150-161)
    float rem0f[D + 1];
    float res[D + 1];
    int sum = 0;
#pragma unroll
    for (int i = 0; i <= D; ++i) {
        const float v = __fmul_rn(e[i], kInv);
        const float up = ceilf(v) * kDp1;
        const float down = floorf(v) * kDp1;
        const float du = __fsub_rn(up, e[i]);
        const float dd = __fsub_rn(e[i], down);
        const bool take_up = du < dd;
        rem0f[i] = take_up ? up : down;
        res[i] = take_up ? -du : dd;  // == e - rem0 with one rounding, as .cuh:167-169
        s.rem0[i] = (int)rem0f[i];
        sum += s.rem0[i];
    }
    sum /= (D + 1);

    // rank of each residual; a tie raises the later index (.cuh:166-173)
#pragma unroll
    for (int i = 0; i <= D; ++i) s.rank[i] = 0;
#pragma unroll
    for (int i = 0; i < D; ++i) {
#pragma unroll
        for (int j = i + 1; j <= D; ++j) {
            const bool lt = res[i] < res[j];
            s.rank[i] += lt ? 1 : 0;
            s.rank[j] += lt ? 0 : 1;
        }
    }
    // bring the point back onto the plane (.cuh:177-186)
    float delta[D + 1];
#pragma unroll
    for (int i = 0; i <= D; ++i) {
        int r = s.rank[i] + sum;
        if (r < 0) {
            r += D + 1;
            s.rem0[i] += D + 1;
            rem0f[i] += kDp1;
        } else if (r > D) {
            r -= D + 1;
            s.rem0[i] -= D + 1;
            rem0f[i] -= kDp1;
        }
        s.rank[i] = r;
        delta[i] = __fmul_rn(__fsub_rn(e[i], rem0f[i]), kInv);  // .cuh:194
    }
    // sorted_res[k] = delta of the coordinate with rank k (ranks are a permutation)
#pragma unroll
    for (int k = 0; k <= D; ++k) {
        float v = 0.0f;
#pragma unroll
        for (int i = 0; i <= D; ++i) v = (s.rank[i] == k) ? delta[i] : v;
        s.sorted_res[k] = v;
    }
    // .cuh:193-199: b[D-rank_i] += delta_i; b[D+1-rank_i] -= delta_i; b[0] += 1 + b[D+1].
    // Every b[m], m>=1, receives exactly one +delta and one -delta, so it equals the single
    // rounded difference below whatever the visiting order; b[0] = delta(rank D) + (1 - delta(rank 0)).
#pragma unroll
    for (int m = 1; m <= D; ++m) s.bary[m] = __fsub_rn(s.sorted_res[D - m], s.sorted_res[D + 1 - m]);
    s.bary[0] = __fadd_rn(s.sorted_res[D], __fsub_rn(1.0f, s.sorted_res[0]));
}

// Hashes of the D+1 vertices (before the modulo).  key_i(r) = rem0_i + r - (D+1)[rank_i > D-r]
// (.cuh:216-220) and hash(key) = sum_i key_i * M^(D-i) mod 2^32 (.cuh:24-31), hence
// h(r) = h(0) + r*S - (D+1) * sum_i [rank_i > D-r] M^(D-i).
template <int D>
__device__ __forceinline__ void vertex_hashes(const Simplex<D>& s, uint32_t (&h)[D + 1]) {
    uint32_t base = 0u, all = 0u;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        base += (uint32_t)s.rem0[i] * hash_pow(D - i);
        all += hash_pow(D - i);
    }
    uint32_t lowered = 0u;  // sum of M^(D-i) over coordinates already lowered by D+1
#pragma unroll
    for (int r = 0; r <= D; ++r) {
        if (r > 0) {
#pragma unroll
            for (int i = 0; i < D; ++i) lowered += (s.rank[i] == D + 1 - r) ? hash_pow(D - i) : 0u;
        }
        h[r] = base + (uint32_t)r * all - (uint32_t)(D + 1) * lowered;
    }
}

template <int D>
__device__ __forceinline__ void vertex_key(const Simplex<D>& s, int r, int (&key)[D]) {
#pragma unroll
    for (int i = 0; i < D; ++i) key[i] = s.rem0[i] + r - ((s.rank[i] > D - r) ? (D + 1) : 0);
}

// aligned 8-byte gather of one table entry (both features) through the read-only path
__device__ __forceinline__ float2 gather2(const float* __restrict__ level_base, uint32_t slot) {
    return __ldg(reinterpret_cast<const float2*>(level_base) + slot);
}

// one 8-byte vector reduction: both features of a table-gradient entry in a single L2 atomic
__device__ __forceinline__ void red_add2(float* level_base, uint32_t slot, float x, float y) {
    float* p = level_base + 2ull * slot;
    asm volatile("red.relaxed.gpu.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(x), "f"(y) : "memory");
}

__device__ __forceinline__ void red_add1(float* p, float x) {
    asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(x) : "memory");
}

}  // namespace permuto
