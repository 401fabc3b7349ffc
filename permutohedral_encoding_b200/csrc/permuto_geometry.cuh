// Per-(point, level) geometry of the permutohedral lattice: elevate, find the enclosing
// simplex, barycentric weights, hash the d+1 vertex keys.
//
// Behaviour follows kernels/permutohedral_encoding/EncodingGPU.cuh:130-223 and :22-45 of the
// reference (paths relative to its project root): the integer results (remainder-0 point,
// ranks, keys, slots) are bit-identical to it; the barycentric weights agree to fp32 rounding
// (about 1e-7 absolute) but not bit for bit, because nvcc contracts the reference's
// `b[..] += (e - rem0) * inv` into fused multiply-adds in its own way.  The code is
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
    uint32_t hash[D + 1];  // hash of the vertex with remainder r, before the modulo
};

// -1 if a < b else 0, in one instruction
__device__ __forceinline__ int minus_one_if_less(float a, float b) {
    int d;
    asm("set.lt.s32.f32 %0, %1, %2;" : "=r"(d) : "f"(a), "f"(b));
    return d;
}

// pos: D floats.  shift, scale: this level's rows.  Rounding of every operation of the elevate
// step is explicit, because simplex selection at fine levels hinges on single ulps of the
// elevated coordinates (they reach 1e5..1e6).  The sequence below is what nvcc's default
// -fmad=true makes of the reference source (.cuh:130-138), established by comparing against the
// reference's own outputs for every pos_dim (cf_i = t_i*scale_i, t_i = pos_i + shift_i):
//   i = D      : e[D] = -(D*cf_D), sm = cf_D
//   2 <= i < D : e[i] = fma(-i, cf_i, sm), sm = sm + cf_i       (cf_i rounded, it feeds i*cf_i)
//   i = 1      : e[1] = fma(-t_1, scale_1, sm), e[0] = fma(t_1, scale_1, sm)
//
// Everything after the elevate step produces the reference's integers (.cuh:146-223) with far
// fewer instructions than a transcription would:
//  * ceil(v)*(D+1) is floor(v)*(D+1) + (D+1) unless v is an integer, in which case the
//    reference's choice is the lower multiple whatever the comparison says; both products are
//    exact while |e| < 2^22, and a rarely taken branch keeps the reference's own formula above;
//  * ranks come from one set.lt per pair and three-input adds; the wrap of rank and rem0 is a
//    mask when D+1 is a power of two;
//  * barycentric weights and vertex hashes are read off the rank-sorted residuals / hash powers
//    (selected with compares, never indexed dynamically): every b[m], m >= 1, receives exactly
//    one +delta and one -delta in the reference (.cuh:193-199), so it equals one rounded
//    difference whatever the visiting order, and the hash is linear over Z/2^32:
//    h(r) = h(0) + r*S - (D+1) * sum_{i<D} [rank_i > D-r] M^(D-i)  (.cuh:24-31, :216-220).
template <int D>
__device__ __forceinline__ void locate_simplex(const float (&pos)[D], const float* __restrict__ shift,
                                               const float* __restrict__ scale, Simplex<D>& s) {
    constexpr float kInv = 1.0f / (D + 1);
    constexpr float kDp1 = (float)(D + 1);
    constexpr bool kPow2 = ((D + 1) & D) == 0;
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
    float v[D + 1], down[D + 1], up[D + 1];
    float biggest = 0.0f;
#pragma unroll
    for (int i = 0; i <= D; ++i) {
        v[i] = __fmul_rn(e[i], kInv);
        down[i] = floorf(v[i]) * kDp1;
        up[i] = (v[i] != floorf(v[i])) ? down[i] + kDp1 : down[i];
        biggest = fmaxf(biggest, fabsf(e[i]));
    }
    if (biggest >= 4194304.0f) {  // products no longer exact: the reference's own expression
#pragma unroll
        for (int i = 0; i <= D; ++i) up[i] = ceilf(v[i]) * kDp1;
    }
    float rem0f[D + 1], res[D + 1];
    float sumf = 0.0f;
#pragma unroll
    for (int i = 0; i <= D; ++i) {
        const float du = __fsub_rn(up[i], e[i]);
        const float dd = __fsub_rn(e[i], down[i]);
        const bool take_up = du < dd;
        rem0f[i] = take_up ? up[i] : down[i];
        res[i] = take_up ? -du : dd;  // == e - rem0 with one rounding, as .cuh:167-169
        sumf += rem0f[i];
    }
    const int sum = __float2int_rn(sumf * kInv);  // exact: every rem0 is a multiple of D+1

    // rank of each residual; a tie raises the later index (.cuh:166-173):
    // rank_i = i + sum_{j<i} c_ji - sum_{j>i} c_ij with c_ab = -[res_a < res_b]
    int rk[D + 1];
#pragma unroll
    for (int i = 0; i <= D; ++i) rk[i] = i + sum;
#pragma unroll
    for (int i = 0; i < D; ++i) {
#pragma unroll
        for (int j = i + 1; j <= D; ++j) {
            const int c = minus_one_if_less(res[i], res[j]);
            rk[i] -= c;
            rk[j] += c;
        }
    }
    // bring the point back onto the plane (.cuh:177-186)
    float delta[D + 1];
#pragma unroll
    for (int i = 0; i <= D; ++i) {
        const int r = rk[i];
        const float off = (r < 0) ? kDp1 : ((r > D) ? -kDp1 : 0.0f);
        rk[i] = kPow2 ? (r & D) : ((r < 0) ? r + D + 1 : ((r > D) ? r - (D + 1) : r));
        rem0f[i] += off;
        s.rank[i] = rk[i];
        s.rem0[i] = (int)rem0f[i];
        delta[i] = __fmul_rn(__fsub_rn(e[i], rem0f[i]), kInv);  // .cuh:194
    }
    // sorted[k] = delta of the coordinate whose rank is k; pw[k] = its hash power (0 for i = D)
    float sorted[D + 1];
    uint32_t pw[D + 1];
#pragma unroll
    for (int k = 0; k <= D; ++k) {
        float dv = delta[D];
        uint32_t pv = 0u;
#pragma unroll
        for (int i = D - 1; i >= 0; --i) {
            const bool is = rk[i] == k;
            dv = is ? delta[i] : dv;
            pv = is ? hash_pow(D - i) : pv;
        }
        sorted[k] = dv;
        pw[k] = pv;
    }
#pragma unroll
    for (int m = 1; m <= D; ++m) s.bary[m] = __fsub_rn(sorted[D - m], sorted[D + 1 - m]);
    s.bary[0] = __fadd_rn(sorted[D], __fsub_rn(1.0f, sorted[0]));

    uint32_t base = 0u, all = 0u;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        base += (uint32_t)s.rem0[i] * hash_pow(D - i);
        all += hash_pow(D - i);
    }
    uint32_t lowered = 0u;  // hash powers of the coordinates already lowered by D+1
    s.hash[0] = base;
#pragma unroll
    for (int r = 1; r <= D; ++r) {
        lowered += pw[D + 1 - r];
        s.hash[r] = base + (uint32_t)r * all - (uint32_t)(D + 1) * lowered;
    }
}

template <int D>
__device__ __forceinline__ void vertex_key(const Simplex<D>& s, int r, int (&key)[D]) {
#pragma unroll
    for (int i = 0; i < D; ++i) key[i] = s.rem0[i] + r - ((s.rank[i] > D - r) ? (D + 1) : 0);
}

__device__ __forceinline__ void red_add1(float* p, float x) {
    asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(x) : "memory");
}

}  // namespace permuto
