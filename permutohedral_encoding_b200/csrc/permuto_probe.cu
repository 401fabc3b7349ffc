// Ceiling probe for the access pattern of the lattice kernels: independent random 8- or 16-byte
// gathers, or vector reductions, over a caller-provided region, from every SM at full occupancy.
// The lattice kernels are bound by how many such operations per second the memory system
// sustains, not by bytes, so this is the denominator their achieved rate is compared with.
// The reference has no counterpart.
#include <cstdint>
#include <cuda_runtime.h>

#include "permuto_b200.h"
#include "permuto_internal.h"

namespace {

__device__ __forceinline__ uint32_t mix(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352dU;
    x ^= x >> 15;
    x *= 0x846ca68bU;
    x ^= x >> 16;
    return x;
}

// KIND 0: 8-byte gather, 1: 16-byte gather, 2: red.v2.f32, 3: red.v4.f32
template <int KIND>
__global__ void __launch_bounds__(256) probe_kernel(float* region, uint32_t entries, int per_thread) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    float acc = 0.f;
    for (int it = 0; it < per_thread; it += 4) {
        uint32_t s[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) s[j] = mix(t * 977u + (uint32_t)(it + j) + 12345u) % entries;
        if (KIND == 0) {
            float2 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __ldg(reinterpret_cast<const float2*>(region) + s[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc += v[j].x + v[j].y;
        } else if (KIND == 1) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __ldg(reinterpret_cast<const float4*>(region) + s[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc += v[j].x + v[j].w;
        } else if (KIND == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("red.relaxed.gpu.global.add.v2.f32 [%0], {%1, %2};" ::"l"(region + 2ull * s[j]), "f"(0.f),
                             "f"(0.f)
                             : "memory");
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(region + 4ull * s[j]),
                             "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f)
                             : "memory");
        }
    }
    if (acc == 123.456f) region[0] = acc;  // keeps the gathers alive; never true for a zeroed region
}

}  // namespace

extern "C" int permuto_probe_random_access(int32_t kind, float* region, int64_t region_bytes, int32_t accesses_per_thread,
                                           int64_t* total_accesses, void* stream) {
    using permuto::set_error;
    if (!region || kind < 0 || kind > 3)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "probe: region must not be NULL and kind must be 0..3 (got %d)", kind);
    if (accesses_per_thread < 4 || (accesses_per_thread & 3))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "probe: accesses_per_thread must be a positive multiple of 4 (got %d)",
                         accesses_per_thread);
    const int entry_bytes = (kind == 0 || kind == 2) ? 8 : 16;
    if (region_bytes < entry_bytes || region_bytes / entry_bytes > 0x7fffffffLL)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "probe: region_bytes out of range");
    if (reinterpret_cast<uintptr_t>(region) % 16 != 0)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "probe: region must be 16-byte aligned");
    const int sms = permuto::sm_count();
    if (sms <= 0) return set_error(PERMUTO_ERR_CUDA, "probe: cannot query the device");
    const int blocks = sms * 32;
    const uint32_t entries = (uint32_t)(region_bytes / entry_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (kind) {
        case 0: probe_kernel<0><<<blocks, 256, 0, st>>>(region, entries, accesses_per_thread); break;
        case 1: probe_kernel<1><<<blocks, 256, 0, st>>>(region, entries, accesses_per_thread); break;
        case 2: probe_kernel<2><<<blocks, 256, 0, st>>>(region, entries, accesses_per_thread); break;
        default: probe_kernel<3><<<blocks, 256, 0, st>>>(region, entries, accesses_per_thread); break;
    }
    if (total_accesses) *total_accesses = (int64_t)blocks * 256 * accesses_per_thread;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PERMUTO_OK : set_error(PERMUTO_ERR_CUDA, "probe launch: %s", cudaGetErrorString(e));
}
