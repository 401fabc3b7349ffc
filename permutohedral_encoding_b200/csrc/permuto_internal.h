// Internal launch interface between the C-ABI translation unit and the per-dimension kernel
// translation units (one object file per pos_dim so that they compile in parallel).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "permuto_b200.h"

namespace permuto {

// Everything a kernel needs to walk the lattice for a range of levels.
struct Problem {
    const float* positions;
    int64_t pos_stride_n;
    int64_t pos_stride_d;
    const void* table;    // [L, C, F], fp32 or (table_half) fp16
    const float* scale;   // [L, D]
    const float* shift;   // [L, D]
    const float* anneal;  // [L]
    int64_t n_points;
    int32_t nr_levels;
    uint32_t capacity;
    int32_t cap_is_pow2;
    int32_t table_half;   // the value table is stored as fp16 (gathers only; gradients stay fp32)
    int32_t nr_feat;      // F: features per level, 2, 4 or 8
    int32_t width;        // F * (L + extra): row length of features / gradients
    int32_t level_begin;  // levels [level_begin, level_end) are processed
    int32_t level_end;
    int32_t extra_levels; // concat rows
    float points_scaling;
    int32_t rows_vec8_ok; // feature rows may be moved with 32-byte vector accesses
    int32_t pos_vec_ok;   // positions are contiguous rows on a base aligned to the row size (pos_dim 2, 4)
    int32_t levels_per_pass; // in: requested (0 = automatic); set by the launcher for the kernel
};

struct ForwardArgs {
    Problem p;
    float* features;
};

// forward fused with the network that consumes the features: one linear layer
// (out = features @ weight^T + bias) or a whole small MLP
constexpr int kMaxMlpLayers = 6;
struct MlpLayer {
    const float* weight;   // [out_features, in_features] row-major (the layout of torch.nn.Linear.weight)
    const float* bias;     // [out_features] or null
    int32_t in_features;
    int32_t out_features;
};
struct ForwardLinearArgs {
    Problem p;
    MlpLayer layer[kMaxMlpLayers];  // layer[0].in_features == p.width
    int32_t nr_layers;
    int32_t activation;    // PERMUTO_ACT_*, applied after every layer but the last
    float* out;            // [N, out_features of the last layer]
    int32_t k_pad;         // p.width rounded up to a multiple of 8 (one tf32 MMA consumes 8)
    int32_t tmem_cols;     // tensor-memory columns per block: a power of two >= 32
    int32_t tmem_half;     // column offset of the second accumulator range (hidden layers ping-pong)
    int32_t* status;       // device word set non-zero when a wait on the tensor core ran out
    int32_t out_vec8_ok;   // out rows can be written with 256-bit stores
};

struct BackwardArgs {
    Problem p;
    const float* grad_features;
    float* lattice_grad;    // may be null
    float* positions_grad;  // may be null
    int32_t aggregate;      // merge colliding scatter-adds inside a warp
    int32_t concat_grad;    // add the gradient that reaches the positions through the concatenated raw points
};

struct DoubleBackwardArgs {
    Problem p;
    const float* double_positions_grad;
    const float* grad_features;
    float* lattice_grad;        // may be null
    float* grad_grad_features;  // may be null
    int32_t aggregate;
};

struct DebugArgs {
    Problem p;
    int32_t* keys;
    int32_t* slots;
    float* bary;
    int32_t* rank;
};

// Records the message permuto_last_error() returns on this thread and hands back `code`;
// every failing entry point goes through it (defined in permuto_cabi.cu).
int set_error(int code, const char* fmt, ...);

// Number of multiprocessors of the current device (cached per device); 0 if the query fails.
int sm_count();

// Defined once per pos_dim in permuto_dim.cu (compiled with -DPERMUTO_DIM=d).
#define PERMUTO_DECLARE_DIM(d)                                                        \
    cudaError_t launch_forward_dim##d(const ForwardArgs&, cudaStream_t);              \
    cudaError_t launch_forward_linear_dim##d(const ForwardLinearArgs&, cudaStream_t); \
    cudaError_t launch_backward_dim##d(const BackwardArgs&, cudaStream_t);            \
    cudaError_t launch_double_backward_dim##d(const DoubleBackwardArgs&, cudaStream_t); \
    cudaError_t launch_debug_dim##d(const DebugArgs&, cudaStream_t);
PERMUTO_DECLARE_DIM(2)
PERMUTO_DECLARE_DIM(3)
PERMUTO_DECLARE_DIM(4)
PERMUTO_DECLARE_DIM(5)
PERMUTO_DECLARE_DIM(6)
PERMUTO_DECLARE_DIM(7)
#undef PERMUTO_DECLARE_DIM

}  // namespace permuto
