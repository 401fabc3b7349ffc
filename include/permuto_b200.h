/*
 * permuto_b200 -- C ABI of the B200 (sm_100a) permutohedral-lattice hash encoding.
 *
 * This is the boundary a binding of the reference project would target instead of its
 * pybind11 module `permutohedral_encoding_bindings._<cc>_C` (reference: src/PyBridge.cxx:13-45,
 * include/permutohedral_encoding/Encoding.cuh:14-188).  Plain pointers and sizes only: the
 * caller owns every buffer, the library allocates nothing, keeps no state between calls (beyond
 * the cached multiprocessor count of each device and the per-thread error message) and
 * never frees caller memory.  All device pointers must belong to the CUDA device that is
 * current on the calling thread; work is enqueued on `stream` (a cudaStream_t passed as
 * void*, NULL = the legacy default stream) and the functions return without synchronising.
 *
 * Layouts (all fp32, element strides):
 *   positions            [N, pos_dim]      arbitrary strides (pos_stride_n, pos_stride_d)
 *   lattice_values       [L, capacity, F]  contiguous (the reference parameter layout), F = nr_feat_per_level;
 *                                          fp32, or fp16 when the configuration says so
 *   scale_factor         [L, pos_dim]      contiguous, from permuto_scale_factor()
 *   random_shift         [L, pos_dim]      contiguous
 *   anneal_window        [L]               contiguous
 *   features / gradients [N, W]            contiguous, W = F*(L + extra_levels), column
 *                                          F*level + feature -- the ordering the reference
 *                                          module returns (src/pytorch_modules/modules.py:87)
 *   lattice_grad         [L, capacity, F]  contiguous, the parameter's own layout
 *   positions_grad       [N, pos_dim]      contiguous
 *
 * Alignment (checked; a violation returns PERMUTO_ERR_INVALID_ARGUMENT):
 *   lattice_values                          4*F bytes (2*F for an fp16 table): all features of a slot
 *                                           move in one access
 *   features, grad_features, lattice_grad,
 *   grad_grad_features                      8 bytes for F = 2, 16 bytes for F = 4 and 8
 *   32-byte alignment of the feature / gradient rows (base pointer and W*4 a multiple of 32)
 *   is not required but selects the fast path that moves 8 floats of a row per access; offset
 *   views that break it fall back to per-level accesses with identical results.
 *   positions: 4 bytes; contiguous rows on a base aligned to pos_dim*4 bytes are read with one
 *   vector load when pos_dim is 2 or 4.
 *
 * Every function returns PERMUTO_OK or a negative status; permuto_last_error() gives the
 * message of the last failure on the calling thread (every failing entry point sets it, the
 * measurement aid included).  Nothing throws or aborts.
 */
#ifndef PERMUTO_B200_H
#define PERMUTO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PERMUTO_ABI_VERSION 2

enum {
    PERMUTO_OK = 0,
    PERMUTO_ERR_INVALID_ARGUMENT = -1, /* NULL pointer, bad size or stride                    */
    PERMUTO_ERR_UNSUPPORTED = -2,      /* pos_dim outside 2..7 or nr_feat_per_level not 2/4/8 */
    PERMUTO_ERR_CUDA = -3              /* a CUDA runtime call or kernel launch failed         */
};

/* Fixed description of one encoding.  Replaces the reference's EncodingFixedParams
 * (include/permutohedral_encoding/Encoding.cuh:31-53) minus the tensors, which are passed
 * per call. */
typedef struct permuto_config {
    int32_t pos_dim;           /* 2..7 (Encoding.cuh:138-157)                                 */
    int32_t nr_feat_per_level; /* 2 (the reference's only width, Encoding.cuh:140-143), or 4 / 8,
                                  which the reference lists as not yet implemented            */
    int32_t nr_levels;         /* L >= 1                                                      */
    int32_t capacity;          /* slots per level, any value >= 1 (power of two is faster)    */
    int32_t concat_points;     /* 0/1: append ceil(pos_dim/2) levels holding the raw points   */
    float points_scaling;      /* factor applied to the concatenated points                   */
    int32_t levels_per_pass;   /* scheduling hint: levels one sweep over the points handles, a
                                  multiple of 8/F; 0 = chosen from the capacity (no reference
                                  counterpart; results do not depend on it)                    */
    int32_t table_dtype;       /* storage type of lattice_values: PERMUTO_TABLE_F32 (the reference's)
                                  or PERMUTO_TABLE_F16 (storage only: arithmetic, outputs and every
                                  gradient stay fp32; the reference only hints at a half-precision
                                  table, kernels/permutohedral_encoding/EncodingGPU.cuh:12)     */
} permuto_config;

enum { PERMUTO_TABLE_F32 = 0, PERMUTO_TABLE_F16 = 1 };

/* Per-call lattice inputs shared by every entry point.  Replaces the reference's
 * EncodingInput (Encoding.cuh:14-29) plus the scale/shift tensors of EncodingFixedParams. */
typedef struct permuto_inputs {
    int64_t nr_positions; /* N >= 1 (src/Encoding.cu:42: zero points is an error)            */
    const float *positions;
    int64_t pos_stride_n;
    int64_t pos_stride_d;
    const void *lattice_values; /* float, or __half when cfg->table_dtype == PERMUTO_TABLE_F16 */
    const float *scale_factor;
    const float *random_shift;
    const float *anneal_window;
} permuto_inputs;

/* Flags of permuto_backward / permuto_double_backward. */
enum {
    PERMUTO_ZERO_OUTPUTS = 1,      /* clear lattice_grad (the selected levels) and positions_grad before accumulating */
    PERMUTO_NO_AGGREGATE = 2,      /* do not merge colliding scatter-adds inside a warp before the atomics            */
    PERMUTO_KEEP_POSITIONS_GRAD = 4, /* with ZERO_OUTPUTS: leave positions_grad as it is (a later bucket of levels)    */
    PERMUTO_CONCAT_POSITIONS_GRAD = 8 /* backward, concat_points: also add points_scaling * grad of the concatenated
                                         coordinates to positions_grad.  Off by default because the reference omits
                                         this term (src/Encoding.cu:129-134: its backward skips the extra levels)   */
};

int permuto_abi_version(void);
const char *permuto_last_error(void);

/* Number of extra output levels when concat_points is set: ceil(pos_dim / nr_feat_per_level)
 * (src/Encoding.cu:71-74). */
int permuto_extra_levels(int32_t pos_dim, int32_t nr_feat_per_level, int32_t concat_points);

/* Host computation of scale_factor[L, pos_dim] (host pointer out).  Replaces
 * EncodingFixedParams::compute_scale_factor_tensor (Encoding.cuh:55-69) and reproduces its
 * rounding: fp32(1/sqrt((i+1)(i+2))) * fp32(1/fp32(sigma)). */
int permuto_scale_factor(const double *sigmas, int32_t nr_levels, int32_t pos_dim, float *out_host);

/* Forward: features [N, W].  Replaces Encoding<P,2>::forward (src/Encoding.cu:54-108) and the
 * module's permute/reshape copy (src/pytorch_modules/modules.py:87). */
int permuto_forward(const permuto_config *cfg, const permuto_inputs *in, float *features, void *stream);

/* Forward fused with the first linear layer of the network that consumes the features:
 *     out[N, out_features] = features[N, W] @ weight[out_features, W]^T + bias
 * without the features ever being written to memory.  The reference's users run exactly this pair
 * (examples/train_toy_example.py:18-26, README.md:39-40: PermutoEncoding followed by
 * torch.nn.Linear(encoding.output_dims(), 32)); the reference itself has no fused form.
 * weight is row-major [out_features, W] (the layout of torch.nn.Linear.weight), bias [out_features]
 * or NULL, out_features a multiple of 16 in 16..256, W = F*(L + extra_levels) at most 256.
 * The product runs on the tensor cores with both operands rounded to tf32 (10-bit mantissa) and
 * fp32 accumulation: |out - exact| <= about 1e-3 * sum_k |features_k * weight_k| per output.
 * status, if not NULL, is a device int32 the kernel sets non-zero when its bounded wait for the
 * tensor core ran out (it then writes no output for that block); the caller clears and reads it.
 * Inference path: no gradients are produced. */
int permuto_forward_linear(const permuto_config *cfg, const permuto_inputs *in, const float *weight,
                           const float *bias, int32_t out_features, float *out, int32_t *status,
                           void *stream);

/* One layer of the network behind the encoding: y = x @ weight^T + bias, weight row-major
 * [out_features, in_features] (torch.nn.Linear layout), bias [out_features] or NULL; device pointers. */
typedef struct permuto_mlp_layer {
    const float *weight;
    const float *bias;
    int32_t in_features;
    int32_t out_features;
} permuto_mlp_layer;

enum { PERMUTO_ACT_NONE = 0, PERMUTO_ACT_RELU = 1, PERMUTO_ACT_GELU = 2 /* exact, erf-based: torch.nn.GELU() */ };

/* Forward fused with the WHOLE small network that consumes the features, e.g. the reference's
 * toy example (examples/train_toy_example.py:18-26): Linear(48,32) GELU Linear(32,32) GELU
 * Linear(32,32) GELU Linear(32,1).  One kernel: neither the features nor any hidden activation is
 * written to memory; every layer with a width that is a multiple of 16 runs on the tensor cores
 * (tf32 operands, fp32 accumulation in tensor memory), a narrower last layer (1..15 outputs) as
 * fp32 dot products in registers.  `layers` is a HOST array of nr_layers (1..6) descriptors with
 * layers[0].in_features == W and layers[i].in_features == layers[i-1].out_features; hidden widths
 * are multiples of 16 in 16..64; the last layer has 1..16 outputs, or a multiple of 16 up to 64
 * (up to 256 when it is the only layer).  `activation` is applied after every layer but the last.
 * out is [N, out_features of the last layer]; status as for permuto_forward_linear.  Inference path. */
int permuto_forward_mlp(const permuto_config *cfg, const permuto_inputs *in, const permuto_mlp_layer *layers,
                        int32_t nr_layers, int32_t activation, float *out, int32_t *status, void *stream);

/* First-order backward.  Replaces Encoding<P,2>::backward (src/Encoding.cu:111-215).
 * grad_features [N, W].  lattice_grad and positions_grad may each be NULL (not required).
 * Only levels in [level_begin, level_end) are processed -- pass 0 and nr_levels for all; a
 * caller that overlaps a gradient all-reduce with the rest of backward calls once per bucket
 * of levels.  positions_grad accumulates over the processed levels. */
int permuto_backward(const permuto_config *cfg, const permuto_inputs *in, const float *grad_features,
                     float *lattice_grad, float *positions_grad, int32_t level_begin,
                     int32_t level_end, uint32_t flags, void *stream);

/* Double backward of the position gradient.  Replaces
 * Encoding<P,2>::double_backward_from_positions (src/Encoding.cu:218-334).
 * double_positions_grad [N, pos_dim] contiguous = d loss / d positions_grad;
 * grad_features [N, W] = the upstream gradient the first backward received.
 * Outputs (each may be NULL): lattice_grad [L, capacity, F]; grad_grad_features [N, W]
 * (= d loss / d grad_features; the concat columns are written as zero). */
int permuto_double_backward(const permuto_config *cfg, const permuto_inputs *in,
                            const float *double_positions_grad, const float *grad_features,
                            float *lattice_grad, float *grad_grad_features, uint32_t flags,
                            void *stream);

/* Debug view of the lattice geometry (the reference has no counterpart; it exists so that
 * keys and hash slots can be compared bit for bit).  Any output may be NULL.
 *   keys  int32 [N, L, pos_dim+1, pos_dim]   slots int32 [N, L, pos_dim+1]
 *   bary  fp32  [N, L, pos_dim+1]            rank  int32 [N, L, pos_dim+1] */
int permuto_debug_lattice(const permuto_config *cfg, const permuto_inputs *in, int32_t *keys,
                          int32_t *slots, float *bary, int32_t *rank, void *stream);

/* Flags of permuto_adam_step. */
enum {
    PERMUTO_ADAM_SKIP_UNTOUCHED = 1, /* leave entries alone whose gradient and both moments are zero (exact when
                                        weight_decay == 0; ignored otherwise)                                    */
    PERMUTO_ADAM_ZERO_GRAD = 2       /* clear the gradient in the same pass (the next backward then accumulates
                                        without PERMUTO_ZERO_OUTPUTS)                                            */
};

/* One AdamW step (amsgrad off) over n fp32 elements -- the lattice values, their gradient and the two
 * moment arrays, all [L, capacity, F] contiguous and 16-byte aligned -- in a single kernel.  Replaces the
 * optimizer the reference's training loops run over the table (examples/performance.py:161,101:
 * torch.optim.AdamW(betas=(0.9, 0.99), eps=1e-15, weight_decay=0); examples/train_toy_example.py:30) and
 * follows torch's update order (hyper-parameters are doubles, combined in double and rounded to fp32
 * once, as torch does with Python scalars); `step` counts from 1.  The moments start as zeros (caller-allocated). */
int permuto_adam_step(float *values, float *grad, float *exp_avg, float *exp_avg_sq, int64_t n, double lr,
                      double beta1, double beta2, double eps, double weight_decay, int64_t step,
                      uint32_t flags, void *stream);

/* Measurement aid with no counterpart in the reference: launches, from every SM at full
 * occupancy, `accesses_per_thread` (a multiple of 4) independent random accesses per thread over
 * the caller's region (device memory, 16-byte aligned, zero-filled by the caller; the reductions
 * add zeros, so the region keeps its contents).  kind 0 = 8-byte gather, 1 = 16-byte gather,
 * 2 = red.global.add.v2.f32, 3 = red.global.add.v4.f32.  The caller times the stream; the
 * lattice kernels' achieved operations per second are compared with these ceilings. */
int permuto_probe_random_access(int32_t kind, float *region, int64_t region_bytes, int32_t accesses_per_thread,
                                int64_t *total_accesses, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PERMUTO_B200_H */
