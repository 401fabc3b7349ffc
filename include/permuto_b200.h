/*
 * permuto_b200 -- C ABI of the B200 (sm_100a) permutohedral-lattice hash encoding.
 *
 * This is the boundary a binding of the reference project would target instead of its
 * pybind11 module `permutohedral_encoding_bindings._<cc>_C` (reference: src/PyBridge.cxx:13-45,
 * include/permutohedral_encoding/Encoding.cuh:14-188).  Plain pointers and sizes only: the
 * caller owns every buffer, the library allocates nothing, keeps no state between calls and
 * never frees caller memory.  All device pointers must belong to the CUDA device that is
 * current on the calling thread; work is enqueued on `stream` (a cudaStream_t passed as
 * void*, NULL = the legacy default stream) and the functions return without synchronising.
 *
 * Layouts (all fp32, element strides):
 *   positions            [N, pos_dim]      arbitrary strides (pos_stride_n, pos_stride_d)
 *   lattice_values       [L, capacity, F]  contiguous (the reference parameter layout), F = nr_feat_per_level
 *   scale_factor         [L, pos_dim]      contiguous, from permuto_scale_factor()
 *   random_shift         [L, pos_dim]      contiguous
 *   anneal_window        [L]               contiguous
 *   features / gradients [N, W]            contiguous, W = F*(L + extra_levels), column
 *                                          F*level + feature -- the ordering the reference
 *                                          module returns (src/pytorch_modules/modules.py:87)
 *   lattice_grad         [L, capacity, F]  contiguous, the parameter's own layout
 *   positions_grad       [N, pos_dim]      contiguous
 *
 * Every function returns PERMUTO_OK or a negative status; permuto_last_error() gives the
 * message of the last failure on the calling thread.  Nothing throws or aborts.
 */
#ifndef PERMUTO_B200_H
#define PERMUTO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PERMUTO_ABI_VERSION 1

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
} permuto_config;

/* Per-call lattice inputs shared by every entry point.  Replaces the reference's
 * EncodingInput (Encoding.cuh:14-29) plus the scale/shift tensors of EncodingFixedParams. */
typedef struct permuto_inputs {
    int64_t nr_positions; /* N >= 1 (src/Encoding.cu:42: zero points is an error)            */
    const float *positions;
    int64_t pos_stride_n;
    int64_t pos_stride_d;
    const float *lattice_values;
    const float *scale_factor;
    const float *random_shift;
    const float *anneal_window;
} permuto_inputs;

/* Flags of permuto_backward / permuto_double_backward. */
enum {
    PERMUTO_ZERO_OUTPUTS = 1,      /* clear lattice_grad (the selected levels) and positions_grad before accumulating */
    PERMUTO_NO_AGGREGATE = 2,      /* do not merge colliding scatter-adds inside a warp before the atomics            */
    PERMUTO_KEEP_POSITIONS_GRAD = 4 /* with ZERO_OUTPUTS: leave positions_grad as it is (a later bucket of levels)     */
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
