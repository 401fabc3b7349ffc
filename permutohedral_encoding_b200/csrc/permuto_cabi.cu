// extern "C" surface declared in include/permuto_b200.h: argument validation, output
// clearing and dispatch on pos_dim.  Replaces the host launchers of the reference
// (src/Encoding.cu:54-334) and its pybind bridge (src/PyBridge.cxx:13-45).
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "permuto_b200.h"
#include "permuto_internal.h"

namespace {
thread_local char g_error[512] = "";
}

namespace permuto {

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices] = {};  // 0 = not asked yet; racing writers store the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices) cached[dev] = sms;
    return sms;
}

}  // namespace permuto

namespace {

using permuto::set_error;

int cuda_fail(cudaError_t e, const char* what) {
    return set_error(PERMUTO_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int extra_levels(int pos_dim, int nr_feat, int concat) { return concat ? (pos_dim + nr_feat - 1) / nr_feat : 0; }

// Checks shared by every entry point; the messages mirror the reference's CHECKs
// (src/Encoding.cu:37-45, :63-66) and factory errors (Encoding.cuh:142,155).
int build_problem(const permuto_config* cfg, const permuto_inputs* in, permuto::Problem& p) {
    if (!cfg || !in) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "cfg and in must not be NULL");
    if (cfg->pos_dim < 2 || cfg->pos_dim > 7)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "Encoding: pos_dim must be 2,3,4,5,6 or 7 (got %d)", cfg->pos_dim);
    if (cfg->nr_feat_per_level != 2 && cfg->nr_feat_per_level != 4 && cfg->nr_feat_per_level != 8)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "Encoding: nr_feat_per_level must be 2, 4 or 8 (got %d)",
                    cfg->nr_feat_per_level);
    if (cfg->nr_levels < 1 || cfg->nr_levels > 65535)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "nr_levels must be in 1..65535 (got %d)", cfg->nr_levels);
    if (cfg->capacity < 1) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "capacity must be >= 1");
    if (in->nr_positions < 1) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "Why do we have 0 points");
    if (in->nr_positions > (int64_t)0x7fffffff)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "nr_positions must be below 2^31");
    if (!in->positions || !in->lattice_values || !in->scale_factor || !in->random_shift || !in->anneal_window)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "positions, lattice_values, scale_factor, random_shift and "
                                                  "anneal_window must not be NULL");
    const int F = cfg->nr_feat_per_level;
    if (cfg->table_dtype != PERMUTO_TABLE_F32 && cfg->table_dtype != PERMUTO_TABLE_F16)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "table_dtype must be PERMUTO_TABLE_F32 or PERMUTO_TABLE_F16 (got %d)",
                         cfg->table_dtype);
    const int entry_bytes = (cfg->table_dtype == PERMUTO_TABLE_F16 ? 2 : 4) * F;
    if (!aligned(in->lattice_values, (size_t)entry_bytes))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT,
                    "lattice_values must be %d-byte aligned (all features of a slot are moved at once)", entry_bytes);
    const int extra = extra_levels(cfg->pos_dim, F, cfg->concat_points);
    p.positions = in->positions;
    p.pos_stride_n = in->pos_stride_n;
    p.pos_stride_d = in->pos_stride_d;
    p.table = in->lattice_values;
    p.scale = in->scale_factor;
    p.shift = in->random_shift;
    p.anneal = in->anneal_window;
    p.n_points = in->nr_positions;
    p.nr_levels = cfg->nr_levels;
    p.capacity = (uint32_t)cfg->capacity;
    p.cap_is_pow2 = (cfg->capacity & (cfg->capacity - 1)) == 0;
    p.nr_feat = F;
    p.table_half = cfg->table_dtype == PERMUTO_TABLE_F16 ? 1 : 0;
    p.width = F * (cfg->nr_levels + extra);
    p.level_begin = 0;
    p.level_end = cfg->nr_levels;
    p.extra_levels = extra;
    p.points_scaling = cfg->points_scaling;
    p.rows_vec8_ok = 0;
    p.pos_vec_ok = (in->pos_stride_d == 1 && in->pos_stride_n == cfg->pos_dim &&
                    aligned(in->positions, 4 * (size_t)cfg->pos_dim)) ? 1 : 0;
    p.levels_per_pass = cfg->levels_per_pass < 0 ? 0 : cfg->levels_per_pass;
    return PERMUTO_OK;
}

// feature rows can be moved 32 bytes at a time when every row segment starts on a 32-byte
// boundary: base aligned, row pitch a multiple of 32 bytes, first level on an 8-float boundary
bool rows_vec8(const permuto::Problem& p, const void* a, const void* b) {
    if ((p.width * 4) % 32 != 0 || (p.level_begin * p.nr_feat) % 8 != 0) return false;
    if (a && !aligned(a, 32)) return false;
    if (b && !aligned(b, 32)) return false;
    return true;
}

// alignment of per-level accesses to rows and table entries: 8 bytes for F = 2, 16 for F = 4 and 8
size_t row_align(const permuto::Problem& p) { return p.nr_feat == 2 ? 8 : 16; }

#define PERMUTO_DISPATCH(fn, args, st)                                  \
    switch (cfg->pos_dim) {                                             \
        case 2: err = permuto::fn##_dim2(args, st); break;              \
        case 3: err = permuto::fn##_dim3(args, st); break;              \
        case 4: err = permuto::fn##_dim4(args, st); break;              \
        case 5: err = permuto::fn##_dim5(args, st); break;              \
        case 6: err = permuto::fn##_dim6(args, st); break;              \
        default: err = permuto::fn##_dim7(args, st); break;             \
    }

}  // namespace

extern "C" {

int permuto_abi_version(void) { return PERMUTO_ABI_VERSION; }

const char* permuto_last_error(void) { return g_error; }

int permuto_extra_levels(int32_t pos_dim, int32_t nr_feat_per_level, int32_t concat_points) {
    if (nr_feat_per_level < 1) return 0;
    return extra_levels(pos_dim, nr_feat_per_level, concat_points);
}

int permuto_scale_factor(const double* sigmas, int32_t nr_levels, int32_t pos_dim, float* out_host) {
    if (!sigmas || !out_host) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "sigmas and out_host must not be NULL");
    if (nr_levels < 1) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "nr_levels must be >= 1");
    if (pos_dim < 2 || pos_dim > 7)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "Encoding: pos_dim must be 2,3,4,5,6 or 7 (got %d)", pos_dim);
    for (int l = 0; l < nr_levels; ++l) {
        // the sigma list reaches the reference as std::vector<float>; its tensor-by-scalar
        // division multiplies the fp32 element by the fp32 reciprocal of the divisor
        const float sigma = (float)sigmas[l];
        const float inv_sigma = 1.0f / sigma;
        for (int i = 0; i < pos_dim; ++i) {
            const float base = (float)(1.0 / std::sqrt((double)((i + 1) * (i + 2))));
            volatile float prod = base * inv_sigma;  // one fp32 rounding, never fused or widened
            out_host[l * pos_dim + i] = prod;
        }
    }
    return PERMUTO_OK;
}

int permuto_forward(const permuto_config* cfg, const permuto_inputs* in, float* features, void* stream) {
    permuto::ForwardArgs a;
    if (int rc = build_problem(cfg, in, a.p)) return rc;
    if (!features) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "features must not be NULL");
    if (!aligned(features, row_align(a.p))) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "features must be %d-byte aligned", (int)row_align(a.p));
    a.features = features;
    a.p.rows_vec8_ok = rows_vec8(a.p, features, nullptr);
    cudaError_t err;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PERMUTO_DISPATCH(launch_forward, a, st)
    if (err != cudaSuccess) return cuda_fail(err, "permuto_forward launch");
    return PERMUTO_OK;
}

int permuto_forward_mlp(const permuto_config* cfg, const permuto_inputs* in, const permuto_mlp_layer* layers,
                        int32_t nr_layers, int32_t activation, float* out, int32_t* status, void* stream) {
    permuto::ForwardLinearArgs a;
    if (int rc = build_problem(cfg, in, a.p)) return rc;
    if (!layers || !out) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "layers and out must not be NULL");
    if (nr_layers < 1 || nr_layers > permuto::kMaxMlpLayers)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "nr_layers must be in 1..%d (got %d)", permuto::kMaxMlpLayers, nr_layers);
    if (activation != PERMUTO_ACT_NONE && activation != PERMUTO_ACT_RELU && activation != PERMUTO_ACT_GELU)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "activation must be PERMUTO_ACT_NONE, _RELU or _GELU (got %d)", activation);
    if (a.p.width > 256)
        return set_error(PERMUTO_ERR_UNSUPPORTED, "the fused layers take feature rows of at most 256 columns (got %d)",
                         a.p.width);
    int widest = 0;  // over the layers that run on the tensor core
    for (int i = 0; i < nr_layers; ++i) {
        const permuto_mlp_layer& ly = layers[i];
        const int expect = i == 0 ? a.p.width : layers[i - 1].out_features;
        if (!ly.weight) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "layer %d: weight must not be NULL", i);
        if (ly.in_features != expect)
            return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "layer %d: in_features is %d but its input has %d columns", i,
                             ly.in_features, expect);
        const bool is_last = i == nr_layers - 1;
        const int h = ly.out_features;
        const bool on_tensor_core = h % 16 == 0 && h >= 16;
        if (nr_layers == 1) {
            if (!on_tensor_core || h > 256)
                return set_error(PERMUTO_ERR_UNSUPPORTED, "out_features must be a multiple of 16 in 16..256 (got %d)", h);
        } else if (!is_last) {
            if (!on_tensor_core || h > 64)
                return set_error(PERMUTO_ERR_UNSUPPORTED, "layer %d: a hidden width must be a multiple of 16 in 16..64 (got %d)", i, h);
        } else if (!(on_tensor_core && h <= 64) && !(h >= 1 && h < 16)) {
            return set_error(PERMUTO_ERR_UNSUPPORTED,
                             "layer %d: the last layer must have 1..16 outputs or a multiple of 16 up to 64 (got %d)", i, h);
        }
        if (on_tensor_core && h > widest) widest = h;
        a.layer[i].weight = ly.weight;
        a.layer[i].bias = ly.bias;
        a.layer[i].in_features = ly.in_features;
        a.layer[i].out_features = h;
    }
    const int last_out = layers[nr_layers - 1].out_features;
    if (!aligned(out, last_out % 16 == 0 ? 16 : 4)) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "out must be 16-byte aligned");
    a.nr_layers = nr_layers;
    a.activation = activation;
    a.out = out;
    a.k_pad = (a.p.width + 7) / 8 * 8;
    int half = 16;  // two accumulator ranges for the hidden layers to alternate between
    while (half < widest) half <<= 1;
    int cols = 32;  // allocation granularity of tensor memory: a power of two, at least 32 columns
    while (cols < (nr_layers == 1 ? widest : 2 * half)) cols <<= 1;
    a.tmem_cols = cols;
    a.tmem_half = half;
    a.status = status;
    a.out_vec8_ok = (last_out % 16 == 0 && aligned(out, 32)) ? 1 : 0;
    cudaError_t err;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PERMUTO_DISPATCH(launch_forward_linear, a, st)
    if (err != cudaSuccess) return cuda_fail(err, "permuto_forward_mlp launch");
    return PERMUTO_OK;
}

int permuto_forward_linear(const permuto_config* cfg, const permuto_inputs* in, const float* weight, const float* bias,
                           int32_t out_features, float* out, int32_t* status, void* stream) {
    if (!cfg || !in) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "cfg and in must not be NULL");
    if (!weight || !out) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "weight and out must not be NULL");
    permuto_mlp_layer one;
    one.weight = weight;
    one.bias = bias;
    one.in_features = cfg->nr_feat_per_level * (cfg->nr_levels + extra_levels(cfg->pos_dim, cfg->nr_feat_per_level,
                                                                              cfg->concat_points));
    one.out_features = out_features;
    return permuto_forward_mlp(cfg, in, &one, 1, PERMUTO_ACT_NONE, out, status, stream);
}

int permuto_backward(const permuto_config* cfg, const permuto_inputs* in, const float* grad_features,
                     float* lattice_grad, float* positions_grad, int32_t level_begin, int32_t level_end,
                     uint32_t flags, void* stream) {
    permuto::BackwardArgs a;
    if (int rc = build_problem(cfg, in, a.p)) return rc;
    if (!grad_features) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "grad_features must not be NULL");
    if (!aligned(grad_features, row_align(a.p)))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "grad_features must be %d-byte aligned", (int)row_align(a.p));
    if (lattice_grad && !aligned(lattice_grad, row_align(a.p)))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "lattice_grad must be %d-byte aligned", (int)row_align(a.p));
    if (level_begin < 0 || level_end > cfg->nr_levels || level_begin > level_end)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "level range [%d, %d) outside [0, %d)", level_begin, level_end,
                    cfg->nr_levels);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    a.p.level_begin = level_begin;
    a.p.level_end = level_end;
    a.grad_features = grad_features;
    a.lattice_grad = lattice_grad;
    a.positions_grad = positions_grad;
    a.aggregate = (flags & PERMUTO_NO_AGGREGATE) ? 0 : 1;
    a.concat_grad = (flags & PERMUTO_CONCAT_POSITIONS_GRAD) ? 1 : 0;
    a.p.rows_vec8_ok = rows_vec8(a.p, grad_features, nullptr);
    if (flags & PERMUTO_ZERO_OUTPUTS) {
        cudaError_t e = cudaSuccess;
        if (lattice_grad && level_end > level_begin)
            e = cudaMemsetAsync(lattice_grad + (size_t)level_begin * a.p.capacity * a.p.nr_feat, 0,
                                (size_t)(level_end - level_begin) * a.p.capacity * a.p.nr_feat * sizeof(float), st);
        if (e == cudaSuccess && positions_grad && !(flags & PERMUTO_KEEP_POSITIONS_GRAD))
            e = cudaMemsetAsync(positions_grad, 0, (size_t)a.p.n_points * cfg->pos_dim * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e, "permuto_backward clearing outputs");
    }
    if ((!lattice_grad && !positions_grad) || level_end == level_begin) return PERMUTO_OK;
    cudaError_t err;
    PERMUTO_DISPATCH(launch_backward, a, st)
    if (err != cudaSuccess) return cuda_fail(err, "permuto_backward launch");
    return PERMUTO_OK;
}

int permuto_double_backward(const permuto_config* cfg, const permuto_inputs* in, const float* double_positions_grad,
                            const float* grad_features, float* lattice_grad, float* grad_grad_features,
                            uint32_t flags, void* stream) {
    permuto::DoubleBackwardArgs a;
    if (int rc = build_problem(cfg, in, a.p)) return rc;
    if (!double_positions_grad) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "double_positions_grad must not be NULL");
    if (lattice_grad && !grad_features)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "grad_features is needed for the lattice gradient");
    if (grad_features && !aligned(grad_features, row_align(a.p)))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "grad_features must be %d-byte aligned", (int)row_align(a.p));
    if (lattice_grad && !aligned(lattice_grad, row_align(a.p)))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "lattice_grad must be %d-byte aligned", (int)row_align(a.p));
    if (grad_grad_features && !aligned(grad_grad_features, row_align(a.p)))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "grad_grad_features must be %d-byte aligned", (int)row_align(a.p));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    a.double_positions_grad = double_positions_grad;
    a.grad_features = grad_features;
    a.lattice_grad = lattice_grad;
    a.grad_grad_features = grad_grad_features;
    a.aggregate = (flags & PERMUTO_NO_AGGREGATE) ? 0 : 1;
    a.p.rows_vec8_ok = rows_vec8(a.p, grad_features, grad_grad_features);
    if ((flags & PERMUTO_ZERO_OUTPUTS) && lattice_grad) {
        cudaError_t e = cudaMemsetAsync(lattice_grad, 0, (size_t)a.p.nr_levels * a.p.capacity * a.p.nr_feat * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e, "permuto_double_backward clearing outputs");
    }
    if (!lattice_grad && !grad_grad_features) return PERMUTO_OK;
    cudaError_t err;
    PERMUTO_DISPATCH(launch_double_backward, a, st)
    if (err != cudaSuccess) return cuda_fail(err, "permuto_double_backward launch");
    return PERMUTO_OK;
}

int permuto_debug_lattice(const permuto_config* cfg, const permuto_inputs* in, int32_t* keys, int32_t* slots,
                          float* bary, int32_t* rank, void* stream) {
    permuto::DebugArgs a;
    if (int rc = build_problem(cfg, in, a.p)) return rc;
    a.keys = keys;
    a.slots = slots;
    a.bary = bary;
    a.rank = rank;
    if (!keys && !slots && !bary && !rank) return PERMUTO_OK;
    cudaError_t err;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PERMUTO_DISPATCH(launch_debug, a, st)
    if (err != cudaSuccess) return cuda_fail(err, "permuto_debug_lattice launch");
    return PERMUTO_OK;
}

}  // extern "C"
