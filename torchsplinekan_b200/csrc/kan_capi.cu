// C ABI of the library (declared in include/kan_b200.h): argument validation,
// mode resolution, workspace sizing and dispatch to the kernel launchers.
#include "../../include/kan_b200.h"
#include "kan_internal.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

using namespace kanb200;

namespace {

// Scratch handed to the SIMT / regulariser launchers starts after the status
// header, so the first word of every workspace keeps the same meaning.
inline void* ws_body(void* ws, size_t bytes) {
    return (ws && bytes > kWsHeader) ? static_cast<char*>(ws) + kWsHeader : nullptr;
}
inline size_t ws_body_bytes(void* ws, size_t bytes) { return (ws && bytes > kWsHeader) ? bytes - kWsHeader : 0; }

thread_local char g_err[512] = "";
int g_basis_impl = 1;

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    if (e == cudaErrorMemoryAllocation)
        return fail(KANB200_EWORKSPACE, "%s: workspace missing or too small", what);
    return fail(KANB200_ECUDA, "%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
}

bool make_shape(int64_t N, int64_t I, int64_t O, int G, int k, LayerShape& s) {
    s.N = N;
    s.I = (int)I;
    s.O = (int)O;
    s.G = G;
    s.K = k;
    return true;
}

// Whether a layer call takes the narrow-layer kernels (AUTO only): a handful of outputs, where the
// 256-output tile of the tensor-core kernels and the 64-wide tiles of the float64 matrix-instruction
// kernels mostly compute padding, and enough samples to fill the GPU with blocks of 64.  Measured
// (us, forward / backward, narrow against the kernels it replaces): 64 -> 1 at 131072 rows float32
// 156 / 464 against 288 / 1018, float64 242 / 799 against 279 / 874; where they lose -- 256 -> 10 at
// 8192 rows 278 / 260 against 74 / 156, float64 64 -> 16 at 4096 rows 162 / 172 against 64 / 116 --
// they are not chosen.
bool layer_uses_narrow(int mode, int dtype, const LayerShape& s) {
    if (mode != KANB200_MODE_AUTO || !narrow_layer_supported(s.O, s.R(), s.K)) return false;
    return s.O <= 4 && s.N >= 32768 && (dtype == KANB200_F64 || dtype == KANB200_F32);
}

// Whether the from-x edge statistic takes the tensor-core kernel for this problem.
bool edge_x_uses_tc(int mode, int dtype, const LayerShape& s) {
    if (dtype != KANB200_F32 || mode == KANB200_MODE_SIMT || !tc_edge_supported(s)) return false;
    // layers of at most 16 outputs have a kernel of their own on the FMA pipes (the tensor-core tile
    // is 128 outputs wide whatever the layer has)
    if (mode == KANB200_MODE_AUTO) return s.N >= 256 && s.O > 16;
    return true;
}

// The same for its backward (needs the SiLU / no-base form: no caller-provided base values).
bool edge_x_bwd_uses_tc(int mode, int dtype, const LayerShape& s, bool custom_base) {
    if (dtype != KANB200_F32 || mode == KANB200_MODE_SIMT || custom_base || !tc_edge_bwd_supported(s)) return false;
    // from about 2^23 edge-samples on: below, the table, the two weight images and the finalize pass
    // cost more than the FMA kernels need for the whole job
    // (outputs are padded to a tile of 128, so the cost follows N I max(O, 128))
    if (mode == KANB200_MODE_AUTO)
        return s.N >= 256 && s.O > 16 && s.N * s.I * (int64_t)(s.O > 128 ? s.O : 128) >= ((int64_t)1 << 23);
    return true;
}

}  // namespace

extern "C" {

KANB200_API const char* kanb200_last_error(void) { return g_err; }

KANB200_API int kanb200_version(void) { return 100; }

KANB200_API int kanb200_set_basis_impl(int impl) {
    if (impl != 0 && impl != 1) return fail(KANB200_EINVAL, "basis impl must be 0 (recurrence) or 1 (local)");
    g_basis_impl = impl;
    return KANB200_OK;
}

KANB200_API int kanb200_get_basis_impl(void) { return g_basis_impl; }

KANB200_API int kanb200_set_accumulation_chunks(int forward_blocks, int param_blocks, int input_blocks) {
    if (forward_blocks < 0 || param_blocks < 0 || input_blocks < 0)
        return fail(KANB200_EINVAL, "accumulation chunk lengths must not be negative");
    tc_set_chunks(forward_blocks, param_blocks, input_blocks);
    return KANB200_OK;
}

KANB200_API int kanb200_check_shapes(int64_t N, int64_t I, int64_t O, int G, int k, int dtype) {
    if (dtype != KANB200_F32 && dtype != KANB200_F64)
        return fail(KANB200_EINVAL, "only FP32 and FP64 inputs are supported");
    if (k < 1 || k > 3) return fail(KANB200_EINVAL, "spline_order must be 1, 2 or 3; got %d", k);
    if (G < 1) return fail(KANB200_EINVAL, "grid has %d knots, too few for spline_order %d", G + 2 * k + 1, k);
    if (N < 0 || I < 1 || O < 1) return fail(KANB200_EINVAL, "bad sizes N=%lld I=%lld O=%lld",
                                             (long long)N, (long long)I, (long long)O);
    if (G + 2 * k > KANB200_MAX_DEG0_BASIS)
        return fail(KANB200_EINVAL, "CUDA kernel supports G + 2k <= %d (got G=%d, k=%d); use backend='reference' "
                                    "for larger grids", KANB200_MAX_DEG0_BASIS, G, k);
    if (I > KANB200_MAX_IN_FEATURES)
        return fail(KANB200_EINVAL, "CUDA kernel supports in_features <= %d, got %lld", KANB200_MAX_IN_FEATURES,
                    (long long)I);
    if (O > (int64_t)1 << 24) return fail(KANB200_EINVAL, "out_features too large: %lld", (long long)O);
    return KANB200_OK;
}

KANB200_API int kanb200_resolve_mode_for(int op, int mode, int dtype, int64_t N, int64_t I, int64_t O, int G,
                                         int k) {
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    const bool tc_ok = dtype == KANB200_F32 && tc_supported(s);
    if (mode == KANB200_MODE_AUTO) {
        if (!tc_ok || N < 256 || I < 8) return KANB200_MODE_SIMT;
        // The tensor-core kernels handle ragged tiles, but a call costs three to six launches (table,
        // operand images, contraction, finalize) against one to three for the gather kernels, about
        // 35 us in all.
        // Backward: they pay from about 2^24 edge-samples (N I O) on, and for narrow layers (whose
        // outputs are padded to a 256-wide tile, so the cost follows N I) from 2^19 input values on
        // (measured, us, gather / tensor cores: 256 -> 10 at 1024 rows 68 / 112, at 4096 rows 182 / 122;
        // 64 -> 64 at 1024 rows 56 / 71, at 4096 rows 109 / 82; 256 -> 256 at 1024 rows 250 / 124).
        // Forward: the gather kernel walks every input feature per output tile and loses much earlier
        // (256 -> 10 at 256 .. 4096 rows 241 / 76; 64 -> 64 84 / 35; 784 -> 256 at 256 rows 988 / 202;
        // 32 -> 8 at 1024 rows 33 / 34): from 2^16 input values on.
        const int64_t narrow = op == KANB200_OP_FORWARD ? ((int64_t)1 << 16) : ((int64_t)1 << 19);
        if (N * I * O >= ((int64_t)1 << 24) || N * I >= narrow) return KANB200_MODE_TC_BF16X3;
        return KANB200_MODE_SIMT;
    }
    if (mode == KANB200_MODE_SIMT) return mode;
    if (mode == KANB200_MODE_TC_BF16X3 || mode == KANB200_MODE_TC_BF16X1)
        return tc_ok ? mode : fail(KANB200_EUNSUPPORTED, "tensor-core modes need float32 and spline order k <= 3");
    return fail(KANB200_EINVAL, "unknown mode %d", mode);
}

KANB200_API int kanb200_resolve_mode(int mode, int dtype, int64_t N, int64_t I, int64_t O, int G, int k) {
    return kanb200_resolve_mode_for(KANB200_OP_BACKWARD, mode, dtype, N, I, O, G, k);
}

KANB200_API size_t kanb200_workspace_bytes(int op, int mode, int dtype, int64_t N, int64_t I, int64_t O, int G, int k,
                               int need_x, int need_param) {
    if (kanb200_check_shapes(N, I, O, G, k, dtype) != KANB200_OK) return 0;
    if (N == 0) return 0;                       // an empty batch launches nothing that needs scratch
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    if (op == KANB200_OP_BASIS) {
        // the table-driven basis kernels; 0 = the recurrence kernels run and need nothing
        return dtype == KANB200_F32 && basis_table_supported(s) ? kWsHeader + tc_table_bytes(s) : 0;
    }
    if (op == KANB200_OP_EDGE_X_FWD || op == KANB200_OP_EDGE_X_BWD) {
        if (N < 1) return 0;
        const bool b = op == KANB200_OP_EDGE_X_BWD;
        if (!b && edge_x_uses_tc(mode, dtype, s)) return tc_edge_workspace(s);
        size_t tc_bytes = 0;
        if (b && edge_x_bwd_uses_tc(mode, dtype, s, false)) tc_bytes = tc_edge_bwd_workspace(s, true);
        const size_t fma_bytes = kWsHeader + (dtype == KANB200_F32 ? edge_workspace<float>(N, s.I, s.O, s.R(), b)
                                                                     : edge_workspace<double>(N, s.I, s.O, s.R(), b));
        if (b) return tc_bytes > fma_bytes ? tc_bytes : fma_bytes;      // a call with base values takes the FMA path
        return kWsHeader + (dtype == KANB200_F32 ? edge_workspace<float>(N, s.I, s.O, s.R(), b)
                                                 : edge_workspace<double>(N, s.I, s.O, s.R(), b));
    }
    if (op == KANB200_OP_EDGE_FWD || op == KANB200_OP_EDGE_BWD) {
        const bool b = op == KANB200_OP_EDGE_BWD;
        if (N < 1) return 0;
        return kWsHeader + (dtype == KANB200_F32 ? edge_workspace<float>(N, s.I, s.O, s.R(), b)
                                                 : edge_workspace<double>(N, s.I, s.O, s.R(), b));
    }
    if (layer_uses_narrow(mode, dtype, s)) {
        if (op == KANB200_OP_FORWARD || !need_param) return 0;
        return kWsHeader + (dtype == KANB200_F32 ? narrow_layer_workspace<float>(N, s.I, s.O, s.R())
                                                 : narrow_layer_workspace<double>(N, s.I, s.O, s.R()));
    }
    const int m = kanb200_resolve_mode_for(op == KANB200_OP_FORWARD ? KANB200_OP_FORWARD : KANB200_OP_BACKWARD, mode,
                                           dtype, N, I, O, G, k);
    if (m < 0) return 0;
    if (m == KANB200_MODE_SIMT) {
        if (dtype == KANB200_F64 && dense64_supported(s)) {
            return dense64_workspace(op == KANB200_OP_FORWARD, s, need_x != 0, need_param != 0);
        }
        if (op == KANB200_OP_FORWARD) return 0;
        const size_t b = dtype == KANB200_F32 ? simt_backward_workspace<float>(s, need_param != 0)
                                              : simt_backward_workspace<double>(s, need_param != 0);
        return b ? kWsHeader + b : 0;
    }
    return tc_workspace(op, s, need_x != 0, need_param != 0);
}

KANB200_API int kanb200_basis(int dtype, const void* x, const void* grid, void* H, int64_t N, int64_t I, int G, int k,
                  void* stream) {
    int rc = kanb200_check_shapes(N, I, 1, G, k, dtype);
    if (rc) return rc;
    if (N == 0) return KANB200_OK;
    if (!x || !grid || !H) return fail(KANB200_EINVAL, "kan_basis: NULL pointer");
    LayerShape s;
    make_shape(N, I, 1, G, k, s);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = dtype == KANB200_F32
                        ? simt_basis<float>((const float*)x, (const float*)grid, (float*)H, s, st)
                        : simt_basis<double>((const double*)x, (const double*)grid, (double*)H, s, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_basis");
}

KANB200_API int kanb200_basis_ws(int dtype, const void* x, const void* grid, void* H, int64_t N, int64_t I, int G,
                                 int k, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, 1, G, k, dtype);
    if (rc) return rc;
    LayerShape s;
    make_shape(N, I, 1, G, k, s);
    const bool table = dtype == KANB200_F32 && basis_table_supported(s) && workspace &&
                       workspace_bytes >= kWsHeader + tc_table_bytes(s) && ((uintptr_t)H & 15) == 0;
    if (!table) return kanb200_basis(dtype, x, grid, H, N, I, G, k, stream);
    if (!x || !grid || !H) return fail(KANB200_EINVAL, "kan_basis: NULL pointer");
    cudaStream_t st = (cudaStream_t)stream;
    float* tab = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWsHeader);
    cudaError_t e = tc_build_table((const float*)grid, tab, s, st);
    if (e == cudaSuccess) e = simt_basis_table((const float*)x, tab, tc_table_stride(s), (float*)H, s, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_basis");
}

KANB200_API int kanb200_basis_grad_ws(int dtype, const void* x, const void* grid, const void* gH, void* gx,
                                      int64_t N, int64_t I, int G, int k, void* workspace, size_t workspace_bytes,
                                      void* stream) {
    int rc = kanb200_check_shapes(N, I, 1, G, k, dtype);
    if (rc) return rc;
    LayerShape s;
    make_shape(N, I, 1, G, k, s);
    const bool table = dtype == KANB200_F32 && basis_table_supported(s) && workspace &&
                       workspace_bytes >= kWsHeader + tc_table_bytes(s) && ((uintptr_t)gH & 15) == 0;
    if (!table) return kanb200_basis_grad(dtype, x, grid, gH, gx, N, I, G, k, stream);
    if (!x || !grid || !gH || !gx) return fail(KANB200_EINVAL, "kan_basis_grad: NULL pointer");
    cudaStream_t st = (cudaStream_t)stream;
    float* tab = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWsHeader);
    cudaError_t e = tc_build_table((const float*)grid, tab, s, st);
    if (e == cudaSuccess)
        e = simt_basis_grad_table((const float*)x, tab, tc_table_stride(s), (const float*)gH, (float*)gx, s, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_basis_grad");
}

KANB200_API int kanb200_basis_grad(int dtype, const void* x, const void* grid, const void* gH, void* gx,
                       int64_t N, int64_t I, int G, int k, void* stream) {
    int rc = kanb200_check_shapes(N, I, 1, G, k, dtype);
    if (rc) return rc;
    if (N == 0) return KANB200_OK;
    if (!x || !grid || !gH || !gx) return fail(KANB200_EINVAL, "kan_basis_grad: NULL pointer");
    LayerShape s;
    make_shape(N, I, 1, G, k, s);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = dtype == KANB200_F32
                        ? simt_basis_grad<float>((const float*)x, (const float*)grid, (const float*)gH, (float*)gx, s, st)
                        : simt_basis_grad<double>((const double*)x, (const double*)grid, (const double*)gH,
                                                  (double*)gx, s, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_basis_grad");
}

KANB200_API int kanb200_forward(int dtype, int mode, const void* x, const void* grid, const void* base_weight,
                    const void* spline_weight, const void* spline_scaler, void* y,
                    int64_t N, int64_t I, int64_t O, int G, int k,
                    void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, dtype);
    if (rc) return rc;
    if (N == 0) return KANB200_OK;
    if (!x || !grid || !spline_weight || !y) return fail(KANB200_EINVAL, "kan_forward: NULL pointer");
    const int m = kanb200_resolve_mode_for(KANB200_OP_FORWARD, mode, dtype, N, I, O, G, k);
    if (m < 0) return m;
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (layer_uses_narrow(mode, dtype, s)) {
        e = dtype == KANB200_F32
                ? narrow_layer_forward<float>((const float*)x, (const float*)grid, (const float*)base_weight,
                                              (const float*)spline_weight, (const float*)spline_scaler, (float*)y, N,
                                              s.I, s.O, s.R(), k, st)
                : narrow_layer_forward<double>((const double*)x, (const double*)grid, (const double*)base_weight,
                                               (const double*)spline_weight, (const double*)spline_scaler, (double*)y,
                                               N, s.I, s.O, s.R(), k, st);
    } else if (m == KANB200_MODE_SIMT && dtype == KANB200_F64 && dense64_supported(s)) {
        e = dense64_forward((const double*)x, (const double*)grid, (const double*)base_weight,
                            (const double*)spline_weight, (const double*)spline_scaler, (double*)y, s,
                            workspace, workspace_bytes, st);
    } else if (m == KANB200_MODE_SIMT) {
        e = dtype == KANB200_F32
                ? simt_forward<float>((const float*)x, (const float*)grid, (const float*)base_weight,
                                      (const float*)spline_weight, (const float*)spline_scaler, (float*)y, s, st)
                : simt_forward<double>((const double*)x, (const double*)grid, (const double*)base_weight,
                                       (const double*)spline_weight, (const double*)spline_scaler, (double*)y, s, st);
    } else {
        e = tc_forward(m == KANB200_MODE_TC_BF16X3 ? 3 : 1, (const float*)x, (const float*)grid,
                       (const float*)base_weight, (const float*)spline_weight, (const float*)spline_scaler,
                       (float*)y, s, workspace, workspace_bytes, st);
    }
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_forward");
}

KANB200_API size_t kanb200_prepared_bytes(int dtype, int64_t I, int64_t O, int G, int k, int has_base) {
    LayerShape s;
    make_shape(1, I, O, G, k, s);
    if (dtype != KANB200_F32 || kanb200_check_shapes(1, I, O, G, k, dtype) != KANB200_OK || !tc_supported(s)) return 0;
    return tc_prepared_bytes(s, has_base != 0);
}

KANB200_API int kanb200_prepare_forward(int dtype, const void* grid, const void* base_weight,
                                        const void* spline_weight, const void* spline_scaler, int64_t I, int64_t O,
                                        int G, int k, void* prepared, size_t prepared_bytes, void* stream) {
    int rc = kanb200_check_shapes(1, I, O, G, k, dtype);
    if (rc) return rc;
    if (!grid || !spline_weight || !prepared) return fail(KANB200_EINVAL, "prepare_forward: NULL pointer");
    LayerShape s;
    make_shape(1, I, O, G, k, s);
    if (dtype != KANB200_F32 || !tc_supported(s))
        return fail(KANB200_EUNSUPPORTED, "prepare_forward: the prepared form needs float32 and spline order k <= 3");
    cudaError_t e = tc_prepare_forward((const float*)grid, (const float*)base_weight, (const float*)spline_weight,
                                       (const float*)spline_scaler, s, prepared, prepared_bytes,
                                       (cudaStream_t)stream);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "prepare_forward");
}

KANB200_API int kanb200_forward_prepared(int dtype, int mode, const void* x, const void* prepared,
                                         size_t prepared_bytes, int has_base, void* y, int64_t N, int64_t I,
                                         int64_t O, int G, int k, void* workspace, size_t workspace_bytes,
                                         void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, dtype);
    if (rc) return rc;
    if (N == 0) return KANB200_OK;
    if (!x || !prepared || !y) return fail(KANB200_EINVAL, "forward_prepared: NULL pointer");
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    if (dtype != KANB200_F32 || !tc_supported(s))
        return fail(KANB200_EUNSUPPORTED, "forward_prepared: the prepared form needs float32 and spline order k <= 3");
    if (mode == KANB200_MODE_SIMT) return fail(KANB200_EINVAL, "forward_prepared: runs on the tensor cores only");
    if (mode != KANB200_MODE_AUTO && mode != KANB200_MODE_TC_BF16X3 && mode != KANB200_MODE_TC_BF16X1)
        return fail(KANB200_EINVAL, "unknown mode %d", mode);
    cudaError_t e = tc_forward_prepared(mode == KANB200_MODE_TC_BF16X1 ? 1 : 3, (const float*)x, prepared,
                                        prepared_bytes, has_base != 0, (float*)y, s, workspace, workspace_bytes,
                                        (cudaStream_t)stream);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "forward_prepared");
}

KANB200_API int kanb200_backward(int dtype, int mode, const void* grad_out, const void* x, const void* grid,
                     const void* base_weight, const void* spline_weight, const void* spline_scaler,
                     void* grad_x, void* grad_base_weight, void* grad_spline_weight, void* grad_spline_scaler,
                     int64_t N, int64_t I, int64_t O, int G, int k,
                     void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, dtype);
    if (rc) return rc;
    if (!spline_weight || (N > 0 && (!grad_out || !x || !grid)))
        return fail(KANB200_EINVAL, "kan_backward: NULL pointer");
    if (grad_spline_scaler && !spline_scaler)
        return fail(KANB200_EINVAL, "kan_backward: grad_spline_scaler requested without spline_scaler");
    if (!base_weight) grad_base_weight = nullptr;
    const int m = kanb200_resolve_mode(mode, dtype, N, I, O, G, k);
    if (m < 0) return m;
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (layer_uses_narrow(mode, dtype, s)) {
        void* body = ws_body(workspace, workspace_bytes);
        const size_t body_bytes = ws_body_bytes(workspace, workspace_bytes);
        e = dtype == KANB200_F32
                ? narrow_layer_backward<float>((const float*)grad_out, (const float*)x, (const float*)grid,
                                               (const float*)base_weight, (const float*)spline_weight,
                                               (const float*)spline_scaler, (float*)grad_x, (float*)grad_base_weight,
                                               (float*)grad_spline_weight, (float*)grad_spline_scaler, N, s.I, s.O,
                                               s.R(), k, body, body_bytes, st)
                : narrow_layer_backward<double>((const double*)grad_out, (const double*)x, (const double*)grid,
                                                (const double*)base_weight, (const double*)spline_weight,
                                                (const double*)spline_scaler, (double*)grad_x,
                                                (double*)grad_base_weight, (double*)grad_spline_weight,
                                                (double*)grad_spline_scaler, N, s.I, s.O, s.R(), k, body, body_bytes,
                                                st);
    } else if (m == KANB200_MODE_SIMT && dtype == KANB200_F64 && dense64_supported(s)) {
        e = dense64_backward((const double*)grad_out, (const double*)x, (const double*)grid,
                             (const double*)base_weight, (const double*)spline_weight, (const double*)spline_scaler,
                             (double*)grad_x, (double*)grad_base_weight, (double*)grad_spline_weight,
                             (double*)grad_spline_scaler, s, workspace, workspace_bytes, st);
    } else if (m == KANB200_MODE_SIMT) {
        e = dtype == KANB200_F32
                ? simt_backward<float>((const float*)grad_out, (const float*)x, (const float*)grid,
                                       (const float*)base_weight, (const float*)spline_weight,
                                       (const float*)spline_scaler, (float*)grad_x, (float*)grad_base_weight,
                                       (float*)grad_spline_weight, (float*)grad_spline_scaler, s,
                                       ws_body(workspace, workspace_bytes),
                                       ws_body_bytes(workspace, workspace_bytes), st)
                : simt_backward<double>((const double*)grad_out, (const double*)x, (const double*)grid,
                                        (const double*)base_weight, (const double*)spline_weight,
                                        (const double*)spline_scaler, (double*)grad_x, (double*)grad_base_weight,
                                        (double*)grad_spline_weight, (double*)grad_spline_scaler, s,
                                        ws_body(workspace, workspace_bytes),
                                        ws_body_bytes(workspace, workspace_bytes), st);
    } else {
        e = tc_backward(m == KANB200_MODE_TC_BF16X3 ? 3 : 1, (const float*)grad_out, O, (const float*)x,
                        (const float*)grid, (const float*)base_weight, (const float*)spline_weight,
                        (const float*)spline_scaler, (float*)grad_x, (float*)grad_base_weight,
                        (float*)grad_spline_weight, (float*)grad_spline_scaler, s, workspace, workspace_bytes, st);
    }
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_backward");
}

KANB200_API int kanb200_backward_param_rows(int mode, const void* grad_out, const void* x, const void* grid,
                                            const void* base_weight, const void* spline_weight,
                                            const void* spline_scaler, void* grad_base_weight,
                                            void* grad_spline_weight, void* grad_spline_scaler,
                                            int64_t N, int64_t I, int64_t O, int G, int k,
                                            int64_t o_begin, int64_t o_end,
                                            void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, KANB200_F32);
    if (rc) return rc;
    if (o_begin < 0 || o_end > O || o_begin >= o_end)
        return fail(KANB200_EINVAL, "kan_backward_param_rows: rows [%lld, %lld) outside [0, %lld)",
                    (long long)o_begin, (long long)o_end, (long long)O);
    if (N < 1) return fail(KANB200_EINVAL, "kan_backward_param_rows: empty batch");
    if (!spline_weight || !grad_out || !x || !grid)
        return fail(KANB200_EINVAL, "kan_backward_param_rows: NULL pointer");
    if (grad_spline_scaler && !spline_scaler)
        return fail(KANB200_EINVAL, "kan_backward_param_rows: grad_spline_scaler requested without spline_scaler");
    if (mode != KANB200_MODE_TC_BF16X3 && mode != KANB200_MODE_TC_BF16X1)
        return fail(KANB200_EUNSUPPORTED, "kan_backward_param_rows: tensor-core modes only");
    if (!base_weight) grad_base_weight = nullptr;
    const int64_t rows = o_end - o_begin;
    LayerShape s;
    make_shape(N, I, rows, G, k, s);
    if (!tc_supported(s)) return fail(KANB200_EUNSUPPORTED, "kan_backward_param_rows: shape not supported");
    const size_t oi = (size_t)o_begin * (size_t)I, oir = oi * (size_t)(G + k);
    auto off = [](const void* p, size_t n) -> const float* { return p ? (const float*)p + n : nullptr; };
    auto offw = [](void* p, size_t n) -> float* { return p ? (float*)p + n : nullptr; };
    cudaError_t e = tc_backward(mode == KANB200_MODE_TC_BF16X3 ? 3 : 1, (const float*)grad_out + o_begin, O,
                                (const float*)x, (const float*)grid, off(base_weight, oi), off(spline_weight, oir),
                                off(spline_scaler, oi), nullptr, offw(grad_base_weight, oi),
                                offw(grad_spline_weight, oir), offw(grad_spline_scaler, oi), s, workspace,
                                workspace_bytes, (cudaStream_t)stream);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "kan_backward_param_rows");
}

static int check_edge(int dtype, int64_t N, int64_t I, int64_t O, int R) {
    if (dtype != KANB200_F32 && dtype != KANB200_F64)
        return fail(KANB200_EINVAL, "edge_abs_mean: only FP32/FP64 supported");
    if (R < 1 || R > 72) return fail(KANB200_EINVAL, "edge_abs_mean: R must be <= 72, got %d", R);
    if (I < 1 || I > KANB200_MAX_IN_FEATURES) return fail(KANB200_EINVAL, "edge_abs_mean: too many input features");
    if (N < 1) return fail(KANB200_EINVAL, "edge_abs_mean: need at least one sample");
    if (O < 1) return fail(KANB200_EINVAL, "edge_abs_mean: bad out_features");
    return KANB200_OK;
}

KANB200_API int kanb200_edge_abs_mean(int dtype, const void* s, const void* H, const void* bw, const void* W, void* a,
                          int64_t N, int64_t I, int64_t O, int R,
                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_edge(dtype, N, I, O, R);
    if (rc) return rc;
    if (!H || !W || !a) return fail(KANB200_EINVAL, "edge_abs_mean: NULL pointer");
    if ((s == nullptr) != (bw == nullptr))
        return fail(KANB200_EINVAL, "edge_abs_mean: s and base_weight must both be given or both be absent");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = dtype == KANB200_F32
                        ? edge_abs_mean_fwd<float>((const float*)s, (const float*)H, (const float*)bw, (const float*)W,
                                                   (float*)a, N, (int)I, (int)O, R, ws_body(workspace, workspace_bytes),
                                                   ws_body_bytes(workspace, workspace_bytes), st)
                        : edge_abs_mean_fwd<double>((const double*)s, (const double*)H, (const double*)bw,
                                                    (const double*)W, (double*)a, N, (int)I, (int)O, R,
                                                    ws_body(workspace, workspace_bytes),
                                                    ws_body_bytes(workspace, workspace_bytes), st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean");
}

KANB200_API int kanb200_edge_abs_mean_x(int dtype, int mode, const void* x, const void* s_val, const void* grid,
                                        const void* bw, const void* W, void* a,
                                        int64_t N, int64_t I, int64_t O, int G, int k,
                                        void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, dtype);
    if (rc) return rc;
    if (N < 1) return fail(KANB200_EINVAL, "edge_abs_mean: need at least one sample");
    if (!x || !grid || !W || !a) return fail(KANB200_EINVAL, "edge_abs_mean_x: NULL pointer");
    if (s_val && !bw) return fail(KANB200_EINVAL, "edge_abs_mean_x: base values given without base_weight");
    if (mode < KANB200_MODE_AUTO || mode > KANB200_MODE_TC_BF16X1) return fail(KANB200_EINVAL, "unknown mode %d", mode);
    LayerShape s;
    make_shape(N, I, O, G, k, s);
    cudaStream_t st = (cudaStream_t)stream;
    if (edge_x_uses_tc(mode, dtype, s)) {
        cudaError_t e = tc_edge_forward(mode == KANB200_MODE_TC_BF16X1 ? 1 : 3, (const float*)x, (const float*)s_val,
                                        (const float*)grid, (const float*)bw, (const float*)W, (float*)a, s,
                                        workspace, workspace_bytes, st);
        return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_x");
    }
    if (mode == KANB200_MODE_TC_BF16X3 || mode == KANB200_MODE_TC_BF16X1)
        return fail(KANB200_EUNSUPPORTED, "edge_abs_mean_x: tensor-core modes need float32 and G + k <= 8");
    cudaError_t e =
        dtype == KANB200_F32
            ? edge_abs_mean_x_fwd<float>((const float*)x, (const float*)s_val, (const float*)grid, (const float*)bw,
                                         (const float*)W, (float*)a, N, (int)I, (int)O, G + k, k,
                                         ws_body(workspace, workspace_bytes), ws_body_bytes(workspace, workspace_bytes), st)
            : edge_abs_mean_x_fwd<double>((const double*)x, (const double*)s_val, (const double*)grid,
                                          (const double*)bw, (const double*)W, (double*)a, N, (int)I, (int)O, G + k, k,
                                          ws_body(workspace, workspace_bytes), ws_body_bytes(workspace, workspace_bytes),
                                          st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_x");
}

KANB200_API int kanb200_edge_abs_mean_x_backward(int dtype, int mode, const void* grad_a, const void* x,
                                                 const void* s_val,
                                                 const void* grid, const void* bw, const void* W,
                                                 void* gx, void* ds, void* dbw, void* dW,
                                                 int64_t N, int64_t I, int64_t O, int G, int k,
                                                 void* workspace, size_t workspace_bytes, void* stream) {
    int rc = kanb200_check_shapes(N, I, O, G, k, dtype);
    if (rc) return rc;
    if (N < 1) return fail(KANB200_EINVAL, "edge_abs_mean: need at least one sample");
    if (!grad_a || !x || !grid || !W) return fail(KANB200_EINVAL, "edge_abs_mean_x_backward: NULL pointer");
    if (s_val && !bw) return fail(KANB200_EINVAL, "edge_abs_mean_x_backward: base values given without base_weight");
    if (ds && !s_val) return fail(KANB200_EINVAL, "edge_abs_mean_x_backward: ds requested without base values s");
    if (mode < KANB200_MODE_AUTO || mode > KANB200_MODE_TC_BF16X1) return fail(KANB200_EINVAL, "unknown mode %d", mode);
    cudaStream_t st = (cudaStream_t)stream;
    LayerShape shape;
    make_shape(N, I, O, G, k, shape);
    if (edge_x_bwd_uses_tc(mode, dtype, shape, s_val != nullptr)) {
        cudaError_t e = tc_edge_backward((const float*)grad_a, (const float*)x, (const float*)grid, (const float*)bw,
                                         (const float*)W, (float*)gx, (float*)dbw, (float*)dW, shape, workspace,
                                         workspace_bytes, st);
        return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_x_backward");
    }
    if (mode == KANB200_MODE_TC_BF16X3 || mode == KANB200_MODE_TC_BF16X1)
        return fail(KANB200_EUNSUPPORTED, "edge_abs_mean_x_backward: tensor-core modes need float32, G + k <= 8, "
                                          "at most 256 outputs and no caller-provided base values");
    cudaError_t e =
        dtype == KANB200_F32
            ? edge_abs_mean_x_bwd<float>((const float*)grad_a, (const float*)x, (const float*)s_val, (const float*)grid,
                                         (const float*)bw, (const float*)W, (float*)gx, (float*)ds, (float*)dbw,
                                         (float*)dW, N, (int)I, (int)O, G + k, k, ws_body(workspace, workspace_bytes),
                                         ws_body_bytes(workspace, workspace_bytes), st)
            : edge_abs_mean_x_bwd<double>((const double*)grad_a, (const double*)x, (const double*)s_val,
                                          (const double*)grid, (const double*)bw, (const double*)W, (double*)gx,
                                          (double*)ds, (double*)dbw, (double*)dW, N, (int)I, (int)O, G + k, k,
                                          ws_body(workspace, workspace_bytes), ws_body_bytes(workspace, workspace_bytes),
                                          st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_x_backward");
}

KANB200_API size_t kanb200_edge_penalty_workspace_bytes(void) { return edge_penalty_workspace_bytes(); }

KANB200_API int kanb200_edge_penalty(int dtype, const void* a, int64_t n, double mu1, double mu2, void* value,
                                     void* grad, void* workspace, size_t workspace_bytes, void* stream) {
    if (dtype != KANB200_F32 && dtype != KANB200_F64) return fail(KANB200_EINVAL, "edge_penalty: bad dtype");
    if (!a || !value || n < 1) return fail(KANB200_EINVAL, "edge_penalty: NULL pointer or no entries");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = dtype == KANB200_F32
                        ? edge_penalty<float>((const float*)a, n, mu1, mu2, (float*)value, (float*)grad, workspace,
                                              workspace_bytes, st)
                        : edge_penalty<double>((const double*)a, n, mu1, mu2, (double*)value, (double*)grad, workspace,
                                               workspace_bytes, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_penalty");
}

KANB200_API int kanb200_set_forward_variant(int variant) {
    tc_set_forward_variant(variant);
    return KANB200_OK;
}

KANB200_API int kanb200_set_edge_sign_recheck(int on) {
    tc_edge_set_sign_recheck(on != 0);
    return KANB200_OK;
}

KANB200_API int kanb200_get_edge_sign_recheck(void) { return tc_edge_get_sign_recheck() ? 1 : 0; }

KANB200_API int kanb200_edge_abs_mean_noalloc(int dtype, const void* s, const void* H, const void* bw,
                                               const void* W, void* a, int64_t N, int64_t I, int64_t O, int R,
                                               void* stream) {
    int rc = check_edge(dtype, N, I, O, R);
    if (rc) return rc;
    if (!H || !W || !a) return fail(KANB200_EINVAL, "edge_abs_mean_noalloc: NULL pointer");
    if ((s == nullptr) != (bw == nullptr))
        return fail(KANB200_EINVAL, "edge_abs_mean_noalloc: s and base_weight must both be given or both be absent");
    const size_t need = dtype == KANB200_F32 ? edge_workspace<float>(N, (int)I, (int)O, R, false)
                                             : edge_workspace<double>(N, (int)I, (int)O, R, false);
    if (need > edge_static_scratch_bytes())
        return fail(KANB200_EWORKSPACE,
                    "edge_abs_mean_noalloc: this shape needs %zu bytes of scratch, the built-in buffer holds %zu; "
                    "use kanb200_edge_abs_mean with a caller-provided workspace",
                    need, edge_static_scratch_bytes());
    void* scratch = nullptr;
    cudaError_t e = edge_static_scratch(&scratch);
    if (e != cudaSuccess) return cuda_fail(e, "edge_abs_mean_noalloc (scratch address)");
    cudaStream_t st = (cudaStream_t)stream;
    e = dtype == KANB200_F32
            ? edge_abs_mean_fwd<float>((const float*)s, (const float*)H, (const float*)bw, (const float*)W, (float*)a,
                                       N, (int)I, (int)O, R, scratch, edge_static_scratch_bytes(), st)
            : edge_abs_mean_fwd<double>((const double*)s, (const double*)H, (const double*)bw, (const double*)W,
                                        (double*)a, N, (int)I, (int)O, R, scratch, edge_static_scratch_bytes(), st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_noalloc");
}

KANB200_API int kanb200_edge_abs_mean_backward(int dtype, const void* grad_a, const void* s, const void* H, const void* bw,
                                   const void* W, void* ds, void* dH, void* dbw, void* dW,
                                   int64_t N, int64_t I, int64_t O, int R,
                                   void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_edge(dtype, N, I, O, R);
    if (rc) return rc;
    if (!H || !W || !grad_a) return fail(KANB200_EINVAL, "edge_abs_mean_backward: NULL pointer");
    if ((s == nullptr) != (bw == nullptr))
        return fail(KANB200_EINVAL, "edge_abs_mean_backward: s and base_weight must both be given or both be absent");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e =
        dtype == KANB200_F32
            ? edge_abs_mean_bwd<float>((const float*)grad_a, (const float*)s, (const float*)H, (const float*)bw,
                                       (const float*)W, (float*)ds, (float*)dH, (float*)dbw, (float*)dW, N, (int)I,
                                       (int)O, R, ws_body(workspace, workspace_bytes),
                                       ws_body_bytes(workspace, workspace_bytes), st)
            : edge_abs_mean_bwd<double>((const double*)grad_a, (const double*)s, (const double*)H, (const double*)bw,
                                        (const double*)W, (double*)ds, (double*)dH, (double*)dbw, (double*)dW, N,
                                        (int)I, (int)O, R, ws_body(workspace, workspace_bytes),
                                        ws_body_bytes(workspace, workspace_bytes), st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "edge_abs_mean_backward");
}

KANB200_API int kanb200_refit_transfer(int dtype, const void* x, const void* grid_old, const void* grid_new,
                                       double* gram, double* transfer, int* info,
                                       int64_t N, int64_t I, int G, int k, void* stream) {
    int rc = kanb200_check_shapes(N, I, 1, G, k, dtype);
    if (rc) return rc;
    if (N < 1) return fail(KANB200_EINVAL, "refit_transfer: need at least one sample");
    if (!x || !grid_old || !grid_new || !gram || !transfer || !info)
        return fail(KANB200_EINVAL, "refit_transfer: NULL pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const int R = G + k;
    cudaError_t e = dtype == KANB200_F32
                        ? refit_moments<float>((const float*)x, (const float*)grid_old, (const float*)grid_new, gram,
                                               transfer, N, (int)I, R, k, st)
                        : refit_moments<double>((const double*)x, (const double*)grid_old, (const double*)grid_new,
                                                gram, transfer, N, (int)I, R, k, st);
    if (e == cudaSuccess) e = refit_solve(gram, transfer, info, (int)I, R, st);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "refit_transfer");
}

KANB200_API int kanb200_check_status(void* workspace, void* stream) {
    if (!workspace) return KANB200_OK;
    int code = 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(&code, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "check_status");
    if (code != 0) {
        cudaMemsetAsync(workspace, 0, sizeof(int), st);
        return fail(KANB200_EDEVICE, "a tensor-core kernel gave up waiting (status %d)", code);
    }
    return KANB200_OK;
}

KANB200_API int kanb200_allreduce_set_wait_limit_ms(int ms) {
    if (ms < 1 || ms > 600000) return fail(KANB200_EINVAL, "allreduce: wait limit must be between 1 ms and 10 min");
    allreduce_set_wait_limit_ms((unsigned)ms);
    return KANB200_OK;
}

KANB200_API size_t kanb200_allreduce_pad_bytes(int world, int blocks) {
    if (world < 1 || world > KANB200_MAX_RANKS || blocks < 1) return 0;
    return allreduce_pad_bytes(world, blocks);
}

KANB200_API int kanb200_allreduce_sum_f32_ranges(const void* const* peer_bases, void* multicast_base,
                                                 const size_t* offsets, const size_t* n_floats, int n_ranges,
                                                 size_t pad_offset, int rank, int world, int local_ranks,
                                                 int blocks, int threads, float scale, int* status, void* stream) {
    if (world < 1 || world > KANB200_MAX_RANKS)
        return fail(KANB200_EINVAL, "allreduce: world size %d outside [1, %d]", world, KANB200_MAX_RANKS);
    if (local_ranks < 1 || rank < 0 || rank + local_ranks > world)
        return fail(KANB200_EINVAL, "allreduce: ranks [%d, %d) outside world of size %d", rank, rank + local_ranks,
                    world);
    if (blocks < 1 || blocks > 1024) return fail(KANB200_EINVAL, "allreduce: blocks must be in [1, 1024]");
    if (threads < 32 || threads > 512 || threads % 32 != 0 || threads < world)
        return fail(KANB200_EINVAL, "allreduce: threads must be a multiple of 32 in [32, 512]");
    if (!peer_bases || !status) return fail(KANB200_EINVAL, "allreduce: peer_bases and status must not be NULL");
    for (int p = 0; p < world; ++p)
        if (!peer_bases[p]) return fail(KANB200_EINVAL, "allreduce: peer_bases[%d] is NULL", p);
    if (n_ranges < 1 || n_ranges > KANB200_MAX_SEGMENTS || !offsets || !n_floats)
        return fail(KANB200_EINVAL, "allreduce: between 1 and %d ranges", KANB200_MAX_SEGMENTS);
    const size_t pad = allreduce_pad_bytes(world, blocks);
    if (pad_offset % 4 != 0) return fail(KANB200_EINVAL, "allreduce: signal pad must be 4-byte aligned");
    for (int i = 0; i < n_ranges; ++i) {
        if (n_floats[i] % 4 != 0 || offsets[i] % 16 != 0)
            return fail(KANB200_EINVAL, "allreduce: n_floats must be a multiple of 4 and the payload 16-byte aligned");
        if (!(pad_offset >= offsets[i] + n_floats[i] * 4 || pad_offset + pad <= offsets[i]))
            return fail(KANB200_EINVAL, "allreduce: signal pad overlaps the payload");
    }
    if (multicast_base && local_ranks != 1)
        return fail(KANB200_EINVAL, "allreduce: several ranks in one launch use peer loads (multicast_base NULL)");
    cudaError_t e = allreduce_sum(const_cast<void* const*>(peer_bases), multicast_base, offsets, n_floats, n_ranges,
                                  pad_offset, rank, world, local_ranks, blocks, threads, scale, status,
                                  (cudaStream_t)stream);
    return e == cudaSuccess ? KANB200_OK : cuda_fail(e, "allreduce_sum");
}

KANB200_API int kanb200_allreduce_sum_f32(const void* const* peer_bases, void* multicast_base,
                                          size_t payload_offset, size_t pad_offset, size_t n_floats,
                                          int rank, int world, int local_ranks, int blocks, float scale,
                                          int* status, void* stream) {
    return kanb200_allreduce_sum_f32_ranges(peer_bases, multicast_base, &payload_offset, &n_floats, 1, pad_offset,
                                            rank, world, local_ranks, blocks, 512, scale, status, stream);
}

}  // extern "C"
