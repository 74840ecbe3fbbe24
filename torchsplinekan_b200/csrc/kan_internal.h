// Internal launcher interface between the C-ABI file and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace kanb200 {

struct LayerShape {
    int64_t N;      // samples
    int I, O;       // in / out features
    int G, K;       // grid intervals, spline order
    int R() const { return G + K; }
    int T() const { return G + 2 * K + 1; }
};

// ---- SIMT path (kan_simt.cu), T = float or double ---------------------------
template <typename T>
cudaError_t simt_basis(const T* x, const T* grid, T* H, const LayerShape& s, cudaStream_t st);
template <typename T>
cudaError_t simt_basis_grad(const T* x, const T* grid, const T* gH, T* gx, const LayerShape& s, cudaStream_t st);
template <typename T>
cudaError_t simt_forward(const T* x, const T* grid, const T* bw, const T* sw, const T* scaler, T* y,
                         const LayerShape& s, cudaStream_t st);
template <typename T>
size_t simt_backward_workspace(const LayerShape& s, bool need_param);
template <typename T>
cudaError_t simt_backward(const T* dY, const T* x, const T* grid, const T* bw, const T* sw, const T* scaler,
                          T* gx, T* gbw, T* gsw, T* gscaler, const LayerShape& s,
                          void* ws, size_t ws_bytes, cudaStream_t st);

// Sums `splits` partial parameter-gradient slabs and applies the scaler
// algebra: gsw = scaler * D, gscaler = sum_r sw * D, gbw = base slot.
// Element (o,i,r) of a slab sits at o*ldo + i*sI + r, its base slot at
// o*ldo + boff + i*sB.
template <typename T>
cudaError_t finalize_param_grads(const T* partial, int splits, int64_t split_stride,
                                 int64_t ldo, int sI, int64_t boff, int sB,
                                 const T* sw, const T* scaler, T* gsw, T* gscaler, T* gbw,
                                 int O, int I, int R, cudaStream_t st);

// ---- float64 layers on the FP64 matrix instruction (kan_dense64.cu) ----------
// From 512 rows on; workspace = status header, the weight image (forward, input gradient) and the
// per-split slabs of the parameter gradients, in that order.
bool dense64_supported(const LayerShape& s);
size_t dense64_workspace(bool forward, const LayerShape& s, bool need_x, bool need_param);
cudaError_t dense64_forward(const double* x, const double* grid, const double* bw, const double* sw,
                            const double* scaler, double* y, const LayerShape& s, void* ws, size_t ws_bytes,
                            cudaStream_t st);
cudaError_t dense64_backward(const double* dY, const double* x, const double* grid, const double* bw,
                             const double* sw, const double* scaler, double* gx, double* gbw, double* gsw,
                             double* gscaler, const LayerShape& s, void* ws, size_t ws_bytes, cudaStream_t st);

// Table-driven dense basis / basis gradient (float, R == 8, at most 12 knots, N >= 256, N I >= 2^21): `tab` is
// the polynomial table built by tc_build_table, `fs` its floats per feature.
bool basis_table_supported(const LayerShape& s);
cudaError_t simt_basis_table(const float* x, const float* tab, int fs, float* H, const LayerShape& s,
                             cudaStream_t st);
cudaError_t simt_basis_grad_table(const float* x, const float* tab, int fs, const float* gH, float* gx,
                                  const LayerShape& s, cudaStream_t st);

// ---- edge statistic (kan_reg.cu) -------------------------------------------
template <typename T>
size_t edge_workspace(int64_t N, int I, int O, int R, bool backward);
template <typename T>
cudaError_t edge_abs_mean_fwd(const T* s, const T* H, const T* bw, const T* W, T* a,
                              int64_t N, int I, int O, int R, void* ws, size_t ws_bytes, cudaStream_t st);
template <typename T>
cudaError_t edge_abs_mean_bwd(const T* ga, const T* s, const T* H, const T* bw, const T* W,
                              T* ds, T* dH, T* dbw, T* dW,
                              int64_t N, int I, int O, int R, void* ws, size_t ws_bytes, cudaStream_t st);

// Layers of at most 16 outputs (classifier heads, scalar outputs) on the FMA pipes: one kernel for the
// forward; one kernel for all gradients plus a small pass for the scaler algebra (per-split slabs, no
// atomics).  Any float type, k <= 3, at most 16 basis functions per feature.
bool narrow_layer_supported(int O, int R, int k);
template <typename T>
size_t narrow_layer_workspace(int64_t N, int I, int O, int R);
template <typename T>
cudaError_t narrow_layer_forward(const T* x, const T* grid, const T* bw, const T* sw, const T* scaler, T* y, int64_t N,
                                 int I, int O, int R, int k, cudaStream_t st);
template <typename T>
cudaError_t narrow_layer_backward(const T* dY, const T* x, const T* grid, const T* bw, const T* sw, const T* scaler,
                                  T* gx, T* gbw, T* gsw, T* gscaler, int64_t N, int I, int O, int R, int k, void* ws,
                                  size_t ws_bytes, cudaStream_t st);

// value = mu1 sum(a) + mu2 entropy(a / sum(a)) and its gradient with respect to a (NULL = not needed):
// the scalar head of the activation regulariser in one launch.
template <typename T>
cudaError_t edge_penalty(const T* a, int64_t n, double mu1, double mu2, T* value, T* grad, void* ws, size_t ws_bytes,
                         cudaStream_t st);
size_t edge_penalty_workspace_bytes();      // scratch of the two-launch form (without it: one block)

// The same operators straight from the layer input x (no H, no dH): see kan_reg.cu.  Scratch as for
// edge_abs_mean_fwd / _bwd.
template <typename T>
cudaError_t edge_abs_mean_x_fwd(const T* x, const T* s, const T* grid, const T* bw, const T* W, T* a,
                                int64_t N, int I, int O, int R, int k, void* ws, size_t ws_bytes, cudaStream_t st);
template <typename T>
cudaError_t edge_abs_mean_x_bwd(const T* ga, const T* x, const T* s, const T* grid, const T* bw, const T* W,
                                T* gx, T* ds, T* dbw, T* dW, int64_t N, int I, int O, int R, int k,
                                void* ws, size_t ws_bytes, cudaStream_t st);

// Fixed device scratch of the allocation-free edge statistic (kan_reg.cu).
size_t edge_static_scratch_bytes();
cudaError_t edge_static_scratch(void** ptr);

// ---- tensor-core path (kan_tc.cu), fp32 I/O ---------------------------------
bool tc_supported(const LayerShape& s);
size_t tc_workspace(int op, const LayerShape& s, bool need_x, bool need_param);
// Inference with fixed parameters: table + weight image built once into a caller-owned buffer
// (tc_prepare_forward), then only the contraction per call (tc_forward_prepared; ws = status header).
size_t tc_prepared_bytes(const LayerShape& s, bool has_base);
cudaError_t tc_prepare_forward(const float* grid, const float* bw, const float* sw, const float* scaler,
                               const LayerShape& s, void* prepared, size_t prepared_bytes, cudaStream_t st);
cudaError_t tc_forward_prepared(int split_terms, const float* x, const void* prepared, size_t prepared_bytes,
                                bool has_base, float* y, const LayerShape& s, void* ws, size_t ws_bytes,
                                cudaStream_t st);
cudaError_t tc_forward(int split_terms, const float* x, const float* grid, const float* bw, const float* sw,
                       const float* scaler, float* y, const LayerShape& s,
                       void* ws, size_t ws_bytes, cudaStream_t st);
// ldy = row stride of dY in elements (s.O for a dense matrix; larger when the call covers a range
// of output columns of a wider matrix)
cudaError_t tc_backward(int split_terms, const float* dY, int64_t ldy, const float* x, const float* grid,
                        const float* bw, const float* sw, const float* scaler, float* gx, float* gbw, float* gsw,
                        float* gscaler, const LayerShape& s, void* ws, size_t ws_bytes, cudaStream_t st);

// Shortens the accumulation chains of the tensor-core kernels (values above the built-in lengths
// are clamped to them; 0 keeps the current value).
void tc_set_chunks(int fwd_kb, int bwd_kb, int dx_kb);

// Forward kernel variant: -1 = chosen by shape (tensor-memory operand for up to 256 outputs), 0 = generated
// operand in shared memory, 1 = in tensor memory.
void tc_set_forward_variant(int v);

// The per-span polynomial table on its own: bytes, floats per feature, and the kernel that fills it.
size_t tc_table_bytes(const LayerShape& s);
int tc_table_stride(const LayerShape& s);
cudaError_t tc_build_table(const float* grid, float* tab, const LayerShape& s, cudaStream_t st);

// Edge statistic straight from x on the tensor cores (kan_tc_edge.cu): float32, G + k <= 8.
// W is the effective coefficient tensor (scaler applied); s_val, when not NULL, replaces silu(x).
bool tc_edge_supported(const LayerShape& s);
size_t tc_edge_workspace(const LayerShape& s);
cudaError_t tc_edge_forward(int split_terms, const float* x, const float* s_val, const float* grid, const float* bw,
                            const float* W, float* a, const LayerShape& s, void* ws, size_t ws_bytes,
                            cudaStream_t st);

// Backward of the same statistic on the tensor cores: float32, G + k <= 8, at most 256 outputs,
// SiLU or no base branch.  gx, dbw, dW may be NULL.
bool tc_edge_bwd_supported(const LayerShape& s);
size_t tc_edge_bwd_workspace(const LayerShape& s, bool need_x);
cudaError_t tc_edge_backward(const float* ga, const float* x, const float* grid, const float* bw, const float* W,
                             float* gx, float* dbw, float* dW, const LayerShape& s, void* ws, size_t ws_bytes,
                             cudaStream_t st);

// Whether the backward kernel evaluates a phi whose tensor-core value is at rounding level again in
// float32 before taking its sign (default: yes).
void tc_edge_set_sign_recheck(bool on);
bool tc_edge_get_sign_recheck();

// Coefficient refit after a knot update (kan_refit.cu): per-feature moment matrices
// G = sum b_new b_new^T, M = sum b_new b_old^T (float64 [I, R, R]) and the in-place solve X = G^-1 M.
template <typename T>
cudaError_t refit_moments(const T* x, const T* grid_old, const T* grid_new, double* Gm, double* Mm, int64_t N, int I,
                          int R, int k, cudaStream_t st);
cudaError_t refit_solve(double* Gm, double* Mm, int* info, int I, int R, cudaStream_t st);

// Gradient all-reduce over symmetric memory (kan_collective.cu).
size_t allreduce_pad_bytes(int world, int blocks);
void allreduce_set_wait_limit_ms(unsigned ms);
cudaError_t allreduce_sum(void* const* peer_bases, void* multicast_base, const size_t* offsets, const size_t* n_floats,
                          int n_segments, size_t pad_off, int rank, int world, int local_ranks, int blocks,
                          int threads, float scale, int* status, cudaStream_t st);

// Workspaces start with a 256-byte header whose first word is a status code
// written by kernels whose bounded waits ran out.  The word is sticky: kernels
// only ever change it from 0 to a code, and only kanb200_check_status clears it.
constexpr size_t kWsHeader = 256;

}  // namespace kanb200
