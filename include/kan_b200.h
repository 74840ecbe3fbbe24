/*
 * kan_b200.h -- C ABI of the B200 (sm_100a) KANLinear hot path.
 *
 * Every entry point takes raw DEVICE pointers, plain sizes and a CUDA stream
 * (passed as void*, 0 = default stream), launches on that stream without
 * synchronising, and returns 0 on success or a negative KANB200_E* code.
 * kanb200_last_error() returns the message of the calling thread's last
 * failure.  Nothing here allocates device memory: scratch space is provided
 * by the caller (size from kanb200_workspace_bytes).  There is no CPU path.
 *
 * Shapes (row-major, contiguous):  x [N,I], grid [I,T] with T = G+2k+1,
 * base_weight [O,I], spline_weight [O,I,R] with R = G+k, spline_scaler [O,I],
 * y / grad_out [N,O], basis H [N,I,R].  dtype: KANB200_F32 or KANB200_F64.
 * A NULL base_weight / spline_scaler pointer means "absent" (the reference
 * passes an empty tensor: csrc/kan_ops.h:22-24).
 *
 * Each declaration cites the function of the reference project
 * (yefanliuming/TORCHSPLINEKAN) that it replaces.
 */
#ifndef KAN_B200_H
#define KAN_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define KANB200_API __attribute__((visibility("default")))
#else
#define KANB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define KANB200_F32 0
#define KANB200_F64 1

/* Arithmetic used for the contraction (fp32 inputs only; fp64 always SIMT). */
#define KANB200_MODE_AUTO     0  /* tensor cores when the shape allows, else SIMT   */
#define KANB200_MODE_SIMT     1  /* fp32/fp64 FMA pipes, gathers the k+1 non-zeros   */
#define KANB200_MODE_TC_BF16X3 2 /* tcgen05, operands split hi+lo bf16, 3 MMAs/step  */
#define KANB200_MODE_TC_BF16X1 3 /* tcgen05, single bf16 MMA (fast, ~3e-3 relative)  */

#define KANB200_OK            0
#define KANB200_EINVAL       -1  /* bad argument (shape, limit, NULL, dtype)         */
#define KANB200_EUNSUPPORTED -2  /* valid request the chosen mode cannot run         */
#define KANB200_EWORKSPACE   -3  /* workspace missing or too small                   */
#define KANB200_ECUDA        -4  /* CUDA runtime error at launch                     */
#define KANB200_EDEVICE      -5  /* a kernel reported a timed-out wait (status word) */

/* Limits shared with the reference (csrc/kan_ops.h:15-17). */
#define KANB200_MAX_DEG0_BASIS  71     /* G + 2k                          */
#define KANB200_MAX_IN_FEATURES 65535

#define KANB200_OP_FORWARD  0
#define KANB200_OP_BACKWARD 1
#define KANB200_OP_EDGE_FWD 2
#define KANB200_OP_EDGE_BWD 3
#define KANB200_OP_BASIS    4  /* kanb200_basis_ws / kanb200_basis_grad_ws (O is ignored) */
#define KANB200_OP_EDGE_X_FWD 5 /* kanb200_edge_abs_mean_x */
#define KANB200_OP_EDGE_X_BWD 6 /* kanb200_edge_abs_mean_x_backward */

KANB200_API const char* kanb200_last_error(void);
KANB200_API int kanb200_version(void);

/* Process-global basis-kernel selector kept for API compatibility
 * (kan_set_basis_impl / kan_get_basis_impl, csrc/kan_cuda.cu:274-279):
 * 0 and 1 are accepted (both run the local k+1 evaluation here), anything
 * else is KANB200_EINVAL. */
KANB200_API int kanb200_set_basis_impl(int impl);
KANB200_API int kanb200_get_basis_impl(void);

/* The tensor-core accumulator truncates on every accumulation, so long reductions are cut into
 * chains whose partial results are added in float32 with round-to-nearest.  The built-in chain
 * lengths (forward: 24 blocks of 64 columns; parameter gradients: 16 blocks of 64 samples; input
 * gradient: 24 blocks of 64 outputs) hold the stated 1e-5 tolerance.  This call can only SHORTEN
 * them (larger values are clamped, 0 keeps a value): more accurate, slightly slower.  Process-wide.
 * No counterpart in the reference (its GEMMs are cuBLAS calls). */
KANB200_API int kanb200_set_accumulation_chunks(int forward_blocks, int param_blocks, int input_blocks);

/* Shape / limit validation run by every entry point before any launch
 * (kan_check_inputs, csrc/kan_ops.h:27-78). */
KANB200_API int kanb200_check_shapes(int64_t N, int64_t I, int64_t O, int G, int k, int dtype);

/* The kernel family a call takes: what KANB200_MODE_AUTO resolves to for this problem (a given mode is
 * only validated).  The rule differs by direction -- op = KANB200_OP_FORWARD or KANB200_OP_BACKWARD --
 * because the gather forward loses to the tensor cores on much smaller problems than the gather
 * backward does.  kanb200_resolve_mode is the backward rule (kept for existing callers). */
KANB200_API int kanb200_resolve_mode_for(int op, int mode, int dtype, int64_t N, int64_t I, int64_t O, int G, int k);
KANB200_API int kanb200_resolve_mode(int mode, int dtype, int64_t N, int64_t I, int64_t O, int G, int k);

/* Bytes of caller-provided scratch the given op needs (0 = none). */
KANB200_API size_t kanb200_workspace_bytes(int op, int mode, int dtype,
                               int64_t N, int64_t I, int64_t O, int G, int k,
                               int need_x, int need_param);

/* H[n,i,r] = B_{r,k}(x[n,i]) on knots grid[i,:]
 * (kan_basis_cuda, csrc/kan_cuda.cu:666-680). */
KANB200_API int kanb200_basis(int dtype, const void* x, const void* grid, void* H,
                  int64_t N, int64_t I, int G, int k, void* stream);

/* gx[n,i] = sum_r gH[n,i,r] dB_r/dx
 * (kan_basis_grad_cuda, csrc/kan_cuda.cu:682-699). */
/* The same two operators with caller scratch (kanb200_workspace_bytes(KANB200_OP_BASIS, ...)):
 * float32 inputs with G + k = 8 then run from a per-span polynomial table built into the scratch
 * (about twice the rate of the recurrence); anything else, or a NULL / short workspace, behaves
 * exactly like the calls without scratch. */
KANB200_API int kanb200_basis_ws(int dtype, const void* x, const void* grid, void* H, int64_t N, int64_t I, int G,
                                 int k, void* workspace, size_t workspace_bytes, void* stream);
KANB200_API int kanb200_basis_grad_ws(int dtype, const void* x, const void* grid, const void* gH, void* gx,
                                      int64_t N, int64_t I, int G, int k, void* workspace, size_t workspace_bytes,
                                      void* stream);

KANB200_API int kanb200_basis_grad(int dtype, const void* x, const void* grid, const void* gH, void* gx,
                       int64_t N, int64_t I, int G, int k, void* stream);

/* y = silu(x) bw^T + H(x) (spline_weight * spline_scaler)^T, basis never
 * materialised (kan_forward_cuda, csrc/kan_cuda.cu:469-532; the dense basis
 * output of that function is produced separately by kanb200_basis). */
KANB200_API int kanb200_forward(int dtype, int mode,
                    const void* x, const void* grid, const void* base_weight,
                    const void* spline_weight, const void* spline_scaler,
                    void* y, int64_t N, int64_t I, int64_t O, int G, int k,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Inference with fixed parameters (the use export_inference serves, spline_kan/kan_linear.py:471-496:
 * the scaler folded into the coefficients once).  Here everything that depends on the parameters
 * only -- the per-span polynomial table of the knots and the bf16 hi/lo image of the effective
 * weights (base_weight columns included) -- is built ONCE into a caller-owned device buffer and every
 * later call runs the contraction alone: one launch per layer instead of three.
 *   kanb200_prepared_bytes    size of that buffer; 0 = no prepared form for this configuration
 *                             (float64, k > 3): use kanb200_forward
 *   kanb200_prepare_forward   fills it (base_weight / spline_scaler may be NULL as in kanb200_forward)
 *   kanb200_forward_prepared  y = layer(x) from x and the buffer; has_base must repeat whether
 *                             base_weight was given; mode AUTO / TC_BF16X3 / TC_BF16X1; workspace:
 *                             kanb200_workspace_bytes(KANB200_OP_FORWARD, KANB200_MODE_TC_BF16X3, ...)
 *                             bytes, at least the 256-byte status header (with less than that figure a
 *                             small batch runs the chains of a tile one after the other instead of
 *                             side by side).  Same results as kanb200_forward in the same
 *                             tensor-core mode and with the same workspace size, bit for bit. */
KANB200_API size_t kanb200_prepared_bytes(int dtype, int64_t I, int64_t O, int G, int k, int has_base);
KANB200_API int kanb200_prepare_forward(int dtype, const void* grid, const void* base_weight,
                                        const void* spline_weight, const void* spline_scaler, int64_t I, int64_t O,
                                        int G, int k, void* prepared, size_t prepared_bytes, void* stream);
KANB200_API int kanb200_forward_prepared(int dtype, int mode, const void* x, const void* prepared,
                                         size_t prepared_bytes, int has_base, void* y, int64_t N, int64_t I,
                                         int64_t O, int G, int k, void* workspace, size_t workspace_bytes,
                                         void* stream);

/* First-order backward; any of the four outputs may be NULL = not needed
 * (kan_backward_cuda_ex, csrc/kan_cuda.cu:537-630).  The basis is recomputed
 * from x, nothing saved by the forward is required. */
KANB200_API int kanb200_backward(int dtype, int mode, const void* grad_out,
                     const void* x, const void* grid, const void* base_weight,
                     const void* spline_weight, const void* spline_scaler,
                     void* grad_x, void* grad_base_weight,
                     void* grad_spline_weight, void* grad_spline_scaler,
                     int64_t N, int64_t I, int64_t O, int G, int k,
                     void* workspace, size_t workspace_bytes, void* stream);

/* a[o,i] = mean_n | s[n,i] bw[o,i] + sum_r H[n,i,r] W[o,i,r] |; s and bw may
 * both be NULL (edge_abs_mean_cuda, csrc/kan_reg_cuda.cu:263-280).  No atomics:
 * per-split partial sums go to the workspace and are reduced in a fixed order. */
KANB200_API int kanb200_edge_abs_mean(int dtype, const void* s, const void* H, const void* bw, const void* W,
                          void* a, int64_t N, int64_t I, int64_t O, int R,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Same result as kanb200_edge_abs_mean, for callers that cannot hand over scratch memory.
 * No counterpart in the reference.  Some hosts plan all device memory ahead of time -- a serving
 * process that gives its whole heap to a static planner at start-up, a plugin interface that only
 * passes the tensors of the operator -- and have nothing to allocate a workspace from when the
 * call is made.  For them the per-split partial sums go to a 4 MiB buffer built into the library
 * (a file-scope __device__ array: every GPU that loads the library keeps it until the process
 * exits).  Limits and rules:
 *   - shapes whose partial sums need more than 4 MiB (splits * O * I * sizeof(dtype); see
 *     kanb200_workspace_bytes(KANB200_OP_EDGE_FWD, ...) minus its 256-byte header) are refused
 *     with KANB200_EWORKSPACE and a message; nothing is launched;
 *   - the call itself allocates nothing (no cudaMalloc / cudaFree, no allocating library call);
 *   - the first call on each device looks up the buffer's device address (cudaGetSymbolAddress,
 *     with that device current) and caches it; make that first call during set-up, before any
 *     stream capture is started;
 *   - all calls on a device share the one buffer, which keeps the previous call's contents.
 *     Every slot a call reads is written earlier by the same call, so nothing needs clearing,
 *     but two calls that overlap on the GPU (different streams) race on it: serialise them. */
KANB200_API int kanb200_edge_abs_mean_noalloc(int dtype, const void* s, const void* H, const void* bw,
                                              const void* W, void* a,
                                              int64_t N, int64_t I, int64_t O, int R, void* stream);

/* The same statistic evaluated straight from the layer input, the basis never stored:
 *     a[o,i] = mean_n | s[n,i] bw[o,i] + sum_r B_r(x[n,i]) W[o,i,r] |
 * with s = silu(x) when s is NULL (and bw given), or the caller's base values s [N,I] (layers with
 * another base activation); bw NULL = no base term.  W [O,I,R] is the effective coefficient
 * tensor (spline_weight * spline_scaler).  Replaces the pair kan_basis_cuda + edge_abs_mean_cuda
 * of the reference's forward_with_regularization (spline_kan/kan_linear.py:381-416,
 * csrc/kan_reg_cuda.cu:263-280) without the [N,I,R] intermediate.  float32 with G + k <= 8 runs
 * on the tensor cores (one K = 16 MMA step per feature, |phi| summed from tensor memory); other
 * shapes and float64 run on the FMA pipes.  mode as for kanb200_forward. */
KANB200_API int kanb200_edge_abs_mean_x(int dtype, int mode, const void* x, const void* s, const void* grid,
                                        const void* bw, const void* W, void* a,
                                        int64_t N, int64_t I, int64_t O, int G, int k,
                                        void* workspace, size_t workspace_bytes, void* stream);

/* Gradients of kanb200_edge_abs_mean_x for the incoming grad_a [O,I]; NULL output = not needed:
 *   gx [N,I]   input gradient through the basis (sum_r dH dB_r/dx), plus ds * silu'(x) when s is NULL;
 *   ds [N,I]   gradient of the caller's base values (only when s is given);
 *   dbw [O,I], dW [O,I,R]  parameter gradients (dW with respect to the effective coefficients).
 * The [N,I,R] tensors H and dH of edge_abs_mean_backward_cuda + kan_basis_grad_cuda
 * (csrc/kan_reg_cuda.cu:284-312, csrc/kan_cuda.cu:682-699) are never formed.  No atomics.
 * float32 with G + k <= 8, at most 256 outputs and s == NULL runs on the tensor cores: sign(phi) is
 * written to shared memory as an exact bf16 operand and both gradients are two more small matrix
 * products per feature, chained behind the one that forms phi.  Other cases run on the FMA pipes.
 * mode as for kanb200_forward (the two tensor-core modes select the same kernel here: the sign of
 * phi is always taken from the three-term product). */
KANB200_API int kanb200_edge_abs_mean_x_backward(int dtype, int mode, const void* grad_a, const void* x, const void* s,
                                                 const void* grid, const void* bw, const void* W,
                                                 void* gx, void* ds, void* dbw, void* dW,
                                                 int64_t N, int64_t I, int64_t O, int G, int k,
                                                 void* workspace, size_t workspace_bytes, void* stream);

/* The tensor-core backward takes sign(phi) from a split-bf16 product, which gives phi to about 5e-6 of
 * its terms.  With the re-check on (the default) a phi below 2e-5 of a bound on its terms is evaluated
 * again in float32 before its sign is taken, so the gradients are those of a float32 evaluation
 * (relative L2 error against float64 3e-7 instead of 7e-5 .. 2e-4); switching it off makes the kernel
 * about a third faster.  Process-wide; returns KANB200_OK. */
KANB200_API int kanb200_set_edge_sign_recheck(int on);

/* Scalar head of the activation regulariser from the per-edge statistic a (n = O*I entries, any shape):
 *   value[0] = mu1 * A + mu2 * S,  A = sum a,  p = max(a / max(A, tiny), tiny),  S = -sum p log p,
 *   grad[j]  = d value / d a_j = mu1 - mu2 (log p_j + S) / A   (NULL = not needed)
 * (regularization_from_edge_means, spline_kan/reference_backend.py:149-170, which the reference
 * evaluates as a chain of tensor operations and differentiates through autograd).  Sums in float64;
 * tiny = the dtype's smallest normal, as in the reference's clamps.  With a workspace of
 * kanb200_edge_penalty_workspace_bytes() bytes (plain scratch, no status header) two launches share
 * the work over the whole GPU; with workspace == NULL, or fewer than 4096 entries, one block does it
 * all in one launch. */
KANB200_API size_t kanb200_edge_penalty_workspace_bytes(void);
KANB200_API int kanb200_edge_penalty(int dtype, const void* a, int64_t n, double mu1, double mu2, void* value,
                                     void* grad, void* workspace, size_t workspace_bytes, void* stream);

/* Which tensor-core forward kernel runs (same results): 1 = the generated operand is stored in tensor
 * memory and the MMA reads it from there (shared memory only carries the weight tiles; one
 * 256-output tile per generated tile), 0 = generated operand in shared memory, two 256-output
 * sub-tiles per generated tile, -1 (default) = by shape: tensor memory for up to 256 outputs.
 * Process-wide. */
KANB200_API int kanb200_set_forward_variant(int variant);
KANB200_API int kanb200_get_edge_sign_recheck(void);

/* Gradients of kanb200_edge_abs_mean; NULL output = not needed
 * (edge_abs_mean_backward_cuda, csrc/kan_reg_cuda.cu:284-312). */
KANB200_API int kanb200_edge_abs_mean_backward(int dtype, const void* grad_a,
                                   const void* s, const void* H, const void* bw, const void* W,
                                   void* ds, void* dH, void* dbw, void* dW,
                                   int64_t N, int64_t I, int64_t O, int R,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* Coefficient refit after the knots of a layer moved: the least-squares part of update_grid
 * (ReferenceKANLayer.update_grid + curve2coeff, spline_kan/reference_backend.py:218-265, 442-493, where
 * every old curve is sampled at every input into an [O, B, I] tensor and one system per feature is
 * solved on the CPU).  For samples x [N,I] and knot rows grid_old / grid_new [I, G+2k+1] it returns, per
 * input feature, the float64 matrix  transfer[i] = G_i^-1 M_i  [R, R]  with
 *     G_i = sum_n b_new(x[n,i]) b_new(x[n,i])^T,   M_i = sum_n b_new(x[n,i]) b_old(x[n,i])^T,
 * so that the refitted coefficients of EVERY output are  c_new[o,i,:] = transfer[i] c_old[o,i,:]
 * (the normal equations of fitting the new basis to the old curve at the samples; the curves
 * themselves are never formed).  gram [I,R,R] receives the Cholesky factors (scratch).  info[i] != 0
 * marks a feature whose G_i is not safely positive definite (a pivot below 1e-10 of its largest
 * diagonal entry: too few distinct samples for some basis function); its transfer matrix is not
 * valid and the caller refits that feature by a minimum-norm solver.  All device pointers. */
KANB200_API int kanb200_refit_transfer(int dtype, const void* x, const void* grid_old, const void* grid_new,
                                       double* gram, double* transfer, int* info,
                                       int64_t N, int64_t I, int G, int k, void* stream);

/* Reads (and clears) the status word the tensor-core kernels keep at the start
 * of a workspace; synchronises the stream.  0 = every wait completed.  The word
 * is sticky: kernels only change it from 0 to a code and nothing but this call
 * clears it, so a timed-out wait in one call is still reported after any number
 * of later calls on the same workspace.  The caller zeroes the first 256 bytes
 * of a workspace once, before its first use.  Bytes 8..15 of that header may hold a
 * device-accessible pointer to an int (e.g. in mapped pinned host memory) that a reporting kernel
 * also sets, so that a host can notice a report without synchronising; NULL (the zeroed header) =
 * none.  (No counterpart in the reference, whose kernels have no waits.) */
KANB200_API int kanb200_check_status(void* workspace, void* stream);

/* Parameter gradients of the output rows [o_begin, o_end) only (tensor-core modes, float32): the
 * pointers are those of the FULL tensors as in kanb200_backward; rows outside the range are not
 * touched.  Calling it range by range lets a data-parallel host start the all-reduce of one
 * range while the next is being computed.  Workspace as for kanb200_backward with need_param. */
KANB200_API int kanb200_backward_param_rows(int mode, const void* grad_out, const void* x, const void* grid,
                                            const void* base_weight, const void* spline_weight,
                                            const void* spline_scaler, void* grad_base_weight,
                                            void* grad_spline_weight, void* grad_spline_scaler,
                                            int64_t N, int64_t I, int64_t O, int G, int k,
                                            int64_t o_begin, int64_t o_end,
                                            void* workspace, size_t workspace_bytes, void* stream);

/* ---- data-parallel gradient all-reduce over NVLink (no counterpart in the reference, which
 * is single-device; it is what batch-sharded training of KANLinear needs after
 * kanb200_backward) ------------------------------------------------------------------------
 * Every rank owns one allocation of the same size that every rank of the node has mapped
 * ("symmetric" memory: cuMem / IPC peer mappings, e.g. torch.distributed._symmetric_memory):
 *     [payload_offset, +n_floats*4)   float32 gradients (n_floats a multiple of 4, 16-byte aligned)
 *     [pad_offset, +kanb200_allreduce_pad_bytes(world, blocks))   signal words, zero before first use
 * One call per rank, on its own stream, replaces every rank's payload with `scale` times the sum
 * over the ranks.  peer_bases[p] is THIS process's mapping of rank p's allocation (world entries,
 * host array).  multicast_base, when not NULL, is a multicast mapping of the same allocations
 * (NVSwitch): the kernel then reduces in the switch (multimem.ld_reduce / multimem.st);
 * otherwise the owner of each slice loads it from every peer and stores the sum to every peer.
 * local_ranks > 1 runs ranks rank .. rank+local_ranks-1 of ONE device inside a single launch
 * (peer loads only) - the way to exercise the protocol on one GPU.  *status (device int) is set
 * to 1 when a bounded wait on another rank ran out (kanb200_allreduce_set_wait_limit_ms); the pad
 * must then be zeroed. */
#define KANB200_MAX_RANKS 16
#define KANB200_MAX_SEGMENTS 4
KANB200_API size_t kanb200_allreduce_pad_bytes(int world, int blocks);
/* How long a rank waits for another one inside the kernel before it gives up with *status = 1
 * (process-wide; default 10 s). */
KANB200_API int kanb200_allreduce_set_wait_limit_ms(int ms);
KANB200_API int kanb200_allreduce_sum_f32(const void* const* peer_bases, void* multicast_base,
                                          size_t payload_offset, size_t pad_offset, size_t n_floats,
                                          int rank, int world, int local_ranks, int blocks, float scale,
                                          int* status, void* stream);

/* The same reduction over up to KANB200_MAX_SEGMENTS ranges of the allocation in one launch
 * (offsets[i] bytes from the base, n_floats[i] floats), with `threads` threads per block (a
 * multiple of 32 up to 512; 128 lets a block share an SM with one of the tensor-core kernels). */
KANB200_API int kanb200_allreduce_sum_f32_ranges(const void* const* peer_bases, void* multicast_base,
                                                 const size_t* offsets, const size_t* n_floats, int n_ranges,
                                                 size_t pad_offset, int rank, int world, int local_ranks,
                                                 int blocks, int threads, float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KAN_B200_H */
