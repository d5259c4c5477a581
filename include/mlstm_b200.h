/* C ABI of the B200 mLSTM kernel library (libmlstm_b200.so).
 *
 * Plain pointers and sizes only.  Every pointer is a DEVICE pointer unless stated otherwise; all
 * tensors are contiguous row-major, [B, NH, S, D] for q, k, v, o, h and their gradients and
 * [B, NH, S] for f, i, m, b and their gradients (the reference's hand-computed offsets,
 * mlstm_matmul.py:46-55).  Every entry point only enqueues work on `stream` (a cudaStream_t passed
 * as void*; NULL = the default stream) and returns at once with 0 or a negative MLSTM_E_* code; it
 * never prints, aborts or synchronises.  Scratch memory is a caller-owned workspace whose size the
 * matching *_workspace() function reports (pass it the same flags as the call: fp32 inputs on the
 * tensor cores need room for converted copies of the operands).  Between calls the library keeps no
 * device state of its own, with one exception: mlstm_forward_f16_static() works in a fixed array
 * inside the library's device image (see there).  Host-side caches (tensor-map encoder entry point,
 * per-device kernel attributes) are guarded for concurrent callers.
 * The first 256 bytes of a workspace hold a device status word that kernels set when they give up on
 * an internal wait; mlstm_read_status() copies it to the host (this one call synchronises the stream);
 * mlstm_forward_f16_static_status() does the same for the built-in array.
 */
#ifndef MLSTM_B200_H
#define MLSTM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define MLSTM_DT_F32 0
#define MLSTM_DT_F16 1
#define MLSTM_DT_BF16 2

/* status codes */
#define MLSTM_OK 0
#define MLSTM_E_ARG (-1)         /* null pointer, non-positive size, unknown dtype or flag      */
#define MLSTM_E_SHAPE (-2)       /* shape outside what the kernels accept                        */
#define MLSTM_E_ALIGN (-3)       /* a tensor pointer is not 16-byte aligned                      */
#define MLSTM_E_UNSUPPORTED (-4) /* the tensor-core path was demanded for a case it cannot do    */
#define MLSTM_E_WORKSPACE (-5)   /* workspace missing or too small                               */
#define MLSTM_E_CUDA (-6)        /* a CUDA runtime or driver call failed                         */
#define MLSTM_E_TIMEOUT (-7)     /* a kernel gave up on an internal wait (see mlstm_read_status) */
#define MLSTM_E_STATIC_LIMIT (-8) /* S beyond what mlstm_forward_f16_static's built-in scratch holds */

/* flags */
#define MLSTM_F_FORCE_SIMT 1 /* use the CUDA-core kernels even where the tensor-core path applies */
#define MLSTM_F_FORCE_TC 2   /* fail with MLSTM_E_UNSUPPORTED instead of using the CUDA-core path */
#define MLSTM_F_ALLOW_TF32 4 /* fp32 inputs may use the tensor cores with single tf32 products (fp32 accumulate,
                                error about 5e-4).  Without it fp32 inputs keep fp32-level accuracy, as the
                                reference's tl.dot(..., allow_tf32=False) (mlstm_matmul.py:19): for D = 64 and
                                128 on the tensor cores with every operand split into two bf16 halves and three
                                products per fp32 product (error about 1e-5), else IEEE fp32 on the CUDA cores */
#define MLSTM_F_NO_SPLIT 8   /* fp32 inputs: do not use the split tensor-core form (IEEE fp32 on the CUDA cores) */

const char* mlstm_status_string(int status);
/* Text of the last CUDA failure behind an MLSTM_E_CUDA on this host thread (which call, which error). */
const char* mlstm_last_error_detail(void);

/* Whether the tcgen05 path handles this case (D in {64, 128, 256}): 1 for 16-bit inputs, 2 for fp32
 * inputs (single tf32 products with MLSTM_F_ALLOW_TF32; split bf16 products by default at D = 64, 128), else 0.
 * The scan entry, the parallel forward (float32 h) and the parallel backward also take D = 512 .. 4096 in multiples
 * of 256 on the tensor cores (two passes: gated S x S matrices to scratch, then plain contractions). */
int mlstm_tc_supported(int S, int D, int dtype);

/* Parallel (matmul) forward.
 * Replaces the launch in Triton_mLSTM.forward / mlstm_matmul (mlstm_matmul.py:121-129, 371-381) of
 * mlstm_matmul_kernel (mlstm_matmul.py:37-101).
 *   q, k, v [B,NH,S,D], f, i [B,NH,S] of `dtype`; h [B,NH,S,D] of `h_dtype` (MLSTM_DT_F32 as the
 *   reference's Python path, or the input type); m, b [B,NH,S] fp32 (the reference's saved M, B).
 * D in {64, 128, 256}: one fused pass.  D = 512 .. 4096 in multiples of 256 with float32 h (16-bit inputs, or
 * float32 inputs with MLSTM_F_ALLOW_TF32): two tensor-core passes; the workspace then holds the gated matrices
 * of as many slices as fit 512 MB at once.  Everything else: the CUDA-core kernels.
 */
size_t mlstm_mm_fwd_workspace(int B, int NH, int S, int D, int dtype, int flags);
int mlstm_mm_fwd(const void* q, const void* k, const void* v, const void* f, const void* i, void* h, float* m,
                 float* b, void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype,
                 int h_dtype, int flags, void* stream);

/* Parallel (matmul) backward.
 * Replaces the three launches of Triton_mLSTM.backward (mlstm_matmul.py:383-405):
 * mlstm_matmul_kernel_backward_db (:132-197), mlstm_matmul_kernel_backward (:200-316) and
 * mlstm_matmul_kernel_df (:319-333).
 *   dh, h of `h_dtype`; q, k, v, f, i and the outputs dq, dk, dv, df, di of `dtype`; m, b fp32 as
 *   written by mlstm_mm_fwd.  df[..., 0] is exactly 0 (mlstm_matmul.py:316, 392).
 * D in {64, 128, 256}: three fused passes (dQ, dK, dV).  D = 512 .. 4096 in multiples of 256 (16-bit inputs, or
 * float32 inputs with MLSTM_F_ALLOW_TF32): the normalised gated matrix and its gradient go to scratch (as many
 * slices at once as fit 512 MB), then dQ = dT K, dK = dT^T Q, dV = W^T dH as plain contractions: five
 * contractions in all.  Everything else: the CUDA-core kernels.
 */
size_t mlstm_mm_bwd_workspace(int B, int NH, int S, int D, int dtype, int h_dtype, int flags);
int mlstm_mm_bwd(const void* dh, const void* q, const void* k, const void* v, const void* f, const void* i,
                 const void* h, const float* m, const float* b, void* dq, void* dk, void* dv, void* df, void* di,
                 void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int h_dtype,
                 int flags, void* stream);

/* Forward scan with output gate: h = mLSTM(q, k, v, f, i) * silu(o).
 * Replaces the four launches of mlstm_scan (mlstm_scan.py:281-327): stabilize_fi (:47-69),
 * precompute_mlstm_triton_scan (:74-137), reduce_mlstm_triton (:143-195), mlstm_triton_scan
 * (:200-278).  q, k, v, o [B,NH,S,D], f, i [B,NH,S] of `dtype`; h fp32 [B,NH,S,D].
 * Three forms, chosen by shape: head dimensions above 256 (the reference demo, D = 1024) run as two
 * tensor-core passes (gated S x S matrix once, then W V); sequences much longer than the head dimension
 * run chunkwise (per-block states, inter-block carry, output from the carried state; 16-bit, D = 128 or 256);
 * everything else is the parallel forward with the output gate in its epilogue.
 */
size_t mlstm_scan_fwd_workspace(int B, int NH, int S, int D, int dtype, int flags);
int mlstm_scan_fwd(const void* q, const void* k, const void* v, const void* f, const void* i, const void* o,
                   void* h, void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype,
                   int flags, void* stream);

/* Output gate as a step of its own, for the training path: h = h_inner * silu(o) and its derivative
 * dh_inner = dh * silu(o), d_o = dh * h_inner * silu'(o), over n elements (what the reference leaves open at
 * mlstm_matmul.py:36 "Integrate o" and computes only in the forward scan, mlstm_scan.py:273-278).
 * h_inner, h, dh, dh_inner of `h_dtype`; o, d_o of `o_dtype` (h_dtype fp32 with any o_dtype, or both equal). */
int mlstm_ogate_fwd(const void* h_inner, const void* o, void* h, long long n, int h_dtype, int o_dtype, void* stream);
int mlstm_ogate_bwd(const void* dh, const void* h_inner, const void* o, void* dh_inner, void* d_o, long long n, int h_dtype,
                    int o_dtype, void* stream);

/* Single-head fp16 forward of the C++ driver.
 * Replaces the launch mlstm_forward<64,16,128,16,8,8><<<S/64,128,smem>>>(Q,K,V,F,I,H,S)
 * (cuda-src/mlstm_forward.cu:12-15, 235-238).  Q, K, V, H [S,D] half, F, I [S] half.
 */
size_t mlstm_forward_f16_workspace(unsigned S, unsigned D);
int mlstm_forward_f16(const void* Q, const void* K, const void* V, const void* F, const void* I, void* H,
                      unsigned S, unsigned D, void* workspace, size_t workspace_bytes, void* stream);

/* Single-head fp16 backward of the C++ driver, complete: dQ, dK, dV [S,D] half and dF, dI [S] half from
 * dH, Q, K, V [S,D] half and F, I [S] half.
 * Replaces the two launches matmul_backward_db<64,16,128,16,8,8><<<S/64,128,smem>>>(dH,Q,K,V,F,I,M,B,dB,S) and
 * matmul_backward<...><<<S/64,128,smem>>>(dH,dB,Q,K,V,dQ,dK,dV,F,I,dI,M,B,S) (cuda-src/mlstm_backward.cu:11-12,
 * 177-178, 621-628) and the never-instantiated backward_df (:525-558).  The reference's kernels stop at dB, dQ and
 * dK (dV is a TODO there, :506-508, and dI / dF are not finished); they take M and B from a host computation.
 * Here the forward is recomputed inside the call for h, m and b, so the argument list needs neither.
 */
size_t mlstm_backward_f16_workspace(unsigned S, unsigned D);
int mlstm_backward_f16(const void* dH, const void* Q, const void* K, const void* V, const void* F, const void* I,
                       void* dQ, void* dK, void* dV, void* dF, void* dI, unsigned S, unsigned D, void* workspace,
                       size_t workspace_bytes, void* stream);

/* The same forward as mlstm_forward_f16 for callers that cannot supply scratch memory.
 * No counterpart in the reference: its launcher has no scratch because its kernel needs none.
 * Who needs it: callers that are not allowed to call cudaMalloc at the point of use (on a
 * latency-critical path, because cudaMalloc/cudaFree stall the whole device; in a process with a
 * fixed memory budget and no allocator of its own) and that use the reference driver's argument list
 * (Q, K, V, F, I, H, S), which has no room for a workspace.  The scratch is a fixed array inside the
 * library's device image: MLSTM_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the
 * process exits.  Limits and rules:
 *   - S <= MLSTM_STATIC_MAX_S, else MLSTM_E_STATIC_LIMIT (use mlstm_forward_f16 with a workspace);
 *   - the first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 *     that device current): make that first call outside any stream capture;
 *   - it calls no cudaMalloc, cudaFree or other allocating routine, on any call;
 *   - all calls on a device share the one array; calls whose kernels may overlap on the GPU race.
 *     Order them on one stream or with events;
 *   - the array starts with the same status word as a workspace; because its address is private to
 *     the library, mlstm_forward_f16_static_status() reads it (after synchronising `stream`):
 *     MLSTM_OK, or MLSTM_E_TIMEOUT with the kernel's code in *host_status. */
#define MLSTM_STATIC_MAX_S 16384u
#define MLSTM_STATIC_SCRATCH_BYTES 332032u /* forward scratch of one head at S = MLSTM_STATIC_MAX_S */
int mlstm_forward_f16_static(const void* Q, const void* K, const void* V, const void* F, const void* I, void* H,
                             unsigned S, unsigned D, void* stream);
int mlstm_forward_f16_static_status(int* host_status, void* stream);

/* Chunkwise forward for long sequences, with a state that can be carried across segments (GPUs).
 * The reference has no such entry point; the mechanism it extends is the scan path's inter-block carry
 * (mlstm_scan.py:143-195, operators :15-26).  16-bit inputs, D = 128 or 256, chunk a multiple of 128.
 * mlstm_scan_fwd uses it by itself for sequences much longer than the head dimension.
 * A segment is processed in this order (all on one stream, one workspace):
 *   mlstm_chunk_gate_summary  (optional) local {F_end, A_end} per slice with no carry
 *   mlstm_chunk_prepare       gates (with carry_in[bh] = {F, A} of the preceding segments, or NULL) and
 *                             the per-block states; summary_out[bh] = {F_end, A_end} incl. the carry (or NULL)
 *   mlstm_chunk_local_state   (optional) the state this segment adds: S_end [B,NH,D,D] (key, value),
 *                             z_end [B,NH,D], stabilised by A_end
 *   mlstm_chunk_apply         h for the segment (times silu(o) when o is given), given the inbound state
 *                             (S_in, z_in stabilised by the carried-in A, or NULL/NULL); optionally the
 *                             outbound state S_out, z_out
 * summary / carry arrays are device doubles [B*NH][2] in natural-log units. */
size_t mlstm_chunk_workspace(int B, int NH, int S, int D, int dtype, int chunk);
int mlstm_chunk_gate_summary(const void* f, const void* i, double* summary, void* workspace, size_t workspace_bytes,
                             int B, int NH, int S, int D, int dtype, int chunk, void* stream);
int mlstm_chunk_prepare(const void* k, const void* v, const void* f, const void* i, const double* carry_in,
                        double* summary_out, void* workspace, size_t workspace_bytes, int B, int NH, int S, int D,
                        int dtype, int chunk, void* stream);
int mlstm_chunk_local_state(void* workspace, size_t workspace_bytes, float* S_end, float* z_end, int B, int NH, int S,
                            int D, int dtype, int chunk, void* stream);
int mlstm_chunk_apply(const void* q, const void* k, const void* v, const void* o, const float* S_in, const float* z_in,
                      void* h, int h_dtype, float* S_out, float* z_out, void* workspace, size_t workspace_bytes, int B,
                      int NH, int S, int D, int dtype, int chunk, void* stream);

/* Backward of the chunkwise forward, in time linear in S (the reference's scan is forward only, README.md:97;
 * the gradient formulas are those of mlstm_matmul.py:336-365 split into the part inside a block and the part
 * carried across blocks).  For a segment processed with no inbound state.
 *   mlstm_chunk_read_mb   after mlstm_chunk_apply: copies the stabiliser m and the row sums b [B,NH,S] fp32 out
 *                         of the workspace (what the parallel forward returns as M and B)
 *   mlstm_chunk_bwd       dh, h of `h_dtype` (fp32 or the input type); q, k, v, f, i and dq, dk, dv, df, di of
 *                         `dtype`; m, b as read above.  Its workspace is its own (mlstm_chunk_bwd_workspace);
 *                         the gates and block states are recomputed in it.  df[..., 0] is exactly 0. */
int mlstm_chunk_read_mb(const void* workspace, size_t workspace_bytes, float* m, float* b, int B, int NH, int S, int D,
                        int dtype, int chunk, void* stream);
size_t mlstm_chunk_bwd_workspace(int B, int NH, int S, int D, int dtype, int h_dtype, int chunk);
int mlstm_chunk_bwd(const void* dh, const void* q, const void* k, const void* v, const void* f, const void* i,
                    const void* h, const float* m, const float* b, void* dq, void* dk, void* dv, void* df, void* di,
                    void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int h_dtype,
                    int chunk, void* stream);

/* Sequence-parallel form of the chunkwise forward: rank r of `world` holds the r-th contiguous segment
 * of every sequence, and ONE exchange connects the ranks (the carry combine of mlstm_scan.py:15-26
 * applied to whole segments; the reference itself has no multi-GPU code).
 *   mlstm_chunk_sp_local   everything that needs no other rank: gates, per-block states, and this
 *                          segment's record [B*NH][mlstm_chunk_sp_record_floats(D)] fp32 =
 *                          S (D*D, key-major) | z (D) | {F_end, A_end} as two doubles; the state is
 *                          stabilised by the segment's own prefix maximum and F counts from zero
 *   -- the caller all-gathers the records into gathered[world][B*NH][record] (NCCL, or any copy) --
 *   mlstm_chunk_sp_apply   folds the records of the lower ranks into this segment's inbound state and
 *                          carry (one kernel), carries it through the blocks and writes h (times
 *                          silu(o) when o is given).  carry_out (optional): {F_in, A_in} per slice.
 * Both calls use the same workspace (mlstm_chunk_workspace) and stream. */
size_t mlstm_chunk_sp_record_floats(int D);
int mlstm_chunk_sp_local(const void* k, const void* v, const void* f, const void* i, float* record, void* workspace,
                         size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int chunk, void* stream);
int mlstm_chunk_sp_apply(const void* q, const void* k, const void* v, const void* o, const float* gathered, int world,
                         int rank, void* h, int h_dtype, double* carry_out, void* workspace, size_t workspace_bytes,
                         int B, int NH, int S, int D, int dtype, int chunk, void* stream);

/* Copies the workspace's device status word to *host_status after synchronising `stream`.
 * Returns MLSTM_OK, or MLSTM_E_TIMEOUT when the word is non-zero, or MLSTM_E_CUDA. */
int mlstm_read_status(const void* workspace, int* host_status, void* stream);

/* Self-test of the bounded waits (no counterpart in the reference, whose kernels have no waits to bound):
 * one warp waits on a barrier that nothing completes, gives up after `limit_cycles` SM cycles (1 ..
 * 2e9; a few million = about a millisecond) and stores the code 4000 in the workspace's status word,
 * exactly as a contraction kernel does when one of its waits runs out.  mlstm_read_status() then returns
 * MLSTM_E_TIMEOUT, and the device stays usable.  `workspace`: at least 256 bytes. */
int mlstm_selftest_wait_timeout(void* workspace, size_t workspace_bytes, long long limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLSTM_B200_H */
