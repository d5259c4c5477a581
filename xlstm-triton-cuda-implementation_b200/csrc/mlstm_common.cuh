// Shared definitions of the mLSTM kernels: status codes, element types, the per-row gate vectors
// and the one elementwise rule that all four contraction passes share.
//
// Decomposition used by every kernel of this library (per batch*head slice, rows r, columns c):
//   F_t  = inclusive cumulative sum of logsigmoid(f)          (reference: mlstm_matmul.py:59, 73-82, 106)
//   a_t  = i_t - F_t,   A_t = max_{s<=t} a_s,   m_t = F_t + A_t (the reference's running row maximum,
//                                                               mlstm_matmul.py:84, is this prefix maximum)
//   exp(d_tilde_rc - m_r) = exp(a_c - A_r)   for c <= r        (mlstm_matmul.py:85-86)
// so the stabiliser is known before the contraction starts and no accumulator is ever rescaled.
// With n_r = max(|b_r|, exp(-m_r)) + 1e-6 (mlstm_matmul.py:95) all four passes have the form
//   T = X Y^T  (contraction over the head dimension)
//   W = (T + g) * exp2(ec[c] + er[r])   on the causal side of the diagonal, 0 elsewhere
//   ACC += W Z (contraction over the streamed tile's 128 rows)
// with (scale = 1/sqrt(D), log2 units, "gA" = A*log2e, "ga" = a*log2e, ln_r = log2(scale / n_r);
// the gate pass stores ga and -gA, the backward preparation -gA + ln, each re-centred per block of
// REF_BLOCK positions around a double reference, see gates.cu):
//   FWD  rows = queries  X=Q  Y=K  Z=V   er = -gA_r + log2(scale)  ec = ga_c       g = 0         out = ACC / n_r
//   DQ   rows = queries  X=dH Y=V  Z=K   er = -gA_r + ln_r         ec = ga_c       g = db_r n_r  out = ACC
//   DK   rows = keys     X=V  Y=dH Z=Q   er = ga_r                 ec = -gA_c+ln_c g = db_c n_c  out = ACC
//   DV   rows = keys     X=K  Y=Q  Z=dH  er = ga_r                 ec = -gA_c+ln_c g = 0         out = ACC
// (backward formulas: mlstm_matmul.py:183-197, 256-316, 336-365).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/mlstm_b200.h"

namespace mlstm {

// FWDC and STATE are the two passes of the chunkwise forward (chunk.cu): STATE builds, per block of
// `chunk_tiles` tiles, U = sum_j w_j k_j v_j^T (rows = key dimensions, X = identity, Y = K, Z = V);
// FWDC is FWD restricted to the query's own block plus one step that applies the block's inbound
// state (Y = identity, Z = state), so T = Q and W = Q scaled per row.
// DQC, DKC, DVC are the backward passes of the chunkwise form: DQ / DK / DV restricted to the row tile's own
// block plus one step that applies a carried state (the inbound state S_k for dQ; for dK and dV the state
// R_k = sum over later positions t of exp(A_end(k) - A_t) (scale / n_t) q_t dh_t^T carried BACK over the blocks).
enum Mode : int { FWD = 0, DQ = 1, DK = 2, DV = 3, FWDC = 4, STATE = 5, DQC = 6, DKC = 7, DVC = 8 };

constexpr int TILE = 128;      // rows of a tensor-core tile; gate vectors are padded to a multiple of it
constexpr int REF_BLOCK = 64;  // positions per reference block of the re-centred gate vectors (gates.cu)

__host__ __device__ constexpr int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Arguments of one contraction pass, shared by the tensor-core and the SIMT kernels.
struct PassParams {
    int S;      // sequence length
    int Spad;   // S rounded up to TILE: stride of every gate vector per slice
    int BH;     // batch * heads
    int D;      // head dimension
    const void* X;  // stationary operand  [BH, S, D]
    const void* Y;  // first streamed operand
    const void* Z;  // second streamed operand
    // er[r] + ec[c] = col_rel[c] + float(row_rel[r] + row_ref[r / REF_BLOCK] + col_ref[c / REF_BLOCK] + er_add):
    // the gate vectors are stored relative to a double reference per block of REF_BLOCK positions
    const float* row_rel;   // [BH, Spad]
    const double* row_ref;  // [BH, Spad / REF_BLOCK]
    const float* row_g;     // g per row (DQ) or nullptr
    const float* col_rel;   // [BH, Spad]
    const float* col_w;     // [BH, Spad] exp2(col_rel): the tensor-core kernel's factorised path off the diagonal
    const double* col_ref;  // [BH, Spad / REF_BLOCK]
    const float* col_g;     // g per column (DK) or nullptr
    float er_add;           // constant term of er (FWD: log2(scale))
    void* out;           // [BH, S, D], element type chosen by the kernel template
    // FWD only
    const float* m;      // [BH, S] stabiliser, written by the gate pass
    float* b_out;        // [BH, S] row sums of the gated tile (the reference's B output) or nullptr
    const void* ogate;   // [BH, S, D] optional output gate pre-activation (scan API), input type
    // DQ / DK only: dot_out[r] = sum_d ACC[r, d] * dot_src[r, d], taken on the fp32 accumulator
    const void* dot_src; // [BH, S, D] input type (q for DQ, k for DK)
    float* dot_out;      // [parts][BH, Spad]: the tensor-core passes write one partial per gate group (4 parts,
                         // dot_part_stride floats apart; df_kernel adds them up), the CUDA-core pass one total
    long long dot_part_stride;
    // chunkwise passes only
    int chunk_tiles;         // tiles per block
    int NB;                  // blocks per slice
    const double* An_bound;  // [BH, NB + 1]  -A*log2e at the block boundaries (entry 0: the inbound carry)
    const void* ident;       // [128, 128] identity in the input type
    const void* states;      // FWDC and the chunkwise backward passes: [BH, NB, D, D] the state applied to every block
                             // (input type; rows = the contraction index of the state step)
    const float* zstate;     // FWDC, DQC: [BH, NB, D] inbound normaliser vector of every block
    const float* rvec;       // DKC: [BH, NB, D] vector part of the state carried back from the later blocks
    int state_reverse;       // STATE: rows carry +A_end(previous block) (contributions to the backward's carried state)
    // FWDC, optional: a carry that became known after the gate pass (sequence-parallel segments).
    // late_bound[bh] = -(A_in + F_in) * log2e, the inbound prefix maximum in this segment's own
    // coordinates; every stabiliser -A*log2e of the slice (rows, block boundaries) becomes
    // min(local value, late_bound[bh]) and m grows by the difference.  +inf = no carry.
    const double* late_bound;
    int* status;         // device word; a kernel that gave up on a wait stores a non-zero code
    int* sched;          // tensor-core passes: 12 device words, one work-item counter per pass mode
    int sched_zeroed;    // the counters were cleared by an earlier kernel of the call (else the launcher clears its own)
    int slice_set;       // tensor-core passes: slices interleaved in the work-item order (set by the launcher)
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// x * sigmoid(x) with the fast exponential and the fast division (a few ulp; an IEEE division costs about
// twenty instructions per element in the epilogues that apply the output gate)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Causal side of the diagonal.  Rows are queries in FWD/DQ (column <= row is valid) and keys in
// DK/DV (column >= row is valid).
template <int MODE>
__device__ __forceinline__ bool causal_ok(int row, int col) {
    return (MODE == FWD || MODE == DQ || MODE == FWDC || MODE == DQC) ? (col <= row) : (col >= row);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute (launch_pdl
// below) may start while the kernel before it in the stream is still running; grid_dep_wait() returns once that kernel
// has completed and its writes are visible (at once when the launch had no such attribute), so everything in front of
// it must touch no global memory.  grid_dep_launch() says that the kernel after this one may be started now.  The
// kernels of this library begin with both (the tensor-core kernels after their shared-memory / TMEM prologue), and the
// tensor-core passes are launched this way: their launch and prologue overlap the tail of the kernel before them.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <bool PDL = true, typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = PDL ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// The small kernels (gate pass, scans, preparation, conversions) are launched the ordinary way: launched programmatically
// as well, their many early, waiting CTAs cost the chunkwise paths 3 to 9 % (measured).  They still begin with
// grid_dep_launch(), so that the tensor-core pass after them starts its prologue under their tail.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_plain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    return launch_pdl<false>(kern, grid, block, smem, st, static_cast<Args&&>(args)...);
}

// Remembers the last CUDA failure of this host thread for mlstm_last_error_detail(); returns MLSTM_E_CUDA.
int note_cuda_error(cudaError_t err, const char* where);

// Launchers implemented in the .cu files.  All return an MLSTM_* status and never synchronise.
int launch_gates_fwd(const void* f, const void* i, float* ga_rel, float* gAn_rel, double* a_ref, double* An_ref, float* m,
                     int BH, int S, int Spad, int dtype, cudaStream_t st, const double* carry_in = nullptr,
                     double* summary_out = nullptr, double* An_bound = nullptr, int chunk_len = 0,
                     double* scratch = nullptr, float* ga_w = nullptr, int* zero_words = nullptr, int n_zero = 0);
// zero_words / n_zero: device words the gate pass clears (the call's status block: status word and the work-item
// counters of the passes that follow; STATUS_WORDS covers them all)
constexpr int STATUS_WORDS = 64;
// bytes of `scratch` that let launch_gates_fwd cut long slices into segments (0: not worth it)
size_t gates_scratch_bytes(int BH, int Spad);
// chunk.cu
int launch_identity(void* ident, int D, int dtype, cudaStream_t st);
// rec (optional): per-slice records of rec_stride floats that receive S_end | z_end | summary {F, A} (two doubles)
int launch_state_scan(const void* U, const float* zU, const double* An_bound, const float* S_in, const float* z_in,
                      void* states16, float* zstate, float* S_end, float* z_end, int BH, int NB, int D, int dtype,
                      cudaStream_t st, const double* late_bound = nullptr, float* rec = nullptr, size_t rec_stride = 0,
                      const double* summary = nullptr, void* statesT16 = nullptr, int reverse = 0, int* zero_word = nullptr);
int launch_bwd_prep(const void* h, const void* dh, const float* b, const float* m, const float* gAn, float* gB,
                    float* gBw, float* g, void* dh16, int BH, int S, int Spad, int D, int h_dtype, int dtype, cudaStream_t st);
// dI, R: `nparts` partial vectors each, `part_stride` floats apart (see PassParams::dot_out).  scratch (optional,
// gates_scratch_bytes(BH, Spad) bytes): long slices are then scanned in segments, one block each.
int launch_df(const void* f, const float* dI, const float* R, void* df, void* di, int BH, int S, int Spad, int dtype,
              cudaStream_t st, int nparts = 1, long long part_stride = 0, double* scratch = nullptr);
constexpr int TC_DOT_PARTS = 4;   // gate groups of the tensor-core passes
int launch_pass_simt(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st);
int launch_pass_tc(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st);
bool tc_supported(int S, int D, int in_dtype);
int launch_round_tf32(const void* in, void* out, long long n, cudaStream_t st);
// fp32 [rows, D] -> bf16 [rows, 2 D] (hi | mid): the operands of the split tensor-core form (mm_tc.cu)
int launch_split_bf16(const void* in, void* out, long long rows, int D, cudaStream_t st);
// the same for up to four tensors of one shape in one launch
int launch_split_bf16_multi(const void* const* in, void* const* out, int count, long long rows, int D, cudaStream_t st);
bool tc_x3_supported(int S, int D);
int launch_pass_tc_x3(int mode, const PassParams& p, cudaStream_t st);
int launch_ogate_fwd(const void* h_inner, const void* o, void* h, long long n, int h_dtype, int o_dtype, cudaStream_t st);
int launch_ogate_bwd(const void* dh, const void* h_inner, const void* o, void* dh_inner, void* d_o, long long n, int h_dtype,
                     int o_dtype, cudaStream_t st);

// Two-pass forward for head dimensions above 256 (scan_gemm.cu); o may be null (no output gate).  Gate vectors as written by
// launch_gates_fwd for all BH slices; bpart and W are scratch of scan_gemm_bpart_bytes / scan_gemm_w_bytes;
// counters: two device words, zeroed by the caller.
struct ScanGemmArgs {
    int S, Spad, BH, D;
    const float *ga, *gAn, *gaw;
    const double *a_ref, *An_ref;
    const float* m;
    float* b;        // [BH, S] row sums out (optional)
    float* bpart;
    int* status;
    int* counters;
};
bool scan_gemm_supported(int S, int D, int in_dtype);
size_t scan_gemm_w_bytes(int BH, int S, int dtype);
size_t scan_gemm_bpart_bytes(int BH, int S, int dtype);
int launch_scan_gemm(const void* q, const void* k, const void* v, const void* o, float* h, void* W, const ScanGemmArgs& a,
                     int dtype, cudaStream_t st);
// The parallel backward in the same two passes (head dimensions above 256).  q, k, v, dh and the outputs dq, dk, dv
// in the input type; gate vectors of launch_gates_fwd and launch_bwd_prep (gB, g) for all BH slices; Wn, dT: scratch
// of scan_gemm_bwd_matrix_bytes each; R, dI: [D / 256][BH, Spad] row-dot partials (dot_stride apart) for launch_df;
// counters: five device words (zeroed by the launches).
struct ScanGemmBwdArgs {
    int S, Spad, BH, D;
    const void *q, *k, *v, *dh;
    void *dq, *dk, *dv;
    const float *ga, *gaw, *gB, *g;
    const double *a_ref, *An_ref;
    void *Wn, *dT;
    float *R, *dI;
    long long dot_stride;
    int* status;
    int* counters;
};
size_t scan_gemm_bwd_matrix_bytes(int BH, int S, int dtype);
int launch_scan_gemm_bwd(const ScanGemmBwdArgs& a, int dtype, cudaStream_t st);

}  // namespace mlstm
