// Chunkwise forward of the mLSTM for long sequences, with an inbound / outbound state so that a
// sequence can be split into contiguous segments across GPUs.
//
// The reference has no such entry point; its only long-sequence mechanism is the inter-block carry of
// the scan path (mlstm_scan.py:143-195: per-block (C, n) states reduced over blocks).  This file
// gives that mechanism the stabiliser algebra of the parallel path: with the prefix maximum A known
// up front (gates.cu), every weight is exp(a_j - A_ref) <= 1 and the carry is a plain linear
// recurrence
//     S_{k+1} = exp(A_end(k-1) - A_end(k)) S_k + U_k,    U_k = sum_{j in block k} exp(a_j - A_end(k)) k_j v_j^T
// (S is indexed [key, value]; z is the same with v dropped: the normaliser vector).  A query t of block k
// gets   num_t = intra-block part + exp(A_end(k-1) - A_t) (q_t S_k) / sqrt(D)   and the same for b_t.
// Both contractions run on the tensor-core pass kernel (modes STATE and FWDC, mm_tc.cu).
#include "mlstm_common.cuh"

namespace mlstm {
namespace {

constexpr size_t WS_ALIGN = 256;
inline size_t al(size_t x) { return (x + WS_ALIGN - 1) / WS_ALIGN * WS_ALIGN; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T16>
__global__ void identity_kernel(T16* ident, int D) {   // D x D
    grid_dep_wait();
    grid_dep_launch();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < D * D) ident[idx] = from_f32<T16>((idx / D) == (idx % D) ? 1.0f : 0.0f);
}

// One thread owns four consecutive elements of a slice's state (D x D matrix and D-vector, the normaliser) and walks
// the blocks in order.  It writes the INBOUND state of every block (16-bit matrix for the tensor cores, fp32 vector;
// skipped when `states` is null) and, optionally, the state after the last block (S_end / z_end with per-slice
// strides, so that they can sit inside a packed record).
// Work split: a CTA owns 512 elements of the matrix: whole rows when only the row-major copy is written; when a
// transposed copy is wanted too, a patch of 32 rows x 16 columns (thread t: row t / 4, columns 4 (t % 4) .. +3), so
// that it writes 32 bytes per row of the row-major copy and, through a transpose in shared memory, 64 bytes per row of
// the transposed copy (written element by element from registers, the
// transposed copy cost 16 times its size in memory transactions: 0.4 ms per scan at 256 blocks of 128 x 128).
// The CTAs behind the patches own the vector.
// late_bound (optional, per slice): a carry that became known after the gate pass, see PassParams;
// block contributions U_k were stabilised by the local block-end maximum and are rescaled to the
// later, larger one on the way in.
// statesT (optional): the same per-block matrices transposed ([value, key]), for passes whose state step
// contracts over the value dimension.  reverse: walk the blocks from the last to the first, which turns
// the same recurrence into the backward's carried state R_{k-1} = exp(A_end(k-1) - A_end(k)) R_k + P_k
// (block k then receives what the LATER blocks contribute).
constexpr int SCAN_TB = 1024;       // blocks per tile of the factor tables of state_scan_kernel
constexpr int SCAN_THREADS_S = 128;
constexpr int PATCH_ROWS = 32, PATCH_COLS = 16;

template <typename T16>
__global__ void __launch_bounds__(SCAN_THREADS_S)
state_scan_kernel(const T16* __restrict__ U, const float* __restrict__ zU, const double* __restrict__ An_bound,
                  const float* __restrict__ S_in, const float* __restrict__ z_in, T16* __restrict__ states,
                  float* __restrict__ zstate, float* __restrict__ S_end, float* __restrict__ z_end, size_t S_end_stride,
                  size_t z_end_stride, int NB, int D, const double* __restrict__ late_bound,
                  const double* __restrict__ summary, double* __restrict__ summary_dst, size_t summary_dst_stride,
                  T16* __restrict__ statesT, int reverse, int* __restrict__ zero_word) {
    grid_dep_wait();
    grid_dep_launch();
    const int bh = blockIdx.y;
    const int DD = D * D;
    // the work-item counter of the pass that follows in the same call (its launcher then needs no memset of its own)
    if (zero_word && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *zero_word = 0;
    // patch shape: 32 x 16 when a transposed copy is written, else whole rows (512 consecutive elements per CTA)
    const int pcols = statesT ? PATCH_COLS : D;
    const int prows = 4 * SCAN_THREADS_S / pcols;
    const int npc = D / pcols;
    const int npatch = (D / prows) * npc;
    if (blockIdx.x == 0 && threadIdx.x == 0 && summary_dst) {
        double* dst = reinterpret_cast<double*>(reinterpret_cast<float*>(summary_dst) + bh * summary_dst_stride);
        dst[0] = summary[2 * bh];
        dst[1] = summary[2 * bh + 1];
    }
    const bool is_vec = static_cast<int>(blockIdx.x) >= npatch;     // uniform over the CTA
    const int prow0 = (blockIdx.x / npc) * prows, pcol0 = (blockIdx.x % npc) * pcols;
    const int lrow = threadIdx.x / (pcols / 4), lcol = (threadIdx.x % (pcols / 4)) * 4;
    const int off = is_vec ? ((blockIdx.x - npatch) * SCAN_THREADS_S + threadIdx.x) * 4 : (prow0 + lrow) * D + pcol0 + lcol;
    const bool valid = !is_vec || off < D;     // threads past the end still help with the factor tables and the barriers
    const size_t per_block = is_vec ? D : DD;
    // block contributions: the matrices in the 16-bit input type (as the tensor-core pass wrote them), the vectors in fp32
    const float* srcz = zU + static_cast<size_t>(bh) * NB * per_block + off;
    const T16* srcU = U + static_cast<size_t>(bh) * NB * per_block + off;
    const float* init = is_vec ? z_in : S_in;
    float4 s = (init && valid) ? *reinterpret_cast<const float4*>(init + static_cast<size_t>(bh) * per_block + off)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
    const double* bound = An_bound + static_cast<size_t>(bh) * (NB + 1);
    const double lb = late_bound ? late_bound[bh] : INFINITY;
    // The two factors of a block (decay of the carried state, rescaling of the block's own contribution) are the
    // same for every element: the CTA computes them once per tile of SCAN_TB blocks into shared memory (evaluated
    // per thread and block they were most of the kernel's instructions: 107 per warp and block against about 20 now).
    __shared__ float sd[SCAN_TB], sc[SCAN_TB];
    // transposed patches on their way out: [column][row], two buffers so that one barrier per block is enough
    __shared__ __align__(16) T16 tp[2][PATCH_COLS][PATCH_ROWS + 8];
    const bool transposing = statesT != nullptr && !is_vec;
    const int trow = threadIdx.x >> 3, tcol = (threadIdx.x & 7) * 4;   // this thread's piece of the transposed patch
    int tbuf = 0;
    // blocks whose contributions are fetched ahead of the serial update
    constexpr int PF = 16;
    for (int t0 = 0; t0 < NB; t0 += SCAN_TB) {
        const int tn = min(SCAN_TB, NB - t0);
        __syncthreads();   // the previous tile's factors are no longer read
        for (int j = threadIdx.x; j < tn; j += blockDim.x) {
            const int kb = reverse ? NB - 1 - (t0 + j) : t0 + j;
            const double b1 = bound[kb + 1], b0 = bound[kb];
            const double b1c = fmin(b1, lb), b0c = fmin(b0, lb);
            // exp(A_end(k-1) - A_end(k)); 0 for the first block when there is no inbound carry (bound = +inf)
            sd[j] = exp2f(static_cast<float>(b1c - b0c));
            sc[j] = exp2f(static_cast<float>(b1c - b1));   // 1 unless the late carry raised the block's stabiliser
        }
        __syncthreads();
        if (is_vec && !valid) continue;
        for (int k0 = 0; k0 < tn; k0 += PF) {
            float4 u[PF];
            if (is_vec) {     // (uniform over the CTA: the loads of either kind go out as one batch)
#pragma unroll
                for (int j = 0; j < PF; j++) {
                    if (k0 + j < tn) {
                        const int kb = reverse ? NB - 1 - (t0 + k0 + j) : t0 + k0 + j;
                        u[j] = __ldg(reinterpret_cast<const float4*>(srcz + static_cast<size_t>(kb) * per_block));
                    }
                }
            } else {
                uint2 raw[PF];
#pragma unroll
                for (int j = 0; j < PF; j++) {
                    if (k0 + j < tn) {
                        const int kb = reverse ? NB - 1 - (t0 + k0 + j) : t0 + k0 + j;
                        raw[j] = __ldg(reinterpret_cast<const uint2*>(srcU + static_cast<size_t>(kb) * per_block));
                    }
                }
#pragma unroll
                for (int j = 0; j < PF; j++) {
                    const T16* e4 = reinterpret_cast<const T16*>(&raw[j]);
                    u[j] = make_float4(to_f32<T16>(e4[0]), to_f32<T16>(e4[1]), to_f32<T16>(e4[2]), to_f32<T16>(e4[3]));
                }
            }
#pragma unroll
            for (int j = 0; j < PF; j++) {
                if (k0 + j >= tn) break;
                const int k = reverse ? NB - 1 - (t0 + k0 + j) : t0 + k0 + j;
                if (is_vec) {
                    if (zstate) *reinterpret_cast<float4*>(zstate + (static_cast<size_t>(bh) * NB + k) * D + off) = s;
                } else if (states || statesT) {
                    T16 o[4] = {from_f32<T16>(s.x), from_f32<T16>(s.y), from_f32<T16>(s.z), from_f32<T16>(s.w)};
                    if (states)
                        *reinterpret_cast<uint2*>(states + (static_cast<size_t>(bh) * NB + k) * DD + off) = *reinterpret_cast<uint2*>(o);
                    if (transposing) {   // (uniform over the CTA)
                        tp[tbuf][lcol + 0][lrow] = o[0];
                        tp[tbuf][lcol + 1][lrow] = o[1];
                        tp[tbuf][lcol + 2][lrow] = o[2];
                        tp[tbuf][lcol + 3][lrow] = o[3];
                        __syncthreads();
                        T16* dstT = statesT + (static_cast<size_t>(bh) * NB + k) * DD + static_cast<size_t>(pcol0 + trow) * D + prow0 + tcol;
                        *reinterpret_cast<uint2*>(dstT) = *reinterpret_cast<const uint2*>(&tp[tbuf][trow][tcol]);
                        tbuf ^= 1;
                    }
                }
                const float d = sd[k0 + j], c = sc[k0 + j];
                // a decay of exactly 0 (nothing carried in) must also wipe an inbound state that is not finite
                s.x = (d == 0.0f ? 0.0f : d * s.x) + c * u[j].x;
                s.y = (d == 0.0f ? 0.0f : d * s.y) + c * u[j].y;
                s.z = (d == 0.0f ? 0.0f : d * s.z) + c * u[j].z;
                s.w = (d == 0.0f ? 0.0f : d * s.w) + c * u[j].w;
            }
        }
    }
    if (!valid) return;
    float* dst = is_vec ? z_end : S_end;
    const size_t stride = is_vec ? z_end_stride : S_end_stride;
    if (dst) *reinterpret_cast<float4*>(dst + static_cast<size_t>(bh) * stride + off) = s;
}

// Vector part of what block k contributes to the backward's carried state:
//   p_k[d] = sum_{t in block k} beta_t g_t q_t[d],  beta_t = exp(A_end(k-1) - A_t) scale / n_t,  g_t = db_t n_t
// (the matrix part sum_t beta_t q_t dh_t^T comes from the tensor-core STATE pass).  One block of D threads per
// (block, slice); log2 beta_t = gB_rel[t] + An_ref[t / 64] - bound[k] with the vectors of the backward preparation.
// The weights beta_t g_t of the block's positions are computed once (into shared memory), then every thread adds up
// its dimension over them: evaluated per thread and position they were most of the kernel.
constexpr int RVEC_MAX_CHUNK = 2048;   // positions of a block whose weights fit the table; longer blocks take several rounds

template <typename T16>
__global__ void rvec_partial_kernel(const T16* __restrict__ q, const float* __restrict__ gB_rel,
                                    const double* __restrict__ An_ref, const double* __restrict__ An_bound,
                                    const float* __restrict__ g, float* __restrict__ out, int S, int Spad, int NB, int chunk,
                                    int D) {
    grid_dep_wait();
    grid_dep_launch();
    __shared__ float wt[RVEC_MAX_CHUNK];
    const int k = blockIdx.x, bh = blockIdx.y, d = threadIdx.x;
    const double b0 = An_bound[static_cast<size_t>(bh) * (NB + 1) + k];
    const int t0 = k * chunk, t1 = min(t0 + chunk, S);
    float acc = 0.0f;
    for (int r0 = t0; r0 < t1; r0 += RVEC_MAX_CHUNK) {
        const int rn = min(RVEC_MAX_CHUNK, t1 - r0);
        __syncthreads();
        for (int j = threadIdx.x; j < rn; j += blockDim.x) {
            const int t = r0 + j;
            const size_t vi = static_cast<size_t>(bh) * Spad + t;
            const float e = gB_rel[vi] + static_cast<float>(An_ref[static_cast<size_t>(bh) * (Spad / REF_BLOCK) + t / REF_BLOCK] - b0);
            wt[j] = exp2f(e) * g[vi];   // exp2(-inf) = 0 for the first block when nothing is carried in
        }
        __syncthreads();
        const T16* qp = q + (static_cast<size_t>(bh) * S + r0) * D + d;
#pragma unroll 8
        for (int j = 0; j < rn; j++) acc = fmaf(wt[j], to_f32<T16>(qp[static_cast<size_t>(j) * D]), acc);
    }
    out[(static_cast<size_t>(bh) * NB + k) * D + d] = acc;
}

// Sequence-parallel fold: from the gathered records of all segments (per slice: S | z | {F_end, A_end},
// every segment's state stabilised by its OWN prefix maximum and its F counted from zero) to the
// inbound state of segment `rank` and its late carry.  With F_in(g) the log-forget total before
// segment g, segment g's stabiliser in global terms is A_g - F_in(g); the inbound maximum is
// A_in = max_{g < rank} of those, S_in = sum_g exp(A_g - F_in(g) - A_in) S_g (weights <= 1), and the
// late bound handed to the kernels is -(A_in + F_in(rank)) * log2e (+inf for the first segment).
// This is the combine of the reference's scan operators (mlstm_scan.py:15-26) over segment summaries.
__global__ void sp_fold_kernel(const float* __restrict__ gathered, int rank, int BH, int D, size_t rec_stride,
                               float* __restrict__ S_in, float* __restrict__ z_in, double* __restrict__ late_bound,
                               double* __restrict__ carry) {
    grid_dep_wait();
    grid_dep_launch();
    const int bh = blockIdx.y;
    const int DD = D * D;
    const int e = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (e >= DD + D) return;
    auto rec = [&](int g) { return gathered + (static_cast<size_t>(g) * BH + bh) * rec_stride; };
    auto tail = [&](int g) { return reinterpret_cast<const double*>(rec(g) + DD + D); };
    double Fin = 0.0, Ain = -INFINITY;
    for (int g = 0; g < rank; g++) {
        const double* t = tail(g);
        Ain = fmax(Ain, t[1] - Fin);
        Fin += t[0];
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    double Fg = 0.0;
    for (int g = 0; g < rank; g++) {
        const double* t = tail(g);
        const float w = static_cast<float>(exp(t[1] - Fg - Ain));
        Fg += t[0];
        const float4 x = __ldg(reinterpret_cast<const float4*>(rec(g) + e));
        acc.x = fmaf(w, x.x, acc.x); acc.y = fmaf(w, x.y, acc.y); acc.z = fmaf(w, x.z, acc.z); acc.w = fmaf(w, x.w, acc.w);
    }
    if (e >= DD) *reinterpret_cast<float4*>(z_in + static_cast<size_t>(bh) * D + (e - DD)) = acc;
    else *reinterpret_cast<float4*>(S_in + static_cast<size_t>(bh) * DD + e) = acc;
    if (e == 0) {
        late_bound[bh] = rank == 0 ? static_cast<double>(INFINITY) : -(Ain + Fin) * 1.4426950408889634;
        if (carry) {
            carry[2 * bh] = Fin;
            carry[2 * bh + 1] = Ain;
        }
    }
}

struct ChunkWs {
    int* status;
    float *ga, *gAn, *gaw, *m, *b, *zU, *zstate, *S_in, *z_in;
    void* U;          // per-block contributions to the state, 16-bit
    double *a_ref, *An_ref, *An_bound, *gscratch, *summary, *late;
    void *ident, *states;
    int NB;
    size_t bytes;
};

ChunkWs carve(void* ws, int BH, int S, int D, int chunk) {
    ChunkWs w{};
    uint8_t* base = static_cast<uint8_t*>(ws);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? base + off : nullptr;
        off += al(bytes);
        return p;
    };
    const size_t Spad = round_up(S, TILE);
    const size_t vec = static_cast<size_t>(BH) * Spad * sizeof(float);
    w.NB = (S + chunk - 1) / chunk;
    const size_t nblk = static_cast<size_t>(BH) * w.NB;
    w.status = static_cast<int*>(take(WS_ALIGN));
    w.ga = static_cast<float*>(take(vec));
    w.gAn = static_cast<float*>(take(vec));
    w.gaw = static_cast<float*>(take(vec));
    w.a_ref = static_cast<double*>(take(vec / REF_BLOCK * 2));
    w.An_ref = static_cast<double*>(take(vec / REF_BLOCK * 2));
    w.m = static_cast<float*>(take(static_cast<size_t>(BH) * S * sizeof(float)));
    w.b = static_cast<float*>(take(static_cast<size_t>(BH) * S * sizeof(float)));
    w.An_bound = static_cast<double*>(take(static_cast<size_t>(BH) * (w.NB + 1) * sizeof(double)));
    const size_t gs = gates_scratch_bytes(BH, static_cast<int>(Spad));
    w.gscratch = gs ? static_cast<double*>(take(gs)) : nullptr;
    w.ident = take(static_cast<size_t>(D) * D * 2);
    w.U = take(nblk * D * D * 2);
    w.zU = static_cast<float*>(take(nblk * D * sizeof(float)));
    w.states = take(nblk * D * D * 2);
    w.zstate = static_cast<float*>(take(nblk * D * sizeof(float)));
    // sequence-parallel stages: this segment's gate summary, the folded inbound state and the late carry
    w.summary = static_cast<double*>(take(static_cast<size_t>(BH) * 2 * sizeof(double)));
    w.late = static_cast<double*>(take(static_cast<size_t>(BH) * sizeof(double)));
    w.S_in = static_cast<float*>(take(static_cast<size_t>(BH) * D * D * sizeof(float)));
    w.z_in = static_cast<float*>(take(static_cast<size_t>(BH) * D * sizeof(float)));
    w.bytes = off;
    return w;
}

int check_chunk_args(int B, int NH, int S, int D, int dtype, int chunk) {
    if (B <= 0 || NH <= 0 || S <= 0 || D <= 0 || chunk <= 0) return MLSTM_E_ARG;
    if (dtype != MLSTM_DT_F16 && dtype != MLSTM_DT_BF16) return MLSTM_E_UNSUPPORTED;  // tensor-core path only
    if (D != 128 && D != 256) return MLSTM_E_UNSUPPORTED;
    if (chunk % TILE != 0) return MLSTM_E_SHAPE;
    if (static_cast<long long>(B) * NH > 65535) return MLSTM_E_SHAPE;
    return MLSTM_OK;
}

// h of the segment from the per-block inbound states (FWDC pass)
int launch_fwdc(const void* q, const void* k, const void* v, const void* o, void* h, int h_dtype, const ChunkWs& w, int BH,
                int S, int Spad, int D, int dtype, int chunk, const double* late_bound, cudaStream_t st) {
    PassParams p{};
    p.S = S; p.Spad = Spad; p.BH = BH; p.D = D; p.status = w.status; p.sched = w.status + 8;
    p.sched_zeroed = 1;   // by the state scan in front of this pass
    p.X = q; p.Y = k; p.Z = v;
    p.row_rel = w.gAn; p.row_ref = w.An_ref; p.col_rel = w.ga; p.col_w = w.gaw; p.col_ref = w.a_ref;
    p.er_add = -0.5f * log2f(static_cast<float>(D));
    p.out = h; p.m = w.m; p.b_out = w.b; p.ogate = o;
    p.chunk_tiles = chunk / TILE; p.NB = w.NB; p.An_bound = w.An_bound; p.ident = w.ident;
    p.states = w.states; p.zstate = w.zstate;
    p.late_bound = late_bound;
    return launch_pass_tc(FWDC, p, dtype, h_dtype, st);
}

}  // namespace

int launch_identity(void* ident, int D, int dtype, cudaStream_t st) {
    const int n = D * D;
    cudaError_t ce;
    if (dtype == MLSTM_DT_BF16)
        ce = launch_plain(identity_kernel<__nv_bfloat16>, dim3((n + 255) / 256), dim3(256), 0, st, static_cast<__nv_bfloat16*>(ident), D);
    else
        ce = launch_plain(identity_kernel<__half>, dim3((n + 255) / 256), dim3(256), 0, st, static_cast<__half*>(ident), D);
    return ce == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

int launch_state_scan(const void* U, const float* zU, const double* An_bound, const float* S_in, const float* z_in,
                      void* states16, float* zstate, float* S_end, float* z_end, int BH, int NB, int D, int dtype,
                      cudaStream_t st, const double* late_bound, float* rec, size_t rec_stride, const double* summary,
                      void* statesT16, int reverse, int* zero_word) {
    // small CTAs: a slice has about 4 K threads of work, which should spread over all SMs
    const int threads = SCAN_THREADS_S;
    if (D % PATCH_ROWS != 0 || D > 4 * threads) return MLSTM_E_SHAPE;
    const int npatch = D * D / (4 * threads);
    dim3 grid(npatch + (D / 4 + threads - 1) / threads, BH);
    size_t s_stride = static_cast<size_t>(D) * D, z_stride = D;
    double* sum_dst = nullptr;
    if (rec) {   // S_end | z_end | summary inside per-slice records
        S_end = rec;
        z_end = rec + s_stride;
        sum_dst = reinterpret_cast<double*>(rec + s_stride + D);
        s_stride = z_stride = rec_stride;
    }
    cudaError_t ce;
    if (dtype == MLSTM_DT_BF16)
        ce = launch_plain(state_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, st, static_cast<const __nv_bfloat16*>(U), zU, An_bound, S_in, z_in,
                        static_cast<__nv_bfloat16*>(states16), zstate, S_end, z_end, s_stride, z_stride, NB, D, late_bound, summary,
                        sum_dst, rec_stride, static_cast<__nv_bfloat16*>(statesT16), reverse, zero_word);
    else
        ce = launch_plain(state_scan_kernel<__half>, grid, dim3(threads), 0, st, static_cast<const __half*>(U), zU, An_bound, S_in, z_in,
                        static_cast<__half*>(states16), zstate, S_end, z_end, s_stride, z_stride, NB, D, late_bound, summary, sum_dst,
                        rec_stride, static_cast<__half*>(statesT16), reverse, zero_word);
    if (ce != cudaSuccess) return MLSTM_E_CUDA;
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

}  // namespace mlstm

using namespace mlstm;

extern "C" {

size_t mlstm_chunk_workspace(int B, int NH, int S, int D, int dtype, int chunk) {
    if (check_chunk_args(B, NH, S, D, dtype, chunk) != MLSTM_OK) return 0;
    return carve(nullptr, B * NH, S, D, chunk).bytes;
}

int mlstm_chunk_gate_summary(const void* f, const void* i, double* summary, void* workspace, size_t workspace_bytes, int B,
                             int NH, int S, int D, int dtype, int chunk, void* stream) {
    if (!f || !i || !summary) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    ChunkWs w = carve(workspace, B * NH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes) return MLSTM_E_WORKSPACE;
    return launch_gates_fwd(f, i, nullptr, nullptr, nullptr, nullptr, nullptr, B * NH, S, round_up(S, TILE), dtype,
                            static_cast<cudaStream_t>(stream), nullptr, summary, nullptr, 0, w.gscratch);
}

int mlstm_chunk_prepare(const void* k, const void* v, const void* f, const void* i, const double* carry_in,
                        double* summary_out, void* workspace, size_t workspace_bytes, int B, int NH, int S, int D,
                        int dtype, int chunk, void* stream) {
    if (!k || !v || !f || !i) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(k) || !aligned16(v)) return MLSTM_E_ALIGN;
    const int BH = B * NH, Spad = round_up(S, TILE);
    ChunkWs w = carve(workspace, BH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // (the gate pass also clears the status word and the work-item counters)
    if ((rc = launch_gates_fwd(f, i, w.ga, w.gAn, w.a_ref, w.An_ref, w.m, BH, S, Spad, dtype, st, carry_in, summary_out,
                               w.An_bound, chunk, w.gscratch, w.gaw, w.status, STATUS_WORDS)) != MLSTM_OK)
        return rc;
    if ((rc = launch_identity(w.ident, D, dtype, st)) != MLSTM_OK) return rc;
    // U_k[key, value] = sum_j exp(a_j - A_end(k)) k_j[key] v_j[value];  zU_k[key] = sum_j exp(...) k_j[key]
    PassParams p{};
    p.S = S; p.Spad = Spad; p.BH = BH; p.D = D; p.status = w.status; p.sched = w.status + 8; p.sched_zeroed = 1;
    p.X = k;  // unused by STATE (the stationary operand is the identity); keeps the tensor map valid
    p.Y = k; p.Z = v;
    p.col_rel = w.ga; p.col_w = w.gaw; p.col_ref = w.a_ref;
    p.row_rel = w.gAn; p.row_ref = w.An_ref;  // unused by STATE
    p.out = w.U; p.b_out = w.zU;
    p.chunk_tiles = chunk / TILE; p.NB = w.NB; p.An_bound = w.An_bound; p.ident = w.ident;
    return launch_pass_tc(STATE, p, dtype, dtype, st);
}

int mlstm_chunk_local_state(void* workspace, size_t workspace_bytes, float* S_end, float* z_end, int B, int NH, int S,
                            int D, int dtype, int chunk, void* stream) {
    if (!S_end || !z_end) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    ChunkWs w = carve(workspace, B * NH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes) return MLSTM_E_WORKSPACE;
    // the recurrence is linear: the state this segment adds is the scan from a zero state, with the
    // first decay taken from the carried-in stabiliser (a zero state makes that decay irrelevant)
    return launch_state_scan(w.U, w.zU, w.An_bound, nullptr, nullptr, w.states, w.zstate, S_end, z_end, B * NH, w.NB, D,
                             dtype, static_cast<cudaStream_t>(stream));
}

int mlstm_chunk_apply(const void* q, const void* k, const void* v, const void* o, const float* S_in, const float* z_in,
                      void* h, int h_dtype, float* S_out, float* z_out, void* workspace, size_t workspace_bytes, int B,
                      int NH, int S, int D, int dtype, int chunk, void* stream) {
    if (!q || !k || !v || !h) return MLSTM_E_ARG;
    if ((S_in == nullptr) != (z_in == nullptr)) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    if (h_dtype != MLSTM_DT_F32 && h_dtype != dtype) return MLSTM_E_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(h) || !aligned16(S_in) ||
        !aligned16(z_in))
        return MLSTM_E_ALIGN;
    const int BH = B * NH, Spad = round_up(S, TILE);
    ChunkWs w = carve(workspace, BH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // (the scan also clears the work-item counter of the output pass)
    if ((rc = launch_state_scan(w.U, w.zU, w.An_bound, S_in, z_in, w.states, w.zstate, S_out, z_out, BH, w.NB, D, dtype,
                                st, nullptr, nullptr, 0, nullptr, nullptr, 0, w.status + 8 + FWDC)) != MLSTM_OK)
        return rc;
    return launch_fwdc(q, k, v, o, h, h_dtype, w, BH, S, Spad, D, dtype, chunk, nullptr, st);
}

// ------------------------------------------------------------------------------------------------
// Backward of the chunkwise forward (no inbound state): dq, dk, dv, df, di in time linear in S.
// Within a block the three parallel backward passes run restricted to the block (modes DQC, DKC, DVC of
// the tensor-core pass); across blocks dQ uses the forward's inbound state S_k, and dK, dV use a state
// carried BACK over the blocks,
//   R_k = sum_{t after block k} exp(A_end(k) - A_t) (scale / n_t) q_t dh_t^T   (+ the vector r_k with g_t q_t),
// built like the forward states: per-block contributions from one STATE pass (Y = Q, Z = dH, column
// weights from the backward preparation), then the block recurrence walked in reverse.  dI and the row
// sums behind dF are row dots of the complete fp32 accumulators, as in the parallel backward
// (mlstm_matmul.py:256-316, 319-333 give the quantities; the reference has no chunkwise backward).
struct ChunkBwdWs {
    ChunkWs f;
    float *gB, *gBw, *g, *dI, *Rdot, *rvec;
    void *dh16, *statesT, *statesT2;
    size_t bytes;
};
static ChunkBwdWs carve_bwd_chunk(void* ws, int BH, int S, int D, int chunk, bool need_dh16) {
    ChunkBwdWs w{};
    w.f = carve(ws, BH, S, D, chunk);
    uint8_t* base = static_cast<uint8_t*>(ws);
    size_t off = w.f.bytes;
    auto take = [&](size_t bytes) {
        void* p = base ? base + off : nullptr;
        off += al(bytes);
        return p;
    };
    const size_t vec = static_cast<size_t>(BH) * round_up(S, TILE) * sizeof(float);
    const size_t nblk = static_cast<size_t>(BH) * w.f.NB;
    w.gB = static_cast<float*>(take(vec));
    w.gBw = static_cast<float*>(take(vec));
    w.g = static_cast<float*>(take(vec));
    w.dI = static_cast<float*>(take(vec * TC_DOT_PARTS));     // partial row dots, one per gate group
    w.Rdot = static_cast<float*>(take(vec * TC_DOT_PARTS));
    w.rvec = static_cast<float*>(take(nblk * D * sizeof(float)));
    w.statesT = take(nblk * D * D * 2);
    w.statesT2 = take(nblk * D * D * 2);
    w.dh16 = need_dh16 ? take(static_cast<size_t>(BH) * S * D * 2) : nullptr;
    w.bytes = off;
    return w;
}

size_t mlstm_chunk_bwd_workspace(int B, int NH, int S, int D, int dtype, int h_dtype, int chunk) {
    if (check_chunk_args(B, NH, S, D, dtype, chunk) != MLSTM_OK) return 0;
    return carve_bwd_chunk(nullptr, B * NH, S, D, chunk, h_dtype != dtype).bytes;
}

int mlstm_chunk_bwd(const void* dh, const void* q, const void* k, const void* v, const void* f, const void* i, const void* h,
                    const float* m, const float* b, void* dq, void* dk, void* dv, void* df, void* di, void* workspace,
                    size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int h_dtype, int chunk, void* stream) {
    if (!dh || !q || !k || !v || !f || !i || !h || !m || !b || !dq || !dk || !dv || !df || !di) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    if (h_dtype != MLSTM_DT_F32 && h_dtype != dtype) return MLSTM_E_ARG;
    if (!aligned16(dh) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(h) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return MLSTM_E_ALIGN;
    const int BH = B * NH, Spad = round_up(S, TILE);
    const bool need16 = h_dtype != dtype;
    ChunkBwdWs w = carve_bwd_chunk(workspace, BH, S, D, chunk, need16);
    if (!workspace || workspace_bytes < w.bytes || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const ChunkWs& c = w.f;
    // gates and forward states, as in the forward (the gate pass also clears the status word and the work-item counters)
    if ((rc = launch_gates_fwd(f, i, c.ga, c.gAn, c.a_ref, c.An_ref, nullptr, BH, S, Spad, dtype, st, nullptr, nullptr,
                               c.An_bound, chunk, c.gscratch, c.gaw, c.status, STATUS_WORDS)) != MLSTM_OK)
        return rc;
    if ((rc = launch_identity(c.ident, D, dtype, st)) != MLSTM_OK) return rc;
    PassParams p{};
    p.S = S; p.Spad = Spad; p.BH = BH; p.D = D; p.status = c.status; p.sched = c.status + 8; p.sched_zeroed = 1;
    p.chunk_tiles = chunk / TILE; p.NB = c.NB; p.An_bound = c.An_bound; p.ident = c.ident;
    p.dot_part_stride = static_cast<long long>(BH) * Spad;
    p.X = k; p.Y = k; p.Z = v;
    p.col_rel = c.ga; p.col_w = c.gaw; p.col_ref = c.a_ref; p.row_rel = c.gAn; p.row_ref = c.An_ref;
    p.out = c.U; p.b_out = c.zU;
    if ((rc = launch_pass_tc(STATE, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    // inbound states of the blocks, transposed (dQ's state step contracts over the value dimension), and z
    if ((rc = launch_state_scan(c.U, c.zU, c.An_bound, nullptr, nullptr, nullptr, c.zstate, nullptr, nullptr, BH, c.NB, D,
                                dtype, st, nullptr, nullptr, 0, nullptr, w.statesT, 0)) != MLSTM_OK)
        return rc;
    // delta = dh . h, n, db -> the backward's per-row vectors (and dh in the input type)
    if ((rc = launch_bwd_prep(h, dh, b, m, c.gAn, w.gB, w.gBw, w.g, w.dh16, BH, S, Spad, D, h_dtype, dtype, st)) != MLSTM_OK)
        return rc;
    const void* dhp = need16 ? w.dh16 : dh;
    // what every block contributes to the state carried back: P_k = sum_t beta_t q_t dh_t^T (tensor cores), p_k (vector)
    p.X = q; p.Y = q; p.Z = dhp;
    p.col_rel = w.gB; p.col_w = w.gBw; p.col_ref = c.An_ref;
    p.out = c.U; p.b_out = nullptr; p.state_reverse = 1;
    p.sched_zeroed = 0;     // the second STATE pass of the call: its counter is cleared again by the launcher
    if ((rc = launch_pass_tc(STATE, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    p.state_reverse = 0;
    p.sched_zeroed = 1;
    {
        dim3 grid(c.NB, BH);
        if (dtype == MLSTM_DT_BF16)
            launch_plain(rvec_partial_kernel<__nv_bfloat16>, grid, dim3(D), 0, st, static_cast<const __nv_bfloat16*>(q), w.gB, c.An_ref,
                       c.An_bound, w.g, c.zU, S, Spad, c.NB, chunk, D);
        else
            launch_plain(rvec_partial_kernel<__half>, grid, dim3(D), 0, st, static_cast<const __half*>(q), w.gB, c.An_ref, c.An_bound, w.g,
                       c.zU, S, Spad, c.NB, chunk, D);
        if (cudaGetLastError() != cudaSuccess) return MLSTM_E_CUDA;
    }
    // the block recurrence in reverse: R_k [key, value] (for dV), its transpose (for dK) and r_k
    if ((rc = launch_state_scan(c.U, c.zU, c.An_bound, nullptr, nullptr, c.states, w.rvec, nullptr, nullptr, BH, c.NB, D,
                                dtype, st, nullptr, nullptr, 0, nullptr, w.statesT2, 1)) != MLSTM_OK)
        return rc;
    // dQ = ((dH V^T + g_r) * decay) K within the block, + beta (S_k dh + g z_k) from the inbound state
    p.X = dhp; p.Y = v; p.Z = k;
    p.row_rel = w.gB; p.row_ref = c.An_ref; p.row_g = w.g; p.col_rel = c.ga; p.col_w = c.gaw; p.col_ref = c.a_ref; p.col_g = nullptr;
    p.states = w.statesT; p.zstate = c.zstate;
    p.out = dq; p.dot_src = q; p.dot_out = w.Rdot;
    if ((rc = launch_pass_tc(DQC, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    // dK = ((V dH^T + g_c) * decay) Q within the block, + gamma (R_k v + r_k) from the later blocks
    p.X = v; p.Y = dhp; p.Z = q;
    p.row_rel = c.ga; p.row_ref = c.a_ref; p.row_g = nullptr; p.col_rel = w.gB; p.col_w = w.gBw; p.col_ref = c.An_ref; p.col_g = w.g;
    p.states = w.statesT2; p.rvec = w.rvec;
    p.out = dk; p.dot_src = k; p.dot_out = w.dI;
    if ((rc = launch_pass_tc(DKC, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    // dV = ((K Q^T) * decay / n) dH within the block, + gamma R_k^T k from the later blocks
    p.X = k; p.Y = q; p.Z = dhp;
    p.col_g = nullptr; p.states = c.states;
    p.out = dv; p.dot_src = nullptr; p.dot_out = nullptr;
    if ((rc = launch_pass_tc(DVC, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    return launch_df(f, w.dI, w.Rdot, df, di, BH, S, Spad, dtype, st, TC_DOT_PARTS, static_cast<long long>(BH) * Spad, c.gscratch);
}

int mlstm_chunk_read_mb(const void* workspace, size_t workspace_bytes, float* m, float* b, int B, int NH, int S, int D, int dtype,
                        int chunk, void* stream) {
    if (!m || !b) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    ChunkWs w = carve(const_cast<void*>(workspace), B * NH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(B) * NH * S * sizeof(float);
    if (cudaMemcpyAsync(m, w.m, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return MLSTM_E_CUDA;
    if (cudaMemcpyAsync(b, w.b, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return MLSTM_E_CUDA;
    return MLSTM_OK;
}

size_t mlstm_chunk_sp_record_floats(int D) { return D > 0 ? static_cast<size_t>(D) * D + D + 4 : 0; }

int mlstm_chunk_sp_local(const void* k, const void* v, const void* f, const void* i, float* record, void* workspace,
                         size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int chunk, void* stream) {
    if (!record) return MLSTM_E_ARG;
    if (!aligned16(record)) return MLSTM_E_ALIGN;
    ChunkWs w = carve(workspace, B * NH, S, D, chunk);
    // gates and block states with no carry; this segment's own summary goes to the workspace
    int rc = mlstm_chunk_prepare(k, v, f, i, nullptr, workspace ? w.summary : nullptr, workspace, workspace_bytes, B, NH, S, D,
                                 dtype, chunk, stream);
    if (rc != MLSTM_OK) return rc;
    // the state the segment adds, stabilised by its own last prefix maximum, written into the record with the summary
    return launch_state_scan(w.U, w.zU, w.An_bound, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, B * NH, w.NB, D,
                             dtype, static_cast<cudaStream_t>(stream), nullptr, record, mlstm_chunk_sp_record_floats(D),
                             w.summary);
}

int mlstm_chunk_sp_apply(const void* q, const void* k, const void* v, const void* o, const float* gathered, int world,
                         int rank, void* h, int h_dtype, double* carry_out, void* workspace, size_t workspace_bytes, int B,
                         int NH, int S, int D, int dtype, int chunk, void* stream) {
    if (!q || !k || !v || !h || !gathered) return MLSTM_E_ARG;
    if (world <= 0 || rank < 0 || rank >= world) return MLSTM_E_ARG;
    int rc = check_chunk_args(B, NH, S, D, dtype, chunk);
    if (rc != MLSTM_OK) return rc;
    if (h_dtype != MLSTM_DT_F32 && h_dtype != dtype) return MLSTM_E_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(h) || !aligned16(gathered))
        return MLSTM_E_ALIGN;
    const int BH = B * NH, Spad = round_up(S, TILE);
    ChunkWs w = carve(workspace, BH, S, D, chunk);
    if (!workspace || workspace_bytes < w.bytes) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    {
        const int threads = 256;
        const int work = (D * D + D) / 4;
        dim3 grid((work + threads - 1) / threads, BH);
        sp_fold_kernel<<<grid, threads, 0, st>>>(gathered, rank, BH, D, mlstm_chunk_sp_record_floats(D), w.S_in, w.z_in,
                                                 w.late, carry_out);
        if (cudaGetLastError() != cudaSuccess) return MLSTM_E_CUDA;
    }
    if ((rc = launch_state_scan(w.U, w.zU, w.An_bound, w.S_in, w.z_in, w.states, w.zstate, nullptr, nullptr, BH, w.NB, D,
                                dtype, st, w.late, nullptr, 0, nullptr, nullptr, 0, w.status + 8 + FWDC)) != MLSTM_OK)
        return rc;
    return launch_fwdc(q, k, v, o, h, h_dtype, w, BH, S, Spad, D, dtype, chunk, w.late, st);
}

}  // extern "C"
