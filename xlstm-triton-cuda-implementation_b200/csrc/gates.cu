// Gate passes of the parallel mLSTM: everything that is O(S) or O(S*D) per slice and needs no
// contraction.  They take the place of the in-kernel log-sigmoid cumulative sums and running
// maxima of the reference (mlstm_matmul.py:59, 73-84; cuda-src/gpu_utils.cuh:125-144), of its
// db kernel (mlstm_matmul.py:132-197, reduced here to a row dot product by the identity
// sum_c C~_rc dC_rc = n_r (dh_r . h_r)) and of its dF kernel (mlstm_matmul.py:319-333).
#include <atomic>
#include <cooperative_groups.h>

#include "mlstm_common.cuh"

namespace mlstm {
namespace {

constexpr double LOG2E_D = 1.4426950408889634;
constexpr int SCAN_THREADS = 1024;
constexpr int GATE_SEG_TOKENS = 4096;  // positions per block when a slice is cut into segments

// Inclusive block scans over SCAN_THREADS elements (one per thread) with a running carry.
__device__ __forceinline__ double block_scan_add(double x, double* warp_tot, double& carry_smem_view) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) warp_tot[warp] = x;
    __syncthreads();
    if (warp == 0) {
        double t = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            double y = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += y;
        }
        warp_tot[lane] = t;
    }
    __syncthreads();
    const double before = (warp > 0 ? warp_tot[warp - 1] : 0.0) + carry_smem_view;
    const double total = warp_tot[31];
    __syncthreads();
    if (threadIdx.x == 0) carry_smem_view += total;
    __syncthreads();
    return x + before;
}

// Exclusive running maximum over the block's threads, seeded with the carry; the carry then takes the block's
// total in.
__device__ __forceinline__ double block_scan_max_excl(double x, double* warp_tot, double& carry_smem_view) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x = fmax(x, y);
    }
    if (lane == 31) warp_tot[warp] = x;
    double excl = __shfl_up_sync(0xffffffffu, x, 1);
    if (lane == 0) excl = -INFINITY;
    __syncthreads();
    if (warp == 0) {
        double t = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            double y = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t = fmax(t, y);
        }
        warp_tot[lane] = t;
    }
    __syncthreads();
    const double before = fmax(warp > 0 ? warp_tot[warp - 1] : -INFINITY, carry_smem_view);
    const double total = warp_tot[31];
    __syncthreads();
    if (threadIdx.x == 0) carry_smem_view = fmax(carry_smem_view, total);
    __syncthreads();
    return fmax(excl, before);
}

// Four consecutive positions per thread and round (a round = 4096 positions = one segment): the two block scans,
// with their barriers, run once per round on the threads' totals.
constexpr int GATE_V = 4;
static_assert(GATE_SEG_TOKENS == GATE_V * SCAN_THREADS && REF_BLOCK % GATE_V == 0 && 32 % (REF_BLOCK / GATE_V) == 0,
              "a round is one segment; a reference block is a group of lanes inside a warp");

// One block per slice.  With F = cumsum(logsigmoid f), a = i - F, A = running maximum of a (all in
// double), it writes m = F + A and the two gate vectors in log2 units, re-centred per block of
// REF_BLOCK positions so that fp32 keeps its relative accuracy however long the sequence is:
//   ga_rel[t]  = (a_t - a_max(block)) * log2e  <= 0  a_ref[block]  = a_max * log2e        (double)
//   gAn_rel[t] = (A_first(block) - A_t) * log2e <= 0 An_ref[block] = -A_first * log2e     (double)
//   ga_w[t]    = exp2(ga_rel[t])  (optional): off the diagonal the kernels use exp2(x + y) = exp2(x) exp2(y)
//                with the row factor exp2(row term + references) <= const computed once per row and block
// A kernel forms exp2(col_rel[c] + float(row_rel[r] + row_ref[r / REF_BLOCK] + col_ref[c / REF_BLOCK])),
// the bracket in double once per block of columns.  Padding (t >= S): ga_rel = -inf (a padded column
// contributes exactly zero), gAn_rel = 0, references 0.  m may be null.
// Chunkwise / sequence-parallel extras (all optional): carry_in[bh] = {F, A} at the end of the
// preceding segment (natural-log units; absent = {0, -inf}); summary_out[bh] = {F, A} at the end of
// this segment; An_bound[bh][0] = -A_in*log2e and An_bound[bh][k+1] = -A*log2e at the last position
// of block k (blocks of chunk_len positions).  The vector outputs may be null (summary only).
// Long sequences are cut into segments of seg_tokens positions, one block each (blockIdx.x =
// slice * nseg + segment; carry_in and summary_out are then per block): first a summary-only launch
// with no carries, then gates_fold_kernel turns the segment summaries into per-segment carries, then
// the full launch.  nseg = 1 is the plain one-block-per-slice form.
// COOP (long slices, all segments resident at once, cooperative launch): the three steps in one kernel.  Every block
// scans its segment with no carry, publishes the segment's {F, A} totals in coop_local, the grid meets, every block
// folds the totals of the segments before it (carry_in and summary_out are then per SLICE) and shifts what it holds in
// registers: F += F_in, a -= F_in, A = max(A - F_in, A_in).  One pass over f and i, one launch.
template <typename T, bool COOP = false>
__global__ void __launch_bounds__(SCAN_THREADS) gates_fwd_kernel(const T* __restrict__ f, const T* __restrict__ i,
                                                                 float* __restrict__ ga_rel, float* __restrict__ gAn_rel,
                                                                 float* __restrict__ ga_w,
                                                                 double* __restrict__ a_ref, double* __restrict__ An_ref,
                                                                 float* __restrict__ m, int S, int Spad,
                                                                 const double* __restrict__ carry_in,
                                                                 double* __restrict__ summary_out,
                                                                 double* __restrict__ An_bound, int chunk_len, int nseg,
                                                                 int seg_tokens, int* __restrict__ zero_words, int n_zero,
                                                                 double* __restrict__ coop_local) {
    __shared__ double wsum[32];
    __shared__ double wmax[32];
    [[maybe_unused]] __shared__ double fold_in[2];
    grid_dep_wait();
    grid_dep_launch();
    // the call's status word and work-item counters start at zero: cleared here, by the call's first kernel,
    // instead of by memsets of their own in front of every pass
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < n_zero) zero_words[threadIdx.x] = 0;
    __shared__ double carry_sum;
    __shared__ double carry_max;
    const int bh = blockIdx.x / nseg;
    const int seg = blockIdx.x - bh * nseg;
    const int t_begin = seg * seg_tokens;
    const int t_end = min(t_begin + seg_tokens, Spad);
    const int nref = Spad / REF_BLOCK;
    const int nb = chunk_len > 0 ? (S + chunk_len - 1) / chunk_len : 0;
    constexpr int LANES_PER_REF = REF_BLOCK / GATE_V;   // 16 threads share a reference block
    if (threadIdx.x == 0) {
        carry_sum = (carry_in && !COOP) ? carry_in[2 * blockIdx.x] : 0.0;
        carry_max = (carry_in && !COOP) ? carry_in[2 * blockIdx.x + 1] : -INFINITY;
        if (!COOP && An_bound && seg == 0) An_bound[static_cast<size_t>(bh) * (nb + 1)] = -carry_max * LOG2E_D;
    }
    __syncthreads();
    for (int base = t_begin; base < t_end; base += GATE_V * SCAN_THREADS) {
        const int t0 = base + GATE_V * threadIdx.x;     // this thread's first position (a multiple of four)
        double F[GATE_V], a[GATE_V], A[GATE_V];
        double run = 0.0;
#pragma unroll
        for (int j = 0; j < GATE_V; j++) {
            const int t = t0 + j;
            double lf = 0.0;
            a[j] = 0.0;
            if (t < S) {
                // logsigmoid in fp32 (relative error 1e-7 per term), summed in double
                const float x = to_f32<T>(f[static_cast<size_t>(bh) * S + t]);
                lf = static_cast<double>(x < 0.0f ? x - log1pf(expf(x)) : -log1pf(expf(-x)));
                a[j] = static_cast<double>(to_f32<T>(i[static_cast<size_t>(bh) * S + t]));   // i for now
            }
            run += lf;
            F[j] = run;    // relative to the thread's first position
        }
        const double incl = block_scan_add(run, wsum, carry_sum);   // carry + everything up to and including this thread
        const double offs = incl - run;
        double amax = -INFINITY;
#pragma unroll
        for (int j = 0; j < GATE_V; j++) {
            F[j] += offs;
            a[j] = (t0 + j < S) ? a[j] - F[j] : -INFINITY;
            amax = fmax(amax, a[j]);
            A[j] = amax;   // running maximum inside the thread
        }
        const double pre = block_scan_max_excl(amax, wmax, carry_max);
#pragma unroll
        for (int j = 0; j < GATE_V; j++) A[j] = fmax(A[j], pre);
        if constexpr (COOP) {
            // (the host launches this form with one round per block: the segment is in registers)
            if (threadIdx.x == 0) {
                coop_local[2 * blockIdx.x] = carry_sum;       // the segment's totals, no carry
                coop_local[2 * blockIdx.x + 1] = carry_max;
                __threadfence();
            }
            cooperative_groups::this_grid().sync();
            if (threadIdx.x == 0) {
                double Fin = carry_in ? carry_in[2 * bh] : 0.0;
                double Ain = carry_in ? carry_in[2 * bh + 1] : -INFINITY;
                for (int s2 = 0; s2 < seg; s2++) {     // a position's a = i - F shifts by -F_in when F_in precedes it
                    const double* tot = coop_local + 2 * (static_cast<size_t>(bh) * nseg + s2);
                    Ain = fmax(Ain, tot[1] - Fin);
                    Fin += tot[0];
                }
                fold_in[0] = Fin;
                fold_in[1] = Ain;
                if (An_bound && seg == 0) An_bound[static_cast<size_t>(bh) * (nb + 1)] = -Ain * LOG2E_D;
                if (summary_out && seg == nseg - 1) {
                    summary_out[2 * bh] = Fin + carry_sum;
                    summary_out[2 * bh + 1] = fmax(Ain, carry_max - Fin);
                }
            }
            __syncthreads();
            const double Fin = fold_in[0], Ain = fold_in[1];
            amax = -INFINITY;
#pragma unroll
            for (int j = 0; j < GATE_V; j++) {
                F[j] += Fin;
                a[j] -= Fin;                       // (-inf in the padding stays -inf)
                A[j] = fmax(A[j] - Fin, Ain);
                amax = fmax(amax, a[j]);
            }
        }
        // reference of a: the block's maximum (so ga_rel <= 0 and exp2(ga_rel) cannot overflow);
        // reference of -A: the block's first element, which is its maximum because A never decreases
        double bm = amax;
#pragma unroll
        for (int o = LANES_PER_REF / 2; o > 0; o >>= 1) bm = fmax(bm, __shfl_xor_sync(0xffffffffu, bm, o));
        const double ra = (bm == -INFINITY) ? 0.0 : bm;
        const int lead = (threadIdx.x & 31) & ~(LANES_PER_REF - 1);      // lane that holds the block's first position
        double rA = __shfl_sync(0xffffffffu, A[0], lead);
        if (base + GATE_V * (static_cast<int>(threadIdx.x) & ~(LANES_PER_REF - 1)) >= S) rA = 0.0;   // block of pure padding
        if (t0 < Spad && ga_rel) {
            float rel[GATE_V], w[GATE_V], An[GATE_V];
#pragma unroll
            for (int j = 0; j < GATE_V; j++) {
                const bool in = t0 + j < S;
                rel[j] = in ? static_cast<float>((a[j] - ra) * LOG2E_D) : -INFINITY;
                w[j] = exp2f(rel[j]);   // in (0, 1]; 0 in the padding
                An[j] = in ? static_cast<float>((rA - A[j]) * LOG2E_D) : 0.0f;
            }
            const size_t vi = static_cast<size_t>(bh) * Spad + t0;    // Spad and t0 are multiples of four
            *reinterpret_cast<float4*>(ga_rel + vi) = make_float4(rel[0], rel[1], rel[2], rel[3]);
            if (ga_w) *reinterpret_cast<float4*>(ga_w + vi) = make_float4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<float4*>(gAn_rel + vi) = make_float4(An[0], An[1], An[2], An[3]);
            if ((threadIdx.x & (LANES_PER_REF - 1)) == 0) {
                a_ref[static_cast<size_t>(bh) * nref + t0 / REF_BLOCK] = ra * LOG2E_D;
                An_ref[static_cast<size_t>(bh) * nref + t0 / REF_BLOCK] = -rA * LOG2E_D;
            }
        }
#pragma unroll
        for (int j = 0; j < GATE_V; j++) {
            const int t = t0 + j;
            if (t < S && m) m[static_cast<size_t>(bh) * S + t] = static_cast<float>(F[j] + A[j]);
            if (t < S && An_bound && ((t + 1) % chunk_len == 0 || t == S - 1))
                An_bound[static_cast<size_t>(bh) * (nb + 1) + t / chunk_len + 1] = -A[j] * LOG2E_D;
        }
    }
    if (!COOP && threadIdx.x == 0 && summary_out) {
        summary_out[2 * blockIdx.x] = carry_sum;
        summary_out[2 * blockIdx.x + 1] = carry_max;
    }
}

// One thread per slice: segment summaries taken with no carry ({F_loc, A_loc}) -> the carry of every
// segment and the slice's own summary.  A position's a = i - F shifts by -F_in when F_in precedes it,
// so a segment's prefix maximum in slice terms is A_loc - F_in.
__global__ void gates_fold_kernel(const double* __restrict__ local, const double* __restrict__ slice_carry,
                                  double* __restrict__ seg_carry, double* __restrict__ slice_summary, int BH, int nseg) {
    grid_dep_wait();
    grid_dep_launch();
    const int bh = blockIdx.x * blockDim.x + threadIdx.x;
    if (bh >= BH) return;
    double F = slice_carry ? slice_carry[2 * bh] : 0.0;
    double A = slice_carry ? slice_carry[2 * bh + 1] : -INFINITY;
    for (int s = 0; s < nseg; s++) {
        const size_t k = (static_cast<size_t>(bh) * nseg + s) * 2;
        seg_carry[k] = F;
        seg_carry[k + 1] = A;
        A = fmax(A, local[k + 1] - F);
        F += local[k];
    }
    if (slice_summary) {
        slice_summary[2 * bh] = F;
        slice_summary[2 * bh + 1] = A;
    }
}

// One warp per row: delta = dh.h, n, db, and from them the two per-row vectors of the backward:
//   gB_rel = gAn_rel + log2(scale / n)  (same block references as gAn_rel),   g = db * n
// (db = sign(b) * (-delta / n) * [|b| > exp(-m)], mlstm_matmul.py:194-196 with the sum replaced by
// n*delta).  Optionally writes dh converted to the 16-bit input type for the tensor-core passes.
// Rows are read with 16-byte accesses.  Padding rows: gB_rel = -inf, g = 0.
constexpr int PREP_ROWS = 4;   // positions per warp in bwd_prep_kernel

template <typename HT, typename T16>
__global__ void bwd_prep_kernel(const HT* __restrict__ h, const HT* __restrict__ dh, const float* __restrict__ b,
                                const float* __restrict__ m, const float* __restrict__ gAn_rel,
                                float* __restrict__ gB_rel, float* __restrict__ gB_w, float* __restrict__ g,
                                T16* __restrict__ dh16, int BH, int S, int Spad, int D, float log2_scale) {
    grid_dep_wait();
    grid_dep_launch();
    // A warp takes PREP_ROWS consecutive positions of one slice (Spad is a multiple of 128): all of their row
    // loads and the per-position scalars are requested before anything is used, so a warp pays the memory
    // latency once instead of twice per position.
    constexpr int VEC = 16 / sizeof(HT);
    const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long first = static_cast<long long>(warp_global) * PREP_ROWS;
    if (first >= static_cast<long long>(BH) * Spad) return;
    const int bh = static_cast<int>(first / Spad), t0 = static_cast<int>(first % Spad);
    // lane r < PREP_ROWS finishes position t0 + r
    const int tl = t0 + lane;
    const bool mine = lane < PREP_ROWS;
    const bool mine_valid = mine && tl < S;
    float bb = 0.0f, mm = 0.0f, ga = 0.0f;
    if (mine_valid) {
        const size_t idx = static_cast<size_t>(bh) * S + tl;
        bb = b[idx];
        mm = m[idx];
        ga = gAn_rel[first + lane];
    }
    float delta[PREP_ROWS];
#pragma unroll
    for (int r = 0; r < PREP_ROWS; r++) {
        delta[r] = 0.0f;
        if (t0 + r < S) {
            const size_t row = (static_cast<size_t>(bh) * S + t0 + r) * D;
            for (int d = lane * VEC; d < D; d += 32 * VEC) {
                const uint4 hraw = *reinterpret_cast<const uint4*>(h + row + d);
                const uint4 draw = *reinterpret_cast<const uint4*>(dh + row + d);
                const HT* hv = reinterpret_cast<const HT*>(&hraw);
                const HT* dv = reinterpret_cast<const HT*>(&draw);
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    const float x = to_f32<HT>(dv[j]);
                    delta[r] += x * to_f32<HT>(hv[j]);
                    if (dh16) dh16[row + d + j] = from_f32<T16>(x);
                }
            }
        }
    }
    float my_delta = 0.0f;
#pragma unroll
    for (int r = 0; r < PREP_ROWS; r++) {
        float x = delta[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        if (lane == r) my_delta = x;
    }
    if (mine) {
        const size_t o = static_cast<size_t>(first) + lane;
        if (!mine_valid) {   // padding positions
            gB_rel[o] = -INFINITY;
            gB_w[o] = 0.0f;
            g[o] = 0.0f;
        } else {
            const float em = expf(-mm);
            const float n = fmaxf(fabsf(bb), em) + 1e-6f;
            const float sgn = bb > 0.0f ? 1.0f : (bb < 0.0f ? -1.0f : 0.0f);
            const float db = (fabsf(bb) > em) ? sgn * (-my_delta / n) : 0.0f;
            const float gg = db * n;
            g[o] = isfinite(gg) ? gg : 0.0f;
            const float rel = ga + (log2_scale - log2f(n));
            gB_rel[o] = rel;
            gB_w[o] = exp2f(rel);   // the same quantity as a factor, for the off-diagonal tiles
        }
    }
}

// dF_t = sigmoid(-f_t) * sum_{s<t} (dI_s - R_s), dF_0 = 0, and dI converted to the output type
// (mlstm_matmul.py:316, 319-333).  One block per slice, or, for long slices, one block per segment of
// seg_tokens positions (blockIdx.x = slice * nseg + segment) that starts from the sum of the segments before it:
// seg_totals[slice * nseg + s] from df_total_kernel.
// dI and R arrive as partial row dots (one per gate group of the tensor-core passes): fixed order of addition.
__device__ __forceinline__ void df_terms(const float* __restrict__ dI, const float* __restrict__ R, size_t idx, int nparts,
                                         long long part_stride, float& dIv, float& Rv) {
    dIv = 0.0f;
    Rv = 0.0f;
    for (int k = 0; k < nparts; k++) {
        dIv += dI[k * part_stride + idx];
        Rv += R[k * part_stride + idx];
    }
}

__global__ void __launch_bounds__(SCAN_THREADS) df_total_kernel(const float* __restrict__ dI, const float* __restrict__ R,
                                                                double* __restrict__ seg_totals, int S, int Spad, int nparts,
                                                                long long part_stride, int nseg, int seg_tokens) {
    __shared__ double wsum[32];
    grid_dep_wait();
    grid_dep_launch();
    const int bh = blockIdx.x / nseg, seg = blockIdx.x - bh * nseg;
    const int t_begin = seg * seg_tokens, t_end = min(t_begin + seg_tokens, S);
    double x = 0.0;
    for (int t = t_begin + threadIdx.x; t < t_end; t += SCAN_THREADS) {
        float dIv, Rv;
        df_terms(dI, R, static_cast<size_t>(bh) * Spad + t, nparts, part_stride, dIv, Rv);
        x += static_cast<double>(dIv) - static_cast<double>(Rv);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = x;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int w = 0; w < SCAN_THREADS / 32; w++) tot += wsum[w];
        seg_totals[blockIdx.x] = tot;
    }
}

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS) df_kernel(const T* __restrict__ f, const float* __restrict__ dI,
                                                          const float* __restrict__ R, T* __restrict__ df,
                                                          T* __restrict__ di, int S, int Spad, int nparts,
                                                          long long part_stride, const double* __restrict__ seg_totals,
                                                          int nseg, int seg_tokens) {
    __shared__ double wsum[32];
    __shared__ double carry_sum;
    grid_dep_wait();
    grid_dep_launch();
    const int bh = blockIdx.x / nseg, seg = blockIdx.x - bh * nseg;
    const int t_begin = seg * seg_tokens, t_end = min(t_begin + seg_tokens, S);
    if (threadIdx.x == 0) {
        double c = 0.0;
        for (int s2 = 0; s2 < seg; s2++) c += seg_totals[bh * nseg + s2];
        carry_sum = c;
    }
    __syncthreads();
    for (int base = t_begin; base < t_end; base += SCAN_THREADS) {
        const int t = base + threadIdx.x;
        const bool in = t < t_end;
        double x = 0.0;
        float dIv = 0.0f;
        if (in) {
            float Rv;
            df_terms(dI, R, static_cast<size_t>(bh) * Spad + t, nparts, part_stride, dIv, Rv);
            x = static_cast<double>(dIv) - static_cast<double>(Rv);
        }
        const double G = block_scan_add(x, wsum, carry_sum);  // inclusive
        if (in) {
            const float fv = to_f32<T>(f[static_cast<size_t>(bh) * S + t]);
            const double sig = 1.0 / (1.0 + exp(static_cast<double>(fv)));  // sigmoid(-f)
            const double val = t == 0 ? 0.0 : sig * (G - x);
            df[static_cast<size_t>(bh) * S + t] = from_f32<T>(static_cast<float>(val));
            di[static_cast<size_t>(bh) * S + t] = from_f32<T>(dIv);
        }
    }
}

// Output gate, elementwise: h = h_inner * silu(o) (mlstm_scan.py:273-278; the "integrate o" note at
// mlstm_matmul.py:36) and its derivative: dh_inner = dh * silu(o), do = dh * h_inner * silu'(o) with
// silu'(x) = sigma(x) (1 + x (1 - sigma(x))).  Eight elements per thread, 16-byte accesses on the 16-bit side.
template <typename HT, typename OT, bool BWD>
__global__ void ogate_kernel(const HT* __restrict__ dh, const HT* __restrict__ h_inner, const OT* __restrict__ o,
                             HT* __restrict__ out_h, OT* __restrict__ out_o, long long n) {
    grid_dep_wait();
    grid_dep_launch();
    const long long base = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (base >= n) return;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const long long e = base + j;
        if (e >= n) break;
        const float x = to_f32<OT>(o[e]);
        const float sg = 1.0f / (1.0f + __expf(-x));
        const float hi = to_f32<HT>(h_inner[e]);
        if (BWD) {
            const float g = to_f32<HT>(dh[e]);
            out_h[e] = from_f32<HT>(g * x * sg);
            out_o[e] = from_f32<OT>(g * hi * sg * (1.0f + x * (1.0f - sg)));
        } else {
            out_h[e] = from_f32<HT>(hi * x * sg);
        }
    }
}

template <bool BWD>
static int ogate_dispatch(const void* dh, const void* h_inner, const void* o, void* out_h, void* out_o, long long n, int h_dtype,
                          int o_dtype, cudaStream_t st) {
    const int threads = 256;
    const long long blocks = (n + threads * 8 - 1) / (threads * 8);
    if (blocks <= 0 || blocks > 0x7fffffffLL) return MLSTM_E_SHAPE;
#define OGATE_LAUNCH(HT, OT)                                                                                              \
    ogate_kernel<HT, OT, BWD><<<(unsigned)blocks, threads, 0, st>>>((const HT*)dh, (const HT*)h_inner, (const OT*)o, (HT*)out_h, \
                                                                    (OT*)out_o, n)
    if (h_dtype == MLSTM_DT_F32) {
        if (o_dtype == MLSTM_DT_F32) OGATE_LAUNCH(float, float);
        else if (o_dtype == MLSTM_DT_F16) OGATE_LAUNCH(float, __half);
        else if (o_dtype == MLSTM_DT_BF16) OGATE_LAUNCH(float, __nv_bfloat16);
        else return MLSTM_E_ARG;
    } else if (h_dtype == MLSTM_DT_F16 && o_dtype == MLSTM_DT_F16) {
        OGATE_LAUNCH(__half, __half);
    } else if (h_dtype == MLSTM_DT_BF16 && o_dtype == MLSTM_DT_BF16) {
        OGATE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    } else {
        return MLSTM_E_ARG;
    }
#undef OGATE_LAUNCH
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

// Round fp32 values to the nearest tf32 (10 mantissa bits).  The tensor cores drop the low 13 bits
// of fp32 operands; rounding first halves the error and removes its bias.
__global__ void round_tf32_kernel(const float4* __restrict__ in, float4* __restrict__ out, long long n4) {
    grid_dep_wait();
    grid_dep_launch();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    const float4 x = in[idx];
    uint4 y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y.x) : "f"(x.x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y.y) : "f"(x.y));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y.z) : "f"(x.z));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y.w) : "f"(x.w));
    out[idx] = *reinterpret_cast<float4*>(&y);
}

// fp32 -> two bf16 halves: hi = bf16(x), mid = bf16(x - hi), written side by side as rows of 2 D values
// (hi | mid).  x - hi is exact in fp32, so hi + mid carries 16 mantissa bits of x.  Four values per thread;
// blockIdx.y selects one of up to four tensors of the same shape.
struct SplitPtrs {
    const float4* in[4];
    __nv_bfloat16* out[4];
};
__global__ void split_bf16_kernel(const SplitPtrs ptrs, long long n4, int D) {
    grid_dep_wait();
    grid_dep_launch();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    const float4* __restrict__ in = ptrs.in[blockIdx.y];
    __nv_bfloat16* __restrict__ out = ptrs.out[blockIdx.y];
    const float4 x = in[idx];
    const long long e = idx * 4;
    const long long row = e / D;
    const int col = static_cast<int>(e - row * D);
    __nv_bfloat162 h01 = __floats2bfloat162_rn(x.x, x.y), h23 = __floats2bfloat162_rn(x.z, x.w);
    const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
    __nv_bfloat162 m01 = __floats2bfloat162_rn(x.x - f01.x, x.y - f01.y), m23 = __floats2bfloat162_rn(x.z - f23.x, x.w - f23.y);
    __nv_bfloat16* dst = out + row * 2 * D + col;
    uint2 hv, mv;
    hv.x = *reinterpret_cast<uint32_t*>(&h01); hv.y = *reinterpret_cast<uint32_t*>(&h23);
    mv.x = *reinterpret_cast<uint32_t*>(&m01); mv.y = *reinterpret_cast<uint32_t*>(&m23);
    *reinterpret_cast<uint2*>(dst) = hv;
    *reinterpret_cast<uint2*>(dst + D) = mv;
}

}  // namespace

int launch_split_bf16_multi(const void* const* in, void* const* out, int count, long long rows, int D, cudaStream_t st) {
    if (count < 1 || count > 4) return MLSTM_E_ARG;
    const long long n4 = rows * D / 4;
    const int threads = 256;
    const long long blocks = (n4 + threads - 1) / threads;
    if (blocks <= 0 || blocks > 0x7fffffffLL || (D & 3)) return MLSTM_E_SHAPE;
    SplitPtrs ptrs{};
    for (int k = 0; k < count; k++) {
        ptrs.in[k] = static_cast<const float4*>(in[k]);
        ptrs.out[k] = static_cast<__nv_bfloat16*>(out[k]);
    }
    return launch_plain(split_bf16_kernel, dim3(static_cast<unsigned>(blocks), count), dim3(threads), 0, st, ptrs, n4, D) == cudaSuccess
               ? MLSTM_OK : MLSTM_E_CUDA;
}

int launch_split_bf16(const void* in, void* out, long long rows, int D, cudaStream_t st) {
    return launch_split_bf16_multi(&in, &out, 1, rows, D, st);
}

int launch_ogate_fwd(const void* h_inner, const void* o, void* h, long long n, int h_dtype, int o_dtype, cudaStream_t st) {
    return ogate_dispatch<false>(nullptr, h_inner, o, h, nullptr, n, h_dtype, o_dtype, st);
}

int launch_ogate_bwd(const void* dh, const void* h_inner, const void* o, void* dh_inner, void* d_o, long long n, int h_dtype,
                     int o_dtype, cudaStream_t st) {
    return ogate_dispatch<true>(dh, h_inner, o, dh_inner, d_o, n, h_dtype, o_dtype, st);
}

int launch_round_tf32(const void* in, void* out, long long n, cudaStream_t st) {
    const long long n4 = n / 4;
    const int threads = 256;
    const long long blocks = (n4 + threads - 1) / threads;
    if (blocks > 0x7fffffffLL || (n & 3)) return MLSTM_E_SHAPE;
    return launch_plain(round_tf32_kernel, dim3((unsigned)blocks), dim3(threads), 0, st, static_cast<const float4*>(in),
                      static_cast<float4*>(out), n4) == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

namespace {
// Blocks of the cooperative gate kernel that can be resident on the current device at once (cached per device).
template <typename T>
int coop_capacity() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    int v = cached[dev].load(std::memory_order_acquire);
    if (v > 0) return v;
    int per_sm = 0, sms = 0, coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gates_fwd_kernel<T, true>, SCAN_THREADS, 0) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    v = per_sm * sms;
    if (v > 0) cached[dev].store(v, std::memory_order_release);
    return v;
}

template <typename T>
int gates_launch_typed(const void* f, const void* i, float* ga, float* gA, double* a_ref, double* An_ref, float* m, int BH,
                       int S, int Spad, cudaStream_t st, const double* carry_in, double* summary_out, double* An_bound,
                       int chunk_len, double* scratch, float* ga_w, int* zero_words, int n_zero) {
    const int nseg = scratch ? (Spad + GATE_SEG_TOKENS - 1) / GATE_SEG_TOKENS : 1;
    if (n_zero > SCAN_THREADS) return MLSTM_E_ARG;
    if (nseg <= 1) {
        return launch_plain(gates_fwd_kernel<T, false>, dim3(BH), dim3(SCAN_THREADS), 0, st, (const T*)f, (const T*)i, ga, gA, ga_w, a_ref,
                            An_ref, m, S, Spad, carry_in, summary_out, An_bound, chunk_len, 1, Spad, zero_words, n_zero,
                            static_cast<double*>(nullptr)) == cudaSuccess
                   ? MLSTM_OK : MLSTM_E_CUDA;
    }
    double* local = scratch;                                         // [BH * nseg][2]
    if ((ga || m || An_bound) && BH * nseg <= coop_capacity<T>()) {
        // all segments fit on the device at once: one cooperative launch does summaries, fold and gates
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(BH * nseg);
        cfg.blockDim = dim3(SCAN_THREADS);
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeCooperative;
        attr.val.cooperative = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        cudaError_t ce = cudaLaunchKernelEx(&cfg, gates_fwd_kernel<T, true>, (const T*)f, (const T*)i, ga, gA, ga_w, a_ref, An_ref, m, S,
                                            Spad, carry_in, summary_out, An_bound, chunk_len, nseg, GATE_SEG_TOKENS, zero_words, n_zero,
                                            local);
        if (ce == cudaSuccess) return MLSTM_OK;
        cudaGetLastError();   // (not launched: take the three-launch path)
    }
    double* seg_carry = scratch + static_cast<size_t>(BH) * nseg * 2;  // [BH * nseg][2]
    // (typed null pointers for the summary-only launch: the launcher converts arguments to the kernel's parameter types)
    float* nof = nullptr;
    double* nod = nullptr;
    const double* nocd = nullptr;
    int* noi = nullptr;
    cudaError_t ce = launch_plain(gates_fwd_kernel<T, false>, dim3(BH * nseg), dim3(SCAN_THREADS), 0, st, (const T*)f, (const T*)i, nof, nof,
                                  nof, nod, nod, nof, S, Spad, nocd, local, nod, 0, nseg, GATE_SEG_TOKENS, zero_words, n_zero, nod);
    if (ce == cudaSuccess)
        ce = launch_plain(gates_fold_kernel, dim3((BH + 127) / 128), dim3(128), 0, st, (const double*)local, carry_in, seg_carry,
                        summary_out, BH, nseg);
    if (ce == cudaSuccess && (ga || m || An_bound))
        ce = launch_plain(gates_fwd_kernel<T, false>, dim3(BH * nseg), dim3(SCAN_THREADS), 0, st, (const T*)f, (const T*)i, ga, gA, ga_w,
                          a_ref, An_ref, m, S, Spad, (const double*)seg_carry, nod, An_bound, chunk_len, nseg, GATE_SEG_TOKENS, noi, 0,
                          nod);
    return ce == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}
}  // namespace

size_t gates_scratch_bytes(int BH, int Spad) {
    const size_t nseg = (static_cast<size_t>(Spad) + GATE_SEG_TOKENS - 1) / GATE_SEG_TOKENS;
    return nseg > 1 ? static_cast<size_t>(BH) * nseg * 4 * sizeof(double) : 0;
}

int launch_gates_fwd(const void* f, const void* i, float* ga, float* gA, double* a_ref, double* An_ref, float* m, int BH,
                     int S, int Spad, int dtype, cudaStream_t st, const double* carry_in, double* summary_out,
                     double* An_bound, int chunk_len, double* scratch, float* ga_w, int* zero_words, int n_zero) {
    switch (dtype) {
        case MLSTM_DT_F32:
            return gates_launch_typed<float>(f, i, ga, gA, a_ref, An_ref, m, BH, S, Spad, st, carry_in, summary_out, An_bound,
                                             chunk_len, scratch, ga_w, zero_words, n_zero);
        case MLSTM_DT_F16:
            return gates_launch_typed<__half>(f, i, ga, gA, a_ref, An_ref, m, BH, S, Spad, st, carry_in, summary_out, An_bound,
                                              chunk_len, scratch, ga_w, zero_words, n_zero);
        case MLSTM_DT_BF16:
            return gates_launch_typed<__nv_bfloat16>(f, i, ga, gA, a_ref, An_ref, m, BH, S, Spad, st, carry_in, summary_out,
                                                     An_bound, chunk_len, scratch, ga_w, zero_words, n_zero);
    }
    return MLSTM_E_ARG;
}

template <typename HT>
static int bwd_prep_dispatch(const void* h, const void* dh, const float* b, const float* m, const float* gA, float* gB,
                             float* gBw, float* g, void* dh16, int BH, int S, int Spad, int D, int dtype, cudaStream_t st) {
    const long long warps = static_cast<long long>(BH) * Spad / PREP_ROWS;   // Spad is a multiple of 128
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) return MLSTM_E_SHAPE;
    const float log2_scale = -0.5f * log2f(static_cast<float>(D));
    if (dtype == MLSTM_DT_BF16)
        launch_plain(bwd_prep_kernel<HT, __nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, st, 
            (const HT*)h, (const HT*)dh, b, m, gA, gB, gBw, g, (__nv_bfloat16*)dh16, BH, S, Spad, D, log2_scale);
    else
        launch_plain(bwd_prep_kernel<HT, __half>, dim3((unsigned)blocks), dim3(threads), 0, st, (const HT*)h, (const HT*)dh, b, m, gA, gB, gBw, g,
                                                                         (__half*)dh16, BH, S, Spad, D, log2_scale);
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

int launch_bwd_prep(const void* h, const void* dh, const float* b, const float* m, const float* gA, float* gB, float* gBw,
                    float* g, void* dh16, int BH, int S, int Spad, int D, int h_dtype, int dtype, cudaStream_t st) {
    switch (h_dtype) {
        case MLSTM_DT_F32: return bwd_prep_dispatch<float>(h, dh, b, m, gA, gB, gBw, g, dh16, BH, S, Spad, D, dtype, st);
        case MLSTM_DT_F16: return bwd_prep_dispatch<__half>(h, dh, b, m, gA, gB, gBw, g, dh16, BH, S, Spad, D, dtype, st);
        case MLSTM_DT_BF16:
            return bwd_prep_dispatch<__nv_bfloat16>(h, dh, b, m, gA, gB, gBw, g, dh16, BH, S, Spad, D, dtype, st);
    }
    return MLSTM_E_ARG;
}

int launch_df(const void* f, const float* dI, const float* R, void* df, void* di, int BH, int S, int Spad, int dtype,
              cudaStream_t st, int nparts, long long part_stride, double* scratch) {
    // long slices, when the caller has scratch for the segment totals (gates_scratch_bytes covers it): one block per segment
    const int nseg = scratch ? (S + GATE_SEG_TOKENS - 1) / GATE_SEG_TOKENS : 1;
    const int seg_tokens = nseg > 1 ? GATE_SEG_TOKENS : S;
    if (nseg > 1)
        launch_plain(df_total_kernel, dim3(BH * nseg), dim3(SCAN_THREADS), 0, st, dI, R, scratch, S, Spad, nparts, part_stride, nseg, seg_tokens);
    const int blocks = BH * nseg;
    switch (dtype) {
        case MLSTM_DT_F32:
            launch_plain(df_kernel<float>, dim3(blocks), dim3(SCAN_THREADS), 0, st, (const float*)f, dI, R, (float*)df, (float*)di, S, Spad,
                       nparts, part_stride, (const double*)scratch, nseg, seg_tokens);
            break;
        case MLSTM_DT_F16:
            launch_plain(df_kernel<__half>, dim3(blocks), dim3(SCAN_THREADS), 0, st, (const __half*)f, dI, R, (__half*)df, (__half*)di, S,
                       Spad, nparts, part_stride, (const double*)scratch, nseg, seg_tokens);
            break;
        case MLSTM_DT_BF16:
            launch_plain(df_kernel<__nv_bfloat16>, dim3(blocks), dim3(SCAN_THREADS), 0, st, (const __nv_bfloat16*)f, dI, R,
                       (__nv_bfloat16*)df, (__nv_bfloat16*)di, S, Spad, nparts, part_stride, (const double*)scratch, nseg, seg_tokens);
            break;
        default: return MLSTM_E_ARG;
    }
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

}  // namespace mlstm
