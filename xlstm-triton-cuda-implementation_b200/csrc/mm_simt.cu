// CUDA-core (fp32 FMA) contraction pass of the parallel mLSTM: the same four passes as the
// tensor-core kernel (mlstm_common.cuh), for fp32 inputs, head dimensions the tcgen05 path does
// not take, and as an on-device cross-check.  fp32 dot products match the reference's
// tl.dot(..., allow_tf32=False) arithmetic (mlstm_matmul.py:15-19).
//
// One block = 64 stationary rows x 64 output columns (blockIdx.z picks the column chunk of the
// head dimension); it streams 64-row tiles on the causal side, forms T over the whole head
// dimension in chunks of 32, gates it, and accumulates W Z for its column chunk.
#include "mlstm_common.cuh"

namespace mlstm {
namespace {

constexpr int BT = 64;   // tile rows / streamed rows
constexpr int BK = 32;   // head-dimension chunk of the first contraction
constexpr int BV = 64;   // output columns per block

template <int MODE, typename InT, typename OutT>
__global__ void __launch_bounds__(256) mlstm_simt_pass(const PassParams p) {
    grid_dep_wait();
    grid_dep_launch();
    constexpr bool ROWS_ARE_Q = (MODE == FWD || MODE == DQ);
    // the X/Y chunks of the first contraction and the Z tile of the second are live at different
    // times and share storage
    __shared__ __align__(16) float pool[BT * (BV + 4)];
    __shared__ float Ws[BT][BT + 1];
    float (*Xs)[BK + 1] = reinterpret_cast<float (*)[BK + 1]>(pool);
    float (*Ys)[BK + 1] = reinterpret_cast<float (*)[BK + 1]>(pool + BT * (BK + 1));
    float (*Zs)[BV + 4] = reinterpret_cast<float (*)[BV + 4]>(pool);
    static_assert(2 * BT * (BK + 1) <= BT * (BV + 4), "X/Y chunks must fit in the Z tile's storage");

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int S = p.S, D = p.D;
    const int NT = (S + BT - 1) / BT;
    const int bh = blockIdx.y;
    const int w = blockIdx.x;
    const int tile = ROWS_ARE_Q ? (NT - 1 - w) : w;
    const int t_begin = ROWS_ARE_Q ? 0 : tile;
    const int t_end = ROWS_ARE_Q ? tile : (NT - 1);
    const int v0 = blockIdx.z * BV;
    const size_t slice = static_cast<size_t>(bh) * S * D;
    const size_t vec = static_cast<size_t>(bh) * p.Spad;
    const InT* X = reinterpret_cast<const InT*>(p.X) + slice;
    const InT* Y = reinterpret_cast<const InT*>(p.Y) + slice;
    const InT* Z = reinterpret_cast<const InT*>(p.Z) + slice;

    static_assert(BT == REF_BLOCK, "one streamed tile = one reference block of the gate vectors");
    const size_t ref = static_cast<size_t>(bh) * (p.Spad / REF_BLOCK);
    double er_d[4];
    float gr_[4];
    int rows[4];
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
        rows[rr] = tile * BT + ty * 4 + rr;
        er_d[rr] = static_cast<double>(p.row_rel[vec + rows[rr]]) + p.row_ref[ref + tile] + static_cast<double>(p.er_add);
        gr_[rr] = (MODE == DQ) ? p.row_g[vec + rows[rr]] : 0.0f;
    }
    float acc[4][4] = {};
    float rowsum[4] = {};

    for (int st = t_begin; st <= t_end; st++) {
        float tacc[4][4] = {};
        for (int d0 = 0; d0 < D; d0 += BK) {
#pragma unroll
            for (int k = 0; k < (BT * BK) / 256; k++) {
                const int idx = tid + k * 256, r = idx / BK, c = idx % BK;
                const int xr = tile * BT + r, yr = st * BT + r, d = d0 + c;
                Xs[r][c] = (xr < S && d < D) ? to_f32<InT>(X[static_cast<size_t>(xr) * D + d]) : 0.0f;
                Ys[r][c] = (yr < S && d < D) ? to_f32<InT>(Y[static_cast<size_t>(yr) * D + d]) : 0.0f;
            }
            __syncthreads();
#pragma unroll
            for (int d = 0; d < BK; d++) {
                float xv[4], yv[4];
#pragma unroll
                for (int rr = 0; rr < 4; rr++) xv[rr] = Xs[ty * 4 + rr][d];
#pragma unroll
                for (int cc = 0; cc < 4; cc++) yv[cc] = Ys[tx * 4 + cc][d];
#pragma unroll
                for (int rr = 0; rr < 4; rr++)
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) tacc[rr][cc] = fmaf(xv[rr], yv[cc], tacc[rr][cc]);
            }
            __syncthreads();
        }
        // gate the tile
        float er[4];
#pragma unroll
        for (int rr = 0; rr < 4; rr++) er[rr] = static_cast<float>(er_d[rr] + p.col_ref[ref + st]);
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int col = st * BT + tx * 4 + cc;
            const float ec = p.col_rel[vec + col];
            const float gc = (MODE == DK) ? p.col_g[vec + col] : 0.0f;
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
                float wv = (tacc[rr][cc] + gc + gr_[rr]) * exp2f(ec + er[rr]);
                if (!causal_ok<MODE>(rows[rr], col) || col >= S) wv = 0.0f;
                Ws[ty * 4 + rr][tx * 4 + cc] = wv;
                rowsum[rr] += wv;
            }
        }
        // streamed Z tile, this block's column chunk
#pragma unroll
        for (int k = 0; k < (BT * BV) / 256; k++) {
            const int idx = tid + k * 256, r = idx / BV, c = idx % BV;
            const int zr = st * BT + r, d = v0 + c;
            Zs[r][c] = (zr < S && d < D) ? to_f32<InT>(Z[static_cast<size_t>(zr) * D + d]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BT; kk++) {
            const float4 z4 = *reinterpret_cast<const float4*>(&Zs[kk][tx * 4]);
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
                const float wv = Ws[ty * 4 + rr][kk];
                acc[rr][0] = fmaf(wv, z4.x, acc[rr][0]);
                acc[rr][1] = fmaf(wv, z4.y, acc[rr][1]);
                acc[rr][2] = fmaf(wv, z4.z, acc[rr][2]);
                acc[rr][3] = fmaf(wv, z4.w, acc[rr][3]);
            }
        }
        __syncthreads();
    }

    // epilogue
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
        float bsum = rowsum[rr];
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) bsum += __shfl_xor_sync(0xffffffffu, bsum, o);
        const int row = rows[rr];
        const bool row_ok = row < S;
        float inv_n = 1.0f;
        if (MODE == FWD) {
            const float mrow = row_ok ? p.m[static_cast<size_t>(bh) * S + row] : 0.0f;
            inv_n = 1.0f / (fmaxf(fabsf(bsum), expf(-mrow)) + 1e-6f);
            if (row_ok && tx == 0 && blockIdx.z == 0 && p.b_out) p.b_out[static_cast<size_t>(bh) * S + row] = bsum;
        }
        float dot = 0.0f;
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int d = v0 + tx * 4 + cc;
            if (row_ok && d < D) {
                const size_t off = slice + static_cast<size_t>(row) * D + d;
                float val = acc[rr][cc] * inv_n;
                if ((MODE == DQ || MODE == DK) && p.dot_src)
                    dot += val * to_f32<InT>(reinterpret_cast<const InT*>(p.dot_src)[off]);
                if (MODE == FWD && p.ogate) val *= silu_f(to_f32<InT>(reinterpret_cast<const InT*>(p.ogate)[off]));
                reinterpret_cast<OutT*>(p.out)[off] = from_f32<OutT>(val);
            }
        }
        if ((MODE == DQ || MODE == DK) && p.dot_out) {
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (tx == 0 && row_ok) atomicAdd(&p.dot_out[vec + row], dot);
        }
    }
}

template <int MODE, typename InT, typename OutT>
int launch_one(const PassParams& p, cudaStream_t st) {
    const int NT = (p.S + BT - 1) / BT;
    dim3 grid(NT, p.BH, (p.D + BV - 1) / BV);
    if (p.BH > 65535 || grid.z > 65535) return MLSTM_E_SHAPE;
    mlstm_simt_pass<MODE, InT, OutT><<<grid, 256, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}

template <int MODE, typename InT>
int launch_out(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (out_dtype == MLSTM_DT_F32) return launch_one<MODE, InT, float>(p, st);
    if (out_dtype == in_dtype) return launch_one<MODE, InT, InT>(p, st);
    return MLSTM_E_ARG;
}

template <int MODE>
int launch_in(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    switch (in_dtype) {
        case MLSTM_DT_F32: return launch_out<MODE, float>(p, in_dtype, out_dtype, st);
        case MLSTM_DT_F16: return launch_out<MODE, __half>(p, in_dtype, out_dtype, st);
        case MLSTM_DT_BF16: return launch_out<MODE, __nv_bfloat16>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_ARG;
}

}  // namespace

int launch_pass_simt(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if ((mode == DQ || mode == DK) && p.dot_out) {
        // row dots are accumulated with atomics over the column chunks
        if (cudaMemsetAsync(p.dot_out, 0, static_cast<size_t>(p.BH) * p.Spad * sizeof(float), st) != cudaSuccess)
            return MLSTM_E_CUDA;
    }
    switch (mode) {
        case FWD: return launch_in<FWD>(p, in_dtype, out_dtype, st);
        case DQ: return launch_in<DQ>(p, in_dtype, out_dtype, st);
        case DK: return launch_in<DK>(p, in_dtype, out_dtype, st);
        case DV: return launch_in<DV>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_ARG;
}

}  // namespace mlstm
