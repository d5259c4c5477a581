// C++ driver interface of the B200 mLSTM backward, in the shape of the reference driver's launches
// (cuda-src/mlstm_backward.cu:11-12, 177-178, 621-628):
//
//     matmul_backward_db<BS, WS, D, M, N, K><<<S / BS, 128, smem>>>(dH, Q, K, V, F, I, M, B, dB, S);
//     matmul_backward<BS, WS, D, M, N, K><<<S / BS, 128, smem>>>(dH, dB, Q, K, V, dQ, dK, dV, F, I, dI, M, B, S);
// become
//     mlstm_backward<BS, WS, D, M, N, K>(dH, Q, K, V, F, I, dQ, dK, dV, dF, dI, S);
//
// One call produces all five gradients (the reference's kernels leave dV, dI and dF unfinished and its
// host check covers dB, dQ and dK only).  M, B and dB are internal here: the forward is recomputed
// inside the call, so there is nothing for the host to precompute.  dH, Q, K, V, dQ, dK, dV: [S, D_DIM]
// half; F, I, dF, dI: [S] half; device pointers owned by the caller; default stream unless one is given.
// The tile parameters are kept for source compatibility and checked for plausibility only.  Returns an
// MLSTM_* status.  Scratch memory: one grow-only device buffer per host thread and device, as in mlstm_forward.cuh;
// callers that manage memory themselves use mlstm_backward_f16() from mlstm_b200.h.
// Link with libmlstm_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "mlstm_b200.h"
#include "mlstm_forward.cuh"

template <unsigned BS_DIM, unsigned WS_DIM, unsigned D_DIM, unsigned MMA_M_DIM, unsigned MMA_N_DIM, unsigned MMA_K_DIM>
inline int mlstm_backward(const half* dH, const half* Q, const half* K, const half* V, const half* F, const half* I,
                          half* dQ, half* dK, half* dV, half* dF, half* dI, const unsigned S_DIM, cudaStream_t stream = 0) {
    static_assert(BS_DIM > 0 && WS_DIM > 0 && MMA_M_DIM > 0 && MMA_N_DIM > 0 && MMA_K_DIM > 0,
                  "tile parameters must be positive");
    static_assert(D_DIM % 8 == 0, "head dimension must be a multiple of 8");
    const size_t bytes = mlstm_backward_f16_workspace(S_DIM, D_DIM);
    if (bytes == 0) return MLSTM_E_SHAPE;
    void* ws = mlstm_driver_detail::scratch(bytes, stream);
    if (!ws) return MLSTM_E_CUDA;
    return mlstm_backward_f16(dH, Q, K, V, F, I, dQ, dK, dV, dF, dI, S_DIM, D_DIM, ws, bytes, stream);
}
