// C++ driver interface of the B200 mLSTM forward, source-compatible with the reference driver's
// call site (cuda-src/mlstm_forward.cu:12-15, 235-238):
//
//     mlstm_forward<BS_DIM, WS_DIM, D_DIM, MMA_M, MMA_N, MMA_K><<<S / BS_DIM, 128, smem>>>(Q, K, V, F, I, H, S);
// becomes
//     mlstm_forward<BS_DIM, WS_DIM, D_DIM, MMA_M, MMA_N, MMA_K>(Q, K, V, F, I, H, S);       // same arguments
//
// Q, K, V, H: [S, D_DIM] half, F, I: [S] half, device pointers owned by the caller, default stream
// unless one is given.  The template parameters of the reference kernel are kept so that a call
// site compiles unchanged; only D_DIM selects anything (the head dimension).  The tile parameters
// described the reference's mma.sync tiling; they are checked for plausibility and otherwise unused,
// the tcgen05 kernel picks its own tiles.  Returns an MLSTM_* status (the reference's launch returned
// nothing and reported errors through CUDA_CHECK, cuda-src/cpu_utils.cuh:10-27).
//
// The kernels need a little scratch memory.  This header keeps one grow-only device buffer per host
// thread for it (allocated with cudaMalloc on first use or growth, never freed before exit); callers
// that manage memory themselves call mlstm_forward_f16() from mlstm_b200.h with their own workspace.
// Link with libmlstm_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "mlstm_b200.h"

namespace mlstm_driver_detail {
inline void* scratch(size_t bytes) {
    thread_local void* buf = nullptr;
    thread_local size_t cap = 0;
    thread_local int dev_of_buf = -1;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (bytes > cap || dev != dev_of_buf) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
        buf = p;  // the previous buffer may still be in use by queued work: it is left to process exit
        cap = bytes;
        dev_of_buf = dev;
    }
    return buf;
}
}  // namespace mlstm_driver_detail

template <unsigned BS_DIM, unsigned WS_DIM, unsigned D_DIM, unsigned MMA_M_DIM, unsigned MMA_N_DIM, unsigned MMA_K_DIM>
inline int mlstm_forward(const half* Q, const half* K, const half* V, const half* F, const half* I, half* H,
                         const unsigned S_DIM, cudaStream_t stream = 0) {
    static_assert(BS_DIM > 0 && WS_DIM > 0 && MMA_M_DIM > 0 && MMA_N_DIM > 0 && MMA_K_DIM > 0,
                  "tile parameters must be positive");
    static_assert(D_DIM % 8 == 0, "head dimension must be a multiple of 8");
    const size_t bytes = mlstm_forward_f16_workspace(S_DIM, D_DIM);
    if (bytes == 0) return MLSTM_E_SHAPE;
    void* ws = mlstm_driver_detail::scratch(bytes);
    if (!ws) return MLSTM_E_CUDA;
    return mlstm_forward_f16(Q, K, V, F, I, H, S_DIM, D_DIM, ws, bytes, stream);
}
