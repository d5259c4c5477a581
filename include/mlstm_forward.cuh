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
// thread AND device for it: allocated with cudaMalloc on first use on that device, replaced by a larger
// one when a longer sequence comes (the smaller buffer is released with cudaFreeAsync on the stream that
// last used it, i.e. after the work queued there), never touched otherwise.  The current device must be
// the one that owns `stream`.  mlstm_driver_scratch_status() reads the status word of the calling
// thread's buffer on the current device (0 = no kernel gave up on a wait).  Callers that manage memory
// themselves call mlstm_forward_f16() from mlstm_b200.h with their own workspace, and callers that must
// not allocate at all mlstm_forward_f16_static().
// Link with libmlstm_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "mlstm_b200.h"

namespace mlstm_driver_detail {
constexpr int MAX_DEVICES = 64;
struct Scratch {
    void* buf = nullptr;
    size_t cap = 0;
    cudaStream_t last_stream = 0;
};
inline Scratch* slots() {
    thread_local Scratch per_device[MAX_DEVICES];
    return per_device;
}
inline void* scratch(size_t bytes, cudaStream_t stream) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    Scratch& s = slots()[dev];
    if (bytes > s.cap) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
        if (s.buf) cudaFreeAsync(s.buf, s.last_stream);   // ordered after the work that last used it
        s.buf = p;
        s.cap = bytes;
    }
    s.last_stream = stream;
    return s.buf;
}
}  // namespace mlstm_driver_detail

// Status word of this thread's scratch buffer on the current device (synchronises `stream`).
inline int mlstm_driver_scratch_status(int* host_status, cudaStream_t stream = 0) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= mlstm_driver_detail::MAX_DEVICES) return MLSTM_E_CUDA;
    void* buf = mlstm_driver_detail::slots()[dev].buf;
    if (!buf) {
        *host_status = 0;
        return MLSTM_OK;
    }
    return mlstm_read_status(buf, host_status, stream);
}

template <unsigned BS_DIM, unsigned WS_DIM, unsigned D_DIM, unsigned MMA_M_DIM, unsigned MMA_N_DIM, unsigned MMA_K_DIM>
inline int mlstm_forward(const half* Q, const half* K, const half* V, const half* F, const half* I, half* H,
                         const unsigned S_DIM, cudaStream_t stream = 0) {
    static_assert(BS_DIM > 0 && WS_DIM > 0 && MMA_M_DIM > 0 && MMA_N_DIM > 0 && MMA_K_DIM > 0,
                  "tile parameters must be positive");
    static_assert(D_DIM % 8 == 0, "head dimension must be a multiple of 8");
    const size_t bytes = mlstm_forward_f16_workspace(S_DIM, D_DIM);
    if (bytes == 0) return MLSTM_E_SHAPE;
    void* ws = mlstm_driver_detail::scratch(bytes, stream);
    if (!ws) return MLSTM_E_CUDA;
    return mlstm_forward_f16(Q, K, V, F, I, H, S_DIM, D_DIM, ws, bytes, stream);
}
