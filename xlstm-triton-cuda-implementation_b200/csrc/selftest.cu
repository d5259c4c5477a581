// Self-test of the bounded-wait protocol that every kernel of this library relies on.
//
// All device-side waits (mbarrier phases that a TMA copy, an MMA commit or another warp completes) go
// through ptx::mbar_wait, which gives up after a cycle limit, raises the CTA's abort word and makes the
// kernel store a code in the workspace's status word instead of hanging.  The contraction kernels
// cannot be made to take that path on purpose without breaking them, so this file exercises the same
// wait primitive in isolation: one warp waits on a barrier that nothing ever arrives on, with a limit
// chosen by the caller (a millisecond is plenty), and reports through the same status word.  Nothing
// here traps, faults or spins without a bound; the context stays usable.
#include "mlstm_common.cuh"
#include "ptx_sm100.cuh"

namespace mlstm {
namespace {

constexpr int SELFTEST_CODE = 4000;

__global__ void wait_timeout_kernel(int* status, long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_word = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    // phase 0 of the barrier never completes: there is no arrival anywhere in this kernel
    const bool ok = ptx::mbar_wait_warp<64>(&bar, 0, &abort_word, limit_cycles);
    __syncthreads();
    if (!ok && threadIdx.x == 0) atomicExch(status, SELFTEST_CODE);
}

}  // namespace
}  // namespace mlstm

extern "C" int mlstm_selftest_wait_timeout(void* workspace, size_t workspace_bytes, long long limit_cycles, void* stream) {
    using namespace mlstm;
    if (!workspace || workspace_bytes < 256) return MLSTM_E_WORKSPACE;
    if (limit_cycles <= 0 || limit_cycles > 2000000000LL) return MLSTM_E_ARG;   // at most about a second
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* status = static_cast<int*>(workspace);
    if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return MLSTM_E_CUDA;
    wait_timeout_kernel<<<1, 32, 0, st>>>(status, limit_cycles);
    return cudaGetLastError() == cudaSuccess ? MLSTM_OK : MLSTM_E_CUDA;
}
