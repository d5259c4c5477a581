// Host-side helpers shared by the tensor-core translation units (mm_tc.cu defines them).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "mlstm_common.cuh"

namespace mlstm {

// Tensor map of a [N2, N1, N0] tensor (N0 contiguous): boxes of 128 bytes x box_rows rows, 128-byte
// swizzle (with 32-byte atoms if atom32), zero fill outside the tensor.
int tc_make_map(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, bool atom32, int box_rows);
// Same tensor for TMA stores of output tiles: boxes of 64 bytes x box_rows rows with the 64-byte swizzle
// (in shared memory the 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3) of that row; the buffer
// is 512-byte aligned).
int tc_make_map_out(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, int box_rows);
// Several 128-byte column groups per box (4-D view of the same tensor), see mm_tc.cu
int tc_make_map_groups(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, bool atom32, int box_rows,
                       int box_groups);
int tc_sm_count();    // SMs of the current device (cached), -1 on error
int tc_slice_set();   // slices interleaved in the work-item order

// CTA-pair form of the tensor-core pass (mm_tc_pair.cu): head dimension 256, 16-bit inputs
bool tc_pair_supported(int S, int D, int in_dtype);
int launch_pass_tc_pair(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st);

}  // namespace mlstm
