// Test infrastructure: builds the reference project's own host-side mLSTM forward
// (mlstmCpu, cuda-src/cpu_utils.cuh:126-170) and its input generator
// (rand_half / fillMatrix, cuda-src/cpu_utils.cuh:43-55) into a shared library, straight from
// the reference checkout.  Nothing of the reference is copied here: the header is included from
// where it lies (-I<reference root>), and the result goes to oracle/_ref/ only.
//
// Exports:
//   ref_fill(seed, Q,K,V,F,I, S, D)  the reference demo's input recipe: srand(seed) then
//                                    fillMatrix on Q,K,V,F,I in this order
//                                    (cuda-src/mlstm_forward.cu:210-215)
//   ref_mlstm_cpu(Q,K,V,F,I,H,S,D)   mlstmCpu
#include <cstdint>
#include <cstdlib>
#include "cuda-src/cpu_utils.cuh"

extern "C" void ref_fill(unsigned seed, half* Q, half* K, half* V, half* F, half* I,
                         unsigned S, unsigned D) {
    srand(seed);
    fillMatrix(Q, S * D);
    fillMatrix(K, S * D);
    fillMatrix(V, S * D);
    fillMatrix(F, S);
    fillMatrix(I, S);
}

extern "C" void ref_mlstm_cpu(half* Q, half* K, half* V, half* F, half* I, half* H,
                              unsigned S, unsigned D) {
    mlstmCpu(Q, K, V, F, I, H, S, D);
}
