// Test program in the shape of the reference driver's main (cuda-src/mlstm_forward.cu:192-263):
// fill Q, K, V, F, I with the reference recipe (srand(100), uniform [-1, 1) halves), run the host
// oracle, launch through include/mlstm_forward.cuh with the reference's template arguments, copy H
// back and count elements further than 0.01 from the oracle (the reference's check,
// cuda-src/cpu_utils.cuh:30-40).  Exit code 0 only when nothing mismatches.  Links the CPU oracle
// (oracle/libmlstm_oracle.so) as the checker: test infrastructure, not shipped.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../include/mlstm_forward.cuh"

extern "C" int mlstm_cpu_forward(const float* Q, const float* K, const float* V, const float* F, const float* I,
                                 float* H, unsigned S, unsigned D, int eps_inside_max);

static void fill(std::vector<half>& a) {
    for (auto& x : a) x = __float2half(-1.0f + 2.0f * (static_cast<float>(rand()) / static_cast<float>(RAND_MAX)));
}
static std::vector<float> widen(const std::vector<half>& a) {
    std::vector<float> o(a.size());
    for (size_t k = 0; k < a.size(); k++) o[k] = __half2float(a[k]);
    return o;
}

int main(int argc, char** argv) {
    constexpr unsigned BS_DIM = 64, WS_DIM = 16, MMA_M_DIM = 16, MMA_N_DIM = 8, MMA_K_DIM = 8, D = 128;
    const unsigned S = argc > 1 ? static_cast<unsigned>(atoi(argv[1])) : 64 * 10;
    std::vector<half> Q(S * D), K(S * D), V(S * D), F(S), I(S), H(S * D);
    srand(100);
    fill(Q); fill(K); fill(V); fill(F); fill(I);

    std::vector<float> Href(S * D);
    if (mlstm_cpu_forward(widen(Q).data(), widen(K).data(), widen(V).data(), widen(F).data(), widen(I).data(),
                          Href.data(), S, D, 1) != 0) return 2;

    half *dQ, *dK, *dV, *dF, *dI, *dH;
    const size_t mat = sizeof(half) * S * D, vec = sizeof(half) * S;
    if (cudaMalloc(&dQ, mat) || cudaMalloc(&dK, mat) || cudaMalloc(&dV, mat) || cudaMalloc(&dF, vec) ||
        cudaMalloc(&dI, vec) || cudaMalloc(&dH, mat)) return 3;
    cudaMemcpy(dQ, Q.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(dK, K.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(dV, V.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(dF, F.data(), vec, cudaMemcpyHostToDevice);
    cudaMemcpy(dI, I.data(), vec, cudaMemcpyHostToDevice);

    const int rc = mlstm_forward<BS_DIM, WS_DIM, D, MMA_M_DIM, MMA_N_DIM, MMA_K_DIM>(dQ, dK, dV, dF, dI, dH, S);
    if (rc != MLSTM_OK) { printf("launch failed: %s\n", mlstm_status_string(rc)); return 4; }
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed: %s\n", cudaGetErrorString(cudaGetLastError())); return 5; }
    int code = -1;   // a kernel that gave up on an internal wait leaves its code in the scratch buffer's status word
    if (mlstm_driver_scratch_status(&code) != MLSTM_OK) { printf("kernel status %d\n", code); return 6; }
    // a longer and then a shorter call on the same thread: the header's scratch grows once and is reused
    if (mlstm_forward<BS_DIM, WS_DIM, D, MMA_M_DIM, MMA_N_DIM, MMA_K_DIM>(dQ, dK, dV, dF, dI, dH, S) != MLSTM_OK) return 7;
    if (cudaDeviceSynchronize() != cudaSuccess) return 8;
    cudaMemcpy(H.data(), dH, mat, cudaMemcpyDeviceToHost);

    unsigned count = 0;
    float worst = 0.0f;
    for (unsigned k = 0; k < S * D; k++) {
        const float d = std::fabs(__half2float(H[k]) - __half2float(__float2half(Href[k])));
        worst = std::fmax(worst, d);
        if (d > 0.01f) count++;
    }
    printf("Check H\nNon_matching count: %u\nNon_matching percent: %f\nworst abs diff: %g\n", count,
           100.0f * count / static_cast<float>(S * D), worst);
    cudaFree(dQ); cudaFree(dK); cudaFree(dV); cudaFree(dF); cudaFree(dI); cudaFree(dH);
    return count == 0 ? 0 : 1;
}
