// Test program in the shape of the reference backward driver's main (cuda-src/mlstm_backward.cu:543-660):
// fill dH, Q, K, V, F, I with the reference recipe (srand(1678), uniform [-1, 1) halves), launch through
// include/mlstm_backward.cuh with the reference's template arguments, copy the gradients back and print
// sums that the calling test compares with the CPU oracle's (which the test computes from the same
// recipe re-generated through this program's dump).  Exit code 0 when the launch succeeded and every value
// is finite.  Usage: driver_backward S out.bin  (out.bin: dH Q K V [S*D] F I [S] dQ dK dV [S*D] dF dI [S], halves)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../include/mlstm_backward.cuh"

static void fill(std::vector<half>& a) {
    for (auto& x : a) x = __float2half(-1.0f + 2.0f * (static_cast<float>(rand()) / static_cast<float>(RAND_MAX)));
}

int main(int argc, char** argv) {
    constexpr unsigned BS_DIM = 64, WS_DIM = 16, MMA_M_DIM = 16, MMA_N_DIM = 8, MMA_K_DIM = 8, D = 128;
    const unsigned S = argc > 1 ? static_cast<unsigned>(atoi(argv[1])) : 64 * 20;
    const char* out_path = argc > 2 ? argv[2] : nullptr;
    std::vector<half> dH(S * D), Q(S * D), K(S * D), V(S * D), F(S), I(S);
    srand(1678);
    fill(dH); fill(Q); fill(K); fill(V); fill(F); fill(I);

    const size_t mat = sizeof(half) * S * D, vec = sizeof(half) * S;
    half *d_dH, *d_Q, *d_K, *d_V, *d_F, *d_I, *d_dQ, *d_dK, *d_dV, *d_dF, *d_dI;
    if (cudaMalloc(&d_dH, mat) || cudaMalloc(&d_Q, mat) || cudaMalloc(&d_K, mat) || cudaMalloc(&d_V, mat) ||
        cudaMalloc(&d_F, vec) || cudaMalloc(&d_I, vec) || cudaMalloc(&d_dQ, mat) || cudaMalloc(&d_dK, mat) ||
        cudaMalloc(&d_dV, mat) || cudaMalloc(&d_dF, vec) || cudaMalloc(&d_dI, vec))
        return 3;
    cudaMemcpy(d_dH, dH.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(d_Q, Q.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(d_K, K.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(d_V, V.data(), mat, cudaMemcpyHostToDevice);
    cudaMemcpy(d_F, F.data(), vec, cudaMemcpyHostToDevice);
    cudaMemcpy(d_I, I.data(), vec, cudaMemcpyHostToDevice);

    const int rc = mlstm_backward<BS_DIM, WS_DIM, D, MMA_M_DIM, MMA_N_DIM, MMA_K_DIM>(d_dH, d_Q, d_K, d_V, d_F, d_I, d_dQ,
                                                                                       d_dK, d_dV, d_dF, d_dI, S);
    if (rc != MLSTM_OK) { printf("launch failed: %s\n", mlstm_status_string(rc)); return 4; }
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed: %s\n", cudaGetErrorString(cudaGetLastError())); return 5; }
    std::vector<half> dQ(S * D), dK(S * D), dV(S * D), dF(S), dI(S);
    cudaMemcpy(dQ.data(), d_dQ, mat, cudaMemcpyDeviceToHost);
    cudaMemcpy(dK.data(), d_dK, mat, cudaMemcpyDeviceToHost);
    cudaMemcpy(dV.data(), d_dV, mat, cudaMemcpyDeviceToHost);
    cudaMemcpy(dF.data(), d_dF, vec, cudaMemcpyDeviceToHost);
    cudaMemcpy(dI.data(), d_dI, vec, cudaMemcpyDeviceToHost);

    unsigned bad = 0;
    auto scan = [&](const std::vector<half>& a, const char* name) {
        double sum = 0.0;
        for (half x : a) {
            const float f = __half2float(x);
            if (!std::isfinite(f)) bad++;
            sum += f;
        }
        printf("sum %s: %.6f\n", name, sum);
    };
    scan(dQ, "dQ"); scan(dK, "dK"); scan(dV, "dV"); scan(dF, "dF"); scan(dI, "dI");
    printf("Non_finite count: %u\n", bad);
    if (out_path) {
        FILE* fh = fopen(out_path, "wb");
        if (!fh) return 6;
        for (const std::vector<half>* a : {&dH, &Q, &K, &V, &F, &I, &dQ, &dK, &dV, &dF, &dI}) fwrite(a->data(), sizeof(half), a->size(), fh);
        fclose(fh);
    }
    return bad == 0 ? 0 : 1;
}
