// A C++ host that shards one PCMM over the GPUs of one process through the C ABI alone (include/ckks_b200.h): the
// columns of the product are split between the GPUs, every output row has one owner
// (ckks_b200_pcmm_set_row_owners), and each GPU's multiply stores the words it computes into the owner's buffer, its
// own or a peer's.  Afterwards every GPU must hold ALL columns of ITS rows, equal word for word to the same rows of the
// whole product computed on GPU 0.  With one GPU the same calls run with a world of one.
//   usage: shard_driver <world> [M K N1 rank]        exit code 0: every rank's rows match
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "ckks_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e__ = (x); if (e__ != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e__)); return 3; } } while (0)
#define CHECK_LIB(x) do { int s__ = (x); if (s__ != CKKS_B200_OK) { printf("%s: %s\n", #x, ckks_b200_last_error()); return 4; } } while (0)

int main(int argc, char** argv) {
    const int world = argc > 1 ? atoi(argv[1]) : 1;
    const int M = argc > 2 ? atoi(argv[2]) : 96, K = argc > 3 ? atoi(argv[3]) : 64;
    const int N1 = argc > 4 ? atoi(argv[4]) : 64, rank = argc > 5 ? atoi(argv[5]) : 7;
    int devices = 0;
    CHECK_CUDA(cudaGetDeviceCount(&devices));
    if (world < 1 || world > 8 || world > devices) { printf("world %d, devices %d\n", world, devices); return 2; }
    // the head of the reference's logN = 16 chain (src/ckks/include/Params.cuh:118-150); any odd moduli would do
    const uint64_t q[3] = {0x20000018e0001ull, 0x2000001c00001ull, 0x2000001ca0001ull};
    const int limbs = 3;
    const long C = (long)(rank + 1) * N1;
    const size_t ct_words = (size_t)limbs * C, out_words = (size_t)M * limbs * C;
    const double scaler = 1073741824.0;

    std::mt19937_64 gen(17);
    std::vector<uint64_t> X((size_t)K * ct_words);
    for (int n = 0; n < K; n++)
        for (int i = 0; i < limbs; i++)
            for (long c = 0; c < C; c++) X[((size_t)n * limbs + i) * C + c] = gen() % q[i];
    std::vector<float> W((size_t)M * K);
    std::uniform_real_distribution<float> uni(-1.f, 1.f);
    for (float& w : W) w = uni(gen);

    std::vector<ckks_b200_pcmm*> pc(world, nullptr);
    std::vector<uint64_t*> dX(world), dOut(world);
    std::vector<float*> dW(world);
    std::vector<cudaStream_t> st(world);
    std::vector<std::vector<const uint64_t*>> ptrs(world);
    for (int g = 0; g < world; g++) {
        CHECK_CUDA(cudaSetDevice(g));
        for (int p = 0; p < world; p++) {
            if (p == g) continue;
            int ok = 0;
            CHECK_CUDA(cudaDeviceCanAccessPeer(&ok, g, p));
            if (!ok) { printf("GPU %d cannot address GPU %d\n", g, p); return 2; }
            cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { printf("peer access %d -> %d: %s\n", g, p, cudaGetErrorString(e)); return 3; }
            cudaGetLastError();
        }
        CHECK_CUDA(cudaStreamCreateWithFlags(&st[g], cudaStreamNonBlocking));
        CHECK_LIB(ckks_b200_pcmm_create(&pc[g], g, N1, rank, q, limbs));
        CHECK_CUDA(cudaMalloc(&dX[g], X.size() * 8));
        CHECK_CUDA(cudaMalloc(&dOut[g], out_words * 8));
        CHECK_CUDA(cudaMalloc(&dW[g], W.size() * 4));
        CHECK_CUDA(cudaMemcpy(dX[g], X.data(), X.size() * 8, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dW[g], W.data(), W.size() * 4, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemset(dOut[g], 0xff, out_words * 8));
        for (int n = 0; n < K; n++) ptrs[g].push_back(dX[g] + (size_t)n * ct_words);
    }

    // the whole product on GPU 0
    CHECK_CUDA(cudaSetDevice(0));
    uint64_t* dRef = nullptr;
    CHECK_CUDA(cudaMalloc(&dRef, out_words * 8));
    CHECK_LIB(ckks_b200_pcmm_ppmm(pc[0], dW[0], ptrs[0].data(), dRef, M, K, N1, K, scaler, 0, C, CKKS_B200_PCMM_TENSOR, st[0]));
    CHECK_LIB(ckks_b200_pcmm_check(pc[0], st[0]));
    std::vector<uint64_t> ref(out_words);
    CHECK_CUDA(cudaMemcpy(ref.data(), dRef, out_words * 8, cudaMemcpyDeviceToHost));

    // the sharded product: weights prepared once per GPU, then every GPU's launch is only enqueued
    const long tiles = (C + 31) / 32;
    for (int g = 0; g < world; g++) {
        CHECK_CUDA(cudaSetDevice(g));
        CHECK_LIB(ckks_b200_pcmm_set_row_owners(pc[g], dOut.data(), world, g));
        CHECK_LIB(ckks_b200_pcmm_prepare_weights(pc[g], dW[g], M, K, scaler, st[g]));
    }
    for (int g = 0; g < world; g++) {
        CHECK_CUDA(cudaSetDevice(g));
        const long c0 = tiles * g / world * 32, c1 = g + 1 == world ? C : tiles * (g + 1) / world * 32;
        CHECK_LIB(ckks_b200_pcmm_ppmm(pc[g], nullptr, ptrs[g].data(), dOut[g], M, K, N1, K, scaler, c0, c1, CKKS_B200_PCMM_TENSOR, st[g]));
    }
    for (int g = 0; g < world; g++) {
        CHECK_CUDA(cudaSetDevice(g));
        CHECK_LIB(ckks_b200_pcmm_check(pc[g], st[g]));          // waits for the stream: this GPU's stores have landed everywhere
    }

    int bad = 0;
    std::vector<uint64_t> got(out_words);
    for (int g = 0; g < world; g++) {
        int r0 = 0, r1 = 0;
        CHECK_LIB(ckks_b200_pcmm_row_owner_range(M, world, g, &r0, &r1));
        CHECK_CUDA(cudaSetDevice(g));
        CHECK_CUDA(cudaMemcpy(got.data(), dOut[g], out_words * 8, cudaMemcpyDeviceToHost));
        size_t wrong = 0, foreign = 0;
        for (int m = 0; m < M; m++)
            for (size_t x = 0; x < ct_words; x++) {
                const uint64_t v = got[(size_t)m * ct_words + x];
                if (m >= r0 && m < r1) wrong += v != ref[(size_t)m * ct_words + x];
                else foreign += v != ~0ull;                       // rows of other owners stay untouched here
            }
        printf("rank %d owns rows [%d, %d): %zu wrong words, %zu words written into rows it does not own\n", g, r0, r1, wrong, foreign);
        bad += wrong != 0 || foreign != 0;
    }
    for (int g = 0; g < world; g++) {
        cudaSetDevice(g);
        ckks_b200_pcmm_destroy(pc[g]);
        cudaFree(dX[g]); cudaFree(dOut[g]); cudaFree(dW[g]);
    }
    cudaFree(dRef);
    printf(bad ? "MISMATCH\n" : "all ranks hold their rows\n");
    return bad ? 1 : 0;
}
