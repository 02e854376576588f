// C++ driver written like the reference's test_rlwe_decomp.cu but against
// include/ckks_b200/compat.hpp (the reference's class names over the C ABI).
// Reads a case from a binary file, runs NTT forward / inverse and PPMM, writes the
// results to a second file; tests/test_compat_cpp.py compares them with the oracle.
//   in : u64 header {q0, q1, logN, N1, rank, M, K}, poly [2][N] u64, X [K][2][C] u64, W [M][K] f32
//   out: ntt [2][N], roundtrip [2][N], ppmm_output [M][2][C], ciphertext 5 limb 0 [C], scale ratio (f64)
#include <cstdio>
#include <vector>

#include "ckks_b200/compat.hpp"

using namespace ckks_b200;

int main(int argc, char** argv) {
    if (argc < 3) { printf("usage: compat_driver in.bin out.bin\n"); return 2; }
    FILE* fi = fopen(argv[1], "rb");
    if (!fi) return 3;
    uint64_tt hdr[7];
    if (fread(hdr, 8, 7, fi) != 7) return 3;
    uint64_tt q0 = hdr[0], q1 = hdr[1];
    int logN = (int)hdr[2], N1 = (int)hdr[3], rank = (int)hdr[4], M = (int)hdr[5], Kn = (int)hdr[6];
    long N = 1L << logN, C = (long)(rank + 1) * N1;
    std::vector<uint64_tt> poly(2 * N), X((size_t)Kn * 2 * C);
    std::vector<float> W((size_t)M * Kn);
    if (fread(poly.data(), 8, poly.size(), fi) != poly.size()) return 3;
    if (fread(X.data(), 8, X.size(), fi) != X.size()) return 3;
    if (fread(W.data(), 4, W.size(), fi) != W.size()) return 3;
    fclose(fi);

    Context_23 context(logN, {}, {q0, q1}, {});
    uint64_tt* d;
    cudaMalloc(&d, 16 * N);
    cudaMemcpy(d, poly.data(), 16 * N, cudaMemcpyHostToDevice);
    context.ToNTTInplace(d, 0, 0, 1, 2, 2);
    std::vector<uint64_tt> fwd(2 * N), back(2 * N);
    cudaMemcpy(fwd.data(), d, 16 * N, cudaMemcpyDeviceToHost);
    context.FromNTTInplace(d, 0, 0, 1, 2, 2);
    cudaMemcpy(back.data(), d, 16 * N, cudaMemcpyDeviceToHost);

    PCMM_Context pcmm_context(N1, rank, {}, {q0, q1});
    PCMM_Scheme pcmm_scheme(pcmm_context);
    std::vector<MLWECiphertext*> cts;
    for (int n = 0; n < Kn; n++) {
        cts.push_back(new MLWECiphertext(N1, 1, 1, rank, (long double)(1LL << 49)));
        cudaMemcpy(cts[n]->cipher_device, X.data() + (size_t)n * 2 * C, 16 * C, cudaMemcpyHostToDevice);
    }
    float* dW;
    cudaMalloc(&dW, sizeof(float) * W.size());
    cudaMemcpy(dW, W.data(), sizeof(float) * W.size(), cudaMemcpyHostToDevice);
    pcmm_scheme.PPMM(dW, cts, M, Kn, N1, Kn);
    pcmm_scheme.PPMM(dW, cts, M, Kn, N1 / 2, Kn);      // wrong K: prints the reference's message and returns
    cudaDeviceSynchronize();
    std::vector<uint64_tt> out((size_t)M * 2 * C), ct5(C);
    cudaMemcpy(out.data(), pcmm_scheme.ppmm_output, 8 * out.size(), cudaMemcpyDeviceToHost);
    cudaMemcpy(ct5.data(), cts[5]->cipher_device, 8 * C, cudaMemcpyDeviceToHost);
    double ratio = (double)(cts[0]->scale / (long double)(1LL << 49));

    FILE* fo = fopen(argv[2], "wb");
    if (!fo) return 4;
    fwrite(fwd.data(), 8, fwd.size(), fo);
    fwrite(back.data(), 8, back.size(), fo);
    fwrite(out.data(), 8, out.size(), fo);
    fwrite(ct5.data(), 8, ct5.size(), fo);
    fwrite(&ratio, 8, 1, fo);
    fclose(fo);
    for (auto c : cts) delete c;
    cudaFree(d);
    cudaFree(dW);
    return 0;
}
