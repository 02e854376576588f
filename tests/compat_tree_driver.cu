// A driver written against include/ckks_llm_compat/ the way the reference's own drivers are written against its
// headers: the same include lines, the same object construction and the same calls on the ring-packed matrix-multiply
// path.  The statements marked [ref] are the reference's own lines (test_rlwe_decomp.cu:9-13,24-57,107-127,140,168,173 and
// src/bert/Bert.cuh:398-412,425,471-487), kept as they stand there; what is between them sets up inputs and checks
// results.  Built with  nvcc -I include/ckks_llm_compat ... -lckks_b200  and nothing else from the reference.
//
//   compat_tree_driver decomp <logN> <N1> [dump.bin]   one ciphertext, rank x rank weights (test_rlwe_decomp.cu)
//   compat_tree_driver bert                             N = 2^16, N1 = 128: three ciphertexts of 256 features, 768 x 768 weights
//
// Prints the precision of the decrypted result against the plaintext product; with a dump file writes what the Python
// test needs to redo every step with the CPU oracle.
#include <iostream>
#include <string>
#include <sstream>
#include <vector>
#include <cmath>

using namespace std;

#include "src/ckks/include/Context_23.cuh"                  // [ref] test_rlwe_decomp.cu:9
#include "src/ckks/include/TimeUtils.cuh"                   // [ref] :10
#include "src/ckks/include/pcmm/PCMM_Context.cuh"           // [ref] :11
#include "src/ckks/include/pcmm/PCMM_Scheme.cuh"            // [ref] :12
#include "src/ckks/include/precision.cuh"                   // [ref] :13

static void dump(FILE* f, const void* device, size_t words) {
    vector<uint64_tt> h(words);
    cudaMemcpy(h.data(), device, words * 8, cudaMemcpyDeviceToHost);
    fwrite(h.data(), 8, words, f);
}

static int run_decomp(int logN, int PCMM_N1, const char* dump_path) {
    int logslots = logN - 1;

    Context_23 context(logN, logslots, 192);                // [ref] :24
    Scheme_23 scheme(context);                              // [ref] :25
    cudaDeviceSynchronize();

    int N = context.N;                                      // [ref] :30-33
    int slots = context.slots;
    int L = context.L;
    int K = context.K;

    int mlwe_rank = N / PCMM_N1;                            // [ref] :35
    vector<uint64_tt> p_ringpack = {context.pVec[context.p_num - 1]};          // [ref] :37
    vector<uint64_tt> q_ringpack = {context.qVec[0], context.qVec[1]};         // [ref] :38
    int p_ringpack_count = p_ringpack.size();               // [ref] :39
    int q_ringpack_count = q_ringpack.size();               // [ref] :40

    SecretKey sk(context);                                  // [ref] :42

    SchemeAlgo scheme_algo(context, scheme, sk);            // [ref] :44

    PCMM_Context pcmm_context(PCMM_N1, mlwe_rank, p_ringpack, q_ringpack, context);   // [ref] :49
    PCMM_Scheme pcmm_scheme(pcmm_context, scheme, sk);      // [ref] :50

    int pq_ringpack_count = pcmm_context.pq_ringpack.size();        // [ref] :52

    MLWESecretKey mlwe_sk(PCMM_N1, pq_ringpack_count, mlwe_rank);   // [ref] :54
    pcmm_scheme.convertMLWESKfromRLWESK(mlwe_sk, sk);       // [ref] :55
    scheme.addEncKey(sk);                                   // [ref] :56
    pcmm_scheme.addRepakcingKey(mlwe_sk, sk);               // [ref] :57
    (void)K; (void)p_ringpack_count;

    double* real_mes_host = new double[N];                  // [ref] :59-60
    randomDoubleArray(real_mes_host, N, 1./10);
    double* real_msg1;
    cudaMalloc(&real_msg1, sizeof(double) * N);
    cudaMemcpy(real_msg1, real_mes_host, sizeof(double) * N, cudaMemcpyHostToDevice);

    int target_level = 1;
    int mat_M = mlwe_rank, mat_N = mlwe_rank;               // [ref] :82-87
    float* plain_mat_host = new float[mat_M * mat_N];
    std::uniform_real_distribution<float> randnum(-1./10, 1./10);
    for(int i = 0; i < mat_M * mat_N; i++){
        plain_mat_host[i] = randnum(rng);
    }

    double* plain_gemm_host = new double[N];                // [ref] :89-99
    memset(plain_gemm_host, 0, sizeof(double) * N);
    for(int idx_M = 0; idx_M < mat_M; idx_M++){
        for(int idx_K = 0; idx_K < PCMM_N1; idx_K++){
            for(int idx_N = 0; idx_N < mat_N; idx_N++){
                plain_gemm_host[idx_M + idx_K*mat_M] += plain_mat_host[idx_N + idx_M*mat_N] * real_mes_host[idx_N + idx_K*mat_N];
            }
        }
    }

    float* plain_mat_device;                                // [ref] :101-103
    cudaMalloc(&plain_mat_device, sizeof(float) * mat_M * mat_N);
    cudaMemcpy(plain_mat_device, plain_mat_host, sizeof(float) * mat_M * mat_N, cudaMemcpyHostToDevice);

    int decomp_num = N / PCMM_N1;                           // [ref] :107-114
    vector<MLWECiphertext*> mlwe_cipher_decomposed;
    for(int i = 0; i < decomp_num; i++){
        MLWECiphertext* mlwe_cipher = new MLWECiphertext(PCMM_N1, q_ringpack_count - 1, q_ringpack_count - 1, mlwe_rank, NTL::RR(context.precision));
        mlwe_cipher_decomposed.push_back(mlwe_cipher);
    }

    Plaintext plain_m1_coeffs_encode(N, L, target_level, slots, NTL::RR(context.precision));   // [ref] :116
    Plaintext m2_dec(N, L, target_level, slots, NTL::RR(context.precision));                   // [ref] :118
    Ciphertext c1(N, L, L, slots, NTL::RR(context.precision));                                 // [ref] :120
    Ciphertext c2(N, L, L, slots, NTL::RR(context.precision));                                 // [ref] :121

    double* real_msg_dec;                                   // [ref] :123-124
    cudaMalloc(&real_msg_dec, sizeof(double) * N);

    context.encode_coeffs(real_msg1, plain_m1_coeffs_encode);       // [ref] :130
    scheme.encryptMsg(c1, plain_m1_coeffs_encode);          // [ref] :137

    FILE* f = dump_path ? fopen(dump_path, "wb") : nullptr;
    if (f) {
        uint64_tt hdr[8] = {(uint64_tt)logN, (uint64_tt)PCMM_N1, p_ringpack[0], q_ringpack[0], q_ringpack[1], (uint64_tt)L, (uint64_tt)mat_M, 0};
        fwrite(hdr, 8, 8, f);
        fwrite(plain_mat_host, 4, (size_t)mat_M * mat_N, f);
        dump(f, c1.cipher_device, (size_t)2 * (L + 1) * N);
        dump(f, pcmm_scheme.repacking_keys_device, (size_t)4 * N * mlwe_rank);
    }

    pcmm_scheme.rlweCipherDecompose(c1, mlwe_cipher_decomposed, decomp_num, 0);        // [ref] :140
    if (f) for (int i = 0; i < decomp_num; i++) dump(f, mlwe_cipher_decomposed[i]->cipher_device, (size_t)2 * (mlwe_rank + 1) * PCMM_N1);

    pcmm_scheme.PPMM(plain_mat_device, mlwe_cipher_decomposed, mat_M, mat_N, PCMM_N1, decomp_num);   // [ref] :168
    pcmm_scheme.PPMM(plain_mat_device, mlwe_cipher_decomposed, mat_M, mat_N, PCMM_N1 / 2, decomp_num); // wrong K: the reference's message, no work
    if (f) dump(f, pcmm_scheme.ppmm_output, (size_t)mat_M * 2 * (mlwe_rank + 1) * PCMM_N1);

    pcmm_scheme.mlweCipherPacking(c2, mlwe_cipher_decomposed, decomp_num, 0);          // [ref] :173
    if (f) { dump(f, c2.cipher_device, (size_t)2 * (L + 1) * N); fclose(f); }

    scheme.decryptMsg(m2_dec, sk, c2);                      // [ref] :179-180
    context.decode_coeffs(m2_dec, real_msg_dec);

    vector<double> real_values_computed(N);                 // [ref] :185-196
    cudaMemcpy(real_values_computed.data(), real_msg_dec, sizeof(double) * N, cudaMemcpyDeviceToHost);
    vector<double> real_values_want(N);
    memcpy(real_values_want.data(), plain_gemm_host, sizeof(double) * N);
    auto status_real = GetPrecisionStats(real_values_computed, real_values_want);
    cout<<status_real.String();
    double want_max = 0;
    for (double v : real_values_want) want_max = max(want_max, fabs(v));
    printf("relative error %.3e (2^%.1f), after-ppmm scale ratio %.6f, result level %d\n", status_real.max_err / want_max,
           log2(status_real.max_err / want_max), (double)(mlwe_cipher_decomposed[0]->scale / NTL::RR(context.precision)).v, c2.l);
    for (auto c : mlwe_cipher_decomposed) delete c;
    return status_real.max_err / want_max < ldexp(1.0, -20) ? 0 : 1;
}

// The BERT layer shape the reference runs (src/bert/Bert.cuh:398-487): 768 input features for 128 tokens in three
// ciphertexts of 256 features each (extracted with a gap of two), 768 x 768 weights, three packings of 256 rows.
static int run_bert() {
    const int logN = 16, PCMM_N1 = 128;
    Context_23 context(logN, logN - 1, 192);
    Scheme_23 scheme(context);
    int N = context.N, slots = context.slots, L = context.L;
    int mlwe_rank = N / PCMM_N1;
    vector<uint64_tt> p_ringpack = {context.pVec[context.p_num - 1]};
    vector<uint64_tt> q_ringpack = {context.qVec[0], context.qVec[1]};
    int q_ringpack_count = q_ringpack.size();
    SecretKey sk(context);
    PCMM_Context pcmm_context(PCMM_N1, mlwe_rank, p_ringpack, q_ringpack, context);
    Bootstrapper bootstrapper(context, scheme);
    PCMM_Scheme pcmm_scheme(pcmm_context, scheme, bootstrapper, sk);        // [ref] test_pcmm_boot.cu:50
    MLWESecretKey mlwe_sk(PCMM_N1, (int)pcmm_context.pq_ringpack.size(), mlwe_rank);
    pcmm_scheme.convertMLWESKfromRLWESK(mlwe_sk, sk);
    scheme.addEncKey(sk);
    pcmm_scheme.addRepakcingKey(mlwe_sk, sk);

    const int feats = 768, toks = PCMM_N1;
    vector<float> W((size_t)feats * feats);
    std::normal_distribution<float> wdist(0.f, 0.02f);
    for (auto& w : W) w = wdist(rng);
    vector<double> X((size_t)feats * toks);                 // [feature][token], ~N(0,1) clipped to [-8, 8], scaled to the driver's 0.1 range
    std::normal_distribution<double> xdist(0.0, 1.0);
    for (auto& x : X) x = max(-8.0, min(8.0, xdist(rng))) / 80.0;
    float* plain_mat;
    cudaMalloc(&plain_mat, sizeof(float) * W.size());
    cudaMemcpy(plain_mat, W.data(), sizeof(float) * W.size(), cudaMemcpyHostToDevice);

    vector<MLWECiphertext*> mlwe_cipher_buffer;
    for (int i = 0; i < feats; i++)
        mlwe_cipher_buffer.push_back(new MLWECiphertext(PCMM_N1, q_ringpack_count - 1, q_ringpack_count - 1, mlwe_rank, NTL::RR(context.precision)));
    Ciphertext* res_cipher[3];
    double* msg_device;
    cudaMalloc(&msg_device, sizeof(double) * N);
    for (int c = 0; c < 3; c++) {
        // feature i of this ciphertext, token t -> coefficient 2*i + t*rank (the comb a decomposition into 256 extracts)
        vector<double> msg(N, 0.0);
        for (int i = 0; i < 256; i++)
            for (int t = 0; t < toks; t++) msg[2 * i + (size_t)t * mlwe_rank] = X[(size_t)(c * 256 + i) * toks + t];
        cudaMemcpy(msg_device, msg.data(), sizeof(double) * N, cudaMemcpyHostToDevice);
        Plaintext plain(N, L, 1, slots, NTL::RR(context.precision));
        context.encode_coeffs(msg_device, plain);
        res_cipher[c] = new Ciphertext(N, L, L, slots, NTL::RR(context.precision));
        scheme.encryptMsg(*res_cipher[c], plain);
    }

    pcmm_scheme.realData_coeffShift(*res_cipher[0], 0);                                 // [ref] Bert.cuh:403
    pcmm_scheme.rlweCipherDecompose(*res_cipher[0], mlwe_cipher_buffer, 256, 0);        // [ref] :404
    pcmm_scheme.rlweCipherDecompose(*res_cipher[1], mlwe_cipher_buffer, 256, 256);      // [ref] :408
    pcmm_scheme.rlweCipherDecompose(*res_cipher[2], mlwe_cipher_buffer, 256, 512);      // [ref] :412

    CUDATimer cuTimer;                                                                  // [ref] :423-427
    cuTimer.start();
    pcmm_scheme.PPMM(plain_mat, mlwe_cipher_buffer, 768, 768, 128, 768);
    cout << "ppmm time "  << cuTimer.stop() << endl;
    cout << "after ppmm scale: " << mlwe_cipher_buffer[0]->scale << endl;

    pcmm_scheme.mlweCipherPacking(*res_cipher[0], mlwe_cipher_buffer, 256, 0);          // [ref] :471
    pcmm_scheme.mlweCipherPacking(*res_cipher[1], mlwe_cipher_buffer, 256, 256);        // [ref] :480
    pcmm_scheme.mlweCipherPacking(*res_cipher[2], mlwe_cipher_buffer, 256, 512);        // [ref] :489

    double worst = 0, want_max = 0;
    vector<double> got(N);
    for (int c = 0; c < 3; c++) {
        Plaintext dec(N, L, 1, slots, NTL::RR(context.precision));
        scheme.decryptMsg(dec, sk, *res_cipher[c]);
        context.decode_coeffs(dec, msg_device);
        cudaMemcpy(got.data(), msg_device, sizeof(double) * N, cudaMemcpyDeviceToHost);
        for (int i = 0; i < 256; i++)
            for (int t = 0; t < toks; t++) {
                double want = 0;
                for (int n = 0; n < feats; n++) want += (double)W[(size_t)(c * 256 + i) * feats + n] * X[(size_t)n * toks + t];
                worst = max(worst, fabs(got[2 * i + (size_t)t * mlwe_rank] - want));
                want_max = max(want_max, fabs(want));
            }
    }
    printf("bert 768x768: relative error %.3e (2^%.1f), result level %d\n", worst / want_max, log2(worst / want_max), res_cipher[0]->l);
    for (auto c : mlwe_cipher_buffer) delete c;
    for (auto c : res_cipher) delete c;
    return worst / want_max < ldexp(1.0, -20) ? 0 : 1;
}

int main(int argc, char* argv[])
{
    if (argc >= 4 && string(argv[1]) == "decomp") return run_decomp(atoi(argv[2]), atoi(argv[3]), argc > 4 ? argv[4] : nullptr);
    if (argc >= 2 && string(argv[1]) == "bert") return run_bert();
    printf("usage: compat_tree_driver decomp <logN> <N1> [dump.bin] | bert\n");
    return 2;
}
