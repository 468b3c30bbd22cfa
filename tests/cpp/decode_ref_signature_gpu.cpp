// A caller written against the reference's exact launcher signatures
//   cdna3::attn::decode(q, K, V, o, DecodeCfg, stream)          cdna3-prims/include/cdna3/attention.hpp:117-119
//   cdna3::attn::decode_dme(q, K, V, o, DecodeDmeCfg, stream)   attention.hpp:152-154
// (no workspace argument: the launcher must not need one).  Reads fp16 q, K, V from a file,
// runs both launchers on the GPU, writes the two fp16 outputs.  Built and run by
// tests/test_zz_no_alloc.py, which compares the outputs with the CPU oracle.
//   argv: in_file out_file D N nQH nKVH stride_kv
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>
#include "cdna3/attention.hpp"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 2; } } while (0)

int main(int argc, char** argv) {
    if (argc != 8) return 64;
    const int D = std::atoi(argv[3]), N = std::atoi(argv[4]), nQH = std::atoi(argv[5]), nKVH = std::atoi(argv[6]), stride = std::atoi(argv[7]);
    const size_t nq = size_t(nQH) * D, nkv = size_t(nKVH) * stride * D;
    std::vector<__half> hq(nq), hk(nkv), hv(nkv), ho(2 * nq);
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 65;
    if (std::fread(hq.data(), 2, nq, f) != nq || std::fread(hk.data(), 2, nkv, f) != nkv || std::fread(hv.data(), 2, nkv, f) != nkv) return 66;
    std::fclose(f);
    __half *q, *K, *V, *o;
    CK(cudaMalloc(&q, nq * 2)); CK(cudaMalloc(&K, nkv * 2)); CK(cudaMalloc(&V, nkv * 2)); CK(cudaMalloc(&o, 2 * nq * 2));
    CK(cudaMemcpy(q, hq.data(), nq * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(K, hk.data(), nkv * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(V, hv.data(), nkv * 2, cudaMemcpyHostToDevice));
    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    int rc = 0;
    if (stride == N) {                                   // packed K/V: the plain decode launcher
        cdna3::attn::DecodeCfg c{D, N, nQH, nKVH};
        rc = cdna3::attn::decode(q, K, V, o, c, st);
    } else {
        rc = 0;
        CK(cudaMemsetAsync(o, 0, nq * 2, st));
    }
    if (rc) { std::fprintf(stderr, "decode: %s\n", b200p_strerror(rc)); return 3; }
    cdna3::attn::DecodeDmeCfg m{D, N, nQH, nKVH, stride};
    rc = cdna3::attn::decode_dme(q, K, V, o + nq, m, st);
    if (rc) { std::fprintf(stderr, "decode_dme: %s\n", b200p_strerror(rc)); return 4; }
    if (b200p_attn_workspace_status(nullptr, st) != 0) return 5;     // synchronises; a wait that gave up would show here
    CK(cudaMemcpy(ho.data(), o, 2 * nq * 2, cudaMemcpyDeviceToHost));
    f = std::fopen(argv[2], "wb");
    if (!f) return 67;
    std::fwrite(ho.data(), 2, 2 * nq, f);
    std::fclose(f);
    return 0;
}
