// Host-only translation unit: the reference-shaped C++ API compiles with a plain C++
// compiler and links against libb200p.so.  Mirrors the call shapes of
// cdna3-prims/tests/validate_attention_api.hip:95,128 and
// cdna3-prims/tests/validate_decode_dme.hip:109-117 (no device work is done here).
#include <cstdio>
#include "cdna3/attention.hpp"
#include "b200p_runtime.h"

int main() {
    cdna3::attn::PrefillCfg pcfg{128, 256, 256, 4, 2, 1, 1};
    cdna3::attn::DecodeCfg dcfg{128, 512, 32, 8};
    cdna3::attn::DecodeDmeCfg mcfg{64, 256, 14, 2, 1024};
    // argument errors are reported before any launch, with or without a GPU
    int e1 = cdna3::attn::prefill<__half>(nullptr, nullptr, nullptr, nullptr, pcfg);
    cdna3::attn::PrefillCfg bad = pcfg; bad.D = 96;
    int e2 = cdna3::attn::prefill<__half>(nullptr, nullptr, nullptr, nullptr, bad);
    int e3 = cdna3::attn::decode<__half>(nullptr, nullptr, nullptr, nullptr, dcfg, nullptr, 0);
    int e4 = cdna3::attn::decode_dme<__nv_bfloat16>(nullptr, nullptr, nullptr, nullptr, mcfg);
    size_t ws = cdna3::attn::decode_workspace_bytes(dcfg);
    // the plain C entry points that have no counterpart in the reference's headers
    b200p_decode_args a{};
    a.D = 128; a.N = 512; a.nQHeads = 32; a.nKVHeads = 8; a.stride_kv = 512; a.batch = 1; a.dtype = B200P_BF16;
    int e5 = b200p_attn_decode_dyn(nullptr, nullptr, nullptr, nullptr, &a, nullptr, 0, nullptr, 0, nullptr);
    b200p_peer_exchange px{};
    int e6 = b200p_attn_decode_push(nullptr, nullptr, nullptr, &a, nullptr, 0, &px, 1, nullptr);
    int e7 = b200p_attn_merge_lse_wait(&px, 1, 8, 128, B200P_BF16, nullptr, nullptr, 0, nullptr);
    int e8 = b200p_skinny_gemm(B200P_BF16, 0, 1, nullptr, nullptr, nullptr, nullptr, nullptr, 2, 64, 64, 64, 64, 1e-6f, nullptr);
    std::printf("%d %d %d %d %zu %d %d %d %d %s\n", e1, e2, e3, e4, ws, e5, e6, e7, e8, b200p_version());
    return (e1 == B200P_E_NULL && e2 == B200P_E_DIM && e3 < 0 && e4 < 0 && ws > 0 &&
            e5 == B200P_E_NULL && e6 < 0 && e7 == B200P_E_NULL && e8 == B200P_E_NULL) ? 0 : 1;
}
