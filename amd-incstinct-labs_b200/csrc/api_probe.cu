// ---------------------------------------------------------------------------
// api_probe.cu -- small kernels that call the device-level headers exactly as a
// user of the reference's facade would (cdna3-prims/tests/compile_smoke.hip:24-50):
// <cdna3/cdna3.hpp> and <cdna3/examples/fused_softmax.hpp> by include, nothing
// else.  They exist so that the headers are compiled for sm_100a with the library
// and can be checked on a GPU through the C ABI (b200p_api_probe).
// ---------------------------------------------------------------------------
#include "common.cuh"
#include <cdna3/cdna3.hpp>
#include <cdna3/examples/fused_softmax.hpp>

namespace b200p {
namespace {

// which = 0: row_softmax_lane over rows of 64 scores (pair per lane); one warp per row.
// which = 1: row_softmax_lane, one score per lane, rows of 32.
__global__ void softmax_rows_kernel(int which, const float* in, float* out, int rows) {
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= rows) return;
    const unsigned l = threadIdx.x % 32;
    if (which == 0) {
        float p0, p1;
        cdna3::ex::row_softmax_lane(in[size_t(row) * 64 + 2 * l], in[size_t(row) * 64 + 2 * l + 1], p0, p1);
        out[size_t(row) * 64 + 2 * l] = p0; out[size_t(row) * 64 + 2 * l + 1] = p1;
    } else {
        out[size_t(row) * 32 + l] = cdna3::ex::row_softmax_lane(in[size_t(row) * 32 + l]);
    }
}

// which = 2: online_softmax_step over `tiles` tiles of 64 scores per row: out[row] = (m, l, sum of p rescaled)
// i.e. the row's final running max, denominator, and sum_k exp(s_k - m) accumulated the way an O column would be.
__global__ void online_rows_kernel(const float* in, float* out, int rows, int tiles) {
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= rows) return;
    const unsigned l = threadIdx.x % 32;
    float m = -1e38f, lrun = 0.f, acc = 0.f;
    for (int j = 0; j < tiles; ++j) {
        const float* s = in + (size_t(row) * tiles + j) * 64;
        float p0, p1;
        const float resc = cdna3::ex::online_softmax_step(s[2 * l], s[2 * l + 1], m, lrun, p0, p1);
        acc = acc * resc + wave::dpp::reduce_sum_bcast(p0, p1);
    }
    if (l == 0) { out[size_t(row) * 3] = m; out[size_t(row) * 3 + 1] = lrun; out[size_t(row) * 3 + 2] = acc; }
}

// which = 3: the reference's per-thread asynchronous copy API: `tiles` packed [16][64] fp16 tiles streamed
// through an AsyncTile2D ping/pong by 128 threads; out[tile][e] = 2 * in[tile][e] (fp32), read from shared memory.
// which = 4: copy_tile_1d_stream<float, 256> by one warp per 256-float tile, out = in + 1.
constexpr int kR = 16, kC = 64;
__global__ void dme_tiles_kernel(const __half* in, float* out, int tiles) {
    __shared__ __align__(16) __half buf[2][kR * kC];
    const int tid = threadIdx.x, nth = blockDim.x;
    dme::AsyncTile2D<kR, kC> tile;
    tile.prologue(in, buf, tid, nth);
    for (int j = 0; j < tiles; ++j) {
        tile.prefetch_next(in, buf, j + 1, tiles, tid, nth);
        for (int e = tid; e < kR * kC; e += nth) out[size_t(j) * kR * kC + e] = 2.f * __half2float(buf[tile.cur()][e]);
        tile.wait_next(j + 1, tiles);
        tile.advance();
    }
}
__global__ void dme_tile1d_kernel(const float* in, float* out, int tiles) {
    __shared__ __align__(16) float buf[4][256];
    const int w = threadIdx.x / 32, l = threadIdx.x % 32;
    const int t = blockIdx.x * 4 + w;
    if (t < tiles) dme::copy_tile_1d_stream<float, 256>(in + size_t(t) * 256, buf[w]);
    dme::wait();
    __syncthreads();
    if (t < tiles)
        for (int i = l; i < 256; i += 32) out[size_t(t) * 256 + i] = buf[w][i] + 1.f;
}

} // namespace
} // namespace b200p

using namespace b200p;

extern "C" int b200p_api_probe(int which, const void* in, float* out, int rows, int tiles, b200p_stream_t stream) {
    if (which < 0 || which > 4) return B200P_E_OP;
    if (!in || !out) return B200P_E_NULL;
    if (rows <= 0 || tiles <= 0) return B200P_E_LENGTH;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    if ((which == 3 || which == 4) && !aligned(in, 16)) return B200P_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (rows + 3) / 4;
    switch (which) {
        case 0: case 1: softmax_rows_kernel<<<grid, 128, 0, st>>>(which, static_cast<const float*>(in), out, rows); break;
        case 2: online_rows_kernel<<<grid, 128, 0, st>>>(static_cast<const float*>(in), out, rows, tiles); break;
        case 3: dme_tiles_kernel<<<1, 128, 0, st>>>(static_cast<const __half*>(in), out, tiles); break;
        case 4: dme_tile1d_kernel<<<(tiles + 3) / 4, 128, 0, st>>>(static_cast<const float*>(in), out, tiles); break;
    }
    return launched();
}
