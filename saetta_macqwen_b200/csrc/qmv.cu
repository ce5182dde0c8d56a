// Quantised matrix times a few vectors: the projections on either side of the attention path.
//
// Stands in for GpuQuant::record (qmv, kernels/qmv.metal:12-48, kernels/quant.metal:9-62) and
// rows::record_proj (qmv_pk / qmv_mma, src/rows.rs:47-110, kernels/rows.metal) of the reference:
// y[r][row] = sum_c W[row][c] x[r][c] for m <= 8 rows of x, W an MLX affine matrix
// (src/quant.rs:1-30): a row is a little-endian bit stream of 5-, 6- or 8-bit integers in u32
// words, every 64 values share a bfloat16 scale and bias, w = scale * q + bias, so a group
// contributes scale * sum(q x) + bias * sum(x).
//
// HBM-bound on the weights, which are read once for all m rows.  A warp owns four consecutive rows
// of W; a lane walks the row in chunks of 32 values (= BITS consecutive words, so a warp's loads of
// one row are contiguous), unpacks them with funnel shifts and multiplies them into up to eight
// accumulators.  x is small and comes through the read-only cache.
#include "host.hpp"

namespace saetta {

constexpr int kQmvRows = 4;  // rows of W per warp
constexpr int kQmvWarps = 8; // warps per block

template <int BITS>
__device__ __forceinline__ float unpack_at(const uint32_t (&w)[BITS + 1], int i) {
    const int bit = i * BITS, word = bit >> 5, shift = bit & 31;
    const uint32_t v = __funnelshift_r(w[word], w[word + 1], shift); // bits shift.. of the 64-bit pair
    return float(v & ((1u << BITS) - 1));
}

template <int BITS, int M>
__global__ void __launch_bounds__(kQmvWarps * 32)
qmv_rows_kernel(const uint32_t *__restrict__ words, const uint16_t *__restrict__ scales,
                const uint16_t *__restrict__ biases, const float *__restrict__ x, float *__restrict__ y,
                uint32_t rows, uint32_t cols, uint32_t y_stride) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row0 = (blockIdx.x * kQmvWarps + warp) * kQmvRows;
    if (row0 >= rows) return;
    const uint32_t row_words = cols * BITS / 32, groups = cols / 64, chunks = cols / 32;
    float acc[kQmvRows][M];
#pragma unroll
    for (int r = 0; r < kQmvRows; r++)
#pragma unroll
        for (int j = 0; j < M; j++) acc[r][j] = 0.f;

    for (uint32_t k = lane; k < chunks; k += 32) { // chunk k = values 32k .. 32k+31 = half a group
        float xsum[M];
#pragma unroll
        for (int j = 0; j < M; j++) {
            const float4 *xp = reinterpret_cast<const float4 *>(x + size_t(j) * cols + k * 32);
            float t = 0.f;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float4 v = __ldg(xp + c);
                t += (v.x + v.y) + (v.z + v.w);
            }
            xsum[j] = t;
        }
#pragma unroll
        for (int r = 0; r < kQmvRows; r++) {
            const uint32_t row = row0 + r;
            if (row >= rows) break;
            const uint32_t *wp = words + size_t(row) * row_words + size_t(k) * BITS;
            uint32_t w[BITS + 1];
#pragma unroll
            for (int c = 0; c < BITS; c++) w[c] = wp[c];
            w[BITS] = 0u;
            float qx[M];
#pragma unroll
            for (int j = 0; j < M; j++) qx[j] = 0.f;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float q0 = unpack_at<BITS>(w, 4 * c), q1 = unpack_at<BITS>(w, 4 * c + 1);
                const float q2 = unpack_at<BITS>(w, 4 * c + 2), q3 = unpack_at<BITS>(w, 4 * c + 3);
#pragma unroll
                for (int j = 0; j < M; j++) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + size_t(j) * cols + k * 32) + c);
                    qx[j] = fmaf(q0, v.x, fmaf(q1, v.y, fmaf(q2, v.z, fmaf(q3, v.w, qx[j]))));
                }
            }
            const size_t g = size_t(row) * groups + (k >> 1);
            const float s = __uint_as_float(uint32_t(scales[g]) << 16), b = __uint_as_float(uint32_t(biases[g]) << 16);
#pragma unroll
            for (int j = 0; j < M; j++) acc[r][j] = fmaf(s, qx[j], fmaf(b, xsum[j], acc[r][j]));
        }
    }
#pragma unroll
    for (int r = 0; r < kQmvRows; r++)
#pragma unroll
        for (int j = 0; j < M; j++) {
            float v = acc[r][j];
#pragma unroll
            for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && row0 + r < rows) y[size_t(j) * y_stride + row0 + r] = v;
        }
}

template <int BITS>
static int launch_qmv(size_t m, const uint32_t *w, const uint16_t *s, const uint16_t *b, const float *x, float *y,
                      uint32_t rows, uint32_t cols, uint32_t y_stride, cudaStream_t st) {
    const unsigned grid = (rows + kQmvWarps * kQmvRows - 1) / (kQmvWarps * kQmvRows), block = kQmvWarps * 32;
    switch (m) {
#define SAETTA_QMV(M)                                                                              \
    case M:                                                                                        \
        qmv_rows_kernel<BITS, M><<<grid, block, 0, st>>>(w, s, b, x, y, rows, cols, y_stride);     \
        break;
        SAETTA_QMV(1)
        SAETTA_QMV(2)
        SAETTA_QMV(3)
        SAETTA_QMV(4)
        SAETTA_QMV(5)
        SAETTA_QMV(6)
        SAETTA_QMV(7)
        SAETTA_QMV(8)
#undef SAETTA_QMV
    default:
        return fail(SAETTA_ERR_BAD_SHAPE, "qmv: 1 to 8 rows");
    }
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

} // namespace saetta

using namespace saetta;

extern "C" int saetta_qmv_rows(int device, const uint32_t *words_dev, const uint16_t *scales_dev, const uint16_t *biases_dev,
                               int bits, size_t rows, size_t cols, size_t m, const float *x_dev, float *y_dev,
                               size_t y_stride, void *stream) {
    if (!words_dev || !scales_dev || !biases_dev || !x_dev || !y_dev) return fail(SAETTA_ERR_BAD_ARG, "qmv: null pointer");
    if (bits != 5 && bits != 6 && bits != 8) return fail(SAETTA_ERR_UNSUPPORTED, "qmv: 5, 6 or 8 bits");
    if (!rows || !cols || cols % 64) return fail(SAETTA_ERR_BAD_SHAPE, "qmv: cols must be a multiple of the group, 64");
    if (!m || m > SAETTA_MAX_ROWS) return fail(SAETTA_ERR_BAD_SHAPE, "qmv: 1 to 8 rows");
    if (y_stride < rows) return fail(SAETTA_ERR_BAD_SHAPE, "qmv: y rows overlap");
    if ((reinterpret_cast<uintptr_t>(x_dev) & 15) || (reinterpret_cast<uintptr_t>(words_dev) & 3))
        return fail(SAETTA_ERR_BAD_ARG, "qmv: x must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "qmv: cannot select the device");
    auto st = (cudaStream_t)stream;
    const uint32_t r = uint32_t(rows), c = uint32_t(cols), ys = uint32_t(y_stride);
    if (bits == 5) return launch_qmv<5>(m, words_dev, scales_dev, biases_dev, x_dev, y_dev, r, c, ys, st);
    if (bits == 6) return launch_qmv<6>(m, words_dev, scales_dev, biases_dev, x_dev, y_dev, r, c, ys, st);
    return launch_qmv<8>(m, words_dev, scales_dev, biases_dev, x_dev, y_dev, r, c, ys, st);
}
