// Quantised matrix times a few vectors: the projections on either side of the attention path.
//
// Stands in for GpuQuant::record (qmv, kernels/qmv.metal:12-48, kernels/quant.metal:9-62) and
// rows::record_proj (qmv_pk / qmv_mma, src/rows.rs:47-110, kernels/rows.metal) of the reference:
// y[r][row] = sum_c W[row][c] x[r][c] for m <= 8 rows of x, W an MLX affine matrix
// (src/quant.rs:1-30): a row is a little-endian bit stream of 5-, 6- or 8-bit integers in u32
// words, every 64 values share a bfloat16 scale and bias, w = scale * q + bias, so a group
// contributes scale * sum(q x) + bias * sum(x).
//
// HBM-bound on the weights, which are read once for all m rows.  Two kernels:
//
//  * qmv_units_kernel, for rows of a multiple of 1024 values (every projection of the model).  A row
//    is cut into units of 128 values = BITS 16-byte words; a team of 8, 16 or 32 lanes shares two
//    rows of W and a lane owns one unit of each, so that everything it needs is in flight as 2 x BITS
//    128-bit loads before any arithmetic starts.  x is staged once per block in shared memory, its
//    16-byte words swizzled inside a unit so that the lanes of a team, which read the same word of
//    different units, fall on different banks (read straight from global memory the same pattern
//    costs one cache line per lane per load and bounds the kernel); the staging pass also leaves
//    the sum of x over every group of 64 (sixteen lanes hold a group and add it up by exchange).  An integer is turned into a float without a
//    conversion instruction: its bits are moved to the top of the mantissa of 1.0, which gives
//    1 + q / 2^BITS exactly, so sum(q x) = 2^BITS (sum(f x) - sum(x)) with sum(x) already at hand.
//  * qmv_rows_kernel, for any other multiple of 64: a warp owns two rows, a lane walks them in chunks of
//    32 values (BITS consecutive 32-bit words) and reads x through the read-only cache.
#include "host.hpp"

#include <utility>

namespace saetta {

constexpr int kQmvRows = 2;  // rows of W per warp
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

#pragma unroll 1
    for (uint32_t k = lane; k < chunks; k += 32) { // chunk k = values 32k .. 32k+31 = half a group
        // the rows' 32 integers first (their loads are all in flight together), then x once per row of x
        float q[kQmvRows][32];
        float s[kQmvRows], b[kQmvRows];
#pragma unroll
        for (int r = 0; r < kQmvRows; r++) {
            const uint32_t row = min(row0 + r, rows - 1); // a row past the end repeats the last one; its sums are dropped
            const uint32_t *wp = words + size_t(row) * row_words + size_t(k) * BITS;
            uint32_t w[BITS + 1];
#pragma unroll
            for (int c = 0; c < BITS; c++) w[c] = __ldg(wp + c);
            w[BITS] = 0u;
#pragma unroll
            for (int i = 0; i < 32; i++) q[r][i] = unpack_at<BITS>(w, i);
            const size_t g = size_t(row) * groups + (k >> 1);
            s[r] = __uint_as_float(uint32_t(__ldg(scales + g)) << 16), b[r] = __uint_as_float(uint32_t(__ldg(biases + g)) << 16);
        }
#pragma unroll
        for (int j = 0; j < M; j++) {
            const float4 *xp = reinterpret_cast<const float4 *>(x + size_t(j) * cols + k * 32);
            float qx[kQmvRows], xsum = 0.f;
#pragma unroll
            for (int r = 0; r < kQmvRows; r++) qx[r] = 0.f;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float4 v = __ldg(xp + c);
                xsum += (v.x + v.y) + (v.z + v.w);
#pragma unroll
                for (int r = 0; r < kQmvRows; r++)
                    qx[r] = fmaf(q[r][4 * c], v.x, fmaf(q[r][4 * c + 1], v.y, fmaf(q[r][4 * c + 2], v.z, fmaf(q[r][4 * c + 3], v.w, qx[r]))));
            }
#pragma unroll
            for (int r = 0; r < kQmvRows; r++) acc[r][j] = fmaf(s[r], qx[r], fmaf(b[r], xsum, acc[r][j]));
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

constexpr int kQmvThreads = 128; // threads per block of the units kernel

// value i of a unit as 1 + q / 2^BITS: its BITS bits moved to the top of the mantissa of 1.0
template <int BITS, int I>
__device__ __forceinline__ float unit_value(const uint32_t (&w)[4 * BITS]) {
    constexpr int bit = I * BITS, word = bit >> 5, p = bit & 31, P = 23 - BITS;
    uint32_t v;
    if constexpr (p < P) {
        v = w[word] << (P - p); // p + BITS <= 32: the integer lies inside this word
    } else if constexpr (p == P) {
        v = w[word];
    } else {
        const uint32_t hi = word + 1 < 4 * BITS ? w[word + 1 < 4 * BITS ? word + 1 : word] : 0u;
        v = __funnelshift_r(w[word], hi, p - P);
    }
    return __uint_as_float((v & (((1u << BITS) - 1) << P)) | 0x3f800000u);
}

template <int BITS, int M, int RR, int C>
__device__ __forceinline__ void unit_word(const uint32_t (&w)[RR][4 * BITS], const float4 *xu, uint32_t x_words,
                                          uint32_t sw, float (&qx)[RR][M]) {
    float f[RR][4];
#pragma unroll
    for (int r = 0; r < RR; r++) {
        f[r][0] = unit_value<BITS, 4 * C>(w[r]), f[r][1] = unit_value<BITS, 4 * C + 1>(w[r]);
        f[r][2] = unit_value<BITS, 4 * C + 2>(w[r]), f[r][3] = unit_value<BITS, 4 * C + 3>(w[r]);
    }
#pragma unroll
    for (int j = 0; j < M; j++) {
        const float4 v = xu[size_t(j) * x_words + (uint32_t(C) ^ sw)];
#pragma unroll
        for (int r = 0; r < RR; r++)
            qx[r][j] = fmaf(f[r][0], v.x, fmaf(f[r][1], v.y, fmaf(f[r][2], v.z, fmaf(f[r][3], v.w, qx[r][j]))));
    }
}

template <int BITS, int M, int RR, int C0, int... Cs>
__device__ __forceinline__ void unit_half(const uint32_t (&w)[RR][4 * BITS], const float4 *xu, uint32_t x_words,
                                          uint32_t sw, float (&qx)[RR][M], std::integer_sequence<int, Cs...>) {
    (unit_word<BITS, M, RR, C0 + Cs>(w, xu, x_words, sw, qx), ...);
}

template <int BITS, int M, int RR>
__global__ void __launch_bounds__(kQmvThreads)
qmv_units_kernel(const uint32_t *__restrict__ words, const uint16_t *__restrict__ scales,
                 const uint16_t *__restrict__ biases, const float *__restrict__ x, float *__restrict__ y,
                 uint32_t rows, uint32_t cols, uint32_t y_stride, uint32_t team) {
    extern __shared__ __align__(16) float qmv_smem[];
    const uint32_t x_words = cols >> 2, units = cols >> 7, groups = cols >> 6;
    float4 *xs = reinterpret_cast<float4 *>(qmv_smem); // [M][cols / 4], swizzled inside every unit of 32
    float *gs = qmv_smem + size_t(M) * cols;          // [M][groups]: sum of x over each group
    const uint32_t tid = threadIdx.x, tl = tid & (team - 1), team_id = tid / team;
    const uint32_t row0 = (blockIdx.x * (kQmvThreads / team) + team_id) * RR;
    const size_t row_words = size_t(cols) * BITS / 32;

    uint32_t w[RR][4 * BITS], sb[RR][2];
    auto load = [&](uint32_t u) {
#pragma unroll
        for (int r = 0; r < RR; r++) {
            const uint32_t row = min(row0 + r, rows - 1); // a row past the end repeats the last one; its sums are dropped
            const uint4 *wp = reinterpret_cast<const uint4 *>(words + size_t(row) * row_words) + size_t(u) * BITS;
#pragma unroll
            for (int c = 0; c < BITS; c++) {
                const uint4 q = __ldg(wp + c);
                w[r][4 * c] = q.x, w[r][4 * c + 1] = q.y, w[r][4 * c + 2] = q.z, w[r][4 * c + 3] = q.w;
            }
            const size_t g = size_t(row) * groups + 2 * u; // both groups of the unit: two bfloat16 in one word
            sb[r][0] = __ldg(reinterpret_cast<const uint32_t *>(scales + g));
            sb[r][1] = __ldg(reinterpret_cast<const uint32_t *>(biases + g));
        }
    };
    uint32_t u = tl;
    load(u); // in flight while x is staged

    // x_words is a multiple of 256: every thread makes the same number of passes, and sixteen consecutive
    // lanes hold one group of 64, whose sum they form with four exchanges
    for (uint32_t i = tid; i < M * x_words; i += kQmvThreads) {
        const uint32_t j = i / x_words, k = i - j * x_words, unit = k >> 5, c = k & 31;
        const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
        xs[j * x_words + (unit << 5) + (c ^ (unit & 7))] = v;
        float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int off = 8; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if ((tid & 15) == 0) gs[j * groups + (k >> 4)] = sum;
    }
    __syncthreads();

    float acc[RR][M];
#pragma unroll
    for (int r = 0; r < RR; r++)
#pragma unroll
        for (int j = 0; j < M; j++) acc[r][j] = 0.f;
    while (true) {
        const float4 *xu = xs + (u << 5);
        const uint32_t sw = u & 7;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float qx[RR][M];
#pragma unroll
            for (int r = 0; r < RR; r++)
#pragma unroll
                for (int j = 0; j < M; j++) qx[r][j] = 0.f;
            if (h == 0) unit_half<BITS, M, RR, 0>(w, xu, x_words, sw, qx, std::make_integer_sequence<int, 16>{});
            else unit_half<BITS, M, RR, 16>(w, xu, x_words, sw, qx, std::make_integer_sequence<int, 16>{});
#pragma unroll
            for (int r = 0; r < RR; r++) {
                const uint32_t s16 = h ? sb[r][0] & 0xffff0000u : sb[r][0] << 16, b16 = h ? sb[r][1] & 0xffff0000u : sb[r][1] << 16;
                const float s = __uint_as_float(s16) * float(1 << BITS), b = __uint_as_float(b16);
#pragma unroll
                for (int j = 0; j < M; j++) {
                    const float xsum = gs[j * groups + 2 * u + h];
                    acc[r][j] = fmaf(s, qx[r][j] - xsum, fmaf(b, xsum, acc[r][j]));
                }
            }
        }
        u += team;
        if (u >= units) break;
        load(u);
    }
#pragma unroll
    for (int r = 0; r < RR; r++)
#pragma unroll
        for (int j = 0; j < M; j++) {
            float v = acc[r][j];
            if (team > 16) v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (team > 8) v += __shfl_xor_sync(0xffffffffu, v, 8);
#pragma unroll
            for (int off = 4; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (tl == 0 && row0 + r < rows) y[size_t(j) * y_stride + row0 + r] = v;
        }
}

constexpr size_t kQmvMaxShared = 200 * 1024;

template <int BITS, int M>
static int launch_qmv_m(const uint32_t *w, const uint16_t *s, const uint16_t *b, const float *x, float *y, uint32_t rows,
                        uint32_t cols, uint32_t y_stride, cudaStream_t st) {
    const size_t shared = (size_t(M) * cols + size_t(M) * (cols / 64)) * sizeof(float);
    const bool aligned = !(reinterpret_cast<uintptr_t>(w) & 15) && !((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(b)) & 3);
    if (cols % 1024 == 0 && shared <= kQmvMaxShared && aligned) {
        constexpr int RR = 2; // rows of W per lane (four measured the same at m = 4 and cost 70 more registers)
        const uint32_t units = cols / 128, team = units % 32 == 0 ? 32 : units % 16 == 0 ? 16 : 8;
        const uint32_t block_rows = kQmvThreads / team * RR;
        if (shared > 48 * 1024)
            SAETTA_CUDA(cudaFuncSetAttribute(qmv_units_kernel<BITS, M, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared)));
        qmv_units_kernel<BITS, M, RR><<<(rows + block_rows - 1) / block_rows, kQmvThreads, shared, st>>>(w, s, b, x, y, rows, cols, y_stride, team);
    } else {
        const unsigned grid = (rows + kQmvWarps * kQmvRows - 1) / (kQmvWarps * kQmvRows);
        qmv_rows_kernel<BITS, M><<<grid, kQmvWarps * 32, 0, st>>>(w, s, b, x, y, rows, cols, y_stride);
    }
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

template <int BITS>
static int launch_qmv(size_t m, const uint32_t *w, const uint16_t *s, const uint16_t *b, const float *x, float *y,
                      uint32_t rows, uint32_t cols, uint32_t y_stride, cudaStream_t st) {
    switch (m) {
#define SAETTA_QMV(M) \
    case M:           \
        return launch_qmv_m<BITS, M>(w, s, b, x, y, rows, cols, y_stride, st);
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
