// Split-KV decode / verify attention over an f32, binary16 or bfloat16 cache,
// in f32 arithmetic on the CUDA cores.
//
// Stands in for attention_partial (kernels/attention.metal:25-121) and
// attention_partial_rows_chunks (kernels/attention_rows.metal:359-571) of the
// reference: the "exact" path its f32-tolerance checks use.  Dot products are
// sequential f32 sums like the CPU's, so the f32 configuration meets its 5e-6
// bound.  This is the small-configuration path; the bandwidth-bound one is
// decode_quant.cu.
#include "host.hpp"

namespace saetta {

constexpr int kXTile = 32;
constexpr float kLog2eX = 1.4426950408889634f;

struct ExactArgs {
    const void *k, *v; // [capacity][kv_heads][256]
    const float *q;    // [m][heads][256]
    float *parts;      // [splits][m][heads][kPartStride]
    const saetta_token_params *params;
    uint32_t m, row_step, capacity, kv_heads;
    float scale;
};

template <int MODE> // 0 binary16, 1 bfloat16, 2 f32
__device__ __forceinline__ float load_kv(const void *p, size_t i) {
    if (MODE == 2) return reinterpret_cast<const float *>(p)[i];
    if (MODE == 0) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}

// grid (splits, kv_heads), 256 threads.  R = 8 * MROWS query rows share the tile.
template <int MODE, int MROWS>
__global__ void __launch_bounds__(256) decode_exact_kernel(const ExactArgs a) {
    constexpr int R = 8 * MROWS;
    extern __shared__ float sm[];
    float *Ks = sm;                      // [32][257]
    float *Vs = Ks + kXTile * 257;       // [32][256]
    float *Qs = Vs + kXTile * 256;       // [R][256]
    float *Ss = Qs + R * 256;            // [R][32]
    float *Ms = Ss + R * kXTile;         // [R] running max (log2 units)
    float *Ls = Ms + R;                  // [R]
    float *As = Ls + R;                  // [R] rescale of this tile

    const uint32_t kv = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t heads = a.kv_heads * kHeadsPerKv;
    const uint32_t kv_len = a.params->kv_len;
    const uint32_t longest = min(kv_len + (a.m - 1) * a.row_step, a.capacity);
    const uint32_t tiles = (longest + kXTile - 1) / kXTile;
    const uint32_t t_begin = uint32_t(uint64_t(blockIdx.x) * tiles / gridDim.x);
    const uint32_t t_end = uint32_t(uint64_t(blockIdx.x + 1) * tiles / gridDim.x);

    for (uint32_t x = tid; x < R * 256; x += 256) {
        const uint32_t r = x >> 8, d = x & 255, row = r >> 3, h = kv * kHeadsPerKv + (r & 7);
        Qs[x] = row < a.m ? a.q[(size_t(row) * heads + h) * kDim + d] : 0.f;
    }
    if (tid < R) Ms[tid] = -INFINITY, Ls[tid] = 0.f;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
    __syncthreads();

    const size_t row_stride = size_t(a.kv_heads) * kDim;
    for (uint32_t t = t_begin; t < t_end; t++) {
        const uint32_t tok0 = t * kXTile;
        for (uint32_t x = tid; x < kXTile * 256; x += 256) {
            const uint32_t tt = x >> 8, d = x & 255;
            const size_t src = size_t(tok0 + tt) * row_stride + kv * kDim + d;
            const bool live = tok0 + tt < longest;
            Ks[tt * 257 + d] = live ? load_kv<MODE>(a.k, src) : 0.f;
            Vs[tt * 256 + d] = live ? load_kv<MODE>(a.v, src) : 0.f;
        }
        __syncthreads();
        // scores: lane = token, one query row per pass of a warp
        for (uint32_t r = warp; r < R; r += 8) {
            const float *qr = Qs + r * 256, *kr = Ks + lane * 257;
            float s = 0.f;
#pragma unroll 8
            for (int d = 0; d < 256; d++) s = __fadd_rn(s, __fmul_rn(qr[d], kr[d]));
            s = s * a.scale * kLog2eX;
            const uint32_t n_row = min(kv_len + (r >> 3) * a.row_step, a.capacity);
            if (tok0 + lane >= n_row) s = -INFINITY;
            float mx = s;
#pragma unroll
            for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_old = Ms[r], m_new = fmaxf(m_old, mx);
            const float p = m_new == -INFINITY ? 0.f : exp2f(s - m_new);
            float sum = p;
#pragma unroll
            for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            Ss[r * kXTile + lane] = p;
            if (lane == 0) {
                const float alpha = m_old == -INFINITY ? 0.f : exp2f(m_old - m_new);
                As[r] = alpha;
                Ms[r] = m_new;
                Ls[r] = Ls[r] * alpha + sum;
            }
        }
        __syncthreads();
        // O[r][d] for d = tid
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] *= As[r];
        for (int tt = 0; tt < kXTile; tt++) {
            const float v = Vs[tt * 256 + tid];
#pragma unroll
            for (int r = 0; r < R; r++) acc[r] = fmaf(Ss[r * kXTile + tt], v, acc[r]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint32_t row = r >> 3, h = kv * kHeadsPerKv + (r & 7);
        if (row >= a.m) continue;
        float *dst = a.parts + ((size_t(blockIdx.x) * a.m + row) * heads + h) * kPartStride;
        dst[tid] = acc[r];
        if (tid == 0) dst[kPartM] = Ms[r], dst[kPartL] = Ls[r];
    }
}

static constexpr size_t exact_smem(int R) {
    return (kXTile * 257 + kXTile * 256 + R * 256 + R * kXTile + 3 * R) * sizeof(float);
}

template <int MODE, int MROWS>
static int configure_one() {
    SAETTA_CUDA(cudaFuncSetAttribute(decode_exact_kernel<MODE, MROWS>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(exact_smem(8 * MROWS))));
    return SAETTA_OK;
}

// Raises the dynamic shared-memory limit of every instantiation on the current device.
int decode_exact_configure(int device) {
    (void)device;
    int rc = SAETTA_OK;
#define SAETTA_CFG(MODE)                                                                      \
    if (!rc) rc = configure_one<MODE, 1>();                                                   \
    if (!rc) rc = configure_one<MODE, 2>();                                                   \
    if (!rc) rc = configure_one<MODE, 4>();                                                   \
    if (!rc) rc = configure_one<MODE, 8>();
    SAETTA_CFG(0)
    SAETTA_CFG(1)
    SAETTA_CFG(2)
#undef SAETTA_CFG
    return rc;
}

template <int MODE, int MROWS>
static int launch_exact_one(const ExactArgs &a, int splits, cudaStream_t stream) {
    constexpr int R = 8 * MROWS;
    const size_t smem = exact_smem(R);
    decode_exact_kernel<MODE, MROWS><<<dim3(splits, a.kv_heads), 256, smem, stream>>>(a);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

template <int MODE>
static int launch_exact_mode(const ExactArgs &a, int splits, cudaStream_t stream) {
    if (a.m == 1) return launch_exact_one<MODE, 1>(a, splits, stream);
    if (a.m == 2) return launch_exact_one<MODE, 2>(a, splits, stream);
    if (a.m <= 4) return launch_exact_one<MODE, 4>(a, splits, stream);
    return launch_exact_one<MODE, 8>(a, splits, stream);
}

int launch_decode_exact(const KvView &kv, const float *q, float *parts, uint32_t m,
                        uint32_t row_step, int splits, uint32_t capacity,
                        const saetta_token_params *params, cudaStream_t stream) {
    ExactArgs a{kv.k, kv.v, q, parts, params, m, row_step, capacity, kv.kv_heads, 0.0625f};
    if (kv.bits == 32) return launch_exact_mode<2>(a, splits, stream);
    if (kv.dtype == SAETTA_BF16) return launch_exact_mode<1>(a, splits, stream);
    return launch_exact_mode<0>(a, splits, stream);
}

} // namespace saetta
