// Attention prep fused with the store into the KV cache.
//
// Stands in for attention_prep / attention_prep_float (kernels/layers.metal:637-697)
// followed by QuantRows::record (src/gpu_layers.rs:373-411; per row in record_rows,
// :483-507), and for the prefill's norm + rope_rows + store sequence
// (src/prefill.rs:1607-1633, 1656-1666; kernels/prefill.metal:553-568): per token,
// RMS-norm and partial RoPE of every query head into q, RMS-norm and RoPE of every
// key head, and key and value into the token's cache slot -- quantised, narrowed
// to 16 bits or as f32, whatever the cache holds.  The reference writes the
// normed keys back as f32 and quantises them in a second pass; here they go
// from registers into the cache, and the f32 copy is optional.
//
// Arithmetic follows the CPU (src/cpu/ops.rs:19-36, 64-74): x * (scale * w) with
// scale = 1 / sqrt(mean(x^2) + eps), and the rotation a*c - b*s, a*s + b*c with the
// angle pos * theta^(-i/half) formed in f64 (the reference's GPU kernel uses f32 and
// loses digits at long positions).  Only the order of the sum of squares differs
// from the CPU's, so results agree to a few ulp, and the codes written to a
// quantised cache are exactly what the quantiser makes of the f32 keys this
// kernel would write back.
//
// HBM-bound element work: one block per token, one warp per head (8 values per
// lane, two 128-bit loads), the 32 sines and cosines once per token.
#include <cmath>

#include "host.hpp"

namespace saetta {

constexpr int kPrepMaxHalf = 64; // rotary pairs at most (rope_dims <= 128)

struct PrepArgs {
    const float *q_and_gate; // [rows][heads][2*256]: q in the first half of each head
    const float *k, *v;      // [rows][kv_heads][256]
    const float *q_norm, *k_norm;
    void *q_out;             // [rows][heads][256] f32 or 16-bit
    float *k_out;            // optional f32 copy of the normed and roped keys
    void *keys, *values;     // cache rows (16/32-bit) or key / value codes
    __half *ks, *kz, *vs, *vz;
    const saetta_token_params *params;
    uint32_t pos, capacity;
    uint32_t heads, kv_heads, half_dims;
    float eps;
    int q_dtype;   // SAETTA_F16, SAETTA_BF16 or SAETTA_F32
    int bits;      // of the cache: 32, 16, 8, 4
    int kv_dtype;  // of a 16-bit cache
    double freq[kPrepMaxHalf]; // theta^(-i/half), as the CPU forms it
};

// The quantiser of kv_quant.cu on the 64 values held by 8 consecutive lanes (8 each).
template <int BITS>
__device__ __forceinline__ void quantize_group(const float (&x)[8], uint32_t lane8, size_t G, uint32_t *data,
                                               __half *scales, __half *biases) {
    float lo = x[0], hi = x[0];
#pragma unroll
    for (int e = 1; e < 8; e++) lo = fminf(lo, x[e]), hi = fmaxf(hi, x[e]);
#pragma unroll
    for (int off = 4; off; off >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off, 8));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off, 8));
    }
    constexpr float levels = float((1u << BITS) - 1);
    const __half sh = __float2half_rn(__fdiv_rn(__fsub_rn(hi, lo), levels));
    const __half zh = __float2half_rn(lo);
    const float sf = __half2float(sh), zf = __half2float(zh);
    const float inv = sf > 0.0f ? __fdiv_rn(1.0f, sf) : 0.0f;
    uint32_t c[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        float r = rintf(__fmul_rn(__fsub_rn(x[e], zf), inv));
        r = r != r ? 0.0f : fminf(fmaxf(r, 0.0f), levels);
        c[e] = static_cast<uint32_t>(r);
    }
    if (BITS == 8) {
        const uint32_t w0 = c[0] | c[1] << 8 | c[2] << 16 | c[3] << 24, w1 = c[4] | c[5] << 8 | c[6] << 16 | c[7] << 24;
        reinterpret_cast<uint2 *>(data)[G * 8 + lane8] = make_uint2(w0, w1);
    } else {
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 8; e++) w |= c[e] << (4 * e);
        data[G * 8 + lane8] = w;
    }
    if (lane8 == 0) scales[G] = sh, biases[G] = zh;
}

__device__ __forceinline__ void store8(void *dst, size_t at, const float (&x)[8], int mode) {
    // mode 0 binary16, 1 bfloat16, 2 f32; `at` counts values
    if (mode == 2) {
        float4 *p = reinterpret_cast<float4 *>(reinterpret_cast<float *>(dst) + at);
        p[0] = make_float4(x[0], x[1], x[2], x[3]), p[1] = make_float4(x[4], x[5], x[6], x[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (mode == 0) {
                w[e] = pack_half2(x[2 * e], x[2 * e + 1]);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t *>(&h);
            }
        }
        *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(dst) + at) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

__global__ void __launch_bounds__(1024, 2) attention_prep_kernel(const PrepArgs a) {
    __shared__ float sn[kPrepMaxHalf], cs[kPrepMaxHalf];
    const uint32_t row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t position = (a.params ? a.params->position : a.pos) + row;
    // warps 0..heads-1: query heads; then kv_heads key heads; then kv_heads value heads
    const bool is_q = warp < a.heads, is_k = !is_q && warp < a.heads + a.kv_heads;
    const uint32_t j = is_q ? warp : is_k ? warp - a.heads : warp - a.heads - a.kv_heads;
    const float *src = is_q   ? a.q_and_gate + (size_t(row) * a.heads + j) * 2 * kDim
                       : is_k ? a.k + (size_t(row) * a.kv_heads + j) * kDim
                              : a.v + (size_t(row) * a.kv_heads + j) * kDim;
    // the loads go out first, so that the sines and cosines below are computed while they are in flight
    const float4 v0 = reinterpret_cast<const float4 *>(src)[lane * 2], v1 = reinterpret_cast<const float4 *>(src)[lane * 2 + 1];
    float wn[8];
    if (is_q || is_k) {
        const float4 *w = reinterpret_cast<const float4 *>((is_q ? a.q_norm : a.k_norm) + lane * 8);
        const float4 w0 = w[0], w1 = w[1];
        wn[0] = w0.x, wn[1] = w0.y, wn[2] = w0.z, wn[3] = w0.w, wn[4] = w1.x, wn[5] = w1.y, wn[6] = w1.z, wn[7] = w1.w;
    }
    if (threadIdx.x < a.half_dims) {
        // angle in f64 as the CPU forms it, brought into [-pi, pi] in f64 (2 pi in two pieces), then the
        // f32 sine and cosine of the remainder: within 2 ulp of rounding the f64 functions
        const double angle = double(position) * a.freq[threadIdx.x];
        const double turns = rint(angle * 0.15915494309189535);
        const double rem = fma(-turns, 2.4492935982947064e-16, fma(-turns, 6.283185307179586, angle));
        float s, c;
        sincosf(float(rem), &s, &c);
        sn[threadIdx.x] = s, cs[threadIdx.x] = c;
    }
    __syncthreads();
    float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    if (is_q || is_k) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss = __fadd_rn(ss, __fmul_rn(x[e], x[e]));
#pragma unroll
        for (int off = 16; off; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(kDim)), a.eps)));
#pragma unroll
        for (int e = 0; e < 8; e++) x[e] = __fmul_rn(x[e], __fmul_rn(scale, wn[e]));
        // RoPE: value i < half pairs with i + half.  Lanes whose dims lie below 2*half take part.
        const uint32_t half = a.half_dims; // a multiple of 8
        const uint32_t d0 = lane * 8;
        const uint32_t lanes_half = half / 8; // lanes per half
        // the partner lane holds the other member of every pair of this lane (same e)
        const bool lower = d0 < half, rot = d0 < 2 * half;
        const uint32_t partner = lower ? lane + lanes_half : lane - lanes_half;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float other = __shfl_sync(0xffffffffu, x[e], rot ? partner : lane);
            if (rot) {
                const uint32_t r = (lower ? d0 : d0 - half) + e;
                const float s = sn[r], c = cs[r];
                const float av = lower ? x[e] : other, bv = lower ? other : x[e];
                x[e] = lower ? __fsub_rn(__fmul_rn(av, c), __fmul_rn(bv, s)) : __fadd_rn(__fmul_rn(av, s), __fmul_rn(bv, c));
            }
        }
    }
    if (is_q) {
        store8(a.q_out, (size_t(row) * a.heads + j) * kDim + lane * 8, x, a.q_dtype == SAETTA_F32 ? 2 : a.q_dtype);
        return;
    }
    if (is_k && a.k_out) store8(a.k_out, (size_t(row) * a.kv_heads + j) * kDim + lane * 8, x, 2);
    if (position >= a.capacity) return; // never write past the cache; the caller sized it
    if (a.bits == 8 || a.bits == 4) {
        const size_t G = (size_t(position) * a.kv_heads + j) * kGroupsPerHead + lane / 8;
        uint32_t *data = reinterpret_cast<uint32_t *>(is_k ? a.keys : a.values);
        __half *scales = is_k ? a.ks : a.vs, *biases = is_k ? a.kz : a.vz;
        if (a.bits == 8) quantize_group<8>(x, lane & 7, G, data, scales, biases);
        else quantize_group<4>(x, lane & 7, G, data, scales, biases);
    } else {
        const int mode = a.bits == 32 ? 2 : a.kv_dtype == SAETTA_BF16 ? 1 : 0;
        store8(is_k ? a.keys : a.values, (size_t(position) * a.kv_heads + j) * kDim + lane * 8, x, mode);
    }
}

} // namespace saetta

using namespace saetta;

extern "C" int saetta_attention_prep(saetta_prep_params p, size_t rows, const float *q_and_gate_dev, const float *k_dev,
                                     const float *v_dev, const float *q_norm_dev, const float *k_norm_dev, void *q_out_dev,
                                     int q_dtype, saetta_kv_cache *cache, const saetta_token_params *params_dev, size_t pos,
                                     float *k_out_dev, void *stream) {
    if (!q_and_gate_dev || !k_dev || !v_dev || !q_norm_dev || !k_norm_dev || !q_out_dev || !cache)
        return fail(SAETTA_ERR_BAD_ARG, "attention prep: null pointer");
    if (p.head_dim != kDim || p.heads != p.kv_heads * kHeadsPerKv || !p.kv_heads)
        return fail(SAETTA_ERR_BAD_SHAPE, "attention prep: head_dim must be 256 and heads 8 per kv head");
    if (p.heads + 2 * p.kv_heads > 32) return fail(SAETTA_ERR_BAD_SHAPE, "attention prep: at most 32 heads in all (one warp each)");
    if (p.rope_dims % 16 || p.rope_dims > 2 * kPrepMaxHalf || p.rope_dims > p.head_dim)
        return fail(SAETTA_ERR_BAD_SHAPE, "attention prep: rope_dims must be a multiple of 16, at most 128");
    if (cache->kv_heads != p.kv_heads || cache->head_dim != p.head_dim)
        return fail(SAETTA_ERR_BAD_SHAPE, "attention prep: cache and parameters disagree on the heads");
    if (q_dtype != SAETTA_F16 && q_dtype != SAETTA_BF16 && q_dtype != SAETTA_F32)
        return fail(SAETTA_ERR_BAD_ARG, "attention prep: unknown q dtype");
    if (!params_dev && pos + rows > cache->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "attention prep: rows past the cache's capacity");
    if ((reinterpret_cast<uintptr_t>(q_and_gate_dev) | reinterpret_cast<uintptr_t>(k_dev) | reinterpret_cast<uintptr_t>(v_dev) |
         reinterpret_cast<uintptr_t>(q_out_dev) | reinterpret_cast<uintptr_t>(k_out_dev) | reinterpret_cast<uintptr_t>(q_norm_dev) |
         reinterpret_cast<uintptr_t>(k_norm_dev)) & 15)
        return fail(SAETTA_ERR_BAD_ARG, "attention prep: buffers must be 16-byte aligned");
    if (!rows) return SAETTA_OK;
    DeviceGuard guard(cache->device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "attention prep: cannot select the device");
    PrepArgs a = {};
    a.q_and_gate = q_and_gate_dev, a.k = k_dev, a.v = v_dev, a.q_norm = q_norm_dev, a.k_norm = k_norm_dev;
    a.q_out = q_out_dev, a.k_out = k_out_dev;
    a.params = params_dev, a.pos = uint32_t(pos), a.capacity = uint32_t(cache->capacity);
    a.heads = p.heads, a.kv_heads = p.kv_heads, a.half_dims = p.rope_dims / 2, a.eps = p.eps;
    a.q_dtype = q_dtype, a.bits = cache->bits, a.kv_dtype = cache->dtype;
    if (cache->bits == 8 || cache->bits == 4) {
        a.keys = cache->k.data, a.values = cache->v.data;
        a.ks = (__half *)cache->k.scales, a.kz = (__half *)cache->k.biases;
        a.vs = (__half *)cache->v.scales, a.vz = (__half *)cache->v.biases;
    } else {
        a.keys = cache->keys, a.values = cache->values;
    }
    // src/cpu/ops.rs:66-68: freq = theta^(-i / half) in f64
    for (uint32_t i = 0; i < a.half_dims; i++) a.freq[i] = std::pow(double(p.rope_theta), -double(i) / double(a.half_dims));
    const unsigned threads = (p.heads + 2 * p.kv_heads) * 32;
    attention_prep_kernel<<<unsigned(rows), threads, 0, (cudaStream_t)stream>>>(a);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}
