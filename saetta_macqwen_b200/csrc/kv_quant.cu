// KV-cache quantise-on-append and dequantise kernels.
//
// Stands in for kernels/kv_quant.metal:15-82 of the reference (kv_quantize<8|4>,
// kv_dequantize<8|4>) and the to_half copy of kernels/prefill.metal:1428-1432.
// The arithmetic follows src/kv_quant.rs:54-105 operation by operation with
// explicit round-to-nearest intrinsics, so codes, scales and biases are the
// CPU's bit for bit (the reference's own Metal kernel is allowed one code of
// slack because of a fast reciprocal; this one is not).
//
// HBM-bound byte work: one group of 64 values is handled by 16 lanes with one
// 128-bit load each; every code word is written once, coalesced.
#include "host.hpp"

namespace saetta {

struct QuantSideArgs {
    const float *x;   // [rows][per_token*64]
    uint32_t *data;   // [capacity*per_token][2*bits]
    __half *scales;   // [capacity*per_token]
    __half *biases;
};

template <int BITS>
__global__ void __launch_bounds__(256)
kv_quantize_kernel(QuantSideArgs s0, QuantSideArgs s1, uint32_t per_token, uint32_t groups,
                   uint32_t pos, const saetta_token_params *params) {
    const QuantSideArgs s = blockIdx.y ? s1 : s0;
    const uint32_t lane16 = threadIdx.x & 15;
    const uint32_t g = blockIdx.x * 16 + (threadIdx.x >> 4); // group among the new rows
    if (g >= groups) return;                                  // whole 16-lane team leaves together
    const uint32_t first = (params ? params->position : pos) * per_token;
    const float4 v = reinterpret_cast<const float4 *>(s.x)[g * 16 + lane16];

    // f32::min / f32::max folds (src/kv_quant.rs:62-63): a NaN operand is ignored.
    float lo = fminf(fminf(v.x, v.y), fminf(v.z, v.w));
    float hi = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
#pragma unroll
    for (int off = 8; off; off >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off, 16));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off, 16));
    }
    constexpr float levels = float((1u << BITS) - 1);
    const __half sh = __float2half_rn(__fdiv_rn(__fsub_rn(hi, lo), levels));
    const __half zh = __float2half_rn(lo);
    const float sf = __half2float(sh), zf = __half2float(zh);
    const float inv = sf > 0.0f ? __fdiv_rn(1.0f, sf) : 0.0f;
    auto code = [&](float x) -> uint32_t {
        float r = rintf(__fmul_rn(__fsub_rn(x, zf), inv)); // round_ties_even
        r = r != r ? 0.0f : fminf(fmaxf(r, 0.0f), levels); // clamp, then `as u32`
        return static_cast<uint32_t>(r);
    };
    uint32_t w = code(v.x) | code(v.y) << BITS | code(v.z) << (2 * BITS) | code(v.w) << (3 * BITS);
    const size_t G = size_t(first) + g;
    if (BITS == 8) {
        s.data[G * 16 + lane16] = w;
    } else {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, w, 1, 16);
        if (!(lane16 & 1)) s.data[G * 8 + (lane16 >> 1)] = w | other << 16;
    }
    if (lane16 == 0) {
        s.scales[G] = sh;
        s.biases[G] = zh;
    }
}

int launch_kv_quantize(int bits, uint32_t per_token, const float *x0, const QuantRows *r0,
                       const float *x1, const QuantRows *r1, size_t rows, size_t pos,
                       const saetta_token_params *params, cudaStream_t stream) {
    if (!rows) return SAETTA_OK;
    QuantSideArgs a0{x0, (uint32_t *)r0->data, (__half *)r0->scales, (__half *)r0->biases};
    QuantSideArgs a1 = a0;
    if (r1) a1 = QuantSideArgs{x1, (uint32_t *)r1->data, (__half *)r1->scales, (__half *)r1->biases};
    const uint32_t groups = uint32_t(rows * per_token);
    dim3 grid((groups + 15) / 16, r1 ? 2 : 1);
    if (bits == 8)
        kv_quantize_kernel<8><<<grid, 256, 0, stream>>>(a0, a1, per_token, groups, uint32_t(pos), params);
    else
        kv_quantize_kernel<4><<<grid, 256, 0, stream>>>(a0, a1, per_token, groups, uint32_t(pos), params);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

// kv_dequantize: out = round16(s * q + z), multiply then add (src/kv_quant.rs:100).
// One thread expands 8 codes into one 128-bit store.
template <int BITS, bool BF16>
__global__ void __launch_bounds__(256)
kv_dequantize_kernel(const uint32_t *__restrict__ data, const __half *__restrict__ scales,
                     const __half *__restrict__ biases, uint4 *__restrict__ out, size_t octets) {
    const size_t o = size_t(blockIdx.x) * 256 + threadIdx.x; // 8 values each
    if (o >= octets) return;
    const size_t g = o >> 3;
    const float s = __half2float(scales[g]), z = __half2float(biases[g]);
    uint32_t q[8];
    if (BITS == 8) {
        const uint2 w = reinterpret_cast<const uint2 *>(data)[o];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            q[i] = (w.x >> (8 * i)) & 255u;
            q[4 + i] = (w.y >> (8 * i)) & 255u;
        }
    } else {
        const uint32_t w = data[o];
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = (w >> (4 * i)) & 15u;
    }
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a = __fadd_rn(__fmul_rn(s, float(q[2 * i])), z);
        const float b = __fadd_rn(__fmul_rn(s, float(q[2 * i + 1])), z);
        if (BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            r[i] = *reinterpret_cast<uint32_t *>(&h);
        } else {
            r[i] = pack_half2(a, b);
        }
    }
    out[o] = make_uint4(r[0], r[1], r[2], r[3]);
}

// Rows [first, first + tokens) of `rows` as 16-bit values into the same rows of out ([row][values]).
int launch_kv_dequantize(const QuantRows *rows, void *out, int dtype, size_t first, size_t tokens,
                         cudaStream_t stream) {
    const size_t octets = tokens * rows->per_token * 8;
    if (!octets) return SAETTA_OK;
    const unsigned grid = unsigned((octets + 255) / 256);
    const size_t g0 = first * rows->per_token; // first group
    auto d = (const uint32_t *)rows->data + g0 * 2 * size_t(rows->bits);
    auto s = (const __half *)rows->scales + g0, z = (const __half *)rows->biases + g0;
    out = static_cast<uint4 *>(out) + g0 * 8;
    if (rows->bits == 8 && dtype == SAETTA_F16)
        kv_dequantize_kernel<8, false><<<grid, 256, 0, stream>>>(d, s, z, (uint4 *)out, octets);
    else if (rows->bits == 8)
        kv_dequantize_kernel<8, true><<<grid, 256, 0, stream>>>(d, s, z, (uint4 *)out, octets);
    else if (dtype == SAETTA_F16)
        kv_dequantize_kernel<4, false><<<grid, 256, 0, stream>>>(d, s, z, (uint4 *)out, octets);
    else
        kv_dequantize_kernel<4, true><<<grid, 256, 0, stream>>>(d, s, z, (uint4 *)out, octets);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

// Store of new rows into a 16-bit or f32 cache: MODE 0 binary16, 1 bfloat16, 2 f32.
template <int MODE>
__global__ void __launch_bounds__(256)
kv_store_plain_kernel(const float *__restrict__ k, const float *__restrict__ v, void *keys,
                      void *values, uint32_t row_values, size_t quads, uint32_t pos,
                      const saetta_token_params *params) {
    const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x; // 4 values each
    if (i >= quads) return;
    const float *src = blockIdx.y ? v : k;
    void *dst = blockIdx.y ? values : keys;
    const size_t first = size_t(params ? params->position : pos) * row_values / 4;
    const float4 x = reinterpret_cast<const float4 *>(src)[i];
    if (MODE == 2) {
        reinterpret_cast<float4 *>(dst)[first + i] = x;
    } else if (MODE == 0) {
        reinterpret_cast<uint2 *>(dst)[first + i] = make_uint2(pack_half2(x.x, x.y), pack_half2(x.z, x.w));
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
        reinterpret_cast<uint2 *>(dst)[first + i] =
            make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
    }
}

// bfloat16 -> binary16 copy of cache rows, 8 values per thread.  Exact for every
// value binary16 can hold (bfloat16 has the shorter significand); magnitudes
// past 65504 saturate instead of becoming infinite.
__global__ void __launch_bounds__(256)
bf16_to_f16_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, size_t octets) {
    const size_t o = size_t(blockIdx.x) * 256 + threadIdx.x;
    if (o >= octets) return;
    uint4 v = in[o];
    uint32_t *w = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a = fminf(fmaxf(__uint_as_float(w[i] << 16), -65504.f), 65504.f);
        const float b = fminf(fmaxf(__uint_as_float(w[i] & 0xffff0000u), -65504.f), 65504.f);
        w[i] = pack_half2(a, b);
    }
    out[o] = v;
}

int launch_bf16_to_f16(const void *in, void *out, size_t values, cudaStream_t stream) {
    const size_t octets = values / 8;
    if (!octets) return SAETTA_OK;
    bf16_to_f16_kernel<<<unsigned((octets + 255) / 256), 256, 0, stream>>>((const uint4 *)in, (uint4 *)out, octets);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

int launch_kv_store_plain(int mode, const float *k, const float *v, void *keys, void *values,
                          size_t row_values, size_t rows, size_t pos,
                          const saetta_token_params *params, cudaStream_t stream) {
    const size_t quads = rows * row_values / 4;
    if (!quads) return SAETTA_OK;
    dim3 grid(unsigned((quads + 255) / 256), 2);
    if (mode == 0)
        kv_store_plain_kernel<0><<<grid, 256, 0, stream>>>(k, v, keys, values, uint32_t(row_values), quads, uint32_t(pos), params);
    else if (mode == 1)
        kv_store_plain_kernel<1><<<grid, 256, 0, stream>>>(k, v, keys, values, uint32_t(row_values), quads, uint32_t(pos), params);
    else
        kv_store_plain_kernel<2><<<grid, 256, 0, stream>>>(k, v, keys, values, uint32_t(row_values), quads, uint32_t(pos), params);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

} // namespace saetta
