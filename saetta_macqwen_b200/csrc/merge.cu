// Log-sum-exp merge of split-KV partial results, with the output gate.
//
// Stands in for attention_reduce (kernels/attention.metal:367-409) and
// attention_reduce_rows (kernels/attention_rows.metal:296-342) of the
// reference: M = max m_p, l = sum l_p 2^(m_p - M), O = sum O_p 2^(m_p - M),
// out = O / l * sigmoid(gate).  Maxima are in log2 units.  Parts are added in
// index order, so the result does not depend on scheduling.
#include "host.hpp"

namespace saetta {

constexpr int kFragFloats = 2048;
constexpr int kPartKv = kFragFloats + 16;

size_t decode_quant_part_floats(size_t kv_heads) { return kv_heads * size_t(kPartKv); }

__device__ __forceinline__ float gate_of(float g) { return 1.0f / (1.0f + expf(-g)); }

// grid (8, rows * kv_heads): 256 fragment elements of one (row, kv head) per block.
__global__ void __launch_bounds__(256)
merge_frag_kernel(const float *__restrict__ parts, uint32_t nparts,
                  const uint32_t *__restrict__ first_part, uint32_t rows, uint32_t kv_heads,
                  const float *__restrict__ q_and_gate, float *__restrict__ out,
                  float *__restrict__ part_out) {
    const uint32_t row = blockIdx.y / kv_heads, kv = blockIdx.y % kv_heads;
    uint32_t p0 = 0, p1 = nparts;
    if (first_part) {
        p0 = first_part[row];
        p1 = first_part[row + 1];
    }
    const uint32_t prow = first_part ? 0 : row, prows = first_part ? 1 : rows;
    const uint32_t e = blockIdx.x * 256 + threadIdx.x; // fragment element
    const uint32_t r = e >> 5, lane = e & 31;
    const uint32_t head = 2 * (lane & 3) + (r & 1);
    const size_t stride = size_t(prows) * kv_heads * kPartKv;
    const float *base = parts + (size_t(prow) * kv_heads + kv) * kPartKv;

    float M = -INFINITY;
    for (uint32_t p = p0; p < p1; p++) M = fmaxf(M, base[p * stride + kFragFloats + head]);
    float acc = 0.f, l = 0.f;
#pragma unroll 4
    for (uint32_t p = p0; p < p1; p++) {
        const float *pp = base + p * stride;
        const float mp = pp[kFragFloats + head];
        if (mp == -INFINITY) continue;
        const float w = exp2f(mp - M);
        l = fmaf(pp[kFragFloats + 8 + head], w, l);
        acc = fmaf(pp[e], w, acc);
    }
    const uint32_t mt = r >> 2, c = r & 3;
    const uint32_t dim = 64 * (mt >> 2) + 8 * (lane >> 2) + (mt & 3) + (c >= 2 ? 4 : 0);
    const size_t rh = size_t(row) * kv_heads * kHeadsPerKv + kv * kHeadsPerKv + head;
    if (out) {
        const float g = q_and_gate[rh * 2 * kDim + kDim + dim];
        out[rh * kDim + dim] = acc / l * gate_of(g);
    } else {
        part_out[rh * kPartStride + dim] = acc;
        if (dim == 0) {
            part_out[rh * kPartStride + kPartM] = M;
            part_out[rh * kPartStride + kPartL] = l;
        }
    }
}

int launch_merge_frag(const float *parts, uint32_t nparts, const uint32_t *first_part,
                      uint32_t rows, uint32_t kv_heads, const float *q_and_gate, float *out,
                      float *part_out, cudaStream_t stream) {
    if (!rows) return SAETTA_OK;
    merge_frag_kernel<<<dim3(8, rows * kv_heads), 256, 0, stream>>>(parts, nparts, first_part, rows,
                                                                     kv_heads, q_and_gate, out, part_out);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

// grid (heads, rows), 256 threads = one per dim.
__global__ void __launch_bounds__(256)
merge_logical_kernel(const float *__restrict__ parts, uint32_t nparts, uint32_t rows,
                     uint32_t heads, const float *__restrict__ q_and_gate,
                     float *__restrict__ out, float *__restrict__ part_out) {
    const uint32_t head = blockIdx.x, row = blockIdx.y, dim = threadIdx.x;
    const size_t rh = size_t(row) * heads + head;
    const size_t stride = size_t(rows) * heads * kPartStride;
    const float *base = parts + rh * kPartStride;
    float M = -INFINITY;
    for (uint32_t p = 0; p < nparts; p++) M = fmaxf(M, base[p * stride + kPartM]);
    float acc = 0.f, l = 0.f;
#pragma unroll 4
    for (uint32_t p = 0; p < nparts; p++) {
        const float *pp = base + p * stride;
        const float mp = pp[kPartM];
        if (mp == -INFINITY) continue;
        const float w = exp2f(mp - M);
        l = fmaf(pp[kPartL], w, l);
        acc = fmaf(pp[dim], w, acc);
    }
    if (out) {
        const float g = q_and_gate[rh * 2 * kDim + kDim + dim];
        out[rh * kDim + dim] = acc / l * gate_of(g);
    } else {
        part_out[rh * kPartStride + dim] = acc;
        if (dim == 0) {
            part_out[rh * kPartStride + kPartM] = M;
            part_out[rh * kPartStride + kPartL] = l;
        }
    }
}

int launch_merge_logical(const float *parts, uint32_t nparts, uint32_t rows, uint32_t heads,
                         const float *q_and_gate, float *out, float *part_out,
                         cudaStream_t stream) {
    if (!rows) return SAETTA_OK;
    merge_logical_kernel<<<dim3(heads, rows), 256, 0, stream>>>(parts, nparts, rows, heads, q_and_gate,
                                                                out, part_out);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

} // namespace saetta
