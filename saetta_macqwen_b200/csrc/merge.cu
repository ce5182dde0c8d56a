// Log-sum-exp merge of split-KV partial results, with the output gate.
//
// Stands in for attention_reduce (kernels/attention.metal:367-409) and
// attention_reduce_rows (kernels/attention_rows.metal:296-342) of the
// reference: M = max m_p, l = sum l_p 2^(m_p - M), O = sum O_p 2^(m_p - M),
// out = O / l * sigmoid(gate).  Maxima are in log2 units.  Parts are added in
// index order, so the result does not depend on scheduling.
#include "merge_role.cuh"

namespace saetta {

size_t decode_quant_part_floats(size_t kv_heads) { return kv_heads * size_t(kPartKv); }

__device__ __forceinline__ float gate_of(float g) { return 1.0f / (1.0f + expf(-g)); }

// grid (32, rows * kv_heads), 1024 threads: 64 fragment elements of one (row, kv
// head) per block, the parts dealt round-robin to 16 thread groups, and every thread's loads
// issued together (the merge is latency-bound, not bandwidth-bound).  Sums are formed in a
// fixed order.
constexpr int kMergeGroups = 16;
constexpr int kMergeElems = 64;
constexpr int kMergeMaxParts = 512; // m and l of at most this many parts are staged in shared memory

__global__ void __launch_bounds__(kMergeGroups * kMergeElems)
merge_frag_kernel(const float *__restrict__ parts, uint32_t nparts,
                  const uint32_t *__restrict__ first_part, uint32_t rows, uint32_t kv_heads,
                  const float *__restrict__ q_and_gate, float *__restrict__ out,
                  float *__restrict__ part_out, const PeerPush push) {
    __shared__ float w_s[kMergeMaxParts][8]; // first m, then the weight 2^(m_p - M), per part and head
    __shared__ float l_s[kMergeMaxParts][8];
    __shared__ float M_s[8], L_s[8];
    __shared__ float red[kMergeGroups][kMergeElems];
    const uint32_t row = blockIdx.y / kv_heads, kv = blockIdx.y % kv_heads;
    pdl_wait(); // the partials come from the kernel before
    pdl_launch_dependents();
    const uint32_t xseq = push.world ? *push.seq_done + 1 : 0; // the exchange this launch publishes
    uint32_t p0 = 0, p1 = nparts;
    if (first_part) {
        p0 = first_part[row];
        p1 = first_part[row + 1];
    }
    const uint32_t prow = first_part ? 0 : row, prows = first_part ? 1 : rows;
    const size_t stride = size_t(prows) * kv_heads * kPartKv;
    const float *base = parts + (size_t(prow) * kv_heads + kv) * kPartKv;
    const uint32_t tid = threadIdx.x, grp = tid / kMergeElems, el = tid % kMergeElems;
    const uint32_t e = blockIdx.x * kMergeElems + el; // fragment element
    const uint32_t r = e >> 5, lane = e & 31;
    const uint32_t head = 2 * (lane & 3) + (r & 1);

    // The merge is a chain of latencies (the parts sit in L2), so every thread asks for all it needs at once:
    // its first kMergeBatch values before the weights are formed, the m / l words in one round.
    constexpr int kMergeBatch = 12; // x 16 groups = 192 parts per round: one round for a decode over all SMs
    float acc = 0.f;
    if (tid < 8) M_s[tid] = -INFINITY, L_s[tid] = 0.f; // what a row without parts (an empty shard) merges to
    for (uint32_t c0 = p0; c0 < p1; c0 += kMergeMaxParts) { // one pass unless a sequence has > 512 parts
        const uint32_t n = min(p1 - c0, uint32_t(kMergeMaxParts));
        float v[kMergeBatch];
#pragma unroll
        for (int k = 0; k < kMergeBatch; k++) {
            const uint32_t p = grp + k * kMergeGroups;
            v[k] = p < n ? base[(c0 + p) * stride + e] : 0.f;
        }
        __syncthreads();
        for (uint32_t xb = tid; xb < n * 16; xb += 4 * blockDim.x) {
            float ml[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t x = xb + k * blockDim.x;
                ml[k] = x < n * 16 ? base[(c0 + (x >> 4)) * stride + kFragFloats + (x & 15)] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t x = xb + k * blockDim.x, p = x >> 4, j = x & 15;
                if (x < n * 16) {
                    if (j < 8) w_s[p][j] = ml[k]; else l_s[p][j - 8] = ml[k];
                }
            }
        }
        __syncthreads();
        if (tid < 256) { // warp h reduces head h
            const uint32_t h = tid >> 5, ln = tid & 31;
            float mx = -INFINITY;
            for (uint32_t p = ln; p < n; p += 32) mx = fmaxf(mx, w_s[p][h]);
#pragma unroll
            for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float Mold = c0 == p0 ? -INFINITY : M_s[h];
            const float Mnew = fmaxf(Mold, mx);
            float lsum = 0.f;
            for (uint32_t p = ln; p < n; p += 32) {
                const float mp = w_s[p][h];
                const float w = mp == -INFINITY ? 0.f : exp2f(mp - Mnew);
                w_s[p][h] = w;
                lsum += l_s[p][h] * w;
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
            if (ln == 0) {
                const float carry = Mold == -INFINITY ? 0.f : exp2f(Mold - Mnew);
                L_s[h] = (c0 == p0 ? 0.f : L_s[h] * carry) + lsum;
                M_s[h] = Mnew;
                red[0][h] = carry;     // reuse: the rescale of what was accumulated so far
            }
        }
        __syncthreads();
        if (c0 != p0) acc *= red[0][head];
        __syncthreads();
        float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < kMergeBatch; k++) {
            const uint32_t p = grp + k * kMergeGroups;
            if (p < n) a4[k & 3] = fmaf(v[k], w_s[p][head], a4[k & 3]);
        }
        for (uint32_t pb = grp + kMergeBatch * kMergeGroups; pb < n; pb += kMergeBatch * kMergeGroups) { // > 192 parts
#pragma unroll
            for (int k = 0; k < kMergeBatch; k++) {
                const uint32_t p = pb + k * kMergeGroups;
                v[k] = p < n ? base[(c0 + p) * stride + e] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < kMergeBatch; k++) {
                const uint32_t p = pb + k * kMergeGroups;
                if (p < n) a4[k & 3] = fmaf(v[k], w_s[p][head], a4[k & 3]);
            }
        }
        acc += (a4[0] + a4[1]) + (a4[2] + a4[3]);
    }
    __syncthreads();
    red[grp][el] = acc;
    __syncthreads();
    if (grp) return;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kMergeGroups; k++) sum += red[k][el];
    const float M = M_s[head], l = L_s[head];
    const uint32_t mt = r >> 2, c = r & 3;
    const uint32_t dim = 64 * (mt >> 2) + 8 * (lane >> 2) + (mt & 3) + (c >= 2 ? 4 : 0);
    const size_t rh = size_t(row) * kv_heads * kHeadsPerKv + kv * kHeadsPerKv + head;
    if (out) {
        const float g = q_and_gate[rh * 2 * kDim + kDim + dim];
        out[rh * kDim + dim] = sum / l * gate_of(g);
    } else if (!push.world) {
        part_out[rh * kPartStride + dim] = sum;
        if (dim == 0) {
            part_out[rh * kPartStride + kPartM] = M;
            part_out[rh * kPartStride + kPartL] = l;
        }
    } else {
        // Straight into this rank's place in every rank's mailbox (remote stores over NVLink, this
        // rank's own copy included).  Every word carries the exchange number, so the reader needs no
        // flag and this kernel no fence: a word is there once its number is.
        const size_t at = (size_t(xseq & 1) * push.world + push.rank) * push.slot_floats + rh * kPartStride;
        for (uint32_t r = 0; r < push.world; r++) {
            unsigned long long *dst = push.parts[r] + at;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + dim), "l"(peer_word(sum, xseq)) : "memory");
            if (dim == 0) {
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartM), "l"(peer_word(M, xseq)) : "memory");
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartL), "l"(peer_word(l, xseq)) : "memory");
            }
        }
        if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) *push.seq_sent = xseq; // read by the collecting kernel only
    }
}

int launch_merge_frag(const float *parts, uint32_t nparts, const uint32_t *first_part,
                      uint32_t rows, uint32_t kv_heads, const float *q_and_gate, float *out,
                      float *part_out, cudaStream_t stream, const PeerPush *push) {
    if (!rows) return SAETTA_OK;
    PeerPush none = {};
    SAETTA_CUDA(launch_pdl(merge_frag_kernel, dim3(kFragFloats / kMergeElems, rows * kv_heads),
                           dim3(kMergeGroups * kMergeElems), 0, stream, parts, nparts, first_part, rows, kv_heads,
                           q_and_gate, out, part_out, push ? *push : none));
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
