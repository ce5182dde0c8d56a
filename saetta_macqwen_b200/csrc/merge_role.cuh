// The log-sum-exp merge of split-KV partials as a ROLE inside the decode kernels.
//
// Stands in for attention_reduce (kernels/attention.metal:367-409) and
// attention_reduce_rows (kernels/attention_rows.metal:296-342) of the reference,
// which are separate dispatches there.  Here a decode launch carries, after its
// split-KV CTAs, a few merge CTAs (higher block indices, so the hardware hands
// them out only after every split-KV CTA of the launch has been handed out).
// Each split-KV CTA, once its partial is in memory, fences and adds one to a
// ticket word; the merge CTAs wait (bounded) until the ticket shows every part,
// then each reduces its own slice of the fragment elements over all parts, in
// part order, and applies the gate -- or leaves the merged (O, m, l), or stores
// it into the peers' mailboxes.  One launch per layer instead of two: the kernel
// boundary between partial and merge, and the merge's own launch, are gone, and
// the next layer's CTAs move onto the SMs the split-KV CTAs leave while the
// merge CTAs still work.
//
// Waiting is safe because the waited-for CTAs are already resident or done; the
// wait is bounded all the same and raises kStatusMergeTimeout instead of hanging.
#pragma once

#include "host.hpp"

namespace saetta {

constexpr int kFragFloats = 2048;         // 8 heads x 256 dims of one (row, kv head) in MMA-fragment order
constexpr int kPartKv = kFragFloats + 16; // + m[8] (log2 units), l[8]
constexpr int kMergeRoleMaxParts = 160;   // parts one merge CTA stages m and l of
constexpr uint32_t kStatusMergeTimeout = 8u;
// Words of an op's status block: [0] status bits, [kTicketWord + pass] parts finished, [kDoneWord + pass] merge CTAs finished.
constexpr int kTicketWord = 8, kDoneWord = 16, kStatusWords = 32;
constexpr int kMergeRoleSmem = 2 * kMergeRoleMaxParts * 8 * 4 + 64 + 5 * 128 * 16;

// Merge CTAs per pass for `rows` query rows per pass: 64 or 128 float4 slots of one (row, kv head) each.
__host__ __device__ inline uint32_t merge_role_ctas(uint32_t rows_per_pass) { return rows_per_pass == 1 ? 16u : 32u; }

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// What a split-KV CTA does once all of its partial has been written: the threads that wrote meet at a
// barrier, then ONE of them calls this -- a gpu-scope fence (cumulative: it orders the writes of the
// other threads too, which the barrier made visible to this one) and the ticket.
__device__ __forceinline__ void ticket_arrive(uint32_t *words, uint32_t pass) {
    __threadfence();
    atomicAdd(words + kTicketWord + pass, 1u);
}

// Merge CTA `idx` of `mo.n_merge` of pass `pass` (query rows row0 .. row0 + rows_pass - 1 of m).
// parts [nparts][m][2][kPartKv]; THREADS threads; smem: kMergeRoleSmem bytes.
template <int THREADS>
__device__ __forceinline__ void merge_role(const float *__restrict__ parts, uint32_t nparts, uint32_t m, uint32_t row0,
                                           uint32_t rows_pass, const MergeOut &mo, uint32_t *words, uint32_t pass,
                                           uint32_t idx, uint8_t *smem) {
    constexpr int KB = 27; // loads in flight per thread and round
    float(*w_s)[8] = reinterpret_cast<float(*)[8]>(smem);               // m, then the weight 2^(m_p - M)
    float(*l_s)[8] = w_s + kMergeRoleMaxParts;
    float *M_s = reinterpret_cast<float *>(l_s + kMergeRoleMaxParts);   // [8], then L [8]
    float4 *red = reinterpret_cast<float4 *>(M_s + 16);                 // [part group - 1][slot]
    __shared__ uint32_t s_ok;

    const uint32_t tid = threadIdx.x;
    const uint32_t S = rows_pass * 2u * 512u / mo.n_merge; // float4 slots of this CTA: 64 or 128, inside one (row, kv)
    const uint32_t PG = THREADS / S;                       // thread groups the parts are dealt to
    const uint32_t sl = tid % S, pg = tid / S;
    const uint32_t unit = idx * S + sl;
    const uint32_t row = row0 + unit / 1024u, kv = (unit >> 9) & 1u, slot = unit & 511u;
    const bool live = row < m && pg < PG;
    const uint32_t r = slot >> 3; // fragment register index of the slot's four elements (lanes 4*(slot&7) ..+3)
    const uint32_t mt = r >> 2, cc = r & 3;
    const uint32_t dim = 64 * (mt >> 2) + 8 * (slot & 7) + (mt & 3) + (cc >= 2 ? 4 : 0);
    const size_t rh0 = (size_t(row) * 2 + kv) * kHeadsPerKv + (r & 1); // + 2c: the head of element c

    pdl_launch_dependents();
    pdl_wait(); // the gate, and whoever still reads `out`, belong to the launches before
    float gate[4] = {0.f, 0.f, 0.f, 0.f};
    if (live && pg == 0 && mo.out) {
#pragma unroll
        for (int c = 0; c < 4; c++) gate[c] = mo.q_and_gate[(rh0 + 2 * c) * 2 * kDim + kDim + dim];
    }
    const uint32_t xseq = mo.push.world ? *mo.push.seq_done + 1 : 0; // the exchange this launch publishes

    if (tid == 0) {
        bool ok = false;
        unsigned long long t0 = 0;
        for (uint32_t n = 0;; n++) {
            if (ld_acquire_u32(words + kTicketWord + pass) >= nparts) { ok = true; break; }
            if ((n & 15) == 15) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                if (!t0) t0 = t;
                else if (t - t0 > 1000000000ull) break; // one second
            }
            __nanosleep(40);
        }
        if (!ok) atomicOr(words, kStatusMergeTimeout);
        s_ok = ok ? 1u : 0u;
    }
    __syncthreads();
    if (s_ok) {
        const size_t stride = size_t(m) * 2 * kPartKv;
        const float *base = parts + (size_t(row < m ? row : 0) * 2 + kv) * kPartKv;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 v[KB];
#pragma unroll
        for (int k = 0; k < KB; k++) {
            const uint32_t p = pg + k * PG;
            v[k] = live && p < nparts ? __ldcg(reinterpret_cast<const float4 *>(base + p * stride) + slot) : zero;
        }
        {   // m and l of every part: all of a thread's loads in one round
            constexpr int KM = (kMergeRoleMaxParts * 16 + THREADS - 1) / THREADS;
            float ml[KM];
#pragma unroll
            for (int k = 0; k < KM; k++) {
                const uint32_t x = tid + k * THREADS;
                ml[k] = x < nparts * 16 ? __ldcg(base + (x >> 4) * stride + kFragFloats + (x & 15)) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < KM; k++) {
                const uint32_t x = tid + k * THREADS;
                if (x < nparts * 16) {
                    if ((x & 15) < 8) w_s[x >> 4][x & 7] = ml[k]; else l_s[x >> 4][x & 7] = ml[k];
                }
            }
        }
        __syncthreads();
        if (tid < 256) { // warp h reduces head h
            const uint32_t h = tid >> 5, ln = tid & 31;
            float mx = -INFINITY;
            for (uint32_t p = ln; p < nparts; p += 32) mx = fmaxf(mx, w_s[p][h]);
#pragma unroll
            for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float lsum = 0.f;
            for (uint32_t p = ln; p < nparts; p += 32) {
                const float mp = w_s[p][h];
                const float w = mp == -INFINITY ? 0.f : exp2f(mp - mx);
                w_s[p][h] = w;
                lsum += l_s[p][h] * w;
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
            if (ln == 0) M_s[h] = mx, M_s[8 + h] = lsum;
        }
        __syncthreads();
        float4 acc = zero;
        const uint32_t hb = r & 1;
        for (uint32_t k0 = 0;; k0 += KB) {
#pragma unroll
            for (int k = 0; k < KB; k++) {
                const uint32_t p = pg + (k0 + k) * PG;
                if (p < nparts) {
                    acc.x = fmaf(v[k].x, w_s[p][hb], acc.x), acc.y = fmaf(v[k].y, w_s[p][2 + hb], acc.y);
                    acc.z = fmaf(v[k].z, w_s[p][4 + hb], acc.z), acc.w = fmaf(v[k].w, w_s[p][6 + hb], acc.w);
                }
            }
            if (pg + (k0 + KB) * PG >= nparts) break; // (uniform per thread group; no barrier inside)
#pragma unroll
            for (int k = 0; k < KB; k++) {
                const uint32_t p = pg + (k0 + KB + k) * PG;
                v[k] = live && p < nparts ? __ldcg(reinterpret_cast<const float4 *>(base + p * stride) + slot) : zero;
            }
        }
        if (pg >= 1 && pg < PG) red[(pg - 1) * S + sl] = acc;
        __syncthreads();
        if (live && pg == 0) {
            for (uint32_t k = 1; k < PG; k++) {
                const float4 o = red[(k - 1) * S + sl];
                acc.x += o.x, acc.y += o.y, acc.z += o.z, acc.w += o.w;
            }
            const float sum[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const size_t rh = rh0 + 2 * c;
                const float M = M_s[2 * c + hb], l = M_s[8 + 2 * c + hb];
                if (mo.out) {
                    mo.out[rh * kDim + dim] = sum[c] / l * (1.0f / (1.0f + expf(-gate[c])));
                } else if (!mo.push.world) {
                    mo.part_out[rh * kPartStride + dim] = sum[c];
                    if (dim == 0) mo.part_out[rh * kPartStride + kPartM] = M, mo.part_out[rh * kPartStride + kPartL] = l;
                } else {
                    // Straight into this rank's place in every rank's mailbox (plain stores over NVLink, this
                    // rank's own copy included).  Every word carries the exchange number: the reader needs
                    // no flag and this kernel no fence.
                    const size_t at = (size_t(xseq & 1) * mo.push.world + mo.push.rank) * mo.push.slot_floats + rh * kPartStride;
                    for (uint32_t pr = 0; pr < mo.push.world; pr++) {
                        unsigned long long *dst = mo.push.parts[pr] + at;
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + dim), "l"(peer_word(sum[c], xseq)) : "memory");
                        if (dim == 0) {
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartM), "l"(peer_word(M, xseq)) : "memory");
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartL), "l"(peer_word(l, xseq)) : "memory");
                        }
                    }
                }
            }
        }
        if (mo.push.world && idx == 0 && pass == 0 && tid == 0) *mo.push.seq_sent = xseq; // read by the collecting kernel only
    }
    // The last merge CTA of the pass to finish clears the two counters for the next launch (which
    // touches them only after its own dependency wait, i.e. after this grid has completed).
    __syncthreads();
    if (tid == 0) {
        if (atomicAdd(words + kDoneWord + pass, 1u) == mo.n_merge - 1) {
            words[kTicketWord + pass] = 0;
            words[kDoneWord + pass] = 0;
        }
    }
}
#endif

} // namespace saetta
