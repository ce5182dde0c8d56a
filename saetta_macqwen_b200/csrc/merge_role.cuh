// The log-sum-exp merge of split-KV partials as a ROLE inside the decode kernels.
//
// Stands in for attention_reduce (kernels/attention.metal:367-409) and
// attention_reduce_rows (kernels/attention_rows.metal:296-342) of the reference,
// which are separate dispatches there.  Here a decode launch carries, after its
// split-KV CTAs, a few merge CTAs (higher block indices, so the hardware hands
// them out only after every split-KV CTA of the launch has been handed out).
// Each split-KV CTA, once its partial is in memory, fences and adds one to a
// ticket word; the merge CTAs wait (bounded) until the ticket shows every part,
// then each reduces its own slices of the fragment elements over all parts, in
// part order, and applies the gate -- or leaves the merged (O, m, l), or stores
// it into the peers' mailboxes.  One launch per layer instead of two: the kernel
// boundary between partial and merge, and the merge's own launch, are gone, and
// the next layer's CTAs move onto the SMs the split-KV CTAs leave while the
// merge CTAs still work.
//
// The partials are laid out for the merge, not for the writer: slice-major,
// [row][kv head][slice of 128 fragment elements][part][128], then the maxima and
// sums [row][kv head][part][m[8], l[8]].  A merge CTA's input -- one slice of
// every part -- is then ONE contiguous range, which a single bulk (TMA engine)
// copy brings into shared memory at several times the rate of per-thread loads
// (measured: 27 128-bit loads per thread of 16 CTAs took 5.8 us, their SMs'
// load/store units being the limit at about 40 GB/s each).
//
// Waiting is safe because the waited-for CTAs are already resident or done; the
// wait is bounded all the same and raises kStatusMergeTimeout instead of hanging.
#pragma once

#include "host.hpp"

namespace saetta {

constexpr int kFragFloats = 2048;         // 8 heads x 256 dims of one (row, kv head) in MMA-fragment order
constexpr int kPartKv = kFragFloats + 16; // + m[8] (log2 units), l[8]
constexpr int kSliceFloats = 128;         // fragment elements of one slice
constexpr int kSlices = kFragFloats / kSliceFloats; // 16 per (row, kv head)
constexpr int kMergeRoleMaxParts = 160;   // parts a merge CTA has room for
constexpr uint32_t kStatusMergeTimeout = 8u;
// Words of an op's status block: [0] status bits, [kTicketWord + pass] parts finished, [kDoneWord + pass] merge CTAs finished,
// [kAllDoneWord] merge CTAs of all passes finished.
constexpr int kTicketWord = 8, kDoneWord = 16, kAllDoneWord = 24, kStatusWords = 32;
// shared memory of a merge CTA: two slice buffers, m/l of every part, the weights, the (m, l) of the warps, the warps' sums, 3 barriers
constexpr int kMergeRoleSmem = 2 * kMergeRoleMaxParts * kSliceFloats * 4 + kMergeRoleMaxParts * 16 * 4 +
                               kMergeRoleMaxParts * 8 * 4 + (12 * 16 + 16) * 4 + 384 * 16 + 32;

// Merge CTAs per pass for `rows` query rows per pass; each takes rows * 2 * 16 / this many slices of one (row, kv head).
// (one slice per merge CTA for one row, two for more: 32, 32, 64 CTAs for 1, 2, 4 rows per pass)
__host__ __device__ inline uint32_t merge_role_ctas(uint32_t rows_per_pass) { return rows_per_pass == 4 ? 64u : 32u; }

// Where the split-KV CTA `part` of `nparts` puts fragment element e of (row, kv head) of its partial
// (rows = m), and its maxima and sums.  `sliced`: the layout above; else [part][row][kv head][kPartKv]
// (what merge.cu's kernel reads: the ragged batch).
struct PartWriter {
    float *o;          // fragment register fr (32 lanes) at reg(fr) + lane
    float *ml;         // m[8], l[8]
    size_t sub_stride; // floats between consecutive slices of this part
    __host__ __device__ float *reg(int fr) const {
        constexpr int kRegsPerSlice = kSliceFloats / 32;
        return o + size_t(fr / kRegsPerSlice) * sub_stride + (fr % kRegsPerSlice) * 32;
    }
};
__host__ __device__ inline PartWriter part_writer(float *parts, bool sliced, uint32_t nparts, uint32_t m, uint32_t row,
                                                   uint32_t kv, uint32_t part) {
    PartWriter w;
    if (sliced) {
        const size_t rk = size_t(row) * 2 + kv;
        w.o = parts + (rk * kSlices * nparts + part) * kSliceFloats;
        w.sub_stride = size_t(nparts) * kSliceFloats;
        w.ml = parts + size_t(m) * 2 * kFragFloats * nparts + (rk * nparts + part) * 16;
    } else {
        w.o = parts + ((size_t(part) * m + row) * 2 + kv) * kPartKv;
        w.sub_stride = kSliceFloats;
        w.ml = w.o + kFragFloats;
    }
    return w;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Polls one mailbox word (a float and the number of the exchange it belongs to, written by one 64-bit
// store) until it carries exchange number `seq`; false after about a second.
__device__ __forceinline__ bool mailbox_poll(const unsigned long long *p, uint32_t seq, float &v) {
    unsigned long long t0 = 0;
    for (uint32_t n = 0;; n++) {
        unsigned long long w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if (uint32_t(w >> 32) == seq) {
            v = __uint_as_float(uint32_t(w));
            return true;
        }
        if ((n & 63) == 63) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (!t0) t0 = t;
            else if (t - t0 > 1000000000ull) return false;
        }
    }
}

// What a split-KV CTA does once all of its partial has been written: the threads that wrote meet at a
// barrier, then ONE of them calls this -- a gpu-scope fence (cumulative: it orders the writes of the
// other threads too, which the barrier made visible to this one) and the ticket.
__device__ __forceinline__ void ticket_arrive(uint32_t *words, uint32_t pass) {
    __threadfence();
    atomicAdd(words + kTicketWord + pass, 1u);
}

// Merge CTA `idx` of `mo.n_merge` of pass `pass` (query rows row0 .. row0 + rows_pass - 1 of m).
// parts: the sliced layout; THREADS = 384 threads; smem: kMergeRoleSmem bytes, 128-byte aligned.
//
// Every step here is a short chain of latencies on an otherwise idle SM (measured in isolation: a
// first version with one warp per head for the weights, a rolled loop over the parts and one warp for
// the last sums took 5.4 us from the ticket to the result, of which the copies were 0.3), so each is
// spread over all twelve warps, its loads are issued together, and nothing is done twice.
template <int THREADS>
__device__ __forceinline__ void merge_role(const float *__restrict__ parts, uint32_t nparts, uint32_t m, uint32_t row0,
                                           uint32_t rows_pass, const MergeOut &mo, uint32_t *words, uint32_t pass,
                                           uint32_t idx, uint8_t *smem) {
    static_assert(THREADS == 384 && kSliceFloats == 128, "twelve warps; a slice is one float4 per lane");
    constexpr int NW = THREADS / 32;                                    // warps = thread groups the parts are dealt to
    constexpr int KP = (kMergeRoleMaxParts + NW - 1) / NW;              // parts per warp and slice, at most
    constexpr int KM = (kMergeRoleMaxParts + THREADS / 8 - 1) / (THREADS / 8); // parts per thread for the weights, at most
    float *buf = reinterpret_cast<float *>(smem);                       // [2][parts][128]
    float *ml_s = buf + 2 * kMergeRoleMaxParts * kSliceFloats;          // [parts][m[8], l[8]]
    float4 *w_t = reinterpret_cast<float4 *>(ml_s + kMergeRoleMaxParts * 16); // [head & 1][part]: weights of heads hb, 2+hb, 4+hb, 6+hb
    float *comb = reinterpret_cast<float *>(w_t + 2 * kMergeRoleMaxParts);    // [warp][head][m, l]; then L [8] at comb + 192
    float4 *red = reinterpret_cast<float4 *>(comb + NW * 16 + 16);      // [warp][slot]
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + NW * 32);       // slice buffer 0, 1, m/l
    __shared__ uint32_t s_ok;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // this CTA's slices: `cnt` (1 or 2) consecutive ones of one (row, kv head)
    const uint32_t cnt = rows_pass * 2u * kSlices / mo.n_merge;
    const uint32_t unit0 = idx * cnt;
    const uint32_t row = row0 + unit0 / (2u * kSlices), kv = (unit0 / kSlices) & 1u, sub0 = unit0 % kSlices;
    const bool live_row = row < m;
    const size_t rk = size_t(live_row ? row : 0) * 2 + kv;
    const float *o_base = parts + (rk * kSlices * nparts) * kSliceFloats; // + sub * nparts * 128
    const float *ml_base = parts + size_t(m) * 2 * kFragFloats * nparts + rk * nparts * 16;

    if (tid == 0) {
        mbar_init(&bars[0], 1), mbar_init(&bars[1], 1), mbar_init(&bars[2], 1);
        s_ok = 0; // 1: every part is in, 2: the wait for the parts gave up
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait(); // the gate, and whoever still reads `out`, belong to the launches before
    const uint32_t xseq = mo.push.world ? *mo.push.seq_done + 1 : 0; // the exchange this launch publishes

    // Output element of thread t < 128 of slice `sub`: float c of float4 slot t / 4.  Fragment register
    // r = sub * 4 + slot / 8 holds, in lane 4 * (slot & 7) + c, head 2c + (r & 1) at dim:
    auto out_of = [&](uint32_t sub, uint32_t &head, uint32_t &dim) {
        const uint32_t slot = tid >> 2, c = tid & 3;
        const uint32_t r = sub * 4 + (slot >> 3), mt = r >> 2, cc = r & 3;
        head = 2 * c + (r & 1);
        dim = 64 * (mt >> 2) + 8 * (slot & 7) + (mt & 3) + (cc >= 2 ? 4 : 0);
    };
    float gate[2] = {0.f, 0.f};
    if (tid < 128 && live_row && mo.out) { // asked for now, needed at the very end
        for (uint32_t i = 0; i < cnt && i < 2; i++) {
            uint32_t head, dim;
            out_of(sub0 + i, head, dim);
            gate[i] = mo.q_and_gate[((size_t(row) * 2 + kv) * kHeadsPerKv + head) * 2 * kDim + kDim + dim];
        }
    }

    // Lane 0 of every warp polls the ticket (twelve loads in flight instead of one: the ticket is seen a
    // round trip to L2 earlier on average); the first to see it issues the copies.
    if (lane == 0) {
        bool ok = false;
        unsigned long long t0 = 0;
        for (uint32_t n = 0;; n++) {
            if (*reinterpret_cast<volatile uint32_t *>(&s_ok) != 0u) break; // another warp saw it (or gave up)
            uint32_t v;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(words + kTicketWord + pass) : "memory");
            if (v >= nparts) { ok = true; break; }
            if ((n & 15) == 15) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                if (!t0) t0 = t;
                else if (t - t0 > 1000000000ull) break; // one second
            }
        }
        if (ok) {
            __threadfence(); // acquire: what the ticket holders wrote before their tickets is visible from here on
            if (atomicCAS(&s_ok, 0u, 1u) == 0u && live_row) {
                // The partials were written through the generic proxy by other SMs; the copies read them
                // through the async proxy.
                asm volatile("fence.proxy.async;" ::: "memory");
                mbar_expect_tx(&bars[2], nparts * 64);
                bulk_g2s(ml_s, ml_base, nparts * 64, &bars[2]);
                for (uint32_t i = 0; i < cnt; i++) {
                    mbar_expect_tx(&bars[i], nparts * kSliceFloats * 4);
                    bulk_g2s(buf + i * kMergeRoleMaxParts * kSliceFloats, o_base + size_t(sub0 + i) * nparts * kSliceFloats,
                             nparts * kSliceFloats * 4, &bars[i]);
                }
            }
        } else if (*reinterpret_cast<volatile uint32_t *>(&s_ok) == 0u) {
            if (atomicCAS(&s_ok, 0u, 2u) == 0u) atomicOr(words, kStatusMergeTimeout); // gave up: nothing is merged
        }
    }
    __syncthreads();
    volatile uint32_t never = 0; // these waits end when the copies land; nothing aborts them
    if (s_ok == 1 && live_row) {
        // ---- weights.  Thread t: head t & 7, parts t / 8, t / 8 + 48, ...; (m, l) pairs are combined in a
        // fixed order: within the thread, across the four lanes of a head, across the warps.
        bool landed = mbar_wait(&bars[2], 0, &never, 2000000u);
        const uint32_t h = tid & 7, j = tid >> 3;
        float mp[KM], lp[KM];
#pragma unroll
        for (int k = 0; k < KM; k++) {
            const uint32_t p = j + k * (THREADS / 8);
            mp[k] = p < nparts ? ml_s[p * 16 + h] : -INFINITY;
            lp[k] = p < nparts ? ml_s[p * 16 + 8 + h] : 0.f;
        }
        // pass 1: the maximum per head -- over the thread's parts, the four lanes of the head, the warps
        float mx = mp[0];
#pragma unroll
        for (int k = 1; k < KM; k++) mx = fmaxf(mx, mp[k]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        if (lane < 8) comb[warp * 8 + h] = mx;
        __syncthreads();
        float M = comb[h];
#pragma unroll
        for (int w = 1; w < NW; w++) M = fmaxf(M, comb[w * 8 + h]);
        // pass 2: the weights 2^(m_p - M) and the sum of l_p times them, added up in the same fixed order
        float wk[KM], lsum = 0.f;
#pragma unroll
        for (int k = 0; k < KM; k++) {
            wk[k] = mp[k] == -INFINITY ? 0.f : exp2f(mp[k] - M);
            lsum = fmaf(lp[k], wk[k], lsum);
            const uint32_t p = j + k * (THREADS / 8);
            if (p < nparts) reinterpret_cast<float *>(w_t + (h & 1) * kMergeRoleMaxParts + p)[h >> 1] = wk[k];
        }
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 8);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 16);
        if (lane < 8) comb[NW * 8 + warp * 8 + h] = lsum;
        __syncthreads();
        if (tid < 8) {
            float L = comb[NW * 8 + h];
#pragma unroll
            for (int w = 1; w < NW; w++) L += comb[NW * 8 + w * 8 + h];
            comb[NW * 16 + h] = L, comb[NW * 16 + 8 + h] = M;
        }
        // (the sums L are first read by the output threads, after the barrier that follows the first slice)
        // ---- the slices: warp g adds up parts g, g + 12, ... of float4 slot `lane`; then 128 threads add the warps
        for (uint32_t i = 0; i < cnt; i++) {
            const uint32_t sub = sub0 + i;
            const uint32_t hb = (lane >> 3) & 1; // register r = sub * 4 + lane / 8 holds heads 2c + (r & 1)
            landed = mbar_wait(&bars[i & 1], 0, &never, 2000000u) && landed;
            const float4 *src = reinterpret_cast<const float4 *>(buf + (i & 1) * kMergeRoleMaxParts * kSliceFloats) + lane;
            const float4 *wsrc = w_t + hb * kMergeRoleMaxParts;
            float4 v[KP], wv[KP];
#pragma unroll
            for (int k = 0; k < KP; k++) {
                const uint32_t p = warp + k * NW;
                v[k] = p < nparts ? src[p * 32] : make_float4(0.f, 0.f, 0.f, 0.f);
                wv[k] = p < nparts ? wsrc[p] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < KP; k++)
                acc.x = fmaf(v[k].x, wv[k].x, acc.x), acc.y = fmaf(v[k].y, wv[k].y, acc.y),
                acc.z = fmaf(v[k].z, wv[k].z, acc.z), acc.w = fmaf(v[k].w, wv[k].w, acc.w);
            red[warp * 32 + lane] = acc;
            __syncthreads();
            if (tid < 128) {
                const float *rp = reinterpret_cast<const float *>(red) + tid;
                float part[NW];
#pragma unroll
                for (int g = 0; g < NW; g++) part[g] = rp[g * 128];
                float sum = part[0];
#pragma unroll
                for (int g = 1; g < NW; g++) sum += part[g];
                uint32_t head, dim;
                out_of(sub, head, dim);
                const size_t rh = (size_t(row) * 2 + kv) * kHeadsPerKv + head;
                const float l = comb[NW * 16 + head], Mh = comb[NW * 16 + 8 + head];
                if (!mo.push.world) {
                    if (mo.out) {
                        mo.out[rh * kDim + dim] = sum / l * (1.0f / (1.0f + expf(-gate[i & 1])));
                    } else {
                        mo.part_out[rh * kPartStride + dim] = sum;
                        if (dim == 0) mo.part_out[rh * kPartStride + kPartM] = Mh, mo.part_out[rh * kPartStride + kPartL] = l;
                    }
                } else {
                    // Straight into this rank's place in every rank's mailbox (plain stores over NVLink).
                    // Every word carries the exchange number: the reader needs no flag and this kernel no
                    // fence.  A launch that also collects keeps its own values in registers.
                    const bool collect = mo.out != nullptr;
                    const size_t at = (size_t(xseq & 1) * mo.push.world + mo.push.rank) * mo.push.slot_floats + rh * kPartStride;
                    for (uint32_t pr = 0; pr < mo.push.world; pr++) {
                        if (collect && pr == mo.push.rank) continue;
                        unsigned long long *dst = mo.push.parts[pr] + at;
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + dim), "l"(peer_word(sum, xseq)) : "memory");
                        if (dim == 0) {
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartM), "l"(peer_word(Mh, xseq)) : "memory");
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + kPartL), "l"(peer_word(l, xseq)) : "memory");
                        }
                    }
                    if (collect) {
                        // ... and the peers' values of the same element out of this rank's own mailbox, as
                        // they land; then the merge over the ranks, in rank order, and the gate.
                        const unsigned long long *mine = mo.push.parts[mo.push.rank] + size_t(xseq & 1) * mo.push.world * mo.push.slot_floats + rh * kPartStride;
                        float o_r[kMaxPeers], m_r[kMaxPeers], l_r[kMaxPeers];
                        bool ok = true;
#pragma unroll
                        for (uint32_t pr = 0; pr < kMaxPeers; pr++) {
                            o_r[pr] = sum, m_r[pr] = Mh, l_r[pr] = l;
                            if (pr < mo.push.world && pr != mo.push.rank && ok) {
                                const unsigned long long *src = mine + size_t(pr) * mo.push.slot_floats;
                                ok = mailbox_poll(src + kPartM, xseq, m_r[pr]) && mailbox_poll(src + kPartL, xseq, l_r[pr]) &&
                                     mailbox_poll(src + dim, xseq, o_r[pr]);
                            }
                        }
                        if (!ok) {
                            atomicOr(mo.push.status, kStatusFullTimeout); // a peer never published: `out` stays as it is
                        } else {
                            float Mx = -INFINITY;
#pragma unroll
                            for (uint32_t pr = 0; pr < kMaxPeers; pr++)
                                if (pr < mo.push.world) Mx = fmaxf(Mx, m_r[pr]);
                            float acc = 0.f, lt = 0.f;
#pragma unroll
                            for (uint32_t pr = 0; pr < kMaxPeers; pr++) {
                                if (pr >= mo.push.world || m_r[pr] == -INFINITY) continue;
                                const float w = exp2f(m_r[pr] - Mx);
                                lt = fmaf(l_r[pr], w, lt);
                                acc = fmaf(o_r[pr], w, acc);
                            }
                            mo.out[rh * kDim + dim] = acc / lt * (1.0f / (1.0f + expf(-gate[i & 1])));
                        }
                    }
                }
            }
            if (i + 1 < cnt) __syncthreads(); // `red` is free again
        }
        if (!landed && tid == 0) atomicOr(words, kStatusMergeTimeout);
    }
    // The last merge CTA of the pass to finish clears the pass's two counters for the next launch (which
    // touches them only after its own dependency wait, i.e. after this grid has completed); the last of
    // the whole launch moves the exchange numbers on -- only then, so that every merge CTA of the
    // launch has read them before they change.
    __syncthreads();
    if (tid == 0) {
        if (atomicAdd(words + kDoneWord + pass, 1u) == mo.n_merge - 1) {
            words[kTicketWord + pass] = 0;
            words[kDoneWord + pass] = 0;
        }
        if (mo.push.world && atomicAdd(words + kAllDoneWord, 1u) == mo.n_merge * mo.passes - 1) {
            words[kAllDoneWord] = 0;
            *mo.push.seq_sent = xseq;
            if (mo.out) *mo.push.seq_done = xseq; // this launch collected too
        }
    }
}
#endif

} // namespace saetta
