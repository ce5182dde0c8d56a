// Split-KV decode / MTP-verify attention over the 8- and 4-bit KV cache.
//
// Stands in for attention_partial_mma_q<8|4> (kernels/attention.metal:242-360)
// and attention_partial_rows<8|4> (kernels/attention_rows.metal:108-292) of the
// reference; the merge over parts is in merge.cu.  The design is this file's
// own and is shaped by HBM bandwidth:
//
//  * One persistent CTA per SM owns a contiguous range of 32-token tiles.  A
//    producer warp streams each tile -- key codes, value codes and the four
//    scale/bias arrays, six contiguous spans covering BOTH kv heads -- into a
//    ring of shared-memory stages with bulk (TMA engine) copies signalled on
//    mbarriers, so every cache byte crosses HBM once and many tiles are in
//    flight per SM.
//  * Eight consumer warps each own one kv head, one query row (decode) or two
//    (MTP verify), and a share of the 16-token sub-tiles.  Codes go from shared
//    memory to registers with 128/64-bit loads and are turned into binary16 MMA
//    fragments with byte permutes (code c becomes the half 1024+c, minus 1024:
//    exact), so a code is dequantised once for all eight query heads of its kv
//    head -- and, with several rows, for two rows.
//  * One row: the score MMA's 16 rows are the heads' query halves (hi, lo: f32
//    precision), the value MMA is O^T[dim][head] += V^T P^T (16 dims per
//    instruction).  Two rows: the 16 rows are the two rows' heads in both
//    products, the value MMA is O[head][dim] += P V (8 dims per instruction),
//    and the query fragments sit in shared memory to leave registers for the
//    128 accumulators.  Either way the score fragment's layout is the layout
//    the value product needs: P never moves between lanes.
//  * Scores are accumulated per 64-value group and only then multiplied by the
//    group's scale: x = s*c + z is applied exactly as s*(q.c) + z*sum(q), in f32.
//  * Online softmax per warp with shuffles; the running maximum is only moved
//    when it grows by more than 2^8 (the accumulators stay in range and are
//    rarely rescaled).  P is multiplied by the value scales before the product;
//    the value biases ride along as one more MMA.
//  * Every wait on an mbarrier is bounded; a wait that gives up sets a bit in
//    the status word, raises the CTA's abort flag and the CTA drains and leaves.
#include <algorithm>

#include <mutex>

#include "merge_role.cuh"

namespace saetta {

constexpr int kTile = 32;     // tokens per stage
constexpr int kSub = 16;      // tokens per MMA sub-tile
constexpr int kWarps = 8;     // consumer warps
constexpr int kThreads = (kWarps + 4) * 32; // two consumer warpgroups + the producer's warpgroup
constexpr int kKv = 2;        // kv heads covered by one stage
constexpr float kLog2e = 1.4426950408889634f;
// Tiles of a CTA's range pulled into L2 before the dependency wait.  Measured 0 / 4 / 8 / 16: four is best
// (deeper prefetches queue ahead of the ring's own copies when the wait turns out to be short).
constexpr int kPrefetchTiles = 4;
constexpr float kRescale = 8.0f; // move the running maximum when it grows by more than 2^8

template <int BITS>
struct Stage {
    static constexpr int kCodeRow = kKv * kDim * BITS / 8; // bytes of codes per token, both kv heads
    static constexpr int kCodes = kTile * kCodeRow;
    static constexpr int kParamRow = kKv * kGroupsPerHead * 2; // 16 bytes per token
    static constexpr int kParams = kTile * kParamRow;
    static constexpr int kK = 0, kV = kCodes, kKs = 2 * kCodes, kKz = kKs + kParams,
                         kVs = kKz + kParams, kVz = kVs + kParams;
    static constexpr int kBytes = 2 * kCodes + 4 * kParams;
    static constexpr int kStages = BITS == 8 ? 5 : 8;
};

constexpr int kQFragBytes = 16 * 32 * 16;              // one set of query fragments: [group][k-step][lane] x 128 bit
constexpr int kQAuxBytes = 4 * 128 * 4;                // per set: code-offset terms and sums [row][group][head]
// One area with two users: the segment merge of batched one-row launches (one buffer per kv head),
// or the query fragments of row-pair launches (up to four sets).
constexpr int kMergeBytes = 4 * kQFragBytes;
static_assert(kMergeBytes >= kKv * kFragFloats * 4, "merge buffers fit");
template <int BITS>
constexpr int smem_bytes() {
    // (a launch's merge CTAs use the same allocation for their own buffers)
    return std::max(Stage<BITS>::kStages * Stage<BITS>::kBytes + kMergeBytes + kQAuxBytes + kWarps * 2 * 16 * 4 +
                        2 * Stage<BITS>::kStages * 8 + 32,
                    kMergeRoleSmem);
}

struct DecodeArgs {
    Segment seg;               // the one segment of a single-sequence launch (tiles filled on device)
    const Segment *segs;       // batched: descriptors, else null
    const uint32_t *cta_first; // batched: CTA c runs segs[cta_first[c] .. cta_first[c+1])
    const float *q;            // [rows][16][256]
    float *parts;              // [part][rows][kv][kPartKv]
    uint32_t *status;          // the op's status words (merge_role.cuh)
    const saetta_token_params *params;
    uint32_t m;        // query rows
    uint32_t row_step; // row r sees kv_len + r*row_step keys
    uint32_t capacity;
    uint32_t n_decode; // split-KV CTAs (= parts); blocks past them run the merge role
    MergeOut mo;
};

__device__ __forceinline__ uint32_t lop_and_or(uint32_t w, uint32_t mask, uint32_t magic) {
    return (w & mask) | magic;
}

// The dimension (within the thread's 16 of a group) that the B fragment of
// k-step j, register `reg`, element e pairs with; must mirror how the key codes
// are cut into A fragments below.
template <int BITS>
__device__ __forceinline__ constexpr int q_dim(int j, int reg, int e) {
    if (BITS == 8) return 4 * j + 2 * reg + e;          // bytes 4j..4j+3 of the 16
    return 8 * (j >> 1) + 2 * (j & 1) + reg + 4 * e;    // nibbles {n, n+4} of word j/2
}

template <int BITS, int ROWS>
__global__ void __launch_bounds__(kThreads, 1) decode_quant_kernel(const DecodeArgs a) {
    using St = Stage<BITS>;
    constexpr int NS = St::kStages;
    extern __shared__ __align__(128) uint8_t smem[];
    if (blockIdx.x >= a.n_decode) { // the blocks after the split-KV CTAs merge what those leave
        merge_role<kThreads>(a.parts, a.n_decode, a.m, blockIdx.y * ROWS, ROWS, a.mo, a.status, blockIdx.y,
                             blockIdx.x - a.n_decode, smem);
        return;
    }
    uint8_t *stages = smem;
    float *merge = reinterpret_cast<float *>(smem + NS * St::kBytes);
    float *qsums = merge + kMergeBytes / 4;
    float *ml = qsums + kQAuxBytes / 4; // [warp][row of the warp][m of 8 heads, l of 8 heads]
    uint64_t *full = reinterpret_cast<uint64_t *>(ml + kWarps * 2 * 16);
    uint64_t *empty = full + NS;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(empty + NS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        abort_flag[0] = 0;
        abort_flag[1] = 0; // a word that stays 0, for waits that must ignore the abort flag
        mbar_fence_init();
    }
    __syncthreads();

    // The tile range of a single-sequence launch's CTA for a given kv_len.
    auto tile_range = [&](uint32_t kv_len, uint32_t &tb, uint32_t &te) {
        const uint32_t longest = min(kv_len + (a.m - 1) * a.row_step, a.capacity);
        const uint32_t tiles = (longest + kTile - 1) / kTile;
        tb = uint32_t(uint64_t(blockIdx.x) * tiles / a.n_decode);
        te = uint32_t(uint64_t(blockIdx.x + 1) * tiles / a.n_decode);
    };
    auto issue_tile = [&](const Segment &s, uint32_t t, uint32_t st) { // one elected lane
        uint8_t *dst = stages + st * St::kBytes;
        mbar_expect_tx(&full[st], St::kBytes);
        const size_t tok = size_t(t) * kTile;
        bulk_g2s(dst + St::kK, (const uint8_t *)s.k + tok * St::kCodeRow, St::kCodes, &full[st]);
        bulk_g2s(dst + St::kV, (const uint8_t *)s.v + tok * St::kCodeRow, St::kCodes, &full[st]);
        bulk_g2s(dst + St::kKs, (const uint8_t *)s.ks + tok * St::kParamRow, St::kParams, &full[st]);
        bulk_g2s(dst + St::kKz, (const uint8_t *)s.kz + tok * St::kParamRow, St::kParams, &full[st]);
        bulk_g2s(dst + St::kVs, (const uint8_t *)s.vs + tok * St::kParamRow, St::kParams, &full[st]);
        bulk_g2s(dst + St::kVz, (const uint8_t *)s.vz + tok * St::kParamRow, St::kParams, &full[st]);
    };

    // While the launch before this one drains, pull the head of this CTA's tile range into L2 (and warm
    // the TLB).  The range comes from a possibly stale kv_len: it is only a hint, every value is read
    // again after the wait; L2 is the point of coherence, so lines brought in early still show what
    // the launch before writes afterwards.  (Filling the copy ring itself this early, or right after
    // the wait from the early kv_len, was measured and lost: in a chain of layers the copies compete
    // with the merge CTAs of the layer before, and the query conversion after the wait covers the
    // first tile's latency anyway.)
    if (warp == kWarps && lane == 0 && !a.segs) {
        const uint32_t kv_hint = *reinterpret_cast<const volatile uint32_t *>(&a.params->kv_len);
        uint32_t tb, te;
        tile_range(kv_hint, tb, te);
        const uint32_t nt = min(te - tb, uint32_t(kPrefetchTiles));
        const size_t tok = size_t(tb) * kTile;
        for (uint32_t t = 0; t < nt; t += 2) { // two tiles (32 KB of 8-bit codes) per request
            const uint32_t n = min(nt - t, 2u);
            l2_prefetch((const uint8_t *)a.seg.k + (tok + t * kTile) * St::kCodeRow, n * St::kCodes);
            l2_prefetch((const uint8_t *)a.seg.v + (tok + t * kTile) * St::kCodeRow, n * St::kCodes);
        }
        if (nt) {
            l2_prefetch((const uint8_t *)a.seg.ks + tok * St::kParamRow, nt * St::kParams);
            l2_prefetch((const uint8_t *)a.seg.kz + tok * St::kParamRow, nt * St::kParams);
            l2_prefetch((const uint8_t *)a.seg.vs + tok * St::kParamRow, nt * St::kParams);
            l2_prefetch((const uint8_t *)a.seg.vz + tok * St::kParamRow, nt * St::kParams);
        }
    }
    pdl_wait();              // q, the token parameters and the new rows of the cache may come from the launch before
    pdl_launch_dependents(); // the next launch's CTAs may take the SMs this grid's CTAs leave

    // The segments this CTA runs.
    uint32_t seg_lo = 0, seg_hi = 1;
    if (a.segs) {
        seg_lo = a.cta_first[blockIdx.x];
        seg_hi = a.cta_first[blockIdx.x + 1];
    }
    const uint32_t row0 = blockIdx.y * ROWS; // first query row of this pass

    auto load_segment = [&](uint32_t si) -> Segment {
        if (a.segs) return a.segs[si];
        Segment s = a.seg;
        const uint32_t kv_len = a.params->kv_len;
        tile_range(kv_len, s.tile_begin, s.tile_end);
        s.kv_len = kv_len;
        s.part = blockIdx.x;
        s.seq = 0;
        return s;
    };

    auto producer_role = [&]() {
        // ---------------------------------------------------------------- producer
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t si = seg_lo; si < seg_hi && ok; si++) {
            const Segment s = load_segment(si);
            for (uint32_t t = s.tile_begin; t < s.tile_end; t++, it++) {
                const uint32_t st = it % NS, round = it / NS;
                if (!mbar_wait(&empty[st], (round & 1) ^ 1, abort_flag)) {
                    if (lane == 0) {
                        atomicOr(a.status, kStatusEmptyTimeout);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                if (lane == 0) issue_tile(s, t, st);
                __syncwarp();
            }
        }
        // Leave only once every copy this warp issued has landed (bounded): the
        // shared memory must not be handed to another CTA with copies in flight.
        const uint32_t issued = it;
        for (uint32_t k = issued > NS ? issued - NS : 0; k < issued; k++)
            mbar_wait(&full[k % NS], (k / NS) & 1, abort_flag, 2000000u);
    };
    // Registers move from the producer's warpgroup (only one of its warps works, and it needs
    // few) to the two consumer warpgroups, whose accumulators and query fragments would
    // otherwise spill inside the inner loop.  What the consumers gain must be what the producers
    // gave up -- 128 x (168 - 40) = 256 x (232 - 168): the pool is the CTA's allocation at launch
    // (384 x 168), not the SM's register file, and an increase beyond it would block for good.
    // (Sixteen consumer warps at 112 registers, fragments in shared memory, were measured: 18 %
    // slower at 8 bits, no faster at 4.)
    if (warp >= kWarps) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == kWarps) producer_role();
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");

    // -------------------------------------------------------------------- consumers
    if constexpr (ROWS == 1) {
        constexpr int NSLOT = kWarps / kKv; // warps sharing one kv head
        const int kv = warp & 1;
        const int row_in_pass = (warp >> 1) % ROWS;
        const int slot = (warp >> 1) / ROWS;
        const uint32_t row = row0 + row_in_pass;
        const bool row_live = row < a.m;
        const int g = lane >> 2, i = lane & 3;
        constexpr uint32_t kMagic = 0x64646464u, k1024 = 0x64006400u, k64 = 0x54005400u;
        // Value codes are centred before the P V product: v = s*(c - C) + (z + C*s) with C = 128, or 7.5
        // for 4-bit.  For zero-mean values the two terms then no longer cancel, so the 16-bit rounding
        // of P costs 3x less relative error.  The 4-bit centre is the exact middle of the codes: with
        // C = 8 the centred codes average -0.5, both sums drift apart in proportion to the tokens a
        // warp has added up, and the tensor cores' truncating f32 adds turn that drift into an error
        // that does not shrink with the length (measured: 1.3e-3 relative at 28000 tokens per warp).
        // Every nibble rides on 64 (ulp 1/16, so 71.5 is exact): 1152 = 0x6480, 71.5 = 0x5478.
        constexpr uint32_t k1152 = 0x64806480u, k71_5 = 0x54785478u;
        constexpr float kVCentre = BITS == 8 ? 128.f : 7.5f;

        uint32_t it = 0;
        bool alive = true; // false once a wait gave up: skip the tiles, keep the barriers
        for (uint32_t si = seg_lo; si < seg_hi; si++) {
            // The query row is asked for before the token parameters are: with one sequence per launch its
            // address depends on neither, and the two round trips then overlap.
            const uint32_t seq = a.segs ? a.segs[si].seq : 0u;
            float4 qraw[4][4];
            {
                const float *qp = a.q + ((size_t(seq) * a.m + (row_live ? row : 0)) * 16 + kv * 8 + g) * kDim;
#pragma unroll
                for (int G = 0; G < 4; G++)
#pragma unroll
                    for (int c = 0; c < 4; c++) qraw[G][c] = *reinterpret_cast<const float4 *>(qp + G * 64 + i * 16 + c * 4);
            }
            const Segment s = load_segment(si);
            const uint32_t n_row = min(s.kv_len + row * a.row_step, a.capacity); // keys this row sees

            // Query fragments of head kv*8+g: 16 dims per group, scaled by log2(e)/16 and rounded to binary16
            // (the B operand of the score product, as in the several-row path); what the code offsets add to
            // q.c per group, for the two heads of this lane's score columns; the group sums for the bias term.
            uint32_t qh[4][8];
            uint32_t qzb = 0;
            float qoff2[4][2];
            {
                float qs[4];
#pragma unroll
                for (int G = 0; G < 4; G++) {
                    float x[16];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float4 v = qraw[G][c];
                        x[4 * c] = v.x, x[4 * c + 1] = v.y, x[4 * c + 2] = v.z, x[4 * c + 3] = v.w;
                    }
                    float hi[16], sum = 0.f, off = 0.f;
#pragma unroll
                    for (int d = 0; d < 16; d++) {
                        hi[d] = __half2float(__float2half_rn(x[d] * (kLog2e * 0.0625f)));
                        sum += hi[d];
                        // 8-bit: every code rides on 1024; 4-bit: even dims (low nibbles) on 1024, odd on 64
                        off += hi[d] * ((BITS == 4 && (d & 1)) ? 64.f : 1024.f);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const int d0 = q_dim<BITS>(j, r, 0), d1 = q_dim<BITS>(j, r, 1);
                            qh[G][2 * j + r] = pack_half2(hi[d0], hi[d1]);
                        }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    off += __shfl_xor_sync(0xffffffffu, off, 1);
                    off += __shfl_xor_sync(0xffffffffu, off, 2);
                    qs[G] = sum;
                    qoff2[G][0] = __shfl_sync(0xffffffffu, off, 8 * i), qoff2[G][1] = __shfl_sync(0xffffffffu, off, 8 * i + 4);
                }
                // B fragment of the bias-term MMA, column g = head g: k-slots 0..3 = the high halves of the
                // four group sums (lanes i = 0, 1 hold two each), k-slots 4..7 = their low halves (i = 2, 3).
                const float s0 = (i & 1) ? qs[2] : qs[0], s1 = (i & 1) ? qs[3] : qs[1];
                const float h0 = __half2float(__float2half_rn(s0)), h1 = __half2float(__float2half_rn(s1));
                qzb = i < 2 ? pack_half2(h0, h1) : pack_half2(s0 - h0, s1 - h1);
            }

            float O[16][4];
            float Ob[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < 16; e++) O[e][0] = O[e][1] = O[e][2] = O[e][3] = 0.f;
            float Mref = -INFINITY, lsum = 0.f; // of head g (this thread's row of the score MMA)

            for (uint32_t t = s.tile_begin; alive && t < s.tile_end; t++, it++) {
                const uint32_t st = it % NS, round = it / NS;
                if (!mbar_wait(&full[st], round & 1, abort_flag)) {
                    if (lane == 0) {
                        atomicOr(a.status, kStatusFullTimeout);
                        *abort_flag = 1;
                    }
                    alive = false;
                    break;
                }
                const uint8_t *sg = stages + st * St::kBytes;
#pragma unroll 1
                for (int sub = 0; sub < kTile / kSub; sub++) {
                    const uint32_t q_idx = 2 * (t - s.tile_begin) + sub;
                    const uint32_t tok0 = t * kTile + sub * kSub; // first token of the sub-tile
                    if (!row_live || (q_idx % NSLOT) != uint32_t(slot) || tok0 >= n_row) continue;
                    const bool partial = tok0 + kSub > n_row;
                    const int lt = sub * kSub; // token offset inside the stage

                    // ------------------------------------------------ scores S[token][head], then transposed
                    // One MMA row per token (16 of them), one column per query head, 16 dims per instruction:
                    // the key codes are the A operand (lane (g, i) feeds tokens g and g+8), the query the B
                    // operand.  Half the instructions of a product with the heads as rows, whose rows 8..15 had
                    // nothing better to hold than the queries' low halves.
                    float S[2][2];
                    {
                        const uint8_t *kc = sg + St::kK + kv * (kDim * BITS / 8);
                        const int tA = lt + g, tB = tA + 8;
                        const uint2 sKA = *reinterpret_cast<const uint2 *>(sg + St::kKs + tA * St::kParamRow + kv * 8);
                        const uint2 sKB = *reinterpret_cast<const uint2 *>(sg + St::kKs + tB * St::kParamRow + kv * 8);
                        const float2 sA[2] = {h2f2(sKA.x), h2f2(sKA.y)}, sB[2] = {h2f2(sKB.x), h2f2(sKB.y)};
                        float sc[4] = {0.f, 0.f, 0.f, 0.f}; // (token g | g+8) x (head 2i | 2i+1)
#pragma unroll
                        for (int G = 0; G < 4; G++) {
                            float acc[4] = {0.f, 0.f, 0.f, 0.f};
                            if (BITS == 8) {
                                const uint4 rA = *reinterpret_cast<const uint4 *>(kc + tA * St::kCodeRow + G * 64 + i * 16);
                                const uint4 rB = *reinterpret_cast<const uint4 *>(kc + tB * St::kCodeRow + G * 64 + i * 16);
                                const uint32_t wA[4] = {rA.x, rA.y, rA.z, rA.w}, wB[4] = {rB.x, rB.y, rB.z, rB.w};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    // operands stay 1024 + c; 1024 * sum(q) is taken off the group sum below
                                    mma_f16(acc, prmt(wA[j], kMagic, 0x4140), prmt(wB[j], kMagic, 0x4140), prmt(wA[j], kMagic, 0x4342),
                                            prmt(wB[j], kMagic, 0x4342), qh[G][2 * j], qh[G][2 * j + 1]);
                                }
                            } else {
                                const uint2 rA = *reinterpret_cast<const uint2 *>(kc + tA * St::kCodeRow + G * 32 + i * 8);
                                const uint2 rB = *reinterpret_cast<const uint2 *>(kc + tB * St::kCodeRow + G * 32 + i * 8);
                                const uint32_t wA[2] = {rA.x, rA.y}, wB[2] = {rB.x, rB.y};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    const uint32_t xA = wA[j >> 1] >> (8 * (j & 1)), xB = wB[j >> 1] >> (8 * (j & 1));
                                    // low nibbles ride on 1024, high nibbles on 64: (1024, 64) * the matching
                                    // partial sums of q come off below
                                    mma_f16(acc, lop_and_or(xA, 0x000f000fu, k1024), lop_and_or(xB, 0x000f000fu, k1024),
                                            lop_and_or(xA, 0x00f000f0u, k64), lop_and_or(xB, 0x00f000f0u, k64), qh[G][2 * j], qh[G][2 * j + 1]);
                                }
                            }
                            const float scA = G == 0 ? sA[0].x : G == 1 ? sA[0].y : G == 2 ? sA[1].x : sA[1].y;
                            const float scB = G == 0 ? sB[0].x : G == 1 ? sB[0].y : G == 2 ? sB[1].x : sB[1].y;
                            sc[0] = fmaf(scA, acc[0] - qoff2[G][0], sc[0]);
                            sc[1] = fmaf(scA, acc[1] - qoff2[G][1], sc[1]);
                            sc[2] = fmaf(scB, acc[2] - qoff2[G][0], sc[2]);
                            sc[3] = fmaf(scB, acc[3] - qoff2[G][1], sc[3]);
                        }
                        {   // bias term: sum_G z[token][G] * qsum[head][G]; k-slots 0..3 meet the sums' high halves,
                            // 4..7 (the same biases again) their low halves
                            float accz[4] = {0.f, 0.f, 0.f, 0.f};
                            const uint32_t zA = *reinterpret_cast<const uint32_t *>(sg + St::kKz + tA * St::kParamRow + kv * 8 + (i & 1) * 4);
                            const uint32_t zB = *reinterpret_cast<const uint32_t *>(sg + St::kKz + tB * St::kParamRow + kv * 8 + (i & 1) * 4);
                            mma_f16(accz, zA, zB, 0u, 0u, qzb, 0u);
                            sc[0] += accz[0], sc[1] += accz[1], sc[2] += accz[2], sc[3] += accz[3];
                        }
                        // To the layout the rest works in -- lane (g, i) owns head g at tokens 2i, 2i+1 of each
                        // 8-token half -- by transposing the 8x8 blocks of 16-bit halves across the warp.
#pragma unroll
                        for (int nt = 0; nt < 2; nt++) {
                            const uint32_t c0 = __float_as_uint(sc[2 * nt]), c1 = __float_as_uint(sc[2 * nt + 1]);
                            const uint32_t ylo = movmatrix_trans(prmt(c0, c1, 0x5410)), yhi = movmatrix_trans(prmt(c0, c1, 0x7632));
                            S[nt][0] = __uint_as_float(prmt(ylo, yhi, 0x5410));
                            S[nt][1] = __uint_as_float(prmt(ylo, yhi, 0x7632));
                            if (partial) {
                                if (tok0 + nt * 8 + 2 * i >= n_row) S[nt][0] = -INFINITY;
                                if (tok0 + nt * 8 + 2 * i + 1 >= n_row) S[nt][1] = -INFINITY;
                            }
                        }
                    }

                    // ------------------------------------------------ online softmax of head g (log2 units)
                    float mx = fmaxf(fmaxf(S[0][0], S[0][1]), fmaxf(S[1][0], S[1][1]));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const bool need = mx > Mref + kRescale;
                    if (__any_sync(0xffffffffu, need)) {
                        const float f = need ? exp2f(Mref - mx) : 1.f; // exp2f(-inf) = 0 on the first tile
                        if (need) Mref = mx, lsum *= f;
                        // the accumulators' columns are heads 2i, 2i+1: fetch their factors from lanes g = 2i, 2i+1
                        const float f0 = __shfl_sync(0xffffffffu, f, 8 * i), f1 = __shfl_sync(0xffffffffu, f, 8 * i + 4);
#pragma unroll
                        for (int e = 0; e < 16; e++) {
                            O[e][0] *= f0, O[e][1] *= f1, O[e][2] *= f0, O[e][3] *= f1;
                        }
                        Ob[0] *= f0, Ob[1] *= f1, Ob[2] *= f0, Ob[3] *= f1;
                    }
                    const float p00 = exp2f(S[0][0] - Mref), p01 = exp2f(S[0][1] - Mref);
                    const float p10 = exp2f(S[1][0] - Mref), p11 = exp2f(S[1][1] - Mref);
                    lsum += (p00 + p01) + (p10 + p11);

                    // ------------------------------------------------ P (x value scales) as B fragments
                    // B[k = token][n = head]: this lane's pairs (2i, 2i+1) and (8+2i, 9+2i) of head g are
                    // exactly its own score columns, so no data moves between lanes.
                    const int T0 = lt + 2 * i, T1 = T0 + 1, T2 = T0 + 8, T3 = T0 + 9;
                    uint2 sV[4];
                    sV[0] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T0 * St::kParamRow + kv * 8);
                    sV[1] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T1 * St::kParamRow + kv * 8);
                    sV[2] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T2 * St::kParamRow + kv * 8);
                    sV[3] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T3 * St::kParamRow + kv * 8);
                    if (partial) { // stale rows may hold anything: keep them out of 0 * x
                        if (tok0 + 2 * i >= n_row) sV[0] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 1 >= n_row) sV[1] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 8 >= n_row) sV[2] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 9 >= n_row) sV[3] = make_uint2(0u, 0u);
                    }
                    // P'[token][head] = P * value scale of (token, group): the two tokens of a pair have
                    // their own scales, gathered into one half2 by a byte permute
                    const uint32_t pu0 = pack_half2(p00, p01), pu1 = pack_half2(p10, p11);
                    uint32_t pbf[4][2];
                    {
                        float2 sf[4][2]; // [token of the lane's four][groups 0,1 | 2,3]
#pragma unroll
                        for (int k = 0; k < 4; k++) sf[k][0] = h2f2(sV[k].x), sf[k][1] = h2f2(sV[k].y);
#pragma unroll
                        for (int G = 0; G < 4; G++) {
                            const float a = (G & 1) ? sf[0][G >> 1].y : sf[0][G >> 1].x, b = (G & 1) ? sf[1][G >> 1].y : sf[1][G >> 1].x;
                            const float c = (G & 1) ? sf[2][G >> 1].y : sf[2][G >> 1].x, d = (G & 1) ? sf[3][G >> 1].y : sf[3][G >> 1].x;
                            pbf[G][0] = pack_half2(p00 * a, p01 * b); // f32 product, one rounding
                            pbf[G][1] = pack_half2(p10 * c, p11 * d);
                        }
                    }

                    // ------------------------------------------------ O^T[dim][head] += V^T P^T
                    {   // value biases: rows 0..3 of one more MMA hold sum_t P[t][h] (z + C s)[t][G]
                        const int gq = g & 3;
                        const uint8_t *vz = sg + St::kVz + kv * 8 + gq * 2;
                        uint32_t z0 = *reinterpret_cast<const uint16_t *>(vz + T0 * St::kParamRow);
                        uint32_t z1 = *reinterpret_cast<const uint16_t *>(vz + T1 * St::kParamRow);
                        uint32_t z2 = *reinterpret_cast<const uint16_t *>(vz + T2 * St::kParamRow);
                        uint32_t z3 = *reinterpret_cast<const uint16_t *>(vz + T3 * St::kParamRow);
                        if (partial) {
                            if (tok0 + 2 * i >= n_row) z0 = 0;
                            if (tok0 + 2 * i + 1 >= n_row) z1 = 0;
                            if (tok0 + 2 * i + 8 >= n_row) z2 = 0;
                            if (tok0 + 2 * i + 9 >= n_row) z3 = 0;
                        }
                        // this lane's group is gq: its scales sit in half gq of the pairs gathered above
                        const uint32_t sel = (gq & 1) ? 0x7632u : 0x5410u;
                        const uint32_t s01 = prmt(gq < 2 ? sV[0].x : sV[0].y, gq < 2 ? sV[1].x : sV[1].y, sel);
                        const uint32_t s23 = prmt(gq < 2 ? sV[2].x : sV[2].y, gq < 2 ? sV[3].x : sV[3].y, sel);
                        const uint32_t cc = pack_half2(kVCentre, kVCentre);
                        const uint32_t a0 = g < 4 ? hfma2_u32(s01, cc, z0 | z1 << 16) : 0u;
                        const uint32_t a2 = g < 4 ? hfma2_u32(s23, cc, z2 | z3 << 16) : 0u;
                        mma_f16(Ob, a0, 0u, a2, 0u, pu0, pu1);
                    }
                    const uint8_t *vc = sg + St::kV + kv * (kDim * BITS / 8);
#pragma unroll
                    for (int G = 0; G < 4; G++) {
                        if (BITS == 8) {
                            const uint2 t0 = *reinterpret_cast<const uint2 *>(vc + T0 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t1 = *reinterpret_cast<const uint2 *>(vc + T1 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t2 = *reinterpret_cast<const uint2 *>(vc + T2 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t3 = *reinterpret_cast<const uint2 *>(vc + T3 * St::kCodeRow + G * 64 + g * 8);
                            // [T0.b0 T1.b0 T0.b1 T1.b1] and [T0.b2 T1.b2 T0.b3 T1.b3], per dim row and token pair
                            const uint32_t x01[2] = {prmt(t0.x, t1.x, 0x5140), prmt(t0.x, t1.x, 0x7362)};
                            const uint32_t u01[2] = {prmt(t0.y, t1.y, 0x5140), prmt(t0.y, t1.y, 0x7362)};
                            const uint32_t x23[2] = {prmt(t2.x, t3.x, 0x5140), prmt(t2.x, t3.x, 0x7362)};
                            const uint32_t u23[2] = {prmt(t2.y, t3.y, 0x5140), prmt(t2.y, t3.y, 0x7362)};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const uint32_t sel = (e & 1) ? 0x4342u : 0x4140u;
                                // 1024 + c minus 1152: the centred code c - 128 (see kVCentre)
                                const uint32_t a0 = hsub2_u32(prmt(x01[e >> 1], kMagic, sel), k1152);
                                const uint32_t a1 = hsub2_u32(prmt(u01[e >> 1], kMagic, sel), k1152);
                                const uint32_t a2 = hsub2_u32(prmt(x23[e >> 1], kMagic, sel), k1152);
                                const uint32_t a3 = hsub2_u32(prmt(u23[e >> 1], kMagic, sel), k1152);
                                mma_f16(O[4 * G + e], a0, a1, a2, a3, pbf[G][0], pbf[G][1]);
                            }
                        } else {
                            const uint32_t t0 = *reinterpret_cast<const uint32_t *>(vc + T0 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t1 = *reinterpret_cast<const uint32_t *>(vc + T1 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t2 = *reinterpret_cast<const uint32_t *>(vc + T2 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t3 = *reinterpret_cast<const uint32_t *>(vc + T3 * St::kCodeRow + G * 32 + g * 4);
                            // low half-word: T0's nibbles 0..3 (dim row g), high: T1's; .y side: nibbles 4..7 (row g+8)
                            const uint32_t x01 = prmt(t0, t1, 0x5410), u01 = prmt(t0, t1, 0x7632);
                            const uint32_t x23 = prmt(t2, t3, 0x5410), u23 = prmt(t2, t3, 0x7632);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                // nibble e of each half-word into bits 4..7 of its byte: 64 + n, minus 71.5
                                auto code = [&](uint32_t w) {
                                    const uint32_t x = e == 0 ? w << 4 : e == 1 ? w : e == 2 ? w >> 4 : w >> 8;
                                    return hsub2_u32(lop_and_or(x, 0x00f000f0u, k64), k71_5);
                                };
                                mma_f16(O[4 * G + e], code(x01), code(u01), code(x23), code(u23), pbf[G][0], pbf[G][1]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }

            // ---------------------------------------------------------------- end of segment
            // l of head g over the four lanes that share it; then every lane takes m and l of the
            // heads of its accumulator columns (2i, 2i+1) from lanes g = 2i and g = 2i+1.
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            float Mc2[2], l[2];
            Mc2[0] = __shfl_sync(0xffffffffu, Mref, 8 * i), Mc2[1] = __shfl_sync(0xffffffffu, Mref, 8 * i + 4);
            l[0] = __shfl_sync(0xffffffffu, lsum, 8 * i), l[1] = __shfl_sync(0xffffffffu, lsum, 8 * i + 4);
#pragma unroll
            for (int G = 0; G < 4; G++) {
                const float b0 = __shfl_sync(0xffffffffu, Ob[0], 4 * G + i);
                const float b1 = __shfl_sync(0xffffffffu, Ob[1], 4 * G + i);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    O[4 * G + e][0] += b0, O[4 * G + e][1] += b1;
                    O[4 * G + e][2] += b0, O[4 * G + e][3] += b1;
                }
            }
            // where this part's fragment register r (32 lanes) and its maxima and sums go
            const PartWriter pw = part_writer(a.parts, a.mo.n_merge != 0, a.n_decode, a.m, row_live ? row : 0, kv, s.part);
            auto dst_reg = [&](int r) { return pw.reg(r) + lane; };
            if (NSLOT == 1) {
                if (row_live) {
#pragma unroll
                    for (int e = 0; e < 16; e++)
#pragma unroll
                        for (int c = 0; c < 4; c++) *dst_reg(4 * e + c) = O[e][c];
                    if (g == 0) {
                        pw.ml[2 * i] = Mc2[0], pw.ml[2 * i + 1] = Mc2[1];
                        pw.ml[8 + 2 * i] = l[0], pw.ml[8 + 2 * i + 1] = l[1];
                    }
                }
            } else {
                // Warps that share a (kv, row) agree on one maximum, scale, and add up
                // in a fixed order through shared memory (deterministic).
                if (g == 0) {
                    ml[warp * 16 + 2 * i] = Mc2[0], ml[warp * 16 + 2 * i + 1] = Mc2[1];
                    ml[warp * 16 + 8 + 2 * i] = l[0], ml[warp * 16 + 8 + 2 * i + 1] = l[1];
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
                float Mc[2] = {-INFINITY, -INFINITY}, lc[2] = {0.f, 0.f};
#pragma unroll
                for (int sl = 0; sl < NSLOT; sl++) {
                    const int w = ((sl * ROWS + row_in_pass) << 1) | kv;
                    Mc[0] = fmaxf(Mc[0], ml[w * 16 + 2 * i]);
                    Mc[1] = fmaxf(Mc[1], ml[w * 16 + 2 * i + 1]);
                }
#pragma unroll
                for (int sl = 0; sl < NSLOT; sl++) {
                    const int w = ((sl * ROWS + row_in_pass) << 1) | kv;
                    const float m0 = ml[w * 16 + 2 * i], m1 = ml[w * 16 + 2 * i + 1];
                    lc[0] += m0 == -INFINITY ? 0.f : ml[w * 16 + 8 + 2 * i] * exp2f(m0 - Mc[0]);
                    lc[1] += m1 == -INFINITY ? 0.f : ml[w * 16 + 8 + 2 * i + 1] * exp2f(m1 - Mc[1]);
                }
                const float f0 = Mc2[0] == -INFINITY ? 0.f : exp2f(Mc2[0] - Mc[0]);
                const float f1 = Mc2[1] == -INFINITY ? 0.f : exp2f(Mc2[1] - Mc[1]);
                if (!a.segs) {
                    // One segment per launch: after the barrier above no warp reads the copy ring any
                    // more, so every warp parks its scaled accumulators in the ring at once; then each
                    // warp adds up its share of the elements in slot order (fixed, hence deterministic).
                    float *mine = reinterpret_cast<float *>(stages) + warp * kFragFloats;
#pragma unroll
                    for (int e = 0; e < 16; e++)
#pragma unroll
                        for (int c = 0; c < 4; c++) mine[(4 * e + c) * 32 + lane] = O[e][c] * ((c & 1) ? f1 : f0);
                    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
                    if (row_live) {
                        constexpr int per = 64 / NSLOT;
#pragma unroll
                        for (int r = 0; r < per; r++) {
                            float v = 0.f;
#pragma unroll
                            for (int sl = 0; sl < NSLOT; sl++) {
                                const int w = ((sl * ROWS + row_in_pass) << 1) | kv;
                                v += reinterpret_cast<const float *>(stages)[w * kFragFloats + (slot * per + r) * 32 + lane];
                            }
                            *dst_reg(slot * per + r) = v;
                        }
                        if (slot == 0 && g == 0) {
                            pw.ml[2 * i] = Mc[0], pw.ml[2 * i + 1] = Mc[1];
                            pw.ml[8 + 2 * i] = lc[0], pw.ml[8 + 2 * i + 1] = lc[1];
                        }
                    }
                } else {
                float *buf = merge + (row_in_pass * kKv + kv) * kFragFloats;
#pragma unroll 1
                for (int sl = 0; sl < NSLOT; sl++) {
                    if (sl == slot) {
#pragma unroll
                        for (int e = 0; e < 16; e++)
#pragma unroll
                            for (int c = 0; c < 4; c++) {
                                const float v = O[e][c] * ((c & 1) ? f1 : f0);
                                float *p = buf + (4 * e + c) * 32 + lane;
                                *p = sl ? *p + v : v;
                            }
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
                }
                if (row_live) {
                    constexpr int per = 64 / NSLOT;
#pragma unroll
                    for (int r = 0; r < per; r++) *dst_reg(slot * per + r) = buf[(slot * per + r) * 32 + lane];
                    if (slot == 0 && g == 0) {
                        pw.ml[2 * i] = Mc[0], pw.ml[2 * i + 1] = Mc[1];
                        pw.ml[8 + 2 * i] = lc[0], pw.ml[8 + 2 * i + 1] = lc[1];
                    }
                }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); // merge buffers free again
            }
        }
        // The partial is written: tell the merge CTAs of this launch (the writers meet, then one
        // of them fences and takes the ticket).
        if (a.mo.n_merge) {
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            if (threadIdx.x == 0) ticket_arrive(a.status, blockIdx.y);
        }
    } else {
        // Several query rows (MTP verify): a warp owns one kv head and two query rows.  The 16 rows
        // of every MMA are the 8 heads of the kv head for the first row, then for the second, so the
        // two rows share every dequantised fragment; keys and values are the B operands (8 tokens /
        // 8 dims per instruction) and P is the A operand of the value product.  Queries are rounded
        // to 16 bits here (one row keeps a low half instead).
        constexpr int NR = 2;
        constexpr int NP = ROWS / NR;                 // row groups per pass
        constexpr int NSLOT = kWarps / (kKv * NP);    // warps sharing one (kv, row group)
        constexpr int GP = 4 / NSLOT;                 // groups whose query fragments one warp prepares
        static_assert(NSLOT == 2 || NSLOT == 4, "two or four warps per (kv head, row group)");
        static_assert(kKv * NP * kQFragBytes <= kMergeBytes, "query fragments fit");
        const int kv = warp & 1;
        const int pair = (warp >> 1) % NP;
        const int slot = (warp >> 1) / NP;
        const int combo = pair * kKv + kv;
        const uint32_t rowA = row0 + pair * NR;       // first query row of this warp
        const int g = lane >> 2, i = lane & 3;
        // Query fragments live in shared memory, one 128-bit A operand per (group, k-step, lane), in
        // the area one-row launches use as their merge buffer.
        uint4 *qf = reinterpret_cast<uint4 *>(merge) + combo * 512;
        float *qaux = qsums + combo * 128; // off[r][G][head], sum[r][G][head]
        constexpr uint32_t kMagic = 0x64646464u, k1024 = 0x64006400u, k64 = 0x54005400u;
        // Value codes are centred before the P V product: v = s*(c - C) + (z + C*s) with C = 128, or 7.5
        // for 4-bit.  For zero-mean values the two terms then no longer cancel, so the 16-bit rounding
        // of P costs 3x less relative error.  The 4-bit centre is the exact middle of the codes: with
        // C = 8 the centred codes average -0.5, both sums drift apart in proportion to the tokens a
        // warp has added up, and the tensor cores' truncating f32 adds turn that drift into an error
        // that does not shrink with the length (measured: 1.3e-3 relative at 28000 tokens per warp).
        // Every nibble rides on 64 (ulp 1/16, so 71.5 is exact): 1152 = 0x6480, 71.5 = 0x5478.
        constexpr uint32_t k1152 = 0x64806480u, k71_5 = 0x54785478u;
        constexpr float kVCentre = BITS == 8 ? 128.f : 7.5f;

        uint32_t it = 0;
        bool alive = true; // false once a wait gave up: skip the tiles, keep the barriers
        for (uint32_t si = seg_lo; si < seg_hi; si++) {
            const Segment s = load_segment(si);
            uint32_t n_row[NR];      // keys each of the warp's rows sees (0 for a row past m)
            uint32_t n_any = 0, n_all = 0xffffffffu;
#pragma unroll
            for (int r = 0; r < NR; r++) {
                n_row[r] = rowA + r < a.m ? min(s.kv_len + (rowA + r) * a.row_step, a.capacity) : 0u;
                n_any = max(n_any, n_row[r]);
                if (rowA + r < a.m) n_all = min(n_all, n_row[r]);
            }

            // ------------------------------------------------ query fragments
            // Head kv*8+g, 16 dims per lane and group, scaled by log2(e)/16.  The warps that share the
            // set split the groups between them.
#pragma unroll
            for (int gi = 0; gi < GP; gi++) {
                const int G = slot * GP + gi;
                uint32_t fa[8], fb[8]; // MMA rows g and g+8
#pragma unroll
                for (int r = 0; r < NR; r++) {
                    const uint32_t qrow = rowA + r < a.m ? rowA + r : 0;
                    const float *qp = a.q + ((size_t(s.seq) * a.m + qrow) * 16 + kv * 8 + g) * kDim + G * 64 + i * 16;
                    float x[16];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float4 v = *reinterpret_cast<const float4 *>(qp + c * 4);
                        x[4 * c] = v.x, x[4 * c + 1] = v.y, x[4 * c + 2] = v.z, x[4 * c + 3] = v.w;
                    }
                    float hi[16], sum = 0.f, off = 0.f;
#pragma unroll
                    for (int d = 0; d < 16; d++) {
                        x[d] *= kLog2e * 0.0625f;
                        hi[d] = __half2float(__float2half_rn(x[d]));
                        sum += hi[d];
                        // 8-bit: every code rides on 1024; 4-bit: even dims (low nibbles) on 1024, odd on 64
                        off += hi[d] * ((BITS == 4 && (d & 1)) ? 64.f : 1024.f);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int w = 0; w < 2; w++) {
                            const int d0 = q_dim<BITS>(j, w, 0), d1 = q_dim<BITS>(j, w, 1);
                            if (r == 0) fa[2 * j + w] = pack_half2(hi[d0], hi[d1]);
                            else fb[2 * j + w] = pack_half2(hi[d0], hi[d1]);
                        }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    off += __shfl_xor_sync(0xffffffffu, off, 1);
                    off += __shfl_xor_sync(0xffffffffu, off, 2);
                    if (i == 0) qaux[(r * 4 + G) * 8 + g] = off, qaux[64 + (r * 4 + G) * 8 + g] = sum;
                }
#pragma unroll
                for (int j = 0; j < 4; j++)
                    qf[(G * 4 + j) * 32 + lane] = make_uint4(fa[2 * j], fb[2 * j], fa[2 * j + 1], fb[2 * j + 1]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            float qoff[NR][4]; // per row and group: what the code offsets (1024; 64 for high nibbles) add to q.c
#pragma unroll
            for (int r = 0; r < NR; r++)
#pragma unroll
                for (int G = 0; G < 4; G++) qoff[r][G] = qaux[(r * 4 + G) * 8 + g];
            // A fragment of the bias-term MMA: k-slots 0..3 = groups (lanes i < 2 hold two each); row g =
            // the first row's group sums (high halves), row g+8 = their low halves or the second row's sums.
            uint32_t qza0 = 0, qza1 = 0;
            if (i < 2) {
                const float s0 = qaux[64 + (2 * i) * 8 + g], s1 = qaux[64 + (2 * i + 1) * 8 + g];
                const float h0 = __half2float(__float2half_rn(s0)), h1 = __half2float(__float2half_rn(s1));
                qza0 = pack_half2(h0, h1);
                qza1 = pack_half2(qaux[64 + (4 + 2 * i) * 8 + g], qaux[64 + (4 + 2 * i + 1) * 8 + g]);
            }

            // O[n-tile (group G, byte e)][c]: c0, c1 = MMA row g (dims G*64 + (2i | 2i+1)*8 + e), c2, c3 = row g+8.
            float O[32][4];
            float Ob[4] = {0.f, 0.f, 0.f, 0.f}; // sum_t P (z + C s): columns 2i, 2i+1 = groups (lanes i < 2)
            float Mref[NR], lsum[NR];           // of head g, per query row
#pragma unroll
            for (int e = 0; e < 32; e++) O[e][0] = O[e][1] = O[e][2] = O[e][3] = 0.f;
#pragma unroll
            for (int r = 0; r < NR; r++) Mref[r] = -INFINITY, lsum[r] = 0.f;

            for (uint32_t t = s.tile_begin; alive && t < s.tile_end; t++, it++) {
                const uint32_t st = it % NS, round = it / NS;
                if (!mbar_wait(&full[st], round & 1, abort_flag)) {
                    if (lane == 0) {
                        atomicOr(a.status, kStatusFullTimeout);
                        *abort_flag = 1;
                    }
                    alive = false;
                    break;
                }
                const uint8_t *sg = stages + st * St::kBytes;
#pragma unroll 1
                for (int sub = 0; sub < kTile / kSub; sub++) {
                    const uint32_t q_idx = 2 * (t - s.tile_begin) + sub;
                    const uint32_t tok0 = t * kTile + sub * kSub; // first token of the sub-tile
                    if ((q_idx % NSLOT) != uint32_t(slot) || tok0 >= n_any) continue;
                    const bool partial = tok0 + kSub > n_all;
                    const int lt = sub * kSub; // token offset inside the stage

                    // ------------------------------------------------ scores S[head][token]
                    // Columns = 8 tokens per n-tile nt.  Lane (g, i) feeds token g of each n-tile and owns
                    // head g (both MMA rows) at tokens 2i, 2i+1.
                    float S[NR][2][2];
                    {
                        const uint8_t *kc = sg + St::kK + kv * (kDim * BITS / 8);
                        float2 sKf[2][2][2]; // [nt][token 2i | 2i+1][groups 0,1 | 2,3]
#pragma unroll
                        for (int nt = 0; nt < 2; nt++)
#pragma unroll
                            for (int c = 0; c < 2; c++) {
                                const uint2 v = *reinterpret_cast<const uint2 *>(sg + St::kKs + (lt + nt * 8 + 2 * i + c) * St::kParamRow + kv * 8);
                                sKf[nt][c][0] = h2f2(v.x), sKf[nt][c][1] = h2f2(v.y);
                            }
                        float sc[NR][2][2];
#pragma unroll
                        for (int r = 0; r < NR; r++) sc[r][0][0] = sc[r][0][1] = sc[r][1][0] = sc[r][1][1] = 0.f;
#pragma unroll
                        for (int G = 0; G < 4; G++) {
                            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                            uint32_t w[2][4];
#pragma unroll
                            for (int nt = 0; nt < 2; nt++) {
                                const int trow = lt + nt * 8 + g; // token this lane loads
                                if (BITS == 8) {
                                    const uint4 rr = *reinterpret_cast<const uint4 *>(kc + trow * St::kCodeRow + G * 64 + i * 16);
                                    w[nt][0] = rr.x, w[nt][1] = rr.y, w[nt][2] = rr.z, w[nt][3] = rr.w;
                                } else {
                                    const uint2 rr = *reinterpret_cast<const uint2 *>(kc + trow * St::kCodeRow + G * 32 + i * 8);
                                    w[nt][0] = rr.x, w[nt][1] = rr.x >> 8, w[nt][2] = rr.y, w[nt][3] = rr.y >> 8;
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const uint4 A = qf[(G * 4 + j) * 32 + lane];
#pragma unroll
                                for (int nt = 0; nt < 2; nt++) {
                                    uint32_t b0, b1;
                                    if (BITS == 8) {
                                        // operands stay 1024 + c; 1024 * sum(q) is taken off the group sum below
                                        b0 = prmt(w[nt][j], kMagic, 0x4140), b1 = prmt(w[nt][j], kMagic, 0x4342);
                                    } else {
                                        // low nibbles ride on 1024, high nibbles on 64: (1024, 64) * the matching
                                        // partial sums of q come off below
                                        b0 = lop_and_or(w[nt][j], 0x000f000fu, k1024), b1 = lop_and_or(w[nt][j], 0x00f000f0u, k64);
                                    }
                                    mma_f16(acc[nt], A.x, A.y, A.z, A.w, b0, b1);
                                }
                            }
#pragma unroll
                            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                                for (int c = 0; c < 2; c++) {
                                    const float2 pr = sKf[nt][c][G >> 1];
                                    const float scale = (G & 1) ? pr.y : pr.x;
                                    sc[0][nt][c] = fmaf(scale, acc[nt][c] - qoff[0][G], sc[0][nt][c]);
                                    sc[1][nt][c] = fmaf(scale, acc[nt][c + 2] - qoff[1][G], sc[1][nt][c]);
                                }
                        }
#pragma unroll
                        for (int nt = 0; nt < 2; nt++) {
                            // bias term: sum_G z[token][G] * qsum[head][G] (k-slots 0..3 = groups)
                            float accz[4] = {0.f, 0.f, 0.f, 0.f};
                            uint32_t zb = *reinterpret_cast<const uint32_t *>(sg + St::kKz + (lt + nt * 8 + g) * St::kParamRow + kv * 8 + (i & 1) * 4);
                            if (i >= 2) zb = 0u;
                            mma_f16(accz, qza0, qza1, 0u, 0u, zb, 0u);
#pragma unroll
                            for (int c = 0; c < 2; c++) {
                                S[0][nt][c] = sc[0][nt][c] + accz[c];
                                S[1][nt][c] = sc[1][nt][c] + accz[c + 2];
                            }
                        }
                        if (partial) {
#pragma unroll
                            for (int r = 0; r < NR; r++)
#pragma unroll
                                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                                    for (int c = 0; c < 2; c++)
                                        if (tok0 + nt * 8 + 2 * i + c >= n_row[r]) S[r][nt][c] = -INFINITY;
                        }
                    }

                    // ------------------------------------------------ online softmax of head g (log2 units)
                    float p[NR][4];
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        float mx = fmaxf(fmaxf(S[r][0][0], S[r][0][1]), fmaxf(S[r][1][0], S[r][1][1]));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                        if (mx > Mref[r] + kRescale) { // uniform over the four lanes of the head
                            const float f = exp2f(Mref[r] - mx); // exp2f(-inf) = 0 on the first tile
                            Mref[r] = mx, lsum[r] *= f;
#pragma unroll
                            for (int e = 0; e < 32; e++) {
                                O[e][2 * r] *= f, O[e][2 * r + 1] *= f;
                            }
                            Ob[2 * r] *= f, Ob[2 * r + 1] *= f;
                        }
                        const float mu = Mref[r] == -INFINITY ? 0.f : Mref[r]; // a row with no key yet: every p is 0
                        p[r][0] = exp2f(S[r][0][0] - mu), p[r][1] = exp2f(S[r][0][1] - mu);
                        p[r][2] = exp2f(S[r][1][0] - mu), p[r][3] = exp2f(S[r][1][1] - mu);
                        lsum[r] += (p[r][0] + p[r][1]) + (p[r][2] + p[r][3]);
                    }
                    __syncwarp(); // the rescale branch is per head; the MMAs below need the whole warp

                    // ------------------------------------------------ O[head][dim] += P V
                    // P is the A operand: this lane's score columns (tokens 2i, 2i+1 and 8+2i, 9+2i of head
                    // g) are exactly the A fragment's elements, so no data moves between lanes.
                    const int T0 = lt + 2 * i, T1 = T0 + 1, T2 = T0 + 8, T3 = T0 + 9;
                    uint2 sV[4];
                    sV[0] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T0 * St::kParamRow + kv * 8);
                    sV[1] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T1 * St::kParamRow + kv * 8);
                    sV[2] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T2 * St::kParamRow + kv * 8);
                    sV[3] = *reinterpret_cast<const uint2 *>(sg + St::kVs + T3 * St::kParamRow + kv * 8);
                    if (partial) { // stale rows may hold anything: keep them out of 0 * x
                        if (tok0 + 2 * i >= n_any) sV[0] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 1 >= n_any) sV[1] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 8 >= n_any) sV[2] = make_uint2(0u, 0u);
                        if (tok0 + 2 * i + 9 >= n_any) sV[3] = make_uint2(0u, 0u);
                    }
                    // A fragment of x[0..3] (MMA row g) and y[0..3] (row g+8) at the lane's four tokens
                    auto a_frag = [&](const float (&x)[4], const float (&y)[4], uint32_t (&A)[4]) {
                        A[0] = pack_half2(x[0], x[1]), A[2] = pack_half2(x[2], x[3]);
                        A[1] = pack_half2(y[0], y[1]), A[3] = pack_half2(y[2], y[3]);
                    };
                    {   // value biases: one MMA with B[token][n = group] = z + C s (columns 4..7 empty)
                        const int gq = g & 3;
                        const uint8_t *vz = sg + St::kVz + kv * 8 + gq * 2;
                        uint32_t z0 = *reinterpret_cast<const uint16_t *>(vz + T0 * St::kParamRow);
                        uint32_t z1 = *reinterpret_cast<const uint16_t *>(vz + T1 * St::kParamRow);
                        uint32_t z2 = *reinterpret_cast<const uint16_t *>(vz + T2 * St::kParamRow);
                        uint32_t z3 = *reinterpret_cast<const uint16_t *>(vz + T3 * St::kParamRow);
                        if (partial) {
                            if (tok0 + 2 * i >= n_any) z0 = 0;
                            if (tok0 + 2 * i + 1 >= n_any) z1 = 0;
                            if (tok0 + 2 * i + 8 >= n_any) z2 = 0;
                            if (tok0 + 2 * i + 9 >= n_any) z3 = 0;
                        }
                        // this lane's group is gq: its scales sit in half gq of the pairs gathered above
                        const uint32_t sel = (gq & 1) ? 0x7632u : 0x5410u;
                        const uint32_t s01 = prmt(gq < 2 ? sV[0].x : sV[0].y, gq < 2 ? sV[1].x : sV[1].y, sel);
                        const uint32_t s23 = prmt(gq < 2 ? sV[2].x : sV[2].y, gq < 2 ? sV[3].x : sV[3].y, sel);
                        const uint32_t cc = pack_half2(kVCentre, kVCentre);
                        const uint32_t b0 = g < 4 ? hfma2_u32(s01, cc, z0 | z1 << 16) : 0u;
                        const uint32_t b1 = g < 4 ? hfma2_u32(s23, cc, z2 | z3 << 16) : 0u;
                        uint32_t A[4];
                        a_frag(p[0], p[1], A);
                        mma_f16(Ob, A[0], A[1], A[2], A[3], b0, b1);
                    }
                    const uint8_t *vc = sg + St::kV + kv * (kDim * BITS / 8);
#pragma unroll
                    for (int G = 0; G < 4; G++) {
                        uint32_t A[4];
                        {   // P times the value scales of group G: f32 product, one rounding
                            float cs[4], x[4], y[4];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const float2 pr = h2f2(G < 2 ? sV[k].x : sV[k].y);
                                cs[k] = (G & 1) ? pr.y : pr.x;
                                x[k] = p[0][k] * cs[k], y[k] = p[1][k] * cs[k];
                            }
                            a_frag(x, y, A);
                        }
                        if (BITS == 8) {
                            // 8 dims (G*64 + g*8 ..) of the lane's four tokens
                            const uint2 t0 = *reinterpret_cast<const uint2 *>(vc + T0 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t1 = *reinterpret_cast<const uint2 *>(vc + T1 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t2 = *reinterpret_cast<const uint2 *>(vc + T2 * St::kCodeRow + G * 64 + g * 8);
                            const uint2 t3 = *reinterpret_cast<const uint2 *>(vc + T3 * St::kCodeRow + G * 64 + g * 8);
                            // [T0.b0 T1.b0 T0.b1 T1.b1] and [T0.b2 T1.b2 T0.b3 T1.b3]; .y: bytes 4..7
                            const uint32_t x01[4] = {prmt(t0.x, t1.x, 0x5140), prmt(t0.x, t1.x, 0x7362),
                                                     prmt(t0.y, t1.y, 0x5140), prmt(t0.y, t1.y, 0x7362)};
                            const uint32_t x23[4] = {prmt(t2.x, t3.x, 0x5140), prmt(t2.x, t3.x, 0x7362),
                                                     prmt(t2.y, t3.y, 0x5140), prmt(t2.y, t3.y, 0x7362)};
#pragma unroll
                            for (int e = 0; e < 8; e++) { // n-tile e: dim G*64 + n*8 + e in column n
                                const uint32_t sel = (e & 1) ? 0x4342u : 0x4140u;
                                // 1024 + c minus 1152: the centred code c - 128 (see kVCentre)
                                const uint32_t b0 = hsub2_u32(prmt(x01[e >> 1], kMagic, sel), k1152);
                                const uint32_t b1 = hsub2_u32(prmt(x23[e >> 1], kMagic, sel), k1152);
                                mma_f16(O[G * 8 + e], A[0], A[1], A[2], A[3], b0, b1);
                            }
                        } else {
                            const uint32_t t0 = *reinterpret_cast<const uint32_t *>(vc + T0 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t1 = *reinterpret_cast<const uint32_t *>(vc + T1 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t2 = *reinterpret_cast<const uint32_t *>(vc + T2 * St::kCodeRow + G * 32 + g * 4);
                            const uint32_t t3 = *reinterpret_cast<const uint32_t *>(vc + T3 * St::kCodeRow + G * 32 + g * 4);
                            // low half-word: T0's nibbles 0..3, high: T1's; second word: nibbles 4..7
                            const uint32_t x01[2] = {prmt(t0, t1, 0x5410), prmt(t0, t1, 0x7632)};
                            const uint32_t x23[2] = {prmt(t2, t3, 0x5410), prmt(t2, t3, 0x7632)};
#pragma unroll
                            for (int e = 0; e < 8; e++) { // nibble e of the 8
                                // nibble e & 3 of each half-word into bits 4..7 of its byte: 64 + n, minus 71.5
                                auto code = [&](uint32_t w) {
                                    const uint32_t x = (e & 3) == 0 ? w << 4 : (e & 3) == 1 ? w : (e & 3) == 2 ? w >> 4 : w >> 8;
                                    return hsub2_u32(lop_and_or(x, 0x00f000f0u, k64), k71_5);
                                };
                                mma_f16(O[G * 8 + e], A[0], A[1], A[2], A[3], code(x01[e >> 2]), code(x23[e >> 2]));
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }

            // ---------------------------------------------------------------- end of segment
#pragma unroll
            for (int r = 0; r < NR; r++) { // l of head g over the four lanes that share it
                lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 1);
                lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 2);
            }
#pragma unroll
            for (int G = 0; G < 4; G++) { // the bias sums of group G sit in lane i = G/2 of the head's four
                const int src = (lane & ~3) | (G >> 1);
                const float b0 = __shfl_sync(0xffffffffu, Ob[G & 1], src);
                const float b1 = __shfl_sync(0xffffffffu, Ob[2 + (G & 1)], src);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    O[G * 8 + e][0] += b0, O[G * 8 + e][1] += b0;
                    O[G * 8 + e][2] += b1, O[G * 8 + e][3] += b1;
                }
            }
            // Warps that share a (kv, row group) agree on one maximum per row, scale, and add up in a
            // fixed order through shared memory (deterministic).
            if (i == 0) {
#pragma unroll
                for (int r = 0; r < NR; r++) {
                    float *m = ml + (warp * NR + r) * 16;
                    m[g] = Mref[r], m[8 + g] = lsum[r];
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            float Mc[NR], lc[NR], f[NR];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                Mc[r] = -INFINITY, lc[r] = 0.f;
#pragma unroll
                for (int sl = 0; sl < NSLOT; sl++) Mc[r] = fmaxf(Mc[r], ml[((((sl * NP + pair) << 1) | kv) * NR + r) * 16 + g]);
#pragma unroll
                for (int sl = 0; sl < NSLOT; sl++) {
                    const float *m = ml + ((((sl * NP + pair) << 1) | kv) * NR + r) * 16;
                    lc[r] += m[g] == -INFINITY ? 0.f : m[8 + g] * exp2f(m[g] - Mc[r]);
                }
                f[r] = Mref[r] == -INFINITY ? 0.f : exp2f(Mref[r] - Mc[r]);
            }
            // After the barrier above no warp reads the copy ring any more, so every warp parks its
            // scaled accumulators in the ring at once, in the fragment order of the one-row path (the
            // merge kernel knows only that one): head h, dim d sits at
            // (4*mt + c)*32 + 4*((d >> 3) & 7) + (h >> 1), mt = 4*(d >> 6) + (d & 3), c = (h & 1) + ((d >> 1) & 2).
            // Then each warp adds up its share of the elements in slot order (fixed, hence deterministic).
            float *ring = reinterpret_cast<float *>(stages);
#pragma unroll
            for (int r = 0; r < NR; r++) {
                float *mine = ring + (warp * NR + r) * kFragFloats + (g & 1) * 32 + (g >> 1);
#pragma unroll
                for (int e = 0; e < 32; e++)
#pragma unroll
                    for (int cc = 0; cc < 2; cc++) // head g, dim 64*(e >> 3) + 8*(2i + cc) + (e & 7)
                        mine[(4 * (4 * (e >> 3) + (e & 3)) + 2 * ((e >> 2) & 1)) * 32 + 4 * (2 * i + cc)] = O[e][2 * r + cc] * f[r];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
#pragma unroll
            for (int r = 0; r < NR; r++) {
                if (rowA + r >= a.m) continue;
                const PartWriter pw = part_writer(a.parts, a.mo.n_merge != 0, a.n_decode, a.m, rowA + r, kv, s.part);
                constexpr int per = 64 / NSLOT;
#pragma unroll
                for (int k = 0; k < per; k++) {
                    float v = 0.f;
#pragma unroll
                    for (int sl = 0; sl < NSLOT; sl++) {
                        const int w = ((sl * NP + pair) << 1) | kv;
                        v += ring[(w * NR + r) * kFragFloats + (slot * per + k) * 32 + lane];
                    }
                    const int fr = slot * per + k; // fragment register
                    pw.reg(fr)[lane] = v;
                }
                if (slot == 0 && i == 0) pw.ml[g] = Mc[r], pw.ml[8 + g] = lc[r];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); // ring, merge buffer and query fragments free again
        }
        // The partial is written: tell the merge CTAs of this launch (the writers meet, then one
        // of them fences and takes the ticket).
        if (a.mo.n_merge) {
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            if (threadIdx.x == 0) ticket_arrive(a.status, blockIdx.y);
        }
    }
}

template <int BITS, int ROWS>
static int launch_one(const DecodeArgs &a, dim3 grid, cudaStream_t stream) {
    SAETTA_CUDA(launch_pdl(decode_quant_kernel<BITS, ROWS>, grid, dim3(kThreads), smem_bytes<BITS>(), stream, a));
    return SAETTA_OK;
}

template <int BITS>
static int launch_rows(DecodeArgs &a, cudaStream_t stream) {
    // blocks [0, n_decode) are the split-KV CTAs, the n_merge after them merge (per pass)
    const uint32_t rows_pass = a.m == 1 ? 1 : a.m == 2 ? 2 : 4;
    a.mo.n_merge = merge_role_ctas(rows_pass);
    const dim3 grid(a.n_decode + a.mo.n_merge, rows_pass == 4 ? (a.m + 3) / 4 : 1);
    a.mo.passes = grid.y;
    if (rows_pass == 1) return launch_one<BITS, 1>(a, grid, stream);
    if (rows_pass == 2) return launch_one<BITS, 2>(a, grid, stream);
    return launch_one<BITS, 4>(a, grid, stream);
}

int decode_quant_configure(int device) {
    (void)device;
#define SAETTA_SET(BITS, ROWS)                                                               \
    SAETTA_CUDA(cudaFuncSetAttribute(decode_quant_kernel<BITS, ROWS>,                        \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<BITS>()))
    SAETTA_SET(8, 1);
    SAETTA_SET(8, 2);
    SAETTA_SET(8, 4);
    SAETTA_SET(4, 1);
    SAETTA_SET(4, 2);
    SAETTA_SET(4, 4);
#undef SAETTA_SET
    return SAETTA_OK;
}

int launch_decode_quant(const KvView &kv, const float *q, float *parts, uint32_t *status,
                        uint32_t m, uint32_t row_step, int splits, uint32_t capacity,
                        const saetta_token_params *params, const MergeOut &mo, cudaStream_t stream) {
    if (splits < 1 || splits > kMergeRoleMaxParts) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: 1..160 split-KV parts");
    DecodeArgs a{};
    a.seg.k = kv.k, a.seg.v = kv.v, a.seg.ks = kv.ks, a.seg.kz = kv.kz, a.seg.vs = kv.vs, a.seg.vz = kv.vz;
    a.segs = nullptr, a.cta_first = nullptr;
    a.q = q, a.parts = parts, a.status = status, a.params = params;
    a.m = m, a.row_step = row_step, a.capacity = capacity;
    a.n_decode = uint32_t(splits), a.mo = mo;
    return kv.bits == 8 ? launch_rows<8>(a, stream) : launch_rows<4>(a, stream);
}

int launch_decode_quant_batched(int bits, const Segment *segments_dev, const uint32_t *cta_first_dev,
                                int ctas, const float *q, float *parts, uint32_t *status,
                                cudaStream_t stream) {
    DecodeArgs a{};
    a.segs = segments_dev, a.cta_first = cta_first_dev;
    a.q = q, a.parts = parts, a.status = status, a.params = nullptr;
    a.m = 1, a.row_step = 0, a.capacity = 0xffffffffu;
    a.n_decode = uint32_t(ctas), a.mo = MergeOut{}; // the ragged batch keeps its merge as a launch of its own (merge.cu)
    return bits == 8 ? launch_one<8, 1>(a, dim3(ctas, 1), stream) : launch_one<4, 1>(a, dim3(ctas, 1), stream);
}

// ----------------------------------------------------------------- fixed-scratch entry point
//
// Scratch for saetta_decode_record_quant_static: the split-KV partials and the
// status words live in these file-scope device arrays instead of cudaMalloc'd
// buffers.  Every GPU that loads the library holds these bytes until exit.
constexpr int kStaticMaxRows = 2;
constexpr int kStaticMaxSplits = kMergeRoleMaxParts;
constexpr size_t kStaticFloats = size_t(kStaticMaxSplits) * kStaticMaxRows * kKv * kPartKv; // 5.3 MB
static __device__ __align__(256) float g_static_parts[kStaticFloats];
static __device__ __align__(256) uint32_t g_static_status[64]; // laid out as an op's status words
static_assert(kStatusWords <= 64, "the status words fit");

struct StaticScratch {
    float *parts = nullptr;   // device address of g_static_parts on that device
    uint32_t *status = nullptr;
    int splits = 0;
};
static StaticScratch g_static[64];

// Looks up, once per device and with that device current, the device addresses
// of the two arrays above.  In host code their names are only host-side handles:
// a kernel must be given what cudaGetSymbolAddress returns.
static int static_scratch(int device, StaticScratch **out) {
    if (device < 0 || device >= 64) return fail(SAETTA_ERR_BAD_ARG, "static decode: device index out of range");
    static std::mutex init_mutex; // first calls from several host threads may meet here
    std::lock_guard<std::mutex> lock(init_mutex);
    StaticScratch &s = g_static[device];
    if (!s.parts) {
        void *parts = nullptr, *status = nullptr;
        SAETTA_CUDA(cudaGetSymbolAddress(&parts, g_static_parts));
        SAETTA_CUDA(cudaGetSymbolAddress(&status, g_static_status));
        if (int rc = decode_quant_configure(device)) return rc;
        s.splits = std::min(sm_count(device), kStaticMaxSplits);
        s.status = static_cast<uint32_t *>(status);
        s.parts = static_cast<float *>(parts);
    }
    *out = &s;
    return SAETTA_OK;
}

int decode_quant_static(int device, const KvView &kv, size_t capacity, const float *q, uint32_t m,
                        const float *q_and_gate, float *out, const saetta_token_params *params,
                        cudaStream_t stream) {
    if (m < 1 || m > uint32_t(kStaticMaxRows))
        return fail(SAETTA_ERR_BAD_SHAPE, "static decode: at most 2 query rows fit the fixed scratch (use saetta_decode_create for more)");
    if (kv.bits != 8 && kv.bits != 4) return fail(SAETTA_ERR_BAD_SHAPE, "static decode: the rows must hold 8- or 4-bit codes");
    if (kv.kv_heads != kKv) return fail(SAETTA_ERR_BAD_SHAPE, "static decode: built for 2 kv heads");
    if (capacity % kTile || !capacity) return fail(SAETTA_ERR_BAD_SHAPE, "static decode: capacity must be a positive multiple of 32");
    if (capacity > 0xffffffe0ull) return fail(SAETTA_ERR_BAD_SHAPE, "static decode: capacity too large");
    StaticScratch *s = nullptr;
    if (int rc = static_scratch(device, &s)) return rc;
    const int splits = int(std::min<size_t>(size_t(s->splits), capacity / kTile));
    // The launch overwrites every partial it later reads, and its merge CTAs put the two counters
    // in the status words back to zero, so nothing has to be cleared between calls.
    MergeOut mo{};
    mo.q_and_gate = q_and_gate, mo.out = out;
    return launch_decode_quant(kv, q, s->parts, s->status, m, 1, splits, uint32_t(capacity), params, mo, stream);
}

// The status word of the fixed-scratch path on `device` (bits of bounded waits that gave up); with
// `clear` it is put back to zero after being read.
int decode_quant_static_status(int device, cudaStream_t stream, uint32_t *status, bool clear) {
    StaticScratch *s = nullptr;
    if (int rc = static_scratch(device, &s)) return rc;
    SAETTA_CUDA(cudaMemcpyAsync(status, s->status, 4, cudaMemcpyDeviceToHost, stream));
    if (clear) SAETTA_CUDA(cudaMemsetAsync(s->status, 0, 4, stream));
    SAETTA_CUDA(cudaStreamSynchronize(stream));
    return SAETTA_OK;
}

} // namespace saetta
