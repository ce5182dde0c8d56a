// Split-KV decode / MTP-verify attention over a 16-bit (binary16 or bfloat16) KV cache, on the tensor cores.
//
// Stands in for attention_partial_mma (kernels/attention.metal:127-236) and
// attention_partial_rows<16> (kernels/attention_rows.metal:108-292) of the
// reference, whose default cache holds half rows [capacity][kv_heads][256]; the
// merge over parts is in merge.cu.  Same shape as the quantised kernel next door
// (decode_quant.cu), minus the dequantisation:
//
//  * One persistent CTA per SM owns a contiguous range of 32-token tiles.  A
//    producer warp streams each tile into a ring of shared-memory stages with
//    TMA tensor copies signalled on mbarriers: per side eight slabs of 32 tokens
//    x 64 dims (128-byte rows, 128-byte swizzle), so that neither the key loads
//    nor ldmatrix below meet bank conflicts.  (One bulk copy per token row into
//    padded rows was tried first: 64 requests of 1 KB per tile held the kernel
//    at 3.6 TB/s, the TMA unit's rate for small requests.)
//  * Eight consumer warps each own one kv head and a share of the 16-token
//    sub-tiles.  Scores: mma.sync m16n8k16 with the 16 rows = high and low halves
//    of the 8 query heads (the query keeps f32 precision), K straight from shared
//    memory as the B operand (a lane's 128-bit load is two k-steps; the query
//    fragments are built for that order of dims).  Values: ldmatrix.trans turns
//    [token][dim] rows into the A fragments of O^T[dim][head] += V^T P^T.
//  * Online softmax and the end-of-range merge as in the quantised kernel; the
//    partials leave in the same fragment order, so merge.cu and the exchange
//    across GPUs serve both.
//  * One query row per pass, or -- for several rows -- two, which then share every
//    load of the cache: the 16 MMA rows are the two rows' heads (queries rounded to
//    binary16, P a single operand).  m rows are ceil(m/2) passes (gridDim.y).
//    Every wait on an mbarrier is bounded.
#include <cuda.h>

#include <algorithm>

#include "merge_role.cuh"

namespace saetta {

namespace half_decode {

constexpr int kTile = 32;   // tokens per stage
constexpr int kSub = 16;    // tokens per MMA sub-tile
constexpr int kWarps = 8;   // consumer warps
constexpr int kThreads = (kWarps + 4) * 32;
constexpr int kKv = 2;
constexpr int kRowBytes = kKv * kDim * 2;   // one token of one side in the cache
constexpr int kSlab = kTile * 128;          // 32 tokens x 64 dims, 128-byte rows
constexpr int kSideBytes = kKv * 4 * kSlab; // the tile's keys (or values): slab = kv*4 + dims/64
constexpr int kStageBytes = 2 * kSideBytes;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescale = 8.0f;
constexpr int kPrefetchTiles = 2;
constexpr int kSmem = 1024 /*align*/ + kStages * kStageBytes + kWarps * 2 * 16 * 4 + 2 * kStages * 8 + 32; // also what a launch's merge CTAs use
static_assert(kMergeRoleSmem <= kSmem - 1024, "the merge role fits a CTA's shared memory");
static_assert(kWarps * 2 * kFragFloats * 4 <= kStages * kStageBytes, "the end-of-range merge parks in the ring");

struct Args {
    const uint8_t *k, *v; // [capacity][2][256] binary16
    const float *q;       // [m][16][256]
    float *parts;         // [part][m][kv][kPartKv]
    uint32_t *status;     // the op's status words (merge_role.cuh)
    const saetta_token_params *params;
    uint32_t m, row_step, capacity;
    uint32_t n_decode;    // split-KV CTAs (= parts); the blocks after them run the merge role
    MergeOut mo;
};

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

// D += A(16x16, row) * B(16x8, col), bfloat16 operands, f32 accumulate.
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Two floats as a pair of 16-bit values of the cache's type, and back.
template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    return pack_half2(lo, hi);
}
template <bool BF16>
__device__ __forceinline__ float2 unpack16(uint32_t w) {
    if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    return h2f2(w);
}
template <bool BF16>
__device__ __forceinline__ void mma16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (BF16) mma_bf16(c, a0, a1, a2, a3, b0, b1);
    else mma_f16(c, a0, a1, a2, a3, b0, b1);
}

// NR query rows per pass; BF16: the cache holds bfloat16 (one row per pass only: with 8-bit significands
// both the query and P need their second halves).
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Byte offset, inside a side of a stage, of 16-byte chunk `chunk` (of the 32 of a kv head's row) of token `tok`.
__device__ __forceinline__ uint32_t swz(uint32_t kv, uint32_t tok, uint32_t chunk) {
    return (kv * 4 + (chunk >> 3)) * kSlab + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4);
}

template <int NR, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
decode_half_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a) {
    static_assert(NR == 1 || !BF16, "two rows per pass need binary16");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    if (blockIdx.x >= a.n_decode) { // the blocks after the split-KV CTAs merge what those leave
        merge_role<kThreads>(a.parts, a.n_decode, a.m, blockIdx.y * NR, NR, a.mo, a.status, blockIdx.y, blockIdx.x - a.n_decode, smem);
        return;
    }
    uint8_t *stages = smem;
    float *ml = reinterpret_cast<float *>(smem + kStages * kStageBytes); // [warp][m of 8 heads, l of 8 heads]
    uint64_t *full = reinterpret_cast<uint64_t *>(ml + kWarps * 2 * 16);
    uint64_t *empty = full + kStages;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(empty + kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        abort_flag[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t row0 = blockIdx.y * NR; // the first query row of this pass
    auto range = [&](uint32_t kv_len, uint32_t &tb, uint32_t &te, uint32_t &n_any) {
        const uint32_t last = min(row0 + NR, a.m) - 1; // the pass's last live row sees the most keys
        n_any = min(kv_len + last * a.row_step, a.capacity);
        const uint32_t tiles = (n_any + kTile - 1) / kTile;
        tb = uint32_t(uint64_t(blockIdx.x) * tiles / a.n_decode);
        te = uint32_t(uint64_t(blockIdx.x + 1) * tiles / a.n_decode);
    };
    auto issue_tile = [&](uint32_t t, uint32_t st) { // the producer warp, all lanes
        uint8_t *dst = stages + st * kStageBytes;
        if (lane == 0) mbar_expect_tx(&full[st], kStageBytes);
        __syncwarp();
        // lanes 0..7: the key slabs, 8..15: the value slabs (slab = kv*4 + dims/64)
        if (lane < 16) {
            const int sl = lane & 7;
            tma_load_3d(dst + (lane >> 3) * kSideBytes + sl * kSlab, lane < 8 ? &map_k : &map_v, &full[st], (sl & 3) * 64,
                        sl >> 2, int(t * kTile));
        }
        __syncwarp();
    };
    // While the launch before this one drains, pull the head of this CTA's range into L2 (the range
    // comes from a possibly stale kv_len: a hint only, everything is read again after the wait).
    if (warp == kWarps && lane == 0) {
        uint32_t tb, te, n_hint;
        range(*reinterpret_cast<const volatile uint32_t *>(&a.params->kv_len), tb, te, n_hint);
        const uint32_t nt = min(te - tb, uint32_t(kPrefetchTiles));
        for (uint32_t t = 0; t < nt; t++) {
            l2_prefetch(a.k + size_t(tb + t) * kTile * kRowBytes, kTile * kRowBytes);
            l2_prefetch(a.v + size_t(tb + t) * kTile * kRowBytes, kTile * kRowBytes);
        }
    }
    pdl_wait();              // q, the token parameters and the new rows of the cache may come from the launch before
    pdl_launch_dependents(); // the next launch's CTAs may take the SMs this grid's CTAs leave
    uint32_t tile_begin, tile_end, n_any;
    range(a.params->kv_len, tile_begin, tile_end, n_any);
    uint32_t n_row[NR]; // keys each row of the pass sees (0 for a row past m)
    uint32_t n_all = n_any;
#pragma unroll
    for (int r = 0; r < NR; r++) {
        n_row[r] = row0 + r < a.m ? min(a.params->kv_len + (row0 + r) * a.row_step, a.capacity) : 0u;
        if (row0 + r < a.m) n_all = min(n_all, n_row[r]);
    }

    if (warp >= kWarps) {
        // ---------------------------------------------------------------- producer
        // (same register pool rule as in decode_quant.cu: 128 x (168 - 40) = 256 x (232 - 168))
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp != kWarps) return;
        uint32_t it = 0;
        for (uint32_t t = tile_begin; t < tile_end; t++, it++) {
            const uint32_t st = it % kStages, round = it / kStages;
            if (!mbar_wait(&empty[st], (round & 1) ^ 1, abort_flag)) {
                if (lane == 0) {
                    atomicOr(a.status, kStatusEmptyTimeout);
                    *abort_flag = 1;
                }
                break;
            }
            issue_tile(t, st);
        }
        // Leave only once every copy this warp issued has landed (bounded): the shared memory must
        // not be handed to another CTA with copies in flight.
        const uint32_t issued = it;
        for (uint32_t k = issued > kStages ? issued - kStages : 0; k < issued; k++)
            mbar_wait(&full[k % kStages], (k / kStages) & 1, abort_flag, 2000000u);
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");

    // -------------------------------------------------------------------- consumers
    constexpr int NSLOT = kWarps / kKv; // warps sharing one kv head
    const int kv = warp & 1, slot = warp >> 1;
    const int g = lane >> 2, i = lane & 3;

    // Query fragments of head kv*8+g, scaled by log2(e)/16.  One row per pass: split into two halves, the
    // 16 MMA rows are the heads' high and low halves.  Two rows: rows 0..7 are the first row's heads,
    // 8..15 the second's, rounded to binary16.  k-step ks covers, for lane i, dims
    // 32*(ks/2) + 8*i + 4*(ks%2) + {0,1 | 2,3}: what a 128-bit load of K holds.
    uint32_t qh[16][2], ql[16][2];
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const uint32_t qrow = row0 + r < a.m ? row0 + r : 0;
        const float *qp = a.q + ((size_t(qrow) * 16) + kv * 8 + g) * kDim;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const float4 v0 = *reinterpret_cast<const float4 *>(qp + b * 32 + i * 8);
            const float4 v1 = *reinterpret_cast<const float4 *>(qp + b * 32 + i * 8 + 4);
            const float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            float hi[8], lo[8];
#pragma unroll
            for (int d = 0; d < 8; d++) {
                const float s = x[d] * (kLog2e * 0.0625f);
                hi[d] = unpack16<BF16>(pack16<BF16>(s, 0.f)).x;
                lo[d] = s - hi[d]; // rounded when packed
            }
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    if (r == 0) qh[2 * b + j][e] = pack16<BF16>(hi[4 * j + 2 * e], hi[4 * j + 2 * e + 1]);
                    if (NR == 1) ql[2 * b + j][e] = pack16<BF16>(lo[4 * j + 2 * e], lo[4 * j + 2 * e + 1]);
                    if (NR == 2 && r == 1) ql[2 * b + j][e] = pack16<BF16>(hi[4 * j + 2 * e], hi[4 * j + 2 * e + 1]);
                }
        }
    }

    float O[NR][16][4];
    float Mref[NR], lsum[NR]; // of head g (this thread's row of the score MMA), per query row
#pragma unroll
    for (int r = 0; r < NR; r++) {
#pragma unroll
        for (int e = 0; e < 16; e++) O[r][e][0] = O[r][e][1] = O[r][e][2] = O[r][e][3] = 0.f;
        Mref[r] = -INFINITY, lsum[r] = 0.f;
    }

    uint32_t it = 0;
    for (uint32_t t = tile_begin; t < tile_end; t++, it++) {
        const uint32_t st = it % kStages, round = it / kStages;
        if (!mbar_wait(&full[st], round & 1, abort_flag)) {
            if (lane == 0) {
                atomicOr(a.status, kStatusFullTimeout);
                *abort_flag = 1;
            }
            break; // skip the tiles, keep the barriers below
        }
        const uint8_t *sk = stages + st * kStageBytes;
        const uint8_t *sv = sk + kSideBytes;
#pragma unroll 1
        for (int sub = 0; sub < kTile / kSub; sub++) {
            const uint32_t q_idx = 2 * (t - tile_begin) + sub;
            const uint32_t tok0 = t * kTile + sub * kSub; // first token of the sub-tile
            if ((q_idx % NSLOT) != uint32_t(slot) || tok0 >= n_any) continue;
            const bool partial = tok0 + kSub > n_all;
            const int lt = sub * kSub;

            // ------------------------------------------------ scores S[row][head][token]
            float S[NR][2][2];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const uint32_t ktok = lt + nt * 8 + g; // token g of the 8-token tile
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(sk + swz(kv, ktok, b * 4 + i));
                    mma16<BF16>(acc, qh[2 * b][0], ql[2 * b][0], qh[2 * b][1], ql[2 * b][1], w.x, w.y);
                    mma16<BF16>(acc, qh[2 * b + 1][0], ql[2 * b + 1][0], qh[2 * b + 1][1], ql[2 * b + 1][1], w.z, w.w);
                }
                if (NR == 1) {
                    S[0][nt][0] = acc[0] + acc[2], S[0][nt][1] = acc[1] + acc[3];
                } else {
                    S[0][nt][0] = acc[0], S[0][nt][1] = acc[1], S[NR - 1][nt][0] = acc[2], S[NR - 1][nt][1] = acc[3];
                }
                if (partial) { // rows past the end may hold anything: assigned, never computed with
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        if (tok0 + nt * 8 + 2 * i >= n_row[r]) S[r][nt][0] = -INFINITY;
                        if (tok0 + nt * 8 + 2 * i + 1 >= n_row[r]) S[r][nt][1] = -INFINITY;
                    }
                }
            }

            // ------------------------------------------------ online softmax of head g (log2 units)
            uint32_t pb[NR][2], pl[2];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                float mx = fmaxf(fmaxf(S[r][0][0], S[r][0][1]), fmaxf(S[r][1][0], S[r][1][1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const bool need = mx > Mref[r] + kRescale;
                if (__any_sync(0xffffffffu, need)) {
                    const float f = need ? exp2f(Mref[r] - mx) : 1.f; // exp2f(-inf) = 0 on the first tile
                    if (need) Mref[r] = mx, lsum[r] *= f;
                    // the accumulators' columns are heads 2i, 2i+1: fetch their factors from lanes g = 2i, 2i+1
                    const float f0 = __shfl_sync(0xffffffffu, f, 8 * i), f1 = __shfl_sync(0xffffffffu, f, 8 * i + 4);
#pragma unroll
                    for (int e = 0; e < 16; e++) O[r][e][0] *= f0, O[r][e][1] *= f1, O[r][e][2] *= f0, O[r][e][3] *= f1;
                }
                const float mu = Mref[r] == -INFINITY ? 0.f : Mref[r]; // a row with no key yet: every p is 0
                const float p00 = exp2f(S[r][0][0] - mu), p01 = exp2f(S[r][0][1] - mu);
                const float p10 = exp2f(S[r][1][0] - mu), p11 = exp2f(S[r][1][1] - mu);
                lsum[r] += (p00 + p01) + (p10 + p11);
                // B[k = token][n = head]: the lane's own score columns, no data moves between lanes.
                pb[r][0] = pack16<BF16>(p00, p01), pb[r][1] = pack16<BF16>(p10, p11);
                if (NR == 1) {
                    // One row: P goes in as two binary16 halves (what the first rounding dropped is the
                    // second operand), so the value product keeps f32 precision as the score product
                    // does; the kernel is bound by the cache's bytes, the second MMA is free.
                    const float2 h0 = unpack16<BF16>(pb[0][0]), h1 = unpack16<BF16>(pb[0][1]);
                    pl[0] = pack16<BF16>(p00 - h0.x, p01 - h0.y), pl[1] = pack16<BF16>(p10 - h1.x, p11 - h1.y);
                }
            }

            // ------------------------------------------------ O^T[dim][head] += V^T P^T
            // ldmatrix.trans: lanes 8j..8j+7 give the rows of matrix j -- tokens 0..7 (j < 2) or 8..15 of the
            // sub-tile at dims 0..7 (j even) or 8..15 of the 16-dim slice -- and get back token pairs of one dim.
            const uint32_t vtok = lt + ((lane >> 4) << 3) + (lane & 7), vhalf = (lane >> 3) & 1;
            uint32_t mask01 = 0xffffffffu, mask23 = 0xffffffffu;
            if (partial) { // what lies past the longest row may be anything: keep it out of 0 * x
                mask01 = (tok0 + 2 * i < n_any ? 0xffffu : 0u) | (tok0 + 2 * i + 1 < n_any ? 0xffff0000u : 0u);
                mask23 = (tok0 + 2 * i + 8 < n_any ? 0xffffu : 0u) | (tok0 + 2 * i + 9 < n_any ? 0xffff0000u : 0u);
            }
#pragma unroll
            for (int mt = 0; mt < 16; mt++) {
                uint32_t av[4];
                ldmatrix_x4_trans(av, sv + swz(kv, vtok, mt * 2 + vhalf));
                if (partial) av[0] &= mask01, av[1] &= mask01, av[2] &= mask23, av[3] &= mask23;
#pragma unroll
                for (int r = 0; r < NR; r++) mma16<BF16>(O[r][mt], av[0], av[1], av[2], av[3], pb[r][0], pb[r][1]);
                if (NR == 1) mma16<BF16>(O[0][mt], av[0], av[1], av[2], av[3], pl[0], pl[1]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
    }

    // ---------------------------------------------------------------- end of range
    // Warps that share a kv head agree on one maximum per row, scale, and add up in a fixed order
    // (deterministic).  After the first barrier no warp reads the copy ring any more (a producer that
    // gave up has raised the status word; the result is void then): every warp parks its scaled
    // accumulators there in the merge kernel's fragment order -- head h, dim d at
    // (4*mt + c)*32 + 4*((d >> 3) & 7) + (h >> 1), mt = 4*(d >> 6) + (d & 3), c = (h & 1) + ((d >> 1) & 2)
    // -- and then each warp adds up its share.
    float Mc2[NR][2], l[NR][2];
#pragma unroll
    for (int r = 0; r < NR; r++) {
        lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 1);
        lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 2);
        Mc2[r][0] = __shfl_sync(0xffffffffu, Mref[r], 8 * i), Mc2[r][1] = __shfl_sync(0xffffffffu, Mref[r], 8 * i + 4);
        l[r][0] = __shfl_sync(0xffffffffu, lsum[r], 8 * i), l[r][1] = __shfl_sync(0xffffffffu, lsum[r], 8 * i + 4);
        if (g == 0) {
            float *m = ml + (warp * NR + r) * 16;
            m[2 * i] = Mc2[r][0], m[2 * i + 1] = Mc2[r][1];
            m[8 + 2 * i] = l[r][0], m[8 + 2 * i + 1] = l[r][1];
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
    float Mc[NR][2], lc[NR][2];
    float *ring = reinterpret_cast<float *>(stages);
#pragma unroll
    for (int r = 0; r < NR; r++) {
        Mc[r][0] = Mc[r][1] = -INFINITY, lc[r][0] = lc[r][1] = 0.f;
#pragma unroll
        for (int sl = 0; sl < NSLOT; sl++) {
            const float *m = ml + ((((sl << 1) | kv)) * NR + r) * 16;
            Mc[r][0] = fmaxf(Mc[r][0], m[2 * i]), Mc[r][1] = fmaxf(Mc[r][1], m[2 * i + 1]);
        }
#pragma unroll
        for (int sl = 0; sl < NSLOT; sl++) {
            const float *m = ml + ((((sl << 1) | kv)) * NR + r) * 16;
            const float m0 = m[2 * i], m1 = m[2 * i + 1];
            lc[r][0] += m0 == -INFINITY ? 0.f : m[8 + 2 * i] * exp2f(m0 - Mc[r][0]);
            lc[r][1] += m1 == -INFINITY ? 0.f : m[8 + 2 * i + 1] * exp2f(m1 - Mc[r][1]);
        }
        const float f0 = Mc2[r][0] == -INFINITY ? 0.f : exp2f(Mc2[r][0] - Mc[r][0]);
        const float f1 = Mc2[r][1] == -INFINITY ? 0.f : exp2f(Mc2[r][1] - Mc[r][1]);
        float *mine = ring + (warp * NR + r) * kFragFloats + i;
#pragma unroll
        for (int mt = 0; mt < 16; mt++)
#pragma unroll
            for (int c = 0; c < 4; c++) { // head 2i + (c & 1), dim 16*mt + g + 8*(c >> 1)
                const int mtq = 4 * (mt >> 2) + (g & 3), cq = (c & 1) + 2 * ((g >> 2) & 1);
                mine[(4 * mtq + cq) * 32 + 4 * ((2 * mt + (c >> 1)) & 7)] = O[r][mt][c] * ((c & 1) ? f1 : f0);
            }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
#pragma unroll
    for (int r = 0; r < NR; r++) {
        if (row0 + r >= a.m) continue;
        const PartWriter pw = part_writer(a.parts, a.mo.n_merge != 0, a.n_decode, a.m, row0 + r, kv, blockIdx.x);
        constexpr int per = 64 / NSLOT;
#pragma unroll
        for (int k = 0; k < per; k++) {
            float v = 0.f;
#pragma unroll
            for (int sl = 0; sl < NSLOT; sl++) v += ring[((((sl << 1) | kv)) * NR + r) * kFragFloats + (slot * per + k) * 32 + lane];
            const int fr = slot * per + k; // fragment register
            pw.reg(fr)[lane] = v;
        }
        if (slot == 0 && g == 0) {
            pw.ml[2 * i] = Mc[r][0], pw.ml[2 * i + 1] = Mc[r][1];
            pw.ml[8 + 2 * i] = lc[r][0], pw.ml[8 + 2 * i + 1] = lc[r][1];
        }
    }
    // The partial is written: tell the merge CTAs of this launch (the writers meet, then one of
    // them fences and takes the ticket).
    if (a.mo.n_merge) {
        asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
        if (threadIdx.x == 0) ticket_arrive(a.status, blockIdx.y);
    }
}

} // namespace half_decode

int decode_half_configure(int device) {
    (void)device;
    SAETTA_CUDA(cudaFuncSetAttribute(half_decode::decode_half_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     half_decode::kSmem));
    SAETTA_CUDA(cudaFuncSetAttribute(half_decode::decode_half_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     half_decode::kSmem));
    SAETTA_CUDA(cudaFuncSetAttribute(half_decode::decode_half_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     half_decode::kSmem));
    return SAETTA_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

int launch_decode_half(const KvView &kv, const float *q, float *parts, uint32_t *status, uint32_t m, uint32_t row_step,
                       int splits, uint32_t capacity, const saetta_token_params *params, const MergeOut &mo,
                       cudaStream_t stream) {
    if (splits < 1 || splits > kMergeRoleMaxParts) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: 1..160 split-KV parts");
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(SAETTA_ERR_CUDA, "decode attention: cuTensorMapEncodeTiled is not available");
    // rows [capacity][2][256]: a box is one slab, 64 dims of one kv head x 32 tokens, 128-byte swizzle
    CUtensorMap mk, mv;
    const CUtensorMapDataType dt = kv.dtype == SAETTA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    for (int side = 0; side < 2; side++) {
        const cuuint64_t dims[3] = {cuuint64_t(kDim), cuuint64_t(half_decode::kKv), cuuint64_t(capacity)};
        const cuuint64_t strides[2] = {kDim * 2, cuuint64_t(half_decode::kKv) * kDim * 2};
        const cuuint32_t box[3] = {64, 1, half_decode::kTile}, el[3] = {1, 1, 1};
        CUresult r = enc(side ? &mv : &mk, dt, 3, const_cast<void *>(side ? kv.v : kv.k), dims, strides, box, el,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(SAETTA_ERR_CUDA, "decode attention: tensor map for the cache rejected");
    }
    half_decode::Args a{};
    a.k = static_cast<const uint8_t *>(kv.k), a.v = static_cast<const uint8_t *>(kv.v);
    a.q = q, a.parts = parts, a.status = status, a.params = params;
    a.m = m, a.row_step = row_step, a.capacity = capacity;
    // blocks [0, n_decode): one part per CTA (CTAs past the last tile leave an empty part); the n_merge
    // blocks after them merge the parts of their pass
    a.n_decode = uint32_t(splits), a.mo = mo;
    const bool pairs = kv.dtype != SAETTA_BF16 && m > 1; // two rows per pass share every load of the cache
    a.mo.n_merge = merge_role_ctas(pairs ? 2 : 1);
    a.mo.passes = kv.dtype == SAETTA_BF16 ? m : m == 1 ? 1 : (m + 1) / 2; // gridDim.y below
    const unsigned ctas = a.n_decode + a.mo.n_merge;
    if (kv.dtype == SAETTA_BF16)
        SAETTA_CUDA(launch_pdl(half_decode::decode_half_kernel<1, true>, dim3(ctas, m), dim3(half_decode::kThreads),
                               half_decode::kSmem, stream, mk, mv, a));
    else if (m == 1)
        SAETTA_CUDA(launch_pdl(half_decode::decode_half_kernel<1, false>, dim3(ctas, 1), dim3(half_decode::kThreads),
                               half_decode::kSmem, stream, mk, mv, a));
    else
        SAETTA_CUDA(launch_pdl(half_decode::decode_half_kernel<2, false>, dim3(ctas, (m + 1) / 2), dim3(half_decode::kThreads),
                               half_decode::kSmem, stream, mk, mv, a));
    return SAETTA_OK;
}

} // namespace saetta
