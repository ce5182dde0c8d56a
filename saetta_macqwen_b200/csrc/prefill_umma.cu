// Chunked causal prefill attention on the 5th-generation tensor cores.
//
// Stands in for attention_prefill::encode / attention_fa8 and for AttGemm's
// prefill_ag_* passes (src/attention_prefill.rs:39-72, src/attention_gemm.rs:150-362,
// kernels/attention_prefill.metal, kernels/attention_gemm.metal) of the
// reference.  Same contract: token i of the chunk sees keys 0 ..= pos + i of the
// cache (which already holds the chunk's rows), the eight query heads of a kv
// head share its K/V, out = softmax(q K^T scale) V * sigmoid(gate).  The design
// is a single fused flash kernel instead of the reference's separate scores /
// softmax / PV passes through device memory:
//
//  * A tile is 128 query rows = 16 tokens x 8 heads of one kv head (row =
//    token*8 + head, the reference's GQA packing), so one K/V block feeds all
//    eight heads.  Persistent CTAs walk the tiles heaviest first.
//  * Sixteen warps in four warpgroups, registers moved between them with setmaxnreg: the
//    softmax warps (0..3, 168 registers), two tile I/O groups (4..7 and 8..11, 152) and the
//    copying / issuing warps (12..14, 40).
//  * Warp 12 streams 64-key K and V blocks into shared memory with TMA tensor
//    copies (128-byte swizzle, three stages each).
//  * Both left-hand operands live in tensor memory, not shared memory: the Q
//    tile (written once per tile with tcgen05.st) and P (written over the S
//    columns it was computed from).  Shared-memory traffic per block is then
//    only the TMA writes and the K / V operand reads, which is what lets the
//    MMA pipe run near its rate.  TMEM: O 256 columns, Q 128, and 128 for S and P: one S buffer of 64 and two
//    P buffers of 32 (16-bit cache), or two S buffers of 64 with P written over the scores (quantised cache).
//  * Two threads issue tcgen05.mma, because one thread needs longer to issue a
//    block's 20 instructions than the tensor pipe needs to run them: warp 13
//    issues S = Q K^T (128x64x256, A from TMEM) ahead of the softmax, and
//    warp 14 issues O += P V (128x256x64, A from TMEM, V read MN-major straight
//    from its [key][dim] rows).  Measured: a 128x64x16 score instruction occupies
//    the pipe for about 55 ns whatever its N up to 128 (a 128x256x16 P V
//    instruction for its nominal 70 ns), so the sixteen score instructions of a
//    block, not its flops, are most of its time.
//  * The softmax warps (one TMEM lane = one row per thread) read S with
//    tcgen05.ld, do the online softmax in log2 units, write P in V's 16-bit type
//    back to TMEM, and only rescale O in TMEM when the running maximum has grown
//    by more than 2^8.  The tile I/O warps move tiles in and out, two threads per
//    row (dims 0..127 and 128..255): the Q rows of the next tile are fetched into
//    registers early and go into TMEM as soon as the last S of the current tile
//    is done, then comes the current tile's epilogue, which reads O out of tensor
//    memory in one go and frees it before it fetches the gate values, so a tile
//    change stalls the MMAs as little as possible.  The
//    epilogue divides by l and applies the sigmoid gate (256-bit loads and
//    stores), or leaves (O, m, l) partials for a merge (across GPUs, or across the
//    two key halves a long-context tile is cut into).
//  * A quantised cache is read IN PLACE (the reference's attention_rows_q reads the codes per key
//    block, kernels/attention_rows_q.metal:16-31,206-344): the copy warp brings a block's codes,
//    scales and biases into a small staging area with tensor copies, one warpgroup turns them into
//    the binary16 operand tiles in shared memory -- s * c + z with one rounding, the reference's
//    round_trip_as_half (src/kv_quant.rs:121-126) -- in the swizzled layout the tensor cores read,
//    and the other tile I/O warpgroup takes whole rows.  No 16-bit copy of the cache exists in
//    device memory, and a chunk over a long prefix reads 1088 (576) bytes per key instead of 2048.
//  * All mbarrier waits are bounded; a wait that gives up sets the status word
//    and the CTA-wide abort flag, every role leaves its loop, and TMEM is freed.
#include <cuda.h>

#include <algorithm>

#include "host.hpp"

namespace saetta {

constexpr int kBM = 128;      // rows per tile
constexpr int kTokTile = 16;  // tokens per tile
constexpr int kBN = 64;       // keys per block
constexpr int kKChunk = kBN * 128;  // bytes of one 64-dim slab of a K or V block
constexpr int kKBytes = 4 * kKChunk;
constexpr int kPfStages = 3;
constexpr int kPfThreads = 512; // four warpgroups: softmax; tile I/O, first halves of the rows; tile I/O, second halves;
                                // TMA warp, S-MMA warp, P V-MMA warp and a spare
constexpr int kPfSmem = 2 * kPfStages * kKBytes + 1024 /*align*/ + 256 /*barriers*/ + 2 * 2 * kBM * 4 /*l, m per row, two tiles*/;
// Shared memory with a quantised cache (QBITS = 8 or 4): two operand stages, and two stages of codes (K and V
// of one kv head, 64 keys) with the four scale / bias arrays (both kv heads: 16 bytes per key and array).
template <int QBITS>
struct PfLayout {
    static constexpr int kOpStages = QBITS ? 2 : kPfStages;
    static constexpr int kCodeRow = kDim * QBITS / 8;          // bytes of one key's codes of one kv head
    static constexpr int kCodeSide = kBN * kCodeRow;           // 16 KB / 8 KB
    static constexpr int kParamArr = kBN * 16;                 // 1 KB
    static constexpr int kCodeStage = QBITS ? 2 * kCodeSide + 4 * kParamArr : 0;
    static constexpr int kCodeStages = QBITS ? 2 : 0;
    static constexpr int kSmem = 2 * kOpStages * kKBytes + kCodeStages * kCodeStage + 1024 /*align*/ + 256 /*barriers*/ + 2 * 2 * kBM * 4;
};
static_assert(PfLayout<0>::kSmem == kPfSmem, "the 16-bit layout is unchanged");
static_assert(PfLayout<8>::kSmem <= 227 * 1024 && PfLayout<4>::kSmem <= 227 * 1024, "fits a CTA's shared memory");
constexpr int kTmemO = 0, kTmemQ = 256, kTmemS = 384, kTmemP = 448; // TMEM columns: O, Q (2 values per column), S (64), two P buffers (32 each)
constexpr float kLog2ePf = 1.4426950408889634f;
constexpr float kPfRescale = 8.0f;

struct PfParams {
    const void *q; // 16-bit [tokens][heads][256]
    const float *q_and_gate;
    float *out, *part;
    uint32_t *status;
    uint32_t heads, kv_heads, pos, tokens, key_lo, key_hi;
    float scale_log2;
    uint32_t fmt;   // of Q and K: 0 binary16, 1 bfloat16 (also the UMMA format code)
    uint32_t v_fmt; // of V, and therefore of P (both operands of one MMA must share a format)
    uint32_t splits;      // each tile's key range is cut into this many work items (>1: partials per split)
    uint32_t part_stride; // floats between the partial buffers of consecutive splits
    uint32_t key_base;    // global position of row 0 of the K / V buffers
    uint32_t q_bf16;      // q arrives as bfloat16 but the key operands are binary16 (a quantised cache): converted on the way in
};

// ----------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// As tc_mma with the A operand in tensor memory (row m in lane m, two 16-bit values per column).
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 256-bit global accesses (one full 32-byte sector per thread); addresses 32-byte aligned.
struct alignas(32) Float8 {
    float v[8];
};
__device__ __forceinline__ Float8 ld_global_v8(const float *p) {
    Float8 r;
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_global_v8(float *p, const Float8 &r) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]),
                 "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7])
                 : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

#define SAETTA_R32(a, o)                                                                                              \
    "=r"(a[o + 0]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]), "=r"(a[o + 6]),    \
        "=r"(a[o + 7]), "=r"(a[o + 8]), "=r"(a[o + 9]), "=r"(a[o + 10]), "=r"(a[o + 11]), "=r"(a[o + 12]),             \
        "=r"(a[o + 13]), "=r"(a[o + 14]), "=r"(a[o + 15]), "=r"(a[o + 16]), "=r"(a[o + 17]), "=r"(a[o + 18]),          \
        "=r"(a[o + 19]), "=r"(a[o + 20]), "=r"(a[o + 21]), "=r"(a[o + 22]), "=r"(a[o + 23]), "=r"(a[o + 24]),          \
        "=r"(a[o + 25]), "=r"(a[o + 26]), "=r"(a[o + 27]), "=r"(a[o + 28]), "=r"(a[o + 29]), "=r"(a[o + 30]),          \
        "=r"(a[o + 31])
#define SAETTA_W32(a, o)                                                                                              \
    "r"(a[o + 0]), "r"(a[o + 1]), "r"(a[o + 2]), "r"(a[o + 3]), "r"(a[o + 4]), "r"(a[o + 5]), "r"(a[o + 6]),           \
        "r"(a[o + 7]), "r"(a[o + 8]), "r"(a[o + 9]), "r"(a[o + 10]), "r"(a[o + 11]), "r"(a[o + 12]), "r"(a[o + 13]),   \
        "r"(a[o + 14]), "r"(a[o + 15]), "r"(a[o + 16]), "r"(a[o + 17]), "r"(a[o + 18]), "r"(a[o + 19]),                \
        "r"(a[o + 20]), "r"(a[o + 21]), "r"(a[o + 22]), "r"(a[o + 23]), "r"(a[o + 24]), "r"(a[o + 25]),                \
        "r"(a[o + 26]), "r"(a[o + 27]), "r"(a[o + 28]), "r"(a[o + 29]), "r"(a[o + 30]), "r"(a[o + 31])

// 32 consecutive f32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : SAETTA_R32(r, 0)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::SAETTA_W32(r, 0), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle (cute::UMMA::SmemDescriptor:
// start address, leading and stride byte offsets in 16-byte units, version 1,
// layout type 2 in bits 61..63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = uint64_t((saddr & 0x3ffffu) >> 4);
    d |= uint64_t(lbo_bytes >> 4) << 16;
    d |= uint64_t(sbo_bytes >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}

struct PfTile {
    uint32_t tok0, kv, b_begin, nb, split;
};

// Work item `round` of this CTA: (token tile, kv head, key split), heaviest tiles first, snaking
// over the CTAs so that every CTA gets a similar mix.
__device__ __forceinline__ bool pf_tile(const PfParams &p, uint32_t round, PfTile &t) {
    const uint32_t tok_tiles = (p.tokens + kTokTile - 1) / kTokTile;
    const uint32_t per_tok_tile = p.kv_heads * p.splits;
    const uint32_t nitems = tok_tiles * per_tok_tile;
    const uint32_t G = gridDim.x, c = blockIdx.x;
    const uint32_t n = round * G + ((round & 1) ? G - 1 - c : c);
    if (n >= nitems) return false;
    const uint32_t tt = tok_tiles - 1 - n / per_tok_tile, rem = n % per_tok_tile;
    t.kv = rem / p.splits;
    t.split = rem % p.splits;
    t.tok0 = tt * kTokTile;
    const uint32_t hi = min(p.key_hi, p.pos + t.tok0 + kTokTile);
    const uint32_t b0 = p.key_lo / kBN;
    const uint32_t b1 = hi > p.key_lo ? (hi + kBN - 1) / kBN : b0;
    const uint32_t nb = b1 - b0;
    t.b_begin = b0 + uint32_t(uint64_t(nb) * t.split / p.splits);
    t.nb = b0 + uint32_t(uint64_t(nb) * (t.split + 1) / p.splits) - t.b_begin;
    return true;
}

// The six maps of a quantised cache: K and V codes (bytes [keys][kv heads][row]) and the four scale / bias arrays
// (binary16 [keys][kv heads * 4]); unused (copies of map_k) for a 16-bit cache.
struct PfQuantMaps {
    CUtensorMap kc, vc, ks, kz, vs, vz;
};

template <int QBITS>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               const __grid_constant__ PfQuantMaps qm, const PfParams p) {
    using L = PfLayout<QBITS>;
    constexpr int NST = L::kOpStages;
    // 16-bit cache: ONE S buffer, released by the softmax warps as soon as the scores are in their registers, and two P
    // buffers of their own (the next block's scores are computed while this block's softmax runs: measured 5-7 % faster).
    // Quantised cache: two S buffers with P written over the scores (there the converting warps bound the kernel, and
    // scores that run further ahead only take issue slots from them: measured 10 % slower with the single buffer).
    constexpr bool kOwnP = QBITS == 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sK = smem;                  // [NST][kKBytes]
    uint8_t *sV = sK + NST * kKBytes;    // [NST][kKBytes]
    uint8_t *sCode = sV + NST * kKBytes; // [2][K codes, V codes, k scales, k biases, v scales, v biases] (quantised cache only)
    uint64_t *bars = reinterpret_cast<uint64_t *>(sCode + L::kCodeStages * L::kCodeStage);
    uint64_t *q_full = bars + 0, *q_empty = bars + 1, *o_final = bars + 2, *o_empty = bars + 3, *k_full = bars + 4,
             *k_empty = bars + 7, *v_full = bars + 10, *v_empty = bars + 13, *s_full = bars + 16, *p_full = bars + 18,
             *pv_done = bars + 20, *lm_full = bars + 22, *code_full = bars + 26, *code_empty = bars + 28, *s_free = bars + 30;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 24);
    float *row_l = reinterpret_cast<float *>(bars + 32); // [2][128] row sums handed from the softmax warps
    float *row_m = row_l + 2 * kBM;                      // [2][128] running maxima (log2 units)
    volatile uint32_t *abort_flag = tmem_slot + 1;
    volatile uint32_t *never_set = tmem_slot + 2; // stays 0: for waits that must ignore the abort flag

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
                mbar_init(q_full, 8), mbar_init(q_empty, 1), mbar_init(o_final, 1), mbar_init(o_empty, 8);
        // (with a quantised cache the eight tile I/O warps fill the operand stages)
        for (int s = 0; s < NST; s++)
            mbar_init(&k_full[s], QBITS ? 8 : 1), mbar_init(&k_empty[s], 1), mbar_init(&v_full[s], QBITS ? 8 : 1), mbar_init(&v_empty[s], 1);
        for (int s = 0; s < L::kCodeStages; s++) mbar_init(&code_full[s], 1), mbar_init(&code_empty[s], 8);
        for (int s = 0; s < 2; s++)
            mbar_init(&s_full[s], 1), mbar_init(&p_full[s], 4), mbar_init(&pv_done[s], 1), mbar_init(&lm_full[s], 4);
        mbar_init(s_free, 4);
        *abort_flag = 0;
        *never_set = 0;
        mbar_fence_init();
    }
    if (warp == 13) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + kTmemO, tmem_q = tmem + kTmemQ, tmem_s = tmem + kTmemS, tmem_p = tmem + kTmemP;

    auto give_up = [&](uint32_t bit) {
        atomicOr(p.status, bit);
        *abort_flag = 1;
    };

    // Registers follow the work: the softmax warps hold a 64-wide score row and the tile I/O warps
    // chunks of O and of the gate, the issuing and copying threads next to nothing.
    // (Each warpgroup meets its own setmaxnreg, and the code of its roles follows it directly, so
    // that the compiler allocates each role within its own limit.)
    if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 12) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t g = 0, tc = 0;
            bool ok = true;
            PfTile t;
            for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                if (!t.nb) continue;
                for (uint32_t b = 0; b < t.nb; b++, g++) {
                    const uint32_t st = g % NST, ph = (g / NST) & 1;
                    const int key0 = int((t.b_begin + b) * kBN) - int(p.key_base); // row of the buffer
                    if constexpr (QBITS != 0) {
                        // the block's codes (this kv head's) and the four scale / bias arrays (both kv heads: 16
                        // bytes per key, the smallest tensor copy) into a code stage; the converting warpgroup
                        // makes the operand tiles
                        const uint32_t cs = g & 1, cph = (g >> 1) & 1;
                        if (!mbar_wait(&code_empty[cs], cph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); ok = false; break; }
                        uint8_t *dst = sCode + cs * L::kCodeStage;
                        mbar_expect_tx(&code_full[cs], L::kCodeStage);
                        tma_load_3d(dst, &qm.kc, &code_full[cs], 0, int(t.kv), key0);
                        tma_load_3d(dst + L::kCodeSide, &qm.vc, &code_full[cs], 0, int(t.kv), key0);
                        tma_load_2d(dst + 2 * L::kCodeSide, &qm.ks, &code_full[cs], 0, key0);
                        tma_load_2d(dst + 2 * L::kCodeSide + L::kParamArr, &qm.kz, &code_full[cs], 0, key0);
                        tma_load_2d(dst + 2 * L::kCodeSide + 2 * L::kParamArr, &qm.vs, &code_full[cs], 0, key0);
                        tma_load_2d(dst + 2 * L::kCodeSide + 3 * L::kParamArr, &qm.vz, &code_full[cs], 0, key0);
                    } else {
                        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); ok = false; break; }
                        mbar_expect_tx(&k_full[st], kKBytes);
                        for (int c = 0; c < 4; c++) tma_load_3d(sK + st * kKBytes + c * kKChunk, &map_k, &k_full[st], c * 64, int(t.kv), key0);
                        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); ok = false; break; }
                        mbar_expect_tx(&v_full[st], kKBytes);
                        for (int c = 0; c < 4; c++) tma_load_3d(sV + st * kKBytes + c * kKChunk, &map_v, &v_full[st], c * 64, int(t.kv), key0);
                    }
                }
                tc++;
            }
            // On the way out after a failed wait, let the copies already issued land
            // (bounded) so that no copy is in flight when the CTA's shared memory is released.
            if (*abort_flag) {
                if constexpr (QBITS != 0) {
                    for (uint32_t k = g > 2 ? g - 2 : 0; k < g; k++) mbar_wait(&code_full[k & 1], (k >> 1) & 1, never_set, 200000u);
                } else {
                    for (uint32_t k = g > NST ? g - NST : 0; k < g; k++) {
                        mbar_wait(&k_full[k % NST], (k / NST) & 1, never_set, 200000u);
                        mbar_wait(&v_full[k % NST], (k / NST) & 1, never_set, 200000u);
                    }
                }
            }
        }
    } else if (warp == 13) {
        // ------------------------------------------------------------ MMA issuer for S = Q K^T
        // Two threads issue MMAs, this one the score products and warp 14 the P V products: one
        // thread alone spends longer issuing the 20 instructions of a block than the tensor
        // pipe needs to run them.  There is ONE S buffer: the softmax warps release it as soon as the
        // scores are in their registers (s_free), so the next block's scores are computed while the
        // softmax of this one runs; P has buffers of its own.
        if (lane == 0) {
            const uint32_t idesc_s = (1u << 4) | (p.fmt << 7) | (p.fmt << 10) | (uint32_t(kBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
            const uint32_t k_addr = smem_u32(sK);
            uint32_t g = 0, tc = 0;
            bool ok = true;
            PfTile t;
            for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                if (!t.nb) continue;
                if (!mbar_wait(q_full, tc & 1, abort_flag)) { give_up(kStatusFullTimeout); break; }
                for (uint32_t b = 0; b < t.nb; b++, g++) {
                    const uint32_t st = g % NST, ph = (g / NST) & 1, sb = g & 1;
                    if (!mbar_wait(&k_full[st], ph, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                    if (!mbar_wait(kOwnP ? s_free : &pv_done[sb], kOwnP ? (g & 1) ^ 1 : ((g >> 1) & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after();
                    const uint64_t bd0 = umma_desc(k_addr + st * kKBytes, 16, 1024);
#pragma unroll
                    for (int ks = 0; ks < kDim / 16; ks++) {
                        // the descriptor's address field counts 16-byte units: +2 per 16-value k-step
                        // inside a 64-value slab, one slab further every fourth step
                        const uint64_t bd = bd0 + uint64_t(((ks >> 2) * kKChunk + (ks & 3) * 32) >> 4);
                        tc_mma_ts(tmem_s + (kOwnP ? 0 : sb * kBN), tmem_q + ks * 8, bd, idesc_s, ks > 0);
                    }
                    tc_commit(&k_empty[st]);
                    tc_commit(&s_full[sb]);
                }
                if (!ok) break;
                tc_commit(q_empty); // every S of this tile has been issued
                tc++;
            }
        }
    } else if (warp == 14) {
        // ------------------------------------------------------------ MMA issuer for O += P V
        if (lane == 0) {
            const uint32_t idesc_o = (1u << 4) | (p.v_fmt << 7) | (p.v_fmt << 10) | (1u << 16) | (uint32_t(kDim >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
            const uint32_t v_addr = smem_u32(sV);
            uint32_t g = 0, tc = 0;
            bool ok = true;
            PfTile t;
            for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                if (!t.nb) continue;
                for (uint32_t b = 0; b < t.nb; b++, g++) {
                    const uint32_t st = g % NST, ph = (g / NST) & 1, sb = g & 1, sph = (g >> 1) & 1;
                    if (!mbar_wait(&p_full[sb], sph, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    if (!mbar_wait(&v_full[st], ph, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                    if (b == 0 && !mbar_wait(o_empty, (tc & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after();
                    // V is MN-major: 64 dims (128 B) x 8 keys per swizzle atom; next 64 dims one slab on
                    // (leading offset), next 8 keys 1024 B on (stride offset); 16 keys per MMA.
                    const uint64_t bd0 = umma_desc(v_addr + st * kKBytes, kKChunk, 1024);
#pragma unroll
                    for (int ks = 0; ks < kBN / 16; ks++)
                        tc_mma_ts(tmem_o, (kOwnP ? tmem_p + sb * 32 : tmem_s + sb * kBN) + ks * 8, bd0 + uint64_t((ks * 2048) >> 4), idesc_o, (b > 0 || ks > 0) ? 1u : 0u);
                    tc_commit(&v_empty[st]);
                    tc_commit(&pv_done[sb]);
                    if (b + 1 == t.nb) tc_commit(o_final);
                }
                tc++;
            }
        }
    }
    } else if (warp < 4) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
        // ------------------------------------------------------------ softmax and correction
        const uint32_t quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t g = 0, tc = 0;
        bool ok = true;
        PfTile t;
        for (uint32_t round = 0; pf_tile(p, round, t); round++) {
            if (!t.nb) continue;
            const uint32_t tok = t.tok0 + (row >> 3);
            const uint32_t lim_hi = min(p.key_hi, p.pos + tok + 1); // keys [key_lo, lim_hi) are visible
            float m_ref = -INFINITY, l = 0.f;
            for (uint32_t b = 0; ok && b < t.nb; b++, g++) {
                const uint32_t st = g & 1, ph = (g >> 1) & 1;
                const uint32_t key0 = (t.b_begin + b) * kBN;
                if (!mbar_wait(&s_full[st], ph, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld32(tmem_s + lane_addr + (kOwnP ? 0 : st * kBN), sr[0]);
                tmem_ld32(tmem_s + lane_addr + (kOwnP ? 0 : st * kBN) + 32, sr[1]);
                tmem_wait_ld();
                if constexpr (kOwnP) { // the scores are in registers: the S buffer is free for the next block's product
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s_free);
                }

                // raw scores; the positive scale (in log2 units) is folded into the exponent's FFMA
                float s[64];
#pragma unroll
                for (int c = 0; c < 64; c++) s[c] = __uint_as_float(sr[c >> 5][c & 31]);
                const bool edge = key0 < p.key_lo || key0 + kBN > min(p.key_hi, p.pos + t.tok0 + 1);
                if (edge) {
#pragma unroll
                    for (int c = 0; c < 64; c++)
                        if (key0 + c < p.key_lo || key0 + c >= lim_hi) s[c] = -INFINITY;
                }
                float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
                for (int c = 4; c < 64; c++) m4[c & 3] = fmaxf(m4[c & 3], s[c]);
                const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
                // O is only rescaled when the maximum has moved by more than 2^8
                const bool need = mx > m_ref + kPfRescale;
                float factor = 1.f;
                if (need) {
                    factor = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - mx);
                    m_ref = mx;
                    l *= factor;
                }
                if (b > 0 && __any_sync(0xffffffffu, need)) {
                    // P V of the block before must have landed in O before O is touched
                    const uint32_t gp = g - 1;
                    if (!mbar_wait(&pv_done[gp & 1], (gp >> 1) & 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < kDim; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_o + lane_addr + c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int k = 0; k < 32; k++) o[k] = __float_as_uint(__uint_as_float(o[k]) * factor);
                        tmem_st32(tmem_o + lane_addr + c, o);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                // P (two values per column) into its own buffer, or over the first 32 columns of the S buffer it came from
                uint32_t pw[32];
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < 32; k++) {
                    const float a = ex2_approx(fmaf(s[2 * k], p.scale_log2, -m_use));
                    const float bb = ex2_approx(fmaf(s[2 * k + 1], p.scale_log2, -m_use));
                    sum4[k & 3] += a + bb;
                    if (p.v_fmt) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(a, bb);
                        pw[k] = *reinterpret_cast<uint32_t *>(&h);
                    } else {
                        pw[k] = pack_half2(a, bb);
                    }
                }
                if constexpr (kOwnP) { // P buffer g & 1: the P V product of two blocks ago has read it
                    if (!mbar_wait(&pv_done[st], ph ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after();
                }
                tmem_st32((kOwnP ? tmem_p + st * 32 : tmem_s + st * kBN) + lane_addr, pw);
                tmem_wait_st();
                const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                l += sum;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[st]);
            }
            if (!ok) break;
            // hand the row's sum and maximum to the tile I/O warps and go on to the next tile
            row_l[(tc & 1) * kBM + row] = l;
            row_m[(tc & 1) * kBM + row] = m_ref;
            __syncwarp();
            if (lane == 0) mbar_arrive(&lm_full[tc & 1]);
            tc++;
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
        // ------------------------------------------------------------ tile I/O: Q rows in, results out
        // Per tile these warps write its Q rows into tensor memory and, at its end, scale and gate
        // O out to memory.  The Q rows of tile k+1 go in as soon as the last S of tile k has been
        // computed, before tile k's epilogue, so the MMA warp never waits for a tile change.
        // Two threads per row: the warps of the first tile I/O warpgroup take dims 0..127 of Q, the
        // gate and O, those of the second dims 128..255.
        // With a quantised cache the same eight warps also make the operand tiles, between a tile's Q
        // rows and its epilogue: per 64-key block they wait for its codes and for a free operand stage,
        // write K (then V) as s * c + z rounded once to binary16 -- the code as an exact binary16
        // integer (byte permute onto the magic 1024, minus 1024), then one fused multiply-add with the
        // group's scale and bias -- into the four 64-dim slabs of the stage in the tensor cores'
        // 128-byte-swizzled layout, and hand the stage to the MMA warps.  A lane reads 16 bytes of
        // codes; eight lanes cover 128 bytes of a key's row, a warp four keys at a time, the eight
        // warps 8 keys each.  (Four warps of their own for this, one per scheduler, were measured at
        // 2.3 us per block against the 1.1 us the MMAs take: chains of dependent instructions with
        // nothing to switch to.)
        const uint32_t quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t half_lo = warp >= 8 ? 1u : 0u;
        const uint32_t cw = warp - 4;
        constexpr uint32_t kMagic = 0x64646464u, k1024 = 0x64006400u;
        uint32_t cg = 0; // blocks converted so far (the copy warp's and the MMA warps' count)
        auto convert_side = [&](const uint8_t *codes, const uint8_t *sc, const uint8_t *bi, uint8_t *dst, uint32_t kv) {
            constexpr int QB = QBITS ? QBITS : 8;              // (this role is never taken with a 16-bit cache)
            constexpr int kValsPerLoad = 128 / QB;             // values in a lane's 16 bytes: 16 or 32
            constexpr int kLoadsPerRow = kDim * QB / 8 / 128;  // 128-byte pieces of a key's row: 2 or 1
            const uint32_t col = lane & 7;
            // every load of the side first: the compiler may not move a shared-memory load above the
            // stores of the piece before (for all it knows they alias), and one piece after the other
            // is a chain of latencies
            uint4 cin[2][kLoadsPerRow];
            uint32_t sin[2][kLoadsPerRow], zin[2][kLoadsPerRow];
#pragma unroll
            for (int it = 0; it < 2; it++) {
                const uint32_t key = cw * 8 + it * 4 + (lane >> 3);
#pragma unroll
                for (int piece = 0; piece < kLoadsPerRow; piece++) {
                    const uint32_t G = ((piece * 8 + col) * kValsPerLoad) >> 6;
                    cin[it][piece] = *reinterpret_cast<const uint4 *>(codes + key * L::kCodeRow + piece * 128 + col * 16);
                    sin[it][piece] = *reinterpret_cast<const uint16_t *>(sc + key * 16 + (kv * 4 + G) * 2);
                    zin[it][piece] = *reinterpret_cast<const uint16_t *>(bi + key * 16 + (kv * 4 + G) * 2);
                }
            }
#pragma unroll
            for (int it = 0; it < 2; it++) {
                const uint32_t key = cw * 8 + it * 4 + (lane >> 3);
#pragma unroll
                for (int piece = 0; piece < kLoadsPerRow; piece++) {
                    const uint4 cw4 = cin[it][piece];
                    const uint32_t d0 = (piece * 8 + col) * kValsPerLoad; // first dim of these values
                    const uint32_t s2 = prmt(sin[it][piece], 0u, 0x1010), z2 = prmt(zin[it][piece], 0u, 0x1010);
                    const uint32_t w4[4] = {cw4.x, cw4.y, cw4.z, cw4.w};
                    uint32_t h[kValsPerLoad / 2]; // pairs of consecutive dims
                    if (QB == 8) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            h[2 * j] = hfma2_u32(hsub2_u32(prmt(w4[j], kMagic, 0x4140), k1024), s2, z2);
                            h[2 * j + 1] = hfma2_u32(hsub2_u32(prmt(w4[j], kMagic, 0x4342), k1024), s2, z2);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint32_t even = w4[j] & 0x0f0f0f0fu, odd = (w4[j] >> 4) & 0x0f0f0f0fu; // nibbles 0,2,4,6 / 1,3,5,7
                            const uint32_t n03 = prmt(even, odd, 0x5140), n47 = prmt(even, odd, 0x7362); // bytes n0 n1 n2 n3 / n4..n7
                            h[4 * j] = hfma2_u32(hsub2_u32(prmt(n03, kMagic, 0x4140), k1024), s2, z2);
                            h[4 * j + 1] = hfma2_u32(hsub2_u32(prmt(n03, kMagic, 0x4342), k1024), s2, z2);
                            h[4 * j + 2] = hfma2_u32(hsub2_u32(prmt(n47, kMagic, 0x4140), k1024), s2, z2);
                            h[4 * j + 3] = hfma2_u32(hsub2_u32(prmt(n47, kMagic, 0x4342), k1024), s2, z2);
                        }
                    }
                    // 16-byte chunks (8 dims) of the key's 128-byte row in slab d / 64, swizzled by the key.
                    // The eight lanes that share a key store chunks of different slabs at once; which of its
                    // chunks a lane stores first is rotated by the lane's slab, so that the eight stores of
                    // a request fall into eight different 16-byte bank groups (unrotated, lanes of different
                    // slabs write the same chunk number: the stores, the largest user of shared-memory
                    // bandwidth here, then cost twice or four times as much).
                    uint8_t *rowp = dst + (d0 >> 6) * kKChunk + key * 128;
                    constexpr int NC = kValsPerLoad / 8; // chunks per lane: 2 or 4
                    const uint32_t rot = QB == 8 ? (col >> 2) : (col >> 1); // this lane's slab among those of the request
                    if (NC == 2) {
                        if (rot & 1) {
#pragma unroll
                            for (int e = 0; e < 4; e++) { const uint32_t x = h[e]; h[e] = h[4 + e]; h[4 + e] = x; }
                        }
                    } else {
                        if (rot & 1) { // rotate the four chunks left by one
#pragma unroll
                            for (int e = 0; e < 4; e++) { const uint32_t x = h[e]; h[e] = h[4 + e]; h[4 + e] = h[8 + e]; h[8 + e] = h[12 + e]; h[12 + e] = x; }
                        }
                        if (rot & 2) { // ... by two
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const uint32_t x = h[e], y = h[4 + e];
                                h[e] = h[8 + e], h[4 + e] = h[12 + e], h[8 + e] = x, h[12 + e] = y;
                            }
                        }
                    }
#pragma unroll
                    for (int c = 0; c < NC; c++) { // register set c now holds the lane's chunk (c + rot) % NC
                        const uint32_t chunk = ((d0 & 63) >> 3) + ((c + rot) & (NC - 1));
                        *reinterpret_cast<uint4 *>(rowp + ((chunk ^ (key & 7)) << 4)) = make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
                    }
                }
            }
        };

        const uint32_t lane_addr = (quarter * 32) << 16;
        struct RowOf {
            uint32_t tok;
            bool live;
            size_t rh;
            float *part;
        };
        auto row_of = [&](const PfTile &t) {
            RowOf r;
            r.tok = t.tok0 + (row >> 3);
            r.live = r.tok < p.tokens;
            r.rh = size_t(r.tok) * p.heads + t.kv * kHeadsPerKv + (row & 7);
            r.part = p.part ? p.part + size_t(t.split) * p.part_stride : nullptr;
            return r;
        };
        // next work item with keys to visit; items without any get their empty partial here
        auto next_item = [&](uint32_t &round, PfTile &t) -> bool {
            while (pf_tile(p, round, t)) {
                round++;
                if (t.nb) return true;
                const RowOf r = row_of(t);
                if (r.live && r.part) {
                    float *dst = r.part + r.rh * kPartStride;
                    for (uint32_t d = half_lo * 128; d < half_lo * 128 + 128; d++) dst[d] = 0.f;
                    if (!half_lo) dst[kPartM] = -INFINITY, dst[kPartL] = 0.f;
                }
            }
            return false;
        };
        auto convert_item = [&](const PfTile &t) -> bool {
            for (uint32_t b = 0; b < t.nb; b++, cg++) {
                const uint32_t st = cg % NST, ph = (cg / NST) & 1, cs = cg & 1, cph = (cg >> 1) & 1;
                const uint8_t *code = sCode + cs * L::kCodeStage;
                if (!mbar_wait(&code_full[cs], cph, abort_flag)) { give_up(kStatusFullTimeout); return false; }
                if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); return false; }
                convert_side(code, code + 2 * L::kCodeSide, code + 2 * L::kCodeSide + L::kParamArr, sK + st * kKBytes, t.kv);
                fence_async_smem(); // the tensor cores read the stage through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&k_full[st]);
                if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); return false; }
                convert_side(code + L::kCodeSide, code + 2 * L::kCodeSide + 2 * L::kParamArr, code + 2 * L::kCodeSide + 3 * L::kParamArr,
                             sV + st * kKBytes, t.kv);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&v_full[st]);
                    mbar_arrive(&code_empty[cs]);
                }
            }
            return true;
        };
        auto load_q = [&](const PfTile &t, uint32_t k) -> bool {
            const RowOf r = row_of(t);
            const bool row_live = r.live;
            const size_t rh = r.rh;
            if (row_live && p.out) { // pull this row's gate values towards L2 for the epilogue
                const char *gpf = reinterpret_cast<const char *>(p.q_and_gate + rh * 2 * kDim + kDim + half_lo * 128);
#pragma unroll
                for (int j = 0; j < 4; j++) prefetch_l2(gpf + j * 128);
            }
            // this thread's part of its Q row into tensor memory (two values per column), once the
            // MMAs of the tile before no longer read the old one.  The row does not depend on that
            // wait: its first half is fetched into registers before it.
            bool waited = false;
            auto q_half = [&](const uint32_t half) -> bool {
                const uint4 *qrow = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.q) + rh * kDim + half * 128);
                uint4 qv[16];
#pragma unroll
                for (int j = 0; j < 16; j++) qv[j] = row_live ? qrow[j] : make_uint4(0u, 0u, 0u, 0u);
                if (p.q_bf16) { // bfloat16 queries over binary16 operand tiles: exact unless outside binary16's range
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        uint32_t *w = reinterpret_cast<uint32_t *>(&qv[j]);
#pragma unroll
                        for (int e = 0; e < 4; e++) w[e] = pack_half2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
                    }
                }
                if (!waited) {
                    if (!mbar_wait(q_empty, (k & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
                    tc_fence_after();
                    waited = true;
                }
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t w[32];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint4 v = qv[c * 8 + j];
                        w[4 * j] = v.x, w[4 * j + 1] = v.y, w[4 * j + 2] = v.z, w[4 * j + 3] = v.w;
                    }
                    tmem_st32(tmem_q + lane_addr + half * 64 + c * 32, w);
                }
                return true;
            };
            if (!q_half(half_lo)) return false;
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
            return true;
        };
        auto epilogue = [&](const PfTile &t, uint32_t k) -> bool {
            const RowOf r = row_of(t);
            const bool row_live = r.live;
            const size_t rh = r.rh;
            float *part = r.part;
            // A half of O leaves tensor memory in one go (128 values), so that the next tile's P V
            // products wait for four tensor-memory loads and nothing else; the gate values, which come
            // from global memory, are fetched afterwards, one 32-byte step ahead of their use.
            // (256-bit loads and stores: a thread's accesses are whole 32-byte sectors of its row)
            const bool gated = row_live && p.out;
            if (!mbar_wait(&lm_full[k & 1], (k >> 1) & 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
            const float l = row_l[(k & 1) * kBM + row], m_ref = row_m[(k & 1) * kBM + row];
            if (!mbar_wait(o_final, k & 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
            tc_fence_after();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
            auto o_half = [&](const uint32_t half, const bool last) {
                const float *gp = p.q_and_gate + (gated ? rh * 2 * kDim + kDim + half * 128 : 0);
                uint32_t o[4][32];
#pragma unroll
                for (int ch = 0; ch < 4; ch++) tmem_ld32(tmem_o + lane_addr + half * 128 + ch * 32, o[ch]);
                tmem_wait_ld();
                if (last) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_empty); // O has left tensor memory: the next tile's P V products may start
                }
                if (row_live) {
                    if (p.out) {
                        float *op = p.out + rh * kDim + half * 128;
                        Float8 g = ld_global_v8(gp);
#pragma unroll
                        for (int st = 0; st < 16; st++) {
                            Float8 gn = g;
                            if (st + 1 < 16) gn = ld_global_v8(gp + (st + 1) * 8);
                            Float8 v;
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                v.v[e] = __uint_as_float(o[st >> 2][8 * (st & 3) + e]) * __fdividef(inv_l, 1.f + __expf(-g.v[e]));
                            st_global_v8(op + st * 8, v);
                            g = gn;
                        }
                    } else {
                        float4 *op = reinterpret_cast<float4 *>(part + rh * kPartStride + half * 128);
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            op[j] = make_float4(__uint_as_float(o[j >> 3][4 * (j & 7)]), __uint_as_float(o[j >> 3][4 * (j & 7) + 1]),
                                                __uint_as_float(o[j >> 3][4 * (j & 7) + 2]), __uint_as_float(o[j >> 3][4 * (j & 7) + 3]));
                    }
                }
            };
            o_half(half_lo, true);
            if (row_live && part && !half_lo) {
                part[rh * kPartStride + kPartM] = m_ref;
                part[rh * kPartStride + kPartL] = l;
            }
            return true;
        };
        uint32_t round = 0, k = 0;
        PfTile cur, nxt;
        bool have = next_item(round, cur);
        if (have && !load_q(cur, 0)) have = false;
        while (have) {
            if constexpr (QBITS != 0)
                if (!convert_item(cur)) break;
            const bool more = next_item(round, nxt);
            if (more && !load_q(nxt, k + 1)) break;
            if (!epilogue(cur, k)) break;
            cur = nxt, have = more, k++;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 13) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

// ----------------------------------------------------------------- the wide kernel (16-bit caches)
//
// Same tiles, same work items, same results as prefill_kernel<0>; what differs is the shape of the score product.
// A tcgen05.mma of 128 rows x N x 16 occupies the tensor pipe for about 55 ns whatever N is, up to 128, so the
// scores are computed 128 keys at a time (sixteen instructions per 128 keys instead of per 64).  Tensor memory
// has no room for that beside the 256-column O: O 256 + S 128 + P 64 leave 64 columns, so only dims 0..127 of the
// Q tile live in tensor memory; dims 128..255 sit in shared memory (written once per tile, in the swizzled
// K-major layout) and are the A operand of the second half of a block's score instructions.  K travels in
// half-stages of 128 keys x 128 dims (a ring of three), V in stages of 64 keys x 256 dims as before.
// Eight softmax warps, two per row (keys 0..63 and 64..127 of the block): they exchange their maxima through
// shared memory, release S as soon as the scores are in registers (the next block's scores are computed during
// this block's softmax) and write P into its own 64 columns.  Four tile I/O warps, one thread per row.  Two copying
// threads (K; V) and two issuing threads (scores; P V).
constexpr int kWBN = 128;                       // keys per score block
constexpr int kWKHalf = kWBN * 128 * 2;         // bytes of a K half-stage: 128 keys x 128 dims, two slabs of [128][128 B]
constexpr int kWKSlab = kWBN * 128;             // 16 KB
constexpr int kWKStages = 3, kWVStages = 2;
constexpr int kWQHi = kBM * 128 * 2;            // dims 128..255 of the Q tile: 32 KB, two slabs of [128 rows][128 B]
constexpr int kWTmemO = 0, kWTmemQ = 256, kWTmemS = 320, kWTmemP = 448;
constexpr int kWSmem = kWKStages * kWKHalf + kWVStages * kKBytes + kWQHi + 1024 /*align*/ + 512 /*barriers*/ +
                       (2 * 2 + 2) * kBM * 4 /*l per half and tile, m per tile*/ + 2 * 2 * kBM * 8 /*maxima per half and parity, tagged*/;
static_assert(kWSmem <= 227 * 1024, "shared memory of the wide prefill kernel");

__global__ void __launch_bounds__(kPfThreads, 1)
prefill_wide_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const PfParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sK = smem;                              // [3][2 slabs][128 keys][128 B]
    uint8_t *sV = sK + kWKStages * kWKHalf;          // [2][4 slabs][64 keys][128 B]
    uint8_t *sQ = sV + kWVStages * kKBytes;          // [2 slabs][128 rows][128 B]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sQ + kWQHi);
    uint64_t *q_full = bars + 0, *q_empty = bars + 1, *o_final = bars + 2, *o_empty = bars + 3, *k_full = bars + 4,
             *k_empty = bars + 7, *v_full = bars + 10, *v_empty = bars + 12, *s_full = bars + 14, *s_free = bars + 15,
             *p_full = bars + 16, *pv_done = bars + 17, *lm_full = bars + 18;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 20);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    volatile uint32_t *never_set = tmem_slot + 2;
    float *row_l = reinterpret_cast<float *>(bars + 64); // [2 tiles][2 halves][128]
    float *row_m = row_l + 2 * 2 * kBM;                  // [2 tiles][128]
    volatile unsigned long long *xmax = reinterpret_cast<volatile unsigned long long *>(row_m + 2 * kBM); // [2 parities][2 halves][128]: (maximum, block number + 1)

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    xmax[threadIdx.x] = 0ull; // 2 x 2 x 128 words = the block's 512 threads: tag 0 is no block's number
    if (threadIdx.x == 0) {
        mbar_init(q_full, 4), mbar_init(q_empty, 1), mbar_init(o_final, 1), mbar_init(o_empty, 4);
        for (int s = 0; s < kWKStages; s++) mbar_init(&k_full[s], 1), mbar_init(&k_empty[s], 1);
        for (int s = 0; s < kWVStages; s++) mbar_init(&v_full[s], 1), mbar_init(&v_empty[s], 1);
        mbar_init(s_full, 1), mbar_init(s_free, 8), mbar_init(p_full, 8), mbar_init(pv_done, 1);
        mbar_init(&lm_full[0], 8), mbar_init(&lm_full[1], 8);
        *abort_flag = 0;
        *never_set = 0;
        mbar_fence_init();
    }
    if (warp == 13) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + kWTmemO, tmem_q = tmem + kWTmemQ, tmem_s = tmem + kWTmemS, tmem_p = tmem + kWTmemP;
    auto give_up = [&](uint32_t bit) {
        atomicOr(p.status, bit);
        *abort_flag = 1;
    };
    // a work item's keys in blocks of 128 from its first 64-key block on; the last may be half a block
    auto wide_blocks = [](const PfTile &t) { return (t.nb + 1) >> 1; };

    if (warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 12) {
            // ------------------------------------------------------------ K copies: a half-stage = 128 keys x 128 dims
            if (lane == 0) {
                uint32_t hs = 0; // half-stages copied so far
                bool ok = true;
                PfTile t;
                for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                    for (uint32_t w = 0; ok && w < wide_blocks(t); w++)
                        for (uint32_t j = 0; j < 2; j++, hs++) {
                            const uint32_t st = hs % kWKStages, ph = (hs / kWKStages) & 1;
                            const int key0 = int(t.b_begin * kBN + w * kWBN) - int(p.key_base);
                            if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); ok = false; break; }
                            mbar_expect_tx(&k_full[st], kWKHalf);
                            for (int c = 0; c < 2; c++)
                                tma_load_3d(sK + st * kWKHalf + c * kWKSlab, &map_k, &k_full[st], int(j) * 128 + c * 64, int(t.kv), key0);
                        }
                }
                if (*abort_flag)
                    for (uint32_t k = hs > uint32_t(kWKStages) ? hs - kWKStages : 0; k < hs; k++)
                        mbar_wait(&k_full[k % kWKStages], (k / kWKStages) & 1, never_set, 200000u);
            }
        } else if (warp == 15) {
            // ------------------------------------------------------------ V copies: a stage = 64 keys x 256 dims
            if (lane == 0) {
                uint32_t vs = 0;
                bool ok = true;
                PfTile t;
                for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                    for (uint32_t b = 0; b < t.nb; b++, vs++) {
                        const uint32_t st = vs % kWVStages, ph = (vs / kWVStages) & 1;
                        const int key0 = int((t.b_begin + b) * kBN) - int(p.key_base);
                        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { give_up(kStatusEmptyTimeout); ok = false; break; }
                        mbar_expect_tx(&v_full[st], kKBytes);
                        for (int c = 0; c < 4; c++) tma_load_3d(sV + st * kKBytes + c * kKChunk, &map_v, &v_full[st], c * 64, int(t.kv), key0);
                    }
                }
                if (*abort_flag)
                    for (uint32_t k = vs > uint32_t(kWVStages) ? vs - kWVStages : 0; k < vs; k++)
                        mbar_wait(&v_full[k % kWVStages], (k / kWVStages) & 1, never_set, 200000u);
            }
        } else if (warp == 13) {
            // ------------------------------------------------------------ score products: 128 rows x 128 keys x 256 dims
            if (lane == 0) {
                const uint32_t idesc_s = (1u << 4) | (p.fmt << 7) | (p.fmt << 10) | (uint32_t(kWBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
                const uint32_t k_addr = smem_u32(sK), q_addr = smem_u32(sQ);
                uint32_t g = 0, hs = 0, tc = 0;
                bool ok = true;
                PfTile t;
                for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                    if (!t.nb) continue;
                    if (!mbar_wait(q_full, tc & 1, abort_flag)) { give_up(kStatusFullTimeout); break; }
                    for (uint32_t w = 0; ok && w < wide_blocks(t); w++, g++) {
                        if (!mbar_wait(s_free, (g & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                        for (uint32_t j = 0; j < 2; j++, hs++) {
                            const uint32_t st = hs % kWKStages, ph = (hs / kWKStages) & 1;
                            if (!mbar_wait(&k_full[st], ph, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                            tc_fence_after();
#pragma unroll
                            for (int ks = 0; ks < 8; ks++) {
                                // 16 dims per instruction: 32 bytes further inside a 64-dim slab, one slab on after four
                                const uint32_t off = uint32_t((ks >> 2) * kWKSlab + (ks & 3) * 32);
                                const uint64_t bd = umma_desc(k_addr + st * kWKHalf + off, 16, 1024);
                                if (j == 0) tc_mma_ts(tmem_s, tmem_q + ks * 8, bd, idesc_s, ks > 0);
                                else tc_mma(tmem_s, umma_desc(q_addr + off, 16, 1024), bd, idesc_s, 1u);
                            }
                            tc_commit(&k_empty[st]);
                        }
                        if (!ok) break;
                        tc_commit(s_full);
                    }
                    if (!ok) break;
                    tc_commit(q_empty); // every score product of this tile has been issued
                    tc++;
                }
            }
        } else {
            // ------------------------------------------------------------ O += P V, 64 keys (one V stage) at a time
            if (lane == 0) {
                const uint32_t idesc_o = (1u << 4) | (p.v_fmt << 7) | (p.v_fmt << 10) | (1u << 16) | (uint32_t(kDim >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
                const uint32_t v_addr = smem_u32(sV);
                uint32_t g = 0, vs = 0, tc = 0;
                bool ok = true;
                PfTile t;
                for (uint32_t round = 0; ok && pf_tile(p, round, t); round++) {
                    if (!t.nb) continue;
                    for (uint32_t w = 0; ok && w < wide_blocks(t); w++, g++) {
                        if (!mbar_wait(p_full, g & 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                        const uint32_t halves = min(2u, t.nb - 2 * w);
                        for (uint32_t j = 0; j < halves; j++, vs++) {
                            const uint32_t st = vs % kWVStages, ph = (vs / kWVStages) & 1;
                            if (!mbar_wait(&v_full[st], ph, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                            if (w == 0 && j == 0 && !mbar_wait(o_empty, (tc & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                            tc_fence_after();
                            const uint64_t bd0 = umma_desc(v_addr + st * kKBytes, kKChunk, 1024);
#pragma unroll
                            for (int ks = 0; ks < kBN / 16; ks++)
                                tc_mma_ts(tmem_o, tmem_p + j * 32 + ks * 8, bd0 + uint64_t((ks * 2048) >> 4), idesc_o,
                                          (w > 0 || j > 0 || ks > 0) ? 1u : 0u);
                            tc_commit(&v_empty[st]);
                        }
                        if (!ok) break;
                        tc_commit(pv_done);
                        if (w + 1 == wide_blocks(t)) tc_commit(o_final);
                    }
                    tc++;
                }
            }
        }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
        // ------------------------------------------------------------ softmax: two threads per row, 64 keys each
        const uint32_t h = warp >> 2, quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t g = 0, tc = 0;
        bool ok = true;
        PfTile t, last;
        for (uint32_t round = 0; pf_tile(p, round, t); round++) {
            if (!t.nb) continue;
            last = t;
            const uint32_t tok = t.tok0 + (row >> 3);
            const uint32_t item_end = (t.b_begin + t.nb) * kBN;
            const uint32_t lim_hi = min(min(p.key_hi, p.pos + tok + 1), item_end); // this row sees keys [key_lo, lim_hi)
            const uint32_t lim_tile = min(min(p.key_hi, p.pos + t.tok0 + 1), item_end); // below it no row of the tile is masked
            float m_ref = -INFINITY, l = 0.f;
            for (uint32_t w = 0; ok && w < wide_blocks(t); w++, g++) {
                const uint32_t key0 = t.b_begin * kBN + w * kWBN + h * 64;
                if (!mbar_wait(s_full, g & 1, abort_flag)) { give_up(kStatusFullTimeout); ok = false; break; }
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld32(tmem_s + lane_addr + h * 64, sr[0]);
                tmem_ld32(tmem_s + lane_addr + h * 64 + 32, sr[1]);
                tmem_wait_ld();
                tc_fence_before(); // the scores are in registers: S is free for the next block's product
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free);

                float s[64];
#pragma unroll
                for (int c = 0; c < 64; c++) s[c] = __uint_as_float(sr[c >> 5][c & 31]);
                if (key0 < p.key_lo || key0 + 64 > lim_tile) {
#pragma unroll
                    for (int c = 0; c < 64; c++)
                        if (key0 + c < p.key_lo || key0 + c >= lim_hi) s[c] = -INFINITY;
                }
                float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
                for (int c = 4; c < 64; c++) m4[c & 3] = fmaxf(m4[c & 3], s[c]);
                float mxl = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                // The row's other half: each thread leaves (maximum, block number + 1) as one 64-bit word and polls
                // its partner's word of the same parity until it carries this block's number.  No barrier, so a
                // warp that has given up cannot strand its partner; the poll is bounded like every other wait.
                // (Two parities: the partner cannot write block g + 2 before it has read this thread's g + 1.)
                xmax[((g & 1) * 2 + h) * kBM + row] = (static_cast<unsigned long long>(g + 1) << 32) | __float_as_uint(mxl);
                {
                    const volatile unsigned long long *theirs = &xmax[((g & 1) * 2 + (h ^ 1)) * kBM + row];
                    unsigned long long wv = *theirs;
                    unsigned long long t0 = 0;
                    bool got = true;
                    for (uint32_t n = 1; uint32_t(wv >> 32) != g + 1; n++) {
                        if ((n & 63) == 0) {
                            unsigned long long tn;
                            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tn));
                            if (!t0) t0 = tn;
                            if (*abort_flag || tn - t0 > 1000000000ull) { got = false; break; }
                        }
                        wv = *theirs;
                    }
                    if (!__all_sync(0xffffffffu, got)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    mxl = fmaxf(mxl, __uint_as_float(uint32_t(wv)));
                }
                const float mx = mxl * p.scale_log2;
                const bool need = mx > m_ref + kPfRescale; // the same in both halves of a row
                float factor = 1.f;
                if (need) {
                    factor = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - mx);
                    m_ref = mx;
                    l *= factor;
                }
                if (w > 0 && __any_sync(0xffffffffu, need)) {
                    // the P V products of the block before must have landed in O; each half rescales its 128 columns
                    if (!mbar_wait(pv_done, (g & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_o + lane_addr + h * 128 + c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int k = 0; k < 32; k++) o[k] = __float_as_uint(__uint_as_float(o[k]) * factor);
                        tmem_st32(tmem_o + lane_addr + h * 128 + c, o);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                uint32_t pw[32];
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < 32; k++) {
                    const float a = ex2_approx(fmaf(s[2 * k], p.scale_log2, -m_use));
                    const float bb = ex2_approx(fmaf(s[2 * k + 1], p.scale_log2, -m_use));
                    sum4[k & 3] += a + bb;
                    if (p.v_fmt) {
                        __nv_bfloat162 hh = __floats2bfloat162_rn(a, bb);
                        pw[k] = *reinterpret_cast<uint32_t *>(&hh);
                    } else {
                        pw[k] = pack_half2(a, bb);
                    }
                }
                l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                // P has one buffer: the P V products of the block before have read it
                if (!mbar_wait(pv_done, (g & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); ok = false; break; }
                tc_fence_after();
                tmem_st32(tmem_p + lane_addr + h * 32, pw);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
            }
            if (!ok) break;
            row_l[((tc & 1) * 2 + h) * kBM + row] = l;
            if (h == 0) row_m[(tc & 1) * kBM + row] = m_ref;
            __syncwarp();
            if (lane == 0) mbar_arrive(&lm_full[tc & 1]);
            tc++;
        }
        // The CTA's LAST tile leaves through these eight warps, two threads per row (this half's 128 columns): nothing
        // is left for them to do, and a tile's scaled, gated stores are bound by the loads and stores in flight,
        // that is by the number of threads (four warps took 15-19 us for it at the end of a CTA's life).
        if (ok && tc) {
            const uint32_t k = tc - 1;
            const uint32_t tok = last.tok0 + (row >> 3);
            const bool row_live = tok < p.tokens;
            const size_t rh = size_t(tok) * p.heads + last.kv * kHeadsPerKv + (row & 7);
            bool fine = mbar_wait(&lm_full[k & 1], (k >> 1) & 1, abort_flag);
            const float l = row_l[((k & 1) * 2) * kBM + row] + row_l[((k & 1) * 2 + 1) * kBM + row], m_ref = row_m[(k & 1) * kBM + row];
            fine = fine && mbar_wait(o_final, k & 1, abort_flag);
            if (!fine) {
                give_up(kStatusMmaTimeout);
            } else {
                tc_fence_after();
                const float inv_l = l > 0.f ? 1.f / l : 0.f;
                uint32_t o[4][32];
#pragma unroll
                for (int ch = 0; ch < 4; ch++) tmem_ld32(tmem_o + lane_addr + h * 128 + ch * 32, o[ch]);
                tmem_wait_ld();
                if (row_live) {
                    if (p.out) {
                        const float *gp = p.q_and_gate + rh * 2 * kDim + kDim + h * 128;
                        float *op = p.out + rh * kDim + h * 128;
                        Float8 gt[2] = {ld_global_v8(gp), ld_global_v8(gp + 8)};
#pragma unroll
                        for (int st = 0; st < 16; st++) {
                            const Float8 gc = gt[st & 1];
                            if (st + 2 < 16) gt[st & 1] = ld_global_v8(gp + (st + 2) * 8);
                            Float8 v;
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                v.v[e] = __uint_as_float(o[st >> 2][8 * (st & 3) + e]) * __fdividef(inv_l, 1.f + __expf(-gc.v[e]));
                            st_global_v8(op + st * 8, v);
                        }
                    } else {
                        float *part = p.part + size_t(last.split) * p.part_stride;
                        float4 *op = reinterpret_cast<float4 *>(part + rh * kPartStride + h * 128);
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            op[j] = make_float4(__uint_as_float(o[j >> 3][4 * (j & 7)]), __uint_as_float(o[j >> 3][4 * (j & 7) + 1]),
                                                __uint_as_float(o[j >> 3][4 * (j & 7) + 2]), __uint_as_float(o[j >> 3][4 * (j & 7) + 3]));
                    }
                    if (p.part && h == 0) {
                        float *part = p.part + size_t(last.split) * p.part_stride;
                        part[rh * kPartStride + kPartM] = m_ref;
                        part[rh * kPartStride + kPartL] = l;
                    }
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // ------------------------------------------------------------ tile I/O: one thread per row
        const uint32_t quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32) << 16;
        struct RowOf {
            uint32_t tok;
            bool live;
            size_t rh;
            float *part;
        };
        auto row_of = [&](const PfTile &t) {
            RowOf r;
            r.tok = t.tok0 + (row >> 3);
            r.live = r.tok < p.tokens;
            r.rh = size_t(r.tok) * p.heads + t.kv * kHeadsPerKv + (row & 7);
            r.part = p.part ? p.part + size_t(t.split) * p.part_stride : nullptr;
            return r;
        };
        auto next_item = [&](uint32_t &round, PfTile &t) -> bool {
            while (pf_tile(p, round, t)) {
                round++;
                if (t.nb) return true;
                const RowOf r = row_of(t);
                if (r.live && r.part) { // no keys: the empty partial
                    float *dst = r.part + r.rh * kPartStride;
                    for (uint32_t d = 0; d < uint32_t(kDim); d++) dst[d] = 0.f;
                    dst[kPartM] = -INFINITY, dst[kPartL] = 0.f;
                }
            }
            return false;
        };
        auto load_q = [&](const PfTile &t, uint32_t k) -> bool {
            const RowOf r = row_of(t);
            if (r.live && p.out) {
                const char *gpf = reinterpret_cast<const char *>(p.q_and_gate + r.rh * 2 * kDim + kDim);
#pragma unroll
                for (int j = 0; j < 8; j++) prefetch_l2(gpf + j * 128);
            }
            // the whole row into registers first: none of it depends on the wait below
            const uint4 *qrow = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.q) + r.rh * kDim);
            uint4 qv[32];
#pragma unroll
            for (int j = 0; j < 32; j++) qv[j] = r.live ? qrow[j] : make_uint4(0u, 0u, 0u, 0u);
            if (p.q_bf16) { // bfloat16 queries over binary16 key operands: exact unless outside binary16's range
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    uint32_t *wq = reinterpret_cast<uint32_t *>(&qv[j]);
#pragma unroll
                    for (int e = 0; e < 4; e++) wq[e] = pack_half2(__uint_as_float(wq[e] << 16), __uint_as_float(wq[e] & 0xffff0000u));
                }
            }
            // the score products of the tile before no longer read the old Q
            if (!mbar_wait(q_empty, (k & 1) ^ 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2; c++) { // dims 0..127 into tensor memory, two values per column
                uint32_t wq[32];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint4 v = qv[c * 8 + j];
                    wq[4 * j] = v.x, wq[4 * j + 1] = v.y, wq[4 * j + 2] = v.z, wq[4 * j + 3] = v.w;
                }
                tmem_st32(tmem_q + lane_addr + c * 32, wq);
            }
#pragma unroll
            for (int j = 0; j < 16; j++) { // dims 128..255 into shared memory: slab = 64 dims, 16-byte chunks swizzled by the row
                const uint32_t slab = j >> 3, chunk = j & 7;
                *reinterpret_cast<uint4 *>(sQ + slab * (kBM * 128) + row * 128 + ((chunk ^ (row & 7)) << 4)) = qv[16 + j];
            }
            tmem_wait_st();
            fence_async_smem(); // the tensor cores read the shared-memory half through the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
            return true;
        };
        auto epilogue = [&](const PfTile &t, uint32_t k) -> bool {
            const RowOf r = row_of(t);
            const bool row_live = r.live;
            const size_t rh = r.rh;
            float *part = r.part;
            const bool gated = row_live && p.out;
            if (!mbar_wait(&lm_full[k & 1], (k >> 1) & 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
            const float l = row_l[((k & 1) * 2) * kBM + row] + row_l[((k & 1) * 2 + 1) * kBM + row], m_ref = row_m[(k & 1) * kBM + row];
            if (!mbar_wait(o_final, k & 1, abort_flag)) { give_up(kStatusMmaTimeout); return false; }
            tc_fence_after();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
            for (uint32_t half = 0; half < 2; half++) {
                const float *gp = p.q_and_gate + (gated ? rh * 2 * kDim + kDim + half * 128 : 0);
                uint32_t o[4][32];
#pragma unroll
                for (int ch = 0; ch < 4; ch++) tmem_ld32(tmem_o + lane_addr + half * 128 + ch * 32, o[ch]);
                tmem_wait_ld();
                if (half == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_empty); // O has left tensor memory: the next tile's P V products may start
                }
                if (row_live) {
                    if (p.out) {
                        float *op = p.out + rh * kDim + half * 128;
                        // the gate values four 32-byte steps ahead of their use (a thread has a whole row: one step
                        // ahead, sixteen dependent round trips to L2 stood between O's two halves).  Releasing O
                        // before any gate value is read -- first half out raw, gated later from its own stores --
                        // shortened the tile change from 9 to 3 us but made the blocks after it slower, the four
                        // epilogue warps then competing with the softmax warps: 790 against 840 TFLOP/s at position 0
                        Float8 gt[4];
#pragma unroll
                        for (int a = 0; a < 4; a++) gt[a] = ld_global_v8(gp + a * 8);
#pragma unroll
                        for (int st = 0; st < 16; st++) {
                            const Float8 gc = gt[st & 3];
                            if (st + 4 < 16) gt[st & 3] = ld_global_v8(gp + (st + 4) * 8);
                            Float8 v;
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                v.v[e] = __uint_as_float(o[st >> 2][8 * (st & 3) + e]) * __fdividef(inv_l, 1.f + __expf(-gc.v[e]));
                            st_global_v8(op + st * 8, v);
                        }
                    } else {
                        float4 *op = reinterpret_cast<float4 *>(part + rh * kPartStride + half * 128);
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            op[j] = make_float4(__uint_as_float(o[j >> 3][4 * (j & 7)]), __uint_as_float(o[j >> 3][4 * (j & 7) + 1]),
                                                __uint_as_float(o[j >> 3][4 * (j & 7) + 2]), __uint_as_float(o[j >> 3][4 * (j & 7) + 3]));
                    }
                }
            }
            if (row_live && part) {
                part[rh * kPartStride + kPartM] = m_ref;
                part[rh * kPartStride + kPartL] = l;
            }
            return true;
        };
        uint32_t round = 0, k = 0;
        PfTile cur, nxt;
        bool have = next_item(round, cur);
        if (have && !load_q(cur, 0)) have = false;
        while (have) {
            const bool more = next_item(round, nxt);
            if (more && !load_q(nxt, k + 1)) break;
            if (!more) break; // the last tile leaves through the softmax warps
            if (!epilogue(cur, k)) break;
            cur = nxt, have = more, k++;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 13) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

// ----------------------------------------------------------------- host side

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

int prefill_configure(int device) {
    (void)device;
    SAETTA_CUDA(cudaFuncSetAttribute(prefill_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfLayout<0>::kSmem));
    SAETTA_CUDA(cudaFuncSetAttribute(prefill_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfLayout<8>::kSmem));
    SAETTA_CUDA(cudaFuncSetAttribute(prefill_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfLayout<4>::kSmem));
    SAETTA_CUDA(cudaFuncSetAttribute(prefill_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWSmem));
    return SAETTA_OK;
}

int launch_prefill(const PrefillArgs &a, uint32_t *status, cudaStream_t stream) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(SAETTA_ERR_CUDA, "prefill attention: cuTensorMapEncodeTiled is not available");
    const bool quant = a.qbits != 0;
    if (quant && (a.qbits != 8 && a.qbits != 4)) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: 8- or 4-bit codes");
    if (quant && a.kv_heads != 2) return fail(SAETTA_ERR_UNSUPPORTED, "prefill attention: codes are read in place for 2 kv heads");
    if (reinterpret_cast<uintptr_t>(a.q) & 15) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: q must be 16-byte aligned");
    if (!quant && ((reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15))
        return fail(SAETTA_ERR_BAD_ARG, "prefill attention: keys and values must be 16-byte aligned");
    if (a.key_base % kBN || a.key_base > a.key_lo) return fail(SAETTA_ERR_BAD_SHAPE, "prefill attention: the cache's first row must sit at a multiple of 64 at or below the first key");
    // rows of the buffers the kernel may touch: up to the last key it is asked for (copies past that read zeros)
    const cuuint64_t keys_total = std::max<cuuint64_t>(1, std::min<cuuint64_t>(cuuint64_t(a.pos) + a.tokens, a.key_hi) - std::min<cuuint64_t>(a.key_base, a.key_hi));
    const int k_dtype = quant ? SAETTA_F16 : (a.k_dtype < 0 ? a.dtype : a.k_dtype);
    if (k_dtype == SAETTA_BF16 && a.dtype != SAETTA_BF16) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: bfloat16 keys need bfloat16 queries");
    CUtensorMap mk, mv;
    PfQuantMaps qm;
    const cuuint32_t el[3] = {1, 1, 1};
    if (!quant) {
        const CUtensorMapDataType dt = k_dtype == SAETTA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const CUtensorMapDataType dtv = a.v_dtype == SAETTA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        for (int side = 0; side < 2; side++) {
            const cuuint64_t dims[3] = {cuuint64_t(kDim), a.kv_heads, keys_total};
            const cuuint64_t strides[2] = {kDim * 2, cuuint64_t(a.kv_heads) * kDim * 2};
            // the wide kernel takes the keys 128 at a time, the values 64 at a time
            const cuuint32_t box[3] = {64, 1, cuuint32_t(side || a.narrow ? kBN : kWBN)};
            CUresult r = enc(side ? &mv : &mk, side ? dtv : dt, 3, const_cast<void *>(side ? a.v : a.k), dims, strides, box, el,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(SAETTA_ERR_CUDA, "prefill attention: tensor map for the cache rejected");
        }
        qm.kc = qm.vc = qm.ks = qm.kz = qm.vs = qm.vz = mk; // not read
    } else {
        // codes: bytes [keys][kv heads][row]; a box is one kv head's rows of 64 keys, unswizzled
        const cuuint64_t row = cuuint64_t(kDim) * a.qbits / 8;
        for (int side = 0; side < 2; side++) {
            const cuuint64_t dims[3] = {row, a.kv_heads, keys_total};
            const cuuint64_t strides[2] = {row, cuuint64_t(a.kv_heads) * row};
            const cuuint32_t box[3] = {cuuint32_t(row), 1, kBN};
            CUresult r = enc(side ? &qm.vc : &qm.kc, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(side ? a.qv : a.qk), dims, strides,
                             box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(SAETTA_ERR_CUDA, "prefill attention: tensor map for the codes rejected");
        }
        // scales and biases: binary16 [keys][kv heads * 4]; a box is 64 keys' 16 bytes
        const void *arr[4] = {a.qks, a.qkz, a.qvs, a.qvz};
        CUtensorMap *maps[4] = {&qm.ks, &qm.kz, &qm.vs, &qm.vz};
        for (int i = 0; i < 4; i++) {
            const cuuint64_t dims[2] = {cuuint64_t(a.kv_heads) * 4, keys_total};
            const cuuint64_t strides[1] = {cuuint64_t(a.kv_heads) * 4 * 2};
            const cuuint32_t box[2] = {cuuint32_t(a.kv_heads) * 4, kBN};
            CUresult r = enc(maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(arr[i]), dims, strides, box, el,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(SAETTA_ERR_CUDA, "prefill attention: tensor map for the scales rejected");
        }
        mk = mv = qm.kc; // not read
    }
    // operands: binary16 throughout over a quantised cache (bfloat16 queries are converted on the way in)
    const uint32_t fmt = k_dtype == SAETTA_BF16 ? 1u : 0u, v_fmt = quant ? 0u : (a.v_dtype == SAETTA_BF16 ? 1u : 0u);
    PfParams p{a.q, a.q_and_gate, a.out, a.part, status, a.heads, a.kv_heads, a.pos, a.tokens, a.key_lo, a.key_hi,
               a.scale * kLog2ePf, fmt, v_fmt, a.splits ? a.splits : 1u, uint32_t(size_t(a.tokens) * a.heads * kPartStride), a.key_base,
               a.dtype == SAETTA_BF16 && !fmt ? 1u : 0u};
    int dev = 0;
    SAETTA_CUDA(cudaGetDevice(&dev));
    const uint32_t tiles = (a.tokens + kTokTile - 1) / kTokTile * a.kv_heads * (a.splits ? a.splits : 1u);
    const uint32_t grid = std::min<uint32_t>(tiles, uint32_t(sm_count(dev)));
    if (!quant && !a.narrow) prefill_wide_kernel<<<grid, kPfThreads, kWSmem, stream>>>(mk, mv, p);
    else if (!quant) prefill_kernel<0><<<grid, kPfThreads, PfLayout<0>::kSmem, stream>>>(mk, mv, qm, p);
    else if (a.qbits == 8) prefill_kernel<8><<<grid, kPfThreads, PfLayout<8>::kSmem, stream>>>(mk, mv, qm, p);
    else prefill_kernel<4><<<grid, kPfThreads, PfLayout<4>::kSmem, stream>>>(mk, mv, qm, p);
    SAETTA_CUDA(cudaGetLastError());
    return SAETTA_OK;
}

} // namespace saetta
