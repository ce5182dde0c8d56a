// Host-side objects behind the C ABI.  They mirror, one for one, the Rust
// structs of the reference that own device memory on this path:
//   QuantRows        src/kv_quant.rs:158-283
//   KvCache          src/gpu_layers.rs:179-293 (GpuKvCache)
//   RowBackup        src/gpu_cache.rs:192-286
//   Decode           src/attention.rs:19-171 (DecodeAttention), src/rows.rs:307-494 (AttentionRows)
//   AttGemm          src/attention_gemm.rs:93-363
// and declare the kernel launchers implemented in the .cu files.
#pragma once

#include <cstring>

#include <vector>

#include "common.cuh"

struct saetta_quant_rows {
    int device = 0;
    int bits = 8;
    size_t per_token = 0; // groups of 64 per token (values / 64)
    size_t capacity = 0;
    void *data = nullptr;
    void *scales = nullptr;
    void *biases = nullptr;
    bool owns = false;
    size_t data_row_bytes() const { return per_token * 2 * size_t(bits) * 4; }
    size_t param_row_bytes() const { return per_token * 2; }
};

struct saetta_kv_cache {
    int device = 0;
    int bits = 16;
    int dtype = SAETTA_F16; // of a 16-bit cache
    size_t heads = 0, kv_heads = 0, head_dim = 0, capacity = 0;
    void *keys = nullptr;   // 16/32-bit rows, or the key codes
    void *values = nullptr;
    saetta_quant_rows k, v; // views into the buffers of a quantised cache
    size_t row_values() const { return kv_heads * head_dim; }
    size_t plain_row_bytes() const { return row_values() * (bits == 32 ? 4 : 2); }
};

struct saetta_row_backup {
    struct Part {
        void *copy;
        size_t row_bytes;
    };
    std::vector<Part> parts;
    int device = 0;
    size_t from = 0, n = 0;
    bool held = false;
};

struct saetta_decode {
    int device = 0;
    size_t heads = 0, kv_heads = 0, capacity = 0, rows = 1;
    int splits = 0;        // grid of the split-KV kernel
    float *parts = nullptr; // [splits][rows][heads][kPartStride]
    uint32_t *status = nullptr;
};

struct saetta_decode_batch {
    int device = 0;
    size_t heads = 0, kv_heads = 0, max_seqs = 0;
    int ctas = 0;
    size_t max_parts = 0;
    float *parts = nullptr;     // [max_parts][heads][kPartStride]
    void *table_dev = nullptr;  // segment descriptors + per-sequence part ranges
    void *table_host = nullptr; // pinned
    size_t table_bytes = 0;
    void *table_event = nullptr; // recorded after the table's upload
    uint32_t *status = nullptr;
};

struct saetta_att_gemm {
    int device = 0;
    size_t chunk = 0, kv_heads = 0;
    // 16-bit copy of the cache rows the tensor-core kernel reads when the cache itself is quantised (keys
    // and values) or bfloat16 (values only).  It persists across calls: rows below the chunk being
    // encoded that an earlier call already converted are not converted again.
    void *stage_k = nullptr, *stage_v = nullptr;
    size_t stage_tokens = 0; // rows each copy has room for
    bool stage_quant = false; // read 8/4-bit caches through the 16-bit copy instead of in place
    bool narrow = false;      // 16-bit caches: score blocks of 64 keys (the older kernel) instead of 128
    struct Staged {
        const void *src = nullptr; // the buffer the rows came from (identity of the cache side)
        int dtype = 0;
        size_t lo = 0, hi = 0;     // rows [lo, hi) of the copy are valid
    } staged[2];
    float *split_parts = nullptr; // partials of the key splits of a long-context chunk
    size_t split_floats = 0;
    uint32_t *status = nullptr;
};

// peer.cu: where one rank's partial goes in the mailboxes of the ranks of a box.
namespace saetta {
constexpr int kMaxPeers = 8;
struct PeerPush {
    unsigned long long *parts[kMaxPeers]; // each rank's mailbox: [2 slots][world][slot_floats] words of (value, exchange number)
    uint32_t *seq_done;                   // this rank's counter of exchanges collected
    uint32_t *seq_sent;                   // ... and published
    uint32_t *status;                     // the group's status word (a peer that never published)
    uint32_t world, rank, slot_floats;
};
// Where a decode launch's merged result goes: out (gated), part_out (the logical (O, m, l) partial), or
// the peers' mailboxes (push.world != 0) -- and with push.world != 0 AND out, the launch also collects:
// its merge CTAs wait for the peers' partials of the same exchange and write the gated result.
// n_merge and passes are filled in by the launcher.
struct MergeOut {
    const float *q_and_gate = nullptr;
    float *out = nullptr;
    float *part_out = nullptr;
    PeerPush push = {};
    uint32_t n_merge = 0; // merge CTAs per pass; 0: the launch carries no merge role
    uint32_t passes = 1;  // gridDim.y of the launch
};
// One mailbox word: a float with the number of the exchange it belongs to, written by one 64-bit
// store so that the reader sees both or neither.
__host__ __device__ inline unsigned long long peer_word(float v, uint32_t seq) {
#ifdef __CUDA_ARCH__
    return (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(v);
#else
    uint32_t b;
    memcpy(&b, &v, 4);
    return (static_cast<unsigned long long>(seq) << 32) | b;
#endif
}

} // namespace saetta

struct saetta_peer_group {
    int device = 0, rank = 0, world = 1;
    size_t rows_max = 0, heads = 0, slot_floats = 0;
    void *mailbox = nullptr; // the slots, then the two exchange counters and the status word
    float *staging = nullptr;
    void *peer_base[saetta::kMaxPeers] = {};
    bool connected = false;
    saetta::PeerPush push = {};
    size_t words_offset() const { return 2 * size_t(world) * slot_floats * sizeof(unsigned long long); }
};
namespace saetta {

using QuantRows = saetta_quant_rows;

// kv_quant.cu
int launch_kv_quantize(int bits, uint32_t per_token, const float *x0, const QuantRows *r0,
                       const float *x1, const QuantRows *r1, size_t rows, size_t pos,
                       const saetta_token_params *params, cudaStream_t stream);
int launch_kv_dequantize(const QuantRows *rows, void *out, int dtype, size_t first, size_t tokens,
                         cudaStream_t stream);
int launch_bf16_to_f16(const void *in, void *out, size_t values, cudaStream_t stream);
int launch_kv_store_plain(int mode, const float *k, const float *v, void *keys, void *values,
                          size_t row_values, size_t rows, size_t pos,
                          const saetta_token_params *params, cudaStream_t stream);

// What a split-KV launch reads: the cache in any of its storage forms.
struct KvView {
    int bits = 8;            // 32, 16, 8, 4
    int dtype = SAETTA_F16;  // of 16-bit rows
    const void *k = nullptr, *v = nullptr; // rows or codes
    const void *ks = nullptr, *kz = nullptr, *vs = nullptr, *vz = nullptr;
    uint32_t kv_heads = 2;
};

// Publishes the partial in the group's staging buffer (rows x heads x kPartStride floats).
int launch_peer_publish(saetta_peer_group *g, size_t rows, cudaStream_t stream);

// One sequence-segment of a batched launch (decode_quant.cu reads these).
struct Segment {
    const void *k, *v, *ks, *kz, *vs, *vz;
    uint32_t tile_begin, tile_end; // 32-token tiles
    uint32_t kv_len;
    uint32_t part;   // slot in the partials buffer
    uint32_t seq;    // which q / out row
    uint32_t pad[3];
};

// decode_quant.cu: tensor-core split-KV over 8/4-bit codes.
// The merge over the parts and what follows it (gate, logical partial, or the push to the peers) run
// inside the same launch (merge_role.cuh); `status` points at kStatusWords zeroed words.
int launch_decode_quant(const KvView &kv, const float *q, float *parts, uint32_t *status,
                        uint32_t m, uint32_t row_step, int splits, uint32_t capacity,
                        const saetta_token_params *params, const MergeOut &mo, cudaStream_t stream);
size_t decode_quant_part_floats(size_t kv_heads); // floats per (part, row) of the internal partial format
int launch_decode_quant_batched(int bits, const Segment *segments_dev, const uint32_t *cta_first_dev,
                                int ctas, const float *q, float *parts, uint32_t *status,
                                cudaStream_t stream);
int decode_quant_configure(int device);
int decode_quant_static(int device, const KvView &kv, size_t capacity, const float *q, uint32_t m,
                        const float *q_and_gate, float *out, const saetta_token_params *params,
                        cudaStream_t stream);
int decode_quant_static_status(int device, cudaStream_t stream, uint32_t *status, bool clear);

// decode_half.cu: tensor-core split-KV over binary16 rows (2 kv heads); partials in decode_quant.cu's format.
int launch_decode_half(const KvView &kv, const float *q, float *parts, uint32_t *status, uint32_t m, uint32_t row_step,
                       int splits, uint32_t capacity, const saetta_token_params *params, const MergeOut &mo,
                       cudaStream_t stream);
int decode_half_configure(int device);

// decode_exact.cu: f32 arithmetic over f32 / 16-bit rows.
int launch_decode_exact(const KvView &kv, const float *q, float *parts, uint32_t m,
                        uint32_t row_step, int splits, uint32_t capacity,
                        const saetta_token_params *params, cudaStream_t stream);
int decode_exact_configure(int device);

// merge.cu: log-sum-exp merge over parts, then the gate.
//   frag:    parts in the fragment order decode_quant.cu writes, [part][row][kv][2064];
//            first_part (device, [seqs+1]) gives each sequence's part range when
//            non-null (batched), else every row merges parts 0..nparts.
//   logical: parts [part][row][head][kPartStride] (decode_exact.cu, other ranks).
// With out == null the merged (O, m, l) is written to part_out in the logical
// layout instead of the gated result.
// With `push` non-null the merged partial goes, instead of part_out, into this rank's place
// in every peer's mailbox (see peer.cu).
int launch_merge_frag(const float *parts, uint32_t nparts, const uint32_t *first_part,
                      uint32_t rows, uint32_t kv_heads, const float *q_and_gate, float *out,
                      float *part_out, cudaStream_t stream, const PeerPush *push = nullptr);
int launch_merge_logical(const float *parts, uint32_t nparts, uint32_t rows, uint32_t heads,
                         const float *q_and_gate, float *out, float *part_out,
                         cudaStream_t stream);

// prefill_umma.cu: tcgen05 causal chunk attention.
struct PrefillArgs {
    const void *q;       // 16-bit [tokens][heads][256]
    const void *k, *v;   // 16-bit [>= pos+tokens][kv_heads][256]
    int dtype;           // of q and k
    int v_dtype;         // of v: P takes the same type, so binary16 values keep P's 11-bit significand
    const float *q_and_gate; // may be null when part != null
    float *out;          // [tokens][heads][256] or null
    float *part;         // [tokens][heads][kPartStride] or null
    uint32_t heads, kv_heads, pos, tokens;
    uint32_t key_lo, key_hi; // keys considered (clipped by causality), global positions
    float scale;
    uint32_t splits = 1;     // > 1: each tile's keys are cut into `splits` work items, each leaving a
                             // partial in part + split * tokens*heads*kPartStride (out must be null)
    uint32_t key_base = 0;   // global position of row 0 of k and v (a multiple of 64, <= key_lo): a shard
                             // that stores only its own slice of the sequence
    // a quantised cache read in place (qbits 8 or 4; k and v above are then unused): codes, scales, biases
    int qbits = 0;
    bool narrow = false;     // 16-bit cache: the kernel with 64-key score blocks instead of the wide one (kept for comparison)
    int k_dtype = -1;        // of k when it differs from q's (binary16 keys under bfloat16 queries: q is converted on the way in)
    const void *qk = nullptr, *qv = nullptr, *qks = nullptr, *qkz = nullptr, *qvs = nullptr, *qvz = nullptr;
};
int launch_prefill(const PrefillArgs &a, uint32_t *status, cudaStream_t stream);
int prefill_configure(int device);

} // namespace saetta
