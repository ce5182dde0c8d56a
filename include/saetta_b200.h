/*
 * saetta_b200.h -- C ABI of the B200 attention path.
 *
 * One shared library, plain pointers and sizes only.  Every entry point
 * returns a saetta_status; saetta_last_error() gives the message of the last
 * failure on the calling thread.  Nothing unwinds across this boundary.
 *
 * Each block names the interface of the reference project (Rust, paths inside
 * that project) that it stands in for.  Geometry is the reference's: head
 * dimension 256, 8 query heads per kv head, quantisation groups of 64.
 *
 * Conventions shared by all entry points
 *   - pointers named *_dev are device pointers on the object's device;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); work is enqueued, never synchronised, unless stated;
 *   - the per-token inputs (position, kv_len) are read ON THE DEVICE from a
 *     saetta_token_params the caller updates between replays, so a recorded
 *     CUDA graph of these calls serves every position, as the reference's
 *     recorded Plan does (src/plan.rs:1-35);
 *   - handles are not thread-safe; distinct handles on distinct streams may
 *     run concurrently.
 */
#ifndef SAETTA_B200_H
#define SAETTA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum saetta_status {
    SAETTA_OK = 0,
    SAETTA_ERR_BAD_ARG = 1,   /* null pointer, unknown enum value */
    SAETTA_ERR_BAD_SHAPE = 2, /* what the reference asserts: head_dim != 256, heads != 8*kv_heads, m > rows ... */
    SAETTA_ERR_NO_MEM = 3,
    SAETTA_ERR_CUDA = 4,
    SAETTA_ERR_TIMEOUT = 5, /* a bounded device-side wait gave up (see saetta_device_status) */
    SAETTA_ERR_UNSUPPORTED = 6
} saetta_status;

const char *saetta_last_error(void);
/* Library version string and the SM architecture the kernels were built for. */
const char *saetta_version(void);

/* src/plan.rs:17-35 `TokenParams`; kernels read it from device memory. */
typedef struct saetta_token_params {
    uint32_t token;
    uint32_t position;
    uint32_t kv_len; /* position + 1 */
    uint32_t pad;
} saetta_token_params;

/* src/attention_prefill.rs:5-14 `FlashParams`. */
typedef struct saetta_flash_params {
    uint32_t heads;
    uint32_t kv_heads;
    uint32_t pos;    /* position of the chunk's first token; token i sees keys 0 ..= pos + i */
    uint32_t tokens;
    float scale;
} saetta_flash_params;

/* Storage type of 16-bit tensors (the reference stores binary16; the tensor-core
 * prefill also takes bfloat16). */
typedef enum saetta_dtype { SAETTA_F16 = 0, SAETTA_BF16 = 1, SAETTA_F32 = -1 /* only where an entry point says so */ } saetta_dtype;

/* ------------------------------------------------------------------ QuantRows
 * src/kv_quant.rs:158-283 `QuantRows`: the codes, scales and biases of one cache
 * side (keys or values).  Layout (kernels/kv_quant.metal:1-6): group
 * G = token * per_token + g, data u32 [groups][2*bits], scales/biases binary16
 * [groups]; code i of a group sits at bit i*bits of word i*bits/32.
 */
typedef struct saetta_quant_rows saetta_quant_rows;

/* QuantRows::new(gpu, bits, values, capacity): owns its three buffers. */
int saetta_quant_rows_create(int device, int bits, size_t values, size_t capacity,
                             saetta_quant_rows **out);
/* The same object over buffers the caller owns (a `View` of each). */
int saetta_quant_rows_wrap(int device, int bits, size_t values, size_t capacity, void *data_dev,
                           void *scales_dev, void *biases_dev, saetta_quant_rows **out);
void saetta_quant_rows_destroy(saetta_quant_rows *rows);
int saetta_quant_rows_buffers(const saetta_quant_rows *rows, void **data_dev, void **scales_dev,
                              void **biases_dev);
/* QuantRows::record / record_at: quantise one token's `values` f32 at x_dev into
 * the slot at params_dev->position. */
int saetta_quant_rows_record_at(saetta_quant_rows *rows, const float *x_dev,
                                const saetta_token_params *params_dev, void *stream);
/* QuantRows::encode: `tokens` rows of x_dev into the slots from `pos`. */
int saetta_quant_rows_encode(saetta_quant_rows *rows, const float *x_dev, size_t pos,
                             size_t tokens, void *stream);
/* QuantRows::encode_dequantize: tokens 0..tokens as 16-bit values (s*q + z, a
 * multiply then an add in f32, then one rounding) into out_dev. */
int saetta_quant_rows_encode_dequantize(const saetta_quant_rows *rows, void *out_dev,
                                        int dtype, size_t tokens, void *stream);

/* Host-side kv_quant::quantize / dequantize (src/kv_quant.rs:54-105), bit for bit
 * what the kernels write; for callers that prepare a cache on the CPU. */
int saetta_quantize_host(const float *x, size_t n, int bits, uint32_t *data, uint16_t *scales,
                         uint16_t *biases);
int saetta_dequantize_host(const uint32_t *data, const uint16_t *scales, const uint16_t *biases,
                           size_t groups, int bits, float *out);

/* ------------------------------------------------------------------ GpuKvCache
 * src/gpu_layers.rs:179-293 `GpuKvCache`.  bits 16 / 8 / 4 as `KvBits`; bits 32
 * (f32 rows, no counterpart in the reference) exists so the f32 configuration
 * can run on the device.  Capacity is rounded up to SAETTA_KV_ALIGN.  Token p
 * lives in row p of every buffer.
 */
#define SAETTA_KV_ALIGN 128
typedef struct saetta_kv_cache saetta_kv_cache;

int saetta_kv_cache_create(int device, int bits, size_t heads, size_t kv_heads, size_t head_dim,
                           size_t capacity, saetta_kv_cache **out);
void saetta_kv_cache_destroy(saetta_kv_cache *cache);
size_t saetta_kv_cache_capacity(const saetta_kv_cache *cache);
int saetta_kv_cache_bits(const saetta_kv_cache *cache);
/* GpuKvCache::buffers(): keys, values, then k.scales, k.biases, v.scales, v.biases
 * for a quantised cache; row_bytes[i] is the size of one token's row. Returns
 * the number of buffers (2 or 6) in *count. */
int saetta_kv_cache_buffers(const saetta_kv_cache *cache, void *buffers_dev[6],
                            size_t row_bytes[6], int *count);
/* The two QuantRows of a quantised cache (borrowed; NULL for 16/32 bits). */
int saetta_kv_cache_quant(const saetta_kv_cache *cache, saetta_quant_rows **keys,
                          saetta_quant_rows **values);
/* GpuKvCache::resize: new buffers, every old row that fits copied over; blocks
 * until the copy is done.  Ops recorded with the old buffers must be recorded again. */
int saetta_kv_cache_resize(saetta_kv_cache *cache, size_t capacity, void *stream);
/* The store sites (src/gpu_layers.rs:373-411, 483-522, src/prefill.rs:1656-1666):
 * write `rows` rows of k and v (f32 [rows][kv_heads*head_dim], already normed
 * and roped) at params_dev->position + r  /  at pos + r.  A 16-bit cache
 * narrows (the reference's to_half), a quantised one quantises. */
int saetta_kv_cache_store(saetta_kv_cache *cache, const float *k_dev, const float *v_dev,
                          const saetta_token_params *params_dev, size_t rows, void *stream);
int saetta_kv_cache_store_at(saetta_kv_cache *cache, const float *k_dev, const float *v_dev,
                             size_t pos, size_t tokens, void *stream);
/* ------------------------------------------------------------------ projections
 * src/qmv.rs:27-170 `GpuQuant::record` (kernel qmv<5|6|8>, kernels/qmv.metal:12-53) and
 * src/rows.rs:47-110 `record_proj` / `record_qmv_pk` (m rows): y[r][row] = sum_c W[row][c] x[r][c]
 * for m <= 8 rows, W [rows][cols] an MLX affine matrix (src/quant.rs:1-30): words_dev holds
 * rows * cols * bits / 32 u32 words (a little-endian bit stream per row), scales_dev / biases_dev
 * rows * cols / 64 bfloat16 values; x_dev [m][cols] f32; row r of y starts y_stride floats after
 * row r-1.  The q/k/v and o projections on either side of the attention path. */
int saetta_qmv_rows(int device, const uint32_t *words_dev, const uint16_t *scales_dev,
                    const uint16_t *biases_dev, int bits, size_t rows, size_t cols, size_t m,
                    const float *x_dev, float *y_dev, size_t y_stride, void *stream);

/* ------------------------------------------------------------------ record / replay
 * src/plan.rs:52-260 `Plan` and `Built`: dispatches recorded once and replayed
 * for every token, the only thing that changes being the TokenParams buffer.
 * On CUDA the recording is a stream capture and the replay a graph launch:
 *   saetta_plan_create                       Plan::new
 *   saetta_plan_params                       Plan::params (device pointer: pass it to every entry point
 *                                            that takes params_dev while recording)
 *   saetta_plan_begin ... entry points on saetta_plan_stream() ... saetta_plan_build
 *                                            the ops (`op` = stream order), then Plan::build
 *   saetta_plan_parallel_begin / _end        `op_parallel`: a side stream whose ops do not depend on the
 *                                            op before them; _end joins it back
 *   saetta_plan_set_params(token, position)  Plan::set_params(TokenParams::new(token, position))
 *   saetta_plan_run / _commit + _wait / _run_timed   Built::run / commit + Pending::wait / run_timed
 *   saetta_plan_len                          Plan::len (kernel launches recorded)
 * The host copy of TokenParams is uploaded by the graph's first node, so a
 * replay is a single graph launch; that node reads the host copy when the
 * replay executes, so call set_params before commit and not again until the
 * matching wait has returned.  Entry points that allocate (resize, an
 * AttGemm encode beyond what saetta_att_gemm_reserve was given) must not be
 * recorded.
 *   saetta_plan_kernels                      Plan::kernels: the distinct kernels of the recording and how
 *                                            many ops each has (names valid until the next begin / destroy)
 *   saetta_plan_build_where                  Plan::build_where(keep, barriers) (src/plan.rs:190-226): a
 *                                            second replayable object holding only the ops whose kernel
 *                                            name contains one of `keep` (n_keep = 0: all of them), with
 *                                            the recording's order carried over the dropped ops
 *                                            (barriers != 0) or with no order between kernels at all
 *                                            (barriers == 0: wrong results, a lower bound).  Copy nodes --
 *                                            the TokenParams upload among them -- are always kept.  For
 *                                            profiling, as in src/profile.rs:39-121: its results are not the
 *                                            plan's results.
 *   saetta_built_run_timed / _len / _destroy Built::run_timed, the number of ops kept, drop */
typedef struct saetta_plan saetta_plan;
int saetta_plan_create(int device, saetta_plan **out);
void saetta_plan_destroy(saetta_plan *plan);
const saetta_token_params *saetta_plan_params(const saetta_plan *plan);
void *saetta_plan_stream(const saetta_plan *plan);
int saetta_plan_begin(saetta_plan *plan);
int saetta_plan_parallel_begin(saetta_plan *plan, void **side_stream);
int saetta_plan_parallel_end(saetta_plan *plan);
int saetta_plan_build(saetta_plan *plan);
int saetta_plan_len(const saetta_plan *plan, size_t *ops);
int saetta_plan_set_params(saetta_plan *plan, uint32_t token, uint32_t position);
int saetta_plan_commit(saetta_plan *plan);
int saetta_plan_wait(saetta_plan *plan);
int saetta_plan_run(saetta_plan *plan);
int saetta_plan_run_timed(saetta_plan *plan, float *gpu_ms);
typedef struct saetta_built saetta_built;
int saetta_plan_kernels(saetta_plan *plan, const char **names_out, size_t *ops_out, size_t cap, size_t *count);
int saetta_plan_build_where(saetta_plan *plan, const char *const *keep, size_t n_keep, int barriers,
                            saetta_built **out);
void saetta_built_destroy(saetta_built *built);
int saetta_built_len(const saetta_built *built, size_t *ops);
int saetta_built_run_timed(saetta_built *built, float *gpu_ms);

/* ------------------------------------------------------------------ attention prep
 * kernels/layers.metal:637-697 `PrepParams`, `attention_prep` (16-bit cache) and
 * `attention_prep_float` + `QuantRows::record` (quantised cache), called from
 * GpuAttention::record_store (src/gpu_layers.rs:373-411) and per row from
 * record_rows (:483-507); for a chunk, the prefill's norm + rope_rows + store
 * (src/prefill.rs:1607-1633, 1656-1666).  Per token: q = rope(rms_norm(q) * q_norm),
 * k = rope(rms_norm(k) * k_norm), and k, v into the token's cache slot in
 * whatever form the cache holds -- one launch, the keys never pass through
 * memory as f32.  rows tokens at params_dev->position + r (decode / verify; read
 * on the device, capturable) or, with params_dev NULL, at pos + r (prefill).
 * q_and_gate_dev [rows][heads][2*head_dim] (q first), k_dev / v_dev
 * [rows][kv_heads][head_dim] f32; q_out_dev [rows][heads][head_dim] of q_dtype
 * (SAETTA_F32 for decode, 16-bit for the prefill kernels); k_out_dev, when not
 * NULL, also receives the normed and roped keys as f32 (what
 * attention_prep_float leaves in k; may be k_dev itself).  The angle is formed
 * in f64 as the CPU does (src/cpu/ops.rs:64-74), not in f32 as the Metal kernel. */
typedef struct saetta_prep_params {
    uint32_t heads, kv_heads, head_dim;
    uint32_t rope_dims; /* rotary dims (2 * half_dims), a multiple of 16, at most 128 */
    float rope_theta;
    float eps;
} saetta_prep_params;
int saetta_attention_prep(saetta_prep_params p, size_t rows, const float *q_and_gate_dev,
                          const float *k_dev, const float *v_dev, const float *q_norm_dev,
                          const float *k_norm_dev, void *q_out_dev, int q_dtype,
                          saetta_kv_cache *cache, const saetta_token_params *params_dev,
                          size_t pos, float *k_out_dev, void *stream);

/* dtype of a 16-bit cache's rows (SAETTA_F16 unless set otherwise before use). */
int saetta_kv_cache_set_dtype(saetta_kv_cache *cache, int dtype);

/* ------------------------------------------------------------------ RowBackup
 * src/gpu_cache.rs:192-286 `RowBackup`: rows from..from+n of every buffer of
 * every cache copied aside and put back by byte ranges.
 */
typedef struct saetta_row_backup saetta_row_backup;
int saetta_row_backup_create(saetta_row_backup **out);
void saetta_row_backup_destroy(saetta_row_backup *b);
int saetta_row_backup_save(saetta_row_backup *b, saetta_kv_cache *const *caches, size_t n_caches,
                           size_t from, size_t n, void *stream);
int saetta_row_backup_restore(saetta_row_backup *b, saetta_kv_cache *const *caches,
                              size_t n_caches, void *stream);
void saetta_row_backup_clear(saetta_row_backup *b);
uint64_t saetta_row_backup_bytes(const saetta_row_backup *b);

/* ------------------------------------------------------------------ DecodeAttention / AttentionRows
 * src/attention.rs:19-171 `DecodeAttention` and src/rows.rs:307-494
 * `AttentionRows`: out = softmax(q K^T / 16) V * sigmoid(gate) for m rows over
 * the cache; row r sees params_dev->kv_len + r keys.  One object holds the
 * split-KV scratch for one capacity; layers that run one after the other share
 * it.  q [m][heads][256] f32, q_and_gate [m][heads][512] f32 with the gate of
 * head h at h*512+256, out [m][heads][256] f32.
 */
#define SAETTA_MAX_ROWS 8 /* src/rows.rs:9 */
typedef struct saetta_decode saetta_decode;

/* DecodeAttention::new(gpu, heads, kv_heads, head_dim, capacity) when rows == 1,
 * AttentionRows::new(gpu, heads, kv_heads, capacity, rows) otherwise. */
int saetta_decode_create(int device, size_t heads, size_t kv_heads, size_t head_dim,
                         size_t capacity, size_t rows, saetta_decode **out);
void saetta_decode_destroy(saetta_decode *op);
/* DecodeAttention::record / AttentionRows::record: a 16-bit (dtype) or f32
 * (dtype = -1) cache [capacity][kv_heads][256]. */
int saetta_decode_record(saetta_decode *op, size_t m, const float *q_dev, const void *keys_dev,
                         const void *values_dev, int dtype, const float *q_and_gate_dev,
                         float *out_dev, const saetta_token_params *params_dev, void *stream);
/* DecodeAttention::record_quant / AttentionRows::record_quant. */
int saetta_decode_record_quant(saetta_decode *op, size_t m, const float *q_dev,
                               const saetta_quant_rows *keys, const saetta_quant_rows *values,
                               const float *q_and_gate_dev, float *out_dev,
                               const saetta_token_params *params_dev, void *stream);
/* Either of the two, picked by the cache's bits. */
int saetta_decode_record_cache(saetta_decode *op, size_t m, const float *q_dev,
                               const saetta_kv_cache *cache, const float *q_and_gate_dev,
                               float *out_dev, const saetta_token_params *params_dev,
                               void *stream);
/* No counterpart in the reference.  The same computation as
 * saetta_decode_record_quant for m = 1 or 2 rows, for callers that are not
 * allowed to allocate device memory: a host process whose memory pool was sized
 * up front and hands this library no allocator, or a latency-critical decode
 * loop in which cudaMalloc (which serialises the device) must never run.  No
 * op object is needed and nothing is allocated, now or later: the split-KV
 * partials go to a fixed array inside the library's device image (about 5.3 MB,
 * resident on every GPU that loads the library until the process exits).
 * Limits: m <= 2, 2 kv heads, capacity a multiple of 32; anything larger is
 * refused with SAETTA_ERR_BAD_SHAPE and should go through saetta_decode_create.
 * The first call on a device looks up the array's device address and raises the
 * kernel's shared-memory limit; make that call once outside any stream capture.
 * All calls on a device share the one array: two calls that overlap on the GPU
 * (different streams) race on it and give wrong results; calls ordered on one
 * stream are fine, and nothing needs clearing between them. */
int saetta_decode_record_quant_static(int device, size_t m, const float *q_dev,
                                      const saetta_quant_rows *keys,
                                      const saetta_quant_rows *values,
                                      const float *q_and_gate_dev, float *out_dev,
                                      const saetta_token_params *params_dev, void *stream);
/* The status word of saetta_decode_record_quant_static on `device`: its kernels'
 * bounded waits set bits there when one of them gives up (the output of that
 * call is then void), and the word is shared by every call on the device, like
 * the scratch.  Synchronises `stream`, returns SAETTA_ERR_TIMEOUT when the word
 * is not 0, and with clear != 0 puts it back to 0 after reading.  Allocates
 * nothing.  No counterpart in the reference. */
int saetta_decode_static_status(int device, void *stream, uint32_t *status, int clear);
/* Number of split-KV parts the op launches (its grid), and the device status
 * word of its bounded waits: 0 when no wait ever gave up.  Synchronises `stream`. */
int saetta_decode_splits(const saetta_decode *op);
int saetta_decode_device_status(saetta_decode *op, void *stream, uint32_t *status);

/* Batched decode, one row per sequence (no counterpart in the reference, which
 * serves one sequence): sequence i reads caches[i] up to kv_lens_dev[i] keys,
 * q [n][heads][256], q_and_gate [n][heads][512], out [n][heads][256].  All
 * caches share bits, and the op's capacity bounds every kv_len. */
typedef struct saetta_decode_batch saetta_decode_batch;
int saetta_decode_batch_create(int device, size_t heads, size_t kv_heads, size_t head_dim,
                               size_t max_seqs, size_t max_total_tokens,
                               saetta_decode_batch **out);
void saetta_decode_batch_destroy(saetta_decode_batch *op);
int saetta_decode_batch_record(saetta_decode_batch *op, size_t n,
                               saetta_kv_cache *const *caches, const uint32_t *kv_lens_host,
                               const float *q_dev, const float *q_and_gate_dev, float *out_dev,
                               void *stream);

/* ------------------------------------------------------------------ split-KV across GPUs
 * No counterpart in the reference (one GPU).  Each rank holds a disjoint set of
 * KV rows and produces, per (row, head), the partial (m, l, O) of
 * kernels/attention.metal:367-409's merge: part [m][heads][SAETTA_PART_STRIDE]
 * f32 = 256 unnormalised outputs, then the running max (in log2 units) and the
 * sum.  After the ranks' parts are gathered into [ranks][m][heads][stride] (an
 * NCCL all-gather on the caller's side), merge applies the gate.
 */
#define SAETTA_PART_STRIDE 264
/* row_step 1: row r sees params_dev->kv_len + r keys (the shard that holds the
 * new rows); 0: every row sees kv_len keys (the other shards). */
int saetta_decode_partial_cache(saetta_decode *op, size_t m, const float *q_dev,
                                const saetta_kv_cache *cache, float *part_dev, uint32_t row_step,
                                const saetta_token_params *params_dev, void *stream);
int saetta_merge_partials(int device, const float *parts_dev, size_t ranks, size_t rows,
                          size_t heads, const float *q_and_gate_dev, float *out_dev, void *stream);

/* The same merge fused with its exchange: no all-gather.  The kernel that
 * finishes a rank's partial stores it straight into every peer's mailbox over
 * NVLink (plain peer stores, every word tagged with the exchange number), and
 * one kernel per rank polls its own memory, merges what arrived and gates.  One process per GPU: create a
 * group on every rank, exchange the 64-byte handles (any host-side
 * all-gather), connect, then per exchange either
 *   saetta_decode_publish_cache + saetta_peer_collect   (decode / verify), or
 *   a partial written to saetta_peer_group_staging() + saetta_peer_merge
 *   (any other partial, e.g. saetta_att_gemm_partial; publishes, then collects)
 * on every rank.  The sequence counter lives on the device, so the launches can
 * sit in a captured CUDA graph.  The wait for a peer is bounded (about a
 * second); saetta_peer_group_status reports a peer that never published.  All
 * ranks must perform the same number of exchanges, and ONE exchange is outstanding
 * per group at a time: a second publish before the collect of the first reuses its
 * number and overwrites it. */
typedef struct saetta_peer_group saetta_peer_group;
int saetta_peer_group_create(int device, int rank, int world, size_t rows_max, size_t heads,
                             uint8_t handle_out[64], saetta_peer_group **out);
int saetta_peer_group_connect(saetta_peer_group *g, const uint8_t *handles /* [world][64] in rank order */);
void saetta_peer_group_destroy(saetta_peer_group *g);
float *saetta_peer_group_staging(saetta_peer_group *g);
int saetta_peer_merge(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev, float *out_dev,
                      void *stream);
int saetta_peer_collect(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev,
                        float *out_dev, void *stream);
/* For many rows (a prefill chunk's partial in the staging buffer): rank j finalises rows
 * [j*rows/world, (j+1)*rows/world) only (saetta_peer_slice), so every rank sends each peer just that
 * peer's slice and writes just its own rows of out_dev [rows][heads][256]; q_and_gate_dev is indexed by
 * the global row. */
int saetta_peer_merge_sliced(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev,
                             float *out_dev, void *stream);
int saetta_peer_slice(const saetta_peer_group *g, size_t rows, size_t *row_lo, size_t *row_hi);
/* saetta_decode_partial_cache with the partial published to the group instead
 * of written to a buffer (m rows, heads as the group was made for). */
/* saetta_decode_batch_record on one shard of every sequence: sequence i's partial is row i of the
 * exchange (n <= the group's rows_max); follow with saetta_peer_collect(g, n, ...). */
int saetta_decode_batch_publish(saetta_decode_batch *op, size_t n, saetta_kv_cache *const *caches,
                                const uint32_t *kv_lens_host, const float *q_dev,
                                saetta_peer_group *group, void *stream);
int saetta_decode_publish_cache(saetta_decode *op, size_t m, const float *q_dev,
                                const saetta_kv_cache *cache, saetta_peer_group *group,
                                uint32_t row_step, const saetta_token_params *params_dev,
                                void *stream);
/* saetta_decode_publish_cache and saetta_peer_collect as ONE launch: the merge CTAs of the decode
 * launch store this rank's partial into the peers' mailboxes and then wait, in the same kernel, for
 * the peers' partials of the same exchange, merge over the ranks and gate -- no second launch and no
 * kernel boundary between the two.  Same bounded wait and status word as saetta_peer_collect. */
int saetta_decode_exchange_cache(saetta_decode *op, size_t m, const float *q_dev,
                                 const saetta_kv_cache *cache, saetta_peer_group *group,
                                 uint32_t row_step, const float *q_and_gate_dev, float *out_dev,
                                 const saetta_token_params *params_dev, void *stream);
int saetta_peer_group_status(saetta_peer_group *g, void *stream, uint32_t *status);
/* Recovery after a collect that gave up, which leaves the ranks' exchange counters
 * apart (every later collect would time out too) and the status word set.  Call it
 * on EVERY rank with the same `seq`, between two host barriers: the first after each
 * rank's stream has drained (no exchange in flight anywhere), the second before the
 * next exchange.  It empties this rank's mailbox, sets both of its counters to `seq`
 * (the next exchange is number seq + 1) and clears its status word.  A CUDA graph
 * recorded before the reset stays valid: the counters are read on the device. */
int saetta_peer_group_reset(saetta_peer_group *g, uint32_t seq, void *stream);

/* ------------------------------------------------------------------ prefill
 * src/attention_prefill.rs:39-72 `encode` and src/attention_gemm.rs:93-363
 * `AttGemm`: causal attention of a chunk of p.tokens query tokens at p.pos over
 * keys 0 .. p.pos + i, gate fused.  q 16-bit [tokens][heads][256], keys/values
 * the 16-bit cache from position 0 with the chunk's rows already written,
 * q_and_gate f32 [tokens][heads][512], out f32 [tokens][heads][256].
 */
typedef struct saetta_att_gemm saetta_att_gemm;
/* AttGemm::new(gpu, chunk, kv_heads). */
int saetta_att_gemm_create(int device, size_t chunk, size_t kv_heads, saetta_att_gemm **out);
void saetta_att_gemm_destroy(saetta_att_gemm *op);
/* Allocates now all the scratch encodes over caches of up to `tokens` rows need
 * -- the 16-bit copies a quantised (or bfloat16-valued) cache is read through,
 * and the partials of the key splits of a long-context chunk -- as AttGemm::new
 * does (src/attention_gemm.rs:119-148), so that later encodes allocate nothing
 * and can be recorded in a Plan.  Without it an encode grows the scratch when it
 * has to, and refuses to when its stream is being captured. */
int saetta_att_gemm_reserve(saetta_att_gemm *op, size_t tokens);
/* The 16-bit copy persists between encodes: per chunk of a long prompt only the
 * rows from the chunk's first row on are converted, the rows below it are taken
 * as converted by the encode of the chunk before (same buffers, same types).  A
 * caller that rewrites rows BELOW the position of its next chunk outside of this
 * sequence (not a rewind followed by a new prefill from there, which is covered)
 * says so here, and the next encode converts every row it reads again. */
int saetta_att_gemm_invalidate(saetta_att_gemm *op);
/* How encode / partial read an 8/4-bit cache.  Off (the default): in place, per key
 * block, as the reference's attention_rows_q kernels read it
 * (kernels/attention_rows_q.metal:16-31,206-344); no 16-bit copy exists.  On: through
 * the op's 16-bit staging copy, the reference's kv_stage route (src/prefill.rs), of
 * which each call converts only the rows it does not hold yet: faster over long
 * prefixes (every row is converted once instead of once per query tile), for 2 KB
 * of device memory per key and side. */
int saetta_att_gemm_stage_quantised(saetta_att_gemm *op, int on);
/* Which kernel serves a 16-bit cache (and the staging copy): score blocks of 128 keys
 * (the default; about a tenth faster over long prefixes) or of 64 keys (the kernel the
 * quantised in-place route is built on).  Same results to rounding; no counterpart in
 * the reference.  keys: 64 or 128. */
int saetta_att_gemm_score_blocks(saetta_att_gemm *op, int keys);
/* AttGemm::encode: with keys_q/values_q non-NULL the cache is read from those
 * 8/4-bit rows (see saetta_att_gemm_stage_quantised) and keys_dev/values_dev are
 * ignored. */
int saetta_att_gemm_encode(saetta_att_gemm *op, const void *q_dev, int dtype, const void *keys_dev,
                           const void *values_dev, const saetta_quant_rows *keys_q,
                           const saetta_quant_rows *values_q, const float *q_and_gate_dev,
                           float *out_dev, saetta_flash_params p, void *stream);
/* The prefill's row route: src/prefill.rs:1674-1686 selects attention_rows /
 * attention_rows_q8|q4 (the AttentionRows kernels over the chunk's rows) instead of
 * the GEMM path for its exact mode.  Here the chunk goes through a decode op in
 * groups of up to its `rows` rows; row r sees keys 0 ..= pos + r of `cache`, which
 * already holds the chunk's rows.  q_dev is f32 [tokens][heads][256].  An f32 cache
 * gets f32 arithmetic throughout; 16-bit and quantised caches the tensor-core row
 * kernels.  params_scratch_dev: ceil(tokens / rows) saetta_token_params on the
 * device, written by the call.  Not capturable. */
int saetta_prefill_rows_cache(saetta_decode *op, const float *q_dev, const saetta_kv_cache *cache,
                              const float *q_and_gate_dev, float *out_dev, saetta_flash_params p,
                              saetta_token_params *params_scratch_dev, void *stream);
/* attention_prefill::encode: the same computation with no object, over a binary16
 * cache (what the reference's function takes).  dtype must be SAETTA_F16: the
 * tensor-core kernel gives P the values' type, and bfloat16's 8-bit significand
 * would put P's rounding at the tolerance; AttGemm stages bfloat16 values as
 * binary16 in its own scratch, which a call without an object has nowhere to
 * keep, so bfloat16 is refused here with SAETTA_ERR_UNSUPPORTED. */
int saetta_prefill_encode(int device, const void *q_dev, int dtype, const void *keys_dev,
                          const void *values_dev, const float *q_and_gate_dev, float *out_dev,
                          saetta_flash_params p, void *stream);
/* As saetta_att_gemm_encode, but keys [lo, hi) only and the result left as the
 * partial (m, l, O) of SAETTA_PART_STRIDE floats per (token, head) for the
 * cross-GPU merge; hi is clipped per token by causality. */
int saetta_att_gemm_partial(saetta_att_gemm *op, const void *q_dev, int dtype,
                            const void *keys_dev, const void *values_dev,
                            const saetta_quant_rows *keys_q, const saetta_quant_rows *values_q,
                            float *part_dev, saetta_flash_params p, size_t key_lo, size_t key_hi,
                            void *stream);

/* The same for a shard that STORES only its own slice of the sequence (no
 * counterpart in the reference): row 0 of keys_dev / values_dev / the quantised
 * rows is the key at global position key_base (a multiple of 64, at most
 * key_lo), and the buffers hold at least key_hi - key_base rows.  p.pos and
 * key_lo / key_hi stay global positions. */
int saetta_att_gemm_partial_shard(saetta_att_gemm *op, const void *q_dev, int dtype,
                                  const void *keys_dev, const void *values_dev,
                                  const saetta_quant_rows *keys_q, const saetta_quant_rows *values_q,
                                  float *part_dev, saetta_flash_params p, size_t key_base,
                                  size_t key_lo, size_t key_hi, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SAETTA_B200_H */
