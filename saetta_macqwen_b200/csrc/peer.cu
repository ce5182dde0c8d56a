// Split-KV merge across the GPUs of one box, fused with its exchange.
//
// No counterpart in the reference (one GPU).  Each rank's decode / prefill
// kernels produce the (m, l, O) partial of its KV shard.  Instead of an
// all-gather followed by a merge, the kernel that finishes the partial stores
// it straight into every peer's mailbox over NVLink (plain peer stores through
// NVSwitch; no multicast, no library kernel on peer memory), and polls its own
// memory for the peers' words, merges and gates what has arrived: for decode
// and verify that is all one launch per rank (the merge CTAs of the decode
// kernel, merge_role.cuh); the kernels in this file are the two-launch form and
// the route for partials that other kernels leave in the staging buffer.  A
// partial crosses NVLink once, as fire-and-forget stores; nothing waits on a
// remote read or on an acknowledgement.
//
// Mailbox protocol (memory shared between processes with CUDA IPC handles):
// every rank owns two slots, each with room for one partial per rank.  A slot
// holds 64-bit words: a float and the number of the exchange it belongs to,
// written by one 64-bit store.  For exchange number seq a rank writes its
// partial into place (seq & 1, its rank) of every mailbox; the merge polls its
// own slot seq & 1 until each word it needs carries seq, so a value is used as
// soon as it has landed and no flag or fence sits between the ranks (one NVLink
// crossing, not a round trip).  Two slots are enough: a rank cannot write
// exchange seq+2 before every peer has finished reading exchange seq, because
// its own merge of seq+1 waits for the peers' seq+1 words, which they send only
// after their merge of seq.  The exchange numbers live in device memory, so a
// captured CUDA graph of these launches replays correctly: the publishing
// kernel reads the count of exchanges collected and writes the count sent, the
// collecting kernel the other way round, so no kernel reads a word that one of
// its own blocks writes.  The wait is bounded: after the limit the kernel sets
// a status bit and leaves.
#include <algorithm>
#include <cstring>
#include <new>

#include "host.hpp"

namespace saetta {

// One block: copies the staging partial into every mailbox.
__global__ void __launch_bounds__(1024)
publish_kernel(const float *__restrict__ staging, const PeerPush push, uint32_t n_floats) {
    pdl_wait();
    const uint32_t s = *push.seq_done + 1;
    const size_t at = (size_t(s & 1) * push.world + push.rank) * push.slot_floats;
    for (uint32_t i = threadIdx.x; i < n_floats; i += blockDim.x) {
        const unsigned long long w = peer_word(staging[i], s);
        for (uint32_t r = 0; r < push.world; r++)
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(push.parts[r] + at + i), "l"(w) : "memory");
    }
    if (threadIdx.x == 0) *push.seq_sent = s;
}

// Row-sliced publish: rank j finalises rows [j*rows/world, (j+1)*rows/world), so only that slice of
// the staging partial goes to rank j's mailbox (at its natural row offset).  grid (blocks, world).
__global__ void __launch_bounds__(1024)
publish_rows_kernel(const float *__restrict__ staging, const PeerPush push, uint32_t rows, uint32_t row_floats) {
    pdl_wait();
    const uint32_t s = *push.seq_done + 1;
    const uint32_t j = blockIdx.y;
    const size_t lo = size_t(rows) * j / push.world * row_floats, hi = size_t(rows) * (j + 1) / push.world * row_floats;
    unsigned long long *dst = push.parts[j] + (size_t(s & 1) * push.world + push.rank) * push.slot_floats;
    for (size_t i = lo + size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < hi; i += size_t(gridDim.x) * blockDim.x)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + i), "l"(peer_word(staging[i], s)) : "memory");
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *push.seq_sent = s;
}

// Polls one mailbox word until it carries exchange number `s`; false after `limit` polls.
__device__ __forceinline__ bool peer_poll(const unsigned long long *p, uint32_t s, uint32_t limit, float &v) {
    for (uint32_t n = 0; n < limit; n++) {
        unsigned long long w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if (uint32_t(w >> 32) == s) {
            v = __uint_as_float(uint32_t(w));
            return true;
        }
        if (n > 16) __nanosleep(50);
    }
    return false;
}

// grid (heads, rows), 256 threads = one per dim; rows row0 .. row0 + gridDim.y - 1.  Reads this rank's own mailbox only.
__global__ void __launch_bounds__(256)
peer_merge_kernel(const unsigned long long *__restrict__ slots, uint32_t world, const uint32_t *seq_sent,
                  uint32_t *seq_done, uint32_t slot_floats, uint32_t heads, const float *__restrict__ q_and_gate,
                  float *__restrict__ out, uint32_t *status, uint32_t poll_limit, uint32_t row0) {
    pdl_wait();
    __shared__ float ml_s[kMaxPeers][2];
    __shared__ uint32_t s_bad;
    const uint32_t s = *seq_sent;
    const uint32_t head = blockIdx.x, row = row0 + blockIdx.y, dim = threadIdx.x;
    const size_t rh = size_t(row) * heads + head;
    const unsigned long long *base = slots + size_t(s & 1) * world * slot_floats + rh * kPartStride;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    bool ok = true;
    if (threadIdx.x < 2 * world) // m and l of every rank
        ok = peer_poll(base + size_t(threadIdx.x >> 1) * slot_floats + kPartM + (threadIdx.x & 1), s, poll_limit,
                       ml_s[threadIdx.x >> 1][threadIdx.x & 1]);
    float o[kMaxPeers];
#pragma unroll
    for (uint32_t r = 0; r < kMaxPeers; r++) {
        o[r] = 0.f;
        if (r < world && ok) ok = peer_poll(base + size_t(r) * slot_floats + dim, s, poll_limit, o[r]);
    }
    if (!ok) s_bad = 1;
    __syncthreads();
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *seq_done = s;
    if (s_bad) { // a peer never published: leave `out` as it is, the host sees the status word
        if (threadIdx.x == 0) atomicOr(status, kStatusFullTimeout);
        return;
    }
    float M = -INFINITY;
    for (uint32_t r = 0; r < world; r++) M = fmaxf(M, ml_s[r][0]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < kMaxPeers; r++) {
        if (r >= world || ml_s[r][0] == -INFINITY) continue;
        const float w = exp2f(ml_s[r][0] - M);
        l = fmaf(ml_s[r][1], w, l);
        acc = fmaf(o[r], w, acc);
    }
    const float g = q_and_gate[rh * 2 * kDim + kDim + dim];
    out[rh * kDim + dim] = acc / l * (1.0f / (1.0f + expf(-g)));
}

// The 32-bit words after the slots.
static uint32_t *group_words(const saetta_peer_group *g) {
    return reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(g->mailbox) + g->words_offset());
}
constexpr int kSeqDoneWord = 0, kSeqSentWord = 1, kStatusWord = 32;

int launch_peer_publish(saetta_peer_group *g, size_t rows, cudaStream_t stream) {
    const uint32_t n = uint32_t(rows * g->heads * kPartStride);
    SAETTA_CUDA(launch_pdl(publish_kernel, dim3(1), dim3(1024), 0, stream, (const float *)g->staging, g->push, n));
    return SAETTA_OK;
}

} // namespace saetta

using namespace saetta;

extern "C" {

int saetta_peer_group_create(int device, int rank, int world, size_t rows_max, size_t heads, uint8_t handle_out[64],
                             saetta_peer_group **out) {
    if (!out || !handle_out) return fail(SAETTA_ERR_BAD_ARG, "peer group: null pointer");
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return fail(SAETTA_ERR_BAD_SHAPE, "peer group: 1..8 ranks");
    if (!rows_max || !heads) return fail(SAETTA_ERR_BAD_SHAPE, "peer group: empty shape");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "peer group: cannot select the device");
    auto *g = new (std::nothrow) saetta_peer_group();
    if (!g) return fail(SAETTA_ERR_NO_MEM, "peer group: host allocation");
    g->device = device, g->rank = rank, g->world = world, g->rows_max = rows_max, g->heads = heads;
    g->slot_floats = rows_max * heads * kPartStride;
    const size_t bytes = g->words_offset() + 256;
    cudaError_t e = cudaMalloc(&g->mailbox, bytes);
    if (e == cudaSuccess) e = cudaMemset(g->mailbox, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&g->staging, g->slot_floats * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(g->staging, 0, g->slot_floats * sizeof(float));
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, g->mailbox);
    if (e != cudaSuccess) {
        cudaFree(g->mailbox), cudaFree(g->staging);
        delete g;
        return cuda_fail(e, "peer group: mailbox");
    }
    memcpy(handle_out, &h, 64);
    *out = g;
    return SAETTA_OK;
}

int saetta_peer_group_connect(saetta_peer_group *g, const uint8_t *handles /* [world][64], rank order */) {
    if (!g || !handles) return fail(SAETTA_ERR_BAD_ARG, "peer group: null pointer");
    if (g->connected) return fail(SAETTA_ERR_BAD_ARG, "peer group: already connected");
    DeviceGuard guard(g->device);
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank) {
            g->peer_base[r] = g->mailbox;
        } else {
            cudaIpcMemHandle_t h;
            memcpy(&h, handles + size_t(r) * 64, 64);
            SAETTA_CUDA(cudaIpcOpenMemHandle(&g->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess));
        }
        g->push.parts[r] = reinterpret_cast<unsigned long long *>(g->peer_base[r]);
    }
    g->push.seq_done = group_words(g) + kSeqDoneWord, g->push.seq_sent = group_words(g) + kSeqSentWord;
    g->push.status = group_words(g) + kStatusWord;
    g->push.world = uint32_t(g->world), g->push.rank = uint32_t(g->rank), g->push.slot_floats = uint32_t(g->slot_floats);
    g->connected = true;
    return SAETTA_OK;
}

void saetta_peer_group_destroy(saetta_peer_group *g) {
    if (!g) return;
    DeviceGuard guard(g->device);
    for (int r = 0; r < g->world; r++)
        if (r != g->rank && g->peer_base[r]) cudaIpcCloseMemHandle(g->peer_base[r]);
    cudaFree(g->mailbox);
    cudaFree(g->staging);
    delete g;
}

float *saetta_peer_group_staging(saetta_peer_group *g) { return g ? g->staging : nullptr; }

static int peer_check(const saetta_peer_group *g, size_t rows, const void *a, const void *b) {
    if (!g || !a || !b) return fail(SAETTA_ERR_BAD_ARG, "peer merge: null pointer");
    if (!g->connected) return fail(SAETTA_ERR_BAD_ARG, "peer merge: the group is not connected");
    if (!rows || rows > g->rows_max) return fail(SAETTA_ERR_BAD_SHAPE, "peer merge: more rows than the group was made for");
    return SAETTA_OK;
}

static int collect_rows(saetta_peer_group *g, size_t row0, size_t rows, const float *q_and_gate_dev, float *out_dev,
                        cudaStream_t stream) {
    if (!rows) return SAETTA_OK; // (a rank that owns no row still took part through its publish)
    uint32_t *words = group_words(g);
    SAETTA_CUDA(launch_pdl(peer_merge_kernel, dim3(unsigned(g->heads), unsigned(rows)), dim3(256), 0, stream,
                           (const unsigned long long *)g->mailbox, uint32_t(g->world),
                           (const uint32_t *)(words + kSeqSentWord), words + kSeqDoneWord, uint32_t(g->slot_floats),
                           uint32_t(g->heads), q_and_gate_dev, out_dev, words + kStatusWord, 1000000u, uint32_t(row0)));
    return SAETTA_OK;
}

int saetta_peer_collect(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev, float *out_dev, void *stream) {
    if (int rc = peer_check(g, rows, q_and_gate_dev, out_dev)) return rc;
    DeviceGuard guard(g->device);
    return collect_rows(g, 0, rows, q_and_gate_dev, out_dev, (cudaStream_t)stream);
}

int saetta_peer_slice(const saetta_peer_group *g, size_t rows, size_t *row_lo, size_t *row_hi) {
    if (!g || !row_lo || !row_hi) return fail(SAETTA_ERR_BAD_ARG, "peer slice: null pointer");
    *row_lo = rows * size_t(g->rank) / size_t(g->world), *row_hi = rows * size_t(g->rank + 1) / size_t(g->world);
    return SAETTA_OK;
}

int saetta_peer_merge_sliced(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev, float *out_dev, void *stream) {
    if (int rc = peer_check(g, rows, q_and_gate_dev, out_dev)) return rc;
    if (rows < size_t(g->world)) return fail(SAETTA_ERR_BAD_SHAPE, "peer merge: fewer rows than ranks");
    DeviceGuard guard(g->device);
    const uint32_t row_floats = uint32_t(g->heads * kPartStride);
    const size_t per_rank = (rows / g->world + 1) * row_floats;
    const unsigned blocks = unsigned(std::min<size_t>(64, (per_rank + 4095) / 4096));
    SAETTA_CUDA(launch_pdl(publish_rows_kernel, dim3(blocks, unsigned(g->world)), dim3(1024), 0, (cudaStream_t)stream,
                           (const float *)g->staging, g->push, uint32_t(rows), row_floats));
    size_t lo, hi;
    saetta_peer_slice(g, rows, &lo, &hi);
    return collect_rows(g, lo, hi - lo, q_and_gate_dev, out_dev, (cudaStream_t)stream);
}

int saetta_peer_merge(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev, float *out_dev, void *stream) {
    if (int rc = peer_check(g, rows, q_and_gate_dev, out_dev)) return rc;
    DeviceGuard guard(g->device);
    if (int rc = launch_peer_publish(g, rows, (cudaStream_t)stream)) return rc;
    return saetta_peer_collect(g, rows, q_and_gate_dev, out_dev, stream);
}

int saetta_peer_group_status(saetta_peer_group *g, void *stream, uint32_t *status) {
    if (!g || !status) return fail(SAETTA_ERR_BAD_ARG, "peer status: null pointer");
    DeviceGuard guard(g->device);
    const uint32_t *dev = group_words(g) + kStatusWord;
    SAETTA_CUDA(cudaMemcpyAsync(status, dev, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SAETTA_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (*status) return fail(SAETTA_ERR_TIMEOUT, "a peer did not publish its partial in time");
    return SAETTA_OK;
}

// After a collect gave up, the ranks' counters differ (the one that waited counts the exchange as done, the
// one that stayed away never sent it), so every later exchange would use different numbers and slots.
// This puts one rank's group back: its own mailbox emptied (number 0 matches no exchange), both
// counters at `seq`, the status word cleared.  Host-side only; nothing of it runs on a peer's memory.
int saetta_peer_group_reset(saetta_peer_group *g, uint32_t seq, void *stream) {
    if (!g) return fail(SAETTA_ERR_BAD_ARG, "peer reset: null handle");
    DeviceGuard guard(g->device);
    cudaStream_t st = (cudaStream_t)stream;
    SAETTA_CUDA(cudaStreamSynchronize(st));
    SAETTA_CUDA(cudaMemsetAsync(g->mailbox, 0, g->words_offset(), st));
    uint32_t *words = group_words(g);
    const uint32_t counters[2] = {seq, seq};
    static_assert(kSeqDoneWord == 0 && kSeqSentWord == 1, "the two counters are set with one copy");
    SAETTA_CUDA(cudaMemcpyAsync(words, counters, sizeof(counters), cudaMemcpyHostToDevice, st));
    SAETTA_CUDA(cudaMemsetAsync(words + kStatusWord, 0, 4, st));
    SAETTA_CUDA(cudaStreamSynchronize(st));
    return SAETTA_OK;
}

} // extern "C"
