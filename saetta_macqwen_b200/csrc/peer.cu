// Split-KV merge across the GPUs of one box, fused with its exchange.
//
// No counterpart in the reference (one GPU).  Each rank's decode / prefill
// kernels leave the (m, l, O) partial of its KV shard in a local staging
// buffer.  Instead of an all-gather followed by a merge, ONE kernel per rank
// waits for every peer's partial to be published and reads it straight out of
// the peer's memory over NVLink (plain peer loads through NVSwitch; no
// multicast, no library kernel on peer memory), merging and gating as it goes.
//
// Mailbox protocol (memory shared between processes with CUDA IPC handles):
// every rank owns two slots of partials and two flags.  publish_kernel copies
// the staging partial into slot (seq & 1) and then stores seq into that slot's
// flag with release semantics at system scope.  peer_merge_kernel acquires every
// rank's flag until it equals seq, then reads the slots.  Two slots are enough:
// a rank cannot publish exchange seq+2 before every peer has finished reading
// exchange seq, because its own merge of seq+1 waits for the peers' seq+1 flags,
// which they set only after their merge of seq.  The sequence number lives in
// device memory, so a captured CUDA graph of these launches replays correctly.
// The wait is bounded: after the limit the kernel sets a status bit and leaves.
#include <cstring>
#include <new>

#include "host.hpp"

namespace saetta {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
    const float *parts[kMaxPeers];       // each rank's [2][slot_floats]
    const uint32_t *flags[kMaxPeers];    // each rank's [2]
};

__global__ void __launch_bounds__(256)
publish_kernel(const float *__restrict__ staging, float *__restrict__ slots, uint32_t *flags, uint32_t *seq_dev,
               uint32_t n_floats, uint32_t slot_floats) {
    pdl_wait();
    __shared__ uint32_t s_seq;
    if (threadIdx.x == 0) s_seq = *seq_dev + 1;
    __syncthreads();
    const uint32_t s = s_seq;
    float *dst = slots + size_t(s & 1) * slot_floats;
    for (uint32_t i = threadIdx.x; i < n_floats; i += blockDim.x) dst[i] = staging[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        *seq_dev = s;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags + (s & 1)), "r"(s) : "memory");
    }
}

// grid (heads, rows), 256 threads = one per dim.
__global__ void __launch_bounds__(256)
peer_merge_kernel(PeerPtrs peers, uint32_t world, const uint32_t *seq_dev, uint32_t slot_floats, uint32_t heads,
                  const float *__restrict__ q_and_gate, float *__restrict__ out, uint32_t *status,
                  uint32_t poll_limit) {
    pdl_wait();
    __shared__ uint32_t s_ok;
    const uint32_t s = *seq_dev;
    if (threadIdx.x < world) {
        const uint32_t *flag = peers.flags[threadIdx.x] + (s & 1);
        uint32_t v = 0, n = 0;
        do {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v == s) break;
            __nanosleep(200);
        } while (++n < poll_limit);
        if (v != s) atomicOr(status, kStatusFullTimeout);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_ok = (*reinterpret_cast<volatile uint32_t *>(status)) == 0;
    __syncthreads();
    if (!s_ok) return; // a peer never published: leave `out` as it is, the host sees the status word

    const uint32_t head = blockIdx.x, row = blockIdx.y, dim = threadIdx.x;
    const size_t rh = size_t(row) * heads + head;
    float M = -INFINITY;
    for (uint32_t r = 0; r < world; r++)
        M = fmaxf(M, __ldcv(peers.parts[r] + size_t(s & 1) * slot_floats + rh * kPartStride + kPartM));
    float acc = 0.f, l = 0.f;
    for (uint32_t r = 0; r < world; r++) {
        const float *pp = peers.parts[r] + size_t(s & 1) * slot_floats + rh * kPartStride;
        const float mp = __ldcv(pp + kPartM);
        if (mp == -INFINITY) continue;
        const float w = exp2f(mp - M);
        l = fmaf(__ldcv(pp + kPartL), w, l);
        acc = fmaf(__ldcv(pp + dim), w, acc);
    }
    const float g = q_and_gate[rh * 2 * kDim + kDim + dim];
    out[rh * kDim + dim] = acc / l * (1.0f / (1.0f + expf(-g)));
}

} // namespace saetta

using namespace saetta;

struct saetta_peer_group {
    int device = 0, rank = 0, world = 1;
    size_t rows_max = 0, heads = 0, slot_floats = 0;
    void *mailbox = nullptr; // [2][slot_floats] floats, then 2 flags, then the sequence number, then status
    float *staging = nullptr;
    void *peer_base[kMaxPeers] = {};
    bool connected = false;
    PeerPtrs ptrs = {};
    size_t flags_offset() const { return 2 * slot_floats * sizeof(float); }
};

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
    const size_t bytes = g->flags_offset() + 256;
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
        g->ptrs.parts[r] = reinterpret_cast<const float *>(g->peer_base[r]);
        g->ptrs.flags[r] = reinterpret_cast<const uint32_t *>(reinterpret_cast<const char *>(g->peer_base[r]) + g->flags_offset());
    }
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

int saetta_peer_merge(saetta_peer_group *g, size_t rows, const float *q_and_gate_dev, float *out_dev, void *stream) {
    if (!g || !q_and_gate_dev || !out_dev) return fail(SAETTA_ERR_BAD_ARG, "peer merge: null pointer");
    if (!g->connected) return fail(SAETTA_ERR_BAD_ARG, "peer merge: the group is not connected");
    if (!rows || rows > g->rows_max) return fail(SAETTA_ERR_BAD_SHAPE, "peer merge: more rows than the group was made for");
    DeviceGuard guard(g->device);
    auto st = (cudaStream_t)stream;
    char *base = reinterpret_cast<char *>(g->mailbox);
    uint32_t *flags = reinterpret_cast<uint32_t *>(base + g->flags_offset());
    uint32_t *seq = flags + 16, *status = flags + 32;
    const uint32_t n = uint32_t(rows * g->heads * kPartStride);
    SAETTA_CUDA(launch_pdl(publish_kernel, dim3(1), dim3(256), 0, st, (const float *)g->staging,
                           reinterpret_cast<float *>(base), flags, seq, n, uint32_t(g->slot_floats)));
    SAETTA_CUDA(launch_pdl(peer_merge_kernel, dim3(unsigned(g->heads), unsigned(rows)), dim3(256), 0, st, g->ptrs,
                           uint32_t(g->world), (const uint32_t *)seq, uint32_t(g->slot_floats), uint32_t(g->heads),
                           q_and_gate_dev, out_dev, status, 2000000u));
    return SAETTA_OK;
}

int saetta_peer_group_status(saetta_peer_group *g, void *stream, uint32_t *status) {
    if (!g || !status) return fail(SAETTA_ERR_BAD_ARG, "peer status: null pointer");
    DeviceGuard guard(g->device);
    const uint32_t *dev = reinterpret_cast<const uint32_t *>(reinterpret_cast<const char *>(g->mailbox) + g->flags_offset()) + 32;
    SAETTA_CUDA(cudaMemcpyAsync(status, dev, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SAETTA_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (*status) return fail(SAETTA_ERR_TIMEOUT, "a peer did not publish its partial in time");
    return SAETTA_OK;
}

} // extern "C"
