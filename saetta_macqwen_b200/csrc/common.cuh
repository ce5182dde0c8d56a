// Shared definitions of the B200 attention path: geometry, error plumbing and
// the small PTX wrappers (mbarrier, bulk copy, mma.sync) the kernels use.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/saetta_b200.h"

namespace saetta {

constexpr int kDim = 256;      // head dimension (src/attention.rs:17)
constexpr int kHeadsPerKv = 8; // query heads per kv head (src/attention.rs:16)
constexpr int kGroup = 64;     // quantisation group (src/kv_quant.rs:9)
constexpr int kGroupsPerHead = kDim / kGroup;
constexpr int kPartStride = SAETTA_PART_STRIDE; // floats per (row, head) partial: O[256], m, l, pad
constexpr int kPartM = 256;
constexpr int kPartL = 257;

// Device status word bits set by bounded waits that gave up.
constexpr uint32_t kStatusFullTimeout = 1u;
constexpr uint32_t kStatusEmptyTimeout = 2u;
constexpr uint32_t kStatusMmaTimeout = 4u;

void set_error(const std::string &msg);
int fail(int code, const std::string &msg);
int cuda_fail(cudaError_t e, const char *what);

#define SAETTA_CUDA(expr)                                              \
    do {                                                               \
        cudaError_t e_ = (expr);                                       \
        if (e_ != cudaSuccess) return ::saetta::cuda_fail(e_, #expr);  \
    } while (0)

// Sets the device for the lifetime of the scope and puts the old one back.
struct DeviceGuard {
    int old = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&old) != cudaSuccess) { ok = false; return; }
        if (old != device && cudaSetDevice(device) != cudaSuccess) ok = false;
        want = device;
    }
    ~DeviceGuard() {
        if (old >= 0 && old != want) cudaSetDevice(old);
    }
    int want = -1;
};

int sm_count(int device);

// Launch with programmatic dependent launch allowed: the grid may be scheduled while the kernel
// before it in the stream is still draining; the kernel itself calls pdl_wait() before it touches
// anything its predecessor may have written.  With a predecessor that never signals, this is an
// ordinary stream-ordered launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#ifdef __CUDACC__
// ----------------------------------------------------------------- PTX helpers

// Programmatic dependent launch: wait until the grids this one depends on have completed and
// their writes are visible; allow the grids that depend on this one to be scheduled.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up about `limit` x 256 ns after its 64th poll (4,000,000: one second), or as
// soon as *abort is set; returns false then.  The polls run back to back -- try_wait itself
// suspends the thread for a short hardware-defined time -- because a sleep between polls would
// delay the wake-up by more than the hand-offs between the roles of these kernels can afford.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          volatile uint32_t *abort_flag,
                                          uint32_t limit = 4000000u) {
    unsigned long long t0 = 0;
    for (uint32_t n = 0;; n++) {
        if (mbar_test(bar, parity)) return true;
        if ((n & 63) == 63) {
            if (*abort_flag) return false;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (!t0) t0 = t;
            else if (t - t0 > (static_cast<unsigned long long>(limit) << 8)) return false;
        }
    }
}

// Bulk (TMA engine) copy of `bytes` contiguous bytes, global -> shared, signalling
// `bar` with the byte count.  Both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Asks the TMA engine to bring `bytes` contiguous bytes into L2; nothing waits for it.
// Address 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void l2_prefetch(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// D += A(16x16, row) * B(16x8, col), f16 operands, f32 accumulate.
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Transposes an 8x8 matrix of 16-bit values held one 32-bit register per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ float2 h2f2(uint32_t a) { return __half22float2(*reinterpret_cast<__half2 *>(&a)); }
__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}
#endif

} // namespace saetta
