// The C ABI (include/saetta_b200.h): argument checks, object lifetimes, and the
// choice of kernel.  Every misuse the reference answers with assert!/panic!
// (src/attention.rs:49-57, src/rows.rs:390,459, src/kv_quant.rs:57,168) comes
// back as a status code here, before anything is launched.
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <cmath>
#include <functional>
#include <new>

#include <mutex>
#include <vector>

#include "merge_role.cuh"

namespace saetta {

static thread_local std::string g_error;

void set_error(const std::string &msg) { g_error = msg; }
int fail(int code, const std::string &msg) {
    g_error = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char *what) {
    g_error = std::string(what) + ": " + cudaGetErrorString(e);
    return e == cudaErrorMemoryAllocation ? SAETTA_ERR_NO_MEM : SAETTA_ERR_CUDA;
}

int sm_count(int device) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return 148;
    return n;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int alloc_zero(void **p, size_t bytes) {
    SAETTA_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    SAETTA_CUDA(cudaMemset(*p, 0, bytes ? bytes : 16));
    return SAETTA_OK;
}

static bool capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return cs != cudaStreamCaptureStatusNone;
}

static KvView view_of(const saetta_quant_rows *k, const saetta_quant_rows *v) {
    KvView kv;
    kv.bits = k->bits;
    kv.k = k->data, kv.v = v->data;
    kv.ks = k->scales, kv.kz = k->biases, kv.vs = v->scales, kv.vz = v->biases;
    kv.kv_heads = uint32_t(k->per_token / kGroupsPerHead);
    return kv;
}

// One-time per-device raise of the kernels' dynamic shared-memory limits.
static std::mutex g_init_mutex; // first calls from several host threads may meet in the lazy set-up below

static int configure_device(int device) {
    static bool done[64] = {};
    std::lock_guard<std::mutex> lock(g_init_mutex);
    if (device >= 0 && device < 64 && done[device]) return SAETTA_OK;
    int rc = decode_quant_configure(device);
    if (!rc) rc = decode_half_configure(device);
    if (!rc) rc = decode_exact_configure(device);
    if (!rc) rc = prefill_configure(device);
    if (!rc && device >= 0 && device < 64) done[device] = true;
    return rc;
}

} // namespace saetta

using namespace saetta;

extern "C" {

const char *saetta_last_error(void) { return g_error.c_str(); }
const char *saetta_version(void) { return "saetta_b200 0.1 (sm_100a)"; }

// ------------------------------------------------------------------ QuantRows

static int quant_rows_check(int bits, size_t values) {
    if (bits != 8 && bits != 4) return fail(SAETTA_ERR_BAD_SHAPE, "QuantRows: bits must be 8 or 4 (a half cache has no codes)");
    if (!values || values % kGroup) return fail(SAETTA_ERR_BAD_SHAPE, "QuantRows: values must be a multiple of 64");
    return SAETTA_OK;
}

int saetta_quant_rows_create(int device, int bits, size_t values, size_t capacity, saetta_quant_rows **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::new: out is null");
    if (int rc = quant_rows_check(bits, values)) return rc;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "QuantRows::new: cannot select the device");
    auto *r = new (std::nothrow) saetta_quant_rows();
    if (!r) return fail(SAETTA_ERR_NO_MEM, "QuantRows::new: host allocation");
    r->device = device, r->bits = bits, r->per_token = values / kGroup, r->capacity = capacity, r->owns = true;
    const size_t groups = r->per_token * capacity;
    int rc = alloc_zero(&r->data, groups * 2 * size_t(bits) * 4);
    if (!rc) rc = alloc_zero(&r->scales, groups * 2);
    if (!rc) rc = alloc_zero(&r->biases, groups * 2);
    if (rc) {
        saetta_quant_rows_destroy(r);
        return rc;
    }
    *out = r;
    return SAETTA_OK;
}

int saetta_quant_rows_wrap(int device, int bits, size_t values, size_t capacity, void *data_dev, void *scales_dev,
                           void *biases_dev, saetta_quant_rows **out) {
    if (!out || !data_dev || !scales_dev || !biases_dev) return fail(SAETTA_ERR_BAD_ARG, "QuantRows wrap: null pointer");
    if (int rc = quant_rows_check(bits, values)) return rc;
    if (!aligned16(data_dev) || !aligned16(scales_dev) || !aligned16(biases_dev))
        return fail(SAETTA_ERR_BAD_ARG, "QuantRows wrap: buffers must be 16-byte aligned");
    auto *r = new (std::nothrow) saetta_quant_rows();
    if (!r) return fail(SAETTA_ERR_NO_MEM, "QuantRows wrap: host allocation");
    r->device = device, r->bits = bits, r->per_token = values / kGroup, r->capacity = capacity;
    r->data = data_dev, r->scales = scales_dev, r->biases = biases_dev, r->owns = false;
    *out = r;
    return SAETTA_OK;
}

void saetta_quant_rows_destroy(saetta_quant_rows *r) {
    if (!r) return;
    if (r->owns) {
        DeviceGuard guard(r->device);
        cudaFree(r->data);
        cudaFree(r->scales);
        cudaFree(r->biases);
    }
    delete r;
}

int saetta_quant_rows_buffers(const saetta_quant_rows *r, void **data_dev, void **scales_dev, void **biases_dev) {
    if (!r) return fail(SAETTA_ERR_BAD_ARG, "QuantRows: null handle");
    if (data_dev) *data_dev = r->data;
    if (scales_dev) *scales_dev = r->scales;
    if (biases_dev) *biases_dev = r->biases;
    return SAETTA_OK;
}

int saetta_quant_rows_record_at(saetta_quant_rows *r, const float *x_dev, const saetta_token_params *params_dev,
                                void *stream) {
    if (!r || !x_dev || !params_dev) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::record: null pointer");
    if (!aligned16(x_dev)) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::record: x must be 16-byte aligned");
    DeviceGuard guard(r->device);
    return launch_kv_quantize(r->bits, uint32_t(r->per_token), x_dev, r, nullptr, nullptr, 1, 0, params_dev,
                              (cudaStream_t)stream);
}

int saetta_quant_rows_encode(saetta_quant_rows *r, const float *x_dev, size_t pos, size_t tokens, void *stream) {
    if (!r || (!x_dev && tokens)) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::encode: null pointer");
    if (pos + tokens > r->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "QuantRows::encode: pos + tokens exceeds the capacity");
    if (!aligned16(x_dev)) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::encode: x must be 16-byte aligned");
    DeviceGuard guard(r->device);
    return launch_kv_quantize(r->bits, uint32_t(r->per_token), x_dev, r, nullptr, nullptr, tokens, pos, nullptr,
                              (cudaStream_t)stream);
}

int saetta_quant_rows_encode_dequantize(const saetta_quant_rows *r, void *out_dev, int dtype, size_t tokens,
                                        void *stream) {
    if (!r || (!out_dev && tokens)) return fail(SAETTA_ERR_BAD_ARG, "QuantRows::encode_dequantize: null pointer");
    if (dtype != SAETTA_F16 && dtype != SAETTA_BF16) return fail(SAETTA_ERR_BAD_ARG, "encode_dequantize: dtype");
    if (tokens > r->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "encode_dequantize: tokens exceeds the capacity");
    if (!aligned16(out_dev)) return fail(SAETTA_ERR_BAD_ARG, "encode_dequantize: out must be 16-byte aligned");
    DeviceGuard guard(r->device);
    return launch_kv_dequantize(r, out_dev, dtype, 0, tokens, (cudaStream_t)stream);
}

// Host restatement of the kernels' arithmetic (src/kv_quant.rs:54-105); the
// narrowing to binary16 is the hardware-equivalent round-to-nearest-even.
static uint16_t host_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, exp = (x >> 23) & 0xffu;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) return uint16_t(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
    const int e = int(exp) - 112;
    if (e >= 31) return uint16_t(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        man |= 0x800000u;
        const uint32_t shift = uint32_t(14 - e);
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (h & 1))) h++;
        return uint16_t(sign | h);
    }
    uint32_t h = (uint32_t(e) << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
    return uint16_t(sign | h);
}
static float host_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t(h) & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (!man) {
            bits = sign;
        } else {
            float v = float(man) * 5.9604644775390625e-08f;
            memcpy(&bits, &v, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

int saetta_quantize_host(const float *x, size_t n, int bits, uint32_t *data, uint16_t *scales, uint16_t *biases) {
    if (!x || !data || !scales || !biases) return fail(SAETTA_ERR_BAD_ARG, "quantize: null pointer");
    if ((bits != 8 && bits != 4) || n % kGroup) return fail(SAETTA_ERR_BAD_SHAPE, "quantize: bits 8 or 4, length a multiple of 64");
    const float levels = float((1u << bits) - 1);
    const size_t per_word = 32 / size_t(bits);
    size_t w = 0;
    for (size_t g = 0; g < n / kGroup; g++) {
        const float *grp = x + g * kGroup;
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < kGroup; i++) lo = fminf(lo, grp[i]), hi = fmaxf(hi, grp[i]);
        const volatile float range = hi - lo;
        const volatile float sd = range / levels;
        const uint16_t s = host_f16(sd), z = host_f16(lo);
        const float sf = host_f16_to_f32(s), zf = host_f16_to_f32(z);
        const volatile float inv = sf > 0.0f ? 1.0f / sf : 0.0f;
        for (size_t k = 0; k < size_t(kGroup); k += per_word) {
            uint32_t word = 0;
            for (size_t i = 0; i < per_word; i++) {
                const volatile float d = grp[k + i] - zf;
                const volatile float t = d * inv;
                float r = rintf(t);
                if (r != r) r = 0.0f;
                r = r < 0.0f ? 0.0f : (r > levels ? levels : r);
                word |= uint32_t(r) << (i * size_t(bits));
            }
            data[w++] = word;
        }
        scales[g] = s, biases[g] = z;
    }
    return SAETTA_OK;
}

int saetta_dequantize_host(const uint32_t *data, const uint16_t *scales, const uint16_t *biases, size_t groups,
                           int bits, float *out) {
    if (!data || !scales || !biases || !out) return fail(SAETTA_ERR_BAD_ARG, "dequantize: null pointer");
    if (bits != 8 && bits != 4) return fail(SAETTA_ERR_BAD_SHAPE, "dequantize: bits 8 or 4");
    const uint32_t mask = (1u << bits) - 1;
    const size_t per_word = 32 / size_t(bits), words = 2 * size_t(bits);
    size_t o = 0;
    for (size_t g = 0; g < groups; g++) {
        const float s = host_f16_to_f32(scales[g]), z = host_f16_to_f32(biases[g]);
        for (size_t k = 0; k < words; k++)
            for (size_t i = 0; i < per_word; i++) {
                const volatile float p = s * float((data[g * words + k] >> (i * size_t(bits))) & mask);
                out[o++] = p + z;
            }
    }
    return SAETTA_OK;
}

// ------------------------------------------------------------------ GpuKvCache

static int kv_cache_alloc(saetta_kv_cache *c, size_t capacity) {
    c->capacity = capacity;
    if (c->bits == 8 || c->bits == 4) {
        saetta_quant_rows *sides[2] = {&c->k, &c->v};
        for (auto *r : sides) {
            *r = saetta_quant_rows();
            r->device = c->device, r->bits = c->bits, r->per_token = c->row_values() / kGroup, r->capacity = capacity;
            const size_t groups = r->per_token * capacity;
            if (int rc = alloc_zero(&r->data, groups * 2 * size_t(c->bits) * 4)) return rc;
            if (int rc = alloc_zero(&r->scales, groups * 2)) return rc;
            if (int rc = alloc_zero(&r->biases, groups * 2)) return rc;
        }
        c->keys = c->k.data, c->values = c->v.data;
        return SAETTA_OK;
    }
    if (int rc = alloc_zero(&c->keys, capacity * c->plain_row_bytes())) return rc;
    return alloc_zero(&c->values, capacity * c->plain_row_bytes());
}

static void kv_cache_free(saetta_kv_cache *c) {
    if (c->bits == 8 || c->bits == 4) {
        for (auto *r : {&c->k, &c->v}) {
            cudaFree(r->data), cudaFree(r->scales), cudaFree(r->biases);
            r->data = r->scales = r->biases = nullptr;
        }
    } else {
        cudaFree(c->keys), cudaFree(c->values);
    }
    c->keys = c->values = nullptr;
}

static size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int saetta_kv_cache_create(int device, int bits, size_t heads, size_t kv_heads, size_t head_dim, size_t capacity,
                           saetta_kv_cache **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache::new: out is null");
    if (bits != 32 && bits != 16 && bits != 8 && bits != 4) return fail(SAETTA_ERR_BAD_SHAPE, "GpuKvCache: bits must be 32, 16, 8 or 4");
    if (head_dim != size_t(kDim)) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention is written for head dim 256");
    if (!kv_heads || heads != kv_heads * kHeadsPerKv) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention needs 8 q heads per kv head");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "GpuKvCache::new: cannot select the device");
    auto *c = new (std::nothrow) saetta_kv_cache();
    if (!c) return fail(SAETTA_ERR_NO_MEM, "GpuKvCache::new: host allocation");
    c->device = device, c->bits = bits, c->heads = heads, c->kv_heads = kv_heads, c->head_dim = head_dim;
    if (int rc = kv_cache_alloc(c, round_up(capacity ? capacity : 1, SAETTA_KV_ALIGN))) {
        kv_cache_free(c);
        delete c;
        return rc;
    }
    *out = c;
    return SAETTA_OK;
}

void saetta_kv_cache_destroy(saetta_kv_cache *c) {
    if (!c) return;
    DeviceGuard guard(c->device);
    kv_cache_free(c);
    delete c;
}

size_t saetta_kv_cache_capacity(const saetta_kv_cache *c) { return c ? c->capacity : 0; }
int saetta_kv_cache_bits(const saetta_kv_cache *c) { return c ? c->bits : 0; }

int saetta_kv_cache_set_dtype(saetta_kv_cache *c, int dtype) {
    if (!c) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache: null handle");
    if (dtype != SAETTA_F16 && dtype != SAETTA_BF16) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache: dtype");
    c->dtype = dtype;
    return SAETTA_OK;
}

int saetta_kv_cache_buffers(const saetta_kv_cache *c, void *buffers_dev[6], size_t row_bytes[6], int *count) {
    if (!c || !buffers_dev || !row_bytes || !count) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache::buffers: null pointer");
    if (c->bits == 8 || c->bits == 4) {
        void *b[6] = {c->keys, c->values, c->k.scales, c->k.biases, c->v.scales, c->v.biases};
        const size_t d = c->k.data_row_bytes(), p = c->k.param_row_bytes();
        const size_t rb[6] = {d, d, p, p, p, p};
        for (int i = 0; i < 6; i++) buffers_dev[i] = b[i], row_bytes[i] = rb[i];
        *count = 6;
    } else {
        buffers_dev[0] = c->keys, buffers_dev[1] = c->values;
        row_bytes[0] = row_bytes[1] = c->plain_row_bytes();
        *count = 2;
    }
    return SAETTA_OK;
}

int saetta_kv_cache_quant(const saetta_kv_cache *c, saetta_quant_rows **keys, saetta_quant_rows **values) {
    if (!c) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache: null handle");
    const bool q = c->bits == 8 || c->bits == 4;
    if (keys) *keys = q ? const_cast<saetta_quant_rows *>(&c->k) : nullptr;
    if (values) *values = q ? const_cast<saetta_quant_rows *>(&c->v) : nullptr;
    return SAETTA_OK;
}

int saetta_kv_cache_resize(saetta_kv_cache *c, size_t capacity, void *stream) {
    if (!c) return fail(SAETTA_ERR_BAD_ARG, "GpuKvCache::resize: null handle");
    DeviceGuard guard(c->device);
    capacity = round_up(capacity ? capacity : 1, SAETTA_KV_ALIGN);
    saetta_kv_cache old = *c; // keeps the old pointers
    void *ob[6];
    size_t rb[6];
    int n = 0;
    saetta_kv_cache_buffers(&old, ob, rb, &n);
    if (int rc = kv_cache_alloc(c, capacity)) {
        kv_cache_free(c);
        *c = old;
        return rc;
    }
    void *nb[6];
    size_t rb2[6];
    saetta_kv_cache_buffers(c, nb, rb2, &n);
    const size_t rows = old.capacity < capacity ? old.capacity : capacity;
    auto st = (cudaStream_t)stream;
    for (int i = 0; i < n; i++) SAETTA_CUDA(cudaMemcpyAsync(nb[i], ob[i], rows * rb[i], cudaMemcpyDeviceToDevice, st));
    SAETTA_CUDA(cudaStreamSynchronize(st));
    kv_cache_free(&old);
    return SAETTA_OK;
}

static int kv_store(saetta_kv_cache *c, const float *k, const float *v, size_t pos, const saetta_token_params *params,
                    size_t rows, cudaStream_t st) {
    if (!aligned16(k) || !aligned16(v)) return fail(SAETTA_ERR_BAD_ARG, "kv store: k and v must be 16-byte aligned");
    DeviceGuard guard(c->device);
    if (c->bits == 8 || c->bits == 4)
        return launch_kv_quantize(c->bits, uint32_t(c->k.per_token), k, &c->k, v, &c->v, rows, pos, params, st);
    const int mode = c->bits == 32 ? 2 : (c->dtype == SAETTA_BF16 ? 1 : 0);
    return launch_kv_store_plain(mode, k, v, c->keys, c->values, c->row_values(), rows, pos, params, st);
}

int saetta_kv_cache_store(saetta_kv_cache *c, const float *k_dev, const float *v_dev, const saetta_token_params *params_dev,
                          size_t rows, void *stream) {
    if (!c || !k_dev || !v_dev || !params_dev) return fail(SAETTA_ERR_BAD_ARG, "kv store: null pointer");
    if (rows > SAETTA_MAX_ROWS) return fail(SAETTA_ERR_BAD_SHAPE, "kv store: more rows than MAX_ROWS");
    return kv_store(c, k_dev, v_dev, 0, params_dev, rows, (cudaStream_t)stream);
}

int saetta_kv_cache_store_at(saetta_kv_cache *c, const float *k_dev, const float *v_dev, size_t pos, size_t tokens,
                             void *stream) {
    if (!c || ((!k_dev || !v_dev) && tokens)) return fail(SAETTA_ERR_BAD_ARG, "kv store: null pointer");
    if (pos + tokens > c->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "kv store: pos + tokens exceeds the capacity");
    return kv_store(c, k_dev, v_dev, pos, nullptr, tokens, (cudaStream_t)stream);
}

// ------------------------------------------------------------------ RowBackup

int saetta_row_backup_create(saetta_row_backup **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "RowBackup::new: out is null");
    *out = new (std::nothrow) saetta_row_backup();
    return *out ? SAETTA_OK : fail(SAETTA_ERR_NO_MEM, "RowBackup::new: host allocation");
}

void saetta_row_backup_clear(saetta_row_backup *b) {
    if (!b) return;
    if (b->held) {
        DeviceGuard guard(b->device);
        for (auto &p : b->parts) cudaFree(p.copy);
    }
    b->parts.clear();
    b->held = false;
}

void saetta_row_backup_destroy(saetta_row_backup *b) {
    saetta_row_backup_clear(b);
    delete b;
}

uint64_t saetta_row_backup_bytes(const saetta_row_backup *b) {
    uint64_t total = 0;
    if (b && b->held)
        for (auto &p : b->parts) total += uint64_t(p.row_bytes) * b->n;
    return total;
}

int saetta_row_backup_save(saetta_row_backup *b, saetta_kv_cache *const *caches, size_t n_caches, size_t from, size_t n,
                           void *stream) {
    if (!b || (!caches && n_caches)) return fail(SAETTA_ERR_BAD_ARG, "RowBackup::save: null pointer");
    saetta_row_backup_clear(b);
    if (!n || !n_caches) return SAETTA_OK;
    for (size_t i = 0; i < n_caches; i++)
        if (!caches[i] || from + n > caches[i]->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "RowBackup::save: rows outside the cache");
    b->device = caches[0]->device;
    DeviceGuard guard(b->device);
    b->from = from, b->n = n, b->held = true;
    for (size_t i = 0; i < n_caches; i++) {
        void *bufs[6];
        size_t rb[6];
        int cnt = 0;
        saetta_kv_cache_buffers(caches[i], bufs, rb, &cnt);
        for (int j = 0; j < cnt; j++) {
            void *copy = nullptr;
            cudaError_t e = cudaMalloc(&copy, n * rb[j]);
            if (e != cudaSuccess) {
                saetta_row_backup_clear(b);
                return cuda_fail(e, "RowBackup::save: cudaMalloc");
            }
            b->parts.push_back({copy, rb[j]});
            SAETTA_CUDA(cudaMemcpyAsync(copy, (const char *)bufs[j] + from * rb[j], n * rb[j], cudaMemcpyDeviceToDevice,
                                        (cudaStream_t)stream));
        }
    }
    return SAETTA_OK;
}

int saetta_row_backup_restore(saetta_row_backup *b, saetta_kv_cache *const *caches, size_t n_caches, void *stream) {
    if (!b) return fail(SAETTA_ERR_BAD_ARG, "RowBackup::restore: null handle");
    if (!b->held) return SAETTA_OK;
    DeviceGuard guard(b->device);
    size_t k = 0;
    for (size_t i = 0; i < n_caches; i++) {
        void *bufs[6];
        size_t rb[6];
        int cnt = 0;
        saetta_kv_cache_buffers(caches[i], bufs, rb, &cnt);
        for (int j = 0; j < cnt; j++, k++) {
            if (k >= b->parts.size() || b->parts[k].row_bytes != rb[j] || b->from + b->n > caches[i]->capacity)
                return fail(SAETTA_ERR_BAD_SHAPE, "RowBackup::restore: caches differ from the ones saved");
            SAETTA_CUDA(cudaMemcpyAsync((char *)bufs[j] + b->from * rb[j], b->parts[k].copy, b->n * rb[j],
                                        cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        }
    }
    // The copies are freed once the stream has used them.
    SAETTA_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    saetta_row_backup_clear(b);
    return SAETTA_OK;
}

// ------------------------------------------------------------------ DecodeAttention / AttentionRows

int saetta_decode_create(int device, size_t heads, size_t kv_heads, size_t head_dim, size_t capacity, size_t rows,
                         saetta_decode **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "DecodeAttention::new: out is null");
    if (head_dim != size_t(kDim)) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention is written for head dim 256");
    if (!kv_heads || heads != kv_heads * kHeadsPerKv) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention needs 8 q heads per kv head");
    if (!rows || rows > SAETTA_MAX_ROWS) return fail(SAETTA_ERR_BAD_SHAPE, "AttentionRows: rows must be 1..8");
    if (!capacity) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: capacity is 0");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "DecodeAttention::new: cannot select the device");
    if (int rc = configure_device(device)) return rc;
    auto *op = new (std::nothrow) saetta_decode();
    if (!op) return fail(SAETTA_ERR_NO_MEM, "DecodeAttention::new: host allocation");
    op->device = device, op->heads = heads, op->kv_heads = kv_heads, op->capacity = capacity, op->rows = rows;
    const size_t tiles = (capacity + 31) / 32;
    const size_t sms = size_t(sm_count(device));
    op->splits = int(std::min(std::min(tiles, sms), size_t(kMergeRoleMaxParts)));
    const size_t per_row = std::max(decode_quant_part_floats(kv_heads), heads * size_t(kPartStride));
    int rc = alloc_zero((void **)&op->parts, size_t(op->splits) * rows * per_row * sizeof(float));
    if (!rc) rc = alloc_zero((void **)&op->status, kStatusWords * 4);
    if (rc) {
        saetta_decode_destroy(op);
        return rc;
    }
    *out = op;
    return SAETTA_OK;
}

void saetta_decode_destroy(saetta_decode *op) {
    if (!op) return;
    DeviceGuard guard(op->device);
    cudaFree(op->parts);
    cudaFree(op->status);
    delete op;
}

int saetta_decode_splits(const saetta_decode *op) { return op ? op->splits : 0; }

int saetta_decode_device_status(saetta_decode *op, void *stream, uint32_t *status) {
    if (!op || !status) return fail(SAETTA_ERR_BAD_ARG, "device_status: null pointer");
    DeviceGuard guard(op->device);
    SAETTA_CUDA(cudaMemcpyAsync(status, op->status, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SAETTA_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (*status) return fail(SAETTA_ERR_TIMEOUT, "a bounded device-side wait gave up");
    return SAETTA_OK;
}

static int decode_check(const saetta_decode *op, size_t m, const void *q, const void *out, const void *params) {
    if (!op || !q || !out || !params) return fail(SAETTA_ERR_BAD_ARG, "decode attention: null pointer");
    if (!m || m > op->rows) return fail(SAETTA_ERR_BAD_SHAPE, "AttentionRows::record: m exceeds the rows the op was made for");
    if (!aligned16(q)) return fail(SAETTA_ERR_BAD_ARG, "decode attention: q must be 16-byte aligned");
    return SAETTA_OK;
}

static int decode_run(saetta_decode *op, size_t m, const float *q, const KvView &kv, size_t kv_capacity,
                      const float *q_and_gate, float *out, float *part_out, uint32_t row_step,
                      const saetta_token_params *params, cudaStream_t st, saetta_peer_group *group = nullptr) {
    if (kv.kv_heads != op->kv_heads) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: cache and op disagree on kv heads");
    if (kv_capacity > op->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: cache larger than the op's capacity");
    if (kv_capacity % 32) return fail(SAETTA_ERR_BAD_SHAPE, "decode attention: cache capacity must be a multiple of 32");
    DeviceGuard guard(op->device);
    const uint32_t heads = uint32_t(op->heads);
    const bool tensor_quant = kv.bits == 8 || kv.bits == 4;
    const bool tensor_half = kv.bits == 16 && kv.kv_heads == 2 && aligned16(kv.k) && aligned16(kv.v);
    if (tensor_quant || tensor_half) {
        // One launch: the split-KV CTAs, then the merge CTAs that gate the result, leave the merged
        // partial, or store it into the peers' mailboxes (merge_role.cuh).
        if (kv.kv_heads != 2) return fail(SAETTA_ERR_UNSUPPORTED, "quantised decode attention is built for 2 kv heads");
        MergeOut mo;
        mo.q_and_gate = q_and_gate, mo.out = out, mo.part_out = part_out;
        if (group) mo.push = group->push; // with `out` too: the launch publishes AND collects
        // binary16 (the reference's own cache format) or bfloat16 rows run the same shape of kernel
        // without the dequantisation
        return tensor_quant ? launch_decode_quant(kv, q, op->parts, op->status, uint32_t(m), row_step, op->splits,
                                                  uint32_t(kv_capacity), params, mo, st)
                            : launch_decode_half(kv, q, op->parts, op->status, uint32_t(m), row_step, op->splits,
                                                 uint32_t(kv_capacity), params, mo, st);
    }
    if (int rc = launch_decode_exact(kv, q, op->parts, uint32_t(m), row_step, op->splits, uint32_t(kv_capacity), params, st))
        return rc;
    if (!group) return launch_merge_logical(op->parts, uint32_t(op->splits), uint32_t(m), heads, q_and_gate, out, part_out, st);
    // across GPUs: the merged partial into the group's staging buffer, published from there; collected
    // by a launch of its own when the caller asked for the result
    if (int rc = launch_merge_logical(op->parts, uint32_t(op->splits), uint32_t(m), heads, nullptr, nullptr, group->staging, st))
        return rc;
    if (int rc = launch_peer_publish(group, m, st)) return rc;
    return out ? saetta_peer_collect(group, m, q_and_gate, out, st) : SAETTA_OK;
}

int saetta_decode_record(saetta_decode *op, size_t m, const float *q_dev, const void *keys_dev, const void *values_dev,
                         int dtype, const float *q_and_gate_dev, float *out_dev, const saetta_token_params *params_dev,
                         void *stream) {
    if (int rc = decode_check(op, m, q_dev, out_dev, params_dev)) return rc;
    if (!keys_dev || !values_dev || !q_and_gate_dev) return fail(SAETTA_ERR_BAD_ARG, "DecodeAttention::record: null pointer");
    if (dtype != -1 && dtype != SAETTA_F16 && dtype != SAETTA_BF16) return fail(SAETTA_ERR_BAD_ARG, "DecodeAttention::record: dtype");
    KvView kv;
    kv.bits = dtype == -1 ? 32 : 16, kv.dtype = dtype == -1 ? SAETTA_F16 : dtype;
    kv.k = keys_dev, kv.v = values_dev, kv.kv_heads = uint32_t(op->kv_heads);
    return decode_run(op, m, q_dev, kv, op->capacity / 32 * 32, q_and_gate_dev, out_dev, nullptr, 1, params_dev, (cudaStream_t)stream);
}

int saetta_decode_record_quant(saetta_decode *op, size_t m, const float *q_dev, const saetta_quant_rows *keys,
                               const saetta_quant_rows *values, const float *q_and_gate_dev, float *out_dev,
                               const saetta_token_params *params_dev, void *stream) {
    if (int rc = decode_check(op, m, q_dev, out_dev, params_dev)) return rc;
    if (!keys || !values || !q_and_gate_dev) return fail(SAETTA_ERR_BAD_ARG, "DecodeAttention::record_quant: null pointer");
    if (keys->bits != values->bits || keys->per_token != values->per_token || keys->capacity != values->capacity)
        return fail(SAETTA_ERR_BAD_SHAPE, "record_quant: keys and values differ in format");
    return decode_run(op, m, q_dev, view_of(keys, values), keys->capacity, q_and_gate_dev, out_dev, nullptr, 1, params_dev,
                      (cudaStream_t)stream);
}

int saetta_decode_record_quant_static(int device, size_t m, const float *q_dev, const saetta_quant_rows *keys,
                                      const saetta_quant_rows *values, const float *q_and_gate_dev, float *out_dev,
                                      const saetta_token_params *params_dev, void *stream) {
    if (!q_dev || !keys || !values || !q_and_gate_dev || !out_dev || !params_dev)
        return fail(SAETTA_ERR_BAD_ARG, "static decode: null pointer");
    if (!aligned16(q_dev)) return fail(SAETTA_ERR_BAD_ARG, "static decode: q must be 16-byte aligned");
    if (keys->bits != values->bits || keys->per_token != values->per_token || keys->capacity != values->capacity)
        return fail(SAETTA_ERR_BAD_SHAPE, "static decode: keys and values differ in format");
    if (keys->bits != 8 && keys->bits != 4) return fail(SAETTA_ERR_BAD_SHAPE, "static decode: the rows must hold 8- or 4-bit codes");
    if (keys->device != device || values->device != device)
        return fail(SAETTA_ERR_BAD_ARG, "static decode: the rows live on another device than the one named");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "static decode: cannot select the device");
    return decode_quant_static(device, view_of(keys, values), keys->capacity, q_dev, uint32_t(m), q_and_gate_dev,
                               out_dev, params_dev, (cudaStream_t)stream);
}

int saetta_decode_static_status(int device, void *stream, uint32_t *status, int clear) {
    if (!status) return fail(SAETTA_ERR_BAD_ARG, "static decode status: null pointer");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "static decode status: cannot select the device");
    if (int rc = decode_quant_static_status(device, (cudaStream_t)stream, status, clear != 0)) return rc;
    if (*status) return fail(SAETTA_ERR_TIMEOUT, "a bounded device-side wait gave up");
    return SAETTA_OK;
}

static KvView view_of_cache(const saetta_kv_cache *c) {
    if (c->bits == 8 || c->bits == 4) return view_of(&c->k, &c->v);
    KvView kv;
    kv.bits = c->bits, kv.dtype = c->dtype, kv.k = c->keys, kv.v = c->values, kv.kv_heads = uint32_t(c->kv_heads);
    return kv;
}

int saetta_decode_record_cache(saetta_decode *op, size_t m, const float *q_dev, const saetta_kv_cache *cache,
                               const float *q_and_gate_dev, float *out_dev, const saetta_token_params *params_dev,
                               void *stream) {
    if (int rc = decode_check(op, m, q_dev, out_dev, params_dev)) return rc;
    if (!cache || !q_and_gate_dev) return fail(SAETTA_ERR_BAD_ARG, "decode attention: null pointer");
    return decode_run(op, m, q_dev, view_of_cache(cache), cache->capacity, q_and_gate_dev, out_dev, nullptr, 1, params_dev,
                      (cudaStream_t)stream);
}

// The prefill's row route (src/prefill.rs:1674-1686 selects attention_rows / attention_rows_q8|q4 for its exact
// mode: the m-row kernels of AttentionRows over the chunk's rows instead of the GEMM path).  The chunk goes through
// the same op in groups of up to `op->rows` rows: row r of the chunk sees keys 0 ..= pos + r.  An f32 cache gets f32
// arithmetic throughout (decode_exact_kernel); 16-bit and quantised caches their tensor-core row kernels.
// `params_scratch_dev` holds one saetta_token_params per group and is written here (from pageable host memory: the
// call is not capturable).
int saetta_prefill_rows_cache(saetta_decode *op, const float *q_dev, const saetta_kv_cache *cache,
                              const float *q_and_gate_dev, float *out_dev, saetta_flash_params p,
                              saetta_token_params *params_scratch_dev, void *stream) {
    if (!op || !q_dev || !cache || !q_and_gate_dev || !out_dev || !params_scratch_dev)
        return fail(SAETTA_ERR_BAD_ARG, "prefill rows: null pointer");
    if (p.heads != op->heads || p.kv_heads != op->kv_heads) return fail(SAETTA_ERR_BAD_SHAPE, "prefill rows: heads differ from the op's");
    if (size_t(p.pos) + p.tokens > cache->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "prefill rows: the chunk ends beyond the cache");
    if (!p.tokens) return SAETTA_OK;
    if (capturing((cudaStream_t)stream)) return fail(SAETTA_ERR_BAD_ARG, "prefill rows: not capturable (it uploads its row groups' parameters)");
    const size_t per = op->rows, groups = (p.tokens + per - 1) / per;
    std::vector<saetta_token_params> host(groups);
    for (size_t g = 0; g < groups; g++) host[g] = saetta_token_params{0u, uint32_t(p.pos + g * per), uint32_t(p.pos + g * per + 1), 0u};
    DeviceGuard guard(op->device);
    SAETTA_CUDA(cudaMemcpyAsync(params_scratch_dev, host.data(), groups * sizeof(saetta_token_params), cudaMemcpyHostToDevice,
                                (cudaStream_t)stream));
    const size_t q_row = size_t(p.heads) * kDim;
    for (size_t g = 0; g < groups; g++) {
        const size_t r0 = g * per, m = std::min(per, size_t(p.tokens) - r0);
        if (int rc = saetta_decode_record_cache(op, m, q_dev + r0 * q_row, cache, q_and_gate_dev + r0 * 2 * q_row, out_dev + r0 * q_row,
                                                params_scratch_dev + g, stream))
            return rc;
    }
    return SAETTA_OK;
}

int saetta_decode_partial_cache(saetta_decode *op, size_t m, const float *q_dev, const saetta_kv_cache *cache,
                                float *part_dev, uint32_t row_step, const saetta_token_params *params_dev, void *stream) {
    if (int rc = decode_check(op, m, q_dev, part_dev, params_dev)) return rc;
    if (!cache) return fail(SAETTA_ERR_BAD_ARG, "decode attention: null pointer");
    if (row_step > 1) return fail(SAETTA_ERR_BAD_ARG, "decode partial: row_step is 0 or 1");
    return decode_run(op, m, q_dev, view_of_cache(cache), cache->capacity, nullptr, nullptr, part_dev, row_step, params_dev,
                      (cudaStream_t)stream);
}

int saetta_decode_publish_cache(saetta_decode *op, size_t m, const float *q_dev, const saetta_kv_cache *cache,
                                saetta_peer_group *group, uint32_t row_step, const saetta_token_params *params_dev,
                                void *stream) {
    if (!group) return fail(SAETTA_ERR_BAD_ARG, "decode publish: null pointer");
    if (int rc = decode_check(op, m, q_dev, group->staging, params_dev)) return rc;
    if (!cache) return fail(SAETTA_ERR_BAD_ARG, "decode attention: null pointer");
    if (row_step > 1) return fail(SAETTA_ERR_BAD_ARG, "decode partial: row_step is 0 or 1");
    if (!group->connected) return fail(SAETTA_ERR_BAD_ARG, "decode publish: the group is not connected");
    if (group->device != op->device) return fail(SAETTA_ERR_BAD_ARG, "decode publish: op and group live on different devices");
    if (m > group->rows_max || op->heads != group->heads) return fail(SAETTA_ERR_BAD_SHAPE, "decode publish: the group was made for another shape");
    return decode_run(op, m, q_dev, view_of_cache(cache), cache->capacity, nullptr, nullptr, group->staging, row_step,
                      params_dev, (cudaStream_t)stream, group);
}

int saetta_decode_exchange_cache(saetta_decode *op, size_t m, const float *q_dev, const saetta_kv_cache *cache,
                                 saetta_peer_group *group, uint32_t row_step, const float *q_and_gate_dev, float *out_dev,
                                 const saetta_token_params *params_dev, void *stream) {
    if (!group || !q_and_gate_dev) return fail(SAETTA_ERR_BAD_ARG, "decode exchange: null pointer");
    if (int rc = decode_check(op, m, q_dev, out_dev, params_dev)) return rc;
    if (!cache) return fail(SAETTA_ERR_BAD_ARG, "decode attention: null pointer");
    if (row_step > 1) return fail(SAETTA_ERR_BAD_ARG, "decode partial: row_step is 0 or 1");
    if (!group->connected) return fail(SAETTA_ERR_BAD_ARG, "decode exchange: the group is not connected");
    if (group->device != op->device) return fail(SAETTA_ERR_BAD_ARG, "decode exchange: op and group live on different devices");
    if (m > group->rows_max || op->heads != group->heads) return fail(SAETTA_ERR_BAD_SHAPE, "decode exchange: the group was made for another shape");
    return decode_run(op, m, q_dev, view_of_cache(cache), cache->capacity, q_and_gate_dev, out_dev, nullptr, row_step,
                      params_dev, (cudaStream_t)stream, group);
}

int saetta_merge_partials(int device, const float *parts_dev, size_t ranks, size_t rows, size_t heads,
                          const float *q_and_gate_dev, float *out_dev, void *stream) {
    if (!parts_dev || !q_and_gate_dev || !out_dev) return fail(SAETTA_ERR_BAD_ARG, "merge_partials: null pointer");
    if (!ranks || !rows || !heads) return fail(SAETTA_ERR_BAD_SHAPE, "merge_partials: empty shape");
    DeviceGuard guard(device);
    return launch_merge_logical(parts_dev, uint32_t(ranks), uint32_t(rows), uint32_t(heads), q_and_gate_dev, out_dev,
                                nullptr, (cudaStream_t)stream);
}

// ------------------------------------------------------------------ batched decode

struct BatchTable { // host mirror of what the kernels read
    std::vector<Segment> segs;
    std::vector<uint32_t> cta_first, seq_first;
};

int saetta_decode_batch_create(int device, size_t heads, size_t kv_heads, size_t head_dim, size_t max_seqs,
                               size_t max_total_tokens, saetta_decode_batch **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "decode batch: out is null");
    if (head_dim != size_t(kDim) || kv_heads != 2 || heads != 16)
        return fail(SAETTA_ERR_BAD_SHAPE, "batched decode attention is built for 16 q / 2 kv heads of 256");
    if (!max_seqs) return fail(SAETTA_ERR_BAD_SHAPE, "decode batch: max_seqs is 0");
    (void)max_total_tokens;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "decode batch: cannot select the device");
    if (int rc = configure_device(device)) return rc;
    auto *op = new (std::nothrow) saetta_decode_batch();
    if (!op) return fail(SAETTA_ERR_NO_MEM, "decode batch: host allocation");
    op->device = device, op->heads = heads, op->kv_heads = kv_heads, op->max_seqs = max_seqs;
    op->ctas = sm_count(device);
    op->max_parts = max_seqs + size_t(op->ctas); // a sequence adds one part per CTA boundary inside it
    op->table_bytes = op->max_parts * sizeof(Segment) + (size_t(op->ctas) + 1 + max_seqs + 1) * 4;
    int rc = alloc_zero((void **)&op->parts, op->max_parts * decode_quant_part_floats(kv_heads) * sizeof(float));
    if (!rc) rc = alloc_zero(&op->table_dev, op->table_bytes);
    if (!rc) rc = alloc_zero((void **)&op->status, 16);
    if (!rc) {
        cudaError_t e = cudaMallocHost(&op->table_host, op->table_bytes);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaMallocHost");
    }
    if (!rc) {
        cudaEvent_t ev;
        cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaEventCreate");
        else op->table_event = ev;
    }
    if (rc) {
        saetta_decode_batch_destroy(op);
        return rc;
    }
    *out = op;
    return SAETTA_OK;
}

void saetta_decode_batch_destroy(saetta_decode_batch *op) {
    if (!op) return;
    DeviceGuard guard(op->device);
    cudaFree(op->parts);
    cudaFree(op->table_dev);
    cudaFree(op->status);
    if (op->table_host) cudaFreeHost(op->table_host);
    if (op->table_event) cudaEventDestroy((cudaEvent_t)op->table_event);
    delete op;
}

// With `group` the merged partial of every sequence is published to the peers instead of gated into out.
static int batch_run(saetta_decode_batch *op, size_t n, saetta_kv_cache *const *caches, const uint32_t *kv_lens_host,
                     const float *q_dev, const float *q_and_gate_dev, float *out_dev, saetta_peer_group *group,
                     void *stream) {
    if (!op || !caches || !kv_lens_host || !q_dev || (!group && (!q_and_gate_dev || !out_dev)))
        return fail(SAETTA_ERR_BAD_ARG, "decode batch: null pointer");
    if (!n || n > op->max_seqs) return fail(SAETTA_ERR_BAD_SHAPE, "decode batch: more sequences than the op was made for");
    const int bits = caches[0] ? caches[0]->bits : 0;
    if (bits != 8 && bits != 4) return fail(SAETTA_ERR_UNSUPPORTED, "decode batch: caches must be 8- or 4-bit");
    uint64_t total_tiles = 0;
    for (size_t i = 0; i < n; i++) {
        if (!caches[i] || caches[i]->bits != bits || caches[i]->kv_heads != 2)
            return fail(SAETTA_ERR_BAD_SHAPE, "decode batch: caches differ in format");
        // (a shard of a short sequence may be empty: its partial is m = -inf, l = 0)
        if ((!kv_lens_host[i] && !group) || kv_lens_host[i] > caches[i]->capacity)
            return fail(SAETTA_ERR_BAD_SHAPE, "decode batch: kv_len outside the cache");
        total_tiles += (kv_lens_host[i] + 31) / 32;
    }
    DeviceGuard guard(op->device);
    // The pinned table is reused: wait until the previous call's copy has read it.
    if (op->table_event) SAETTA_CUDA(cudaEventSynchronize((cudaEvent_t)op->table_event));
    // Cut the concatenated tile sequence into equal CTA shares; a share that
    // crosses a sequence boundary becomes several segments.
    auto *segs = reinterpret_cast<Segment *>(op->table_host);
    auto *cta_first = reinterpret_cast<uint32_t *>(segs + op->max_parts);
    auto *seq_first = cta_first + op->ctas + 1;
    const uint32_t ctas = uint32_t(op->ctas);
    uint32_t nseg = 0;
    {
        // segments in (sequence, tile) order; parts are numbered in the same order,
        // so a sequence's parts are contiguous.
        size_t seq = 0;
        uint64_t seq_base = 0; // global index of the sequence's first tile
        uint64_t seq_tiles = (kv_lens_host[0] + 31) / 32;
        seq_first[0] = 0;
        for (uint32_t c = 0; c < ctas; c++) {
            cta_first[c] = nseg;
            uint64_t lo = total_tiles * c / ctas, hi = total_tiles * (c + 1) / ctas;
            while (lo < hi) {
                while (lo >= seq_base + seq_tiles) {
                    seq_base += seq_tiles;
                    seq++;
                    seq_tiles = (kv_lens_host[seq] + 31) / 32;
                    seq_first[seq] = nseg;
                }
                const uint64_t end = hi < seq_base + seq_tiles ? hi : seq_base + seq_tiles;
                Segment s{};
                const saetta_kv_cache *kc = caches[seq];
                s.k = kc->k.data, s.v = kc->v.data, s.ks = kc->k.scales, s.kz = kc->k.biases;
                s.vs = kc->v.scales, s.vz = kc->v.biases;
                s.tile_begin = uint32_t(lo - seq_base), s.tile_end = uint32_t(end - seq_base);
                s.kv_len = kv_lens_host[seq], s.part = nseg, s.seq = uint32_t(seq);
                if (nseg >= op->max_parts) return fail(SAETTA_ERR_BAD_SHAPE, "decode batch: part table overflow");
                segs[nseg++] = s;
                lo = end;
            }
        }
        cta_first[ctas] = nseg;
        for (size_t s2 = seq + 1; s2 <= n; s2++) seq_first[s2] = nseg;
    }
    auto st = (cudaStream_t)stream;
    SAETTA_CUDA(cudaMemcpyAsync(op->table_dev, op->table_host, op->table_bytes, cudaMemcpyHostToDevice, st));
    SAETTA_CUDA(cudaEventRecord((cudaEvent_t)op->table_event, st));
    auto *segs_dev = reinterpret_cast<const Segment *>(op->table_dev);
    auto *cta_first_dev = reinterpret_cast<const uint32_t *>(segs_dev + op->max_parts);
    auto *seq_first_dev = cta_first_dev + op->ctas + 1;
    if (int rc = launch_decode_quant_batched(bits, segs_dev, cta_first_dev, op->ctas, q_dev, op->parts, op->status, st))
        return rc;
    return launch_merge_frag(op->parts, nseg, seq_first_dev, uint32_t(n), 2, q_and_gate_dev, out_dev,
                             group ? group->staging : nullptr, st, group ? &group->push : nullptr);
}

int saetta_decode_batch_record(saetta_decode_batch *op, size_t n, saetta_kv_cache *const *caches,
                               const uint32_t *kv_lens_host, const float *q_dev, const float *q_and_gate_dev,
                               float *out_dev, void *stream) {
    return batch_run(op, n, caches, kv_lens_host, q_dev, q_and_gate_dev, out_dev, nullptr, stream);
}

int saetta_decode_batch_publish(saetta_decode_batch *op, size_t n, saetta_kv_cache *const *caches,
                                const uint32_t *kv_lens_host, const float *q_dev, saetta_peer_group *group,
                                void *stream) {
    if (!group) return fail(SAETTA_ERR_BAD_ARG, "decode batch publish: null pointer");
    if (!group->connected) return fail(SAETTA_ERR_BAD_ARG, "decode batch publish: the group is not connected");
    if (op && (group->device != op->device || op->heads != group->heads || n > group->rows_max))
        return fail(SAETTA_ERR_BAD_SHAPE, "decode batch publish: the group was made for another shape or device");
    return batch_run(op, n, caches, kv_lens_host, q_dev, nullptr, nullptr, group, stream);
}

// ------------------------------------------------------------------ prefill

int saetta_att_gemm_create(int device, size_t chunk, size_t kv_heads, saetta_att_gemm **out) {
    if (!out) return fail(SAETTA_ERR_BAD_ARG, "AttGemm::new: out is null");
    if (!chunk || !kv_heads) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm::new: empty shape");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "AttGemm::new: cannot select the device");
    if (int rc = configure_device(device)) return rc;
    auto *op = new (std::nothrow) saetta_att_gemm();
    if (!op) return fail(SAETTA_ERR_NO_MEM, "AttGemm::new: host allocation");
    op->device = device, op->chunk = chunk, op->kv_heads = kv_heads;
    if (int rc = alloc_zero((void **)&op->status, 16)) {
        delete op;
        return rc;
    }
    *out = op;
    return SAETTA_OK;
}

void saetta_att_gemm_destroy(saetta_att_gemm *op) {
    if (!op) return;
    DeviceGuard guard(op->device);
    cudaFree(op->stage_k);
    cudaFree(op->stage_v);
    cudaFree(op->split_parts);
    cudaFree(op->status);
    delete op;
}


constexpr uint32_t kKeySplits = 2;      // work items a long-context tile's keys are cut into
constexpr size_t kSplitFromKeys = 16384; // from this many keys on

// AttGemm::new allocates all of its scratch (src/attention_gemm.rs:119-148); here `reserve` does, for
// caches of up to `tokens` rows: the 16-bit staging copies and the partials of the key splits.
int saetta_att_gemm_reserve(saetta_att_gemm *op, size_t tokens) {
    if (!op) return fail(SAETTA_ERR_BAD_ARG, "AttGemm: null handle");
    DeviceGuard guard(op->device);
    if (tokens >= kSplitFromKeys) {
        const size_t need = size_t(kKeySplits) * op->chunk * op->kv_heads * kHeadsPerKv * kPartStride;
        if (need > op->split_floats) {
            cudaFree(op->split_parts);
            op->split_parts = nullptr, op->split_floats = 0;
            if (int rc = alloc_zero((void **)&op->split_parts, need * sizeof(float))) return rc;
            op->split_floats = need;
        }
    }
    if (tokens <= op->stage_tokens) return SAETTA_OK;
    tokens = round_up(tokens, 1024);
    cudaFree(op->stage_k), cudaFree(op->stage_v);
    op->stage_k = op->stage_v = nullptr, op->stage_tokens = 0;
    op->staged[0] = op->staged[1] = saetta_att_gemm::Staged(); // what the old copies held is gone
    const size_t bytes = tokens * op->kv_heads * kDim * 2;
    if (int rc = alloc_zero(&op->stage_k, bytes)) return rc;
    if (int rc = alloc_zero(&op->stage_v, bytes)) return rc;
    op->stage_tokens = tokens;
    return SAETTA_OK;
}

int saetta_att_gemm_invalidate(saetta_att_gemm *op) {
    if (!op) return fail(SAETTA_ERR_BAD_ARG, "AttGemm: null handle");
    op->staged[0] = op->staged[1] = saetta_att_gemm::Staged();
    return SAETTA_OK;
}

int saetta_att_gemm_stage_quantised(saetta_att_gemm *op, int on) {
    if (!op) return fail(SAETTA_ERR_BAD_ARG, "AttGemm: null handle");
    op->stage_quant = on != 0;
    return SAETTA_OK;
}

int saetta_att_gemm_score_blocks(saetta_att_gemm *op, int keys) {
    if (!op) return fail(SAETTA_ERR_BAD_ARG, "AttGemm: null handle");
    if (keys != 64 && keys != 128) return fail(SAETTA_ERR_BAD_ARG, "AttGemm: score blocks of 64 or 128 keys");
    op->narrow = keys == 64;
    return SAETTA_OK;
}

static int prefill_check(const void *q, int dtype, const saetta_flash_params &p) {
    if (!q) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: q is null");
    if (dtype != SAETTA_F16 && dtype != SAETTA_BF16) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: dtype");
    if (!p.kv_heads || p.heads != p.kv_heads * kHeadsPerKv) return fail(SAETTA_ERR_BAD_SHAPE, "needs 8 q heads per kv head");
    if (!aligned16(q)) return fail(SAETTA_ERR_BAD_ARG, "prefill attention: q must be 16-byte aligned");
    return SAETTA_OK;
}

// Brings rows [lo, hi) of one side's staging copy (row r of the copy = row r of the cache buffer)
// up to date.  Rows the copy already holds from the same buffer in the same type are kept when they
// lie below `fresh_from` (the first row of the chunk being encoded: what lies below it was written
// before the call that staged it and has not changed since, unless the caller says so with
// saetta_att_gemm_invalidate); the rest is converted by `convert(first, count)`.
static int stage_rows(saetta_att_gemm *op, int side, const void *src, int dtype, size_t lo, size_t hi, size_t fresh_from,
                      cudaStream_t st, const std::function<int(size_t, size_t)> &convert) {
    if (hi > op->stage_tokens) {
        if (capturing(st))
            return fail(SAETTA_ERR_BAD_ARG, "AttGemm::encode: the staging copy must grow, which a recording cannot do; call saetta_att_gemm_reserve first");
        if (int rc = saetta_att_gemm_reserve(op, hi)) return rc;
    }
    saetta_att_gemm::Staged &s = op->staged[side];
    size_t from = lo;
    const bool same = s.src == src && s.dtype == dtype && s.lo <= lo && s.hi >= lo;
    if (same) from = std::max(lo, std::min(s.hi, fresh_from));
    if (from < hi)
        if (int rc = convert(from, hi - from)) return rc;
    s.src = src, s.dtype = dtype, s.lo = same ? s.lo : lo, s.hi = hi;
    return SAETTA_OK;
}

// key_base: global position of row 0 of the cache buffers handed in (0 unless a shard stores only its slice).
static int att_gemm_run(saetta_att_gemm *op, const void *q, int dtype, const void *keys, const void *values,
                        const saetta_quant_rows *kq, const saetta_quant_rows *vq, const float *q_and_gate, float *out,
                        float *part, saetta_flash_params p, size_t key_base, size_t key_lo, size_t key_hi, cudaStream_t st) {
    if (int rc = prefill_check(q, dtype, p)) return rc;
    if (!p.tokens) return SAETTA_OK;
    if (p.kv_heads != op->kv_heads) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm::encode: kv heads differ from the op's");
    DeviceGuard guard(op->device);
    const size_t end = size_t(p.pos) + p.tokens;
    if (key_hi > end) key_hi = end;
    if (key_base % 64 || key_base > key_lo)
        return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm: the cache's first row must sit at a multiple of 64 at or below key_lo");
    if (key_hi <= key_lo) key_hi = key_lo; // an empty shard: every row gets the empty partial
    // rows of the buffers the kernel reads, and the first row of the chunk itself
    const size_t lo = key_lo - key_base, hi = key_hi - key_base;
    const size_t fresh = size_t(p.pos) > key_base ? size_t(p.pos) - key_base : 0;
    int v_dtype = dtype, k_dtype = dtype;
    // in place: the kernel turns the codes into operand tiles itself, per key block
    const bool in_place = (kq || vq) && p.kv_heads == 2 && !op->stage_quant;
    if (kq || vq) {
        if (!kq || !vq || kq->bits != vq->bits) return fail(SAETTA_ERR_BAD_ARG, "AttGemm::encode: quant needs both sides");
        if (hi > kq->capacity || hi > vq->capacity) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm::encode: the keys asked for exceed the capacity");
        if (kq->per_token != p.kv_heads * size_t(kGroupsPerHead)) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm::encode: quant rows of another shape");
    }
    if ((kq || vq) && !in_place) {
        // Other head counts, or a caller who asked for it (saetta_att_gemm_stage_quantised: every query tile
        // converts the blocks it reads when the codes are read in place, which costs the tensor pipe about a
        // fifth of its rate; with the copy each row is converted once, for 2 KB per key and side of device
        // memory): the quantised cache is read through a 16-bit copy, as the reference's
        // kv_stage reads it (src/kv_quant.rs:121-126 semantics).  Both sides are staged as binary16
        // (exactly the reference's round_trip_as_half; bfloat16 queries are converted on their way into
        // tensor memory), so P is binary16 too and keeps an 11-bit significand.  Only the rows the copy does not hold yet are dequantised: per chunk of
        // a long prompt, the chunk's own rows.
        if (int rc = stage_rows(op, 0, kq->data, SAETTA_F16, lo, hi, fresh, st, [&](size_t first, size_t n) {
                return launch_kv_dequantize(kq, op->stage_k, SAETTA_F16, first, n, st);
            }))
            return rc;
        if (int rc = stage_rows(op, 1, vq->data, SAETTA_F16, lo, hi, fresh, st, [&](size_t first, size_t n) {
                return launch_kv_dequantize(vq, op->stage_v, SAETTA_F16, first, n, st);
            }))
            return rc;
        keys = op->stage_k, values = op->stage_v;
        k_dtype = v_dtype = SAETTA_F16;
    }
    if (!in_place && (!keys || !values)) return fail(SAETTA_ERR_BAD_ARG, "AttGemm::encode: keys or values null");
    if (!(kq || vq) && dtype == SAETTA_BF16) {
        // P must share V's type in the second MMA; bfloat16's 8-bit significand would put P's
        // rounding at the tolerance, so bfloat16 values go through a binary16 copy (exact in range).
        const size_t row = p.kv_heads * size_t(kDim);
        const void *src = values;
        if (int rc = stage_rows(op, 1, src, SAETTA_F16 + 16 /* converted from bfloat16 */, lo, hi, fresh, st, [&](size_t first, size_t n) {
                return launch_bf16_to_f16(static_cast<const uint16_t *>(src) + first * row,
                                          static_cast<uint16_t *>(op->stage_v) + first * row, n * row, st);
            }))
            return rc;
        values = op->stage_v;
        v_dtype = SAETTA_F16;
    }
    PrefillArgs a{q, keys, values, dtype, v_dtype, q_and_gate, out, part, p.heads, p.kv_heads, p.pos, p.tokens,
                  uint32_t(key_lo), uint32_t(key_hi), p.scale};
    a.key_base = uint32_t(key_base);
    a.k_dtype = k_dtype;
    a.narrow = op->narrow;
    if (in_place) {
        // 8/4-bit rows are read where they are, per key block (kernels/attention_rows_q.metal:16-31): no
        // 16-bit copy of the cache, nothing to reserve
        a.qbits = kq->bits;
        a.qk = kq->data, a.qv = vq->data, a.qks = kq->scales, a.qkz = kq->biases, a.qvs = vq->scales, a.qvz = vq->biases;
    }
    // Long context: every tile has about the same work, and tiles rarely divide evenly over
    // the SMs.  Cut each tile's keys into two work items (twice as many, half as long) and merge
    // their (m, l, O); the merge is a few tens of microseconds against milliseconds of MMA.
    if (out && key_hi - key_lo >= kSplitFromKeys) {
        const size_t need = size_t(kKeySplits) * p.tokens * p.heads * kPartStride;
        if (need > op->split_floats) {
            if (capturing(st))
                return fail(SAETTA_ERR_BAD_ARG, "AttGemm::encode: the key-split partials must be allocated, which a recording cannot do; call saetta_att_gemm_reserve first");
            cudaFree(op->split_parts);
            op->split_parts = nullptr, op->split_floats = 0;
            if (int rc = alloc_zero((void **)&op->split_parts, need * sizeof(float))) return rc;
            op->split_floats = need;
        }
        a.out = nullptr, a.part = op->split_parts, a.splits = kKeySplits;
        if (int rc = launch_prefill(a, op->status, st)) return rc;
        return launch_merge_logical(op->split_parts, kKeySplits, p.tokens, p.heads, q_and_gate, out, nullptr, st);
    }
    return launch_prefill(a, op->status, st);
}

int saetta_att_gemm_encode(saetta_att_gemm *op, const void *q_dev, int dtype, const void *keys_dev, const void *values_dev,
                           const saetta_quant_rows *keys_q, const saetta_quant_rows *values_q, const float *q_and_gate_dev,
                           float *out_dev, saetta_flash_params p, void *stream) {
    if (!op || !q_and_gate_dev || !out_dev) return fail(SAETTA_ERR_BAD_ARG, "AttGemm::encode: null pointer");
    if (p.tokens > op->chunk) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm::encode: more tokens than the chunk the op was made for");
    return att_gemm_run(op, q_dev, dtype, keys_dev, values_dev, keys_q, values_q, q_and_gate_dev, out_dev, nullptr, p, 0, 0,
                        size_t(p.pos) + p.tokens, (cudaStream_t)stream);
}

int saetta_att_gemm_partial(saetta_att_gemm *op, const void *q_dev, int dtype, const void *keys_dev, const void *values_dev,
                            const saetta_quant_rows *keys_q, const saetta_quant_rows *values_q, float *part_dev,
                            saetta_flash_params p, size_t key_lo, size_t key_hi, void *stream) {
    if (!op || !part_dev) return fail(SAETTA_ERR_BAD_ARG, "AttGemm partial: null pointer");
    if (key_lo > key_hi) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm partial: key_lo > key_hi");
    return att_gemm_run(op, q_dev, dtype, keys_dev, values_dev, keys_q, values_q, nullptr, nullptr, part_dev, p, 0, key_lo,
                        key_hi, (cudaStream_t)stream);
}

int saetta_att_gemm_partial_shard(saetta_att_gemm *op, const void *q_dev, int dtype, const void *keys_dev,
                                  const void *values_dev, const saetta_quant_rows *keys_q,
                                  const saetta_quant_rows *values_q, float *part_dev, saetta_flash_params p,
                                  size_t key_base, size_t key_lo, size_t key_hi, void *stream) {
    if (!op || !part_dev) return fail(SAETTA_ERR_BAD_ARG, "AttGemm partial: null pointer");
    if (key_lo > key_hi) return fail(SAETTA_ERR_BAD_SHAPE, "AttGemm partial: key_lo > key_hi");
    return att_gemm_run(op, q_dev, dtype, keys_dev, values_dev, keys_q, values_q, nullptr, nullptr, part_dev, p, key_base,
                        key_lo, key_hi, (cudaStream_t)stream);
}

int saetta_prefill_encode(int device, const void *q_dev, int dtype, const void *keys_dev, const void *values_dev,
                          const float *q_and_gate_dev, float *out_dev, saetta_flash_params p, void *stream) {
    if (!keys_dev || !values_dev || !q_and_gate_dev || !out_dev) return fail(SAETTA_ERR_BAD_ARG, "prefill encode: null pointer");
    if (int rc = prefill_check(q_dev, dtype, p)) return rc;
    if (dtype != SAETTA_F16)
        return fail(SAETTA_ERR_UNSUPPORTED, "prefill encode: binary16 only (bfloat16 values need AttGemm's binary16 staging copy)");
    if (!aligned16(keys_dev) || !aligned16(values_dev)) return fail(SAETTA_ERR_BAD_ARG, "prefill encode: keys and values must be 16-byte aligned");
    if (!p.tokens) return SAETTA_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SAETTA_ERR_CUDA, "prefill encode: cannot select the device");
    if (int rc = configure_device(device)) return rc;
    static uint32_t *status[64] = {};
    if (device < 0 || device >= 64) return fail(SAETTA_ERR_BAD_ARG, "prefill encode: device");
    {
        std::lock_guard<std::mutex> lock(g_init_mutex);
        if (!status[device])
            if (int rc = alloc_zero((void **)&status[device], 16)) return rc;
    }
    PrefillArgs a{q_dev, keys_dev, values_dev, dtype, dtype, q_and_gate_dev, out_dev, nullptr, p.heads, p.kv_heads, p.pos,
                  p.tokens, 0, p.pos + p.tokens, p.scale};
    return launch_prefill(a, status[device], (cudaStream_t)stream);
}

} // extern "C"
