/*
 * CPU oracle for the attention hot path of saetta-macqwen.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, loop for loop and in the
 * same summation order, the reference's own Rust CPU code.  It is the checker
 * the CUDA kernels are compared against and the timed CPU baseline; nothing in
 * the shipped library links or calls it.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (never -ffast-math), so that
 * a*b+c stays an unfused multiply and add as in the Rust code.
 *
 * Parity is pinned against the reference's own fixtures and known answers:
 *   src/cpu/testdata/attention.json  (src/cpu/attention.rs:188-221)
 *   src/cpu/testdata/ops.json        (src/cpu/ops.rs:81-110)
 *   packed-word known answers        (src/kv_quant.rs:319-332)
 *   half-step round-trip bound       (src/kv_quant.rs:302-317)
 *
 * Third-party arithmetic: binary16 conversion comes from crate `half` 2.7.1
 * (Cargo.lock), whose f16::from_f32 / to_f32 are IEEE round-to-nearest-even
 * narrowing and exact widening; restated here in software.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SO_GROUP 64 /* src/kv_quant.rs:9 */

/* ---------------------------------------------------------------- f16 / bf16 */

static uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
static float bits_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* IEEE binary32 -> binary16, round to nearest even (half::f16::from_f32). */
uint16_t so_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xffu;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
    }
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
    if (e <= 0) {                                   /* subnormal or zero */
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e); /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++; /* may carry into exp: correct */
    return (uint16_t)(sign | half);
}

/* binary16 -> binary32, exact (half::f16::to_f32). */
float so_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp - 15 + 127) << 23) | (man << 13));
}

/* binary32 -> bfloat16 (round to nearest even) and back. */
uint16_t so_f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7f800000u) == 0x7f800000u && (x & 0x7fffffu)) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}
float so_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

void so_round_f16(const float *x, float *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_f16_to_f32(so_f32_to_f16(x[i]));
}
void so_round_bf16(const float *x, float *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_bf16_to_f32(so_f32_to_bf16(x[i]));
}
void so_to_f16(const float *x, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_f32_to_f16(x[i]);
}
void so_to_bf16(const float *x, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_f32_to_bf16(x[i]);
}
void so_from_f16(const uint16_t *x, float *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_f16_to_f32(x[i]);
}
void so_from_bf16(const uint16_t *x, float *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = so_bf16_to_f32(x[i]);
}

/* ---------------------------------------------------------------- kv_quant */

/* Rust f32::min / f32::max: a NaN operand is ignored. */
static float rs_min(float a, float b) { return fminf(a, b); }
static float rs_max(float a, float b) { return fmaxf(a, b); }

/*
 * src/kv_quant.rs:54-87 `quantize`.  n is a multiple of 64; bits is 8 or 4.
 * data gets n/64 * 2*bits words, scales and biases n/64 binary16 values each.
 * Returns 0, or -1 on a bad argument (the reference asserts).
 */
int so_quantize(const float *x, size_t n, int bits, uint32_t *data, uint16_t *scales,
                uint16_t *biases) {
    if ((bits != 8 && bits != 4) || n % SO_GROUP) return -1;
    const float levels = (float)((1u << bits) - 1);
    const size_t per_word = 32 / (size_t)bits;
    size_t w = 0;
    for (size_t g = 0; g < n / SO_GROUP; g++) {
        const float *group = x + g * SO_GROUP;
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < SO_GROUP; i++) lo = rs_min(lo, group[i]);
        for (int i = 0; i < SO_GROUP; i++) hi = rs_max(hi, group[i]);
        uint16_t s = so_f32_to_f16((hi - lo) / levels);
        uint16_t z = so_f32_to_f16(lo);
        float sf = so_f16_to_f32(s), zf = so_f16_to_f32(z);
        float inv = sf > 0.0f ? 1.0f / sf : 0.0f;
        for (size_t k = 0; k < SO_GROUP; k += per_word) {
            uint32_t word = 0;
            for (size_t i = 0; i < per_word; i++) {
                float r = rintf((group[k + i] - zf) * inv); /* round_ties_even */
                /* f32::clamp then `as u32` (NaN casts to 0) */
                if (r != r) r = 0.0f;
                if (r < 0.0f) r = 0.0f;
                if (r > levels) r = levels;
                word |= (uint32_t)r << (i * (size_t)bits);
            }
            data[w++] = word;
        }
        scales[g] = s;
        biases[g] = z;
    }
    return 0;
}

/* src/kv_quant.rs:90-105 `dequantize`: s * q + z, a multiply then an add. */
int so_dequantize(const uint32_t *data, const uint16_t *scales, const uint16_t *biases,
                  size_t groups, int bits, float *out) {
    if (bits != 8 && bits != 4) return -1;
    const uint32_t mask = (1u << bits) - 1;
    const size_t per_word = 32 / (size_t)bits, words = 2 * (size_t)bits;
    size_t o = 0;
    for (size_t g = 0; g < groups; g++) {
        float s = so_f16_to_f32(scales[g]), z = so_f16_to_f32(biases[g]);
        for (size_t k = 0; k < words; k++) {
            uint32_t w = data[g * words + k];
            for (size_t i = 0; i < per_word; i++) {
                uint32_t q = (w >> (i * (size_t)bits)) & mask;
                float p = s * (float)q;
                out[o++] = p + z;
            }
        }
    }
    return 0;
}

/* src/kv_quant.rs:129-135 `round_trip` (bits 16 rounds to binary16). */
int so_round_trip(const float *x, size_t n, int bits, float *y) {
    if (bits == 16) {
        so_round_f16(x, y, n);
        return 0;
    }
    if ((bits != 8 && bits != 4) || n % SO_GROUP) return -1;
    size_t groups = n / SO_GROUP;
    uint32_t *data = malloc(groups * 2 * (size_t)bits * 4);
    uint16_t *s = malloc(groups * 2), *z = malloc(groups * 2);
    so_quantize(x, n, bits, data, s, z);
    so_dequantize(data, s, z, groups, bits, y);
    free(data);
    free(s);
    free(z);
    return 0;
}

/* src/kv_quant.rs:121-126 `round_trip_as_half`; to_bf16 != 0 rounds the
 * dequantised values to bfloat16 instead (the storage type the tensor-core
 * prefill kernel feeds its multiplies with). */
int so_round_trip_as_half(const float *x, size_t n, int bits, int to_bf16, float *y) {
    int rc = so_round_trip(x, n, bits, y);
    if (rc) return rc;
    if (to_bf16)
        so_round_bf16(y, y, n);
    else
        so_round_f16(y, y, n);
    return 0;
}

/* ---------------------------------------------------------------- cpu::ops */

/* src/cpu/ops.rs:13-15 `dot`: left-to-right f32 sum of products. */
float so_dot(const float *a, const float *b, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float p = a[i] * b[i];
        s = s + p;
    }
    return s;
}

/* src/cpu/ops.rs:4-11 `matvec`: w is [out][n]. */
void so_matvec(const float *w, const float *x, size_t out, size_t n, float *y) {
    for (size_t r = 0; r < out; r++) y[r] = so_dot(w + r * n, x, n);
}

/*
 * src/cpu/matrix.rs:104-135 `row_dot` over every row (`quant_matvec`, :73-101): y = W x for an MLX
 * affine matrix (src/quant.rs:1-30): a row is a little-endian bit stream of `bits`-wide integers in
 * u32 words, every 64 values share a bfloat16 scale and bias, w = scale * q + bias, and the sum over
 * a group is scale * sum(q x) + bias * sum(x), groups added in order.
 */
static float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
int so_quant_matvec(const uint32_t *words, const uint16_t *scales, const uint16_t *biases, int bits, size_t rows,
                    size_t cols, const float *x, float *y) {
    if ((bits != 4 && bits != 5 && bits != 6 && bits != 8) || cols % 64) return 1;
    const size_t groups = cols / 64, row_words = cols * (size_t)bits / 32;
    float *x_sums = malloc(groups * sizeof(float));
    for (size_t g = 0; g < groups; g++) {
        float t = 0.0f;
        for (size_t i = 0; i < 64; i++) t = t + x[g * 64 + i];
        x_sums[g] = t;
    }
    const uint64_t mask = (1ull << bits) - 1;
    for (size_t r = 0; r < rows; r++) {
        const uint32_t *w = words + r * row_words;
        uint64_t acc = 0;
        unsigned have = 0;
        size_t next = 0;
        float total = 0.0f;
        for (size_t g = 0; g < groups; g++) {
            float dot = 0.0f;
            for (size_t i = 0; i < 64; i++) {
                if (have < (unsigned)bits) {
                    acc |= (uint64_t)w[next++] << have;
                    have += 32;
                }
                float p = (float)(acc & mask) * x[g * 64 + i];
                dot = dot + p;
                acc >>= bits;
                have -= bits;
            }
            float a = bf16_bits_to_f32(scales[r * groups + g]) * dot;
            float b = bf16_bits_to_f32(biases[r * groups + g]) * x_sums[g];
            total = total + (a + b);
        }
        y[r] = total;
    }
    free(x_sums);
    return 0;
}

/* src/cpu/ops.rs:19-36 `rms_norm`. */
void so_rms_norm(float *x, const float *w, size_t n, float eps) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float p = x[i] * x[i];
        ss = ss + p;
    }
    float mean = ss / (float)n;
    float scale = 1.0f / sqrtf(mean + eps);
    for (size_t i = 0; i < n; i++) {
        float sg = scale * w[i];
        x[i] = x[i] * sg;
    }
}

/* src/cpu/ops.rs:38-40 `sigmoid`. */
float so_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

/* src/cpu/ops.rs:51-59 `softmax`. */
void so_softmax(float *x, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = rs_max(max, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - max);
        sum += x[i];
    }
    for (size_t i = 0; i < n; i++) x[i] /= sum;
}

/* src/cpu/ops.rs:64-74 `rope`: value i pairs with i + dims/2, f64 angle. */
void so_rope(float *head, size_t dims, size_t pos, float theta) {
    size_t half = dims / 2;
    for (size_t i = 0; i < half; i++) {
        double freq = pow((double)theta, -((double)i) / (double)half);
        double angle = (double)pos * freq;
        float s = (float)sin(angle), c = (float)cos(angle);
        float a = head[i], b = head[i + half];
        float ac = a * c, bs = b * s, as = a * s, bc = b * c;
        head[i] = ac - bs;
        head[i + half] = as + bc;
    }
}

/* ---------------------------------------------------------------- attention */

/*
 * src/cpu/attention.rs:159-181 `attend`: one query head over the first `len`
 * tokens of kv head `kv`.  keys/values are [len][kv_heads][d].  scratch holds
 * len floats.
 */
void so_attend(const float *q, const float *keys, const float *values, size_t len,
               size_t kv_heads, size_t d, size_t kv, float *scratch, float *out) {
    size_t stride = kv_heads * d, offset = kv * d;
    float scale = 1.0f / sqrtf((float)d);
    for (size_t t = 0; t < len; t++) scratch[t] = so_dot(q, keys + t * stride + offset, d) * scale;
    so_softmax(scratch, len);
    for (size_t i = 0; i < d; i++) out[i] = 0.0f;
    for (size_t t = 0; t < len; t++) {
        float p = scratch[t];
        const float *v = values + t * stride + offset;
        for (size_t i = 0; i < d; i++) {
            float pv = p * v[i];
            out[i] = out[i] + pv;
        }
    }
}

/*
 * The inner part of the layer for `rows` query rows (src/cpu/attention.rs:144-154
 * with the buffer layout of src/attention.rs:68-71 and src/rows.rs:379-381):
 *   q           [rows][heads][d]
 *   q_and_gate  [rows][heads][2d], gate of head h at h*2d + d
 *   keys/values [>= max len][kv_heads][d] f32 (already rounded as the cache stores them)
 *   lens[r]     number of keys row r sees
 *   out         [rows][heads][d] = attend(...) * sigmoid(gate)
 * One (row, head) pair is one unit of work.
 */
typedef struct {
    const float *q, *q_and_gate, *keys, *values;
    const uint32_t *lens;
    float *out;
    size_t rows, heads, kv_heads, d;
    size_t first, step; /* units first, first+step, ... */
} so_job;

static void *so_job_run(void *arg) {
    so_job *j = arg;
    size_t group = j->heads / j->kv_heads, maxlen = 0;
    for (size_t r = 0; r < j->rows; r++)
        if (j->lens[r] > maxlen) maxlen = j->lens[r];
    float *scratch = malloc((maxlen ? maxlen : 1) * sizeof(float));
    for (size_t u = j->first; u < j->rows * j->heads; u += j->step) {
        size_t r = u / j->heads, h = u % j->heads;
        float *o = j->out + (r * j->heads + h) * j->d;
        so_attend(j->q + (r * j->heads + h) * j->d, j->keys, j->values, j->lens[r], j->kv_heads,
                  j->d, h / group, scratch, o);
        const float *g = j->q_and_gate + (r * j->heads + h) * 2 * j->d + j->d;
        for (size_t i = 0; i < j->d; i++) o[i] = o[i] * so_sigmoid(g[i]);
    }
    free(scratch);
    return NULL;
}

int so_attention_rows(const float *q, const float *q_and_gate, const float *keys,
                      const float *values, const uint32_t *lens, size_t rows, size_t heads,
                      size_t kv_heads, size_t d, int threads, float *out) {
    if (!kv_heads || heads % kv_heads || threads < 1) return -1;
    if (threads > 256) threads = 256;
    so_job jobs[256];
    pthread_t tid[256];
    for (int t = 0; t < threads; t++) {
        jobs[t] = (so_job){q, q_and_gate, keys, values, lens, out, rows, heads, kv_heads, d,
                           (size_t)t, (size_t)threads};
    }
    if (threads == 1) {
        so_job_run(&jobs[0]);
        return 0;
    }
    for (int t = 0; t < threads; t++) pthread_create(&tid[t], NULL, so_job_run, &jobs[t]);
    for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    return 0;
}

/*
 * src/cpu/attention.rs:103-156 `attention_at`: the whole layer for one token,
 * appending to a caller-owned cache (keys/values [cap][kv_heads][d], *len tokens
 * held).  rounding: 0 none, 16/8/4 = KvCache::round_to, +100 = as_half too.
 * Used to replay attention.json.
 */
int so_attention_layer(size_t hidden, size_t heads, size_t kv_heads, size_t d, size_t rope_dims,
                       float theta, float eps, const float *q_proj, const float *k_proj,
                       const float *v_proj, const float *o_proj, const float *q_norm,
                       const float *k_norm, const float *x, size_t pos, float *keys, float *values,
                       size_t *len, int rounding, float *y) {
    size_t hd = heads * d, kd = kv_heads * d;
    float *qg = malloc(2 * hd * 4), *q = malloc(hd * 4), *gate = malloc(hd * 4);
    float *k = malloc(kd * 4), *v = malloc(kd * 4), *out = malloc(hd * 4);
    so_matvec(q_proj, x, 2 * hd, hidden, qg);
    for (size_t h = 0; h < heads; h++) {
        memcpy(q + h * d, qg + h * 2 * d, d * 4);
        memcpy(gate + h * d, qg + h * 2 * d + d, d * 4);
    }
    so_matvec(k_proj, x, kd, hidden, k);
    so_matvec(v_proj, x, kd, hidden, v);
    for (size_t h = 0; h < heads; h++) {
        so_rms_norm(q + h * d, q_norm, d, eps);
        so_rope(q + h * d, rope_dims, pos, theta);
    }
    for (size_t h = 0; h < kv_heads; h++) {
        so_rms_norm(k + h * d, k_norm, d, eps);
        so_rope(k + h * d, rope_dims, pos, theta);
    }
    if (rounding) {
        int bits = rounding % 100, as_half = rounding >= 100;
        int rc = as_half ? so_round_trip_as_half(k, kd, bits, 0, k) : so_round_trip(k, kd, bits, k);
        rc |= as_half ? so_round_trip_as_half(v, kd, bits, 0, v) : so_round_trip(v, kd, bits, v);
        if (rc) return rc;
    }
    memcpy(keys + *len * kd, k, kd * 4);
    memcpy(values + *len * kd, v, kd * 4);
    *len += 1;
    float *scratch = malloc(*len * 4);
    size_t group = heads / kv_heads;
    for (size_t h = 0; h < heads; h++)
        so_attend(q + h * d, keys, values, *len, kv_heads, d, h / group, scratch, out + h * d);
    for (size_t i = 0; i < hd; i++) out[i] = out[i] * so_sigmoid(gate[i]);
    so_matvec(o_proj, out, hidden, hd, y);
    free(scratch);
    free(qg);
    free(q);
    free(gate);
    free(k);
    free(v);
    free(out);
    return 0;
}

/* ---------------------------------------------------------------- generators */

/* tests/attention.rs:16-26, src/kv_quant.rs:290-300 `noise`: 64-bit LCG. */
void so_noise(float *x, size_t n, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        x[i] = (float)(s >> 40) / (float)(1ull << 23) - 1.0f;
    }
}

/* src/attention_prefill.rs:103-108 `spread` (before the narrowing to half). */
void so_spread(float *x, size_t n, size_t seed) {
    for (size_t i = 0; i < n; i++) x[i] = (float)((i * 7919 + seed * 104729) % 1999) / 500.0f - 2.0f;
}

/* Seeded N(0,1): splitmix64 -> Box-Muller in f64, narrowed to f32.  Not from
 * the reference (it has no normal generator); used for the benchmark shapes. */
static uint64_t splitmix64(uint64_t *s) {
    uint64_t z = (*s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
void so_normal(float *x, size_t n, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; i += 2) {
        double u1 = ((double)(splitmix64(&s) >> 11) + 1.0) / 9007199254740993.0;
        double u2 = (double)(splitmix64(&s) >> 11) / 9007199254740992.0;
        double r = sqrt(-2.0 * log(u1)), a = 6.283185307179586476925286766559 * u2;
        x[i] = (float)(r * cos(a));
        if (i + 1 < n) x[i + 1] = (float)(r * sin(a));
    }
}
