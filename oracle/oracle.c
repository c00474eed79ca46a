/* CPU restatement (plain C) of the reference's quantized-linear arithmetic. TEST INFRASTRUCTURE ONLY.
 *
 * Used by the test-suite as a second parity checker, by the benchmark's cpu_baseline leg, and to build full-size
 * seeded inputs quickly. No product path links or loads it. Functions name the reference source they follow (paths
 * relative to the reference project root). It is validated byte-for-byte against the NumPy oracle, which is itself
 * pinned to vectors produced by the reference (tests/golden).
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off: no fused multiply-add may be introduced by the compiler)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

/* ---------------------------------------------------------------- helpers ---------------------------------- */

static inline float bf16_to_float(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* native/src/q3/numeric.cuh:17-21 */
static inline uint16_t float_to_bf16(float value) {
    uint32_t u;
    memcpy(&u, &value, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float half_to_float(uint16_t bits) {
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h;
}

static inline uint16_t float_to_half(float value) {
    _Float16 h = (_Float16)value; /* round to nearest even */
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

static const float kE2m1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* Unsigned E4M3, bias 7, subnormals (tools/euhedral_artifacts/nvfp4.py:25-28; native/src/nvfp4/nvfp4.cuh:60-62). */
static inline float e4m3_value(uint32_t code) {
    code &= 0x7fu;
    const uint32_t e = code >> 3, m = code & 7u;
    return e == 0 ? ldexpf((float)m / 8.0f, -6) : ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
}

/* Nearest code 0..126, ties to even, saturating (tools/euhedral_artifacts/nvfp4.py:72-82 over the E4M3 table). */
static inline uint8_t e4m3_encode(float v) {
    if (!(v > 0.0f)) return 0;
    if (v >= 448.0f) return 126;
    if (v < 0.015625f) return (uint8_t)lrint((double)v * 512.0);
    int exp2;
    (void)frexp((double)v, &exp2);
    int e = exp2 - 1;
    long q = lrint(ldexp((double)v, 3 - e));
    if (q == 16) {
        e += 1;
        q = 8;
    }
    long code = (long)(e + 7) * 8 + (q - 8);
    return (uint8_t)(code > 126 ? 126 : code);
}

/* Nearest E2M1 magnitude index, ties to the even index (same table search). */
static inline uint8_t e2m1_encode(float v) {
    uint8_t i = 0;
    if (v > 0.25f) i = 1;
    if (v >= 0.75f) i = 2;
    if (v > 1.25f) i = 3;
    if (v >= 1.75f) i = 4;
    if (v > 2.5f) i = 5;
    if (v >= 3.5f) i = 6;
    if (v > 5.0f) i = 7;
    return i;
}

static inline uint64_t align_up(uint64_t v, uint64_t unit) { return (v + unit - 1) / unit * unit; }

/* ---------------------------------------------------------------- threading -------------------------------- */

typedef void (*range_fn)(void* ctx, uint32_t begin, uint32_t end);
typedef struct {
    range_fn fn;
    void* ctx;
    uint32_t begin, end;
} task_t;

static void* task_main(void* p) {
    task_t* t = (task_t*)p;
    t->fn(t->ctx, t->begin, t->end);
    return NULL;
}

static void parallel_rows(range_fn fn, void* ctx, uint32_t n, int threads) {
    if (threads < 1) threads = 1;
    if ((uint32_t)threads > n) threads = (int)n;
    if (threads <= 1) {
        fn(ctx, 0, n);
        return;
    }
    pthread_t* ids = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    task_t* tasks = (task_t*)malloc(sizeof(task_t) * (size_t)threads);
    for (int i = 0; i < threads; ++i) {
        tasks[i].fn = fn;
        tasks[i].ctx = ctx;
        tasks[i].begin = (uint32_t)((uint64_t)n * (uint64_t)i / (uint64_t)threads);
        tasks[i].end = (uint32_t)((uint64_t)n * (uint64_t)(i + 1) / (uint64_t)threads);
        pthread_create(&ids[i], NULL, task_main, &tasks[i]);
    }
    for (int i = 0; i < threads; ++i) pthread_join(ids[i], NULL);
    free(ids);
    free(tasks);
}

/* ---------------------------------------------------------------- NVFP4 ------------------------------------ */

EXPORT void oracle_nvfp4_offsets(uint32_t n, uint32_t k, uint64_t* scale_off, uint64_t* global_off, uint64_t* size) {
    const uint64_t kp = align_up(k, 128);
    *scale_off = align_up((uint64_t)n * kp / 2, 256);
    *global_off = align_up(*scale_off + (uint64_t)n * kp / 16, 256);
    *size = *global_off + 4;
}

typedef struct {
    const float* w;
    uint8_t* blob;
    uint32_t n, k;
    float global;
} nvfp4_q_ctx;

/* tools/euhedral_artifacts/nvfp4.py:89-105 */
static void nvfp4_quantize_rows(void* p, uint32_t begin, uint32_t end) {
    nvfp4_q_ctx* c = (nvfp4_q_ctx*)p;
    const uint64_t kp = align_up(c->k, 128);
    uint64_t scale_off, global_off, size;
    oracle_nvfp4_offsets(c->n, c->k, &scale_off, &global_off, &size);
    const float g = c->global;
    float block[16];
    for (uint32_t r = begin; r < end; ++r) {
        uint8_t* codes = c->blob + (uint64_t)r * kp / 2;
        uint8_t* scales = c->blob + scale_off + (uint64_t)r * kp / 16;
        for (uint64_t b = 0; b < kp / 16; ++b) {
            float amax = 0.0f;
            for (int i = 0; i < 16; ++i) {
                const uint64_t col = b * 16 + (uint64_t)i;
                block[i] = col < c->k ? c->w[(uint64_t)r * c->k + col] : 0.0f;
                amax = fmaxf(amax, fabsf(block[i]));
            }
            float ratio = 0.0f;
            if (g > 0.0f) {
                ratio = amax / 6.0f;
                ratio = ratio / g;
            }
            const uint8_t sc = e4m3_encode(ratio);
            const float step = e4m3_value(sc) * g;
            scales[b] = sc;
            for (int i = 0; i < 16; i += 2) {
                uint8_t pair = 0;
                for (int h = 0; h < 2; ++h) {
                    const float v = block[i + h];
                    const float scaled = step > 0.0f ? fabsf(v) / step : 0.0f;
                    uint8_t code = e2m1_encode(scaled);
                    if (v < 0.0f && code > 0) code |= 8u;
                    pair |= (uint8_t)(code << (4 * h));
                }
                codes[b * 8 + (uint64_t)i / 2] = pair;
            }
        }
    }
}

/* Whole tensor as the converter writes it (tools/euhedral_artifacts/nvfp4.py:226-266, uncalibrated). `blob` must hold
 * oracle_nvfp4_offsets().size bytes. */
EXPORT void oracle_nvfp4_quantize(const float* weights, uint32_t n, uint32_t k, uint8_t* blob, int threads) {
    nvfp4_q_ctx ctx;
    memset(&ctx, 0, sizeof(ctx));
    ctx.w = weights;
    ctx.blob = blob;
    ctx.n = n;
    ctx.k = k;
    uint64_t scale_off, global_off, size;
    oracle_nvfp4_offsets(n, k, &scale_off, &global_off, &size);
    memset(blob, 0, size);
    float amax = 0.0f;
    for (uint64_t i = 0; i < (uint64_t)n * k; ++i) {
        const float a = fabsf(weights[i]);
        if (a > amax) amax = a;
    }
    ctx.global = amax / 2688.0f;
    parallel_rows(nvfp4_quantize_rows, &ctx, n, threads);
    memcpy(blob + global_off, &ctx.global, 4);
}

typedef struct {
    const uint16_t* x;
    const uint8_t* blob;
    float* y;
    float* dense;
    uint32_t rows, k, n;
} linear_ctx;

/* Dense float32 weights, fp32(e2m1 * sign) * fp32(e4m3 * global) (tools/euhedral_artifacts/nvfp4.py:108-115). */
static void nvfp4_dense_rows(void* p, uint32_t begin, uint32_t end) {
    linear_ctx* c = (linear_ctx*)p;
    const uint64_t kp = align_up(c->k, 128);
    uint64_t scale_off, global_off, size;
    oracle_nvfp4_offsets(c->n, c->k, &scale_off, &global_off, &size);
    float g;
    memcpy(&g, c->blob + global_off, 4);
    for (uint32_t r = begin; r < end; ++r) {
        const uint8_t* codes = c->blob + (uint64_t)r * kp / 2;
        const uint8_t* scales = c->blob + scale_off + (uint64_t)r * kp / 16;
        for (uint32_t col = 0; col < c->k; ++col) {
            const uint32_t code = (codes[col / 2] >> ((col & 1u) * 4u)) & 15u;
            const float value = (code & 8u) ? -kE2m1[code & 7u] : kE2m1[code & 7u];
            const float block = e4m3_value(scales[col / 16]) * g;
            c->dense[(uint64_t)r * c->k + col] = value * block;
        }
    }
}

EXPORT void oracle_nvfp4_dense(const uint8_t* blob, uint32_t n, uint32_t k, float* dense, int threads) {
    linear_ctx ctx = {NULL, blob, NULL, dense, 0, k, n};
    parallel_rows(nvfp4_dense_rows, &ctx, n, threads);
}

/* y[row][out] (float32) = (sum_k x * (e2m1 * e4m3)) * global with FP32 accumulation in K order: the arithmetic of
 * native/src/reference/kernels.cu:125-149 (products exact, global applied to the sum) in a sequential order. */
static void nvfp4_linear_rows(void* p, uint32_t begin, uint32_t end) {
    linear_ctx* c = (linear_ctx*)p;
    const uint64_t kp = align_up(c->k, 128);
    uint64_t scale_off, global_off, size;
    oracle_nvfp4_offsets(c->n, c->k, &scale_off, &global_off, &size);
    float g;
    memcpy(&g, c->blob + global_off, 4);
    float* wrow = (float*)malloc(sizeof(float) * c->k);
    float scale_lut[128];
    for (uint32_t i = 0; i < 128; ++i) scale_lut[i] = e4m3_value(i);
    for (uint32_t out = begin; out < end; ++out) {
        const uint8_t* codes = c->blob + (uint64_t)out * kp / 2;
        const uint8_t* scales = c->blob + scale_off + (uint64_t)out * kp / 16;
        for (uint32_t col = 0; col < c->k; ++col) {
            const uint32_t code = (codes[col / 2] >> ((col & 1u) * 4u)) & 15u;
            const float value = (code & 8u) ? -kE2m1[code & 7u] : kE2m1[code & 7u];
            wrow[col] = value * scale_lut[scales[col / 16] & 0x7fu];
        }
        for (uint32_t row = 0; row < c->rows; ++row) {
            const uint16_t* x = c->x + (uint64_t)row * c->k;
            float sum = 0.0f;
            for (uint32_t col = 0; col < c->k; ++col) sum += bf16_to_float(x[col]) * wrow[col];
            c->y[(uint64_t)row * c->n + out] = sum * g;
        }
    }
    free(wrow);
}

EXPORT void oracle_nvfp4_linear(const uint16_t* x, const uint8_t* blob, float* y, uint32_t rows, uint32_t k, uint32_t n,
        int threads) {
    linear_ctx ctx = {x, blob, y, NULL, rows, k, n};
    parallel_rows(nvfp4_linear_rows, &ctx, n, threads);
}

/* ---------------------------------------------------------------- Q3G64_F16S ------------------------------- */

EXPORT void oracle_q3_offsets(uint32_t n, uint32_t k, uint64_t* scale_off, uint64_t* size) {
    const uint64_t groups = align_up(k, 128) / 64;
    *scale_off = align_up((uint64_t)n * groups * 24, 256);
    *size = *scale_off + (uint64_t)n * groups * 2;
}

typedef struct {
    const float* w;
    uint8_t* blob;
    uint32_t n, k;
} q3_q_ctx;

/* tools/euhedral_artifacts/grouped.py:39-66,129-135 (round to nearest, no calibration). */
static void q3_quantize_rows(void* p, uint32_t begin, uint32_t end) {
    q3_q_ctx* c = (q3_q_ctx*)p;
    const uint64_t groups = align_up(c->k, 128) / 64;
    uint64_t scale_off, size;
    oracle_q3_offsets(c->n, c->k, &scale_off, &size);
    for (uint32_t r = begin; r < end; ++r) {
        for (uint64_t g = 0; g < groups; ++g) {
            float v[64];
            float amax = 0.0f;
            for (int i = 0; i < 64; ++i) {
                const uint64_t col = g * 64 + (uint64_t)i;
                v[i] = col < c->k ? c->w[(uint64_t)r * c->k + col] : 0.0f;
                amax = fmaxf(amax, fabsf(v[i]));
            }
            const float raw = (float)((double)amax / 3.0);
            uint16_t sbits = float_to_half(raw);
            if ((sbits & 0x7fffu) == 0 && amax > 0.0f) sbits = 0x0001u; /* 2^-24 */
            const float scale = half_to_float(sbits);
            const float inverse = scale > 0.0f ? (float)(1.0 / (double)scale) : 0.0f;
            uint8_t* out = c->blob + ((uint64_t)r * groups + g) * 24;
            memset(out, 0, 24);
            for (int i = 0; i < 64; ++i) {
                float q = rintf(v[i] * inverse);
                if (q < -4.0f) q = -4.0f;
                if (q > 3.0f) q = 3.0f;
                const uint32_t field = (uint32_t)((int)q & 7);
                const int bit = 3 * i;
                out[bit >> 3] |= (uint8_t)(field << (bit & 7));
                if ((bit & 7) > 5) out[(bit >> 3) + 1] |= (uint8_t)(field >> (8 - (bit & 7)));
            }
            memcpy(c->blob + scale_off + ((uint64_t)r * groups + g) * 2, &sbits, 2);
        }
    }
}

EXPORT void oracle_q3_quantize(const float* weights, uint32_t n, uint32_t k, uint8_t* blob, int threads) {
    q3_q_ctx ctx = {weights, blob, n, k};
    uint64_t scale_off, size;
    oracle_q3_offsets(n, k, &scale_off, &size);
    memset(blob, 0, size);
    parallel_rows(q3_quantize_rows, &ctx, n, threads);
}

static inline int q3_code(const uint8_t* group, uint32_t index) {
    const uint32_t bit = index * 3u;
    const uint32_t word = (uint32_t)group[bit >> 3] | ((bit >> 3) + 1u < 24u ? (uint32_t)group[(bit >> 3) + 1u] << 8 : 0u);
    const uint32_t field = (word >> (bit & 7u)) & 7u;
    return (int)field - (field >= 4u ? 8 : 0);
}

static void q3_dense_rows(void* p, uint32_t begin, uint32_t end) {
    linear_ctx* c = (linear_ctx*)p;
    const uint64_t groups = align_up(c->k, 128) / 64;
    uint64_t scale_off, size;
    oracle_q3_offsets(c->n, c->k, &scale_off, &size);
    for (uint32_t r = begin; r < end; ++r)
        for (uint32_t col = 0; col < c->k; ++col) {
            const uint64_t g = (uint64_t)r * groups + col / 64;
            uint16_t sbits;
            memcpy(&sbits, c->blob + scale_off + g * 2, 2);
            c->dense[(uint64_t)r * c->k + col] = (float)q3_code(c->blob + g * 24, col % 64) * half_to_float(sbits);
        }
}

EXPORT void oracle_q3_dense(const uint8_t* blob, uint32_t n, uint32_t k, float* dense, int threads) {
    linear_ctx ctx = {NULL, blob, NULL, dense, 0, k, n};
    parallel_rows(q3_dense_rows, &ctx, n, threads);
}

/* y (float32) = sum_k (x * code) * scale, FP32, K order (native/src/reference/kernels.cu:27-41;
 * core/src/test/.../gpu/FirstLayerCpuReference.java:146-173). */
static void q3_linear_rows(void* p, uint32_t begin, uint32_t end) {
    linear_ctx* c = (linear_ctx*)p;
    const uint64_t groups = align_up(c->k, 128) / 64;
    uint64_t scale_off, size;
    oracle_q3_offsets(c->n, c->k, &scale_off, &size);
    float* wrow = (float*)malloc(sizeof(float) * c->k);
    for (uint32_t out = begin; out < end; ++out) {
        for (uint32_t col = 0; col < c->k; ++col) {
            const uint64_t g = (uint64_t)out * groups + col / 64;
            uint16_t sbits;
            memcpy(&sbits, c->blob + scale_off + g * 2, 2);
            wrow[col] = (float)q3_code(c->blob + g * 24, col % 64) * half_to_float(sbits);
        }
        for (uint32_t row = 0; row < c->rows; ++row) {
            const uint16_t* x = c->x + (uint64_t)row * c->k;
            float sum = 0.0f;
            for (uint32_t col = 0; col < c->k; ++col) sum += bf16_to_float(x[col]) * wrow[col];
            c->y[(uint64_t)row * c->n + out] = sum;
        }
    }
    free(wrow);
}

EXPORT void oracle_q3_linear(const uint16_t* x, const uint8_t* blob, float* y, uint32_t rows, uint32_t k, uint32_t n,
        int threads) {
    linear_ctx ctx = {x, blob, y, NULL, rows, k, n};
    parallel_rows(q3_linear_rows, &ctx, n, threads);
}

/* ---------------------------------------------------------------- trellis ---------------------------------- */

/* One codebook value (native/src/trellis/codebook.cuh:33-37): FP16 fma(0x6400 + bytesum(state * 0x83DCD12D), 0x1EEE,
 * 0xC931), one rounding. */
static inline uint16_t trellis_value_bits(uint32_t state) {
    const uint32_t x = state * 0x83DCD12Du;
    const uint32_t sum = 0x6400u + (x & 255u) + ((x >> 8) & 255u) + ((x >> 16) & 255u) + (x >> 24);
    const double a = (double)half_to_float((uint16_t)sum);
    const double b = (double)half_to_float(0x1EEE), c = (double)half_to_float(0xC931);
    const double r = a * b + c; /* exact in double: 11 x 11 bit product plus an 11 bit addend */
    _Float16 h = (_Float16)r;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

/* 16-bit window ending at ring bit S(p) (codebook.cuh:40-61). words: w little-endian int16 of one tile. */
static inline uint32_t trellis_state(const uint16_t* words, int w, int p) {
    const int m = p & 15, ka = w >> 4;
    const int half_step = (w & 15) == 8;
    const int end = (p >> 4) * w + ka * (m + 1) + (half_step ? (m + 1) / 2 : 0);
    const int ring = 16 * w;
    int start = (end - 16) % ring;
    if (start < 0) start += ring;
    uint32_t state = 0;
    for (int i = 0; i < 16; ++i) {
        const int bit = (start + i) % ring;       /* MSB-first within each uint32 */
        const int word32 = bit >> 5, o = bit & 31;
        const uint32_t value = (uint32_t)words[2 * word32] | ((uint32_t)words[2 * word32 + 1] << 16);
        state = (state << 1) | ((value >> (31 - o)) & 1u);
    }
    return state;
}

/* values[256] FP16 bits in tensor-core position order. */
EXPORT void oracle_trellis_decode_tile(const uint16_t* words, int w, uint16_t* values) {
    for (int p = 0; p < 256; ++p) values[p] = trellis_value_bits(trellis_state(words, w, p));
}

typedef struct {
    const uint16_t* x;      /* bf16 [rows][k] */
    const uint16_t* words;  /* [k/16][n/16][w] */
    const uint16_t* suh;    /* f16 [s][k] */
    const uint16_t* svh;    /* f16 [n] */
    const int32_t* ends;
    float* y;               /* [rows][n] */
    int s, rows, k, n, w;
} trellis_ctx;

/* native/src/trellis/codebook.cuh:76-92 */
static void hadamard128(float* v) {
    for (int h = 1; h < 128; h <<= 1)
        for (int t = 0; t < 64; ++t) {
            const int i = (t / h) * 2 * h + (t % h);
            const float a = v[i], b = v[i + h];
            v[i] = a + b;
            v[i + h] = a - b;
        }
    for (int i = 0; i < 128; ++i) v[i] = v[i] * 0.08838834764831845f;
}

/* Column blocks [begin, end) of 128 columns. FP32 throughout, activations not rounded to FP16: the arithmetic of the
 * scalar device oracle native/src/reference/trellis.cuh:14-55. */
static void trellis_linear_blocks(void* p, uint32_t begin, uint32_t end) {
    trellis_ctx* c = (trellis_ctx*)p;
    const int k = c->k, n = c->n, w = c->w, tiles_n = n / 16;
    float* u = (float*)malloc(sizeof(float) * (size_t)k * (size_t)c->rows);
    float* q = (float*)malloc(sizeof(float) * (size_t)k * 128);
    uint16_t tile[256];
    for (uint32_t block = begin; block < end; ++block) {
        const int c0 = (int)block * 128;
        int g = 0;
        while (g + 1 < c->s && c0 >= c->ends[g]) ++g;
        for (int r = 0; r < c->rows; ++r) {
            float* ur = u + (size_t)r * k;
            for (int col = 0; col < k; ++col)
                ur[col] = bf16_to_float(c->x[(size_t)r * k + col]) * half_to_float(c->suh[(size_t)g * k + col]);
            for (int b = 0; b < k / 128; ++b) hadamard128(ur + b * 128);
        }
        for (int ti = 0; ti < k / 16; ++ti)
            for (int tj = 0; tj < 8; ++tj) {
                oracle_trellis_decode_tile(c->words + ((size_t)ti * tiles_n + (size_t)(c0 / 16 + tj)) * w, w, tile);
                for (int pos = 0; pos < 256; ++pos) {
                    const int t = pos >> 3, j = pos & 7;
                    const int row = (t & 3) * 2 + ((j >> 1) & 1) * 8 + (j & 1);
                    const int col = (t >> 2) + (j >> 2) * 8;
                    q[(size_t)(ti * 16 + row) * 128 + tj * 16 + col] = half_to_float(tile[pos]);
                }
            }
        for (int r = 0; r < c->rows; ++r) {
            float z[128];
            for (int col = 0; col < 128; ++col) z[col] = 0.0f;
            const float* ur = u + (size_t)r * k;
            for (int row = 0; row < k; ++row) {
                const float a = ur[row];
                const float* qr = q + (size_t)row * 128;
                for (int col = 0; col < 128; ++col) z[col] += a * qr[col];
            }
            hadamard128(z);
            for (int col = 0; col < 128; ++col)
                c->y[(size_t)r * n + c0 + col] = half_to_float(c->svh[c0 + col]) * z[col];
        }
    }
    free(u);
    free(q);
}

EXPORT void oracle_trellis_linear(const uint16_t* x, const uint16_t* words, const uint16_t* suh, const uint16_t* svh,
        const int32_t* ends, int s, float* y, int rows, int k, int n, int w, int threads) {
    trellis_ctx ctx = {x, words, suh, svh, ends, y, s, rows, k, n, w};
    parallel_rows(trellis_linear_blocks, &ctx, (uint32_t)(n / 128), threads);
}

/* ---------------------------------------------------------------- misc ------------------------------------- */

EXPORT void oracle_float_to_bf16(const float* in, uint16_t* out, uint64_t count) {
    for (uint64_t i = 0; i < count; ++i) out[i] = float_to_bf16(in[i]);
}

EXPORT int oracle_abi_version(void) { return 1; }

/* ---------------------------------------------------------------- trellis tile encoder --------------------- */

/* The reference's tile encoder (quantization/src/main/resources/cuda/trellis.cu:34-399, from exllamav3's dense and
 * fractional Viterbi kernels): a 256-weight tile is quantized to a tail-biting ring of 16-bit states; position i brings
 * d(i) = ka + bit (i mod 16) of `mask` new bits (mask 0: an integer rate, 0xAAAA: the half-step rates). Costs are FP16:
 * the first step costs (value - w)^2 (one rounding for the difference, one for the square), every further step
 * fma(difference, difference, cost of the predecessor) with one rounding; of equal costs the lowest predecessor wins.
 * Two passes (trellis.cu:93-99,393-396): from an open start at position 128 all round, the best end node (ties by the
 * kernels' bit-reversed rank, trellis.cu:63-81) is traced back to the node entering position 0; the second pass starts at
 * position 0 pinned to that node and is traced back in full. Test infrastructure: restated to check an encoder against the
 * reference's golden tiles (tiles-K-idx / -out / -packed). */

static double g_half_value[65536];      /* every FP16 bit pattern as a double */
static uint16_t g_state_value[65536];   /* codebook value (FP16 bits) of every state */
static pthread_once_t g_encoder_once = PTHREAD_ONCE_INIT;

static void encoder_tables(void) {
    for (uint32_t i = 0; i < 65536u; ++i) {
        g_half_value[i] = (double)half_to_float((uint16_t)i);
        g_state_value[i] = trellis_value_bits(i);
    }
}

static inline uint16_t double_to_half_bits(double v) {
    _Float16 h = (_Float16)v; /* one rounding, to nearest even */
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

/* a < b as the kernels compare FP16 costs (__hlt: false when either is NaN) */
static inline int half_less(uint16_t a, uint16_t b) {
    const double x = g_half_value[a], y = g_half_value[b];
    return x < y;
}

static inline uint32_t reverse5(uint32_t v) {
    return ((v & 1u) << 4) | ((v & 2u) << 2) | (v & 4u) | ((v & 8u) >> 2) | ((v & 16u) >> 4);
}

typedef struct {
    const float* tiles;
    uint16_t* indices;
    float* decoded;
    int ka;
    uint32_t mask;
} encode_ctx;

static inline int position_bits(int position, int ka, uint32_t mask) { return ka + (int)((mask >> (position & 15)) & 1u); }

/* One forward pass; history[ri][node] = the predecessor node chosen for `node` at ring position ri. */
static void encoder_forward(const uint16_t* w_bits, int roll, int pre_state, int ka, uint32_t mask, uint16_t* cost_a, uint16_t* cost_b,
        uint16_t** final_costs, uint16_t* history) {
    uint16_t *costs = cost_a, *previous = cost_b;
    for (int i = 0; i < 256; ++i) {
        const int ri = (i + roll) & 255;
        uint16_t* swap = costs;
        costs = previous;
        previous = swap;
        const int kin = position_bits(ri, ka, mask), kout = position_bits(ri + 1, ka, mask);
        const int shift = 16 - kout, nodes = 65536 >> kout, branches = 1 << kout;
        const double w = g_half_value[w_bits[ri]];
        const int write = pre_state >= 0 || ri < 128;
        for (int node = 0; node < nodes; ++node) {
            uint16_t best = 0;
            int best_from = 0;
            for (int branch = 0; branch < branches; ++branch) {
                const int state = (branch << shift) | node, from = state >> kin;
                const double difference = g_half_value[double_to_half_bits(g_half_value[g_state_value[state]] - w)];
                uint16_t cost;
                if (i == 0)
                    cost = pre_state >= 0 && from != pre_state ? 0x7c00u : double_to_half_bits(difference * difference);
                else
                    cost = double_to_half_bits(difference * difference + g_half_value[previous[from]]);
                if (branch == 0 || half_less(cost, best)) {
                    best = cost;
                    best_from = from;
                }
            }
            costs[node] = best;
            if (write) history[(size_t)ri * 65536u + (size_t)node] = (uint16_t)best_from;
        }
    }
    *final_costs = costs;
}

static void encode_tiles_range(void* p, uint32_t begin, uint32_t end) {
    const encode_ctx* c = (const encode_ctx*)p;
    uint16_t* history = (uint16_t*)malloc((size_t)256 * 65536u * sizeof(uint16_t));
    uint16_t* cost_a = (uint16_t*)malloc(65536u * sizeof(uint16_t));
    uint16_t* cost_b = (uint16_t*)malloc(65536u * sizeof(uint16_t));
    for (uint32_t tile = begin; tile < end; ++tile) {
        uint16_t w_bits[256];
        for (int i = 0; i < 256; ++i) w_bits[i] = float_to_half(c->tiles[(size_t)tile * 256u + (size_t)i]);
        uint16_t* costs = NULL;
        /* pass 1: open start at position 128; the best of the last step's nodes, ties by the kernels' rank */
        encoder_forward(w_bits, 128, -1, c->ka, c->mask, cost_a, cost_b, &costs, history);
        const int last_nodes = 65536 >> position_bits(128, c->ka, c->mask);
        uint32_t best_key = 0x7c00ffffu;
        for (int e = 0; e < last_nodes; ++e) {
            const uint32_t v = (uint32_t)e & 1023u;
            const uint32_t rank = (reverse5(v >> 5) << 10) | (reverse5(v & 31u) << 5) | ((uint32_t)e >> 10);
            const uint32_t key = ((uint32_t)costs[e] << 16) | rank;
            if (key < best_key) best_key = key;
        }
        int node = 0;
        if (best_key < 0x7c000000u) {
            const uint32_t rank = best_key & 65535u;
            node = (int)(((rank & 31u) << 10) | (reverse5(rank >> 10) << 5) | reverse5((rank >> 5) & 31u));
        }
        /* back to the node that enters position 0 (ring positions 127 down to 0 carry history in this pass) */
        for (int i = 255; i >= 0; --i) {
            const int ri = (i + 128) & 255;
            node = history[(size_t)ri * 65536u + (size_t)node];
            if (ri == 0) break;
        }
        const int pinned = node;
        /* pass 2: from position 0, pinned; traced back in full */
        encoder_forward(w_bits, 0, pinned, c->ka, c->mask, cost_a, cost_b, &costs, history);
        node = pinned;
        for (int ri = 255; ri >= 0; --ri) {
            const int from = history[(size_t)ri * 65536u + (size_t)node];
            const int state = ((from << position_bits(ri, c->ka, c->mask)) | node) & 0xFFFF;
            node = from;
            c->indices[(size_t)tile * 256u + (size_t)ri] = (uint16_t)state;
            c->decoded[(size_t)tile * 256u + (size_t)ri] = half_to_float(g_state_value[state]);
        }
    }
    free(history);
    free(cost_a);
    free(cost_b);
}

/* tiles float32 [count][256] -> indices u16 [count][256] (the 16-bit state of every position), decoded float32. */
EXPORT void oracle_trellis_encode_tiles(const float* tiles, uint32_t count, int ka, uint32_t mask, uint16_t* indices, float* decoded,
        int threads) {
    pthread_once(&g_encoder_once, encoder_tables);
    encode_ctx c = {tiles, indices, decoded, ka, mask};
    parallel_rows(encode_tiles_range, &c, count, threads);
}
