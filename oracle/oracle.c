/*
 * CPU oracle for the decode-time linear operators (TEST INFRASTRUCTURE ONLY).
 *
 * This file restates, in plain C, the arithmetic of the reference's OpenCL
 * GEMV kernels so that the CUDA path can be checked against it.  It is a
 * checker: only tests, the smoke check and the benchmark's CPU-baseline leg
 * may link or call it.  The shipped library never does.
 *
 * What each function follows (paths are relative to the reference project):
 *   half codec            src/models/lfm2-5-350m/src/utils.cpp:1001-1068
 *   fp16 GEMV             src/models/lfm2-5-350m/src/utils.cpp:35-73 (generic, any K)
 *                         src/models/lfm2-5-350m/kernels/gemv_m1.cl:65-517
 *                         src/models/qwen2-5-0-5b/kernels/gemv_m1.cl:288-690
 *                         src/models/smollm2-135m-instruct/kernels/block_fused.cl:409-465
 *   int8 GEMV             src/models/lfm2-5-350m/kernels/gemv_m1_int8.cl:34-84
 *                         src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl:37-98
 *   Q4 GEMV               src/models/lfm2-5-350m/kernels/gemv_m1_q4.cl:31-127
 *   residual epilogue     src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl:105-167
 *   SwiGLU epilogue       src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl:176-231
 *   silu(gate)*(W3 x)     src/models/lfm2-5-350m/kernels/mlp_fused.cl:19-73
 *   dequantisation        src/models/lfm2-5-350m/scripts/quantize_q4.py:156-166
 *                         src/models/lfm2-5-350m/scripts/quantize_weights.py:135-139
 *
 * Pinning: the dequantisers and the quantiser restatement (oracle/quant.py) are
 * pinned against vectors produced by the reference's own Python quantisers
 * (tests/golden).  The kernel arithmetic is pinned against the reference's
 * unmodified .cl sources compiled for the CPU (oracle/_ref, built by
 * oracle/build_ref.py) when that build is present.
 *
 * Accumulation orders offered (argument `order`):
 *   0  the kernels' own order: 64 work-items, work-item t handles the vec4 (or
 *      8-nibble pixel) t, t+64, ... ; 4-term dot evaluated left to right with
 *      separate multiply and add; binary tree over the 64 partials.
 *   1  same, but each multiply-add contracted to fma (what a fast-math
 *      compiler may do).
 *   2  double precision, sequential (tolerance reference).
 * M > 1 is defined as M independent M = 1 results (the reference loops M = 1
 * for quantised weights: src/models/lfm2-5-350m/src/model.cpp:243-251).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_WG 64

enum { FMT_FP16 = 0, FMT_INT8 = 1, FMT_Q4 = 2 };

/* ---- IEEE binary16 codec, round to nearest even ------------------------- */
float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(113 - shift) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_f32_to_f16(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    uint32_t e8 = (b >> 23) & 0xFFu;
    uint32_t man = b & 0x7FFFFFu;
    if (e8 == 0xFFu) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0u));
    int32_t e = (int32_t)e8 - 112; /* half exponent field */
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) ++q;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) ++q; /* carry into exponent is correct */
    return (uint16_t)(sign | q);
}

/* ---- unpack rules (bit-exact contract) ----------------------------------- */
static inline int q4_code(const uint8_t* row, int k) {
    /* byte k/2: low nibble = even k, high nibble = odd k; value = nibble - 8 */
    return (int)((row[k >> 1] >> (4 * (k & 1))) & 0xF) - 8;
}

/* out[N*K] fp32 = float(q) * float(scale)   (per row for int8, per 32-block for Q4) */
void oracle_dequant(int fmt, int N, int K, const void* W, const uint16_t* scale, float* out) {
    for (int n = 0; n < N; ++n) {
        for (int k = 0; k < K; ++k) {
            float v;
            if (fmt == FMT_FP16) {
                v = oracle_f16_to_f32(((const uint16_t*)W)[(size_t)n * K + k]);
            } else if (fmt == FMT_INT8) {
                v = (float)((const int8_t*)W)[(size_t)n * K + k] * oracle_f16_to_f32(scale[n]);
            } else {
                const uint8_t* row = (const uint8_t*)W + (size_t)n * (K / 2);
                v = (float)q4_code(row, k) * oracle_f16_to_f32(scale[(size_t)n * (K / 32) + k / 32]);
            }
            out[(size_t)n * K + k] = v;
        }
    }
}

/* ---- one output row, full-K sum before any per-row scale ------------------ */
static inline float mul_add(float acc, float a, float b, int order) {
    return order == 1 ? fmaf(a, b, acc) : acc + a * b;
}

static float dot4(const float* a, const float* b, int order) {
    /* dot(float4,float4): left to right */
    if (order == 1) return fmaf(a[3], b[3], fmaf(a[2], b[2], fmaf(a[1], b[1], a[0] * b[0])));
    return ((a[0] * b[0] + a[1] * b[1]) + a[2] * b[2]) + a[3] * b[3];
}

static float tree64(float* p) {
    for (int s = ORACLE_WG / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) p[t] += p[t + s];
    return p[0];
}

/* fp16 / int8 rows: vec4 per work-item per iteration, scalar tail for K % 4 */
static float row_sum_vec4(int fmt, int K, const void* wrow, const float* xf, int order) {
    float part[ORACLE_WG];
    const int K4 = K >> 2;
    for (int t = 0; t < ORACLE_WG; ++t) {
        float acc = 0.f;
        for (int k4 = t; k4 < K4; k4 += ORACLE_WG) {
            float w[4];
            for (int i = 0; i < 4; ++i) {
                int k = 4 * k4 + i;
                w[i] = fmt == FMT_FP16 ? oracle_f16_to_f32(((const uint16_t*)wrow)[k])
                                       : (float)((const int8_t*)wrow)[k];
            }
            acc += dot4(xf + 4 * k4, w, order);
        }
        for (int k = K4 * 4 + t; k < K; k += ORACLE_WG) {
            float w = fmt == FMT_FP16 ? oracle_f16_to_f32(((const uint16_t*)wrow)[k])
                                      : (float)((const int8_t*)wrow)[k];
            acc = mul_add(acc, w, xf[k], order);
        }
        part[t] = acc;
    }
    return tree64(part);
}

/* Q4 rows: one 8-nibble pixel per work-item per iteration; scale folded per pixel */
static float row_sum_q4(int K, const uint8_t* wrow, const uint16_t* srow, const float* xf, int order) {
    float part[ORACLE_WG];
    const int npix = K >> 3;
    for (int t = 0; t < ORACLE_WG; ++t) {
        float acc = 0.f;
        for (int pix = t; pix < npix; pix += ORACLE_WG) {
            const int k0 = pix * 8;
            float d;
            if (order == 1) {
                d = xf[k0] * (float)q4_code(wrow, k0);
                for (int i = 1; i < 8; ++i) d = fmaf(xf[k0 + i], (float)q4_code(wrow, k0 + i), d);
                acc = fmaf(d, oracle_f16_to_f32(srow[pix >> 2]), acc);
            } else {
                d = xf[k0] * (float)q4_code(wrow, k0);
                for (int i = 1; i < 8; ++i) d = d + xf[k0 + i] * (float)q4_code(wrow, k0 + i);
                acc += d * oracle_f16_to_f32(srow[pix >> 2]);
            }
        }
        part[t] = acc;
    }
    return tree64(part);
}

static double row_sum_f64(int fmt, int K, const void* wrow, const uint16_t* srow, const float* xf) {
    double acc = 0.0;
    if (fmt == FMT_Q4) {
        for (int k = 0; k < K; ++k)
            acc += (double)xf[k] * (double)q4_code((const uint8_t*)wrow, k) *
                   (double)oracle_f16_to_f32(srow[k >> 5]);
    } else if (fmt == FMT_INT8) {
        for (int k = 0; k < K; ++k) acc += (double)xf[k] * (double)((const int8_t*)wrow)[k];
    } else {
        for (int k = 0; k < K; ++k)
            acc += (double)xf[k] * (double)oracle_f16_to_f32(((const uint16_t*)wrow)[k]);
    }
    return acc;
}

static size_t row_bytes(int fmt, int K) {
    return fmt == FMT_FP16 ? (size_t)K * 2 : fmt == FMT_INT8 ? (size_t)K : (size_t)K / 2;
}

/*
 * acc[M*N] (fp32) = x[M,K] . W[N,K]^T with the format's scale placement:
 *   int8: (sum over K) * float(scale[n])      -- scale once, at the tail
 *   Q4  : sum over 8-weight partials of d * float(scale[n][k/32])
 * This is the value the kernels hold just before the final half store.
 */
typedef struct {
    int fmt, M, N, K, order, n0, n1;
    const void* W;
    const uint16_t* scale;
    const uint16_t* x;
    float* acc;
} lin_job;

static void* lin_worker(void* arg) {
    lin_job* j = (lin_job*)arg;
    const size_t rb = row_bytes(j->fmt, j->K);
    float* xf = (float*)malloc(sizeof(float) * (size_t)j->K);
    for (int m = 0; m < j->M; ++m) {
        for (int k = 0; k < j->K; ++k) xf[k] = oracle_f16_to_f32(j->x[(size_t)m * j->K + k]);
        for (int n = j->n0; n < j->n1; ++n) {
            const uint8_t* wrow = (const uint8_t*)j->W + rb * (size_t)n;
            const uint16_t* srow = j->fmt == FMT_Q4 ? j->scale + (size_t)n * (j->K / 32) : NULL;
            float v;
            if (j->order == 2) {
                double d = row_sum_f64(j->fmt, j->K, wrow, srow, xf);
                if (j->fmt == FMT_INT8) d *= (double)oracle_f16_to_f32(j->scale[n]);
                v = (float)d;
            } else {
                if (j->fmt == FMT_Q4) v = row_sum_q4(j->K, wrow, srow, xf, j->order);
                else v = row_sum_vec4(j->fmt, j->K, wrow, xf, j->order);
                if (j->fmt == FMT_INT8) v = v * oracle_f16_to_f32(j->scale[n]);
            }
            j->acc[(size_t)m * j->N + n] = v;
        }
    }
    free(xf);
    return NULL;
}

int oracle_linear_acc(int fmt, int M, int N, int K, const void* W, const uint16_t* scale,
                      const uint16_t* x, float* acc, int order, int nthreads) {
    if (fmt < 0 || fmt > 2 || M < 0 || N < 0 || K < 0) return -1;
    if (fmt == FMT_Q4 && (K % 32) != 0) return -1;
    if (nthreads < 1) nthreads = 1;
    if (nthreads > N) nthreads = N > 0 ? N : 1;
    if (nthreads > 256) nthreads = 256;
    lin_job jobs[256];
    pthread_t th[256];
    for (int t = 0; t < nthreads; ++t) {
        lin_job* j = &jobs[t];
        j->fmt = fmt; j->M = M; j->N = N; j->K = K; j->order = order;
        j->n0 = (int)((long long)N * t / nthreads);
        j->n1 = (int)((long long)N * (t + 1) / nthreads);
        j->W = W; j->scale = scale; j->x = x; j->acc = acc;
    }
    if (nthreads == 1) { lin_worker(&jobs[0]); return 0; }
    for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, lin_worker, &jobs[t]);
    for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
    return 0;
}

/* ---- epilogues: what work-item 0 does with the reduced sum --------------- */
/* plain: out = half(acc) */
void oracle_store_half(size_t n, const float* acc, uint16_t* out) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_f32_to_f16(acc[i]);
}
/* residual (in place): r = half(float(r) + acc) */
void oracle_store_residual(size_t n, const float* acc, uint16_t* r) {
    for (size_t i = 0; i < n; ++i) r[i] = oracle_f32_to_f16(oracle_f16_to_f32(r[i]) + acc[i]);
}
/* SwiGLU of two projections: out = half( g / (1 + exp(-g)) * u ) */
void oracle_store_swiglu(size_t n, const float* g, const float* u, uint16_t* out) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_f32_to_f16((g[i] / (1.0f + expf(-g[i]))) * u[i]);
}
/* gate in/out: gate = half( gate * (1 / (1 + exp(-gate))) * acc ) */
void oracle_store_silu_gate(size_t n, const float* acc, uint16_t* gate) {
    for (size_t i = 0; i < n; ++i) {
        float g = oracle_f16_to_f32(gate[i]);
        float sig = 1.0f / (1.0f + expf(-g));
        gate[i] = oracle_f32_to_f16(g * sig * acc[i]);
    }
}

/* ---- RMSNorm feeding the projections --------------------------------------
 * src/models/smollm2-135m-instruct/kernels/rmsnorm.cl:27-104 (USE_FP16 path): one work-group
 * of 64 per row; lane t sums dot(v, v) over the vec4 columns c4 = t, t + 64, ... (then a scalar
 * tail), a binary tree reduces the 64 partials, inv = rsqrt(sum / cols + eps), and every element
 * is stored as half((x * inv) * weight). */
void oracle_rmsnorm_half(int rows, int cols, const uint16_t* x, const uint16_t* weight, float eps, uint16_t* out) {
    const int C4 = cols >> 2;
    for (int r = 0; r < rows; ++r) {
        const uint16_t* xr = x + (size_t)r * cols;
        float p[64];
        for (int t = 0; t < 64; ++t) {
            float acc = 0.0f;
            for (int c4 = t; c4 < C4; c4 += 64) {
                float v[4];
                for (int i = 0; i < 4; ++i) v[i] = oracle_f16_to_f32(xr[c4 * 4 + i]);
                acc += ((v[0] * v[0] + v[1] * v[1]) + v[2] * v[2]) + v[3] * v[3];
            }
            for (int c = C4 * 4 + t; c < cols; c += 64) {
                float v = oracle_f16_to_f32(xr[c]);
                acc += v * v;
            }
            p[t] = acc;
        }
        for (int s2 = 32; s2 > 0; s2 >>= 1)
            for (int t = 0; t < s2; ++t) p[t] += p[t + s2];
        const float inv = 1.0f / sqrtf(p[0] / (float)cols + eps);
        for (int c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] = oracle_f32_to_f16((oracle_f16_to_f32(xr[c]) * inv) * oracle_f16_to_f32(weight[c]));
    }
}

/* arg-max over fp16 logits; the first index wins on ties (the reference's
 * src/models/lfm2-5-350m/kernels/argmax.cl:30-120 resolves ties by work-item order). */
int oracle_argmax_half(size_t n, const uint16_t* v) {
    size_t best = 0;
    float bv = -INFINITY;
    for (size_t i = 0; i < n; ++i) {
        float f = oracle_f16_to_f32(v[i]);
        if (f > bv) { bv = f; best = i; }
    }
    return (int)best;
}
