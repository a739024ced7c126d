/*
 * CPU oracle for the W4A16 matmul path of LLM170 -- TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's CPU algorithm.  It is the
 * checker for the CUDA path: only the tests, the smoke check and the bench's CPU
 * baseline leg may load it.  Nothing in the product library links or calls it.
 *
 * Parity pin: the reference is Rust and cannot be compiled where this oracle is
 * developed, so the oracle is pinned by re-running the reference's own known-answer
 * tests for this path (they are computable, no stored vectors): see
 * tests/test_oracle_kat.py, which cites each reference test it restates.
 *
 * Must be compiled with -ffp-contract=off: the reference accumulates with a separate
 * f32 multiply and f32 add (crates/core/src/quant/lane.rs:62-64).
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* crates/core/src/quant/deq.rs:4-27  (IEEE half -> f32, subnormals/inf/nan kept) */
ORC_API float orc_half_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t frac = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (frac == 0) {
            bits = sign << 31;
        } else {
            uint32_t e = 127 - 15 + 1;
            uint32_t f = frac;
            while ((f & 0x400u) == 0) {
                f <<= 1;
                e -= 1;
            }
            f &= 0x3ffu;
            bits = (sign << 31) | (e << 23) | (f << 13);
        }
    } else if (exp == 0x1f) {
        bits = (sign << 31) | (0xffu << 23) | (frac << 13);
    } else {
        bits = (sign << 31) | ((exp + 112) << 23) | (frac << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* crates/core/src/quant/deq.rs:29-31 */
ORC_API float orc_bf16_to_f32(uint16_t h) {
    uint32_t bits = ((uint32_t)h) << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:187-219  (f32 -> f16, round to nearest even) */
ORC_API uint16_t orc_f32_to_f16(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xFFu);
    uint32_t man = b & 0x7FFFFFu;
    if (exp == 0xFF) {
        return (uint16_t)(sign | 0x7C00u | (man != 0 ? 0x200u : 0u));
    }
    int32_t e = exp - 127 + 15;
    if (e >= 31) {
        return (uint16_t)(sign | 0x7C00u);
    }
    if (e <= 0) {
        if (e < -10) {
            return sign;
        }
        uint32_t m = man | 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = 1u << (shift - 1);
        uint32_t sub = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1);
        if (rem > half || (rem == half && (sub & 1u) == 1u)) {
            sub += 1;
        }
        return (uint16_t)(sign | (uint16_t)sub);
    }
    uint32_t h = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u) == 1u)) {
        h += 1;
    }
    return (uint16_t)(sign | (uint16_t)h);
}

/* crates/core/src/quant/lane.rs:2-13  (fixed pairwise f64 tree over the 64 lanes) */
ORC_API double orc_tree64(const double *v) {
    double a[64];
    memcpy(a, v, sizeof(a));
    for (int i = 0; i < 32; ++i) {
        a[i] += a[i + 32];
    }
    static const int offs[5] = {16, 8, 4, 2, 1};
    for (int o = 0; o < 5; ++o) {
        int off = offs[o];
        for (int i = 0; i < off; ++i) {
            a[i] += a[i + off];
        }
    }
    return a[0];
}

/* crates/core/src/quant/lane.rs:42-70.  Lane l takes elements i = l, l+64, ...; each
 * accumulator is a sequential f32 sum with un-fused multiply and add.  Returns 0 on
 * success, -1 on a violated shape contract (the reference asserts). */
ORC_API int orc_lane_parts_scale(const uint32_t *qrow, const uint32_t *zrow, const float *scale,
                                 const uint16_t *x, int k, int group, double *lane_out) {
    if (group < 32 || group % 32 != 0 || k % group != 0) {
        return -1;
    }
    for (int l = 0; l < 64; ++l) {
        float acc = 0.0f;
        for (int i = l; i < k; i += 64) {
            int g = i / group;
            int32_t q = (int32_t)((qrow[i >> 3] >> (4 * (i & 7))) & 0xFu);
            float w = (float)(q - (int32_t)zrow[g]) * scale[g];
            float p = w * orc_half_to_f32(x[i]);
            acc = acc + p;
        }
        lane_out[l] = (double)acc;
    }
    return 0;
}

/* crates/core/src/quant/lane.rs:32-40 */
ORC_API float orc_dot_row_w4a16_lane_group(const uint32_t *qrow, const uint32_t *zrow,
                                           const float *srow_f32, const uint16_t *x, int k,
                                           int group) {
    double lanes[64];
    if (orc_lane_parts_scale(qrow, zrow, srow_f32, x, k, group, lanes) != 0) {
        return NAN;
    }
    return (float)orc_tree64(lanes);
}

/* crates/core/src/quant/lane.rs:19-30  (g128, f16 scales) */
ORC_API float orc_dot_row_w4a16_lane(const uint32_t *qrow, const uint32_t *zrow,
                                     const uint16_t *srow, const uint16_t *x, int k) {
    if (k % 128 != 0) {
        return NAN;
    }
    int ng = k / 128;
    float *sc = (float *)malloc(sizeof(float) * (size_t)ng);
    for (int g = 0; g < ng; ++g) {
        sc[g] = orc_half_to_f32(srow[g]);
    }
    float r = orc_dot_row_w4a16_lane_group(qrow, zrow, sc, x, k, 128);
    free(sc);
    return r;
}

/* crates/core/src/matmul/cpu.rs:167-194  ((nib-8) as f32 * scale for one row) */
ORC_API void orc_dequant_row_w4a16_split(const uint8_t *q, const uint8_t *s, size_t row, int k,
                                         int group, int scale_bf16, float *out) {
    int nb = k / group;
    const uint8_t *qrow = q + row * (size_t)(k / 2);
    const uint8_t *srow = s + row * (size_t)(k * 2 / group);
    for (int b = 0; b < nb; ++b) {
        uint16_t bits = (uint16_t)(srow[2 * b] | (srow[2 * b + 1] << 8));
        float sc = scale_bf16 ? orc_bf16_to_f32(bits) : orc_half_to_f32(bits);
        for (int i = 0; i < group; ++i) {
            int woff = 4 * (b * (group / 8) + i / 8);
            uint32_t w = (uint32_t)qrow[woff] | ((uint32_t)qrow[woff + 1] << 8) |
                         ((uint32_t)qrow[woff + 2] << 16) | ((uint32_t)qrow[woff + 3] << 24);
            int32_t nib = (int32_t)((w >> (4 * (i % 8))) & 0xFu);
            out[b * group + i] = (float)(nib - 8) * sc;
        }
    }
}

/* All rows of a linear: out[n][k] f32.  Same arithmetic as the row function above. */
ORC_API void orc_dequant_w4a16(const uint8_t *q, const uint8_t *s, int n, int k, int group,
                               int scale_bf16, float *out) {
    for (int r = 0; r < n; ++r) {
        orc_dequant_row_w4a16_split(q, s, (size_t)r, k, group, scale_bf16, out + (size_t)r * k);
    }
}

/* crates/core/src/marlin.rs:2-43  (returns 0 ok, -1 contract violation) */
ORC_API int orc_marlin_repack_q(const uint32_t *q, size_t qlen, int n, int k, uint32_t *out) {
    if (k % 16 != 0 || n % 64 != 0) {
        return -1;
    }
    int k8 = k / 8;
    if (qlen != (size_t)n * (size_t)k8) {
        return -1;
    }
    int kt_n = k / 16, nt_n = n / 64;
    static const int OFF[4] = {0, 1, 8, 9};
    static const int PACK[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    for (int kt = 0; kt < kt_n; ++kt) {
        for (int nt = 0; nt < nt_n; ++nt) {
            uint32_t *tile = out + ((size_t)kt * nt_n + nt) * 128;
            for (int tid = 0; tid < 32; ++tid) {
                int tc_col = tid / 4;
                int tc_row = (tid % 4) * 2;
                for (int warp = 0; warp < 4; ++warp) {
                    int cur_n = nt * 64 + warp * 16 + tc_col;
                    uint32_t vals[8];
                    for (int i = 0; i < 4; ++i) {
                        int kk = kt * 16 + tc_row + OFF[i];
                        vals[i] = (q[(size_t)cur_n * k8 + kk / 8] >> ((kk % 8) * 4)) & 0xFu;
                        vals[4 + i] =
                            (q[(size_t)(cur_n + 8) * k8 + kk / 8] >> ((kk % 8) * 4)) & 0xFu;
                    }
                    uint32_t res = 0;
                    for (int i = 0; i < 8; ++i) {
                        res |= vals[PACK[i]] << (i * 4);
                    }
                    tile[tid * 4 + warp] = res;
                }
            }
        }
    }
    return 0;
}

/* Inverse of the above; restates the `unrepack` helper of the reference's round-trip test,
 * crates/core/src/marlin.rs:75-105.  `q` must be zeroed by the caller. */
ORC_API int orc_marlin_unrepack_q(const uint32_t *packed, int n, int k, uint32_t *q) {
    if (k % 16 != 0 || n % 64 != 0) {
        return -1;
    }
    int k8 = k / 8;
    static const int OFF[4] = {0, 1, 8, 9};
    static const int PACK[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    for (int kt = 0; kt < k / 16; ++kt) {
        for (int nt = 0; nt < n / 64; ++nt) {
            const uint32_t *tile = packed + ((size_t)kt * (n / 64) + nt) * 128;
            for (int tid = 0; tid < 32; ++tid) {
                int tc_col = tid / 4;
                int tc_row = (tid % 4) * 2;
                for (int warp = 0; warp < 4; ++warp) {
                    int cur_n = nt * 64 + warp * 16 + tc_col;
                    uint32_t res = tile[tid * 4 + warp];
                    uint32_t vals[8];
                    for (int i = 0; i < 8; ++i) {
                        vals[PACK[i]] = (res >> (i * 4)) & 0xFu;
                    }
                    for (int i = 0; i < 4; ++i) {
                        int kk = kt * 16 + tc_row + OFF[i];
                        q[(size_t)cur_n * k8 + kk / 8] |= vals[i] << ((kk % 8) * 4);
                        q[(size_t)(cur_n + 8) * k8 + kk / 8] |= vals[4 + i] << ((kk % 8) * 4);
                    }
                }
            }
        }
    }
    return 0;
}

/* crates/core/src/marlin.rs:45-67 */
ORC_API int orc_marlin_permute_scales(const float *s, size_t slen, int n, int k, int gs,
                                      float *out) {
    if (n % 64 != 0 || k % gs != 0) {
        return -1;
    }
    int kg = k / gs;
    if (slen != (size_t)n * (size_t)kg) {
        return -1;
    }
    for (int g = 0; g < kg; ++g) {
        for (int chunk = 0; chunk < n / 64; ++chunk) {
            for (int p = 0; p < 64; ++p) {
                int src = p / 8 + 8 * (p % 8);
                out[(size_t)g * n + chunk * 64 + p] = s[(size_t)(chunk * 64 + src) * kg + g];
            }
        }
    }
    return 0;
}

/* crates/core/src/qwen35/stages/moe.rs:8-31 and crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:168-185.
 * softmax over all n (divide by the full sum), order by (p desc, index asc), keep k,
 * renormalise by the sum of the kept k (summed in kept order). */
ORC_API int orc_select_topk(const float *logits, int n, int k, int32_t *idx_out, float *w_out) {
    float mx = -INFINITY;
    for (int e = 0; e < n; ++e) {
        mx = fmaxf(mx, logits[e]);
    }
    float *p = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    float sum = 0.0f;
    for (int e = 0; e < n; ++e) {
        p[e] = expf(logits[e] - mx);
        sum += p[e];
    }
    for (int e = 0; e < n; ++e) {
        p[e] /= sum;
    }
    int kk = k < n ? k : n;
    unsigned char *used = (unsigned char *)calloc((size_t)(n > 0 ? n : 1), 1);
    for (int r = 0; r < kk; ++r) {
        int best = -1;
        for (int e = 0; e < n; ++e) {
            if (used[e]) {
                continue;
            }
            /* total_cmp order on non-NaN softmax outputs == ordinary > ; ties -> lower index */
            if (best < 0 || p[e] > p[best]) {
                best = e;
            }
        }
        used[best] = 1;
        idx_out[r] = best;
    }
    float wsum = 0.0f;
    for (int r = 0; r < kk; ++r) {
        wsum += p[idx_out[r]];
    }
    for (int r = 0; r < kk; ++r) {
        w_out[r] = p[idx_out[r]] / wsum;
    }
    free(used);
    free(p);
    return kk;
}

/* ---- whole-linear driver: rows split over threads, each output = one lane dot --------
 * Mirrors the reference's row-chunked CPU pool (crates/core/src/matmul/cpu.rs:18-24)
 * with the lane dot of crates/core/src/quant/lane.rs:32-40 as the per-output kernel and the
 * symmetric zero point 8 (crates/server/src/probes/w4a16/gates.rs:113). */
typedef struct {
    const uint32_t *q;
    const uint16_t *s;
    const uint16_t *x;
    float *out;
    int m, n, k, group, scale_bf16;
    int row0, row1;
} orc_job;

static void *orc_linear_worker(void *arg) {
    orc_job *j = (orc_job *)arg;
    int ng = j->k / j->group;
    int k8 = j->k / 8;
    float *sc = (float *)malloc(sizeof(float) * (size_t)ng);
    uint32_t *z8 = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)ng);
    for (int g = 0; g < ng; ++g) {
        z8[g] = 8;
    }
    for (int r = j->row0; r < j->row1; ++r) {
        const uint16_t *srow = j->s + (size_t)r * ng;
        for (int g = 0; g < ng; ++g) {
            sc[g] = j->scale_bf16 ? orc_bf16_to_f32(srow[g]) : orc_half_to_f32(srow[g]);
        }
        const uint32_t *qrow = j->q + (size_t)r * k8;
        for (int t = 0; t < j->m; ++t) {
            j->out[(size_t)t * j->n + r] = orc_dot_row_w4a16_lane_group(
                qrow, z8, sc, j->x + (size_t)t * j->k, j->k, j->group);
        }
    }
    free(sc);
    free(z8);
    return NULL;
}

/* out[m][n] f32 = lane-order dot of every (token, row) pair for rows [row0,row1).
 * Columns outside [row0,row1) are left untouched.  Returns 0 ok, -1 bad shape. */
ORC_API int orc_linear_lane_rows(const uint32_t *q, const uint16_t *s, const uint16_t *x,
                                 float *out, int m, int n, int k, int group, int scale_bf16,
                                 int row0, int row1, int nthreads) {
    if (group < 32 || group % 32 != 0 || k % group != 0 || m < 1 || row0 < 0 || row1 > n ||
        row0 > row1) {
        return -1;
    }
    if (nthreads < 1) {
        nthreads = 1;
    }
    int rows = row1 - row0;
    if (nthreads > rows) {
        nthreads = rows > 0 ? rows : 1;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
    orc_job *jobs = (orc_job *)malloc(sizeof(orc_job) * (size_t)nthreads);
    int per = (rows + nthreads - 1) / nthreads;
    int started = 0;
    for (int i = 1; i < nthreads; ++i) {
        int a = row0 + i * per;
        int b = a + per < row1 ? a + per : row1;
        if (a >= b) {
            break;
        }
        jobs[i] = (orc_job){q, s, x, out, m, n, k, group, scale_bf16, a, b};
        pthread_create(&th[started], NULL, orc_linear_worker, &jobs[i]);
        started++;
    }
    if (rows > 0) {
        /* the first chunk runs on the calling thread */
        jobs[0] = (orc_job){q,  s, x, out, m, n, k, group, scale_bf16, row0,
                            row0 + per < row1 ? row0 + per : row1};
        orc_linear_worker(&jobs[0]);
    }
    for (int i = 0; i < started; ++i) {
        pthread_join(th[i], NULL);
    }
    free(th);
    free(jobs);
    return 0;
}

ORC_API int orc_linear_lane(const uint32_t *q, const uint16_t *s, const uint16_t *x, float *out,
                            int m, int n, int k, int group, int scale_bf16, int nthreads) {
    return orc_linear_lane_rows(q, s, x, out, m, n, k, group, scale_bf16, 0, n, nthreads);
}

/* ---- int8 lm-head (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1472-1518, assets/head.cu:100-225) ----
 * Quantiser: per row of a bf16 [n][k] matrix, scale = absmax/127 (1 when the row is zero) and
 * q = round-half-away-from-zero(v / scale) clamped to [-127, 127] (Rust's f32::round), all in f32. */
ORC_API int orc_head_quant(const uint16_t *w_bf16, int n, int k, int8_t *q, float *scale) {
    if (n < 1 || k < 1) {
        return -1;
    }
    for (int r = 0; r < n; ++r) {
        const uint16_t *row = w_bf16 + (size_t)r * k;
        float amax = 0.0f;
        for (int i = 0; i < k; ++i) {
            float v = fabsf(orc_bf16_to_f32(row[i]));
            amax = v > amax ? v : amax;
        }
        float s = amax > 0.0f ? amax / 127.0f : 1.0f;
        scale[r] = s;
        for (int i = 0; i < k; ++i) {
            float v = roundf(orc_bf16_to_f32(row[i]) / s);
            v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);
            q[(size_t)r * k + i] = (int8_t)v;
        }
    }
    return 0;
}

/* GEMV in the order of w4a16_gemv_i8 / w4a16_gemv_i8_t (assets/head.cu:100-225, built with -fmad=false): 64 lanes,
 * lane l takes the 4-byte words l, l+64, ... of the row and adds its four products one after the other (separate
 * f32 multiply and add); the 64 lane sums are added in f64 as lanes (l, l+32), then offsets 16, 8, 4, 2, 1;
 * out = (float)sum * scale.  x is f32 [t][k], out f32 [t][n]. */
ORC_API int orc_head_gemv_i8(const int8_t *q, const float *scale, const float *x, float *out, int n, int k, int t) {
    if (n < 1 || k < 4 || k % 4 != 0 || t < 1) {
        return -1;
    }
    const int k4 = k / 4;
    for (int r = 0; r < t; ++r) {
        const float *xr = x + (size_t)r * k;
        for (int o = 0; o < n; ++o) {
            const int8_t *w = q + (size_t)o * k;
            double red[64];
            for (int l = 0; l < 64; ++l) {
                float acc = 0.0f;
                for (int i = l; i < k4; i += 64) {
                    acc += (float)w[4 * i] * xr[4 * i];
                    acc += (float)w[4 * i + 1] * xr[4 * i + 1];
                    acc += (float)w[4 * i + 2] * xr[4 * i + 2];
                    acc += (float)w[4 * i + 3] * xr[4 * i + 3];
                }
                red[l] = (double)acc;
            }
            for (int l = 0; l < 32; ++l) {
                red[l] += red[l + 32];
            }
            for (int off = 16; off >= 1; off >>= 1) {
                for (int l = 0; l < off; ++l) {
                    red[l] += red[l + off];
                }
            }
            out[(size_t)r * n + o] = (float)red[0] * scale[o];
        }
    }
    return 0;
}
