/*
 * CPU oracle for the block-sparse attention path of SF-BERT -- TEST INFRASTRUCTURE ONLY.
 * See sfb_oracle.h for the contract and the parity pins.  The shipped library never
 * calls into this file.
 */
#include "sfb_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void orc_set_num_threads(int n)
{
    if (n > 0) omp_set_num_threads(n);
}

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------ */
/* counter-based generator (splitmix64 finaliser)                                   */
uint64_t orc_hash64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

void orc_fill_normal(float *dst, size_t n, uint64_t seed, float stddev)
{
    const double two_pi = 6.283185307179586;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++) {
        uint64_t h = orc_hash64(seed * 0x100000001B3ull + (uint64_t)i);
        uint32_t a = (uint32_t)(h >> 32), b = (uint32_t)h;
        double u1 = ((double)a + 1.0) / 4294967296.0; /* (0,1] */
        double u2 = (double)b / 4294967296.0;         /* [0,1) */
        dst[i] = (float)(sqrt(-2.0 * log(u1)) * cos(two_pi * u2)) * stddev;
    }
}

/* ------------------------------------------------------------------------------ */
/* layouts                                                                          */
#define LAY(h, i, j) layout[((size_t)(h) * nb + (i)) * nb + (j)]

void orc_layout_full(uint8_t *layout, uint32_t heads, uint32_t nb, int causal)
{
    /* no_fusion_test.cu:55-63: keep i >= j; non-causal keeps everything */
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < nb; i++)
            for (uint32_t j = 0; j < nb; j++)
                LAY(h, i, j) = (uint8_t)(!causal || i >= j);
}

void orc_layout_fixed(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t stride, int causal)
{
    memset(layout, 0, (size_t)heads * nb * nb);
    for (uint32_t h = 0; h < heads; h++) {
        /* fixed_fusion_test.cu:58-75: summary column index per head = stride-(h+1) */
        int first = (int)stride - (int)(h + 1);
        for (uint32_t i = 0; i < nb; i++) {
            for (int j = first; j < (int)nb; j += (int)stride)
                if (j >= 0) LAY(h, i, j) = 1;
            /* fixed_fusion_test.cu:78-92: the row's own group of `stride` blocks */
            uint32_t g = i / stride;
            uint32_t right = (g + 1) * stride > nb ? nb : (g + 1) * stride;
            for (uint32_t j = g * stride; j < right; j++) LAY(h, i, j) = 1;
            /* fixed_fusion_test.cu:95-107: causal cut */
            if (causal)
                for (uint32_t j = i + 1; j < nb; j++) LAY(h, i, j) = 0;
        }
    }
}

void orc_layout_stride(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t band, uint32_t every, int causal)
{
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < nb; i++)
            for (uint32_t j = 0; j < nb; j++) {
                int keep = (j <= i && j + band > i) || (every && (j % every) == 0);
                if (causal && j > i) keep = 0;
                LAY(h, i, j) = (uint8_t)keep;
            }
}

void orc_layout_stride_sawtooth(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t chunks)
{
    /* stride_fusion_test.cu:57-70 */
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < nb; i++) {
            uint32_t offset = chunks ? i % chunks : 0;
            for (uint32_t j = 0; j < nb; j++)
                LAY(h, i, j) = (uint8_t)((j + offset >= i) && (j <= i));
        }
}

void orc_layout_local(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t left, uint32_t right)
{
    /* local_fusion_test.cu:54-66 with left=extra_diag, right=0 */
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < nb; i++)
            for (uint32_t j = 0; j < nb; j++)
                LAY(h, i, j) = (uint8_t)((j + left >= i) && (j <= i + right));
}

void orc_layout_bigbird(uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t window,
                        uint32_t g_first, uint32_t g_last, uint32_t nrand, uint64_t seed)
{
    if (nrand > nb) nrand = nb;
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t i = 0; i < nb; i++) {
            /* big_bird_fusion_test.cu:59-81: window, then dense first rows / columns
             * (here also the last g_last) */
            int row_global = (i < g_first) || (i + g_last >= nb);
            for (uint32_t j = 0; j < nb; j++) {
                uint32_t dist = i > j ? i - j : j - i;
                int col_global = (j < g_first) || (j + g_last >= nb);
                LAY(h, i, j) = (uint8_t)(dist <= window || row_global || col_global);
            }
            /* nrand distinct columns of this row: draw t retries with a bumped
             * counter until the column differs from the earlier draws */
            uint32_t drawn[64];
            uint32_t nd = 0;
            uint64_t ctr = 0;
            while (nd < nrand && nd < 64) {
                uint64_t key = (seed << 32) ^ ((uint64_t)h << 48) ^ ((uint64_t)i << 20) ^ ctr;
                uint32_t c = (uint32_t)(orc_hash64(key) % nb);
                ctr++;
                int dup = 0;
                for (uint32_t t = 0; t < nd; t++) dup |= (drawn[t] == c);
                if (dup) continue;
                drawn[nd++] = c;
                LAY(h, i, c) = 1;
            }
        }
}

/* ------------------------------------------------------------------------------ */
/* layout -> LUT                                                                    */
int orc_lut_count(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t *blocks)
{
    uint32_t first = 0;
    for (uint32_t h = 0; h < heads; h++) {
        uint32_t cnt = 0;
        for (size_t e = 0; e < (size_t)nb * nb; e++) cnt += layout[(size_t)h * nb * nb + e] != 0;
        if (h == 0) first = cnt;
        else if (cnt != first) return -1;
    }
    *blocks = first;
    return 0;
}

int orc_lut_build(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                  uint32_t *nt_lut, uint32_t *nn_lut, uint32_t *rblk_lut, uint32_t *nn_max)
{
    uint32_t maxc = 0;
    for (uint32_t h = 0; h < heads; h++) {
        uint32_t *nt = nt_lut + (size_t)h * blocks * 2;
        uint32_t *nn = nn_lut + (size_t)h * (nb + blocks) * 2;
        uint32_t *rb = rblk_lut ? rblk_lut + (size_t)h * blocks * 2 : NULL;
        memset(nn, 0, sizeof(uint32_t) * 2 * (nb + blocks));
        /* stride_fusion_test.cu:87-98: row-major scan, (x,y) = (row, column) */
        uint32_t count = 0;
        for (uint32_t i = 0; i < nb; i++)
            for (uint32_t j = 0; j < nb; j++)
                if (LAY(h, i, j)) {
                    if (count >= blocks) return -1;
                    nt[2 * count] = i;
                    nt[2 * count + 1] = j;
                    count++;
                }
        if (count != blocks) return -1;
        /* stride_fusion_test.cu:114-120: entries (block id, column), per-row counts */
        for (uint32_t k = 0; k < blocks; k++) {
            nn[2 * (nb + k)] = k;
            nn[2 * (nb + k) + 1] = nt[2 * k + 1];
            nn[2 * nt[2 * k] + 1]++;
        }
        /* stride_fusion_test.cu:122-128: offsets start at nb */
        nn[0] = nb;
        for (uint32_t i = 1; i < nb; i++) nn[2 * i] = nn[2 * (i - 1)] + nn[2 * (i - 1) + 1];
        /* stride_fusion_test.cu:130-134 */
        for (uint32_t i = 0; i < nb; i++)
            if (nn[2 * i + 1] > maxc) maxc = nn[2 * i + 1];
        /* stride_fusion_test.cu:215-223: (block id, row) in row order */
        if (rb) {
            uint32_t c = 0;
            for (uint32_t i = 0; i < nb; i++)
                for (uint32_t j = 0; j < nn[2 * i + 1]; j++) {
                    rb[2 * c] = c;
                    rb[2 * c + 1] = i;
                    c++;
                }
        }
    }
    if (nn_max) *nn_max = maxc;
    return 0;
}

/* The column-major twin of nn_lut that the backward matmuls walk (bst_sgemm_xn with TN_OP,
 * blocksparse.h:1005-1010).  The reference builds it for the dense causal layout only
 * (generate_tn_lut, ewops.h:675-701): header[c] = (offset, count) of block column c with the
 * offsets starting at nb, entries (block id in the row-major scan, row block) column by column,
 * rows ascending.  This is that rule for any layout. */
int orc_lut_build_tn(const uint8_t *layout, uint32_t heads, uint32_t nb, uint32_t blocks,
                     uint32_t *tn_lut, uint32_t *tn_max)
{
    uint32_t maxc = 0;
    for (uint32_t h = 0; h < heads; h++) {
        uint32_t *tn = tn_lut + (size_t)h * (nb + blocks) * 2;
        memset(tn, 0, sizeof(uint32_t) * 2 * (nb + blocks));
        uint32_t total = 0;
        for (uint32_t j = 0; j < nb; j++) {
            uint32_t cnt = 0;
            for (uint32_t i = 0; i < nb; i++) cnt += LAY(h, i, j) ? 1u : 0u;
            tn[2 * j] = nb + total;
            tn[2 * j + 1] = cnt;
            total += cnt;
            if (cnt > maxc) maxc = cnt;
        }
        if (total != blocks) return -1;
        uint32_t id = 0;
        uint32_t *fill = (uint32_t *)calloc(nb, sizeof(uint32_t));
        if (!fill) return -1;
        for (uint32_t i = 0; i < nb; i++)
            for (uint32_t j = 0; j < nb; j++)
                if (LAY(h, i, j)) {
                    const uint32_t at = tn[2 * j] + fill[j]++;
                    tn[2 * at] = id++;
                    tn[2 * at + 1] = i;
                }
        free(fill);
    }
    if (tn_max) *tn_max = maxc;
    return 0;
}

/* ------------------------------------------------------------------------------ */
/* element masks                                                                    */
static int keep_elem(int pred, uint32_t ctx, uint32_t bs, uint32_t bi, uint32_t bj, uint32_t r, uint32_t c)
{
    switch (pred) {
    case ORC_MASK_CAUSAL_DIAG: /* no_fusion_test.cu:126-141 */
        return bi != bj || r >= c;
    case ORC_MASK_CAUSAL_ALL:  /* stride_fusion_test.cu:149-160 */
        return r >= c;
    case ORC_MASK_LOCAL: {     /* local_fusion_test.cu:155-174 */
        uint32_t row = bi * bs + r, col = bj * bs + c;
        if (bi == bj && c > r) return 0;
        return !(col > row || col + ctx <= row);
    }
    default:
        return 1;
    }
}

static void put_word(void *base, size_t idx, uint32_t bs, uint64_t w)
{
    if (bs == 64) ((uint64_t *)base)[idx] = w;
    else if (bs == 32) ((uint32_t *)base)[idx] = (uint32_t)w;
    else if (bs == 16) ((uint16_t *)base)[idx] = (uint16_t)w;
    else ((uint8_t *)base)[idx] = (uint8_t)w;
}

static uint64_t get_word(const void *base, size_t idx, uint32_t bs)
{
    if (bs == 64) return ((const uint64_t *)base)[idx];
    if (bs == 32) return ((const uint32_t *)base)[idx];
    if (bs == 16) return ((const uint16_t *)base)[idx];
    return ((const uint8_t *)base)[idx];
}

void orc_mask_pack(const uint32_t *nt_lut, uint32_t heads, uint32_t blocks, uint32_t bs,
                   int pred, uint32_t ctx, void *mask_np, void *mask_t)
{
    for (uint32_t h = 0; h < heads; h++)
        for (uint32_t k = 0; k < blocks; k++) {
            uint32_t bi = nt_lut[((size_t)h * blocks + k) * 2];
            uint32_t bj = nt_lut[((size_t)h * blocks + k) * 2 + 1];
            for (uint32_t r = 0; r < bs; r++) {
                /* stride_fusion_test.cu:165-173: bit c of word r */
                uint64_t w = 0;
                for (uint32_t c = 0; c < bs; c++)
                    w |= (uint64_t)(keep_elem(pred, ctx, bs, bi, bj, r, c) != 0) << c;
                if (mask_np) put_word(mask_np, ((size_t)h * blocks + k) * bs + r, bs, w);
                /* stride_fusion_test.cu:175-179: transposed [r][k] */
                if (mask_t) put_word(mask_t, ((size_t)h * bs + r) * blocks + k, bs, w);
            }
        }
}

/* ------------------------------------------------------------------------------ */
/* bf16 storage rounding                                                            */
uint16_t orc_to_bhalf(float v)
{
    /* ew_op_gpu.h:241-253: exp = bits & 0xff800000 (sign and exponent);
     * f = fma.rz(exp, 2^-8, v) (adds half a bf16 ulp of the magnitude, rounds toward
     * zero, subnormals flushed); result = upper 16 bits. */
    uint32_t u;
    memcpy(&u, &v, 4);
    if ((u & 0x7f800000u) == 0) return (uint16_t)((u >> 16) & 0x8000u); /* ftz */
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)(u >> 16);   /* inf / nan */
    uint32_t eb = u & 0xff800000u;
    float e;
    memcpy(&e, &eb, 4);
    /* the sum is exact in double (both terms share the exponent); truncate toward zero */
    double s = (double)e * 0.00390625 + (double)v;
    float f = (float)s;
    if (fabs((double)f) > fabs(s)) f = nextafterf(f, 0.0f);
    memcpy(&u, &f, 4);
    return (uint16_t)(u >> 16);
}

float orc_from_bhalf(uint16_t v)
{
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ------------------------------------------------------------------------------ */
/* attention                                                                        */
void orc_attention(const float *q, const float *k, const float *v,
                   const uint32_t *nt_lut, const uint32_t *nn_lut, const void *mask_np,
                   uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d,
                   uint32_t blocks, uint32_t lut_heads, uint32_t mask_heads,
                   float scale, float eps, int round_s_bf16,
                   float *s_out, float *p_out, float *o_out)
{
    const size_t L = (size_t)nb * bs;
    const size_t HD = (size_t)H * d;
    const long long pairs = (long long)B * H;
    (void)nt_lut;

#pragma omp parallel
    {
        uint32_t maxrow = 0;
        for (uint32_t hl = 0; hl < (lut_heads > 1 ? lut_heads : 1); hl++)
            for (uint32_t i = 0; i < nb; i++) {
                uint32_t c = nn_lut[((size_t)hl * (nb + blocks) + i) * 2 + 1];
                if (c > maxrow) maxrow = c;
            }
        /* one row of scores / probabilities across the row's blocks */
        float *srow = (float *)malloc(sizeof(float) * (size_t)(maxrow ? maxrow : 1) * bs);
        float *prow = (float *)malloc(sizeof(float) * (size_t)(maxrow ? maxrow : 1) * bs);

#pragma omp for schedule(dynamic, 1) collapse(2)
        for (long long bh = 0; bh < pairs; bh++)
            for (uint32_t i = 0; i < nb; i++) {
                uint32_t b = (uint32_t)(bh / H), h = (uint32_t)(bh % H);
                const uint32_t *nn = nn_lut + (lut_heads > 1 ? (size_t)h * (nb + blocks) * 2 : 0);
                const size_t mhead = mask_heads > 1 ? (size_t)h * blocks * bs : 0;
                uint32_t off = nn[2 * i], cnt = nn[2 * i + 1];
                for (uint32_t r = 0; r < bs; r++) {
                    const float *qrow = q + ((size_t)b * L + (size_t)i * bs + r) * HD + (size_t)h * d;
                    /* scores: matmul.h:60-63, float accumulation over d in order */
                    for (uint32_t e = 0; e < cnt; e++) {
                        uint32_t col = nn[2 * (off + e) + 1];
                        for (uint32_t c = 0; c < bs; c++) {
                            const float *krow = k + ((size_t)b * L + (size_t)col * bs + c) * HD + (size_t)h * d;
                            float sum = 0;
                            for (uint32_t n = 0; n < d; n++) sum += qrow[n] * krow[n];
                            if (round_s_bf16) sum = orc_from_bhalf(orc_to_bhalf(sum));
                            srow[(size_t)e * bs + c] = sum;
                        }
                    }
                    /* ewops.h:70-79: max of the kept, unscaled scores */
                    float mx = -1000000.0f;
                    for (uint32_t e = 0; e < cnt; e++) {
                        uint32_t blk = nn[2 * (off + e)];
                        uint64_t w = mask_np ? get_word(mask_np, mhead + (size_t)blk * bs + r, bs) : ~0ull;
                        for (uint32_t c = 0; c < bs; c++)
                            if ((w >> c) & 1)
                                if (srow[(size_t)e * bs + c] > mx) mx = srow[(size_t)e * bs + c];
                    }
                    /* ewops.h:81-90: exp((x-max)*scale) in double, stored as float, float sum */
                    float sum_of_c = 0.0f;
                    for (uint32_t e = 0; e < cnt; e++) {
                        uint32_t blk = nn[2 * (off + e)];
                        uint64_t w = mask_np ? get_word(mask_np, mhead + (size_t)blk * bs + r, bs) : ~0ull;
                        for (uint32_t c = 0; c < bs; c++) {
                            float p = 0.0f;
                            if ((w >> c) & 1) {
                                p = (float)exp((double)((srow[(size_t)e * bs + c] - mx) * scale));
                                sum_of_c += p;
                            }
                            prow[(size_t)e * bs + c] = p;
                        }
                    }
                    /* ewops.h:92-95 */
                    float den = sum_of_c + eps;
                    for (uint32_t e = 0; e < cnt * bs; e++) prow[e] = den > 0.0f ? prow[e] / den : 0.0f;

                    for (uint32_t e = 0; e < cnt; e++) {
                        uint32_t blk = nn[2 * (off + e)];
                        size_t o = ((((size_t)b * H + h) * blocks + blk) * bs + r) * bs;
                        if (s_out) memcpy(s_out + o, srow + (size_t)e * bs, sizeof(float) * bs);
                        if (p_out) memcpy(p_out + o, prow + (size_t)e * bs, sizeof(float) * bs);
                    }
                    /* matmul.h:11-16: float accumulation over the keys in ascending order */
                    if (o_out) {
                        float *orow = o_out + ((size_t)b * L + (size_t)i * bs + r) * HD + (size_t)h * d;
                        for (uint32_t m = 0; m < d; m++) {
                            float sum = 0;
                            for (uint32_t e = 0; e < cnt; e++) {
                                uint32_t col = nn[2 * (off + e) + 1];
                                const float *vb = v + ((size_t)b * L + (size_t)col * bs) * HD + (size_t)h * d + m;
                                for (uint32_t c = 0; c < bs; c++) sum += prow[(size_t)e * bs + c] * vb[(size_t)c * HD];
                            }
                            orow[m] = sum;
                        }
                    }
                }
            }
        free(srow);
        free(prow);
    }
}

/* ------------------------------------------------------------------------------ */
void orc_bias_residual_layernorm(float *out, float *sum_out, float *mean, float *rstd,
                                 const float *x, const float *bias, const float *resid,
                                 const float *gain, const float *beta,
                                 uint32_t m, uint32_t hidden)
{
#pragma omp parallel
    {
        float *row = (float *)malloc(sizeof(float) * hidden);
#pragma omp for schedule(static)
        for (long long i = 0; i < (long long)m; i++) {
            double s = 0.0, s2 = 0.0;
            for (uint32_t j = 0; j < hidden; j++) {
                float t = x[(size_t)i * hidden + j];
                if (bias) t = t + bias[j];                          /* ewops.h:13-14  */
                if (resid) t = resid[(size_t)i * hidden + j] + t;   /* ewops.h:298-299 */
                row[j] = t;
                s += t;                                             /* layernorm.h:22 */
                s2 += (t * t);                                      /* layernorm.h:23: float product */
            }
            float mu = (float)(s / hidden);                         /* layernorm.h:26 */
            double ms = s2 / hidden;                                /* layernorm.h:28 */
            float rs = (float)(1.0f / (double)sqrt(ms - (mu * mu) + 1e-5)); /* layernorm.h:30 */
            if (mean) mean[i] = mu;
            if (rstd) rstd[i] = rs;
            for (uint32_t j = 0; j < hidden; j++) {
                if (sum_out) sum_out[(size_t)i * hidden + j] = row[j];
                out[(size_t)i * hidden + j] = ((row[j] - mu) * rs) * gain[j] + beta[j]; /* layernorm.h:34 */
            }
        }
        free(row);
    }
}

/* ------------------------------------------------------------------------------ */
void orc_bias_gelu(float *out, const float *x, const float *bias, uint32_t m, uint32_t n)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)m; i++)
        for (uint32_t j = 0; j < n; j++) {
            float a = x[(size_t)i * n + j];
            if (bias) a = a + bias[j];                 /* ewops.h:13-14 */
            float ex = (float)exp(-(1.702 * a));       /* ewops.h:37: double arithmetic, float result */
            float rcp = (float)(1.0 / (ex + 1.0));     /* ewops.h:38 */
            out[(size_t)i * n + j] = a * rcp;          /* ewops.h:40 */
        }
}

/* out = act(x . w + bias): matrixMulNNCPU (matmul.h:101-118: double accumulation over k in ascending order),
 * then bias (ewops.h:10-17) and, for act = 1, gelu (ewops.h:32-43) -- the projections of the encoder layer
 * (transformer_inference_part.cpp:213-234 makes them with cblas_sgemm).  x [m,k], w [k,n] row-major. */
void orc_linear(float *out, const float *x, const float *w, const float *bias, uint32_t m, uint32_t n, uint32_t k, int act)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)m; i++)
        for (uint32_t j = 0; j < n; j++) {
            double sum = 0;
            for (uint32_t t = 0; t < k; t++) sum += (double)x[(size_t)i * k + t] * (double)w[(size_t)t * n + j];
            out[(size_t)i * n + j] = (float)sum;
        }
    if (act == 1) orc_bias_gelu(out, out, bias, m, n);
    else if (bias) {
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < (long long)m; i++)
            for (uint32_t j = 0; j < n; j++) out[(size_t)i * n + j] = out[(size_t)i * n + j] + bias[j];
    }
}

/* out = act(x . wt^T + bias) with wt [n,k] row-major: matrixMulNTCPU (matmul.h:121-132: FLOAT accumulation over k
 * in ascending order -- unlike the NN product, which accumulates in double), the logits product over the tied
 * embedding table (transformer_inference_part.cpp:241). */
void orc_linear_nt(float *out, const float *x, const float *wt, const float *bias, uint32_t m, uint32_t n, uint32_t k, int act)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)m; i++)
        for (uint32_t j = 0; j < n; j++) {
            float sum = 0.f;
            for (uint32_t t = 0; t < k; t++) sum += x[(size_t)i * k + t] * wt[(size_t)j * k + t];
            out[(size_t)i * n + j] = sum;
        }
    if (act == 1) orc_bias_gelu(out, out, bias, m, n);
    else if (bias) {
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < (long long)m; i++)
            for (uint32_t j = 0; j < n; j++) out[(size_t)i * n + j] = out[(size_t)i * n + j] + bias[j];
    }
}

/* out[b,l,:] = table[ids[b,l],:] + pos[l,:]: embedding_lookup (embedding.h:5-12) then tensor_add_matrix
 * (ewops.h:276-282), the front of the encoder stack (transformer_inference_part.cpp:201-209, dropout off).
 * pos may be NULL.  An id outside [0, vocab) gives a row of zeros (the reference would read out of bounds). */
void orc_embedding(float *out, const float *table, const int32_t *ids, const float *pos, uint32_t batch, uint32_t seq_len,
                   uint32_t hidden, uint32_t vocab)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)batch * seq_len; i++) {
        const int32_t id = ids[i];
        const uint32_t l = (uint32_t)(i % seq_len);
        for (uint32_t j = 0; j < hidden; j++) {
            const float e = (id >= 0 && (uint32_t)id < vocab) ? table[(size_t)id * hidden + j] : 0.f;
            out[(size_t)i * hidden + j] = pos ? e + pos[(size_t)l * hidden + j] : e;
        }
    }
}

/* ------------------------------------------------------------------------------ */
/* element-sparse (CSR) attention: the alternative format the reference prototypes    */

/* one (batch, head) worth of generate_csr_full_mask (ewops.h:430-443): row i keeps the columns j <= i.
 * rowptr [L+1], colidx [L(L+1)/2]. */
void orc_csr_full_mask(int32_t *rowptr, int32_t *colidx, uint32_t L)
{
    uint32_t nnz = 0;
    rowptr[0] = 0;
    for (uint32_t i = 0; i < L; i++) {
        for (uint32_t j = 0; j <= i; j++) colidx[nnz++] = (int32_t)j;
        rowptr[i + 1] = (int32_t)nnz;
    }
}

/* the element pattern of a block layout (one head, uint8 [nb][nb]): every element of every kept block, columns
 * ascending.  rowptr [nb*bs+1], colidx [blocks*bs*bs].  Returns the number of nonzeros. */
uint32_t orc_csr_from_layout(const uint8_t *layout, uint32_t nb, uint32_t bs, int32_t *rowptr, int32_t *colidx)
{
    uint32_t nnz = 0;
    rowptr[0] = 0;
    for (uint32_t i = 0; i < nb * bs; i++) {
        const uint32_t bi = i / bs;
        for (uint32_t bj = 0; bj < nb; bj++)
            if (layout[(size_t)bi * nb + bj])
                for (uint32_t c = 0; c < bs; c++) colidx[nnz++] = (int32_t)(bj * bs + c);
        rowptr[i + 1] = (int32_t)nnz;
    }
    return nnz;
}

/* O[b,i,h,:] = sum over the columns j of row i of softmax_j(q_i . k_j) v_j with one CSR pattern for every (batch,
 * head).  The arithmetic is the dense CPU path's (matmul.h:53-78 scores with float accumulation over d, ewops.h:64-98
 * max of the unscaled kept scores, exp((x-max)*scale), divide by sum+1e-6, matmul.h:6-20 P.V over the kept keys in
 * ascending order); the reference's GPU prototype of this format (csr_sddmm / csr_softmax / csr_spmm and
 * fused_attention, cuda_kernels.h:976-1075) computes the same thing one thread per row, with a max that starts at
 * 1e-20 instead of -1e6.  q, k, v, o are [B,L,H,d]; rows without entries give zeros. */
void orc_csr_attention(const float *q, const float *k, const float *v, const int32_t *rowptr, const int32_t *colidx,
                       uint32_t B, uint32_t H, uint32_t L, uint32_t d, float scale, float *o)
{
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (uint32_t b = 0; b < B; b++)
        for (uint32_t h = 0; h < H; h++) {
            float *s = (float *)malloc(sizeof(float) * (L ? L : 1));
            for (uint32_t i = 0; i < L; i++) {
                const int32_t lo = rowptr[i], hi = rowptr[i + 1];
                const float *qi = q + (((size_t)b * L + i) * H + h) * d;
                float *oi = o + (((size_t)b * L + i) * H + h) * d;
                for (uint32_t x = 0; x < d; x++) oi[x] = 0.f;
                if (hi <= lo || !s) continue;
                float mx = -1000000.0f;
                for (int32_t e = lo; e < hi; e++) {
                    const float *kj = k + (((size_t)b * L + (uint32_t)colidx[e]) * H + h) * d;
                    float sum = 0.f;
                    for (uint32_t x = 0; x < d; x++) sum += qi[x] * kj[x];
                    s[e - lo] = sum;
                    if (sum > mx) mx = sum;
                }
                float tot = 0.f;
                for (int32_t e = lo; e < hi; e++) {
                    s[e - lo] = (float)exp((s[e - lo] - mx) * scale);
                    tot += s[e - lo];
                }
                for (int32_t e = lo; e < hi; e++) s[e - lo] /= (tot + 1e-6f);
                for (uint32_t x = 0; x < d; x++) {
                    float acc = 0.f;
                    for (int32_t e = lo; e < hi; e++)
                        acc += s[e - lo] * v[(((size_t)b * L + (uint32_t)colidx[e]) * H + h) * d + x];
                    oi[x] = acc;
                }
            }
            free(s);
        }
}

/* ------------------------------------------------------------------------------ */
void orc_magicu64(uint32_t d, uint32_t *magic, uint32_t *shift)
{
    /* blocksparse.h:1016-1043: smallest p with 2^p > nc*(d-1-(2^p-1)%d) */
    if (d == 1) { *magic = 1; *shift = 0; return; }
    if (d == 2) { *magic = 1; *shift = 1; return; }
    if (d == 4) { *magic = 1; *shift = 2; return; }
    if (d == 8) { *magic = 1; *shift = 3; return; }
    uint32_t nbits = d == 3 ? 65 : 63;
    uint64_t nmax = d == 3 ? 0xffffffffull : 0x7fffffffull;
    uint64_t d64 = d;
    uint64_t nc = ((nmax + 1ull) / d64) * d64 - 1ull;
    for (uint32_t p = 0; p < nbits && p < 64; p++) {
        uint64_t two_p = 1ull << p;
        uint64_t rem = d64 - 1ull - (two_p - 1ull) % d64;
        if (two_p > nc * rem) {
            uint32_t mg = (uint32_t)((two_p + rem) / d64);
            *magic = mg;
            *shift = mg == 1 ? p : p - 32;
            return;
        }
    }
    *magic = 0;
    *shift = 0;
}

/* ------------------------------------------------------------------------------ */
/* backward of the block-sparse path                                               */

/* dx = (dy - sum over the query row of dy*y) * y * scale on the concatenated blocks of every query
 * row (bst_masked_softmax_grad, blocksparse.h:1045-1157; CPU twin softmax_grad, ewops.h:103-122:
 * float accumulation over the keys in ascending order). */
void orc_softmax_grad(const float *dy, const float *y, const uint32_t *nn_lut,
                      uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t blocks,
                      uint32_t lut_heads, float scale, float *dx)
{
    const size_t blk = (size_t)bs * bs;
#pragma omp parallel for schedule(static) collapse(2)
    for (uint32_t b = 0; b < B; b++)
        for (uint32_t h = 0; h < H; h++) {
            const uint32_t *nn = nn_lut + (lut_heads > 1 ? (size_t)h * (nb + blocks) * 2 : 0);
            const size_t base = ((size_t)b * H + h) * blocks * blk;
            for (uint32_t i = 0; i < nb; i++) {
                const uint32_t off = nn[2 * i], cnt = nn[2 * i + 1];
                for (uint32_t r = 0; r < bs; r++) {
                    float sum = 0.f;
                    for (uint32_t e = 0; e < cnt; e++) {
                        const size_t at = base + (size_t)nn[2 * (off + e)] * blk + (size_t)r * bs;
                        for (uint32_t c = 0; c < bs; c++) sum += dy[at + c] * y[at + c];
                    }
                    for (uint32_t e = 0; e < cnt; e++) {
                        const size_t at = base + (size_t)nn[2 * (off + e)] * blk + (size_t)r * bs;
                        for (uint32_t c = 0; c < bs; c++) dx[at + c] = (dy[at + c] - sum) * y[at + c] * scale;
                    }
                }
            }
        }
}

/* C[b, rows of block COLUMN j, h, :] = sum over the blocks k of column j of A[b,h,k]^T . B[b, rows of
 * row(k), h, :]  (bst_sgemm_xn with TN_OP, blocksparse.h:1005-1010; CPU twin multiheadmatmulTN,
 * matmul.h:81-99: float accumulation over the query rows in ascending order).  a is
 * [B,H,blocks,bs,bs], b and c are [B,L,H,d]; columns without blocks give zeros. */
void orc_spmm_tn(const float *a, const float *bm, const uint32_t *tn_lut,
                 uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d, uint32_t blocks,
                 uint32_t lut_heads, float *c)
{
    const size_t blk = (size_t)bs * bs, L = (size_t)nb * bs;
#pragma omp parallel for schedule(static) collapse(2)
    for (uint32_t b = 0; b < B; b++)
        for (uint32_t h = 0; h < H; h++) {
            const uint32_t *tn = tn_lut + (lut_heads > 1 ? (size_t)h * (nb + blocks) * 2 : 0);
            for (uint32_t j = 0; j < nb; j++) {
                const uint32_t off = tn[2 * j], cnt = tn[2 * j + 1];
                for (uint32_t cc = 0; cc < bs; cc++)
                    for (uint32_t x = 0; x < d; x++) {
                        float sum = 0.f;
                        for (uint32_t e = 0; e < cnt; e++) {
                            const float *ab = a + (((size_t)b * H + h) * blocks + tn[2 * (off + e)]) * blk;
                            const size_t row0 = (size_t)tn[2 * (off + e) + 1] * bs;
                            for (uint32_t r = 0; r < bs; r++)
                                sum += ab[(size_t)r * bs + cc] * bm[(((size_t)b * L + row0 + r) * H + h) * d + x];
                        }
                        c[(((size_t)b * L + (size_t)j * bs + cc) * H + h) * d + x] = sum;
                    }
            }
        }
}

/* C[b, rows of block row i, h, :] = sum over the blocks k of row i of A[b,h,k] . B[b, rows of col(k), h, :]
 * (bst_sgemm_xn with NN_OP, blocksparse.h:996-1003; CPU twin multiheadmatmulNN, matmul.h:6-20). */
void orc_spmm_nn(const float *a, const float *bm, const uint32_t *nn_lut,
                 uint32_t B, uint32_t H, uint32_t nb, uint32_t bs, uint32_t d, uint32_t blocks,
                 uint32_t lut_heads, float *c)
{
    const size_t blk = (size_t)bs * bs, L = (size_t)nb * bs;
#pragma omp parallel for schedule(static) collapse(2)
    for (uint32_t b = 0; b < B; b++)
        for (uint32_t h = 0; h < H; h++) {
            const uint32_t *nn = nn_lut + (lut_heads > 1 ? (size_t)h * (nb + blocks) * 2 : 0);
            for (uint32_t i = 0; i < nb; i++) {
                const uint32_t off = nn[2 * i], cnt = nn[2 * i + 1];
                for (uint32_t r = 0; r < bs; r++)
                    for (uint32_t x = 0; x < d; x++) {
                        float sum = 0.f;
                        for (uint32_t e = 0; e < cnt; e++) {
                            const float *ab = a + (((size_t)b * H + h) * blocks + nn[2 * (off + e)]) * blk + (size_t)r * bs;
                            const size_t col0 = (size_t)nn[2 * (off + e) + 1] * bs;
                            for (uint32_t cc = 0; cc < bs; cc++)
                                sum += ab[cc] * bm[(((size_t)b * L + col0 + cc) * H + h) * d + x];
                        }
                        c[(((size_t)b * L + (size_t)i * bs + r) * H + h) * d + x] = sum;
                    }
            }
        }
}

