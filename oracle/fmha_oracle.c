/*
 * TEST INFRASTRUCTURE ONLY (see fmha_oracle.h): CPU restatement of the reference's MXFP8 attention forward path.
 * Each function names the reference lines it follows. Plain C + OpenMP; no part of the product calls into this file.
 */
#include "fmha_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define D 128

/* ------------------------------------------------------------------------------------------------ small numeric helpers */

/* tests/gpu/ref_host.cpp:26-33: e4m3 byte -> value; the two NaN encodings decode to 0. */
double oracle_e4m3_decode(uint8_t b) {
    const int s = (b >> 7) & 1, e = (b >> 3) & 0xF, m = b & 0x7;
    double v;
    if (e == 0xF && m == 0x7) v = 0.0;
    else if (e == 0) v = (m / 8.0) * ldexp(1.0, -6);
    else v = (1.0 + m / 8.0) * ldexp(1.0, e - 7);
    return s ? -v : v;
}

static float g_pos[127];
static int g_pos_ready = 0;
static void init_pos(void) {
    if (g_pos_ready) return;
    for (int i = 0; i < 127; ++i) g_pos[i] = (float)oracle_e4m3_decode((uint8_t)i);
    g_pos_ready = 1;
}

/* tests/gpu/ref_host.cpp:217-227: nearest e4m3, ties to the even byte, saturating at 448 (byte 126). */
uint8_t oracle_e4m3_encode(float x) {
    init_pos();
    const uint8_t sgn = x < 0 ? 0x80 : 0;
    const float a = fabsf(x);
    if (!(a < 448.0f)) return sgn | 126;
    /* largest index whose value is <= a */
    int lo = 0, hi_b = 127;
    while (hi_b - lo > 1) {
        const int mid = (lo + hi_b) / 2;
        if (g_pos[mid] <= a) lo = mid; else hi_b = mid;
    }
    const int hi = lo + 1 < 127 ? lo + 1 : lo;
    const float dl = a - g_pos[lo], dh = g_pos[hi] - a;
    const int pick = dh < dl ? hi : dl < dh ? lo : (lo % 2 == 0 ? lo : hi);
    return sgn | (uint8_t)pick;
}

float oracle_bf16_to_f32(uint16_t x) {
    uint32_t u = (uint32_t)x << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* round to nearest even (crates/amdgpu-tile/src/tileop.rs:232-236) */
uint16_t oracle_f32_to_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the number of OpenMP threads of the parallel loops below (a launcher may have exported OMP_NUM_THREADS=1); returns what is in force. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

size_t oracle_q_bytes(const oracle_shape* sh) { return (size_t)sh->B * sh->S * sh->H * D; }
size_t oracle_kv_bytes(const oracle_shape* sh) { return (size_t)sh->B * sh->SK * sh->HK * D; }
/* tests/gpu/ref_host.cpp:196-198: scale tensors plus zeroed slack of (256+256) / (512+128) rows of H*4 bytes */
size_t oracle_qs_bytes(const oracle_shape* sh) { return (size_t)sh->B * sh->S * sh->H * 4 + (size_t)(256 + 256) * sh->H * 4; }
size_t oracle_ks_bytes(const oracle_shape* sh) { return (size_t)sh->B * sh->SK * sh->HK * 4 + (size_t)(512 + 128) * sh->H * 4; }

/* ------------------------------------------------------------------------------------------------ generators */

typedef struct { uint64_t st; } xs64;
static uint64_t xs_next(xs64* g) { g->st ^= g->st << 13; g->st ^= g->st >> 7; g->st ^= g->st << 17; return g->st; }
static double xs_unif(xs64* g) { return (double)(xs_next(g) >> 11) * (1.0 / 9007199254740992.0); }
static double xs_gauss(xs64* g) {
    double u1 = xs_unif(g), u2 = xs_unif(g);
    if (u1 < 1e-300) u1 = 1e-300;
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
}

/* tests/gpu/ref_host.cpp:239-252 (quant_rows): per 32-element block E8M0 = floor(log2 amax) - 8 (+127, clamped 0..254), elements RNE */
static void quant_rows(xs64* g, uint8_t* dst, uint8_t* scales, long nrows, int heads, double mul) {
    double blk[32];
    for (long r = 0; r < nrows; ++r)
        for (int h = 0; h < heads; ++h)
            for (int bk = 0; bk < 4; ++bk) {
                double amax = 0;
                for (int i = 0; i < 32; ++i) { blk[i] = xs_gauss(g) * mul; amax = fmax(amax, fabs(blk[i])); }
                const int e = amax > 0 ? (int)floor(log2(amax)) - 8 : -127;
                int eb = e + 127; if (eb > 254) eb = 254; if (eb < 0) eb = 0;
                scales[((size_t)r * heads + h) * 4 + bk] = (uint8_t)eb;
                const double inv = ldexp(1.0, -(eb - 127));
                for (int i = 0; i < 32; ++i) dst[((size_t)r * heads + h) * D + 32 * bk + i] = oracle_e4m3_encode((float)(blk[i] * inv));
            }
}

/* The harness's Q / K quantisation rule (tests/gpu/ref_host.cpp:239-252) as a function of f32 inputs, every step in f32 with one rounding
 * (product with `mul`, maximum, power-of-two scaling, RNE saturating e4m3): the statement the device quantiser is checked against bit for
 * bit. For inputs whose product with `mul` is exact this is the harness's arithmetic. */
void oracle_quantize_rows(const float* x, long nrows, float mul, uint8_t* out, uint8_t* scales) {
    for (long r = 0; r < nrows; ++r)
        for (int bk = 0; bk < 4; ++bk) {
            float y[32], amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                volatile float prod = x[(size_t)r * D + 32 * bk + i] * mul;   /* volatile: no fused or extended-precision evaluation */
                y[i] = prod;
                amax = fmaxf(amax, fabsf(y[i]));
            }
            int e = -127;
            if (amax > 0.0f) { int ex; frexpf(amax, &ex); e = ex - 1 - 8; }   /* floor(log2 amax) - 8 */
            int eb = e + 127; if (eb > 254) eb = 254; if (eb < 0) eb = 0;
            scales[(size_t)r * 4 + bk] = (uint8_t)eb;
            for (int i = 0; i < 32; ++i) out[(size_t)r * D + 32 * bk + i] = oracle_e4m3_encode(ldexpf(y[i], 127 - eb));
        }
}

/* The harness's V rule (ref_host.cpp:253-258) in f32: descale = amax / 448 (1 for an all-zero tensor), elements e4m3(x / descale). */
void oracle_quantize_tensor(const float* x, size_t n, uint8_t* out, float* descale) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
    volatile float vd = amax > 0.0f ? amax / 448.0f : 1.0f;
    *descale = vd;
    for (size_t i = 0; i < n; ++i) { volatile float q = x[i] / vd; out[i] = oracle_e4m3_encode(q); }
}

/* The unquantised samples of the `normal` generator, rounded to f32 (Q with its softmax scale already folded in, as the harness draws
 * them): what a quantiser must turn into the generator's bytes. Same stream order as oracle_generate (Q rows, K rows, V flat). */
int oracle_generate_raw_normal(const oracle_shape* sh, float* q_raw, float* k_raw, float* v_raw) {
    const int B = sh->B, H = sh->H, HK = sh->HK, S = sh->S, SK = sh->SK;
    xs64 g = {0x9E3779B97F4A7C15ull};
    const double qmul = 1.4426950408889634 / sqrt((double)D);
    const size_t nq = (size_t)B * S * H * D, nk = (size_t)B * SK * HK * D;
    for (size_t i = 0; i < nq; ++i) q_raw[i] = (float)(xs_gauss(&g) * qmul);
    for (size_t i = 0; i < nk; ++i) k_raw[i] = (float)xs_gauss(&g);
    for (size_t i = 0; i < nk; ++i) v_raw[i] = (float)xs_gauss(&g);
    return 0;
}

static int generate_impl(int mode, const oracle_shape* sh, uint8_t* q, uint8_t* k, uint8_t* v, uint8_t* qs, uint8_t* ks, float* vdescale,
                         uint8_t* v_bs, uint8_t* vscale) {
    static const uint8_t palette[11] = {0x00, 0x20, 0x28, 0x30, 0x38, 0x3C, 0x40, 0xA0, 0xA8, 0xB0, 0xB8};
    const int B = sh->B, H = sh->H, HK = sh->HK, S = sh->S, SK = sh->SK;
    const size_t nq = oracle_q_bytes(sh), nk = oracle_kv_bytes(sh);
    /* tests/gpu/ref_host.cpp:183-207: the 32-bit LCG stream is always drawn first (palette data and E8M0 in 126..128) */
    uint32_t seed = 20260101u;
#define RND() (seed = seed * 1664525u + 1013904223u, (seed >> 16) & 0xFFu)
    for (size_t i = 0; i < nq; ++i) q[i] = palette[RND() % 11];
    for (size_t i = 0; i < nk; ++i) k[i] = palette[RND() % 11];
    for (size_t i = 0; i < nk; ++i) v[i] = palette[RND() % 11];
    memset(qs, 0, oracle_qs_bytes(sh));
    memset(ks, 0, oracle_ks_bytes(sh));
    for (size_t i = 0; i < (size_t)B * S * H * 4; ++i) qs[i] = (uint8_t)(126 + RND() % 3);
    for (size_t i = 0; i < (size_t)B * SK * HK * 4; ++i) ks[i] = (uint8_t)(126 + RND() % 3);
#undef RND
    *vdescale = 1.0f;
    if (mode == ORACLE_DATA_LCG) return 0;
    xs64 g = {0x9E3779B97F4A7C15ull};
    if (mode == ORACLE_DATA_UNIFORM) {   /* ref_host.cpp:232-236: any byte that is not a NaN encoding */
        uint8_t* bufs[3] = {q, k, v};
        const size_t ns[3] = {nq, nk, nk};
        for (int t = 0; t < 3; ++t)
            for (size_t i = 0; i < ns[t]; ++i) {
                uint8_t x;
                do { x = (uint8_t)(xs_next(&g) >> 56); } while ((x & 0x7F) == 0x7F);
                bufs[t][i] = x;
            }
        return 0;
    }
    if (mode != ORACLE_DATA_NORMAL) return -1;
    /* ref_host.cpp:237-259: Q rows (scaled by log2(e)/sqrt(128)), then K rows, then V flat with one f32 descale */
    const double qmul = 1.4426950408889634 / sqrt((double)D);
    quant_rows(&g, q, qs, (long)B * S, H, qmul);
    quant_rows(&g, k, ks, (long)B * SK, HK, 1.0);
    double* vv = (double*)malloc(nk * sizeof(double));
    if (!vv) return -2;
    double vmax = 0;
    for (size_t i = 0; i < nk; ++i) { vv[i] = xs_gauss(&g); vmax = fmax(vmax, fabs(vv[i])); }
    *vdescale = (float)(vmax / 448.0);
    for (size_t i = 0; i < nk; ++i) v[i] = oracle_e4m3_encode((float)(vv[i] / *vdescale));
    if (v_bs && vscale) {
        /* extension (not in the reference): the same V samples quantised per 32 keys per (kv head, column) with the Q/K block rule */
        const int nblk = (SK + 31) / 32;
        for (int b = 0; b < B; ++b)
            for (int kb = 0; kb < nblk; ++kb)
                for (int h = 0; h < HK; ++h)
                    for (int d = 0; d < D; ++d) {
                        double amax = 0;
                        const int t1 = (kb * 32 + 32 < SK) ? kb * 32 + 32 : SK;
                        for (int t = kb * 32; t < t1; ++t) amax = fmax(amax, fabs(vv[(((size_t)b * SK + t) * HK + h) * D + d]));
                        const int e = amax > 0 ? (int)floor(log2(amax)) - 8 : -127;
                        int eb = e + 127; if (eb > 254) eb = 254; if (eb < 0) eb = 0;
                        vscale[(((size_t)b * nblk + kb) * HK + h) * D + d] = (uint8_t)eb;
                        const double inv = ldexp(1.0, -(eb - 127));
                        for (int t = kb * 32; t < t1; ++t) {
                            const size_t idx = (((size_t)b * SK + t) * HK + h) * D + d;
                            v_bs[idx] = oracle_e4m3_encode((float)(vv[idx] * inv));
                        }
                    }
    }
    free(vv);
    return 0;
}

int oracle_generate(int mode, const oracle_shape* sh, uint8_t* q, uint8_t* k, uint8_t* v, uint8_t* qs, uint8_t* ks, float* vdescale) {
    return generate_impl(mode, sh, q, k, v, qs, ks, vdescale, NULL, NULL);
}

int oracle_generate_v_blockscaled(const oracle_shape* sh, uint8_t* v, uint8_t* vscale) {
    const size_t nq = oracle_q_bytes(sh), nk = oracle_kv_bytes(sh);
    uint8_t* q = (uint8_t*)malloc(nq);
    uint8_t* k = (uint8_t*)malloc(nk);
    uint8_t* v0 = (uint8_t*)malloc(nk);
    uint8_t* qs = (uint8_t*)malloc(oracle_qs_bytes(sh));
    uint8_t* ks = (uint8_t*)malloc(oracle_ks_bytes(sh));
    float vd;
    int rc = -2;
    if (q && k && v0 && qs && ks) rc = generate_impl(ORACLE_DATA_NORMAL, sh, q, k, v0, qs, ks, &vd, v, vscale);
    free(q); free(k); free(v0); free(qs); free(ks);
    return rc;
}

/* ------------------------------------------------------------------------------------------------ fp64 oracle */

/* tests/gpu/ref_host.cpp:438-471 (`check`), same operation order: dequantise, scores * ln 2, max-subtracted exp, normalise, * V descale. */
/* `row_list` (may be NULL = rows 0 .. rows-1, as `check` does) names the query rows to evaluate: ref slot i holds row row_list[i]. */
static int reference_impl(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                          float vdescale, const uint8_t* vscale, int rows, const int* row_list, int causal, double* ref) {
    const int B = sh->B, H = sh->H, HK = sh->HK, S = sh->S, SK_all = sh->SK, GQA = sh->H / sh->HK;
    const int rows_eff = row_list ? rows : (rows < S ? rows : S);
    if (row_list) for (int i = 0; i < rows; ++i) if (row_list[i] < 0 || row_list[i] >= S) return -3;
    const double cpu_scale = 0.6931471805599453;
    const int nblk = (SK_all + 31) / 32;
    double tab[256];
    for (int i = 0; i < 256; ++i) tab[i] = oracle_e4m3_decode((uint8_t)i);
#pragma omp parallel
    {
        double* sc = (double*)malloc((size_t)SK_all * sizeof(double));
        double qd[D];
#pragma omp for collapse(3) schedule(dynamic, 1)
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < H; ++h)
                for (int slot = 0; slot < rows_eff; ++slot) {
                    const int i = row_list ? row_list[slot] : slot;
                    const int hk = h / GQA;
                    /* the keys the row sees: all of them, or (causal, crates/amdgpu-stage/src/attention/attn3.rs:298-306) those below
                       min(i + SK - S + 1, SK) */
                    int SK = SK_all;
                    if (causal) { SK = i + SK_all - S + 1; if (SK > SK_all) SK = SK_all; if (SK < 0) SK = 0; }
                    for (int kk = 0; kk < D; ++kk)
                        qd[kk] = tab[q[(((size_t)b * S + i) * H + h) * D + kk]] * ldexp(1.0, (int)qs[(((size_t)b * S + i) * H + h) * 4 + kk / 32] - 127);
                    double mx = -1e300;
                    for (int t = 0; t < SK; ++t) {
                        const uint8_t* kr = k + (((size_t)b * SK_all + t) * HK + hk) * D;
                        const uint8_t* sr = ks + (((size_t)b * SK_all + t) * HK + hk) * 4;
                        double acc = 0.0;
                        for (int kk = 0; kk < D; ++kk) acc += qd[kk] * tab[kr[kk]] * ldexp(1.0, (int)sr[kk / 32] - 127);
                        sc[t] = acc * cpu_scale;
                        mx = fmax(mx, sc[t]);
                    }
                    double den = 0.0;
                    for (int t = 0; t < SK; ++t) { sc[t] = exp(sc[t] - mx); den += sc[t]; }
                    double* o = ref + (((size_t)b * H + h) * rows_eff + slot) * D;
                    for (int d = 0; d < D; ++d) {
                        double acc = 0.0;
                        if (vscale) {
                            for (int t = 0; t < SK; ++t)
                                acc += sc[t] / den * tab[v[(((size_t)b * SK_all + t) * HK + hk) * D + d]] *
                                       ldexp(1.0, (int)vscale[(((size_t)b * nblk + t / 32) * HK + hk) * D + d] - 127);
                        } else {
                            for (int t = 0; t < SK; ++t) acc += sc[t] / den * tab[v[(((size_t)b * SK_all + t) * HK + hk) * D + d]];
                            acc *= vdescale;
                        }
                        o[d] = acc;
                    }
                }
        free(sc);
    }
    return 0;
}

int oracle_reference(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                     float vdescale, const uint8_t* vscale, int rows, double* ref) {
    return reference_impl(sh, q, k, v, qs, ks, vdescale, vscale, rows, NULL, 0, ref);
}

int oracle_reference_causal(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                            float vdescale, int rows, double* ref) {
    return reference_impl(sh, q, k, v, qs, ks, vdescale, NULL, rows, NULL, 1, ref);
}

int oracle_reference_rows(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                          float vdescale, const uint8_t* vscale, const int* row_list, int nrows, int causal, double* ref) {
    if (!row_list || nrows < 1) return -3;
    return reference_impl(sh, q, k, v, qs, ks, vdescale, vscale, nrows, row_list, causal, ref);
}

/* tests/gpu/ref_host.cpp:463-469: err = |got - ref|; bad when !(err <= 0.05 + 0.05 |ref|) (NaN counts); worst, mean, max|ref| */
static int compare_impl(const oracle_shape* sh, const uint16_t* out, const double* ref, int rows, const int* row_list, oracle_stats* st) {
    const int B = sh->B, H = sh->H, S = sh->S;
    const int rows_eff = row_list ? rows : (rows < S ? rows : S);
    double worst = 0.0, sum_abs = 0.0, max_ref = 0.0;
    uint64_t bad = 0, cnt = 0;
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h)
            for (int slot = 0; slot < rows_eff; ++slot)
                for (int d = 0; d < D; ++d) {
                    const int i = row_list ? row_list[slot] : slot;
                    const double acc = ref[(((size_t)b * H + h) * rows_eff + slot) * D + d];
                    const double got = oracle_bf16_to_f32(out[(((size_t)b * S + i) * H + h) * D + d]);
                    const double err = fabs(got - acc);
                    if (err != err) worst = INFINITY; else worst = fmax(worst, err);
                    sum_abs += err;
                    max_ref = fmax(max_ref, fabs(acc));
                    ++cnt;
                    if (!(err <= 0.05 + 0.05 * fabs(acc))) ++bad;
                }
    st->checked = cnt; st->bad = bad; st->worst_err = worst; st->mean_err = cnt ? sum_abs / cnt : 0.0; st->max_ref = max_ref;
    return 0;
}

int oracle_compare(const oracle_shape* sh, const uint16_t* out, const double* ref, int rows, oracle_stats* st) {
    return compare_impl(sh, out, ref, rows, NULL, st);
}

int oracle_compare_rows(const oracle_shape* sh, const uint16_t* out, const double* ref, const int* row_list, int nrows, oracle_stats* st) {
    if (!row_list || nrows < 1) return -3;
    return compare_impl(sh, out, ref, nrows, row_list, st);
}

/* crates/amdgpu-graph/src/dispatch.rs:494-511 */
void oracle_dispatch(uint64_t b, uint64_t h, uint64_t s, uint64_t sk, int* path, uint32_t* splits) {
    const uint64_t blocks256 = ((s + 255) / 256) * h * b, ntiles = (sk + 127) / 128;
    const uint64_t sp = (ntiles >= 16 && blocks256 <= 64) ? 4 : (ntiles >= 32 && blocks256 <= 128) ? 2 : 0;
    if (sp > 0) {
        const uint64_t tps = (ntiles + sp - 1) / sp;
        if ((sp - 1) * tps < ntiles) { *path = 2; *splits = (uint32_t)sp; return; }
    }
    *path = blocks256 <= 64 ? 1 : 0;
    *splits = 0;
}

/* ------------------------------------------------------------------------------------------------ the reference kernels' recipe */

typedef struct {
    float thr, target, conv;
    int lut, lazy;
} recipe_t;

/* crates/amdgpu-tile/src/softmax.rs:26-30 (short copy: thr 120/512, target 131/512, conversion scale 1, LUT) and :88-100
 * (long copy: target s91 = 0x3e7df17e, thr s92 = 0x3e85d086, conversion scale 0.25, no LUT, lazy update); the copy is chosen
 * from the whole sequence's tile count (crates/amdgpu-stage/src/attention/state.rs:73-77). */
static recipe_t recipe_for(int ntiles_total) {
    recipe_t r;
    if (ntiles_total < 4) {
        r.thr = 120.0f / 512.0f; r.target = 131.0f / 512.0f; r.conv = 1.0f; r.lut = 1; r.lazy = 0;
    } else {
        const uint32_t s91 = 0x3e7df17eu, s92 = 0x3e85d086u;
        memcpy(&r.target, &s91, 4); memcpy(&r.thr, &s92, 4);
        r.conv = 0.25f; r.lut = 0; r.lazy = 1;
    }
    return r;
}

static float f16_round(float x) { return (float)(_Float16)x; }

/* crates/amdgpu-tile/src/reduce.rs:94-113 + docs/vendor-spec.md:271-281: u = round(65535 clamp(x,0,1)); optional mantissa LUT
 * subtract; the u16 read as bf16 bits; times the conversion scale; to e4m3 (round to nearest even, saturating). Returns the value of P. */
static float p_from_x(float x, const recipe_t* r) {
    static const int lut[8] = {0, 6, 9, 11, 11, 10, 7, 3};
    float c = x < 0.0f ? 0.0f : (x > 1.0f ? 1.0f : x);
    if (!(x == x)) c = 0.0f;
    uint32_t u = (uint32_t)rintf(65535.0f * c);
    if (r->lut) u = (u - (uint32_t)lut[(u >> 4) & 7]) & 0xFFFFu;
    const float bf = oracle_bf16_to_f32((uint16_t)u);
    return (float)oracle_e4m3_decode(oracle_e4m3_encode(r->conv * bf));
}

typedef struct {
    float b;        /* the reference, kept as two f16 words: b = 4 (hi + lo) (softmax.rs:130-150) */
    float l;        /* row sum of the quantised P */
    float o[D];
} row_state;

/* One query row over the key range [key_lo, key_hi): crates/amdgpu-tile/src/softmax.rs:111-255 (decide / decide_lazy),
 * crates/amdgpu-stage/src/attention/attn3.rs:391-480 (scores carry the reference; P V), reduce.rs:35-49 (key mask). */
static void recipe_row(const recipe_t* rc, const float* qd, const uint8_t* kbase, const uint8_t* ksbase, const uint8_t* vbase, size_t kv_row_stride,
                       size_t ks_row_stride, int key_lo, int key_hi, const double* tab, row_state* st) {
    float x[128];
    st->b = 64.0f;   /* bias words 0x4800 0x4800: b = 4 * (8 + 8) (softmax.rs:73-74) */
    st->l = 0.0f;
    for (int d = 0; d < D; ++d) st->o[d] = 0.0f;
    for (int t0 = key_lo; t0 < key_hi; t0 += 128) {
        const int nv = key_hi - t0 < 128 ? key_hi - t0 : 128;
        float m = -1.0e30f;
        for (int j = 0; j < nv; ++j) {
            const uint8_t* kr = kbase + (size_t)(t0 + j) * kv_row_stride;
            const uint8_t* sr = ksbase + (size_t)(t0 + j) * ks_row_stride;
            /* block-scaled MFMA: exact products per 32-element block, f32 accumulation over the four blocks; Q scale lowered by 2^-9 */
            float s = 0.0f;
            for (int bk = 0; bk < 4; ++bk) {
                double acc = 0.0;
                for (int i = 0; i < 32; ++i) acc += (double)qd[32 * bk + i] * tab[kr[32 * bk + i]];
                s += (float)(acc * ldexp(1.0, (int)sr[bk] - 127));
            }
            x[j] = s * (1.0f / 512.0f) + st->b;
            m = fmaxf(m, x[j]);
        }
        const int grow = rc->thr < m;
        if (grow) {   /* softmax.rs:130-150 / 207-227: new two-word reference, delta, rescale */
            const float b_new = st->b + (rc->target - m);
            const float q4 = b_new * 0.25f;
            const float hq = f16_round(q4);
            const float lq = f16_round(q4 - hq);
            const float b_q = (hq + lq) * 4.0f;
            const float delta = b_q - st->b;
            st->b = b_q;
            for (int j = 0; j < nv; ++j) x[j] += delta;
            const float corr = exp2f(delta * 512.0f);
            for (int d = 0; d < D; ++d) st->o[d] *= corr;
            st->l *= corr;
        }
        for (int j = 0; j < nv; ++j) {
            const float pj = p_from_x(x[j], rc);
            st->l += pj;
            if (pj != 0.0f) {
                const uint8_t* vr = vbase + (size_t)(t0 + j) * kv_row_stride;
                for (int d = 0; d < D; ++d) st->o[d] += pj * (float)tab[vr[d]];
            }
        }
    }
}

static int recipe_impl(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                       float vdescale, int splits, int rows, const int* row_list, uint16_t* out) {
    const int B = sh->B, H = sh->H, HK = sh->HK, S = sh->S, SK = sh->SK, GQA = sh->H / sh->HK;
    const int rows_eff = row_list ? rows : (rows < S ? rows : S);
    if (row_list) for (int i = 0; i < rows; ++i) if (row_list[i] < 0 || row_list[i] >= S) return -3;
    const int ntiles = (SK + 127) / 128;
    const recipe_t rc = recipe_for(ntiles);
    const int nsp = splits > 1 ? splits : 1;
    const int tps = (ntiles + nsp - 1) / nsp;
    if ((nsp - 1) * tps >= ntiles) return -1;   /* every split must own a tile (tests/gpu/ref_host.cpp:117-120) */
    double tab[256];
    for (int i = 0; i < 256; ++i) tab[i] = oracle_e4m3_decode((uint8_t)i);
#pragma omp parallel for collapse(3) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h)
            for (int slot = 0; slot < rows_eff; ++slot) {
                const int i = row_list ? row_list[slot] : slot;
                const int hk = h / GQA;
                float qd[D];
                for (int kk = 0; kk < D; ++kk) {   /* Q scale bytes - 9: scores come out in units of 1/512 (block3.rs:138-147); folded below */
                    qd[kk] = (float)(tab[q[(((size_t)b * S + i) * H + h) * D + kk]] * ldexp(1.0, (int)qs[(((size_t)b * S + i) * H + h) * 4 + kk / 32] - 127));
                }
                const uint8_t* kbase = k + ((size_t)b * SK * HK + hk) * D;
                const uint8_t* vbase = v + ((size_t)b * SK * HK + hk) * D;
                const uint8_t* ksbase = ks + ((size_t)b * SK * HK + hk) * 4;
                uint16_t* orow = out + (((size_t)b * S + i) * H + h) * D;
                row_state st;
                if (nsp == 1) {
                    recipe_row(&rc, qd, kbase, ksbase, vbase, (size_t)HK * D, (size_t)HK * 4, 0, SK, tab, &st);
                    const float fin = (1.0f / st.l) * vdescale;   /* state.rs:79-82 */
                    for (int d = 0; d < D; ++d) orow[d] = oracle_f32_to_bf16(st.o[d] * fin);
                } else {
                    /* block3.rs:291-356 partial (fp16 Ohat, lse = log2 l - 512 b), then epilogue.rs:117-146 */
                    float m = -1.0e30f, den = 0.0f, acc[D];
                    for (int d = 0; d < D; ++d) acc[d] = 0.0f;
                    for (int sp = 0; sp < nsp; ++sp) {
                        const int lo = sp * tps * 128;
                        int hi = (sp + 1) * tps * 128;
                        if (hi > SK) hi = SK;
                        recipe_row(&rc, qd, kbase, ksbase, vbase, (size_t)HK * D, (size_t)HK * 4, lo, hi, tab, &st);
                        const float fin = (1.0f / st.l) * vdescale;
                        const float lse = log2f(st.l) - 512.0f * st.b;
                        const float mn = fmaxf(m, lse);
                        const float a = exp2f(m - mn), w = exp2f(lse - mn);
                        den = den * a + w;
                        for (int d = 0; d < D; ++d) acc[d] = acc[d] * a + w * f16_round(st.o[d] * fin);
                        m = mn;
                    }
                    const float rd = 1.0f / den;
                    for (int d = 0; d < D; ++d) orow[d] = oracle_f32_to_bf16(acc[d] * rd);
                }
            }
    return 0;
}

int oracle_recipe_forward(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                          float vdescale, int splits, int rows, uint16_t* out) {
    return recipe_impl(sh, q, k, v, qs, ks, vdescale, splits, rows, NULL, out);
}

int oracle_recipe_forward_rows(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                               float vdescale, int splits, const int* row_list, int nrows, uint16_t* out) {
    if (!row_list || nrows < 1) return -3;
    return recipe_impl(sh, q, k, v, qs, ks, vdescale, splits, nrows, row_list, out);
}

/* crates/amdgpu-tile/src/epilogue.rs:117-146 on f32 partials */
int oracle_combine_f32(const float* ohat, const float* lse2, uint32_t rows_total, uint32_t splits, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows_total; ++r) {
        float m = -1.0e30f, den = 0.0f, acc[D];
        for (int d = 0; d < D; ++d) acc[d] = 0.0f;
        for (uint32_t s = 0; s < splits; ++s) {
            const float ls = lse2[(size_t)s * rows_total + r];
            const float* o = ohat + ((size_t)s * rows_total + r) * D;
            const float mn = fmaxf(m, ls);
            const float a = exp2f(m - mn), w = exp2f(ls - mn);
            den = den * a + w;
            for (int d = 0; d < D; ++d) acc[d] = acc[d] * a + w * o[d];
            m = mn;
        }
        const float rd = 1.0f / den;
        for (int d = 0; d < D; ++d) out[(size_t)r * D + d] = oracle_f32_to_bf16(acc[d] * rd);
    }
    return 0;
}
