/*
 * TEST INFRASTRUCTURE ONLY. CPU restatement of the reference's MXFP8 attention forward path, used as the checker by tests/,
 * by __graft_entry__.smoke() and by bench.py's CPU-baseline legs. Nothing in the product (amdgpu_rustdsl_b200/) links, imports
 * or calls this code.
 *
 * Parity pin: the generators are bit-exact against the reference harness's own input dumps, and the fp64 oracle agrees with the
 * harness's `check` to its printed precision, both verified against the reference's tests/gpu/ref_host.cpp compiled from the
 * reference tree with a stub HIP runtime (oracle/Makefile, tests/test_oracle_pin.py, fixtures in tests/golden/).
 * The recipe path (`oracle_recipe_*`) restates gfx950 kernel arithmetic whose exact instruction rounding the reference does not
 * state; it is pinned statistically, against the per-shape mean errors the reference publishes (docs/perf-matrix.md:29-53).
 */
#ifndef FMHA_ORACLE_H
#define FMHA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_DATA_LCG = 0, ORACLE_DATA_UNIFORM = 1, ORACLE_DATA_NORMAL = 2 };

typedef struct oracle_shape {
    int B, H, HK, S, SK;
} oracle_shape;

/* Sizes in bytes of the generated buffers (tests/gpu/ref_host.cpp:187-198): q, k (= v), q scales and k scales with their slack. */
size_t oracle_q_bytes(const oracle_shape* sh);
size_t oracle_kv_bytes(const oracle_shape* sh);
size_t oracle_qs_bytes(const oracle_shape* sh);
size_t oracle_ks_bytes(const oracle_shape* sh);

/* e4m3 decode / encode as the reference harness does them (ref_host.cpp:26-33, 217-227). */
double oracle_e4m3_decode(uint8_t b);
uint8_t oracle_e4m3_encode(float x);

/* The harness's three input generators (ref_host.cpp:183-263): fills q, k, v (e4m3 bytes), qs, ks (E8M0 with slack) and *vdescale. */
/* The harness's quantisation rules as functions of f32 inputs (ref_host.cpp:239-258), and the generator's unquantised samples. */
void oracle_quantize_rows(const float* x, long nrows, float mul, uint8_t* out, uint8_t* scales);
void oracle_quantize_tensor(const float* x, size_t n, uint8_t* out, float* descale);
int oracle_generate_raw_normal(const oracle_shape* sh, float* q_raw, float* k_raw, float* v_raw);

int oracle_generate(int mode, const oracle_shape* sh, uint8_t* q, uint8_t* k, uint8_t* v, uint8_t* qs, uint8_t* ks, float* vdescale);

/*
 * Extension data (no reference counterpart): re-quantise V with one E8M0 per 32 keys per (head, column), same rule as the
 * Q/K blocks (floor(log2 amax) - 8, RNE saturating). Draws the same N(0,1) stream position as oracle_generate's V.
 * vscale layout [B][ceil(SK/32)][HK][128]; v is rewritten. Only for ORACLE_DATA_NORMAL.
 */
int oracle_generate_v_blockscaled(const oracle_shape* sh, uint8_t* v, uint8_t* vscale);

/*
 * The fp64 oracle on the dequantised inputs (ref_host.cpp:438-471, the `check` lambda) for the first `rows` query rows of every
 * (b, h): ref[((b*H + h)*rows_eff + i)*128 + d], rows_eff = min(rows, S). vscale may be NULL (reference behaviour).
 */
int oracle_reference(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                     float vdescale, const uint8_t* vscale, int rows, double* ref);

/* The same oracle with the causal mask of the reference's per-tensor sibling family (crates/amdgpu-stage/src/attention/attn3.rs:298-306):
 * row i sees the keys below min(i + SK - S + 1, SK). The reference's MXFP8 path has no mask; this checks the library's extension. */
int oracle_reference_causal(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                            float vdescale, int rows, double* ref);

/* The same oracle for an explicit list of query rows (the reference's `check` only ever looks at the first REF_ROWS rows; the list lets
 * the tests reach the query tiles behind the first). ref[((b*H + h)*nrows + i)*128 + d] belongs to row row_list[i]. `causal` as above. */
int oracle_reference_rows(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                          float vdescale, const uint8_t* vscale, const int* row_list, int nrows, int causal, double* ref);

typedef struct oracle_stats {
    uint64_t checked, bad;
    double worst_err, mean_err, max_ref;
} oracle_stats;

/* The gate statistics of `check` for a bf16 output tensor [B,S,H,128] against `ref` from oracle_reference. */
int oracle_compare(const oracle_shape* sh, const uint16_t* out_bf16, const double* ref, int rows, oracle_stats* st);

int oracle_compare_rows(const oracle_shape* sh, const uint16_t* out_bf16, const double* ref, const int* row_list, int nrows, oracle_stats* st);

/* Shape dispatch (crates/amdgpu-graph/src/dispatch.rs:494-511): path 0 = vs128, 1 = t128, 2 = kvsplit. */
void oracle_dispatch(uint64_t b, uint64_t h, uint64_t s, uint64_t sk, int* path, uint32_t* splits);

/*
 * CPU restatement of the reference kernels' arithmetic ("the reference path" of the accuracy gate), f32:
 * crates/amdgpu-tile/src/softmax.rs (reference shift + lazy rollback), reduce.rs:52-113 (pknorm -> e4m3 P, LUT),
 * attn3.rs:391-480 (scores in units of 1/512, P V), state.rs:73-82, block3.rs:291-300 (fp16 partials + lse),
 * epilogue.rs:89-167 (combine). splits = 0 runs the unsplit kernels, 2/4/8 the kvsplit + combine pair.
 * Computes the first `rows` query rows of every (b,h); out_bf16 is the full [B,S,H,128] tensor (other rows untouched).
 */
int oracle_recipe_forward(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                          float vdescale, int splits, int rows, uint16_t* out_bf16);

int oracle_recipe_forward_rows(const oracle_shape* sh, const uint8_t* q, const uint8_t* k, const uint8_t* v, const uint8_t* qs, const uint8_t* ks,
                               float vdescale, int splits, const int* row_list, int nrows, uint16_t* out_bf16);

/* CPU restatement of the combine kernel on f32 partials (epilogue.rs:117-146): out bf16 [rows_total][128]. */
int oracle_combine_f32(const float* ohat, const float* lse2, uint32_t rows_total, uint32_t splits, uint16_t* out_bf16);

float oracle_bf16_to_f32(uint16_t x);
uint16_t oracle_f32_to_bf16(float x);

int oracle_num_threads(void);
int oracle_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
