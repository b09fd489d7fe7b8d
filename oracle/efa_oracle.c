/* TEST INFRASTRUCTURE - not part of the product.
 *
 * CPU restatement (plain C, fp32 data, double accumulation) of the checker that
 * eager-flash-attention uses for its tensor-parallel attention block, and of its input recipe.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may call this file; the
 * library under test never does.
 *
 * What it follows, by file:line of eager-flash-attention:
 *   oracle_rand_fill       rand_fill                          attn_main.cu:88-96
 *   oracle_ref_inputs      allocate_and_fill + compute_qkv    attn_main.cu:98-153
 *   oracle_attention_rows  baseline_attention + softmax_rows  baseline_attention.cu:29-64, 82-143
 *   oracle_project_rows    reference() projection SGEMM       attn_tests.cu:41-48
 *   oracle_block_rows      reference() incl. the rank sum     attn_tests.cu:27-60
 *   oracle_compare         compare + the pass metric          attn_tests.cu:14-22, 135-137
 *
 * Parity pin: the reference ships no golden vectors; this file is pinned against outputs of the
 * reference's own GPU checker (baseline_attention + cuBLAS projection), dumped on a B200 by
 * oracle/ref_dump.cu and committed under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* scale * U(-1, 1) from the glibc rand() stream; the expression is the reference's, term by term. */
void oracle_rand_fill(float* dst, size_t n, float scale)
{
    for (size_t i = 0; i < n; i++)
        dst[i] = scale * (2.0f * (float)rand() / RAND_MAX - 1.0f);
}

/* Round-to-nearest-even fp32 -> fp16 bit pattern and back. */
uint16_t oracle_f32_to_f16(float x)
{
    _Float16 h = (_Float16)x;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

float oracle_f16_to_f32(uint16_t u)
{
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float)h;
}

void oracle_round_f16(const float* in, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = oracle_f32_to_f16(in[i]);
}

void oracle_widen_f16(const uint16_t* in, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = oracle_f16_to_f32(in[i]);
}

/* Inputs of rank `rank` of R: X seeded `seed` (same on all ranks), weights seeded seed*31+rank+1,
 * drawn in the order X, W_q, W_k, W_v, W_O with scales 1, 0.15, 0.15, 0.10, 0.05; then per local
 * head h: Q_h[S][d_h] = X[S][d] * W_q_h[d][d_h] (and K, V alike) in fp32.
 * Outputs: Q, K, V fp32 [H_local][S][d_h]; W_O fp32 [d_local][d]. */
int oracle_ref_inputs(int S, int d, int H, int R, int rank, int seed,
                      float* Q, float* K, float* V, float* W_O)
{
    if (R <= 0 || H % R != 0 || d % H != 0) return 1;
    const int H_local = H / R, d_h = d / H, d_local = H_local * d_h;
    const size_t wn = (size_t)H_local * d * d_h;
    float* X = (float*)malloc((size_t)S * d * sizeof(float));
    float* Wq = (float*)malloc(wn * sizeof(float));
    float* Wk = (float*)malloc(wn * sizeof(float));
    float* Wv = (float*)malloc(wn * sizeof(float));
    if (!X || !Wq || !Wk || !Wv) return 2;
    srand(seed);
    oracle_rand_fill(X, (size_t)S * d, 1.0f);
    srand(seed * 31 + rank + 1);
    oracle_rand_fill(Wq, wn, 0.15f);
    oracle_rand_fill(Wk, wn, 0.15f);
    oracle_rand_fill(Wv, wn, 0.10f);
    oracle_rand_fill(W_O, (size_t)d_local * d, 0.05f);
    for (int h = 0; h < H_local; h++) {
        const float* W3[3] = {Wq + (size_t)h * d * d_h, Wk + (size_t)h * d * d_h, Wv + (size_t)h * d * d_h};
        float* O3[3] = {Q + (size_t)h * S * d_h, K + (size_t)h * S * d_h, V + (size_t)h * S * d_h};
        for (int t = 0; t < 3; t++) {
            #pragma omp parallel for schedule(static)
            for (int s = 0; s < S; s++) {
                const float* x = X + (size_t)s * d;
                float* o = O3[t] + (size_t)s * d_h;
                for (int j = 0; j < d_h; j++) o[j] = 0.f;
                for (int k = 0; k < d; k++) {
                    const float xv = x[k];
                    const float* wr = W3[t] + (size_t)k * d_h;
                    for (int j = 0; j < d_h; j++) o[j] += xv * wr[j];
                }
            }
        }
    }
    free(X); free(Wq); free(Wk); free(Wv);
    return 0;
}

/* Full-softmax attention for selected query rows of every local head.
 * Q, K, V: fp32 [H_local][S][d_h]. rows: nrows absolute row indices (NULL = rows 0..nrows-1).
 * O: fp32 [nrows][H_local*d_h]. scores = (1/sqrt(d_h)) q.k; causal keeps keys 0..row; natural exp. */
void oracle_attention_rows(const float* Q, const float* K, const float* V,
                           int H_local, int S, int d_h, int causal,
                           const int* rows, int nrows, float* O)
{
    const int d_local = H_local * d_h;
    const float scale = 1.f / sqrtf((float)d_h);
    #pragma omp parallel
    {
        float* sc = (float*)malloc((size_t)S * sizeof(float));
        double* acc = (double*)malloc((size_t)d_h * sizeof(double));
        #pragma omp for schedule(dynamic, 4) collapse(2)
        for (int h = 0; h < H_local; h++) {
            for (int i = 0; i < nrows; i++) {
                const int r = rows ? rows[i] : i;
                const float* q = Q + ((size_t)h * S + r) * d_h;
                const float* Kh = K + (size_t)h * S * d_h;
                const float* Vh = V + (size_t)h * S * d_h;
                const int valid = causal ? r + 1 : S;
                float mx = -INFINITY;
                for (int j = 0; j < valid; j++) {
                    const float* k = Kh + (size_t)j * d_h;
                    double s = 0.0;
                    for (int c = 0; c < d_h; c++) s += (double)q[c] * (double)k[c];
                    sc[j] = (float)(s * (double)scale);
                    if (sc[j] > mx) mx = sc[j];
                }
                double sum = 0.0;
                for (int j = 0; j < valid; j++) sum += exp((double)(sc[j] - mx));
                for (int c = 0; c < d_h; c++) acc[c] = 0.0;
                for (int j = 0; j < valid; j++) {
                    const double p = exp((double)(sc[j] - mx)) / sum;
                    const float* v = Vh + (size_t)j * d_h;
                    for (int c = 0; c < d_h; c++) acc[c] += p * (double)v[c];
                }
                float* o = O + (size_t)i * d_local + (size_t)h * d_h;
                for (int c = 0; c < d_h; c++) o[c] = (float)acc[c];
            }
        }
        free(sc); free(acc);
    }
}

/* out[nrows][d] (+)= O[nrows][d_local] * W_O[d_local][d] */
void oracle_project_rows(const float* O, const float* W_O, int nrows, int d_local, int d,
                         int accumulate, float* out)
{
    #pragma omp parallel
    {
        double* acc = (double*)malloc((size_t)d * sizeof(double));
        #pragma omp for schedule(static)
        for (int i = 0; i < nrows; i++) {
            for (int j = 0; j < d; j++) acc[j] = 0.0;
            for (int k = 0; k < d_local; k++) {
                const double ov = (double)O[(size_t)i * d_local + k];
                const float* wr = W_O + (size_t)k * d;
                for (int j = 0; j < d; j++) acc[j] += ov * (double)wr[j];
            }
            float* o = out + (size_t)i * d;
            for (int j = 0; j < d; j++) o[j] = accumulate ? o[j] + (float)acc[j] : (float)acc[j];
        }
        free(acc);
    }
}

/* One rank's contribution to the block output for selected rows, added into out[nrows][d]:
 * attention over the rank's heads, projection with the rank's W_O slice. Calling it for every
 * rank with accumulate = 1 on a zeroed buffer is the reference's plain sum over ranks. */
int oracle_block_rows(const float* Q, const float* K, const float* V, const float* W_O,
                      int H_local, int S, int d_h, int d, int causal,
                      const int* rows, int nrows, int accumulate, float* out)
{
    const int d_local = H_local * d_h;
    float* O = (float*)malloc((size_t)nrows * d_local * sizeof(float));
    if (!O) return 2;
    oracle_attention_rows(Q, K, V, H_local, S, d_h, causal, rows, nrows, O);
    oracle_project_rows(O, W_O, nrows, d_local, d, accumulate, out);
    free(O);
    return 0;
}

/* max |a - ref| and max |ref|; the reference passes when max_abs / max_ref <= rtol and finite. */
void oracle_compare(const float* a, const float* ref, size_t n, float* max_abs, float* max_ref)
{
    float ma = 0.f, mr = 0.f;
    int bad = 0;
    for (size_t i = 0; i < n; i++) {
        const float dlt = fabsf(a[i] - ref[i]);
        if (!(dlt == dlt) || isinf(dlt)) bad = 1;
        if (dlt > ma) ma = dlt;
        if (fabsf(ref[i]) > mr) mr = fabsf(ref[i]);
    }
    *max_abs = bad ? INFINITY : ma;
    *max_ref = mr;
}
