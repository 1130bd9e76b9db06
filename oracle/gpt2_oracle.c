/*
 * CPU oracle for the GPT-2 forward hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker that the CUDA kernels are compared against; it is
 * never linked into, loaded by, or called from the product library.  Only the
 * tests, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * PARITY PINNING: the reference project (GJ0407790/CUDA-GPT2-Inference) ships
 * no tests, golden vectors or CPU implementation.  This oracle is therefore a
 * restatement of the math in the reference's CUDA kernels, pinned against
 * outputs of those kernels themselves (built from the reference sources by
 * oracle/Makefile into oracle/_ref/ and run on a GPU; the recorded outputs are
 * the fixtures under tests/golden/).  Ops with no reference source
 * (encoder_forward, standalone gelu_forward, the gpt2_forward driver) are
 * "parity unpinned": they follow the definitions stated at each function.
 *
 * Every function cites the reference file:line whose math it restates.
 * Each op exists in two accumulation flavours selected by `precise`:
 *   precise = 0 : fp32 accumulation (the timed CPU baseline),
 *   precise = 1 : fp64 accumulation (the arbiter for tolerances).
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp, no -ffast-math).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Seeded, counter-based generators (identical bytes on every machine).      */
/* ------------------------------------------------------------------------- */

static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* uniform in (0,1], 24 bits */
static inline float u01(uint64_t bits) {
    return (float)((bits >> 40) + 1) * (1.0f / 16777216.0f);
}

/* dst[i] = mean + std * N(0,1); element i depends only on (seed, stream, i).
 * Box-Muller evaluated in double and rounded once, so the bytes do not depend
 * on the libm's float routines. */
ORACLE_API void oracle_fill_normal(float* dst, size_t n, uint64_t seed, uint64_t stream,
                                   float mean, float std) {
    const uint64_t key = splitmix64(seed ^ splitmix64(stream * 0xD6E8FEB86659FD93ull + 1));
#pragma omp parallel for schedule(static)
    for (ptrdiff_t p = 0; p < (ptrdiff_t)((n + 1) / 2); ++p) {
        uint64_t a = splitmix64(key + 2 * (uint64_t)p);
        uint64_t b = splitmix64(key + 2 * (uint64_t)p + 1);
        double u1 = (double)u01(a), u2 = (double)u01(b);
        double r = sqrt(-2.0 * log(u1));
        double th = 6.283185307179586476925 * u2;
        size_t i = 2 * (size_t)p;
        dst[i] = (float)((double)mean + (double)std * r * cos(th));
        if (i + 1 < n) dst[i + 1] = (float)((double)mean + (double)std * r * sin(th));
    }
}

/* token ids uniform in [0, vocab) */
ORACLE_API void oracle_fill_tokens(int32_t* dst, size_t n, uint64_t seed, int32_t vocab) {
    const uint64_t key = splitmix64(seed ^ 0x746F6B656E73ull);
    for (size_t i = 0; i < n; ++i) dst[i] = (int32_t)(splitmix64(key + i) % (uint64_t)vocab);
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP team size of every later call (a launcher may have exported
 * OMP_NUM_THREADS=1 before this library was loaded); returns the size in effect. */
ORACLE_API int oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* encoder_forward: out[b,t,:] = wte[tok[b,t],:] + wpe[t,:]                  */
/* The reference has no source for it (README.md:10 names the step; 0.4 ms in */
/* images/llmc/llmc_breakdown.png).  One fp32 add per element => bit-exact.  */
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_encoder_forward(float* out, const int32_t* inp, const float* wte,
                                       const float* wpe, int B, int T, int C) {
#pragma omp parallel for schedule(static)
    for (int bt = 0; bt < B * T; ++bt) {
        const float* e = wte + (size_t)inp[bt] * C;
        const float* p = wpe + (size_t)(bt % T) * C;
        float* o = out + (size_t)bt * C;
        for (int c = 0; c < C; ++c) o[c] = e[c] + p[c];
    }
}

/* ------------------------------------------------------------------------- */
/* gelu: kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:5-11                 */
/* 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3)))                               */
/* ------------------------------------------------------------------------- */
static inline float gelu_f32(float x) {
    const float k = 0.7978845608028654f; /* sqrt(2/pi) */
    float cube = 0.044715f * x * x * x;
    return 0.5f * x * (1.0f + tanhf(k * (x + cube)));
}
static inline double gelu_f64(double x) {
    const double k = 0.79788456080286535588;
    return 0.5 * x * (1.0 + tanh(k * (x + 0.044715 * x * x * x)));
}

ORACLE_API void oracle_gelu_forward(float* out, const float* inp, size_t N, int precise) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)N; ++i)
        out[i] = precise ? (float)gelu_f64((double)inp[i]) : gelu_f32(inp[i]);
}

/* ------------------------------------------------------------------------- */
/* residual: kernels/residual/1_residual_naive.cuh:9-12   out = inp1 + inp2  */
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_residual_forward(float* out, const float* inp1, const float* inp2, size_t N) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)N; ++i) out[i] = inp1[i] + inp2[i];
}

/* ------------------------------------------------------------------------- */
/* layernorm: kernels/layernorm/1_layernorm_block.cuh:32-60                  */
/*   m = sum(x)/C ; rstd = 1/sqrt(var + 1e-5), var biased ;                  */
/*   out = (x-m)*rstd*w + b ; also stores mean[row], rstd[row].              */
/* precise=0 follows the reference's single-pass form var = E[x^2]-m^2       */
/* (:45-46) in fp32; precise=1 is the two-pass variance in fp64.             */
/* ------------------------------------------------------------------------- */
static void layernorm_row(float* o, float* mean, float* rstd, const float* x, const float* w,
                          const float* b, int C, int precise) {
    if (precise) {
        double s = 0.0;
        for (int c = 0; c < C; ++c) s += x[c];
        double m = s / C, v = 0.0;
        for (int c = 0; c < C; ++c) { double d = x[c] - m; v += d * d; }
        double r = 1.0 / sqrt(v / C + 1e-5);
        for (int c = 0; c < C; ++c) o[c] = (float)((x[c] - m) * r * w[c] + b[c]);
        if (mean) *mean = (float)m;
        if (rstd) *rstd = (float)r;
    } else {
        float s = 0.f, ss = 0.f;
        for (int c = 0; c < C; ++c) { s += x[c]; ss += x[c] * x[c]; }
        float m = s / C;
        float r = 1.0f / sqrtf(ss / C - m * m + 1e-5f);
        for (int c = 0; c < C; ++c) o[c] = r * (x[c] - m) * w[c] + b[c];
        if (mean) *mean = m;
        if (rstd) *rstd = r;
    }
}

ORACLE_API void oracle_layernorm_forward(float* out, float* mean, float* rstd, const float* inp,
                                         const float* weight, const float* bias, int B, int T, int C,
                                         int precise) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < B * T; ++r)
        layernorm_row(out + (size_t)r * C, mean ? mean + r : NULL, rstd ? rstd + r : NULL,
                      inp + (size_t)r * C, weight, bias, C, precise);
}

/* fused residual + layernorm:
 * kernels/fused_residual_layernorm/fused_residual_layernorm.cuh:28-36 (res_out = inp1+inp2,
 * stored) and :59-81 (layernorm of res_out).  The reference kernel's float4 pointer stride
 * (:19,48-50) walks into the following rows; the oracle states the intended math. */
ORACLE_API void oracle_fused_residual_layernorm_forward(float* res_out, float* ln_out, float* mean,
                                                        float* rstd, const float* inp1,
                                                        const float* inp2, const float* weight,
                                                        const float* bias, int B, int T, int C,
                                                        int precise) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < B * T; ++r) {
        float* ro = res_out + (size_t)r * C;
        const float* a = inp1 + (size_t)r * C;
        const float* b2 = inp2 + (size_t)r * C;
        for (int c = 0; c < C; ++c) ro[c] = a[c] + b2[c];
        layernorm_row(ln_out + (size_t)r * C, mean ? mean + r : NULL, rstd ? rstd + r : NULL, ro,
                      weight, bias, C, precise);
    }
}

/* ------------------------------------------------------------------------- */
/* matmul: kernels/matmul/1_matmul_tiling.cuh:25-54                          */
/*   out[m,o] = bias[o] + sum_c inp[m,c]*weight[o,c]   (weight is [OC,C])    */
/* epilogue options of kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:196-212*/
/* (tanh-GELU) and a residual add (kernels/residual/1_residual_naive.cuh).   */
/* act: 0 none, 1 gelu.  residual: NULL or [M,OC], added after act.          */
/* ------------------------------------------------------------------------- */
typedef float v8f __attribute__((vector_size(32)));
typedef double v4d __attribute__((vector_size(32)));

static inline float hsum8(v8f v) {
    return ((v[0] + v[4]) + (v[1] + v[5])) + ((v[2] + v[6]) + (v[3] + v[7]));
}

/* 4 rows x 4 output columns, fp32 accumulate, 8 lanes along K */
static void mm_block_f32(float acc[4][4], const float* a, size_t lda, const float* w, size_t ldw,
                         int K, int mr, int nr) {
    v8f s[4][4];
    for (int i = 0; i < 4; ++i) for (int j = 0; j < 4; ++j) s[i][j] = (v8f){0, 0, 0, 0, 0, 0, 0, 0};
    const float* ap[4];
    const float* wp[4];
    for (int i = 0; i < 4; ++i) ap[i] = a + (size_t)(i < mr ? i : 0) * lda;
    for (int j = 0; j < 4; ++j) wp[j] = w + (size_t)(j < nr ? j : 0) * ldw;
    int k = 0;
    for (; k + 8 <= K; k += 8) {
        v8f av[4], wv[4];
        for (int i = 0; i < 4; ++i) memcpy(&av[i], ap[i] + k, 32);
        for (int j = 0; j < 4; ++j) memcpy(&wv[j], wp[j] + k, 32);
        for (int i = 0; i < 4; ++i) for (int j = 0; j < 4; ++j) s[i][j] += av[i] * wv[j];
    }
    for (int i = 0; i < 4; ++i) for (int j = 0; j < 4; ++j) {
        float t = hsum8(s[i][j]);
        for (int kk = k; kk < K; ++kk) t += ap[i][kk] * wp[j][kk];
        acc[i][j] = t;
    }
}

/* 2 rows x 4 columns, fp64 accumulate */
static void mm_block_f64(double acc[2][4], const float* a, size_t lda, const float* w, size_t ldw,
                         int K, int mr, int nr) {
    v4d s[2][4];
    for (int i = 0; i < 2; ++i) for (int j = 0; j < 4; ++j) s[i][j] = (v4d){0, 0, 0, 0};
    const float* ap[2];
    const float* wp[4];
    for (int i = 0; i < 2; ++i) ap[i] = a + (size_t)(i < mr ? i : 0) * lda;
    for (int j = 0; j < 4; ++j) wp[j] = w + (size_t)(j < nr ? j : 0) * ldw;
    int k = 0;
    for (; k + 4 <= K; k += 4) {
        v4d av[2], wv[4];
        for (int i = 0; i < 2; ++i) av[i] = (v4d){ap[i][k], ap[i][k + 1], ap[i][k + 2], ap[i][k + 3]};
        for (int j = 0; j < 4; ++j) wv[j] = (v4d){wp[j][k], wp[j][k + 1], wp[j][k + 2], wp[j][k + 3]};
        for (int i = 0; i < 2; ++i) for (int j = 0; j < 4; ++j) s[i][j] += av[i] * wv[j];
    }
    for (int i = 0; i < 2; ++i) for (int j = 0; j < 4; ++j) {
        double t = (s[i][j][0] + s[i][j][2]) + (s[i][j][1] + s[i][j][3]);
        for (int kk = k; kk < K; ++kk) t += (double)ap[i][kk] * (double)wp[j][kk];
        acc[i][j] = t;
    }
}

ORACLE_API void oracle_matmul_forward_ex(float* out, const float* inp, const float* weight,
                                         const float* bias, int B, int T, int C, int OC, int act,
                                         const float* residual, int precise) {
    const int M = B * T;
    const int MB = precise ? 2 : 4;
    const int n_mblk = (M + MB - 1) / MB;
    /* column panels keep a slab of the weight in cache while sweeping rows */
    const int NP = 64;
#pragma omp parallel for schedule(dynamic, 1) collapse(1)
    for (int np = 0; np < (OC + NP - 1) / NP; ++np) {
        const int n0 = np * NP, n1 = n0 + NP < OC ? n0 + NP : OC;
        for (int mb = 0; mb < n_mblk; ++mb) {
            const int m0 = mb * MB, mr = M - m0 < MB ? M - m0 : MB;
            for (int n = n0; n < n1; n += 4) {
                const int nr = n1 - n < 4 ? n1 - n : 4;
                double accd[4][4];
                if (precise) {
                    double a2[2][4];
                    mm_block_f64(a2, inp + (size_t)m0 * C, C, weight + (size_t)n * C, C, C, mr, nr);
                    for (int i = 0; i < 2; ++i) for (int j = 0; j < 4; ++j) accd[i][j] = a2[i][j];
                } else {
                    float a4[4][4];
                    mm_block_f32(a4, inp + (size_t)m0 * C, C, weight + (size_t)n * C, C, C, mr, nr);
                    for (int i = 0; i < 4; ++i) for (int j = 0; j < 4; ++j) accd[i][j] = a4[i][j];
                }
                for (int i = 0; i < mr; ++i) for (int j = 0; j < nr; ++j) {
                    size_t o = (size_t)(m0 + i) * OC + (n + j);
                    if (precise) {
                        double v = accd[i][j] + (bias ? (double)bias[n + j] : 0.0);
                        if (act == 1) v = gelu_f64(v);
                        if (residual) v += (double)residual[o];
                        out[o] = (float)v;
                    } else {
                        float v = (float)accd[i][j];
                        if (bias) v += bias[n + j];
                        if (act == 1) v = gelu_f32(v);
                        if (residual) v += residual[o];
                        out[o] = v;
                    }
                }
            }
        }
    }
}

/* reference-shaped signature: kernels/matmul/1_matmul_tiling.cuh:57-65 */
ORACLE_API void oracle_matmul_forward(float* out, const float* inp, const float* weight,
                                      const float* bias, int B, int T, int C, int OC) {
    oracle_matmul_forward_ex(out, inp, weight, bias, B, T, C, OC, 0, NULL, 0);
}

/* ------------------------------------------------------------------------- */
/* causal attention.                                                          */
/* Input packing inp[B,T,3,NH,HS]: kernels/attention/permute.cuh:10-28;       */
/* output [B,T,NH,HS]: permute.cuh:37-48, 3_flash_attention_permute.cuh:306;  */
/* math softmax(scale*q.k) over keys col<=row, scale=1/sqrt(HS):              */
/* kernels/attention/3_flash_attention_permute.cuh:149-153,216-221,342 and    */
/* 1_attention_cublas.cuh:50-61.  Direct (not blockwise) softmax, exact exp.  */
/* lse (nullable) receives log(sum_j exp(scale*q.k_j)) as [B,NH,T]; the       */
/* reference's flash kernels write no statistics (3_...cuh:349).              */
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_attention_forward(float* out, float* lse, const float* inp, int B, int T,
                                         int C, int NH, int precise) {
    const int HS = C / NH;
    const double scale_d = 1.0 / sqrt((double)HS);
    const float scale_f = 1.0f / sqrtf((float)HS);
#pragma omp parallel
    {
        double* sc = (double*)malloc(sizeof(double) * (size_t)T);
        double* acc = (double*)malloc(sizeof(double) * (size_t)HS);
#pragma omp for schedule(dynamic, 4) collapse(2)
        for (int bh = 0; bh < B * NH; ++bh) {
            for (int t = 0; t < T; ++t) {
                const int b = bh / NH, h = bh % NH;
                const float* q = inp + ((size_t)(b * T + t) * 3 * C) + h * HS;
                double mx = -INFINITY;
                for (int j = 0; j <= t; ++j) {
                    const float* k = inp + ((size_t)(b * T + j) * 3 * C) + C + h * HS;
                    if (precise) {
                        double s = 0.0;
                        for (int d = 0; d < HS; ++d) s += (double)q[d] * (double)k[d];
                        sc[j] = s * scale_d;
                    } else {
                        float s = 0.f;
                        for (int d = 0; d < HS; ++d) s += q[d] * k[d];
                        sc[j] = (double)(s * scale_f);
                    }
                    if (sc[j] > mx) mx = sc[j];
                }
                double l = 0.0;
                for (int d = 0; d < HS; ++d) acc[d] = 0.0;
                if (precise) {
                    for (int j = 0; j <= t; ++j) {
                        double p = exp(sc[j] - mx);
                        l += p;
                        const float* v = inp + ((size_t)(b * T + j) * 3 * C) + 2 * C + h * HS;
                        for (int d = 0; d < HS; ++d) acc[d] += p * (double)v[d];
                    }
                    float* o = out + ((size_t)(b * T + t) * C) + h * HS;
                    for (int d = 0; d < HS; ++d) o[d] = (float)(acc[d] / l);
                } else {
                    float lf = 0.f;
                    float accf[256];
                    for (int d = 0; d < HS; ++d) accf[d] = 0.f;
                    for (int j = 0; j <= t; ++j) {
                        float p = expf((float)sc[j] - (float)mx);
                        lf += p;
                        const float* v = inp + ((size_t)(b * T + j) * 3 * C) + 2 * C + h * HS;
                        for (int d = 0; d < HS; ++d) accf[d] += p * v[d];
                    }
                    float* o = out + ((size_t)(b * T + t) * C) + h * HS;
                    for (int d = 0; d < HS; ++d) o[d] = accf[d] / lf;
                    l = lf;
                }
                if (lse) lse[((size_t)b * NH + h) * T + t] = (float)(mx + log(l));
            }
        }
        free(sc);
        free(acc);
    }
}

/* ------------------------------------------------------------------------- */
/* gpt2_forward: operator order of images/gpt2/gpt2_flow.png, README.md:9-15, */
/* with every layernorm but the first fused with the preceding residual add   */
/* (README.md:255-256).  Parameters are one flat fp32 array holding 16        */
/* tensors, each stacked over layers, in this order:                          */
/*   wte[Vp,C] wpe[maxT,C] ln1w[L,C] ln1b[L,C] qkvw[L,3C,C] qkvb[L,3C]        */
/*   attprojw[L,C,C] attprojb[L,C] ln2w[L,C] ln2b[L,C] fcw[L,4C,C] fcb[L,4C]  */
/*   fcprojw[L,C,4C] fcprojb[L,C] lnfw[C] lnfb[C]                             */
/* The lm-head reuses wte as its [Vp,C] weight with no bias.                  */
/* logits: [B,T,Vp].                                                          */
/* ------------------------------------------------------------------------- */
typedef struct {
    int max_seq_len, vocab_size, padded_vocab_size, num_layers, num_heads, channels;
} oracle_gpt2_config;

ORACLE_API size_t oracle_gpt2_param_offsets(const oracle_gpt2_config* cfg, size_t offsets[17]) {
    const size_t C = cfg->channels, L = cfg->num_layers, Vp = cfg->padded_vocab_size,
                 maxT = cfg->max_seq_len;
    const size_t sizes[16] = {Vp * C, maxT * C, L * C, L * C, L * 3 * C * C, L * 3 * C,
                              L * C * C, L * C, L * C, L * C, L * 4 * C * C, L * 4 * C,
                              L * C * 4 * C, L * C, C, C};
    size_t o = 0;
    for (int i = 0; i < 16; ++i) { offsets[i] = o; o += sizes[i]; }
    offsets[16] = o;
    return o;
}

/* Seeded random-init parameters: matrices (incl. wte, wpe) N(0,0.02), layernorm
 * weight 1 / bias 0, linear biases 0.  Tensor i uses stream i of `seed`. */
ORACLE_API void oracle_gpt2_init_params(float* params, const oracle_gpt2_config* cfg, uint64_t seed) {
    size_t off[17];
    oracle_gpt2_param_offsets(cfg, off);
    for (int i = 0; i < 16; ++i) {
        float* p = params + off[i];
        size_t n = off[i + 1] - off[i];
        int is_ln_w = (i == 2 || i == 8 || i == 14);
        int is_zero = (i == 3 || i == 5 || i == 7 || i == 9 || i == 11 || i == 13 || i == 15);
        if (is_ln_w) for (size_t k = 0; k < n; ++k) p[k] = 1.0f;
        else if (is_zero) memset(p, 0, n * sizeof(float));
        else oracle_fill_normal(p, n, seed, (uint64_t)i, 0.0f, 0.02f);
    }
}

/* returns 0 on success, -1 on allocation failure */
ORACLE_API int oracle_gpt2_forward(float* logits, const float* params, const oracle_gpt2_config* cfg,
                                   const int32_t* tokens, int B, int T, int precise) {
    const int C = cfg->channels, L = cfg->num_layers, NH = cfg->num_heads,
              Vp = cfg->padded_vocab_size;
    const size_t M = (size_t)B * T;
    size_t off[17];
    oracle_gpt2_param_offsets(cfg, off);
    const float *wte = params + off[0], *wpe = params + off[1];
    float* buf = (float*)malloc(sizeof(float) * M * C * (size_t)(1 + 1 + 3 + 1 + 1 + 4));
    if (!buf) return -1;
    float* resid = buf;              /* [M,C]  residual stream            */
    float* lnout = resid + M * C;    /* [M,C]                             */
    float* qkv = lnout + M * C;      /* [M,3C]                            */
    float* atty = qkv + M * 3 * C;   /* [M,C]                             */
    float* branch = atty + M * C;    /* [M,C]  attn-proj / fc-proj output */
    float* fch = branch + M * C;     /* [M,4C] gelu(fc)                   */

    oracle_encoder_forward(resid, tokens, wte, wpe, B, T, C);
    oracle_layernorm_forward(lnout, NULL, NULL, resid, params + off[2], params + off[3], B, T, C, precise);
    for (int l = 0; l < L; ++l) {
        const float* qkvw = params + off[4] + (size_t)l * 3 * C * C;
        const float* qkvb = params + off[5] + (size_t)l * 3 * C;
        const float* apw = params + off[6] + (size_t)l * C * C;
        const float* apb = params + off[7] + (size_t)l * C;
        const float* ln2w = params + off[8] + (size_t)l * C;
        const float* ln2b = params + off[9] + (size_t)l * C;
        const float* fcw = params + off[10] + (size_t)l * 4 * C * C;
        const float* fcb = params + off[11] + (size_t)l * 4 * C;
        const float* fpw = params + off[12] + (size_t)l * C * 4 * C;
        const float* fpb = params + off[13] + (size_t)l * C;
        oracle_matmul_forward_ex(qkv, lnout, qkvw, qkvb, B, T, C, 3 * C, 0, NULL, precise);
        oracle_attention_forward(atty, NULL, qkv, B, T, C, NH, precise);
        oracle_matmul_forward_ex(branch, atty, apw, apb, B, T, C, C, 0, NULL, precise);
        oracle_fused_residual_layernorm_forward(resid, lnout, NULL, NULL, resid, branch, ln2w, ln2b,
                                                B, T, C, precise);
        oracle_matmul_forward_ex(fch, lnout, fcw, fcb, B, T, C, 4 * C, 1, NULL, precise);
        oracle_matmul_forward_ex(branch, fch, fpw, fpb, B, T, 4 * C, C, 0, NULL, precise);
        const float* nw = (l + 1 < L) ? params + off[2] + (size_t)(l + 1) * C : params + off[14];
        const float* nb = (l + 1 < L) ? params + off[3] + (size_t)(l + 1) * C : params + off[15];
        oracle_fused_residual_layernorm_forward(resid, lnout, NULL, NULL, resid, branch, nw, nb, B, T,
                                                C, precise);
    }
    oracle_matmul_forward_ex(logits, lnout, wte, NULL, B, T, C, Vp, 0, NULL, precise);
    free(buf);
    return 0;
}
