/*
 * CPU oracle for the gpt-oss-shaped MoE layer.  TEST INFRASTRUCTURE ONLY: the tests,
 * the smoke check and the benchmark's CPU-baseline leg may call it; the product path
 * (libneon_moe.so) never does.
 *
 * PARITY UNPINNED.  The nominal reference (NeonEngine: NeonEngine/src/main.cpp:16-18
 * picks one of three rendering apps; no MoE, router, MXFP4 or tensor code exists in
 * NeonEngine/src or NeonEngine/shaders) has no implementation, test, golden vector or
 * fixture of this path.  This file restates the layer math of the benchmark
 * configuration text:
 *
 *   logits[t,e] = sum_h x[t,h]*Wr[e,h] + br[e] (+ logit_bias[e])
 *   top-k largest logits, ties -> lower expert id; softmax over the k selected
 *   gu[r]  = sum_h x[h]*deq(Wgu[e,r,h]) + bgu[e,r]       rows interleaved: even = gate
 *   a[i]   = g*sigmoid(alpha*g)*(l+1),  g = min(gu[2i],limit), l = clamp(gu[2i+1],+-limit)
 *   y[c]   = sum_i a[i]*deq(Wd[e,c,i]) + bd[e,c]
 *   out[t] = sum_{s<k} w[t,s]*y_s                         fixed slot order
 *
 * Numerics: bf16 -> fp32 exact; e2m1 x 2^(scale-127) exact; all sums in fp64; nothing is
 * rounded between stages; outputs rounded once to fp32.  An optional mode quantises
 * activations to MXFP4 blocks (see oracle_quantize_mxfp4) to check a 4-bit-activation
 * tensor-core path against like-for-like math.
 *
 * It is pinned only against an independent numpy float64 restatement and hand-computed
 * known-answer cases (tests/golden).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16f(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* Dequantise one row of `cols` MXFP4 weights (cols/2 bytes, cols/32 scales) to fp32. */
static void dequant_row(const uint8_t* blk, const uint8_t* sc, int cols, float* out) {
    for (int b = 0; b < cols / 32; ++b) {
        float s = ldexpf(1.0f, (int)sc[b] - 127);
        for (int j = 0; j < 16; ++j) {
            uint8_t v = blk[b * 16 + j];
            out[b * 32 + 2 * j] = kE2M1[v & 15] * s;
            out[b * 32 + 2 * j + 1] = kE2M1[v >> 4] * s;
        }
    }
}

/* Router: logits (fp64 sum, rounded to fp32), top-k with lower-id tie-break, softmax.
 * idx[T,k] sorted by descending logit then ascending id; w[T,k]; logits_out[T,E] optional. */
void oracle_route(const uint16_t* x, const uint16_t* wr, const uint16_t* br, const float* logit_bias,
                  int T, int H, int E, int k, int32_t* idx, float* w, float* logits_out) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        float* lg = (float*)malloc(sizeof(float) * E);
        for (int e = 0; e < E; ++e) {
            double acc = 0.0;
            for (int h = 0; h < H; ++h) acc += (double)bf16f(x[(size_t)t * H + h]) * (double)bf16f(wr[(size_t)e * H + h]);
            acc += (double)bf16f(br[e]);
            if (logit_bias) acc += (double)logit_bias[e];
            lg[e] = (float)acc;
            if (logits_out) logits_out[(size_t)t * E + e] = lg[e];
        }
        char* used = (char*)calloc(E, 1);
        for (int s = 0; s < k; ++s) {
            int best = -1;
            for (int e = 0; e < E; ++e)
                if (!used[e] && (best < 0 || lg[e] > lg[best])) best = e; /* strict > keeps the lower id */
            used[best] = 1;
            idx[t * k + s] = best;
        }
        double m = lg[idx[t * k]], den = 0.0;
        for (int s = 0; s < k; ++s) den += exp((double)lg[idx[t * k + s]] - m);
        for (int s = 0; s < k; ++s) w[t * k + s] = (float)(exp((double)lg[idx[t * k + s]] - m) / den);
        free(used);
        free(lg);
    }
}

/* Dispatch: stable counting sort of the T*k (token, slot) entries by expert.
 * count[E], offset[E+1], perm[T*k] (sorted position -> entry id t*k+s), inv[T*k]. */
void oracle_dispatch(const int32_t* idx, int T, int k, int E, int32_t* count, int32_t* offset,
                     int32_t* perm, int32_t* inv) {
    int n = T * k;
    for (int e = 0; e < E; ++e) count[e] = 0;
    for (int i = 0; i < n; ++i) count[idx[i]]++;
    offset[0] = 0;
    for (int e = 0; e < E; ++e) offset[e + 1] = offset[e] + count[e];
    int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * E);
    for (int e = 0; e < E; ++e) cur[e] = offset[e];
    for (int i = 0; i < n; ++i) {
        int p = cur[idx[i]]++;
        perm[p] = i;
        inv[i] = p;
    }
    free(cur);
}

/* Quantise a vector of n (multiple of 32) values to MXFP4 in place: per block of 32 the
 * E8M0 scale is 2^(floor(log2(amax)) - 2) (so amax lands in [4, 8) -> clipped to 6), and
 * each value is rounded to the nearest e2m1 magnitude, ties to the even code. */
void oracle_quantize_mxfp4(double* v, int n) {
    static const double mags[8] = {0, 0.5, 1, 1.5, 2, 3, 4, 6};
    for (int b = 0; b < n / 32; ++b) {
        double amax = 0;
        for (int j = 0; j < 32; ++j) amax = fmax(amax, fabs(v[b * 32 + j]));
        if (amax == 0) continue;
        int e;
        frexp(amax, &e); /* amax = m*2^e, m in [0.5,1) -> floor(log2) = e-1 */
        double s = ldexp(1.0, (e - 1) - 2);
        for (int j = 0; j < 32; ++j) {
            double a = fabs(v[b * 32 + j]) / s;
            int best = 0;
            double bd = 1e300;
            for (int c = 0; c < 8; ++c) {
                double d = fabs(a - mags[c]);
                if (d < bd || (d == bd && (c & 1) == 0)) { bd = d; best = c; }
            }
            v[b * 32 + j] = copysign(mags[best] * s, v[b * 32 + j]);
        }
    }
}

/* Expert products + SwiGLU + weighted combine for the tokens listed in `tokens`
 * (n_sel token ids, or NULL = all T).  out[n_sel or T, H] fp32.  idx/w are the routing
 * of ALL T tokens.  Experts are global ids in [0,E); weights hold experts
 * [e_lo, e_lo+E_local) only and pairs routed elsewhere contribute nothing (expert-
 * parallel partial sums).  quant_act != 0 quantises x and a to MXFP4 first. */
void oracle_experts(const uint16_t* x, const int32_t* idx, const float* w, int T, int H, int I, int k,
                    int e_lo, int E_local,
                    const uint8_t* gub, const uint8_t* gus, const uint16_t* gubias,
                    const uint8_t* db, const uint8_t* ds, const uint16_t* dbias,
                    float limit, float alpha, const int32_t* tokens, int n_sel, int quant_act,
                    float* out) {
    int n_tok = tokens ? n_sel : T;
    /* per-slot contributions are summed in slot order afterwards: keep them apart */
    double* ys = (double*)calloc((size_t)n_tok * k * H, sizeof(double));
    for (int el = 0; el < E_local; ++el) {
        int e = e_lo + el;
        /* pairs (j, s) of the selected tokens routed to e */
        int np = 0;
        int* pj = (int*)malloc(sizeof(int) * n_tok * k);
        int* ps = (int*)malloc(sizeof(int) * n_tok * k);
        for (int j = 0; j < n_tok; ++j) {
            int t = tokens ? tokens[j] : j;
            for (int s = 0; s < k; ++s)
                if (idx[t * k + s] == e) { pj[np] = j; ps[np] = s; ++np; }
        }
        if (np == 0) { free(pj); free(ps); continue; }
        double* xin = (double*)malloc(sizeof(double) * (size_t)np * H);
        for (int p = 0; p < np; ++p) {
            int t = tokens ? tokens[pj[p]] : pj[p];
            for (int h = 0; h < H; ++h) xin[(size_t)p * H + h] = bf16f(x[(size_t)t * H + h]);
            if (quant_act) oracle_quantize_mxfp4(xin + (size_t)p * H, H);
        }
        double* gu = (double*)malloc(sizeof(double) * (size_t)np * 2 * I);
#pragma omp parallel
        {
            float* row = (float*)malloc(sizeof(float) * (H > I ? H : I));
#pragma omp for schedule(static)
            for (int r = 0; r < 2 * I; ++r) {
                dequant_row(gub + ((size_t)el * 2 * I + r) * (H / 2), gus + ((size_t)el * 2 * I + r) * (H / 32), H, row);
                double bias = bf16f(gubias[(size_t)el * 2 * I + r]);
                for (int p = 0; p < np; ++p) {
                    const double* xp = xin + (size_t)p * H;
                    double s = 0.0;
#pragma omp simd reduction(+ : s)
                    for (int h = 0; h < H; ++h) s += xp[h] * (double)row[h];
                    gu[(size_t)p * 2 * I + r] = s + bias;
                }
            }
            free(row);
        }
        double* a = (double*)malloc(sizeof(double) * (size_t)np * I);
        for (int p = 0; p < np; ++p) {
            for (int i = 0; i < I; ++i) {
                double g = gu[(size_t)p * 2 * I + 2 * i], l = gu[(size_t)p * 2 * I + 2 * i + 1];
                if (g > limit) g = limit;
                if (l > limit) l = limit;
                if (l < -limit) l = -limit;
                a[(size_t)p * I + i] = g / (1.0 + exp(-(double)alpha * g)) * (l + 1.0);
            }
            if (quant_act) oracle_quantize_mxfp4(a + (size_t)p * I, I);
        }
#pragma omp parallel
        {
            float* row = (float*)malloc(sizeof(float) * (H > I ? H : I));
#pragma omp for schedule(static)
            for (int c = 0; c < H; ++c) {
                dequant_row(db + ((size_t)el * H + c) * (I / 2), ds + ((size_t)el * H + c) * (I / 32), I, row);
                double bias = bf16f(dbias[(size_t)el * H + c]);
                for (int p = 0; p < np; ++p) {
                    const double* ap = a + (size_t)p * I;
                    double s = 0.0;
#pragma omp simd reduction(+ : s)
                    for (int i = 0; i < I; ++i) s += ap[i] * (double)row[i];
                    int t = tokens ? tokens[pj[p]] : pj[p];
                    ys[((size_t)pj[p] * k + ps[p]) * H + c] = (double)w[t * k + ps[p]] * (s + bias);
                }
            }
            free(row);
        }
        free(a); free(gu); free(xin); free(pj); free(ps);
    }
    for (int j = 0; j < n_tok; ++j)
        for (int c = 0; c < H; ++c) {
            double s = 0.0;
            for (int sl = 0; sl < k; ++sl) s += ys[((size_t)j * k + sl) * H + c];
            out[(size_t)j * H + c] = (float)s;
        }
    free(ys);
}

/* SwiGLU alone, for unit tests: a[n] from interleaved gu[2n]. */
void oracle_swiglu(const double* gu, int n, float limit, float alpha, double* a) {
    for (int i = 0; i < n; ++i) {
        double g = gu[2 * i], l = gu[2 * i + 1];
        if (g > limit) g = limit;
        if (l > limit) l = limit;
        if (l < -limit) l = -limit;
        a[i] = g / (1.0 + exp(-(double)alpha * g)) * (l + 1.0);
    }
}
