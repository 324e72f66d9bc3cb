/* C restatement of the reference's CPU algorithm for the SSM hot path -- TEST INFRASTRUCTURE and the
 * timed CPU baseline of bench.py; never part of the shipped library.  Parity unpinned: the reference
 * (Rust over an un-vendored Burn) cannot be executed where this was written and ships no golden
 * vectors; this file follows its formulas (file:line cited per function) and is checked against the
 * numpy oracle, which is checked against the reference's own invariants.
 *
 * float32 throughout, like the reference's backend-flex CPU path; pthreads over (batch x head), the
 * axis along which the problems are independent.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

int bm_oracle_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* Minimal parallel-for over [0, n): work items are independent (batch x head / batch x channel)
 * problems; items are handed out through an atomic counter (dynamic schedule). */
typedef void (*item_fn)(int item, void* ctx);
typedef struct { item_fn fn; void* ctx; int n; int next; pthread_mutex_t mu; } pf_state;
static void* pf_worker(void* arg) {
    pf_state* st = (pf_state*)arg;
    for (;;) {
        pthread_mutex_lock(&st->mu);
        int i = st->next++;
        pthread_mutex_unlock(&st->mu);
        if (i >= st->n) break;
        st->fn(i, st->ctx);
    }
    return NULL;
}
static void parallel_for(int n, item_fn fn, void* ctx, int nthreads) {
    if (nthreads <= 0) nthreads = bm_oracle_max_threads();
    if (nthreads > n) nthreads = n;
    pf_state st = {fn, ctx, n, 0, PTHREAD_MUTEX_INITIALIZER};
    if (nthreads <= 1) { pf_worker(&st); return; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * nthreads);
    for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, pf_worker, &st);
    for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
    free(th);
}

/* Serial chunked SSD, K1..K5 of src/mamba2/ssd/serial.rs:138-506, per (b, h):
 *   K1 cum = cumsum(dt*A); K2 CB = C.B^T; K3 S = X^T.(B*dt*exp(Aend-cum)); K4 h' = exp(Aend) h + S;
 *   K5 y = exp(cum) C.h + (CB * exp(cum_t-cum_s)[s<=t] * dt_s).X + D x.
 * x [b,s,h,p], dt [b,s,h], a [h], bm/cm [b,s,g,r], d [h], h0 [b,h,p,r] (may be NULL) -> y, hfinal.
 * seqlen must be a multiple of chunk_len. */
typedef struct {
    const float *x, *dt, *a, *bm, *cm, *d, *h0;
    float *y, *hfinal;
    int B, S, H, P, R, G, Q;
} ssd2_ctx;

static void ssd2_item(int item, void* vctx) {
    const ssd2_ctx* c = (const ssd2_ctx*)vctx;
    const int S = c->S, H = c->H, P = c->P, R = c->R, G = c->G, Q = c->Q, NC = S / Q;
    const int b = item / H, h = item % H, g = h / (H / G);
    float* cum = (float*)malloc(sizeof(float) * Q);
    float* cb = (float*)malloc(sizeof(float) * Q * Q);
    float* hst = (float*)malloc(sizeof(float) * P * R);
    float* snew = (float*)malloc(sizeof(float) * P * R);
    for (int i = 0; i < P * R; ++i) hst[i] = c->h0 ? c->h0[((size_t)b * H + h) * P * R + i] : 0.f;
    for (int n = 0; n < NC; ++n) {
        const size_t s0 = (size_t)n * Q;
        /* K1 */
        float run = 0.f;
        for (int l = 0; l < Q; ++l) {
            run += c->dt[((size_t)b * S + s0 + l) * H + h] * c->a[h];
            cum[l] = run;
        }
        const float aend = cum[Q - 1];
        /* K2 (K5 reads only the lower triangle) */
        for (int t = 0; t < Q; ++t) {
            const float* ct = c->cm + (((size_t)b * S + s0 + t) * G + g) * R;
            for (int s = 0; s <= t; ++s) {
                const float* bs = c->bm + (((size_t)b * S + s0 + s) * G + g) * R;
                float acc = 0.f;
                for (int r = 0; r < R; ++r) acc += ct[r] * bs[r];
                cb[t * Q + s] = acc;
            }
        }
        /* K5 with the state entering the chunk */
        for (int t = 0; t < Q; ++t) {
            const float* ct = c->cm + (((size_t)b * S + s0 + t) * G + g) * R;
            const float* xt = c->x + (((size_t)b * S + s0 + t) * H + h) * P;
            float* yt = c->y + (((size_t)b * S + s0 + t) * H + h) * P;
            const float et = expf(cum[t]);
            for (int p = 0; p < P; ++p) {
                float acc = 0.f;
                for (int r = 0; r < R; ++r) acc += ct[r] * hst[p * R + r];
                yt[p] = et * acc + c->d[h] * xt[p];
            }
            for (int s = 0; s <= t; ++s) {
                const float w = cb[t * Q + s] * expf(cum[t] - cum[s]) * c->dt[((size_t)b * S + s0 + s) * H + h];
                const float* xs = c->x + (((size_t)b * S + s0 + s) * H + h) * P;
                for (int p = 0; p < P; ++p) yt[p] += w * xs[p];
            }
        }
        /* K3 + K4 */
        memset(snew, 0, sizeof(float) * P * R);
        for (int l = 0; l < Q; ++l) {
            const float w = c->dt[((size_t)b * S + s0 + l) * H + h] * expf(aend - cum[l]);
            const float* bl = c->bm + (((size_t)b * S + s0 + l) * G + g) * R;
            const float* xl = c->x + (((size_t)b * S + s0 + l) * H + h) * P;
            for (int p = 0; p < P; ++p) {
                const float xw = xl[p] * w;
                for (int r = 0; r < R; ++r) snew[p * R + r] += xw * bl[r];
            }
        }
        const float ea = expf(aend);
        for (int i = 0; i < P * R; ++i) hst[i] = ea * hst[i] + snew[i];
    }
    memcpy(c->hfinal + ((size_t)b * H + h) * P * R, hst, sizeof(float) * P * R);
    free(cum); free(cb); free(hst); free(snew);
}

int bm_oracle_ssd2_serial(const float* x, const float* dt, const float* a, const float* bm, const float* cm,
                          const float* d, const float* h0, float* y, float* hfinal, int B, int S, int H, int P,
                          int R, int G, int Q, int nthreads) {
    if (S % Q != 0) return -1;
    ssd2_ctx c = {x, dt, a, bm, cm, d, h0, y, hfinal, B, S, H, P, R, G, Q};
    parallel_for(B * H, ssd2_item, &c, nthreads);
    return 0;
}

/* One-token Mamba-2 state update + readout (src/mamba2/mamba2.rs:935-991); state updated in place. */
typedef struct {
    float* state; const float *x, *dt, *a, *bm, *cm, *d; float* y; int B, H, P, R, G;
} step2_ctx;

static void step2_item(int item, void* vctx) {
    const step2_ctx* c = (const step2_ctx*)vctx;
    const int H = c->H, P = c->P, R = c->R, G = c->G;
    const int b = item / H, h = item % H, g = h / (H / G);
    const float dtv = c->dt[b * H + h], da = expf(dtv * c->a[h]);
    const float* bv = c->bm + ((size_t)b * G + g) * R;
    const float* cv = c->cm + ((size_t)b * G + g) * R;
    for (int p = 0; p < P; ++p) {
        float* st = c->state + (((size_t)b * H + h) * P + p) * R;
        const float xp = c->x[((size_t)b * H + h) * P + p];
        float acc = 0.f;
        for (int r = 0; r < R; ++r) {
            st[r] = st[r] * da + dtv * bv[r] * xp;
            acc += st[r] * cv[r];
        }
        c->y[((size_t)b * H + h) * P + p] = acc + c->d[h] * xp;
    }
}

void bm_oracle_step2(float* state, const float* x, const float* dt, const float* a, const float* bm,
                     const float* cm, const float* d, float* y, int B, int H, int P, int R, int G, int nthreads) {
    step2_ctx c = {state, x, dt, a, bm, cm, d, y, B, H, P, R, G};
    parallel_for(B * H, step2_item, &c, nthreads);
}

/* Mamba-1 sequential selective scan (src/mamba1/mamba1.rs:422-523), batch-major tensors. */
typedef struct {
    const float *u, *delta, *a, *bm, *cm, *d, *h0; float *y, *hfinal; int B, S, I, R;
} scan1_ctx;

static void scan1_item(int item, void* vctx) {
    const scan1_ctx* c = (const scan1_ctx*)vctx;
    const int S = c->S, I = c->I, R = c->R;
    const int b = item / I, i = item % I;
    float h[256];
    for (int r = 0; r < R; ++r) h[r] = c->h0 ? c->h0[((size_t)b * I + i) * R + r] : 0.f;
    for (int t = 0; t < S; ++t) {
        const size_t gi = ((size_t)b * S + t) * I + i;
        const float dl = c->delta[gi], uu = c->u[gi];
        const float* bv = c->bm + ((size_t)b * S + t) * R;
        const float* cv = c->cm + ((size_t)b * S + t) * R;
        float acc = 0.f;
        for (int r = 0; r < R; ++r) {
            h[r] = h[r] * expf(dl * c->a[(size_t)i * R + r]) + dl * bv[r] * uu;
            acc += h[r] * cv[r];
        }
        c->y[gi] = acc + c->d[i] * uu;
    }
    for (int r = 0; r < R; ++r) c->hfinal[((size_t)b * I + i) * R + r] = h[r];
}

void bm_oracle_selscan1(const float* u, const float* delta, const float* a, const float* bm, const float* cm,
                        const float* d, const float* h0, float* y, float* hfinal, int B, int S, int I, int R,
                        int nthreads) {
    scan1_ctx c = {u, delta, a, bm, cm, d, h0, y, hfinal, B, S, I, R};
    parallel_for(B * I, scan1_item, &c, nthreads);
}
