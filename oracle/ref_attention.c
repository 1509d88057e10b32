/*
 * Plain-C CPU oracle for the DirectKV decode-attention hot path.
 * TEST INFRASTRUCTURE ONLY: linked or loaded by tests, by the smoke check and by
 * the CPU-baseline leg of the benchmark, never by the product library.
 *
 * Parity status: pinned through tests that compare this file with the torch
 * oracle (oracle/directkv_oracle.py), which is itself checked against outputs
 * of the reference's own Python code stored under tests/golden/.
 *
 * Each function cites the reference file:line it restates (paths relative to
 * the reference project's root).  Build: see oracle/Makefile.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- bf16 <-> fp32 (round to nearest even, as __float2bfloat16) ---------- */
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void dkv_ref_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}

/*
 * The libc rand() input streams of the reference's kernel test.
 * tests/test_directkv_cpu_kv.cu:184-188: value = (rand()/RAND_MAX - 0.5) * mul,
 * where mul = 2*scale for the bf16 inputs (seeds 42..45, scale 0.1) and 0.2 for
 * the past K/V (seed 99, :252-254; K then V drawn from ONE stream, so pass
 * reseed = 0 for V).
 */
void dkv_ref_rand_stream(float* out, int64_t n, float mul, unsigned seed, int reseed) {
    if (reseed) srand(seed);
    for (int64_t i = 0; i < n; ++i) out[i] = ((float)rand() / (float)RAND_MAX - 0.5f) * mul;
}

/*
 * tests/test_directkv_cpu_kv.cu:148-179 for one (batch, head):
 * scores = Q K^T * scale; causal mask j > s_past + i -> -1e30; max-subtracted
 * softmax; O = P V.  Q [S_q, D], K/V [S_kv, D], all fp32 row-major.
 */
void dkv_ref_attention(float* O, const float* Q, const float* K, const float* V,
                       int S_q, int S_kv, int D, float scale, int is_causal, int s_past) {
    float* scores = (float*)malloc(sizeof(float) * (size_t)S_kv);
    for (int i = 0; i < S_q; ++i) {
        float maxv = -1e30f;
        for (int j = 0; j < S_kv; ++j) {
            float s = 0.f;
            for (int d = 0; d < D; ++d) s += Q[(size_t)i * D + d] * K[(size_t)j * D + d];
            s *= scale;
            if (is_causal && j > s_past + i) s = -1e30f;
            scores[j] = s;
            maxv = fmaxf(maxv, s);
        }
        float sumv = 0.f;
        for (int j = 0; j < S_kv; ++j) {
            scores[j] = expf(scores[j] - maxv);
            sumv += scores[j];
        }
        for (int j = 0; j < S_kv; ++j) scores[j] /= sumv;
        for (int d = 0; d < D; ++d) {
            float o = 0.f;
            for (int j = 0; j < S_kv; ++j) o += scores[j] * V[(size_t)j * D + d];
            O[(size_t)i * D + d] = o;
        }
    }
    free(scores);
}

/*
 * tests/test_directkv_cpu_kv.cu:372-385: Y[t, h, d] = sum_hh X[t, hh] * W[h, d, hh]
 * in fp32 over the full hidden size.  X [T, H], W [NH, D, H] bf16 bit patterns;
 * Y [T, NH, D] fp32.
 */
void dkv_ref_project(float* Y, const uint16_t* X, const uint16_t* W, int T, int NH, int D, int H) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < T; ++t)
        for (int hd = 0; hd < NH * D; ++hd) {
            const uint16_t* w = W + (size_t)hd * H;
            const uint16_t* x = X + (size_t)t * H;
            float s = 0.f;
            for (int hh = 0; hh < H; ++hh) s += bf16_to_f32(x[hh]) * bf16_to_f32(w[hh]);
            Y[(size_t)t * NH * D + hd] = s;
        }
}

/*
 * Decode attention of a ragged batch over a slot-indexed bf16 pool: the torch
 * path of directkv/directkv_backend.py:835-859 (gather k_buf[slots], expand KV
 * heads to Q heads, softmax(q k^T * scale) v with no mask) written as loops.
 * slot(t) = page_table[b, t / page_size] * page_size + t % page_size.
 * Q [B, NH_q, D] bf16, pools [n_slots, NH_kv, D] bf16, O [B, NH_q, D] fp32.
 * seq_lens[b] counts every token attended, all of them already in the pool.
 */
void dkv_ref_decode_paged(float* O, const uint16_t* Q, const uint16_t* Kp, const uint16_t* Vp,
                          const int32_t* page_table, int pt_stride, const int32_t* seq_lens,
                          int B, int NH_q, int NH_kv, int D, int page_size, float scale) {
    const int g = NH_q / NH_kv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b)
        for (int hq = 0; hq < NH_q; ++hq) {
            const int S = seq_lens[b];
            const int h = hq / g;
            float qf[512];
            for (int d = 0; d < D; ++d) qf[d] = bf16_to_f32(Q[((size_t)b * NH_q + hq) * D + d]);
            float* sc = (float*)malloc(sizeof(float) * (size_t)(S > 0 ? S : 1));
            float maxv = -1e30f;
            for (int t = 0; t < S; ++t) {
                int64_t slot = (int64_t)page_table[(size_t)b * pt_stride + t / page_size] * page_size + t % page_size;
                const uint16_t* k = Kp + ((size_t)slot * NH_kv + h) * D;
                float s = 0.f;
                for (int d = 0; d < D; ++d) s += qf[d] * bf16_to_f32(k[d]);
                s *= scale;
                sc[t] = s;
                maxv = fmaxf(maxv, s);
            }
            float acc[512];
            for (int d = 0; d < D; ++d) acc[d] = 0.f;
            float sumv = 0.f;
            for (int t = 0; t < S; ++t) {
                int64_t slot = (int64_t)page_table[(size_t)b * pt_stride + t / page_size] * page_size + t % page_size;
                const uint16_t* v = Vp + ((size_t)slot * NH_kv + h) * D;
                float p = expf(sc[t] - maxv);
                sumv += p;
                for (int d = 0; d < D; ++d) acc[d] += p * bf16_to_f32(v[d]);
            }
            for (int d = 0; d < D; ++d) O[((size_t)b * NH_q + hq) * D + d] = acc[d] / sumv;
            free(sc);
        }
}
