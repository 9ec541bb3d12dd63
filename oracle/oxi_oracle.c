/*
 * CPU oracle for the pointer-table KV-cache path (TEST INFRASTRUCTURE ONLY).
 *
 * This file restates, in scalar C, the arithmetic of the reference's batched
 * kernels (crates/oxide-infer-kernels/src/batched_attn.rs, "BA" below) in the
 * same operation order, so that the CUDA library can be checked against it.
 * It is never linked into, imported by, or called from the product library;
 * only the tests, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Parity status: pinned.  The restatement is checked against (1) the known-
 * answer tests the reference holds for this path (uniform-softmax mean
 * position, sliding-window boundary, pat()-seeded attention vs. f64 within the
 * reference's own tolerances, the conv "zero state, unit weights" case) and
 * (2) outputs of the reference's own kernels executed on a B200, committed as
 * fixtures under tests/golden/.
 *
 * Approximate PTX instructions have no CPU equivalent; they are restated as
 * their correctly-rounded functions:
 *   div.approx.ftz(x, 128)  -> x / 128        (exact: power-of-two divisor)
 *   rsqrt.approx.ftz(x)     -> (float)(1/sqrt((double)x))
 *   ex2.approx.ftz(x)       -> exp2f(x), subnormal results flushed to zero
 *   rcp.approx.ftz(x)       -> 1.0f / x
 * so K (after RMSNorm+RoPE) may differ from the GPU by one f16 ulp on a small
 * fraction of elements; V bytes, conv state and conv output are bit-exact.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: every mul/add/fma below is a separate PTX
 * instruction in the reference and must not be fused or split.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NQ 16u
#define NKV 4u
#define HD 128u
#define KV_DIM 512u
#define ATTN_SCALE 0.0883883476f /* BA:1321 */
#define LOG2E 1.44269504f        /* BA:1328 */

/* ---------------------------------------------------------------- fp16 -- */

/* IEEE binary16 -> binary32 (what cvt.f32.f16 does; exact). */
float orc_h2f(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else { /* subnormal: renormalise */
            int sh = 0;
            while (!(m & 0x400u)) { m <<= 1; sh++; }
            m &= 0x3ffu;
            x = sign | ((uint32_t)(113 - sh) << 23) | (m << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* binary32 -> binary16, round-to-nearest-even, subnormals kept
 * (cvt.rn.f16.f32; the host side of the reference uses half::f16::from_f32,
 * same rounding). */
uint16_t orc_f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* >= 65520 rounds to inf */
    if (x < 0x38800000u) {                                   /* below 2^-14: half subnormal */
        if (x < 0x33000000u) return (uint16_t)sign;          /* <= 2^-25 rounds to zero */
        uint32_t e = x >> 23;
        uint32_t m = (x & 0x7fffffu) | 0x800000u;
        uint32_t sh = 126u - e; /* 14..24 */
        uint32_t hm = m >> sh;
        uint32_t rem = m & ((1u << sh) - 1u);
        uint32_t half = 1u << (sh - 1u);
        if (rem > half || (rem == half && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = x - 0x38000000u;
    uint32_t r = hm >> 13;
    uint32_t rem = hm & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

void orc_f2h_array(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = orc_f2h(in[i]);
}
void orc_h2f_array(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = orc_h2f(in[i]);
}

/* ------------------------------------------------- approximate functions -- */

static inline float ex2_ftz(float x) {
    float r = exp2f(x);
    if (r < 1.17549435e-38f) r = 0.0f;
    return r;
}
static inline float rcp_ftz(float x) { return 1.0f / x; }
static inline float rsqrt_ftz(float x) { return (float)(1.0 / sqrt((double)x)); }

/* shfl.sync.down tree 16,8,4,2,1 followed by reading lane 0 (BA:71-80,
 * BA:1310-1320).  A lane whose source is out of range keeps its own value;
 * only lane 0's result is used. */
static inline float warp_tree_sum_lane0(float p[32]) {
    for (int off = 16; off >= 1; off >>= 1) {
        float n[32];
        for (int i = 0; i < 32; i++) n[i] = p[i] + (i + off < 32 ? p[i + off] : p[i]);
        memcpy(p, n, sizeof(n));
    }
    return p[0];
}

/* ------------------------------------------------ deterministic inputs -- */

/* The generator every hot-path test binary of the reference uses
 * (crates/oxide-infer-server/src/bin/test_split_attention.rs:28-34). */
float orc_pat(uint64_t seed, uint64_t idx) {
    uint64_t x = seed * 6364136223846793005ull + idx;
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    return ((float)(x & 0xffffu) / 32767.5f) - 1.0f;
}
void orc_pat_fill(uint64_t seed, float scale, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = orc_pat(seed, i) * scale;
}

/* RoPE table rows (crates/oxide-infer-models/src/rope.rs:158-201): f16 cos/sin
 * [max_pos][head_dim]; inv_freq[i] = 1/theta^(2i/hd) for i < floor(partial*hd)/2,
 * else 0; the 64 angles are repeated for dims 64..127; all maths in f32. */
void orc_rope_table(uint16_t* cos_t, uint16_t* sin_t, uint32_t max_pos, uint32_t hd,
                    float theta, float partial) {
    uint32_t half = hd / 2;
    uint32_t angles = (uint32_t)(partial * (float)hd) / 2;
    float* inv = (float*)calloc(half, sizeof(float));
    for (uint32_t i = 0; i < angles && i < half; i++)
        inv[i] = 1.0f / powf(theta, (float)(2 * i) / (float)hd);
    for (uint32_t pos = 0; pos < max_pos; pos++) {
        for (uint32_t d = 0; d < hd; d++) {
            float a = (float)pos * inv[d % half];
            cos_t[(size_t)pos * hd + d] = orc_f2h(cosf(a));
            sin_t[(size_t)pos * hd + d] = orc_f2h(sinf(a));
        }
    }
    free(inv);
}

/* ------------------------------------------------- projections (lt.gemm) ---- */

/* y [rows][out] = f16( x [rows][in] * w [out][in]^T ), f32 accumulation in index order with fma: the
 * reference's projection GEMMs (lt.gemm(m = out, k = in, n = rows, W, x, y): cuBLASLt, f16 operands,
 * f32 compute, f16 output; lt_gemm.rs:828-900, launched at batch_engine.rs:914-926 and :1241-1245).
 * cuBLASLt does not specify its summation order, so a GPU GEMM agrees with this restatement to
 * about one f16 step of the output, not bit for bit. */
void orc_linear_f16(uint16_t* y, const uint16_t* x, const uint16_t* w, uint32_t rows, uint32_t out_features,
                    uint32_t in_features) {
#pragma omp parallel for schedule(static)
    for (int64_t ro = 0; ro < (int64_t)rows * out_features; ro++) {
        const uint16_t* xr = x + (size_t)(ro / out_features) * in_features;
        const uint16_t* wr = w + (size_t)(ro % out_features) * in_features;
        float a = 0.0f;
        for (uint32_t k = 0; k < in_features; k++) a = fmaf(orc_h2f(xr[k]), orc_h2f(wr[k]), a);
        y[ro] = orc_f2h(a);
    }
}

/* ------------------------------------------------------------ a1..a3 ---- */

/* batched_qk_rmsnorm_fp16, BA:13-118.  In place on x_io [B][heads][hd]. */
void orc_qk_rmsnorm(uint16_t* x_io, const uint16_t* w, float eps, uint32_t heads, uint32_t hd,
                    uint32_t batch) {
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t h = 0; h < heads; h++) {
            uint16_t* x = x_io + ((size_t)b * heads + h) * hd;
            float part[32];
            for (uint32_t lane = 0; lane < 32; lane++) {
                float s = 0.0f;
                for (uint32_t d = lane; d < hd; d += 32) {
                    float fx = orc_h2f(x[d]);
                    s = fmaf(fx, fx, s);
                }
                part[lane] = s;
            }
            float sum = warp_tree_sum_lane0(part);
            float mean = sum / (float)hd;
            mean = mean + eps;
            float r = rsqrt_ftz(mean);
            for (uint32_t d = 0; d < hd; d++) {
                float fx = orc_h2f(x[d]);
                float fw = orc_h2f(w[d]);
                fx = fx * r;
                fx = fx * fw;
                x[d] = orc_f2h(fx);
            }
        }
}

/* batched_rope_fp16, BA:128-219.  In place; rotate-half; table row pos_ids[b]. */
void orc_rope(uint16_t* x_io, const uint16_t* cos_t, const uint16_t* sin_t,
              const uint32_t* pos_ids, uint32_t heads, uint32_t hd, uint32_t batch) {
    uint32_t half = hd / 2;
    uint16_t tmp[512];
    for (uint32_t b = 0; b < batch; b++) {
        const uint16_t* c = cos_t + (size_t)pos_ids[b] * hd;
        const uint16_t* s = sin_t + (size_t)pos_ids[b] * hd;
        for (uint32_t h = 0; h < heads; h++) {
            uint16_t* x = x_io + ((size_t)b * heads + h) * hd;
            for (uint32_t d = 0; d < hd; d++) {
                float fx = orc_h2f(x[d]);
                float fo = d < half ? -orc_h2f(x[d + half]) : orc_h2f(x[d - half]);
                float res = fx * orc_h2f(c[d]);
                res = fmaf(fo, orc_h2f(s[d]), res);
                tmp[d] = orc_f2h(res);
            }
            memcpy(x, tmp, hd * 2);
        }
    }
}

/* batched_kv_copy_fp16, BA:233-287: dst_ptrs[b] + pos*kv_dim <- src[b]. */
void orc_kv_copy(const uint64_t* dst_ptrs, const uint16_t* src, const uint32_t* pos_ids,
                 uint32_t kv_dim, uint32_t batch) {
    for (uint32_t b = 0; b < batch; b++) {
        uint16_t* dst = (uint16_t*)(uintptr_t)dst_ptrs[b] + (size_t)pos_ids[b] * kv_dim;
        memcpy(dst, src + (size_t)b * kv_dim, (size_t)kv_dim * 2);
    }
}

/* ------------------------------------------------------------ a4..a7 ---- */

/* Per-warp key scan shared by the online, split and split4 kernels
 * (BA:1284-1352, BA:1495-1560, BA:2773-3007): lane l owns dims 4l..4l+3.
 * Updates (m, s, acc[128]) over keys [t0, t1). */
static void scan_keys(const uint16_t* q, const uint16_t* kbase, const uint16_t* vbase,
                      uint32_t kvh, uint32_t t0, uint32_t t1, float* m_io, float* s_io,
                      float* acc) {
    float qf[HD];
    for (uint32_t d = 0; d < HD; d++) qf[d] = orc_h2f(q[d]);
    float m = *m_io, s = *s_io;
    for (uint32_t t = t0; t < t1; t++) {
        const uint16_t* k = kbase + ((size_t)t * NKV + kvh) * HD;
        const uint16_t* v = vbase + ((size_t)t * NKV + kvh) * HD;
        float part[32];
        for (uint32_t l = 0; l < 32; l++) {
            float dot = qf[4 * l] * orc_h2f(k[4 * l]);
            dot = fmaf(qf[4 * l + 1], orc_h2f(k[4 * l + 1]), dot);
            dot = fmaf(qf[4 * l + 2], orc_h2f(k[4 * l + 2]), dot);
            dot = fmaf(qf[4 * l + 3], orc_h2f(k[4 * l + 3]), dot);
            part[l] = dot;
        }
        float sc = warp_tree_sum_lane0(part) * ATTN_SCALE;
        if (sc > m) {
            float corr = ex2_ftz((m - sc) * LOG2E);
            for (uint32_t d = 0; d < HD; d++) acc[d] = acc[d] * corr;
            s = s * corr;
            m = sc;
        }
        float w = ex2_ftz((sc - m) * LOG2E);
        s = s + w;
        for (uint32_t d = 0; d < HD; d++) acc[d] = fmaf(w, orc_h2f(v[d]), acc[d]);
    }
    *m_io = m;
    *s_io = s;
}

static inline uint32_t window_start(uint32_t slen, uint32_t window) {
    return (window != 0 && slen > window) ? slen - window : 0; /* BA:1268-1274 */
}

/* batched_gqa_attention_online_fp16, BA:1194-1370. ctx [B][16][128] f16. */
void orc_attn_online(uint16_t* ctx, const uint16_t* q, const uint64_t* k_ptrs,
                     const uint64_t* v_ptrs, const uint32_t* seq_lens, uint32_t batch,
                     uint32_t window) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t bh = 0; bh < (int64_t)batch * NQ; bh++) {
        uint32_t b = (uint32_t)(bh / NQ), h = (uint32_t)(bh % NQ);
        const uint16_t* kb = (const uint16_t*)(uintptr_t)k_ptrs[b];
        const uint16_t* vb = (const uint16_t*)(uintptr_t)v_ptrs[b];
        uint32_t slen = seq_lens[b];
        float m = -1.0e30f, s = 0.0f, acc[HD];
        memset(acc, 0, sizeof(acc));
        scan_keys(q + ((size_t)b * NQ + h) * HD, kb, vb, h >> 2, window_start(slen, window), slen,
                  &m, &s, acc);
        float inv = rcp_ftz(s);
        uint16_t* o = ctx + ((size_t)b * NQ + h) * HD;
        for (uint32_t d = 0; d < HD; d++) o[d] = orc_f2h(acc[d] * inv);
    }
}

/* batched_gqa_attention_split_fp16 / _split4_fp16 (bit-identical by the
 * reference's own test), BA:1389-1589, BA:2665-3035.
 * partial_acc [B][nchunks][16][128] f32, partial_stats [B][nchunks][16][2]. */
void orc_attn_split(const uint16_t* q, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                    const uint32_t* seq_lens, float* partial_acc, float* partial_stats,
                    uint32_t batch, uint32_t window, uint32_t chunk_keys, uint32_t nchunks) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t it = 0; it < (int64_t)batch * nchunks * NQ; it++) {
        uint32_t h = (uint32_t)(it % NQ);
        uint32_t c = (uint32_t)((it / NQ) % nchunks);
        uint32_t b = (uint32_t)(it / ((int64_t)NQ * nchunks));
        const uint16_t* kb = (const uint16_t*)(uintptr_t)k_ptrs[b];
        const uint16_t* vb = (const uint16_t*)(uintptr_t)v_ptrs[b];
        uint32_t slen = seq_lens[b];
        uint32_t t0 = c * chunk_keys + window_start(slen, window);
        uint32_t t1 = t0 + chunk_keys;
        if (t1 > slen) t1 = slen;
        float m = -1.0e30f, s = 0.0f, acc[HD];
        memset(acc, 0, sizeof(acc));
        if (t0 < t1) scan_keys(q + ((size_t)b * NQ + h) * HD, kb, vb, h >> 2, t0, t1, &m, &s, acc);
        size_t pidx = ((size_t)b * nchunks + c) * NQ + h;
        partial_stats[pidx * 2] = m;
        partial_stats[pidx * 2 + 1] = s;
        memcpy(partial_acc + pidx * HD, acc, sizeof(acc));
    }
}

/* batched_gqa_attn_combine_fp16, BA:1597-1717. */
void orc_attn_combine(uint16_t* ctx, const float* partial_acc, const float* partial_stats,
                      uint32_t batch, uint32_t nchunks) {
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < (int64_t)batch * NQ; bh++) {
        uint32_t b = (uint32_t)(bh / NQ), h = (uint32_t)(bh % NQ);
        float m = -1.0e30f, s = 0.0f, acc[HD];
        memset(acc, 0, sizeof(acc));
        for (uint32_t c = 0; c < nchunks; c++) {
            size_t pidx = ((size_t)b * nchunks + c) * NQ + h;
            float mc = partial_stats[pidx * 2], sc = partial_stats[pidx * 2 + 1];
            if (mc > m) {
                float corr = ex2_ftz((m - mc) * LOG2E);
                for (uint32_t d = 0; d < HD; d++) acc[d] = acc[d] * corr;
                s = s * corr;
                m = mc;
            }
            float w = ex2_ftz((mc - m) * LOG2E);
            s = s + w * sc;
            const float* p = partial_acc + pidx * HD;
            for (uint32_t d = 0; d < HD; d++) acc[d] = fmaf(w, p[d], acc[d]);
        }
        float inv = rcp_ftz(s);
        uint16_t* o = ctx + ((size_t)b * NQ + h) * HD;
        for (uint32_t d = 0; d < HD; d++) o[d] = orc_f2h(acc[d] * inv);
    }
}

/* batched_sigmoid_gate_fp16, BA:583-655: ctx (already f16) *= sigmoid(gate). */
void orc_sigmoid_gate(uint16_t* ctx_io, const uint16_t* gate, uint32_t heads, uint32_t hd,
                      uint32_t batch) {
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t h = 0; h < heads; h++) {
            float g = orc_h2f(gate[(size_t)b * heads + h]);
            float e = ex2_ftz((-g) * LOG2E);
            float sig = rcp_ftz(e + 1.0f);
            uint16_t* x = ctx_io + ((size_t)b * heads + h) * hd;
            for (uint32_t d = 0; d < hd; d++) x[d] = orc_f2h(orc_h2f(x[d]) * sig);
        }
}

/* The engine's decode sequence for one attention layer
 * (crates/oxide-infer-server/src/batch_engine.rs:941-1239): norm q, norm k,
 * rope q, rope k, copy k, copy v, split4 + combine (or online when one chunk),
 * gate.  q_io and k_io are modified in place as in the reference. */
void orc_decode_layer(uint16_t* ctx, uint16_t* q_io, uint16_t* k_io, const uint16_t* v_in,
                      const uint16_t* gate, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                      const uint16_t* cos_t, const uint16_t* sin_t, const uint32_t* pos_ids,
                      const uint32_t* seq_lens, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                      uint32_t batch, uint32_t window, float eps, float* scratch_acc,
                      float* scratch_stats, uint32_t nchunks) {
    orc_qk_rmsnorm(q_io, q_norm_w, eps, NQ, HD, batch);
    orc_qk_rmsnorm(k_io, k_norm_w, eps, NKV, HD, batch);
    orc_rope(q_io, cos_t, sin_t, pos_ids, NQ, HD, batch);
    orc_rope(k_io, cos_t, sin_t, pos_ids, NKV, HD, batch);
    orc_kv_copy(k_ptrs, k_io, pos_ids, KV_DIM, batch);
    orc_kv_copy(v_ptrs, v_in, pos_ids, KV_DIM, batch);
    if (nchunks > 1) {
        orc_attn_split(q_io, k_ptrs, v_ptrs, seq_lens, scratch_acc, scratch_stats, batch, window,
                       128, nchunks);
        orc_attn_combine(ctx, scratch_acc, scratch_stats, batch, nchunks);
    } else {
        orc_attn_online(ctx, q_io, k_ptrs, v_ptrs, seq_lens, batch, window);
    }
    if (gate) orc_sigmoid_gate(ctx, gate, NQ, HD, batch);
}

/* ---------------------------------------------------------------- a8 ---- */

/* One prefill chunk through the GEMM attention sequence of
 * BatchEngine::gemm_attention_chunk (batch_engine.rs:439-592): per kv head
 * S = Qpack*K^T in f32, batched_attn_softmax_mask_fp16 (BA:2368-2546) to
 * unnormalised f16 P + f32 sum, O = V^T*P^T rounded to f16, then
 * batched_attn_gate_scatter_fp16 (BA:2561-2645).  The two GEMMs run inside
 * cuBLASLt in the reference (f16 inputs, f32 accumulate, summation order not
 * specified); here they accumulate in f32 in index order, so this function is
 * comparable with the reference only to its own test tolerance (8e-3).
 * q [rows][16][128], gate [rows][16], ctx [rows][16][128]; rows consecutive
 * positions p0.. of one sequence whose K/V are at kbase/vbase. */
void orc_prefill_gemm_chunk(uint16_t* ctx, const uint16_t* q, const uint16_t* gate,
                            const uint16_t* kbase, const uint16_t* vbase, uint32_t rows,
                            uint32_t p0, uint32_t window) {
    uint32_t slen_min = p0 + 1, slen_max = p0 + rows;
    uint32_t t_lo = window ? (slen_min > window ? slen_min - window : 0) : 0;
    uint32_t keys = slen_max - t_lo;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t rh = 0; rh < (int64_t)rows * NQ; rh++) {
        uint32_t r = (uint32_t)(rh / NQ), h = (uint32_t)(rh % NQ), kvh = h >> 2;
        uint32_t slen = p0 + r + 1;
        float* sc = (float*)malloc(sizeof(float) * keys);
        uint16_t* p = (uint16_t*)malloc(sizeof(uint16_t) * keys);
        const uint16_t* qr = q + ((size_t)r * NQ + h) * HD;
        for (uint32_t u = 0; u < keys; u++) {
            const uint16_t* k = kbase + ((size_t)(t_lo + u) * NKV + kvh) * HD;
            float a = 0.0f;
            for (uint32_t d = 0; d < HD; d++) a = fmaf(orc_h2f(qr[d]), orc_h2f(k[d]), a);
            sc[u] = a;
        }
        uint32_t hi = slen - t_lo;
        if (hi > keys) hi = keys;
        uint32_t lo = (window != 0 && slen > window) ? slen - window - t_lo : 0;
        float m = -1.0e30f;
        for (uint32_t u = lo; u < hi; u++) m = fmaxf(m, sc[u] * ATTN_SCALE);
        /* the column sum is reduced thread-strided by 128 then by warp tree
         * then across 4 warps (BA:2476-2535) */
        float tsum[128];
        for (uint32_t t = 0; t < 128; t++) tsum[t] = 0.0f;
        for (uint32_t u = 0; u < keys; u++) {
            float e = 0.0f;
            if (u >= lo && u < hi) {
                float x = sc[u] * ATTN_SCALE;
                x = x - m;
                x = x * LOG2E;
                e = ex2_ftz(x);
                tsum[u % 128] = tsum[u % 128] + e;
            }
            p[u] = orc_f2h(e);
        }
        float wsum[4];
        for (uint32_t w = 0; w < 4; w++) wsum[w] = warp_tree_sum_lane0(tsum + 32 * w);
        float sum = wsum[0];
        sum = sum + wsum[1];
        sum = sum + wsum[2];
        sum = sum + wsum[3];
        float g = orc_h2f(gate[(size_t)r * NQ + h]);
        float sig = rcp_ftz(ex2_ftz((-g) * LOG2E) + 1.0f);
        float scale = sig / sum; /* div.rn.f32, BA:2608 */
        uint16_t* o = ctx + ((size_t)r * NQ + h) * HD;
        for (uint32_t d = 0; d < HD; d++) {
            float a = 0.0f;
            for (uint32_t u = 0; u < keys; u++) {
                const uint16_t* v = vbase + ((size_t)(t_lo + u) * NKV + kvh) * HD;
                a = fmaf(orc_h2f(p[u]), orc_h2f(v[d]), a);
            }
            float of = orc_h2f(orc_f2h(a)); /* PV GEMM output is f16 */
            o[d] = orc_f2h(of * scale);
        }
        free(sc);
        free(p);
    }
}

/* ----------------------------------------------------------- a9, a10 ---- */

/* batched_fused_causal_conv1d_gating_ptr_fp16, BA:727-881.
 * bcx [B][3*hidden] = [B | C | x]; state_ptrs[b] -> [hidden][k_len-1] f16;
 * conv_w [hidden][k_len]; y [B][hidden].  The newest tap enters as the
 * unrounded f32 product, the history taps are the stored f16 products. */
void orc_conv_decode(uint16_t* y, const uint64_t* state_ptrs, const uint16_t* bcx,
                     const uint16_t* conv_w, uint32_t hidden, uint32_t k_len, uint32_t batch) {
    uint32_t km1 = k_len - 1;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)batch; b++) {
        uint16_t* st = (uint16_t*)(uintptr_t)state_ptrs[b];
        const uint16_t* row = bcx + (size_t)b * 3 * hidden;
        for (uint32_t c = 0; c < hidden; c++) {
            float fin = orc_h2f(row[c]) * orc_h2f(row[2 * hidden + c]);
            uint16_t hin = orc_f2h(fin);
            uint16_t* s = st + (size_t)c * km1;
            const uint16_t* w = conv_w + (size_t)c * k_len;
            float sum = 0.0f;
            for (uint32_t k = 0; k < km1; k++) sum = fmaf(orc_h2f(s[k]), orc_h2f(w[k]), sum);
            sum = fmaf(fin, orc_h2f(w[km1]), sum);
            for (uint32_t k = 0; k + 1 < km1; k++) s[k] = s[k + 1];
            s[km1 - 1] = hin;
            sum = sum * orc_h2f(row[hidden + c]);
            y[(size_t)b * hidden + c] = orc_f2h(sum);
        }
    }
}

/* conv_state_prefill_fp16, BA:1049-1176: build every wave row's 6-slot state
 * in pool [rows][hidden][6] from the wave's own B*x history or the request's
 * carry state. origin/local_pos are used as signed 32-bit, as in the PTX. */
void orc_conv_state_prefill(uint16_t* pool, const uint64_t* carry_tbl, const uint32_t* origin_tbl,
                            const uint32_t* pos_tbl, const uint16_t* bcx, uint32_t hidden,
                            uint32_t k_len, uint32_t rows) {
    uint32_t km1 = k_len - 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        int32_t origin = (int32_t)origin_tbl[r], lpos = (int32_t)pos_tbl[r];
        const uint16_t* carry = (const uint16_t*)(uintptr_t)carry_tbl[r];
        uint16_t* dst = pool + (size_t)r * hidden * 6;
        for (uint32_t c = 0; c < hidden; c++)
            for (uint32_t k = 0; k < km1; k++) {
                int32_t j = lpos + (int32_t)k - 6;
                uint16_t v;
                if (j < 0) {
                    v = carry[(size_t)c * 6 + (size_t)(j + 6)];
                } else {
                    const uint16_t* src = bcx + (size_t)(origin + j) * 3 * hidden;
                    v = orc_f2h(orc_h2f(src[c]) * orc_h2f(src[2 * hidden + c]));
                }
                dst[(size_t)c * 6 + k] = v;
            }
    }
}

/* The engine's conv sequence for one prefill wave of one layer
 * (batch_engine.rs:847-899 and the per-chunk copy-back in
 * crates/oxide-infer-server/src/bin/server.rs:1192-1224): gather states into
 * the pool, run the decode kernel on every pool row, then copy each chunk's
 * last pool row into the request's persistent state (carry_tbl of that row).
 * pool is caller scratch [rows][hidden][6]. */
void orc_conv_prefill_wave(uint16_t* y, uint16_t* pool, const uint64_t* carry_tbl,
                           const uint32_t* origin_tbl, const uint32_t* pos_tbl,
                           const uint16_t* bcx, const uint16_t* conv_w, uint32_t hidden,
                           uint32_t k_len, uint32_t rows) {
    orc_conv_state_prefill(pool, carry_tbl, origin_tbl, pos_tbl, bcx, hidden, k_len, rows);
    uint64_t* ptrs = (uint64_t*)malloc(sizeof(uint64_t) * rows);
    for (uint32_t r = 0; r < rows; r++) ptrs[r] = (uint64_t)(uintptr_t)(pool + (size_t)r * hidden * 6);
    orc_conv_decode(y, ptrs, bcx, conv_w, hidden, k_len, rows);
    for (uint32_t r = 0; r < rows; r++) {
        int last = (r + 1 == rows) || (origin_tbl[r + 1] != origin_tbl[r]);
        if (last)
            memcpy((void*)(uintptr_t)carry_tbl[r], pool + (size_t)r * hidden * 6,
                   (size_t)hidden * 6 * 2);
    }
    free(ptrs);
}

/* ---- sampling-side table kernels of the same file (next to the KV path) ------------------- */

/* batched_embed_lookup_fp16 (batched_attn.rs:664-714; launched batch_engine.rs:778):
 * out[b][:] = table[token_ids[b]][:], hidden f16 per row, no bounds check in the reference. */
void orc_embed_lookup(uint16_t* out, const uint16_t* table, const uint32_t* token_ids,
                      uint32_t hidden, uint32_t batch) {
    for (uint32_t b = 0; b < batch; b++)
        memcpy(out + (size_t)b * hidden, table + (size_t)token_ids[b] * hidden, (size_t)hidden * 2);
}

/* batched_argmax_direct_f16 (batched_attn.rs:890-1023), one block of `nthreads` threads per row
 * (256 at batch_engine.rs:1377).  Thread t scans t, t+nthreads, ... keeping the FIRST strict
 * maximum (start -1e30, index 0; NaN never wins: setp.gt is false).  Then the shuffle-down tree
 * inside each warp (offsets 16..1; a lane takes its partner's pair only if strictly greater; a
 * partner past lane 31 returns the lane's own value), lane 0 of each warp to shared memory, and
 * the same tree with offsets 4, 2, 1 over the 8 warp results.  Ties are therefore resolved by the
 * tree, not by the lowest index - restated literally here. */
void orc_argmax(uint32_t* tokens_out, const uint16_t* logits, uint32_t vocab, uint32_t batch,
                uint32_t nthreads) {
#pragma omp parallel for schedule(static)
    for (int64_t bb = 0; bb < (int64_t)batch; bb++) {
        const uint16_t* row = logits + (size_t)bb * vocab;
        float* mx = (float*)malloc(sizeof(float) * nthreads);
        uint32_t* bi = (uint32_t*)malloc(sizeof(uint32_t) * nthreads);
        for (uint32_t t = 0; t < nthreads; t++) {
            float m = -1.0e30f;
            uint32_t best = 0;
            for (uint32_t i = t; i < vocab; i += nthreads) {
                const float f = orc_h2f(row[i]);
                if (f > m) {
                    m = f;
                    best = i;
                }
            }
            mx[t] = m;
            bi[t] = best;
        }
        const uint32_t nwarps = nthreads / 32;
        float wm[8] = {0};
        uint32_t wi[8] = {0};
        for (uint32_t w = 0; w < nwarps && w < 8; w++) {
            float v[32];
            uint32_t ix[32];
            for (int l = 0; l < 32; l++) {
                v[l] = mx[w * 32 + l];
                ix[l] = bi[w * 32 + l];
            }
            for (int off = 16; off >= 1; off >>= 1) {
                float nv[32];
                uint32_t ni[32];
                for (int l = 0; l < 32; l++) {
                    const int p = l + off <= 31 ? l + off : l;
                    const int take = v[p] > v[l];
                    nv[l] = take ? v[p] : v[l];
                    ni[l] = take ? ix[p] : ix[l];
                }
                memcpy(v, nv, sizeof v);
                memcpy(ix, ni, sizeof ix);
            }
            wm[w] = v[0];
            wi[w] = ix[0];
        }
        for (int off = 4; off >= 1; off >>= 1) {  /* threads 0..7; only lane 0's result is used */
            float nv[8];
            uint32_t ni[8];
            for (int l = 0; l < 8; l++) {
                const int p = l + off;
                const int take = p < 8 && wm[p] > wm[l];
                nv[l] = take ? wm[p] : wm[l];
                ni[l] = take ? wi[p] : wi[l];
            }
            memcpy(wm, nv, sizeof wm);
            memcpy(wi, ni, sizeof wi);
        }
        tokens_out[bb] = wi[0];
        free(mx);
        free(bi);
    }
}

/* Sets the number of OpenMP threads of the following calls (a launcher may have exported
 * OMP_NUM_THREADS=1 for its worker processes); n <= 0 leaves it alone. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
