/*
 * TEST INFRASTRUCTURE, not product code: a scalar CPU restatement of the KV append/quantise step, the golden
 * source for "q bits, cache bytes and scales are bit-exact". Only tests/, __graft_entry__.smoke() and bench.py's
 * CPU-baseline legs may load it.
 *
 * Parity status: the reference has no fp8 cache and no test or golden vector for this path, so the quantise rule
 * is pinned by this file's own definition (the rule this path is specified with: per-(token, head) scale = amax / 448, e4m3 round to
 * nearest even) and the e4m3 conversion is pinned exhaustively against torch.float8_e4m3fn
 * (tests/test_oracle.py). The q/k row math restates the reference and is pinned, within one bf16 ulp, against
 * outputs of the reference's own inference/modeling_nanochat.py:qk_norm_rope (tests/golden/).
 *
 * What it follows in the reference:
 *   model/kernels/qk_row.cuh:26-30   rstd = 1 / sqrt(mean(x^2) + FLT_EPSILON), the sum of squares taken per lane
 *                                    (8 lanes, lane t owns dims 8t..8t+7 and 64+8t..64+8t+7), then an xor
 *                                    butterfly over offsets 4, 2, 1 (qk_row.cuh:19-23)
 *   model/kernels/qk_row.cuh:33-41   n = x * rstd * gain; y1 = n1 cos + n2 sin; y2 = n2 cos - n1 sin with partners
 *                                    64 apart
 *   model/kernels/decode.cu:494-505  q, k, v each rounded to bf16 exactly once
 *   model/kernels/decode.cu:556-564  the row's k, v go to cache position pos[b] of slot cache_slot[b]
 *   model/kernels/decode.cu:482-494  the optional value-embedding mix v = bf16(v + 2 sigmoid(w[head] . h) ve[token]):
 *                                    the dot product as FMAs, a warp lane owning 8 consecutive elements of every
 *                                    256-element chunk, then an xor butterfly over offsets 16, 8, 4, 2, 1
 * Deviations, chosen so that a CPU can reproduce the GPU bit for bit: every fp32 operation is individually
 * rounded (compile with -ffp-contract=off; the reference lets nvcc contract FMAs), and rsqrtf (2 ulp, not
 * reproducible on a CPU) is replaced by a correctly rounded sqrt followed by a correctly rounded divide. The
 * gate's sigmoid is evaluated in double precision and rounded once, 2 / (1 + exp(-d)), where the reference uses
 * fp32 expf (not reproducible across libraries); the two agree to within an ulp of fp32.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC (oracle/build_oracle.py).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#define HEAD_DIM 128
#define HALF 64
#define LANES 8
#define VEC 8

static float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* Round to nearest even; NaN stays NaN (quiet). */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* e4m3 (OCP "fn": no infinity, 0x7f NaN, max 448), round to nearest even, finite inputs saturate to +-448. */
uint8_t oracle_f32_to_e4m3(float f) {
    uint32_t u = f32_bits(f);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    u &= 0x7fffffffu;
    if (u > 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* NaN */
    const float a = bits_f32(u);
    if (a < 0.015625f) { /* below 2^-6: subnormal grid of spacing 2^-9 */
        const float q = nearbyintf(a * 512.0f); /* exact product; default rounding mode is to nearest even */
        return (uint8_t)(sign | (uint8_t)q);    /* q = 8 lands on the first normal, 0x08 */
    }
    if (a >= 464.0f) return (uint8_t)(sign | 0x7eu); /* would round to 480 or more: saturate */
    u += 0x7ffffu + ((u >> 20) & 1u);               /* keep 3 mantissa bits */
    const int e = (int)(u >> 23) - 127 + 7;
    const uint32_t m = (u >> 20) & 7u;
    return (uint8_t)(sign | (uint8_t)(e << 3) | (uint8_t)m);
}

float oracle_e4m3_to_f32(uint8_t b) {
    const int e = (b >> 3) & 15, m = b & 7;
    float a;
    if (e == 15 && m == 7) a = NAN;
    else if (e == 0) a = ldexpf((float)m, -9);
    else a = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -a : a;
}

/* One q or k head row: 128 bf16 in, 128 bf16 out. gain fp32[128]; cs, sn fp32[64] at the row's position. */
void oracle_qk_row(const uint16_t *x, const float *gain, const float *cs, const float *sn, uint16_t *y) {
    float ss[LANES];
    for (int t = 0; t < LANES; t++) { /* qk_row.cuh:27-28, per lane, each product and add rounded */
        float acc = 0.f;
        for (int i = 0; i < VEC; i++) {
            const float x1 = oracle_bf16_to_f32(x[VEC * t + i]), x2 = oracle_bf16_to_f32(x[HALF + VEC * t + i]);
            const float p1 = x1 * x1, p2 = x2 * x2;
            const float s = p1 + p2;
            acc = acc + s;
        }
        ss[t] = acc;
    }
    for (int o = LANES / 2; o > 0; o >>= 1) { /* qk_row.cuh:19-23, xor butterfly 4, 2, 1 */
        float next[LANES];
        for (int t = 0; t < LANES; t++) next[t] = ss[t] + ss[t ^ o];
        memcpy(ss, next, sizeof ss);
    }
    const float mean = ss[0] / (float)HEAD_DIM;
    const float root = sqrtf(mean + FLT_EPSILON);
    const float r = 1.0f / root;
    for (int i = 0; i < HALF; i++) { /* qk_row.cuh:36-40, parenthesised as written */
        const float x1 = oracle_bf16_to_f32(x[i]), x2 = oracle_bf16_to_f32(x[HALF + i]);
        const float a1 = x1 * r, a2 = x2 * r;
        const float n1 = a1 * gain[i], n2 = a2 * gain[HALF + i];
        const float t1 = n1 * cs[i], t2 = n2 * sn[i], t3 = n2 * cs[i], t4 = n1 * sn[i];
        y[i] = oracle_f32_to_bf16(t1 + t2);
        y[HALF + i] = oracle_f32_to_bf16(t3 - t4);
    }
}

/* One k or v head row of 128 bf16 values: scale = amax / 448, byte = e4m3(x / scale); amax == 0 gives scale 0 and
 * all bytes 0x00 (the sign of a zero is dropped). */
void oracle_quant_row(const uint16_t *x, uint8_t *bytes, float *scale) {
    float amax = 0.f;
    for (int i = 0; i < HEAD_DIM; i++) amax = fmaxf(amax, fabsf(oracle_bf16_to_f32(x[i])));
    if (!(amax > 0.f)) { /* zero row (inputs are finite by contract) */
        *scale = 0.f;
        memset(bytes, 0, HEAD_DIM);
        return;
    }
    const float s = amax / 448.0f;
    *scale = s;
    for (int i = 0; i < HEAD_DIM; i++) bytes[i] = oracle_f32_to_e4m3(oracle_bf16_to_f32(x[i]) / s);
}

/* The value-embedding gate of one (row, kv head): 2 sigmoid(w . h) over C elements (C a multiple of 256), h bf16 (the
 * layer's normed input), w fp32. decode.cu:485-491's order: lane L of 32 accumulates, by FMA, elements
 * (32 k + L) 8 + j for k = 0 .. C / 256 - 1 and j = 0 .. 7; the lanes' sums are reduced by an xor butterfly. */
float oracle_ve_gate(const uint16_t *h, const float *w, int C) {
    float d[32];
    for (int lane = 0; lane < 32; lane++) {
        float acc = 0.f;
        for (int k = 0; k < C / 256; k++)
            for (int j = 0; j < 8; j++) {
                const int i = (k * 32 + lane) * 8 + j;
                acc = fmaf(oracle_bf16_to_f32(h[i]), w[i], acc);
            }
        d[lane] = acc;
    }
    for (int o = 16; o > 0; o >>= 1) {
        float next[32];
        for (int lane = 0; lane < 32; lane++) next[lane] = d[lane] + d[lane ^ o];
        memcpy(d, next, sizeof d);
    }
    return (float)(2.0 / (1.0 + exp(-(double)d[0])));
}

/* v (128 bf16) <- bf16(v + gate * ve), each product and sum rounded (decode.cu:492-494). */
void oracle_ve_mix(uint16_t *v, float gate, const uint16_t *ve) {
    for (int i = 0; i < HEAD_DIM; i++) {
        const float p = gate * oracle_bf16_to_f32(ve[i]);
        v[i] = oracle_f32_to_bf16(oracle_bf16_to_f32(v[i]) + p);
    }
}

/*
 * The whole step for `rows` tokens, logical (un-paged) outputs:
 *   qkv bf16 [rows][row_stride] (Hq q heads, Hkv k heads, Hkv v heads); pos int32 [rows];
 *   cos, sin fp32 [table_len][64]; q_out bf16 [rows][Hq][128]; k_bf16 [rows][Hkv][128] (the rounded, rotated k
 *   before quantisation, for cross-checks); k_bytes, v_bytes u8 [rows][Hkv][128]; k_scale, v_scale fp32
 *   [rows][Hkv].
 */
static void kv_append_rows(const uint16_t *qkv, const float *q_gain, const float *k_gain, const float *cs,
                           const float *sn, const int32_t *pos, long long rows, int Hq, int Hkv, long long row_stride,
                           uint16_t *q_out, uint16_t *k_bf16, uint8_t *k_bytes, float *k_scale, uint8_t *v_bytes,
                           float *v_scale, const uint16_t *hn, const long long *tokens, const uint16_t *ve_table,
                           const float *ve_gate, int C) {
    for (long long r = 0; r < rows; r++) {
        const uint16_t *row = qkv + r * row_stride;
        const float *c = cs + (size_t)pos[r] * HALF, *s = sn + (size_t)pos[r] * HALF;
        for (int h = 0; h < Hq; h++) oracle_qk_row(row + h * HEAD_DIM, q_gain, c, s, q_out + (r * Hq + h) * HEAD_DIM);
        for (int h = 0; h < Hkv; h++) {
            uint16_t *kb = k_bf16 + (r * Hkv + h) * HEAD_DIM;
            oracle_qk_row(row + (Hq + h) * HEAD_DIM, k_gain, c, s, kb);
            oracle_quant_row(kb, k_bytes + (r * Hkv + h) * HEAD_DIM, k_scale + r * Hkv + h);
            uint16_t v[HEAD_DIM];
            memcpy(v, row + (Hq + Hkv + h) * HEAD_DIM, sizeof v);
            if (ve_table)
                oracle_ve_mix(v, oracle_ve_gate(hn + r * C, ve_gate + (size_t)h * C, C),
                              ve_table + ((size_t)tokens[r] * Hkv + h) * HEAD_DIM);
            oracle_quant_row(v, v_bytes + (r * Hkv + h) * HEAD_DIM, v_scale + r * Hkv + h);
        }
    }
}

void oracle_kv_append(const uint16_t *qkv, const float *q_gain, const float *k_gain, const float *cs,
                      const float *sn, const int32_t *pos, long long rows, int Hq, int Hkv, long long row_stride,
                      uint16_t *q_out, uint16_t *k_bf16, uint8_t *k_bytes, float *k_scale, uint8_t *v_bytes,
                      float *v_scale) {
    kv_append_rows(qkv, q_gain, k_gain, cs, sn, pos, rows, Hq, Hkv, row_stride, q_out, k_bf16, k_bytes, k_scale, v_bytes,
                   v_scale, NULL, NULL, NULL, NULL, 0);
}

/* The same with the value-embedding mix on v: h bf16 [rows][C] (the layer's normed input), tokens int64 [rows],
 * ve_table bf16 [vocab][Hkv][128], ve_gate fp32 [Hkv][C]. */
void oracle_kv_append_ve(const uint16_t *qkv, const float *q_gain, const float *k_gain, const float *cs,
                         const float *sn, const int32_t *pos, long long rows, int Hq, int Hkv, long long row_stride,
                         uint16_t *q_out, uint16_t *k_bf16, uint8_t *k_bytes, float *k_scale, uint8_t *v_bytes,
                         float *v_scale, const uint16_t *h, const long long *tokens, const uint16_t *ve_table,
                         const float *ve_gate, int C) {
    kv_append_rows(qkv, q_gain, k_gain, cs, sn, pos, rows, Hq, Hkv, row_stride, q_out, k_bf16, k_bytes, k_scale, v_bytes,
                   v_scale, h, tokens, ve_table, ve_gate, C);
}

/* Bulk helpers for the Python side. */
void oracle_f32_to_e4m3_n(const float *x, uint8_t *y, long long n) {
    for (long long i = 0; i < n; i++) y[i] = oracle_f32_to_e4m3(x[i]);
}
void oracle_quant_rows(const uint16_t *x, uint8_t *bytes, float *scale, long long rows) {
    for (long long r = 0; r < rows; r++) oracle_quant_row(x + r * HEAD_DIM, bytes + r * HEAD_DIM, scale + r);
}
