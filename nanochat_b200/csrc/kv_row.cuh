/*
 * Row arithmetic of the KV append, shared by kv_append.cu and the attention kernel that appends its own token
 * (decode_attn.cu), so both produce the same bits: one head row of 128 values is handled by 8 lanes, lane t owning
 * dims 8t..8t+7 and their rotation partners 64+8t..64+8t+7 (the ownership of the reference's
 * model/kernels/qk_row.cuh:11-12,44-50). Every fp32 operation is an explicit round-to-nearest intrinsic in the
 * order of oracle/kv_append_oracle.c.
 */
#pragma once

#include "ncb_common.cuh"

constexpr int LANES = 8;
constexpr int VEC = 8;

static __device__ __forceinline__ void unpack_bf16x8(const uint4 &u, float *v) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < VEC / 2; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

static __device__ __forceinline__ void load_bf16x8(const bf16 *p, float *v) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < VEC / 2; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

static __device__ __forceinline__ void load_f32x8(const float *p, float *v) {
    *reinterpret_cast<float4 *>(v) = *reinterpret_cast<const float4 *>(p);
    *reinterpret_cast<float4 *>(v + 4) = *reinterpret_cast<const float4 *>(p + 4);
}

/* The 8-lane group's shuffle mask and butterfly reductions (offsets 4, 2, 1). */
static __device__ __forceinline__ unsigned group_mask() {
    return 0xffu << ((threadIdx.x & 31) & ~(LANES - 1));
}
static __device__ __forceinline__ float group_sum(float v) {
    const unsigned mask = group_mask();
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(mask, v, o));
    return v;
}
static __device__ __forceinline__ float group_max(float v) {
    const unsigned mask = group_mask();
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o));
    return v;
}

/* x1, x2 (this lane's 8 + 8 values) -> normed, gained, rotated values rounded to bf16 and widened again. */
static __device__ __forceinline__ void norm_rotate(float *x1, float *x2, const float *gain, const float *cs,
                                                   const float *sn, int o) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; i++)
        ss = __fadd_rn(ss, __fadd_rn(__fmul_rn(x1[i], x1[i]), __fmul_rn(x2[i], x2[i])));
    ss = group_sum(ss);
    const float mean = __fmul_rn(ss, 1.f / (float)HEAD_DIM); /* a power of two: the same rounding as the division */
    const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(mean, FLT_EPSILON)));
#pragma unroll
    for (int q = 0; q < VEC; q += 4) { /* four dims and their partners at a time: 16 table values live, not 32 */
        const float4 g1 = *reinterpret_cast<const float4 *>(gain + o + q), g2 = *reinterpret_cast<const float4 *>(gain + HALF + o + q);
        const float4 c = *reinterpret_cast<const float4 *>(cs + o + q), s = *reinterpret_cast<const float4 *>(sn + o + q);
        const float g1v[4] = {g1.x, g1.y, g1.z, g1.w}, g2v[4] = {g2.x, g2.y, g2.z, g2.w};
        const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float n1 = __fmul_rn(__fmul_rn(x1[q + i], r), g1v[i]), n2 = __fmul_rn(__fmul_rn(x2[q + i], r), g2v[i]);
            const float y1 = __fadd_rn(__fmul_rn(n1, cv[i]), __fmul_rn(n2, sv[i]));
            const float y2 = __fsub_rn(__fmul_rn(n2, cv[i]), __fmul_rn(n1, sv[i]));
            x1[q + i] = __bfloat162float(__float2bfloat16_rn(y1));
            x2[q + i] = __bfloat162float(__float2bfloat16_rn(y2));
        }
    }
}

/* The optional value-embedding mix of a v head row (the reference's attn_prologue, model/kernels/decode.cu:482-494):
 * v <- bf16(v + g ve), g = 2 sigmoid(w . h) with h the row's normed layer input (bf16 [C]) and w the kv head's gate
 * weights (fp32 [C]), ve the token's table row for this kv head (bf16 [128]). */
struct ValueEmbed {
    const bf16 *h;            /* [rows][C] */
    const long long *tokens;  /* [rows] */
    const bf16 *table;        /* [vocab][Hkv][128] */
    const float *gate;        /* [Hkv][C] */
    int C, vocab;             /* C a multiple of 256 */
};

/* The reference sums the gate's dot product by FMAs per warp lane L (elements (32 k + L) 8 + j) and reduces the 32
 * lanes with an xor butterfly over 16, 8, 4, 2, 1. Here a row has 8 lanes: lane t plays the reference's lanes t, t + 8,
 * t + 16 and t + 24, whose first two butterfly steps (16, then 8) stay inside the thread; the steps 4, 2, 1 are the
 * group's own butterfly. Same sums in the same order, so the gate's bits are those of oracle/kv_append_oracle.c.
 * The sigmoid is evaluated in double precision and rounded once. */
static __device__ __forceinline__ void ve_mix(float *x1, float *x2, const ValueEmbed &ve, long long row, int kv_head,
                                              int Hkv, int t, int o) {
    const bf16 *h = ve.h + (size_t)row * ve.C;
    const float *w = ve.gate + (size_t)kv_head * ve.C;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < ve.C / 256; k++) {
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const int base = (k * 32 + t + 8 * m) * VEC;
            float hv[VEC], wv[VEC];
            load_bf16x8(h + base, hv);
            load_f32x8(w + base, wv);
#pragma unroll
            for (int j = 0; j < VEC; j++) d[m] = __fmaf_rn(hv[j], wv[j], d[m]);
        }
    }
    const float s = group_sum(__fadd_rn(__fadd_rn(d[0], d[2]), __fadd_rn(d[1], d[3])));
    const float g = (float)(2.0 / (1.0 + exp(-(double)s)));
    long long token = ve.tokens[row];
    if (token < 0 || token >= ve.vocab) token = 0; /* as the embedding lookup does */
    const bf16 *e = ve.table + ((size_t)token * Hkv + kv_head) * HEAD_DIM;
    float e1[VEC], e2[VEC];
    load_bf16x8(e + o, e1);
    load_bf16x8(e + HALF + o, e2);
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        x1[i] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(x1[i], __fmul_rn(g, e1[i]))));
        x2[i] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(x2[i], __fmul_rn(g, e2[i]))));
    }
}

static __device__ __forceinline__ uint4 pack_bf16x8(const float *v) {
    uint4 u;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < VEC / 2; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return u;
}

/* scale = amax / 448 over the group's 128 values; bytes = e4m3(x / scale); a zero row gives scale 0, bytes 0.
 * The row's 16 quotients share one correctly rounded reciprocal r = RN(1 / scale): q0 = RN(x r), the remainder
 * e = fma(-scale, q0, x), q = fma(e, r, q0) is the correctly rounded x / scale (Markstein's division step; checked
 * exhaustively for every pair of bf16 mantissas and every exponent difference that does not round to zero, which is
 * the whole input domain here: x and amax are bf16-valued). Three instructions per value instead of an IEEE division;
 * rows whose amax is so small or large that r or an intermediate could leave the normal range take the division. */
static __device__ __forceinline__ float quantise(const float *x1, const float *x2, uint8_t *b1, uint8_t *b2) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; i++) amax = fmaxf(amax, fmaxf(fabsf(x1[i]), fabsf(x2[i])));
    amax = group_max(amax);
    if (!(amax > 0.f)) {
#pragma unroll
        for (int i = 0; i < VEC; i++) b1[i] = b2[i] = 0;
        return 0.f;
    }
    const float scale = __fdiv_rn(amax, 448.f);
    float q1[VEC], q2[VEC];
    if (amax > 0x1p-100f && amax < 0x1p100f) {
        const float r = __frcp_rn(scale);
#pragma unroll
        for (int i = 0; i < VEC; i++) {
            const float a1 = __fmul_rn(x1[i], r), a2 = __fmul_rn(x2[i], r);
            q1[i] = __fmaf_rn(__fmaf_rn(-scale, a1, x1[i]), r, a1);
            q2[i] = __fmaf_rn(__fmaf_rn(-scale, a2, x2[i]), r, a2);
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i++) q1[i] = __fdiv_rn(x1[i], scale), q2[i] = __fdiv_rn(x2[i], scale);
    }
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
        const uint16_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(q1[i], q1[i + 1]), __NV_SATFINITE, __NV_E4M3);
        const uint16_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(q2[i], q2[i + 1]), __NV_SATFINITE, __NV_E4M3);
        b1[i] = (uint8_t)p1, b1[i + 1] = (uint8_t)(p1 >> 8);
        b2[i] = (uint8_t)p2, b2[i + 1] = (uint8_t)(p2 >> 8);
    }
    return scale;
}


/* The same K row as store_k_row below, as one 16-byte store per lane instead of two 8-byte ones: neighbouring lanes
 * swap halves, so that the even lane holds chunk t/2 (its own dims 8t..8t+7 and the neighbour's) and the odd lane chunk
 * 4 + t/2 (the partners). All 8 lanes of the row's group must call it. */
static __device__ __forceinline__ void store_k_row16(uint8_t *page, int j, int t, const uint8_t *b1, const uint8_t *b2) {
    unsigned long long lo, hi;
    memcpy(&lo, b1, 8);
    memcpy(&hi, b2, 8);
    const unsigned mask = group_mask();
    const bool odd = t & 1;
    /* the even lane gives away its partners' half, the odd lane its first half */
    const unsigned long long got = __shfl_xor_sync(mask, odd ? lo : hi, 1);
    uint4 chunk;
    if (odd) {
        chunk = make_uint4((uint32_t)got, (uint32_t)(got >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
        *reinterpret_cast<uint4 *>(page + page_k_chunk(j, 4 + (t >> 1))) = chunk;
    } else {
        chunk = make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)got, (uint32_t)(got >> 32));
        *reinterpret_cast<uint4 *>(page + page_k_chunk(j, t >> 1)) = chunk;
    }
}

/* Lane t's 8 + 8 quantised bytes of a K row into a page (global or shared) at in-page position j: dims 8t..8t+7 sit
 * in chunk t/2 at byte (t&1)*8, the partners in chunk 4 + t/2. */
static __device__ __forceinline__ void store_k_row(uint8_t *page, int j, int t, const uint8_t *b1, const uint8_t *b2) {
    uint2 lo, hi;
    memcpy(&lo, b1, 8);
    memcpy(&hi, b2, 8);
    *reinterpret_cast<uint2 *>(page + page_k_chunk(j, t >> 1) + (t & 1) * 8) = lo;
    *reinterpret_cast<uint2 *>(page + page_k_chunk(j, 4 + (t >> 1)) + (t & 1) * 8) = hi;
}

/* The same for a V row: the page stores V transposed, so these are 16 single bytes. */
static __device__ __forceinline__ void store_v_row(uint8_t *page, int j, int t, const uint8_t *b1, const uint8_t *b2) {
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        page[page_v_byte(j, t * VEC + i)] = b1[i];
        page[page_v_byte(j, HALF + t * VEC + i)] = b2[i];
    }
}
