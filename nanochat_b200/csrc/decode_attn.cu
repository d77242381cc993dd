/*
 * decode_attn_fp8: single-token attention over the paged e4m3 KV cache, split over the KV length, plus the
 * (m, l, o) merge kernel. Replaces the reference's k_attn (model/kernels/decode.cu:567-675) and its in-kernel
 * merge (decode.cu:548,661-674) for an fp8 cache, grouped-query heads and split KV.
 *
 * Roofline: HBM. Each (kv head, position) costs 264 bytes (128 K + 128 V + two fp32 scales) and is read exactly
 * once for all G = Hq / Hkv query heads that share it. Everything else is shaped to keep that stream busy:
 *
 *   - one thread block per (sequence, kv head, chunk of pages); a page (include/nanochat_b200.h) is one contiguous
 *     16,896-byte record fetched by ONE cp.async.bulk that signals an mbarrier. Each of the block's WARPS warps
 *     owns one shared-memory stage and one barrier: it takes every WARPS-th page of the chunk, waits for it,
 *     consumes it and immediately issues its next page into the same stage. Warps never synchronise with each
 *     other until the end, a barrier is only ever waited on by the warp that armed it (so its phases are observed
 *     strictly in order), and three blocks of four warps per SM keep twelve pages (about 200 KB) in flight or in
 *     use per SM while staggering the blocks' start-up and drain phases;
 *   - no fp8 -> float conversion of K or V at all: both contractions run on the tensor cores as
 *     mma.sync.m16n8k32 e4m3 x e4m3 -> fp32 with the CACHE as the A operand (16 positions, or 16 dims, per tile)
 *     and the N = 8 columns holding the group's query heads. bf16 queries and fp32 probabilities do not fit e4m3's
 *     3 mantissa bits, so each is split into two e4m3 terms, x ~ hi + lo / 16, which keeps bf16-level precision
 *     (relative error 2^-8); the two terms of a head are adjacent columns (2 head, 2 head + 1), so G <= 4 fills
 *     one 8-column tile and G <= 8 two (template parameter NT);
 *   - the per-position K scale multiplies the fp32 score, the per-position V scale is folded into the
 *     probability before it is split, and the running maximum tracks score + log2(v scale) so the folded
 *     probabilities stay in (0, 1]; statistics and accumulators are fp32, exponentials are exp2 with log2(e)
 *     folded into the score scale;
 *   - the page layout (swizzled K rows, V stored transposed in 16-position blocks) makes every ldmatrix
 *     conflict-free and lets the score accumulators turn into the PV operand with four shuffles.
 *
 * Positions outside [begin, len) inside the first and last page are masked with selects; their V bytes are zeroed
 * in shared memory first because an e4m3 NaN byte times a zero probability would still be NaN.
 *
 * Every wait is bounded: when a barrier does not flip within about a second the warp records
 * NCB_DEV_WAIT_TIMEOUT in the caller's status word, waits once more (bounded again) for its copy in flight, stops
 * consuming and falls through to the block's final barriers.
 */
#include <algorithm>
#include <functional>
#include <mutex>
#include <map>
#include <array>
#include <vector>

#include "kv_row.cuh"

constexpr int WARPS = 4; /* = stages per block; 12 stages of 16,896 B fit one SM's shared memory */
constexpr int BLOCKS_PER_SM = 12 / WARPS;
constexpr int THREADS = WARPS * 32;
constexpr uint32_t WAIT_TRIES = 1u << 19; /* x <= 2 us suspend hint each: about one second */
constexpr float P_SCALE = 256.f;          /* folded probabilities in (0, 1] -> e4m3 range, exact power of two */
constexpr float LO_SCALE = 16.f;          /* second term's gain: the first term's rounding error is <= 2^-4 ulp-wise */
constexpr float MIN_LOG2_VSCALE = -64.f;
constexpr size_t ATTN_SMEM = (size_t)WARPS * PAGE_BYTES;
static_assert(WARPS * 4 * 2 * PART * sizeof(float) <= ATTN_SMEM, "the merge area reuses the ring");
static_assert(THREADS >= HEAD_DIM && 12 % WARPS == 0, "the final merge maps one thread to one output dim");

struct AttnArgs {
    const bf16 *q;
    const uint8_t *cache;
    const int32_t *lens, *slot_map;
    float *parts; /* [B][Hq][max_chunks][PART] */
    int B, Hq, Hkv, n_slots, pages_per_slot, window, chunk_pages, max_chunks;
    float scale_log2; /* softmax scale * log2(e) */
    int *status;
    int len_add; /* a sequence's length is lens[b] + len_add (1 when lens holds the new token's position) */
    int early;   /* the predecessor launch leaves lens, slot_map and all but the newest cached position alone */
    /* APPEND only: the new token's fused projection row and what its q/k row math needs (kv_append_fp8's inputs) */
    const bf16 *qkv;
    const float *q_gain, *k_gain, *cs, *sn;
    long long qkv_row_stride;
    int table_len;
    ValueEmbed ve; /* APPEND only; table == NULL: the layer has no value embedding */
    bf16 *direct;  /* one chunk per sequence (max_chunks == 1): the block normalises and writes out[B][Hq][128] itself */
};

/* ---- PTX wrappers ------------------------------------------------------------------------------------------- */

static __device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

static __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
static __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
/* True once the barrier's phase of the given parity has completed; gives up after WAIT_TRIES bounded tries. */
static __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t tries = 0; tries < WAIT_TRIES; tries++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(bar), "r"(parity), "r"(2000u)
                     : "memory");
        if (done) return true;
    }
    return false;
}
/* One page from global to shared memory; the barrier receives the byte count when the copy has landed. A page is
 * read once per step, so it is marked evict-first in L2: what else lives there across the launch (weights the
 * neighbouring GEMMs prefetched, the split states) is not pushed out by the cache stream. */
static __device__ __forceinline__ void page_load(uint32_t dst, const void *src, uint32_t bar) {
    mbar_expect_tx(bar, PAGE_BYTES);
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"((uint32_t)PAGE_BYTES), "r"(bar), "l"(policy)
                 : "memory");
}
static __device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                                   uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
/* d += A B, A 16x32 e4m3 (row), B 32x8 e4m3 (col), fp32 accumulators. */
static __device__ __forceinline__ void mma_e4m3(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
/* e4m3 bytes of (hi, lo), hi in bits 8..15. */
static __device__ __forceinline__ uint32_t cvt_e4m3x2(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
/* The two e4m3 bytes of x (low 16 bits) as floats: .x from the low byte. */
static __device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t x) {
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((uint16_t)x));
    return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}
/* x[0..3] -> word of first terms e4m3(x) and word of second terms e4m3((x - first) * 16); byte i from x[i]. */
static __device__ __forceinline__ void split4(const float *x, uint32_t &hi, uint32_t &lo) {
    const uint32_t h01 = cvt_e4m3x2(x[1], x[0]), h23 = cvt_e4m3x2(x[3], x[2]);
    const float2 f01 = e4m3x2_to_float2(h01), f23 = e4m3x2_to_float2(h23);
    const uint32_t l01 = cvt_e4m3x2((x[1] - f01.y) * LO_SCALE, (x[0] - f01.x) * LO_SCALE);
    const uint32_t l23 = cvt_e4m3x2((x[3] - f23.y) * LO_SCALE, (x[2] - f23.x) * LO_SCALE);
    hi = h01 | (h23 << 16);
    lo = l01 | (l23 << 16);
}
static __device__ __forceinline__ float lg2(float x) { /* log2, 0 -> -inf */
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
/* max over the 8 lanes that share lane % 4 (one query head's positions) */
static __device__ __forceinline__ float head_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
static __device__ __forceinline__ float head_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v + __shfl_xor_sync(0xffffffffu, v, 16);
}

/* ---- split-KV kernel ---------------------------------------------------------------------------------------- */

/* A row the kernels refuse (and flag): its length or slot lies outside the cache or, where the row's own token is
 * appended first, beyond the rotary table (table_len 0: no such check). The split and the merge kernels share the
 * test, so a refused row has no states written and none merged: its output is a zero row. */
static __device__ __forceinline__ bool row_rejected(int len, int slot, int pages_per_slot, int n_slots, int table_len) {
    return len > pages_per_slot * PAGE_TOKENS || slot < 0 || slot >= n_slots || (table_len > 0 && len > table_len);
}

/* Zero the V bytes of the page's positions outside [begin, len): an e4m3 NaN byte times a zero probability would
 * still be NaN. One warp; the caller synchronises it afterwards. */
static __device__ __forceinline__ void zero_v_outside(uint8_t *page, int key0, int begin, int len, int lane) {
#pragma unroll
    for (int blk = 0; blk < 4; blk++) { /* 16-position blocks: (group, half) */
        const int first = key0 + 16 * blk;
        uint32_t keep[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {
            keep[w] = 0;
#pragma unroll
            for (int bb = 0; bb < 4; bb++) {
                const int pos = first + 4 * w + bb;
                if (pos >= begin && pos < len) keep[w] |= 0xffu << (8 * bb);
            }
        }
        if ((keep[0] & keep[1] & keep[2] & keep[3]) == 0xffffffffu) continue;
        for (int d = lane; d < HEAD_DIM; d += 32) {
            uint4 *row = reinterpret_cast<uint4 *>(page + PAGE_V + blk * 2048 + d * 16);
            uint4 v = *row;
            v.x &= keep[0], v.y &= keep[1], v.z &= keep[2], v.w &= keep[3];
            *row = v;
        }
    }
}

/* One landed page (64 positions starting at key0) for one warp: scores of the warp's query columns against the page's
 * K rows, the online-softmax update and the accumulation of V, as described at the top of the file. [begin, len) are
 * the attended positions (positions outside them inside the page are masked; their V bytes are zeroed in shared
 * memory first). */
template <int NT>
static __device__ __forceinline__ void attend_page(uint8_t *page, uint32_t page_u, int key0, int begin, int len,
                                                   const uint32_t (&qf)[NT][4][2],
                                                   const float (&qfac)[NT], float (&m)[NT], float (&l)[NT],
                                                   float (&oacc)[NT][8][4], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const bool partial = key0 < begin || key0 + PAGE_TOKENS > len;
    if (partial) {
        zero_v_outside(page, key0, begin, len, lane);
        __syncwarp();
    }
#pragma unroll
    for (int gi = 0; gi < 2; gi++) { /* 32 positions at a time */
        const int first = key0 + 32 * gi;
        if (partial && (first >= len || first + 32 <= begin)) continue;
        /* ---- scores: A = K rows (position 4 r + 2 mt [+ 1 for rows 8..15]), B = q ---- */
        float sc[NT][2][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int c = 0; c < 4; c++) sc[nt][mt][c] = 0.f;
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            const int row = 32 * gi + 4 * (lane & 7) + 2 * mt + ((lane >> 3) & 1);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                uint32_t a0, a1, a2, a3;
                const int c = 2 * ks + (lane >> 4);
                ldmatrix_x4(a0, a1, a2, a3, page_u + PAGE_K + row * HEAD_DIM + ((c ^ (lane & 7)) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; nt++) mma_e4m3(sc[nt][mt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
            }
        }
        /* this lane: head t of each tile, positions first + 4 g + {0, 1, 2, 3} */
        const float4 ks4 = *reinterpret_cast<const float4 *>(page + PAGE_KS + (32 * gi + 4 * g) * 4);
        const float4 vs4 = *reinterpret_cast<const float4 *>(page + PAGE_VS + (32 * gi + 4 * g) * 4);
        const float ksc[4] = {ks4.x, ks4.y, ks4.z, ks4.w}, vsc[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
        bool valid[4];
        float lv[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int pos = first + 4 * g + j;
            valid[j] = !partial || (pos >= begin && pos < len);
            lv[j] = fmaxf(lg2(vsc[j]), MIN_LOG2_VSCALE);
        }
        uint32_t pb[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float x[4], top = -INFINITY;
            bool ok[4]; /* this slot may see position j: inside the span */
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float raw = sc[nt][j >> 1][2 * (j & 1)] + sc[nt][j >> 1][2 * (j & 1) + 1] * (1.f / LO_SCALE);
                x[j] = raw * (ksc[j] * qfac[nt]);
                ok[j] = valid[j];
                top = fmaxf(top, ok[j] ? x[j] + lv[j] : -INFINITY);
            }
            top = fmaxf(head_max(top), m[nt]);
            if (__any_sync(0xffffffffu, top > m[nt])) { /* some head's maximum moved: rescale */
                const float c = m[nt] == -INFINITY ? 0.f : ex2(m[nt] - top);
                l[nt] *= c;
#pragma unroll
                for (int dt = 0; dt < 8; dt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) oacc[nt][dt][e] *= c;
                m[nt] = top;
            }
            float p[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const bool on = ok[j] && top != -INFINITY;
                const float e = on ? ex2(x[j] - top) : 0.f;
                l[nt] += e;
                p[j] = on ? e * (vsc[j] * P_SCALE) : 0.f;
            }
            uint32_t whi, wlo;
            split4(p, whi, wlo);
            /* C layout -> B layout: column g of positions 4 t .. 4 t + 3 (and + 16) lives in lane
             * 4 t + g / 2 (and + 16), first term if g is even */
            const int src = 4 * t + (g >> 1);
            const uint32_t h0 = __shfl_sync(0xffffffffu, whi, src), l0 = __shfl_sync(0xffffffffu, wlo, src);
            const uint32_t h1 = __shfl_sync(0xffffffffu, whi, src + 16), l1 = __shfl_sync(0xffffffffu, wlo, src + 16);
            pb[nt][0] = (g & 1) ? l0 : h0;
            pb[nt][1] = (g & 1) ? l1 : h1;
        }
        /* ---- values: A = V^T rows (dim 16 dt + r), B = folded probabilities ---- */
        const uint32_t vbase = page_u + PAGE_V + gi * 4096 + (lane >> 4) * 2048 + (8 * ((lane >> 3) & 1) + (lane & 7)) * 16;
#pragma unroll
        for (int dt = 0; dt < 8; dt++) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(a0, a1, a2, a3, vbase + dt * 256);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma_e4m3(oacc[nt][dt], a0, a1, a2, a3, pb[nt][0], pb[nt][1]);
        }
    }
}

/* The warp's query columns as MMA B fragments: q_stage holds S slots of 128 fp32 values (bf16-valued), q_scale each
 * slot's amax / 448. qfac[nt]: what turns lane column t's raw score into log2 units. */
template <int NT>
static __device__ __forceinline__ void query_fragments(const float *q_stage, const float *q_scale, int S, float scale_log2,
                                                       uint32_t (&qf)[NT][4][2], float (&qfac)[NT], int lane) {
    const int g = lane >> 2, t = lane & 3;
    /* B fragments of q: column g = (head g / 2 of the tile, term g % 2); b0 = dims 32 ks + 4 t .. + 3,
     * b1 = dims 32 ks + 16 + 4 t .. + 3 */
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int hc = 4 * nt + (g >> 1), hs = 4 * nt + t; /* the head of this lane's B column / C columns */
        const float sc = hc < S ? q_scale[hc] : 0.f, inv = sc > 0.f ? 1.f / sc : 0.f;
        qfac[nt] = (hs < S ? q_scale[hs] : 0.f) * scale_log2;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float x[4];
                uint32_t hi, lo;
#pragma unroll
                for (int i = 0; i < 4; i++)
                    x[i] = hc < S ? q_stage[hc * HEAD_DIM + 32 * ks + 16 * half + 4 * t + i] * inv : 0.f;
                split4(x, hi, lo);
                qf[nt][ks][half] = (g & 1) ? lo : hi;
            }
    }

}

/* APPEND: the block first does kv_append_fp8's work for its own heads of the new token (the q rows of its group
 * into shared memory; if its chunk holds the new position, the k and v rows into the cache in global memory and
 * into the landed page in shared memory), so a decode step needs no separate append launch and no round trip of q
 * through global memory. Meant for one new token per sequence; rows that share a slot need the separate kernels. */
template <int NT, bool APPEND>
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM) k_decode_attn(AttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];       /* WARPS stages of one page; later the merge area */
    __shared__ __align__(8) uint64_t bars[WARPS];          /* one "page landed" barrier per warp */
    __shared__ float q_stage[4 * NT * HEAD_DIM], q_scale[4 * NT];
    __shared__ __align__(16) uint8_t new_kv[2][HEAD_DIM]; /* APPEND: the new token's k and v bytes, natural order */
    __shared__ float new_scale[2];
    float *merge = reinterpret_cast<float *>(smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int chunk = blockIdx.x, kvh = blockIdx.y;
    const int G = a.Hq / a.Hkv;

    /* Launched with programmatic stream serialisation: what this kernel reads comes from kernels before it, and it
     * waits for them here — unless the entry point's contract says that the launch immediately before this one leaves
     * the lengths, the slot map and all but the newest cached position alone (a.early): then the block works out its
     * pages and starts its first page copies BEFORE waiting, under the predecessor's tail. */
    if (!a.early) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = (int)blockIdx.z, S = G; /* the block's row; its query slots: the heads of the kv group */
    const int given = a.lens[b];
    /* direct mode has no merge launch behind it to write the zero rows of idle, refused and empty sequences */
    auto zero_row = [&]() {
        if (a.direct && tid < HEAD_DIM)
            for (int h = 0; h < G; h++) a.direct[((size_t)b * a.Hq + (size_t)kvh * G + h) * HEAD_DIM + tid] = __float2bfloat16_rn(0.f);
    };
    if (given < 0) { /* an idle row: nothing appended, nothing attended, nothing flagged; its output is a zero row */
        zero_row();
        return;
    }
    const int len = given + a.len_add;
    const int slot = a.slot_map ? a.slot_map[b] : b;
    if (row_rejected(len, slot, a.pages_per_slot, a.n_slots, APPEND ? a.table_len : 0)) {
        if (tid == 0 && chunk == 0 && kvh == 0) flag(a.status, APPEND ? NCB_DEV_BAD_POSITION : NCB_DEV_BAD_LENGTH);
        zero_row();
        return; /* the merge kernel makes the same test and writes zeros */
    }
    const Span sp = span_of(len, a.window, a.chunk_pages);
    if (chunk >= sp.n_chunks) {
        if (chunk == 0) zero_row(); /* an empty sequence */
        return;
    }
    const int pg0 = sp.first_page + chunk * sp.chunk;
    const int n = min(sp.chunk, sp.last_page - pg0);
    if (n <= 0) {
        if (chunk == 0) zero_row();
        return;
    }

    const uint8_t *pages = a.cache + (((size_t)slot * a.Hkv + kvh) * a.pages_per_slot + pg0) * PAGE_BYTES;
    uint8_t *page = smem + (size_t)warp * PAGE_BYTES; /* this warp's stage */
    const uint32_t page_u = smem_u32(page), bar = smem_u32(bars + warp);

    /* Pages below the one that holds the newest position were written at least one step ago. The appending variant
     * may take that page early too: it patches the new token's row into the landed page anyway. */
    const bool first_now = !a.early || APPEND || pg0 + warp < (len - 1) / PAGE_TOKENS;
    if (lane == 0) { /* arm this warp's barrier and start its first page before anything else happens */
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (warp < n && first_now) page_load(page_u, pages + (size_t)warp * PAGE_BYTES, bar);
    }
    if (a.early) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0 && warp < n && !first_now) page_load(page_u, pages + (size_t)warp * PAGE_BYTES, bar);
    }
    /* the group's queries as fp32 (bf16 values) and each head's scale amax / 448 */
    const int new_page = (len - 1) / PAGE_TOKENS - pg0; /* APPEND: the chunk page that receives the new token */
    if (APPEND) {
        const int item = tid / LANES, t8 = tid % LANES, o = t8 * VEC;
        const bool owner = new_page >= 0 && new_page < n;
        if (item < G + (owner ? 2 : 0)) { /* q heads of the group, then (owner only) this kv head's k and v */
            const int p = len - 1;
            const bf16 *row = a.qkv + (size_t)b * a.qkv_row_stride;
            const int head = item < G ? kvh * G + item : item == G ? a.Hq + kvh : a.Hq + a.Hkv + kvh;
            float x1[VEC], x2[VEC];
            load_bf16x8(row + (size_t)head * HEAD_DIM + o, x1);
            load_bf16x8(row + (size_t)head * HEAD_DIM + HALF + o, x2);
            const size_t tab = (size_t)p * HALF;
            if (item < G) {
                norm_rotate(x1, x2, a.q_gain, a.cs + tab, a.sn + tab, o);
#pragma unroll
                for (int i = 0; i < VEC; i++) {
                    q_stage[item * HEAD_DIM + o + i] = x1[i];
                    q_stage[item * HEAD_DIM + HALF + o + i] = x2[i];
                }
            } else {
                const bool is_k = item == G;
                if (is_k) norm_rotate(x1, x2, a.k_gain, a.cs + tab, a.sn + tab, o);
                else if (a.ve.table) ve_mix(x1, x2, a.ve, b, kvh, a.Hkv, t8, o);
                uint8_t b1[VEC], b2[VEC];
                const float scale = quantise(x1, x2, b1, b2);
                const int j = p % PAGE_TOKENS;
                uint8_t *home = const_cast<uint8_t *>(pages) + (size_t)new_page * PAGE_BYTES; /* the cache itself */
                if (is_k) {
                    store_k_row(home, j, t8, b1, b2);
                    if (t8 == 0) reinterpret_cast<float *>(home + PAGE_KS)[j] = scale;
                } else {
                    store_v_row(home, j, t8, b1, b2);
                    if (t8 == 0) reinterpret_cast<float *>(home + PAGE_VS)[j] = scale;
                }
                memcpy(new_kv[is_k ? 0 : 1] + o, b1, VEC);
                memcpy(new_kv[is_k ? 0 : 1] + HALF + o, b2, VEC);
                if (t8 == 0) new_scale[is_k ? 0 : 1] = scale;
            }
        }
    } else {
        for (int i = tid; i < S * HEAD_DIM; i += THREADS) /* the group's heads are consecutive */
            q_stage[i] = __bfloat162float(a.q[((size_t)b * a.Hq + (size_t)kvh * G) * HEAD_DIM + i]);
    }
    __syncthreads();
    for (int h = warp; h < S; h += WARPS) {
        float m = 0.f;
        for (int i = lane; i < HEAD_DIM; i += 32) m = fmaxf(m, fabsf(q_stage[h * HEAD_DIM + i]));
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) q_scale[h] = m / 448.f;
    }
    __syncthreads();

    uint32_t qf[NT][4][2];
    float qfac[NT];
    query_fragments<NT>(q_stage, q_scale, S, a.scale_log2, qf, qfac, lane);

    /* the warp's running state: per tile, head t's maximum (log2 units), this lane's share of the sum, and O^T
     * fragments (dims 16 dt + g, + 8; columns = head t's two terms) */
    float m[NT], l[NT], oacc[NT][8][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        m[nt] = -INFINITY;
        l[nt] = 0.f;
#pragma unroll
        for (int dt = 0; dt < 8; dt++)
#pragma unroll
            for (int i = 0; i < 4; i++) oacc[nt][dt][i] = 0.f;
    }

    uint32_t phase = 0;
    for (int i = warp; i < n; phase ^= 1) {
        if (!mbar_wait(bar, phase)) {
            if (lane == 0) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
            mbar_wait(bar, phase); /* the block must not exit under a copy still in flight */
            break;
        }
        const int key0 = (pg0 + i) * PAGE_TOKENS; /* the page's first position */
        if (APPEND && i == new_page) {
            /* the copy of this page raced with the stores of the new token above: whatever it caught of that row,
             * put the row's final bytes and scales into the landed page */
            const int j = (len - 1) % PAGE_TOKENS;
            if (lane < 8)
                *reinterpret_cast<uint4 *>(page + page_k_chunk(j, lane)) = *reinterpret_cast<const uint4 *>(new_kv[0] + 16 * lane);
#pragma unroll
            for (int e = 0; e < 4; e++) page[page_v_byte(j, 4 * lane + e)] = new_kv[1][4 * lane + e];
            if (lane == 0) {
                reinterpret_cast<float *>(page + PAGE_KS)[j] = new_scale[0];
                reinterpret_cast<float *>(page + PAGE_VS)[j] = new_scale[1];
            }
            __syncwarp();
        }
        attend_page<NT>(page, page_u, key0, sp.begin, sp.len, qf, qfac, m, l, oacc, lane);
        __syncwarp(); /* every lane has read the stage */
        i += WARPS; /* a fixed page-to-warp map keeps the summation order, hence the output bits, reproducible */
        if (lane == 0 && i < n) {
            /* order this warp's reads (and the masking writes) of the stage before the copy engine's writes */
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            page_load(page_u, pages + (size_t)i * PAGE_BYTES, bar);
        }
    }
    /* the merge kernel may start occupying free SM resources now; it still waits for this grid to finish */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads(); /* every warp is done with its stage and has no copy in flight: the ring becomes the merge area */

#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int h = 4 * nt + t;
        float *mine = merge + (warp * 4 * NT + h) * PART;
        const float lsum = head_sum(l[nt]);
        if (g == 0) mine[0] = m[nt], mine[1] = lsum;
#pragma unroll
        for (int dt = 0; dt < 8; dt++) {
            mine[4 + 16 * dt + g] = (oacc[nt][dt][0] + oacc[nt][dt][1] * (1.f / LO_SCALE)) * (1.f / P_SCALE);
            mine[4 + 16 * dt + g + 8] = (oacc[nt][dt][2] + oacc[nt][dt][3] * (1.f / LO_SCALE)) * (1.f / P_SCALE);
        }
    }
    __syncthreads();
    if (tid < HEAD_DIM) { /* merge the warps' states per head; thread = dim */
        for (int h = 0; h < S; h++) {
            float top = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; w++) top = fmaxf(top, merge[(w * 4 * NT + h) * PART]);
            float lsum = 0.f, o = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) {
                const float *st = merge + (w * 4 * NT + h) * PART;
                const float c = st[0] == -INFINITY ? 0.f : ex2(st[0] - top);
                lsum += c * st[1];
                o += c * st[4 + tid];
            }
            if (a.direct) { /* the sequence's only chunk: bf16(o / l), the merge kernel's arithmetic on a single state */
                a.direct[((size_t)b * a.Hq + (size_t)kvh * G + h) * HEAD_DIM + tid] =
                    __float2bfloat16_rn(lsum > 0.f ? __fdiv_rn(o, lsum) : 0.f);
                continue;
            }
            float *out = a.parts + (((size_t)b * a.Hq + (size_t)kvh * G + h) * a.max_chunks + chunk) * PART;
            if (tid == 0) out[0] = top, out[1] = lsum;
            out[4 + tid] = o;
        }
    }
}

/* ---- prefill attention --------------------------------------------------------------------------------------- */

/* A prefill pass holds many rows of the same prompt with lengths one apart (the reference runs them through k_attn
 * row by row, model/kernels/decode.cu:859-863,1041-1051). Here a block takes a TILE of consecutive rows of one prompt
 * and one kv head and streams the prompt's pages ONCE through a ring shared by its PF_WARPS warps; a warp owns 16
 * query slots (16 / G rows x the G heads of the kv group) over the whole key range, so there are no partial states,
 * no workspace and no merge launch: the warp normalises and writes its bf16 outputs itself.
 *
 * The arithmetic differs from the decode kernel's, because here the tensor pipe, not HBM, is the limit, and on this
 * architecture every mma.sync with e4m3 operands costs four extra fp32 adds and operand shuffling around the MMA
 * itself (measured: 546 instructions per page for 32 of them). So the page's bytes are widened to f16 in registers
 * (exact: e4m3 is a subset of f16) and both contractions run as m16n8k16 f16 MMAs with the QUERY SLOTS as the M
 * dimension: scores S = Q K^T come out as (slot, key) tiles whose accumulator layout is already the A operand layout
 * of P V, so probabilities need no shuffles, and queries (bf16, exact in f16 after a power-of-two scale) and
 * probabilities (f16, 11 bits) need no two-term split. Key columns are permuted so that one lane's four
 * probabilities of a 16-key step are four consecutive positions: exactly the four V bytes an ldmatrix row hands that
 * lane. K rows are fetched as B operands by ldmatrix straight from the swizzled page (two rows of a matrix share a
 * bank group: a two-way conflict, the price of the permutation), V^T rows likewise, conflict-free.
 * The K scale multiplies the fp32 score, the V scale is folded into the probability, and the running maximum tracks
 * score + log2(v scale), as in the decode kernel.
 *
 * Page ring: PF_STAGES stages, one "landed" mbarrier each. Warps consume pages 0 .. their last page in order; the
 * LAST warp to finish with a stage (a shared counter against the number of warps that need that page) issues the
 * copy of the page PF_STAGES further on into it, so no warp is set aside as a producer. All waits are bounded. */
constexpr int PF_WARPS = 4, PF_STAGES = 4; /* 3 blocks per SM: 12 warps at 168 registers, 12 stages of 16.9 KB */
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_SLOTS = 16; /* query slots per warp: the M of the MMA */
constexpr size_t PF_SMEM = (size_t)PF_STAGES * PAGE_BYTES;

struct PrefillArgs {
    const bf16 *q;         /* [rows][Hq][128] */
    const uint8_t *cache;
    const int32_t *lens, *slot_map, *group_first, *group_rows; /* per row, per row, per block, per block */
    bf16 *out;             /* [rows][Hq][128] */
    int Hq, Hkv, n_slots, pages_per_slot;
    float scale_log2;
    int *status;
};

/* d += A B, A 16x16 f16 (row), B 16x8 f16 (col), fp32 accumulators. */
static __device__ __forceinline__ void mma_f16(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
/* The four e4m3 bytes of x as two f16x2 words (exact): lo from bytes 0, 1, hi from bytes 2, 3. */
static __device__ __forceinline__ void widen_e4m3x4(uint32_t x, uint32_t &lo, uint32_t &hi) {
    uint16_t l, h;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(l), "=h"(h) : "r"(x));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"(l));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"(h));
}
static __device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
/* max / sum over the 4 lanes that share lane / 4 (one query slot's key columns) */
static __device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
static __device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__global__ void __launch_bounds__(PF_THREADS, 3) k_prefill_attn(PrefillArgs a) {
    extern __shared__ __align__(128) uint8_t smem[]; /* the page ring */
    __shared__ __align__(8) uint64_t bars[PF_STAGES];
    __shared__ int finished[PF_STAGES]; /* warps done with the stage's current page */
    __shared__ int warp_len[PF_WARPS];  /* each warp's longest row */
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    /* blocks are dispatched in index order and the groups are listed longest-first: with the kv head as the fastest
     * index the whole launch starts its longest blocks first, not each head's in turn */
    const int group = blockIdx.x / a.Hkv, kvh = blockIdx.x % a.Hkv, G = a.Hq / a.Hkv, rpw = PF_SLOTS / G;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b0 = a.group_first[group];
    const int n_rows = min(a.group_rows[group], PF_WARPS * rpw);
    const int n_active = (n_rows + rpw - 1) / rpw; /* warps that have rows */
    const int len_block = a.lens[b0 + n_rows - 1];  /* rows ascend in position: the last one is the longest */
    const int slot = a.slot_map[b0];
    const bool bad = len_block > a.pages_per_slot * PAGE_TOKENS || slot < 0 || slot >= a.n_slots;
    if (bad && tid == 0 && kvh == 0) flag(a.status, NCB_DEV_BAD_LENGTH);
    const int n_pages = bad || len_block <= 0 ? 0 : (len_block + PAGE_TOKENS - 1) / PAGE_TOKENS;
    const uint32_t ring = smem_u32(smem);
    const uint8_t *pages = a.cache + (((size_t)(bad ? 0 : slot) * a.Hkv + kvh) * a.pages_per_slot) * PAGE_BYTES;
    auto full = [&](int st) { return smem_u32(bars + st); };
    const int r0 = b0 + warp * rpw, rows_w = max(0, min(rpw, b0 + n_rows - r0)), S = rows_w * G;
    const int my_len = rows_w > 0 && !bad ? a.lens[r0 + rows_w - 1] : 0;
    if (lane == 0) warp_len[warp] = my_len;
    if (tid == 0) {
        for (int st = 0; st < PF_STAGES; st++) {
            mbar_init(full(st), 1);
            finished[st] = 0;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < min(n_pages, PF_STAGES); i++)
            page_load(ring + i * PAGE_BYTES, pages + (size_t)i * PAGE_BYTES, full(i));
    }
    __syncthreads();
    if (warp >= n_active) return;

    /* ---- the warp's queries as A fragments: slot g (and g + 8) = row (slot / G), head (slot % G) of the group;
     * k slots (2t, 2t+1) and (2t+8, 2t+9) of step s take dims 16 s + 4 t .. + 3, the order the cache bytes arrive in */
    uint32_t qa[8][4];
    float qfac[2];
    int row_len[2];
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const int sl = g + 8 * rr;
        const bool on = sl < S;
        const int row = r0 + (on ? sl / G : 0);
        const bf16 *src = a.q + ((size_t)row * a.Hq + (size_t)kvh * G + (on ? sl % G : 0)) * HEAD_DIM + 4 * t;
        float x[8][4], amax = 0.f;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            const uint2 u = on ? *reinterpret_cast<const uint2 *>(src + 16 * s) : make_uint2(0u, 0u);
            x[s][0] = __uint_as_float(u.x << 16), x[s][1] = __uint_as_float(u.x & 0xffff0000u);
            x[s][2] = __uint_as_float(u.y << 16), x[s][3] = __uint_as_float(u.y & 0xffff0000u);
#pragma unroll
            for (int e = 0; e < 4; e++) amax = fmaxf(amax, fabsf(x[s][e]));
        }
        amax = quad_max(amax);
        /* bf16 values are exact in f16 once the row's largest magnitude is below 2^15: a power-of-two scale */
        const int expo = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
        const int down = max(0, min(expo - 14, 126));
        const float mul = __uint_as_float((uint32_t)(127 - down) << 23), back = __uint_as_float((uint32_t)(127 + down) << 23);
        qfac[rr] = a.scale_log2 * back;
        row_len[rr] = on ? a.lens[row] : 0;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            qa[s][rr] = pack_f16x2(x[s][0] * mul, x[s][1] * mul);
            qa[s][2 + rr] = pack_f16x2(x[s][2] * mul, x[s][3] * mul);
        }
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, oacc[16][4];
#pragma unroll
    for (int nd = 0; nd < 16; nd++)
#pragma unroll
        for (int e = 0; e < 4; e++) oacc[nd][e] = 0.f;

    /* ldmatrix rows of this lane. K: matrix c = lane / 8 is score tile c, whose column n = lane % 8 is the key
     * 16 (c / 2) + 4 (n / 2) + 2 (c % 2) + n % 2 of a 32-key half page; V^T: matrix = 8 dims, row = dim lane. */
    const int kc = lane >> 3, kn = lane & 7;
    const int krow = 16 * (kc >> 1) + 4 * (kn >> 1) + 2 * (kc & 1) + (kn & 1);
    const uint32_t kswz = (uint32_t)((krow >> 2) & 7) << 4;
    const int my_pages = (my_len + PAGE_TOKENS - 1) / PAGE_TOKENS;
    bool ok = true;
    for (int i = 0; i < my_pages; i++) {
        const int st = i % PF_STAGES;
        if (!mbar_wait(full(st), (i / PF_STAGES) & 1)) {
            if (lane == 0) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
            mbar_wait(full(st), (i / PF_STAGES) & 1); /* the block must not exit under a copy still in flight */
            ok = false;
            break;
        }
        uint8_t *page = smem + (size_t)st * PAGE_BYTES;
        const uint32_t page_u = ring + st * PAGE_BYTES;
        const int key0 = i * PAGE_TOKENS;
        if (key0 + PAGE_TOKENS > len_block) { /* bytes past the block's last position may be anything: zero their V */
            zero_v_outside(page, key0, 0, len_block, lane);
            __syncwarp();
        }
#pragma unroll
        for (int gi = 0; gi < 2; gi++) {
            const int first = key0 + 32 * gi;
            if (first >= my_len) continue;
            /* ---- scores: A = q, B = K rows ---- */
            float sc[4][4];
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int e = 0; e < 4; e++) sc[c][e] = 0.f;
            const uint32_t kbase = page_u + PAGE_K + (32 * gi + krow) * HEAD_DIM;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                uint32_t kr[4];
                ldmatrix_x4(kr[0], kr[1], kr[2], kr[3], kbase + (((uint32_t)s << 4) ^ kswz));
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t b0, b1;
                    widen_e4m3x4(kr[c], b0, b1);
                    mma_f16(sc[c], qa[s][0], qa[s][1], qa[s][2], qa[s][3], b0, b1);
                }
            }
            /* this lane: slots g and g + 8, positions first + 16 h + 4 t + e: tile 2 h + e / 2, column pair e % 2 */
            float ksc[2][4], vsc[2][4], lv[2][4];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float4 k4 = *reinterpret_cast<const float4 *>(page + PAGE_KS + (32 * gi + 16 * h + 4 * t) * 4);
                const float4 v4 = *reinterpret_cast<const float4 *>(page + PAGE_VS + (32 * gi + 16 * h + 4 * t) * 4);
                ksc[h][0] = k4.x, ksc[h][1] = k4.y, ksc[h][2] = k4.z, ksc[h][3] = k4.w;
                vsc[h][0] = v4.x, vsc[h][1] = v4.y, vsc[h][2] = v4.z, vsc[h][3] = v4.w;
#pragma unroll
                for (int e = 0; e < 4; e++) lv[h][e] = fmaxf(lg2(vsc[h][e]), MIN_LOG2_VSCALE);
            }
            const bool diagonal = first + 32 > min(row_len[0], row_len[1]); /* some position is masked for this lane */
            float top[2];
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                float best = -INFINITY;
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float &x = sc[2 * h + (e >> 1)][2 * rr + (e & 1)];
                        x *= ksc[h][e] * qfac[rr];
                        const bool seen = !diagonal || first + 16 * h + 4 * t + e < row_len[rr];
                        best = fmaxf(best, seen ? x + lv[h][e] : -INFINITY);
                    }
                top[rr] = fmaxf(quad_max(best), m[rr]);
            }
            if (__any_sync(0xffffffffu, top[0] > m[0] || top[1] > m[1])) { /* some slot's maximum moved: rescale */
                const float c0 = m[0] == -INFINITY ? 0.f : ex2(m[0] - top[0]);
                const float c1 = m[1] == -INFINITY ? 0.f : ex2(m[1] - top[1]);
                l[0] *= c0, l[1] *= c1;
#pragma unroll
                for (int nd = 0; nd < 16; nd++) {
                    oacc[nd][0] *= c0, oacc[nd][1] *= c0;
                    oacc[nd][2] *= c1, oacc[nd][3] *= c1;
                }
                m[0] = top[0], m[1] = top[1];
            }
            uint32_t pa[2][4]; /* per 16-key step h: A fragments of the folded probabilities */
#pragma unroll
            for (int rr = 0; rr < 2; rr++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float x = sc[2 * h + (e >> 1)][2 * rr + (e & 1)];
                        const bool seen = (!diagonal || first + 16 * h + 4 * t + e < row_len[rr]) && top[rr] != -INFINITY;
                        const float w = seen ? ex2(x - top[rr]) : 0.f;
                        l[rr] += w;
                        p[e] = seen ? w * (vsc[h][e] * P_SCALE) : 0.f;
                    }
                    pa[h][rr] = pack_f16x2(p[0], p[1]);
                    pa[h][2 + rr] = pack_f16x2(p[2], p[3]);
                }
            /* ---- values: A = probabilities, B = V^T rows (dim 8 nd + n), the lane's four positions per row ---- */
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t vbase = page_u + PAGE_V + gi * 4096 + h * 2048 + lane * 16;
#pragma unroll
                for (int qd = 0; qd < 4; qd++) {
                    uint32_t vr[4];
                    ldmatrix_x4(vr[0], vr[1], vr[2], vr[3], vbase + qd * 512);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t b0, b1;
                        widen_e4m3x4(vr[j], b0, b1);
                        mma_f16(oacc[4 * qd + j], pa[h][0], pa[h][1], pa[h][2], pa[h][3], b0, b1);
                    }
                }
            }
        }
        /* done with the stage: the last of the warps that needed this page refills it */
        __syncwarp();
        if (lane == 0) {
            int need = 0;
#pragma unroll
            for (int w = 0; w < PF_WARPS; w++) need += (w < n_active && warp_len[w] > key0) ? 1 : 0;
            __threadfence_block(); /* this warp's reads of the stage come before the count */
            if (atomicAdd(&finished[st], 1) == need - 1) {
                atomicExch(&finished[st], 0);
                if (i + PF_STAGES < n_pages) {
                    __threadfence_block();
                    /* the warps' reads and masking writes of the stage come before the copy engine's writes */
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    page_load(page_u, pages + (size_t)(i + PF_STAGES) * PAGE_BYTES, full(st));
                }
            }
        }
    }
    /* ---- normalise and store: slot g's (and g + 8's) dims 8 nd + 2 t, + 1 ---- */
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const int sl = g + 8 * rr;
        const float lsum = quad_sum(l[rr]);
        if (sl >= S) continue;
        const float inv = ok && lsum > 0.f ? __fdiv_rn(1.f, lsum * P_SCALE) : 0.f;
        bf16 *dst = a.out + ((size_t)(r0 + sl / G) * a.Hq + (size_t)kvh * G + sl % G) * HEAD_DIM + 2 * t;
#pragma unroll
        for (int nd = 0; nd < 16; nd++)
            *reinterpret_cast<__nv_bfloat162 *>(dst + 8 * nd) =
                __floats2bfloat162_rn(oacc[nd][2 * rr] * inv, oacc[nd][2 * rr + 1] * inv);
    }
}

/* ---- merge kernel ------------------------------------------------------------------------------------------- */

struct MergeArgs {
    const float *parts;
    long long rows, part_stride, row_stride; /* state (row, p) at parts + row * row_stride + p * part_stride */
    int n_parts;                             /* > 0: fixed; 0: from lens (the split kernel's chunks) */
    const int32_t *lens, *slot_map;
    int Hq, window, chunk_pages, n_slots, pages_per_slot, max_chunks, len_add;
    bf16 *out;       /* [rows][128] normalised, or NULL */
    float *part_out; /* [rows][PART] merged state, or NULL */
    int table_len;   /* > 0: rows longer than this were refused by the appending split kernel */
};

/* How many chunk states the split kernel left for `row`: 0 for idle and refused rows. */
static __device__ __forceinline__ int states_of(const MergeArgs &a, long long row) {
    if (a.n_parts > 0) return a.n_parts;
    const int b = (int)(row / a.Hq), given = a.lens[b], slot = a.slot_map ? a.slot_map[b] : b;
    if (given < 0) return 0;
    const int len = given + a.len_add;
    if (row_rejected(len, slot, a.pages_per_slot, a.n_slots, a.table_len)) return 0;
    return min(span_of(len, a.window, a.chunk_pages).n_chunks, a.max_chunks);
}

constexpr int MERGE_WARPS = 4;      /* rows with at most 16 states */
constexpr int MERGE_WARPS_WIDE = 8; /* rows with more: every warp still gets its states in one batch of loads */

/* The states of one row folded by a block of W warps: warp w folds states w, w + W, ... into a running
 * state (its loads are independent of the fold, so they overlap), then warp 0 merges the W running states through
 * shared memory. Lane = four output dims. Returns true in warp 0, whose lanes then hold the row's un-normalised state
 * (top in log2 units, lsum, acc); the other warps are done. */
template <int W>
static __device__ __forceinline__ bool merge_row_states(const MergeArgs &a, long long row, float &top, float &lsum,
                                                        float4 &acc) {
    __shared__ float sm[W], sl[W];
    __shared__ float4 so[W][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = states_of(a, row);
    const float *st = a.parts + row * a.row_stride;
    top = -INFINITY, lsum = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int DEPTH = 4; /* states loaded before the first is folded: the loads' latencies overlap */
    for (int p0 = warp; p0 < n; p0 += W * DEPTH) {
        float mp[DEPTH], lp[DEPTH];
        float4 o[DEPTH];
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            const int p = p0 + i * W;
            if (p < n) {
                const float *s = st + p * a.part_stride;
                mp[i] = s[0], lp[i] = s[1];
                o[i] = *reinterpret_cast<const float4 *>(s + 4 + 4 * lane);
            }
        }
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (p0 + i * W < n) { /* folded in index order, as a one-at-a-time loop would */
                const float next = fmaxf(top, mp[i]);
                const float c0 = top == -INFINITY ? 0.f : ex2(top - next), c1 = mp[i] == -INFINITY ? 0.f : ex2(mp[i] - next);
                lsum = lsum * c0 + lp[i] * c1;
                acc.x = acc.x * c0 + o[i].x * c1, acc.y = acc.y * c0 + o[i].y * c1;
                acc.z = acc.z * c0 + o[i].z * c1, acc.w = acc.w * c0 + o[i].w * c1;
                top = next;
            }
        }
    }
    if (lane == 0) sm[warp] = top, sl[warp] = lsum;
    so[warp][lane] = acc;
    __syncthreads();
    if (warp != 0) return false;
    top = sm[0];
#pragma unroll
    for (int w = 1; w < W; w++) top = fmaxf(top, sm[w]);
    lsum = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < W; w++) {
        const float c = sm[w] == -INFINITY ? 0.f : ex2(sm[w] - top);
        const float4 o = so[w][lane];
        lsum += c * sl[w];
        acc.x += c * o.x, acc.y += c * o.y, acc.z += c * o.z, acc.w += c * o.w;
    }
    return true;
}

/* out[row][4 lane .. 4 lane + 3] = acc / lsum as bf16 (the reference's __fdiv_rn then round, decode.cu:674); a row
 * without any position gives zeros. */
static __device__ __forceinline__ void store_normalised(bf16 *out, long long row, int lane, float lsum, const float4 &acc) {
    const bool any = lsum > 0.f;
    const float x = any ? __fdiv_rn(acc.x, lsum) : 0.f, y = any ? __fdiv_rn(acc.y, lsum) : 0.f;
    const float z = any ? __fdiv_rn(acc.z, lsum) : 0.f, w = any ? __fdiv_rn(acc.w, lsum) : 0.f;
    uint2 u;
    *reinterpret_cast<__nv_bfloat162 *>(&u.x) = __floats2bfloat162_rn(x, y);
    *reinterpret_cast<__nv_bfloat162 *>(&u.y) = __floats2bfloat162_rn(z, w);
    *reinterpret_cast<uint2 *>(out + row * HEAD_DIM + 4 * lane) = u;
}

/* One block of W warps per row. */
template <int W>
__global__ void __launch_bounds__(W * 32) k_merge(MergeArgs a) {
    const long long row = blockIdx.x;
    const int lane = threadIdx.x & 31;
    /* launched with programmatic stream serialisation: wait here until the grid before it (the split kernel, whose
     * states this reads) has completed and its writes are visible; a no-op after an ordinary launch */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float top, lsum;
    float4 acc;
    if (!merge_row_states<W>(a, row, top, lsum, acc)) return;
    if (a.part_out) {
        float *o = a.part_out + row * PART;
        if (lane == 0) *reinterpret_cast<float4 *>(o) = make_float4(top, lsum, 0.f, 0.f);
        *reinterpret_cast<float4 *>(o + 4 + 4 * lane) = acc;
    }
    if (a.out) store_normalised(a.out, row, lane, lsum, acc);
}

/* ---- merge + exchange over peer memory ------------------------------------------------------------------------ */

constexpr int MAX_PEERS = 8;
constexpr uint32_t PEER_WAIT_POLLS = 1u << 22; /* x ~100 ns each: roughly half a second */
constexpr int PACKET_WORDS = NCB_PEER_STATE_BYTES / 8; /* one state as 8-byte (fp32 value, call number) words */
static_assert(PACKET_WORDS >= HEAD_DIM + 2, "o[128], then m and l");

/* Every rank owns an "inbox" [2][world][rows][PACKET_WORDS] of 8-byte words that all peers can address, and a private
 * device word pair `epoch` = (calls completed, blocks arrived in the current call). */
struct ExchangeArgs {
    MergeArgs local;         /* this rank's chunk states (the split kernel's workspace) */
    uint2 *inbox[MAX_PEERS]; /* rank q's inbox */
    int world, rank;
    uint32_t *epoch;
    int *status;
};

/* 16 bytes = two (value, call number) words, read in one piece. Volatile: each poll goes to memory. */
static __device__ __forceinline__ uint4 load_packet_pair(const uint2 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

/* The chunk merge of k_merge and the cross-GPU exchange in one launch, one block per row: merge the row's local chunk
 * states, PUSH the rank state into every other rank's inbox with plain stores over NVLink (one direction, no read
 * round trip), then read the other ranks' states of the same row from this rank's own inbox and merge in rank order,
 * so every rank computes bit-identical outputs. A state travels as self-validating 8-byte words (fp32 value, call
 * number), the scheme of low-latency collectives: an 8-byte store lands whole, so a word whose second half equals the
 * current call number holds this call's value; no flags, no fences, nothing ordered after the data. The receiver
 * polls its own memory (bounded) until every word of a state carries the call number. Rows are independent: a block
 * waits only for the same row's blocks on the other GPUs, never for blocks of its own grid.
 * The call number comes from a device word the kernel itself advances (the last block to finish bumps it), so the
 * launch arguments never change and the step can be captured in a CUDA graph. Inboxes alternate between two halves by
 * the call's parity: a rank can run at most one call ahead of a peer (it needs the peer's words of call e to finish
 * call e), so what it writes never lands in a half a slower peer still reads, and a word left by call e - 2 in the
 * same half never passes for call e. */
template <int W>
__global__ void __launch_bounds__(W * 32) k_merge_exchange(ExchangeArgs a) {
    const long long row = blockIdx.x, rows = a.local.rows;
    const int lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.wait;" ::: "memory"); /* this rank's chunk states are complete and visible */
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(a.epoch) + 1u;
    float top, lsum;
    float4 acc;
    if (!merge_row_states<W>(a.local, row, top, lsum, acc)) return;
    const size_t half = (size_t)(epoch & 1u) * a.world * rows * PACKET_WORDS;
    const size_t mine = half + ((size_t)a.rank * rows + row) * PACKET_WORDS;
    const uint4 w01 = make_uint4(__float_as_uint(acc.x), epoch, __float_as_uint(acc.y), epoch);
    const uint4 w23 = make_uint4(__float_as_uint(acc.z), epoch, __float_as_uint(acc.w), epoch);
    const uint4 wml = make_uint4(__float_as_uint(top), epoch, __float_as_uint(lsum), epoch);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; q++) {
        if (q < a.world && q != a.rank) {
            uint2 *o = a.inbox[q] + mine;
            *reinterpret_cast<uint4 *>(o + 4 * lane) = w01;
            *reinterpret_cast<uint4 *>(o + 4 * lane + 2) = w23;
            if (lane == 0) *reinterpret_cast<uint4 *>(o + HEAD_DIM) = wml;
        }
    }
    /* the other ranks' states of this row, from this rank's own inbox */
    float mq[MAX_PEERS], lq[MAX_PEERS];
    float4 oq[MAX_PEERS];
    bool ok = true;
#pragma unroll
    for (int q = 0; q < MAX_PEERS; q++) {
        if (q >= a.world) continue;
        if (q == a.rank) {
            mq[q] = top, lq[q] = lsum, oq[q] = acc;
            continue;
        }
        const uint2 *in = a.inbox[a.rank] + half + ((size_t)q * rows + row) * PACKET_WORDS;
        uint4 r01 = make_uint4(0u, 0u, 0u, 0u), r23 = r01, rml = r01;
        bool got = false;
        for (uint32_t polls = 0; polls < PEER_WAIT_POLLS && ok; polls++) {
            r01 = load_packet_pair(in + 4 * lane);
            r23 = load_packet_pair(in + 4 * lane + 2);
            rml = load_packet_pair(in + HEAD_DIM);
            got = r01.y == epoch && r01.w == epoch && r23.y == epoch && r23.w == epoch && rml.y == epoch && rml.w == epoch;
            if (__all_sync(0xffffffffu, got)) break;
            got = false;
            __nanosleep(64);
        }
        if (!__all_sync(0xffffffffu, got)) ok = false; /* the remaining ranks are not waited for either */
        mq[q] = __uint_as_float(rml.x), lq[q] = __uint_as_float(rml.z);
        oq[q] = make_float4(__uint_as_float(r01.x), __uint_as_float(r01.z), __uint_as_float(r23.x), __uint_as_float(r23.z));
    }
    if (!ok && lane == 0) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
    top = -INFINITY;
#pragma unroll
    for (int q = 0; q < MAX_PEERS; q++)
        if (q < a.world) top = fmaxf(top, mq[q]);
    lsum = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; q++) {
        if (q < a.world) {
            const float c = mq[q] == -INFINITY ? 0.f : ex2(mq[q] - top);
            lsum += c * lq[q];
            acc.x += c * oq[q].x, acc.y += c * oq[q].y, acc.z += c * oq[q].z, acc.w += c * oq[q].w;
        }
    }
    if (ok) store_normalised(a.local.out, row, lane, lsum, acc);
    if (lane == 0) { /* the last row to finish closes the call */
        __threadfence();
        if (atomicAdd(a.epoch + 1, 1u) == (uint32_t)rows - 1u) {
            a.epoch[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(a.epoch) = epoch;
        }
    }
}

/* ---- host side ---------------------------------------------------------------------------------------------- */

/* Host-side facts remembered per device ordinal, under one lock (entry points may be called from several threads). */
static std::mutex g_device_lock;
constexpr int MAX_DEVICES = 64;

static int sm_count() { /* of the current device */
    static int count[MAX_DEVICES] = {};
    int device = 0, c = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return 148;
    std::lock_guard<std::mutex> guard(g_device_lock);
    if (!count[device]) {
        if (cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || c <= 0) c = 148;
        count[device] = c;
    }
    return count[device];
}

static int pages_of(int len) { return (len + PAGE_TOKENS - 1) / PAGE_TOKENS; }

/* The new token's inputs for the appending variant (kv_append_fp8's arguments). */
struct AppendIn {
    const void *qkv, *q_gain, *k_gain, *cos, *sin;
    long long qkv_row_stride;
    int table_len;
    ValueEmbed ve;
};

template <int NT, bool APPEND> static cudaError_t prepare() { /* opt in to the large dynamic shared memory, once per device */
    static bool done[MAX_DEVICES] = {};
    int device = 0;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess) return rc;
    std::lock_guard<std::mutex> guard(g_device_lock);
    if (device >= 0 && device < MAX_DEVICES && done[device]) return cudaSuccess;
    rc = cudaFuncSetAttribute(k_decode_attn<NT, APPEND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)ATTN_SMEM);
    if (rc == cudaSuccess && device >= 0 && device < MAX_DEVICES) done[device] = true;
    return rc;
}

static int launch_split(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *workspace,
                        long long workspace_bytes, int B, int Hq, int Hkv, int n_slots, int pages_per_slot,
                        int max_kv_len, int window, int &chunk_pages, float softmax_scale, void *status,
                        cudaStream_t stream, const AppendIn *app = nullptr, bool early = false, void *direct_out = nullptr) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || n_slots <= 0 || pages_per_slot <= 0 || max_kv_len < 0 ||
        window < 0 || chunk_pages < 0 || !(softmax_scale > 0.f))
        return NCB_ERR_ARG;
    if (Hq / Hkv > 8) return NCB_ERR_UNSUPPORTED;
    if (B > 65535 || Hkv > 65535) return NCB_ERR_ARG;
    /* the default chunk follows the caller's max_kv_len, as decode_attn_workspace_bytes() computed it, before the
     * bound is clipped to the cache: the workspace the caller sized is then never too small */
    if (chunk_pages == 0) chunk_pages = decode_attn_chunk_pages(B, Hkv, max_kv_len);
    if (max_kv_len > pages_per_slot * PAGE_TOKENS) max_kv_len = pages_per_slot * PAGE_TOKENS;
    if (B == 0) return NCB_OK;
    if ((!q && !app) || !kv_cache || !lens || !workspace) return NCB_ERR_ARG;
    if (((uintptr_t)q | (uintptr_t)kv_cache | (uintptr_t)workspace) % 16 != 0) return NCB_ERR_ALIGN;
    if (app) {
        if (!app->qkv || !app->q_gain || !app->k_gain || !app->cos || !app->sin || app->table_len <= 0 ||
            app->qkv_row_stride < (long long)(Hq + 2 * Hkv) * HEAD_DIM)
            return NCB_ERR_ARG;
        const uintptr_t all = (uintptr_t)app->qkv | (uintptr_t)app->q_gain | (uintptr_t)app->k_gain |
                              (uintptr_t)app->cos | (uintptr_t)app->sin;
        if (all % 16 != 0 || app->qkv_row_stride % 8 != 0) return NCB_ERR_ALIGN;
        const ValueEmbed &ve = app->ve;
        if (ve.table) {
            if (!ve.h || !ve.tokens || !ve.gate || ve.C <= 0 || ve.C % 256 || ve.vocab <= 0) return NCB_ERR_ARG;
            if (((uintptr_t)ve.h | (uintptr_t)ve.table | (uintptr_t)ve.gate) % 16 || (uintptr_t)ve.tokens % 8)
                return NCB_ERR_ALIGN;
        }
    }
    if (workspace_bytes < decode_attn_workspace_bytes(B, Hq, max_kv_len, Hkv, chunk_pages)) return NCB_ERR_WORKSPACE;
    const int max_chunks = max(1, (pages_of(max_kv_len) + chunk_pages - 1) / chunk_pages);
    AttnArgs a = {(const bf16 *)q, (const uint8_t *)kv_cache, (const int32_t *)lens, (const int32_t *)slot_map,
                  (float *)workspace, B, Hq, Hkv, n_slots, pages_per_slot, window, chunk_pages, max_chunks,
                  softmax_scale * 1.4426950408889634f, (int *)status, app ? 1 : 0, (app || early) ? 1 : 0};
    if (app) {
        a.qkv = (const bf16 *)app->qkv, a.q_gain = (const float *)app->q_gain, a.k_gain = (const float *)app->k_gain;
        a.cs = (const float *)app->cos, a.sn = (const float *)app->sin;
        a.qkv_row_stride = app->qkv_row_stride, a.table_len = app->table_len;
        a.ve = app->ve;
    }
    a.direct = max_chunks == 1 ? (bf16 *)direct_out : nullptr; /* only a sequence's sole chunk may write the output */
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(max_chunks, Hkv, B);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = ATTN_SMEM;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaError_t rc;
    if (Hq / Hkv <= 4 && !app) {
        if (prepare<1, false>() != cudaSuccess) return NCB_ERR_LAUNCH;
        rc = cudaLaunchKernelEx(&config, k_decode_attn<1, false>, a);
    } else if (!app) {
        if (prepare<2, false>() != cudaSuccess) return NCB_ERR_LAUNCH;
        rc = cudaLaunchKernelEx(&config, k_decode_attn<2, false>, a);
    } else if (Hq / Hkv <= 4) {
        if (prepare<1, true>() != cudaSuccess) return NCB_ERR_LAUNCH;
        rc = cudaLaunchKernelEx(&config, k_decode_attn<1, true>, a);
    } else {
        if (prepare<2, true>() != cudaSuccess) return NCB_ERR_LAUNCH;
        rc = cudaLaunchKernelEx(&config, k_decode_attn<2, true>, a);
    }
    return rc == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

static int launch_merge(const MergeArgs &a, cudaStream_t stream) {
    if (a.rows == 0) return NCB_OK;
    const long long blocks = a.rows; /* a block per row */
    if (blocks > 0x7fffffffLL) return NCB_ERR_ARG;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)blocks);
    const bool wide = a.n_parts == 0 ? a.max_chunks > 4 * MERGE_WARPS : a.n_parts > 4 * MERGE_WARPS;
    config.blockDim = dim3((wide ? MERGE_WARPS_WIDE : MERGE_WARPS) * 32);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1; /* overlap its launch with the split kernel's tail */
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t rc = wide ? cudaLaunchKernelEx(&config, k_merge<MERGE_WARPS_WIDE>, a)
                                : cudaLaunchKernelEx(&config, k_merge<MERGE_WARPS>, a);
    return rc == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

/* What the merge + exchange launch needs besides the local merge (decode_attn_fp8_sharded). */
struct ExchangeIn {
    void *const *inbox;
    int world, rank;
    void *epoch;
};

static int launch_exchange(const MergeArgs &m, const ExchangeIn &x, void *status, cudaStream_t stream) {
    ExchangeArgs a = {};
    a.local = m;
    for (int q = 0; q < x.world; q++) a.inbox[q] = (uint2 *)x.inbox[q];
    a.world = x.world, a.rank = x.rank, a.epoch = (uint32_t *)x.epoch, a.status = (int *)status;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)m.rows);
    const bool wide = m.n_parts == 0 ? m.max_chunks > 4 * MERGE_WARPS : m.n_parts > 4 * MERGE_WARPS;
    config.blockDim = dim3((wide ? MERGE_WARPS_WIDE : MERGE_WARPS) * 32);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t rc = wide ? cudaLaunchKernelEx(&config, k_merge_exchange<MERGE_WARPS_WIDE>, a)
                                : cudaLaunchKernelEx(&config, k_merge_exchange<MERGE_WARPS>, a);
    return rc == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

static int attend(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *workspace,
                  long long workspace_bytes, void *out, void *part_out, int B, int Hq, int Hkv, int n_slots,
                  int pages_per_slot, int max_kv_len, int window, int chunk_pages, float softmax_scale, void *status,
                  void *stream, const AppendIn *app = nullptr, const ExchangeIn *exchange = nullptr) {
    if (!out && !part_out) return NCB_ERR_ARG;
    if (((uintptr_t)out | (uintptr_t)part_out) % 16 != 0) return NCB_ERR_ALIGN;
    /* One chunk per sequence (short caches, or a chunk size at least the cache's pages): the split kernel's blocks
     * normalise and write the output themselves and there is no merge launch (launch_split takes `out` only then). */
    void *direct = (out && !part_out && !exchange) ? out : nullptr;
    const int rc = launch_split(q, kv_cache, lens, slot_map, workspace, workspace_bytes, B, Hq, Hkv, n_slots,
                                pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status,
                                (cudaStream_t)stream, app, exchange != nullptr, direct);
    if (rc != NCB_OK || B == 0) return rc;
    if (max_kv_len > pages_per_slot * PAGE_TOKENS) max_kv_len = pages_per_slot * PAGE_TOKENS;
    const int max_chunks = max(1, (pages_of(max_kv_len) + chunk_pages - 1) / chunk_pages);
    if (direct && max_chunks == 1) return NCB_OK;
    MergeArgs m = {(const float *)workspace, (long long)B * Hq, PART, (long long)max_chunks * PART, 0,
                   (const int32_t *)lens, (const int32_t *)slot_map, Hq, window, chunk_pages, n_slots, pages_per_slot,
                   max_chunks, app ? 1 : 0, (bf16 *)out, (float *)part_out, app ? app->table_len : 0};
    if (exchange) return launch_exchange(m, *exchange, status, (cudaStream_t)stream);
    return launch_merge(m, (cudaStream_t)stream);
}

/* ---- built-in scratch for callers that cannot allocate ------------------------------------------------------- */

/* The per-chunk states of decode_attn_fp8_static. In host code this name is only a handle for
 * cudaGetSymbolAddress; the kernels get the device address that call returns. */
static __device__ __align__(256) unsigned char g_static_scratch[NCB_STATIC_SCRATCH_BYTES];

/* The array's address on the current device, looked up once per device. */
static int static_scratch(void **ptr) {
    static void *address[MAX_DEVICES] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return NCB_ERR_LAUNCH;
    std::lock_guard<std::mutex> guard(g_device_lock);
    if (!address[device]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return NCB_ERR_LAUNCH;
        address[device] = p;
    }
    *ptr = address[device];
    return NCB_OK;
}

/*
 * Chunk size by a model of how the split kernel's blocks fill the GPU. Blocks are dispatched in grid order (chunk
 * fastest, then kv head, then sequence) to `slots` resident places; a block with p pages takes BLOCK_US + PAGE_US *
 * ceil(p / WARPS) (its warps walk their pages one after the other), a block beyond its sequence's chunks IDLE_US.
 * The modelled makespan tracks the measured kernel time up to a constant (the bytes' own streaming time) across
 * chunk sizes, batch shapes and ragged lengths, including the steps where one more wave of blocks appears; the
 * chunk size with the smallest makespan wins, the larger one on ties (fewer states to merge). A chunk size that leaves
 * every sequence ONE chunk is spared the merge launch (the blocks write the output themselves), but the model gives
 * that no credit: on a 12-page cache three pages per warp in one launch measured slower (604 us per d20 step) than one
 * page per warp and a merge launch (552 - 572 us). lens == NULL takes
 * every sequence as max_kv_len long. Chunks stay between one page per warp and 32 pages (longer ones gain nothing
 * and unbalance ragged batches).
 */
static int plan_chunk_pages(const int *lens, int B, int Hkv, int max_kv_len, int window) {
    constexpr double BLOCK_US = 2.0, PAGE_US = 1.2, IDLE_US = 0.3;
    const int slots = BLOCKS_PER_SM * sm_count(), max_pages = pages_of(max_kv_len);
    if (max_pages <= WARPS) return WARPS;
    std::vector<int> pages(B);
    for (int b = 0; b < B; b++) {
        int len = lens ? lens[b] : max_kv_len;
        len = len < 0 ? 0 : len > max_kv_len ? max_kv_len : len;
        const int begin = (window > 0 && len > window) ? len - window : 0;
        pages[b] = pages_of(len) - begin / PAGE_TOKENS;
    }
    int best = WARPS;
    double best_cost = 0.;
    std::vector<double> heap;
    /* launches of more than 32,768 blocks are many waves deep: whole waves of the mean sequence stand in for the
     * dispatch simulation there, which keeps the planner itself under a few milliseconds */
    const bool simulate = (long long)B * Hkv * ((max_pages + WARPS - 1) / WARPS) <= 32768;
    long long total_pages = 0;
    for (int b = 0; b < B; b++) total_pages += pages[b];
    const int mean_pages = (int)((total_pages + B - 1) / B);
    for (int c = WARPS; c <= 32; c++) {
        const int max_chunks = (max_pages + c - 1) / c;
        double end = 0.;
        if (!simulate) {
            const int n = (mean_pages + c - 1) / c, each = n ? (mean_pages + n - 1) / n : 0;
            const long long busy = (long long)B * Hkv * n, idle = (long long)B * Hkv * (max_chunks - n);
            end = (double)((busy + slots - 1) / slots) * (BLOCK_US + PAGE_US * ((each + WARPS - 1) / WARPS)) +
                  (double)idle / slots * IDLE_US;
        } else {
            heap.assign(slots, 0.);
            for (int b = 0; b < B; b++) {
                const int n = (pages[b] + c - 1) / c, each = n ? (pages[b] + n - 1) / n : 0;
                for (int h = 0; h < Hkv; h++)
                    for (int i = 0; i < max_chunks; i++) {
                        const int first = i * each, p = i < n ? (pages[b] - first < each ? pages[b] - first : each) : 0;
                        std::pop_heap(heap.begin(), heap.end(), std::greater<double>());
                        double &t = heap.back();
                        t += p > 0 ? BLOCK_US + PAGE_US * ((p + WARPS - 1) / WARPS) : IDLE_US;
                        if (t > end) end = t;
                        std::push_heap(heap.begin(), heap.end(), std::greater<double>());
                    }
            }
        }
        if (c == WARPS || end <= best_cost) best = c, best_cost = end;
    }
    return best;
}

extern "C" {

int decode_attn_plan_chunk_pages(const int *lens, int B, int Hkv, int max_kv_len, int window) {
    if (B <= 0 || Hkv <= 0 || max_kv_len <= 0) return 1;
    return plan_chunk_pages(lens, B, Hkv, max_kv_len, window);
}

int decode_attn_chunk_pages(int B, int Hkv, int max_kv_len) {
    if (B <= 0 || Hkv <= 0 || max_kv_len <= 0) return 1;
    /* every sequence taken as max_kv_len long; remembered, since eager callers ask on every call. The answer
     * depends on the current device's SM count, so that is part of the key. */
    static std::mutex lock;
    static std::map<std::array<int, 4>, int> known;
    const std::array<int, 4> key = {sm_count(), B, Hkv, max_kv_len};
    std::lock_guard<std::mutex> guard(lock);
    auto hit = known.find(key);
    if (hit != known.end()) return hit->second;
    const int c = plan_chunk_pages(nullptr, B, Hkv, max_kv_len, 0);
    if (known.size() < 4096) known.emplace(key, c);
    return c;
}

long long decode_attn_workspace_bytes(int B, int Hq, int max_kv_len, int Hkv, int chunk_pages) {
    if (B < 0 || Hq <= 0 || Hkv <= 0 || max_kv_len < 0 || chunk_pages < 0) return -1;
    if (chunk_pages == 0) chunk_pages = decode_attn_chunk_pages(B, Hkv, max_kv_len);
    const long long max_chunks = max(1, (pages_of(max_kv_len) + chunk_pages - 1) / chunk_pages);
    return (long long)B * Hq * max_chunks * PART * (long long)sizeof(float);
}

int decode_attn_fp8(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *workspace,
                    long long workspace_bytes, void *out, int B, int Hq, int Hkv, int n_slots, int pages_per_slot,
                    int max_kv_len, int window, int chunk_pages, float softmax_scale, void *status, void *stream) {
    if (!out && B > 0) return NCB_ERR_ARG;
    return attend(q, kv_cache, lens, slot_map, workspace, workspace_bytes, out, nullptr, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream);
}

int decode_attn_fp8_partial(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                            void *workspace, long long workspace_bytes, void *part_out, int B, int Hq, int Hkv,
                            int n_slots, int pages_per_slot, int max_kv_len, int window, int chunk_pages,
                            float softmax_scale, void *status, void *stream) {
    if (!part_out && B > 0) return NCB_ERR_ARG;
    return attend(q, kv_cache, lens, slot_map, workspace, workspace_bytes, nullptr, part_out, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream);
}

int decode_attn_fp8_static(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *out,
                           int B, int Hq, int Hkv, int n_slots, int pages_per_slot, int max_kv_len, int window,
                           int chunk_pages, float softmax_scale, void *status, void *stream) {
    if (!out && B > 0) return NCB_ERR_ARG;
    if (B < 0 || Hq <= 0 || Hkv <= 0 || pages_per_slot <= 0 || max_kv_len < 0 || chunk_pages < 0) return NCB_ERR_ARG;
    if (chunk_pages == 0) chunk_pages = decode_attn_chunk_pages(B, Hkv, max_kv_len);
    if (max_kv_len > pages_per_slot * PAGE_TOKENS) max_kv_len = pages_per_slot * PAGE_TOKENS;
    const long long need = decode_attn_workspace_bytes(B, Hq, max_kv_len, Hkv, chunk_pages);
    if (need > (long long)NCB_STATIC_SCRATCH_BYTES) return NCB_ERR_STATIC_LIMIT;
    void *scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc != NCB_OK) return rc;
    return attend(q, kv_cache, lens, slot_map, scratch, NCB_STATIC_SCRATCH_BYTES, out, nullptr, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream);
}

int decode_step_attn_fp8(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                         const void *pos, const void *slot_map, void *kv_cache, void *workspace,
                         long long workspace_bytes, void *out, int B, int Hq, int Hkv, long long qkv_row_stride,
                         int table_len, int n_slots, int pages_per_slot, int max_kv_len, int window, int chunk_pages,
                         float softmax_scale, void *status, void *stream) {
    if (!out && B > 0) return NCB_ERR_ARG;
    const AppendIn app = {qkv, q_gain, k_gain, cos, sin, qkv_row_stride, table_len};
    return attend(nullptr, kv_cache, pos, slot_map, workspace, workspace_bytes, out, nullptr, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream, &app);
}

int decode_step_attn_fp8_ve(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                            const void *pos, const void *slot_map, void *kv_cache, void *workspace,
                            long long workspace_bytes, void *out, int B, int Hq, int Hkv, long long qkv_row_stride,
                            int table_len, int n_slots, int pages_per_slot, int max_kv_len, int window,
                            int chunk_pages, float softmax_scale, const void *h, const void *tokens,
                            const void *ve_table, const void *ve_gate, int C, int vocab, void *status, void *stream) {
    if (!out && B > 0) return NCB_ERR_ARG;
    AppendIn app = {qkv, q_gain, k_gain, cos, sin, qkv_row_stride, table_len};
    app.ve = {(const bf16 *)h, (const long long *)tokens, (const bf16 *)ve_table, (const float *)ve_gate, C, vocab};
    return attend(nullptr, kv_cache, pos, slot_map, workspace, workspace_bytes, out, nullptr, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream, &app);
}

int prefill_attn_rows_per_block(int Hq, int Hkv) {
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > PF_SLOTS) return 0;
    return PF_WARPS * (PF_SLOTS / (Hq / Hkv));
}

int prefill_attn_fp8(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                     const void *group_first, const void *group_rows, int n_groups, void *out, long long rows, int Hq,
                     int Hkv, int n_slots, int pages_per_slot, float softmax_scale, void *status, void *stream) {
    if (rows < 0 || n_groups < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || n_slots <= 0 || pages_per_slot <= 0 ||
        !(softmax_scale > 0.f))
        return NCB_ERR_ARG;
    if (Hq / Hkv > PF_SLOTS) return NCB_ERR_UNSUPPORTED;
    if (rows == 0 || n_groups == 0) return NCB_OK;
    if (!q || !kv_cache || !lens || !slot_map || !group_first || !group_rows || !out ||
        (long long)n_groups * Hkv > 0x7fffffffLL)
        return NCB_ERR_ARG;
    if (((uintptr_t)q | (uintptr_t)kv_cache | (uintptr_t)out) % 16 != 0) return NCB_ERR_ALIGN;
    {
        static bool done[MAX_DEVICES] = {};
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return NCB_ERR_LAUNCH;
        std::lock_guard<std::mutex> guard(g_device_lock);
        if (!done[device]) {
            if (cudaFuncSetAttribute(k_prefill_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM) != cudaSuccess)
                return NCB_ERR_LAUNCH;
            done[device] = true;
        }
    }
    PrefillArgs a = {(const bf16 *)q, (const uint8_t *)kv_cache, (const int32_t *)lens, (const int32_t *)slot_map,
                     (const int32_t *)group_first, (const int32_t *)group_rows, (bf16 *)out, Hq, Hkv, n_slots, pages_per_slot,
                     softmax_scale * 1.4426950408889634f, (int *)status};
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)((long long)n_groups * Hkv));
    config.blockDim = dim3(PF_THREADS);
    config.dynamicSmemBytes = PF_SMEM;
    config.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, k_prefill_attn, a) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

int decode_attn_fp8_split(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                          void *workspace, long long workspace_bytes, int B, int Hq, int Hkv, int n_slots,
                          int pages_per_slot, int max_kv_len, int window, int chunk_pages, float softmax_scale,
                          void *status, void *stream) {
    return launch_split(q, kv_cache, lens, slot_map, workspace, workspace_bytes, B, Hq, Hkv, n_slots, pages_per_slot,
                        max_kv_len, window, chunk_pages, softmax_scale, status, (cudaStream_t)stream);
}

int decode_attn_fp8_sharded(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                            void *workspace, long long workspace_bytes, void *out, int B, int Hq, int Hkv, int n_slots,
                            int pages_per_slot, int max_kv_len, int window, int chunk_pages, float softmax_scale,
                            void *const *inbox, int world, int rank, void *epoch, void *status, void *stream) {
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) return NCB_ERR_ARG;
    if (B == 0) return NCB_OK; /* every rank passes the same B: nobody sends, nobody waits */
    if (!out || !inbox || !epoch) return NCB_ERR_ARG;
    for (int r = 0; r < world; r++) {
        if (!inbox[r]) return NCB_ERR_ARG;
        if ((uintptr_t)inbox[r] % 16) return NCB_ERR_ALIGN;
    }
    if ((uintptr_t)epoch % 8) return NCB_ERR_ALIGN;
    const ExchangeIn x = {inbox, world, rank, epoch};
    return attend(q, kv_cache, lens, slot_map, workspace, workspace_bytes, out, nullptr, B, Hq, Hkv, n_slots,
                  pages_per_slot, max_kv_len, window, chunk_pages, softmax_scale, status, stream, nullptr, &x);
}

int decode_attn_merge(const void *parts, int n_parts, long long rows, void *out, void *stream) {
    if (n_parts <= 0 || rows < 0) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!parts || !out) return NCB_ERR_ARG;
    if (((uintptr_t)parts | (uintptr_t)out) % 16 != 0) return NCB_ERR_ALIGN;
    MergeArgs m = {(const float *)parts, rows, rows * PART, PART, n_parts, nullptr, nullptr, 1, 0, 1, 1, 1, n_parts, 0,
                   (bf16 *)out, nullptr, 0};
    return launch_merge(m, (cudaStream_t)stream);
}

} /* extern "C" */
