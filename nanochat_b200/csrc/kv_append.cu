/*
 * kv_append_fp8: fused rotary + QK-RMSNorm + per-(token, head) scale + e4m3 pack + append into the paged cache.
 * Replaces the reference's k_prologue (model/kernels/decode.cu:551-565; row math model/kernels/qk_row.cuh:26-51)
 * for an fp8 cache and Hq != Hkv.
 *
 * Work item = one head row of 128 values (a q, k or v head of one token), handled by 8 lanes; lane t owns dims
 * 8t..8t+7 and their rotation partners 64+8t..64+8t+7, the ownership of qk_row.cuh:11-12,44-50. A 128-thread block
 * holds the same head row of 16 consecutive tokens, so that a prefill pass (runs of consecutive positions of one
 * slot) can store its transposed V bytes as 16-byte chunks. At decode sizes the kernel is bound by launch latency
 * and a few KB of traffic per token; it is written for exactness: every fp32 operation is an explicit round-to-nearest intrinsic in the order of
 * oracle/kv_append_oracle.c (no FMA contraction, sqrt + divide instead of rsqrtf), which makes q bits, cache
 * bytes and scales exact functions of the inputs.
 */
#include "kv_row.cuh"

constexpr int BLOCK = 128;
constexpr int ROWS_PER_BLOCK = BLOCK / LANES; /* 16: one run of V positions that share 16-byte chunks */
static_assert(ROWS_PER_BLOCK == 16 && BLOCK == HEAD_DIM, "a V run is 16 positions and the block has a thread per dim");

namespace {

struct AppendArgs {
    const bf16 *qkv;
    const float *q_gain, *k_gain, *cs, *sn;
    const int32_t *pos, *slot_map;
    bf16 *q_out;
    uint8_t *cache;
    long long rows, qkv_row_stride;
    int Hq, Hkv, table_len, n_slots, pages_per_slot;
    int *status;
    ValueEmbed ve; /* table == NULL: no value embedding on this layer */
    int heads_per_block;
};

/* Block (x, y) = rows 16 x .. 16 x + 15 of the head rows y hpb .. y hpb + hpb - 1 (q heads, then k heads, then v heads);
 * 8 lanes per row. A block of a large pass walks over several head rows: positions, slots and the run test are
 * done once, the rows' rotary entries stay in L1 between heads, and the next head's inputs are in flight while the
 * current one is computed. */
__global__ void __launch_bounds__(BLOCK, 6) k_kv_append(AppendArgs a) {
    /* launched with programmatic stream serialisation: wait for the kernel that produced qkv and pos, then let the
     * next kernel's launch overlap this one (it waits the same way before it reads the cache or q) */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ __align__(16) uint8_t vt[HEAD_DIM][ROWS_PER_BLOCK]; /* a V run transposed: [dim][position] */
    const int g = threadIdx.x / LANES, t = threadIdx.x % LANES, o = t * VEC;
    const long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK, row = row0 + g;
    const bool live = row < a.rows;
    int p = 0, slot = 0;
    bool valid = false;
    if (live) {
        p = a.pos[row];
        slot = a.slot_map ? a.slot_map[row] : (int)row;
        valid = !(p < 0 || p >= a.table_len || p >= a.pages_per_slot * PAGE_TOKENS || slot < 0 || slot >= a.n_slots);
        /* a negative position marks an idle row (skipped silently); anything else outside the cache is flagged */
        if (!valid && p >= 0 && t == 0 && blockIdx.y == 0) flag(a.status, NCB_DEV_BAD_POSITION);
    }
    /* A prefill pass appends runs of consecutive positions of one slot. When the block's 16 rows are such a run and
     * start on a 16-position boundary, their V bytes of one dim are 16 contiguous bytes of the page: they are
     * transposed through shared memory and stored as 128 16-byte chunks (2 KB contiguous) instead of 2,048 single
     * bytes. Any other block (decode steps, ragged edges) stores byte by byte. Same bytes either way. */
    const int p0 = a.pos[row0], slot0 = a.slot_map ? a.slot_map[row0] : (int)row0;
    const bool run = __syncthreads_and(live && valid && slot == slot0 && p == p0 + g && p0 % ROWS_PER_BLOCK == 0);
    const bool on = live && valid; /* the same for the 8 lanes of a row; nobody leaves before the loop's barriers */
    const int heads = a.Hq + 2 * a.Hkv, first = blockIdx.y * a.heads_per_block;
    const int last = min(first + a.heads_per_block, heads);
    const bf16 *x = a.qkv + (on ? row : 0) * a.qkv_row_stride;
    const size_t tab = (size_t)(on ? p : 0) * HALF;
    const int j = p % PAGE_TOKENS;
    uint4 raw1 = make_uint4(0, 0, 0, 0), raw2 = raw1;
    if (on && first < last) {
        raw1 = *reinterpret_cast<const uint4 *>(x + (size_t)first * HEAD_DIM + o);
        raw2 = *reinterpret_cast<const uint4 *>(x + (size_t)first * HEAD_DIM + HALF + o);
    }
    for (int which = first; which < last; which++) {
        float x1[VEC], x2[VEC];
        unpack_bf16x8(raw1, x1);
        unpack_bf16x8(raw2, x2);
        if (on && which + 1 < last) { /* the next head row's inputs start now */
            raw1 = *reinterpret_cast<const uint4 *>(x + (size_t)(which + 1) * HEAD_DIM + o);
            raw2 = *reinterpret_cast<const uint4 *>(x + (size_t)(which + 1) * HEAD_DIM + HALF + o);
        }
        const bool is_q = which < a.Hq, is_k = !is_q && which < a.Hq + a.Hkv, is_v = !is_q && !is_k;
        const int head = is_q ? which : is_k ? which - a.Hq : which - a.Hq - a.Hkv;
        uint8_t *page = a.cache + (((size_t)(on ? slot : 0) * a.Hkv + (is_q ? 0 : head)) * a.pages_per_slot +
                                   (on ? p / PAGE_TOKENS : 0)) * PAGE_BYTES;
        uint8_t b1[VEC], b2[VEC];
        if (on) {
            if (!is_v) norm_rotate(x1, x2, is_q ? a.q_gain : a.k_gain, a.cs + tab, a.sn + tab, o);
            else if (a.ve.table) ve_mix(x1, x2, a.ve, row, head, a.Hkv, t, o);
            if (is_q) {
                bf16 *q = a.q_out + ((size_t)row * a.Hq + head) * HEAD_DIM;
                *reinterpret_cast<uint4 *>(q + o) = pack_bf16x8(x1);
                *reinterpret_cast<uint4 *>(q + HALF + o) = pack_bf16x8(x2);
            } else {
                const float scale = quantise(x1, x2, b1, b2);
                if (t == 0) reinterpret_cast<float *>(page + (is_k ? PAGE_KS : PAGE_VS))[j] = scale;
                if (is_k) store_k_row16(page, j, t, b1, b2);
                else if (!run) store_v_row(page, j, t, b1, b2);
            }
        }
        if (is_v && run) { /* block-uniform: every thread of the block is in the run */
            /* a dim's 16 positions are four words; word k of dim d sits at word k ^ ((d >> 3) & 3), which spreads the
             * eight lanes of a row (dims 8 apart, else all on one bank) over four banks */
            const int col = g ^ ((t & 3) << 2);
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                vt[o + i][col] = b1[i];
                vt[HALF + o + i][col] = b2[i];
            }
            __syncthreads();
            const int d = threadIdx.x, j0 = j - g; /* the run's first in-page position; thread = dim */
            const uint32_t *w = reinterpret_cast<const uint32_t *>(vt[d]);
            const int sw = (d >> 3) & 3;
            *reinterpret_cast<uint4 *>(page + page_v_byte(j0, d)) = make_uint4(w[sw], w[1 ^ sw], w[2 ^ sw], w[3 ^ sw]);
            __syncthreads(); /* the next v head row reuses the tile */
        }
    }
}

} /* namespace */

extern "C" {

const char *ncb_status_string(int status) {
    switch (status) {
    case NCB_OK: return "ok";
    case NCB_ERR_ARG: return "invalid argument";
    case NCB_ERR_ALIGN: return "misaligned pointer or stride";
    case NCB_ERR_WORKSPACE: return "workspace too small";
    case NCB_ERR_LAUNCH: return "kernel launch failed";
    case NCB_ERR_UNSUPPORTED: return "unsupported shape (head ratio, tile width)";
    case NCB_ERR_STATIC_LIMIT: return "needs more than the built-in scratch";
    default: return "unknown status";
    }
}

int kv_cache_pages(int max_len) { return max_len <= 0 ? 0 : (max_len + PAGE_TOKENS - 1) / PAGE_TOKENS; }

long long kv_cache_bytes(int n_slots, int kv_heads, int max_len) {
    if (n_slots < 0 || kv_heads < 0 || max_len < 0) return -1;
    return (long long)n_slots * kv_heads * kv_cache_pages(max_len) * PAGE_BYTES;
}

} /* extern "C" */

static int launch_append(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                         const void *pos, const void *slot_map, void *q_out, void *kv_cache, long long rows, int Hq,
                         int Hkv, long long qkv_row_stride, int table_len, int n_slots, int pages_per_slot, void *status,
                         void *stream, const ValueEmbed &ve) {
    if (rows < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || table_len <= 0 || n_slots <= 0 || pages_per_slot <= 0)
        return NCB_ERR_ARG;
    if (qkv_row_stride < (long long)(Hq + 2 * Hkv) * HEAD_DIM) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!qkv || !q_gain || !k_gain || !cos || !sin || !pos || !q_out || !kv_cache) return NCB_ERR_ARG;
    const uintptr_t all = (uintptr_t)qkv | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)cos | (uintptr_t)sin |
                          (uintptr_t)q_out | (uintptr_t)kv_cache;
    if (all % 16 != 0 || qkv_row_stride % 8 != 0) return NCB_ERR_ALIGN;
    if (ve.table) {
        if (!ve.h || !ve.tokens || !ve.gate || ve.C <= 0 || ve.C % 256 || ve.vocab <= 0) return NCB_ERR_ARG;
        if (((uintptr_t)ve.h | (uintptr_t)ve.table | (uintptr_t)ve.gate) % 16 || (uintptr_t)ve.tokens % 8) return NCB_ERR_ALIGN;
    }
    const long long blocks = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    if (blocks > 0x7fffffffLL || Hq + 2 * Hkv > 65535) return NCB_ERR_ARG;
    /* small passes (decode steps): one head row per block, as many blocks as possible; large passes (prefill): a block
     * walks over up to 8 head rows as long as about 2,048 blocks remain, enough to fill every SM several times */
    const int heads = Hq + 2 * Hkv;
    long long hpb = blocks * heads / 2048;
    hpb = hpb < 1 ? 1 : hpb > 8 ? 8 : hpb;
    AppendArgs a = {(const bf16 *)qkv, (const float *)q_gain, (const float *)k_gain, (const float *)cos,
                    (const float *)sin, (const int32_t *)pos, (const int32_t *)slot_map, (bf16 *)q_out,
                    (uint8_t *)kv_cache, rows, qkv_row_stride, Hq, Hkv, table_len, n_slots, pages_per_slot,
                    (int *)status, ve, (int)hpb};
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)blocks, (unsigned)((heads + hpb - 1) / hpb));
    config.blockDim = dim3(BLOCK);
    config.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, k_kv_append, a) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

extern "C" {

int kv_append_fp8(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                  const void *pos, const void *slot_map, void *q_out, void *kv_cache, long long rows, int Hq,
                  int Hkv, long long qkv_row_stride, int table_len, int n_slots, int pages_per_slot, void *status,
                  void *stream) {
    return launch_append(qkv, q_gain, k_gain, cos, sin, pos, slot_map, q_out, kv_cache, rows, Hq, Hkv, qkv_row_stride,
                         table_len, n_slots, pages_per_slot, status, stream, ValueEmbed{});
}

int kv_append_fp8_ve(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                     const void *pos, const void *slot_map, void *q_out, void *kv_cache, long long rows, int Hq,
                     int Hkv, long long qkv_row_stride, int table_len, int n_slots, int pages_per_slot, const void *h,
                     const void *tokens, const void *ve_table, const void *ve_gate, int C, int vocab, void *status,
                     void *stream) {
    const ValueEmbed ve = {(const bf16 *)h, (const long long *)tokens, (const bf16 *)ve_table, (const float *)ve_gate, C,
                           vocab};
    return launch_append(qkv, q_gain, k_gain, cos, sin, pos, slot_map, q_out, kv_cache, rows, Hq, Hkv, qkv_row_stride,
                         table_len, n_slots, pages_per_slot, status, stream, ve);
}

} /* extern "C" */
