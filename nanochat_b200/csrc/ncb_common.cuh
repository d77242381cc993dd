/*
 * Shared by kv_append.cu and decode_attn.cu: the page layout of the fp8 KV cache (described in
 * include/nanochat_b200.h), status codes and small device helpers.
 */
#pragma once

#include <float.h>
#include <stdint.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/nanochat_b200.h"

typedef __nv_bfloat16 bf16;

constexpr int HEAD_DIM = NCB_HEAD_DIM;
constexpr int HALF = HEAD_DIM / 2;
constexpr int PAGE_TOKENS = NCB_PAGE_TOKENS;
constexpr int PAGE_BYTES = NCB_PAGE_BYTES;
constexpr int PAGE_K = 0;                                /* K rows, 64 x 128 B, 16-byte chunks swizzled */
constexpr int PAGE_V = PAGE_TOKENS * HEAD_DIM;           /* V transposed: [group][half][dim][16] */
constexpr int PAGE_KS = 2 * PAGE_TOKENS * HEAD_DIM;      /* fp32 K scales */
constexpr int PAGE_VS = PAGE_KS + PAGE_TOKENS * 4;       /* fp32 V scales */
static_assert(PAGE_VS + PAGE_TOKENS * 4 == PAGE_BYTES, "page layout");
static_assert(PAGE_BYTES % 128 == 0, "pages stay 128-byte aligned");

/* Byte offset, inside a page, of K's 16-byte chunk c (dims 16c..16c+15) of in-page position j. */
static __host__ __device__ __forceinline__ int page_k_chunk(int j, int c) {
    return PAGE_K + j * HEAD_DIM + ((c ^ ((j >> 2) & 7)) << 4);
}
/* Byte offset, inside a page, of V's byte for in-page position j and dim d. */
static __host__ __device__ __forceinline__ int page_v_byte(int j, int d) {
    return PAGE_V + (j >> 5) * 4096 + ((j >> 4) & 1) * 2048 + d * 16 + (j & 15);
}

static __device__ __forceinline__ void flag(int *status, int bit) {
    if (status) atomicOr(status, bit);
}

constexpr int PART = NCB_PART_FLOATS; /* one (m, l, 2 pad, o[128]) attention state, fp32 */

static __device__ __forceinline__ float ex2(float x) { /* exp2, -inf -> 0 */
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

/* Where a sequence's attended positions and pages lie; shared by the split kernel and everything that merges its states. */
struct Span {
    int begin, len, first_page, last_page; /* positions [begin, len), pages [first_page, last_page) */
    int n_chunks, chunk;                   /* the pages cut into n_chunks runs of `chunk` pages (the last may be shorter) */
};
/* chunk_pages is an upper bound: a sequence takes the fewest chunks that respect it and then evens them out, so no
 * block is left with a stub (129 pages at 27 per chunk are 5 chunks of 26, 26, 26, 26, 25). */
static __device__ __forceinline__ Span span_of(int len, int window, int chunk_pages) {
    Span s;
    s.len = len;
    s.begin = (window > 0 && len > window) ? len - window : 0;
    s.first_page = s.begin / PAGE_TOKENS;
    s.last_page = (len + PAGE_TOKENS - 1) / PAGE_TOKENS;
    const int pages = s.last_page - s.first_page;
    s.n_chunks = (pages + chunk_pages - 1) / chunk_pages;
    s.chunk = s.n_chunks > 0 ? (pages + s.n_chunks - 1) / s.n_chunks : 0;
    return s;
}

