/*
 * Shared by stream_gemm.cu and tile_gemm.cu: PTX wrappers for the Blackwell tensor-core path (mbarriers, TMA boxes,
 * tcgen05 matrix descriptors, MMAs, commits and tensor-memory loads) and the host-side cache of TMA tensor maps.
 * Everything here has internal linkage: each library gets its own copy.
 */
#pragma once

#include "ncb_common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int KBLK = 64;                         /* k-values per box: 64 bf16 = one 128-byte swizzle row */
constexpr long long WAIT_CYCLES = 4000000000ll;  /* bound of every barrier wait */

/* ---- PTX wrappers ------------------------------------------------------------------------------------------- */

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
/* True once the barrier's phase of the given parity has completed. Polls without a suspend hint (one thread feeds the
 * whole pipeline, so a late wake-up stalls it) and gives up after WAIT_CYCLES of the SM clock, about two seconds. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const long long start = clock64();
    for (;;) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (done) return true;
        if (clock64() - start > WAIT_CYCLES) return false;
    }
}
/* One box of a 2-d tensor map into shared memory; (c0, c1) = (k, row) element coordinates, c0 a multiple of 64.
 * `policy` is an L2 eviction policy: weights are read once (evict first), activations by every block (evict last). */
__device__ __forceinline__ void tma_load(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
                 "[%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
/* A contiguous run of global memory into L2; 16-byte aligned, a multiple of 16 bytes. */
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
/* Shared-memory matrix descriptor of a K-major tile of 128-byte rows with the 128-byte swizzle: 8-row groups are
 * 1024 bytes apart (stride byte offset), the leading byte offset is unused for this layout, descriptor version 1. */
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
/* D[tmem] (+)= A[smem] . B[smem]^T, bf16 operands, fp32 accumulate, M 128, N from the instruction descriptor, K 16. */
__device__ __forceinline__ void umma_bf16(uint32_t tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
/* The barrier gets one arrival when every MMA issued so far by this thread has completed. */
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
/* 32 consecutive fp32 columns of this thread's tensor-memory lane. */
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float *v) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                   "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                   "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

/* ---- host side: tensor maps ----------------------------------------------------------------------------------- */

typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/* The driver's tensor-map encoder, looked up through the runtime so that the library does not link libcuda. */
EncodeTiled encoder() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiled)p;
    }();
    return fn;
}

/* Tensor map of a row-major bf16 matrix [rows][K] read in boxes of box_rows x 64 with the 128-byte swizzle; rows of
 * a box beyond the matrix read as zero. A map depends only on (pointer, shape, box), so maps are cached. */
bool tensor_map(const void *base, int rows, int K, int box_rows, CUtensorMap *out) {
    struct Key {
        const void *p;
        int rows, K, box;
        bool operator==(const Key &o) const { return p == o.p && rows == o.rows && K == o.K && box == o.box; }
    };
    struct Hash {
        size_t operator()(const Key &k) const {
            size_t h = (size_t)(uintptr_t)k.p;
            h = h * 1000003u ^ (size_t)k.rows;
            h = h * 1000003u ^ (size_t)k.K;
            return h * 1000003u ^ (size_t)k.box;
        }
    };
    static std::mutex lock;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    const Key key = {base, rows, K, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto hit = cache.find(key);
    if (hit != cache.end()) {
        *out = hit->second;
        return true;
    }
    EncodeTiled encode = encoder();
    if (!encode) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {KBLK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 8192) cache.clear(); /* activations of eager callers come and go */
    cache.emplace(key, *out);
    return true;
}

} /* namespace */
