/*
 * y = epilogue(x . W^T) for any number of activation rows on Blackwell's tcgen05 tensor cores: the GEMMs of prefill
 * passes (thousands of prompt rows) and of decode steps above 64 sequences. Replaces, for sm_100a, the reference's
 * Hopper-only slot GEMM k_wgmma with its STORE / RESID / RELU2 epilogues when it runs prompt rows
 * (model/kernels/decode.cu:232-359, driven by dec_prefill, decode.cu:1041-1051) and stands where a library GEMM would.
 *
 * With hundreds of rows the weights are re-used enough for the tensor cores to be the bound, so this is a classic
 * tiled GEMM rather than a weight stream (stream_gemm.cu): D[128 rows][BN features] = x tile (A operand, M = 128) .
 * W tile^T (B operand, N = BN = 256, or 128 for widths that are not a multiple of 256), both K-major bf16, fp32
 * accumulators in tensor memory. One persistent block per SM walks over the output tiles:
 *   - warp 0, one thread: TMA producer. Per 64-wide k-block one box of x (128 rows) and one of W (BN rows) into a ring
 *     of shared-memory stages (cp.async.bulk.tensor, 128-byte swizzle, no multicast), one mbarrier per stage;
 *   - warp 1, one thread: issues tcgen05.mma.cta_group::1.kind::f16 (four K = 16 steps per k-block), releases stages
 *     with tcgen05.commit, and signals a finished accumulator. Tensor memory holds TWO accumulators (2 x BN columns), so
 *     the MMAs of the next tile run while the epilogue drains the previous one;
 *   - warps 2..5: epilogue. Warp w owns the 32 tensor-memory lanes (= rows) its rank allows (w % 4), a thread reads
 *     its row 32 columns at a time (tcgen05.ld), applies the epilogue and writes 64 contiguous bytes.
 * Tiles are dealt to the blocks round-robin; when the last round would occupy at most half of the blocks, its tiles
 * are cut into two half-width units each (N = BN / 2 MMAs on the same stages), which shortens that round to about half.
 * Rows beyond the matrix are zero-filled by TMA on the way in and masked on the way out. The parameter-free RMS norm
 * of the inputs is not fused here: passes of this size keep the normed rows in memory anyway (add_rms_norm).
 * Every mbarrier wait is bounded; on expiry NCB_DEV_WAIT_TIMEOUT is flagged, every role abandons its remaining tiles
 * and the block still frees its tensor memory.
 */
#include "umma.cuh"

namespace {

constexpr int BM = 128;          /* rows per tile = MMA M */
constexpr int THREADS = 192;     /* producer warp, MMA warp, four epilogue warps */
constexpr int A_BYTES = BM * KBLK * 2;

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_RELU2 = 2, EPI_F32 = 3 };

template <int BN> struct Tile {
    static constexpr int B_BYTES = BN * KBLK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          /* 48 KB (BN 256) or 32 KB (BN 128) */
    static constexpr int STAGES = BN == 256 ? 4 : 6;               /* 192 KB of ring either way */
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = 1024 + RING_BYTES + 256;     /* 1024: the ring is aligned by hand; 256: barriers */
    static constexpr int TMEM_COLS = 2 * BN;                       /* two accumulators */
};

struct TileArgs {
    const bf16 *resid; /* [rows][N] for EPI_RESID (may alias y) */
    void *y;           /* [rows][N] bf16, or fp32 for EPI_F32 */
    int rows, N, K;
    int *status;
    int split_from; /* tiles from this index on are worked on as two half-width units each (= tiles: none) */
};

/* A unit of work: a tile, or half of one. */
struct Unit {
    int m0, n0, width;
};

/* Grid = min(tiles, SMs); block b takes units b, b + grid, ...; tile t = (row tile t / n_tiles, feature tile t % n_tiles),
 * so blocks that run at the same time share the x rows and cover neighbouring feature tiles. When the last round of
 * tiles would fill at most half of the blocks (`split_from` < tiles), each of its tiles is cut into two half-width
 * units, so that the round takes about half as long: units [0, split_from) are whole tiles, unit split_from + h is
 * half h % 2 of tile split_from + h / 2. */
template <int BN>
static __device__ __forceinline__ Unit unit_of(int u, int n_tiles, int split_from) {
    if (u < split_from) return {(u / n_tiles) * BM, (u % n_tiles) * BN, BN};
    const int h = u - split_from, t = split_from + h / 2;
    return {(t / n_tiles) * BM, (t % n_tiles) * BN + (h & 1) * (BN / 2), BN / 2};
}

/* The epilogue on 32 consecutive fp32 products of one row, written at element offset `at` of y. */
template <int EPI> static __device__ __forceinline__ void store_columns(const TileArgs &a, size_t at, const float *v) {
    if (EPI == EPI_F32) {
        float4 *out = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.y) + at);
#pragma unroll
        for (int j = 0; j < 8; j++) out[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        uint4 res[4];
        if (EPI == EPI_RESID) {
            const uint4 *r = reinterpret_cast<const uint4 *>(a.resid + at);
#pragma unroll
            for (int j = 0; j < 4; j++) res[j] = r[j];
        }
        uint4 packed[4];
        bf16 *o = reinterpret_cast<bf16 *>(packed);
        const bf16 *rr = reinterpret_cast<const bf16 *>(res);
#pragma unroll
        for (int j = 0; j < 32; j++) {
            bf16 out = __float2bfloat16_rn(v[j]);
            if (EPI == EPI_RESID) out = __float2bfloat16_rn(__bfloat162float(rr[j]) + __bfloat162float(out));
            if (EPI == EPI_RELU2) {
                const float p = fmaxf(__bfloat162float(out), 0.f);
                out = __float2bfloat16_rn(p * p);
            }
            o[j] = out;
        }
        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<bf16 *>(a.y) + at);
#pragma unroll
        for (int j = 0; j < 4; j++) dst[j] = packed[j];
    }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS, 1) k_tile_gemm(const __grid_constant__ CUtensorMap map_x,
                                                          const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_w_half, const TileArgs a) {
    using T = Tile<BN>;
    constexpr int STAGES = T::STAGES;
    extern __shared__ uint8_t raw[];
    const uint32_t raw_addr = smem_u32(raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u; /* swizzled tiles sit on 1024-byte boundaries */
    uint8_t *tail = raw + (ring - raw_addr) + T::RING_BYTES;
    const uint32_t bars = ring + T::RING_BYTES; /* full[STAGES], empty[STAGES], acc_full[2], acc_empty[2] */
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 192);
    volatile int *failed = reinterpret_cast<volatile int *>(tail + 200);
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = a.N / BN, m_tiles = (a.rows + BM - 1) / BM, tiles = n_tiles * m_tiles;
    const int split_from = a.split_from, units = split_from + 2 * (tiles - split_from);
    const int nkb = a.K / KBLK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4); /* one arrival per epilogue warp */
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(T::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    /* x and resid come from the kernel before this one; W does not, but a tile needs both operands */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) { /* producer */
            const uint64_t w_policy = policy_evict_last(), x_policy = policy_evict_last(); /* both are re-read by other tiles */
            uint32_t g = 0; /* k-blocks issued so far, over all of this block's tiles */
            for (int u = blockIdx.x; u < units && !*failed; u += gridDim.x) {
                const Unit un = unit_of<BN>(u, n_tiles, split_from);
                const bool whole = un.width == BN;
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    if (!mbar_wait(empty(s), ((g / STAGES) & 1) ^ 1)) {
                        flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                        *failed = 1;
                        break;
                    }
                    mbar_expect_tx(full(s), A_BYTES + (whole ? T::B_BYTES : T::B_BYTES / 2));
                    tma_load(ring + s * T::STAGE_BYTES, &map_x, kb * KBLK, un.m0, full(s), x_policy);
                    tma_load(ring + s * T::STAGE_BYTES + A_BYTES, whole ? &map_w : &map_w_half, kb * KBLK, un.n0, full(s),
                             w_policy);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) { /* MMA issuer */
            constexpr uint32_t IDESC_BASE = (1u << 4) /* fp32 accumulators */ | (1u << 7) /* A bf16 */ | (1u << 10) /* B bf16 */
                                            | ((uint32_t)(BM >> 4) << 24); /* both K-major; N goes to bits 17.. */
            uint32_t g = 0, it = 0;
            for (int u = blockIdx.x; u < units && !*failed; u += gridDim.x, it++) {
                const uint32_t buf = it & 1;
                const uint32_t idesc = IDESC_BASE | ((uint32_t)(unit_of<BN>(u, n_tiles, split_from).width >> 3) << 17);
                if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1) ^ 1)) { /* the epilogue has drained this accumulator */
                    flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                    *failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    ok = mbar_wait(full(s), (g / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = ring + s * T::STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < KBLK / 16; k++) /* 16 k-values = 32 bytes further along the swizzled row */
                        umma_bf16(acc, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0);
                    umma_commit(empty(s));
                }
                if (!ok) {
                    flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                    *failed = 1;
                    break;
                }
                umma_commit(acc_full(buf));
            }
        }
    } else { /* epilogue warps 2..5: tensor-memory lanes 32 (warp % 4) .. + 31 */
        const int quarter = warp & 3;
        uint32_t it = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, it++) {
            const uint32_t buf = it & 1;
            const Unit un = unit_of<BN>(u, n_tiles, split_from);
            const int m0 = un.m0, n0 = un.n0;
            if (*failed || !mbar_wait(acc_full(buf), (it >> 1) & 1)) {
                if (!*failed && lane == 0) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                *failed = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const bool live = row < a.rows;
            const size_t base = (size_t)row * a.N + n0;
#pragma unroll 1
            for (int c = 0; c < un.width / 32; c++) {
                float v[32];
                tmem_load32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c * 32, v);
                if (!live) continue;
                store_columns<EPI>(a, base + c * 32, v);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(T::TMEM_COLS) : "memory");
}


/* ---- the same GEMM on block pairs (tcgen05 cta_group::2) ----------------------------------------------------------- */

constexpr bool PAIR_BY_DEFAULT = true;

/* Two blocks on neighbouring SMs (a cluster of two) work on ONE 256-row x 256-feature tile: each block stages its own
 * 128 rows of x and its own 128 of the 256 W rows, the leader's single thread issues tcgen05.mma.cta_group::2 (M 256),
 * which multiplies both blocks' x rows by the W rows of BOTH blocks' shared memory, and each block's tensor memory
 * receives its own 128 rows of the product. Per 64-wide k-block a block then loads 32 KB for 128 x 256 x 64 products
 * instead of 48 KB, which is what the single-block form runs short of (its operand loads, not its MMAs, set its pace).
 *   - producers (one thread per block): TMA boxes into the block's own ring; both blocks' copies report their bytes to
 *     the LEADER's "stage full" barrier (a tensor copy with .cta_group::2 may signal the peer's barrier; every block
 *     loads its own boxes, nothing is broadcast);
 *   - MMA thread (leader only): waits for a full stage, issues the four K = 16 steps, and releases the stage in both
 *     blocks with one tcgen05.commit addressed to both blocks of the pair; the same for a finished accumulator;
 *   - epilogue warps (both blocks): as in the single-block kernel on the block's own 128 rows; every warp of both blocks
 *     then arrives on the leader's "accumulator drained" barrier (eight arrivals).
 * The pair leaves together (cluster barrier) after the last tile, then frees its tensor memory. All waits bounded. */
/* A pair's tile is 256 rows x WIDTH features, WIDTH = NSUB * NMMA: NSUB MMAs of N = NMMA per K = 16 step into
 * neighbouring accumulator columns. <256, 1> is the standard tile; <160, 2> (320 wide, one accumulator) exists for
 * widths like 1280, where 256-wide tiles leave a last round that is nearly empty (80 tiles for 74 pairs) and 320-wide
 * tiles fit one round (64). Of an MMA's NMMA W rows each block stages NMMA / 2. */
template <int NMMA, int NSUB> struct Pair {
    static constexpr int WIDTH = NMMA * NSUB;
    static constexpr int SUB_BYTES = (NMMA / 2) * KBLK * 2;        /* this block's W rows of one MMA */
    static constexpr int B_BYTES = NSUB * SUB_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          /* 32 KB (256 wide) or 36 KB (320 wide) */
    static constexpr int STAGES = 6;
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = 1024 + RING_BYTES + 256;
    static constexpr int ACCS = 2 * WIDTH <= 512 ? 2 : 1;          /* accumulators in tensor memory */
    static constexpr int TMEM_COLS = 512;
    static_assert(SUB_BYTES % 1024 == 0 && NMMA % 32 == 0 && NMMA <= 256 && WIDTH <= 512, "swizzle atoms, MMA shape");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
/* The address of this block's shared-memory location `addr` in block `rank` of the cluster. */
__device__ __forceinline__ uint32_t in_block(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
/* tma_load whose barrier may live in the pair's other block (`bar` is a shared::cluster address). */
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
                 "[%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
/* One arrival on the barrier at this offset in BOTH blocks of the pair once every MMA issued so far has completed. */
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

/* A pair's unit: a 256 x WIDTH tile, or (NSUB == 1, last round) one of its two halves. */
template <int WIDTH> static __device__ __forceinline__ Unit pair_unit_of(int u, int n_tiles, int split_from) {
    if (u < split_from) return {(u / n_tiles) * 2 * BM, (u % n_tiles) * WIDTH, WIDTH};
    const int h = u - split_from, t = split_from + h / 2;
    return {(t / n_tiles) * 2 * BM, (t % n_tiles) * WIDTH + (h & 1) * (WIDTH / 2), WIDTH / 2};
}

template <int NMMA, int NSUB, int EPI>
__global__ void __launch_bounds__(THREADS, 1) k_tile_gemm_pair(const __grid_constant__ CUtensorMap map_x,
                                                               const __grid_constant__ CUtensorMap map_w,
                                                               const __grid_constant__ CUtensorMap map_w_half, const TileArgs a) {
    using P = Pair<NMMA, NSUB>;
    constexpr int STAGES = P::STAGES, WIDTH = P::WIDTH, ACCS = P::ACCS;
    extern __shared__ uint8_t raw[];
    const uint32_t raw_addr = smem_u32(raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u;
    uint8_t *tail = raw + (ring - raw_addr) + P::RING_BYTES;
    const uint32_t bars = ring + P::RING_BYTES; /* full[STAGES], empty[STAGES], acc_full[2], acc_empty[2] */
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 192);
    volatile int *failed = reinterpret_cast<volatile int *>(tail + 200);
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    /* the `it`-th unit of this pair uses accumulator it % ACCS; it is the (it / ACCS)-th use of that accumulator */
    auto acc_of = [](uint32_t it) { return ACCS == 2 ? (it & 1u) : 0u; };
    auto use_of = [](uint32_t it) { return ACCS == 2 ? (it >> 1) : it; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank(); /* 0: the pair's leader */
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles = a.N / WIDTH, m_tiles = (a.rows + 2 * BM - 1) / (2 * BM), tiles = n_tiles * m_tiles;
    const int split_from = a.split_from, units = split_from + 2 * (tiles - split_from);
    const int nkb = a.K / KBLK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full(s), 1);  /* the leader producer's arrival; both blocks' copies add their bytes */
            mbar_init(empty(s), 1); /* the pair-wide commit */
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 8); /* four epilogue warps in each block */
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) { /* the same warp in both blocks: the allocation covers both blocks' tensor memory */
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(P::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all(); /* the peer's barriers exist before anything signals them */
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) { /* producer: this block's x rows and W rows */
            const uint64_t w_policy = policy_evict_last(), x_policy = policy_evict_last();
            uint32_t g = 0;
            for (int u = pair; u < units && !*failed; u += n_pairs) {
                const Unit un = pair_unit_of<WIDTH>(u, n_tiles, split_from);
                const bool whole = un.width == WIDTH;
                const int b_bytes = whole ? P::B_BYTES : P::B_BYTES / 2;
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    if (!mbar_wait(empty(s), ((g / STAGES) & 1) ^ 1)) {
                        flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                        *failed = 1;
                        break;
                    }
                    const uint32_t leader_full = in_block(full(s), 0), stage = ring + s * P::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(full(s), 2 * (A_BYTES + b_bytes));
                    tma_load_pair(stage, &map_x, kb * KBLK, un.m0 + (int)rank * BM, leader_full, x_policy);
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < NSUB; j++) /* MMA j's features: the leader's half, then the peer's */
                            tma_load_pair(stage + A_BYTES + j * P::SUB_BYTES, &map_w, kb * KBLK,
                                          un.n0 + j * NMMA + (int)rank * (NMMA / 2), leader_full, w_policy);
                    } else {
                        tma_load_pair(stage + A_BYTES, &map_w_half, kb * KBLK, un.n0 + (int)rank * (NMMA / 4), leader_full,
                                      w_policy);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) { /* MMA issuer of the pair */
            constexpr uint32_t IDESC_BASE = (1u << 4) /* fp32 accumulators */ | (1u << 7) /* A bf16 */ | (1u << 10) /* B bf16 */
                                            | ((uint32_t)((2 * BM) >> 4) << 24); /* M 256 over the pair */
            uint32_t g = 0, it = 0;
            for (int u = pair; u < units && !*failed; u += n_pairs, it++) {
                const uint32_t buf = acc_of(it);
                const bool whole = pair_unit_of<WIDTH>(u, n_tiles, split_from).width == WIDTH;
                const uint32_t idesc = IDESC_BASE | ((uint32_t)((whole ? NMMA : NMMA / 2) >> 3) << 17);
                if (!mbar_wait(acc_empty(buf), (use_of(it) & 1) ^ 1)) { /* both blocks have drained this accumulator */
                    flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                    *failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * WIDTH;
                bool ok = true;
                for (int kb = 0; kb < nkb; kb++, g++) {
                    const int s = g % STAGES;
                    ok = mbar_wait(full(s), (g / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = ring + s * P::STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < KBLK / 16; k++)
#pragma unroll
                        for (int j = 0; j < NSUB; j++)
                            if (j == 0 || whole)
                                umma_bf16_pair(acc + j * NMMA, umma_desc(a_addr + k * 32),
                                               umma_desc(b_addr + j * P::SUB_BYTES + k * 32), idesc, (kb | k) != 0);
                    umma_commit_pair(empty(s));
                }
                if (!ok) {
                    flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                    *failed = 1;
                    break;
                }
                umma_commit_pair(acc_full(buf));
            }
        }
    } else { /* epilogue warps 2..5 of both blocks: this block's tensor-memory lanes 32 (warp % 4) .. + 31 */
        const int quarter = warp & 3;
        uint32_t it = 0;
        for (int u = pair; u < units; u += n_pairs, it++) {
            const uint32_t buf = acc_of(it);
            const Unit un = pair_unit_of<WIDTH>(u, n_tiles, split_from);
            const int m0 = un.m0 + (int)rank * BM, n0 = un.n0;
            if (*failed || !mbar_wait(acc_full(buf), use_of(it) & 1)) {
                if (!*failed && lane == 0) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                *failed = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const bool live = row < a.rows;
            const size_t base = (size_t)row * a.N + n0;
#pragma unroll 1
            for (int c = 0; c < un.width / 32; c++) {
                float v[32];
                tmem_load32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * WIDTH + c * 32, v);
                if (!live) continue;
                store_columns<EPI>(a, base + c * 32, v);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(in_block(acc_empty(buf), 0));
        }
    }
    /* nobody leaves while the leader's MMAs may still read the peer's shared memory or signal its barriers */
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P::TMEM_COLS) : "memory");
}

/* ---- host side ---------------------------------------------------------------------------------------------- */

int sm_count_now() {
    int device = 0, c = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || c <= 0) return 148;
    return c;
}

template <int BN, int EPI>
int launch(const CUtensorMap &map_x, const CUtensorMap &map_w, const CUtensorMap &map_w_half, TileArgs a, cudaStream_t stream) {
    auto kernel = k_tile_gemm<BN, EPI>;
    static std::mutex lock;
    static int prepared_device = -1; /* per instantiation: the attribute has to be set once per device */
    {
        std::lock_guard<std::mutex> guard(lock);
        int device = 0;
        cudaGetDevice(&device);
        if (prepared_device != device) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Tile<BN>::SMEM_BYTES) != cudaSuccess)
                return NCB_ERR_LAUNCH;
            prepared_device = device;
        }
    }
    const int tiles = (a.N / BN) * ((a.rows + BM - 1) / BM), sms = sm_count_now();
    /* a last round of tiles that fills at most half of the blocks is run as half-width units */
    const int rest = tiles % sms;
    a.split_from = (BN == 256 && tiles > sms && rest > 0 && 2 * rest <= sms) ? tiles - rest : tiles;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles < sms ? tiles : sms);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = Tile<BN>::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_w_half, a) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

template <int BN>
int launch_epi(const CUtensorMap &map_x, const CUtensorMap &map_w, const CUtensorMap &map_w_half, const TileArgs &a,
               int epilogue, cudaStream_t stream) {
    switch (epilogue) {
    case EPI_STORE: return launch<BN, EPI_STORE>(map_x, map_w, map_w_half, a, stream);
    case EPI_RESID: return launch<BN, EPI_RESID>(map_x, map_w, map_w_half, a, stream);
    case EPI_RELU2: return launch<BN, EPI_RELU2>(map_x, map_w, map_w_half, a, stream);
    case EPI_F32: return launch<BN, EPI_F32>(map_x, map_w, map_w_half, a, stream);
    default: return NCB_ERR_ARG;
    }
}

/* Pairs of blocks that can be resident at once with `smem_bytes` of dynamic shared memory each (0: no clusters). */
template <typename Kernel> int resident_pairs_of(Kernel kernel, int smem_bytes) {
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = smem_bytes;
    config.gridDim = dim3(2 * sm_count_now());
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) != cudaSuccess) n = 0;
    return n;
}

/* Resident pairs on the current device (the <256, 1, STORE> kernel stands for all: same block shape). */
int resident_pairs() {
    static std::mutex lock;
    static int known[64];
    static bool have[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    std::lock_guard<std::mutex> guard(lock);
    if (!have[device]) {
        auto kernel = k_tile_gemm_pair<160, 2, EPI_STORE>; /* the larger ring of the two */
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Pair<160, 2>::SMEM_BYTES) != cudaSuccess)
            known[device] = 0;
        else
            known[device] = resident_pairs_of(kernel, Pair<160, 2>::SMEM_BYTES);
        have[device] = true;
    }
    return known[device];
}

/* The block-pair form on `pairs` resident pairs. */
template <int NMMA, int NSUB, int EPI>
int launch_pair(const CUtensorMap &map_x, const CUtensorMap &map_w, const CUtensorMap &map_w_half, TileArgs a, int pairs,
                cudaStream_t stream) {
    using P = Pair<NMMA, NSUB>;
    auto kernel = k_tile_gemm_pair<NMMA, NSUB, EPI>;
    static std::mutex lock;
    static int prepared_device = -1;
    {
        std::lock_guard<std::mutex> guard(lock);
        int device = 0;
        cudaGetDevice(&device);
        if (prepared_device != device) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::SMEM_BYTES) != cudaSuccess)
                return NCB_ERR_LAUNCH;
            prepared_device = device;
        }
    }
    const int tiles = (a.N / P::WIDTH) * ((a.rows + 2 * BM - 1) / (2 * BM));
    const int rest = tiles % pairs;
    a.split_from = (NSUB == 1 && tiles > pairs && rest > 0 && 2 * rest <= pairs) ? tiles - rest : tiles;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs));
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = P::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_w_half, a) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

template <int NMMA, int NSUB>
int launch_pair_epi(const CUtensorMap &map_x, const CUtensorMap &map_w, const CUtensorMap &map_w_half, const TileArgs &a,
                    int epilogue, int pairs, cudaStream_t stream) {
    switch (epilogue) {
    case EPI_STORE: return launch_pair<NMMA, NSUB, EPI_STORE>(map_x, map_w, map_w_half, a, pairs, stream);
    case EPI_RESID: return launch_pair<NMMA, NSUB, EPI_RESID>(map_x, map_w, map_w_half, a, pairs, stream);
    case EPI_RELU2: return launch_pair<NMMA, NSUB, EPI_RELU2>(map_x, map_w, map_w_half, a, pairs, stream);
    case EPI_F32: return launch_pair<NMMA, NSUB, EPI_F32>(map_x, map_w, map_w_half, a, pairs, stream);
    default: return NCB_ERR_ARG;
    }
}

/* Rounds a width costs, in units of 256-wide tile rounds: whole rounds, plus about 0.6 of one for a last round that is
 * run as half-width units (NSUB == 1 only), weighted by the width. */
double pair_cost(int rows, int N, int width, bool can_split, int pairs) {
    const int tiles = (N / width) * ((rows + 2 * BM - 1) / (2 * BM));
    const int whole = tiles / pairs, rest = tiles % pairs;
    double rounds = whole;
    if (rest > 0) rounds += (can_split && whole > 0 && 2 * rest <= pairs) ? 0.6 : 1.0;
    return rounds * width;
}

} /* namespace */

extern "C" {

/*
 * y = epilogue(x . W^T) for any number of rows on the tcgen05 tensor cores.
 *   x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3); resid bf16 [rows][N] for epilogue 1 (may
 *   be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding the product), 2 relu^2, 3 fp32 store.
 *   N a multiple of 128, K a multiple of 64; x, w, y and resid 16-byte aligned. status: optional device word,
 *   NCB_DEV_WAIT_TIMEOUT is or-ed in if a bounded wait expired. Launched with programmatic stream serialisation.
 *   form: 1 one block per 128 x 256 (or 128 x 128) tile; 2 a pair of blocks per 256 x 256 or 256 x 320 tile (N a
 *   multiple of 256 or of 640, else NCB_ERR_UNSUPPORTED; the width with fewer, fuller rounds of tiles is taken);
 *   0 the pair form where it applies and there are more than 128 rows, else form 1.
 *   All forms give the same bits: a product's k-blocks are accumulated in the same order.
 */
int tile_gemm_form(const void *x, const void *w, const void *resid, void *y, long long rows, int N, int K, int epilogue,
                   int form, int *status, void *stream) {
    if (rows < 0 || rows > 0x7fffff00LL || N <= 0 || K <= 0 || N % 128 || K % KBLK) return NCB_ERR_ARG;
    if (epilogue < EPI_STORE || epilogue > EPI_F32 || form < 0 || form > 2) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!x || !w || !y || (epilogue == EPI_RESID && !resid)) return NCB_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)resid) % 16) return NCB_ERR_ALIGN;
    const TileArgs a = {(const bf16 *)resid, y, (int)rows, N, K, status, 0};
    CUtensorMap map_x, map_w, map_w_half;
    const bool wide_ok = N % 320 == 0, std_ok = N % 256 == 0;
    if ((form == 2 || (form == 0 && PAIR_BY_DEFAULT && rows > BM)) && (wide_ok || std_ok)) {
        const int pairs = resident_pairs();
        if (pairs > 0) {
            const bool wide = wide_ok && (!std_ok || pair_cost((int)rows, N, 320, false, pairs) < pair_cost((int)rows, N, 256, true, pairs));
            const int nmma = wide ? 160 : 256;
            if (!tensor_map(x, (int)rows, K, BM, &map_x) || !tensor_map(w, N, K, nmma / 2, &map_w) ||
                !tensor_map(w, N, K, nmma / 4, &map_w_half))
                return NCB_ERR_LAUNCH;
            return wide ? launch_pair_epi<160, 2>(map_x, map_w, map_w_half, a, epilogue, pairs, (cudaStream_t)stream)
                        : launch_pair_epi<256, 1>(map_x, map_w, map_w_half, a, epilogue, pairs, (cudaStream_t)stream);
        }
        if (form == 2) return NCB_ERR_UNSUPPORTED;
    } else if (form == 2) {
        return NCB_ERR_UNSUPPORTED;
    }
    const int bn = N % 256 == 0 ? 256 : 128;
    if (!tensor_map(x, (int)rows, K, BM, &map_x) || !tensor_map(w, N, K, bn, &map_w) ||
        !tensor_map(w, N, K, bn / 2, &map_w_half))
        return NCB_ERR_LAUNCH;
    return bn == 256 ? launch_epi<256>(map_x, map_w, map_w_half, a, epilogue, (cudaStream_t)stream)
                     : launch_epi<128>(map_x, map_w, map_w_half, a, epilogue, (cudaStream_t)stream);
}

int tile_gemm(const void *x, const void *w, const void *resid, void *y, long long rows, int N, int K, int epilogue,
              int *status, void *stream) {
    return tile_gemm_form(x, w, resid, y, rows, N, K, epilogue, 0, status, stream);
}

} /* extern "C" */
