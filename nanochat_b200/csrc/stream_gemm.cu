/*
 * y = epilogue(norm?(x) . W^T) for 1 to 256 activation rows as a weight stream on Blackwell's tcgen05 tensor cores.
 * Serves decode steps of 17 to 256 sequences per GPU (the d32-class batch of 32 per GPU), where the reference runs
 * its Hopper-only slot GEMM k_wgmma with the STORE / RESID / RELU2 epilogues (model/kernels/decode.cu:170-208,232-359)
 * and separate k_norm / k_rstd launches (decode.cu:415-456). Same model semantics as decode_step.cu: parameter-free
 * RMS norm with eps FLT_EPSILON, bf16 GEMM outputs, residual add and relu^2 in bf16, fp32 logits.
 *
 * The weights are the only traffic that matters (a 2048 x 8192 projection is 33.5 MB against 128 KB of activations),
 * so the GEMM is "swapped": D[128 features][rows] = W tile (A operand, M = 128) . x^T (B operand, N = rows padded to
 * 32 / 64 / 128 / 256), both K-major, fp32 accumulators in tensor memory. One block:
 *   - thread 0 streams W and x k-blocks (64 k-values = one 128-byte swizzled row per feature) into a ring of
 *     shared-memory stages with cp.async.bulk.tensor (TMA, 128-byte swizzle, no multicast); weight loads for the
 *     first ring fill are issued BEFORE griddepcontrol.wait, so in a captured step the stream starts under the
 *     predecessor's tail;
 *   - thread 32 issues tcgen05.mma.cta_group::1.kind::f16 (4 per k-block) and releases stages with tcgen05.commit;
 *   - warps 2, 3 sum the squares of the staged x boxes for the fused norm. The norm has no gain, so
 *     norm(x) . W^T = rstd[row] * (x . W^T): the scale is applied to the fp32 accumulators in the epilogue.
 * K is split over a thread-block cluster of up to 8 blocks so that short-and-wide projections (16 feature tiles of
 * a 2048 x 2048 matrix) still cover the GPU; after the main loop every block parks its accumulators in its own
 * shared memory, and block r of the cluster reduces rows r, r + S, ... over all blocks through distributed shared
 * memory in a fixed order (deterministic), applies the epilogue and stores. No workspace, no atomics.
 * Every mbarrier wait is bounded; on expiry NCB_DEV_WAIT_TIMEOUT is flagged and the block still walks through both
 * cluster barriers and frees its tensor memory.
 */
#include "umma.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {

constexpr int TILE_F = 128;                      /* output features per block = MMA M */
constexpr int A_BOX_BYTES = TILE_F * KBLK * 2;   /* 16 KB of weights per box */
constexpr int RING_KB_SMALL = 100;               /* ring of the <= 128-row shapes: two blocks per SM */
constexpr int THREADS = 128;
constexpr int MAX_SPLIT = 8;                     /* portable cluster size */

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_RELU2 = 2, EPI_F32 = 3, EPI_MIX = 4 };

template <int NP> struct Shape {
    /* A stage holds KSUB consecutive boxes of W and the matching boxes of x. Wider stages (2 or 4 boxes, i.e. 256
     * or 512 contiguous bytes per feature row and stage) measured no faster than 1. */
    static constexpr int KSUB = 1;
    static constexpr int B_BOX_BYTES = NP * KBLK * 2;
    static constexpr int BOX_BYTES = A_BOX_BYTES + B_BOX_BYTES;
    static constexpr int STAGE_BYTES = KSUB * BOX_BYTES;
    static constexpr int RING_KB = NP == 256 ? 144 : RING_KB_SMALL; /* 256 rows park 128 KB of accumulators */
    static constexpr int STAGES = RING_KB * 1024 / STAGE_BYTES < 8 ? RING_KB * 1024 / STAGE_BYTES : 8;
    static_assert(STAGES >= 2, "at least two stages");
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int PARK_BYTES = NP * TILE_F * 4; /* fp32 accumulators parked over the ring after the main loop */
    static_assert(PARK_BYTES <= RING_BYTES, "the parked accumulators reuse the ring");
    static constexpr int TAIL_BYTES = 256 + NP * 4; /* barriers, tensor-memory slot, per-row sums of squares */
    static constexpr int SMEM_BYTES = 1024 + RING_BYTES + TAIL_BYTES; /* 1024: the ring is aligned by hand */
};

struct GemmArgs {
    const bf16 *x;     /* [rows][K] */
    const bf16 *resid; /* [rows][N] for EPI_RESID (may alias y) */
    void *y;           /* [rows][N] bf16, or fp32 for EPI_F32 */
    int rows, N, K, norm_input;
    const uint8_t *next_w; /* optional: bytes the NEXT kernel will stream, pulled into L2 while this one runs */
    long long next_bytes;
    int *status;
    const bf16 *x0; /* EPI_MIX: [rows][N], the first normed embedding rows */
    float l1, l2;   /* EPI_MIX: the next layer's (resid_lambda, x0_lambda) */
};

__device__ __forceinline__ float sumsq_bf16x8(const uint4 &u) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        s += f.x * f.x + f.y * f.y;
    }
    return s;
}


/* ---- the kernel ---------------------------------------------------------------------------------------------- */

/* Grid (S, N / 128), cluster (S, 1, 1): block (s, t) multiplies feature tile t by k-blocks [s kb / S, (s + 1) kb / S). */
template <int NP, int EPI>
__global__ void __launch_bounds__(THREADS) k_stream_gemm(const __grid_constant__ CUtensorMap map_w,
                                                         const __grid_constant__ CUtensorMap map_x, const GemmArgs a) {
    using Sh = Shape<NP>;
    constexpr int STAGES = Sh::STAGES;
    extern __shared__ uint8_t raw[];
    const uint32_t raw_addr = smem_u32(raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u; /* swizzled tiles sit on 1024-byte boundaries */
    uint8_t *ring_ptr = raw + (ring - raw_addr);
    uint8_t *tail = ring_ptr + Sh::RING_BYTES;
    const uint32_t bars = ring + Sh::RING_BYTES; /* full[STAGES], empty[STAGES], accumulators complete */
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 128);
    float *sumsq = reinterpret_cast<float *>(tail + 256); /* [NP] this block's K slice */
    float *park = reinterpret_cast<float *>(ring_ptr);    /* [NP][128] after the main loop */
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * STAGES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = gridDim.x, rank = blockIdx.x, tile = blockIdx.y;
    const int kb_total = a.K / KBLK;
    const int kb0 = (int)((long long)rank * kb_total / S), kb1 = (int)((long long)(rank + 1) * kb_total / S);
    const int nkb = kb1 - kb0;
    cg::cluster_group cluster = cg::this_cluster();

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), a.norm_input ? 3 : 1); /* the MMAs' commit + the two norm warps */
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) { /* NP columns of tensor memory: lane = feature, column = row */
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NP)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); /* the successor may start streaming its weights */

    constexpr int KSUB = Sh::KSUB;
    const int nst = (nkb + KSUB - 1) / KSUB; /* stages of up to KSUB boxes; stage i holds boxes [i KSUB, ...) */
    auto boxes_of = [&](int i) { return nkb - i * KSUB < KSUB ? nkb - i * KSUB : KSUB; };
    const uint64_t w_policy = policy_evict_first(), x_policy = policy_evict_last();
    auto load_w = [&](int i) {
        const int s = i % STAGES, n = boxes_of(i);
        mbar_expect_tx(full(s), n * Sh::BOX_BYTES);
        for (int b = 0; b < n; b++)
            tma_load(ring + s * Sh::STAGE_BYTES + b * A_BOX_BYTES, &map_w, (kb0 + i * KSUB + b) * KBLK, tile * TILE_F, full(s), w_policy);
    };
    auto load_x = [&](int i) {
        const int s = i % STAGES, n = boxes_of(i);
        for (int b = 0; b < n; b++)
            tma_load(ring + s * Sh::STAGE_BYTES + KSUB * A_BOX_BYTES + b * Sh::B_BOX_BYTES, &map_x,
                     (kb0 + i * KSUB + b) * KBLK, 0, full(s), x_policy);
    };
    if (warp == 0) {
        if (lane == 0) { /* producer */
            const int pre = nst < STAGES ? nst : STAGES;
            for (int i = 0; i < pre; i++) load_w(i); /* weights do not depend on the predecessor */
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < pre; i++) load_x(i);
            for (int i = pre; i < nst; i++) {
                if (!mbar_wait(empty(i % STAGES), ((i / STAGES) & 1) ^ 1)) {
                    flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                    break;
                }
                load_w(i);
                load_x(i);
            }
            if (a.next_w) { /* all of this block's loads are issued: its share of the NEXT kernel's weights starts
                               * towards L2 now (32 KB runs) and arrives under the epilogues and the next launch */
                const long long blocks = (long long)gridDim.x * gridDim.y, me = (long long)tile * gridDim.x + rank;
                const long long share = ((a.next_bytes + blocks - 1) / blocks + 15) & ~15ll;
                const long long from = me * share, to = from + share < a.next_bytes ? from + share : a.next_bytes;
                for (long long at = from; at < to; at += 32768)
                    l2_prefetch(a.next_w + at, (uint32_t)(to - at < 32768 ? to - at : 32768));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) { /* MMA issuer */
            constexpr uint32_t IDESC = (1u << 4) /* fp32 accumulators */ | (1u << 7) /* A bf16 */ | (1u << 10) /* B bf16 */
                                       | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(TILE_F >> 4) << 24); /* both K-major */
            bool ok = true;
            for (int i = 0; i < nst; i++) {
                const int s = i % STAGES, n = boxes_of(i);
                ok = mbar_wait(full(s), (i / STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = ring + s * Sh::STAGE_BYTES, b_addr = a_addr + KSUB * A_BOX_BYTES;
                for (int b = 0; b < n; b++) {
#pragma unroll
                    for (int k = 0; k < KBLK / 16; k++) /* 16 k-values = 32 bytes further along the swizzled row */
                        umma_bf16(tmem, umma_desc(a_addr + b * A_BOX_BYTES + k * 32),
                                  umma_desc(b_addr + b * Sh::B_BOX_BYTES + k * 32), IDESC, (i | b | k) != 0);
                }
                umma_commit(empty(s));
            }
            if (!ok) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
            umma_commit(accum_bar);
        }
    }
    if (tid != 0) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp >= 2 && a.norm_input) {
        /* Sums of squares of x[:, this block's K slice] from the staged x boxes: warp 2 takes the lower half of the
         * rows, warp 3 the upper; 8 lanes read one row's 128 bytes (the swizzle only permutes 16-byte chunks inside
         * a row), so a warp covers 4 rows per load. Each warp releases a stage with its own arrival. */
        constexpr int ROWS_W = NP / 2, PER = ROWS_W / 4;
        float acc[PER];
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] = 0.f;
        const int row0 = (warp - 2) * ROWS_W + (lane >> 3);
        for (int i = 0; i < nst; i++) {
            const int s = i % STAGES, n = boxes_of(i);
            if (!mbar_wait(full(s), (i / STAGES) & 1)) {
                flag(a.status, NCB_DEV_WAIT_TIMEOUT);
                break;
            }
            const uint8_t *xs = ring_ptr + s * Sh::STAGE_BYTES + KSUB * A_BOX_BYTES + (lane & 7) * 16;
            for (int b = 0; b < n; b++) {
#pragma unroll
                for (int j = 0; j < PER; j++)
                    acc[j] += sumsq_bf16x8(*reinterpret_cast<const uint4 *>(xs + b * Sh::B_BOX_BYTES + (row0 + 4 * j) * 128));
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty(s)) : "memory");
        }
#pragma unroll
        for (int j = 0; j < PER; j++) {
            float v = acc[j];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if ((lane & 7) == 0) sumsq[row0 + 4 * j] = v;
        }
    }
    __syncthreads(); /* the norm warps have read their last x box: the ring may now be overwritten */

    /* every thread: accumulators complete; thread tid holds feature tid (tensor-memory lane) of every row (column) */
    if (!mbar_wait(accum_bar, 0)) flag(a.status, NCB_DEV_WAIT_TIMEOUT);
    __syncwarp(); /* the tensor-memory loads below are warp-wide */
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const size_t col = (size_t)tile * TILE_F + tid;
    /* fp32 product (already normed) -> the bf16 epilogues; EPI_MIX: the residual add, then the next layer's stream
     * mix bf16(l1 h + l2 x0) with products and sum individually rounded (inference/modeling_nanochat.py:170-171) */
    auto finish_value = [&](float v, float resid, float x0 = 0.f) {
        bf16 out = __float2bfloat16_rn(v);
        if (EPI == EPI_RESID || EPI == EPI_MIX) out = __float2bfloat16_rn(resid + __bfloat162float(out));
        if (EPI == EPI_MIX)
            out = __float2bfloat16_rn(__fadd_rn(__fmul_rn(a.l1, __bfloat162float(out)), __fmul_rn(a.l2, x0)));
        if (EPI == EPI_RELU2) {
            const float p = fmaxf(__bfloat162float(out), 0.f);
            out = __float2bfloat16_rn(p * p);
        }
        return out;
    };
    auto finish = [&](float v, float resid, float x0, size_t at) {
        if (EPI == EPI_F32)
            reinterpret_cast<float *>(a.y)[at] = v;
        else
            reinterpret_cast<bf16 *>(a.y)[at] = finish_value(v, resid, x0);
    };
    constexpr bool HAS_RESID = EPI == EPI_RESID || EPI == EPI_MIX;
    const float inv_k = 1.f / (float)a.K;

    if (S == 1) { /* no partner: straight from tensor memory to y, 32 rows at a time, loads before stores */
#pragma unroll 1
        for (int c = 0; c < NP / 32; c++) {
            if (c * 32 >= a.rows) break;
            float v[32], res[32], mix[EPI == EPI_MIX ? 32 : 1];
            tmem_load32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, v);
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int r = c * 32 + j;
                res[j] = HAS_RESID && r < a.rows ? __bfloat162float(a.resid[(size_t)r * a.N + col]) : 0.f;
                if (EPI == EPI_MIX) mix[j] = r < a.rows ? __bfloat162float(a.x0[(size_t)r * a.N + col]) : 0.f;
                if (a.norm_input) v[j] *= rsqrtf(sumsq[r] * inv_k + FLT_EPSILON);
            }
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int r = c * 32 + j;
                if (r < a.rows) finish(v[j], res[j], EPI == EPI_MIX ? mix[j] : 0.f, (size_t)r * a.N + col);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 1)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NP) : "memory");
        return;
    }

    /* K split over the cluster: park the partial accumulators, then block `rank` sums rows rank, rank + S, ... over
     * all blocks in a fixed order through distributed shared memory, four rows' loads in flight at a time */
#pragma unroll
    for (int c = 0; c < NP / 32; c++) {
        float v[32];
        tmem_load32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, v);
#pragma unroll
        for (int j = 0; j < 32; j++) park[(c * 32 + j) * TILE_F + tid] = v[j];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster.sync(); /* all blocks' accumulators and sums of squares are parked */
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NP) : "memory");
    /* 32 threads cover a row's 128 features with 16-byte remote loads; the block's four warps take four of its rows
     * at a time, and all of a thread's loads (two row groups x S peers) are issued before the first add */
    const float *peer_park[MAX_SPLIT], *peer_sumsq[MAX_SPLIT];
#pragma unroll
    for (int s = 0; s < MAX_SPLIT; s++) {
        peer_park[s] = cluster.map_shared_rank(park, s < S ? s : 0) + lane * 4;
        peer_sumsq[s] = cluster.map_shared_rank(sumsq, s < S ? s : 0);
    }
    const size_t col4 = (size_t)tile * TILE_F + lane * 4;
    constexpr int RB = 2;
    for (int r0 = rank + warp * S; r0 < a.rows; r0 += 4 * S * RB) {
        float4 pv[RB][MAX_SPLIT];
        float ps[RB][MAX_SPLIT];
        uint2 res[RB], mix[RB];
#pragma unroll
        for (int i = 0; i < RB; i++) {
            const int r = r0 + i * 4 * S;
            const bool ok = r < a.rows;
#pragma unroll
            for (int s = 0; s < MAX_SPLIT; s++) {
                pv[i][s] = ok && s < S ? *reinterpret_cast<const float4 *>(peer_park[s] + r * TILE_F) : make_float4(0.f, 0.f, 0.f, 0.f);
                ps[i][s] = ok && s < S && a.norm_input ? peer_sumsq[s][r] : 0.f;
            }
            res[i] = HAS_RESID && ok ? *reinterpret_cast<const uint2 *>(a.resid + (size_t)r * a.N + col4) : make_uint2(0u, 0u);
            mix[i] = EPI == EPI_MIX && ok ? *reinterpret_cast<const uint2 *>(a.x0 + (size_t)r * a.N + col4) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < RB; i++) {
            const int r = r0 + i * 4 * S;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            float ss = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_SPLIT; s++) {
                v.x += pv[i][s].x, v.y += pv[i][s].y, v.z += pv[i][s].z, v.w += pv[i][s].w;
                ss += ps[i][s];
            }
            if (a.norm_input) {
                const float rstd = rsqrtf(ss * inv_k + FLT_EPSILON);
                v.x *= rstd, v.y *= rstd, v.z *= rstd, v.w *= rstd;
            }
            if (r >= a.rows) continue;
            const size_t at = (size_t)r * a.N + col4;
            if (EPI == EPI_F32) {
                *reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.y) + at) = v;
            } else {
                const __nv_bfloat162 *rr = reinterpret_cast<const __nv_bfloat162 *>(&res[i]);
                const __nv_bfloat162 *mm = reinterpret_cast<const __nv_bfloat162 *>(&mix[i]);
                const float2 r01 = __bfloat1622float2(rr[0]), r23 = __bfloat1622float2(rr[1]);
                const float2 m01 = __bfloat1622float2(mm[0]), m23 = __bfloat1622float2(mm[1]);
                uint2 out;
                __nv_bfloat162 *oo = reinterpret_cast<__nv_bfloat162 *>(&out);
                oo[0] = __halves2bfloat162(finish_value(v.x, r01.x, m01.x), finish_value(v.y, r01.y, m01.y));
                oo[1] = __halves2bfloat162(finish_value(v.z, r23.x, m23.x), finish_value(v.w, r23.y, m23.y));
                *reinterpret_cast<uint2 *>(reinterpret_cast<bf16 *>(a.y) + at) = out;
            }
        }
    }
    cluster.sync(); /* nobody leaves while a peer still reads its shared memory */
}

/* ---- host side ---------------------------------------------------------------------------------------------- */

/* K split S: enough blocks for every SM without a second wave, at least two k-blocks each. */
int auto_split(int rows, int tiles, int kb) {
    const int slots = rows > 128 ? 148 : 296; /* 256-row blocks need an SM each, the others fit two per SM (B200) */
    int s = MAX_SPLIT;                        /* measured: powers of two, as many blocks as fit in one wave */
    while (s > 1 && (tiles * s > slots || s > kb / 2)) s >>= 1;
    return s;
}

template <int NP, int EPI>
int launch(const CUtensorMap &map_w, const CUtensorMap &map_x, const GemmArgs &a, int split, cudaStream_t stream) {
    auto kernel = k_stream_gemm<NP, EPI>;
    static bool prepared = false; /* per instantiation; the attribute belongs to the function on every device */
    static std::mutex lock;
    {
        std::lock_guard<std::mutex> guard(lock);
        int device = 0;
        static int prepared_device = -1;
        cudaGetDevice(&device);
        if (!prepared || prepared_device != device) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<NP>::SMEM_BYTES) !=
                cudaSuccess)
                return NCB_ERR_LAUNCH;
            prepared = true;
            prepared_device = device;
        }
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(split, a.N / TILE_F);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = Shape<NP>::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = split;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, kernel, map_w, map_x, a) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

template <int NP>
int launch_epi(const CUtensorMap &map_w, const CUtensorMap &map_x, const GemmArgs &a, int epilogue, int split,
               cudaStream_t stream) {
    switch (epilogue) {
    case EPI_STORE: return launch<NP, EPI_STORE>(map_w, map_x, a, split, stream);
    case EPI_RESID: return launch<NP, EPI_RESID>(map_w, map_x, a, split, stream);
    case EPI_RELU2: return launch<NP, EPI_RELU2>(map_w, map_x, a, split, stream);
    case EPI_F32: return launch<NP, EPI_F32>(map_w, map_x, a, split, stream);
    case EPI_MIX: return launch<NP, EPI_MIX>(map_w, map_x, a, split, stream);
    default: return NCB_ERR_ARG;
    }
}

} /* namespace */

extern "C" {

/* The K split stream_gemm chooses for `rows` rows and a [N][K] weight matrix when called with split 0. */
int stream_gemm_split(int rows, int N, int K) {
    if (rows < 0 || rows > 256 || N <= 0 || K <= 0 || N % TILE_F || K % KBLK) return 0;
    return auto_split(rows, N / TILE_F, K / KBLK);
}

} /* extern "C" */

/* The checks and the launch shared by stream_gemm and stream_gemm_mix. */
static int run_stream_gemm(const void *x, const void *w, const void *resid, void *y, int rows, int N, int K, int norm_input,
                           int epilogue, int split, const void *next_w, long long next_bytes, int *status, void *stream,
                           const void *x0, float l1, float l2) {
    if (rows < 0 || rows > 256 || N <= 0 || K <= 0 || N % TILE_F || K % KBLK) return NCB_ERR_ARG;
    if (epilogue < EPI_STORE || epilogue > EPI_MIX || split < 0 || split > MAX_SPLIT || split > K / KBLK) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    const bool has_resid = epilogue == EPI_RESID || epilogue == EPI_MIX;
    if (!x || !w || !y || (has_resid && !resid) || (epilogue == EPI_MIX && !x0)) return NCB_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)resid | (uintptr_t)x0) % 16) return NCB_ERR_ALIGN;
    if (next_w && ((uintptr_t)next_w % 16 || next_bytes % 16 || next_bytes < 0)) return NCB_ERR_ALIGN;
    if (split == 0) split = auto_split(rows, N / TILE_F, K / KBLK);
    const int np = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    CUtensorMap map_w, map_x;
    if (!tensor_map(w, N, K, TILE_F, &map_w) || !tensor_map(x, rows, K, np, &map_x)) return NCB_ERR_LAUNCH;
    const GemmArgs a = {(const bf16 *)x, (const bf16 *)resid, y, rows, N, K, norm_input,
                        next_bytes > 0 ? (const uint8_t *)next_w : nullptr, next_bytes, status, (const bf16 *)x0, l1, l2};
    cudaStream_t s = (cudaStream_t)stream;
    switch (np) {
    case 32: return launch_epi<32>(map_w, map_x, a, epilogue, split, s);
    case 64: return launch_epi<64>(map_w, map_x, a, epilogue, split, s);
    case 128: return launch_epi<128>(map_w, map_x, a, epilogue, split, s);
    default: return launch_epi<256>(map_w, map_x, a, epilogue, split, s);
    }
}

extern "C" {

/*
 * y = epilogue(norm?(x) . W^T) for rows <= 256 activation rows on the tcgen05 tensor cores.
 *   x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3); resid bf16 [rows][N] for epilogue 1
 *   (may be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding the product), 2 relu^2, 3 fp32.
 *   norm_input != 0 applies the parameter-free RMS norm (eps FLT_EPSILON) to x, as a per-row scale of the fp32
 *   product. split: blocks per cluster that share a feature tile's K range (1..8, at most K / 64), 0 = automatic.
 *   next_w, next_bytes: optional; the weights the NEXT call on this stream will read (16-byte aligned, a multiple
 *   of 16 bytes). They are prefetched into L2 while this call runs, so a chain of short GEMMs keeps HBM busy across
 *   kernel boundaries. status: optional device word, NCB_DEV_WAIT_TIMEOUT is or-ed in if a bounded wait expired.
 * N must be a multiple of 128, K of 64; x, w, y and resid 16-byte aligned.
 */
int stream_gemm(const void *x, const void *w, const void *resid, void *y, int rows, int N, int K, int norm_input,
                int epilogue, int split, const void *next_w, long long next_bytes, int *status, void *stream) {
    if (epilogue == EPI_MIX) return NCB_ERR_ARG;
    return run_stream_gemm(x, w, resid, y, rows, N, K, norm_input, epilogue, split, next_w, next_bytes, status, stream,
                           nullptr, 1.f, 0.f);
}

/* stream_gemm with the residual epilogue followed by the NEXT layer's stream mix:
 * y = bf16(l1 * bf16(resid + bf16(x . W^T)) + l2 * x0), x0 bf16 [rows][N], 16-byte aligned. */
int stream_gemm_mix(const void *x, const void *w, const void *resid, const void *x0, float l1, float l2, void *y, int rows,
                    int N, int K, int norm_input, int split, const void *next_w, long long next_bytes, int *status,
                    void *stream) {
    return run_stream_gemm(x, w, resid, y, rows, N, K, norm_input, EPI_MIX, split, next_w, next_bytes, status, stream, x0,
                           l1, l2);
}

} /* extern "C" */
