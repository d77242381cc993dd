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
                if (EPI == EPI_F32) {
                    float4 *out = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.y) + base + c * 32);
#pragma unroll
                    for (int j = 0; j < 8; j++) out[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
                    uint4 res[4];
                    if (EPI == EPI_RESID) {
                        const uint4 *r = reinterpret_cast<const uint4 *>(a.resid + base + c * 32);
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
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<bf16 *>(a.y) + base + c * 32);
#pragma unroll
                    for (int j = 0; j < 4; j++) dst[j] = packed[j];
                }
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

} /* namespace */

extern "C" {

/*
 * y = epilogue(x . W^T) for any number of rows on the tcgen05 tensor cores.
 *   x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3); resid bf16 [rows][N] for epilogue 1 (may
 *   be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding the product), 2 relu^2, 3 fp32 store.
 *   N a multiple of 128, K a multiple of 64; x, w, y and resid 16-byte aligned. status: optional device word,
 *   NCB_DEV_WAIT_TIMEOUT is or-ed in if a bounded wait expired. Launched with programmatic stream serialisation.
 */
int tile_gemm(const void *x, const void *w, const void *resid, void *y, long long rows, int N, int K, int epilogue,
              int *status, void *stream) {
    if (rows < 0 || rows > 0x7fffff00LL || N <= 0 || K <= 0 || N % 128 || K % KBLK) return NCB_ERR_ARG;
    if (epilogue < EPI_STORE || epilogue > EPI_F32) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!x || !w || !y || (epilogue == EPI_RESID && !resid)) return NCB_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)resid) % 16) return NCB_ERR_ALIGN;
    const int bn = N % 256 == 0 ? 256 : 128;
    CUtensorMap map_x, map_w, map_w_half;
    if (!tensor_map(x, (int)rows, K, BM, &map_x) || !tensor_map(w, N, K, bn, &map_w) ||
        !tensor_map(w, N, K, bn / 2, &map_w_half))
        return NCB_ERR_LAUNCH;
    const TileArgs a = {(const bf16 *)resid, y, (int)rows, N, K, status, 0};
    return bn == 256 ? launch_epi<256>(map_x, map_w, map_w_half, a, epilogue, (cudaStream_t)stream)
                     : launch_epi<128>(map_x, map_w, map_w_half, a, epilogue, (cudaStream_t)stream);
}

} /* extern "C" */
