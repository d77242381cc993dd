/*
 * The rest of a decode step for small batches (at most 16 rows): weight-streaming GEMMs with fused RMS norm and
 * epilogues, the embedding + first norm, and the greedy choice. Replaces, for sm_100a, the reference's Hopper-only
 * slot GEMM k_wgmma with its STORE / RESID / RELU2 / ARGMAX epilogues (model/kernels/decode.cu:170-208,232-359) and
 * its k_norm / k_rstd / k_commit (decode.cu:415-456,678-688). Model semantics are those of the reference's exported
 * model (inference/modeling_nanochat.py:105-125,163-194): parameter-free RMS norm with eps FLT_EPSILON rounded to
 * bf16, bf16 GEMM outputs, residual adds in bf16, relu^2 in bf16, fp32 logits.
 *
 * At 8 rows a d20 step reads 0.95 GB of weights and computes almost nothing: every GEMM is a stream of W with a
 * handful of activation rows held on chip, bound by HBM and, at these sizes (3 to 170 MB per GEMM), by launch and
 * ramp-up latency. So:
 *   - y^T tile = W tile . x^T on mma.sync.m16n8k16 (bf16, fp32 accumulate) with the ROWS as the M dimension (16 slots,
 *     rows 8..15 zero when there are at most 8) and 8 output features as N. W is the B operand and goes from global
 *     memory straight to registers with one 16-byte load per thread and 32 k-values (a feature row is read in
 *     64-byte runs by four lanes, every sector fully used); the MMA's k slots are permuted identically for A and B so
 *     no shuffle or shared-memory staging is needed;
 *   - a block owns tiles of 8 output features and splits K over its 8 warps; each warp issues all loads of its K
 *     slice before the first MMA (5 to 20 independent 16-byte loads per thread in flight), partial tiles are summed
 *     through shared memory; a block walks over several tiles when there are more tiles than resident blocks, with
 *     the next tile's weights already streaming, so the activations are loaded and normed once per block;
 *   - the RMS norm of the input is fused: activations stay in registers between the sum of squares (block-wide
 *     through shared memory) and the MMAs, so a layer needs no separate norm kernel;
 *   - epilogues: bf16 store, residual add, relu^2, or fp32 store (logits).
 * These kernels wait for their predecessor with griddepcontrol.wait and are launched with programmatic stream
 * serialisation, so inside a captured step the launch of each overlaps the tail of the one before.
 */
#include "ncb_common.cuh"

constexpr int GEMM_WARPS = 8;
constexpr int GEMM_THREADS = GEMM_WARPS * 32;
constexpr int TILE_N = 8;         /* output features per block */
constexpr int MAX_ROWS = 16;
constexpr int MAX_K_ITERS = 20;   /* 32 k-values per iteration and warp: K <= 8 * 20 * 32 = 5120 */

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_RELU2 = 2, EPI_F32 = 3, EPI_MIX = 4 };

struct GemmArgs {
    const bf16 *x;     /* [rows][K] */
    const bf16 *w;     /* [N][K] */
    const bf16 *resid; /* [rows][N] for EPI_RESID (may alias y) */
    void *y;           /* [rows][N] bf16, or fp32 for EPI_F32 */
    int rows, N, K, norm_input;
    const bf16 *x0;    /* EPI_MIX: [rows][N], the first normed embedding rows */
    float l1, l2;      /* EPI_MIX: the next layer's (resid_lambda, x0_lambda) */
};

/* The per-layer stream mix of the reference's model (inference/modeling_nanochat.py:170-171; decode.cu:430-432):
 * h <- bf16(l1 h + l2 x0), both products and the sum rounded in fp32, one bf16 rounding. */
static __device__ __forceinline__ bf16 stream_mix(bf16 h, bf16 x0, float l1, float l2) {
    return __float2bfloat16_rn(__fadd_rn(__fmul_rn(l1, __bfloat162float(h)), __fmul_rn(l2, __bfloat162float(x0))));
}

static __device__ __forceinline__ void mma_bf16(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

static __device__ __forceinline__ float sumsq_bf16x8(const uint4 &u) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        s += f.x * f.x + f.y * f.y;
    }
    return s;
}

static __device__ __forceinline__ uint4 scale_bf16x8(const uint4 &u, float r) {
    uint4 out;
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
    __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&out);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        o[i] = __floats2bfloat162_rn(f.x * r, f.y * r);
    }
    return out;
}

/* ITERS: 32-k iterations per warp (K = GEMM_WARPS * ITERS * 32 exactly); HI: rows 8..15 are in use.
 * A block keeps its activation slice (normed once) in registers and walks over the feature tiles
 * blockIdx.x, blockIdx.x + gridDim.x, ...; while it reduces one tile the next tile's weights are already in flight
 * (PREFETCH: only where two weight slices fit the register file). */
template <int ITERS, bool HI, int EPI, bool NORM>
__global__ void __launch_bounds__(GEMM_THREADS, ITERS > 8 ? 2 : 1) k_skinny_gemm(GemmArgs a) {
    constexpr bool PREFETCH = ITERS <= 8;
    constexpr bool HOLD_X = NORM || PREFETCH; /* long K slices stream x with the MMAs to stay within 128 registers */
    __shared__ float part[GEMM_WARPS][16][TILE_N + 1];
    __shared__ float ss[GEMM_WARPS][16];
    __shared__ float rstd[16];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int tiles = a.N / TILE_N;
    const int k_warp = warp * ITERS * 32;
    const bf16 *wbase = a.w + (size_t)g * a.K + k_warp + 8 * t;

    /* the weights do not depend on the kernel before this one: start streaming them before waiting for it */
    uint4 wv[ITERS], wnext[PREFETCH ? ITERS : 1];
    int tile = blockIdx.x;
    if (tile < tiles) {
        const bf16 *wrow = wbase + (size_t)tile * TILE_N * a.K;
#pragma unroll
        for (int i = 0; i < ITERS; i++) wv[i] = __ldcs(reinterpret_cast<const uint4 *>(wrow + 32 * i)); /* read once */
    }
    if (PREFETCH && tile + (int)gridDim.x < tiles) {
        const bf16 *wrow = wbase + (size_t)(tile + gridDim.x) * TILE_N * a.K;
#pragma unroll
        for (int i = 0; i < ITERS; i++) wnext[i] = __ldcs(reinterpret_cast<const uint4 *>(wrow + 32 * i));
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    uint4 xlo[HOLD_X ? ITERS : 1], xhi[HI && HOLD_X ? ITERS : 1];
    const bool lo_on = g < a.rows, hi_on = HI && g + 8 < a.rows;
    const bf16 *xl = a.x + (size_t)g * a.K + k_warp + 8 * t, *xh = a.x + (size_t)(g + 8) * a.K + k_warp + 8 * t;
    if (HOLD_X) {
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            xlo[i] = lo_on ? *reinterpret_cast<const uint4 *>(xl + 32 * i) : make_uint4(0, 0, 0, 0);
            if (HI) xhi[i] = hi_on ? *reinterpret_cast<const uint4 *>(xh + 32 * i) : make_uint4(0, 0, 0, 0);
        }
    }
    if (NORM) { /* rows' 1 / sqrt(mean(x^2) + eps) over the full K, then x <- bf16(x * rstd) in registers */
        float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            s_lo += sumsq_bf16x8(xlo[i]);
            if (HI) s_hi += sumsq_bf16x8(xhi[i]);
        }
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        if (HI) {
            s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
            s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
        }
        if (t == 0) {
            ss[warp][g] = s_lo;
            ss[warp][g + 8] = HI ? s_hi : 0.f;
        }
        __syncthreads();
        if (tid < 16) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < GEMM_WARPS; w++) s += ss[w][tid];
            rstd[tid] = rsqrtf(s / (float)a.K + FLT_EPSILON);
        }
        __syncthreads();
        const float r_lo = rstd[g], r_hi = rstd[g + 8];
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            xlo[i] = scale_bf16x8(xlo[i], r_lo);
            if (HI) xhi[i] = scale_bf16x8(xhi[i], r_hi);
        }
    }
    for (; tile < tiles; tile += gridDim.x) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f}; /* two chains: MMA latency overlaps */
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            /* k slots (2t, 2t+1) and (2t+8, 2t+9) of the two MMAs take the thread's values 0..1, 2..3 and 4..5, 6..7 */
            uint4 lo, hi = make_uint4(0, 0, 0, 0);
            if (HOLD_X) {
                lo = xlo[i];
                if (HI) hi = xhi[i];
            } else {
                lo = lo_on ? *reinterpret_cast<const uint4 *>(xl + 32 * i) : make_uint4(0, 0, 0, 0);
                if (HI && hi_on) hi = *reinterpret_cast<const uint4 *>(xh + 32 * i);
            }
            mma_bf16(acc, lo.x, hi.x, lo.y, hi.y, wv[i].x, wv[i].y);
            mma_bf16(acc2, lo.z, hi.z, lo.w, hi.w, wv[i].z, wv[i].w);
        }
        /* the tile after next starts streaming now; the next one becomes current */
        const int after = tile + (PREFETCH ? 2 : 1) * (int)gridDim.x;
        if (PREFETCH) {
#pragma unroll
            for (int i = 0; i < ITERS; i++) wv[i] = wnext[i];
        }
        if (after < tiles) {
            const bf16 *wrow = wbase + (size_t)after * TILE_N * a.K;
#pragma unroll
            for (int i = 0; i < ITERS; i++) {
                const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(wrow + 32 * i));
                if (PREFETCH) wnext[i] = v; else wv[i] = v;
            }
        }
        /* C: acc[0], acc[1] = row g, features 2t, 2t+1; acc[2], acc[3] = row g+8 */
        part[warp][g][2 * t] = acc[0] + acc2[0];
        part[warp][g][2 * t + 1] = acc[1] + acc2[1];
        part[warp][g + 8][2 * t] = acc[2] + acc2[2];
        part[warp][g + 8][2 * t + 1] = acc[3] + acc2[3];
        __syncthreads();
        if (tid < 16 * TILE_N) {
            const int row = tid / TILE_N, col = tid % TILE_N;
            if (row < a.rows) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < GEMM_WARPS; w++) v += part[w][row][col];
                const size_t at = (size_t)row * a.N + (size_t)tile * TILE_N + col;
                if (EPI == EPI_F32) {
                    reinterpret_cast<float *>(a.y)[at] = v;
                } else {
                    bf16 out = __float2bfloat16_rn(v);
                    if (EPI == EPI_RESID || EPI == EPI_MIX)
                        out = __float2bfloat16_rn(__bfloat162float(a.resid[at]) + __bfloat162float(out));
                    if (EPI == EPI_MIX) out = stream_mix(out, a.x0[at], a.l1, a.l2);
                    if (EPI == EPI_RELU2) {
                        const float r = fmaxf(__bfloat162float(out), 0.f);
                        out = __float2bfloat16_rn(r * r);
                    }
                    reinterpret_cast<bf16 *>(a.y)[at] = out;
                }
            }
        }
        __syncthreads(); /* the partial sums are consumed before the next tile overwrites them */
    }
}

/* x0[row] = rms_norm(embed[token[row]]), one warp per row (decode.cu:415-443 EMBED, with a bf16 table);
 * h[row] = x0[row], or with mixing the first layer's stream mix bf16(l1 x0 + l2 x0). x0 may be NULL (not kept). */
__global__ void __launch_bounds__(128) k_embed_norm(const bf16 *embed, const long long *tokens, bf16 *h, bf16 *x0, float l1,
                                                    float l2, int mix, int rows, int C, int vocab) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    long long token = tokens[row];
    if (token < 0 || token >= vocab) token = 0;
    const bf16 *e = embed + (size_t)token * C;
    float s = 0.f;
    for (int i = lane * 8; i < C; i += 256) s += sumsq_bf16x8(*reinterpret_cast<const uint4 *>(e + i));
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float r = rsqrtf(s / (float)C + FLT_EPSILON);
    for (int i = lane * 8; i < C; i += 256) {
        uint4 v = scale_bf16x8(*reinterpret_cast<const uint4 *>(e + i), r);
        if (x0) *reinterpret_cast<uint4 *>(x0 + (size_t)row * C + i) = v;
        if (mix) {
            bf16 *b = reinterpret_cast<bf16 *>(&v);
#pragma unroll
            for (int j = 0; j < 8; j++) b[j] = stream_mix(b[j], b[j], l1, l2);
        }
        *reinterpret_cast<uint4 *>(h + (size_t)row * C + i) = v;
    }
}

/* h[row] += y[row] (bf16 add, skipped when y is NULL), n[row] = rms_norm(h[row]); one block of 256 threads per row,
 * the row held in registers between the two passes (C <= 256 * 8 * ROW_VECS). For any number of rows: the norm and
 * residual steps between library GEMMs when a pass has more than 16 rows (decode.cu:415-443 RESID_NORM / NORM). */
constexpr int ROW_THREADS = 256, ROW_VECS = 2;
__global__ void __launch_bounds__(ROW_THREADS) k_add_rms_norm(bf16 *h, const bf16 *y, bf16 *n, int C, const bf16 *x0,
                                                              float l1, float l2) {
    __shared__ float warp_sums[ROW_THREADS / 32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * C;
    uint4 v[ROW_VECS];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_VECS; j++) {
        const int i = (threadIdx.x + j * ROW_THREADS) * 8;
        if (i < C) {
            v[j] = *reinterpret_cast<const uint4 *>(h + base + i);
            if (y) {
                const uint4 w = *reinterpret_cast<const uint4 *>(y + base + i);
                __nv_bfloat162 *a = reinterpret_cast<__nv_bfloat162 *>(&v[j]);
                const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&w);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 fa = __bfloat1622float2(a[e]), fb = __bfloat1622float2(b[e]);
                    a[e] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
                }
            }
            if (x0) { /* the next layer's stream mix, after the residual add */
                const uint4 z = *reinterpret_cast<const uint4 *>(x0 + base + i);
                bf16 *a = reinterpret_cast<bf16 *>(&v[j]);
                const bf16 *b = reinterpret_cast<const bf16 *>(&z);
#pragma unroll
                for (int e = 0; e < 8; e++) a[e] = stream_mix(a[e], b[e], l1, l2);
            }
            if (y || x0) *reinterpret_cast<uint4 *>(h + base + i) = v[j];
            s += sumsq_bf16x8(v[j]);
        }
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
#pragma unroll
    for (int w = 0; w < ROW_THREADS / 32; w++) s += warp_sums[w];
    const float r = rsqrtf(s / (float)C + FLT_EPSILON);
#pragma unroll
    for (int j = 0; j < ROW_VECS; j++) {
        const int i = (threadIdx.x + j * ROW_THREADS) * 8;
        if (i < C) *reinterpret_cast<uint4 *>(n + base + i) = scale_bf16x8(v[j], r);
    }
}

/* u = relu(u)^2 in bf16, in place, 8 values per thread. */
__global__ void __launch_bounds__(256) k_relu2(bf16 *u, long long count) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
    if (i >= count) return;
    uint4 v = *reinterpret_cast<const uint4 *>(u + i);
    __nv_bfloat162 *a = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float2 f = __bfloat1622float2(a[e]);
        const float x = fmaxf(f.x, 0.f), z = fmaxf(f.y, 0.f);
        a[e] = __floats2bfloat162_rn(x * x, z * z);
    }
    *reinterpret_cast<uint4 *>(u + i) = v;
}

/* tokens[row] = argmax(logits[row]) (ties to the lowest id, decode.cu:90-96), pos[row] += 1; one block per row. */
__global__ void __launch_bounds__(1024) k_greedy(const float *logits, long long *tokens, int32_t *pos, int vocab,
                                                 long long *trace, int trace_stride) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (pos[row] < 0) return; /* an idle row (the whole block leaves): no choice, no advance */
    const float *z = logits + (size_t)row * vocab;
    float v = -INFINITY;
    int at = 0x7fffffff;
    for (int i = tid; i < vocab; i += 1024) {
        const float x = z[i];
        if (x > v) v = x, at = i; /* ascending i: the first maximum wins */
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > v || (ov == v && oi < at)) v = ov, at = oi;
    }
    if (lane == 0) best_v[warp] = v, best_i[warp] = at;
    __syncthreads();
    if (warp == 0) {
        v = best_v[lane], at = best_i[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > v || (ov == v && oi < at)) v = ov, at = oi;
        }
        if (lane == 0) {
            const long long choice = at == 0x7fffffff ? 0 : at;
            const int next = pos[row] + 1;
            tokens[row] = choice;
            pos[row] = next;
            if (trace && next >= 0 && next < trace_stride) trace[(size_t)row * trace_stride + next] = choice;
        }
    }
}

/* ---- sampling -------------------------------------------------------------------------------------------------
 * The reference's choice rule (decode.cu:90-120 keys and Gumbel noise, :195-203 temperature and cap, :364-411
 * nucleus): temperature 0 takes the argmax of the raw logits; otherwise the logits are capped (c tanh(s / c)),
 * optionally cut to the nucleus of mass top_p (transformers' TopPLogitsWarper: keep e >= e*, the least e whose
 * cumulative mass from below exceeds (1 - top_p) of the total, found by bisection on the IEEE bits of e in [0, 1])
 * and sampled by Gumbel-max: argmax of s / T - log(-log u), u from Philox4x32-10 at counter (token id, step), key
 * seed. Ties go to the lowest id. An optional bit mask restricts the choice to allowed tokens. */

static __device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int round = 0; round < 10; round++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += 0x9E3779B9u;
        k.y += 0xBB67AE85u;
    }
    return c;
}

/* -log(-log(u)), u in (0, 1) from 52 random bits, exact in double. Restates the reference's noise
 * (model/kernels/decode.cu:100-105) so that a (seed, step, token) triple means the same draw: the counter layout, the
 * 52-bit mantissa and the midpoint u = (2 r + 1) 2^-53 have to be the reference's. */
static __device__ __forceinline__ float gumbel(unsigned long long seed, int step, int token) {
    const uint4 x = philox4x32_10(make_uint4((uint32_t)token, (uint32_t)step, 0u, 0u),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const unsigned long long r = ((unsigned long long)x.x << 32 | x.y) >> 12;
    return (float)-log(-log(ldexp(2.0 * (double)r + 1.0, -53)));
}

constexpr int SAMPLE_THREADS = 1024;

static __device__ float block_sum_ordered(float v, float *scratch) { /* fixed order: lanes, then warps 0..31 */
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < SAMPLE_THREADS / 32; w++) s = __fadd_rn(s, scratch[w]);
    return s;
}

struct SampleArgs {
    const float *logits;       /* [rows][vocab] */
    float *probs;              /* [rows][vocab] scratch for the nucleus */
    const float *temperature, *top_p; /* [rows] */
    const unsigned long long *seed;   /* [rows] */
    const int32_t *first;      /* [rows]: the position of each row's first generated token's input (step = pos - first) */
    const uint32_t *allow;     /* [rows][vocab / 32] or NULL */
    long long *tokens;
    int32_t *pos;
    long long *trace;
    int vocab, trace_stride;
    float softcap;
};

__global__ void __launch_bounds__(SAMPLE_THREADS) k_sample(SampleArgs a) {
    __shared__ float scratch[SAMPLE_THREADS / 32];
    __shared__ float best_v[SAMPLE_THREADS / 32];
    __shared__ int best_i[SAMPLE_THREADS / 32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, V = a.vocab;
    if (a.pos[b] < 0) return; /* an idle row (the whole block leaves): no choice, no advance */
    const float *s = a.logits + (size_t)b * V;
    float *e = a.probs + (size_t)b * V;
    const uint32_t *allow = a.allow ? a.allow + (size_t)b * (V / 32) : nullptr;
    const float T = a.temperature[b], top_p = a.top_p[b];
    const bool sampled = T > 0.f, nucleus = sampled && top_p < 1.f;
    const int step = a.pos[b] - a.first[b];
    const unsigned long long seed = a.seed[b];
    auto ok = [&](int r) { return !allow || ((allow[r >> 5] >> (r & 31)) & 1u); };
    auto value = [&](int r) { /* the score the choice works on, before noise */
        const float z = s[r];
        if (!sampled) return z;
        const float capped = a.softcap > 0.f ? __fmul_rn(a.softcap, tanhf(__fdiv_rn(z, a.softcap))) : z;
        return __fdiv_rn(capped, T);
    };
    float least = 0.f;
    if (nucleus) {
        float m = -INFINITY;
        for (int r = tid; r < V; r += SAMPLE_THREADS)
            if (ok(r)) m = fmaxf(m, value(r));
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) scratch[warp] = m;
        __syncthreads();
        m = -INFINITY;
        for (int w = 0; w < SAMPLE_THREADS / 32; w++) m = fmaxf(m, scratch[w]);
        float sum = 0.f;
        for (int r = tid; r < V; r += SAMPLE_THREADS) {
            e[r] = ok(r) ? expf(__fsub_rn(value(r), m)) : 0.f;
            sum = __fadd_rn(sum, e[r]);
        }
        const float drop = __fmul_rn(__fsub_rn(1.f, top_p), block_sum_ordered(sum, scratch));
        /* The nucleus threshold, restating the reference's rule (model/kernels/decode.cu:382-393): e lies in [0, 1], where
         * IEEE bit patterns order like the values, so the least e* whose mass from below exceeds `drop` is found by
         * bisection on the bits; sums in the fixed order of block_sum_ordered, so the result is reproducible. */
        uint32_t lo = 0u, hi = __float_as_uint(1.f); /* the least bits u with C(u) > drop */
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            const float x = __uint_as_float(mid);
            float below = 0.f;
            for (int r = tid; r < V; r += SAMPLE_THREADS)
                if (e[r] <= x) below = __fadd_rn(below, e[r]);
            if (block_sum_ordered(below, scratch) > drop) hi = mid; else lo = mid + 1;
        }
        least = __uint_as_float(lo);
    }
    float v = -INFINITY;
    int at = 0x7fffffff;
    for (int r = tid; r < V; r += SAMPLE_THREADS) {
        if (!ok(r) || (nucleus && e[r] < least)) continue;
        const float x = sampled ? __fadd_rn(value(r), gumbel(seed, step, r)) : value(r);
        if (x > v || at == 0x7fffffff) v = x, at = r; /* ascending r: the first maximum wins */
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (oi != 0x7fffffff && (at == 0x7fffffff || ov > v || (ov == v && oi < at))) v = ov, at = oi;
    }
    if (lane == 0) best_v[warp] = v, best_i[warp] = at;
    __syncthreads();
    if (warp == 0) {
        v = best_v[lane], at = best_i[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, at, o);
            if (oi != 0x7fffffff && (at == 0x7fffffff || ov > v || (ov == v && oi < at))) v = ov, at = oi;
        }
        if (lane == 0) {
            const long long choice = at == 0x7fffffff ? -1 : at; /* -1: the mask allows nothing */
            const int next = a.pos[b] + 1;
            a.tokens[b] = choice; /* -1 reaches the host; as the next step's input the embedding reads it as token 0 */
            a.pos[b] = next;
            if (a.trace && next >= 0 && next < a.trace_stride) a.trace[(size_t)b * a.trace_stride + next] = choice;
        }
    }
}

/* ---- host side ---------------------------------------------------------------------------------------------- */

template <typename... Args>
static int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, args...) == cudaSuccess ? NCB_OK : NCB_ERR_LAUNCH;
}

/* Blocks for `tiles` feature tiles: everything resident at once when it fits, else an even number of tiles per
 * block (640 tiles on 444 slots -> 320 blocks of 2) so that no block is left with one more than the others. */
template <typename K> static int grid_for(K kernel, int tiles, bool prefetch) {
    if (!prefetch) return tiles; /* without a second weight slice in registers a block's tiles would serialise */
    static int slots = 0; /* per instantiation; the same on every device of a homogeneous box */
    if (!slots) {
        int device = 0, sms = 148, per_sm = 1;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, GEMM_THREADS, 0) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        slots = sms * per_sm;
    }
    const int per_block = (tiles + slots - 1) / slots;
    return (tiles + per_block - 1) / per_block;
}

template <int ITERS, bool HI, bool NORM> static int launch_gemm_epi(const GemmArgs &a, int epilogue, cudaStream_t stream) {
    const int tiles = a.N / TILE_N;
    const dim3 block(GEMM_THREADS);
    switch (epilogue) {
    case EPI_STORE: { auto k = k_skinny_gemm<ITERS, HI, EPI_STORE, NORM>; return launch_pdl(k, dim3(grid_for(k, tiles, ITERS <= 8)), block, stream, a); }
    case EPI_RESID: { auto k = k_skinny_gemm<ITERS, HI, EPI_RESID, NORM>; return launch_pdl(k, dim3(grid_for(k, tiles, ITERS <= 8)), block, stream, a); }
    case EPI_RELU2: { auto k = k_skinny_gemm<ITERS, HI, EPI_RELU2, NORM>; return launch_pdl(k, dim3(grid_for(k, tiles, ITERS <= 8)), block, stream, a); }
    case EPI_F32: { auto k = k_skinny_gemm<ITERS, HI, EPI_F32, NORM>; return launch_pdl(k, dim3(grid_for(k, tiles, ITERS <= 8)), block, stream, a); }
    case EPI_MIX: { auto k = k_skinny_gemm<ITERS, HI, EPI_MIX, NORM>; return launch_pdl(k, dim3(grid_for(k, tiles, ITERS <= 8)), block, stream, a); }
    default: return NCB_ERR_ARG;
    }
}

template <int ITERS> static int launch_gemm_rows(const GemmArgs &a, int epilogue, cudaStream_t stream) {
    constexpr bool CAN_NORM = ITERS <= 8; /* the fused norm keeps the whole K slice of x in registers */
    if (a.norm_input) {
        if (!CAN_NORM) return NCB_ERR_UNSUPPORTED;
        return a.rows > 8 ? launch_gemm_epi<(CAN_NORM ? ITERS : 1), true, true>(a, epilogue, stream)
                          : launch_gemm_epi<(CAN_NORM ? ITERS : 1), false, true>(a, epilogue, stream);
    }
    return a.rows > 8 ? launch_gemm_epi<ITERS, true, false>(a, epilogue, stream)
                      : launch_gemm_epi<ITERS, false, false>(a, epilogue, stream);
}

/* The K / 256 values k_skinny_gemm is instantiated for. */
static bool skinny_depth_ok(int K) {
    switch (K / (GEMM_WARPS * 32)) {
    case 1: case 2: case 3: case 4: case 5: case 6: case 8: case 10: case 12: case 16: case 20: return K % (GEMM_WARPS * 32) == 0;
    default: return false;
    }
}

static int launch_skinny(const GemmArgs &a, int epilogue, cudaStream_t s) {
    const int rows = a.rows, N = a.N, K = a.K;
    if (rows < 0 || rows > MAX_ROWS || N <= 0 || K <= 0 || N % TILE_N || K % (GEMM_WARPS * 32)) return NCB_ERR_ARG;
    if (!skinny_depth_ok(K)) return NCB_ERR_UNSUPPORTED;
    if (rows == 0) return NCB_OK;
    if (!a.x || !a.w || !a.y || ((epilogue == EPI_RESID || epilogue == EPI_MIX) && !a.resid) ||
        (epilogue == EPI_MIX && !a.x0))
        return NCB_ERR_ARG;
    if (((uintptr_t)a.x | (uintptr_t)a.w) % 16 || (uintptr_t)a.y % 4) return NCB_ERR_ALIGN;
    switch (K / (GEMM_WARPS * 32)) {
    case 1: return launch_gemm_rows<1>(a, epilogue, s);
    case 2: return launch_gemm_rows<2>(a, epilogue, s);
    case 3: return launch_gemm_rows<3>(a, epilogue, s);
    case 4: return launch_gemm_rows<4>(a, epilogue, s);
    case 5: return launch_gemm_rows<5>(a, epilogue, s);
    case 6: return launch_gemm_rows<6>(a, epilogue, s);
    case 8: return launch_gemm_rows<8>(a, epilogue, s);
    case 10: return launch_gemm_rows<10>(a, epilogue, s);
    case 12: return launch_gemm_rows<12>(a, epilogue, s);
    case 16: return launch_gemm_rows<16>(a, epilogue, s);
    case 20: return launch_gemm_rows<20>(a, epilogue, s);
    default: return NCB_ERR_UNSUPPORTED;
    }
}

extern "C" {

/* 1 if skinny_gemm takes the shape (rows <= 16, N a multiple of 8, K / 256 one of the instantiated depths, at most
 * 2048 with the fused norm), else 0: callers choose between this kernel and stream_gemm with it. */
int skinny_gemm_supported(int rows, int N, int K, int norm_input) {
    if (rows < 0 || rows > MAX_ROWS || N <= 0 || K <= 0 || N % TILE_N || !skinny_depth_ok(K)) return 0;
    return !(norm_input && K / (GEMM_WARPS * 32) > 8);
}

/*
 * y = epilogue(norm?(x) . W^T) for rows <= 16 activation rows.
 *   x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3); resid bf16 [rows][N] for epilogue 1
 *   (may be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding the product), 2 relu^2, 3 fp32.
 *   norm_input != 0 applies the parameter-free RMS norm (eps FLT_EPSILON, rounded to bf16) to x first.
 * K must be a multiple of 256 and at most 5120 (at most 2048 with norm_input), N a multiple of 8.
 */
int skinny_gemm(const void *x, const void *w, const void *resid, void *y, int rows, int N, int K, int norm_input,
                int epilogue, void *stream) {
    if (epilogue < EPI_STORE || epilogue > EPI_F32) return NCB_ERR_ARG;
    const GemmArgs a = {(const bf16 *)x, (const bf16 *)w, (const bf16 *)resid, y, rows, N, K, norm_input, nullptr, 1.f, 0.f};
    return launch_skinny(a, epilogue, (cudaStream_t)stream);
}

/* skinny_gemm with the residual epilogue followed by the NEXT layer's stream mix:
 * y = bf16(l1 * bf16(resid + bf16(x . W^T)) + l2 * x0), x0 bf16 [rows][N]. */
int skinny_gemm_mix(const void *x, const void *w, const void *resid, const void *x0, float l1, float l2, void *y, int rows,
                    int N, int K, int norm_input, void *stream) {
    const GemmArgs a = {(const bf16 *)x, (const bf16 *)w, (const bf16 *)resid, y, rows, N, K, norm_input, (const bf16 *)x0, l1, l2};
    return launch_skinny(a, EPI_MIX, (cudaStream_t)stream);
}

static int launch_embed(const void *embed, const void *tokens, void *h, void *x0, float l1, float l2, int mix, int rows,
                        int C, int vocab, void *stream) {
    if (rows < 0 || C <= 0 || C % 8 || vocab <= 0) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!embed || !tokens || !h) return NCB_ERR_ARG;
    if (((uintptr_t)embed | (uintptr_t)h | (uintptr_t)x0) % 16) return NCB_ERR_ALIGN;
    return launch_pdl(k_embed_norm, dim3((rows + 3) / 4), dim3(128), (cudaStream_t)stream, (const bf16 *)embed,
                      (const long long *)tokens, (bf16 *)h, (bf16 *)x0, l1, l2, mix, rows, C, vocab);
}

/* h bf16 [rows][C] = rms_norm(embed[tokens]); tokens int64 [rows]; C a multiple of 8. */
int embed_norm(const void *embed, const void *tokens, void *h, int rows, int C, int vocab, void *stream) {
    return launch_embed(embed, tokens, h, nullptr, 1.f, 0.f, 0, rows, C, vocab, stream);
}

/* x0 = rms_norm(embed[tokens]) kept for the later layers' mixes, h = bf16(l1 x0 + l2 x0): the first layer's input. */
int embed_norm_mix(const void *embed, const void *tokens, void *h, void *x0, float l1, float l2, int rows, int C,
                   int vocab, void *stream) {
    if (!x0 && rows > 0) return NCB_ERR_ARG;
    return launch_embed(embed, tokens, h, x0, l1, l2, 1, rows, C, vocab, stream);
}

static int launch_add_norm(void *h, const void *y, void *n, const void *x0, float l1, float l2, long long rows, int C,
                           void *stream) {
    if (rows < 0 || rows > 0x7fffffffLL || C <= 0 || C % 8 || C > ROW_THREADS * 8 * ROW_VECS) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!h || !n) return NCB_ERR_ARG;
    if (((uintptr_t)h | (uintptr_t)y | (uintptr_t)n | (uintptr_t)x0) % 16) return NCB_ERR_ALIGN;
    return launch_pdl(k_add_rms_norm, dim3((unsigned)rows), dim3(ROW_THREADS), (cudaStream_t)stream, (bf16 *)h,
                      (const bf16 *)y, (bf16 *)n, C, (const bf16 *)x0, l1, l2);
}

/* h bf16 [rows][C] += y (same shape; NULL: no add), n = rms_norm(h). C a multiple of 8, at most 4096. */
int add_rms_norm(void *h, const void *y, void *n, long long rows, int C, void *stream) {
    return launch_add_norm(h, y, n, nullptr, 1.f, 0.f, rows, C, stream);
}

/* h += y, then the next layer's stream mix h = bf16(l1 h + l2 x0), then n = rms_norm(h). */
int add_rms_norm_mix(void *h, const void *y, const void *x0, float l1, float l2, void *n, long long rows, int C,
                     void *stream) {
    if (!x0 && rows > 0) return NCB_ERR_ARG;
    return launch_add_norm(h, y, n, x0, l1, l2, rows, C, stream);
}

/* u bf16 [count] = relu(u)^2 in place; count a multiple of 8. */
int relu2_inplace(void *u, long long count, void *stream) {
    if (count < 0 || count % 8) return NCB_ERR_ARG;
    if (count == 0) return NCB_OK;
    if (!u) return NCB_ERR_ARG;
    if ((uintptr_t)u % 16) return NCB_ERR_ALIGN;
    const long long blocks = (count / 8 + 255) / 256;
    if (blocks > 0x7fffffffLL) return NCB_ERR_ARG;
    return launch_pdl(k_relu2, dim3((unsigned)blocks), dim3(256), (cudaStream_t)stream, (bf16 *)u, count);
}

/* tokens[row] = argmax(logits[row]) over fp32 [rows][vocab], ties to the lowest id; pos[row] += 1; if trace (int64
 * [rows][trace_stride]) is given, trace[row][new pos] = the choice, so a host can fetch a whole run at its end. */
int greedy_choice(const void *logits, void *tokens, void *pos, int rows, int vocab, void *trace, int trace_stride,
                  void *stream) {
    if (rows < 0 || vocab <= 0) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!logits || !tokens || !pos) return NCB_ERR_ARG;
    return launch_pdl(k_greedy, dim3(rows), dim3(1024), (cudaStream_t)stream, (const float *)logits,
                      (long long *)tokens, (int32_t *)pos, vocab, (long long *)trace, trace_stride);
}

/*
 * tokens[row] = the reference's choice for logits fp32 [rows][vocab] (see "sampling" above); pos[row] += 1; the
 * choice is logged in trace like greedy_choice does (-1 when the mask allows no token).
 *   temperature, top_p fp32 [rows]; seed uint64 [rows]; first int32 [rows] (step = pos - first picks the noise);
 *   allow uint32 [rows][vocab / 32] or NULL; probs fp32 [rows][vocab] scratch (used when top_p < 1);
 *   softcap: the logit cap c applied to sampled rows (0: none). vocab a multiple of 32.
 */
int sample_choice(const void *logits, void *probs, const void *temperature, const void *top_p, const void *seed,
                  const void *first, const void *allow, float softcap, void *tokens, void *pos, int rows, int vocab,
                  void *trace, int trace_stride, void *stream) {
    if (rows < 0 || vocab <= 0 || vocab % 32 || softcap < 0.f) return NCB_ERR_ARG;
    if (rows == 0) return NCB_OK;
    if (!logits || !probs || !temperature || !top_p || !seed || !first || !tokens || !pos) return NCB_ERR_ARG;
    const SampleArgs a = {(const float *)logits, (float *)probs, (const float *)temperature, (const float *)top_p,
                          (const unsigned long long *)seed, (const int32_t *)first, (const uint32_t *)allow,
                          (long long *)tokens, (int32_t *)pos, (long long *)trace, vocab, trace_stride, softcap};
    return launch_pdl(k_sample, dim3(rows), dim3(SAMPLE_THREADS), (cudaStream_t)stream, a);
}

} /* extern "C" */
