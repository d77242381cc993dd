/*
 * C ABI of the B200 (sm_100a) decode hot path: the fp8 (e4m3) KV-cache append/quantise step and single-token
 * attention over that cache. Every entry point takes plain device pointers, sizes and a cudaStream_t passed as
 * void*, launches on that stream, never synchronises or allocates (unless its comment says otherwise), and
 * returns an NCB_* status instead of aborting. The caller owns every buffer and keeps it alive until the stream
 * has run the launch.
 *
 * The reference binds its kernels the same way: nvcc-built shared objects loaded with ctypes.CDLL and called
 * with pointer(tensor), ints and stream() (native.py:43-65; model/ops/qk_prologue.py:18-20;
 * inference/decoder.py:131-148). The entry points below replace, on the decode path,
 *   k_prologue  (model/kernels/decode.cu:551-565, row math model/kernels/qk_row.cuh:26-51)  -> kv_append_fp8
 *   k_attn      (model/kernels/decode.cu:567-675)                                           -> decode_attn_fp8*
 *   the (m, l, acc) merge inside k_attn (model/kernels/decode.cu:548,661-674)               -> decode_attn_merge
 * and are split over two libraries, kv_append and decode_attn, one per kernel file as in the reference.
 *
 * Cache layout ("pages"). One cache buffer per layer: uint8 [n_slots][Hkv][pages_per_slot][NCB_PAGE_BYTES].
 * A page holds NCB_PAGE_TOKENS = 64 consecutive positions of one (slot, kv head):
 *   [0, 8192)       K rows: position j at j*128; the row's 16-byte chunk c is stored at chunk c ^ ((j >> 2) & 7)
 *   [8192, 16384)   V transposed: 32-position group gi, half h (positions 16h..16h+15 of the group), dim d:
 *                   16 bytes at 8192 + gi*4096 + h*2048 + d*16, byte (j & 15)
 *   [16384, 16640)  K scales, fp32[64]
 *   [16640, 16896)  V scales, fp32[64]
 * so that a (slot, kv head, split) thread block streams one contiguous region with one bulk copy per page and
 * feeds the tensor cores from shared memory without conflicts or transposes. A stored byte b with scale s stands
 * for the value e4m3(b) * s; s = amax / 448 over the row's 128 bf16 values.
 */
#ifndef NANOCHAT_B200_H
#define NANOCHAT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define NCB_HEAD_DIM 128
#define NCB_PAGE_TOKENS 64
#define NCB_PAGE_BYTES 16896
#define NCB_PART_FLOATS 132 /* one partial attention state: m, l, 2 pad, o[128]; fp32 */
#define NCB_STATIC_SCRATCH_BYTES (8u << 20) /* the built-in scratch of decode_attn_fp8_static */
#define NCB_PEER_STATE_BYTES 1056 /* one (m, l, o) state in a peer inbox of decode_attn_fp8_sharded */

enum {
    NCB_OK = 0,
    NCB_ERR_ARG = 1,         /* a size, ratio or pointer argument is out of range or NULL */
    NCB_ERR_ALIGN = 2,       /* a pointer or stride misses its required alignment */
    NCB_ERR_WORKSPACE = 3,   /* the workspace is smaller than decode_attn_workspace_bytes() */
    NCB_ERR_LAUNCH = 4,      /* the CUDA runtime refused the launch; see cudaGetLastError */
    NCB_ERR_UNSUPPORTED = 5, /* a shape this kernel does not take: Hq / Hkv above its limit, a GEMM width its form cannot tile */
    NCB_ERR_STATIC_LIMIT = 6 /* decode_attn_fp8_static: the call needs more than NCB_STATIC_SCRATCH_BYTES */
};

/* Bits a kernel ORs into the caller's optional device status word (int32, may be NULL). */
enum {
    NCB_DEV_BAD_POSITION = 1, /* kv_append_fp8: a row's position or slot is outside the cache; the row was skipped */
    NCB_DEV_WAIT_TIMEOUT = 2, /* decode_attn_fp8: a bounded wait on a copy barrier ran out; outputs are invalid */
    NCB_DEV_BAD_LENGTH = 4    /* decode_attn_fp8: a length or slot is outside the cache; the sequence was skipped */
};

const char *ncb_status_string(int status);

/* ---- library kv_append -------------------------------------------------------------------------------------- */

/* Bytes of one layer's cache for n_slots sequences of at most max_len positions (rounded up to whole pages). */
long long kv_cache_bytes(int n_slots, int kv_heads, int max_len);
/* Pages per (slot, kv head) for max_len positions. */
int kv_cache_pages(int max_len);

/*
 * Fused rotary + QK-RMSNorm + quantise + append for `rows` new tokens (replaces k_prologue, decode.cu:551-565).
 *   qkv       bf16 [rows][qkv_row_stride]: per row Hq q heads, then Hkv k heads, then Hkv v heads of 128
 *   q_gain, k_gain   fp32 [128], shared by the heads (decode.cu:464)
 *   cos, sin  fp32 [table_len][64], indexed by absolute position (decode.cu:498)
 *   pos       int32 [rows]: each row's position; the row's k, v are written at that position
 *   slot_map  int32 [rows] or NULL (row r writes slot r) (decode.cu:556)
 *   q_out     bf16 [rows][Hq][128]: normed, rotated q
 *   kv_cache  the layer's pages (layout above)
 *   status    int32 device word or NULL
 * Arithmetic: every fp32 operation individually rounded in the order fixed by oracle/kv_append_oracle.c, so q
 * bits, cache bytes and scales are exact functions of the inputs. Rows whose position >= pages_per_slot * 64 or
 * >= table_len, or whose slot is outside [0, n_slots), are skipped and flagged in *status. A NEGATIVE position marks
 * an idle row: it is skipped silently (nothing written, nothing flagged), the counterpart of the reference's
 * `active` slot mask (decode.cu:60-62,555), so that one captured step serves a batch whose slots finish at different
 * times.
 */
int kv_append_fp8(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                  const void *pos, const void *slot_map, void *q_out, void *kv_cache, long long rows, int Hq,
                  int Hkv, long long qkv_row_stride, int table_len, int n_slots, int pages_per_slot, void *status,
                  void *stream);

/*
 * kv_append_fp8 with the reference's optional value-embedding mix on v (attn_prologue, decode.cu:482-494; the
 * reference's checkpoints have it on alternating layers, model/modeling.py:35-37): before it is quantised, each v
 * head row becomes bf16(v + g ve[token]) with g = 2 sigmoid(ve_gate[kv head] . h).
 *   h         bf16 [rows][C]: the layer's normed input rows (what the qkv projection read)
 *   tokens    int64 [rows]: the rows' input tokens (outside [0, vocab): token 0, as embed_norm)
 *   ve_table  bf16 [vocab][Hkv][128]; ve_gate fp32 [Hkv][C]; C a multiple of 256
 * The dot product is summed in the reference's order (FMAs per warp lane over 8-element runs of 256-element chunks,
 * then an xor butterfly), the sigmoid is evaluated in double precision and rounded once (the reference's fp32 expf
 * is not reproducible on a CPU), products and sums individually rounded: v bytes and scales stay exact functions of
 * the inputs (oracle/kv_append_oracle.c:oracle_kv_append_ve). ve_table == NULL is kv_append_fp8.
 */
int kv_append_fp8_ve(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                     const void *pos, const void *slot_map, void *q_out, void *kv_cache, long long rows, int Hq,
                     int Hkv, long long qkv_row_stride, int table_len, int n_slots, int pages_per_slot, const void *h,
                     const void *tokens, const void *ve_table, const void *ve_gate, int C, int vocab, void *status,
                     void *stream);

/* ---- library decode_attn ------------------------------------------------------------------------------------ */

/* Pages one thread block covers when chunk_pages == 0 is passed below; depends only on these three values (every
 * sequence is taken as max_kv_len long). */
int decode_attn_chunk_pages(int B, int Hkv, int max_kv_len);
/* The same choice for lengths the HOST knows (lens: host int32[B], clipped to [0, max_kv_len]; NULL = all at
 * max_kv_len): a model of how the split kernel's blocks fill the GPU picks the chunk size that avoids a nearly
 * empty last wave of blocks. Pass the result as chunk_pages (and to decode_attn_workspace_bytes); worth it for
 * ragged batches whose lengths change slowly, such as the steps of one captured decode loop. */
int decode_attn_plan_chunk_pages(const int *lens, int B, int Hkv, int max_kv_len, int window);
/* Workspace bytes for the split partials; chunk_pages == 0 selects decode_attn_chunk_pages(B, Hkv, max_kv_len). Pass
 * the same max_kv_len here and to the attention entry point: they derive the same default chunk from it (the entry
 * point clips max_kv_len to the cache's capacity only afterwards, which can only shrink the need). */
long long decode_attn_workspace_bytes(int B, int Hq, int max_kv_len, int Hkv, int chunk_pages);

/*
 * out[b, h, :] = softmax_j(q[b, h] . K[j] * softmax_scale) V[j] over the cached positions
 * j in [max(0, lens[b] - window), lens[b]) of slot slot_map[b] (replaces k_attn, decode.cu:567-675; the current
 * token is read from the cache, where kv_append_fp8 put it, instead of from registers).
 *   q         bf16 [B][Hq][128]
 *   lens      int32 [B]: cached positions per sequence (0 gives a zero output row; so does a negative value, which
 *             marks an idle row and is not flagged)
 *   slot_map  int32 [B] or NULL
 *   workspace >= decode_attn_workspace_bytes(B, Hq, max_kv_len, Hkv, chunk_pages), 16-byte aligned; contents are
 *             scratch, calls sharing it must be stream-ordered
 *   out       bf16 [B][Hq][128]
 *   max_kv_len   an upper bound of every lens[b]; sizes the grid (lens stay on the device)
 *   window    0 for none, else the number of most recent positions attended (decode.cu:575)
 *   chunk_pages  0 for the built-in choice
 * Two launches: the split-KV kernel (one block per sequence, kv head and chunk of pages; all Hq/Hkv query heads
 * of the kv head share each K/V byte) and the merge kernel. When max_kv_len and chunk_pages leave every sequence one
 * chunk (at most four pages of cache, or a chunk size of at least the cache's pages) the split kernel's blocks
 * normalise and write `out` themselves and there is no second launch; the output bits are the same either way.
 */
int decode_attn_fp8(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *workspace,
                    long long workspace_bytes, void *out, int B, int Hq, int Hkv, int n_slots, int pages_per_slot,
                    int max_kv_len, int window, int chunk_pages, float softmax_scale, void *status, void *stream);

/*
 * As decode_attn_fp8, but leaves the un-normalised state of each (b, h) in part_out, fp32
 * [B][Hq][NCB_PART_FLOATS] = (m in log2 units, l, 0, 0, o[128]) with out = o / l, for merging across GPUs that
 * each hold a slice of the positions (the merge rule of decode.cu:548,661-670 is associative).
 */
int decode_attn_fp8_partial(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                            void *workspace, long long workspace_bytes, void *part_out, int B, int Hq, int Hkv,
                            int n_slots, int pages_per_slot, int max_kv_len, int window, int chunk_pages,
                            float softmax_scale, void *status, void *stream);

/*
 * kv_append_fp8 and decode_attn_fp8 for one new token per sequence in the same two launches as decode_attn_fp8
 * alone (replaces k_prologue + k_attn, decode.cu:859-863, as a pair): every block of the split-KV kernel first does
 * the append's arithmetic for its own heads — q rows stay in shared memory, the block whose chunk holds the new
 * position writes that kv head's k and v bytes and scales into the cache — and then attends over positions
 * [max(0, pos[b] + 1 - window), pos[b] + 1). Same arithmetic as kv_append_fp8 (shared code), so the cache bytes are
 * identical; q is not written out. Arguments as for the two entry points; `pos` int32 [B] takes the place of lens,
 * max_kv_len bounds pos[b] + 1. Rows must address distinct slots (rows sharing a slot, as in prefill, need the
 * separate entry points, where every row's append lands before any row attends). pos[b] < 0 marks an idle row: no
 * append, no attention, a zero output row, no status bit (the reference's inactive slots, decode.cu:555,573).
 * Stream contract: the split kernel starts its first page copies before it waits for the launch before it (programmatic
 * dependent launch), so a kernel launched IMMEDIATELY before this call on the stream that releases its dependents
 * early (every kernel of these libraries does) must not write pos, slot_map or this cache (in a decode step it is the
 * qkv projection; copies, ordinary kernels and anything earlier are always complete).
 */
int decode_step_attn_fp8(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                         const void *pos, const void *slot_map, void *kv_cache, void *workspace,
                         long long workspace_bytes, void *out, int B, int Hq, int Hkv, long long qkv_row_stride,
                         int table_len, int n_slots, int pages_per_slot, int max_kv_len, int window, int chunk_pages,
                         float softmax_scale, void *status, void *stream);

/* decode_step_attn_fp8 with the value-embedding mix of kv_append_fp8_ve on the appended v rows (same arguments, same
 * bytes). */
int decode_step_attn_fp8_ve(const void *qkv, const void *q_gain, const void *k_gain, const void *cos, const void *sin,
                            const void *pos, const void *slot_map, void *kv_cache, void *workspace,
                            long long workspace_bytes, void *out, int B, int Hq, int Hkv, long long qkv_row_stride,
                            int table_len, int n_slots, int pages_per_slot, int max_kv_len, int window,
                            int chunk_pages, float softmax_scale, const void *h, const void *tokens,
                            const void *ve_table, const void *ve_gate, int C, int vocab, void *status, void *stream);

/*
 * Attention for a prefill pass (replaces k_attn over prompt rows, decode.cu:859-863,1041-1051): `rows` query rows,
 * many of which belong to one sequence. Rows are grouped on the host: block z = the group_rows[z] rows starting at
 * row group_first[z] (int32 [n_groups] each; at most prefill_attn_rows_per_block(Hq, Hkv) rows: 64 for Hq == Hkv, 16
 * for four query heads per kv head; at most 16 query heads per kv head), all of one slot with ascending positions.
 * Blocks start in the order of the list, so list the groups that reach furthest into their prompts first. A block
 * streams the sequence's pages once for all its rows (a shared ring consumed by four warps, each owning
 * 16 / (Hq / Hkv) rows over the whole key range; the cache bytes are widened to f16 in registers and both
 * contractions run as f16 tensor-core MMAs) and writes normalised outputs itself: no workspace, no merge launch.
 *   q bf16 [rows][Hq][128]; lens int32 [rows] (row r attends positions [0, lens[r])); slot_map int32 [rows];
 *   out bf16 [rows][Hq][128]. No window. Every row's k, v must already be in the cache (kv_append_fp8).
 * A block whose longest row exceeds the cache, or whose slot is outside it, is flagged (NCB_DEV_BAD_LENGTH) and writes
 * zeros.
 */
int prefill_attn_rows_per_block(int Hq, int Hkv);
int prefill_attn_fp8(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                     const void *group_first, const void *group_rows, int n_groups, void *out, long long rows, int Hq,
                     int Hkv, int n_slots, int pages_per_slot, float softmax_scale, void *status, void *stream);

/*
 * The first of decode_attn_fp8's two launches alone: the split-KV kernel, leaving one state per (b, h, chunk) in
 * the workspace. For timing that kernel by itself and for callers that merge elsewhere; same arguments and
 * checks as decode_attn_fp8 without `out`.
 */
int decode_attn_fp8_split(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                          void *workspace, long long workspace_bytes, int B, int Hq, int Hkv, int n_slots,
                          int pages_per_slot, int max_kv_len, int window, int chunk_pages, float softmax_scale,
                          void *status, void *stream);

/*
 * decode_attn_fp8 for callers that cannot hand over a workspace because they cannot allocate device memory at
 * all: code running inside someone else's memory plan (a serving engine that gives a plug-in only its input and
 * output tensors), hosts that forbid cudaMalloc after start-up, or a thin FFI shim with no allocator behind it.
 * No counterpart in the reference, whose decoder allocates all of its own buffers up front in dec_create.
 *
 * Same arguments and results as decode_attn_fp8 minus the workspace: the per-chunk states go to an array built
 * into the library, NCB_STATIC_SCRATCH_BYTES (8 MiB) of device memory that every GPU loading decode_attn holds
 * until the process exits. A call whose states need more (decode_attn_workspace_bytes() for the same B, Hq,
 * max_kv_len, Hkv, chunk_pages) is refused with NCB_ERR_STATIC_LIMIT; pass a larger chunk_pages to shrink the need.
 * The entry point itself calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * The first call on each device looks up the array's device address (with that device current) and remembers it;
 * make that first call outside any stream capture. Every call on a device shares the one array: calls must be
 * stream-ordered with respect to each other, since two that overlap on the GPU would overwrite each other's
 * states. Nothing in the array has to start at zero; each call writes every state it later reads. The remembered
 * address belongs to the device's primary context: after cudaDeviceReset the library must be reloaded.
 */
int decode_attn_fp8_static(const void *q, const void *kv_cache, const void *lens, const void *slot_map, void *out,
                           int B, int Hq, int Hkv, int n_slots, int pages_per_slot, int max_kv_len, int window,
                           int chunk_pages, float softmax_scale, void *status, void *stream);

/*
 * Merge n_parts states per row: parts fp32 [n_parts][rows][NCB_PART_FLOATS] (e.g. the all-gathered part_out of
 * every rank, rows = B * Hq) into out bf16 [rows][128]. A state with m = -inf counts as empty; a row whose states
 * are all empty gives zeros.
 */
int decode_attn_merge(const void *parts, int n_parts, long long rows, void *out, void *stream);

/*
 * decode_attn_fp8 for sequences whose positions are sharded by length over the GPUs of one box (each rank's cache
 * holds a contiguous slice of every sequence; lens are the LOCAL lengths): the split-KV launch, then ONE launch that
 * merges this rank's chunk states, exchanges the (m, l, o) state of every row with the other ranks over peer memory
 * (NVLink) and merges across ranks, so that every rank ends with the full out bf16 [B][Hq][128], bit-identical on all
 * ranks (states are merged in rank order). No collective library on the data path. The merge rule of
 * decode.cu:548,661-670 is associative, which is what makes the sharding exact. No counterpart in the reference,
 * which runs on one GPU.
 *   inbox   host array of `world` (<= 8) device pointers, the same on every rank: inbox[r] is rank r's buffer of
 *           2 * world * B * Hq * NCB_PEER_STATE_BYTES bytes, addressable from every GPU (peer-mapped / symmetric
 *           memory), 16-byte aligned, zeroed once before the first call (and the ranks synchronised)
 *   epoch   this rank's own two device uint32 words, zeroed once; the kernel advances the first by one per call, so
 *           the launch arguments never change and a step can be captured in a CUDA graph and replayed
 * Per row the second launch stores the rank state into every other rank's inbox (plain peer stores) as 8-byte words
 * (fp32 value, call number) that validate themselves: no flags and no fences, an arrived word whose second half is
 * the current call number holds this call's value. It then polls — bounded, about half a second — its own inbox until
 * every word of the other ranks' states of the row carries the call number, and merges the `world` states. Every rank
 * must make the same sequence of calls with the same B and Hq; a rank may run ahead of a peer by at most one call, and
 * the inbox's two halves alternate between calls so nothing still being read is overwritten. If a wait runs out,
 * NCB_DEV_WAIT_TIMEOUT is set in *status and the row's `out` is not written; the kernel still returns. Other
 * arguments as decode_attn_fp8. Stream contract: as for decode_step_attn_fp8, the kernel launched immediately before
 * this call must not write lens, slot_map or cached positions below lens[b] - 1 (appending the newest token there is
 * fine: the page that holds it is only read after the wait).
 */
int decode_attn_fp8_sharded(const void *q, const void *kv_cache, const void *lens, const void *slot_map,
                            void *workspace, long long workspace_bytes, void *out, int B, int Hq, int Hkv, int n_slots,
                            int pages_per_slot, int max_kv_len, int window, int chunk_pages, float softmax_scale,
                            void *const *inbox, int world, int rank, void *epoch, void *status, void *stream);

/* ---- library decode_step ------------------------------------------------------------------------------------
 * The rest of a decode step for at most 16 rows; replaces the reference's Hopper-only slot GEMM k_wgmma with its
 * epilogues (model/kernels/decode.cu:170-208,232-359), k_norm / k_rstd (decode.cu:415-456) and k_commit
 * (decode.cu:678-688). All three are launched with programmatic stream serialisation. */

/*
 * y = epilogue(norm?(x) . W^T). x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3);
 * resid bf16 [rows][N] for epilogue 1 (may be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding
 * the product), 2 relu^2, 3 fp32 store. norm_input != 0 first applies the parameter-free RMS norm (eps
 * FLT_EPSILON, rounded to bf16) to x. rows <= 16; K a multiple of 256, at most 5120 (2048 with norm_input); N a
 * multiple of 8.
 */
int skinny_gemm(const void *x, const void *w, const void *resid, void *y, int rows, int N, int K, int norm_input,
                int epilogue, void *stream);
/* 1 if skinny_gemm takes the shape, else 0 (for choosing between it and stream_gemm without a failed call). */
int skinny_gemm_supported(int rows, int N, int K, int norm_input);
/*
 * The per-layer stream mix of the reference's model, h <- bf16(resid_lambda h + x0_lambda x0) with x0 the first normed
 * embedding rows (inference/modeling_nanochat.py:170-171; k_norm RESID_NORM, decode.cu:430-432), fused where the
 * stream is written: skinny_gemm_mix is skinny_gemm's residual epilogue followed by the NEXT layer's mix,
 *   y = bf16(l1 * bf16(resid + bf16(x . W^T)) + l2 * x0),   x0 bf16 [rows][N];
 * embed_norm_mix keeps x0 = rms_norm(embed[tokens]) and writes h = bf16(l1 x0 + l2 x0), the first layer's input;
 * add_rms_norm_mix is add_rms_norm with the mix between the add and the norm. Products and the sum are individually
 * rounded fp32 operations, then one bf16 rounding.
 */
int skinny_gemm_mix(const void *x, const void *w, const void *resid, const void *x0, float l1, float l2, void *y, int rows,
                    int N, int K, int norm_input, void *stream);
int embed_norm_mix(const void *embed, const void *tokens, void *h, void *x0, float l1, float l2, int rows, int C,
                   int vocab, void *stream);
int add_rms_norm_mix(void *h, const void *y, const void *x0, float l1, float l2, void *n, long long rows, int C,
                     void *stream);
/* h bf16 [rows][C] = rms_norm(embed[tokens]); embed bf16 [vocab][C]; tokens int64 [rows]; C a multiple of 8. */
int embed_norm(const void *embed, const void *tokens, void *h, int rows, int C, int vocab, void *stream);
/* h bf16 [rows][C] += y (same shape, or NULL for no add), in bf16; n bf16 [rows][C] = rms_norm(h). Any number of
 * rows; C a multiple of 8, at most 4096. The norm / residual steps between library GEMMs (decode.cu:415-456). */
int add_rms_norm(void *h, const void *y, void *n, long long rows, int C, void *stream);
/* u bf16 [count] = relu(u)^2 in place (the MLP activation, decode.cu:170-208 EPI_RELU2); count a multiple of 8. */
int relu2_inplace(void *u, long long count, void *stream);
/* tokens[row] (int64) = argmax of logits fp32 [rows][vocab], ties to the lowest id; pos[row] (int32) += 1; with
 * trace (int64 [rows][trace_stride], may be NULL) also trace[row][new pos[row]] = the choice. Rows with pos[row] < 0
 * are idle: token and position stay as they are. */
int greedy_choice(const void *logits, void *tokens, void *pos, int rows, int vocab, void *trace, int trace_stride,
                  void *stream);

/*
 * The reference's sampled choice (decode.cu:90-120,195-203,364-411): per row, temperature 0 takes the argmax of the
 * raw logits; otherwise logits are capped (softcap * tanh(s / softcap), softcap 0: none), optionally cut to the
 * nucleus of mass top_p (keep e >= e*, the least e whose cumulative mass from below exceeds (1 - top_p) of the
 * total; bisection on IEEE bits) and sampled by Gumbel-max with Philox4x32-10 noise at counter (token id,
 * pos - first), key seed. Ties to the lowest id; `allow` (uint32 [rows][vocab / 32], may be NULL) masks tokens.
 * tokens[row] = choice (-1 if the mask allows nothing; embed_norm reads a token outside the vocabulary as token 0),
 * pos[row] += 1, trace as greedy_choice; idle rows (pos[row] < 0) are left alone.
 * logits fp32 [rows][vocab]; probs fp32 [rows][vocab] scratch; temperature, top_p fp32 [rows]; seed uint64 [rows];
 * first int32 [rows]; vocab a multiple of 32.
 */
int sample_choice(const void *logits, void *probs, const void *temperature, const void *top_p, const void *seed,
                  const void *first, const void *allow, float softcap, void *tokens, void *pos, int rows, int vocab,
                  void *trace, int trace_stride, void *stream);

/* ---- library stream_gemm ------------------------------------------------------------------------------------
 * The same GEMM for 1 to 256 rows on the tcgen05 tensor cores (TMA-staged weight stream, accumulators in tensor
 * memory, K split over a thread-block cluster and reduced through distributed shared memory); replaces k_wgmma with
 * its epilogues (model/kernels/decode.cu:170-208,232-359) and k_norm / k_rstd (decode.cu:415-456) for decode batches
 * above 16 sequences per GPU. */

/* The K split (blocks per cluster) stream_gemm chooses for `rows` rows and a [N][K] weight matrix when called with
 * split 0; 0 for shapes it does not take. */
int stream_gemm_split(int rows, int N, int K);

/*
 * y = epilogue(norm?(x) . W^T). x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3);
 * resid bf16 [rows][N] for epilogue 1 (may be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding
 * the product), 2 relu^2, 3 fp32 store. norm_input != 0 applies the parameter-free RMS norm (eps FLT_EPSILON) to x,
 * as a per-row scale of the fp32 product. rows <= 256; N a multiple of 128; K a multiple of 64; x, w, y, resid
 * 16-byte aligned. split: 1..8 blocks share one feature tile's K range (at most K / 64), 0 = automatic. next_w, next_bytes:
 * optional (NULL, 0): the weights the next call on this stream will read, 16-byte aligned and a multiple of 16
 * bytes; they are prefetched into L2 while this call runs. status: optional device word for NCB_DEV_WAIT_TIMEOUT.
 * Launched with programmatic stream serialisation.
 */
int stream_gemm(const void *x, const void *w, const void *resid, void *y, int rows, int N, int K, int norm_input,
                int epilogue, int split, const void *next_w, long long next_bytes, int *status, void *stream);

/* stream_gemm's residual epilogue followed by the NEXT layer's stream mix (see skinny_gemm_mix):
 * y = bf16(l1 * bf16(resid + bf16(x . W^T)) + l2 * x0), x0 bf16 [rows][N], 16-byte aligned. */
int stream_gemm_mix(const void *x, const void *w, const void *resid, const void *x0, float l1, float l2, void *y, int rows,
                    int N, int K, int norm_input, int split, const void *next_w, long long next_bytes, int *status,
                    void *stream);

/* ---- library tile_gemm --------------------------------------------------------------------------------------
 * The same GEMM for any number of rows as a tiled tcgen05 kernel (128 rows x 256 features per tile, TMA-staged operands,
 * two accumulators in tensor memory so that the epilogue of one tile overlaps the MMAs of the next, one persistent
 * block per SM): the GEMMs of prefill passes and of decode steps above 64 sequences, where the reference runs k_wgmma
 * over prompt rows (model/kernels/decode.cu:232-359,1041-1051). */

/*
 * y = epilogue(x . W^T). x bf16 [rows][K]; w bf16 [N][K]; y bf16 [rows][N] (fp32 for epilogue 3); resid bf16 [rows][N]
 * for epilogue 1 (may be y itself). epilogue: 0 store, 1 residual add (in bf16, after rounding the product), 2 relu^2,
 * 3 fp32 store. Any rows >= 0; N a multiple of 128 (tiles are 256 wide when N is a multiple of 256); K a multiple of
 * 64; all pointers 16-byte aligned. No fused input norm: passes of this size keep the normed rows in memory
 * (add_rms_norm). status: optional device word for NCB_DEV_WAIT_TIMEOUT. Launched with programmatic stream
 * serialisation.
 */
int tile_gemm(const void *x, const void *w, const void *resid, void *y, long long rows, int N, int K, int epilogue,
              int *status, void *stream);

/*
 * tile_gemm with the kernel form chosen by the caller. form 1: one block per 128 x 256 (or 128 x 128) tile. form 2: a
 * pair of blocks on neighbouring SMs per 256 x 256 or 256 x 320 tile (tcgen05 cta_group::2: each block stages its own
 * 128 rows of x and half of the W tile, so a block loads a third less per product; the 320-wide tile is taken where it
 * makes fewer, fuller rounds, e.g. N = 1280); N must be a multiple of 256 or 640, else NCB_ERR_UNSUPPORTED. form 0:
 * tile_gemm's own choice (pairs where they apply and rows > 128). All forms give the same bits. No counterpart in the
 * reference (its GEMM is one kernel form).
 */
int tile_gemm_form(const void *x, const void *w, const void *resid, void *y, long long rows, int N, int K, int epilogue,
                   int form, int *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif
