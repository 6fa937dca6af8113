/*
 * pace_b200.h - C ABI of the B200 (sm_100a) KV-cache hot path.
 *
 * Every entry point takes plain pointers and sizes, returns an int status
 * (PACE_OK == 0) and never throws.  Device pointers are marked "device";
 * `stream` is a cudaStream_t passed as void*.  All work is stream-ordered: no
 * call synchronises unless it says so.
 *
 * The library replaces, for CUDA callers, what the reference does on the CPU in
 *   pace/llm/cache.py            (append, growth, rollback, beam gather)
 *   csrc/ops/attention.cpp       (the pace::attention custom op)
 *   csrc/ops/kernels/attention_kernels.cpp (the four-primitive SDPA sequence)
 * Each declaration cites the reference interface it stands in for.
 */
#ifndef PACE_B200_H_
#define PACE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- return codes (host side) ------------------------------------------ */
#define PACE_OK 0
#define PACE_ERR_INVALID 1     /* an argument failed validation; nothing was launched */
#define PACE_ERR_CUDA 2        /* the CUDA runtime reported an error (see pace_last_cuda_error) */
#define PACE_ERR_UNSUPPORTED 3 /* valid request outside what the kernels are built for */

/* ---- sticky device status bits (pool->status[0]) ----------------------- */
#define PACE_DEV_POOL_EXHAUSTED 1 /* reserve: free list ran dry                    */
#define PACE_DEV_OVER_REMOVE 2    /* truncate: remove_len > cached length          */
#define PACE_DEV_BAD_INDEX 4      /* a sequence slot / page id was out of range    */
#define PACE_DEV_TABLE_FULL 8     /* a sequence needs more pages than its table row*/
#define PACE_DEV_WAIT_TIMEOUT 16  /* a bounded in-kernel wait gave up               */

/*
 * Paged KV pool descriptor.  Geometry + device pointers; plain data, copied by
 * value into kernels.  Storage may come from pace_kv_pool_create() or from the
 * caller (pace_kv_pool_bytes + pace_kv_pool_bind, e.g. a torch allocation).
 *
 *   pages        bf16 [n_layers][2 (K,V)][n_pages][n_kv_heads][page_tokens][head_dim]
 *   block_table  int32 [max_seqs][max_pages_per_seq]  logical page -> physical page
 *   seq_len      int32 [n_layers][max_seqs]  cached tokens, per layer
 *                (the reference keeps one seq_len per layer object, cache.py:184)
 *   seq_pages    int32 [max_seqs]   pages a slot owns; capacity = seq_pages*page_tokens
 *   page_ref     int32 [n_pages]    reference counts (beam gather shares pages)
 *   free_stack   int32 [n_pages]    free physical pages; counters[0] = number free
 *   counters     int32 [8 + n_layers] [0] free pages, [2] pages shared after a gather, [8 + layer] append ticket
 *   status       int32 [4]          [0] sticky PACE_DEV_* bits
 *   table_tmp    int32 [max_seqs][max_pages_per_seq + 1]   scratch of pace_kv_gather
 *
 * page_tokens is the physical page size (the Python host uses 64: one page is one K/V chunk of
 * the attention kernels).  The reference's capacity (whole `tokens_per_split` segments,
 * cache.py:177-181, 292-313) is host bookkeeping on top of the pages and does not depend on it;
 * a page of exactly tokens_per_split tokens makes the two coincide.
 *
 * Between calls the pool's memory belongs to the library: only its kernels write it.
 */
typedef struct pace_kv_pool {
  int32_t n_layers, n_kv_heads, head_dim, page_tokens;
  int32_t n_pages, max_seqs, max_pages_per_seq, owns_memory;
  void* pages;          /* device */
  int32_t* block_table; /* device */
  int32_t* seq_len;     /* device */
  int32_t* seq_pages;   /* device */
  int32_t* page_ref;    /* device */
  int32_t* free_stack;  /* device */
  int32_t* counters;    /* device */
  int32_t* status;      /* device */
  int32_t* table_tmp;   /* device */
} pace_kv_pool_t;

const char* pace_last_cuda_error(void);
const char* pace_version(void);

/* ---- pool lifetime ------------------------------------------------------
 * Reference: BMCKVCache.__init__ / _create_new_segment allocate torch buffers
 * (pace/llm/cache.py:175-193, 242-266); here one pool per model instance is
 * carved into pages once and segments become block-table entries. */
int pace_kv_pool_bytes(const pace_kv_pool_t* geom, uint64_t* pages_bytes, uint64_t* meta_bytes);
int pace_kv_pool_bind(pace_kv_pool_t* pool, void* pages_mem, void* meta_mem); /* host-only pointer carving */
int pace_kv_pool_create(pace_kv_pool_t* pool);  /* cudaMalloc for pages+meta of the filled-in geometry, then reset */
int pace_kv_pool_destroy(pace_kv_pool_t* pool); /* frees what pace_kv_pool_create allocated */
int pace_kv_pool_reset(const pace_kv_pool_t* pool, void* stream); /* all slots empty, all pages free */
/* Sticky status and the kernels' bounded waits.  Every in-kernel wait (on a ring stage, on a result
 * slot) gives up after about a quarter of a second, raises PACE_DEV_WAIT_TIMEOUT and lets its thread
 * block return; the first wait of a block to give up also releases the block's other waits, so a block
 * leaves after one such interval, not one per role.  While the bit stands, every later attention launch
 * on the pool returns at once without touching its output: the host reads the word
 * (pace_kv_pool_query), deals with the cause and clears it (pace_kv_pool_clear_status) to restore
 * service.  (No counterpart in the reference, which has no device.)
 *
 * pace_selftest_wait_timeout makes one wait run out on purpose, harmlessly: a one-block kernel waits on
 * a barrier nobody arrives on for about limit_us microseconds (1 .. 1e6), gives up and raises the bit
 * on this pool.  For health checks and for testing the host's handling of the bit. */
int pace_selftest_wait_timeout(const pace_kv_pool_t* pool, int32_t limit_us, void* stream);
/* Synchronising read of {status bits, free pages, 0, 0}. */
int pace_kv_pool_query(const pace_kv_pool_t* pool, int32_t out[4], void* stream);
int pace_kv_pool_clear_status(const pace_kv_pool_t* pool, void* stream);

/* Give back every page of the listed slots and zero their lengths (all layers).
 * Reference: cache objects are dropped with the manager (generator.py:396-410). */
int pace_kv_seq_release(const pace_kv_pool_t* pool, const int32_t* seq_ids /*device*/, int32_t batch, void* stream);

/* ---- append -------------------------------------------------------------
 * Reference: BMCKVCache.update_cache / DynamicKVCache.update_cache
 * (pace/llm/cache.py:268-326, 370-400).
 *
 * pace_kv_reserve makes sure every listed slot owns ceil((seq_len[layer]+n)/page_tokens)
 * pages (popping the free list; copy-on-write of a shared last page after a beam
 * gather).  pace_kv_append copies n new K/V rows per sequence into the slots
 * [seq_len, seq_len+n) and then advances seq_len[layer].  k_new / v_new are bf16
 * [batch][n_kv_heads][n_new][head_dim] addressed through element strides (the last
 * dimension is contiguous), so the transposed view a model produces needs no copy.
 * n_new_per_seq (device, optional) gives ragged counts <= n_new. */
int pace_kv_reserve(const pace_kv_pool_t* pool, int32_t layer, const int32_t* seq_ids, int32_t batch,
                    int32_t n_new, const int32_t* n_new_per_seq, void* stream);
int pace_kv_append(const pace_kv_pool_t* pool, int32_t layer, const int32_t* seq_ids, int32_t batch,
                   int32_t n_new, const int32_t* n_new_per_seq, const void* k_new, const void* v_new,
                   int64_t stride_b, int64_t stride_h, int64_t stride_t, void* stream);
/* Ordering of the two append entry points against an attention launch in front of them on the
 * stream: the library remembers, per stream, the pool and layer its newest attention launch reads.
 * An append to ANOTHER layer (the decoder-layer pattern attn(l), append(l+1), attn(l+1)) starts
 * while that launch is still running (programmatic dependent launch) - it touches nothing the
 * launch reads.  An append to the SAME pool and layer, or a pace_kv_append_rope whose q_out is the
 * q of that launch, is ordered behind its completion like any other kernel. */

/* One launch for a whole decode step: the rows of layers [layer_begin, layer_end) at once.
 * Reference: the same BMCKVCache.update_cache (cache.py:268-326), called once per layer per
 * generated token (llama.py:159); here the per-layer calls of a step collapse into one kernel that
 * runs after the step's last attention launch, which is possible because the attention entry
 * points can take the step's new row straight from the caller's buffer (PACE_ATTN_PENDING_ROW).
 * k_new / v_new are bf16 [layer][batch][n_kv_heads][n_new][head_dim] through element strides
 * (stride_l first; head_dim contiguous, rows 16-byte aligned); layer `layer_begin` is at offset 0.
 * Every listed layer's seq_len advances by the same counts.  pace_kv_reserve for the step must have
 * run (any one layer: pages are shared by all layers).  k_new = v_new = NULL advances the lengths
 * only: for a step whose rows every layer's attention launch has stored already
 * (PACE_ATTN_PENDING_ROW).  The kernel is ordered behind everything in
 * front of it on the stream and in front of everything behind it (no programmatic overlap). */
int pace_kv_append_layers(const pace_kv_pool_t* pool, int32_t layer_begin, int32_t layer_end,
                          const int32_t* seq_ids, int32_t batch, int32_t n_new, const int32_t* n_new_per_seq,
                          const void* k_new, const void* v_new, int64_t stride_l, int64_t stride_b,
                          int64_t stride_h, int64_t stride_t, void* stream);

/* ---- RoPE + append in one pass -----------------------------------------------
 * Reference: the step in front of the append in every decoder layer,
 * pace/llm/models/llama.py:130-165: q/k/v are viewed as heads, RotaryEmbedding's
 * callable rotates q and k (pace/ops/rotary_embedding.py:375-441: table rows picked
 * by position id, cast to the activations' dtype, NeoX halves or GPT-J pairs, every
 * product and sum rounded to that dtype), then update_cache stores k and v.
 *
 * pace_kv_append_rope reads the projection outputs once, writes the rotated queries
 * to q_out (which may be q itself) and the rotated keys and the values straight into
 * the slots [seq_len, seq_len + n) of the paged cache, then advances seq_len[layer]
 * as pace_kv_append does (pace_kv_reserve must have run).  All tensors are bf16
 * addressed as [batch][token][head][head_dim] through element strides (head_dim
 * contiguous, 16-byte aligned rows): the untransposed output of a fused or split
 * QKV projection needs no copy.  cos/sin are the operator's fp32 tables
 * [table_rows][rotary_dim / 2]; table_row[b * row_stride_b + t] names the row of
 * token t of sequence b (the position id, already shifted for longrope).
 * rotary_dim <= head_dim, a multiple of 16; elements beyond it pass through.
 * A row index outside the table raises PACE_DEV_BAD_INDEX and leaves that token
 * unrotated. */
typedef struct {
  const void* q;        int64_t q_stride_b, q_stride_t, q_stride_h;
  const void* k;        int64_t k_stride_b, k_stride_t, k_stride_h;
  const void* v;        int64_t v_stride_b, v_stride_t, v_stride_h;
  void* q_out;          int64_t o_stride_b, o_stride_t, o_stride_h;
  const int32_t* table_row; /* device */
  int64_t row_stride_b;
  const float* cos_table;   /* device, fp32 [table_rows][rotary_dim / 2] */
  const float* sin_table;
  int32_t table_rows;
  int32_t rotary_dim;
  int32_t gptj_pairs;       /* 0: NeoX halves (d, d + rotary_dim / 2); 1: GPT-J pairs (2d, 2d + 1) */
  int32_t n_q_heads;
  /* Deferred append (decode steps): when k_stage is not NULL the rotated keys and the values go to
   * these staging rows, bf16 [batch][n_kv_heads][token][head_dim] through element strides, instead of
   * the pool, and seq_len is left alone - the rows then ride along with the layer's decode launch
   * (PACE_ATTN_PENDING_ROW) and are committed by pace_kv_append_layers. */
  void* k_stage;
  void* v_stage;
  int64_t stage_stride_b, stage_stride_h, stage_stride_t;
} pace_rope_args_t;
int pace_kv_append_rope(const pace_kv_pool_t* pool, int32_t layer, const int32_t* seq_ids, int32_t batch,
                        int32_t n_new, const int32_t* n_new_per_seq, const pace_rope_args_t* rope, void* stream);

/* ---- rollback -------------------------------------------------------------
 * Reference: BMCKVCache.remove_cache (cache.py:224-240): seq_len -= n, pages kept,
 * data untouched.  Over-removal leaves the length alone and raises
 * PACE_DEV_OVER_REMOVE.  layers [layer_begin, layer_end).  remove_per_seq (device,
 * optional) overrides the scalar per sequence (PARD with per-sequence acceptance). */
int pace_kv_truncate(const pace_kv_pool_t* pool, int32_t layer_begin, int32_t layer_end,
                     const int32_t* seq_ids, int32_t batch, int32_t remove_len,
                     const int32_t* remove_per_seq, void* stream);

/* ---- PARD acceptance ---------------------------------------------------------
 * Reference: Generator._postprocess_speculated_tokens (pace/llm/generator.py:669-713), one sequence
 * at a time on the host there.  Per sequence b of the batch: accept the leading matches among the
 * first d - 1 draft tokens (draft i is accepted while target_next[b][i] == drafts[b][i] and
 * i < n_target[b]; with `forced` given, while forced[b][i] != 0 instead), always keep one more token
 * (the target's own), and say how far the two caches roll back:
 *     keep[b]          = 1 + accepted                                  in [1, d]
 *     target_remove[b] = d - keep + 1  if keep < d,  else 0            (generator.py:696-702)
 *     draft_remove[b]  = d - 1                                         (generator.py:706)
 *     kept[b][0 .. keep)  the tokens that join the history: the accepted ones (the target's tokens;
 *                         the drafts when acceptance is forced) and then target_next[b][min(keep - 1, n_target[b] - 1)]
 * The arrays feed pace_kv_truncate (remove_per_seq) and the next step's ragged counts directly:
 * nothing of a speculative step has to come back to the host.  drafts int64 [batch][d], target_next
 * int64 [batch][d + 1] (n_target[b] of them valid), forced uint8 [batch][d - 1] or NULL, kept int64
 * [batch][d]; all device. */
int pace_pard_accept(const int64_t* drafts, const int64_t* target_next, const int32_t* n_target,
                     const uint8_t* forced, int32_t batch, int32_t d, int32_t* keep, int32_t* target_remove,
                     int32_t* draft_remove, int64_t* kept, void* stream);

/* ---- beam gather ----------------------------------------------------------
 * Reference: KVCacheBase.update_cache_with_beam_indices (cache.py:161-167):
 * row i of the batch becomes a copy of old row beam_idx[i].  Index-only here: the
 * block-table rows and lengths are permuted and page reference counts adjusted. */
int pace_kv_gather(const pace_kv_pool_t* pool, const int32_t* seq_ids, const int64_t* beam_idx /*device*/,
                   int32_t batch, void* stream);

/* ---- cache read-back --------------------------------------------------------
 * Materialises what the reference's update_cache returns (cache.py:326): dense
 * bf16 [batch][n_kv_heads][cap_tokens][head_dim] K and V, rows beyond a slot's
 * pages zero-filled. */
int pace_kv_read_dense(const pace_kv_pool_t* pool, int32_t layer, const int32_t* seq_ids, int32_t batch,
                       void* k_out, void* v_out, int32_t cap_tokens, void* stream);

/* ---- attention --------------------------------------------------------------
 * Reference: pace::attention (csrc/ops/attention.cpp:18-97, schema :104-108) and
 * kernels::attention_kernel Method 1 (csrc/ops/kernels/attention_kernels.cpp:218-257):
 * softmax(Q K^T / sqrt(D) + mask) V with fp32 accumulation, output in Q's dtype.
 *
 * Paged form: K/V come from the pool (layer, slots); the additive mask of the
 * reference (causal tail + left padding + BMC padding columns, llama.py:294-310)
 * is expressed by integers: kv_len = seq_len[layer][slot] (the q_len newest
 * tokens included), query i sees keys [kv_start, kv_len - q_len + i].
 * q / out are bf16 [batch][n_q_heads][q_len][head_dim] through element strides.
 * GQA: n_q_heads = G * n_kv_heads, query head h reads KV head h / G, which is
 * what the reference obtains by repeat_kv before caching (llama.py:152-158). */
typedef struct pace_attn_args {
  const pace_kv_pool_t* pool;
  int32_t layer;
  int32_t batch;
  int32_t n_q_heads;
  int32_t q_len;            /* 1 = decode; d+1 = verify; chunk = prefill */
  const int32_t* seq_ids;   /* device [batch]; NULL = slots 0..batch-1 */
  const int32_t* kv_start;  /* device [batch] or NULL (no left padding) */
  const int32_t* q_lens;    /* device [batch] or NULL: ragged query counts <= q_len */
  const void* q;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  void* out;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  float scale;              /* 0 -> 1/sqrt(head_dim) */
  void* workspace;          /* device scratch, pace_attn_workspace_bytes(); zero it once after allocation */
  uint64_t workspace_bytes;
  uint32_t flags;           /* PACE_ATTN_* bits, 0 = none */
  /* PACE_ATTN_PENDING_ROW only: the step's new K and V row of every (sequence, kv head), bf16
   * [batch][n_kv_heads][head_dim] through element strides (head_dim contiguous, rows 16-byte aligned). */
  const void* k_pending;
  const void* v_pending;
  int64_t pending_stride_b, pending_stride_h;
  /* At most this many thread blocks (a caller that shares the GPU with work on another stream);
   * 0 = the kernels' own choice, one per SM or two for the four-warp decode form.  Any value gives
   * the same result: the kernels cut the work into as many contiguous ranges as there are blocks. */
  int32_t max_ctas;
} pace_attn_args_t;

/* Never cut one (sequence, KV head) stream of keys across thread blocks.  The kernels normally decide
 * this on the device from the cached lengths: cutting balances ragged batches, but the pieces meet in
 * the workspace, and because the host cannot know the outcome a K/V append launched behind the
 * attention launch has to hold its completion until that launch has completed (the next attention
 * launch orders itself after the append only).  A launch with this bit set touches no workspace, the
 * append behind it completes on its own, and the next layer's attention launch learns of this one's
 * completion directly: about 0.5 us less per layer.  Set it when batch * n_kv_heads is not small
 * against the number of SMs and the lengths are about even (the host mirror of the reference's one
 * seq_len per layer, cache.py:184, is enough to tell).  It only changes the schedule, never the result. */
#define PACE_ATTN_WHOLE_UNITS 1u

/* Decode (q_len == 1) over the cache PLUS one row per sequence that is not in the cache yet: the
 * launch first stores k_pending / v_pending in the row's slot of the pool - row number seq_len of
 * the sequence, whose page pace_kv_reserve must have provided - and then attends over keys
 * [kv_start, seq_len].  seq_len itself is NOT advanced.  The result is what pace_kv_append of that
 * row followed by a plain decode launch gives.  This takes the per-layer append out of the chain of
 * a decode step (llama.py:159-165 does update_cache, then attention, in every layer): the rows stay
 * in the caller's staging buffer, every layer's attention launch follows the previous layer's
 * directly, and one pace_kv_append_layers after the last layer advances all layers' lengths (it
 * stores the rows again, which changes nothing).  A row that is never committed is simply a stale
 * row beyond seq_len, as after a rollback.  Served by the tensor-core kernels for every group size
 * below 33 query heads per KV head; PACE_ERR_UNSUPPORTED otherwise. */
#define PACE_ATTN_PENDING_ROW 2u

/* Decode launches normally begin by waiting for the kernel in front of them on the stream
 * (a programmatic dependent launch: only the set-up overlaps).  When the library knows that its own
 * newest launch on the stream was an attention launch - so nothing of the pool this launch reads
 * (lengths, block table, pages) can have been written by the kernel directly in front - a
 * whole-unit decode launch starts streaming K/V pages at once and waits only before it touches q,
 * the pending rows and out.  The K/V stream then runs beside the tail of the kernel in front (the
 * previous layer's attention, or the projection that produces q).  This bit forbids that: set it
 * if seq_ids, kv_start or the pool were written by a kernel of your own directly in front. */
#define PACE_ATTN_NO_EARLY_KV 4u

/* Decode: keep the form with eight consumer warps and one thread block per SM (the kernels fall
 * back to it by themselves when the workspace or shared memory has no room for two blocks per SM). */
#define PACE_ATTN_ONE_CTA_PER_SM 8u

uint64_t pace_attn_workspace_bytes(int32_t batch, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                   int32_t q_len);
/* q_len == 1.  The grouped query heads of a KV head are packed into one mma.sync tile (any group
 * size); groups of 1 or 2 (plain multi-head attention) run on the CUDA-core kernel instead, whose
 * packed fp32 FMAs cost less than a tile that is seven eighths padding. */
int pace_attn_decode(const pace_attn_args_t* a, void* stream);
/* The CUDA-core decode kernel whatever the group size (1, 2, 4 or 8 query heads per KV head;
 * PACE_ERR_UNSUPPORTED otherwise): 8 lanes per K/V row, packed fp32 FMAs, warp-shuffle online
 * softmax - the form the reference's head-by-head CPU loop maps to most directly.  pace_attn_decode
 * picks it only for groups of 1 or 2; pace_attn_verify with q_len = 1 is the tensor-core form. */
int pace_attn_decode_cuda_cores(const pace_attn_args_t* a, void* stream);
/* q_len >= 1 query tokens per sequence, causal among themselves (PARD verify: d + 1 tokens; a
 * prefill chunk: hundreds).  Tiles of 33 and more query rows (tokens x grouped heads) run on the
 * tcgen05 tensor cores, smaller ones on mma.sync.  pace_attn_prefill is the same entry point under
 * the name the chunked-prefill caller expects. */
int pace_attn_verify(const pace_attn_args_t* a, void* stream);
int pace_attn_prefill(const pace_attn_args_t* a, void* stream);

/* Decode attention without any allocation.  (No counterpart in the reference: its CPU op
 * allocates its score tensor on every call, attention_kernels.cpp:222-226.)
 *
 * For hosts that cannot allocate device memory where a decode step runs - an engine that owns the
 * whole device and lends this library nothing, a serving loop whose memory was fixed at start-up,
 * a thread that must not enter the allocator - and so cannot supply pace_attn_decode's workspace.
 * Same arguments and result as pace_attn_decode; `workspace` / `workspace_bytes` are ignored and
 * the scratch is a fixed device array inside the library (about 3.4 MB per GPU, held until the
 * process exits).  Limits, refused with PACE_ERR_UNSUPPORTED beyond them: at most 16 query heads per
 * KV head, head_dim <= 128, batch * n_kv_heads <= 65536, at most 192 SMs.  The first call on a device
 * resolves the array's address there (make it before any stream capture) and keeps it for the life
 * of the process: after a cudaDeviceReset the kept address is stale and the entry point must not be
 * used again in that process.  Calls share the array: issue them on one stream, or otherwise keep
 * them from overlapping on the GPU. */
int pace_attn_decode_static(const pace_attn_args_t* a, void* stream);

/* Dense form with the reference op's exact operands: q [B,N,S,H], k/v [B,Nkv,L,H]
 * contiguous bf16, additive mask [B,1,mask_rows,L] (mask_rows 1 or S; bf16 or fp32;
 * may be NULL), out [B,N,S,H].  Reference: pace::attention, attention.cpp:18-97. */
int pace_attention_dense(const void* q, const void* k, const void* v, const void* mask, int32_t mask_is_fp32,
                         int32_t mask_rows, void* out, int32_t B, int32_t N, int32_t Nkv, int32_t S, int32_t L,
                         int32_t H, void* workspace, uint64_t workspace_bytes, void* stream);

/* ---- op timing -------------------------------------------------------------------
 * Reference: PROFILE_PACE_FUNCTION / TimingLogger (csrc/core/logging.h:144-212, used at
 * csrc/ops/attention.cpp:24), switched on by the environment variable PACE_LOG_LEVEL=profile.
 * With that value set when the library is loaded, the attention, append, rollback, gather and linear
 * entry points record a CUDA event on their stream before and after their launches and a line
 *     [PACE profile] pace::<op>,<shapes>,<milliseconds>
 * goes to stderr once both events have completed: at a later profiled call, at pace_profile_flush
 * (which waits for the outstanding ones and returns how many it wrote or dropped) or at process exit.
 * The time is device time between the two events.  Calls made while their stream is being captured
 * into a CUDA graph are not timed.  No other value of the variable changes anything. */
int pace_profile_enabled(void);
int pace_profile_flush(void);

/* ---- weight-streaming linear layer for decode steps ------------------------------
 * Reference: the Linear operator's GEMM back ends on a decoder layer's projections and MLP
 * (pace/ops/backends/tpp.py:19-63, pace/ops/backends/imbps.py:19-92, csrc/ops/libxsmm_linear.cpp:225-241).
 * y[M][N] = x[M][K] w[N][K]^T, bf16 in and out, fp32 accumulation, no bias; M <= 32 tokens, N and K
 * multiples of 128 (PACE_ERR_UNSUPPORTED otherwise: larger token counts are compute-bound and belong to
 * a library GEMM).  Row pitches are in elements (x_stride, w_stride multiples of 8, bases 16-byte
 * aligned).  `workspace` is pace_linear_workspace_bytes(largest N) bytes of 32-byte aligned device memory, zeroed once
 * after allocation and not shared by launches that can overlap on the GPU (one per stream); the kernel
 * leaves it zeroed.  `status` (device, may be NULL) takes PACE_DEV_WAIT_TIMEOUT if a bounded wait runs
 * out.  Launched as a programmatic dependent: the weights are fetched while the kernel in front still
 * runs, only x waits for it. */
uint64_t pace_linear_workspace_bytes(int32_t n_max);
int pace_linear_skinny(const void* x, int64_t x_stride, const void* w, int64_t w_stride, void* y, int64_t y_stride,
                       int32_t M, int32_t N, int32_t K, void* workspace, uint64_t workspace_bytes, int32_t* status,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PACE_B200_H_ */
