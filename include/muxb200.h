/*
 * muxb200 — C ABI of the B200 (sm_100a) paged decode attention path for
 * MuxServe's FlexStore head-granular unified KV pool.
 *
 * Plain pointers, sizes and strides only: no torch types, no exceptions.
 * Every entry point validates its arguments on the host and returns 0 or a
 * negative mux_status_t BEFORE anything is launched; kernels are enqueued on
 * the stream the caller passes and never synchronise the host.
 *
 * Pool geometry (muxserve/flexstore/manager.py:456-468 in the reference):
 *   key pool    [num_blocks][head_size/x][block_size][x]   x = 16 / sizeof(elem)
 *   value pool  [num_blocks][head_size][block_size]
 * A block holds block_size tokens of ONE head of ONE layer of ONE model; the
 * pool has no layer and no head dimension.  head_size is 128.
 */
#ifndef MUXB200_H_
#define MUXB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  MUX_OK = 0,
  MUX_ERR_NULL_POINTER = -1,
  MUX_ERR_BAD_DTYPE = -2,
  MUX_ERR_BAD_HEAD_SIZE = -3,     /* only 128 (muxserve/flexstore/manager.py:336-337) */
  MUX_ERR_BAD_BLOCK_SIZE = -4,    /* only 8, 16, 32 (muxserve/arg_utils.py:61-65) */
  MUX_ERR_MISALIGNED = -5,        /* a pointer or stride breaks the 16-byte rule */
  MUX_ERR_BAD_SHAPE = -6,         /* negative / inconsistent sizes */
  MUX_ERR_BAD_GROUP = -7,         /* q heads not a multiple of kv heads, or group too large */
  MUX_ERR_WORKSPACE_TOO_SMALL = -8,
  MUX_ERR_CUDA = -9,              /* a CUDA runtime call failed; see mux_last_cuda_error */
  MUX_ERR_BAD_HANDLE = -10,
  MUX_ERR_BUFFER_TOO_SMALL = -11,
  MUX_ERR_UNKNOWN_REQUEST = -12,
  MUX_ERR_TOO_LARGE = -13         /* beyond a stated fixed capacity */
} mux_status_t;

typedef enum { MUX_DTYPE_F16 = 0, MUX_DTYPE_BF16 = 1 } mux_dtype_t;

/* Bits of the device status word (mux_device_status). */
#define MUX_DEV_BAD_BLOCK_ID 1u   /* a block id outside [0, num_blocks) was met; block 0 was read in its place */
#define MUX_DEV_WAIT_TIMEOUT 2u   /* a bounded wait on a staged copy ran out */
#define MUX_DEV_BAD_CONTEXT 4u    /* a context length above max_context_len (or < 0) was met */
#define MUX_DEV_BAD_SLOT 8u       /* a slot outside the pool was met and skipped */
#define MUX_DEV_BAD_HEAD_MAPPING 16u /* head_mapping does not give every kv head num_q_heads/num_kv_heads q heads */
#define MUX_DEV_INTERNAL 32u      /* a kernel found a precondition of its own broken (shared-memory alignment) and left */
#define MUX_DEV_BAD_GROUP 64u     /* an item_group outside [1, max_group] was met; at most max_group heads were computed */

/* Bits of the `flags` field of the attention argument structs.
 *
 * MUX_ATTN_EARLY_KV: the kernels of this library are launched with programmatic dependent launch: a launch
 * may become resident while the kernels just ahead of it in the stream are still draining, and normally
 * waits for them before it reads anything.  With this bit the caller states that the launch's index data
 * (block_tables, context lengths, seq_rows, head_mapping, the item arrays, units) and the KV blocks the
 * block lists name are NOT written by the (up to two) kernels directly ahead of it in the stream; each CTA
 * then resolves its item and stages its first KV blocks before it waits, and only q, the new K/V rows and
 * all writes (pool, workspace, out) stay behind the wait.  True for a decode step through
 * mux_decode_attention(_mixed): the kernel ahead of a layer's attention produced q/k/v, and the previous
 * layer's attention appended to blocks of its own layer.  NOT true for mux_paged_attention right after
 * mux_reshape_and_cache of the same layer, nor right after mux_block_table_append: leave the bit clear there. */
#define MUX_ATTN_EARLY_KV 1

const char* mux_strerror(int status);
/* cudaError_t of the last failing CUDA call made by this library on the calling thread. */
int mux_last_cuda_error(void);
/* Library ABI version (bumped when a struct below changes). */
int mux_abi_version(void);

/* ------------------------------------------------------------------------
 * reshape_and_cache — append new tokens' K/V rows to the pool.
 *
 * Replaces the MuxServe-vLLM fork's cache op reached from
 * muxserve/flexserver/models/llama.py:160-161 (PagedAttentionWithRoPE) with
 * slots produced by csrc/batch_scheduler.h:42-67:
 *   s = slot_mapping[t, h];  b = s / block_size;  o = s % block_size
 *   key_pool  [b][d / x][o][d % x] = k[t, h, d]
 *   value_pool[b][d][o]            = v[t, h, d]
 * A negative slot skips the row.  k and v may be strided views of a fused
 * qkv tensor (llama.py:157-158): strides are in elements.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* k;               /* [num_tokens, num_kv_heads, head_size] */
  const void* v;
  int64_t k_token_stride;      /* elements between tokens */
  int64_t k_head_stride;       /* elements between heads (normally head_size) */
  int64_t v_token_stride;
  int64_t v_head_stride;
  void* key_cache;
  void* value_cache;
  int64_t num_blocks;          /* pool size in blocks */
  const int64_t* slot_mapping; /* slot of (token t, head h) at [t*slot_token_stride + h*slot_head_stride] */
  int64_t slot_token_stride;   /* elements; L*H for the reference's [T, L, H] tensor sliced at one layer */
  int64_t slot_head_stride;    /* elements; 1 for that slice */
  int32_t num_tokens;
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t block_size;
  int32_t dtype;               /* mux_dtype_t */
  int32_t reserved;
} mux_cache_write_args_t;

int mux_reshape_and_cache(const mux_cache_write_args_t* args, void* cuda_stream);

/* ------------------------------------------------------------------------
 * paged_attention — decode attention of one new query token per sequence
 * over block-table-indirected KV blocks.
 *
 * Replaces the fork's attention op reached from llama.py:160-161; argument
 * meaning follows paged_attention(out, q, key_cache, value_cache,
 * head_mapping, scale, block_tables, context_lens, block_size,
 * max_context_len).  In MuxServe mode block_tables for one layer is
 * [num_seqs, num_kv_heads, max_blocks] (muxserve/flexserver/llm_runtime.py:327):
 * every (sequence, kv head) has its own block list.
 *   out[s, hq, :] = softmax_j(scale * q[s, hq, :] . K_j) . V_j ,  j < context_lens[s]
 * with kv head h = head_mapping[hq] (NULL = hq / (num_q_heads/num_kv_heads)).
 * Every block list must have ceil(max_context_len / block_size) readable
 * entries (the width the reference gives the table); entries at or beyond
 * ceil(context_len / block_size) may hold anything (the reference leaves them
 * uninitialised): they are never used as block ids.
 *
 * Long contexts are split into partitions of partition_size tokens that are
 * combined through the caller's workspace (flash-decoding).  Sizes come from
 * mux_paged_attention_workspace_size; workspace may be NULL when that is 0, its
 * contents need no initialisation, and two launches that may overlap on the GPU
 * must not share it.
 * ---------------------------------------------------------------------- */
typedef struct {
  void* out;                   /* [num_seqs, num_q_heads, head_size] */
  const void* q;
  int64_t q_seq_stride;        /* elements between sequences */
  int64_t q_head_stride;       /* elements between q heads (normally head_size) */
  int64_t out_seq_stride;
  int64_t out_head_stride;
  const void* key_cache;
  const void* value_cache;
  int64_t num_blocks;
  const int32_t* head_mapping; /* [num_q_heads] device, or NULL for contiguous groups */
  const int32_t* block_tables; /* device */
  int64_t bt_seq_stride;       /* elements */
  int64_t bt_head_stride;      /* elements; 0 = all kv heads read ONE list (and so the same K/V, a pool block holding
                                  one head): meaningful for num_kv_heads == 1 or read-only probing, and refused by
                                  mux_decode_attention when num_kv_heads > 1 (its kv heads would append to one slot) */
  const int32_t* context_lens; /* [num_seqs] device */
  const int32_t* seq_rows;     /* NULL, or [num_seqs] device: sequence s uses row seq_rows[s] of block_tables
                                  (a persistent table kept on the device, see mux_block_table_append) */
  float scale;
  int32_t num_seqs;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t block_size;
  int32_t max_context_len;
  int32_t dtype;               /* mux_dtype_t */
  int32_t partition_size;      /* tokens, multiple of block_size; 0 = library heuristic */
  int32_t num_stages;          /* depth of the shared-memory block ring (multiple of 4, <= 16); 0 = default */
  int32_t flags;               /* MUX_ATTN_* bits, 0 = none */
  int32_t num_units;           /* 0, or the length of `units` */
  /* Optional work list (see mux_attn_mixed_args_t.units): units[u] = item | partition << 24 with
   * item = sequence * num_kv_heads + kv head, every partition of every sequence with context_lens > 0 exactly
   * once, fullest first.  For a host that knows the context lengths it uploads (the reference's scheduler does,
   * csrc/batch_scheduler.cpp:135-140): the launch then has no CTA for a partition a sequence does not have.
   * partition_size must be given explicitly; num_seqs * num_kv_heads < 2^24.  Negative entries are padding
   * (a list kept at a fixed length for a captured CUDA graph): their CTAs leave at once.  A sequence with an empty
   * context should be listed with its partition 0 (that CTA writes the zero rows); left out, its rows of `out` are
   * not written.  The list is read BEFORE the launch waits for the kernels ahead of it in the stream: it must be
   * complete by then (uploaded by a copy, or written by a kernel that is not the one directly ahead). */
  const int32_t* units;        /* device, [num_units] */
} mux_attn_args_t;

size_t mux_paged_attention_workspace_size(const mux_attn_args_t* args);
int mux_paged_attention(const mux_attn_args_t* args, void* workspace,
                        size_t workspace_bytes, void* cuda_stream);

/* No counterpart in the reference.  Same operation and arguments as
 * mux_paged_attention, for callers that cannot allocate device memory while
 * they run (a worker whose footprint was fixed at start-up, a process sharing
 * the GPU that must not grow, a path on which cudaMalloc is not permitted):
 * the flash-decoding scratch is a fixed MUX_STATIC_SCRATCH_BYTES array inside
 * the library image, so the call itself never allocates or frees anything.
 *  - Returns MUX_ERR_TOO_LARGE when mux_paged_attention_workspace_size(args)
 *    exceeds MUX_STATIC_SCRATCH_BYTES; fall back to mux_paged_attention then.
 *  - The first call on each device resolves the array's device address; make
 *    that first call outside of any stream capture.
 *  - All calls on a device share the one array: two calls whose kernels can
 *    overlap on the GPU (different streams, no ordering) race on it.  Calls on
 *    one stream, or otherwise ordered, are safe; stale contents are harmless
 *    because every value read is written earlier in the same call.
 *  - Every GPU that loads the library holds the array until process exit. */
#define MUX_STATIC_SCRATCH_BYTES (16u << 20)
int mux_paged_attention_static_scratch(const mux_attn_args_t* args, void* cuda_stream);

/* ------------------------------------------------------------------------
 * paged_attention, mixed-model form — ONE launch serves the decode batches
 * of several colocated models that share the pool.  No counterpart in the
 * reference, which runs each model in its own processes
 * (muxserve/muxsched/scheduler.py:167-208); the per-item fields restate what
 * the single-model call derives from (sequence, kv head).
 *
 * An item is one (sequence, kv head) pair of some model:
 *   q rows  [item_q_row[i], item_q_row[i] + item_group[i])  of the packed
 *   q / out matrices [total_q_rows, head_size] attend over the block list
 *   block_tables[i, :] with context length item_context_len[i] and softmax
 *   scale item_scale[i].
 * ---------------------------------------------------------------------- */
typedef struct {
  void* out;                     /* packed [total_q_rows, head_size] */
  const void* q;
  int64_t q_row_stride;          /* elements (normally head_size) */
  int64_t out_row_stride;
  const void* key_cache;
  const void* value_cache;
  int64_t num_blocks;
  const int32_t* block_tables;   /* [num_items, max_blocks] device */
  int64_t bt_item_stride;        /* elements */
  const int32_t* item_context_len; /* [num_items] device */
  const int32_t* item_q_row;     /* [num_items] device */
  const int32_t* item_group;     /* [num_items] device, each in [1, max_group] */
  const float* item_scale;       /* [num_items] device */
  int32_t num_items;
  int32_t max_group;             /* upper bound of item_group, <= 8 */
  int32_t head_size;
  int32_t block_size;
  int32_t max_context_len;
  int32_t dtype;
  int32_t partition_size;
  int32_t num_stages;
  int32_t flags;                 /* MUX_ATTN_* bits, 0 = none */
  int32_t num_units;             /* 0, or the length of `units` */
  /* Optional work list.  Without it the launch has one CTA per (item, partition index up to the longest item's
   * count) and the CTAs past an item's last partition leave at once; with context lengths as skewed as a
   * multiplexed batch's most CTAs are of that kind.  The host knows the lengths, so it may list the real
   * (item, partition) pairs instead: units[u] = item | partition << 24, every partition of every item with
   * item_context_len > 0 exactly once, in the order they should start (longest first).  partition_size must
   * then be given explicitly (the list depends on it); num_items < 2^24. */
  const int32_t* units;          /* device, [num_units] */
} mux_attn_mixed_args_t;

size_t mux_paged_attention_mixed_workspace_size(const mux_attn_mixed_args_t* args);
int mux_paged_attention_mixed(const mux_attn_mixed_args_t* args, void* workspace,
                              size_t workspace_bytes, void* cuda_stream);

/* ------------------------------------------------------------------------
 * decode step — reshape_and_cache and paged_attention of one layer in ONE launch.
 *
 * What PagedAttentionWithRoPE does back to back at muxserve/flexserver/models/llama.py:160-161
 * for a decode batch (one new token per sequence): the new K/V row of every
 * (sequence, kv head) is appended at position context_len - 1 of that pair's
 * block list, i.e. slot block_table[(ctx-1)/block_size]*block_size + (ctx-1)%block_size,
 * the slot csrc/batch_scheduler.h:58-67 puts in slot_mapping, and attention runs over
 * all context_len tokens.  Same results as mux_reshape_and_cache followed by
 * mux_paged_attention, bit for bit.
 * A step may append several tokens per sequence (new_tokens, up to MUX_MAX_FUSED_NEW_TOKENS; the reference
 * itself appends one): k / v then hold new_tokens consecutive rows per sequence, token-major, for positions
 * context_len - new_tokens .. context_len - 1 (context_len counts them all), and the one query of the sequence
 * attends over everything.  With rotary, new key j is rotated at its own position, the query at context_len - 1.
 * ---------------------------------------------------------------------- */
#define MUX_MAX_FUSED_NEW_TOKENS 16
typedef struct {
  mux_attn_args_t attn;
  const void* k;            /* [num_seqs * new_tokens, num_kv_heads, head_size] new rows (strided views allowed) */
  const void* v;
  int64_t k_seq_stride;     /* elements */
  int64_t k_head_stride;
  int64_t v_seq_stride;
  int64_t v_head_stride;
  const void* cos_sin_cache; /* NULL, or rotary cache [max_position][64 cos | 64 sin] in the tensor dtype: q and the */
  int64_t max_position;      /* new k are rotated at position context_len - 1 first (see mux_rotary_embedding) */
  int32_t new_tokens;        /* rows per (sequence, kv head); 0 means 1 */
  int32_t reserved;
} mux_decode_args_t;

/* workspace: mux_paged_attention_workspace_size(&args->attn) */
int mux_decode_attention(const mux_decode_args_t* args, void* workspace, size_t workspace_bytes,
                         void* cuda_stream);

typedef struct {
  mux_attn_mixed_args_t attn;
  const void* k;            /* [num_items * new_tokens, head_size]: new_tokens consecutive rows per item */
  const void* v;
  int64_t k_row_stride;     /* elements */
  int64_t v_row_stride;
  const void* cos_sin_cache; /* as in mux_decode_args_t; one cache for all models of the launch */
  int64_t max_position;
  int32_t new_tokens;        /* as in mux_decode_args_t */
  int32_t reserved;
} mux_decode_mixed_args_t;

/* workspace: mux_paged_attention_mixed_workspace_size(&args->attn) */
int mux_decode_attention_mixed(const mux_decode_mixed_args_t* args, void* workspace,
                               size_t workspace_bytes, void* cuda_stream);

/* ------------------------------------------------------------------------
 * rotary position embedding of q and k, in place — the step PagedAttentionWithRoPE applies before
 * the cache write (parameters at muxserve/flexserver/models/llama.py:138-147: rotary_dim = head
 * size, GPT-NeoX pairing of element d with d + 64).  fp32 arithmetic, one rounding.
 * ---------------------------------------------------------------------- */
typedef struct {
  void* q;                    /* [num_tokens, num_q_heads, 128], may be NULL when num_q_heads == 0 */
  void* k;                    /* [num_tokens, num_kv_heads, 128] */
  int64_t q_token_stride, q_head_stride, k_token_stride, k_head_stride;   /* elements */
  const int64_t* positions;   /* [num_tokens] device */
  const void* cos_sin_cache;  /* [max_position][64 cos | 64 sin], tensor dtype, device */
  int64_t max_position;
  int32_t num_tokens, num_q_heads, num_kv_heads, head_size;
  int32_t dtype;
  int32_t reserved;
} mux_rotary_args_t;

int mux_rotary_embedding(const mux_rotary_args_t* args, void* cuda_stream);

/* ------------------------------------------------------------------------
 * prompt-phase attention — causal self-attention of every prompt over its own tokens, the step
 * PagedAttentionWithRoPE runs on the prompt rows of a batch (muxserve/flexserver/models/llama.py:160-161,
 * prompt lengths from input_metadata.prompt_lens, muxserve/flexserver/llm_runtime.py:298-330) before
 * their K/V rows go to the pool through mux_reshape_and_cache with the slots of
 * csrc/batch_scheduler.h:42-56.  The rows of all prompts are concatenated:
 * prompt i owns rows cu_seqlens[i] .. cu_seqlens[i+1]-1, row t attends to rows <= t of its own prompt.
 * q head h reads kv head h / (num_q_heads / num_kv_heads).  Runs on tcgen05 tensor cores (TMA-staged
 * 128 x 128 tiles, accumulators in tensor memory).  No workspace.
 * ---------------------------------------------------------------------- */
typedef struct {
  void* out;                 /* [total_tokens, num_q_heads, 128] */
  const void* q;             /* [total_tokens, num_q_heads, 128] */
  const void* k;             /* [total_tokens, num_kv_heads, 128] */
  const void* v;
  int64_t out_seq_stride, out_head_stride;   /* elements; multiples of 8, innermost dimension contiguous */
  int64_t q_seq_stride, q_head_stride;
  int64_t k_seq_stride, k_head_stride;
  int64_t v_seq_stride, v_head_stride;
  const int32_t* cu_seqlens; /* device, [num_seqs + 1], cu_seqlens[0] = 0, non-decreasing */
  float scale;               /* > 0 */
  int32_t num_seqs;
  int32_t total_tokens;      /* rows of q / k / v / out; normally cu_seqlens[num_seqs].  Rows of v between a prompt's end
                                and total_tokens share 64-row steps with real rows and must hold finite values
                                (they are weighted by 0, and 0 * NaN would poison the step) */
  int32_t max_prompt_len;    /* host-known upper bound of every prompt length (sizes the grid) */
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t dtype;
  int32_t block_size;        /* of the pool below; ignored when key_cache is NULL */
  /* Optional: the prompt-phase cache write in the same launch.  When key_cache is not NULL every K/V row is also
   * written to its slot, exactly as mux_reshape_and_cache(k, v, ..., slot_mapping) would (negative slot = skip the
   * row, slot outside the pool = MUX_DEV_BAD_SLOT and skipped): the CTA that holds a K/V step of its own query
   * rows in shared memory copies it to the pool while the attention of the last steps runs. */
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;   /* device, [total_tokens, num_kv_heads] by the two strides (elements), or NULL */
  int64_t slot_token_stride, slot_head_stride;
  int64_t num_blocks;
  /* Instead of slot_mapping (used when slot_mapping is NULL): this layer's block lists, as the decode ops take
   * them.  Token t of prompt i, kv head h goes to slot block_tables[i][h][t / block_size] * block_size +
   * t % block_size — the slots getPromptSlots (csrc/batch_scheduler.h:42-56) would have listed, without the
   * [tokens, layers, heads] int64 array.  A negative block id skips the tokens of that block. */
  const int32_t* block_tables;   /* device, [num_seqs, num_kv_heads, max_blocks] by the two strides (elements) */
  int64_t bt_seq_stride, bt_head_stride;
  int32_t max_blocks_per_seq;
  int32_t num_units;             /* 0, or the number of (prompt, q head, query tile) triples in `units` */
  /* Optional work list for a host that knows the prompt lengths (the reference's does: input_metadata.prompt_lens is
   * a host list): units[2u] = prompt, units[2u + 1] = q head | query tile << 16, one entry per 128-row query tile
   * of every (prompt, q head), longest prompts first and the tiles of one (prompt, head) together, last tile first.
   * Without it the grid is (tiles of the longest prompt) x heads x prompts and the CTAs of shorter prompts' missing
   * tiles leave at once.  Negative prompt = padding. */
  const int32_t* units;          /* device, [num_units][2] */
} mux_prefill_args_t;

int mux_prefill_attention(const mux_prefill_args_t* args, void* cuda_stream);

/* ------------------------------------------------------------------------
 * Persistent block tables on the device.  The reference rebuilds and uploads the whole
 * [L, S, H, max_blocks] table every step (csrc/batch_scheduler.cpp:156-169,
 * muxserve/flexserver/llm_runtime.py:322-327); a decode step changes it only where a sequence
 * crosses a block boundary.  This call scatters n newly granted blocks into a table that stays on
 * the device:  tables[l][upd_row[i]][h][upd_block[i]] = upd_ids[i][l][h]  for all l, h.
 * upd_ids rows have the [layer][head] order in which the allocator grants a logical block
 * (csrc/batch_scheduler.h:19-20).  All pointers are device memory.
 * ---------------------------------------------------------------------- */
int mux_block_table_append(int32_t* tables, int64_t layer_stride, int64_t row_stride, int64_t head_stride,
                           int32_t num_layers, int32_t num_rows, int32_t num_kv_heads, int32_t max_blocks,
                           const int32_t* upd_row, const int32_t* upd_block, const int32_t* upd_ids,
                           int32_t num_updates, void* cuda_stream);

/* ------------------------------------------------------------------------
 * Tensor-parallel output all-reduce over NVLink peer memory.
 *
 * Replaces the NCCL all-reduce (sum over the TP group) of the row-parallel o_proj output,
 * muxserve/flexserver/models/llama.py:131-137,162 (the fork's ParallelLinear.row), for the 16-bit
 * [tokens, hidden] messages of a decode step, which are latency-bound: one kernel per rank, plain peer
 * stores / loads and epoch flags, every wait bounded (MUX_DEV_WAIT_TIMEOUT when one runs out).
 * Every rank ends up with the same bits (fp32 sums in rank order).
 *
 * Set-up (host), with the rank's own GPU current throughout: each rank creates one exchange buffer of
 * mux_tp_allreduce_buffer_size() bytes (mux_tp_buffer_create: its own zeroed allocation), exports it
 * (mux_tp_buffer_export: a CUDA IPC handle, 64 bytes, to be carried to the other ranks by any host channel),
 * imports the other ranks' handles (mux_tp_buffer_import: maps the peer's memory for THIS device and enables
 * peer access to the peer's GPU) and synchronises with them once before the first call.  All ranks must make
 * the same sequence of calls (count, dtype, algo, num_ctas); calls of one communicator are ordered on
 * one stream per rank.  in == out is allowed.  Ranks of one process may pass plain device pointers.
 * ---------------------------------------------------------------------- */
#define MUX_TP_MAX_WORLD 8
#define MUX_TP_CTRL_BYTES 32768                /* flags and call counters at the start of every exchange buffer */
#define MUX_TP_AUTO 0
#define MUX_TP_ONE_SHOT 1                      /* each rank pushes its message to all, sums locally */
#define MUX_TP_TWO_SHOT 2                      /* reduce-scatter by peer loads + all-gather by peer stores */
#define MUX_TP_ONE_SHOT_MAX_PUSH_BYTES (4 << 20)  /* MUX_TP_AUTO: one-shot while (world - 1) * message stays within this */
typedef struct {
  int32_t world;                      /* 2 .. MUX_TP_MAX_WORLD */
  int32_t rank;
  void* buffers[MUX_TP_MAX_WORLD];    /* exchange buffer of every rank as mapped in THIS process; [rank] is local */
  int64_t buffer_bytes;               /* size of each */
} mux_tp_comm_t;

size_t mux_tp_allreduce_buffer_size(int32_t world, size_t max_message_bytes);
#define MUX_TP_IPC_HANDLE_BYTES 64
int mux_tp_buffer_create(size_t bytes, void** ptr);     /* on the current device, zeroed */
int mux_tp_buffer_destroy(void* ptr);                   /* what mux_tp_buffer_create returned */
int mux_tp_buffer_export(const void* ptr, unsigned char handle[MUX_TP_IPC_HANDLE_BYTES]);
int mux_tp_buffer_import(const unsigned char handle[MUX_TP_IPC_HANDLE_BYTES], void** ptr);
int mux_tp_buffer_release(void* ptr);                   /* what mux_tp_buffer_import returned */
/* out = sum over ranks of in; count elements (multiple of 8) of dtype.  Every launch has 32 CTAs; num_ctas says how
 * many of them move data (0 = heuristic), the others only exchange flags.
 * MUX_ERR_TOO_LARGE when the message does not fit the exchange buffers. */
int mux_tp_allreduce(const mux_tp_comm_t* comm, const void* in, void* out, int64_t count, int32_t dtype,
                     int32_t algo, int32_t num_ctas, void* cuda_stream);
/* ------------------------------------------------------------------------
 * o_proj GEMM fused with the all-reduce of its result: what the row-parallel output projection of the
 * reference's attention layer does in two steps (muxserve/flexserver/models/llama.py:131-137,162: the fork's
 * ParallelLinear.row, then the NCCL all-reduce over the TP group), in ONE kernel per rank:
 *   out[t, n] = sum over ranks r of round16( sum_k a_r[t, k] * w_r[n, k] )      (fp32 inside, rank order)
 * a_r = the rank's attention output [m, k] (k = local q heads * 128), w_r = the rank's slice [n, k] of the
 * o_proj weight (nn.Linear's [out_features, in_features] layout, sliced along in_features), out [m, n] on every
 * rank.  The GEMM runs on tcgen05 tensor cores (TMA-staged operands, accumulators in tensor memory); every
 * 128 x 64 output tile is exchanged as soon as it is finished: pushed to the tile's owner rank, summed there,
 * pushed back to all (plain peer stores, bounded waits).  m <= 128; n a multiple of 64, <= MUX_TP_OPROJ_MAX_COLS;
 * k a multiple of 64; strides in elements, multiples of 8.  comm == NULL (or world 1): the GEMM alone.
 * A communicator used for this call must be used ONLY for it, always with the same n, by all ranks in the same
 * order (its exchange buffer: mux_tp_allreduce_buffer_size(world, m_max * n * 2)).
 * ---------------------------------------------------------------------- */
#define MUX_TP_OPROJ_MAX_COLS 16384
/* The caller states that `w` is not written by the kernels directly ahead in the stream (model weights never are):
 * the launch is made programmatically dependent and starts streaming the first weight tiles while those kernels
 * drain; `a`, the exchange buffers and `out` are touched only after they have completed. */
#define MUX_OPROJ_EARLY_W 1
typedef struct {
  const void* a;
  int64_t a_row_stride;
  const void* w;
  int64_t w_row_stride;
  void* out;
  int64_t out_row_stride;
  int32_t m, n, k;
  int32_t dtype;
  int32_t algo;        /* MUX_TP_AUTO, or force MUX_TP_ONE_SHOT (every rank sums every tile) / MUX_TP_TWO_SHOT (tile owners) */
  int32_t flags;       /* 0 or MUX_OPROJ_EARLY_W */
} mux_oproj_args_t;
int mux_tp_oproj_allreduce(const mux_tp_comm_t* comm, const mux_oproj_args_t* args, void* cuda_stream);
/* All ranks of a world as one cooperative launch on ONE GPU (tests of the protocol): args[r] are rank r's
 * operands, maps_scratch is 2 * world * 128 bytes of device memory (64-byte aligned) for the ranks' copy descriptors. */
int mux_tp_oproj_allreduce_emulated(int32_t world, void* const* buffers, int64_t buffer_bytes,
                                    const mux_oproj_args_t* args, void* maps_scratch, void* cuda_stream);

/* The same device code for a whole world on ONE GPU: rank r uses buffers[r], ins[r], outs[r]; all ranks'
 * CTAs form one cooperative launch (they wait on one another).  For tests of the protocol without
 * several GPUs; fails with MUX_ERR_CUDA when the grid cannot be resident at once. */
int mux_tp_allreduce_emulated(int32_t world, void* const* buffers, int64_t buffer_bytes, const void* const* ins,
                              void* const* outs, int64_t count, int32_t dtype, int32_t algo, int32_t num_ctas,
                              void* cuda_stream);

/* Self-test of the failure path: launches one warp that waits, with the same bounded wait the
 * kernels use, on a barrier nothing completes.  The wait gives up after a (shortened) poll limit, well under a second, sets MUX_DEV_WAIT_TIMEOUT and the kernel ends normally: the context stays usable. */
int mux_selftest_wait_timeout(void* cuda_stream);

/* Reads and clears the device status word (MUX_DEV_* bits) of the current
 * device.  Synchronises the given stream. Returns a negative mux_status_t on failure.
 * The word is copied and then cleared by two operations on `cuda_stream`: bits that kernels on OTHER
 * streams set between the two are lost, so read it from the stream the work ran on (or after a device sync). */
int mux_device_status(void* cuda_stream);

/* ------------------------------------------------------------------------
 * Host side: block allocator.  Same observable behaviour as KVStorage in the
 * reference (csrc/memory_manager.cpp:4-157): block ids, free-list order,
 * preemption index, return encodings and counters.
 * ---------------------------------------------------------------------- */
typedef struct mux_kv_storage mux_kv_storage_t;

mux_kv_storage_t* mux_kv_storage_create(int32_t num_blocks);        /* memory_manager.cpp:4-10 */
void mux_kv_storage_destroy(mux_kv_storage_t* s);
/* memory_manager.cpp:12-23.  Pops `size` ids from the tail of the free list. */
int mux_kv_storage_allocate(mux_kv_storage_t* s, int32_t size, int32_t* out_ids);
/* memory_manager.cpp:25-142.  alloc_info = rows [request id, logical blocks, has_blocks];
 * writes [preempt_idx, block ids...] to out and its length to *out_len.  Call with
 * out == NULL to learn the length that the same call would write WITHOUT changing state. */
int mux_kv_storage_allocate_batch(mux_kv_storage_t* s, const int32_t* alloc_info,
                                  int32_t num_requests, int32_t num_layers, int32_t num_heads,
                                  int32_t* out, int64_t out_capacity, int64_t* out_len);
/* memory_manager.cpp:144-157.  Returns the number of freed blocks (>= 0). */
int64_t mux_kv_storage_free_batch(mux_kv_storage_t* s, const int32_t* request_ids, int32_t n);
int32_t mux_kv_storage_new_blocks_allocated(const mux_kv_storage_t* s);  /* memory_manager.h:18 */
int32_t mux_kv_storage_num_blocks_allocated(const mux_kv_storage_t* s);
int64_t mux_kv_storage_num_free(const mux_kv_storage_t* s);
/* Copies the free list (allocation order: the tail is handed out first). */
int mux_kv_storage_free_list(const mux_kv_storage_t* s, int32_t* out, int64_t capacity);
/* Invariant check: every id in [0,num_blocks) is in exactly one of free list / one owner. */
int mux_kv_storage_check(const mux_kv_storage_t* s);

/* ------------------------------------------------------------------------
 * Host side: per-model step builder.  Same observable behaviour as
 * BatchScheduler / Request in the reference (csrc/batch_scheduler.h:9-106,
 * csrc/batch_scheduler.cpp:5-199), except that block-table padding, which the
 * reference leaves uninitialised, is written as 0.
 * ---------------------------------------------------------------------- */
typedef struct mux_batch_scheduler mux_batch_scheduler_t;

mux_batch_scheduler_t* mux_batch_scheduler_create(int32_t num_layers, int32_t num_heads,
                                                  int32_t max_seq_len, int32_t block_size);
void mux_batch_scheduler_destroy(mux_batch_scheduler_t* b);
/* batch_scheduler.cpp:12-20 */
int mux_batch_scheduler_add_request(mux_batch_scheduler_t* b, const int32_t* prompt,
                                    int32_t prompt_len, int32_t req_id, int32_t max_tokens);
/* batch_scheduler.cpp:22-48.  out has 3*n+1 entries. last_tokens may be NULL (prefill). */
int mux_batch_scheduler_try_batch(mux_batch_scheduler_t* b, const int32_t* req_ids, int32_t n,
                                  const int32_t* last_tokens, int32_t n_last, int32_t* out);
/* batch_scheduler.cpp:51-97.  out receives [numTokens, numContexts, maxContextLen,
 * maxBlocksPerSeq, L, H, prompt lens...]; *out_len its length. */
int mux_batch_scheduler_get_batch_info(mux_batch_scheduler_t* b, const int32_t* block_request,
                                       int32_t n, const int32_t* block_info, int64_t block_info_len,
                                       int32_t* out, int32_t out_capacity, int32_t* out_len);
/* batch_scheduler.cpp:99-193.  Buffers are host memory sized by the caller from
 * get_batch_info, as muxserve/flexserver/llm_runtime.py:300-312 does:
 *   tokens, positions [padded_len] int32;  context_lens [numContexts] int32;
 *   block_tables [numTokens, maxBlocksPerSeq, L, H] int32;  slot_mapping [numTokens, L, H] int64. */
int mux_batch_scheduler_get_batch(mux_batch_scheduler_t* b, const int32_t* block_request, int32_t n,
                                  const int32_t* block_info, int64_t block_info_len,
                                  int32_t* tokens, int32_t* positions, int32_t padded_len,
                                  int32_t* context_lens, int32_t num_contexts,
                                  int32_t* block_tables, int64_t block_tables_len,
                                  int64_t* slot_mapping, int64_t slot_mapping_len);
/* Same step as get_batch for a decode batch, but block tables are written in the
 * layout the kernels consume, [L, numContexts, H, maxBlocksPerSeq], which the reference
 * reaches by a device permute (llm_runtime.py:327). */
int mux_batch_scheduler_get_batch_decode_layered(
    mux_batch_scheduler_t* b, const int32_t* block_request, int32_t n,
    const int32_t* block_info, int64_t block_info_len,
    int32_t* tokens, int32_t* positions, int32_t padded_len,
    int32_t* context_lens, int32_t num_contexts,
    int32_t* block_tables, int64_t block_tables_len,
    int64_t* slot_mapping, int64_t slot_mapping_len);
/* The flattened descriptors of ONE fused attention launch per layer index over the decode batches of several
 * colocated models (mux_paged_attention_mixed / mux_decode_attention_mixed), straight from their step builders.
 * No counterpart in the reference, which runs every model in its own processes (muxserve/muxsched/scheduler.py:167-208);
 * the tables are the ones csrc/batch_scheduler.cpp:156-169 would emit per model.  Call after every model's
 * get_batch_info of the step.  Models are laid out deepest first (spans[] tells where), so the models that still
 * have layer l are a prefix of the items and of the packed q / out rows.  With tp > 1 the schedulers hold the LOCAL
 * heads of rank tp_rank and every model's rows are its full [sequences, tp * local q heads]: this rank's heads at
 * their global position (the TP all-reduce of the ranks' out matrices is then the models' whole output). */
typedef struct {
  const mux_batch_scheduler_t* scheduler;
  const int32_t* request_ids;   /* the model's decode batch, in batch order */
  int32_t num_requests;
  int32_t num_q_heads;          /* local; a multiple (<= 8x) of the scheduler's head count */
  float scale;
} mux_mixed_model_t;
typedef struct {
  int32_t model;                /* index into the caller's models[] */
  int32_t first_item, num_items, first_row, num_rows, num_layers;
} mux_mixed_span_t;
/* totals[5] receives {items, rows, layers of the deepest model, largest group, max context length}.
 * block_tables == NULL: sizing call (totals[0..3] and spans only).  Otherwise block_tables is
 * [layers][items][max_blocks] int32 (unused entries 0) and the four item arrays have `items` entries. */
int mux_batch_scheduler_get_batch_mixed(const mux_mixed_model_t* models, int32_t num_models, int32_t tp,
                                        int32_t tp_rank, int32_t max_blocks, int32_t* item_context_len,
                                        int32_t* item_q_row, int32_t* item_group, float* item_scale,
                                        int32_t* block_tables, int64_t block_tables_len, mux_mixed_span_t* spans,
                                        int32_t* totals);
int mux_batch_scheduler_release_requests(mux_batch_scheduler_t* b, const int32_t* req_ids, int32_t n);
/* batch_scheduler.h:88-92.  Each copies up to capacity entries and returns the full length. */
int32_t mux_batch_scheduler_preempt_requests(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity);
int32_t mux_batch_scheduler_prompt_info(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity);
/* pairs [request id, max tokens] */
int32_t mux_batch_scheduler_batch_reqs(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity);
/* Introspection for tests: [contextLen, numPhysicalBlocks, logicalBlockIdx, logicalBlockOffset, numOutputs]. */
int mux_batch_scheduler_request_state(const mux_batch_scheduler_t* b, int32_t req_id, int32_t out[5]);

#ifdef __cplusplus
}
#endif
#endif /* MUXB200_H_ */
