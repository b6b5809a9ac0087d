/* peerkv.h -- C ABI of the B200 peer-parallel split-K decode-attention library.
 *
 * Plain pointers, sizes and an opaque stream handle; no torch or C++ types.
 * Every entry point returns 0 on success and a negative PKV_E* code otherwise;
 * pkv_last_error() gives the message of the calling thread's last failure.
 * Device-side trouble (a wait that ran out, a block-table id outside the pool)
 * never traps: it is recorded in a status word that pkv_shard_status() /
 * pkv_exchange_status() read back.
 *
 * The library replaces, in the PeerKV project:
 *   - the pybind module of csrc/peer_fused_attn_ext.cu:139-145 and its host
 *     orchestration (:37-137), JIT-loaded by umallm/peerkv/fused_attn.py:32-46;
 *   - the kernels of csrc/peer_attn_kernels.cuh (attn_split_gqa :14-47,
 *     attn_combine :50-61, merge2_h :64-73);
 *   - the per-sequence gather loop of umallm/peerkv/paged.py:48-97 (the kernels
 *     read the paged pool through the block table directly).
 * All pointers are device pointers on the device of the object they are passed
 * to unless a comment says otherwise.  The caller owns q, the KV pool, block
 * tables and outputs; the library owns only the scratch inside its objects.
 */
#ifndef PEERKV_H_
#define PEERKV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKV_ABI_VERSION 1

/* return codes */
#define PKV_OK            0
#define PKV_E_INVALID    -1   /* bad argument (message says which) */
#define PKV_E_CUDA       -2   /* a CUDA runtime / driver call failed */
#define PKV_E_UNSUPPORTED -3  /* shape outside what the kernels cover */
#define PKV_E_STATE      -4   /* object not ready (e.g. peer not attached) */

/* element types */
#define PKV_F16      0
#define PKV_BF16     1
#define PKV_INT8     2   /* codes; one fp16 scale per (token, kv-head) row */
#define PKV_FP8_E4M3 3   /* e4m3fn codes; same scales */
#define PKV_F32      4

/* device status bits (OR-ed; 0 = healthy) */
#define PKV_ST_PIPE_TIMEOUT   0x1u  /* an on-chip copy barrier was not completed in time */
#define PKV_ST_BAD_PAGE       0x2u  /* block-table entry outside [0, n_pages) was skipped */
#define PKV_ST_Q_TIMEOUT      0x4u  /* the query for this epoch never arrived */
#define PKV_ST_PARTIAL_TIMEOUT 0x8u /* a peer's partial for this epoch never arrived */

typedef struct pkv_shard pkv_shard;       /* one GPU's attention context */
typedef struct pkv_exchange pkv_exchange; /* one GPU's mailboxes for q and partials */

/* A KV pool as the kernels see it.  Address of element (page, tok, head, d) is
 *   base + page*page_stride + tok*token_stride + head*head_stride + d   (elements).
 * vLLM's [2, nb, bs, Hkv, D] cache is k = cache[0], v = cache[1], page_stride =
 * bs*Hkv*D, token_stride = Hkv*D, head_stride = D.  The reference op's
 * contiguous [Hkv, T, D] shard (csrc/peer_fused_attn_ext.cu:8-16) is one page of
 * T tokens: page_size = T, token_stride = D, head_stride = T*D.
 * Strides must be multiples of 8 elements (16 bytes for 1-byte codes), bases
 * 16-byte aligned, head_dim 128.  k_scale / v_scale ([page][tok][head] fp16,
 * dense) are NULL unless dtype is PKV_INT8 or PKV_FP8_E4M3; quantised pools also need
 * page_size to be a multiple of 16 and n_kv_heads <= 8 or a multiple of 8.  At most 8
 * query heads per kv head. */
typedef struct pkv_kv_view {
  const void* k;
  const void* v;
  const void* k_scale;
  const void* v_scale;
  int32_t dtype;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t page_size;
  int64_t n_pages;
  int64_t page_stride;
  int64_t token_stride;
  int64_t head_stride;
} pkv_kv_view;

/* One decode step over ONE shard: a single query token per sequence.
 *   q            [batch, n_q_heads, head_dim], q_dtype PKV_F16 or PKV_BF16
 *   block_table  [batch, block_table_stride] int32 page ids of THIS pool, in
 *                sequence order; NULL means page j of sequence b is b*block_table_stride + j
 *   seq_lens     [batch] int32 tokens of each sequence that live in THIS shard
 *                (0 allowed; only a sequence's last listed page may be partial)
 *   scale        softmax scale (the reference default is 1/sqrt(head_dim)) */
typedef struct pkv_decode_args {
  const void* q;
  int32_t q_dtype;
  int32_t batch;
  int32_t n_q_heads;
  int32_t reserved0;
  pkv_kv_view kv;
  const int32_t* block_table;
  int64_t block_table_stride;
  const int32_t* seq_lens;
  float scale;
  int32_t reserved1;
} pkv_decode_args;

const char* pkv_last_error(void);
int pkv_abi_version(void);

/* ---- one GPU ------------------------------------------------------------ */

/* Allocates the split-K scratch of one GPU once (no allocation per call; the
 * reference allocates 6-14 tensors per call, csrc/peer_fused_attn_ext.cu:56-92).
 * A shard is used from one host thread, and its launches must not overlap on the GPU
 * (one stream, or ordered streams): they share the scratch, and each launch records
 * per-SM timings that the next one uses to split the work. */
int pkv_shard_create(pkv_shard** out, int device, int max_batch, int n_q_heads);
int pkv_shard_destroy(pkv_shard* s);
/* Reads (and clears) the device status word; synchronises `stream` first. */
int pkv_shard_status(pkv_shard* s, void* stream, uint32_t* status_out);

/* Cumulative counters of the shard since its creation; synchronises `stream` first.
 * launches = decode kernels run; units = (16-token tile, kv-head) pairs those kernels
 * read, so KV bytes read = units * 16 * 128 * 2 * element size.  Feeds the per-call
 * counters the reference plans (umallm/observability/metrics.py:31-46). */
int pkv_shard_stats(pkv_shard* s, void* stream, uint64_t* launches_out, uint64_t* units_out);

/* Shard partial in the reference's (O, lse) convention
 * (umallm/peer_parallel_attn.py:46-71): o_part [batch, n_q_heads, 128] fp32,
 * normalised; lse_part [batch, n_q_heads] fp32, natural log; an empty shard
 * gives O = 0 and lse = -inf.  o_part / lse_part may point into a peer GPU's
 * memory (P2P mapped): that is how a peer hands its partial to the home GPU. */
int pkv_decode_partial(pkv_shard* s, const pkv_decode_args* a, float* o_part,
                       float* lse_part, void* stream);

/* Whole attention on one GPU: out [batch, n_q_heads, 128] in out_dtype
 * (PKV_F16 / PKV_BF16 / PKV_F32); lse_out may be NULL.  Replaces the Tp == 0
 * path of peer_fused_attn (csrc/peer_fused_attn_ext.cu:66-74). */
int pkv_decode(pkv_shard* s, const pkv_decode_args* a, void* out, int32_t out_dtype,
               float* lse_out, void* stream);

/* pkv_decode for callers that must not allocate device memory.  No counterpart in the
 * reference (its op allocates fresh scratch tensors on every call).
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they need
 * attention: a plugin running inside another runtime's memory pool whose budget is
 * already fully handed out, a serving process that pre-sizes all GPU memory at start-up
 * and treats any later allocation as a fault, or code on a path where the allocator's
 * implicit device synchronisation is not acceptable.  For them the split-K scratch
 * lives in arrays that are part of the library image itself: about 16 MB per GPU, held
 * by every GPU that loads the library until the process ends.
 *
 * Same arguments and result as pkv_decode, minus the shard object.  Limits, checked
 * with a clear error: at most 32 sequences and 64 query heads per call (and a GPU of
 * at most 192 SMs).  The call makes no cudaMalloc / cudaFree and uses no allocating
 * library routine; the caller still owns q, the KV pool, tables and outputs.
 *
 * The first call on a device does the one-time set-up for that device (looks up the
 * arrays' device addresses, raises the kernel's shared-memory limit), so make it
 * before starting any stream capture.  All calls on a device share the one scratch:
 * each call first clears the words that must start at zero, and two calls whose
 * kernels overlap on the GPU (different streams, no ordering between them) race on
 * it -- order them, or use pkv_decode with separate shards. */
int pkv_decode_static(int device, const pkv_decode_args* a, void* out, int32_t out_dtype,
                      float* lse_out, void* stream);
/* Reads (and clears) the status word of pkv_decode_static's scratch on `device`;
 * synchronises `stream` first.  The bits of all static calls since the last read
 * accumulate.  Allocates nothing.  No counterpart in the reference. */
int pkv_static_status(int device, void* stream, uint32_t* status_out);

/* Measurement aid: launches ONLY the split-K kernel of pkv_decode (per-CTA partials
 * stay in the shard's scratch, no combine), so its duration can be timed alone with
 * events on `stream`.  No counterpart in the reference. */
int pkv_decode_splits_only(pkv_shard* s, const pkv_decode_args* a, void* stream);
/* Measurement aid: every later launch on the shard records %globaltimer stamps per CTA
 * into buf (device memory of the shard's GPU, 8 x 64-bit words per CTA, room for 1024
 * CTAs, zeroed by the caller before each launch); NULL switches it off.  Words: 0 CTA
 * start, 1 query published (home) / first query rows seen (peer), 2 last tile consumed,
 * 3 last local combine done, 4 last peer row complete (home), 5 last output row written.
 * No counterpart in the reference. */
int pkv_shard_trace(pkv_shard* s, uint64_t* buf);

/* Single-pass N-way LSE merge (replaces merge2_h, csrc/peer_attn_kernels.cuh:64-73,
 * and the fold of umallm/peer_parallel_attn.py:169-172).  Part i is at
 * o_parts + i*o_part_stride (floats), lse_parts + i*lse_part_stride; rows =
 * batch*n_q_heads.  lse_out may be NULL. */
int pkv_merge_partials(int device, const float* o_parts, int64_t o_part_stride,
                       const float* lse_parts, int64_t lse_part_stride, int32_t n_parts,
                       int32_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                       float* lse_out, void* stream);

/* Per-(token, kv-head) absmax quantiser; rows = tokens*kv_heads rows of 128
 * values in src_dtype (PKV_F16 / PKV_BF16), codes [rows, 128] 1 byte each,
 * scales [rows] fp16.  fmt PKV_INT8 or PKV_FP8_E4M3.  No counterpart in the
 * reference (its umallm/compression.py is a 4-bit group quantiser). */
int pkv_quantize_kv(int device, const void* src, int32_t src_dtype, int64_t rows,
                    void* codes, void* scales, int32_t fmt, void* stream);

/* Splits a global block table into one local table per GPU, on the device, with no
 * host round trip (replaces the .item() loop of umallm/peerkv/paged.py:52-61).
 *   mode 0: ids in [bases[d], bases[d+1]) live on GPU d at local id gid - bases[d]
 *           (the reference's peer_base rule is n_dev = 2, bases = {0, peer_base});
 *   mode 1: id gid lives on GPU gid mod n_dev at local id gid div n_dev (bases unused).
 * block_table [batch, block_table_stride] int32 and seq_lens [batch] int32 are on
 * `device`; out_tables[d] ([batch, out_stride] int32) and out_lens[d] ([batch] int32)
 * are host arrays of n_dev device pointers that may point into other GPUs' memory
 * (P2P mapped).  Sequence order is kept, so only a GPU's last listed page of a
 * sequence can be partial. */
int pkv_split_block_table(int device, const int32_t* block_table, int64_t block_table_stride,
                          const int32_t* seq_lens, int32_t batch, int32_t page_size,
                          int32_t n_dev, int32_t mode, const int64_t* bases,
                          int32_t* const* out_tables, int64_t out_stride,
                          int32_t* const* out_lens, void* stream);

/* Appends new tokens' K and V (key / value [n_tokens, n_kv_heads, 128], 16-bit, rows
 * kv_token_stride elements apart) to a KV cache whose blocks are spread over n_dev GPUs:
 * slot_mapping[t] = block id * block_size + offset (negative = padding, skipped); block id
 * g belongs to the GPU d with the largest bases[d] <= g, at local block g - bases[d] (the
 * reference's peer_base rule, umallm/peerkv/paged.py:52-61, for N GPUs).  Runs on `device`,
 * which holds key, value and slot_mapping; k_pools[d] / v_pools[d] (host arrays of n_dev
 * device pointers, element strides per pool) may point into other GPUs' memory (P2P
 * mapped), so the append needs no second stream.  A slot outside every pool is skipped
 * and sets PKV_ST_BAD_PAGE in *status_word (a device word of `device`, may be NULL).
 * This is the write side that the reference lists as missing for its sharded path
 * (umallm/peerkv/register.py:21-27); it replaces vLLM's reshape_and_cache for such a
 * cache. */
/* Attention partial for MANY query rows over one contiguous KV shard (sharded prefill):
 * q (batch, n_q_heads, sq, 128), k / v (batch, n_kv_heads, sk, 128), 16-bit, element
 * strides given (multiples of 8, unit last stride).  With causal != 0 query row i sees key
 * j iff k_pos0 + j <= q_pos0 + i (the diagonal of a ring: q_pos0 == k_pos0); otherwise
 * every key.  o_part [batch, n_q_heads, sq, 128] fp32 normalised, lse_part [batch,
 * n_q_heads, sq] natural log, -inf and O = 0 for a row that sees no key: the convention of
 * pkv_decode_partial, so pkv_merge_partials merges shards.  The shard is read once per
 * 64 query rows and head.  Replaces the aten flash-attention calls of
 * umallm/peer_parallel_attn.py:60-66 (flash_partial) and :95-101 (_causal_partial). */
int pkv_prefill_partial(int device, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                        int64_t q_stride_s, const void* k, const void* v, int64_t kv_stride_b,
                        int64_t kv_stride_h, int64_t kv_stride_s, int32_t batch,
                        int32_t n_q_heads, int32_t n_kv_heads, int32_t sq, int32_t sk,
                        int32_t head_dim, int32_t dtype, float scale, int32_t causal,
                        int64_t q_pos0, int64_t k_pos0, float* o_part, float* lse_part,
                        void* stream);

/* Copy-back staging, the fallback when the peers hold KV but may not lend compute
 * (umallm/vllm_integration/peerkv_staging.py:82-131; chosen under R1-busy,
 * umallm/elastic_policy.py:346-350).  The home tensor has c_local real blocks followed by
 * c_scratch scratch blocks.  Every entry of block_table [batch, stride] (global ids, on
 * `device`) that names a peer block (id >= c_local = bases[1]; GPU d owns ids from
 * bases[d], n_blocks[d] of them, pools k_pools[d] / v_pools[d] with block stride
 * page_strides[d] elements, P2P mapped; index 0 unused) is copied into the next free
 * scratch block -- block_elems elements of elem_size bytes for K and again for V -- and
 * out_table gets the entry rewritten to that scratch block; local entries are copied
 * through.  A single-GPU pkv_decode over the home tensor with out_table then gives the
 * exact result.  scratch_words: `batch` int32 of device scratch.  More peer entries than
 * scratch blocks, or an id outside every pool, sets PKV_ST_BAD_PAGE in *status_word (a
 * device word) and leaves that entry pointing at the first scratch block.  No host
 * synchronisation; the reference's version finds the unique ids on the host. */
int pkv_stage_peer_blocks(int device, const int32_t* block_table, int64_t block_table_stride,
                          const int32_t* seq_lens, int32_t batch, int32_t block_size,
                          int32_t n_dev, const int64_t* bases, const int64_t* n_blocks,
                          const void* const* k_pools, const void* const* v_pools,
                          const int64_t* page_strides, void* k_home, void* v_home,
                          int64_t home_page_stride, int64_t c_local, int64_t c_scratch,
                          int64_t block_elems, int32_t elem_size, int32_t* out_table,
                          int32_t* scratch_words, uint32_t* status_word, void* stream);

/* Lets kernels running on `device` load from and store to `peer_device`'s memory (a
 * no-op when already enabled or when both are the same GPU).  pkv_exchange_attach does
 * this for its two devices; callers that hand P2P pool pointers to pkv_kv_append or
 * pkv_split_block_table without an exchange call it themselves. */
int pkv_enable_peer_access(int device, int peer_device);
int pkv_kv_append(int device, const void* key, const void* value, int64_t kv_token_stride,
                  const int64_t* slot_mapping, int32_t n_tokens, int32_t n_kv_heads,
                  int32_t head_dim, int32_t block_size, int32_t n_dev, const int64_t* bases,
                  const int64_t* n_blocks, void* const* k_pools, void* const* v_pools,
                  const int64_t* page_strides, const int64_t* token_strides,
                  const int64_t* head_strides, uint32_t* status_word, void* stream);

/* ---- several GPUs ------------------------------------------------------- */

/* Mailboxes of one GPU, allocated once: a q inbox of 8-byte {payload, epoch} words, and
 * `world` partial slots ([max_batch, n_q_heads, 128] O + [max_batch, n_q_heads] lse
 * each, as 8-byte {fp32, epoch} words).  rank 0..world-1; the home rank
 * is the one that owns q and runs the merge.  Replaces the per-call stream/event/scratch
 * set-up of csrc/peer_fused_attn_ext.cu:81-97 and its cudaMemcpyAsync hops
 * (:100-101,120-123).
 *
 * Protocol.  Epochs count steps and only grow.  The home GPU stores the query rows into
 * each peer's inbox as 8-byte words, 4 bytes of q and the low 32 bits of the epoch: an
 * aligned 8-byte store arrives whole, so a word that shows this step's epoch holds this
 * step's q, and neither a fence nor a flag follows.  A peer re-reads (bounded) the words
 * it needs until they show the epoch, and writes anything into the home GPU's slot only
 * after it has seen the first word of that sequence.
 * A peer stores the (O, lse) rows of a (sequence, kv-head) into its slot on the home GPU
 * in the same word format; the home GPU polls the lse words of a pair, checks every O
 * word of it, and merges the pair as soon as all of them show the epoch.  The low 32
 * bits of the epoch repeat after 2^32 steps; a word can only be taken for a newer one
 * if it was written exactly a multiple of 2^32 steps earlier and never since.
 * The home GPU publishes epoch e+1 only after its
 * merge of epoch e has ended, so neither the inbox nor a slot is rewritten while it can
 * still be read, also when steps are enqueued back to back without a host
 * synchronisation.  Every step entry point validates, launches, and only then advances
 * the epoch: a call that returns an error leaves the epoch unchanged.  All ranks must
 * issue the same number of steps; after an error, or a step that one rank did not
 * issue, bring the ranks back together with pkv_exchange_resync. */
int pkv_exchange_create(pkv_exchange** out, int device, int rank, int world,
                        int max_batch, int n_q_heads);
int pkv_exchange_destroy(pkv_exchange* x);
/* 64-byte inter-process handle of this GPU's mailbox slab (other process opens it). */
int pkv_exchange_export(pkv_exchange* x, void* handle64);
/* Map peer `peer_rank`'s slab from its exported handle (one process per GPU). */
int pkv_exchange_import(pkv_exchange* x, int peer_rank, const void* handle64);
/* Same process, several devices: map `peer`'s slab directly (enables peer access). */
int pkv_exchange_attach(pkv_exchange* x, int peer_rank, pkv_exchange* peer);
int pkv_exchange_status(pkv_exchange* x, void* stream, uint32_t* status_out);
/* Current epoch (number of steps begun). */
int pkv_exchange_epoch(pkv_exchange* x, uint64_t* epoch_out);
/* Sets the epoch (>= the current one): every rank passes the same value, e.g. the
 * largest epoch any rank has reached, after a failed or skipped step. */
int pkv_exchange_resync(pkv_exchange* x, uint64_t epoch);

/* CUDA-graph capture of a sequence of steps (a whole decode step of L layers as one
 * graph per GPU, csrc/peer_rt_bench.cu:134-154 and csrc/peer_fused_decoder.cu:433-455 in
 * the reference).  The kernels take their epoch as `*base + relative`, base being a
 * device word of the exchange, so a captured launch stays valid on replay:
 *   pkv_exchange_capture_begin(x);  cudaStreamBeginCapture(stream, ...);
 *   ... pkv_home_step / pkv_peer_step calls on `stream` ...
 *   pkv_exchange_capture_end(x, stream, &steps);   -- adds the node that advances base
 *   cudaStreamEndCapture(stream, &graph);
 * and after every cudaGraphLaunch of it call pkv_exchange_replayed(x) so that the host's
 * epoch follows.  Every rank captures the same steps and replays the same number of
 * times.  No allocation happens in any of these calls. */
int pkv_exchange_capture_begin(pkv_exchange* x);
int pkv_exchange_capture_end(pkv_exchange* x, void* stream, uint64_t* steps_out);
int pkv_exchange_replayed(pkv_exchange* x);

/* Measurement aid: what a hop over the fabric costs, with the primitives the decode kernels
 * use.  Rank A calls it with role 0 and rank B with role 1 (peer_rank = the other one), at
 * about the same time, after both called pkv_exchange_hop_probe_reset and synchronised.
 * The two single-warp kernels bounce a flag `iters` times; with payload_bytes > 0 (a
 * multiple of 512) every bounce first stores that many bytes into the other GPU's q inbox
 * and passes a system fence, as a partial return does.  Roles 2 and 3 are 0 and 1 with the
 * bounce done the way the query publish does it: the payload as {payload, marker} words,
 * no fence, no flag, the receiver polling the last 512 bytes.  out (2 x uint64 of device memory on
 * this rank's GPU): elapsed ns of this side; 1 if a wait ran out (bounded, 2 s).  One-way
 * latency = out[0] of role 0 / (2 * iters).  Not to be mixed with steps in flight (the
 * inbox is overwritten).  No counterpart in the reference. */
int pkv_exchange_hop_probe(pkv_exchange* x, int32_t peer_rank, int32_t role, int32_t iters,
                           int32_t payload_bytes, uint64_t* out, void* stream);
int pkv_exchange_hop_probe_reset(pkv_exchange* x, void* stream);

/* Home rank, start of a step in the three-call form (publish, partial, merge): advances
 * the epoch, stores q ([batch, n_q_heads, 128], 16-bit) into every attached peer's q
 * inbox with P2P stores ({payload, epoch} words).  Replaces the q broadcast +
 * event fork of peer_fused_attn_ext.cu:100-102,114.  pkv_home_step does all three in
 * one launch and is the form to use. */
int pkv_home_publish_q(pkv_exchange* x, const void* q, int32_t batch, void* stream);
/* Peer rank, one step: advances the epoch, waits (bounded, device side, per sequence)
 * for the q of this epoch, computes the shard partial and stores it into the home
 * rank's slot for this rank as {fp32, epoch} words.  a->q is ignored unless q_override != 0; with q_override the kernel reads
 * a->q at once and waits for nothing, so the caller must order the step after the home
 * GPU's previous merge itself. */
int pkv_peer_step(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, int32_t home_rank,
                  int32_t q_override, void* stream);
/* Home rank, one whole step in ONE launch: the kernel first stores q into the peers'
 * inboxes, all warps sharing the rows, then streams the home shard; it combines its
 * splits and, pair by pair, waits (bounded, device side) for the rows of the ranks in
 * wait_mask and folds them in; a rank without its bit is left out of the merge.  out [batch, n_q_heads, 128] in out_dtype;
 * lse_out may be NULL.  An empty home pool (n_pages 0) is fine.  Same result as
 * pkv_home_publish_q + pkv_home_partial + pkv_home_merge; replaces the host
 * orchestration of csrc/peer_fused_attn_ext.cu:94-135. */
int pkv_home_step(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, uint32_t wait_mask,
                  void* out, int32_t out_dtype, float* lse_out, void* stream);
/* Home rank: its own shard's partial into its own slot (after pkv_home_publish_q). */
int pkv_home_partial(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, void* stream);
/* Home rank: waits (bounded, device side, per row) until the slots of the ranks in
 * `wait_mask` (bit r = rank r takes part; this rank's own slot always does) show this
 * step's epoch in every word, then merges them into out [batch, n_q_heads, 128] of
 * out_dtype.  A rank without its bit is left out.  Replaces the event join + merge2_h of
 * peer_fused_attn_ext.cu:128-131. */
int pkv_home_merge(pkv_exchange* x, int32_t batch, uint32_t wait_mask, void* out,
                   int32_t out_dtype, float* lse_out, void* stream);

/* ---- the rest of a decoder layer (the full-step configuration) ------------- */

/* The small kernels around the attention call of one decoder layer, for a decode batch
 * of `rows` tokens; the projections in between stay library GEMMs, as in the reference
 * (csrc/peer_fused_decoder.cu:100-109).  dtype PKV_F16 or PKV_BF16 throughout.
 *
 * pkv_add_rmsnorm: if delta != NULL, x += delta in place (the residual add); then
 *   out = x * rsqrt(mean(x^2) + eps) * weight.  x, delta, out [rows, hidden], weight
 *   [hidden]; hidden a multiple of 8.  Replaces add_kernel + rmsnorm_kernel
 *   (csrc/peer_fused_decoder.cu:51-71, 87-95).
 * pkv_rope_append: qkv [batch, (n_q_heads + 2 n_kv_heads) * head_dim] (q heads, k heads,
 *   v heads); rotate-half RoPE at angle positions[b] * inv_freq[i] on q and k; q goes to
 *   q_out [batch, n_q_heads, head_dim]; the rotated k and v are stored into the pools at
 *   page pages[b], token slot slots[b] (element strides as in pkv_kv_view); pools NULL =
 *   no append.  No counterpart in the reference (its layer has neither RoPE nor an
 *   append, :205-206).
 * pkv_swiglu: out[r, f] = silu(gate_up[r, f]) * gate_up[r, ffn + f]; ffn a multiple of 8.
 *   Replaces swiglu_kernel (:73-85). */
int pkv_add_rmsnorm(int device, void* x, const void* delta, const void* weight, void* out,
                    int32_t rows, int32_t hidden, float eps, int32_t dtype, void* stream);
int pkv_rope_append(int device, const void* qkv, const int64_t* positions, const float* inv_freq,
                    int32_t batch, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                    void* q_out, void* k_pool, void* v_pool, int64_t page_stride,
                    int64_t token_stride, int64_t head_stride, const int64_t* pages,
                    const int64_t* slots, int32_t dtype, void* stream);
int pkv_swiglu(int device, const void* gate_up, void* out, int32_t rows, int32_t ffn,
               int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PEERKV_H_ */
