// Paged, GQA-packed split-K flash-decode partial kernel for one KV shard (sm_100a).
//
// Replaces attn_split_gqa (PeerKV csrc/peer_attn_kernels.cuh:14-47) and the
// per-sequence gather of umallm/peerkv/paged.py:48-97: the kernel walks the block
// table itself and never copies KV.
//
// Work unit = a TILE of 16 tokens of one page, all (up to 8) kv-heads.  The tiles
// of all sequences form one flat list; the grid is persistent (one CTA per SM) and
// CTA c owns the contiguous range [c*per, (c+1)*per) of it, so load is balanced by
// tokens, not by sequences.  Where a range crosses a sequence boundary the CTA
// flushes one partial (unnormalised O, running max m, running sum l) to slot
// c + seq; a sequence is therefore covered by the consecutive slots of the CTAs
// that touched it, and the warp that finishes a (sequence, kv-head) last merges them in
// the kernel's tail (replaces attn_combine, csrc/peer_attn_kernels.cuh:50-61).
//
// Inside a CTA: warps 8 and 9 are the producers of a K ring and a V ring of 32 KiB
// slots; 16 lanes each issue one 2 KiB TMA box per tile (8 heads x 2 halves of the
// head dimension, [16 tok][64 d], 128-byte swizzle so ldmatrix is bank-conflict
// free), a head's boxes completing on that head's own mbarrier.  Warps 0..7 each own
// one kv-head and consume the tiles with tensor-core MMAs in the "swapped" form
//     S^T[16 tok x 8 qheads] = K[16 x 128] . Q^T[128 x 8]
//     O^T[128 d  x 8 qheads] += V^T[128 x 16] . P^T[16 x 8]
// so the G = Hq/Hkv query heads of a group ride in the N = 8 dimension and one
// K/V read serves the whole group.  Softmax statistics are per column (q head),
// reduced with three xor-shuffles; P is transposed into the B-fragment layout
// with movmatrix.  Decode is HBM-bound: the tensor cores are used because the
// CUDA-core form needs ~8 issue cycles per KV row, more than HBM leaves.
#pragma once
#include "ptx.cuh"

namespace pkv {

constexpr int kHeadDim = 128;
constexpr int kTileTok = 16;
constexpr int kHeadsPerCta = 8;
constexpr int kProducerWarps = 2;   // one feeds the K ring, one the V ring
// Consumer warps per kv-head (WPH): 1, or 2 taking alternate tiles where the per-tile
// work is heavier than HBM leaves time for (1-byte pools).  Warp order in a CTA:
// 8*WPH consumers, 2 producers, 1 service warp.
constexpr int kMaxWph = 2;
__host__ __device__ constexpr int cta_threads(int wph) { return (kHeadsPerCta * wph + kProducerWarps + 1) * 32; }
constexpr int kMaxBatch = 4096;
constexpr int kMaxCtas = 256;       // CTAs along x (one per SM)
constexpr int kGroupCtas = 16;      // CTAs per first-level group of the two-level split-K merge
constexpr int kGroupThreshold = 32; // slots per (sequence, kv-head) above which the merge is two-level

constexpr uint32_t kPollLimit = 1u << 20;  // polls of mbarrier.try_wait before giving up

enum : uint32_t {
  kStPipeTimeout = 0x1u,
  kStBadPage = 0x2u,
  kStQTimeout = 0x4u,
  kStPartialTimeout = 0x8u,
};

constexpr int kMaxWorld = 16;       // ranks of one exchange
constexpr int kTraceWords = 8;      // 64-bit time stamps per CTA when a trace buffer is given

struct DecodeParams {
  const void* q;               // [B][Hq][128] 16-bit
  const int32_t* block_table;  // may be null (identity)
  const int32_t* seq_lens;     // [B]
  const void* k_scale;         // quantised pools only: fp16 [page][tok][head]
  const void* v_scale;
  int64_t bt_stride;
  int64_t n_pages;
  int batch;
  int n_q_heads;
  int n_kv_heads;
  int group;           // n_q_heads / n_kv_heads, 1..8
  int page_size;       // tokens per page
  int tiles_per_page;  // ceil(page_size / 16)
  int head_major;      // 1: pool dims are (d, tok, head, page); 0: (d, head, tok, page)
  int n_cta_x;
  int force_empty;     // 1: the pool holds no page; every sequence counts as empty here
  float scale_log2;    // softmax scale * log2(e)
  float* part_o;       // [slots][Hq][128]
  float* part_ml;      // [slots][Hq][2]  (m in log2 units, l)
  uint32_t* status;
  // Epochs are `*epoch_base + <relative value>`: the base is a device word that a captured
  // graph bumps once per replay, so the same launch parameters stay valid.  Null = 0.
  const uint64_t* epoch_base;
  // peer rank: the query arrives in this inbox as 8-byte {payload, epoch} words, [B][Hq][64]
  // (a 16-bit pair per word); a word whose upper half is the step's epoch is this step's.
  // The first word of a sequence also tells that the home GPU has finished reading the rows
  // of the previous step, so this rank's slot there may be overwritten.  Null: q is local.
  const unsigned long long* q_ll;
  uint64_t epoch_rel;
  uint64_t q_timeout_ns;
  // fused combine: the last CTA to finish a sequence merges that sequence's slots
  int fuse;                    // 0: leave the per-CTA partials in part_o / part_ml
  int out_dtype;               // 0 f16, 1 bf16, 4 f32
  void* out;                   // [B][Hq][128] final output, or null
  float* o_part;               // [B][Hq][128] f32 normalised shard partial, or null (may be P2P)
  float* lse_part;             // [B][Hq] natural log, or null (may be P2P)
  // peer rank: the rows go to the home GPU as {fp32, epoch} words instead (P2P), [B][Hq][128]
  // and [B][Hq]; nothing else announces them
  unsigned long long* o_ll;
  unsigned long long* lse_ll;
  unsigned int* seq_counter;   // [batch][n_kv_heads], zero between launches
  unsigned int* grp_counter;   // [(CTA groups + batch)][n_kv_heads], zero between launches
  int grp_slot0;               // first slot index of the per-group partials
  int unit_slot0;              // first of the per-sequence slots the home GPU folds its own splits into
  int sib_slot0;               // first slot index of the second warps' parking slots (two warps per head)
  // adaptive split of the tile list: per-CTA (duration ns, tiles, weight) of the previous
  // launch on this shard; written for the next one.  Word 0 is the CTA count they refer to.
  const uint32_t* obs_read;
  uint32_t* obs_write;
  // home GPU only -- q publish in the prologue: all warps store q [B][Hq][128] into every
  // peer's inbox as {payload, epoch} words; nothing else announces it.
  int pub_n;
  unsigned long long* pub_ll[kMaxWorld];
  // home GPU only -- final merge in the tail: after a (sequence, kv-head) is combined locally
  // the same warp re-reads (bounded) the peers' rows of that pair until every word shows
  // this step's epoch, and folds them in.
  int mg_n;                    // partial slots (ranks); 0 = no merge
  int mg_self;                 // this rank's slot (its own rows never leave the registers)
  uint32_t mg_wait_mask;       // bit r: rank r sends a partial this step
  const unsigned long long* mg_o;     // slot r at mg_o + r * mg_o_stride: [B][Hq][128] words
  const unsigned long long* mg_lse;   // slot r at mg_lse + r * mg_lse_stride: [B][Hq] words
  int64_t mg_o_stride, mg_lse_stride;
  uint64_t mg_timeout_ns;
  uint32_t* mg_status;         // the exchange's status word
  // cumulative counters of the shard: [0] launches, [1] (16-token tile, kv-head) units read; or null
  unsigned long long* stats;
  // measurement aid: [CTAs][kTraceWords] %globaltimer stamps, or null
  //   0 CTA start   1 q published (home) / first q rows seen (peer)   2 last tile consumed
  //   3 last local combine done   4 last peer row complete (home)   5 last row written
  unsigned long long* trace;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_max(const DecodeParams& p, int word) {
  if (p.trace)
    atomicMax(p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * kTraceWords + word, global_ns());
}
__device__ __forceinline__ void trace_first(const DecodeParams& p, int word) {
  if (p.trace) {
    unsigned long long* w = p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * kTraceWords + word;
    atomicCAS(w, 0ull, global_ns());
  }
}

// Barrier `id` (1..15) over the first `n` threads' worth of warps; n a multiple of 32.
__device__ __forceinline__ void bar_sync(int id, int n) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int n) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// Tiles of a sequence with `len` tokens in this shard.
__device__ __forceinline__ int seq_tiles(int len, int page_size, int tiles_per_page) {
  int full = len / page_size;
  int rem = len - full * page_size;
  return full * tiles_per_page + (rem + kTileTok - 1) / kTileTok;
}

// Exclusive prefix of tiles per sequence into smem `prefix[0..batch]`.
// Called by the first `nthr` threads of the block (all but the service warp); ends with
// a barrier among them.
__device__ __forceinline__ void build_tile_prefix(int* prefix, const int32_t* seq_lens, int batch,
                                                  int page_size, int tiles_per_page, bool force_empty,
                                                  int nthr) {
  const int tid = threadIdx.x;
  for (int b = tid; b < batch; b += nthr) {
    int len = force_empty ? 0 : seq_lens[b];
    prefix[b + 1] = len > 0 ? seq_tiles(len, page_size, tiles_per_page) : 0;
  }
  if (tid == 0) prefix[0] = 0;
  bar_sync(1, nthr);
  if (tid < 32) {
    int carry = 0;
    for (int base = 1; base <= batch; base += 32) {
      int i = base + tid;
      int v = i <= batch ? prefix[i] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, o);
        if (tid >= o) v += n;
      }
      v += carry;
      if (i <= batch) prefix[i] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  bar_sync(1, nthr);
}

// Largest s with prefix[s] <= g (prefix non-decreasing, prefix[batch] > g).
__device__ __forceinline__ int find_seq(const int* prefix, int batch, int g) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= g) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void store_out4(void* out, int dtype, int64_t idx, float4 v) {
  if (dtype == 4) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx) = v;
  } else if (dtype == 1) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + idx) =
        make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  } else {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + idx) =
        make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
}

// Online-softmax fold of one slot (running max m in log2 units, sum l, unnormalised row o)
// into the accumulator; a slot with m = -inf carries no tokens and is skipped.
__device__ __forceinline__ void fold_slot(float& M, float& L, float4& acc, float m, float l,
                                          const float4& o) {
  if (m == -INFINITY) return;
  const float mn = fmaxf(M, m);
  const float ca = fast_exp2(M - mn), cs = fast_exp2(m - mn);
  L = L * ca + l * cs;
  acc.x = acc.x * ca + o.x * cs; acc.y = acc.y * ca + o.y * cs;
  acc.z = acc.z * ca + o.z * cs; acc.w = acc.w * ca + o.w * cs;
  M = mn;
}

// One warp merges the partial slots c0..c1 (absolute slot indices) of sequence b for up to four query
// heads qh0.. and writes their rows; each lane owns 4 of the 128 dims.  c1 < c0 means
// the shard holds no token of the sequence.  This runs in the kernel's tail, where a
// dependent chain of L2 round trips is what costs, so each step first issues all
// loads of NS slots x NH heads (statistics and rows, none depending on another and no
// shuffle in between) and only then does the arithmetic.
//
// On the home GPU the peers' shard partials are folded in as well.  They arrive as
// {fp32, epoch} words: a round of loads is repeated (bounded) until every word of it shows
// `tag`, the low half of this step's epoch.  Returns false, with the exchange's status bit
// set, if that did not happen in time; once one wait has run out, later ones of the same
// launch give up at once.
template <int NH, int NS, int NP>   // heads per pass; slots per round; peer partials per round
__device__ __forceinline__ bool combine_heads(const DecodeParams& p, uint32_t tag, int b, int qh0, int nh,
                                              int c0, int c1, int lane, int emit_slot = -1) {
  float4 acc[NH];
  float M[NH], L[NH];
#pragma unroll
  for (int i = 0; i < NH; ++i) {
    acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    M[i] = -INFINITY; L[i] = 0.f;
  }
  const float2* ml2 = reinterpret_cast<const float2*>(p.part_ml);
  for (int base = c0; base <= c1; base += NS) {
    static_assert(NS * NH <= 32, "one lane per (slot, head) statistic");
    float4 os[NS][NH];
    // the statistics of row (jj, i) are loaded by lane jj * NH + i alone and handed round
    // afterwards: every lane loading every row's pair would cost 2 * NS * NH registers
    float2 ml_mine = make_float2(-INFINITY, 0.f);
    {
      const int jj = lane / NH, i = lane - jj * NH;
      if (jj < NS) ml_mine = __ldcg(ml2 + (int64_t)min(base + jj, c1) * p.n_q_heads + qh0 + (i < nh ? i : 0));
    }
#pragma unroll
    for (int jj = 0; jj < NS; ++jj) {
      const int c = min(base + jj, c1);           // clamped: a valid row even past the end
      const int64_t row0 = (int64_t)c * p.n_q_heads + qh0;
#pragma unroll
      for (int i = 0; i < NH; ++i) {
        const int64_t row = row0 + (i < nh ? i : 0);
        os[jj][i] = __ldcg(reinterpret_cast<const float4*>(p.part_o + row * kHeadDim) + lane);
      }
    }
#pragma unroll
    for (int jj = 0; jj < NS; ++jj) {
#pragma unroll
      for (int i = 0; i < NH; ++i) {
        const float m = __shfl_sync(0xffffffffu, ml_mine.x, jj * NH + i);
        const float l = __shfl_sync(0xffffffffu, ml_mine.y, jj * NH + i);
        if (base + jj <= c1) fold_slot(M[i], L[i], acc[i], m, l, os[jj][i]);
      }
    }
  }
  if (emit_slot >= 0) {
    // first level of a two-level merge: the result stays an unnormalised slot
#pragma unroll
    for (int i = 0; i < NH; ++i) {
      if (i < nh) {
        const int64_t row = (int64_t)emit_slot * p.n_q_heads + qh0 + i;
        *reinterpret_cast<float4*>(p.part_o + row * kHeadDim + lane * 4) = acc[i];
        if (lane == 0) *reinterpret_cast<float2*>(p.part_ml + row * 2) = make_float2(M[i], L[i]);
      }
    }
    return true;
  }
  // The peers' shard partials are slots too: (m = lse * log2 e, l = 1, o = O normalised).
  // They are {fp32, epoch} words.  While they are not there yet, only the lse words of the
  // awaited rows are polled, one per lane (a writer stores a row's lse word last).  Then the
  // rows are loaded as whole words, NP ranks x NH heads per round, and a round is repeated
  // (bounded) until every word of it shows the epoch.
  if (p.mg_n > 0) {
    static_assert(NP * NH <= 32, "one lane per (rank, head) lse word");
    const uint32_t mask = p.mg_wait_mask & ~(1u << p.mg_self);
    const int64_t row0 = (int64_t)b * p.n_q_heads + qh0;
    const unsigned long long t0 = global_ns();
    auto give_up = [&]() {
      int stop = 0;
      if (lane == 0) {
        if ((*reinterpret_cast<const volatile uint32_t*>(p.mg_status) & kStPartialTimeout) ||
            global_ns() - t0 > p.mg_timeout_ns) {
          atomicOr(p.mg_status, kStPartialTimeout);
          stop = 1;
        }
      }
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (!stop) __nanosleep(32);
      return stop != 0;
    };
    for (;;) {
      bool fresh = true;
      for (int idx = lane; idx < p.mg_n * NH; idx += 32) {
        const int r = idx / NH, i = idx - r * NH;
        if (((mask >> r) & 1u) && i < nh)
          fresh = fresh && (uint32_t)(ld_ll(p.mg_lse + r * p.mg_lse_stride + row0 + i) >> 32) == tag;
      }
      if (__all_sync(0xffffffffu, fresh)) break;
      if (give_up()) return false;
    }
    for (int r0 = 0; r0 < p.mg_n; r0 += NP) {
      float4 os[NP][NH];
      float lse_mine = -INFINITY;
      for (;;) {
        bool fresh = true;
        {
          const int jj = lane / NH, i = lane - jj * NH, r = r0 + jj;
          if (jj < NP && r < p.mg_n && ((mask >> r) & 1u) && i < nh) {
            const unsigned long long w = ld_ll(p.mg_lse + r * p.mg_lse_stride + row0 + i);
            fresh = (uint32_t)(w >> 32) == tag;
            lse_mine = __uint_as_float((uint32_t)w);
          }
        }
#pragma unroll
        for (int jj = 0; jj < NP; ++jj) {
          const int r = min(r0 + jj, p.mg_n - 1);               // clamped: always a row of the slab
          const bool use = r0 + jj < p.mg_n && ((mask >> r) & 1u);
#pragma unroll
          for (int i = 0; i < NH; ++i) {
            const bool row_fresh =
                ld_ll_row4(p.mg_o + r * p.mg_o_stride + (row0 + (i < nh ? i : 0)) * kHeadDim + lane * 4, tag, os[jj][i]);
            fresh = fresh && (row_fresh || !use || i >= nh);
          }
        }
        if (__all_sync(0xffffffffu, fresh)) break;
        if (give_up()) return false;
      }
#pragma unroll
      for (int jj = 0; jj < NP; ++jj) {
        const int r = r0 + jj;
        const bool use = r < p.mg_n && ((mask >> r) & 1u);
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          const float ls = __shfl_sync(0xffffffffu, lse_mine, jj * NH + i);
          if (use && i < nh) fold_slot(M[i], L[i], acc[i], ls * 1.4426950408889634f, 1.f, os[jj][i]);
        }
      }
    }
    if (lane == 0) trace_max(p, 4);
  }
#pragma unroll
  for (int i = 0; i < NH; ++i) {
    if (i < nh) {
      const float inv = L[i] > 0.f ? 1.f / L[i] : 0.f;
      float4 v = acc[i];
      v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
      const int64_t idx = ((int64_t)b * p.n_q_heads + qh0 + i) * kHeadDim + lane * 4;
      const float lse = L[i] > 0.f ? (M[i] + log2f(L[i])) * 0.6931471805599453f : -INFINITY;
      const int64_t row = (int64_t)b * p.n_q_heads + qh0 + i;
      if (p.out) store_out4(p.out, p.out_dtype, idx, v);
      if (p.o_part) *reinterpret_cast<float4*>(p.o_part + idx) = v;
      if (p.lse_part && lane == 0) p.lse_part[row] = lse;
      if (p.o_ll) st_ll_row(p.o_ll + row * kHeadDim, p.lse_ll + row, v, lse, tag, lane);
    }
  }
  if (lane == 0) trace_max(p, 5);
  return true;
}

// LIGHT: the CTA runs two consumer warps per head and has few registers per thread:
// one head per pass, eight slots and four peer partials per round (wider forms spill).
template <bool LIGHT>
__device__ __forceinline__ bool combine_group(const DecodeParams& p, uint32_t tag, int b, int qh0, int nq,
                                              int c0, int c1, int lane, int emit_slot = -1) {
  bool ok = true;
  if constexpr (LIGHT) {
    for (int i = 0; i < nq && ok; ++i) ok = combine_heads<1, 8, 4>(p, tag, b, qh0 + i, 1, c0, c1, lane, emit_slot);
  } else {
    for (int i = 0; i < nq && ok; i += 4)
      ok = combine_heads<4, 6, 3>(p, tag, b, qh0 + i, min(4, nq - i), c0, c1, lane, emit_slot);
  }
  return ok;
}

// A warp's poll of the query inbox found words of an older step: lane 0 decides whether to
// keep polling (true) or to give up -- the CTA aborted elsewhere, or the query is overdue.
__device__ __forceinline__ bool q_keep_waiting(const DecodeParams& p, unsigned long long t0, int lane,
                                               volatile int* abort_flag) {
  int go = 1;
  if (lane == 0) {
    if (*abort_flag) {
      go = 0;                                         // the CTA gave up elsewhere: just leave
    } else if (global_ns() - t0 > p.q_timeout_ns) {
      atomicOr(p.status, kStQTimeout);
      *abort_flag = 1;
      go = 0;
    }
  }
  go = __shfl_sync(0xffffffffu, go, 0);
  if (go) __nanosleep(64);
  return go != 0;
}

// Bounded wait of one warp (lane 0 polls) until query word `w` shows this step's epoch
// (peer ranks).  The home GPU publishes the query of step e only after its merge of step e-1
// has ended, so once any word of a sequence is fresh this rank's slot on the home GPU may
// be overwritten.
__device__ __forceinline__ bool wait_q_word(const DecodeParams& p, uint64_t epoch, const unsigned long long* w,
                                            int lane, volatile int* abort_flag) {
  const unsigned long long t0 = global_ns();
  for (;;) {
    int ok = 1;
    if (lane == 0) ok = (uint32_t)(ld_ll(w) >> 32) == (uint32_t)epoch;
    if (__shfl_sync(0xffffffffu, ok, 0)) return true;
    if (!q_keep_waiting(p, t0, lane, abort_flag)) return false;
  }
}

// An on-chip wait ended without its barrier: unless the CTA had already aborted for
// another reason (a query that never came), that is a pipeline time-out.
__device__ __forceinline__ void pipe_failed(const DecodeParams& p, volatile int* abort_flag) {
  if (!*abort_flag) {
    atomicOr(p.status, kStPipeTimeout);
    *abort_flag = 1;
  }
}

// Waits for a phase of an on-chip barrier.  Gives up when the CTA has aborted or the
// deadline (%globaltimer) has passed.
__device__ __forceinline__ bool pipe_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long deadline) {
  for (uint32_t w = 0;; ++w) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((w & 63u) == 63u && global_ns() > deadline) return false;
  }
}

// Where each CTA's range of the flat tile list starts: bound[c] .. bound[c+1].
// SMs do not stream at the same rate (the same ones are a few per cent slower launch
// after launch), so an equal split leaves the slowest CTA running alone at the end.
// Each launch therefore records, per CTA, how long its tiles took; the next launch on
// the same shard splits the list in proportion to those rates (damped, clamped to
// [0.5, 2]).  Small problems, a first launch, or a changed grid use the equal split, and
// every CTA computes the same bounds from the same inputs.  Called by the first `nthr`
// threads of the block; ends with a barrier among them.
__device__ __forceinline__ void build_cta_bounds(int* bound, float* wtmp, int total, int n_cta,
                                                 const uint32_t* obs, int nthr) {
  const int tid = threadIdx.x;
  const bool adaptive = obs && obs[0] == (uint32_t)n_cta && total >= 8 * n_cta && n_cta <= kMaxCtas;
  if (!adaptive) {
    const int per = (total + n_cta - 1) / n_cta;
    for (int c = tid; c <= n_cta; c += nthr) {
      bound[c] = min(total, c * per);
      if (c < min(n_cta, kMaxCtas)) wtmp[c] = 1.f;
    }
    bar_sync(1, nthr);
    return;
  }
  // rates of the previous launch
  for (int c = tid; c < n_cta; c += nthr) {
    const float dur = (float)obs[1 + 3 * c], tiles = (float)obs[2 + 3 * c];
    wtmp[c] = (dur > 0.f && tiles > 0.f) ? tiles / dur : 0.f;
  }
  bar_sync(1, nthr);
  if (tid < 32) {
    float sum = 0.f; int cnt = 0;
    for (int c = tid; c < n_cta; c += 32) if (wtmp[c] > 0.f) { sum += wtmp[c]; ++cnt; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    }
    const float mean = cnt > 0 ? sum / cnt : 1.f;
    // weight = half the weight used last time + half the observed relative rate
    float carry = 0.f;
    for (int base = 0; base < n_cta; base += 32) {
      const int c = base + tid;
      float w = 0.f;
      if (c < n_cta) {
        const float rel = wtmp[c] > 0.f ? wtmp[c] / mean : 1.f;
        const float prev = __uint_as_float(obs[3 + 3 * c]);
        const float pw = (prev > 0.25f && prev < 4.f) ? prev : 1.f;
        w = fminf(fmaxf(0.5f * pw + 0.5f * rel, 0.5f), 2.f);
        wtmp[c] = w;
      }
      float v = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, v, o);
        if (tid >= o) v += n;
      }
      v += carry;
      if (c < n_cta) reinterpret_cast<float*>(bound)[c + 1] = v;     // inclusive prefix, as float for now
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
    const float tot_w = carry;
    __syncwarp();
    for (int c = tid; c < n_cta; c += 32) {
      const float cum = reinterpret_cast<float*>(bound)[c + 1];
      int b = (int)((double)total * (double)cum / (double)tot_w);
      b = min(max(b, 0), total);
      if (c == n_cta - 1) b = total;
      bound[c + 1] = b;
    }
    if (tid == 0) bound[0] = 0;
  }
  bar_sync(1, nthr);
}

// The CTA whose range holds tile g: largest c with bound[c] <= g.
__device__ __forceinline__ int find_cta(const int* bound, int n_cta, int g) {
  int lo = 0, hi = n_cta;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (bound[mid] <= g) lo = mid; else hi = mid;
  }
  return lo;
}

// KV element kinds (the PKV_* dtype codes of the C ABI)
constexpr int kKvF16 = 0, kKvBF16 = 1, kKvInt8 = 2, kKvFp8 = 3;

template <int NSTAGE, int ES>   // ES = bytes per KV element (2, or 1 for quantised codes)
struct SmemLayout {
  static constexpr int kHeadBytes = kTileTok * kHeadDim * ES;        // one head of a tile: 4 KiB / 2 KiB
  static constexpr int kSlotBytes = kHeadsPerCta * kHeadBytes;        // one K or V tile: 32 / 16 KiB
  static constexpr int kVOff = NSTAGE * kSlotBytes;                   // V ring after the K ring
  static constexpr int kDataBytes = 2 * NSTAGE * kSlotBytes;
  // quantised pools: fp16 scales of a tile, [16 tok][8 heads], per ring and slot
  static constexpr int kScaleSlot = kTileTok * kHeadsPerCta * 2;      // 256 B
  static constexpr int kScaleOff = kDataBytes;
  static constexpr int kScaleBytes = ES == 1 ? 2 * NSTAGE * kScaleSlot : 0;
  // barriers: full[ring][slot][head], empty[ring][slot], scale_full[ring][slot]
  static constexpr int kBarOff = kScaleOff + kScaleBytes;
  static constexpr int kNumBars = 2 * NSTAGE * kHeadsPerCta + 4 * NSTAGE;
  static constexpr int kAbortOff = kBarOff + kNumBars * 8;
  static constexpr int kSibOff = kAbortOff + 16;                       // [8] per-head hand-over counters (WPH = 2),
                                                                       // then [8] help flags, [8] lo, [8] hi
  static constexpr int kBoundOff = kSibOff + 128;                      // tile range bounds per CTA
  static constexpr int kWeightOff = kBoundOff + (kMaxCtas + 1) * 4;    // split weights (floats)
  static constexpr int kPrefixOff = kWeightOff + kMaxCtas * 4;
  static constexpr int kTotal = kPrefixOff + (kMaxBatch + 1) * 4 + 1024;  // +1024: manual alignment
};

// 1-byte codes -> fp16 pairs, exactly.  int8: bias the byte to unsigned, plant it in the
// mantissa of 1024.0 (0x6400 | u = 1024 + u) and subtract 1152; e4m3: the hardware cvt.
// `SEL_A` / `SEL_B` pick which two bytes of `r` form each pair (prmt selectors).
// UNBIAS = false (int8 only) leaves every value 1152 too large; the caller takes
// 1152 * sum(q) off the dot product instead, which is exact in the fp32 accumulator for
// the 128-term sums it is used on and saves two instructions per register.
template <bool FP8, bool UNBIAS = true>
__device__ __forceinline__ void codes_to_half2(uint32_t r, uint32_t sel_a, uint32_t sel_b,
                                               uint32_t& a, uint32_t& b) {
  if constexpr (FP8) {
    // selectors here choose two source bytes into the low 16 bits (upper bytes zero)
    uint32_t pa, pb;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(pa) : "r"(r), "r"(0u), "r"(sel_a));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(pb) : "r"(r), "r"(0u), "r"(sel_b));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(a) : "h"(static_cast<unsigned short>(pa)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(b) : "h"(static_cast<unsigned short>(pb)));
  } else {
    const uint32_t x = r ^ 0x80808080u;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(a) : "r"(x), "r"(0x64646464u), "r"(sel_a));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(b) : "r"(x), "r"(0x64646464u), "r"(sel_b));
    if constexpr (UNBIAS) {
      const uint32_t bias = 0x64806480u;   // 1152.0 twice
      asm("sub.f16x2 %0, %1, %2;" : "=r"(a) : "r"(a), "r"(bias));
      asm("sub.f16x2 %0, %1, %2;" : "=r"(b) : "r"(b), "r"(bias));
    }
  }
}

// prmt selectors for codes_to_half2.  K (row-wise bytes): pairs (b0,b1) and (b2,b3).
// V (after the transposed load): pairs (b0,b2) and (b1,b3).  int8 pairs are planted as
// [0x64:hi][0x64:lo]; e4m3 pairs are packed into the low 16 bits for the hardware cvt.
template <bool FP8> __device__ __forceinline__ constexpr uint32_t kQuantSelK0() { return FP8 ? 0x4410u : 0x4140u; }
template <bool FP8> __device__ __forceinline__ constexpr uint32_t kQuantSelK1() { return FP8 ? 0x4432u : 0x4342u; }
template <bool FP8> __device__ __forceinline__ constexpr uint32_t kQuantSelV0() { return FP8 ? 0x4420u : 0x4240u; }
template <bool FP8> __device__ __forceinline__ constexpr uint32_t kQuantSelV1() { return FP8 ? 0x4431u : 0x4341u; }

// two bf16 (packed) -> two fp16 (packed), round to nearest
__device__ __forceinline__ uint32_t bf16x2_to_half2(uint32_t v) {
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v);
  const __half2 h = __floats2half2_rn(__low2float(b), __high2float(b));
  return *reinterpret_cast<const uint32_t*>(&h);
}

// KVT: kKvF16 / kKvBF16 (16-bit pools; q has the same type) or kKvInt8 / kKvFp8 (1-byte
// codes with one fp16 scale per (token, kv-head); q is fp16 or bf16 per QBF16 and the
// MMAs run in fp16, into which both code formats convert exactly).
template <int KVT, bool QBF16, int NSTAGE, int WPH>
__global__ void __launch_bounds__(cta_threads(WPH), 1)
decode_partial_kernel(const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
  constexpr bool kQuant = KVT >= kKvInt8;
  constexpr bool BF16 = KVT == kKvBF16;        // operand type of the MMAs
  constexpr int ES = kQuant ? 1 : 2;
  constexpr int kConsumerWarps = kHeadsPerCta * WPH;
  constexpr int kServiceWarp = kConsumerWarps + kProducerWarps;
  using L = SmemLayout<NSTAGE, ES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  int* prefix = reinterpret_cast<int*>(sgen + L::kPrefixOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kAbortOff);
  const uint32_t bar0 = sbase + L::kBarOff;
  // ring 0 = K, ring 1 = V
  auto full = [&](int ring, int s, int h) {
    return bar0 + 8u * ((ring * NSTAGE + s) * kHeadsPerCta + h);
  };
  auto empty = [&](int ring, int s) {
    return bar0 + 8u * (2 * NSTAGE * kHeadsPerCta + ring * NSTAGE + s);
  };
  auto scale_full = [&](int ring, int s) {
    return bar0 + 8u * (2 * NSTAGE * kHeadsPerCta + 2 * NSTAGE + ring * NSTAGE + s);
  };
  auto scale_smem = [&](int ring, int s) {
    return sbase + L::kScaleOff + (ring * NSTAGE + s) * L::kScaleSlot;
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hb = blockIdx.y;                   // block of 8 kv-heads
  const int head0 = hb * kHeadsPerCta;
  const int heads_here = min(kHeadsPerCta, p.n_kv_heads - head0);

  if (threadIdx.x == 0) {
    for (int ring = 0; ring < 2; ++ring)
      for (int s = 0; s < NSTAGE; ++s) {
        for (int h = 0; h < kHeadsPerCta; ++h) mbar_init(full(ring, s, h), 1);
        mbar_init(empty(ring, s), heads_here);   // one arrival per consumer warp with a head
        mbar_init(scale_full(ring, s), 1);
      }
    *abort_flag = 0;
    for (int h = 0; h < 4 * kHeadsPerCta; ++h) reinterpret_cast<volatile int*>(sgen + L::kSibOff)[h] = 0;
    fence_barrier_init();
  }
  // The kernel is launched with programmatic stream serialisation: its CTAs may be placed
  // as soon as the last CTA of the kernel before it in the stream has left, without waiting
  // for that kernel's memory to drain.  Nothing of global memory is touched above this
  // line; below it everything the previous kernel wrote is visible.  The kernel does NOT
  // trigger its own dependents early: CTAs placed on whichever SM frees first land on other
  // SMs than last time, and the split of the tile list, which learns per CTA index how fast
  // its SM streams, then balances worse (measured: 5 % slower steps).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint64_t epoch = (p.epoch_base ? *reinterpret_cast<const volatile uint64_t*>(p.epoch_base) : 0ull) +
                         p.epoch_rel;
  int* bound = reinterpret_cast<int*>(sgen + L::kBoundOff);
  float* cta_weight = reinterpret_cast<float*>(sgen + L::kWeightOff);
  // The service warp (the last one) does not help with the tile list: the other warps build
  // it among themselves (barrier 1) and announce it on barrier 2, where the service warp
  // picks it up.
  constexpr int kWorkThreads = (kConsumerWarps + kProducerWarps) * 32;
  if (p.pub_n > 0) {
    // Home GPU: before anything else, and while the memory system is still idle, EVERY warp
    // of the grid pushes a slice of the query out: a chunk is 512 bytes of q (one 16-byte word
    // per lane) of one sequence for one peer, stored as 1 KiB of {payload, epoch} words.  No
    // fence, no counter, no flag: each 8-byte word proves itself to its reader.
    const int row16 = p.n_q_heads * (kHeadDim * 2 / 16);          // 16-byte words per sequence
    const int cpp = (row16 + 31) / 32;                            // chunks per (sequence, peer)
    const int n_chunks = p.batch * p.pub_n * cpp;
    const int n_warps_cta = blockDim.x >> 5;
    const int gw = (blockIdx.y * gridDim.x + blockIdx.x) * n_warps_cta + warp;
    const int n_gw = gridDim.x * gridDim.y * n_warps_cta;
    for (int c = gw; c < n_chunks; c += n_gw) {
      const int pair = c / cpp, word = (c - pair * cpp) * 32 + lane;
      const int b = pair / p.pub_n, j = pair - b * p.pub_n;
      if (word < row16) {
        const int64_t i = (int64_t)b * row16 + word;
        st_ll_q16(p.pub_ll[j] + 4 * i, __ldcg(reinterpret_cast<const uint4*>(p.q) + i), (uint32_t)epoch);
      }
    }
    if (lane == 0 && gw < n_chunks) trace_max(p, 1);
  }
  if (warp == kServiceWarp) {
    bar_sync(2, kWorkThreads + 32);
  } else {
    build_tile_prefix(prefix, p.seq_lens, p.batch, p.page_size, p.tiles_per_page, p.force_empty != 0,
                      kWorkThreads);
    build_cta_bounds(bound, cta_weight, prefix[p.batch], p.n_cta_x, p.obs_read, kWorkThreads);
    __threadfence_block();
    bar_arrive(2, kWorkThreads + 32);
  }
  const int total = prefix[p.batch];
  const int g0 = bound[blockIdx.x];
  const int g1 = bound[blockIdx.x + 1];
  const unsigned long long t_start = global_ns();
  // every on-chip wait ends by then: the longest legitimate stall (a peer whose query is
  // late) plus two seconds
  const unsigned long long pipe_deadline = t_start + p.q_timeout_ns + 2000000000ull;
  if (threadIdx.x == 0) trace_first(p, 0);
  if (p.stats && threadIdx.x == 0 && blockIdx.x == 0) {
    if (blockIdx.y == 0) atomicAdd(p.stats, 1ull);
    atomicAdd(p.stats + 1, (unsigned long long)total * (unsigned long long)heads_here);   // (tile, kv-head) units
  }
  if (p.obs_write && warp == 0 && lane == 0 && blockIdx.y == 0) {
    if (blockIdx.x == 0) p.obs_write[0] = (uint32_t)p.n_cta_x;
    if (g0 >= g1) {                       // nothing to time: keep the weight, no rate
      p.obs_write[1 + 3 * blockIdx.x] = 0u;
      p.obs_write[2 + 3 * blockIdx.x] = 0u;
      p.obs_write[3 + 3 * blockIdx.x] = __float_as_uint(1.f);
    }
  }
  if (warp == kServiceWarp) {
    // ---------------------------- service warp ---------------------------- //
    // Sequences with no token in this shard have no CTA of their own.  Their rows
    // (neutral, or -- on the home GPU -- the merge of the peers' rows) are written by the
    // service warps: unit (empty sequence e, kv-head h) goes to the service warp of CTA
    // (e * heads_here + h) mod gridDim.x, so a ragged batch whose sequences mostly live on
    // other GPUs does not serialise its merge in one warp.
    if (p.fuse) {
      int unit = 0;
      for (int b = 0; b < p.batch; ++b) {
        if (prefix[b + 1] != prefix[b]) continue;
        for (int h = 0; h < heads_here; ++h, ++unit) {
          if (unit % (int)gridDim.x != (int)blockIdx.x) continue;
          const int qh0 = (head0 + h) * p.group;
          // a peer's rows land in the home GPU's slot: not before the query of this epoch is
          // here, which is also when the home GPU has finished reading the previous rows
          if (p.q_ll && !wait_q_word(p, epoch, p.q_ll + (int64_t)b * p.n_q_heads * (kHeadDim / 2), lane, abort_flag))
            return;
          combine_group<(WPH > 1)>(p, (uint32_t)epoch, b, qh0, p.group, 0, -1, lane);
        }
      }
    }
    return;
  }
  if (g0 >= g1) return;

  if (warp >= kConsumerWarps) {   // warps 8, 9 (the service warp has returned)
    // ------------------------------ producers ----------------------------- //
    // Warp 8 feeds the K ring, warp 9 the V ring.  Lane -> (head, half of the head
    // dimension); each lane issues one 2 KiB box per tile, and each head's two
    // boxes complete on that head's own barrier so its consumer warp can start as
    // soon as ITS rows have landed.
    const int ring = warp - kConsumerWarps;
    const CUtensorMap* map = ring ? &tm_v : &tm_k;
    if (lane == 0) prefetch_tensormap(map);
    const uint64_t stream_policy = l2_policy_evict_first();
    // 16-bit pools: lane -> (head, half of D), 16 lanes, a [64 d][16 tok] box each.
    // 1-byte pools: lane -> head, 8 lanes, a [128 d][16 tok] box each (also 2 KiB), and
    // lanes 8.. copy the tile's fp16 scales.
    const int hh = kQuant ? (lane & 7) : ((lane >> 1) & 7);
    const int dh = kQuant ? 0 : (lane & 1);
    const bool lane_active = lane < (kQuant ? 8 : 16) && hh < heads_here;
    const unsigned int box_lanes = kQuant ? (0xffu >> (kHeadsPerCta - heads_here))
                                          : (0xffffu >> (2 * (kHeadsPerCta - heads_here)));
    const uint32_t ring_base = sbase + (ring ? L::kVOff : 0);
    const uint32_t dst_off = hh * L::kHeadBytes + dh * 2048;
    // scale copies: every kv-head of the pool sits in this CTA (Hkv <= 8): the tile's
    // [16 tok][Hkv] scales are one contiguous run; otherwise one 16-byte row per token.
    const bool scale_one = p.n_kv_heads <= kHeadsPerCta;
    const uint8_t* scale_base = reinterpret_cast<const uint8_t*>(ring ? p.v_scale : p.k_scale);

    int s = find_seq(prefix, p.batch, g0);
    int it = 0;
    bool ok = true;
    for (int g = g0; g < g1 && ok;) {
      while (prefix[s + 1] <= g) ++s;
      const int seg_end = min(g1, prefix[s + 1]);
      int ti = g - prefix[s];                       // tile index inside the sequence
      const int n = seg_end - g;
      for (int base = 0; base < n && ok; base += 32) {
        // one coalesced block-table read per 32 tiles
        const int my_tile = ti + base + lane;
        int my_page = 0;
        if (base + lane < n) {
          const int pj = my_tile / p.tiles_per_page;
          my_page = p.block_table ? p.block_table[(int64_t)s * p.bt_stride + pj]
                                  : (int)((int64_t)s * p.bt_stride + pj);
          if (my_page < 0 || my_page >= p.n_pages) {
            atomicOr(p.status, kStBadPage);
            my_page = 0;
          }
        }
        const int cnt = min(32, n - base);
        int tpos = (ti + base) % p.tiles_per_page;
        for (int j = 0; j < cnt; ++j, ++it) {
          const int stage = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          const int page = __shfl_sync(0xffffffffu, my_page, j);
          const int tok0 = tpos * kTileTok;
          if (++tpos == p.tiles_per_page) tpos = 0;
          int got = 1;
          if (lane == 0) {
            got = pipe_wait(empty(ring, stage), ph ^ 1, abort_flag, pipe_deadline) ? 1 : 0;
            if (!got) pipe_failed(p, abort_flag);
          }
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) { ok = false; break; }
          if (lane_active) {
            const uint32_t bar = full(ring, stage, hh);
            if (dh == 0) mbar_arrive_expect_tx(bar, L::kHeadBytes);
            __syncwarp(box_lanes);
            const uint32_t dst = ring_base + stage * L::kSlotBytes + dst_off;
            if (p.head_major) tma_load_4d(dst, map, bar, dh * 64, tok0, head0 + hh, page, stream_policy);
            else              tma_load_4d(dst, map, bar, dh * 64, head0 + hh, tok0, page, stream_policy);
          }
          if constexpr (kQuant) {
            // scales of the tile: dense [page][tok][head] fp16
            const int64_t row0 = ((int64_t)page * p.page_size + tok0) * p.n_kv_heads + head0;
            const uint32_t sdst = scale_smem(ring, stage);
            const uint32_t sbar = scale_full(ring, stage);
            if (scale_one) {
              if (lane == 8) {
                const uint32_t bytes = kTileTok * p.n_kv_heads * 2;
                mbar_arrive_expect_tx(sbar, bytes);
                bulk_load(sdst, scale_base + row0 * 2, bytes, sbar, stream_policy);
              }
            } else if (lane >= 8 && lane < 8 + kTileTok) {
              if (lane == 8) mbar_arrive_expect_tx(sbar, kTileTok * 16);
              __syncwarp(0x00ffff00u);
              const int r = lane - 8;
              bulk_load(sdst + r * 16, scale_base + (row0 + (int64_t)r * p.n_kv_heads) * 2, 16, sbar, stream_policy);
            }
          }
        }
      }
      g = seg_end;
    }
    if (!ok) {
      // Give copies already in flight a bounded chance to land before the CTA
      // (and its shared memory) goes away.
      if (lane_active && dh == 0) {
        for (int back = 1; back <= NSTAGE && back <= it; ++back) {
          const int jt = it - back;
          mbar_wait_bounded(full(ring, jt % NSTAGE, hh), (jt / NSTAGE) & 1, kPollLimit);
        }
      }
      if (kQuant && lane == 8) {
        for (int back = 1; back <= NSTAGE && back <= it; ++back) {
          const int jt = it - back;
          mbar_wait_bounded(scale_full(ring, jt % NSTAGE), (jt / NSTAGE) & 1, kPollLimit);
        }
      }
    }
    return;
  }

  // -------------------------------- consumers -------------------------------- //
  const int hh = warp & (kHeadsPerCta - 1);     // kv-head inside the block of 8
  const int par = warp / kHeadsPerCta;          // which of the WPH alternating tile streams
  if (hh >= heads_here) return;                 // no head for this warp in a partial block
  const bool active = true;
  const int kvh = head0 + hh;
  const int g = lane >> 2, t = lane & 3;        // MMA fragment row / column-pair ids
  const int G = p.group;
  const uint32_t koff = hh * L::kHeadBytes;
  const uint32_t voff = L::kVOff + hh * L::kHeadBytes;
  const int scale_stride = p.n_kv_heads <= kHeadsPerCta ? p.n_kv_heads : kHeadsPerCta;  // halves per token row
  // ldmatrix lane addressing (row inside the [16 tok][64 d] swizzled block)
  const int krow = lane & 15, kcsel = lane >> 4;
  const int vrow = (lane & 7) + ((lane >> 4) << 3), vcsel = (lane >> 3) & 1;
  const uint32_t krow_off = krow * 128, kx = krow & 7;
  const uint32_t vrow_off = vrow * 128, vx = vrow & 7;

  const bool ps16 = (p.page_size % kTileTok) == 0;

  // What the last CTA of a (sequence, kv-head) does for q heads qh0 .. qh0+nq-1 once the
  // pair's slots lo..hi are complete: the final merge and the rows' way out.
  auto finish_unit = [&](int seq, int qh0, int nq, int lo, int hi) {
    if (p.mg_n > 0) {
      // Home GPU: the peers' rows of this pair are needed, and they usually arrive later
      // than this.  Fold the pair's own slots into one (unnormalised) slot first, so
      // that what is left to do once the rows are here is one round of loads.
      const int us = p.unit_slot0 + seq;
      combine_group<(WPH > 1)>(p, (uint32_t)epoch, seq, qh0, nq, lo, hi, lane, us);
      __threadfence_block();
      __syncwarp();
      lo = hi = us;
    }
    if (lane == 0) trace_max(p, 3);
    combine_group<(WPH > 1)>(p, (uint32_t)epoch, seq, qh0, nq, lo, hi, lane);
  };

  int s = find_seq(prefix, p.batch, g0);
  for (int gt = g0; gt < g1;) {
    while (prefix[s + 1] <= gt) ++s;
    const int seg_end = min(g1, prefix[s + 1]);
    const int len = p.seq_lens[s];

    // On a peer the query rows of this step are pushed by the home GPU as {payload, epoch}
    // words: the loads below are repeated (bounded) until every word carries this epoch.
    const int64_t q_row = (int64_t)s * p.n_q_heads + (int64_t)kvh * G + g;
    const unsigned long long* q_ll_row = p.q_ll ? p.q_ll + q_row * (kHeadDim / 2) : nullptr;
    // A peer's kernel usually starts before the home GPU's: until the query is there, one
    // lane polls one word of this kv-head's rows (a thousand warps re-reading whole rows
    // would load the very L2 lines the query is being written to).
    if (p.q_ll &&
        !wait_q_word(p, epoch, p.q_ll + ((int64_t)s * p.n_q_heads + (int64_t)kvh * G) * (kHeadDim / 2), lane, abort_flag))
      return;

    // Q^T B-fragments: column n = g is q head kvh*G + g (zero beyond the group).
    // 16-bit pools: k-step ks covers d = 16ks..16ks+15 in the natural order.
    // 1-byte pools: the K codes go into 8-bit MMAs (m16n8k32) as they lie in shared memory,
    // so q has to become 8-bit terms: k-step kp covers d = 32kp..32kp+31, register 0 of a
    // term holds d = 32kp+4t..+3 and register 1 d = 32kp+16+4t..+3, one byte each.
    //   int8 codes: q is scaled to 16-bit integers per head (absmax -> 32767) and split into
    //     a signed high byte and an unsigned low byte: two integer MMAs per k-step,
    //     score = (256 acc_hi + acc_lo) * absmax / 32767, exact in int32.
    //   e4m3 codes: q is scaled by a power of two per head (absmax into [128, 256)) and split
    //     into two e4m3 terms q = t1 + t2, t2 the rounding of what t1 left: eight significant
    //     bits, which holds a bf16 value exactly (down to 2^-17 of the head's absmax) and
    //     rounds an fp16 one to that precision.  A product of two e4m3 values is exact in the
    //     fp32 accumulator.
    constexpr int kQTerms = 2;
    uint32_t qf[kQuant ? kQTerms * 4 : 8][2];
    float qmul0 = 1.f, qmul1 = 1.f;      // what the 8-bit terms of score columns 2t, 2t+1 must be multiplied by
    if constexpr (!kQuant) {
      const bool have = active && g < G;
      if (q_ll_row) {
        const unsigned long long t0 = global_ns();
        for (;;) {
          bool fresh = true;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const unsigned long long w0 = have ? ld_ll(q_ll_row + ks * 8 + t) : ll_word(0u, (uint32_t)epoch);
            const unsigned long long w1 = have ? ld_ll(q_ll_row + ks * 8 + 4 + t) : ll_word(0u, (uint32_t)epoch);
            qf[ks][0] = (uint32_t)w0;
            qf[ks][1] = (uint32_t)w1;
            fresh = fresh && (uint32_t)(w0 >> 32) == (uint32_t)epoch && (uint32_t)(w1 >> 32) == (uint32_t)epoch;
          }
          if (__all_sync(0xffffffffu, fresh)) break;
          if (!q_keep_waiting(p, t0, lane, abort_flag)) return;
        }
        if (warp == 0 && lane == 0) trace_first(p, 1);
      } else {
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(p.q) + q_row * (kHeadDim / 2);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          qf[ks][0] = have ? __ldcg(qrow + ks * 8 + t) : 0u;
          qf[ks][1] = have ? __ldcg(qrow + ks * 8 + 4 + t) : 0u;
        }
      }
    } else {
      const uint16_t* qrow = reinterpret_cast<const uint16_t*>(p.q) + q_row * kHeadDim;
      const bool have = active && g < G;
      auto widen = [](const uint2& raw, float (&v)[4]) {
        if constexpr (QBF16) {
          const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          v[0] = __low2float(x); v[1] = __high2float(x); v[2] = __low2float(y); v[3] = __high2float(y);
        } else {
          const __half2 x = *reinterpret_cast<const __half2*>(&raw.x);
          const __half2 y = *reinterpret_cast<const __half2*>(&raw.y);
          v[0] = __low2float(x); v[1] = __high2float(x); v[2] = __low2float(y); v[3] = __high2float(y);
        }
      };
      uint2 qraw[8];
      if (q_ll_row) {
        const unsigned long long t0 = global_ns();
        for (;;) {
          bool fresh = true;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int d0 = 32 * (i >> 1) + 16 * (i & 1) + 4 * t;      // two words: d0, d0+1 | d0+2, d0+3
            unsigned long long w0 = ll_word(0u, (uint32_t)epoch), w1 = w0;
            if (have) ld_ll_x2(q_ll_row + d0 / 2, w0, w1);
            qraw[i] = make_uint2((uint32_t)w0, (uint32_t)w1);
            fresh = fresh && (uint32_t)(w0 >> 32) == (uint32_t)epoch && (uint32_t)(w1 >> 32) == (uint32_t)epoch;
          }
          if (__all_sync(0xffffffffu, fresh)) break;
          if (!q_keep_waiting(p, t0, lane, abort_flag)) return;
        }
        if (warp == 0 && lane == 0) trace_first(p, 1);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int d0 = 32 * (i >> 1) + 16 * (i & 1) + 4 * t;
          qraw[i] = have ? __ldcg(reinterpret_cast<const uint2*>(qrow + d0)) : make_uint2(0u, 0u);
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v[4];
        widen(qraw[i], v);
#pragma unroll
        for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(v[e]));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));      // the head's 128 dims
      const bool live = amax > 1e-30f && amax < 3e38f;
      float pre, post;
      if constexpr (KVT == kKvInt8) {
        pre = live ? 32767.f / amax : 0.f;
        post = live ? amax * (1.f / 32767.f) : 0.f;
      } else {
        const int e2 = (int)((__float_as_uint(amax) >> 23) & 255u) - 127;      // amax in [2^e2, 2^(e2+1))
        pre = live ? __uint_as_float((uint32_t)(127 + 7 - e2) << 23) : 0.f;
        post = live ? __uint_as_float((uint32_t)(127 - 7 + e2) << 23) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int kp = i >> 1, half = i & 1;
        float qv[4];
        widen(qraw[i], qv);
        if constexpr (KVT == kKvInt8) {
          uint32_t hi = 0u, lo = 0u;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int qi = __float2int_rn(qv[e] * pre);             // |qi| <= 32767
            hi |= ((uint32_t)(qi >> 8) & 255u) << (8 * e);
            lo |= ((uint32_t)qi & 255u) << (8 * e);
          }
          qf[kp][half] = hi;
          qf[4 + kp][half] = lo;
        } else {
          float r[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) r[e] = qv[e] * pre;
#pragma unroll
          for (int term = 0; term < kQTerms; ++term) {
            const uint32_t p01 = pack_e4m3x2(r[0], r[1]), p23 = pack_e4m3x2(r[2], r[3]);
            qf[term * 4 + kp][half] = p01 | (p23 << 16);
            const float2 f01 = unpack_e4m3x2(p01), f23 = unpack_e4m3x2(p23);
            r[0] -= f01.x; r[1] -= f01.y; r[2] -= f23.x; r[3] -= f23.y;
          }
        }
      }
      qmul0 = __shfl_sync(0xffffffffu, post, (2 * t) * 4) * p.scale_log2;
      qmul1 = __shfl_sync(0xffffffffu, post, (2 * t + 1) * 4) * p.scale_log2;
    }
    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int n_seq_tiles = prefix[s + 1] - prefix[s];

    const int tile_base = prefix[s];
    for (; gt < seg_end; ++gt) {
      // tile counter of this CTA, its ring slot and phase, and the tile's index in its sequence:
      // all derived from gt, so that nothing but gt is carried around the loop
      const int it = gt - g0;
      if (WPH > 1 && (it & (WPH - 1)) != par) continue;   // the sibling warp's tile
      const int stage = it % NSTAGE;
      const uint32_t ph = (uint32_t)(it / NSTAGE) & 1u;
      const int ti = gt - tile_base;
      // valid tokens of this tile: 16 except on a sequence's last tile (pages that are a
      // multiple of 16 tokens), else from the tile's position inside its page
      int valid = kTileTok;
      if (ps16) {
        if (ti == n_seq_tiles - 1) valid = len - ti * kTileTok;
      } else {
        const int pj = ti / p.tiles_per_page;
        const int tok0 = (ti - pj * p.tiles_per_page) * kTileTok;
        valid = min(kTileTok, min(p.page_size - tok0, len - pj * p.page_size - tok0));
      }
      const uint32_t sk = sbase + stage * L::kSlotBytes + koff;
      const uint32_t sv = sbase + stage * L::kSlotBytes + voff;

      bool got = pipe_wait(full(0, stage, hh), ph, abort_flag, pipe_deadline);
      if (!got) { if (lane == 0) pipe_failed(p, abort_flag); return; }

      float sc[4];
      if (active) {
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (kQuant) {
          // [16 tok][128 B] codes: one ldmatrix.x4 = two 16-byte chunks = the A fragment of
          // one k-step of 32 dims (r0: tok g, bytes 4t..; r1: tok g+8; r2, r3: the next chunk).
          if constexpr (KVT == kKvInt8) {
            int ih[4] = {0, 0, 0, 0}, il[4] = {0, 0, 0, 0};
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {
              uint32_t r[4];
              const uint32_t chunk = (kp << 1) | kcsel;
              ldmatrix_x4(r, sk + krow_off + ((chunk ^ kx) << 4));
              mma_16832_s8<false>(ih, r, qf[kp][0], qf[kp][1]);
              mma_16832_s8<true>(il, r, qf[4 + kp][0], qf[4 + kp][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) sa[i] = (float)(ih[i] * 256 + il[i]);
          } else {
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {
              uint32_t r[4];
              const uint32_t chunk = (kp << 1) | kcsel;
              ldmatrix_x4(r, sk + krow_off + ((chunk ^ kx) << 4));
              mma_16832_e4m3(sa, r, qf[kp][0], qf[kp][1]);
              mma_16832_e4m3(sa, r, qf[4 + kp][0], qf[4 + kp][1]);
            }
          }
          // per-token K scales (rows g and g+8 of the score tile)
          got = pipe_wait(scale_full(0, stage), ph, abort_flag, pipe_deadline);
          if (!got) { if (lane == 0) pipe_failed(p, abort_flag); return; }
          const __half* ksc = reinterpret_cast<const __half*>(sgen + L::kScaleOff + stage * L::kScaleSlot);
          const float k0 = __half2float(ksc[g * scale_stride + hh]);
          const float k1 = __half2float(ksc[(g + 8) * scale_stride + hh]);
          sc[0] = sa[0] * (k0 * qmul0); sc[1] = sa[1] * (k0 * qmul1);
          sc[2] = sa[2] * (k1 * qmul0); sc[3] = sa[3] * (k1 * qmul1);
        } else {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t a[4];
            const uint32_t chunk = ((ks & 3) << 1) | kcsel;
            ldmatrix_x4(a, sk + (ks >> 2) * 2048 + krow_off + ((chunk ^ kx) << 4));
            if (ks & 1) mma_16816<BF16>(sb, a, qf[ks][0], qf[ks][1]);
            else        mma_16816<BF16>(sa, a, qf[ks][0], qf[ks][1]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) sc[i] = (sa[i] + sb[i]) * p.scale_log2;
        }
        if (valid < kTileTok) {
          if (g >= valid) { sc[0] = -INFINITY; sc[1] = -INFINITY; }
          if (g + 8 >= valid) { sc[2] = -INFINITY; sc[3] = -INFINITY; }
        }
        // column (q head) maxima over the 16 tokens
        float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float al0 = fast_exp2(m0 - mn0), al1 = fast_exp2(m1 - mn1);
        m0 = mn0; m1 = mn1;
        sc[0] = fast_exp2(sc[0] - mn0); sc[2] = fast_exp2(sc[2] - mn0);
        sc[1] = fast_exp2(sc[1] - mn1); sc[3] = fast_exp2(sc[3] - mn1);
        l0 = l0 * al0 + sc[0] + sc[2];
        l1 = l1 * al1 + sc[1] + sc[3];
        if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1;
          }
        }
      }

      // the K tile is now in registers (scores): hand its slot back before the PV half
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(0, stage));

      got = pipe_wait(full(1, stage, hh), ph, abort_flag, pipe_deadline);
      if (!got) { if (lane == 0) pipe_failed(p, abort_flag); return; }

      if (active) {
        if constexpr (kQuant) {
          // fold the per-token V scales into P (tokens g and g+8; 0 past the end so that a
          // garbage scale there cannot poison the sum)
          const bool gots = pipe_wait(scale_full(1, stage), ph, abort_flag, pipe_deadline);
          if (!gots) { if (lane == 0) pipe_failed(p, abort_flag); return; }
          const __half* vsc = reinterpret_cast<const __half*>(
              sgen + L::kScaleOff + (NSTAGE + stage) * L::kScaleSlot);
          const float v0 = g < valid ? __half2float(vsc[g * scale_stride + hh]) : 0.f;
          const float v1 = g + 8 < valid ? __half2float(vsc[(g + 8) * scale_stride + hh]) : 0.f;
          sc[0] *= v0; sc[1] *= v0; sc[2] *= v1; sc[3] *= v1;
        }
        // P^T as the B operand: transpose the two 8x8 (tok x head) blocks.
        const uint32_t b0 = movmatrix_trans(pack2<BF16>(sc[0], sc[1]));
        const uint32_t b1 = movmatrix_trans(pack2<BF16>(sc[2], sc[3]));
        // Rows of a partial tile beyond `valid` may hold anything (even NaN bit
        // patterns): blank them in the A fragments instead of touching smem.
        uint32_t mk01 = 0xffffffffu, mk23 = 0xffffffffu;
        if (valid < kTileTok) {
          mk01 = (2 * t < valid ? 0x0000ffffu : 0u) | (2 * t + 1 < valid ? 0xffff0000u : 0u);
          mk23 = (2 * t + 8 < valid ? 0x0000ffffu : 0u) | (2 * t + 9 < valid ? 0xffff0000u : 0u);
        }
        [[maybe_unused]] const uint32_t bias_a[4] = {0x64806480u, 0x64806480u, 0x64806480u, 0x64806480u};
        [[maybe_unused]] const uint32_t nb0 = b0 ^ 0x80008000u, nb1 = b1 ^ 0x80008000u;      // -P
        if constexpr (kQuant) {
          // Transposed 8x8 "b16" loads over code bytes deliver, per thread, the byte pairs
          // (d = 2g, 2g+1) of tokens 2t and 2t+1: bytes (0,2) are row d = 16c+2g of V^T and
          // bytes (1,3) row d = 16c+2g+1.  So MMA row g is d = 16c+2g and row g+8 is
          // d = 16c+2g+1; the flush below writes O with that mapping.
#pragma unroll
          for (int jp = 0; jp < 4; ++jp) {
            uint32_t r[4], a[4];
            const uint32_t chunk = (jp << 1) | kcsel;
            ldmatrix_x4_trans(r, sv + krow_off + ((chunk ^ kx) << 4));
            // r0: toks 0-7, chunk 2jp; r1: toks 8-15, chunk 2jp; r2, r3: chunk 2jp+1
            // int8 codes enter as (code + 1152), three instructions per register instead of
            // five; a second MMA with the constant 1152 and -P takes the bias off again.  Its
            // rounding error is 2^-24 * 1152 * sum(P) per tile at most, i.e. below 1e-4 code
            // units of the normalised output.  Rows past `valid` are zero in the first MMA
            // and carry P = 0 in the second.
            constexpr bool F8 = KVT == kKvFp8;
            codes_to_half2<F8, F8>(r[0], kQuantSelV0<F8>(), kQuantSelV1<F8>(), a[0], a[1]);
            codes_to_half2<F8, F8>(r[1], kQuantSelV0<F8>(), kQuantSelV1<F8>(), a[2], a[3]);
            if (valid < kTileTok) { a[0] &= mk01; a[1] &= mk01; a[2] &= mk23; a[3] &= mk23; }
            mma_16816<false>(o[2 * jp], a, b0, b1);
            if constexpr (!F8) mma_16816<false>(o[2 * jp], bias_a, nb0, nb1);
            codes_to_half2<F8, F8>(r[2], kQuantSelV0<F8>(), kQuantSelV1<F8>(), a[0], a[1]);
            codes_to_half2<F8, F8>(r[3], kQuantSelV0<F8>(), kQuantSelV1<F8>(), a[2], a[3]);
            if (valid < kTileTok) { a[0] &= mk01; a[1] &= mk01; a[2] &= mk23; a[3] &= mk23; }
            mma_16816<false>(o[2 * jp + 1], a, b0, b1);
            if constexpr (!F8) mma_16816<false>(o[2 * jp + 1], bias_a, nb0, nb1);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t a[4];
            const uint32_t chunk = ((j & 3) << 1) | vcsel;
            ldmatrix_x4_trans(a, sv + (j >> 2) * 2048 + vrow_off + ((chunk ^ vx) << 4));
            if (valid < kTileTok) { a[0] &= mk01; a[1] &= mk01; a[2] &= mk23; a[3] &= mk23; }
            mma_16816<BF16>(o[j], a, b0, b1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(1, stage));
    }
    if (gt >= g1 && p.obs_write && warp == 0 && lane == 0 && blockIdx.y == 0) {
      // this CTA's tiles are done: what the next launch's split is computed from
      const unsigned long long t_end = global_ns();
      p.obs_write[1 + 3 * blockIdx.x] = (uint32_t)min(t_end - t_start, 0xffffffffull);
      p.obs_write[2 + 3 * blockIdx.x] = (uint32_t)(g1 - g0);
      p.obs_write[3 + 3 * blockIdx.x] = __float_as_uint(cta_weight[blockIdx.x]);
    }
    if (gt >= g1 && warp == 0 && lane == 0) trace_max(p, 2);
    // flush this (CTA, sequence) partial
    if (active) {
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
      }
      const int h0 = 2 * t, h1 = 2 * t + 1;
      // Two warps per head (1-byte pools): the second warp parks its partial in a slot of
      // its own and hands over; the first folds it into its registers, so the CTA leaves
      // ONE slot per (sequence, kv-head) as with one warp per head.  Both warps walk the
      // same segments in the same order, so the hand-over counter is the sequence number + 1.
      const int slot = (WPH > 1 && par == 1) ? p.sib_slot0 + blockIdx.x + s : blockIdx.x + s;
      const int64_t hbase = (int64_t)slot * p.n_q_heads + (int64_t)kvh * G;
      if constexpr (WPH > 1) {
        volatile int* sib = reinterpret_cast<volatile int*>(sgen + L::kSibOff) + hh;
        if (par == 0) {
          int ok = 1;
          if (lane == 0) {
            ok = 0;
            for (uint32_t w = 0;; ++w) {
              if (*sib > s) { ok = 1; break; }
              if (*abort_flag) break;
              if ((w & 63u) == 63u && global_ns() > pipe_deadline) { pipe_failed(p, abort_flag); break; }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) return;
          __syncwarp();
          const int64_t sbase = (int64_t)(p.sib_slot0 + blockIdx.x + s) * p.n_q_heads + (int64_t)kvh * G;
          const float2 sm0 = h0 < G ? __ldcg(reinterpret_cast<const float2*>(p.part_ml) + sbase + h0) : make_float2(-INFINITY, 0.f);
          const float2 sm1 = h1 < G ? __ldcg(reinterpret_cast<const float2*>(p.part_ml) + sbase + h1) : make_float2(-INFINITY, 0.f);
          const float mn0 = fmaxf(m0, sm0.x), mn1 = fmaxf(m1, sm1.x);
          // factors of own and sibling rows; a side without tokens (m = -inf) counts as zero
          const float a0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - mn0), b0s = sm0.x == -INFINITY ? 0.f : fast_exp2(sm0.x - mn0);
          const float a1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - mn1), b1s = sm1.x == -INFINITY ? 0.f : fast_exp2(sm1.x - mn1);
          l0 = l0 * a0 + sm0.y * b0s; l1 = l1 * a1 + sm1.y * b1s;
          m0 = mn0; m1 = mn1;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int d = 16 * j + 2 * g;          // 1-byte pools: rows g, g+8 of m-tile j are d, d+1
            float s00 = 0.f, s02 = 0.f, s01 = 0.f, s03 = 0.f;
            if (h0 < G) {
              const float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_o + (sbase + h0) * kHeadDim + d));
              s00 = v.x; s02 = v.y;
            }
            if (h1 < G) {
              const float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_o + (sbase + h1) * kHeadDim + d));
              s01 = v.x; s03 = v.y;
            }
            o[j][0] = o[j][0] * a0 + s00 * b0s; o[j][2] = o[j][2] * a0 + s02 * b0s;
            o[j][1] = o[j][1] * a1 + s01 * b1s; o[j][3] = o[j][3] * a1 + s03 * b1s;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // accumulator rows g and g+8 of m-tile j: d = 16j+g, 16j+g+8 (16-bit pools) or
        // d = 16j+2g, 16j+2g+1 (1-byte pools, see the PV loop)
        const int d = kQuant ? 16 * j + 2 * g : 16 * j + g;
        const int d2 = kQuant ? d + 1 : d + 8;
        if (h0 < G) {
          p.part_o[(hbase + h0) * kHeadDim + d] = o[j][0];
          p.part_o[(hbase + h0) * kHeadDim + d2] = o[j][2];
        }
        if (h1 < G) {
          p.part_o[(hbase + h1) * kHeadDim + d] = o[j][1];
          p.part_o[(hbase + h1) * kHeadDim + d2] = o[j][3];
        }
      }
      if (g == 0) {
        if (h0 < G) { p.part_ml[(hbase + h0) * 2] = m0; p.part_ml[(hbase + h0) * 2 + 1] = l0; }
        if (h1 < G) { p.part_ml[(hbase + h1) * 2] = m1; p.part_ml[(hbase + h1) * 2 + 1] = l1; }
      }
      if constexpr (WPH > 1) {
        if (par == 1) {
          __threadfence();
          __syncwarp();
          if (lane == 0) reinterpret_cast<volatile int*>(sgen + L::kSibOff)[hh] = s + 1;
          if (!p.fuse) continue;
          // The first warp of the pair counts the CTA in.  If that made this CTA the last one
          // of the (sequence, kv-head), the merge of the pair's slots is shared: the first
          // warp takes the first half of the group's q heads, this one the second half.
          volatile int* help = reinterpret_cast<volatile int*>(sgen + L::kSibOff) + kHeadsPerCta + hh;
          int verdict = 0;
          if (lane == 0) {
            for (uint32_t w = 0;; ++w) {
              const int v = *help;
              if (v == s + 1 || v == -(s + 1)) { verdict = v; break; }
              if (*abort_flag) break;
              if ((w & 63u) == 63u && global_ns() > pipe_deadline) { pipe_failed(p, abort_flag); break; }
            }
          }
          verdict = __shfl_sync(0xffffffffu, verdict, 0);
          if (verdict == 0) return;
          __syncwarp();
          const int first = (G + 1) / 2;
          if (verdict > 0 && G > first) {
            const int lo2 = help[kHeadsPerCta], hi2 = help[2 * kHeadsPerCta];
            finish_unit(s, kvh * G + first, G - first, lo2, hi2);
          }
          continue;
        }
      }
    }

    if (p.fuse) {
      // Each consumer warp is on its own: it counts its (sequence, kv-head) in, and
      // the warp that arrives last for that pair merges the pair's slots.  No
      // CTA-wide meeting, so the other warps run straight into the next sequence.
      const int t0s = prefix[s], t1s = prefix[s + 1];
      const int c0 = find_cta(bound, p.n_cta_x, t0s), c1 = find_cta(bound, p.n_cta_x, t1s - 1);
      const int slot_lo = c0 + s, slot_hi = c1 + s;
      __threadfence();
      __syncwarp();
      int last = 0;
      int lo = slot_lo, hi = slot_hi;          // what the final merge reads
      if (slot_hi - slot_lo + 1 <= kGroupThreshold) {
        if (lane == 0) {
          unsigned int* ctr = p.seq_counter + (size_t)s * p.n_kv_heads + kvh;
          const unsigned int prev = atomicAdd(ctr, 1u);
          last = prev == (unsigned int)(slot_hi - slot_lo);
          if (last) *ctr = 0;
          __threadfence();
        }
        last = __shfl_sync(0xffffffffu, last, 0);
      } else {
        // A sequence spread over many CTAs (small batches): merge in two levels so the
        // last warp does not walk a hundred slots alone.  CTAs are grouped by
        // c / kGroupCtas; the last warp of a group folds the group's slots into one
        // group slot, then counts the group in; the last group folds the group slots.
        const int gi = blockIdx.x / kGroupCtas, g_lo = c0 / kGroupCtas, g_hi = c1 / kGroupCtas;
        const int cg0 = max(c0, gi * kGroupCtas), cg1 = min(c1, gi * kGroupCtas + kGroupCtas - 1);
        int glast = 0;
        if (lane == 0) {
          unsigned int* ctr = p.grp_counter + (size_t)(gi + s) * p.n_kv_heads + kvh;
          const unsigned int prev = atomicAdd(ctr, 1u);
          glast = prev == (unsigned int)(cg1 - cg0);
          if (glast) *ctr = 0;
          __threadfence();
        }
        glast = __shfl_sync(0xffffffffu, glast, 0);
        if (glast) {
          combine_group<(WPH > 1)>(p, (uint32_t)epoch, s, kvh * G, G, cg0 + s, cg1 + s, lane, p.grp_slot0 + gi + s);
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            unsigned int* ctr = p.seq_counter + (size_t)s * p.n_kv_heads + kvh;
            const unsigned int prev = atomicAdd(ctr, 1u);
            last = prev == (unsigned int)(g_hi - g_lo);
            if (last) *ctr = 0;
            __threadfence();
          }
          last = __shfl_sync(0xffffffffu, last, 0);
          lo = p.grp_slot0 + g_lo + s;
          hi = p.grp_slot0 + g_hi + s;
        }
      }
      int mine = G;                       // q heads of the group this warp merges
      if constexpr (WPH > 1) {
        // tell the second warp of the pair whether there is a merge to share, and over which slots
        volatile int* help = reinterpret_cast<volatile int*>(sgen + L::kSibOff) + kHeadsPerCta + hh;
        if (lane == 0) {
          help[kHeadsPerCta] = lo;
          help[2 * kHeadsPerCta] = hi;
          __threadfence_block();
          *help = last ? s + 1 : -(s + 1);
        }
        mine = (G + 1) / 2;
      }
      if (last) finish_unit(s, kvh * G, mine, lo, hi);
    }
  }
}

}  // namespace pkv
