// Cross-GPU exchange kernels: q publish (home -> peers, P2P stores), the single-pass
// N-way LSE merge (on the slots of an exchange: bounded re-reading of {fp32, epoch} words) and the KV
// quantiser.  Replaces merge2_h (PeerKV csrc/peer_attn_kernels.cuh:64-73) and the
// cudaMemcpyAsync + event fork/join of csrc/peer_fused_attn_ext.cu:100-102,112-128.
#pragma once
#include "decode_kernel.cuh"

namespace pkv {

struct PublishParams {
  const uint4* q;          // [batch][row16] 16-byte words of q
  int batch, row16;        // sequences; 16-byte words per sequence (Hq * 16)
  unsigned long long* dst[kMaxWorld];   // peers' q inboxes (P2P mapped), one block per peer
  const uint64_t* epoch_base;
  uint64_t epoch_rel;
};

// The stand-alone q publish (the fused home step does the same in its own prologue).
// One 1024-thread block per destination peer: each 16-byte word of q goes out as four
// 8-byte {payload, epoch} words, which need neither a fence nor a flag behind them.
__global__ void __launch_bounds__(1024) publish_q_kernel(const PublishParams p) {
  unsigned long long* dst = p.dst[blockIdx.x];
  const uint64_t epoch = (p.epoch_base ? *reinterpret_cast<const volatile uint64_t*>(p.epoch_base) : 0ull) +
                         p.epoch_rel;
  const int64_t n16 = (int64_t)p.batch * p.row16;
  for (int64_t i0 = 0; i0 < n16; i0 += 4096) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + threadIdx.x + 1024 * u;
      if (i < n16) v[u] = __ldcg(p.q + i);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + threadIdx.x + 1024 * u;
      if (i < n16) st_ll_q16(dst + 4 * i, v[u], (uint32_t)epoch);
    }
  }
}

// Measurement aid: round-trip time of the two things a step sends over the fabric, with
// the primitives the decode kernels use.  Two single-warp kernels on two GPUs bounce a flag
// `iters` times; with payload_words > 0 each bounce first stores that many 512-byte lines
// into the other GPU's inbox and passes a system fence, as a partial return does.  role 0
// starts, role 1 answers; out[0] = elapsed ns of this side, out[1] = 1 if a wait ran out
// (every wait is bounded by `timeout_ns`).
// With `ll` set the bounce is what the query publish does instead: the payload goes out as
// 8-byte {payload, marker} words (16 bytes per lane and line), no fence and no flag, and the
// other side polls the words of the last line themselves.  The markers have their top bit
// set, so that none of them passes for the epoch of one of an exchange's first 2^31 steps.
__global__ void __launch_bounds__(32) hop_probe_kernel(int role, int ll, int iters, int payload_words,
                                                       uint4* remote_buf, const uint4* my_buf,
                                                       uint64_t* remote_flag, const uint64_t* my_flag,
                                                       unsigned long long timeout_ns, unsigned long long* out) {
  const int lane = threadIdx.x;
  unsigned long long t0, bad = 0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  auto wait_for = [&](uint32_t v) {
    unsigned long long s, n;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(s));
    if (ll) {
      const unsigned long long* w = reinterpret_cast<const unsigned long long*>(my_buf + (payload_words - 1) * 32 + lane);
      for (;;) {
        unsigned long long a, b;
        ld_ll_x2(w, a, b);
        const bool here = (uint32_t)(a >> 32) == (0x80000000u | v) && (uint32_t)(b >> 32) == (0x80000000u | v);
        if (__all_sync(0xffffffffu, here)) break;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n));
        if (__any_sync(0xffffffffu, n - s > timeout_ns)) { bad = 1; break; }
      }
    } else {
      if (lane == 0) {
        while (ld_acquire_sys_u64(my_flag) < v) {
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n));
          if (n - s > timeout_ns) { bad = 1; break; }
        }
      }
      bad = __shfl_sync(0xffffffffu, bad, 0);
    }
  };
  for (int i = 1; i <= iters && !bad; ++i) {
    if (role == 1) { wait_for((uint32_t)i); if (bad) break; }
    if (ll) {
      for (int w = 0; w < payload_words; ++w)
        st_ll_x2(reinterpret_cast<unsigned long long*>(remote_buf + w * 32 + lane),
                 ll_word((uint32_t)w, 0x80000000u | (uint32_t)i), ll_word((uint32_t)lane, 0x80000000u | (uint32_t)i));
    } else {
      if (payload_words > 0) {
        for (int w = 0; w < payload_words; ++w) remote_buf[w * 32 + lane] = make_uint4(i, 0u, lane, 0u);
        __threadfence_system();
        __syncwarp();
      }
      if (lane == 0) st_release_sys_u64(remote_flag, (uint64_t)i);
    }
    if (role == 0) wait_for((uint32_t)i);
  }
  if (lane == 0) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    out[0] = t1 - t0;
    out[1] = bad;
  }
}

// Adds `step` to a device-resident epoch base: the last node of a captured decode step.
__global__ void bump_epoch_kernel(uint64_t* base, uint64_t step) { *base += step; }

struct MergeParams {
  const float* o_parts;     // part i at o_parts + i*o_stride: [rows][128]
  const float* lse_parts;   // part i at lse_parts + i*lse_stride: [rows]
  int64_t o_stride, lse_stride;
  int n_parts, rows;
  void* out;
  int out_dtype;
  float* lse_out;
  // the slots of an exchange instead of o_parts / lse_parts: {fp32, epoch} words, same
  // strides (in words); the parts with bit i of wait_mask are re-read (bounded) until every
  // word shows the epoch, the others are left out
  const unsigned long long* o_ll;
  const unsigned long long* lse_ll;
  uint32_t wait_mask;
  const uint64_t* epoch_base;
  uint64_t epoch_rel;
  uint64_t timeout_ns;
  uint32_t* status;
};

// One warp per (sequence, q head) row; each lane owns 4 of the 128 output dims.
__global__ void __launch_bounds__(256) merge_partials_kernel(const MergeParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= p.rows) return;
  if (p.o_ll) {
    const uint64_t epoch = (p.epoch_base ? *reinterpret_cast<const volatile uint64_t*>(p.epoch_base) : 0ull) +
                           p.epoch_rel;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float M = -INFINITY, wsum = 0.f;
    for (int i = 0; i < p.n_parts; ++i) {
      if (!((p.wait_mask >> i) & 1u)) continue;
      float4 v;
      float li;
      uint64_t t0, now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      for (;;) {
        const unsigned long long* o_row = p.o_ll + i * p.o_stride + (int64_t)row * kHeadDim;
        const unsigned long long lw = ld_ll(p.lse_ll + i * p.lse_stride + row);
        const bool row_fresh = ld_ll_row4(o_row + lane * 4, (uint32_t)epoch, v);
        if (__all_sync(0xffffffffu, row_fresh && (uint32_t)(lw >> 32) == (uint32_t)epoch)) {
          li = __uint_as_float((uint32_t)lw);
          break;
        }
        int give_up = 0;
        if (lane == 0) {
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if ((*reinterpret_cast<const volatile uint32_t*>(p.status) & kStPartialTimeout) ||
              now - t0 > p.timeout_ns) {
            atomicOr(p.status, kStPartialTimeout);
            give_up = 1;
          }
        }
        if (__shfl_sync(0xffffffffu, give_up, 0)) return;   // status says why; the row is left untouched
        __nanosleep(32);
      }
      if (li == -INFINITY) continue;
      const float mn = fmaxf(M, li);
      const float ca = __expf(M - mn), cs = __expf(li - mn);
      acc.x = acc.x * ca + v.x * cs; acc.y = acc.y * ca + v.y * cs;
      acc.z = acc.z * ca + v.z * cs; acc.w = acc.w * ca + v.w * cs;
      wsum = wsum * ca + cs;
      M = mn;
    }
    if (wsum > 0.f) {
      const float inv = 1.f / wsum;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    store_out4(p.out, p.out_dtype, (int64_t)row * kHeadDim + lane * 4, acc);
    if (p.lse_out && lane == 0) p.lse_out[row] = wsum > 0.f ? M + __logf(wsum) : -INFINITY;
    return;
  }
  float L = -INFINITY;
  for (int i = 0; i < p.n_parts; ++i) L = fmaxf(L, __ldcg(p.lse_parts + i * p.lse_stride + row));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
  if (L > -INFINITY) {
    for (int i = 0; i < p.n_parts; ++i) {
      const float li = __ldcg(p.lse_parts + i * p.lse_stride + row);
      if (li == -INFINITY) continue;
      const float w = __expf(li - L);
      const float4 v = __ldcg(reinterpret_cast<const float4*>(
                                  p.o_parts + i * p.o_stride + (int64_t)row * kHeadDim) + lane);
      acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
      wsum += w;
    }
    const float inv = 1.f / wsum;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  const int64_t idx = (int64_t)row * kHeadDim + lane * 4;
  store_out4(p.out, p.out_dtype, idx, acc);
  if (p.lse_out && lane == 0) p.lse_out[row] = L > -INFINITY ? L + __logf(wsum) : -INFINITY;
}

// Per-row absmax quantiser (one warp per row of 128 values, 4 per lane).
//   a = max|x|; s32 = a/QMAX (1 if a == 0); stored scale s = fp16_rn(s32), bumped to
//   the smallest fp16 subnormal if that rounded to 0; code = q(x / float(s)) with a
//   true fp32 division; int8: rint + clamp to +-127; e4m3: clamp to +-448 then RNE.
template <bool BF16>
__global__ void __launch_bounds__(256)
quantize_kv_kernel(const void* __restrict__ src, int64_t rows, uint8_t* __restrict__ codes,
                   __half* __restrict__ scales, int fmt) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  float x[4];
  const uint2 raw = *(reinterpret_cast<const uint2*>(
                          reinterpret_cast<const uint16_t*>(src) + row * kHeadDim) + lane);
  if constexpr (BF16) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  } else {
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  }
  float a = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
  const float qmax = fmt == 2 ? 127.f : 448.f;
  float s32 = __fdiv_rn(a, qmax);
  if (a == 0.f) s32 = 1.f;
  __half s16 = __float2half_rn(s32);
  if (__half2float(s16) == 0.f) s16 = __ushort_as_half((unsigned short)1);
  const float sf = __half2float(s16);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float y = __fdiv_rn(x[i], sf);
    uint32_t c;
    if (fmt == 2) {
      const float r = fminf(fmaxf(rintf(y), -127.f), 127.f);
      c = static_cast<uint32_t>(static_cast<int>(r)) & 0xffu;
    } else {
      const float yc = fminf(fmaxf(y, -448.f), 448.f);
      uint16_t pr;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pr) : "f"(0.f), "f"(yc));
      c = pr & 0xffu;
    }
    packed |= c << (8 * i);
  }
  *(reinterpret_cast<uint32_t*>(codes + row * kHeadDim) + lane) = packed;
  if (lane == 0) scales[row] = s16;
}

// Appends the new tokens' K and V to a KV cache whose blocks are spread over several GPUs
// (the sharded counterpart of vLLM's reshape_and_cache: slot = block id * block_size +
// offset).  Runs on the GPU that holds key / value / slot_mapping; the pools of the other
// GPUs are written through P2P mappings, so the append needs no second stream and is
// ordered before the step's attention by stream order alone (the query of the step is
// published to the peers only by a later kernel on the same stream).
//   owner d of block id g: the largest d with bases[d] <= g; local block = g - bases[d].
// One warp per (token, kv-head); a negative slot is padding and is skipped.
struct AppendParams {
  const void* key;              // [n_tokens][n_kv_heads][128] 16-bit, token stride kv_token_stride
  const void* value;
  const int64_t* slot_mapping;  // [n_tokens]
  int64_t kv_token_stride;      // elements
  int n_tokens, n_kv_heads, block_size, n_dev;
  int64_t bases[kMaxWorld];
  int64_t n_blocks[kMaxWorld];  // blocks of GPU d's pool (ids beyond are skipped and flagged)
  uint16_t* k_pool[kMaxWorld];  // may be P2P mapped
  uint16_t* v_pool[kMaxWorld];
  int64_t page_stride[kMaxWorld], token_stride[kMaxWorld], head_stride[kMaxWorld];   // elements
  uint32_t* status;             // kStBadPage on a slot outside every pool (may be null)
};

__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (unit >= (int64_t)p.n_tokens * p.n_kv_heads) return;
  const int tok = (int)(unit / p.n_kv_heads), h = (int)(unit % p.n_kv_heads);
  const int64_t slot = p.slot_mapping[tok];
  if (slot < 0) return;
  const int64_t gid = slot / p.block_size;
  const int off = (int)(slot - gid * p.block_size);
  int d = 0;
  for (int k = 1; k < p.n_dev; ++k) if (gid >= p.bases[k]) d = k;
  const int64_t local = gid - p.bases[d];
  if (local < 0 || local >= p.n_blocks[d]) {
    if (p.status && lane == 0) atomicOr(p.status, kStBadPage);
    return;
  }
  const int64_t src = (int64_t)tok * p.kv_token_stride + (int64_t)h * kHeadDim;
  const int64_t dst = local * p.page_stride[d] + (int64_t)off * p.token_stride[d] + (int64_t)h * p.head_stride[d];
  // 128 x 16 bit = 256 bytes per row: 8 bytes per lane
  const uint2 kv = *(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.key) + src) + lane);
  const uint2 vv = *(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.value) + src) + lane);
  *(reinterpret_cast<uint2*>(p.k_pool[d] + dst) + lane) = kv;
  *(reinterpret_cast<uint2*>(p.v_pool[d] + dst) + lane) = vv;
}

// Copy-back staging: the fallback when the peers hold KV but may not lend compute
// (PeerKV umallm/vllm_integration/peerkv_staging.py:82-131, chosen under R1-busy,
// umallm/elastic_policy.py:346-350).  Every block-table entry that names a peer block is
// copied over NVLink into a scratch block at the tail of the home GPU's tensor and the
// entry is rewritten to that scratch block, so a single-GPU decode can run over the
// home tensor alone.  No host round trip: kernel 1 counts each sequence's peer entries,
// kernel 2 ranks them (scratch slot = number of peer entries before it, sequence-major)
// and copies; an entry that finds no scratch slot left is flagged and left pointing at
// scratch block 0.  A block shared by two sequences is staged twice.
struct StageParams {
  const int32_t* block_table;   // [batch][bt_stride] global ids
  const int32_t* seq_lens;      // [batch]
  int32_t* out_table;           // [batch][bt_stride] ids into the home tensor (local or scratch)
  int32_t* row_count;           // [batch] scratch words: peer entries per sequence
  int64_t bt_stride;
  int batch, block_size, n_dev;
  int64_t c_local, c_scratch;   // blocks of the home tensor: [0, c_local) real, then c_scratch scratch blocks
  int64_t bases[kMaxWorld];     // first id of GPU d's blocks (bases[0] = 0; d >= 1 are the peers)
  int64_t n_blocks[kMaxWorld];
  const uint4* k_pool[kMaxWorld];   // peers' pools (P2P mapped); [0] unused
  const uint4* v_pool[kMaxWorld];
  int64_t page_stride16[kMaxWorld]; // peers' block strides in 16-byte words
  uint4* k_home;                // the home tensor (destination)
  uint4* v_home;
  int64_t home_page_stride16;
  int64_t block_words16;        // 16-byte words of one block of K (contiguous inside a block)
  uint32_t* status;
};

__global__ void __launch_bounds__(256) stage_count_kernel(const StageParams p) {
  __shared__ int red[8];
  const int b = blockIdx.x;
  const int n_blk = (p.seq_lens[b] + p.block_size - 1) / p.block_size;
  const int32_t* row = p.block_table + (int64_t)b * p.bt_stride;
  int cnt = 0;
  for (int j = threadIdx.x; j < n_blk; j += blockDim.x) cnt += row[j] >= p.c_local ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    p.row_count[b] = t;
  }
}

// grid (batch): one block per sequence walks its entries in order, 8 warps = 8 entries at a time.
__global__ void __launch_bounds__(256) stage_copy_kernel(const StageParams p) {
  __shared__ int s_base, red[8];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {                                                           // peer entries of the sequences before this one
    int part = 0;
    for (int i = threadIdx.x; i < b; i += blockDim.x) part += p.row_count[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) red[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      int base = 0;
      for (int w = 0; w < 8; ++w) base += red[w];
      s_base = base;
    }
    __syncthreads();
  }
  const int n_blk = (p.seq_lens[b] + p.block_size - 1) / p.block_size;
  const int32_t* row = p.block_table + (int64_t)b * p.bt_stride;
  int32_t* out = p.out_table + (int64_t)b * p.bt_stride;
  int before = s_base;                                        // peer entries ranked so far
  for (int j0 = 0; j0 < n_blk; j0 += 32) {
    const int j = j0 + lane;
    const int64_t gid = j < n_blk ? row[j] : 0;
    const bool peer = j < n_blk && gid >= p.c_local;
    const unsigned int bal = __ballot_sync(0xffffffffu, peer);
    const int slot = before + __popc(bal & ((1u << lane) - 1u));
    before += __popc(bal);
    if (j < n_blk && warp == 0) {                              // one warp writes the table
      int32_t v = (int32_t)gid;
      if (peer) {
        if (slot < p.c_scratch) v = (int32_t)(p.c_local + slot);
        else { v = (int32_t)p.c_local; atomicOr(p.status, kStBadPage); }
      }
      out[j] = v;
    }
    // the copies: entry e of this group of 32 is taken by warp e mod 8
    for (int e = warp; e < 32; e += 8) {
      const bool e_peer = (bal >> e) & 1u;
      if (!e_peer) continue;
      const int e_slot = before - __popc(bal) + __popc(bal & ((1u << e) - 1u));
      if (e_slot >= p.c_scratch) continue;
      const int64_t e_gid = __shfl_sync(0xffffffffu, gid, e);
      int d = 1;
      for (int k = 2; k < p.n_dev; ++k) if (e_gid >= p.bases[k]) d = k;
      const int64_t local = e_gid - p.bases[d];
      if (local < 0 || local >= p.n_blocks[d]) { if (lane == 0) atomicOr(p.status, kStBadPage); continue; }
      const uint4* sk = p.k_pool[d] + local * p.page_stride16[d];
      const uint4* sv = p.v_pool[d] + local * p.page_stride16[d];
      uint4* dk = p.k_home + (p.c_local + e_slot) * p.home_page_stride16;
      uint4* dv = p.v_home + (p.c_local + e_slot) * p.home_page_stride16;
      for (int64_t i = lane; i < p.block_words16; i += 128) {
        uint4 a[4], c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t w = i + 32 * u;
          if (w < p.block_words16) { a[u] = sk[w]; c[u] = sv[w]; }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t w = i + 32 * u;
          if (w < p.block_words16) { dk[w] = a[u]; dv[w] = c[u]; }
        }
      }
    }
  }
}

// Splits a global block table into per-GPU local tables (the device-side form of
// the id test in PeerKV umallm/peerkv/paged.py:52-61, generalised to N GPUs).
//   mode 0 (ranges):      owner d = largest d with bases[d] <= gid, local id = gid - bases[d]
//   mode 1 (round robin): owner d = gid mod n_dev,                  local id = gid div n_dev
// One warp per (sequence, device): a stable ballot compaction keeps sequence
// order, so a sequence's partial last page stays last in its owner's list.
struct SplitParams {
  const int32_t* block_table;   // [batch][bt_stride] global ids
  const int32_t* seq_lens;      // [batch] tokens
  int64_t bt_stride;
  int batch, page_size, n_dev, mode;
  int64_t bases[kMaxWorld];
  int32_t* out_table[kMaxWorld];  // [batch][out_stride] each; may be P2P mapped
  int32_t* out_lens[kMaxWorld];   // [batch] each
  int64_t out_stride;
};

__global__ void __launch_bounds__(32) split_block_table_kernel(const SplitParams p) {
  const int b = blockIdx.x, d = blockIdx.y, lane = threadIdx.x;
  const int len = p.seq_lens[b];
  const int n_blk = len > 0 ? (len + p.page_size - 1) / p.page_size : 0;
  const int32_t* row = p.block_table + (int64_t)b * p.bt_stride;
  int32_t* out = p.out_table[d] + (int64_t)b * p.out_stride;
  int cnt = 0;
  bool owns_last = false;
  for (int j0 = 0; j0 < n_blk; j0 += 32) {
    const int j = j0 + lane;
    bool mine = false;
    int local = 0;
    if (j < n_blk) {
      const int64_t gid = row[j];
      if (p.mode == 1) {
        mine = (gid % p.n_dev) == d;
        local = (int)(gid / p.n_dev);
      } else {
        int owner = 0;
        for (int k = 1; k < p.n_dev; ++k) if (gid >= p.bases[k]) owner = k;
        mine = owner == d;
        local = (int)(gid - p.bases[d]);
      }
      if (mine && j == n_blk - 1) owns_last = true;
    }
    const unsigned int bal = __ballot_sync(0xffffffffu, mine);
    if (mine) out[cnt + __popc(bal & ((1u << lane) - 1u))] = local;
    cnt += __popc(bal);
  }
  owns_last = __any_sync(0xffffffffu, owns_last);
  if (lane == 0) {
    int tok = cnt * p.page_size;
    if (owns_last) tok -= n_blk * p.page_size - len;
    p.out_lens[d][b] = tok;
  }
}

}  // namespace pkv
