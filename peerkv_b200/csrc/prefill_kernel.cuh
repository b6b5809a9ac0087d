// Flash-attention partial for MANY query rows over one contiguous KV shard, optionally
// causal: what sharded (ring / context-parallel) prefill runs per (query shard, key shard)
// pair.  Replaces the aten flash-attention calls of PeerKV umallm/peer_parallel_attn.py
// (flash_partial :60-66 and _causal_partial :95-101) with a kernel that returns the
// (O, lse) partial in the same convention as the decode path, so the same merge applies.
//
// One CTA = 64 query rows of one (batch, q head): 4 warps x 16 rows.  The K and V shard is
// streamed once per CTA in tiles of 64 keys through a two-stage cp.async ring (shared
// memory, XOR-swizzled rows so every ldmatrix is bank-conflict free); S = Q K^T and
// O += P V run on the tensor cores (mma.sync m16n8k16, fp32 accumulate), the softmax is
// online per row.  Causal shards skip every key tile that lies wholly in the future and
// mask inside the diagonal tile.  KV traffic per CTA is Sk rows, i.e. Sq/64 reads of the
// shard per head instead of one per query row.
#pragma once
#include "ptx.cuh"

namespace pkv {

constexpr int kPfRows = 64;      // query rows per CTA
constexpr int kPfKeys = 64;      // keys per tile
constexpr int kPfThreads = 128;
constexpr int kPfTileBytes = kPfKeys * kHeadDim * 2;                  // 16 KiB
constexpr int kPfSmem = kPfRows * kHeadDim * 2 + 4 * kPfTileBytes;    // Q + 2 x (K, V) = 80 KiB

struct PrefillParams {
  const void* q;            // (B, Hq, Sq, 128) 16-bit, element strides below, unit last stride
  const void* k;            // (B, Hkv, Sk, 128)
  const void* v;
  int64_t q_sb, q_sh, q_ss;
  int64_t kv_sb, kv_sh, kv_ss;
  int n_q_heads, group;     // group = Hq / Hkv
  int sq, sk;
  int causal;               // 1: query row i sees key j iff k_pos0 + j <= q_pos0 + i
  int64_t q_pos0, k_pos0;
  float scale_log2;
  float* o_part;            // [B][Hq][Sq][128] fp32, normalised
  float* lse_part;          // [B][Hq][Sq] natural log; -inf for a row that sees no key
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;        // n = 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// byte offset of 16-byte chunk `c` (0..15) of row `r` in a [rows][128 x 16-bit] tile
__device__ __forceinline__ uint32_t pf_off(int r, int c) {
  return (uint32_t)r * 256u + (uint32_t)(((c & 8) | ((c ^ r) & 7)) << 4);
}

// rows [row0, row0 + 64) of a (rows, 128) 16-bit matrix -> a swizzled tile; rows >= n_rows are zeros
__device__ __forceinline__ void pf_load_tile(uint32_t smem, const uint16_t* base, int64_t row_stride, int row0,
                                             int n_rows) {
#pragma unroll
  for (int i = 0; i < (kPfKeys * 16) / kPfThreads; ++i) {
    const int idx = threadIdx.x + i * kPfThreads;
    const int r = idx >> 4, c = idx & 15;
    const bool ok = row0 + r < n_rows;
    const uint16_t* src = base + (int64_t)(ok ? row0 + r : 0) * row_stride + c * 8;
    cp_async16(smem + pf_off(r, c), src, ok);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(kPfThreads) prefill_partial_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t pf_smem[];
  const uint32_t sq_ = smem_u32(pf_smem);
  const uint32_t skv = sq_ + kPfRows * kHeadDim * 2;      // stage s: K at skv + s*2*tile, V right after
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int b = blockIdx.z, h = blockIdx.y, row0 = blockIdx.x * kPfRows;
  const int kvh = h / p.group;
  const uint16_t* qb = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_sb + h * p.q_sh;
  const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.k) + b * p.kv_sb + kvh * p.kv_sh;
  const uint16_t* vb = reinterpret_cast<const uint16_t*>(p.v) + b * p.kv_sb + kvh * p.kv_sh;

  // keys this CTA can see at all: a causal CTA stops at its last row's position
  int n_keys = p.sk;
  if (p.causal) {
    const int64_t last_q = p.q_pos0 + min(row0 + kPfRows, p.sq) - 1;
    const int64_t lim = last_q - p.k_pos0 + 1;
    n_keys = (int)max((int64_t)0, min((int64_t)p.sk, lim));
  }
  const int n_tiles = (n_keys + kPfKeys - 1) / kPfKeys;

  pf_load_tile(sq_, qb, p.q_ss, row0, p.sq);
  if (n_tiles > 0) {
    pf_load_tile(skv, kb, p.kv_ss, 0, n_keys);
    pf_load_tile(skv + kPfTileBytes, vb, p.kv_ss, 0, n_keys);
  }
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8 of this warp
  uint32_t qf[8][4];
  const int wr = warp * 16;                                       // this warp's rows inside the CTA tile
  const int64_t qpos_a = p.q_pos0 + row0 + wr + g, qpos_b = qpos_a + 8;

  for (int it = 0; it < n_tiles; ++it) {
    const int st = it & 1;
    if (it + 1 < n_tiles) {
      const uint32_t nxt = skv + (st ^ 1) * 2 * kPfTileBytes;
      pf_load_tile(nxt, kb, p.kv_ss, (it + 1) * kPfKeys, n_keys);
      pf_load_tile(nxt + kPfTileBytes, vb, p.kv_ss, (it + 1) * kPfKeys, n_keys);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        ldmatrix_x4(qf[ks], sq_ + pf_off(wr + (lane & 15), 2 * ks + (lane >> 4)));
    }
    const uint32_t sk_ = skv + st * 2 * kPfTileBytes, sv_ = sk_ + kPfTileBytes;

    // S = Q K^T for 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        uint32_t r[4];
        ldmatrix_x4(r, sk_ + pf_off(8 * j + (lane & 7), 4 * kp + (lane >> 3)));
        mma_16816<BF16>(s[j], qf[2 * kp], r[0], r[1]);
        mma_16816<BF16>(s[j], qf[2 * kp + 1], r[2], r[3]);
      }
    }
    // scale, mask (end of the shard, causal diagonal), row maxima
    const int key0 = it * kPfKeys;
    const bool edge = key0 + kPfKeys > n_keys || (p.causal && p.k_pos0 + key0 + kPfKeys - 1 > p.q_pos0 + row0 + wr);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[j][e] * p.scale_log2;
        if (edge) {
          const int key = key0 + 8 * j + 2 * t + (e & 1);
          const int64_t qpos = (e & 2) ? qpos_b : qpos_a;
          if (key >= n_keys || (p.causal && p.k_pos0 + key > qpos)) v = -INFINITY;
        }
        s[j][e] = v;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    // a row that has seen no key yet keeps m = -inf: use 0 as the reference so exp2 stays finite
    const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    const float al0 = fast_exp2(m0 - ref0), al1 = fast_exp2(m1 - ref1);
    m0 = mn0; m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] = fast_exp2(s[j][0] - ref0); s[j][1] = fast_exp2(s[j][1] - ref0);
      s[j][2] = fast_exp2(s[j][2] - ref1); s[j][3] = fast_exp2(s[j][3] - ref1);
      rs0 += s[j][0] + s[j][1];
      rs1 += s[j][2] + s[j][3];
    }
    l0 = l0 * al0 + rs0;
    l1 = l1 * al1 + rs1;
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }

    // O += P V : k-step kk covers keys 16kk..16kk+15 = score tiles 2kk, 2kk+1.  A bf16 P
    // keeps 8 significant bits, which alone would cost up to 2^-9 of the value spread in the
    // output when a row sees only a few keys; bf16 therefore sends P as two terms (the
    // rounding and what it left), fp16 (11 bits) as one.
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4], a2[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x0 = s[2 * kk + (e >> 1)][(e & 1) * 2], x1 = s[2 * kk + (e >> 1)][(e & 1) * 2 + 1];
        a[e] = pack2<BF16>(x0, x1);
        if constexpr (BF16) {
          const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a[e]));
          a2[e] = pack2<true>(x0 - r.x, x1 - r.y);
        }
      }
#pragma unroll
      for (int c = 0; c < 16; c += 2) {
        uint32_t r[4];
        ldmatrix_x4_trans(r, sv_ + pf_off(16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8, c + (lane >> 4)));
        mma_16816<BF16>(o[c], a, r[0], r[1]);
        mma_16816<BF16>(o[c + 1], a, r[2], r[3]);
        if constexpr (BF16) {
          mma_16816<true>(o[c], a2, r[0], r[1]);
          mma_16816<true>(o[c + 1], a2, r[2], r[3]);
        }
      }
    }
    __syncthreads();          // everyone is done with this stage before it is refilled
  }
  if (n_tiles == 0) cp_async_wait<0>();

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int ra = row0 + wr + g, rb = ra + 8;
  const int64_t base = ((int64_t)b * p.n_q_heads + h) * p.sq;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int d = 8 * j + 2 * t;
    if (ra < p.sq) *reinterpret_cast<float2*>(p.o_part + (base + ra) * kHeadDim + d) = make_float2(o[j][0] * inv0, o[j][1] * inv0);
    if (rb < p.sq) *reinterpret_cast<float2*>(p.o_part + (base + rb) * kHeadDim + d) = make_float2(o[j][2] * inv1, o[j][3] * inv1);
  }
  if (t == 0) {
    if (ra < p.sq) p.lse_part[base + ra] = l0 > 0.f ? (m0 + log2f(l0)) * 0.6931471805599453f : -INFINITY;
    if (rb < p.sq) p.lse_part[base + rb] = l1 > 0.f ? (m1 + log2f(l1)) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace pkv
