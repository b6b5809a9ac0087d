// The small kernels of a decoder layer around the attention call: RMSNorm with the
// residual add fused in, RoPE with the append of the new token's K/V to the paged pool,
// and SwiGLU.  They replace rmsnorm_kernel / add_kernel / swiglu_kernel / copy_kernel of
// PeerKV csrc/peer_fused_decoder.cu:51-95 (which has neither RoPE nor a KV append,
// :205-206) for batch > 1.  All are a few KB of traffic per launch: what matters is
// that each is ONE launch, so a captured decode step has few nodes between its GEMMs.
#pragma once
#include "ptx.cuh"

namespace pkv {

template <bool BF16> struct Elem16;
template <> struct Elem16<true> {
  using T = __nv_bfloat16; using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float2 up(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<const T2*>(&v)); }
  static __device__ __forceinline__ uint32_t down(float a, float b) { T2 r = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&r); }
  static __device__ __forceinline__ float round(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }
};
template <> struct Elem16<false> {
  using T = __half; using T2 = __half2;
  static __device__ __forceinline__ float2 up(uint32_t v) { return __half22float2(*reinterpret_cast<const T2*>(&v)); }
  static __device__ __forceinline__ uint32_t down(float a, float b) { T2 r = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&r); }
  static __device__ __forceinline__ float round(float a) { return __half2float(__float2half_rn(a)); }
};

// One block per row.  With `delta` the row is first updated in place, x += delta (the
// residual add, rounded to the 16-bit type as a separate add would), then
// out = x * rsqrt(mean(x^2) + eps) * weight, in fp32 with one rounding at the end.
// hidden must be a multiple of 8; any number of threads.
template <bool BF16>
__global__ void __launch_bounds__(512) add_rmsnorm_kernel(void* __restrict__ x_, const void* __restrict__ delta_,
                                                          const void* __restrict__ w_, void* __restrict__ out_,
                                                          int hidden, float eps) {
  using E = Elem16<BF16>;
  extern __shared__ float row_sm[];                 // the row in fp32
  __shared__ float red[32];
  const int64_t base = (int64_t)blockIdx.x * hidden;
  uint4* x = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(x_) + base);
  const uint4* delta = delta_ ? reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(delta_) + base) : nullptr;
  const uint4* w = reinterpret_cast<const uint4*>(w_);
  uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out_) + base);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 v = x[i];
    uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
    float f[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 a = E::up(pv[k]); f[2 * k] = a.x; f[2 * k + 1] = a.y; }
    if (delta) {
      const uint4 dv = delta[i];
      const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = E::up(pd[k]);
        f[2 * k] = E::round(f[2 * k] + a.x); f[2 * k + 1] = E::round(f[2 * k + 1] + a.y);
        pv[k] = E::down(f[2 * k], f[2 * k + 1]);
      }
      x[i] = v;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) { row_sm[i * 8 + k] = f[k]; ss += f[k] * f[k]; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / (float)hidden + eps);
  }
  __syncthreads();
  const float rstd = red[0];
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    const uint4 wv = w[i];
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv);
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = E::up(pw[k]);
      po[k] = E::down(row_sm[i * 8 + 2 * k] * rstd * a.x, row_sm[i * 8 + 2 * k + 1] * rstd * a.y);
    }
    out[i] = o;
  }
}

struct RopeParams {
  const void* qkv;           // [B][(Hq + 2 Hkv) * D]: q heads, then k heads, then v heads
  const int64_t* positions;  // [B] index of the new token
  const float* inv_freq;     // [D / 2]
  void* q_out;               // [B][Hq][D]
  void* k_pool;              // paged pools (may be null: no append)
  void* v_pool;
  const int64_t* pages;      // [B] page of this GPU's pool that takes the new token
  const int64_t* slots;      // [B] token slot inside that page
  int64_t page_stride, token_stride, head_stride;   // elements
  int n_q_heads, n_kv_heads, head_dim;
};

// grid (B, Hq + 2 Hkv), D/2 threads.  Rotate-half RoPE (x1, x2 = the two halves of a head:
// out1 = x1 cos - x2 sin, out2 = x2 cos + x1 sin, angle = position * inv_freq[i], fp32) on
// the q and k heads; q goes to q_out, the rotated k and the plain v go straight into the
// page slot of the pool.
template <bool BF16>
__global__ void rope_append_kernel(const RopeParams p) {
  using E = Elem16<BF16>;
  using T = typename E::T;
  const int b = blockIdx.x, h = blockIdx.y, i = threadIdx.x, half = p.head_dim / 2;
  const T* src = reinterpret_cast<const T*>(p.qkv) + ((int64_t)b * (p.n_q_heads + 2 * p.n_kv_heads) + h) * p.head_dim;
  T* dst;
  if (h < p.n_q_heads) {
    dst = reinterpret_cast<T*>(p.q_out) + ((int64_t)b * p.n_q_heads + h) * p.head_dim;
  } else {
    if (!p.k_pool) return;
    const bool is_v = h >= p.n_q_heads + p.n_kv_heads;
    const int kh = h - p.n_q_heads - (is_v ? p.n_kv_heads : 0);
    dst = reinterpret_cast<T*>(is_v ? p.v_pool : p.k_pool) + p.pages[b] * p.page_stride +
          p.slots[b] * p.token_stride + kh * p.head_stride;
    if (is_v) {
      dst[i] = src[i];
      dst[i + half] = src[i + half];
      return;
    }
  }
  const float ang = (float)p.positions[b] * p.inv_freq[i];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  float x1, x2;
  if constexpr (BF16) { x1 = __bfloat162float(src[i]); x2 = __bfloat162float(src[i + half]); }
  else { x1 = __half2float(src[i]); x2 = __half2float(src[i + half]); }
  const float o1 = x1 * cs - x2 * sn, o2 = x2 * cs + x1 * sn;
  if constexpr (BF16) { dst[i] = __float2bfloat16_rn(o1); dst[i + half] = __float2bfloat16_rn(o2); }
  else { dst[i] = __float2half_rn(o1); dst[i + half] = __float2half_rn(o2); }
}

// out[r][f] = silu(gu[r][f]) * gu[r][ffn + f], eight elements per thread; ffn % 8 == 0.
template <bool BF16>
__global__ void __launch_bounds__(256) swiglu_kernel(const void* __restrict__ gu_, void* __restrict__ out_,
                                                     int rows, int ffn) {
  using E = Elem16<BF16>;
  const int64_t n8 = (int64_t)rows * (ffn / 8);
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  const int r = (int)(idx / (ffn / 8)), c = (int)(idx % (ffn / 8));
  const uint4* gu = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(gu_) + (int64_t)r * 2 * ffn);
  const uint4 gv = gu[c], uv = gu[ffn / 8 + c];
  const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
  const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uv);
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = E::up(pg[k]), u = E::up(pu[k]);
    // silu in fp32, rounded to the 16-bit type before the product (as two separate ops would)
    const float s0 = E::round(g.x / (1.f + __expf(-g.x))), s1 = E::round(g.y / (1.f + __expf(-g.y)));
    po[k] = E::down(s0 * u.x, s1 * u.y);
  }
  reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out_) + (int64_t)r * ffn)[c] = o;
}

}  // namespace pkv
