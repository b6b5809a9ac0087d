// TEST / BENCH INFRASTRUCTURE ONLY -- not part of the product.
//
// Compiles the REFERENCE's own split-K GQA decode kernels (PeerKV
// csrc/peer_attn_kernels.cuh: attn_split_gqa, attn_combine, merge2_h) for sm_100a from
// the reference checkout, where they lie, and exposes one C entry point that runs the
// reference's two-shard flow (csrc/peer_fused_attn_ext.cu:100-131) with both shards on
// one GPU: split + combine per shard, then merge2_h.  Used by bench.py to report "the
// reference's kernel on this GPU" beside ours on the single-layer configuration.
// Built by oracle/Makefile into oracle/_ref/ (git-ignored); the reference sources are
// included by path at build time and never copied into this repository.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include PEERKV_REF_KERNELS   // -DPEERKV_REF_KERNELS='"<reference>/csrc/peer_attn_kernels.cuh"'

namespace {
float *g_spO = nullptr, *g_spM = nullptr, *g_spL = nullptr, *g_l = nullptr;
__half* g_O = nullptr;
int g_cap_H = 0, g_cap_S = 0;
}

extern "C" int ref_attn_two_shards(const void* q, const void* K0, const void* V0, int T0,
                                   const void* K1, const void* V1, int T1, int H, int HKV, int D,
                                   int S, float scale, void* out, void* stream) {
  if (D != 128) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (H > g_cap_H || S > g_cap_S) {
    cudaFree(g_spO); cudaFree(g_spM); cudaFree(g_spL); cudaFree(g_l); cudaFree(g_O);
    cudaMalloc(&g_spO, sizeof(float) * 2 * H * S * D);
    cudaMalloc(&g_spM, sizeof(float) * 2 * H * S);
    cudaMalloc(&g_spL, sizeof(float) * 2 * H * S);
    cudaMalloc(&g_l, sizeof(float) * 2 * H);
    cudaMalloc(&g_O, sizeof(__half) * 2 * H * D);
    g_cap_H = H; g_cap_S = S;
  }
  const __half* qh = static_cast<const __half*>(q);
  for (int sh = 0; sh < 2; ++sh) {
    const __half* K = static_cast<const __half*>(sh ? K1 : K0);
    const __half* V = static_cast<const __half*>(sh ? V1 : V0);
    const int T = sh ? T1 : T0;
    float* spO = g_spO + (size_t)sh * H * S * D;
    float* spM = g_spM + (size_t)sh * H * S;
    float* spL = g_spL + (size_t)sh * H * S;
    attn_split_gqa<<<H * S, 32, 0, st>>>(qh, K, V, spO, spM, spL, H, HKV, T, D, S, scale);
    attn_combine<<<H, D, 0, st>>>(spO, spM, spL, g_O + (size_t)sh * H * D, g_l + (size_t)sh * H, H, D, S);
  }
  merge2_h<<<(H * D + 127) / 128, 128, 0, st>>>(g_O, g_l, g_O + (size_t)H * D, g_l + H,
                                               static_cast<__half*>(out), H, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
