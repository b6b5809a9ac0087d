// C ABI of the library (declared in include/peerkv.h): argument checking, tensor-map
// construction, persistent scratch and kernel launches.  No allocation, stream or
// event creation happens on the per-step entry points.
#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/peerkv.h"
#include "merge_kernel.cuh"
#include "layer_kernels.cuh"
#include "prefill_kernel.cuh"

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define PKV_CUDA(expr)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (expr);                                                            \
    if (e_ != cudaSuccess)                                                              \
      return fail(PKV_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_),   \
                  __FILE__, __LINE__);                                                  \
  } while (0)

// A named range around each entry point's work, for timelines taken with a profiler
// (header-only NVTX: costs a few nanoseconds when nothing listens).
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* base;
  int32_t dtype, n_kv_heads, page_size;
  int64_t n_pages, page_stride, token_stride, head_stride;
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
constexpr size_t kMapCache = 256;   // tensor maps kept per shard: two per layer of a model and pool
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  uint64_t stamp;
};

bool is_16bit(int dt) { return dt == PKV_F16 || dt == PKV_BF16; }
bool is_quant(int dt) { return dt == PKV_INT8 || dt == PKV_FP8_E4M3; }

}  // namespace

struct pkv_shard {
  int device = 0;
  int num_sms = 0;
  int max_batch = 0;
  int n_q_heads = 0;
  int n_slots = 0;
  int grp_slot0 = 0;
  size_t grp_counter_off = 0;        // word offset of the group counters inside `counters`
  float* part_o = nullptr;
  float* part_ml = nullptr;
  uint32_t* status = nullptr;       // device word
  unsigned int* counters = nullptr;  // [n_counter_words]: 64 spare words, then per (sequence, kv-head)
  unsigned long long* trace = nullptr;   // caller's time-stamp buffer (pkv_shard_trace), or null
  size_t n_counter_words = 0;
  uint32_t* obs[2] = {nullptr, nullptr};   // per-CTA timings of the last launch / for the next one
  int obs_parity = 0;
  std::vector<MapEntry> maps;
  uint64_t stamp = 0;
  bool attr_set = false;
  bool cache_maps = true;
};

struct pkv_exchange {
  int device = 0, rank = 0, world = 1, max_batch = 0, n_q_heads = 0;
  uint8_t* slab = nullptr;                  // this GPU's mailboxes (cudaMalloc)
  uint8_t* peer_slab[pkv::kMaxWorld] = {};  // mapped slabs by rank (own slab at [rank])
  bool imported[pkv::kMaxWorld] = {};       // opened with cudaIpcOpenMemHandle
  uint32_t* status = nullptr;               // local: status word; epoch base at byte 128
  uint64_t epoch = 0;                       // steps begun (absolute)
  uint64_t base_host = 0;                   // host mirror of the device-resident epoch base
  uint64_t cap_epoch0 = 0, cap_steps = 0;   // graph capture: epoch at its start, steps it holds
  bool capturing = false;
  size_t off_q = 0, off_o = 0, off_lse = 0, off_probe = 0, slab_bytes = 0;
  size_t o_part_elems = 0, lse_part_elems = 0;
};

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Partial slot `slot` in rank `owner_rank`'s slab, as 8-byte {fp32, epoch} words:
// O [max_batch][n_q_heads][128] and lse [max_batch][n_q_heads].
unsigned long long* slot_o(pkv_exchange* x, int owner_rank, int slot) {
  return reinterpret_cast<unsigned long long*>(x->peer_slab[owner_rank] + x->off_o) + (size_t)slot * x->o_part_elems;
}
unsigned long long* slot_lse(pkv_exchange* x, int owner_rank, int slot) {
  return reinterpret_cast<unsigned long long*>(x->peer_slab[owner_rank] + x->off_lse) + (size_t)slot * x->lse_part_elems;
}
// query inbox of rank `owner_rank`: [max_batch][n_q_heads][64] 8-byte {payload, epoch} words
unsigned long long* q_inbox(pkv_exchange* x, int owner_rank) {
  return reinterpret_cast<unsigned long long*>(x->peer_slab[owner_rank] + x->off_q);
}
uint64_t* epoch_base_dev(pkv_exchange* x) {
  return reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(x->status) + 128);
}

}  // namespace


namespace {

int build_map(pkv_shard* s, const void* base, const pkv_kv_view& kv, CUtensorMap* out) {
  MapKey key;
  memset(&key, 0, sizeof key);
  key.base = base; key.dtype = kv.dtype; key.n_kv_heads = kv.n_kv_heads;
  key.page_size = kv.page_size; key.n_pages = kv.n_pages; key.page_stride = kv.page_stride;
  key.token_stride = kv.token_stride; key.head_stride = kv.head_stride;
  if (s->cache_maps)
    for (auto& e : s->maps)
      if (e.key == key) { e.stamp = ++s->stamp; *out = e.map; return PKV_OK; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(PKV_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const uint64_t es = is_16bit(kv.dtype) ? 2 : 1;
  const bool head_major = kv.head_stride >= kv.token_stride;
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  dims[0] = pkv::kHeadDim;
  box[0] = static_cast<cuuint32_t>(128 / es);   // 128 bytes: one swizzle row
  if (head_major) {
    dims[1] = kv.page_size; dims[2] = kv.n_kv_heads;
    strides[0] = kv.token_stride * es; strides[1] = kv.head_stride * es;
    box[1] = pkv::kTileTok; box[2] = 1;
  } else {
    dims[1] = kv.n_kv_heads; dims[2] = kv.page_size;
    strides[0] = kv.head_stride * es; strides[1] = kv.token_stride * es;
    box[1] = 1; box[2] = pkv::kTileTok;
  }
  dims[3] = kv.n_pages;
  strides[2] = kv.page_stride * es;
  box[3] = 1;
  CUtensorMapDataType dt = kv.dtype == PKV_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : kv.dtype == PKV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  MapEntry e;
  e.key = key;
  CUresult r = enc(&e.map, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(PKV_E_CUDA,
                "cuTensorMapEncodeTiled failed (%d) for pool %p: heads %d page_size %d pages %lld "
                "strides (page %lld, tok %lld, head %lld)",
                (int)r, base, kv.n_kv_heads, kv.page_size, (long long)kv.n_pages,
                (long long)kv.page_stride, (long long)kv.token_stride, (long long)kv.head_stride);
  *out = e.map;
  if (!s->cache_maps) return PKV_OK;   // encoding is host arithmetic only; nothing is stored
  e.stamp = ++s->stamp;
  if (s->maps.size() < kMapCache) {
    s->maps.push_back(e);
  } else {
    size_t victim = 0;
    for (size_t i = 1; i < s->maps.size(); ++i)
      if (s->maps[i].stamp < s->maps[victim].stamp) victim = i;
    s->maps[victim] = e;
  }
  return PKV_OK;
}

int check_args(const pkv_shard* s, const pkv_decode_args* a) {
  if (!s || !a) return fail(PKV_E_INVALID, "null shard or args");
  const pkv_kv_view& kv = a->kv;
  if (a->batch < 0 || a->batch > s->max_batch)
    return fail(PKV_E_INVALID, "batch %d outside [0, max_batch=%d]", a->batch, s->max_batch);
  if (a->n_q_heads != s->n_q_heads)
    return fail(PKV_E_INVALID, "n_q_heads %d differs from the shard's %d", a->n_q_heads,
                s->n_q_heads);
  if (kv.head_dim != pkv::kHeadDim)
    return fail(PKV_E_UNSUPPORTED, "head_dim %d: the kernels require 128", kv.head_dim);
  if (kv.n_kv_heads <= 0 || a->n_q_heads % kv.n_kv_heads)
    return fail(PKV_E_INVALID, "n_q_heads %d is not a multiple of n_kv_heads %d", a->n_q_heads,
                kv.n_kv_heads);
  const int group = a->n_q_heads / kv.n_kv_heads;
  if (group > 8)
    return fail(PKV_E_UNSUPPORTED, "GQA group %d: at most 8 query heads per kv head", group);
  if (!is_16bit(a->q_dtype)) return fail(PKV_E_INVALID, "q_dtype must be PKV_F16 or PKV_BF16");
  if (is_16bit(kv.dtype)) {
    if (kv.dtype != a->q_dtype)
      return fail(PKV_E_INVALID, "16-bit KV (%d) and q (%d) must share a dtype", kv.dtype,
                  a->q_dtype);
  } else if (is_quant(kv.dtype)) {
    if (kv.n_pages > 0 && (!kv.k_scale || !kv.v_scale))
      return fail(PKV_E_INVALID, "quantised KV needs k_scale and v_scale");
    if (kv.page_size % pkv::kTileTok)
      return fail(PKV_E_UNSUPPORTED, "quantised KV: page_size %d must be a multiple of 16", kv.page_size);
    if (kv.n_kv_heads > pkv::kHeadsPerCta && kv.n_kv_heads % pkv::kHeadsPerCta)
      return fail(PKV_E_UNSUPPORTED, "quantised KV: n_kv_heads %d must be <= 8 or a multiple of 8",
                  kv.n_kv_heads);
    if ((reinterpret_cast<uintptr_t>(kv.k_scale) | reinterpret_cast<uintptr_t>(kv.v_scale)) & 15)
      return fail(PKV_E_INVALID, "scale arrays must be 16-byte aligned");
  } else {
    return fail(PKV_E_INVALID, "kv dtype %d unknown", kv.dtype);
  }
  if (a->batch > 0) {
    if (!a->q || !a->seq_lens) return fail(PKV_E_INVALID, "null q or seq_lens");
    if (kv.n_pages > 0 && (!kv.k || !kv.v)) return fail(PKV_E_INVALID, "null k or v pool");
    if (kv.page_size <= 0) return fail(PKV_E_INVALID, "page_size %d", kv.page_size);
    const int64_t es = is_16bit(kv.dtype) ? 2 : 1;
    const int64_t mod = 16 / es;
    if (kv.page_stride % mod || kv.token_stride % mod || kv.head_stride % mod)
      return fail(PKV_E_INVALID, "KV strides must be multiples of 16 bytes");
    if ((reinterpret_cast<uintptr_t>(kv.k) | reinterpret_cast<uintptr_t>(kv.v)) & 15)
      return fail(PKV_E_INVALID, "KV pool bases must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(a->q) & 3) return fail(PKV_E_INVALID, "q must be 4-byte aligned");
  }
  return PKV_OK;
}

struct LaunchOut {
  void* out = nullptr;
  int out_dtype = PKV_F32;
  float* o_part = nullptr;
  float* lse_part = nullptr;
  unsigned long long* o_ll = nullptr;     // the rows as {fp32, epoch} words (a slot of an exchange)
  unsigned long long* lse_ll = nullptr;
  const unsigned long long* q_ll = nullptr;   // peer: the query inbox ({payload, epoch} words)
  const uint64_t* epoch_base = nullptr;
  uint64_t epoch_rel = 0;
  bool skip_combine = false;
  pkv_exchange* home = nullptr;   // set: publish q, wait for the peers and merge in the same kernel
  uint32_t wait_mask = 0;
};

constexpr int kStages = 3;    // 16-bit pools: 3 K slots + 3 V slots of 32 KiB
constexpr int kStagesQ = 6;   // 1-byte pools: 6 + 6 slots of 16 KiB
constexpr int kWphQ = 2;      // 1-byte pools: two consumer warps per kv-head, alternate tiles
using L16 = pkv::SmemLayout<kStages, 2>;
using L8 = pkv::SmemLayout<kStagesQ, 1>;

template <typename K>
int set_smem(K kernel, int bytes) {
  PKV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return PKV_OK;
}

int set_kernel_attrs() {
  int rc = set_smem(pkv::decode_partial_kernel<pkv::kKvBF16, true, kStages, 1>, L16::kTotal);
  if (!rc) rc = set_smem(pkv::decode_partial_kernel<pkv::kKvF16, false, kStages, 1>, L16::kTotal);
  if (!rc) rc = set_smem(pkv::decode_partial_kernel<pkv::kKvInt8, true, kStagesQ, kWphQ>, L8::kTotal);
  if (!rc) rc = set_smem(pkv::decode_partial_kernel<pkv::kKvInt8, false, kStagesQ, kWphQ>, L8::kTotal);
  if (!rc) rc = set_smem(pkv::decode_partial_kernel<pkv::kKvFp8, true, kStagesQ, kWphQ>, L8::kTotal);
  if (!rc) rc = set_smem(pkv::decode_partial_kernel<pkv::kKvFp8, false, kStagesQ, kWphQ>, L8::kTotal);
  return rc;
}
constexpr uint64_t kWaitNs = 2000000000ull;  // bound of every cross-GPU device-side wait

int launch_decode(pkv_shard* s, const pkv_decode_args* a, const LaunchOut& lo, cudaStream_t st) {
  int rc = check_args(s, a);
  if (rc) return rc;
  if (a->batch == 0) return PKV_OK;
  DeviceGuard guard(s->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", s->device);
  if (!s->attr_set) {
    rc = set_kernel_attrs();
    if (rc) return rc;
    s->attr_set = true;
  }
  const pkv_kv_view& kv = a->kv;
  const int n_hb = (kv.n_kv_heads + pkv::kHeadsPerCta - 1) / pkv::kHeadsPerCta;
  const int n_cta_x = s->num_sms / n_hb > 0 ? s->num_sms / n_hb : 1;
  if (n_cta_x > pkv::kMaxCtas)
    return fail(PKV_E_UNSUPPORTED, "%d CTAs per head block exceed the kernel's %d", n_cta_x, pkv::kMaxCtas);

  pkv::DecodeParams p;
  memset(&p, 0, sizeof p);
  p.q = a->q;
  p.block_table = a->block_table;
  p.seq_lens = a->seq_lens;
  p.bt_stride = a->block_table_stride;
  p.n_pages = kv.n_pages;
  p.batch = a->batch;
  p.n_q_heads = a->n_q_heads;
  p.n_kv_heads = kv.n_kv_heads;
  p.group = a->n_q_heads / kv.n_kv_heads;
  p.page_size = kv.page_size;
  p.tiles_per_page = (kv.page_size + pkv::kTileTok - 1) / pkv::kTileTok;
  p.head_major = kv.head_stride >= kv.token_stride ? 1 : 0;
  p.n_cta_x = n_cta_x;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.part_o = s->part_o;
  p.part_ml = s->part_ml;
  p.status = s->status;
  p.q_ll = lo.q_ll;
  p.epoch_base = lo.epoch_base;
  p.epoch_rel = lo.epoch_rel;
  p.q_timeout_ns = kWaitNs;
  p.o_ll = lo.o_ll;
  p.lse_ll = lo.lse_ll;
  p.force_empty = kv.n_pages > 0 ? 0 : 1;
  p.trace = s->trace;
  p.stats = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(s->status) + 64);
  p.k_scale = kv.k_scale;
  p.v_scale = kv.v_scale;
  p.fuse = lo.skip_combine ? 0 : 1;
  p.out = lo.out;
  p.out_dtype = lo.out_dtype;
  p.o_part = lo.o_part;
  p.lse_part = lo.lse_part;
  p.seq_counter = s->counters + 64;
  p.grp_counter = s->counters + s->grp_counter_off;
  p.grp_slot0 = s->grp_slot0;
  p.sib_slot0 = s->grp_slot0 / pkv::kMaxWph;
  p.unit_slot0 = s->n_slots - s->max_batch;
  if (s->obs[0] && n_cta_x <= pkv::kMaxCtas) {
    p.obs_read = s->obs[s->obs_parity];
    p.obs_write = s->obs[s->obs_parity ^ 1];
    s->obs_parity ^= 1;
  }
  if (lo.home) {
    pkv_exchange* x = lo.home;
    p.mg_n = x->world;
    p.mg_self = x->rank;
    p.mg_wait_mask = lo.wait_mask & ~(1u << x->rank);
    p.mg_o = slot_o(x, x->rank, 0);
    p.mg_lse = slot_lse(x, x->rank, 0);
    p.mg_o_stride = (int64_t)x->o_part_elems;
    p.mg_lse_stride = (int64_t)x->lse_part_elems;
    p.mg_timeout_ns = kWaitNs;
    p.mg_status = x->status;
    for (int r = 0; r < x->world; ++r) {
      if (r == x->rank) continue;
      p.pub_ll[p.pub_n++] = q_inbox(x, r);
    }
  }

  Range range(lo.home ? "pkv:home_step(publish+partial+merge)" : lo.q_ll ? "pkv:peer_step(partial)" : "pkv:decode");
  // An empty pool goes through the same kernel: every sequence counts as empty, no tile is
  // ever loaded (the zeroed tensor maps are not touched), and the service warps write the
  // neutral rows (O = 0, lse = -inf) or, on the home GPU, the merge of the peers' rows.
  CUtensorMap tk, tv;
  memset(&tk, 0, sizeof tk);
  memset(&tv, 0, sizeof tv);
  if (kv.n_pages > 0) {
    rc = build_map(s, kv.k, kv, &tk);
    if (rc) return rc;
    rc = build_map(s, kv.v, kv, &tv);
    if (rc) return rc;
  }
  dim3 grid(n_cta_x, n_hb);
  const dim3 block(pkv::cta_threads(is_quant(kv.dtype) ? kWphQ : 1));
  const bool qbf = a->q_dtype == PKV_BF16;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = is_quant(kv.dtype) ? L8::kTotal : L16::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddepcontrol.wait in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  switch (kv.dtype) {
    case PKV_BF16: PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvBF16, true, kStages, 1>, tk, tv, p)); break;
    case PKV_F16: PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvF16, false, kStages, 1>, tk, tv, p)); break;
    case PKV_INT8:
      if (qbf) PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvInt8, true, kStagesQ, kWphQ>, tk, tv, p));
      else     PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvInt8, false, kStagesQ, kWphQ>, tk, tv, p));
      break;
    default:
      if (qbf) PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvFp8, true, kStagesQ, kWphQ>, tk, tv, p));
      else     PKV_CUDA(cudaLaunchKernelEx(&cfg, pkv::decode_partial_kernel<pkv::kKvFp8, false, kStagesQ, kWphQ>, tk, tv, p));
      break;
  }
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;   // the combine is fused into the kernel's tail
}

int read_status(int device, uint32_t* dev_word, cudaStream_t st, uint32_t* out) {
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  uint32_t v = 0;
  PKV_CUDA(cudaMemcpyAsync(&v, dev_word, sizeof v, cudaMemcpyDeviceToHost, st));
  PKV_CUDA(cudaStreamSynchronize(st));
  if (v) {
    PKV_CUDA(cudaMemsetAsync(dev_word, 0, sizeof v, st));
    PKV_CUDA(cudaStreamSynchronize(st));
  }
  if (out) *out = v;
  return PKV_OK;
}

}  // namespace

extern "C" {

const char* pkv_last_error(void) { return g_err.c_str(); }
int pkv_abi_version(void) { return PKV_ABI_VERSION; }

int pkv_shard_create(pkv_shard** out, int device, int max_batch, int n_q_heads) {
  if (!out) return fail(PKV_E_INVALID, "null out");
  if (max_batch <= 0 || max_batch > pkv::kMaxBatch)
    return fail(PKV_E_INVALID, "max_batch %d outside [1, %d]", max_batch, pkv::kMaxBatch);
  if (n_q_heads <= 0 || n_q_heads > 1024) return fail(PKV_E_INVALID, "n_q_heads %d", n_q_heads);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  int sms = 0, major = 0;
  PKV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  PKV_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10)
    return fail(PKV_E_UNSUPPORTED, "device %d has compute capability %d.x; this library is sm_100a only",
                device, major);
  pkv_shard* s = new pkv_shard();
  s->device = device;
  s->num_sms = sms;
  s->max_batch = max_batch;
  s->n_q_heads = n_q_heads;
  s->grp_slot0 = (sms + max_batch) * pkv::kMaxWph;                 // per-CTA slots, then per-group slots
  // ... then per-group slots (CTA group + sequence), then one slot per sequence for the home GPU's own fold
  s->n_slots = s->grp_slot0 + (sms + pkv::kGroupCtas - 1) / pkv::kGroupCtas + max_batch + max_batch;
  s->maps.reserve(kMapCache);
  const size_t o_bytes = (size_t)s->n_slots * n_q_heads * pkv::kHeadDim * sizeof(float);
  const size_t ml_bytes = (size_t)s->n_slots * n_q_heads * 2 * sizeof(float);
  cudaError_t e = cudaMalloc(&s->part_o, o_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&s->part_ml, ml_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&s->status, 256);
  if (e == cudaSuccess) e = cudaMemset(s->status, 0, 256);
  s->grp_counter_off = 64 + (size_t)n_q_heads * max_batch;
  s->n_counter_words = s->grp_counter_off +
                       (size_t)(pkv::kMaxCtas / pkv::kGroupCtas + max_batch) * n_q_heads;   // n_kv_heads <= n_q_heads
  const size_t obs_words = 1 + 3 * pkv::kMaxCtas;
  if (e == cudaSuccess) e = cudaMalloc(&s->counters, (s->n_counter_words + 2 * obs_words) * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(s->counters, 0, (s->n_counter_words + 2 * obs_words) * sizeof(unsigned int));
  s->obs[0] = s->counters + s->n_counter_words;
  s->obs[1] = s->obs[0] + obs_words;
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    pkv_shard_destroy(s);
    return fail(PKV_E_CUDA, "scratch allocation failed: %s", cudaGetErrorString(e));
  }
  *out = s;
  return PKV_OK;
}

int pkv_shard_destroy(pkv_shard* s) {
  if (!s) return PKV_OK;
  DeviceGuard guard(s->device);
  cudaFree(s->part_o);
  cudaFree(s->part_ml);
  cudaFree(s->status);
  cudaFree(s->counters);
  delete s;
  return PKV_OK;
}

int pkv_shard_status(pkv_shard* s, void* stream, uint32_t* status_out) {
  if (!s) return fail(PKV_E_INVALID, "null shard");
  uint32_t v = 0;
  int rc = read_status(s->device, s->status, static_cast<cudaStream_t>(stream), &v);
  if (rc) return rc;
  if (v) {
    // a wait gave up mid-kernel: the arrival counters may be left half-counted
    DeviceGuard guard(s->device);
    PKV_CUDA(cudaMemsetAsync(s->counters, 0, s->n_counter_words * sizeof(unsigned int),
                             static_cast<cudaStream_t>(stream)));
    PKV_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  }
  if (status_out) *status_out = v;
  return PKV_OK;
}

int pkv_shard_stats(pkv_shard* s, void* stream, uint64_t* launches_out, uint64_t* units_out) {
  if (!s) return fail(PKV_E_INVALID, "null shard");
  DeviceGuard guard(s->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", s->device);
  unsigned long long v[2] = {0, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PKV_CUDA(cudaMemcpyAsync(v, reinterpret_cast<uint8_t*>(s->status) + 64, sizeof v, cudaMemcpyDeviceToHost, st));
  PKV_CUDA(cudaStreamSynchronize(st));
  if (launches_out) *launches_out = v[0];
  if (units_out) *units_out = v[1];
  return PKV_OK;
}

int pkv_decode_partial(pkv_shard* s, const pkv_decode_args* a, float* o_part, float* lse_part,
                       void* stream) {
  if (!o_part || !lse_part) return fail(PKV_E_INVALID, "null o_part or lse_part");
  LaunchOut lo;
  lo.o_part = o_part;
  lo.lse_part = lse_part;
  return launch_decode(s, a, lo, static_cast<cudaStream_t>(stream));
}

int pkv_decode(pkv_shard* s, const pkv_decode_args* a, void* out, int32_t out_dtype,
               float* lse_out, void* stream) {
  if (!out) return fail(PKV_E_INVALID, "null out");
  if (out_dtype != PKV_F16 && out_dtype != PKV_BF16 && out_dtype != PKV_F32)
    return fail(PKV_E_INVALID, "out_dtype %d", out_dtype);
  LaunchOut lo;
  lo.out = out;
  lo.out_dtype = out_dtype;
  lo.lse_part = lse_out;
  return launch_decode(s, a, lo, static_cast<cudaStream_t>(stream));
}

int pkv_decode_splits_only(pkv_shard* s, const pkv_decode_args* a, void* stream) {
  LaunchOut lo;
  lo.skip_combine = true;
  return launch_decode(s, a, lo, static_cast<cudaStream_t>(stream));
}

int pkv_merge_partials(int device, const float* o_parts, int64_t o_part_stride,
                       const float* lse_parts, int64_t lse_part_stride, int32_t n_parts,
                       int32_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                       float* lse_out, void* stream) {
  if (!o_parts || !lse_parts || !out) return fail(PKV_E_INVALID, "null pointer");
  if (head_dim != pkv::kHeadDim) return fail(PKV_E_UNSUPPORTED, "head_dim %d: 128 required", head_dim);
  if (n_parts <= 0 || rows < 0) return fail(PKV_E_INVALID, "n_parts %d rows %d", n_parts, rows);
  if (out_dtype != PKV_F16 && out_dtype != PKV_BF16 && out_dtype != PKV_F32)
    return fail(PKV_E_INVALID, "out_dtype %d", out_dtype);
  if (rows == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv::MergeParams m;
  memset(&m, 0, sizeof m);
  m.o_parts = o_parts; m.lse_parts = lse_parts;
  m.o_stride = o_part_stride; m.lse_stride = lse_part_stride;
  m.n_parts = n_parts; m.rows = rows;
  m.out = out; m.out_dtype = out_dtype; m.lse_out = lse_out;
  Range range("pkv:merge");
  pkv::merge_partials_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(m);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_quantize_kv(int device, const void* src, int32_t src_dtype, int64_t rows, void* codes,
                    void* scales, int32_t fmt, void* stream) {
  if (!src || !codes || !scales) return fail(PKV_E_INVALID, "null pointer");
  if (!is_16bit(src_dtype)) return fail(PKV_E_INVALID, "src_dtype must be PKV_F16 or PKV_BF16");
  if (!is_quant(fmt)) return fail(PKV_E_INVALID, "fmt must be PKV_INT8 or PKV_FP8_E4M3");
  if (rows < 0 || rows > (int64_t)0x7fffffff * 8) return fail(PKV_E_INVALID, "rows %lld", (long long)rows);
  if (rows == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  const unsigned int blocks = static_cast<unsigned int>((rows + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (src_dtype == PKV_BF16)
    pkv::quantize_kv_kernel<true><<<blocks, 256, 0, st>>>(src, rows, static_cast<uint8_t*>(codes),
                                                          static_cast<__half*>(scales), fmt);
  else
    pkv::quantize_kv_kernel<false><<<blocks, 256, 0, st>>>(src, rows, static_cast<uint8_t*>(codes),
                                                           static_cast<__half*>(scales), fmt);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}


int pkv_split_block_table(int device, const int32_t* block_table, int64_t block_table_stride,
                          const int32_t* seq_lens, int32_t batch, int32_t page_size,
                          int32_t n_dev, int32_t mode, const int64_t* bases,
                          int32_t* const* out_tables, int64_t out_stride,
                          int32_t* const* out_lens, void* stream) {
  if (!block_table || !seq_lens || !out_tables || !out_lens) return fail(PKV_E_INVALID, "null pointer");
  if (n_dev < 1 || n_dev > pkv::kMaxWorld) return fail(PKV_E_INVALID, "n_dev %d", n_dev);
  if (mode != 0 && mode != 1) return fail(PKV_E_INVALID, "mode %d", mode);
  if (mode == 0 && !bases) return fail(PKV_E_INVALID, "mode 0 needs bases");
  if (page_size <= 0 || batch < 0) return fail(PKV_E_INVALID, "page_size %d batch %d", page_size, batch);
  if (batch == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv::SplitParams p;
  memset(&p, 0, sizeof p);
  p.block_table = block_table; p.seq_lens = seq_lens; p.bt_stride = block_table_stride;
  p.batch = batch; p.page_size = page_size; p.n_dev = n_dev; p.mode = mode;
  p.out_stride = out_stride;
  for (int d = 0; d < n_dev; ++d) {
    p.bases[d] = bases ? bases[d] : 0;
    if (!out_tables[d] || !out_lens[d]) return fail(PKV_E_INVALID, "null output for device %d", d);
    p.out_table[d] = out_tables[d];
    p.out_lens[d] = out_lens[d];
  }
  pkv::split_block_table_kernel<<<dim3(batch, n_dev), 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_prefill_partial(int device, const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                        const void* k, const void* v, int64_t kv_stride_b, int64_t kv_stride_h,
                        int64_t kv_stride_s, int32_t batch, int32_t n_q_heads, int32_t n_kv_heads, int32_t sq,
                        int32_t sk, int32_t head_dim, int32_t dtype, float scale, int32_t causal,
                        int64_t q_pos0, int64_t k_pos0, float* o_part, float* lse_part, void* stream) {
  if (!q || !o_part || !lse_part) return fail(PKV_E_INVALID, "null pointer");
  if (head_dim != pkv::kHeadDim) return fail(PKV_E_UNSUPPORTED, "head_dim %d: the kernels require 128", head_dim);
  if (!is_16bit(dtype)) return fail(PKV_E_INVALID, "dtype must be PKV_F16 or PKV_BF16");
  if (batch < 0 || sq < 0 || sk < 0 || n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads)
    return fail(PKV_E_INVALID, "batch %d sq %d sk %d heads %d/%d", batch, sq, sk, n_q_heads, n_kv_heads);
  if (batch > 65535 || n_q_heads > 65535) return fail(PKV_E_UNSUPPORTED, "batch and heads must fit a grid dimension");
  if (sk > 0 && (!k || !v)) return fail(PKV_E_INVALID, "null k or v");
  if ((q_stride_b | q_stride_h | q_stride_s | kv_stride_b | kv_stride_h | kv_stride_s) % 8)
    return fail(PKV_E_INVALID, "strides must be multiples of 8 elements (16 bytes)");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return fail(PKV_E_INVALID, "q, k and v must be 16-byte aligned");
  if (batch == 0 || sq == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  static bool attr_done[64] = {};
  if (device < 64 && !attr_done[device]) {
    PKV_CUDA(cudaFuncSetAttribute(pkv::prefill_partial_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pkv::kPfSmem));
    PKV_CUDA(cudaFuncSetAttribute(pkv::prefill_partial_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pkv::kPfSmem));
    attr_done[device] = true;
  }
  pkv::PrefillParams p;
  memset(&p, 0, sizeof p);
  p.q = q; p.k = k; p.v = v;
  p.q_sb = q_stride_b; p.q_sh = q_stride_h; p.q_ss = q_stride_s;
  p.kv_sb = kv_stride_b; p.kv_sh = kv_stride_h; p.kv_ss = kv_stride_s;
  p.n_q_heads = n_q_heads; p.group = n_q_heads / n_kv_heads; p.sq = sq; p.sk = sk;
  p.causal = causal ? 1 : 0; p.q_pos0 = q_pos0; p.k_pos0 = k_pos0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o_part = o_part; p.lse_part = lse_part;
  Range range("pkv:prefill_partial");
  const dim3 grid((sq + pkv::kPfRows - 1) / pkv::kPfRows, n_q_heads, batch);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PKV_BF16) pkv::prefill_partial_kernel<true><<<grid, pkv::kPfThreads, pkv::kPfSmem, st>>>(p);
  else                   pkv::prefill_partial_kernel<false><<<grid, pkv::kPfThreads, pkv::kPfSmem, st>>>(p);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_stage_peer_blocks(int device, const int32_t* block_table, int64_t block_table_stride,
                          const int32_t* seq_lens, int32_t batch, int32_t block_size, int32_t n_dev,
                          const int64_t* bases, const int64_t* n_blocks, const void* const* k_pools,
                          const void* const* v_pools, const int64_t* page_strides, void* k_home, void* v_home,
                          int64_t home_page_stride, int64_t c_local, int64_t c_scratch, int64_t block_elems,
                          int32_t elem_size, int32_t* out_table, int32_t* scratch_words, uint32_t* status_word,
                          void* stream) {
  if (!block_table || !seq_lens || !bases || !n_blocks || !k_pools || !v_pools || !page_strides || !k_home ||
      !v_home || !out_table || !scratch_words || !status_word)
    return fail(PKV_E_INVALID, "null pointer");
  if (n_dev < 2 || n_dev > pkv::kMaxWorld) return fail(PKV_E_INVALID, "n_dev %d (the home GPU and at least one peer)", n_dev);
  if (batch < 0 || block_size <= 0 || c_local < 0 || c_scratch < 0 || elem_size <= 0)
    return fail(PKV_E_INVALID, "batch %d block_size %d c_local %lld c_scratch %lld", batch, block_size,
                (long long)c_local, (long long)c_scratch);
  if ((block_elems * elem_size) % 16 || (home_page_stride * elem_size) % 16 ||
      ((reinterpret_cast<uintptr_t>(k_home) | reinterpret_cast<uintptr_t>(v_home)) & 15))
    return fail(PKV_E_INVALID, "blocks must be multiples of 16 bytes and 16-byte aligned");
  if (bases[1] != c_local) return fail(PKV_E_INVALID, "bases[1] must equal c_local");
  if (batch == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv::StageParams p;
  memset(&p, 0, sizeof p);
  p.block_table = block_table; p.seq_lens = seq_lens; p.out_table = out_table; p.row_count = scratch_words;
  p.bt_stride = block_table_stride; p.batch = batch; p.block_size = block_size; p.n_dev = n_dev;
  p.c_local = c_local; p.c_scratch = c_scratch;
  for (int d = 0; d < n_dev; ++d) {
    p.bases[d] = bases[d]; p.n_blocks[d] = n_blocks[d];
    if (d == 0) continue;
    if (!k_pools[d] || !v_pools[d]) return fail(PKV_E_INVALID, "null pool for device %d", d);
    if ((page_strides[d] * elem_size) % 16 ||
        ((reinterpret_cast<uintptr_t>(k_pools[d]) | reinterpret_cast<uintptr_t>(v_pools[d])) & 15))
      return fail(PKV_E_INVALID, "pool %d: blocks must be 16-byte aligned", d);
    p.k_pool[d] = static_cast<const uint4*>(k_pools[d]); p.v_pool[d] = static_cast<const uint4*>(v_pools[d]);
    p.page_stride16[d] = page_strides[d] * elem_size / 16;
  }
  p.k_home = static_cast<uint4*>(k_home); p.v_home = static_cast<uint4*>(v_home);
  p.home_page_stride16 = home_page_stride * elem_size / 16;
  p.block_words16 = block_elems * elem_size / 16;
  p.status = status_word;
  Range range("pkv:stage_peer_blocks(copy-back)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pkv::stage_count_kernel<<<batch, 256, 0, st>>>(p);
  pkv::stage_copy_kernel<<<batch, 256, 0, st>>>(p);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_enable_peer_access(int device, int peer_device) {
  if (device == peer_device) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  int can = 0;
  PKV_CUDA(cudaDeviceCanAccessPeer(&can, device, peer_device));
  if (!can) return fail(PKV_E_UNSUPPORTED, "device %d cannot access device %d", device, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
  else if (e != cudaSuccess)
    return fail(PKV_E_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", peer_device, cudaGetErrorString(e));
  return PKV_OK;
}

int pkv_kv_append(int device, const void* key, const void* value, int64_t kv_token_stride,
                  const int64_t* slot_mapping, int32_t n_tokens, int32_t n_kv_heads, int32_t head_dim,
                  int32_t block_size, int32_t n_dev, const int64_t* bases, const int64_t* n_blocks,
                  void* const* k_pools, void* const* v_pools, const int64_t* page_strides,
                  const int64_t* token_strides, const int64_t* head_strides, uint32_t* status_word,
                  void* stream) {
  if (!key || !value || !slot_mapping || !bases || !n_blocks || !k_pools || !v_pools || !page_strides ||
      !token_strides || !head_strides)
    return fail(PKV_E_INVALID, "null pointer");
  if (head_dim != pkv::kHeadDim) return fail(PKV_E_UNSUPPORTED, "head_dim %d: 128 required", head_dim);
  if (n_dev < 1 || n_dev > pkv::kMaxWorld) return fail(PKV_E_INVALID, "n_dev %d", n_dev);
  if (n_tokens < 0 || n_kv_heads <= 0 || block_size <= 0)
    return fail(PKV_E_INVALID, "n_tokens %d n_kv_heads %d block_size %d", n_tokens, n_kv_heads, block_size);
  if (kv_token_stride % 4 || ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 7))
    return fail(PKV_E_INVALID, "key / value rows must be 8-byte aligned");
  if (n_tokens == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv::AppendParams p;
  memset(&p, 0, sizeof p);
  p.key = key; p.value = value; p.slot_mapping = slot_mapping; p.kv_token_stride = kv_token_stride;
  p.n_tokens = n_tokens; p.n_kv_heads = n_kv_heads; p.block_size = block_size; p.n_dev = n_dev;
  p.status = status_word;
  for (int d = 0; d < n_dev; ++d) {
    if (!k_pools[d] || !v_pools[d]) return fail(PKV_E_INVALID, "null pool for device %d", d);
    if (d > 0 && bases[d] < bases[d - 1]) return fail(PKV_E_INVALID, "bases must ascend");
    if (page_strides[d] % 4 || token_strides[d] % 4 || head_strides[d] % 4 ||
        ((reinterpret_cast<uintptr_t>(k_pools[d]) | reinterpret_cast<uintptr_t>(v_pools[d])) & 7))
      return fail(PKV_E_INVALID, "pool %d: strides and bases must keep rows 8-byte aligned", d);
    p.bases[d] = bases[d]; p.n_blocks[d] = n_blocks[d];
    p.k_pool[d] = static_cast<uint16_t*>(k_pools[d]); p.v_pool[d] = static_cast<uint16_t*>(v_pools[d]);
    p.page_stride[d] = page_strides[d]; p.token_stride[d] = token_strides[d]; p.head_stride[d] = head_strides[d];
  }
  const int64_t units = (int64_t)n_tokens * n_kv_heads;
  pkv::kv_append_kernel<<<static_cast<unsigned int>((units + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------- //
// several GPUs
// ------------------------------------------------------------------------- //
extern "C" {

int pkv_exchange_create(pkv_exchange** out, int device, int rank, int world, int max_batch,
                        int n_q_heads) {
  if (!out) return fail(PKV_E_INVALID, "null out");
  if (world < 1 || world > pkv::kMaxWorld || rank < 0 || rank >= world)
    return fail(PKV_E_INVALID, "rank %d / world %d (max %d)", rank, world, pkv::kMaxWorld);
  if (max_batch <= 0 || max_batch > pkv::kMaxBatch || n_q_heads <= 0)
    return fail(PKV_E_INVALID, "max_batch %d n_q_heads %d", max_batch, n_q_heads);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv_exchange* x = new pkv_exchange();
  x->device = device; x->rank = rank; x->world = world;
  x->max_batch = max_batch; x->n_q_heads = n_q_heads;
  x->o_part_elems = (size_t)max_batch * n_q_heads * pkv::kHeadDim;
  x->lse_part_elems = align_up((size_t)max_batch * n_q_heads, 64);
  x->off_q = 0;
  x->off_o = align_up((size_t)max_batch * n_q_heads * (pkv::kHeadDim / 2) * 8, 256);   // 4 payload bytes per 8-byte word
  x->off_lse = x->off_o + align_up(world * x->o_part_elems * 8, 256);
  x->off_probe = x->off_lse + align_up(world * x->lse_part_elems * 8, 256);   // one flag for pkv_exchange_hop_probe
  x->slab_bytes = x->off_probe + 256;
  cudaError_t e = cudaMalloc(&x->slab, x->slab_bytes);
  if (e == cudaSuccess) e = cudaMemset(x->slab, 0, x->slab_bytes);
  const size_t status_bytes = 512;   // status word, epoch base at byte 128
  if (e == cudaSuccess) e = cudaMalloc(&x->status, status_bytes);
  if (e == cudaSuccess) e = cudaMemset(x->status, 0, status_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    pkv_exchange_destroy(x);
    return fail(PKV_E_CUDA, "mailbox allocation failed: %s", cudaGetErrorString(e));
  }
  x->peer_slab[rank] = x->slab;
  *out = x;
  return PKV_OK;
}

int pkv_exchange_destroy(pkv_exchange* x) {
  if (!x) return PKV_OK;
  DeviceGuard guard(x->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < x->world; ++r)
    if (x->imported[r] && x->peer_slab[r]) cudaIpcCloseMemHandle(x->peer_slab[r]);
  cudaFree(x->slab);
  cudaFree(x->status);
  delete x;
  return PKV_OK;
}

int pkv_exchange_export(pkv_exchange* x, void* handle64) {
  if (!x || !handle64) return fail(PKV_E_INVALID, "null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  DeviceGuard guard(x->device);
  cudaIpcMemHandle_t h;
  PKV_CUDA(cudaIpcGetMemHandle(&h, x->slab));
  memcpy(handle64, &h, 64);
  return PKV_OK;
}

int pkv_exchange_import(pkv_exchange* x, int peer_rank, const void* handle64) {
  if (!x || !handle64) return fail(PKV_E_INVALID, "null pointer");
  if (peer_rank < 0 || peer_rank >= x->world || peer_rank == x->rank)
    return fail(PKV_E_INVALID, "peer_rank %d", peer_rank);
  DeviceGuard guard(x->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  PKV_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  x->peer_slab[peer_rank] = static_cast<uint8_t*>(p);
  x->imported[peer_rank] = true;
  return PKV_OK;
}

int pkv_exchange_attach(pkv_exchange* x, int peer_rank, pkv_exchange* peer) {
  if (!x || !peer) return fail(PKV_E_INVALID, "null pointer");
  if (peer_rank < 0 || peer_rank >= x->world || peer_rank == x->rank || peer->rank != peer_rank)
    return fail(PKV_E_INVALID, "peer_rank %d", peer_rank);
  if (peer->world != x->world || peer->max_batch != x->max_batch || peer->n_q_heads != x->n_q_heads)
    return fail(PKV_E_INVALID, "exchanges were created with different shapes");
  if (peer->device != x->device) {
    DeviceGuard guard(x->device);
    int can = 0;
    PKV_CUDA(cudaDeviceCanAccessPeer(&can, x->device, peer->device));
    if (!can) return fail(PKV_E_UNSUPPORTED, "device %d cannot access device %d", x->device, peer->device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
    else if (e != cudaSuccess)
      return fail(PKV_E_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", peer->device, cudaGetErrorString(e));
  }
  x->peer_slab[peer_rank] = peer->slab;
  return PKV_OK;
}

int pkv_exchange_status(pkv_exchange* x, void* stream, uint32_t* status_out) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  return read_status(x->device, x->status, static_cast<cudaStream_t>(stream), status_out);
}

int pkv_exchange_epoch(pkv_exchange* x, uint64_t* epoch_out) {
  if (!x || !epoch_out) return fail(PKV_E_INVALID, "null pointer");
  *epoch_out = x->epoch;
  return PKV_OK;
}

int pkv_exchange_resync(pkv_exchange* x, uint64_t epoch) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  if (x->capturing) return fail(PKV_E_STATE, "resync during a graph capture");
  if (epoch < x->epoch) return fail(PKV_E_INVALID, "epochs only grow: %llu < %llu",
                                    (unsigned long long)epoch, (unsigned long long)x->epoch);
  x->epoch = epoch;
  return PKV_OK;
}

int pkv_exchange_capture_begin(pkv_exchange* x) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  if (x->capturing) return fail(PKV_E_STATE, "capture already begun");
  x->capturing = true;
  x->cap_epoch0 = x->epoch;
  return PKV_OK;
}

int pkv_exchange_capture_end(pkv_exchange* x, void* stream, uint64_t* steps_out) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  if (!x->capturing) return fail(PKV_E_STATE, "no capture begun");
  DeviceGuard guard(x->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", x->device);
  const uint64_t steps = x->epoch - x->cap_epoch0;
  // last node of the captured step: the next replay's epochs start where this one's end
  pkv::bump_epoch_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch_base_dev(x), steps);
  PKV_CUDA(cudaGetLastError());
  x->capturing = false;
  x->cap_steps = steps;
  x->epoch = x->cap_epoch0;     // nothing has run yet: a capture only records
  if (steps_out) *steps_out = steps;
  return PKV_OK;
}

int pkv_exchange_replayed(pkv_exchange* x) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  if (x->capturing || !x->cap_steps) return fail(PKV_E_STATE, "no captured step to account for");
  x->epoch += x->cap_steps;
  x->base_host += x->cap_steps;
  return PKV_OK;
}

namespace {
int check_step(pkv_exchange* x, const pkv_decode_args* a) {
  if (a->batch <= 0 || a->batch > x->max_batch)
    return fail(PKV_E_INVALID, "batch %d outside [1, %d]", a->batch, x->max_batch);
  if (a->n_q_heads != x->n_q_heads) return fail(PKV_E_INVALID, "n_q_heads mismatch");
  return PKV_OK;
}
}  // namespace

// Every step entry point validates first, launches, and only then commits the new epoch:
// a call that fails leaves the exchange where it was.
int pkv_home_publish_q(pkv_exchange* x, const void* q, int32_t batch, void* stream) {
  if (!x || !q) return fail(PKV_E_INVALID, "null pointer");
  if (batch <= 0 || batch > x->max_batch) return fail(PKV_E_INVALID, "batch %d", batch);
  if (reinterpret_cast<uintptr_t>(q) & 15) return fail(PKV_E_INVALID, "q must be 16-byte aligned");
  pkv::PublishParams p;
  memset(&p, 0, sizeof p);
  p.q = static_cast<const uint4*>(q);
  p.batch = batch;
  p.row16 = x->n_q_heads * (pkv::kHeadDim * 2 / 16);
  p.epoch_base = epoch_base_dev(x);
  p.epoch_rel = x->epoch + 1 - x->base_host;
  int n = 0;
  for (int r = 0; r < x->world; ++r) {
    if (r == x->rank) continue;
    if (!x->peer_slab[r]) return fail(PKV_E_STATE, "rank %d is not attached", r);
    p.dst[n++] = q_inbox(x, r);
  }
  if (n > 0) {
    DeviceGuard guard(x->device);
    if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", x->device);
    Range range("pkv:publish_q");
    pkv::publish_q_kernel<<<n, 1024, 0, static_cast<cudaStream_t>(stream)>>>(p);
    PKV_CUDA(cudaGetLastError());
  }
  x->epoch += 1;
  return PKV_OK;
}

int pkv_peer_step(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, int32_t home_rank,
                  int32_t q_override, void* stream) {
  if (!x || !s || !a) return fail(PKV_E_INVALID, "null pointer");
  if (home_rank < 0 || home_rank >= x->world || home_rank == x->rank)
    return fail(PKV_E_INVALID, "home_rank %d", home_rank);
  if (!x->peer_slab[home_rank]) return fail(PKV_E_STATE, "home rank %d is not attached", home_rank);
  int rc = check_step(x, a);
  if (rc) return rc;
  pkv_decode_args aa = *a;
  LaunchOut lo;
  lo.epoch_base = epoch_base_dev(x);
  lo.epoch_rel = x->epoch + 1 - x->base_host;
  if (!q_override) {
    aa.q = x->slab + x->off_q;           // not read: the kernel takes the rows from the inbox words
    lo.q_ll = q_inbox(x, x->rank);
  }
  lo.o_ll = slot_o(x, home_rank, x->rank);
  lo.lse_ll = slot_lse(x, home_rank, x->rank);
  rc = launch_decode(s, &aa, lo, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  x->epoch += 1;
  return PKV_OK;
}

int pkv_home_partial(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, void* stream) {
  if (!x || !s || !a) return fail(PKV_E_INVALID, "null pointer");
  int rc = check_step(x, a);
  if (rc) return rc;
  LaunchOut lo;
  lo.epoch_base = epoch_base_dev(x);          // the step pkv_home_publish_q has begun
  lo.epoch_rel = x->epoch - x->base_host;
  lo.o_ll = slot_o(x, x->rank, x->rank);
  lo.lse_ll = slot_lse(x, x->rank, x->rank);
  return launch_decode(s, a, lo, static_cast<cudaStream_t>(stream));
}

int pkv_home_step(pkv_exchange* x, pkv_shard* s, const pkv_decode_args* a, uint32_t wait_mask,
                  void* out, int32_t out_dtype, float* lse_out, void* stream) {
  if (!x || !s || !a || !out) return fail(PKV_E_INVALID, "null pointer");
  int rc = check_step(x, a);
  if (rc) return rc;
  if (out_dtype != PKV_F16 && out_dtype != PKV_BF16 && out_dtype != PKV_F32)
    return fail(PKV_E_INVALID, "out_dtype %d", out_dtype);
  if (reinterpret_cast<uintptr_t>(a->q) & 15) return fail(PKV_E_INVALID, "q must be 16-byte aligned");
  for (int r = 0; r < x->world; ++r)
    if (!x->peer_slab[r]) return fail(PKV_E_STATE, "rank %d is not attached", r);
  LaunchOut lo;
  lo.out = out;
  lo.out_dtype = out_dtype;
  lo.lse_part = lse_out;
  lo.home = x;
  lo.wait_mask = wait_mask;
  lo.epoch_base = epoch_base_dev(x);
  lo.epoch_rel = x->epoch + 1 - x->base_host;
  rc = launch_decode(s, a, lo, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  x->epoch += 1;
  return PKV_OK;
}

int pkv_home_merge(pkv_exchange* x, int32_t batch, uint32_t wait_mask, void* out,
                   int32_t out_dtype, float* lse_out, void* stream) {
  if (!x || !out) return fail(PKV_E_INVALID, "null pointer");
  if (batch <= 0 || batch > x->max_batch) return fail(PKV_E_INVALID, "batch %d", batch);
  if (out_dtype != PKV_F16 && out_dtype != PKV_BF16 && out_dtype != PKV_F32)
    return fail(PKV_E_INVALID, "out_dtype %d", out_dtype);
  DeviceGuard guard(x->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", x->device);
  pkv::MergeParams m;
  memset(&m, 0, sizeof m);
  m.o_ll = slot_o(x, x->rank, 0);
  m.lse_ll = slot_lse(x, x->rank, 0);
  m.o_stride = (int64_t)x->o_part_elems;
  m.lse_stride = (int64_t)x->lse_part_elems;
  m.n_parts = x->world;
  m.rows = batch * x->n_q_heads;
  m.out = out; m.out_dtype = out_dtype; m.lse_out = lse_out;
  m.wait_mask = wait_mask | (1u << x->rank);
  m.epoch_base = epoch_base_dev(x);
  m.epoch_rel = x->epoch - x->base_host;
  m.timeout_ns = kWaitNs;
  m.status = x->status;
  Range range("pkv:home_merge(wait+merge)");
  pkv::merge_partials_kernel<<<(m.rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(m);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_exchange_hop_probe(pkv_exchange* x, int32_t peer_rank, int32_t role, int32_t iters, int32_t payload_bytes,
                           uint64_t* out, void* stream) {
  if (!x || !out) return fail(PKV_E_INVALID, "null pointer");
  if (peer_rank < 0 || peer_rank >= x->world || peer_rank == x->rank || !x->peer_slab[peer_rank])
    return fail(PKV_E_STATE, "rank %d is not an attached peer", peer_rank);
  if (role < 0 || role > 3 || iters <= 0 || iters > 1000000) return fail(PKV_E_INVALID, "role %d iters %d", role, iters);
  const int ll = role >> 1;
  role &= 1;
  const size_t inbox = (size_t)x->max_batch * x->n_q_heads * pkv::kHeadDim * 4;
  if (payload_bytes < 0 || payload_bytes % 512 || (size_t)payload_bytes > inbox || (ll && payload_bytes == 0))
    return fail(PKV_E_INVALID, "payload_bytes %d: a multiple of 512, at most the q inbox (%zu), not 0 with roles 2/3",
                payload_bytes, inbox);
  DeviceGuard guard(x->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", x->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pkv::hop_probe_kernel<<<1, 32, 0, st>>>(
      role, ll, iters, payload_bytes / 512, reinterpret_cast<uint4*>(x->peer_slab[peer_rank] + x->off_q),
      reinterpret_cast<const uint4*>(x->slab + x->off_q),
      reinterpret_cast<uint64_t*>(x->peer_slab[peer_rank] + x->off_probe),
      reinterpret_cast<const uint64_t*>(x->slab + x->off_probe), kWaitNs, reinterpret_cast<unsigned long long*>(out));
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_exchange_hop_probe_reset(pkv_exchange* x, void* stream) {
  if (!x) return fail(PKV_E_INVALID, "null exchange");
  DeviceGuard guard(x->device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", x->device);
  PKV_CUDA(cudaMemsetAsync(x->slab + x->off_probe, 0, 256, static_cast<cudaStream_t>(stream)));
  return PKV_OK;
}

int pkv_shard_trace(pkv_shard* s, uint64_t* buf) {
  if (!s) return fail(PKV_E_INVALID, "null shard");
  s->trace = reinterpret_cast<unsigned long long*>(buf);
  return PKV_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------- //
// pkv_decode_static: the same decode with its scratch in static device memory
// ------------------------------------------------------------------------- //
namespace {

constexpr int kStaticMaxBatch = 32;
constexpr int kStaticMaxQHeads = 64;
constexpr int kStaticMaxSms = 192;
constexpr int kStaticMaxDevices = 16;
constexpr size_t kStaticGrpSlot0 = (size_t)(kStaticMaxSms + kStaticMaxBatch) * pkv::kMaxWph;
constexpr size_t kStaticSlots = kStaticGrpSlot0 + kStaticMaxSms / pkv::kGroupCtas + 1 + 2 * kStaticMaxBatch;
constexpr size_t kStaticObsWords = 1 + 3 * pkv::kMaxCtas;
constexpr size_t kStaticGrpOff = 64 + (size_t)kStaticMaxBatch * kStaticMaxQHeads;    // relative to the counters
constexpr size_t kStaticWords = 64 + kStaticGrpOff +
    (size_t)(pkv::kMaxCtas / pkv::kGroupCtas + kStaticMaxBatch) * kStaticMaxQHeads;   // cleared per call

// One copy per GPU that loads the library, held until the process exits (16 MB).
// In host code these names are only handles for cudaGetSymbolAddress, never pointers.
static __device__ __align__(256) float g_static_part_o[kStaticSlots * kStaticMaxQHeads * pkv::kHeadDim];
static __device__ __align__(256) float g_static_part_ml[kStaticSlots * kStaticMaxQHeads * 2];
static __device__ __align__(256) unsigned int g_static_words[kStaticWords + 2 * kStaticObsWords];

pkv_shard g_static_shard[kStaticMaxDevices];
bool g_static_ready[kStaticMaxDevices];
std::mutex g_static_mutex;

// First call on a device: resolve the device addresses of the static arrays with that
// device current, and raise the kernels' shared-memory limit.
int static_setup(int device) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ready[device]) return PKV_OK;
  int sms = 0, major = 0;
  PKV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  PKV_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10)
    return fail(PKV_E_UNSUPPORTED, "device %d has compute capability %d.x; sm_100a only", device, major);
  if (sms > kStaticMaxSms)
    return fail(PKV_E_UNSUPPORTED, "device %d has %d SMs; the static scratch is sized for %d", device,
                sms, kStaticMaxSms);
  float *po = nullptr, *pml = nullptr;
  unsigned int* pw = nullptr;
  PKV_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&po), g_static_part_o));
  PKV_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&pml), g_static_part_ml));
  PKV_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&pw), g_static_words));
  pkv_shard& s = g_static_shard[device];
  s.device = device;
  s.num_sms = sms;
  s.max_batch = kStaticMaxBatch;
  s.n_q_heads = 0;                       // set per call
  s.n_slots = static_cast<int>(kStaticSlots);
  s.part_o = po;
  s.part_ml = pml;
  s.status = reinterpret_cast<uint32_t*>(pw);          // words [0, 64): status block
  s.counters = pw + 64;                                // 64 global words, then per (sequence, kv-head)
  s.n_counter_words = kStaticWords - 64;
  s.grp_counter_off = kStaticGrpOff;
  s.grp_slot0 = static_cast<int>(kStaticGrpSlot0);
  s.obs[0] = pw + kStaticWords;           // survive from call to call (not cleared)
  s.obs[1] = s.obs[0] + kStaticObsWords;
  s.cache_maps = false;                                // tensor maps are encoded on the stack
  { int rc = set_kernel_attrs(); if (rc) return rc; }
  s.attr_set = true;
  g_static_ready[device] = true;
  return PKV_OK;
}

}  // namespace

extern "C" int pkv_decode_static(int device, const pkv_decode_args* a, void* out, int32_t out_dtype,
                                 float* lse_out, void* stream) {
  if (!a || !out) return fail(PKV_E_INVALID, "null args or out");
  if (device < 0 || device >= kStaticMaxDevices) return fail(PKV_E_INVALID, "device %d", device);
  if (out_dtype != PKV_F16 && out_dtype != PKV_BF16 && out_dtype != PKV_F32)
    return fail(PKV_E_INVALID, "out_dtype %d", out_dtype);
  if (a->batch < 0 || a->batch > kStaticMaxBatch)
    return fail(PKV_E_INVALID, "batch %d exceeds the static scratch (at most %d sequences per call); "
                "use pkv_decode with a pkv_shard for larger batches", a->batch, kStaticMaxBatch);
  if (a->n_q_heads <= 0 || a->n_q_heads > kStaticMaxQHeads)
    return fail(PKV_E_INVALID, "n_q_heads %d exceeds the static scratch (at most %d query heads); "
                "use pkv_decode with a pkv_shard", a->n_q_heads, kStaticMaxQHeads);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  int rc = static_setup(device);
  if (rc) return rc;
  pkv_shard& s = g_static_shard[device];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The arrays keep whatever the previous call left: the arrival counters must start at
  // zero (a call that gave up on a wait may have left them half-counted).  The status
  // word is left alone: its bits stay until pkv_static_status reads them.
  PKV_CUDA(cudaMemsetAsync(s.counters, 0, s.n_counter_words * sizeof(unsigned int), st));
  std::lock_guard<std::mutex> lock(g_static_mutex);
  s.n_q_heads = a->n_q_heads;
  LaunchOut lo;
  lo.out = out;
  lo.out_dtype = out_dtype;
  lo.lse_part = lse_out;
  return launch_decode(&s, a, lo, st);
}

// ------------------------------------------------------------------------- //
// the small kernels of a decoder layer around the attention call
// ------------------------------------------------------------------------- //
extern "C" {

int pkv_add_rmsnorm(int device, void* x, const void* delta, const void* weight, void* out, int32_t rows,
                    int32_t hidden, float eps, int32_t dtype, void* stream) {
  if (!x || !weight || !out) return fail(PKV_E_INVALID, "null pointer");
  if (!is_16bit(dtype)) return fail(PKV_E_INVALID, "dtype must be PKV_F16 or PKV_BF16");
  if (rows < 0 || hidden <= 0 || hidden % 8 || hidden > 12000)
    return fail(PKV_E_INVALID, "rows %d hidden %d (a multiple of 8, at most 12000)", rows, hidden);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(PKV_E_INVALID, "pointers must be 16-byte aligned");
  if (rows == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  const size_t sm = (size_t)hidden * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PKV_BF16) pkv::add_rmsnorm_kernel<true><<<rows, 512, sm, st>>>(x, delta, weight, out, hidden, eps);
  else                   pkv::add_rmsnorm_kernel<false><<<rows, 512, sm, st>>>(x, delta, weight, out, hidden, eps);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_rope_append(int device, const void* qkv, const int64_t* positions, const float* inv_freq, int32_t batch,
                    int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, void* q_out, void* k_pool,
                    void* v_pool, int64_t page_stride, int64_t token_stride, int64_t head_stride,
                    const int64_t* pages, const int64_t* slots, int32_t dtype, void* stream) {
  if (!qkv || !positions || !inv_freq || !q_out) return fail(PKV_E_INVALID, "null pointer");
  if (!is_16bit(dtype)) return fail(PKV_E_INVALID, "dtype must be PKV_F16 or PKV_BF16");
  if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || head_dim % 2 || head_dim > 2048)
    return fail(PKV_E_INVALID, "batch %d heads %d/%d head_dim %d", batch, n_q_heads, n_kv_heads, head_dim);
  if ((k_pool || v_pool) && (!k_pool || !v_pool || !pages || !slots))
    return fail(PKV_E_INVALID, "an append needs k_pool, v_pool, pages and slots");
  if (batch == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  pkv::RopeParams p;
  memset(&p, 0, sizeof p);
  p.qkv = qkv; p.positions = positions; p.inv_freq = inv_freq; p.q_out = q_out;
  p.k_pool = k_pool; p.v_pool = v_pool; p.pages = pages; p.slots = slots;
  p.page_stride = page_stride; p.token_stride = token_stride; p.head_stride = head_stride;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
  const dim3 grid(batch, n_q_heads + 2 * n_kv_heads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PKV_BF16) pkv::rope_append_kernel<true><<<grid, head_dim / 2, 0, st>>>(p);
  else                   pkv::rope_append_kernel<false><<<grid, head_dim / 2, 0, st>>>(p);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

int pkv_swiglu(int device, const void* gate_up, void* out, int32_t rows, int32_t ffn, int32_t dtype, void* stream) {
  if (!gate_up || !out) return fail(PKV_E_INVALID, "null pointer");
  if (!is_16bit(dtype)) return fail(PKV_E_INVALID, "dtype must be PKV_F16 or PKV_BF16");
  if (rows < 0 || ffn <= 0 || ffn % 8) return fail(PKV_E_INVALID, "rows %d ffn %d (a multiple of 8)", rows, ffn);
  if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(PKV_E_INVALID, "pointers must be 16-byte aligned");
  if (rows == 0) return PKV_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  const int64_t n8 = (int64_t)rows * (ffn / 8);
  const unsigned int blocks = static_cast<unsigned int>((n8 + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PKV_BF16) pkv::swiglu_kernel<true><<<blocks, 256, 0, st>>>(gate_up, out, rows, ffn);
  else                   pkv::swiglu_kernel<false><<<blocks, 256, 0, st>>>(gate_up, out, rows, ffn);
  PKV_CUDA(cudaGetLastError());
  return PKV_OK;
}

}  // extern "C"

extern "C" int pkv_static_status(int device, void* stream, uint32_t* status_out) {
  if (device < 0 || device >= kStaticMaxDevices) return fail(PKV_E_INVALID, "device %d", device);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(PKV_E_CUDA, "cannot select device %d", device);
  int rc = static_setup(device);
  if (rc) return rc;
  return read_status(device, g_static_shard[device].status, static_cast<cudaStream_t>(stream), status_out);
}
