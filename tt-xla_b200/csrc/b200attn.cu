// Host side of the C ABI declared in include/b200attn.h: argument checks, tensor-map
// encoding and kernel launches.  Single translation unit; built for sm_100a only.
#include "../../include/b200attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <initializer_list>
#include <mutex>

#include "decode.cuh"
#include "decode_fp8.cuh"
#include "kv_scatter.cuh"
#include "prefill.cuh"
#include "rope_scatter.cuh"
#include "rowlinear_ar.cuh"
#include "step_metadata.cuh"

namespace b200attn {

static_assert(kDecTicketBytes == B200ATTN_DECODE_TICKET_BYTES, "header and kernels agree");

// Diagnostics block: code, pad, globaltimer stamp of the latest timeout (see ptx.cuh).
__device__ __align__(16) int g_err_word[4] = {0, 0, 0, 0};

// Work counters of the prefill kernel's dynamic item list: a launch uses word (tag % slots) and
// claims it by its tag (see prefill_draw), so nothing has to be cleared between launches.
__device__ unsigned long long g_pf_sched[kPfSchedSlots];
static std::atomic<uint32_t> g_pf_launch_seq{0};

// Split-KV scratch of b200attn_paged_decode_static.  In host code this name is only a handle
// for cudaGetSymbolAddress; kernels get the device address looked up below.
static __device__ __align__(256) unsigned char g_static_workspace[B200ATTN_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
#ifdef B200ATTN_PF_TRACE
static unsigned long long* g_pf_trace = nullptr;
#endif

struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int* err_word = nullptr;
  unsigned long long* pf_sched = nullptr;
};

static std::mutex g_mutex;
static DeviceInfo g_devices[kMaxDevices];
static void* g_static_workspace_addr[kMaxDevices] = {};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

// Per-device set-up on first use: SM count, address of the diagnostics word, and the
// driver's tensor-map encoder (looked up at run time so the library has no link-time
// dependency on libcuda and still loads on a machine without a driver).
static int get_device(DeviceInfo** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return B200ATTN_ERR_NO_DEVICE;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_devices[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return B200ATTN_ERR_NO_DEVICE;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_err_word) != cudaSuccess) {
      cudaGetLastError();
      return B200ATTN_ERR_NO_DEVICE;
    }
    d.err_word = static_cast<int*>(p);
    if (cudaGetSymbolAddress(&p, g_pf_sched) != cudaSuccess) {
      cudaGetLastError();
      return B200ATTN_ERR_NO_DEVICE;
    }
    d.pf_sched = static_cast<unsigned long long*>(p);
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) !=
              cudaSuccess ||
          q != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        return B200ATTN_ERR_NO_DEVICE;
      }
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    d.ready = true;
  }
  *out = &d;
  return B200ATTN_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A serving loop encodes the same few tensor maps step after step (the caches and activation
// buffers keep their addresses): the last few encodings are kept per host thread.
struct MapKey {
  const void* base;
  uint64_t rows, cols, row_stride;
  uint32_t box_rows, kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && row_stride == o.row_stride &&
           box_rows == o.box_rows && kind == o.kind;
  }
};
constexpr int kMapCacheSize = 16;
struct MapCache {
  MapKey keys[kMapCacheSize];
  CUtensorMap maps[kMapCacheSize];
  int used = 0, next = 0;
  bool find(const MapKey& k, CUtensorMap* out) const {
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) {
        *out = maps[i];
        return true;
      }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    keys[next] = k;
    maps[next] = m;
    next = (next + 1) % kMapCacheSize;
    if (used < kMapCacheSize) ++used;
  }
};
static thread_local MapCache t_map_cache;

// bf16 matrix [rows, cols] with `row_stride` elements between rows; boxes of
// [box_rows x 64 columns] land in shared memory with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                    uint64_t row_stride, uint32_t box_rows) {
  const MapKey key{base, rows, cols, row_stride, box_rows, 0u};
  if (t_map_cache.find(key, map)) return B200ATTN_OK;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return B200ATTN_ERR_TENSOR_MAP;
  t_map_cache.put(key, *map);
  return B200ATTN_OK;
}

// e4m3 cache [rows, 128] (one byte per element): boxes of [box_rows x 128 bytes], 128-byte swizzle.
static int make_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  const MapKey key{base, rows, 128, 128, box_rows, 1u};
  if (t_map_cache.find(key, map)) return B200ATTN_OK;
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return B200ATTN_ERR_TENSOR_MAP;
  t_map_cache.put(key, *map);
  return B200ATTN_OK;
}

// The opt-in to more than 48 KiB of dynamic shared memory is a per-kernel, per-device setting:
// made once, not before every launch.
template <typename Kernel>
static cudaError_t allow_dynamic_smem(Kernel kern, int bytes, bool* done_for_device) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (done_for_device[dev]) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done_for_device[dev] = true;
  return e;
}

static int check_cache_geometry(int num_kv_heads, int head_size, int block_size,
                                int64_t num_blocks) {
  if (num_kv_heads <= 0 || num_blocks <= 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (head_size != 64 && head_size != 128) return B200ATTN_ERR_UNSUPPORTED;
  if (block_size != 32 && block_size != 64) return B200ATTN_ERR_UNSUPPORTED;
  if (num_blocks * num_kv_heads * block_size > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  return B200ATTN_OK;
}

// ------------------------------------------------------------------------------ scatter
static int launch_scatter(int mode, ScatterParams& p, int head_size, void* stream) {
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (!p.k_cache || !p.v_cache || !p.k_new || !p.v_new) return B200ATTN_ERR_NULL_POINTER;
  if (!aligned16(p.k_cache) || !aligned16(p.v_cache) || !aligned16(p.k_new) ||
      !aligned16(p.v_new))
    return B200ATTN_ERR_MISALIGNED;
  p.vec_per_head = head_size / 8;
  p.err_word = dev->err_word;
  if (p.num_tokens == 0) return B200ATTN_OK;
  const int64_t total = p.num_tokens * p.num_kv_heads * p.vec_per_head;
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(dev->sm_count) * 8;  // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (mode) {
    case kScatterSlots:
      kv_scatter_kernel<kScatterSlots><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
      break;
    case kScatterUpdate:
      kv_scatter_kernel<kScatterUpdate><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
      break;
    default:
      kv_scatter_kernel<kScatterFill><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
      break;
  }
  return static_cast<int>(cudaGetLastError());
}

static int fill_scatter_common(ScatterParams& p, void* k_cache, void* v_cache, const void* k_new,
                               const void* v_new, int64_t new_token_stride, int num_kv_heads,
                               int head_size, int block_size, int64_t num_blocks,
                               int cache_dtype = B200ATTN_CACHE_BF16) {
  if (cache_dtype != B200ATTN_CACHE_BF16 && cache_dtype != B200ATTN_CACHE_FP8_E4M3)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (int rc = check_cache_geometry(num_kv_heads, head_size, block_size, num_blocks)) return rc;
  if (new_token_stride < static_cast<int64_t>(num_kv_heads) * head_size)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (new_token_stride % 8 != 0) return B200ATTN_ERR_MISALIGNED;
  p = ScatterParams{};
  p.k_cache = static_cast<uint4*>(k_cache);
  p.v_cache = static_cast<uint4*>(v_cache);
  p.k_new = static_cast<const uint4*>(k_new);
  p.v_new = static_cast<const uint4*>(v_new);
  p.new_token_stride_v = new_token_stride / 8;
  p.cache_fp8 = cache_dtype == B200ATTN_CACHE_FP8_E4M3;
  p.num_kv_heads = num_kv_heads;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  return B200ATTN_OK;
}

template <int HD, int BS, int STAGES>
static int launch_decode(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p,
                         int num_users, cudaStream_t s) {
  using L = DecodeSmem<HD, BS, STAGES>;
  auto kern = paged_decode_splitkv_kernel<HD, BS, STAGES>;
  static bool smem_allowed[kMaxDevices] = {};
  cudaError_t e = allow_dynamic_smem(kern, L::kTotalBytes, smem_allowed);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(p.num_splits, p.num_kv_heads, num_users);
  kern<<<grid, kDecThreads, L::kTotalBytes, s>>>(tk, tv, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (p.num_splits > 1 && !p.tickets) {
    dim3 cgrid(p.num_q_heads, num_users);
    decode_combine_kernel<HD><<<cgrid, HD, 0, s>>>(p);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

template <int BS, int STAGES>
static int launch_decode_fp8(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p,
                             int num_users, cudaStream_t s) {
  using L = DecodeFp8Smem<BS, STAGES>;
  auto kern = paged_decode_fp8_kernel<BS, STAGES>;
  static bool smem_allowed[kMaxDevices] = {};
  cudaError_t e = allow_dynamic_smem(kern, L::kTotalBytes, smem_allowed);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(p.num_splits, p.num_kv_heads, num_users);
  kern<<<grid, kDecThreads, L::kTotalBytes, s>>>(tk, tv, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (p.num_splits > 1 && !p.tickets) {
    dim3 cgrid(p.num_q_heads, num_users);
    decode_combine_kernel<128><<<cgrid, 128, 0, s>>>(p);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

template <int HD, int BS, bool WIN>
static int launch_prefill_win(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const PrefillParams& p, int sm_count, cudaStream_t s) {
  using L = PrefillSmem<HD>;
  auto kern = prefill_tcgen05_kernel<HD, BS, WIN>;
  static bool smem_allowed[kMaxDevices] = {};
  cudaError_t e = allow_dynamic_smem(kern, L::kTotalBytes, smem_allowed);
  if (e != cudaSuccess) return static_cast<int>(e);
  // persistent: one CTA per SM (the kernel holds all of an SM's shared and tensor memory)
  dim3 grid(static_cast<unsigned>(p.total_items < sm_count ? p.total_items : sm_count));
  kern<<<grid, kPfThreads, L::kTotalBytes, s>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

// The sliding-window variant is a separate instantiation, so full causal attention carries none
// of its masking or bookkeeping.
template <int HD, int BS>
static int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const PrefillParams& p, int sm_count, cudaStream_t s) {
  return p.window > 0 ? launch_prefill_win<HD, BS, true>(tq, tk, tv, p, sm_count, s)
                      : launch_prefill_win<HD, BS, false>(tq, tk, tv, p, sm_count, s);
}

template <int NB, int S, int W>
static int launch_rowlinear(const CUtensorMap& tw, const CUtensorMap& tx, const RowLinearParams& p,
                            int tiles, cudaStream_t s) {
  using L = RowLinearSmem<NB>;
  auto kern = rowlinear_allreduce_kernel<NB, S, W>;
  static bool smem_allowed[kMaxDevices] = {};
  cudaError_t e = allow_dynamic_smem(kern, L::kTotalBytes, smem_allowed);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(S, static_cast<unsigned>(tiles), 1);
  cfg.blockDim = dim3(kRlThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kTotalBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Programmatic dependent launch: CTAs may start (and fetch weights) while the kernel before
  // drains; the kernel waits for that kernel's completion before it touches anything else.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  // Every cluster has to be resident at once (a CTA waits for the same CTA on its peers); the
  // answer depends only on the instantiation, so it is asked once.
  static int max_clusters[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int resident = 0;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (max_clusters[dev] == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_UNSUPPORTED;
      }
      max_clusters[dev] = n > 0 ? n : -1;
    }
    resident = max_clusters[dev];
  }
  if (resident < tiles) return B200ATTN_ERR_TOO_LARGE;
  e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return static_cast<int>(e);
}

template <int NB, int W>
static int launch_rowlinear_w(int split, const CUtensorMap& tw, const CUtensorMap& tx,
                              const RowLinearParams& p, int tiles, cudaStream_t s) {
  switch (split) {
    case 8: return launch_rowlinear<NB, 8, W>(tw, tx, p, tiles, s);
    case 4: return launch_rowlinear<NB, 4, W>(tw, tx, p, tiles, s);
    case 2: return launch_rowlinear<NB, 2, W>(tw, tx, p, tiles, s);
    default: return launch_rowlinear<NB, 1, W>(tw, tx, p, tiles, s);
  }
}

// the instantiation whose source-rank loops are the shortest that cover the call's world size
template <int NB>
static int launch_rowlinear_nb(int split, const CUtensorMap& tw, const CUtensorMap& tx,
                               const RowLinearParams& p, int tiles, cudaStream_t s) {
  if (p.world <= 2) return launch_rowlinear_w<NB, 2>(split, tw, tx, p, tiles, s);
  if (p.world <= 4) return launch_rowlinear_w<NB, 4>(split, tw, tx, p, tiles, s);
  return launch_rowlinear_w<NB, 8>(split, tw, tx, p, tiles, s);
}

}  // namespace b200attn

using namespace b200attn;

extern "C" {

int b200attn_version(void) { return B200ATTN_VERSION; }

const char* b200attn_status_string(int status) {
  switch (status) {
    case B200ATTN_OK: return "ok";
    case B200ATTN_ERR_NULL_POINTER: return "a required pointer is NULL";
    case B200ATTN_ERR_UNSUPPORTED:
      return "unsupported geometry (head_size must be 64 or 128, block_size 32 or 64, "
             "q heads per kv head <= 16 for decode)";
    case B200ATTN_ERR_MISALIGNED: return "pointer or stride is not 16-byte aligned";
    case B200ATTN_ERR_WORKSPACE: return "decode workspace missing or too small";
    case B200ATTN_ERR_BAD_ARGUMENT: return "bad argument (negative size or inconsistent head counts)";
    case B200ATTN_ERR_NO_DEVICE: return "no usable CUDA device (this library has no CPU path)";
    case B200ATTN_ERR_TENSOR_MAP: return "the driver refused the TMA tensor map for this layout";
    case B200ATTN_ERR_TOO_LARGE: return "size beyond the supported maximum";
    default:
      if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
      return "unknown status";
  }
}

int b200attn_paged_update_cache(void* k_cache, void* v_cache, const void* k_new,
                                const void* v_new, int64_t new_token_stride,
                                const int32_t* update_indices, const int32_t* page_table,
                                int64_t page_table_stride, int page_table_width, int num_users,
                                int num_kv_heads, int head_size, int block_size,
                                int64_t num_blocks, void* stream) {
  return b200attn_paged_update_cache_ex(
      k_cache, v_cache, k_new, v_new, new_token_stride, update_indices, page_table,
      page_table_stride, page_table_width, num_users, num_kv_heads, head_size, block_size,
      num_blocks, B200ATTN_CACHE_BF16, stream);
}

int b200attn_paged_update_cache_ex(void* k_cache, void* v_cache, const void* k_new,
                                const void* v_new, int64_t new_token_stride,
                                const int32_t* update_indices, const int32_t* page_table,
                                int64_t page_table_stride, int page_table_width, int num_users,
                                int num_kv_heads, int head_size, int block_size,
                                int64_t num_blocks, int cache_dtype, void* stream) {
  if (num_users < 0 || page_table_width <= 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (!update_indices || !page_table) return B200ATTN_ERR_NULL_POINTER;
  ScatterParams p;
  if (int rc = fill_scatter_common(p, k_cache, v_cache, k_new, v_new, new_token_stride,
                                   num_kv_heads, head_size, block_size, num_blocks, cache_dtype))
    return rc;
  p.positions = update_indices;
  p.page_table = page_table;
  p.page_table_stride = page_table_stride;
  p.page_table_width = page_table_width;
  p.num_tokens = num_users;
  return launch_scatter(kScatterUpdate, p, head_size, stream);
}

int b200attn_paged_fill_cache(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                              int64_t new_token_stride, const int32_t* fill_page_table,
                              int64_t page_table_stride, int page_table_width,
                              const int32_t* batch_idx, int num_users, int tokens_per_user,
                              int num_kv_heads, int head_size, int block_size,
                              int64_t num_blocks, void* stream) {
  return b200attn_paged_fill_cache_ex(
      k_cache, v_cache, k_new, v_new, new_token_stride, fill_page_table, page_table_stride,
      page_table_width, batch_idx, num_users, tokens_per_user, num_kv_heads, head_size,
      block_size, num_blocks, B200ATTN_CACHE_BF16, stream);
}

int b200attn_paged_fill_cache_ex(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                              int64_t new_token_stride, const int32_t* fill_page_table,
                              int64_t page_table_stride, int page_table_width,
                              const int32_t* batch_idx, int num_users, int tokens_per_user,
                              int num_kv_heads, int head_size, int block_size,
                              int64_t num_blocks, int cache_dtype, void* stream) {
  if (num_users < 0 || tokens_per_user < 0 || page_table_width <= 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (!fill_page_table) return B200ATTN_ERR_NULL_POINTER;
  if ((static_cast<int64_t>(tokens_per_user) + block_size - 1) / block_size > page_table_width)
    return B200ATTN_ERR_BAD_ARGUMENT;
  ScatterParams p;
  if (int rc = fill_scatter_common(p, k_cache, v_cache, k_new, v_new, new_token_stride,
                                   num_kv_heads, head_size, block_size, num_blocks, cache_dtype))
    return rc;
  p.page_table = fill_page_table;
  p.page_table_stride = page_table_stride;
  p.page_table_width = page_table_width;
  p.batch_idx = batch_idx;
  p.tokens_per_user = tokens_per_user > 0 ? tokens_per_user : 1;
  p.num_tokens = static_cast<int64_t>(num_users) * tokens_per_user;
  return launch_scatter(kScatterFill, p, head_size, stream);
}

int b200attn_kv_scatter_slots(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                              int64_t new_token_stride, const int64_t* slot_mapping,
                              int num_tokens, int num_kv_heads, int head_size, int block_size,
                              int64_t num_blocks, void* stream) {
  return b200attn_kv_scatter_slots_ex(
      k_cache, v_cache, k_new, v_new, new_token_stride, slot_mapping, num_tokens, num_kv_heads,
      head_size, block_size, num_blocks, B200ATTN_CACHE_BF16, stream);
}

int b200attn_kv_scatter_slots_ex(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                              int64_t new_token_stride, const int64_t* slot_mapping,
                              int num_tokens, int num_kv_heads, int head_size, int block_size,
                              int64_t num_blocks, int cache_dtype, void* stream) {
  if (num_tokens < 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (!slot_mapping) return B200ATTN_ERR_NULL_POINTER;
  ScatterParams p;
  if (int rc = fill_scatter_common(p, k_cache, v_cache, k_new, v_new, new_token_stride,
                                   num_kv_heads, head_size, block_size, num_blocks, cache_dtype))
    return rc;
  p.slot_mapping = slot_mapping;
  p.num_tokens = num_tokens;
  return launch_scatter(kScatterSlots, p, head_size, stream);
}

int b200attn_dequant_pages_fp8(void* k_dst, void* v_dst, const void* k_cache, const void* v_cache,
                               const int32_t* page_table, int64_t page_table_stride,
                               int page_table_width, const int32_t* cu_q, const int32_t* q_start,
                               int num_seqs, int num_kv_heads, int head_size, int block_size,
                               int64_t num_blocks, void* stream) {
  if (!k_dst || !v_dst || !k_cache || !v_cache || !page_table || !cu_q)
    return B200ATTN_ERR_NULL_POINTER;
  if (num_seqs < 0 || page_table_width <= 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (int rc = check_cache_geometry(num_kv_heads, head_size, block_size, num_blocks)) return rc;
  if (!aligned16(k_dst) || !aligned16(v_dst) || !aligned16(k_cache) || !aligned16(v_cache))
    return B200ATTN_ERR_MISALIGNED;
  if (static_cast<int64_t>(num_seqs) * page_table_width * num_kv_heads * block_size > 0x7fffffffLL)
    return B200ATTN_ERR_TOO_LARGE;
  if (num_seqs > 65535) return B200ATTN_ERR_TOO_LARGE;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (num_seqs == 0) return B200ATTN_OK;
  DequantPagesParams p{};
  p.k_src = static_cast<const uint8_t*>(k_cache);
  p.v_src = static_cast<const uint8_t*>(v_cache);
  p.k_dst = static_cast<__nv_bfloat16*>(k_dst);
  p.v_dst = static_cast<__nv_bfloat16*>(v_dst);
  p.page_table = page_table;
  p.page_table_stride = page_table_stride;
  p.page_table_width = page_table_width;
  p.cu_q = cu_q;
  p.q_start = q_start;
  p.block_size = block_size;
  p.page_elems = num_kv_heads * block_size * head_size;
  p.num_blocks = num_blocks;
  p.err_word = dev->err_word;
  dim3 grid(static_cast<unsigned>(page_table_width), static_cast<unsigned>(num_seqs));
  dequant_pages_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int b200attn_build_step_metadata(const int32_t* num_computed, const int32_t* num_scheduled,
                                 const int32_t* block_table, int64_t block_table_stride,
                                 int num_requests, int rows, int page_table_width,
                                 int fill_page_table_width, int tokens_per_row, int block_size,
                                 int32_t* cache_position, int32_t* page_table,
                                 int32_t* fill_page_table, int64_t* slot_mapping, void* stream) {
  if (!num_computed || !num_scheduled || !block_table || !cache_position || !page_table ||
      !fill_page_table || !slot_mapping)
    return B200ATTN_ERR_NULL_POINTER;
  if (num_requests < 0 || rows < num_requests || page_table_width <= 0 ||
      fill_page_table_width <= 0 || fill_page_table_width > page_table_width ||
      tokens_per_row <= 0 || block_size <= 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (rows == 0) return B200ATTN_OK;
  StepMetadataParams p{num_computed, num_scheduled, block_table, block_table_stride,
                       num_requests, rows, page_table_width, fill_page_table_width,
                       tokens_per_row, block_size, cache_position, page_table, fill_page_table,
                       slot_mapping};
  build_step_metadata_kernel<<<static_cast<unsigned>(rows), 128, 0,
                               static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int b200attn_rope_kv_scatter_slots(void* q, int64_t q_stride, void* k, int64_t k_stride,
                                   const void* v, int64_t v_stride, const int64_t* positions,
                                   const float* inv_freq, int rotary_dim, int is_neox_style,
                                   void* k_cache, void* v_cache, const int64_t* slot_mapping,
                                   int num_tokens, int num_q_heads, int num_kv_heads,
                                   int head_size, int block_size, int64_t num_blocks,
                                   void* stream) {
  if (!q || !k || !positions || !inv_freq) return B200ATTN_ERR_NULL_POINTER;
  if (slot_mapping && (!v || !k_cache || !v_cache)) return B200ATTN_ERR_NULL_POINTER;
  if (num_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (!is_neox_style) return B200ATTN_ERR_UNSUPPORTED;
  if (head_size != 64 && head_size != 128) return B200ATTN_ERR_UNSUPPORTED;
  if (rotary_dim <= 0 || rotary_dim > head_size || rotary_dim % 16 != 0)
    return B200ATTN_ERR_UNSUPPORTED;
  if (slot_mapping)
    if (int rc = check_cache_geometry(num_kv_heads, head_size, block_size, num_blocks)) return rc;
  if (!aligned16(q) || !aligned16(k) || (v && !aligned16(v)) || q_stride % 8 || k_stride % 8 ||
      (v && v_stride % 8) || (k_cache && !aligned16(k_cache)) || (v_cache && !aligned16(v_cache)))
    return B200ATTN_ERR_MISALIGNED;
  if (q_stride < static_cast<int64_t>(num_q_heads) * head_size ||
      k_stride < static_cast<int64_t>(num_kv_heads) * head_size)
    return B200ATTN_ERR_BAD_ARGUMENT;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (num_tokens == 0) return B200ATTN_OK;
  RopeScatterParams p{};
  p.q = static_cast<__nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.k = static_cast<__nv_bfloat16*>(k);
  p.k_stride = k_stride;
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.v_stride = v_stride;
  p.positions = positions;
  p.inv_freq = inv_freq;
  p.rotary_dim = rotary_dim;
  p.k_cache = static_cast<uint4*>(k_cache);
  p.v_cache = static_cast<uint4*>(v_cache);
  p.slot_mapping = slot_mapping;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.head_size = head_size;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.err_word = dev->err_word;
  rope_kv_scatter_kernel<<<static_cast<unsigned>(num_tokens), 256, 0,
                           static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// -------------------------------------------------------------------------------- decode
int b200attn_decode_auto_splits(int num_users, int num_kv_heads, int head_size,
                                int max_context_len) {
  if (num_users <= 0 || num_kv_heads <= 0 || max_context_len <= 0) return 1;
  int sm = 148;
  DeviceInfo* dev;
  if (get_device(&dev) == B200ATTN_OK) sm = dev->sm_count;
  // Cost model fitted to a sweep of split counts on B200 (20 batch shapes, times in
  // microseconds).  A launch costs ~6 us whatever it does; a CTA alone on its SM streams one
  // 64-token K+V tile (32 KiB at head_size 128) in ~0.54 us, and all CTAs together share
  // ~7.0 TB/s; the end of a launch is ragged in proportion to the longest CTA (a quarter of its
  // streaming time); CTAs beyond the resident set cost ~6 us per extra wave of start-up; more
  // than one split costs ~2 us for the merge by the last split to arrive plus ~0.1 us per split.
  const double tile_bytes = 2.0 * kDecTile * head_size * 2.0;
  const double bw = 7.0e6;                                   // bytes per us
  const int occ = head_size > 64 ? 2 : 3;                    // resident CTAs per SM
  // ... but never faster than ~0.45 us per tile: below 32 KiB a tile's time is the round trip of
  // its loads and barriers, not its bytes (head_size 64: 13.3 us with one split against 10.2 us
  // with four on eight users of up to 1024 tokens)
  const double t_bytes = 0.54 * tile_bytes / 32768.0;
  const double t_alone = t_bytes > 0.45 ? t_bytes : 0.45;
  const int64_t tiles = (max_context_len + kDecTile - 1) / kDecTile;
  const int64_t base = static_cast<int64_t>(num_users) * num_kv_heads;
  const double slots = static_cast<double>(occ) * sm;
  const int max_s = static_cast<int>(tiles < 128 ? tiles : 128);
  int best_s = 1;
  double best_t = 0.0;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t chunk = (tiles + s - 1) / s;
    const double ctas = static_cast<double>(base) * s;
    const double shared = ctas * chunk * tile_bytes / bw;
    const double alone = chunk * t_alone;
    double t = 6.0 + (shared > alone ? shared : alone) + 0.25 * alone;
    if (s > 1) t += 2.0 + 0.1 * s;
    if (ctas > slots) t += 6.0 * (ctas / slots - 1.0);
    if (s == 1 || t < best_t * 0.995) {
      best_t = t;
      best_s = s;
    }
  }
  return best_s;
}

size_t b200attn_decode_workspace_bytes(int num_users, int num_q_heads, int head_size,
                                       int num_splits) {
  if (num_splits <= 1 || num_users <= 0 || num_q_heads <= 0 || head_size <= 0) return 0;
  const size_t rows = static_cast<size_t>(num_users) * num_q_heads * num_splits;
  size_t o_bytes = rows * head_size * sizeof(float);
  o_bytes = (o_bytes + 255) & ~static_cast<size_t>(255);
  return kDecTicketBytes + o_bytes + rows * sizeof(float2);
}


int b200attn_paged_decode(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                          const void* k_cache, const void* v_cache, const int32_t* page_table,
                          int64_t page_table_stride, int page_table_width, const int32_t* cur_pos,
                          int num_users, int num_q_heads, int num_kv_heads, int head_size,
                          int block_size, int64_t num_blocks, float scale, int max_context_len,
                          int num_splits, void* workspace, size_t workspace_bytes, void* stream) {
  return b200attn_paged_decode_ex(out, out_row_stride, q, q_row_stride, k_cache, v_cache,
                                  page_table, page_table_stride, page_table_width, cur_pos,
                                  num_users, num_q_heads, num_kv_heads, head_size, block_size,
                                  num_blocks, scale, 0, nullptr, B200ATTN_CACHE_BF16,
                                  max_context_len, num_splits, workspace, workspace_bytes, stream);
}

int b200attn_paged_decode_ex(void* out, int64_t out_row_stride, const void* q,
                             int64_t q_row_stride, const void* k_cache, const void* v_cache,
                             const int32_t* page_table, int64_t page_table_stride,
                             int page_table_width, const int32_t* cur_pos, int num_users,
                             int num_q_heads, int num_kv_heads, int head_size, int block_size,
                             int64_t num_blocks, float scale, int sliding_window,
                             const float* sinks, int cache_dtype, int max_context_len,
                             int num_splits, void* workspace, size_t workspace_bytes,
                             void* stream) {
  return b200attn_paged_decode_step(out, out_row_stride, q, q_row_stride,
                                    const_cast<void*>(k_cache), const_cast<void*>(v_cache),
                                    nullptr, nullptr, 0, 1, page_table, page_table_stride,
                                    page_table_width, cur_pos, num_users, num_q_heads, num_kv_heads,
                                    head_size, block_size, num_blocks, scale, sliding_window, sinks,
                                    cache_dtype, max_context_len, num_splits, workspace,
                                    workspace_bytes, stream);
}

int b200attn_paged_decode_step(void* out, int64_t out_row_stride, const void* q,
                               int64_t q_row_stride, void* k_cache, void* v_cache,
                               const void* k_new, const void* v_new, int64_t new_token_stride,
                               int wrap_negative_positions, const int32_t* page_table,
                               int64_t page_table_stride, int page_table_width,
                               const int32_t* cur_pos, int num_users, int num_q_heads,
                               int num_kv_heads, int head_size, int block_size,
                               int64_t num_blocks, float scale, int sliding_window,
                               const float* sinks, int cache_dtype, int max_context_len,
                               int num_splits, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if ((k_new == nullptr) != (v_new == nullptr)) return B200ATTN_ERR_NULL_POINTER;
  if (k_new) {
    if (!aligned16(k_new) || !aligned16(v_new) || new_token_stride % 8 != 0)
      return B200ATTN_ERR_MISALIGNED;
    if (new_token_stride < static_cast<int64_t>(num_kv_heads) * head_size)
      return B200ATTN_ERR_BAD_ARGUMENT;
  }
  if (sliding_window < 0 || !(scale > 0.f)) return B200ATTN_ERR_BAD_ARGUMENT;
  if (cache_dtype != B200ATTN_CACHE_BF16 && cache_dtype != B200ATTN_CACHE_FP8_E4M3)
    return B200ATTN_ERR_BAD_ARGUMENT;
  const bool fp8 = cache_dtype == B200ATTN_CACHE_FP8_E4M3;
  if (fp8 && head_size != 128) return B200ATTN_ERR_UNSUPPORTED;
  if (!out || !q || !k_cache || !v_cache || !page_table || !cur_pos)
    return B200ATTN_ERR_NULL_POINTER;
  if (num_users < 0 || num_q_heads <= 0 || page_table_width <= 0 || num_splits < 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (num_splits > kDecMaxSplits) return B200ATTN_ERR_TOO_LARGE;
  if (int rc = check_cache_geometry(num_kv_heads, head_size, block_size, num_blocks)) return rc;
  if (num_q_heads % num_kv_heads != 0) return B200ATTN_ERR_BAD_ARGUMENT;
  const int group = num_q_heads / num_kv_heads;
  if (group > 16) return B200ATTN_ERR_UNSUPPORTED;
  if (!aligned16(out) || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) ||
      q_row_stride % 8 != 0 || out_row_stride % 8 != 0)
    return B200ATTN_ERR_MISALIGNED;
  if (q_row_stride < static_cast<int64_t>(num_q_heads) * head_size ||
      out_row_stride < static_cast<int64_t>(num_q_heads) * head_size)
    return B200ATTN_ERR_BAD_ARGUMENT;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (num_users == 0) return B200ATTN_OK;
  if (num_users > 65535 || num_kv_heads > 65535) return B200ATTN_ERR_TOO_LARGE;

  if (max_context_len <= 0) max_context_len = page_table_width * block_size;
  if (sliding_window > 0 && max_context_len > sliding_window + kDecTile)
    max_context_len = sliding_window + kDecTile;       // what a user streams at most
  if (num_splits == 0)
    num_splits = b200attn_decode_auto_splits(num_users, num_kv_heads, head_size, max_context_len);
  const size_t need = b200attn_decode_workspace_bytes(num_users, num_q_heads, head_size, num_splits);
  if (num_splits > 1 && (!workspace || workspace_bytes < need || !aligned16(workspace)))
    return B200ATTN_ERR_WORKSPACE;

  CUtensorMap tk, tv;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * num_kv_heads * block_size;
  if (fp8) {
    if (int rc = make_map_u8(&tk, k_cache, rows, block_size)) return rc;
    if (int rc = make_map_u8(&tv, v_cache, rows, block_size)) return rc;
  } else {
    if (int rc = make_map(&tk, k_cache, rows, head_size, head_size, block_size)) return rc;
    if (int rc = make_map(&tv, v_cache, rows, head_size, head_size, block_size)) return rc;
  }

  DecodeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_row_stride = q_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.page_table = page_table;
  p.page_table_stride = page_table_stride;
  p.page_table_width = page_table_width;
  p.cur_pos = cur_pos;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = group;
  p.num_splits = num_splits;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = sliding_window;
  p.sinks = sinks;
  p.k_new = static_cast<const uint4*>(k_new);
  p.v_new = static_cast<const uint4*>(v_new);
  p.new_token_stride_v = new_token_stride / 8;
  p.k_cache_w = static_cast<uint8_t*>(k_cache);
  p.v_cache_w = static_cast<uint8_t*>(v_cache);
  p.cache_fp8 = fp8 ? 1 : 0;
  p.wrap_negative = wrap_negative_positions ? 1 : 0;
  p.err_word = dev->err_word;
  if (num_splits > 1) {
    const size_t rows_p = static_cast<size_t>(num_users) * num_q_heads * num_splits;
    size_t o_bytes = rows_p * head_size * sizeof(float);
    o_bytes = (o_bytes + 255) & ~static_cast<size_t>(255);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    // One arrival counter per (user, KV head) when they fit the ticket region: the last split
    // to arrive merges the partials inside the same launch.  Larger batches fall back to the
    // separate combine launch.
    if (static_cast<size_t>(num_users) * num_kv_heads * sizeof(unsigned int) <= kDecTicketBytes)
      p.tickets = reinterpret_cast<unsigned int*>(ws);
    p.part_o = reinterpret_cast<float*>(ws + kDecTicketBytes);
    p.part_ml = reinterpret_cast<float2*>(ws + kDecTicketBytes + o_bytes);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fp8)
    return block_size == 64 ? launch_decode_fp8<64, 6>(tk, tv, p, num_users, s)
                            : launch_decode_fp8<32, 6>(tk, tv, p, num_users, s);
  if (head_size == 128 && block_size == 64) return launch_decode<128, 64, 3>(tk, tv, p, num_users, s);
  if (head_size == 128 && block_size == 32) return launch_decode<128, 32, 3>(tk, tv, p, num_users, s);
  if (head_size == 64 && block_size == 64) return launch_decode<64, 64, 4>(tk, tv, p, num_users, s);
  return launch_decode<64, 32, 4>(tk, tv, p, num_users, s);
}

// ------------------------------------------------------------------------------- prefill

int b200attn_prefill(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                     const void* k_src, const void* v_src, int kv_is_paged,
                     int64_t kv_token_stride, const int32_t* page_table,
                     int64_t page_table_stride, int page_table_width, const int32_t* cu_q,
                     const int32_t* cu_q_host, const int32_t* q_start, int num_seqs, int total_q,
                     int num_q_heads, int num_kv_heads, int head_size, int block_size,
                     int64_t num_blocks, float scale, void* stream) {
  return b200attn_prefill_ex(out, out_row_stride, q, q_row_stride, k_src, v_src, kv_is_paged,
                             kv_token_stride, page_table, page_table_stride, page_table_width,
                             cu_q, cu_q_host, q_start, num_seqs, total_q, num_q_heads,
                             num_kv_heads, head_size, block_size, num_blocks, scale, 0, stream);
}

int b200attn_prefill_ex(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                        const void* k_src, const void* v_src, int kv_is_paged,
                        int64_t kv_token_stride, const int32_t* page_table,
                        int64_t page_table_stride, int page_table_width, const int32_t* cu_q,
                        const int32_t* cu_q_host, const int32_t* q_start, int num_seqs,
                        int total_q, int num_q_heads, int num_kv_heads, int head_size,
                        int block_size, int64_t num_blocks, float scale, int sliding_window,
                        void* stream) {
  if (sliding_window < 0 || !(scale > 0.f)) return B200ATTN_ERR_BAD_ARGUMENT;
  if (!out || !q || !k_src || !v_src || !cu_q || !cu_q_host) return B200ATTN_ERR_NULL_POINTER;
  if (num_seqs < 0 || total_q < 0 || num_q_heads <= 0 || num_kv_heads <= 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (num_q_heads % num_kv_heads != 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (head_size != 64 && head_size != 128) return B200ATTN_ERR_UNSUPPORTED;
  if (!aligned16(out) || !aligned16(q) || !aligned16(k_src) || !aligned16(v_src) ||
      q_row_stride % 8 != 0 || out_row_stride % 8 != 0)
    return B200ATTN_ERR_MISALIGNED;
  if (q_row_stride < static_cast<int64_t>(num_q_heads) * head_size ||
      out_row_stride < static_cast<int64_t>(num_q_heads) * head_size)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (kv_is_paged) {
    if (!page_table || page_table_width <= 0) return B200ATTN_ERR_NULL_POINTER;
    if (int rc = check_cache_geometry(num_kv_heads, head_size, block_size, num_blocks)) return rc;
  } else {
    if (q_start) return B200ATTN_ERR_BAD_ARGUMENT;
    if (kv_token_stride % 8 != 0) return B200ATTN_ERR_MISALIGNED;
    if (kv_token_stride < static_cast<int64_t>(num_kv_heads) * head_size)
      return B200ATTN_ERR_BAD_ARGUMENT;
    if (block_size != 32 && block_size != 64) block_size = 64;  // unused by this form
  }
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (num_seqs == 0 || total_q == 0) return B200ATTN_OK;

  int total_tiles = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int len = cu_q_host[s + 1] - cu_q_host[s];
    if (len < 0) return B200ATTN_ERR_BAD_ARGUMENT;
    total_tiles += (len + kPfRowsPerItem - 1) / kPfRowsPerItem;
  }
  // rows are addressed absolutely (cu_q[s] + row), so the offsets must start at 0 and end inside q
  if (cu_q_host[0] != 0 || cu_q_host[num_seqs] > total_q) return B200ATTN_ERR_BAD_ARGUMENT;
  if (total_tiles == 0) return B200ATTN_OK;
  if (static_cast<int64_t>(total_tiles) * num_q_heads > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;

  CUtensorMap tq, tk, tv;
  if (int rc = make_map(&tq, q, total_q, static_cast<uint64_t>(num_q_heads) * head_size,
                        q_row_stride, kPfM))
    return rc;
  if (kv_is_paged) {
    const uint64_t rows = static_cast<uint64_t>(num_blocks) * num_kv_heads * block_size;
    if (int rc = make_map(&tk, k_src, rows, head_size, head_size, block_size)) return rc;
    if (int rc = make_map(&tv, v_src, rows, head_size, head_size, block_size)) return rc;
  } else {
    const uint64_t cols = static_cast<uint64_t>(num_kv_heads) * head_size;
    if (int rc = make_map(&tk, k_src, total_q, cols, kv_token_stride, kPfN)) return rc;
    if (int rc = make_map(&tv, v_src, total_q, cols, kv_token_stride, kPfN)) return rc;
  }

  PrefillParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.page_table = page_table;
  p.page_table_stride = page_table_stride;
  p.page_table_width = page_table_width;
  p.cu_q = cu_q;
  p.q_start = q_start;
  p.num_seqs = num_seqs;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_q_heads / num_kv_heads;
  p.kv_is_paged = kv_is_paged ? 1 : 0;
  p.window = sliding_window;
  p.total_items = total_tiles * num_q_heads;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err_word = dev->err_word;
  uint32_t tag = ++g_pf_launch_seq;
  if (tag == 0) tag = ++g_pf_launch_seq;      // 0 marks a clear counter word
  p.sched_tag = tag;
  p.sched = dev->pf_sched + tag % kPfSchedSlots;
#ifdef B200ATTN_PF_TRACE
  p.trace = g_pf_trace;
#endif
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (head_size == 128 && block_size == 64) return launch_prefill<128, 64>(tq, tk, tv, p, dev->sm_count, s);
  if (head_size == 128) return launch_prefill<128, 32>(tq, tk, tv, p, dev->sm_count, s);
  if (block_size == 64) return launch_prefill<64, 64>(tq, tk, tv, p, dev->sm_count, s);
  return launch_prefill<64, 32>(tq, tk, tv, p, dev->sm_count, s);
}

#ifdef B200ATTN_PF_TRACE
// Debug builds only: device buffer [CTAs][6][8] of cycle counters the prefill kernel fills.
void b200attn_debug_set_prefill_trace(unsigned long long* dev_buffer) { g_pf_trace = dev_buffer; }
#endif

int b200attn_paged_decode_static(void* out, int64_t out_row_stride, const void* q,
                                 int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                 const int32_t* page_table, int64_t page_table_stride,
                                 int page_table_width, const int32_t* cur_pos, int num_users,
                                 int num_q_heads, int num_kv_heads, int head_size, int block_size,
                                 int64_t num_blocks, float scale, int max_context_len,
                                 int num_splits, void* stream) {
  if (num_users < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_splits < 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (head_size != 64 && head_size != 128) return B200ATTN_ERR_UNSUPPORTED;
  if (page_table_width <= 0) return B200ATTN_ERR_BAD_ARGUMENT;
  if (num_splits > 0) {
    if (b200attn_decode_workspace_bytes(num_users, num_q_heads, head_size, num_splits) >
        B200ATTN_STATIC_WORKSPACE_BYTES)
      return B200ATTN_ERR_TOO_LARGE;
  } else {
    int ctx = max_context_len > 0 ? max_context_len : page_table_width * block_size;
    num_splits = b200attn_decode_auto_splits(num_users, num_kv_heads, head_size, ctx);
    while (num_splits > 1 &&
           b200attn_decode_workspace_bytes(num_users, num_q_heads, head_size, num_splits) >
               B200ATTN_STATIC_WORKSPACE_BYTES)
      --num_splits;
  }
  // Per-device set-up, once, with that device current: the device address of the array.
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return B200ATTN_ERR_NO_DEVICE;
  }
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_static_workspace_addr[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_static_workspace);
      if (e != cudaSuccess || !p) {
        cudaGetLastError();
        return e != cudaSuccess ? static_cast<int>(e) : B200ATTN_ERR_NO_DEVICE;
      }
      g_static_workspace_addr[dev] = p;
    }
    ws = g_static_workspace_addr[dev];
  }
  // The arrival counters this call uses must start at zero whatever an earlier (possibly
  // aborted) call left behind.
  if (num_splits > 1 && num_users > 0) {
    size_t n = static_cast<size_t>(num_users) * num_kv_heads * sizeof(unsigned int);
    if (n > kDecTicketBytes) n = kDecTicketBytes;
    cudaError_t e = cudaMemsetAsync(ws, 0, n, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return b200attn_paged_decode(out, out_row_stride, q, q_row_stride, k_cache, v_cache,
                               page_table, page_table_stride, page_table_width, cur_pos,
                               num_users, num_q_heads, num_kv_heads, head_size, block_size,
                               num_blocks, scale, max_context_len, num_splits, ws,
                               B200ATTN_STATIC_WORKSPACE_BYTES, stream);
}

int b200attn_read_error_word(int32_t* out_host, void* stream) {
  if (!out_host) return B200ATTN_ERR_NULL_POINTER;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(out_host, dev->err_word, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(dev->err_word, 0, sizeof(int), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && *out_host != 0) {
    // a launch that gave up may have left a prefill work counter half-way: clear them all
    e = cudaMemsetAsync(dev->pf_sched, 0, sizeof(unsigned long long) * kPfSchedSlots, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  }
  return static_cast<int>(e);
}

int b200attn_peek_error_word_async(int32_t* out_pinned_host, void* stream) {
  if (!out_pinned_host) return B200ATTN_ERR_NULL_POINTER;
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  return static_cast<int>(cudaMemcpyAsync(out_pinned_host, dev->err_word, sizeof(int),
                                          cudaMemcpyDeviceToHost,
                                          static_cast<cudaStream_t>(stream)));
}

// ------------------------------------------------------------------------------ row-parallel
// linear with fused all-reduce
static inline int rl_token_rows(int tokens) { return tokens <= 32 ? 32 : (tokens <= 64 ? 64 : 128); }

// bytes of one (parity, source rank) staging area: 8-byte units, one per bf16 pair
static inline size_t rl_area_bytes(int max_tokens, int max_n) {
  const size_t tiles = (static_cast<size_t>(max_n) + kRlTileN - 1) / kRlTileN;
  return tiles * rl_token_rows(max_tokens) * (kRlTileN * 8 / 2);
}

size_t b200attn_comm_bytes(int world, int max_tokens, int max_n) {
  if (world < 1 || world > kRlMaxWorld || max_tokens < 1 || max_tokens > kRlMaxTokens ||
      max_n < 8)
    return 0;
  return kRlStageOff + static_cast<size_t>(2) * (world + 1) * rl_area_bytes(max_tokens, max_n);
}

// K splits = CTAs per cluster: as many as keep every CTA resident and give each a K step.
static void rl_plan(int sm_count, int n_total, int k_local, int* tiles, int* k_steps, int* split,
                    int* per) {
  *tiles = (n_total + kRlTileN - 1) / kRlTileN;
  *k_steps = (k_local + kRlKStep - 1) / kRlKStep;
  *split = 1;
  *per = *k_steps;
  for (int cand : {8, 4, 2}) {
    const int c_per = (*k_steps + cand - 1) / cand;
    if (*tiles * cand <= sm_count && (cand - 1) * c_per < *k_steps) {
      *split = cand;
      *per = c_per;
      return;
    }
  }
}

int b200attn_rowlinear_plan(int num_tokens, int n_total, int k_local, int* token_rows,
                            int* k_splits) {
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (!token_rows || !k_splits) return B200ATTN_ERR_NULL_POINTER;
  if (num_tokens < 1 || num_tokens > kRlMaxTokens || n_total <= 0 || k_local <= 0)
    return B200ATTN_ERR_BAD_ARGUMENT;
  int tiles, k_steps, per;
  rl_plan(dev->sm_count, n_total, k_local, &tiles, &k_steps, k_splits, &per);
  *token_rows = rl_token_rows(num_tokens);
  return B200ATTN_OK;
}

int b200attn_comm_alloc(size_t bytes, void** dev_ptr) {
  if (!dev_ptr) return B200ATTN_ERR_NULL_POINTER;
  if (bytes < kRlStageOff) return B200ATTN_ERR_BAD_ARGUMENT;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    cudaGetLastError();
    return static_cast<int>(e);
  }
  *dev_ptr = p;
  return B200ATTN_OK;
}

int b200attn_comm_free(void* dev_ptr) {
  return dev_ptr ? static_cast<int>(cudaFree(dev_ptr)) : B200ATTN_OK;
}

int b200attn_comm_export(const void* dev_ptr, unsigned char* handle64) {
  if (!dev_ptr || !handle64) return B200ATTN_ERR_NULL_POINTER;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(e);
  }
  memcpy(handle64, &h, 64);
  return B200ATTN_OK;
}

int b200attn_comm_import(const unsigned char* handle64, void** peer_ptr) {
  if (!handle64 || !peer_ptr) return B200ATTN_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(e);
  }
  *peer_ptr = p;
  return B200ATTN_OK;
}

int b200attn_comm_close(void* peer_ptr) {
  return peer_ptr ? static_cast<int>(cudaIpcCloseMemHandle(peer_ptr)) : B200ATTN_OK;
}

int b200attn_rowlinear_allreduce(void* out, int64_t out_row_stride, const void* x,
                                 int64_t x_row_stride, const void* w, int64_t w_row_stride,
                                 int num_tokens, int n_total, int k_local, int rank, int world,
                                 void* const* comm_bufs, int max_tokens, int max_n,
                                 int reduce_mode, uint64_t peer_timeout_ns, void* stream) {
  DeviceInfo* dev;
  if (int rc = get_device(&dev)) return rc;
  if (!out || !x || !w) return B200ATTN_ERR_NULL_POINTER;
  if (num_tokens < 0 || n_total <= 0 || k_local <= 0 || world < 1 || world > kRlMaxWorld ||
      rank < 0 || rank >= world || reduce_mode < 0 || reduce_mode > 2)
    return B200ATTN_ERR_BAD_ARGUMENT;
  if (num_tokens > kRlMaxTokens) return B200ATTN_ERR_TOO_LARGE;
  if (num_tokens == 0) return B200ATTN_OK;
  if ((n_total & 7) || (k_local & 7) || (out_row_stride & 7) || (x_row_stride & 7) ||
      (w_row_stride & 7))
    return B200ATTN_ERR_UNSUPPORTED;
  if (!aligned16(out) || !aligned16(x) || !aligned16(w)) return B200ATTN_ERR_MISALIGNED;
  int tiles, k_steps, split, per;
  rl_plan(dev->sm_count, n_total, k_local, &tiles, &k_steps, &split, &per);
  if (tiles > dev->sm_count) return B200ATTN_ERR_TOO_LARGE;
  RowLinearParams p{};
  if (world > 1) {
    if (!comm_bufs) return B200ATTN_ERR_NULL_POINTER;
    if (num_tokens > max_tokens || n_total > max_n || max_tokens > kRlMaxTokens)
      return B200ATTN_ERR_WORKSPACE;
    for (int r = 0; r < world; ++r) {
      if (!comm_bufs[r]) return B200ATTN_ERR_NULL_POINTER;
      p.comm[r] = static_cast<uint8_t*>(comm_bufs[r]);
    }
  }
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.num_tokens = num_tokens;
  p.n_total = n_total;
  p.k_steps = k_steps;
  p.steps_per_split = per;
  p.rank = rank;
  p.world = world;
  p.src_stride = world > 1 ? rl_area_bytes(max_tokens, max_n) : 0;
  p.two_shot = reduce_mode == 0 ? (world > 2) : (reduce_mode == 2);
  p.peer_timeout_ns = peer_timeout_ns ? peer_timeout_ns : 1000ull * 1000 * 1000;
  p.err_word = dev->err_word;
  const int nb = rl_token_rows(num_tokens);
  CUtensorMap tw, tx;
  if (int rc = make_map(&tw, w, n_total, k_local, w_row_stride, kRlTileN)) return rc;
  if (int rc = make_map(&tx, x, num_tokens, k_local, x_row_stride, nb)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nb == 32) return launch_rowlinear_nb<32>(split, tw, tx, p, tiles, s);
  if (nb == 64) return launch_rowlinear_nb<64>(split, tw, tx, p, tiles, s);
  return launch_rowlinear_nb<128>(split, tw, tx, p, tiles, s);
}

}  // extern "C"
