// Paged GQA decode attention: split-KV streaming kernel + split combine.
//
// Grid (split, kv_head, user).  One CTA owns one KV head of one user and the G = nq/nkv
// query heads that share it, so every K/V byte is read from HBM once.  A producer warp walks
// the user's page-table slice and pulls one 64-token tile of K and V per stage into a
// shared-memory ring with TMA (128-byte swizzled boxes of [block_size x 64] elements, one
// mbarrier per stage).  Four consumer warps each take 16 tokens of the tile:
// S = Q.K^T and O += P.V run on mma.sync m16n8k16 with the G query rows padded to 16 (the
// kernel is HBM-bound; tensor throughput is irrelevant), the softmax is the online
// (running max / running sum) form in fp32 with warp-shuffle row reductions.  The four
// warps' partial (m, l, O) are merged through shared memory at the end, and the CTA writes
// either the final bf16 rows (one split) or an fp32 partial; the split that finishes last for a
// (user, KV head) merges the partials (decode_split_finish), so one launch does it all.
#pragma once
#include "kv_scatter.cuh"
#include "ptx.cuh"

namespace b200attn {

constexpr int kDecTile = 64;           // tokens per pipeline stage
constexpr int kDecConsumerWarps = 4;   // 16 tokens each
constexpr int kDecThreads = (kDecConsumerWarps + 1) * 32;

struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_row_stride;
  __nv_bfloat16* out;
  int64_t out_row_stride;
  const int32_t* page_table;
  int64_t page_table_stride;
  int page_table_width;
  const int32_t* cur_pos;
  float* part_o;    // [users, nq, splits, hd]
  float2* part_ml;  // [users, nq, splits]  (running max in log2 units, running sum)
  unsigned int* tickets;   // [users, nkv] arrival counters of the splits, zero between launches;
                           // NULL: the partials are merged by decode_combine_kernel instead
  int num_q_heads;
  int num_kv_heads;
  int group;        // nq / nkv
  int num_splits;
  int64_t num_blocks;
  float scale_log2; // softmax scale * log2(e)
  int window;       // sliding window size in keys (0 = attend to the whole context)
  const float* sinks;  // [num_q_heads] attention-sink logits (scaled domain), or NULL
  // Optional fused cache write of this step's K / V rows (the decode step's paged_update_cache):
  const uint4* k_new;  // [users, nkv, hd] bf16 rows in 16-byte vectors, or NULL (no write)
  const uint4* v_new;
  int64_t new_token_stride_v;   // vectors between users
  uint8_t* k_cache_w;  // cache bases as plain pointers for the write
  uint8_t* v_cache_w;
  int cache_fp8;       // 1: the caches hold e4m3
  int wrap_negative;   // 1: a negative position wraps like the reference's CPU indexing, 0: skip
  int* err_word;
};

// The decode step's cache write, done by the one warp that is about to stream the tile holding
// the new token: user u's K / V rows of KV head `kvh` go to position cur_pos[u], addressed
// exactly as kv_scatter_kernel<kScatterUpdate> does (floor division, negative column wrap).
// Every lane ends with a proxy fence so that the TMA loads issued afterwards by this warp read
// the rows just written.
template <int HD, int BS>
__device__ __forceinline__ void decode_write_new_token(const DecodeParams& p, int user, int kvh,
                                                       int lane) {
  constexpr int kVec = HD / 8;   // 16-byte vectors of 8 values per row
  const int pos = p.cur_pos[user];
  if (pos < 0 && !p.wrap_negative) return;
  int col = floordiv_i32(pos, BS);
  const int off = pos - col * BS;
  if (col < 0) col += p.page_table_width;
  bool ok = col >= 0 && col < p.page_table_width;
  int64_t blk = 0;
  if (ok) {
    blk = p.page_table[static_cast<int64_t>(user) * p.page_table_stride + col];
    ok = blk >= 0 && blk < p.num_blocks;
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.err_word, kDevBadIndex);
    return;
  }
  const int64_t row = (blk * p.num_kv_heads + kvh) * BS + off;
  for (int i = lane; i < 2 * kVec; i += 32) {
    const bool is_v = i >= kVec;
    const int v = is_v ? i - kVec : i;
    const uint4 val = __ldg((is_v ? p.v_new : p.k_new) +
                            static_cast<int64_t>(user) * p.new_token_stride_v + kvh * kVec + v);
    uint8_t* base = is_v ? p.v_cache_w : p.k_cache_w;
    if (p.cache_fp8)
      reinterpret_cast<uint2*>(base)[row * kVec + v] = bf16x8_to_e4m3x8(val);
    else
      reinterpret_cast<uint4*>(base)[row * kVec + v] = val;
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  __syncwarp();
}

// Folds an attention sink into a row's (max, sum): the sink is one more softmax column that
// contributes to the denominator only.  Returns the factor the accumulated values scale by.
__device__ __forceinline__ float apply_sink(float& m, float& l, float sink_log2) {
  const float m2 = fmaxf(m, sink_log2);
  const float f = (m == -INFINITY) ? 0.f : fast_exp2(m - m2);
  l = l * f + fast_exp2(sink_log2 - m2);
  m = m2;
  return f;
}

constexpr int kDecMaxSplits = 256;       // bounds the merge scratch in shared memory
constexpr int kDecTicketBytes = 65536;   // ticket region at the start of the split-KV workspace

// End of a split's work when the launch has more than one split: the split's partial (max, sum,
// O) for the G query heads is already in global memory.  The split takes a ticket of its
// (user, KV head); whoever arrives last finds every other partial published (each writer fences
// before its ticket), merges them and writes the bf16 rows.  Nobody waits for anybody, so
// nothing can hang, and no second launch is needed.  Called by the kDecConsumerWarps * 32
// threads `tid` = 0..127 with `scratch` = free shared memory of (32 * splits + 40) floats.
template <int HD>
__device__ __forceinline__ void decode_split_finish(const DecodeParams& p, int user, int kvh,
                                                    float* scratch, int tid) {
  constexpr int kThreads = kDecConsumerWarps * 32;
  const int S = p.num_splits;
  const int G = p.group;
  float* fac = scratch;                    // [G][S] running max of a split, then its merge factor
  float* sl = scratch + 16 * S;            // [G][S] running sum of a split
  float* row_m = sl + 16 * S;              // [G] merged max
  float* row_l = row_m + 16;               // [G] merged sum
  volatile int* last_flag = reinterpret_cast<volatile int*>(row_l + 16);
  unsigned int* ticket = p.tickets + static_cast<int64_t>(user) * p.num_kv_heads + kvh;

  __threadfence();                         // this thread's partial stores, device-wide
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
  if (tid == 0) *last_flag = atomicAdd(ticket, 1u) == static_cast<unsigned int>(S - 1);
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
  if (!*last_flag) return;
  __threadfence();

  const int64_t row0 = (static_cast<int64_t>(user) * p.num_q_heads + kvh * G) * S;
  for (int i = tid; i < G * S; i += kThreads) {
    const float2 ml = __ldcg(p.part_ml + row0 + i);
    fac[i] = ml.x;
    sl[i] = ml.y;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
  const int warp = tid >> 5, lane = tid & 31;
  for (int r = warp; r < G; r += kDecConsumerWarps) {
    float m = -INFINITY;
    for (int s = lane; s < S; s += 32) m = fmaxf(m, fac[r * S + s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (int s = lane; s < S; s += 32) {
      const float ms = fac[r * S + s];
      const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - m);   // empty splits carry -inf
      fac[r * S + s] = f;
      l += f * sl[r * S + s];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
      row_m[r] = m;
      row_l[r] = l;
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
  for (int i = tid; i < G * HD; i += kThreads) {
    const int r = i / HD, d = i - r * HD;
    const float* src = p.part_o + (row0 + static_cast<int64_t>(r) * S) * HD + d;
    float acc = 0.f;
    int s = 0;
    for (; s + 4 <= S; s += 4) {
      // an empty split published no O rows: its factor is 0 and its memory must not be read
      // into the sum (0 * garbage may be NaN)
      const float f0 = fac[r * S + s], f1 = fac[r * S + s + 1];
      const float f2 = fac[r * S + s + 2], f3 = fac[r * S + s + 3];
      const float x0 = f0 != 0.f ? __ldcg(src + static_cast<int64_t>(s) * HD) : 0.f;
      const float x1 = f1 != 0.f ? __ldcg(src + static_cast<int64_t>(s + 1) * HD) : 0.f;
      const float x2 = f2 != 0.f ? __ldcg(src + static_cast<int64_t>(s + 2) * HD) : 0.f;
      const float x3 = f3 != 0.f ? __ldcg(src + static_cast<int64_t>(s + 3) * HD) : 0.f;
      acc += f0 * x0;
      acc += f1 * x1;
      acc += f2 * x2;
      acc += f3 * x3;
    }
    for (; s < S; ++s) {
      const float f = fac[r * S + s];
      if (f != 0.f) acc += f * __ldcg(src + static_cast<int64_t>(s) * HD);
    }
    float m = row_m[r], l = row_l[r];
    const int head = kvh * G + r;
    if (p.sinks) acc *= apply_sink(m, l, p.sinks[head] * 1.4426950408889634f);
    p.out[static_cast<int64_t>(user) * p.out_row_stride + head * HD + d] =
        __float2bfloat16(l > 0.f ? acc / l : 0.f);
  }
  if (tid == 0) *ticket = 0u;              // leave the counter as the next launch expects it
}

template <int HD, int BS, int STAGES>
struct DecodeSmem {
  static constexpr int kSub = HD / 64;                 // 64-element (128 B) column groups
  static constexpr int kPages = kDecTile / BS;         // pages per tile
  static constexpr int kBoxBytes = BS * 128;           // one TMA box
  static constexpr int kTensorBytes = kPages * kSub * kBoxBytes;  // K (or V) of one tile
  static constexpr int kStageBytes = 2 * kTensorBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kBarrierBytes = 2 * STAGES * 8 + 16;
  static constexpr int kTotalBytes = kRingBytes + kBarrierBytes + 1024;  // 1 KiB alignment slack
};

template <int HD, int BS, int STAGES>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_splitkv_kernel(const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
  using L = DecodeSmem<HD, BS, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + L::kRingBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + STAGES);

  // A CTA of this launch just gave up on a wait: do not repeat the timeout per CTA.
  if (timeout_drain_window(p.err_word)) return;

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int user = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int ctx = p.cur_pos[user] + 1;  // keys 0 .. cur_pos
  const int lo = (p.window > 0 && ctx > p.window) ? ctx - p.window : 0;   // first key attended
  const int n_tiles = ctx > 0 ? (ctx + kDecTile - 1) / kDecTile : 0;
  const int t_lo = lo / kDecTile;
  const int tiles_per_split = (n_tiles - t_lo + p.num_splits - 1) / p.num_splits;
  const int t_begin = t_lo + split * tiles_per_split;
  const int t_end = min(n_tiles, t_begin + tiles_per_split);
  const int G = p.group;

  if (t_begin >= t_end) {
    // A row without context (negative position) still gets the reference's cache write.
    if (p.k_new && n_tiles == 0 && split == 0 && warp == 0)
      decode_write_new_token<HD, BS>(p, user, kvh, lane);
    // Nothing for this split: publish an empty partial (or zeros when it is the only split).
    if (p.num_splits > 1) {
      if (threadIdx.x < G) {
        const int64_t row = (static_cast<int64_t>(user) * p.num_q_heads + kvh * G + threadIdx.x) *
                                p.num_splits + split;
        p.part_ml[row] = make_float2(-INFINITY, 0.f);
      }
      if (p.tickets && threadIdx.x < kDecConsumerWarps * 32)
        decode_split_finish<HD>(p, user, kvh, reinterpret_cast<float*>(ring), threadIdx.x);
    } else {
      for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int r = i / HD, d = i - r * HD;
        p.out[static_cast<int64_t>(user) * p.out_row_stride + (kvh * G + r) * HD + d] =
            __float2bfloat16(0.f);
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kDecConsumerWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kDecConsumerWarps) {
    // ------------------------------------------------------------------ producer warp
    if (lane == 0) {
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
    }
    const uint64_t policy = l2_policy_evict_first();
    // the split that streams the last tile writes the new token's rows first
    if (p.k_new && t_end == n_tiles) decode_write_new_token<HD, BS>(p, user, kvh, lane);
    const int n_pages = (ctx + BS - 1) / BS;
    const int32_t* pt = p.page_table + static_cast<int64_t>(user) * p.page_table_stride;
    const int first_page = t_begin * L::kPages;
    // Each lane keeps one page id of a 32-page window; the next window is fetched early.
    int win_base = first_page;
    auto fetch = [&](int base) {
      // pages past the end repeat the last one
      const int idx = min(min(base + lane, n_pages - 1), p.page_table_width - 1);
      return pt[idx];
    };
    int cur_ids = fetch(win_base);
    int nxt_ids = fetch(win_base + 32);
    for (int t = t_begin; t < t_end; ++t) {
      const int it = t - t_begin;
      const int stage = it % STAGES;
      const uint32_t parity = ((it / STAGES) & 1) ^ 1;
      mbar_wait(&empty_bar[stage], parity, abort_flag, p.err_word);
      uint8_t* kdst = ring + stage * L::kStageBytes;
      uint8_t* vdst = kdst + L::kTensorBytes;
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
#pragma unroll
      for (int pg = 0; pg < L::kPages; ++pg) {
        const int page_idx = t * L::kPages + pg;
        if (page_idx - win_base >= 32) {
          win_base += 32;
          cur_ids = nxt_ids;
          nxt_ids = fetch(win_base + 32);
        }
        int64_t blk = __shfl_sync(0xffffffffu, cur_ids, page_idx - win_base);
        if (blk < 0 || blk >= p.num_blocks) {
          if (lane == 0) atomicExch(p.err_word, kDevBadIndex);
          blk = 0;
        }
        if (lane == 0) {
          const int32_t y = static_cast<int32_t>((blk * p.num_kv_heads + kvh) * BS);
#pragma unroll
          for (int s = 0; s < L::kSub; ++s) {
            tma_load_2d(kdst + (pg * L::kSub + s) * L::kBoxBytes, &tm_k, &full_bar[stage], s * 64,
                        y, policy);
            tma_load_2d(vdst + (pg * L::kSub + s) * L::kBoxBytes, &tm_v, &full_bar[stage], s * 64,
                        y, policy);
          }
        }
      }
    }
    return;  // consumers wait on every full barrier, so no copy is in flight at kernel end
  }

  // -------------------------------------------------------------------- consumer warps
  const int g = lane >> 2;   // fragment row (query head within the group); g + 8 is the second row
  const int tq = lane & 3;

  // Q fragments: A operand rows = query heads of this KV head (rows >= G are zero).
  uint32_t qf[HD / 16][4];
  {
    const __nv_bfloat16* qrow = p.q + static_cast<int64_t>(user) * p.q_row_stride +
                                static_cast<int64_t>(kvh) * G * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int d0 = ks * 16 + tq * 2;
      const uint32_t lo0 = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + g * HD + d0) : 0u;
      const uint32_t lo8 = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + g * HD + d0 + 8) : 0u;
      const uint32_t hi0 =
          (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * HD + d0) : 0u;
      const uint32_t hi8 =
          (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * HD + d0 + 8) : 0u;
      qf[ks][0] = lo0;
      qf[ks][1] = hi0;
      qf[ks][2] = lo8;
      qf[ks][3] = hi8;
    }
  }

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY;  // running max, rows g and g+8 (log2 units)
  float l_lo = 0.f, l_hi = 0.f;              // running sum (this thread's share of the row)

  // Per-lane ldmatrix row addressing inside a tile.
  //   K (non-transposed): matrix m = lane/8 -> n-tile m/2, k-half m%2; row = token.
  //   V (transposed):     matrix m = lane/8 -> token half m%2, d-tile offset m/2.
  const int lm = lane >> 3, lr = lane & 7;
  const int k_tok = warp * 16 + (lm >> 1) * 8 + lr;
  const int v_tok = warp * 16 + (lm & 1) * 8 + lr;
  const int k_page = k_tok / BS, k_row = k_tok % BS;
  const int v_page = v_tok / BS, v_row = v_tok % BS;

  for (int t = t_begin; t < t_end; ++t) {
    const int it = t - t_begin;
    const int stage = it % STAGES;
    mbar_wait(&full_bar[stage], (it / STAGES) & 1, abort_flag, p.err_word);
    const uint32_t kbase = smem_u32(ring + stage * L::kStageBytes);
    const uint32_t vbase = kbase + L::kTensorBytes;
    const int tok0 = t * kDecTile + warp * 16;   // first token of this warp's slice

    if (tok0 < ctx && tok0 + 16 > lo) {       // at least one of this warp's keys is attended
      const bool tail = (tok0 + 16 > ctx) || (tok0 < lo);
      if (tail) {
        // Zero this warp's V rows past the context so that stale or non-finite cache
        // contents cannot reach the accumulator through 0 * x.
        for (int i = lane; i < 16 * (HD / 8); i += 32) {
          const int r = i / (HD / 8), c = i % (HD / 8);
          const int tok = warp * 16 + r;
          if (t * kDecTile + tok >= ctx) {
            const int pg = tok / BS, row = tok % BS;
            const uint32_t a = vbase + ((pg * L::kSub + (c >> 3)) * BS + row) * 128 +
                               (((c & 7) ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
          }
        }
        fence_proxy_async_smem();  // the next TMA write to this stage follows generic writes
        __syncwarp();
      }

      // ---- S = Q K^T for 16 tokens (two 8-token n-tiles)
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int cc = ks * 2 + (lm & 1);  // 16-byte chunk along head_size
        const uint32_t a = kbase + ((k_page * L::kSub + (cc >> 3)) * BS + k_row) * 128 +
                           (((cc & 7) ^ (k_row & 7)) << 4);
        uint32_t b[4];
        ldmatrix_x4(b, a);
        mma_bf16_16816(s[0], qf[ks], b[0], b[1]);
        mma_bf16_16816(s[1], qf[ks], b[2], b[3]);
      }

      // ---- online softmax (log2 domain)
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] *= p.scale_log2;
      if (tail) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int tok = tok0 + i * 8 + tq * 2 + (j & 1);
            if (tok >= ctx || tok < lo) s[i][j] = -INFINITY;
          }
      }
      float mx_lo = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float mx_hi = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      // the guard above leaves at least one unmasked key, so mn_* is finite here.
      const float c_lo = fast_exp2(m_lo - mn_lo), c_hi = fast_exp2(m_hi - mn_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      float pr[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        pr[i][0] = fast_exp2(s[i][0] - mn_lo);
        pr[i][1] = fast_exp2(s[i][1] - mn_lo);
        pr[i][2] = fast_exp2(s[i][2] - mn_hi);
        pr[i][3] = fast_exp2(s[i][3] - mn_hi);
      }
      l_lo = l_lo * c_lo + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
      l_hi = l_hi * c_hi + (pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3]);
      if (__any_sync(0xffffffffu, (c_lo != 1.f) || (c_hi != 1.f))) {
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[i][0] *= c_lo;
          o[i][1] *= c_lo;
          o[i][2] *= c_hi;
          o[i][3] *= c_hi;
        }
      }
      uint32_t pa[4];
      pa[0] = pack_bf16x2(pr[0][0], pr[0][1]);
      pa[1] = pack_bf16x2(pr[0][2], pr[0][3]);
      pa[2] = pack_bf16x2(pr[1][0], pr[1][1]);
      pa[3] = pack_bf16x2(pr[1][2], pr[1][3]);

      // ---- O += P V  (k = this warp's 16 tokens, n = head_size)
#pragma unroll
      for (int dn = 0; dn < HD / 8; dn += 2) {
        const int cc = dn + (lm >> 1);
        const uint32_t a = vbase + ((v_page * L::kSub + (cc >> 3)) * BS + v_row) * 128 +
                           (((cc & 7) ^ (v_row & 7)) << 4);
        uint32_t b[4];
        ldmatrix_x4_trans(b, a);
        mma_bf16_16816(o[dn], pa, b[0], b[1]);
        mma_bf16_16816(o[dn + 1], pa, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
  }

  // -------------------------------------------------------------------- merge the 4 warps
  // Row sums: finish the quad reduction.
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // All consumer warps are past their last full-barrier wait: the ring is free to reuse.
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32));
  float* mo = reinterpret_cast<float*>(ring);                       // [4 warps][16 rows][HD]
  float* mm = mo + kDecConsumerWarps * 16 * HD;                     // [4][16] max
  float* ml = mm + kDecConsumerWarps * 16;                          // [4][16] sum
  static_assert((kDecConsumerWarps * 16 * (HD + 2)) * 4 <= L::kRingBytes, "merge scratch fits");
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    const int d = i * 8 + tq * 2;
    *reinterpret_cast<float2*>(mo + (warp * 16 + g) * HD + d) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * HD + d) = make_float2(o[i][2], o[i][3]);
  }
  if (tq == 0) {
    mm[warp * 16 + g] = m_lo;
    mm[warp * 16 + g + 8] = m_hi;
    ml[warp * 16 + g] = l_lo;
    ml[warp * 16 + g + 8] = l_hi;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerWarps * 32));

  for (int i = threadIdx.x; i < G * HD; i += kDecConsumerWarps * 32) {
    const int r = i / HD, d = i - r * HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecConsumerWarps; ++w) m = fmaxf(m, mm[w * 16 + r]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kDecConsumerWarps; ++w) {
      const float mw = mm[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
      acc += f * mo[(w * 16 + r) * HD + d];
      l += f * ml[w * 16 + r];
    }
    const int head = kvh * G + r;
    if (p.num_splits == 1) {
      if (p.sinks) acc *= apply_sink(m, l, p.sinks[head] * 1.4426950408889634f);
      p.out[static_cast<int64_t>(user) * p.out_row_stride + head * HD + d] =
          __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      const int64_t row =
          (static_cast<int64_t>(user) * p.num_q_heads + head) * p.num_splits + split;
      p.part_o[row * HD + d] = acc;
      if (d == 0) p.part_ml[row] = make_float2(m, l);
    }
  }
  if (p.num_splits > 1 && p.tickets)
    decode_split_finish<HD>(p, user, kvh, reinterpret_cast<float*>(ring), threadIdx.x);
}

// Merges the split partials of one (user, q head) row and writes bf16.
template <int HD>
__global__ void __launch_bounds__(HD) decode_combine_kernel(const DecodeParams p) {
  const int head = blockIdx.x;
  const int user = blockIdx.y;
  const int d = threadIdx.x;
  const int64_t row0 = (static_cast<int64_t>(user) * p.num_q_heads + head) * p.num_splits;
  float m = -INFINITY;
  for (int s = 0; s < p.num_splits; ++s) m = fmaxf(m, p.part_ml[row0 + s].x);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < p.num_splits; ++s) {
    const float2 ml = p.part_ml[row0 + s];
    if (ml.x == -INFINITY) continue;
    const float f = fast_exp2(ml.x - m);
    acc += f * p.part_o[(row0 + s) * HD + d];
    l += f * ml.y;
  }
  if (p.sinks) acc *= apply_sink(m, l, p.sinks[head] * 1.4426950408889634f);
  p.out[static_cast<int64_t>(user) * p.out_row_stride + head * HD + d] =
      __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace b200attn
