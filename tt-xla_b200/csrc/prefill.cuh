// Causal varlen / chunked prefill attention on tcgen05 tensor cores.
//
// Persistent kernel: one CTA per SM walks a list of work items; an item is 2 x 128 query
// rows (tiles A and B) of one sequence x one query head.  KV is consumed in tiles of 128
// keys, shared by both query tiles.  Ten warps:
//   warp 0      TMA producer: per item Q_A and Q_B, then K_0, V_0, K_1, V_1, ... into a ring
//               of swizzled [128 rows x 128 B] sub-tiles (paged source: one box per page;
//               fresh source: one box per 64-wide column group).  It runs ahead of the other
//               warps, so the loads of the next item overlap the tail of the current one.
//   warp 1      allocates tensor memory once (S_A, S_B, O_A, O_B = 512 columns) and issues
//               tcgen05.mma from one lane in the order
//                   PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1), ...
//               so that the tensor pipe works for one query tile while the other tile's
//               softmax runs; at an item boundary it goes straight on to QK(0) of the next
//               item while the softmax warps are still in their epilogue.
//   warps 2-5   softmax warpgroup of tile A, warps 6-9 of tile B; one thread per query row:
//               tcgen05.ld the row of S, causal mask on diagonal tiles, running max with a
//               lazy rescale threshold, ex2 via packed fp32 FMA, row sum, P as packed bf16 back
//               into tensor memory over the first 64 columns of its S buffer (the PV MMA takes
//               its A operand from tensor memory); rescales its O row in tensor memory when the
//               running max moved; per item it normalises O by 1/l and stores bf16.
// Items are ordered heaviest first (by the index of the 256-row block inside its sequence,
// highest first, heads of one block adjacent) and dealt to the CTAs in rounds of alternating
// direction (0..G-1, G-1..0, ...), which evens out the per-CTA sums of a sorted list.
// Every mbarrier wait is bounded; tensor memory is always freed before exit.
#pragma once
#include "ptx.cuh"

namespace b200attn {

constexpr int kPfM = 128;        // query rows per tile
constexpr int kPfQTiles = 2;     // query tiles per item
constexpr int kPfRowsPerItem = kPfM * kPfQTiles;
constexpr int kPfN = 128;        // keys per KV tile
constexpr int kPfThreads = 320;
constexpr float kPfRescaleThreshold = 8.f;  // log2 units
constexpr int kPfSeqCache = 2048;           // sequences whose cu_q is cached in shared memory
constexpr int kPfLevelOrderMaxSeqs = 64;    // above this, items keep plain sequence order
constexpr int kPfItemTable = 96;            // rounds whose item is decoded once, up front

struct PrefillParams {
  __nv_bfloat16* out;
  int64_t out_row_stride;
  const int32_t* page_table;
  int64_t page_table_stride;
  int page_table_width;
  const int32_t* cu_q;
  const int32_t* q_start;
  int num_seqs;
  int num_q_heads;
  int num_kv_heads;
  int group;
  int kv_is_paged;
  int window;          // sliding window size in keys (0 = full causal attention)
  int total_items;     // (256-row blocks over all sequences) x num_q_heads
  int64_t num_blocks;
  float scale_log2;
  int* err_word;
};

template <int HD>
struct PrefillSmem {
  static constexpr int kSub = HD / 64;
  static constexpr int kSubBytes = 128 * 128;             // 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;     // one Q, K or V tile
  static constexpr int kSlots = (HD == 128) ? 4 : 8;      // ring slots (one K or V tile each)
  static constexpr int kQOff = 0;
  static constexpr int kRingOff = kPfQTiles * kTileBytes;
  static constexpr int kSeqOff = kRingOff + kSlots * kTileBytes;
  static constexpr int kItemOff = kSeqOff + (kPfSeqCache + 4) * 4;   // keeps 16-byte alignment
  static constexpr int kBarOff = kItemOff + kPfItemTable * 16;
  static constexpr int kNumBars = 2 + 2 * kSlots + 4 * kPfQTiles;
  static constexpr int kTotalBytes = kBarOff + kNumBars * 8 + 16 + 1024;
  static_assert(kItemOff % 16 == 0, "16-byte vector access alignment");
  static_assert(kBarOff % 8 == 0, "barrier alignment");
  static_assert(kTotalBytes <= 232448, "shared memory budget");
};

// Compact result of the item-order search (one per round, kept in shared memory).
struct PrefillItemKey {
  int seq;    // -1 = no such item
  int q0;
  int head;
  int start;
};

// What every role needs to know about one work item.
struct PrefillItem {
  int seq, head, q0, seq_q_begin, seq_len_q, start;
  int rows_valid[kPfQTiles], first_pos[kPfQTiles];
  // KV tiles are counted relative to the item's first tile j0 (0 without a sliding window):
  // query tile w works on relative tiles skip[w] .. n_rel[w]-1.
  int j0, skip[kPfQTiles], n_rel[kPfQTiles];
  int n_max;          // relative tiles of the item (the larger n_rel)
};

// Item index -> (sequence, 256-row block, head).  `cu` is cu_q (shared-memory copy when the
// batch fits the cache).  Heaviest first: blocks ranked by their index inside their sequence,
// highest first across sequences; the heads of one block are adjacent.  The search costs
// microseconds, so the kernel runs it once per round up front (one thread per round) and the
// roles read the result from shared memory.
__device__ __forceinline__ PrefillItemKey prefill_find_item(const PrefillParams& p,
                                                           const int32_t* cu, int item) {
  PrefillItemKey key{-1, 0, 0, 0};
  if (item >= p.total_items) return key;
  key.head = item % p.num_q_heads;
  const int t = item / p.num_q_heads;
  auto nblk = [&](int s) { return (cu[s + 1] - cu[s] + kPfRowsPerItem - 1) / kPfRowsPerItem; };
  int seq = -1, blk = 0;
  if (p.num_seqs <= kPfLevelOrderMaxSeqs) {
    int max_n = 0;
    for (int s = 0; s < p.num_seqs; ++s) max_n = max(max_n, nblk(s));
    auto at_or_above = [&](int r) {   // number of blocks whose index is >= r; decreasing in r
      int n = 0;
      for (int s = 0; s < p.num_seqs; ++s) n += max(0, nblk(s) - r);
      return n;
    };
    if (max_n == 0 || t >= at_or_above(0)) return key;
    int lo = 0, hi = max_n - 1;       // largest r with at_or_above(r) > t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (at_or_above(mid) > t) lo = mid; else hi = mid - 1;
    }
    int idx = t - at_or_above(lo + 1);
    for (int s = 0; s < p.num_seqs; ++s) {
      if (nblk(s) > lo) {
        if (idx == 0) {
          seq = s;
          break;
        }
        --idx;
      }
    }
    blk = lo;
  } else {
    int acc = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int n = nblk(s);
      if (t < acc + n) {
        seq = s;
        blk = n - 1 - (t - acc);      // later blocks of a sequence first
        break;
      }
      acc += n;
    }
  }
  if (seq < 0) return key;
  key.seq = seq;
  key.q0 = blk * kPfRowsPerItem;
  key.start = p.q_start ? p.q_start[seq] : 0;
  return key;
}

__device__ __forceinline__ bool prefill_expand_item(const PrefillParams& p,
                                                    const PrefillItemKey& key, const int32_t* cu,
                                                    PrefillItem& it) {
  if (key.seq < 0) return false;
  it.seq = key.seq;
  it.head = key.head;
  it.q0 = key.q0;
  it.start = key.start;
  it.seq_q_begin = cu[key.seq];
  it.seq_len_q = cu[key.seq + 1] - it.seq_q_begin;
#pragma unroll
  for (int w = 0; w < kPfQTiles; ++w) {
    it.rows_valid[w] = max(0, min(kPfM, it.seq_len_q - it.q0 - w * kPfM));
    it.first_pos[w] = it.start + it.q0 + w * kPfM;
  }
  // first key any row of tile A may attend (tile A starts lowest)
  const int lo = (p.window > 0 && it.first_pos[0] + 1 > p.window) ? it.first_pos[0] + 1 - p.window : 0;
  it.j0 = lo / kPfN;
#pragma unroll
  for (int w = 0; w < kPfQTiles; ++w) {
    const int n_abs =
        it.rows_valid[w] > 0 ? (it.first_pos[w] + it.rows_valid[w] - 1) / kPfN + 1 : 0;
    const int lo_w =
        (p.window > 0 && it.first_pos[w] + 1 > p.window) ? it.first_pos[w] + 1 - p.window : 0;
    it.n_rel[w] = n_abs > 0 ? n_abs - it.j0 : 0;
    it.skip[w] = n_abs > 0 ? lo_w / kPfN - it.j0 : 0;
  }
  it.n_max = max(it.n_rel[0], it.n_rel[1]);   // tile A never ends later than tile B
  return true;
}

// Item handled by CTA `cta` of `num_ctas` in round `round` (alternating direction per round).
__device__ __forceinline__ int prefill_item_of(int round, int cta, int num_ctas) {
  return round * num_ctas + ((round & 1) ? (num_ctas - 1 - cta) : cta);
}

template <int HD, int BS, bool WIN>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
  using L = PrefillSmem<HD>;
  constexpr int kSub = L::kSub;
  constexpr int kSlots = L::kSlots;
  constexpr int kPagesPerTile = kPfN / BS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem + L::kQOff;
  uint8_t* ring = smem + L::kRingOff;
  int32_t* cu_smem = reinterpret_cast<int32_t*>(smem + L::kSeqOff);
  PrefillItemKey* item_table = reinterpret_cast<PrefillItemKey*>(smem + L::kItemOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                   // Q tiles of the item landed (TMA -> MMA)
  uint64_t* q_empty = bars + 1;              // last QK of the item retired (MMA -> TMA)
  uint64_t* full = bars + 2;                 // [kSlots]
  uint64_t* empty = full + kSlots;           // [kSlots]
  uint64_t* s_full = empty + kSlots;         // [2]  S of tile A / B ready (MMA -> softmax)
  uint64_t* p_full = s_full + kPfQTiles;     // [2]  P of tile A / B written (softmax -> MMA)
  uint64_t* pv_done = p_full + kPfQTiles;    // [2]  PV of tile A / B retired (MMA -> softmax)
  uint64_t* o_empty = pv_done + kPfQTiles;   // [2]  O of tile A / B read out (softmax -> MMA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A CTA of this launch just gave up on a wait: do not repeat the timeout per CTA.
  if (timeout_drain_window(p.err_word)) return;

  const bool cu_cached = p.num_seqs <= kPfSeqCache;
  if (cu_cached)
    for (int s = threadIdx.x; s <= p.num_seqs; s += blockDim.x) cu_smem[s] = p.cu_q[s];
  const int32_t* cu = cu_cached ? cu_smem : p.cu_q;
  if (cu_cached) __syncthreads();
  const int num_rounds = (p.total_items + gridDim.x - 1) / gridDim.x;
  for (int r = threadIdx.x; r < min(num_rounds, kPfItemTable); r += blockDim.x)
    item_table[r] = prefill_find_item(p, cu, prefill_item_of(r, blockIdx.x, gridDim.x));
  auto get_item = [&](int round, PrefillItem& it) {
    const PrefillItemKey key =
        round < kPfItemTable ? item_table[round]
                             : prefill_find_item(p, cu, prefill_item_of(round, blockIdx.x, gridDim.x));
    return prefill_expand_item(p, key, cu, it);
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < kPfQTiles; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_empty[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_A [0,128)  S_B [128,256)  O_A [256,256+HD)  O_B [384,384+HD)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
    }
    const uint64_t pol_q = l2_policy_evict_first();
    const uint64_t pol_kv = l2_policy_evict_last();
    uint32_t ring_i = 0, item_n = 0;
    for (int round = 0; round < num_rounds; ++round) {
      PrefillItem it;
      if (!get_item(round, it)) continue;
      const int kvh = it.head / p.group;
      // Q may be overwritten once every QK of the previous item has retired.
      mbar_wait(q_empty, (item_n & 1) ^ 1, abort_flag, p.err_word);
      ++item_n;
      if (lane == 0) {
        mbar_arrive_expect_tx(q_full, kPfQTiles * L::kTileBytes);
#pragma unroll
        for (int w = 0; w < kPfQTiles; ++w)
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_2d(q_smem + w * L::kTileBytes + s * L::kSubBytes, &tm_q, q_full,
                        it.head * HD + s * 64, it.seq_q_begin + it.q0 + w * kPfM, pol_q);
      }
      const int32_t* pt = p.page_table + static_cast<int64_t>(it.seq) * p.page_table_stride;
      const int last_pos = it.start + min(it.seq_len_q, it.q0 + kPfRowsPerItem) - 1;
      const int n_pages = last_pos / BS + 1;      // pages holding keys 0 .. last_pos
      for (int i = 0; i < 2 * it.n_max; ++i, ++ring_i) {
        const int j = (WIN ? it.j0 : 0) + (i >> 1);          // absolute KV tile
        const bool is_v = i & 1;
        const int slot = ring_i % kSlots;
        mbar_wait(&empty[slot], ((ring_i / kSlots) & 1) ^ 1, abort_flag, p.err_word);
        uint8_t* dst = ring + slot * L::kTileBytes;
        const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
        if (lane == 0) mbar_arrive_expect_tx(&full[slot], L::kTileBytes);
        if (p.kv_is_paged) {
          int my_id = 0;
          if (lane < kPagesPerTile) {
            int idx = min(j * kPagesPerTile + lane, n_pages - 1);
            idx = min(idx, p.page_table_width - 1);
            my_id = pt[idx];
          }
#pragma unroll
          for (int pg = 0; pg < kPagesPerTile; ++pg) {
            int64_t blk = __shfl_sync(0xffffffffu, my_id, pg);
            if (blk < 0 || blk >= p.num_blocks) {
              if (lane == 0) atomicExch(p.err_word, kDevBadIndex);
              blk = 0;
            }
            if (lane == 0) {
              const int32_t y = static_cast<int32_t>((blk * p.num_kv_heads + kvh) * BS);
#pragma unroll
              for (int s = 0; s < kSub; ++s)
                tma_load_2d(dst + s * L::kSubBytes + pg * BS * 128, tm, &full[slot], s * 64, y,
                            pol_kv);
            }
          }
        } else if (lane == 0) {
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_2d(dst + s * L::kSubBytes, tm, &full[slot], kvh * HD + s * 64,
                        it.seq_q_begin + j * kPfN, pol_kv);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the schedule (so addresses and descriptors stay warp-uniform);
    // lane 0 issues.  Descriptor words are built once per tile: the k-step only adds a
    // constant to the low word, so consecutive tcgen05.mma are a couple of instructions apart.
    constexpr uint32_t idesc_qk = umma_idesc_bf16(kPfM, kPfN, false, false);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(kPfM, HD, false, true);
    // high descriptor word: SBO = 1024 B, descriptor version 1, 128-byte swizzle
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
    constexpr uint32_t kLboV = (static_cast<uint32_t>(L::kSubBytes) >> 4) << 16;  // V: next 64 d
    constexpr uint32_t kLboK = 1u << 16;                                          // unused field
    const bool leader = lane == 0;
    auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
    uint32_t ring_base = 0;            // ring index of K_0 of the current item
    uint32_t item_n = 0;
    uint32_t tiles_done[kPfQTiles] = {0, 0};   // KV tiles finished per query tile (all items)
    uint32_t items_done[kPfQTiles] = {0, 0};   // items in which the query tile was active
    auto wait_ring = [&](uint32_t i) {
      mbar_wait(&full[i % kSlots], (i / kSlots) & 1, abort_flag, p.err_word);
      tc_fence_after_sync();
    };
    auto release_ring = [&](uint32_t i) {
      if (leader) umma_commit(&empty[i % kSlots]);
    };
    auto issue_qk = [&](int w, uint32_t k_ring) {   // S_w = Q_w K^T
      const uint32_t q_lo = (smem_u32(q_smem + w * L::kTileBytes) >> 4) | kLboK;
      const uint32_t k_lo = (smem_u32(ring + (k_ring % kSlots) * L::kTileBytes) >> 4) | kLboK;
      const uint32_t d = tmem_base + w * kPfN;
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * L::kSubBytes + (kk & 3) * 32) >> 4;
          umma_ss(d, desc(q_lo + off), desc(k_lo + off), idesc_qk, kk > 0);
        }
        umma_commit(&s_full[w]);
      }
    };
    auto issue_pv = [&](int w, bool first, uint32_t v_ring) {   // O_w (+)= P_w V_j
      mbar_wait(&p_full[w], tiles_done[w] & 1, abort_flag, p.err_word);
      if (first)    // O_w of the previous item must have been read out before it is overwritten
        mbar_wait(&o_empty[w], (items_done[w] & 1) ^ 1, abort_flag, p.err_word);
      tc_fence_after_sync();
      const uint32_t p_tmem = tmem_base + w * kPfN;   // P over the first 64 columns of S_w
      const uint32_t v_lo = (smem_u32(ring + (v_ring % kSlots) * L::kTileBytes) >> 4) | kLboV;
      const uint32_t d = tmem_base + 256 + w * 128;
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < kPfN / 16; ++kk) {
          // A: 16 keys = 8 packed 32-bit columns per step; B: 16 keys = 2048 B further on
          umma_ts(d, p_tmem + kk * 8, desc(v_lo + kk * (2048 >> 4)), idesc_pv,
                  !first || (kk > 0));
        }
        umma_commit(&pv_done[w]);
      }
      ++tiles_done[w];
    };
    for (int round = 0; round < num_rounds; ++round) {
      PrefillItem it;
      if (!get_item(round, it)) continue;
      mbar_wait(q_full, item_n & 1, abort_flag, p.err_word);
      ++item_n;
      wait_ring(ring_base);                         // K_0
#pragma unroll
      for (int w = 0; w < kPfQTiles; ++w)
        if (it.n_rel[w] > 0 && (!WIN || it.skip[w] == 0)) issue_qk(w, ring_base);
      release_ring(ring_base);
      if (it.n_max == 1 && leader) umma_commit(q_empty);
      for (int j = 0; j < it.n_max; ++j) {
        wait_ring(ring_base + 2 * j + 1);           // V_j
        const bool has_next = j + 1 < it.n_max;
        bool next_k_ready = false;
#pragma unroll
        for (int w = 0; w < kPfQTiles; ++w) {
          const int skip_w = WIN ? it.skip[w] : 0;
          if (j >= skip_w && j < it.n_rel[w]) issue_pv(w, j == skip_w, ring_base + 2 * j + 1);
          if (j + 1 >= skip_w && j + 1 < it.n_rel[w]) {
            if (!next_k_ready) {
              wait_ring(ring_base + 2 * j + 2);   // K_{j+1}
              next_k_ready = true;
            }
            issue_qk(w, ring_base + 2 * j + 2);
          }
        }
        release_ring(ring_base + 2 * j + 1);
        if (has_next) {
          release_ring(ring_base + 2 * j + 2);
          // the last QK of the item has been issued: Q is free once it retires
          if (j + 2 == it.n_max && leader) umma_commit(q_empty);
        }
      }
#pragma unroll
      for (int w = 0; w < kPfQTiles; ++w)
        if (it.n_rel[w] > 0) ++items_done[w];
      ring_base += 2 * it.n_max;
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int w = (warp - 2) >> 2;                       // 0 = tile A, 1 = tile B
    const int row = (warp & 3) * 32 + lane;              // tensor-memory lane == query row
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + w * kPfN + lane_addr;
    const uint32_t o_addr = tmem_base + 256 + w * 128 + lane_addr;
    const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint32_t tiles_done = 0;            // KV tiles this warpgroup has finished (all items)
    for (int round = 0; round < num_rounds; ++round) {
      PrefillItem it;
      if (!get_item(round, it)) continue;
      if (it.n_rel[w] <= 0) continue;
      const int q_pos = it.first_pos[w] + row;
      float m_run = -INFINITY, l_run = 0.f;
      const int skip_w = WIN ? it.skip[w] : 0;
      for (int jr = skip_w; jr < it.n_rel[w]; ++jr, ++tiles_done) {
        const int j = (WIN ? it.j0 : 0) + jr;    // absolute KV tile
        const bool first = jr == skip_w;
        mbar_wait(&s_full[w], tiles_done & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        uint32_t sreg[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, sreg[c]);
        tmem_wait_ld();

        const int key0 = j * kPfN;
        if (key0 + kPfN - 1 > it.first_pos[w]) {   // tile crosses the diagonal for some row
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (key0 + c * 32 + k > q_pos) sreg[c][k] = 0xff800000u;   // -inf
        }
        if (WIN && key0 < it.first_pos[w] + kPfM - p.window) {   // below some row's window
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (key0 + c * 32 + k + p.window <= q_pos) sreg[c][k] = 0xff800000u;   // -inf
        }
        // row max of the raw scores (scale > 0), four independent chains
        float mx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mx[c] = max3(__uint_as_float(sreg[c][0]), __uint_as_float(sreg[c][1]),
                       __uint_as_float(sreg[c][2]));
#pragma unroll
          for (int k = 3; k + 1 < 32; k += 2)
            mx[c] = max3(mx[c], __uint_as_float(sreg[c][k]), __uint_as_float(sreg[c][k + 1]));
          mx[c] = fmaxf(mx[c], __uint_as_float(sreg[c][31]));
        }
        const float mx_s = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        float m_new = m_run;
        if (mx_s - m_run > kPfRescaleThreshold) m_new = mx_s;   // also taken when m_run = -inf
        // a row whose keys are all masked so far (possible only under a sliding window) keeps
        // m = -inf: its weights and its correction factor are 0, not exp2(-inf + inf)
        const float corr = (WIN && m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
        const bool rescale = (m_new != m_run) && !first;
        m_run = m_new;
        // p = 2^(s*scale - m): packed FMA, then ex2; two packed running sums.  Each 32-key
        // chunk goes straight back to tensor memory as 16 packed bf16x2 columns.  QK_j has
        // retired (s_full), and PV_{j-1} was issued before it, so S_w / P_w / O_w are quiescent.
        const float m_sub = (WIN && m_new == -INFINITY) ? 0.f : m_new;
        const uint64_t negm2 = pack_f32x2(-m_sub, -m_sub);
        uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t preg[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const uint64_t x2 = fma_f32x2(
                pack_f32x2(__uint_as_float(sreg[c][k]), __uint_as_float(sreg[c][k + 1])), scale2,
                negm2);
            float x0, x1;
            unpack_f32x2(x2, x0, x1);
            const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
            sum2[(k >> 1) & 1] = add_f32x2(sum2[(k >> 1) & 1], pack_f32x2(e0, e1));
            preg[k >> 1] = pack_bf16x2(e0, e1);
          }
          tmem_st_32x16(s_addr + c * 16, preg);
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(sum2[0], a0, a1);
          unpack_f32x2(sum2[1], b0, b1);
          l_run = l_run * corr + ((a0 + a1) + (b0 + b1));
        }
        // O row rescale (rare: only when the running max moved by more than the threshold).
        if (!first && __any_sync(0xffffffffu, rescale)) {
          const float f = rescale ? corr : 1.f;
          const uint64_t f2 = pack_f32x2(f, f);
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t oreg[32];
            tmem_ld_32x32(o_addr + c * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              float y0, y1;
              unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(oreg[k]),
                                                __uint_as_float(oreg[k + 1])), f2), y0, y1);
              oreg[k] = __float_as_uint(y0);
              oreg[k + 1] = __float_as_uint(y1);
            }
            tmem_st_32x32(o_addr + c * 32, oreg);
          }
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&p_full[w]);
      }
      // ---- item epilogue: O / l -> bf16 rows.  O_w is handed back to the MMA warp as soon as
      // it sits in registers, so PV_0 of the next item does not wait for the global stores.
      mbar_wait(&pv_done[w], (tiles_done - 1) & 1, abort_flag, p.err_word);
      tc_fence_after_sync();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      uint32_t oreg[HD / 32][32];
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) tmem_ld_32x32(o_addr + c * 32, oreg[c]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&o_empty[w]);
      uint32_t packed[HD / 2];
#pragma unroll
      for (int c = 0; c < HD / 32; ++c)
#pragma unroll
        for (int k = 0; k < 32; k += 2)
          packed[(c * 32 + k) >> 1] = pack_bf16x2(__uint_as_float(oreg[c][k]) * inv_l,
                                                  __uint_as_float(oreg[c][k + 1]) * inv_l);
      if (row < it.rows_valid[w]) {
        __nv_bfloat16* orow =
            p.out + static_cast<int64_t>(it.seq_q_begin + it.q0 + w * kPfM + row) * p.out_row_stride +
            static_cast<int64_t>(it.head) * HD;
#pragma unroll
        for (int k = 0; k < HD / 2; k += 4)
          *reinterpret_cast<uint4*>(orow + 2 * k) =
              make_uint4(packed[k], packed[k + 1], packed[k + 2], packed[k + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200attn
