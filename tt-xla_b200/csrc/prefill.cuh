// Causal varlen / chunked prefill attention on tcgen05 tensor cores.
//
// Persistent kernel: one CTA per SM walks a list of work items; an item is 128 query rows of
// one sequence x one query head.  KV is consumed in tiles of 128 keys.  Four warpgroups:
//   warpgroup 0   warps 0 and 2: TMA producers.  Warp 0 loads, per item, the Q tile (two Q
//                 buffers, so the next item's Q lands while this one is still in use) and the K
//                 tiles; warp 2 loads the V tiles.  K and V have rings of their own (swizzled
//                 [128 rows x 128 B] sub-tiles; paged source: one box per page; fresh source:
//                 one box per 64-wide column group): QK runs ahead of PV, so a K tile must not
//                 queue behind the V tiles that are still waiting for their P.
//                 warps 1 and 3: tcgen05.mma issuers, one lane each.  Warp 1 (which also owns the
//                 tensor-memory allocation: S_0, S_1, S_2, O = 512 columns) issues S_{t%3} =
//                 Q K_t^T as soon as K_t has landed and the PV that read the buffer three tiles
//                 ago has retired; warp 3 issues O (+)= P_t V_t as soon as the softmax has
//                 written P_t.  Two issuers because the tensor pipe's queue is short: a single
//                 thread that also waits on four barriers per tile leaves the pipe idle half of
//                 the time (measured).  The tile counter t runs on across items, so the QKs of
//                 the next item are in flight while the last tiles of this one are still in
//                 their softmax; only the first PV of an item waits for the epilogue to have
//                 read the item before out of O.  One tcgen05.commit per MMA group: the barrier
//                 that tells the softmax "S is ready" is the same one that tells the K producer
//                 "the slot is free", and likewise for PV / the V producer / the epilogue.
//   warpgroups 1, 2   softmax of the even / odd tiles, one thread per query row: tcgen05.ld the
//                 row of S, causal mask on the diagonal tile, row max; the running max of a row
//                 is handed from tile to tile through shared memory (the only serial link
//                 between the two warpgroups: a tile's exponentials need the max of the tile
//                 before, nothing else of it, so the exponentials of consecutive tiles overlap);
//                 ex2 via packed fp32 FMA, row sum kept per warpgroup, P as packed bf16 back into
//                 tensor memory over the first 64 columns of its S buffer (the PV MMA takes its A
//                 operand from tensor memory); rescales the O row in tensor memory in the rare
//                 case that the running max moved by more than a threshold.
//   warpgroup 3   epilogue: per item, waits for the last PV, merges the two warpgroups' row
//                 sums, reads O, hands it back, normalises by 1/l and stores bf16 rows.
// Registers follow the roles (setmaxnreg): the two softmax warpgroups hold a whole S row each.
// Items are ordered heaviest first (by the index of the 128-row block inside its sequence,
// highest first, heads of one block adjacent) and handed out dynamically: a CTA takes the next
// item of the list from a global counter when it is about to need one (longest-processing-time
// -first list scheduling, which also absorbs the run-to-run differences between CTAs that a
// static deal cannot); its first item is the one with its own index, so no atomic stands before
// the first loads.  The counter needs no clearing launch: its word carries a tag that is unique
// to the launch, a CTA that finds another tag claims the word for this launch with a
// compare-and-swap, and the CTA that draws the last end marker puts the word back to zero (so
// that a replay of a captured launch, which carries the same tag, starts afresh).
// Every mbarrier wait is bounded; tensor memory is always freed before exit.
// Code size is a first-order cost here: four roles run different code on every SM
// sub-partition, and whatever runs once per item (mask, epilogue, taking an item) runs out of a
// cold instruction cache.  Hence the compact wait (pf_wait), the rolled rare loops, and the item
// order tabulated once instead of searched per item.
#pragma once
#include "ptx.cuh"

namespace b200attn {

constexpr int kPfM = 128;        // query rows per item
constexpr int kPfRowsPerItem = kPfM;
constexpr int kPfN = 128;        // keys per KV tile
constexpr int kPfThreads = 512;  // four warpgroups
constexpr float kPfRescaleThreshold = 8.f;  // log2 units
// One pair of exponentials in every kPfPolyEvery is computed on the FMA pipe (a cubic on the
// fractional part, the integer part added to the exponent field) instead of the MUFU: the
// special-function unit is the busiest pipe of the softmax warps, the FMA pipe the idlest.
// Relative error of the cubic 1.0e-4, far below the bf16 rounding of P.  0 = MUFU only, which is
// the default: on config 2 every fourth pair measured 834 TFLOP/s, every second 779, none 918
// (the softmax warps are short of issue slots, not of MUFU throughput).
#ifndef B200ATTN_PF_POLY_EVERY
#define B200ATTN_PF_POLY_EVERY 0
#endif
constexpr int kPfPolyEvery = B200ATTN_PF_POLY_EVERY;

constexpr int kPfSeqCache = 1024;           // sequences whose cu_q is cached in shared memory
constexpr int kPfLevelOrderMaxSeqs = 64;    // above this, items keep plain sequence order
constexpr int kPfQueue = 16;                // items in flight inside a CTA (fetched .. epilogue)
constexpr int kPfBlockTab = 1024;           // 128-row blocks whose place in the list is tabulated
constexpr int kPfSchedSlots = 64;           // counter words; a launch uses word tag % 64
// register budgets per warpgroup (sum = 4 x 128, the per-thread budget the kernel launches with)
constexpr int kPfRegsProducer = 88;
constexpr int kPfRegsSoftmax = 184;
constexpr int kPfRegsEpilogue = 56;

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
  unsigned long long* sched;   // this launch's counter word: (tag << 32) | next item
  uint32_t sched_tag;          // unique per launch on a device, never 0
#ifdef B200ATTN_PF_TRACE
  unsigned long long* trace;   // [CTA][role 0..5][8] cycles spent per wait site (debug builds only)
#endif
};

// Debug builds (-DB200ATTN_PF_TRACE) time every wait site with clock64; product builds compile
// the macros away.
#ifdef B200ATTN_PF_TRACE
#define PF_TRACE_DECL unsigned long long tr_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long tr_t0 = 0;
#define PF_TRACE_BEGIN() tr_t0 = clock64()
#define PF_TRACE_END(site) tr_acc[site] += clock64() - tr_t0
#define PF_TRACE_FLUSH(role)                                                        \
  if (lane == 0 && p.trace)                                                          \
    for (int i_ = 0; i_ < 8; ++i_)                                                   \
      p.trace[(static_cast<size_t>(blockIdx.x) * 6 + (role)) * 8 + i_] = tr_acc[i_];
// timeline of one CTA: clock of event `ev` of KV tile `t` (counted over the CTA's items)
#define PF_TL(ev, t)                                                                 \
  if (p.trace && blockIdx.x == 5 && (t) < 160u && (threadIdx.x & 31) == 0)           \
    p.trace[148 * 6 * 8 + (t) * 16 + (ev)] = clock64();
// ... and of item-level event `ev` of the CTA's n-th item
#define PF_TLI(ev, n)                                                                \
  if (p.trace && blockIdx.x == 5 && (n) < 32u && (threadIdx.x & 31) == 0)            \
    p.trace[148 * 6 * 8 + 160 * 16 + (n) * 8 + (ev)] = clock64();
#else
#define PF_TL(ev, t)
#define PF_TLI(ev, n)
#define PF_TRACE_DECL
#define PF_TRACE_BEGIN()
#define PF_TRACE_END(site)
#define PF_TRACE_FLUSH(role)
#endif

template <int HD>
struct PrefillSmem {
  static constexpr int kSub = HD / 64;
  static constexpr int kSubBytes = 128 * 128;             // 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;     // one Q, K or V tile
  // K ring and V ring.  At most 3 tiles per ring: a producer learns that slot t % kRing is free
  // from the S / PV barrier of tile t - kRing, which is shared with tile t - kRing + 3.
  static constexpr int kRing = (HD == 128) ? 2 : 3;       // tiles per ring
  static constexpr int kSlots = 2 * kRing;
  static constexpr int kQOff = 0;                         // two Q buffers (by item parity)
  static constexpr int kRingOff = 2 * kTileBytes;
  static constexpr int kSeqOff = kRingOff + kSlots * kTileBytes;
  static constexpr int kPrefixOff = kSeqOff + (kPfSeqCache + 4) * 4;   // blocks before a sequence
  static constexpr int kItemOff = kPrefixOff + (kPfSeqCache + 4) * 4;  // keeps 16-byte alignment
  static constexpr int kTabOff = kItemOff + kPfQueue * 48;             // list position -> block
  static constexpr int kMaxOff = kTabOff + kPfBlockTab * 4;            // running max [tile parity][row]
  static constexpr int kStatOff = kMaxOff + 2 * kPfM * 4;            // (max, sum) [item parity][group][row]
  static constexpr int kBarOff = kStatOff + 2 * 2 * kPfM * 8;
  // q_full[2] q_empty[2] k_full[kRing] v_full[kRing] k_empty[kRing] v_empty[kRing] s_full[3] p_full[3] pv_done[3] m_ready[2]
  // o_full o_empty stat_full[2] stat_empty[2]
  static constexpr int kNumBars = 4 + 2 * kSlots + 17 + kPfQueue;
  static constexpr int kTotalBytes = kBarOff + kNumBars * 8 + 16 + 1024;
  static_assert(kItemOff % 16 == 0, "16-byte vector access alignment");
  static_assert(kBarOff % 8 == 0, "barrier alignment");
  static_assert(kTotalBytes <= 232448, "shared memory budget");
};

// Compact result of the item-order search.
struct PrefillItemKey {
  int seq;    // -1 = no such item
  int q0;
  int head;
  int start;
};

// What every role needs to know about one work item.
struct alignas(16) PrefillItem {
  int seq, head, q0, seq_q_begin, seq_len_q, start;   // seq < 0: end of the CTA's work
  int rows_valid;     // query rows of the item that exist (the last block of a sequence is ragged)
  int first_pos;      // absolute position of the item's first query row
  int j0;             // first KV tile any row attends (0 without a sliding window)
  int n_tiles;        // KV tiles j0 .. j0 + n_tiles - 1
  int pad[2];
};
static_assert(sizeof(PrefillItem) == 48, "queue entries are copied as three 16-byte vectors");

// List position -> (sequence, 128-row block, head) for lists too long to tabulate (more than
// kPfBlockTab blocks or kPfSeqCache sequences): plain sequence order, later blocks of a
// sequence first, found by a scan of cu_q.  Tabulated lists (the common case) are ordered
// heaviest first, see the table build in the kernel's prologue.
__device__ __forceinline__ PrefillItemKey prefill_find_item(const PrefillParams& p,
                                                           const int32_t* cu, uint32_t item) {
  PrefillItemKey key{-1, 0, 0, 0};
  if (item >= static_cast<uint32_t>(p.total_items)) return key;
  key.head = item % p.num_q_heads;
  const int t = item / p.num_q_heads;
  int acc = 0;
  for (int s = 0; s < p.num_seqs; ++s) {
    const int n = (cu[s + 1] - cu[s] + kPfRowsPerItem - 1) / kPfRowsPerItem;
    if (t < acc + n) {
      key.seq = s;
      key.q0 = (n - 1 - (t - acc)) * kPfRowsPerItem;
      key.start = p.q_start ? p.q_start[s] : 0;
      break;
    }
    acc += n;
  }
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
  it.rows_valid = max(0, min(kPfM, it.seq_len_q - it.q0));
  it.first_pos = it.start + it.q0;
  // first key the first row may attend (it starts lowest)
  const int lo = (p.window > 0 && it.first_pos + 1 > p.window) ? it.first_pos + 1 - p.window : 0;
  it.j0 = lo / kPfN;
  const int n_abs = it.rows_valid > 0 ? (it.first_pos + it.rows_valid - 1) / kPfN + 1 : 0;
  it.n_tiles = n_abs - it.j0;
  return it.n_tiles > 0;
}

// The launch's counter word is (tag << 32) | next list position.  CTA b starts with item b, so
// a freshly claimed word stands at num_ctas (prefill_claim, early in every CTA's prologue).
// Drawing the next position is one atomicAdd, issued well before its result is needed
// (prefill_draw_resolve).  Positions >= total are end markers; every CTA that had a first item
// draws exactly one, and the CTA that draws the last of them (position total + num_ctas - 1)
// clears the word.  An add that found another launch's tag in the word did not count: the
// word is claimed and the draw repeated.
__device__ __forceinline__ void prefill_claim(unsigned long long* word, uint32_t tag,
                                              uint32_t num_ctas) {
  const unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(word);
  if (static_cast<uint32_t>(cur >> 32) != tag)
    atomicCAS(word, cur, (static_cast<unsigned long long>(tag) << 32) | num_ctas);
}
__device__ __forceinline__ uint32_t prefill_draw_resolve(unsigned long long* word, uint32_t tag,
                                                         uint32_t total, uint32_t num_ctas,
                                                         unsigned long long drawn) {
  for (int tries = 0; tries < 4096; ++tries) {
    if (static_cast<uint32_t>(drawn >> 32) == tag) {
      const uint32_t idx = static_cast<uint32_t>(drawn);
      if (idx == total + num_ctas - 1u)
        *reinterpret_cast<volatile unsigned long long*>(word) = 0ull;
      return idx;
    }
    // Add again only once the word is this launch's: adds on a word that is still to be
    // claimed would make every claim's compare fail.
    const unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(word);
    if (static_cast<uint32_t>(cur >> 32) == tag)
      drawn = atomicAdd(word, 1ull);
    else
      atomicCAS(word, cur, (static_cast<unsigned long long>(tag) << 32) | num_ctas);
  }
  return 0xffffffffu;   // never seen; reads as an end marker
}

// Bounded mbarrier wait of this kernel.  The kernel has some forty wait sites, and its code size
// is what its instruction fetch stalls follow, so a site is a probe, a polling loop and two
// checks; giving up only raises the CTA's abort flag (every later wait of the CTA then returns
// at once, its results are garbage), and the CTA reports to the diagnostics word once, on its
// way out.
__device__ __forceinline__ bool pf_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > kWaitTimeoutNs) {
      *abort_flag = 1;
      return false;
    }
  }
}

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <int HD, int BS, bool WIN>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
  using L = PrefillSmem<HD>;
  constexpr int kSub = L::kSub;
  constexpr int kPagesPerTile = kPfN / BS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem + L::kQOff;
  uint8_t* ring = smem + L::kRingOff;
  int32_t* cu_smem = reinterpret_cast<int32_t*>(smem + L::kSeqOff);
  int32_t* prefix_smem = reinterpret_cast<int32_t*>(smem + L::kPrefixOff);
  PrefillItem* item_q = reinterpret_cast<PrefillItem*>(smem + L::kItemOff);
  float* m_sh = reinterpret_cast<float*>(smem + L::kMaxOff);          // [tile parity][row]
  float2* stat_sh = reinterpret_cast<float2*>(smem + L::kStatOff);    // [item parity][group][row]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                   // [2] Q of the item landed (TMA -> MMA)
  uint64_t* q_empty = bars + 2;              // [2] last QK of the item retired (MMA -> TMA)
  constexpr int kRing = L::kRing;
  uint64_t* k_full = bars + 4;               // [kRing] K tile landed (TMA -> MMA)
  uint64_t* v_full = k_full + kRing;         // [kRing]
  // S of tile t in buffer t%3 ready = QK(t) retired: wakes the softmax, and tells the K producer
  // that the K slot is free again
  uint64_t* s_full = v_full + kRing;         // [3]
  uint64_t* p_full = s_full + 3;             // [3] P of the tile written (softmax -> PV issuer)
  // PV(t) retired: S_{t%3} may be overwritten (QK issuer), the V slot is free (V producer), O may
  // be rescaled (softmax), and after an item's last tile O is complete (epilogue)
  uint64_t* pv_done = p_full + 3;            // [3]
  uint64_t* m_ready = pv_done + 3;           // [2] running max after an even / odd tile published
  uint64_t* o_empty = m_ready + 2;           // O of the item read out (epilogue -> PV issuer)
  uint64_t* stat_full = o_empty + 1;         // [2] both groups' (max, sum) written
  uint64_t* stat_empty = stat_full + 2;      // [2] ... and read by the epilogue
  uint64_t* item_full = stat_empty + 2;      // [kPfQueue] the n-th item of this CTA is in the queue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = warp >> 2;               // warpgroup = role
#ifdef B200ATTN_PF_TRACE
  const long long tr_entry = clock64();
#endif

  // A CTA of this launch just gave up on a wait: do not repeat the timeout per CTA.
  if (timeout_drain_window(p.err_word)) return;
  if (threadIdx.x == 96) prefill_claim(p.sched, p.sched_tag, gridDim.x);

  const bool cu_cached = p.num_seqs <= kPfSeqCache;
  if (cu_cached)
    for (int s = threadIdx.x; s <= p.num_seqs; s += blockDim.x) cu_smem[s] = p.cu_q[s];
  const int32_t* cu = cu_cached ? cu_smem : p.cu_q;
  // For the item search: batches of many sequences get the number of 128-row blocks before
  // each sequence, small batches (level order) the block count of each sequence.
  const bool use_prefix = cu_cached && p.num_seqs > kPfLevelOrderMaxSeqs;
  if (cu_cached) __syncthreads();
  if (cu_cached && !use_prefix)
    for (int s = threadIdx.x; s < p.num_seqs; s += blockDim.x)
      prefix_smem[s] = (cu[s + 1] - cu[s] + kPfRowsPerItem - 1) / kPfRowsPerItem;
  if (use_prefix && warp == 0) {
    // each lane sums a run of consecutive sequences, a warp scan turns the run totals into offsets
    const int per = (p.num_seqs + 31) / 32;
    const int s0 = lane * per, s1 = min(p.num_seqs, s0 + per);
    int run = 0;
    for (int s = s0; s < s1; ++s) run += (cu[s + 1] - cu[s] + kPfRowsPerItem - 1) / kPfRowsPerItem;
    int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int acc = incl - run;
    for (int s = s0; s < s1; ++s) {
      prefix_smem[s] = acc;
      acc += (cu[s + 1] - cu[s] + kPfRowsPerItem - 1) / kPfRowsPerItem;
    }
  }
  // Small lists are tabulated once (list position -> sequence, block), so that taking an item
  // costs the drawing thread one look-up instead of a search.  Every (sequence, block) pair
  // computes its own position: in the level order, the blocks with a higher index plus the
  // earlier sequences that have a block of this index; in sequence order, the blocks of the
  // sequences before plus the later blocks of its own.
  if (cu_cached && p.total_items / p.num_q_heads <= kPfBlockTab) {
    __syncthreads();
    uint32_t* blk_tab = reinterpret_cast<uint32_t*>(smem + L::kTabOff);   // (sequence << 16) | block
    const int S = p.num_seqs;
    if (!use_prefix) {
      const int lanes_per_seq = static_cast<int>(blockDim.x) / S;    // S <= 64 < blockDim.x
      const int s_mine = static_cast<int>(threadIdx.x) % S;
      if (static_cast<int>(threadIdx.x) < S * lanes_per_seq) {
        const int n_mine = prefix_smem[s_mine];
        for (int r = static_cast<int>(threadIdx.x) / S; r < n_mine; r += lanes_per_seq) {
          int pos = 0;
          for (int s2 = 0; s2 < S; ++s2) {
            const int n2 = prefix_smem[s2];
            pos += max(0, n2 - 1 - r) + ((s2 < s_mine && n2 > r) ? 1 : 0);
          }
          blk_tab[pos] = (static_cast<uint32_t>(s_mine) << 16) | static_cast<uint32_t>(r);
        }
      }
    } else {
      for (int s2 = threadIdx.x; s2 < S; s2 += blockDim.x) {
        const int n2 = (cu[s2 + 1] - cu[s2] + kPfRowsPerItem - 1) / kPfRowsPerItem;
        for (int r = 0; r < n2; ++r)
          blk_tab[prefix_smem[s2] + n2 - 1 - r] = (static_cast<uint32_t>(s2) << 16) | static_cast<uint32_t>(r);
      }
    }
  }
  // The n-th item of this CTA: false at the end marker (and once a wait of this CTA has been
  // abandoned).  The K producer's lane 0 wrote the entry, fully expanded, so that taking it is a
  // wait and three vector loads for everybody else.
  auto take_item = [&](uint32_t n, PrefillItem& it) {
    pf_wait(&item_full[n % kPfQueue], (n / kPfQueue) & 1, abort_flag);
    if (*abort_flag) return false;
    const uint4* src = reinterpret_cast<const uint4*>(&item_q[n % kPfQueue]);
    uint4* dst = reinterpret_cast<uint4*>(&it);
    dst[0] = src[0];
    dst[1] = src[1];
    dst[2] = src[2];
    return it.seq >= 0;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&m_ready[i], 128);
      mbar_init(&stat_full[i], 256);
      mbar_init(&stat_empty[i], 128);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(o_empty, 128);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
    }
    for (int i = 0; i < kPfQueue; ++i) mbar_init(&item_full[i], 1);
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
  // columns: S_0 [0,128)  S_1 [128,256)  S_2 [256,384)  O [384,384+HD)

  if (group == 0) {
    setmaxnreg_dec<kPfRegsProducer>();
    if (warp == 0 || warp == 2) {
      // ------------------------------------------------------------------ TMA producers
      // warp 0: Q and K tiles; warp 2: V tiles.  Ring slot of tile t (counted over all items of
      // this CTA): t % kRing of the K ring / of the V ring.
      const bool is_v = warp == 2;
      if (lane == 0) {
        prefetch_tensormap(is_v ? &tm_v : &tm_k);
        if (!is_v) prefetch_tensormap(&tm_q);
      }
      const uint64_t pol_q = l2_policy_evict_first();
      const uint64_t pol_kv = l2_policy_evict_last();
      const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
      uint64_t* full = is_v ? v_full : k_full;
      uint64_t* retired = is_v ? pv_done : s_full;    // the MMA group that read a slot has retired
      uint8_t* my_ring = ring + (is_v ? kRing * L::kTileBytes : 0);
      uint32_t t = 0, item_n = 0;
      PF_TRACE_DECL
#ifdef B200ATTN_PF_TRACE
      const long long tr_start = clock64();
#endif
      // The K producer is the role that runs furthest ahead: its lane 0 draws the CTA's items
      // from the launch's list and queues them for everybody.  The atomic that draws item n + 1
      // is issued behind the second-to-last K tile of item n and its result is looked at once
      // the last K tile of item n has been issued, so its latency stays off the loads' path.
      bool more = !is_v && lane == 0;
      unsigned long long drawn = 0;
      const bool use_tab = cu_cached && p.total_items / p.num_q_heads <= kPfBlockTab;
      const uint32_t* blk_tab = reinterpret_cast<const uint32_t*>(smem + L::kTabOff);
      auto draw = [&]() {
        if (more) drawn = atomicAdd(p.sched, 1ull);
      };
      auto publish = [&](uint32_t n) {
        if (more) {
          // the first item of a CTA is the one with its own index: the list is drawn from
          // position gridDim.x on, and no atomic stands before the first loads
          const uint32_t idx =
              n == 0 ? blockIdx.x
                     : prefill_draw_resolve(p.sched, p.sched_tag,
                                            static_cast<uint32_t>(p.total_items), gridDim.x, drawn);
          PrefillItemKey key{-1, 0, 0, 0};
          if (idx < static_cast<uint32_t>(p.total_items)) {
            if (use_tab) {
              const uint32_t e = blk_tab[idx / p.num_q_heads];
              key.seq = static_cast<int>(e >> 16);
              key.q0 = static_cast<int>(e & 0xffffu) * kPfRowsPerItem;
              key.head = idx % p.num_q_heads;
              key.start = p.q_start ? p.q_start[key.seq] : 0;
            } else {
              key = prefill_find_item(p, cu, idx);
            }
          }
          PrefillItem full;
          if (!prefill_expand_item(p, key, cu, full)) full.seq = -1;
          more = full.seq >= 0;
          item_q[n % kPfQueue] = full;
          mbar_arrive(&item_full[n % kPfQueue]);
        }
      };
      publish(0);
      for (uint32_t n = 0;; ++n) {
        __syncwarp();
        PrefillItem it;
        if (!take_item(n, it)) break;
        const int kvh = it.head / p.group;
        if (!is_v) {
          const int ip = item_n & 1;
          // the Q buffer is free once every QK of the item two back has retired
          PF_TRACE_BEGIN();
          pf_wait(&q_empty[ip], ((item_n >> 1) & 1) ^ 1, abort_flag);
          PF_TRACE_END(0);
          if (lane == 0) {
            mbar_arrive_expect_tx(&q_full[ip], L::kTileBytes);
#pragma unroll
            for (int s = 0; s < kSub; ++s)
              tma_load_2d(q_smem + ip * L::kTileBytes + s * L::kSubBytes, &tm_q, &q_full[ip],
                          it.head * HD + s * 64, it.seq_q_begin + it.q0, pol_q);
          }
        }
        ++item_n;
        const int32_t* pt = p.page_table + static_cast<int64_t>(it.seq) * p.page_table_stride;
        const int last_pos = it.first_pos + it.rows_valid - 1;
        const int n_pages = last_pos / BS + 1;      // pages holding keys 0 .. last_pos
        for (int i = 0; i < it.n_tiles; ++i, ++t) {
          const int j = it.j0 + i;                             // absolute KV tile
          const int slot = t % kRing;
          if (t >= static_cast<uint32_t>(kRing)) {     // the slot held tile t - kRing
            const uint32_t u = t - kRing;
            PF_TRACE_BEGIN();
            pf_wait(&retired[u % 3u], (u / 3u) & 1, abort_flag);
            PF_TRACE_END(1);
          }
          PF_TL(is_v ? 14 : 13, t)
          uint8_t* dst = my_ring + slot * L::kTileBytes;
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
          // late, so that the CTA commits to its next item when it is about to need it (a
          // draw at the start of a long item would hand this CTA work that an idle one should
          // take), but a tile before the result is looked at
          if (i == max(0, it.n_tiles - 2)) draw();
        }
        publish(n + 1);
      }
#ifdef B200ATTN_PF_TRACE
      tr_acc[7] = clock64() - tr_start;
      tr_acc[6] = t;
#endif
      PF_TRACE_FLUSH(is_v ? 1 : 0)
    } else {
      // ------------------------------------------------------------------ MMA issuers
      // warp 1: QK, warp 3: PV.  The whole warp walks the schedule (so addresses and descriptors
      // stay warp-uniform); lane 0 issues.
      const bool is_pv = warp == 3;
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kPfM, kPfN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kPfM, HD, false, true);
      // high descriptor word: SBO = 1024 B, descriptor version 1, 128-byte swizzle
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLboV = (static_cast<uint32_t>(L::kSubBytes) >> 4) << 16;  // V: next 64 d
      constexpr uint32_t kLboK = 1u << 16;                                          // unused field
      const bool leader = lane == 0;
      PF_TRACE_DECL
#ifdef B200ATTN_PF_TRACE
      const long long tr_start = clock64();
#endif
      auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
      uint8_t* k_ring = ring;
      uint8_t* v_ring = ring + kRing * L::kTileBytes;
      uint32_t t = 0, item_no = 0;
      for (;;) {
        PrefillItem it;
        PF_TLI(is_pv ? 0 : 2, item_no)
        if (!take_item(item_no, it)) break;
        PF_TLI(is_pv ? 1 : 3, item_no)
        const int n = it.n_tiles;
        const int ip = item_no & 1;
        if (!is_pv) {
          PF_TRACE_BEGIN();
          pf_wait(&q_full[ip], (item_no >> 1) & 1, abort_flag);
          PF_TRACE_END(0);
          PF_TLI(4, item_no)
        }
        const uint32_t q_lo = (smem_u32(q_smem + ip * L::kTileBytes) >> 4) | kLboK;
        const int last_pos = it.first_pos + it.rows_valid - 1;
        for (int j = 0; j < n; ++j, ++t) {
          const uint32_t b = t % 3u;
          const uint32_t slot = t % kRing;
          if (!is_pv) {
            // ---- S_b = Q K_t^T
            PF_TRACE_BEGIN();
            pf_wait(&k_full[slot], (t / kRing) & 1, abort_flag);
            PF_TRACE_END(1);
            PF_TL(0, t)
            if (t >= 3) {     // S_b still holds P of tile t-3 until its PV has retired
              PF_TRACE_BEGIN();
              pf_wait(&pv_done[b], ((t - 3) / 3u) & 1, abort_flag);
              PF_TRACE_END(2);
            }
            PF_TL(1, t)
            tc_fence_after_sync();
            const uint32_t k_lo = (smem_u32(k_ring + slot * L::kTileBytes) >> 4) | kLboK;
            const uint32_t d = tmem_base + b * kPfN;
            if (leader) {
#pragma unroll
              for (int kk = 0; kk < HD / 16; ++kk) {
                const uint32_t off = ((kk >> 2) * L::kSubBytes + (kk & 3) * 32) >> 4;
                umma_ss(d, desc(q_lo + off), desc(k_lo + off), idesc_qk, kk > 0);
              }
              umma_commit(&s_full[b]);
              // the last QK of the item has been issued: its Q buffer is free once it retires
              if (j == n - 1) umma_commit(&q_empty[ip]);
            }
            PF_TL(2, t)
          } else {
            // ---- O (+)= P_t V_t
            uint8_t* vt = v_ring + slot * L::kTileBytes;
            PF_TRACE_BEGIN();
            pf_wait(&v_full[slot], (t / kRing) & 1, abort_flag);
            PF_TRACE_END(1);
            PF_TL(3, t)
            if (j == n - 1) {
              // Keys past the item's last query row are masked in P, but 0 x (stale, possibly
              // non-finite cache contents) would still poison the row: zero those V rows.
              const int first_dead = last_pos + 1 - (it.j0 + j) * kPfN;     // row inside the tile
              if (first_dead < kPfN) {
                const int vecs = (kPfN - first_dead) * 8;   // 16-byte vectors per 64-wide sub-tile
                for (int s = 0; s < kSub; ++s)
                  for (int i = lane; i < vecs; i += 32)
                    *reinterpret_cast<uint4*>(vt + s * L::kSubBytes + first_dead * 128 + i * 16) =
                        make_uint4(0u, 0u, 0u, 0u);
                fence_proxy_async_smem();
                __syncwarp();
              }
            }
            PF_TRACE_BEGIN();
            pf_wait(&p_full[b], (t / 3u) & 1, abort_flag);
            PF_TRACE_END(3);
            PF_TL(4, t)
            if (j == 0) {   // O of the item before must have been read out before it is overwritten
              PF_TRACE_BEGIN();
              pf_wait(o_empty, (item_no & 1) ^ 1, abort_flag);
              PF_TRACE_END(4);
            }
            PF_TL(5, t)
            tc_fence_after_sync();
            const uint32_t p_tmem = tmem_base + b * kPfN;   // P over the first 64 columns of S_b
            const uint32_t v_lo = (smem_u32(vt) >> 4) | kLboV;
            const uint32_t d = tmem_base + 3 * kPfN;
            if (leader) {
#pragma unroll
              for (int kk = 0; kk < kPfN / 16; ++kk) {
                // A: 16 keys = 8 packed 32-bit columns per step; B: 16 keys = 2048 B further on
                umma_ts(d, p_tmem + kk * 8, desc(v_lo + kk * (2048 >> 4)), idesc_pv,
                        (j > 0) || (kk > 0));
              }
              umma_commit(&pv_done[b]);
            }
            PF_TL(6, t)
          }
        }
        ++item_no;
      }
#ifdef B200ATTN_PF_TRACE
      tr_acc[7] = clock64() - tr_start;
      tr_acc[6] = t;
      tr_acc[5] = tr_start - tr_entry;     // prologue: entry to the start of the role
#endif
      PF_TRACE_FLUSH(is_pv ? 5 : 2)
    }
  } else if (group <= 2) {
    // ------------------------------------------------------------------ softmax, even / odd tiles
    setmaxnreg_inc<kPfRegsSoftmax>();
    const uint32_t w = group - 1;                        // parity of the tiles this group takes
    const int row = (warp & 3) * 32 + lane;              // tensor-memory lane == query row
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t o_addr = tmem_base + 3 * kPfN + lane_addr;
    const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint32_t t0 = 0;                    // global index of the item's first tile
    uint32_t item_no = 0;
    PF_TRACE_DECL
#ifdef B200ATTN_PF_TRACE
    const long long tr_start = clock64();
#endif
    for (;;) {
      PrefillItem it;
      if (!take_item(item_no, it)) break;
      const int ip = item_no & 1;
      const int q_pos = it.first_pos + row;
      float l_run = 0.f, m_last = -INFINITY;   // this group's row sum, relative to m_last
      for (int jr = 0; jr < it.n_tiles; ++jr) {
        const uint32_t t = t0 + jr;
        if ((t & 1u) != w) continue;
        const uint32_t b = t % 3u;                       // S / P buffer of the tile
        const uint32_t s_addr = tmem_base + b * kPfN + lane_addr;
        const int j = it.j0 + jr;                        // absolute KV tile
        PF_TRACE_BEGIN();
        pf_wait(&s_full[b], (t / 3u) & 1, abort_flag);
        PF_TRACE_END(0);
#ifdef B200ATTN_PF_TRACE
        const long long tr_tile = clock64();
        if ((warp & 3) == 0) { PF_TL(7, t) }
#endif
        tc_fence_after_sync();
#ifdef B200ATTN_PF_NOSOFTMAX
        if (t > 0) pf_wait(&m_ready[w ^ 1u], (((t + 1) >> 1) - 1) & 1, abort_flag);
        mbar_arrive(&m_ready[w]);
        tc_fence_before_sync();
        mbar_arrive(&p_full[b]);
        continue;
#endif
        uint32_t sreg[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, sreg[c]);
        tmem_wait_ld();
#ifdef B200ATTN_PF_TRACE
        const long long tr_ld = clock64();
        tr_acc[3] += tr_ld - tr_tile;
        if ((warp & 3) == 0) { PF_TL(8, t) }
#endif

        const int key0 = j * kPfN;
        if (key0 + kPfN - 1 > it.first_pos) {   // tile crosses the diagonal for some row
          const int lim = q_pos - key0;                                // the row sees keys 0 .. lim
          const int lim_w = it.first_pos + (warp & 3) * 32 - key0;     // ... of the warp's first row
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (lim_w < c * 32 + 31) {    // warp-uniform: some row of the warp loses a key of this chunk
#pragma unroll
              for (int kx = 0; kx < 32; ++kx)
                asm("{\n\t.reg .pred p;\n\t"
                    "setp.lt.s32 p, %1, %2;\n\t"
                    "selp.b32 %0, 0xff800000, %0, p;\n\t}"       // -inf
                    : "+r"(sreg[c][kx])
                    : "r"(lim), "r"(c * 32 + kx));
            }
          }
        }
#ifdef B200ATTN_PF_TRACE
        if ((warp & 3) == 0) { PF_TL(15, t) }
#endif
        if (WIN && key0 < it.first_pos + kPfM - p.window) {   // below some row's window
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int kx = 0; kx < 32; ++kx)
              if (key0 + c * 32 + kx + p.window <= q_pos) sreg[c][kx] = 0xff800000u;   // -inf
        }
        // row max of the raw scores (scale > 0), four independent chains
        float mx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mx[c] = max3(__uint_as_float(sreg[c][0]), __uint_as_float(sreg[c][1]),
                       __uint_as_float(sreg[c][2]));
#pragma unroll
          for (int kx = 3; kx + 1 < 32; kx += 2)
            mx[c] = max3(mx[c], __uint_as_float(sreg[c][kx]), __uint_as_float(sreg[c][kx + 1]));
          mx[c] = fmaxf(mx[c], __uint_as_float(sreg[c][31]));
        }
        const float mx_s = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
#ifdef B200ATTN_PF_TRACE
        const long long tr_mx = clock64();
        tr_acc[4] += tr_mx - tr_ld;
        if ((warp & 3) == 0) { PF_TL(9, t) }
#endif
        // running max after the tile before (the other group publishes it as soon as it has it)
        float m_prev = -INFINITY;
        if (t > 0) {
          const uint32_t other = (t + 1) >> 1;           // tiles of the other parity before t
          PF_TRACE_BEGIN();
          pf_wait(&m_ready[w ^ 1u], (other - 1) & 1, abort_flag);
          PF_TRACE_END(1);
          if (jr > 0) m_prev = m_sh[(w ^ 1u) * kPfM + row];
        }
        float m_new = m_prev;
        if (mx_s - m_prev > kPfRescaleThreshold) m_new = mx_s;   // also taken when m_prev = -inf
        m_sh[w * kPfM + row] = m_new;
        mbar_arrive(&m_ready[w]);
        // a row whose keys are all masked so far (possible only under a sliding window) keeps
        // m = -inf: its weights and its correction factor are 0, not exp2(-inf + inf)
        const bool rescale = (jr > 0) && (m_new != m_prev);
        // p = 2^(s*scale - m): packed FMA, then ex2; two packed running sums.  Each 32-key
        // chunk goes straight back to tensor memory as 16 packed bf16x2 columns.  QK of this
        // tile has retired (s_full) and the PV that read the buffer before was issued ahead of
        // it, so the S / P columns are quiescent.
#ifdef B200ATTN_PF_TRACE
        const long long tr_ex = clock64();
        if ((warp & 3) == 0) { PF_TL(10, t) }
#endif
        const float m_sub = (WIN && m_new == -INFINITY) ? 0.f : m_new;
        const uint64_t negm2 = pack_f32x2(-m_sub, -m_sub);
        uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t preg[16];
#pragma unroll
          for (int kx = 0; kx < 32; kx += 2) {
            const uint64_t x2 = fma_f32x2(
                pack_f32x2(__uint_as_float(sreg[c][kx]), __uint_as_float(sreg[c][kx + 1])), scale2,
                negm2);
            float x0, x1, e0, e1;
            unpack_f32x2(x2, x0, x1);
            if (kPfPolyEvery > 0 && ((kx >> 1) % (kPfPolyEvery > 0 ? kPfPolyEvery : 1)) ==
                                        (kPfPolyEvery - 1)) {
              exp2_poly_f32x2(x0, x1, e0, e1);
            } else {
              e0 = fast_exp2(x0);
              e1 = fast_exp2(x1);
            }
            sum2[(kx >> 1) & 1] = add_f32x2(sum2[(kx >> 1) & 1], pack_f32x2(e0, e1));
            preg[kx >> 1] = pack_bf16x2(e0, e1);
          }
          tmem_st_32x16(s_addr + c * 16, preg);
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(sum2[0], a0, a1);
          unpack_f32x2(sum2[1], b0, b1);
          // this group's sum is relative to the max at ITS previous tile
          const float f = (m_last == -INFINITY) ? 0.f : fast_exp2(m_last - m_new);
          l_run = l_run * f + ((a0 + a1) + (b0 + b1));
          m_last = m_new;
        }
#ifdef B200ATTN_PF_TRACE
        const long long tr_ex1 = clock64();
        tr_acc[5] += tr_ex1 - tr_ex;
        if ((warp & 3) == 0) { PF_TL(11, t) }
#endif
        // O row rescale (rare: only when the running max moved by more than the threshold):
        // every PV up to the tile before must have retired; PV of this tile waits for p_full.
        if (__any_sync(0xffffffffu, rescale)) {
          pf_wait(&pv_done[(t - 1) % 3u], ((t - 1) / 3u) & 1, abort_flag);
          tc_fence_after_sync();
          const float corr =
              !rescale ? 1.f : ((WIN && m_prev == -INFINITY) ? 0.f : fast_exp2(m_prev - m_new));
          const uint64_t f2 = pack_f32x2(corr, corr);
#pragma unroll 1   // rare path: keep it small
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t oreg[32];
            tmem_ld_32x32(o_addr + c * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int kx = 0; kx < 32; kx += 2) {
              float y0, y1;
              unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(oreg[kx]),
                                                __uint_as_float(oreg[kx + 1])), f2), y0, y1);
              oreg[kx] = __float_as_uint(y0);
              oreg[kx + 1] = __float_as_uint(y1);
            }
            tmem_st_32x32(o_addr + c * 32, oreg);
          }
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&p_full[b]);
#ifdef B200ATTN_PF_TRACE
        tr_acc[6] += clock64() - tr_ex1;
        if ((warp & 3) == 0) { PF_TL(12, t) }
#endif
      }
      // ---- item end: hand this group's (max, sum) of the row to the epilogue
      PF_TRACE_BEGIN();
      pf_wait(&stat_empty[ip], ((item_no >> 1) & 1) ^ 1, abort_flag);
      PF_TRACE_END(2);
      stat_sh[(ip * 2 + w) * kPfM + row] = make_float2(m_last, l_run);
      mbar_arrive(&stat_full[ip]);
      t0 += it.n_tiles;
      ++item_no;
    }
#ifdef B200ATTN_PF_TRACE
    tr_acc[7] = clock64() - tr_start;
#endif
    if (warp == 4 || warp == 8) { PF_TRACE_FLUSH(3 + w) }
  } else {
    // ------------------------------------------------------------------ epilogue
    setmaxnreg_dec<kPfRegsEpilogue>();
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t item_no = 0;
    uint32_t t_end = 0;                 // tiles of all items up to and including this one
    PF_TRACE_DECL
#ifdef B200ATTN_PF_TRACE
    const long long tr_start = clock64();
#endif
    for (;;) {
      PrefillItem it;
      if (!take_item(item_no, it)) break;
      const int ip = item_no & 1;
      const uint32_t ph = (item_no >> 1) & 1;
      t_end += it.n_tiles;
      const uint32_t o_addr = tmem_base + 3 * kPfN + lane_addr;
      PF_TRACE_BEGIN();
      pf_wait(&stat_full[ip], ph, abort_flag);
      PF_TRACE_END(0);
      if ((warp & 3) == 0) { PF_TLI(5, item_no) }
      const float2 s0 = stat_sh[(ip * 2 + 0) * kPfM + row];
      const float2 s1 = stat_sh[(ip * 2 + 1) * kPfM + row];
      mbar_arrive(&stat_empty[ip]);
      // O is relative to the max after the last tile, which is the larger of the two
      const float m_fin = fmaxf(s0.x, s1.x);
      const float l = (s0.x == -INFINITY ? 0.f : s0.y * fast_exp2(s0.x - m_fin)) +
                      (s1.x == -INFINITY ? 0.f : s1.y * fast_exp2(s1.x - m_fin));
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      PF_TRACE_BEGIN();      // the PV of the item's last tile
      pf_wait(&pv_done[(t_end - 1) % 3u], ((t_end - 1) / 3u) & 1, abort_flag);
      PF_TRACE_END(1);
#ifdef B200ATTN_PF_TRACE
      const long long tr_ep = clock64();
      if ((warp & 3) == 0) { PF_TLI(6, item_no) }
#endif
      tc_fence_after_sync();
      __nv_bfloat16* orow =
          p.out + static_cast<int64_t>(it.seq_q_begin + it.q0 + row) * p.out_row_stride +
          static_cast<int64_t>(it.head) * HD;
      const bool store = row < it.rows_valid;
#pragma unroll 1   // once per item: small code matters more than the unrolled form's few cycles
      for (int c = 0; c < HD / 16; ++c) {
        uint32_t oreg[16];
        tmem_ld_32x16(o_addr + c * 16, oreg);
        tmem_wait_ld();
        if (c == HD / 16 - 1) {      // O sits in registers: hand the buffer back to the MMA warp
          tc_fence_before_sync();
          mbar_arrive(o_empty);
#ifdef B200ATTN_PF_TRACE
          tr_acc[2] += clock64() - tr_ep;
          if ((warp & 3) == 0) { PF_TLI(7, item_no) }
#endif
        }
        uint32_t packed[8];
#pragma unroll
        for (int kx = 0; kx < 16; kx += 2)
          packed[kx >> 1] = pack_bf16x2(__uint_as_float(oreg[kx]) * inv_l,
                                        __uint_as_float(oreg[kx + 1]) * inv_l);
        if (store) {
          *reinterpret_cast<uint4*>(orow + c * 16) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(orow + c * 16 + 8) =
              make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
      ++item_no;
    }
#ifdef B200ATTN_PF_TRACE
    tr_acc[7] = clock64() - tr_start;
    tr_acc[6] = item_no;
#endif
    (void)item_no;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) report_wait_timeout(p.err_word);
}

}  // namespace b200attn
