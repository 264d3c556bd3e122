// Causal varlen / chunked prefill attention on tcgen05 tensor cores.
//
// One CTA = 128 query rows of one sequence x one query head.  KV is consumed in tiles of
// 128 keys.  Six warps:
//   warp 0      TMA producer: Q once, then K_j, V_j, K_j+1, ... into a 4-slot ring of
//               [2 x 128 rows x 128 B] swizzled sub-tiles (paged source: one box per page;
//               fresh source: one box per 64-wide column group).
//   warp 1      allocates tensor memory and issues tcgen05.mma from one thread:
//               S_j = Q K_j^T (two S buffers, so S_j+1 is computed while S_j is in softmax)
//               and O += P_j V_j (V as an MN-major B operand straight from the paged layout).
//   warps 2-5   one thread per query row: tcgen05.ld the row of S, scale + causal mask,
//               running max with a lazy rescale threshold, exp2, row sum, P as bf16 into a
//               swizzled shared-memory tile (the A operand of the PV MMA); rescales its O
//               row in tensor memory when the running max moved; at the end normalises O by
//               1/l and stores bf16.
// Every mbarrier wait is bounded; tensor memory is always freed before exit.
#pragma once
#include "ptx.cuh"

namespace b200attn {

constexpr int kPfM = 128;        // query rows per CTA
constexpr int kPfN = 128;        // keys per tile
constexpr int kPfThreads = 192;
constexpr int kPfSlots = 4;      // ring slots (each holds one K or one V tile)
constexpr float kPfRescaleThreshold = 8.f;  // log2 units

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
  int64_t num_blocks;
  float scale_log2;
  int* err_word;
};

template <int HD>
struct PrefillSmem {
  static constexpr int kSub = HD / 64;
  static constexpr int kSubBytes = 128 * 128;             // 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;     // Q, K or V tile
  static constexpr int kPBytes = 2 * kSubBytes;           // P: 128 rows x 128 keys bf16
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kTileBytes;
  static constexpr int kRingOff = kPOff + kPBytes;
  static constexpr int kBarOff = kRingOff + kPfSlots * kTileBytes;
  static constexpr int kNumBars = 1 + 2 * kPfSlots + 2 + 2 + 2;
  static constexpr int kTotalBytes = kBarOff + kNumBars * 8 + 16 + 1024;
};

template <int HD, int BS>
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
  uint8_t* p_smem = smem + L::kPOff;
  uint8_t* ring = smem + L::kRingOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* full = bars + 1;                 // [kPfSlots]
  uint64_t* empty = full + kPfSlots;         // [kPfSlots]
  uint64_t* s_full = empty + kPfSlots;       // [2]
  uint64_t* s_empty = s_full + 2;            // [2]
  uint64_t* p_full = s_empty + 2;            // [1]
  uint64_t* pv_done = p_full + 1;            // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A CTA of this launch already gave up on a wait: do not repeat the timeout per CTA.
  if (*reinterpret_cast<volatile int*>(p.err_word) == kDevWaitTimeout) return;

  // ---- which (sequence, query tile) is this CTA?  Heavy (late) tiles are scheduled first.
  int tile_linear = gridDim.x - 1 - blockIdx.x;
  int seq = -1, q0 = 0, seq_q_begin = 0, seq_len_q = 0;
  {
    int acc = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int b = p.cu_q[s], e = p.cu_q[s + 1];
      const int nt = (e - b + kPfM - 1) / kPfM;
      if (tile_linear < acc + nt) {
        seq = s;
        q0 = (tile_linear - acc) * kPfM;
        seq_q_begin = b;
        seq_len_q = e - b;
        break;
      }
      acc += nt;
    }
  }
  if (seq < 0) return;  // uniform for the whole CTA; nothing allocated yet
  const int head = blockIdx.y;
  const int kvh = head / p.group;
  const int start = p.q_start ? p.q_start[seq] : 0;
  const int rows_valid = min(kPfM, seq_len_q - q0);
  const int first_pos = start + q0;                   // absolute position of row 0
  const int last_pos = first_pos + rows_valid - 1;    // last valid row
  const int n_tiles = last_pos / kPfN + 1;            // key tiles 0 .. n_tiles-1

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kPfSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
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
  const uint32_t tmem_s0 = tmem_base;          // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;     // O: columns [256, 256+HD)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      const uint64_t pol_q = l2_policy_evict_first();
      mbar_arrive_expect_tx(q_full, L::kTileBytes);
#pragma unroll
      for (int s = 0; s < kSub; ++s)
        tma_load_2d(q_smem + s * L::kSubBytes, &tm_q, q_full, head * HD + s * 64,
                    seq_q_begin + q0, pol_q);
    }
    const uint64_t pol_kv = l2_policy_evict_last();
    const int32_t* pt = p.page_table + static_cast<int64_t>(seq) * p.page_table_stride;
    const int n_pages = (last_pos + BS) / BS;   // pages holding keys 0 .. last_pos
    for (int i = 0; i < 2 * n_tiles; ++i) {
      const int j = i >> 1;
      const bool is_v = i & 1;
      const int slot = i % kPfSlots;
      mbar_wait(&empty[slot], ((i / kPfSlots) & 1) ^ 1, abort_flag, p.err_word);
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
                      seq_q_begin + j * kPfN, pol_kv);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kPfM, kPfN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kPfM, HD, false, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t p_addr = smem_u32(p_smem);
      auto issue_qk = [&](int j) {
        const int i = 2 * j, slot = i % kPfSlots;
        mbar_wait(&full[slot], (i / kPfSlots) & 1, abort_flag, p.err_word);
        if (j >= 2) mbar_wait(&s_empty[j & 1], ((j - 2) >> 1) & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(ring + slot * L::kTileBytes);
        const uint32_t d = tmem_s0 + (j & 1) * kPfN;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * L::kSubBytes + (kk & 3) * 32;
          umma_ss(d, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                  umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk > 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&empty[slot]);
      };
      mbar_wait(q_full, 0, abort_flag, p.err_word);
      issue_qk(0);
      for (int j = 0; j < n_tiles; ++j) {
        if (j + 1 < n_tiles) issue_qk(j + 1);
        const int i = 2 * j + 1, slot = i % kPfSlots;
        mbar_wait(&full[slot], (i / kPfSlots) & 1, abort_flag, p.err_word);
        mbar_wait(p_full, j & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(ring + slot * L::kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kPfN / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * L::kSubBytes + (kk & 3) * 32;
          umma_ss(tmem_o, umma_smem_desc_sw128(p_addr + a_off, 16, 1024),
                  umma_smem_desc_sw128(v_addr + kk * 2048, L::kSubBytes, 1024), idesc_pv,
                  (j > 0) || (kk > 0));
        }
        umma_commit(pv_done);
        umma_commit(&empty[slot]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int row = (warp & 3) * 32 + lane;              // tensor-memory lane == query row
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_pos = first_pos + row;
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.err_word);
      tc_fence_after_sync();
      uint32_t sreg[4][32];
      const uint32_t s_addr = tmem_s0 + (j & 1) * kPfN + lane_addr;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, sreg[c]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&s_empty[j & 1]);

      const int key0 = j * kPfN;
      const bool need_mask = key0 + kPfN - 1 > first_pos;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          float v = __uint_as_float(sreg[c][k]) * p.scale_log2;
          if (need_mask && (key0 + c * 32 + k > q_pos)) v = -INFINITY;
          sreg[c][k] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      float m_new = m_run;
      if (mx - m_run > kPfRescaleThreshold) m_new = mx;   // also taken when m_run = -inf
      const float corr = fast_exp2(m_run - m_new);
      const bool rescale = (m_new != m_run) && (j > 0);
      m_run = m_new;
      float sum = 0.f;
      uint32_t preg[64];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          const float e0 = fast_exp2(__uint_as_float(sreg[c][k]) - m_new);
          const float e1 = fast_exp2(__uint_as_float(sreg[c][k + 1]) - m_new);
          sum += e0 + e1;
          preg[(c * 32 + k) >> 1] = pack_bf16x2(e0, e1);
        }
      l_run = l_run * corr + sum;

      if (j > 0) {
        // PV_{j-1} must have retired before P is overwritten or O is rescaled.
        mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, rescale)) {
          const float f = rescale ? corr : 1.f;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t oreg[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) oreg[k] = __float_as_uint(__uint_as_float(oreg[k]) * f);
            tmem_st_32x32(tmem_o + lane_addr + c * 32, oreg);
          }
          tmem_wait_st();
        }
      }
      // P row -> swizzled K-major tile: 16-byte chunk jj covers keys jj*8 .. jj*8+7.
      const uint32_t p_row = smem_u32(p_smem) + row * 128;
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const uint32_t a = p_row + (jj >> 3) * L::kSubBytes + (((jj & 7) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(preg[jj * 4]),
                     "r"(preg[jj * 4 + 1]), "r"(preg[jj * 4 + 2]), "r"(preg[jj * 4 + 3])
                     : "memory");
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16 rows
    mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag, p.err_word);
    tc_fence_after_sync();
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.out + static_cast<int64_t>(seq_q_begin + q0 + row) * p.out_row_stride +
                          static_cast<int64_t>(head) * HD;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t oreg[32];
      tmem_ld_32x32(tmem_o + lane_addr + c * 32, oreg);
      tmem_wait_ld();
      if (row < rows_valid) {
#pragma unroll
        for (int k = 0; k < 32; k += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(oreg[k]) * inv_l, __uint_as_float(oreg[k + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(oreg[k + 2]) * inv_l,
                            __uint_as_float(oreg[k + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(oreg[k + 4]) * inv_l,
                            __uint_as_float(oreg[k + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(oreg[k + 6]) * inv_l,
                            __uint_as_float(oreg[k + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + k) = v;
        }
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
