// Causal varlen / chunked prefill attention on tcgen05 tensor cores.
//
// One CTA = 2 x 128 query rows (tiles A and B) of one sequence x one query head.  KV is
// consumed in tiles of 128 keys, shared by both query tiles.  Ten warps:
//   warp 0      TMA producer: Q_A and Q_B once, then K_0, V_0, K_1, V_1, ... into a ring of
//               swizzled [128 rows x 128 B] sub-tiles (paged source: one box per page; fresh
//               source: one box per 64-wide column group).
//   warp 1      allocates tensor memory (S_A, S_B, O_A, O_B = 512 columns) and issues
//               tcgen05.mma from one thread in the order
//                   PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1), ...
//               so that the tensor pipe works for one query tile while the other tile's
//               softmax runs.  S = Q K^T has both operands K-major; O += P V takes V as an
//               MN-major B operand straight from the paged [key][d] layout.
//   warps 2-5   softmax warpgroup of tile A, warps 6-9 of tile B; one thread per query row:
//               tcgen05.ld the row of S, causal mask on diagonal tiles, running max with a
//               lazy rescale threshold, ex2 via packed fp32 FMA, row sum, P as bf16 into a
//               swizzled shared-memory tile (the A operand of the PV MMA); rescales its O row
//               in tensor memory when the running max moved; at the end normalises O by 1/l
//               and stores bf16.
// Every mbarrier wait is bounded; tensor memory is always freed before exit.
#pragma once
#include "ptx.cuh"

namespace b200attn {

constexpr int kPfM = 128;        // query rows per tile
constexpr int kPfQTiles = 2;     // query tiles per CTA
constexpr int kPfRowsPerCta = kPfM * kPfQTiles;
constexpr int kPfN = 128;        // keys per KV tile
constexpr int kPfThreads = 320;
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
  static constexpr int kTileBytes = kSub * kSubBytes;     // one Q, K or V tile
  static constexpr int kPBytes = 2 * kSubBytes;           // P: 128 rows x 128 keys bf16
  static constexpr int kSlots = (HD == 128) ? 3 : 6;      // ring slots (one K or V tile each)
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kPfQTiles * kTileBytes;
  static constexpr int kRingOff = kPOff + kPfQTiles * kPBytes;
  static constexpr int kBarOff = kRingOff + kSlots * kTileBytes;
  static constexpr int kNumBars = 1 + 2 * kSlots + 3 * kPfQTiles;
  static constexpr int kTotalBytes = kBarOff + kNumBars * 8 + 16 + 1024;
  static_assert(kTotalBytes <= 232448, "shared memory budget");
};

template <int HD, int BS>
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
  uint8_t* p_smem = smem + L::kPOff;
  uint8_t* ring = smem + L::kRingOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* full = bars + 1;                 // [kSlots]
  uint64_t* empty = full + kSlots;           // [kSlots]
  uint64_t* s_full = empty + kSlots;         // [2]  S of tile A / B ready (MMA -> softmax)
  uint64_t* p_full = s_full + kPfQTiles;     // [2]  P of tile A / B written (softmax -> MMA)
  uint64_t* pv_done = p_full + kPfQTiles;    // [2]  PV of tile A / B retired (MMA -> softmax)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A CTA of this launch already gave up on a wait: do not repeat the timeout per CTA.
  if (*reinterpret_cast<volatile int*>(p.err_word) == kDevWaitTimeout) return;

  // ---- which (sequence, 256-row query block) is this CTA?  Heavy (late) blocks go first.
  int tile_linear = gridDim.x - 1 - blockIdx.x;
  int seq = -1, q0 = 0, seq_q_begin = 0, seq_len_q = 0;
  {
    int acc = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int b = p.cu_q[s], e = p.cu_q[s + 1];
      const int nt = (e - b + kPfRowsPerCta - 1) / kPfRowsPerCta;
      if (tile_linear < acc + nt) {
        seq = s;
        q0 = (tile_linear - acc) * kPfRowsPerCta;
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
  // Per query tile: valid rows, first absolute position, number of KV tiles it attends to.
  int rows_valid[kPfQTiles], first_pos[kPfQTiles], n_tiles[kPfQTiles];
#pragma unroll
  for (int w = 0; w < kPfQTiles; ++w) {
    rows_valid[w] = max(0, min(kPfM, seq_len_q - q0 - w * kPfM));
    first_pos[w] = start + q0 + w * kPfM;
    n_tiles[w] = rows_valid[w] > 0 ? (first_pos[w] + rows_valid[w] - 1) / kPfN + 1 : 0;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);   // tile A never needs more KV tiles than B

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < kPfQTiles; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
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
      const uint64_t pol_q = l2_policy_evict_first();
      mbar_arrive_expect_tx(q_full, kPfQTiles * L::kTileBytes);
#pragma unroll
      for (int w = 0; w < kPfQTiles; ++w)
#pragma unroll
        for (int s = 0; s < kSub; ++s)
          tma_load_2d(q_smem + w * L::kTileBytes + s * L::kSubBytes, &tm_q, q_full,
                      head * HD + s * 64, seq_q_begin + q0 + w * kPfM, pol_q);
    }
    const uint64_t pol_kv = l2_policy_evict_last();
    const int32_t* pt = p.page_table + static_cast<int64_t>(seq) * p.page_table_stride;
    const int last_pos = start + min(seq_len_q, q0 + kPfRowsPerCta) - 1;
    const int n_pages = last_pos / BS + 1;      // pages holding keys 0 .. last_pos
    for (int i = 0; i < 2 * n_max; ++i) {
      const int j = i >> 1;
      const bool is_v = i & 1;
      const int slot = i % kSlots;
      mbar_wait(&empty[slot], ((i / kSlots) & 1) ^ 1, abort_flag, p.err_word);
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
      auto wait_item = [&](int i) {
        mbar_wait(&full[i % kSlots], (i / kSlots) & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
      };
      auto release_item = [&](int i) { umma_commit(&empty[i % kSlots]); };
      auto issue_qk = [&](int w, int j) {   // S_w = Q_w K_j^T
        const uint32_t q_addr = smem_u32(q_smem + w * L::kTileBytes);
        const uint32_t k_addr = smem_u32(ring + ((2 * j) % kSlots) * L::kTileBytes);
        const uint32_t d = tmem_base + w * kPfN;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * L::kSubBytes + (kk & 3) * 32;
          umma_ss(d, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                  umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk > 0);
        }
        umma_commit(&s_full[w]);
      };
      auto issue_pv = [&](int w, int j) {   // O_w += P_w V_j
        mbar_wait(&p_full[w], j & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        const uint32_t p_addr = smem_u32(p_smem + w * L::kPBytes);
        const uint32_t v_addr = smem_u32(ring + ((2 * j + 1) % kSlots) * L::kTileBytes);
        const uint32_t d = tmem_base + 256 + w * 128;
#pragma unroll
        for (int kk = 0; kk < kPfN / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * L::kSubBytes + (kk & 3) * 32;
          umma_ss(d, umma_smem_desc_sw128(p_addr + a_off, 16, 1024),
                  umma_smem_desc_sw128(v_addr + kk * 2048, L::kSubBytes, 1024), idesc_pv,
                  (j > 0) || (kk > 0));
        }
        umma_commit(&pv_done[w]);
      };
      mbar_wait(q_full, 0, abort_flag, p.err_word);
      wait_item(0);
#pragma unroll
      for (int w = 0; w < kPfQTiles; ++w)
        if (n_tiles[w] > 0) issue_qk(w, 0);
      release_item(0);
      for (int j = 0; j < n_max; ++j) {
        wait_item(2 * j + 1);                       // V_j
        const bool has_next = j + 1 < n_max;
        bool next_k_ready = false;
#pragma unroll
        for (int w = 0; w < kPfQTiles; ++w) {
          if (j < n_tiles[w]) {
            issue_pv(w, j);
            if (j + 1 < n_tiles[w]) {
              if (!next_k_ready) {
                wait_item(2 * j + 2);               // K_{j+1}
                next_k_ready = true;
              }
              issue_qk(w, j + 1);
            }
          }
        }
        release_item(2 * j + 1);
        if (has_next) release_item(2 * j + 2);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int w = (warp - 2) >> 2;                       // 0 = tile A, 1 = tile B
    const int row = (warp & 3) * 32 + lane;              // tensor-memory lane == query row
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + w * kPfN + lane_addr;
    const uint32_t o_addr = tmem_base + 256 + w * 128 + lane_addr;
    const int q_pos = first_pos[w] + row;
    const int my_tiles = n_tiles[w];
    const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < my_tiles; ++j) {
      mbar_wait(&s_full[w], j & 1, abort_flag, p.err_word);
      tc_fence_after_sync();
      uint32_t sreg[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, sreg[c]);
      tmem_wait_ld();

      const int key0 = j * kPfN;
      if (key0 + kPfN - 1 > first_pos[w]) {     // tile crosses the diagonal for some row
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (key0 + c * 32 + k > q_pos) sreg[c][k] = 0xff800000u;   // -inf
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
      const float corr = fast_exp2(m_run - m_new);
      const bool rescale = (m_new != m_run) && (j > 0);
      m_run = m_new;
      if (j > 0) {
        // PV_{j-1} must have retired before P is overwritten or O is rescaled.  It was issued
        // before QK_j, whose completion s_full just signalled, so this wait does not block.
        mbar_wait(&pv_done[w], (j - 1) & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
      }
      // p = 2^(s*scale - m): packed FMA, then ex2; two packed running sums.  Each 32-key chunk
      // goes straight to the swizzled K-major P tile (16-byte piece jj covers keys jj*8..+7).
      const uint64_t negm2 = pack_f32x2(-m_new, -m_new);
      const uint32_t p_row = smem_u32(p_smem + w * L::kPBytes) + row * 128;
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
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int jj = c * 4 + q4;
          const uint32_t a = p_row + (jj >> 3) * L::kSubBytes + (((jj & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(preg[q4 * 4]),
                       "r"(preg[q4 * 4 + 1]), "r"(preg[q4 * 4 + 2]), "r"(preg[q4 * 4 + 3])
                       : "memory");
        }
      }
      {
        float a0, a1, b0, b1;
        unpack_f32x2(sum2[0], a0, a1);
        unpack_f32x2(sum2[1], b0, b1);
        l_run = l_run * corr + ((a0 + a1) + (b0 + b1));
      }
      // O row rescale (rare: only when the running max moved by more than the threshold).
      if (j > 0) {
        if (__any_sync(0xffffffffu, rescale)) {
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
          tmem_wait_st();
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_full[w]);
    }
    // ---- epilogue: O / l -> bf16 rows
    if (my_tiles > 0) {
      mbar_wait(&pv_done[w], (my_tiles - 1) & 1, abort_flag, p.err_word);
      tc_fence_after_sync();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow =
          p.out + static_cast<int64_t>(seq_q_begin + q0 + w * kPfM + row) * p.out_row_stride +
          static_cast<int64_t>(head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t oreg[32];
        tmem_ld_32x32(o_addr + c * 32, oreg);
        tmem_wait_ld();
        if (row < rows_valid[w]) {
#pragma unroll
          for (int k = 0; k < 32; k += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(oreg[k]) * inv_l,
                              __uint_as_float(oreg[k + 1]) * inv_l);
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
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200attn
