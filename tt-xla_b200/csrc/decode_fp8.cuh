// Paged GQA decode attention over an fp8 (e4m3) KV cache, head_size 128.
//
// The cache dtype is one of the plugin's KV-cache options (attention.py:42-51: "fp8" / "fp8_e4m3"
// -> torch.float8_e4m3fn); values are stored unscaled, as the reference's cache write stores them
// (attention.py:692-700: clamp to the finite range, then cast).  Decode is HBM-bound, so a cache
// of half the bytes streams twice the tokens per second.
//
// Same structure as the bf16 kernel (grid (split, kv_head, user); producer warp + four consumer
// warps; 64-token tiles in a TMA-fed ring; online softmax; 4-warp merge; fp32 partials for the
// combine kernel).  What differs is how the tiles reach the tensor cores:
//   * a tile row is one token's 128 head elements = 128 bytes = one swizzled row;
//   * K: an 8x8 `ldmatrix` of 16-bit units hands thread (g, tq) four CONSECUTIVE e4m3 of token g.
//     The contraction index of an MMA may be permuted freely as long as both operands agree, so
//     those four become the thread's k-slots {2tq, 2tq+1, 2tq+8, 2tq+9} and the Q fragments are
//     loaded with the same permutation once per CTA;
//   * V: the transposed `ldmatrix` hands thread (g, tq) the byte pairs (d = 2g, 2g+1) of tokens
//     2tq and 2tq+1.  A byte permute regroups them into two B fragments, one for the even and
//     one for the odd head elements of the 16-byte chunk; the accumulators therefore hold the
//     head elements in a permuted order that the merge step undoes;
//   * e4m3 pairs widen to f16 pairs exactly (`cvt.rn.f16x2.e4m3x2`), so the MMAs run in f16 with
//     fp32 accumulation; Q (bf16) and the softmax weights are rounded to f16 (11 significant
//     bits, more than bf16 keeps).
#pragma once
#include "decode.cuh"

namespace b200attn {

template <int BS, int STAGES>
struct DecodeFp8Smem {
  static constexpr int kPages = kDecTile / BS;
  static constexpr int kBoxBytes = BS * 128;                  // one TMA box: BS tokens x 128 B
  static constexpr int kTensorBytes = kPages * kBoxBytes;     // K (or V) of one tile: 8 KiB
  static constexpr int kStageBytes = 2 * kTensorBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kBarrierBytes = 2 * STAGES * 8 + 16;
  static constexpr int kTotalBytes = kRingBytes + kBarrierBytes + 1024;
};

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// two e4m3 (low 16 bits of v) -> f16x2, exact
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t v) {
  uint32_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t byte_perm(uint32_t v, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(v), "r"(sel));
  return r;
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

template <int BS, int STAGES>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_fp8_kernel(const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
  constexpr int HD = 128;
  using L = DecodeFp8Smem<BS, STAGES>;
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
    int win_base = t_begin * L::kPages;
    auto fetch = [&](int base) {
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
          tma_load_2d(kdst + pg * L::kBoxBytes, &tm_k, &full_bar[stage], 0, y, policy);
          tma_load_2d(vdst + pg * L::kBoxBytes, &tm_v, &full_bar[stage], 0, y, policy);
        }
      }
    }
    return;  // consumers wait on every full barrier, so no copy is in flight at kernel end
  }

  // -------------------------------------------------------------------- consumer warps
  const int g = lane >> 2;   // fragment row (query head within the group); g + 8 is the second row
  const int tq = lane & 3;

  // Q fragments in f16 with the contraction permutation of the K loads: within k-step ks the
  // thread's slots {2tq, 2tq+1} hold head elements 16ks + 4tq + {0, 1}, slots {2tq+8, 2tq+9}
  // hold 16ks + 4tq + {2, 3}.  Rows >= G are zero.
  uint32_t qf[HD / 16][4];
  {
    const __nv_bfloat16* qrow = p.q + static_cast<int64_t>(user) * p.q_row_stride +
                                static_cast<int64_t>(kvh) * G * HD;
    auto load4 = [&](int row, int d0, uint32_t& first, uint32_t& second) {
      if (row < G) {
        const uint2 v = *reinterpret_cast<const uint2*>(qrow + row * HD + d0);   // 4 bf16
        first = pack_f16x2(bf16_bits_to_f32(v.x & 0xffffu), bf16_bits_to_f32(v.x >> 16));
        second = pack_f16x2(bf16_bits_to_f32(v.y & 0xffffu), bf16_bits_to_f32(v.y >> 16));
      } else {
        first = 0u;
        second = 0u;
      }
    };
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int d0 = ks * 16 + tq * 4;
      load4(g, d0, qf[ks][0], qf[ks][2]);
      load4(g + 8, d0, qf[ks][1], qf[ks][3]);
    }
  }

  // o[2c + e][j]: head element 16c + 4tq + 2(j & 1) + e of row g (j < 2) or g + 8 (j >= 2)
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY;  // running max, rows g and g+8 (log2 units)
  float l_lo = 0.f, l_hi = 0.f;              // running sum (this thread's share of the row)

  // Per-lane ldmatrix row addressing inside a tile (rows of 128 bytes, 16-byte chunks XOR-swizzled
  // with the row's low three bits).
  //   K: matrix m = lane/8 -> token half m/2 (n-tile), chunk parity m%2 (k-step of a pair).
  //   V (transposed): matrix m = lane/8 -> token half m%2, chunk parity m/2.
  const int lm = lane >> 3, lr = lane & 7;
  const int k_tok = warp * 16 + (lm >> 1) * 8 + lr;
  const int v_tok = warp * 16 + (lm & 1) * 8 + lr;
  const uint32_t k_row_off = static_cast<uint32_t>(((k_tok / BS) * BS + k_tok % BS) * 128);
  const uint32_t v_row_off = static_cast<uint32_t>(((v_tok / BS) * BS + v_tok % BS) * 128);
  const int k_sw = (k_tok % BS) & 7, v_sw = (v_tok % BS) & 7;

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
        for (int i = lane; i < 16 * 8; i += 32) {
          const int r = i >> 3, c = i & 7;
          const int tok = warp * 16 + r;
          if (t * kDecTile + tok >= ctx) {
            const int row = tok % BS;
            const uint32_t a = vbase + ((tok / BS) * BS + row) * 128 + ((c ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
          }
        }
        fence_proxy_async_smem();  // the next TMA write to this stage follows generic writes
        __syncwarp();
      }

      // ---- S = Q K^T for 16 tokens (two 8-token n-tiles); one ldmatrix feeds two k-steps
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < HD / 32; ++kp) {
        const int cc = kp * 2 + (lm & 1);   // 16-byte chunk = k-step
        uint32_t b[4];
        ldmatrix_x4(b, kbase + k_row_off + ((cc ^ k_sw) << 4));
        // b[0]: tokens 0-7, k-step 2kp   b[1]: tokens 0-7, k-step 2kp+1
        // b[2]: tokens 8-15, k-step 2kp  b[3]: tokens 8-15, k-step 2kp+1
        mma_f16_16816(s[0], qf[2 * kp], e4m3x2_to_f16x2(b[0]), e4m3x2_to_f16x2(b[0] >> 16));
        mma_f16_16816(s[0], qf[2 * kp + 1], e4m3x2_to_f16x2(b[1]), e4m3x2_to_f16x2(b[1] >> 16));
        mma_f16_16816(s[1], qf[2 * kp], e4m3x2_to_f16x2(b[2]), e4m3x2_to_f16x2(b[2] >> 16));
        mma_f16_16816(s[1], qf[2 * kp + 1], e4m3x2_to_f16x2(b[3]), e4m3x2_to_f16x2(b[3] >> 16));
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
      pa[0] = pack_f16x2(pr[0][0], pr[0][1]);
      pa[1] = pack_f16x2(pr[0][2], pr[0][3]);
      pa[2] = pack_f16x2(pr[1][0], pr[1][1]);
      pa[3] = pack_f16x2(pr[1][2], pr[1][3]);

      // ---- O += P V  (k = this warp's 16 tokens, n = head elements).  One transposed ldmatrix
      // covers 16 tokens x two 16-byte chunks = four n-tiles (even / odd elements of each chunk).
#pragma unroll
      for (int cp = 0; cp < HD / 32; ++cp) {
        const int cc = cp * 2 + (lm >> 1);
        uint32_t b[4];
        ldmatrix_x4_trans(b, vbase + v_row_off + ((cc ^ v_sw) << 4));
        // b[0]: tokens 0-7 of chunk 2cp, b[1]: tokens 8-15 of chunk 2cp, b[2] / b[3]: chunk 2cp+1.
        // In each: byte0 = V[2tq][2g], byte1 = V[2tq][2g+1], byte2 = V[2tq+1][2g], byte3 = V[2tq+1][2g+1].
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t lo8 = b[2 * h], hi8 = b[2 * h + 1];
          const int c = 2 * cp + h;
          mma_f16_16816(o[2 * c], pa, e4m3x2_to_f16x2(byte_perm(lo8, 0x3120u)),
                        e4m3x2_to_f16x2(byte_perm(hi8, 0x3120u)));
          mma_f16_16816(o[2 * c + 1], pa, e4m3x2_to_f16x2(byte_perm(lo8, 0x3120u) >> 16),
                        e4m3x2_to_f16x2(byte_perm(hi8, 0x3120u) >> 16));
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
  }

  // -------------------------------------------------------------------- merge the 4 warps
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
  for (int c = 0; c < HD / 16; ++c) {
    // undo the even / odd split: elements 16c + 4tq + {0, 1, 2, 3}
    const int d = c * 16 + tq * 4;
    *reinterpret_cast<float4*>(mo + (warp * 16 + g) * HD + d) =
        make_float4(o[2 * c][0], o[2 * c + 1][0], o[2 * c][1], o[2 * c + 1][1]);
    *reinterpret_cast<float4*>(mo + (warp * 16 + g + 8) * HD + d) =
        make_float4(o[2 * c][2], o[2 * c + 1][2], o[2 * c][3], o[2 * c + 1][3]);
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

}  // namespace b200attn
