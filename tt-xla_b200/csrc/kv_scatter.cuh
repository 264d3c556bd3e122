// KV-cache write: scatters new K and V rows into the paged caches.
//
// One (token, kv head) row of the cache is head_size*2 bytes contiguous, so every thread
// moves one 16-byte vector and a warp's stores are fully coalesced (an e4m3 cache gets the
// vector's 8 values as 8 bytes).  K and V go in the same
// launch.  The three addressing forms differ only in how a token finds its block and offset.
#pragma once
#include "ptx.cuh"

namespace b200attn {

enum ScatterMode : int {
  kScatterSlots = 0,   // slot_mapping[t] (int64), negative = skip
  kScatterUpdate = 1,  // decode: update_indices[u] + page_table[u, :]
  kScatterFill = 2     // prefill: fill_page_table[batch_idx[u], t / bs], offset t % bs
};

struct ScatterParams {
  uint4* k_cache;
  uint4* v_cache;
  const uint4* k_new;
  const uint4* v_new;
  int64_t new_token_stride_v;  // in 16-byte vectors
  const int64_t* slot_mapping;
  const int32_t* positions;   // update_indices
  const int32_t* page_table;
  int64_t page_table_stride;
  int page_table_width;
  const int32_t* batch_idx;
  int tokens_per_user;
  int64_t num_tokens;
  int num_kv_heads;
  int block_size;
  int64_t num_blocks;
  int vec_per_head;           // head_size * 2 / 16
  int cache_fp8;              // 1: the caches hold e4m3 (8 bytes per vector), 0: bf16
  int* err_word;
};

// 8 bf16 -> 8 e4m3, round to nearest even, saturating at +-448 (what clamping to the finite
// range and casting does, attention.py:692-700); NaN stays NaN.
__device__ __forceinline__ uint2 bf16x8_to_e4m3x8(const uint4 v) {
  auto pair = [](uint32_t w) -> uint32_t {       // two bf16 -> two e4m3 in the low 16 bits
    uint16_t r;
    const float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
  };
  return make_uint2(pair(v.x) | (pair(v.y) << 16), pair(v.z) | (pair(v.w) << 16));
}

// Python-style floor division and modulo (the reference's CPU branch indexes with torch
// `//` and `%`, which floor).
__device__ __forceinline__ int floordiv_i32(int a, int b) {
  int q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}

template <int MODE>
__global__ void __launch_bounds__(256) kv_scatter_kernel(const ScatterParams p) {
  const int vec_per_token = p.num_kv_heads * p.vec_per_head;
  const int64_t total = p.num_tokens * vec_per_token;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_token;
    const int rem = static_cast<int>(i - t * vec_per_token);
    const int h = rem / p.vec_per_head;
    const int v = rem - h * p.vec_per_head;

    int64_t blk;
    int off;
    if (MODE == kScatterSlots) {
      const int64_t slot = p.slot_mapping[t];
      if (slot < 0) continue;
      blk = slot / p.block_size;
      off = static_cast<int>(slot - blk * p.block_size);
    } else if (MODE == kScatterUpdate) {
      const int pos = p.positions[t];
      int col = floordiv_i32(pos, p.block_size);
      off = pos - col * p.block_size;
      if (col < 0) col += p.page_table_width;  // torch negative-index wrap-around
      if (col < 0 || col >= p.page_table_width) {
        if (v == 0 && h == 0) atomicExch(p.err_word, kDevBadIndex);
        continue;
      }
      blk = p.page_table[t * p.page_table_stride + col];
    } else {
      const int64_t u = t / p.tokens_per_user;
      const int tt = static_cast<int>(t - u * p.tokens_per_user);
      const int col = tt / p.block_size;
      off = tt - col * p.block_size;
      const int64_t row = p.batch_idx ? p.batch_idx[u] : u;
      if (col >= p.page_table_width) {
        if (v == 0 && h == 0) atomicExch(p.err_word, kDevBadIndex);
        continue;
      }
      blk = p.page_table[row * p.page_table_stride + col];
    }
    if (blk < 0 || blk >= p.num_blocks) {
      if (v == 0 && h == 0) atomicExch(p.err_word, kDevBadIndex);
      continue;
    }
    const int64_t src = t * p.new_token_stride_v + rem;
    const int64_t dst =
        ((blk * p.num_kv_heads + h) * p.block_size + off) * p.vec_per_head + v;
    const uint4 kv = __ldg(p.k_new + src);
    const uint4 vv = __ldg(p.v_new + src);
    if (p.cache_fp8) {
      reinterpret_cast<uint2*>(p.k_cache)[dst] = bf16x8_to_e4m3x8(kv);
      reinterpret_cast<uint2*>(p.v_cache)[dst] = bf16x8_to_e4m3x8(vv);
    } else {
      p.k_cache[dst] = kv;
      p.v_cache[dst] = vv;
    }
  }
}

}  // namespace b200attn
