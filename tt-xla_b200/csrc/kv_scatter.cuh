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

// ------------------------------------------------------------------------------------------
// Widening of the pages a prefill batch reads from an e4m3 cache into a bf16 page pool.
//
// The tcgen05 prefill kernel takes 16-bit K / V tiles.  Over an fp8 cache the prefix pages of
// the batch's sequences are first copied, widened, into a compact scratch pool laid out
// [sequence][page slot] (slot i of sequence s = page_table[s, i]), and the kernel then reads that
// pool through the identity page table.  Every e4m3 value is exactly representable in bf16, so
// the attention sees exactly the cache's values.  HBM-bound: 1 byte read + 2 written per element
// of the context; the attention over it is tensor-bound and an order of magnitude longer.
struct DequantPagesParams {
  const uint8_t* k_src;       // [num_blocks, nkv, bs, hd] e4m3
  const uint8_t* v_src;
  __nv_bfloat16* k_dst;       // [num_seqs * width, nkv, bs, hd] bf16
  __nv_bfloat16* v_dst;
  const int32_t* page_table;
  int64_t page_table_stride;
  int page_table_width;
  const int32_t* cu_q;        // [num_seqs + 1]
  const int32_t* q_start;     // [num_seqs] or NULL (0)
  int block_size;
  int page_elems;             // nkv * bs * hd
  int64_t num_blocks;
  int* err_word;
};

__device__ __forceinline__ uint4 e4m3x8_to_bf16x8(const uint2 v) {
  auto widen = [](uint32_t two) -> uint32_t {   // two e4m3 (low 16 bits) -> two bf16
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(static_cast<uint16_t>(two)));
    float lo, hi;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
        : "=f"(lo), "=f"(hi)
        : "r"(h));
    return pack_bf16x2(lo, hi);
  };
  return make_uint4(widen(v.x), widen(v.x >> 16), widen(v.y), widen(v.y >> 16));
}

// grid (page slot, sequence); one CTA widens one page of K and of V.
__global__ void __launch_bounds__(256) dequant_pages_kernel(const DequantPagesParams p) {
  const int slot = blockIdx.x, seq = blockIdx.y;
  const int len = p.cu_q[seq + 1] - p.cu_q[seq];
  const int ctx = (p.q_start ? p.q_start[seq] : 0) + len;          // keys 0 .. ctx-1 are read
  if (len <= 0 || slot >= (ctx + p.block_size - 1) / p.block_size) return;
  int64_t blk = p.page_table[static_cast<int64_t>(seq) * p.page_table_stride + slot];
  if (blk < 0 || blk >= p.num_blocks) {
    if (threadIdx.x == 0) atomicExch(p.err_word, kDevBadIndex);
    return;
  }
  const int64_t dst_page = static_cast<int64_t>(seq) * p.page_table_width + slot;
  const int vecs = p.page_elems / 8;                               // 8 elements per thread step
  const uint2* ks = reinterpret_cast<const uint2*>(p.k_src + blk * p.page_elems);
  const uint2* vs = reinterpret_cast<const uint2*>(p.v_src + blk * p.page_elems);
  uint4* kd = reinterpret_cast<uint4*>(p.k_dst + dst_page * p.page_elems);
  uint4* vd = reinterpret_cast<uint4*>(p.v_dst + dst_page * p.page_elems);
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    kd[i] = e4m3x8_to_bf16x8(__ldg(ks + i));
    vd[i] = e4m3x8_to_bf16x8(__ldg(vs + i));
  }
}

}  // namespace b200attn
