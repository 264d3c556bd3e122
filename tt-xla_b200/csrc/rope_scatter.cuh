// Rotary embedding fused with the KV-cache write (slot-mapping form).
//
// One CTA per token.  The token's cos / sin row is computed once into shared memory exactly as
// the plugin's rotary layer does it (fp32 position x inv_freq, fp32 cos / sin, rounded to bf16),
// then every 16-byte vector pair (x1, x2) of the rotated part of each q and k head is combined
// with the reference's bf16 rounding after every multiply and add, q and k are written back in
// place, and the rotated k and the untouched v go straight to their cache slot: k makes one trip
// through registers instead of three through HBM (rotary write, scatter read, scatter write).
#pragma once
#include "ptx.cuh"

namespace b200attn {

struct RopeScatterParams {
  __nv_bfloat16* q;
  int64_t q_stride;       // elements between token rows
  __nv_bfloat16* k;
  int64_t k_stride;
  const __nv_bfloat16* v;
  int64_t v_stride;
  const int64_t* positions;
  const float* inv_freq;  // [rotary_dim / 2]
  int rotary_dim;
  uint4* k_cache;
  uint4* v_cache;
  const int64_t* slot_mapping;   // may be NULL: rotate only
  int num_q_heads;
  int num_kv_heads;
  int head_size;
  int block_size;
  int64_t num_blocks;
  int* err_word;
};

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// (x1, x2) -> (x1*c - x2*s, x2*c + x1*s) with a bf16 rounding after every operation.
__device__ __forceinline__ void rope_pair(uint32_t& a, uint32_t& b, const __nv_bfloat16* cs,
                                          const __nv_bfloat16* sn) {
  // a, b hold two consecutive bf16 each (low half = even element)
  float x1[2] = {__uint_as_float(a << 16), __uint_as_float(a & 0xffff0000u)};
  float x2[2] = {__uint_as_float(b << 16), __uint_as_float(b & 0xffff0000u)};
  float o1[2], o2[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float c = __bfloat162float(cs[i]), s = __bfloat162float(sn[i]);
    o1[i] = bf16_round(bf16_round(x1[i] * c) - bf16_round(x2[i] * s));
    o2[i] = bf16_round(bf16_round(x2[i] * c) + bf16_round(x1[i] * s));
  }
  a = pack_bf16x2(o1[0], o1[1]);
  b = pack_bf16x2(o2[0], o2[1]);
}

__global__ void __launch_bounds__(256) rope_kv_scatter_kernel(const RopeScatterParams p) {
  __shared__ __nv_bfloat16 cs[128];
  __shared__ __nv_bfloat16 sn[128];
  const int64_t t = blockIdx.x;
  const int half = p.rotary_dim / 2;
  const float pos = static_cast<float>(p.positions[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float f = pos * p.inv_freq[i];
    cs[i] = __float2bfloat16_rn(cosf(f));
    sn[i] = __float2bfloat16_rn(sinf(f));
  }
  __syncthreads();

  const int hd = p.head_size;
  const int vec_per_head = hd / 8;
  const int pair_vecs = half / 8;                 // 16-byte vectors in each rotated half
  const int tail_vecs = (hd - p.rotary_dim) / 8;  // not rotated
  int64_t blk = -1;
  int off = 0;
  if (p.slot_mapping) {
    const int64_t slot = p.slot_mapping[t];
    if (slot >= 0) {
      blk = slot / p.block_size;
      off = static_cast<int>(slot - blk * p.block_size);
      if (blk >= p.num_blocks) {
        if (threadIdx.x == 0) atomicExch(p.err_word, kDevBadIndex);
        blk = -1;
      }
    }
  }
  // ---- rotated halves of the q heads, then of the k heads
  const int rot_units = (p.num_q_heads + p.num_kv_heads) * pair_vecs;
  for (int u = threadIdx.x; u < rot_units; u += blockDim.x) {
    const int head = u / pair_vecs, pv = u - head * pair_vecs;
    const bool is_k = head >= p.num_q_heads;
    const int h = is_k ? head - p.num_q_heads : head;
    __nv_bfloat16* row = is_k ? p.k + t * p.k_stride + static_cast<int64_t>(h) * hd
                              : p.q + t * p.q_stride + static_cast<int64_t>(h) * hd;
    uint4 a = *reinterpret_cast<const uint4*>(row + pv * 8);
    uint4 b = *reinterpret_cast<const uint4*>(row + half + pv * 8);
    const __nv_bfloat16* c = cs + pv * 8;
    const __nv_bfloat16* s = sn + pv * 8;
    rope_pair(a.x, b.x, c, s);
    rope_pair(a.y, b.y, c + 2, s + 2);
    rope_pair(a.z, b.z, c + 4, s + 4);
    rope_pair(a.w, b.w, c + 6, s + 6);
    *reinterpret_cast<uint4*>(row + pv * 8) = a;
    *reinterpret_cast<uint4*>(row + half + pv * 8) = b;
    if (is_k && blk >= 0) {
      const int64_t dst = ((blk * p.num_kv_heads + h) * p.block_size + off) * vec_per_head;
      p.k_cache[dst + pv] = a;
      p.k_cache[dst + pair_vecs + pv] = b;
    }
  }
  if (blk < 0) return;
  // ---- unrotated tail of the k heads, and all of v
  const int copy_units = p.num_kv_heads * (tail_vecs + vec_per_head);
  for (int u = threadIdx.x; u < copy_units; u += blockDim.x) {
    const int h = u / (tail_vecs + vec_per_head);
    const int i = u - h * (tail_vecs + vec_per_head);
    const int64_t dst = ((blk * p.num_kv_heads + h) * p.block_size + off) * vec_per_head;
    if (i < tail_vecs) {
      const int vi = 2 * pair_vecs + i;
      p.k_cache[dst + vi] =
          *reinterpret_cast<const uint4*>(p.k + t * p.k_stride + static_cast<int64_t>(h) * hd + vi * 8);
    } else {
      const int vi = i - tail_vecs;
      p.v_cache[dst + vi] =
          *reinterpret_cast<const uint4*>(p.v + t * p.v_stride + static_cast<int64_t>(h) * hd + vi * 8);
    }
  }
}

}  // namespace b200attn
