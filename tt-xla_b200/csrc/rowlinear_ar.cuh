// Row-parallel linear layer with the tensor-parallel all-reduce fused into its epilogue, for
// decode-sized batches (up to 128 token rows):
//
//     out[t, n] = sum over ranks r of  bf16( sum_k x_r[t, k] * w_r[n, k] )      (fp32 sums)
//
// Every rank holds its own K slice of the activations (x_r [tokens, K/world]) and of the weight
// (w_r [N, K/world], the torch Linear layout) and all ranks launch this kernel on the same
// sequence of calls.  What the reference expresses as a row-sharded weight whose partial sums the
// compiler all-reduces (vllm_tt/vllm_distributed_utils.py:356-363, `partition_row_parallel_linear`;
// vLLM's RowParallelLinear.forward = GEMM then tensor_model_parallel_all_reduce, which also adds
// bf16 partials) is one launch here.
//
// Work split: the weight is the HBM stream, so it is the M operand.  A cluster of S CTAs owns one
// tile of 128 output columns and splits K between its CTAs (grid = S x N/128 <= number of SMs:
// every CTA of every rank is resident, and a CTA only ever waits for the same CTA on its peers).
// Per CTA:
//   warp 0     TMA producer: per 64-wide K step one [128 x 64] box of w and one [NB x 64] box of x
//              (NB = 32 / 64 / 128 token rows; rows beyond the token count are zero-filled by the
//              tensor map's bounds) into a ring of swizzled stages.
//   warp 1     tcgen05.mma issuer: D[128 columns x NB tokens] (+)= W_stage . X_stage^T, both operands
//              K-major from shared memory, fp32 accumulator in tensor memory.
//   warps 2-5  epilogue, one thread per output column:
//              1. split-K: CTA s finishes token rows [s*NB/S, (s+1)*NB/S).  Every CTA stores each
//                 share of its D straight into the owning CTA's shared memory (distributed shared
//                 memory stores), one cluster barrier, then the owner adds the S pieces in CTA order.
//              2. all-reduce: the partial goes to EVERY peer as 8-byte units {bf16 pair, epoch}
//                 (32 lanes write 256 contiguous bytes; plain peer stores over NVLink).  An 8-byte
//                 store lands whole, so the unit carries its own arrival flag: no fence, no separate
//                 flag round trip.  The receiver spins (bounded) on the units addressed to it,
//                 adds the bf16 partials of all ranks, its own included, in rank order (so every
//                 rank produces the same bits) and writes bf16.
// The push of one tile overlaps the K loops of tiles still running; nothing is read from a peer's
// memory.
//
// Call sequencing without host help (so the launch can sit in a CUDA graph): the communicator
// header holds an epoch word; every CTA uses epoch+1 as this call's unit flag and the last CTA out
// stores it back.  Staging is double-buffered by epoch parity: a rank can be at most one call
// ahead of a peer (it needs the peer's partials of call e+1 to finish e+1, and the peer pushes
// those only after it has finished call e), so units of call e+2 never overwrite units of call e
// that are still being read.
#pragma once
#include "ptx.cuh"

namespace b200attn {

constexpr int kRlMaxWorld = 8;
constexpr int kRlTileN = 128;        // output columns per cluster (the MMA's M)
constexpr int kRlMaxTokens = 128;    // token rows of one launch (the MMA's N)
constexpr int kRlKStep = 64;         // K elements per stage: one 128-byte swizzle row of bf16
constexpr int kRlThreads = 192;
constexpr int kRlMaxSplit = 8;       // CTAs per cluster
constexpr size_t kRlStageOff = 32768;   // staging starts here; the header sits below

struct RowLinearComm {       // the first bytes of a communicator buffer
  uint32_t epoch;            // calls completed on this rank
  uint32_t ticket;           // CTAs of the running call that have finished
  uint32_t out_of_step;      // a wait for a peer ran out on this rank: the ranks no longer agree
                             // on the epoch, and every later call through this communicator only
                             // runs its GEMM; a new communicator starts clean
};

struct RowLinearParams {
  __nv_bfloat16* out;
  int64_t out_row_stride;    // elements
  int num_tokens, n_total;
  int k_steps;               // 64-wide K steps of this rank's slice
  int steps_per_split;       // K steps per CTA of a cluster (the last CTA may get fewer)
  int rank, world;
  int two_shot;              // 0: every rank reduces everything; 1: reduce at a slot's owner
  size_t src_stride;         // bytes of one staging area; world + 1 areas per parity
  uint8_t* comm[kRlMaxWorld];   // communicator buffer of every rank as mapped here; own at [rank]
  uint64_t peer_timeout_ns;
  int* err_word;
};

template <int NB>
struct RowLinearSmem {
  static constexpr int kWBytes = kRlTileN * 128;       // 16 KiB
  static constexpr int kXBytes = NB * 128;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = NB == 32 ? 8 : (NB == 64 ? 7 : 5);
  static constexpr int kWOff = 0;
  static constexpr int kXOff = kStages * kWBytes;
  static constexpr int kRingBytes = kStages * kStageBytes;
  // split-K exchange: [source CTA][token of this CTA's share][column] fp32 = NB * 128 * 4 bytes
  // whatever S is.  Apart from the ring: the other CTAs store into it while this one may still
  // be in its K loop.
  static constexpr int kXchOff = kRingBytes;
  static constexpr int kXchBytes = NB * kRlTileN * 4;
  static constexpr int kBarOff = kXchOff + kXchBytes;
  static constexpr int kNumBars = 2 * kStages + 1;
  static constexpr int kMiscBytes = 64;                 // tensor-memory slot, flags, health words
  static constexpr int kTotalBytes = kBarOff + kNumBars * 8 + kMiscBytes + 1024;   // + alignment
  static_assert(kTotalBytes <= 232448, "over the shared memory of one CTA");
};

// One 8-byte unit: two bf16 partial sums (token rows t, t+1 of one column) and the call's epoch.
// Areas per parity: one per source rank, then one for results (two-shot mode).  Units of one
// area: [slot = tile * S + share][pair of the share][column].
__device__ __forceinline__ uint2* rl_unit(uint8_t* comm, const RowLinearParams& p, uint32_t parity,
                                          int src, int slot, int pairs_per_share, int pair, int col) {
  uint8_t* area =
      comm + kRlStageOff + (static_cast<size_t>(parity) * (p.world + 1) + src) * p.src_stride;
  return reinterpret_cast<uint2*>(area) +
         (static_cast<size_t>(slot) * pairs_per_share + pair) * kRlTileN + col;
}
__device__ __forceinline__ uint2 ld_volatile_u2(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_u2(uint2* p, uint32_t x, uint32_t y) {
  asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory offset in CTA `cta` of this cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Programmatic dependent launch: blocks until the kernels this launch depends on have completed
// and their writes are visible (a no-op for an ordinary launch).
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// NB: token rows of the MMA (32 / 64 / 128).  S: CTAs per cluster = K splits (1 / 2 / 4 / 8).
// W: bound of the loops over source ranks (2 / 4 / 8 >= world).  The exchange is straight-line
// code unrolled over sources x units that every CTA runs once, out of a cold instruction cache:
// with the loops bounded at 8 sources a two-rank call spent a microsecond more fetching it.
template <int NB, int S, int W>
__global__ void __launch_bounds__(kRlThreads, 1)
rowlinear_allreduce_kernel(const __grid_constant__ CUtensorMap tm_w,
                           const __grid_constant__ CUtensorMap tm_x, const RowLinearParams p) {
  using L = RowLinearSmem<NB>;
  constexpr int kStages = L::kStages;
  constexpr int kShare = NB / S;          // token rows this CTA finishes
  constexpr int kPairs = kShare / 2;
  static_assert(kShare >= 2 && kShare % 2 == 0, "shares are whole bf16 pairs");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* xch = reinterpret_cast<float*>(smem + L::kXchOff);   // [source CTA][share row][column]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint32_t* misc = reinterpret_cast<uint32_t*>(acc_full + 1);
  uint32_t* tmem_slot = misc;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  uint32_t* epoch_slot = misc + 2;
  volatile int* dead_slot = reinterpret_cast<volatile int*>(misc + 3);
  volatile uint32_t* health = misc + 4;                       // [source CTA], written by the cluster

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split = static_cast<int>(cluster_cta_rank());   // == blockIdx.x
  const int tile = blockIdx.y;
  const int n0 = tile * kRlTileN;
  const int ks_begin = split * p.steps_per_split;
  const int my_steps = min(p.k_steps, ks_begin + p.steps_per_split) - ks_begin;
  uint8_t* own = p.comm[p.rank];
  RowLinearComm* hdr = reinterpret_cast<RowLinearComm*>(own);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NB);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  cluster_arrive();     // #0: this CTA is up (its shared memory may be stored to from now on)
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_w);
      prefetch_tensormap(&tm_x);
      const uint64_t pol_x = l2_policy_evict_last();
      const uint64_t pol_w = l2_policy_evict_first();
      // The weight does not depend on the kernels before this one: its first stages are on
      // their way while those kernels drain (when the launch is a programmatic dependent one).
      const int ahead = min(my_steps, kStages);
      for (int i = 0; i < ahead; ++i) {
        mbar_arrive_expect_tx(&full[i], L::kStageBytes);
        tma_load_2d(smem + L::kWOff + i * L::kWBytes, &tm_w, &full[i], (ks_begin + i) * kRlKStep,
                    n0, pol_w);
      }
      grid_dependency_wait();
      for (int i = 0; i < ahead; ++i)
        tma_load_2d(smem + L::kXOff + i * L::kXBytes, &tm_x, &full[i], (ks_begin + i) * kRlKStep, 0,
                    pol_x);
      for (int i = ahead; i < my_steps; ++i) {
        const int slot = i % kStages;
        mbar_wait(&empty[slot], ((i / kStages) & 1) ^ 1, abort_flag, p.err_word);
        mbar_arrive_expect_tx(&full[slot], L::kStageBytes);
        const int k0 = (ks_begin + i) * kRlKStep;
        tma_load_2d(smem + L::kWOff + slot * L::kWBytes, &tm_w, &full[slot], k0, n0, pol_w);
        tma_load_2d(smem + L::kXOff + slot * L::kXBytes, &tm_x, &full[slot], k0, 0, pol_x);
      }
    }
    __syncwarp();
    cluster_wait();     // #0
    cluster_arrive();   // #1 (this warp stores to nobody)
    cluster_wait();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(kRlTileN, NB, false, false);
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO, version, SW128
    auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
    const bool leader = lane == 0;
    {
      for (int i = 0; i < my_steps; ++i) {
        const int slot = i % kStages;
        mbar_wait(&full[slot], (i / kStages) & 1, abort_flag, p.err_word);
        tc_fence_after_sync();
        if (leader) {
          const uint32_t a_lo = (smem_u32(smem + L::kWOff + slot * L::kWBytes) >> 4) | (1u << 16);
          const uint32_t b_lo = (smem_u32(smem + L::kXOff + slot * L::kXBytes) >> 4) | (1u << 16);
#pragma unroll
          for (int kk = 0; kk < kRlKStep / 16; ++kk)
            umma_ss(tmem_base, desc(a_lo + ((kk * 32) >> 4)), desc(b_lo + ((kk * 32) >> 4)), idesc,
                    i > 0 || kk > 0);
          umma_commit(&empty[slot]);
        }
        __syncwarp();
      }
      if (leader) umma_commit(acc_full);
    }
    __syncwarp();
    cluster_wait();     // #0
    cluster_arrive();   // #1
    cluster_wait();
  } else {
    // ------------------------------------------------------------------ epilogue + all-reduce
    const int et = threadIdx.x - 64;                       // 0..127
    const int col = (warp & 3) * 32 + lane;                // tensor-memory lane == output column
    const bool col_ok = n0 + col < p.n_total;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // Everything below reads or writes memory other kernels touch: wait for them first.
    grid_dependency_wait();
    if (et == 0) {
      // A wait of an earlier call through this communicator ran out: the ranks are no longer
      // in step.  The GEMM still runs (its loads are already on their way), but nothing is
      // published or waited for.
      *dead_slot = p.world > 1 && *reinterpret_cast<volatile uint32_t*>(&hdr->out_of_step) != 0u;
      *epoch_slot = p.world > 1 ? *reinterpret_cast<volatile uint32_t*>(&hdr->epoch) + 1u : 1u;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const uint32_t epoch = *epoch_slot;
    const uint32_t parity = epoch & 1u;
    const bool dead = *dead_slot != 0;
    mbar_wait(acc_full, 0, abort_flag, p.err_word);
    tc_fence_after_sync();
    cluster_wait();     // #0: every CTA of the cluster is up
    if (!dead) {
      // split-K: token row t of this CTA's D goes to CTA t / kShare, into its slab of our rows
      const uint32_t xch_addr = smem_u32(xch) + static_cast<uint32_t>(split * kShare * kRlTileN + col) * 4u;
      uint32_t dst_base[S];
#pragma unroll
      for (int d = 0; d < S; ++d) dst_base[d] = cluster_map(xch_addr, d);
#pragma unroll
      for (int c = 0; c < NB / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + lane_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const int token = c * 32 + k;
          st_cluster_f32(dst_base[token / kShare] +
                             static_cast<uint32_t>((token % kShare) * kRlTileN) * 4u,
                         __uint_as_float(r[k]));
        }
      }
    }
    if (et < S) {
      const uint32_t ok = (!dead && !*abort_flag) ? 1u : 0u;
      st_cluster_u32(cluster_map(smem_u32(const_cast<uint32_t*>(health)) + split * 4u, et), ok);
    }
    __syncwarp();
    cluster_arrive();   // #1: every piece and every health word has been stored
    cluster_wait();
    const int t_begin = split * kShare;
    float part[kShare];
    bool healthy = true;
#pragma unroll
    for (int i = 0; i < kShare; ++i) {
      float a = xch[i * kRlTileN + col];
#pragma unroll
      for (int r = 1; r < S; ++r) a += xch[(r * kShare + i) * kRlTileN + col];
      part[i] = a;
    }
#pragma unroll
    for (int r = 0; r < S; ++r) healthy = healthy && health[r] != 0;
    // A broken pipeline anywhere in the cluster publishes nothing: the peers' own bounded waits
    // then report the failure instead of summing garbage.
    const bool active = healthy && col_ok;
    const int slot = tile * S + split;
    __nv_bfloat16* o = p.out + static_cast<int64_t>(t_begin) * p.out_row_stride + n0 + col;

    if (p.world == 1) {
      if (active) {
#pragma unroll
        for (int i = 0; i < kShare; ++i)
          if (t_begin + i < p.num_tokens)
            o[static_cast<int64_t>(i) * p.out_row_stride] = __float2bfloat16_rn(part[i]);
      }
    } else {
      // One shot (two ranks): every rank sends its partial to every peer and reduces everything.
      // Two shots (more ranks): (tile, share) `slot` has an owner rank; the others send their
      // partial to the owner only, the owner reduces and sends the bf16 result back to everyone,
      // so a rank's traffic stays about two partials whatever the number of ranks.
      const int owner = p.two_shot ? slot % p.world : -1;
      const bool i_reduce = owner < 0 || owner == p.rank;     // this CTA adds the partials up
      const int result_area = p.world;                        // area index after the ranks' own
      uint32_t mine[kPairs];
#pragma unroll
      for (int u = 0; u < kPairs; ++u) mine[u] = pack_bf16x2(part[2 * u], part[2 * u + 1]);
      if (active && (owner < 0 || owner != p.rank)) {
        for (int peer = 0; peer < p.world; ++peer) {
          if (peer == p.rank || (owner >= 0 && peer != owner)) continue;
          uint2* dst = rl_unit(p.comm[peer], p, parity, p.rank, slot, kPairs, 0, col);
#pragma unroll
          for (int u = 0; u < kPairs; ++u)
            if (t_begin + 2 * u < p.num_tokens) st_u2(dst + u * kRlTileN, mine[u], epoch);
        }
      }
      constexpr int kChunk = kPairs < 8 ? kPairs : 8;
      bool gave_up = !active;
#pragma unroll
      for (int c = 0; c < kPairs; c += kChunk) {
        uint2 got[W][kChunk];
        // wanted: the partial of every peer when this CTA reduces, else the owner's result
        // (kept in row 0)
#pragma unroll
        for (int src = 0; src < W; ++src)
#pragma unroll
          for (int u = 0; u < kChunk; ++u) {
            const bool from_src = i_reduce ? (src < p.world && src != p.rank) : (src == 0);
            const bool wanted = from_src && !gave_up && t_begin + 2 * (c + u) < p.num_tokens;
            got[src][u].x = 0u;
            got[src][u].y = wanted ? epoch - 1u : epoch;
          }
        // Rounds of polling: every unit that has not landed yet is re-read, all reads of a round
        // in flight together, so a round costs one memory round trip whatever the unit count.
        uint64_t t0 = 0;
        for (uint32_t round = 1;; ++round) {
#pragma unroll
          for (int src = 0; src < W; ++src) {
            if (i_reduce ? src < p.world : src == 0) {
              const uint2* from =
                  rl_unit(own, p, parity, i_reduce ? src : result_area, slot, kPairs, c, col);
#pragma unroll
              for (int u = 0; u < kChunk; ++u)
                if (got[src][u].y != epoch) got[src][u] = ld_volatile_u2(from + u * kRlTileN);
            }
          }
          bool pending = false;
#pragma unroll
          for (int src = 0; src < W; ++src)
#pragma unroll
            for (int u = 0; u < kChunk; ++u) pending = pending || got[src][u].y != epoch;
          if (!pending) break;
          if ((round & 31u) == 0u) {
            if (*abort_flag) {
              gave_up = true;
              break;
            }
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
              t0 = now;
            } else if (now - t0 > p.peer_timeout_ns) {
              *abort_flag = 1;
              *reinterpret_cast<volatile uint32_t*>(&hdr->out_of_step) = 1u;
              report_wait_timeout(p.err_word);
              gave_up = true;
              break;
            }
          }
        }
        if (!gave_up) {
#pragma unroll
          for (int u = 0; u < kChunk; ++u) {
            const int t = t_begin + 2 * (c + u);
            if (t >= p.num_tokens) continue;
            uint32_t res;
            if (i_reduce) {
              float a0 = 0.f, a1 = 0.f;
#pragma unroll
              for (int src = 0; src < W; ++src) {
                if (src < p.world) {
                  const uint32_t v = (src == p.rank) ? mine[c + u] : got[src][u].x;
                  a0 += bf16_lo(v);
                  a1 += bf16_hi(v);
                }
              }
              res = pack_bf16x2(a0, a1);
              if (owner >= 0) {
                for (int peer = 0; peer < p.world; ++peer)
                  if (peer != p.rank)
                    st_u2(rl_unit(p.comm[peer], p, parity, result_area, slot, kPairs, c + u, col),
                          res, epoch);
              }
            } else {
              res = got[0][u].x;
            }
            unsigned short* o16 = reinterpret_cast<unsigned short*>(o);
            o16[static_cast<int64_t>(2 * (c + u)) * p.out_row_stride] =
                static_cast<unsigned short>(res & 0xffffu);
            if (t + 1 < p.num_tokens)
              o16[static_cast<int64_t>(2 * (c + u) + 1) * p.out_row_stride] =
                  static_cast<unsigned short>(res >> 16);
          }
        }
      }
    }
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, NB);
  }
  if (threadIdx.x == 0 && p.world > 1) {
    // last CTA out publishes the epoch for the next call (the next launch on the stream reads it)
    if (atomicAdd(&hdr->ticket, 1u) == gridDim.x * gridDim.y - 1) {
      hdr->ticket = 0;
      *reinterpret_cast<volatile uint32_t*>(&hdr->epoch) = *epoch_slot;
    }
  }
}

}  // namespace b200attn
