// FP8 (e4m3 x e4m3) GEMM with 128x128 weight-block scales and per-token
// per-128-column activation scales, fp32 accumulation, bf16/fp16 output:
//
//   Y[m, n] = sum_kb ( sum_{k in kb} X8[m, k] * W8[n, k] ) * a_scale[m, kb] * w_scale[n / 128, kb]
//
// sm_100a design
//   * tcgen05.mma kind::f8f6f4 (UMMA 128 x BN x 32), operands staged in shared
//     memory by TMA (2-D tiled loads, 128-byte swizzle, no multicast), fp32
//     accumulators in tensor memory.
//   * The scales change every 128 columns of K, so each K block is accumulated
//     in its own TMEM buffer (two buffers, ping-pong) and the epilogue warps
//     promote it into fp32 registers with that block's scale (tcgen05.ld +
//     FFMA) while the tensor core already works on the next block.
//   * Warp roles: E epilogue warps (E = 4 or 8), one TMA producer warp, one
//     MMA-issuer warp that also owns the TMEM allocation.
//   * Two orientations share the kernel.  "Normal" (many tokens): the 128 UMMA
//     rows are tokens, the BN columns are weight rows.  "Swapped" (few tokens,
//     decode): the 128 UMMA rows are weight rows and the BN columns are tokens,
//     so a handful of tokens still fills the tensor core's M and the kernel is
//     a pure weight-streaming (HBM-bound) loop.
//   * Schedule: grid = (tiles, split).  When a shape has fewer output tiles
//     than SMs (decode), the K range of every tile is cut into `split` (<= 8)
//     parts that run as one thread-block cluster; each CTA parks its fp32
//     partial in its own shared memory and, after a cluster barrier, reduces a
//     slice of the tile by reading its peers through distributed shared
//     memory in a fixed order (deterministic; no global partials, no atomics,
//     no spinning).  With enough tiles split = 1 and CTAs store directly.
//   * Every mbarrier wait is bounded; a wait that runs out sets
//     MIE_STATUS_WAIT_TIMEOUT, the roles fall through to the common exit and
//     TMEM is released.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "umma.cuh"

namespace mie {
namespace {

constexpr int kTileR = 128;  // UMMA M
constexpr int kBlockK = 128; // bytes of K per pipeline stage = one scale block
constexpr int kUmmaK = 32;   // fp8 elements per tcgen05.mma

__device__ __forceinline__ void epi_bar_sync(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// --------------------------------------------------------------------------
// Kernel
// --------------------------------------------------------------------------
struct GemmParams {
  // Row operand rows / column operand rows (see the orientation note above).
  int rows_r, rows_c, k;
  int m, n;               // logical problem (tokens, weight rows)
  const float* a_scale;   // [k_blocks][a_scale_ld]  (token scales, K-block major)
  int a_scale_ld;
  const float* w_scale;   // [ceil(n/128)][w_scale_ld]
  int w_scale_ld;
  void* y;                // [m][ldy] bf16 or fp16
  long long ldy;
  int out_f16;
  int* status;
  long long* trace;       // optional [CTAs][16] globaltimer stamps (profiling aid), or null
};

__device__ __forceinline__ void trace_stamp(const GemmParams& p, int slot) {
  if (p.trace != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[(size_t)(blockIdx.x * gridDim.y + blockIdx.y) * 16 + slot] = (long long)t;
  }
}

// Scale staging: per chunk of kChunkKb K blocks the epilogue warps pull every
// scale they will need into shared memory in one batch, so no global-memory
// latency sits between two K blocks.
template <int BN, bool kSwap>
struct ScaleStage {
  static constexpr int kWidth = kSwap ? BN : kTileR;             // token scales per K block
  static constexpr int kChunkKb = kSwap ? (4096 / BN > 32 ? 32 : 4096 / BN) : 16;
  static constexpr int kWBlocks = kSwap ? 1 : (BN + 127) / 128;  // weight scale blocks per tile column range
  static constexpr int kFloats = kChunkKb * kWidth + kChunkKb * kWBlocks;
};

template <int BN, int E, bool kSwap>
struct GemmSmem {
  static constexpr int kStageBytes = kTileR * kBlockK + BN * kBlockK;
  static constexpr int kScaleBytes = ScaleStage<BN, kSwap>::kFloats * 4;
  // Narrow column tiles (few tokens) use few registers: two CTAs share an SM, which halves the cost of a
  // partial last wave and doubles the TMA requests in flight per SM.
  static constexpr int kCtasPerSm = BN <= 32 ? 2 : 1;
  static constexpr int kBudget = (kCtasPerSm == 2 ? 100 : 200) * 1024 - kScaleBytes;
  static constexpr int kStages = (kBudget / kStageBytes) > 12 ? 12 : (kBudget / kStageBytes);
  static constexpr int kBarBytes = (2 * kStages + 16) * 8;
  static constexpr int kTotal = kStages * kStageBytes + kBarBytes + kScaleBytes + 64 + 1024;
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_smem(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Largest split * ceil(chunks / split) over the allowed split factors (1..8).
constexpr int max_reduction_chunks(int chunks) {
  int worst = chunks;
  for (int split = 2; split <= 8; ++split) {
    const int used = split * ((chunks + split - 1) / split);
    if (used > worst) worst = used;
  }
  return worst;
}

template <int BN, int E, bool kSwap>
__global__ void __launch_bounds__((E + 2) * 32, (BN <= 32 ? 2 : 1))
    fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_c,
                    const GemmParams p) {
  using S = GemmSmem<BN, E, kSwap>;
  using SS = ScaleStage<BN, kSwap>;
  constexpr int kStages = S::kStages;
  constexpr int kCols = E == 8 ? BN / 2 : BN;  // accumulator columns owned by one epilogue warp
  // Accumulator ring in TMEM: as many BN-column buffers as fit (at most 8), so the MMA issuer can run
  // several K blocks ahead of the promotion.
  constexpr int kAcc = (512 / S::kCtasPerSm) / BN > 8 ? 8 : (512 / S::kCtasPerSm) / BN;
  constexpr uint32_t kTmemCols = kAcc * BN < 32 ? 32 : kAcc * BN;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  static_assert(kCols % 16 == 0, "column slice must be a multiple of 16");
  // The stage ring doubles as the landing zone of the cluster reduction: split slots of ceil(BN/8/split)
  // 8-column chunks each, at most (BN/8 + 7) chunks in total.
  static_assert(kStages * S::kStageBytes >= max_reduction_chunks(BN / 8) * 8 * kTileR * 4,
                "stage ring too small for the reduction");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 8;
  float* sscale = reinterpret_cast<float*>(tmem_empty + 8);  // staged scales of the current K chunk
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sscale + SS::kFloats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (p.k + kBlockK - 1) / kBlockK;
  const int tiles_r = (p.rows_r + kTileR - 1) / kTileR;
  const int split = gridDim.y, rank = blockIdx.y, tile = blockIdx.x;  // cluster = (1, split, 1)
  const int tr = tile % tiles_r, tc = tile / tiles_r;
  const int kb_first = (int)((long long)kb_total * rank / split);
  const int kb_last = (int)((long long)kb_total * (rank + 1) / split);  // exclusive

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < kAcc; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], E);
    }
    mbar_fence_init();
    tma_prefetch_desc(&map_r);
    tma_prefetch_desc(&map_c);
  }
  if (warp == E + 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers, tensor-map prefetch and the TMEM allocation above overlap the tail of the previous kernel.
  chain_wait();
  chain_release();
  if (threadIdx.x == 0) {
    trace_stamp(p, 0);
    trace_stamp(p, 1);
  }

  // Epilogue state that outlives the role branch (the reduction below needs it).
  constexpr int kEpiThreads = E * 32;
  const int quad = warp & 3, half = E == 8 ? (warp >> 2) & 1 : 0;
  const int row_in_tile = quad * 32 + lane;
  const int col0 = half * kCols;
  float acc[kCols];

  if (warp == E) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const uint64_t stream_policy = l2_evict_first_policy();
      uint32_t n = 0;
      for (int kb = kb_first; kb < kb_last; ++kb, ++n) {
        const int s = n % kStages;
        if (!mbar_wait_bounded(&empty_bar[s], ((n / kStages) & 1u) ^ 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        uint8_t* dst = stage_base + (size_t)s * S::kStageBytes;
        mbar_expect_tx(&full_bar[s], S::kStageBytes);
        if (kSwap)  // decode-time weights are streamed once: keep them from flushing L2
          tma_load_2d_hint(dst, &map_r, &full_bar[s], kb * kBlockK, tr * kTileR, stream_policy);
        else
          tma_load_2d(dst, &map_r, &full_bar[s], kb * kBlockK, tr * kTileR);
        tma_load_2d(dst + kTileR * kBlockK, &map_c, &full_bar[s], kb * kBlockK, tc * BN);
        if (n == 0) trace_stamp(p, 2);
      }
      trace_stamp(p, 3);
    }
  } else if (warp == E + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f8(BN);
      uint32_t n = 0;
      for (int kb = kb_first; kb < kb_last; ++kb, ++n) {
        const int s = n % kStages, b = n % kAcc;
        if (!mbar_wait_bounded(&full_bar[s], (n / kStages) & 1u) ||
            !mbar_wait_bounded(&tmem_empty[b], ((n / kAcc) & 1u) ^ 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        if (n == 0) trace_stamp(p, 4);
        const uint32_t a_addr = smem_u32(stage_base + (size_t)s * S::kStageBytes);
        const uint32_t b_addr = a_addr + kTileR * kBlockK;
        const uint64_t da = smem_desc_k128(a_addr), db = smem_desc_k128(b_addr);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          umma_f8(tmem_base + b * BN, da + (uint64_t)(k * kUmmaK / 16), db + (uint64_t)(k * kUmmaK / 16), idesc,
                  k > 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs have read it
        umma_commit(&tmem_full[b]);  // hands the K block's accumulator to the epilogue
      }
      trace_stamp(p, 5);
    }
  } else {
    // ---------------- Epilogue warps: promote every K block with its scales ----------------
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int epi_tid = threadIdx.x;  // epilogue warps are warps 0..E-1
    const int wblk = tr;              // swapped mode: the tile's 128 weight rows are one scale block
    uint32_t n = 0;
    bool ok = true;
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
    for (int kb0 = kb_first; kb0 < kb_last && ok; kb0 += SS::kChunkKb) {
      const int kc = kb_last - kb0 < SS::kChunkKb ? kb_last - kb0 : SS::kChunkKb;
      // Stage this chunk's scales (all loads in flight together).
      epi_bar_sync(kEpiThreads);  // the previous chunk's readers are done
      float* s_w = sscale + SS::kChunkKb * SS::kWidth;
      if (kSwap) {
        // Products a_scale[token] * w_scale, one per (K block, column).
        for (int i = epi_tid; i < kc * BN; i += kEpiThreads) {
          const int kk = i / BN, tok = tc * BN + i % BN;
          const float ws = p.w_scale[(long long)wblk * p.w_scale_ld + kb0 + kk];
          sscale[i] = tok < p.m ? p.a_scale[(long long)(kb0 + kk) * p.a_scale_ld + tok] * ws : 0.f;
        }
      } else {
        for (int i = epi_tid; i < kc * kTileR; i += kEpiThreads) {
          const int kk = i / kTileR, tok = tr * kTileR + i % kTileR;
          sscale[i] = tok < p.m ? p.a_scale[(long long)(kb0 + kk) * p.a_scale_ld + tok] : 0.f;
        }
        for (int i = epi_tid; i < kc * SS::kWBlocks; i += kEpiThreads) {
          const int kk = i / SS::kWBlocks, blk = (tc * BN) / 128 + i % SS::kWBlocks;
          s_w[i] = blk * 128 < p.n ? p.w_scale[(long long)blk * p.w_scale_ld + kb0 + kk] : 0.f;
        }
      }
      epi_bar_sync(kEpiThreads);
      if (epi_tid == 0 && n == 0) trace_stamp(p, 6);
      for (int kk = 0; kk < kc; ++kk, ++n) {
        const int b = n % kAcc;
        float s_row = 0.f;
        if (!kSwap) s_row = sscale[kk * kTileR + row_in_tile] * s_w[kk * SS::kWBlocks + (col0 / 128)];
        const float* s_col = sscale + kk * BN + col0;  // swapped mode: one product per column
        if (!mbar_wait_bounded(&tmem_full[b], (n / kAcc) & 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          ok = false;
          break;
        }
        tc_fence_after();
        if (epi_tid == 0 && n == 0) trace_stamp(p, 7);
        const uint32_t taddr = lane_addr + (uint32_t)(b * BN + col0);
        if constexpr (kCols % 64 == 0) {
          // Two loads in flight per wait: halves the TMEM round trips per K block.
#pragma unroll
          for (int c = 0; c < kCols; c += 64) {
            float d0[32], d1[32];
            tmem_ld32(taddr + c, d0);
            tmem_ld32(taddr + c + 32, d1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(d0[j], kSwap ? s_col[c + j] : s_row, acc[c + j]);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              acc[c + 32 + j] = fmaf(d1[j], kSwap ? s_col[c + 32 + j] : s_row, acc[c + 32 + j]);
          }
        } else if constexpr (kCols % 32 == 0) {
#pragma unroll
          for (int c = 0; c < kCols; c += 32) {
            float d[32];
            tmem_ld32(taddr + c, d);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(d[j], kSwap ? s_col[c + j] : s_row, acc[c + j]);
          }
        } else {
          float d[16];
          tmem_ld16(taddr, d);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = fmaf(d[j], kSwap ? s_col[j] : s_row, acc[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[b]);
      }
    }
    if (epi_tid == 0) trace_stamp(p, 8);
  }

  // ---------------- output: direct (split == 1) or reduced across the cluster ----------------
  const int r_glob = tr * kTileR + row_in_tile;  // token (normal) or weight row (swapped)
  if (split == 1) {
    if (warp < E) {
      if (kSwap) {
        if (r_glob < p.n) {
#pragma unroll
          for (int j = 0; j < kCols; ++j) {
            const int tok = tc * BN + col0 + j;
            if (tok < p.m) {
              if (p.out_f16)
                reinterpret_cast<__half*>(p.y)[(long long)tok * p.ldy + r_glob] = __float2half_rn(acc[j]);
              else
                reinterpret_cast<__nv_bfloat16*>(p.y)[(long long)tok * p.ldy + r_glob] = __float2bfloat16_rn(acc[j]);
            }
          }
        }
      } else if (r_glob < p.m) {
        const int n0 = tc * BN + col0;
        uint16_t* yrow = reinterpret_cast<uint16_t*>(p.y) + (long long)r_glob * p.ldy + n0;
        const bool vec = (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) && (n0 + kCols <= p.n);
        if (vec) {
#pragma unroll
          for (int j = 0; j < kCols; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              w[q] = p.out_f16 ? Mma16816<__half>::pack(acc[j + 2 * q], acc[j + 2 * q + 1])
                               : Mma16816<__nv_bfloat16>::pack(acc[j + 2 * q], acc[j + 2 * q + 1]);
            }
            *reinterpret_cast<uint4*>(yrow + j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < kCols; ++j) {
            if (n0 + j < p.n) {
              if (p.out_f16)
                reinterpret_cast<__half*>(yrow)[j] = __float2half_rn(acc[j]);
              else
                reinterpret_cast<__nv_bfloat16*>(yrow)[j] = __float2bfloat16_rn(acc[j]);
            }
          }
        }
      }
    }
  } else {
    // Every MMA of this CTA has completed (the epilogue consumed the last accumulator), so the stage ring
    // is free.  Rank d owns the 8-column chunks [d * slice, (d + 1) * slice) of the tile: every CTA pushes
    // its partial of those columns into slot [its own rank] of the owner's ring (remote shared-memory
    // stores), the cluster barrier publishes them, and the owner adds the slots in rank order.
    constexpr int kChunks = BN / 8;
    const int slice = (kChunks + split - 1) / split;            // chunks per owner
    const int slice_floats = slice * 8 * kTileR;                 // one slot
    const uint32_t red_addr = smem_u32(stage_base);
    cluster_sync_all();  // every CTA of the cluster is done with its own stage ring
    if (warp < E) {
#pragma unroll
      for (int j = 0; j < kCols; ++j) {
        const int col = col0 + j, owner = (col >> 3) / slice;
        const int local_col = col - owner * slice * 8;
        const uint32_t local = red_addr + (uint32_t)((rank * slice_floats + local_col * kTileR + row_in_tile) * 4);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)owner));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(acc[j]) : "memory");
      }
    }
    if (threadIdx.x == 0) trace_stamp(p, 9);
    cluster_sync_all();
    if (warp < E) {
      const float* red = reinterpret_cast<const float*>(stage_base);
      const int chunk_lo = rank * slice, chunk_hi = (rank + 1) * slice < kChunks ? (rank + 1) * slice : kChunks;
      for (int ch = chunk_lo + (E == 8 ? (warp >> 2) : 0); ch < chunk_hi; ch += (E == 8 ? 2 : 1)) {
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
        for (int peer = 0; peer < split; ++peer) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            sum[j] += red[peer * slice_floats + ((ch - chunk_lo) * 8 + j) * kTileR + row_in_tile];
        }
        if (kSwap) {
          if (r_glob < p.n) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int tok = tc * BN + ch * 8 + j;
              if (tok < p.m) {
                if (p.out_f16)
                  reinterpret_cast<__half*>(p.y)[(long long)tok * p.ldy + r_glob] = __float2half_rn(sum[j]);
                else
                  reinterpret_cast<__nv_bfloat16*>(p.y)[(long long)tok * p.ldy + r_glob] =
                      __float2bfloat16_rn(sum[j]);
              }
            }
          }
        } else if (r_glob < p.m) {
          const int n0 = tc * BN + ch * 8;
          uint16_t* yrow = reinterpret_cast<uint16_t*>(p.y) + (long long)r_glob * p.ldy + n0;
          const bool vec = (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) && (n0 + 8 <= p.n);
          if (vec) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              w[q] = p.out_f16 ? Mma16816<__half>::pack(sum[2 * q], sum[2 * q + 1])
                               : Mma16816<__nv_bfloat16>::pack(sum[2 * q], sum[2 * q + 1]);
            }
            *reinterpret_cast<uint4*>(yrow) = make_uint4(w[0], w[1], w[2], w[3]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (n0 + j < p.n) {
                if (p.out_f16)
                  reinterpret_cast<__half*>(yrow)[j] = __float2half_rn(sum[j]);
                else
                  reinterpret_cast<__nv_bfloat16*>(yrow)[j] = __float2bfloat16_rn(sum[j]);
              }
            }
          }
        }
      }
    }
    // No CTA reads a peer after the barrier above, so nothing more is needed before exit.
  }
  if (threadIdx.x == 0) trace_stamp(p, 11);

  tc_fence_before();
  __syncthreads();
  if (warp == E + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) trace_stamp(p, 12);
}

// --------------------------------------------------------------------------
// Activation quantiser: per token, per 128 columns.  One half-warp per group.
// --------------------------------------------------------------------------
template <typename T>
__global__ void quantize_kernel(const T* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                                float* __restrict__ scales, int scale_ld, int m, int k) {
  const int groups = (k + 127) / 128;
  const long long hw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;  // half-warp id
  const int l16 = threadIdx.x & 15;
  const bool live = hw < (long long)m * groups;  // dead lanes still take part in the shuffles
  const int row = live ? (int)(hw / groups) : 0, grp = live ? (int)(hw % groups) : 0;
  const int c0 = grp * 128 + l16 * 8;
  float v[8];
  const T* src = x + (long long)row * ldx + c0;
  if (!live) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  } else if (c0 + 8 <= k && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_float<T>(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = c0 + j < k ? to_float<T>(src[j]) : 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!live) return;
  const float scale = __fdiv_rn(amax, 448.0f);  // raw scale is what gets stored (0 for a zero group)
  const float denom = fmaxf(scale, 1e-12f);
  uint32_t packed[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(v[4 * h], denom), __fdiv_rn(v[4 * h + 1], denom)), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(v[4 * h + 2], denom), __fdiv_rn(v[4 * h + 3], denom)), __NV_SATFINITE, __NV_E4M3);
    packed[h] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  uint8_t* dst = q + (long long)row * ldq + c0;
  if (c0 + 8 <= k && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
  } else {
    const uint8_t* b = reinterpret_cast<const uint8_t*>(packed);
    for (int j = 0; j < 8; ++j)
      if (c0 + j < k) dst[j] = b[j];
  }
  if (l16 == 0) scales[(long long)grp * scale_ld + row] = scale;
}

// --------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------
struct Map2Key {
  const void* ptr;
  long long rows, k, ld;
  int box_rows;
  bool operator==(const Map2Key& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows;
  }
};
struct Map2Hash {
  size_t operator()(const Map2Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.k;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

int operand_map(const void* ptr, long long rows, long long k, long long ld, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<Map2Key, CUtensorMap, Map2Hash> cache;
  Map2Key key{ptr, rows, k, ld, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t dims[2] = {(uint64_t)k, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)ld};
  const uint32_t box[2] = {(uint32_t)kBlockK, (uint32_t)box_rows};
  const int rc = make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 16384) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

// K-split factor for a shape with `tiles` output tiles of `kb_total` K blocks.  Cost model in units of
// one K block of a 256-column tile: waves * (K blocks per CTA + fixed cost) + the cluster reduction
// (which grows with the tile width).  Only cluster sizes 1, 2 and 4 are used: 3 and 8 co-schedule badly
// with one 200 KB CTA per SM (measured), and larger splits leave too little work per CTA.
int choose_split(long long tiles, int kb_total, int bn, int ctas_per_sm, int max_split) {
  const int slots = sm_count() * ctas_per_sm;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 4; s *= 2) {
    if (s > kb_total || (max_split > 0 && s > max_split)) break;
    const long long ctas = tiles * s;
    const double waves = (double)((ctas + slots - 1) / slots);
    const double cost = waves * ((kb_total + s - 1) / s + 4.0) + (s > 1 ? bn / 32.0 : 0.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

template <int BN, int E, bool kSwap>
int launch_gemm(const CUtensorMap& mr, const CUtensorMap& mc, const GemmParams& p, long long tiles, int split,
                cudaStream_t stream) {
  using S = GemmSmem<BN, E, kSwap>;
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(fp8_gemm_kernel<BN, E, kSwap>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  S::kTotal));
    configured[dev] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)tiles, (unsigned)split, 1);
  config.blockDim = dim3((E + 2) * 32, 1, 1);
  config.dynamicSmemBytes = S::kTotal;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)split;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = chained_launch_enabled() ? 2 : 1;
  MIE_CUDA(cudaLaunchKernelEx(&config, fp8_gemm_kernel<BN, E, kSwap>, mr, mc, p));
  MIE_LAUNCH_CHECK("fp8_gemm_kernel");
  return MIE_OK;
}

// Column-tile width for the swapped orientation: smallest of 16/32/64/128 covering m.
int swap_bn(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_fp8_quantize(const void* x, int64_t ldx, int32_t dtype, void* q, int64_t ldq, float* scales,
                                int32_t scale_ld, int32_t m, int32_t k, void* stream) {
  MIE_CHECK_ARG(x && q && scales, "null pointer");
  MIE_CHECK_ARG(dtype == MIE_DTYPE_BF16 || dtype == MIE_DTYPE_F16, "activation must be bf16 or fp16");
  MIE_CHECK_ARG(m >= 0 && k >= 1 && scale_ld >= m && ldx >= k && ldq >= k, "invalid quantiser shape");
  if (m == 0) return MIE_OK;
  const long long half_warps = (long long)m * ((k + 127) / 128);
  const int threads = 256;
  const long long blocks = (half_warps * 16 + threads - 1) / threads;
  if (dtype == MIE_DTYPE_BF16)
    quantize_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, scales, scale_ld, m, k);
  else
    quantize_kernel<__half><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        (const __half*)x, ldx, (uint8_t*)q, ldq, scales, scale_ld, m, k);
  MIE_LAUNCH_CHECK("quantize_kernel");
  return MIE_OK;
}

extern "C" int mie_fp8_gemm(const void* x8, int64_t ldx, const float* a_scale, int32_t a_scale_ld, const void* w8,
                            int64_t ldw, const float* w_scale, int32_t w_scale_ld, void* y, int64_t ldy,
                            int32_t out_dtype, int32_t m, int32_t n, int32_t k, int32_t max_split, int32_t* status,
                            int64_t* trace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MIE_CHECK_ARG(x8 && a_scale && w8 && w_scale && y, "null pointer");
  MIE_CHECK_ARG(m >= 0 && n >= 1 && k >= 1, "invalid GEMM shape %d x %d x %d", m, n, k);
  MIE_CHECK_ARG(out_dtype == MIE_DTYPE_BF16 || out_dtype == MIE_DTYPE_F16, "output must be bf16 or fp16");
  MIE_CHECK_ARG(ldx % 16 == 0 && ldw % 16 == 0, "operand row strides must be multiples of 16 bytes");
  MIE_CHECK_ARG(((reinterpret_cast<uintptr_t>(x8) | reinterpret_cast<uintptr_t>(w8)) & 15) == 0,
                "operands must be 16-byte aligned");
  MIE_CHECK_ARG(ldy >= n && a_scale_ld >= m && w_scale_ld >= (k + 127) / 128, "invalid leading dimension");
  if (m == 0) return MIE_OK;

  const bool swap = m <= 128;
  const int bn = swap ? swap_bn(m) : 256;
  const int kb = (k + kBlockK - 1) / kBlockK;
  const long long tiles_r = swap ? (n + kTileR - 1) / kTileR : (m + kTileR - 1) / kTileR;
  const long long tiles_c = swap ? (m + bn - 1) / bn : (n + bn - 1) / bn;
  const long long tiles = tiles_r * tiles_c;
  MIE_CHECK_ARG(tiles <= 0x7fffffff, "too many output tiles (%lld)", tiles);
  const int split = choose_split(tiles, kb, bn, bn <= 32 ? 2 : 1, max_split);

  GemmParams p;
  p.rows_r = swap ? n : m;
  p.rows_c = swap ? m : n;
  p.k = k;
  p.m = m;
  p.n = n;
  p.a_scale = a_scale;
  p.a_scale_ld = a_scale_ld;
  p.w_scale = w_scale;
  p.w_scale_ld = w_scale_ld;
  p.y = y;
  p.ldy = ldy;
  p.out_f16 = out_dtype == MIE_DTYPE_F16;
  p.status = status;
  p.trace = reinterpret_cast<long long*>(trace);

  CUtensorMap mr, mc;
  if (swap) {
    if (int rc = operand_map(w8, n, k, ldw, kTileR, &mr)) return rc;
    if (int rc = operand_map(x8, m, k, ldx, bn, &mc)) return rc;
    switch (bn) {
      case 16: return launch_gemm<16, 4, true>(mr, mc, p, tiles, split, stream);
      case 32: return launch_gemm<32, 4, true>(mr, mc, p, tiles, split, stream);
      case 64: return launch_gemm<64, 4, true>(mr, mc, p, tiles, split, stream);
      default: return launch_gemm<128, 4, true>(mr, mc, p, tiles, split, stream);
    }
  }
  if (int rc = operand_map(x8, m, k, ldx, kTileR, &mr)) return rc;
  if (int rc = operand_map(w8, n, k, ldw, bn, &mc)) return rc;
  return launch_gemm<256, 8, false>(mr, mc, p, tiles, split, stream);
}
