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
//     in its own TMEM buffer (a ring) and the promotion warps add it into fp32
//     registers with that block's scale (tcgen05.ld + FFMA) while the tensor
//     core already works on the next block.
//   * Two kernels.  Up to 128 tokens (decode): fp8_gemm_kernel, "swapped" - the
//     128 UMMA rows are weight rows and the BN = 16..128 columns are tokens, so
//     a handful of tokens still fills the tensor core's M and the kernel is a
//     pure weight-streaming (HBM-bound) loop; E = 4 promotion warps, one TMA
//     producer warp, one MMA-issuer warp that also owns the TMEM allocation.
//     More than 128 tokens: fp8_gemm_wide_kernel (described at its definition).
//   * A shape with fewer output tiles than SMs cuts the K range of every tile
//     into parts that run as one thread-block cluster and are reduced through
//     distributed shared memory in a fixed order (deterministic; no global
//     partials, no atomics, no spinning).
//   * Every mbarrier wait is bounded; a wait that runs out sets
//     MIE_STATUS_WAIT_TIMEOUT, the roles fall through to the common exit and
//     TMEM is released.
#include <cstdlib>
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
  int m, n, k;            // tokens, weight rows, reduction length
  const float* a_scale;   // [k_blocks][a_scale_ld]  (token scales, K-block major)
  int a_scale_ld;
  const float* w_scale;   // [ceil(n/128)][w_scale_ld]
  int w_scale_ld;
  void* y;                // [m][ldy] bf16 or fp16
  long long ldy;
  int out_f16;
  int* status;
  int prefetch;           // weights of the first K blocks are requested before the launch-chain wait
  // Wide kernel only: this launch covers output tiles [tile_begin, tile_end).  late_wait: the launch-chain
  // wait is taken at the end of the kernel instead of the start (second launch of a two-launch GEMM, whose
  // inputs are already known to be complete because the first launch waited for them).
  int tile_begin, tile_end, late_wait;
};

// Scale staging: per chunk of kChunkKb K blocks the promotion warps pull every
// scale product they will need into shared memory in one batch, so no
// global-memory latency sits between two K blocks.
template <int BN>
struct ScaleStage {
  static constexpr int kChunkKb = 4096 / BN > 32 ? 32 : 4096 / BN;
  static constexpr int kFloats = kChunkKb * BN;  // one a_scale * w_scale product per (K block, token)
};

constexpr int kNarrowEpiWarps = 4;  // promotion warps of fp8_gemm_kernel (one per TMEM lane quadrant)

template <int BN>
struct GemmSmem {
  static constexpr int kStageBytes = kTileR * kBlockK + BN * kBlockK;
  static constexpr int kScaleBytes = ScaleStage<BN>::kFloats * 4;
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

// Largest split * ceil(chunks / split) over the allowed split factors (1..8).
constexpr int max_reduction_chunks(int chunks) {
  int worst = chunks;
  for (int split = 2; split <= 8; ++split) {
    const int used = split * ((chunks + split - 1) / split);
    if (used > worst) worst = used;
  }
  return worst;
}

__device__ __forceinline__ void store_out(const GemmParams& p, long long token, int col, float v) {
  if (p.out_f16)
    reinterpret_cast<__half*>(p.y)[token * p.ldy + col] = __float2half_rn(v);
  else
    reinterpret_cast<__nv_bfloat16*>(p.y)[token * p.ldy + col] = __float2bfloat16_rn(v);
}

// Up to 128 tokens.  The 128 UMMA rows are weight rows (one 128-row scale block per tile), the BN columns
// are tokens.  Warps 0..3 promote, warp 4 is the TMA producer, warp 5 issues the MMAs and owns TMEM.
// grid = (tiles, split), cluster = (1, split, 1): CTA `rank` of a cluster takes the rank-th part of K.
template <int BN>
__global__ void __launch_bounds__((kNarrowEpiWarps + 2) * 32, (BN <= 32 ? 2 : 1))
    fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmParams p) {
  using S = GemmSmem<BN>;
  using SS = ScaleStage<BN>;
  constexpr int E = kNarrowEpiWarps;
  constexpr int kStages = S::kStages;
  // Accumulator ring in TMEM: as many BN-column buffers as fit (at most 8), so the MMA issuer can run
  // several K blocks ahead of the promotion.
  constexpr int kAcc = (512 / S::kCtasPerSm) / BN > 8 ? 8 : (512 / S::kCtasPerSm) / BN;
  constexpr uint32_t kTmemCols = kAcc * BN < 32 ? 32 : kAcc * BN;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  static_assert(BN % 16 == 0, "token tile must be a multiple of 16");
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
  float* sscale = reinterpret_cast<float*>(tmem_empty + 8);  // staged scale products of the current K chunk
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sscale + SS::kFloats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (p.k + kBlockK - 1) / kBlockK;
  const int tiles_w = (p.n + kTileR - 1) / kTileR;
  const int split = gridDim.y, rank = blockIdx.y, tile = blockIdx.x;
  const int tw = tile % tiles_w, tt = tile / tiles_w;  // weight-row tile, token tile
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
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
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
  // So can the weights (the caller promises that the kernel queued before this one does not write them):
  // the producer requests the weight half of its first stages before the launch-chain wait and adds the
  // activation half afterwards.
  uint32_t prefetched = 0;
  if (p.prefetch && warp == E && lane == 0) {
    const uint64_t stream_policy = l2_evict_first_policy();
    for (int kb = kb_first; kb < kb_last && prefetched < (uint32_t)kStages; ++kb, ++prefetched) {
      mbar_expect_tx(&full_bar[prefetched], S::kStageBytes);
      tma_load_2d_hint(stage_base + (size_t)prefetched * S::kStageBytes, &map_w, &full_bar[prefetched], kb * kBlockK,
                       tw * kTileR, stream_policy);
    }
  }
  chain_wait();
  chain_release();

  // Promotion state that outlives the role branch (the reduction below needs it).
  constexpr int kEpiThreads = E * 32;
  const int row_in_tile = (warp & 3) * 32 + lane;
  float acc[BN];

  if (warp == E) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const uint64_t stream_policy = l2_evict_first_policy();  // weights are streamed once per call
      uint32_t n = 0;
      for (int kb = kb_first; kb < kb_last; ++kb, ++n) {
        const int s = n % kStages;
        uint8_t* dst = stage_base + (size_t)s * S::kStageBytes;
        if (n < prefetched) {  // the weight half is already on its way
          tma_load_2d(dst + kTileR * kBlockK, &map_x, &full_bar[s], kb * kBlockK, tt * BN);
          continue;
        }
        if (!mbar_wait_bounded(&empty_bar[s], ((n / kStages) & 1u) ^ 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        mbar_expect_tx(&full_bar[s], S::kStageBytes);
        tma_load_2d_hint(dst, &map_w, &full_bar[s], kb * kBlockK, tw * kTileR, stream_policy);
        tma_load_2d(dst + kTileR * kBlockK, &map_x, &full_bar[s], kb * kBlockK, tt * BN);
      }
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
        const uint32_t a_addr = smem_u32(stage_base + (size_t)s * S::kStageBytes);
        const uint32_t b_addr = a_addr + kTileR * kBlockK;
        const uint64_t da = smem_desc_k128(a_addr), db = smem_desc_k128(b_addr);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          umma_f8(tmem_base + b * BN, da + (uint64_t)(k * kUmmaK / 16), db + (uint64_t)(k * kUmmaK / 16), idesc,
                  k > 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs have read it
        umma_commit(&tmem_full[b]);  // hands the K block's accumulator to the promotion warps
      }
    }
  } else {
    // ---------------- Promotion warps: add every K block with its scales ----------------
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const int epi_tid = threadIdx.x;  // promotion warps are warps 0..E-1
    uint32_t n = 0;
    bool ok = true;
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    for (int kb0 = kb_first; kb0 < kb_last && ok; kb0 += SS::kChunkKb) {
      const int kc = kb_last - kb0 < SS::kChunkKb ? kb_last - kb0 : SS::kChunkKb;
      // Stage this chunk's scale products a_scale[token] * w_scale (all loads in flight together).
      epi_bar_sync(kEpiThreads);  // the previous chunk's readers are done
      for (int i = epi_tid; i < kc * BN; i += kEpiThreads) {
        const int kk = i / BN, tok = tt * BN + i % BN;
        const float ws = p.w_scale[(long long)tw * p.w_scale_ld + kb0 + kk];
        sscale[i] = tok < p.m ? p.a_scale[(long long)(kb0 + kk) * p.a_scale_ld + tok] * ws : 0.f;
      }
      epi_bar_sync(kEpiThreads);
      for (int kk = 0; kk < kc; ++kk, ++n) {
        const int b = n % kAcc;
        const float* s_col = sscale + kk * BN;
        if (!mbar_wait_bounded(&tmem_full[b], (n / kAcc) & 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = lane_addr + (uint32_t)(b * BN);
        if constexpr (BN % 64 == 0) {
          // Two loads in flight per wait: halves the TMEM round trips per K block.
#pragma unroll
          for (int c = 0; c < BN; c += 64) {
            float d0[32], d1[32];
            tmem_ld32(taddr + c, d0);
            tmem_ld32(taddr + c + 32, d1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(d0[j], s_col[c + j], acc[c + j]);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c + 32 + j] = fmaf(d1[j], s_col[c + 32 + j], acc[c + 32 + j]);
          }
        } else if constexpr (BN % 32 == 0) {
          float d[32];
          tmem_ld32(taddr, d);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = fmaf(d[j], s_col[j], acc[j]);
        } else {
          float d[16];
          tmem_ld16(taddr, d);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = fmaf(d[j], s_col[j], acc[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[b]);
      }
    }
  }

  // ---------------- output: direct (split == 1) or reduced across the cluster ----------------
  const int w_row = tw * kTileR + row_in_tile;  // weight row = output column
  if (split == 1) {
    if (warp < E && w_row < p.n) {
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        const int tok = tt * BN + j;
        if (tok < p.m) store_out(p, tok, w_row, acc[j]);
      }
    }
  } else {
    // Every MMA of this CTA has completed (the promotion consumed the last accumulator), so the stage ring
    // is free.  Rank d owns the 8-token chunks [d * slice, (d + 1) * slice) of the tile: every CTA pushes
    // its partial of those tokens into slot [its own rank] of the owner's ring (remote shared-memory
    // stores), the cluster barrier publishes them, and the owner adds the slots in rank order.
    constexpr int kChunks = BN / 8;
    const int slice = (kChunks + split - 1) / split;            // chunks per owner
    const int slice_floats = slice * 8 * kTileR;                 // one slot
    const uint32_t red_addr = smem_u32(stage_base);
    cluster_sync_all();  // every CTA of the cluster is done with its own stage ring
    if (warp < E) {
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        const int owner = (j >> 3) / slice;
        const int local_col = j - owner * slice * 8;
        const uint32_t local = red_addr + (uint32_t)((rank * slice_floats + local_col * kTileR + row_in_tile) * 4);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)owner));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(acc[j]) : "memory");
      }
    }
    cluster_sync_all();
    if (warp < E) {
      const float* red = reinterpret_cast<const float*>(stage_base);
      const int chunk_lo = rank * slice, chunk_hi = (rank + 1) * slice < kChunks ? (rank + 1) * slice : kChunks;
      for (int ch = chunk_lo; ch < chunk_hi; ++ch) {
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
        for (int peer = 0; peer < split; ++peer) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            sum[j] += red[peer * slice_floats + ((ch - chunk_lo) * 8 + j) * kTileR + row_in_tile];
        }
        if (w_row < p.n) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int tok = tt * BN + ch * 8 + j;
            if (tok < p.m) store_out(p, tok, w_row, sum[j]);
          }
        }
      }
    }
    // No CTA reads a peer after the barrier above, so nothing more is needed before exit.
  }

  tc_fence_before();
  __syncthreads();
  if (warp == E + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------
// Wide kernel (more than 128 tokens): tokens are the 128 UMMA rows, 256 weight rows the columns.
//
//   * Schedule, grid = (CTAs, split).  With at least as many tiles as SMs the grid is persistent (split =
//     1, one CTA per SM): CTA c takes tiles c, c + P, c + 2P, ... whole and stores a finished tile while
//     the tensor core already works on the next one.  A shape with fewer tiles than SMs runs one tile per
//     2- or 4-CTA cluster, each CTA taking a slice of K: every CTA parks its fp32 partial in its own (then
//     idle) stage ring in a swizzled [row][4-column group] layout, and after a cluster barrier reads the
//     column slice it owns from every peer with 16-byte distributed-shared-memory loads, adds the partials
//     in rank order (a fixed order: results do not depend on timing) and stores bf16.  No global scratch.
//   * 12 warps: 8 promotion warps (two warpgroups), one TMA producer, one MMA issuer, two idle.  The
//     producer warpgroup hands most of its registers to the promotion warps (setmaxnreg), which keep the
//     128 x 256 fp32 result in registers (128 per thread) next to two 32-column landing buffers.
//   * Two 256-column accumulators ping-pong in TMEM.  Promotion of one K block: two rounds of two TMEM loads
//     in flight; the multiply-adds (packed fp32x2) of one landing buffer run while the other is being
//     refilled, and the first loads of the next K block are issued before the last columns of the current
//     one are consumed.  The accumulator goes back to the MMA issuer as soon as its last load has landed.
// --------------------------------------------------------------------------
constexpr int kWideBN = 256;
constexpr int kWideEpiWarps = 8;
constexpr int kWideThreads = 384;
constexpr int kWideStages = 4;
constexpr int kWideStageBytes = kTileR * kBlockK + kWideBN * kBlockK;  // 48 KiB
constexpr int kWideChunkKb = 16;                                        // K blocks of scales staged at a time
constexpr int kWideScaleFloats = kWideChunkKb * (kTileR + 2);
constexpr int kWideStoreBytes = kWideEpiWarps * 2048;  // per promotion warp: 32 rows x 32 columns of 16-bit output
constexpr int kWideSmemBytes = kWideStages * kWideStageBytes + kWideStoreBytes + (2 * kWideStages + 4) * 8 +
                               kWideScaleFloats * 4 + 64 + 1024;
static_assert(kWideStages * kWideStageBytes >= kTileR * kWideBN * 4, "stage ring too small for the fp32 partial tile");

struct WideItem {
  int tm, tn, k0, k1;
};

// Work of CTA (x, rank) of a (gridDim.x, split) grid over the tiles [first, tiles).  split == 1: tiles
// first + x, first + x + gridDim.x, ... whole.  split > 1 (one cluster per tile): tile first + x, the
// rank-th part of its K range.
__device__ __forceinline__ bool wide_item(int first, int tiles, int tiles_m, int kb_total, int split, int rank,
                                          int idx, WideItem& it) {
  const int tile = first + blockIdx.x + idx * gridDim.x;
  if (tile >= tiles || (split > 1 && idx > 0)) return false;
  it.tm = tile % tiles_m;
  it.tn = tile / tiles_m;
  it.k0 = (int)((long long)kb_total * rank / split);
  it.k1 = (int)((long long)kb_total * (rank + 1) / split);
  return true;
}

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

__device__ __forceinline__ void tmem_ld_wait_pin(float (&a)[32], float (&b)[32]) {
  // The wait is what makes the registers of the earlier tcgen05.ld valid; naming them as in/out operands
  // keeps every later use of a and b behind it.
  uint32_t* r = reinterpret_cast<uint32_t*>(a);
  uint32_t* q = reinterpret_cast<uint32_t*>(b);
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31]), "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]),
                 "+r"(q[5]), "+r"(q[6]), "+r"(q[7]), "+r"(q[8]), "+r"(q[9]), "+r"(q[10]), "+r"(q[11]),
                 "+r"(q[12]), "+r"(q[13]), "+r"(q[14]), "+r"(q[15]), "+r"(q[16]), "+r"(q[17]), "+r"(q[18]),
                 "+r"(q[19]), "+r"(q[20]), "+r"(q[21]), "+r"(q[22]), "+r"(q[23]), "+r"(q[24]), "+r"(q[25]),
                 "+r"(q[26]), "+r"(q[27]), "+r"(q[28]), "+r"(q[29]), "+r"(q[30]), "+r"(q[31])
               :
               : "memory");
}

// acc[0..32) += d[0..32) * s, two columns per instruction.
__device__ __forceinline__ void promote32(float* acc, const float (&d)[32], float s) {
  const float2 s2 = make_float2(s, s);
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const float2 r = __ffma2_rn(make_float2(d[j], d[j + 1]), s2, make_float2(acc[j], acc[j + 1]));
    acc[j] = r.x;
    acc[j + 1] = r.y;
  }
}

// Cluster reduction of a K-split tile: this CTA adds the 4-column groups [g_lo, g_lo + 64 / kSplit) of the
// tile over all ranks, in rank order, and stores them.  A thread owns 32 / kSplit (row, group) items and has
// the loads of all of them, from every rank, in flight together (one exposed round trip instead of many).
template <int kSplit>
__device__ __forceinline__ void wide_cluster_reduce(const GemmParams& p, uint32_t park_addr, int rank, int epi_tid,
                                                    int tok0, int col_base) {
  constexpr int kGroups = 64 / kSplit, kItems = kTileR * kGroups / (kWideEpiWarps * 32);
  const int g_lo = kGroups * rank;
  const bool vec = (p.ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 7) == 0);
  float4 part[kItems][kSplit];
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const int i = epi_tid + u * (kWideEpiWarps * 32);
    const int row = i / kGroups, g = g_lo + i % kGroups;
    const uint32_t slot = park_addr + (uint32_t)((row * 64 + (g ^ (row & 7))) * 16);
#pragma unroll
    for (int peer = 0; peer < kSplit; ++peer) part[u][peer] = ld_cluster_f4(slot, (uint32_t)peer);
  }
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const int i = epi_tid + u * (kWideEpiWarps * 32);
    const int row = i / kGroups, g = g_lo + i % kGroups;
    float4 sum = part[u][0];
#pragma unroll
    for (int peer = 1; peer < kSplit; ++peer) {
      sum.x += part[u][peer].x;
      sum.y += part[u][peer].y;
      sum.z += part[u][peer].z;
      sum.w += part[u][peer].w;
    }
    const int tok = tok0 + row, n0 = col_base + g * 4;
    if (tok < p.m && n0 < p.n) {
      uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + (long long)tok * p.ldy + n0;
      if (vec && n0 + 4 <= p.n) {
        uint2 w;
        w.x = p.out_f16 ? Mma16816<__half>::pack(sum.x, sum.y) : Mma16816<__nv_bfloat16>::pack(sum.x, sum.y);
        w.y = p.out_f16 ? Mma16816<__half>::pack(sum.z, sum.w) : Mma16816<__nv_bfloat16>::pack(sum.z, sum.w);
        *reinterpret_cast<uint2*>(dst) = w;
      } else {
        const float v[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (n0 + j < p.n) {
            if (p.out_f16)
              reinterpret_cast<__half*>(dst)[j] = __float2half_rn(v[j]);
            else
              reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16_rn(v[j]);
          }
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kWideThreads, 1)
    fp8_gemm_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const GemmParams p) {
  constexpr int BN = kWideBN, E = kWideEpiWarps, kStages = kWideStages, kAcc = 2;
  constexpr int kCols = BN / 2;  // columns owned by one promotion warp
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* store_base = smem + kStages * kWideStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(store_base + kWideStoreBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + kAcc;
  float* sscale = reinterpret_cast<float*>(tmem_empty + kAcc);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sscale + kWideScaleFloats);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (p.k + kBlockK - 1) / kBlockK;
  const int tiles_m = (p.m + kTileR - 1) / kTileR;
  const int tiles = p.tile_end;
  const int split = gridDim.y, rank = blockIdx.y;  // cluster = (1, split, 1)

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
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_w);
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
  // So can the weights (nothing on the stream writes them): the producer requests the weight half of its
  // first stages before the launch-chain wait and adds the activation half afterwards.
  uint32_t prefetched = 0;
  if (p.prefetch && warp == E && lane == 0) {
    WideItem first;
    if (wide_item(p.tile_begin, tiles, tiles_m, kb_total, split, rank, 0, first)) {
      for (int kb = first.k0; kb < first.k1 && prefetched < (uint32_t)kStages; ++kb, ++prefetched) {
        mbar_expect_tx(&full_bar[prefetched], kWideStageBytes);
        tma_load_2d(stage_base + (size_t)prefetched * kWideStageBytes + kTileR * kBlockK, &map_w,
                    &full_bar[prefetched], kb * kBlockK, first.tn * BN);
      }
    }
  }
  if (!p.late_wait) chain_wait();
  chain_release();

  // K blocks this CTA will process (the promotion pipeline needs to know when the last one is reached).
  uint32_t total_blocks = 0;
  {
    WideItem it;
    for (int idx = 0; wide_item(p.tile_begin, tiles, tiles_m, kb_total, split, rank, idx, it); ++idx) total_blocks += (uint32_t)(it.k1 - it.k0);
  }

  if (warp >= E) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == E && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t n = 0;
      bool ok = true;
      WideItem it;
      for (int idx = 0; ok && wide_item(p.tile_begin, tiles, tiles_m, kb_total, split, rank, idx, it); ++idx) {
        for (int kb = it.k0; kb < it.k1; ++kb, ++n) {
          const int s = n % kStages;
          uint8_t* dst = stage_base + (size_t)s * kWideStageBytes;
          if (n < prefetched) {  // the weight half is already on its way
            tma_load_2d(dst, &map_x, &full_bar[s], kb * kBlockK, it.tm * kTileR);
            continue;
          }
          if (!mbar_wait_bounded(&empty_bar[s], ((n / kStages) & 1u) ^ 1u)) {
            raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], kWideStageBytes);
          tma_load_2d(dst, &map_x, &full_bar[s], kb * kBlockK, it.tm * kTileR);
          tma_load_2d(dst + kTileR * kBlockK, &map_w, &full_bar[s], kb * kBlockK, it.tn * BN);
        }
      }
    } else if (warp == E + 1 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = instr_desc_f8(BN);
      for (uint32_t n = 0; n < total_blocks; ++n) {
        const int s = n % kStages, b = n % kAcc;
        if (!mbar_wait_bounded(&full_bar[s], (n / kStages) & 1u) ||
            !mbar_wait_bounded(&tmem_empty[b], ((n / kAcc) & 1u) ^ 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(stage_base + (size_t)s * kWideStageBytes);
        const uint64_t da = smem_desc_k128(a_addr), db = smem_desc_k128(a_addr + kTileR * kBlockK);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          umma_f8(tmem_base + b * BN, da + (uint64_t)(k * kUmmaK / 16), db + (uint64_t)(k * kUmmaK / 16), idesc,
                  k > 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs have read it
        umma_commit(&tmem_full[b]);  // hands the K block's accumulator to the promotion warps
      }
    }
    __syncwarp();
    if (split > 1) {
      cluster_sync_all();  // partials parked
      cluster_sync_all();  // peers have read this CTA's partial
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---------------- Promotion warps ----------------
    constexpr int kEpiThreads = E * 32;
    const int quad = warp & 3, half = warp >> 2;
    const int row_in_tile = quad * 32 + lane;
    const int col0 = half * kCols;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col0;
    const int epi_tid = threadIdx.x;
    float acc[kCols];
    float buf_a[32], buf_b[32];
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
    uint32_t n = 0;
    bool ok = true;
    // First accumulator: its first 64 columns start the pipeline.
    if (total_blocks > 0) {
      ok = mbar_wait_bounded(&tmem_full[0], 0);
      if (!ok) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      tc_fence_after();
      if (ok) {
        tmem_ld32(lane_addr, buf_a);
        tmem_ld32(lane_addr + 32, buf_b);
      }
    }
    WideItem it;
    for (int idx = 0; ok && wide_item(p.tile_begin, tiles, tiles_m, kb_total, split, rank, idx, it); ++idx) {
      const int tok0 = it.tm * kTileR;
      for (int kb0 = it.k0; kb0 < it.k1 && ok; kb0 += kWideChunkKb) {
        const int kc = it.k1 - kb0 < kWideChunkKb ? it.k1 - kb0 : kWideChunkKb;
        // Stage this chunk's scales (all loads in flight together).
        epi_bar_sync(kEpiThreads);  // the previous chunk's readers are done
        float* s_w = sscale + kWideChunkKb * kTileR;
        for (int i = epi_tid; i < kc * kTileR; i += kEpiThreads) {
          const int kk = i / kTileR, tok = tok0 + i % kTileR;
          sscale[i] = tok < p.m ? p.a_scale[(long long)(kb0 + kk) * p.a_scale_ld + tok] : 0.f;
        }
        for (int i = epi_tid; i < kc * 2; i += kEpiThreads) {
          const int kk = i >> 1, blk = it.tn * 2 + (i & 1);
          s_w[i] = blk * 128 < p.n ? p.w_scale[(long long)blk * p.w_scale_ld + kb0 + kk] : 0.f;
        }
        epi_bar_sync(kEpiThreads);
        for (int kk = 0; kk < kc; ++kk, ++n) {
          const int b = n & 1;
          const float s = sscale[kk * kTileR + row_in_tile] * s_w[kk * 2 + half];
          const uint32_t taddr = lane_addr + (uint32_t)(b * BN);
          tmem_ld_wait_pin(buf_a, buf_b);  // columns 0..63 have landed
          promote32(acc, buf_a, s);
          tmem_ld32(taddr + 64, buf_a);
          promote32(acc + 32, buf_b, s);
          tmem_ld32(taddr + 96, buf_b);
          tmem_ld_wait_pin(buf_a, buf_b);  // columns 64..127 have landed
          // Every load of this accumulator has landed: hand the buffer back to the MMA issuer.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[b]);
          promote32(acc + 64, buf_a, s);
          const bool more = n + 1 < total_blocks;
          if (more) {
            if (!mbar_wait_bounded(&tmem_full[b ^ 1], ((n + 1) >> 1) & 1u)) {
              raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
              ok = false;
            }
            tc_fence_after();
            if (ok) tmem_ld32(lane_addr + (uint32_t)((b ^ 1) * BN), buf_a);
          }
          promote32(acc + 96, buf_b, s);
          if (more && ok) tmem_ld32(lane_addr + (uint32_t)((b ^ 1) * BN) + 32, buf_b);
          if (!ok) break;
        }
      }
      if (!ok) break;

      const int r_glob = tok0 + row_in_tile;
      if (split == 1) {
        const int n0 = it.tn * BN + col0;
        const bool vec = (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) && (n0 + kCols <= p.n);
        if (vec) {
          // Rows leave through a per-warp staging area so that global stores are whole 64-byte row
          // segments: a lane parks 32 columns of its own row (4 x 16 bytes, unit u of row r at
          // r * 4 + ((u + r / 2) & 3): conflict-free both ways), then four lanes store one row segment.
          uint4* stage = reinterpret_cast<uint4*>(store_base + warp * 2048);
          const int out_row = lane >> 2, unit = lane & 3;
#pragma unroll
          for (int c = 0; c < kCols; c += 32) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j = c + u * 8 + 2 * q;
                w[q] = p.out_f16 ? Mma16816<__half>::pack(acc[j], acc[j + 1])
                                 : Mma16816<__nv_bfloat16>::pack(acc[j], acc[j + 1]);
              }
              stage[lane * 4 + ((u + (lane >> 1)) & 3)] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            __syncwarp();
#pragma unroll
            for (int r8 = 0; r8 < 32; r8 += 8) {
              const int r = r8 + out_row;
              const uint4 v = stage[r * 4 + ((unit + (r >> 1)) & 3)];
              const int tok = tok0 + quad * 32 + r;
              if (tok < p.m) {
                uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + (long long)tok * p.ldy + n0 + c + unit * 8;
                *reinterpret_cast<uint4*>(dst) = v;
              }
            }
            __syncwarp();
          }
        } else if (r_glob < p.m) {
          uint16_t* yrow = reinterpret_cast<uint16_t*>(p.y) + (long long)r_glob * p.ldy + n0;
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
      } else {
        // Park the partial: float4 (row, g) lives at slot row * 64 + (g ^ (row & 7)), so that both the
        // row-per-lane writes here and the column-group-per-lane reads below are free of bank conflicts.
        // Every MMA of this CTA has completed (its last accumulator was consumed), so the ring is idle.
        float4* park = reinterpret_cast<float4*>(stage_base);
#pragma unroll
        for (int j = 0; j < kCols; j += 4) {
          const int g = (col0 + j) >> 2;
          park[row_in_tile * 64 + (g ^ (row_in_tile & 7))] = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        }
        cluster_sync_all();
        if (split == 2)
          wide_cluster_reduce<2>(p, smem_u32(stage_base), rank, epi_tid, tok0, it.tn * BN);
        else
          wide_cluster_reduce<4>(p, smem_u32(stage_base), rank, epi_tid, tok0, it.tn * BN);
        cluster_sync_all();  // no CTA leaves while a peer may still read its partial
      }
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
    }
    if (!ok) {
      tmem_ld_wait();  // nothing of this thread stays in flight
      if (split > 1) {  // a CTA that gave up still meets its peers at the two cluster barriers
        cluster_sync_all();
        cluster_sync_all();
      }
    }
  }

  // Second launch of a two-launch GEMM: it ran beside the first one, and must not complete before it
  // (the kernel queued behind only waits for this one).
  if (p.late_wait) chain_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == E + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
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
// (which grows with the tile width).  Cluster sizes 1, 2 and 4 are used, and 8 for the narrow tiles that
// run two 100 KB CTAs per SM (o / down at up to 32 tokens: 160 CTAs instead of 80); 3 and 8 co-schedule
// badly with one 200 KB CTA per SM (measured), and larger splits leave too little work per CTA.
int choose_split(long long tiles, int kb_total, int bn, int ctas_per_sm, int max_split) {
  const int slots = sm_count() * ctas_per_sm;
  int best = 1;
  double best_cost = 1e30;
  const int limit = ctas_per_sm == 2 ? 8 : 4;
  for (int s = 1; s <= limit; s *= 2) {
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

template <int BN>
int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, long long tiles, int split,
                cudaStream_t stream) {
  using S = GemmSmem<BN>;
  constexpr int E = kNarrowEpiWarps;
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(fp8_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
  MIE_CUDA(cudaLaunchKernelEx(&config, fp8_gemm_kernel<BN>, mw, mx, p));
  MIE_LAUNCH_CHECK("fp8_gemm_kernel");
  return MIE_OK;
}

// Column-tile width for the swapped orientation: smallest of 16/32/64/128 covering m.
int swap_bn(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

// Schedule of the wide kernel.  `tiles` output tiles of `kb` K blocks on P SMs (one 200 KB CTA each):
//   tiles <= P      one launch; whole tiles, or one tile per 2-/4-CTA cluster with the K range cut when all
//                   clusters still fit one wave;
//   tiles > P       the whole waves (floor(tiles / P) * P tiles) run as one persistent launch; the
//                   remaining R tiles would otherwise cost a full extra round on R of the P SMs, so when
//                   R * s <= P they go to a second launch of one s-CTA cluster per tile (s = 2 or 4) that
//                   starts on the SMs the first launch frees and finishes in 1 / s of a round.
// Costs in units of one K block of the main loop; the cluster reduction and the fill / drain of a CTA are
// worth a few blocks each.
struct WidePlan {
  int main_tiles;  // tiles of the persistent launch (0: none)
  int main_split;  // K split of the main launch (> 1 only when it is the only launch)
  int tail_split;  // K split of the tail launch (0: no tail launch)
};

WidePlan plan_wide(long long tiles, int kb, int max_split) {
  const int slots = sm_count();
  WidePlan plan{(int)tiles, 1, 0};
  if (tiles <= slots) {
    double best_cost = 1e30;
    for (int s = 1; s <= 4; s *= 2) {
      if (s > kb || (max_split > 0 && s > max_split)) break;
      if (s > 1 && tiles * s > slots) break;  // clusters only when all of them run in one wave
      const double cost = (double)((kb + s - 1) / s) + 4.0 + (s > 1 ? 3.0 : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        plan.main_split = s;
      }
    }
    return plan;
  }
  const long long rest = tiles % slots;
  if (rest == 0) return plan;
  double best_cost = (double)kb;  // the tail as one more whole round of the persistent launch
  for (int s = 2; s <= 4; s *= 2) {
    if (s > kb || (max_split > 0 && s > max_split) || rest * s > slots) break;
    const double cost = (double)((kb + s - 1) / s) + 3.0 + 2.0;  // reduction + the second launch's start-up
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      plan.main_tiles = (int)(tiles - rest);
      plan.tail_split = s;
    }
  }
  return plan;
}

int launch_wide_range(const CUtensorMap& mx, const CUtensorMap& mw, GemmParams p, int tile_begin, int tile_end,
                      int split, bool late_wait, cudaStream_t stream) {
  p.tile_begin = tile_begin;
  p.tile_end = tile_end;
  p.late_wait = late_wait ? 1 : 0;
  const int count = tile_end - tile_begin;
  const int ctas = split > 1 ? count : (count < sm_count() ? count : sm_count());
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)ctas, (unsigned)split, 1);
  config.blockDim = dim3(kWideThreads, 1, 1);
  config.dynamicSmemBytes = kWideSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)split;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = chained_launch_enabled() ? 2 : 1;
  MIE_CUDA(cudaLaunchKernelEx(&config, fp8_gemm_wide_kernel, mx, mw, p));
  MIE_LAUNCH_CHECK("fp8_gemm_wide_kernel");
  return MIE_OK;
}

int launch_wide(const CUtensorMap& mx, const CUtensorMap& mw, const GemmParams& p, int max_split,
                cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(fp8_gemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kWideSmemBytes));
    configured[dev] = true;
  }
  const int kb = (p.k + kBlockK - 1) / kBlockK;
  const long long tiles = (long long)((p.m + kTileR - 1) / kTileR) * ((p.n + kWideBN - 1) / kWideBN);
  MIE_CHECK_ARG(tiles <= 0x7fffffff, "too many output tiles (%lld)", tiles);
  const WidePlan plan = plan_wide(tiles, kb, max_split);
  if (int rc = launch_wide_range(mx, mw, p, 0, plan.main_tiles, plan.main_split, false, stream)) return rc;
  if (plan.tail_split > 0) {
    // Only with launch chaining on does the tail start before the main launch has drained; without it the
    // stream simply runs the two launches one after the other.
    return launch_wide_range(mx, mw, p, plan.main_tiles, (int)tiles, plan.tail_split, chained_launch_enabled(),
                             stream);
  }
  return MIE_OK;
}

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
                            int32_t out_dtype, int32_t m, int32_t n, int32_t k, int32_t max_split, int32_t flags,
                            int32_t* status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MIE_CHECK_ARG(x8 && a_scale && w8 && w_scale && y, "null pointer");
  MIE_CHECK_ARG(m >= 0 && n >= 1 && k >= 1, "invalid GEMM shape %d x %d x %d", m, n, k);
  MIE_CHECK_ARG(out_dtype == MIE_DTYPE_BF16 || out_dtype == MIE_DTYPE_F16, "output must be bf16 or fp16");
  MIE_CHECK_ARG(ldx % 16 == 0 && ldw % 16 == 0, "operand row strides must be multiples of 16 bytes");
  MIE_CHECK_ARG(((reinterpret_cast<uintptr_t>(x8) | reinterpret_cast<uintptr_t>(w8)) & 15) == 0,
                "operands must be 16-byte aligned");
  MIE_CHECK_ARG(ldy >= n && a_scale_ld >= m && w_scale_ld >= (k + 127) / 128, "invalid leading dimension");
  MIE_CHECK_ARG((flags & ~(MIE_GEMM_NO_WEIGHT_PREFETCH)) == 0, "unknown flag bits %d", flags);
  if (m == 0) return MIE_OK;

  // Up to 128 tokens stream the weights through the narrow kernel, unless that needs a second wave of
  // full-K tiles (more 128-row weight tiles than SMs at more than 32 tokens, where only one of its CTAs
  // fits an SM: gate_up): the wide kernel's 256-row tiles then finish in one round.  Between 129 and 256
  // tokens a weight of at most 12 row tiles (N <= 1536: the merged qkv of a 4- or 8-way head shard) is
  // still faster there, as two token tiles (measured 9.7 vs 12.6 us at N = 768, 10.8 vs 13.1 at N = 1536;
  // at N = 2560 the wide kernel wins).
  const int tiles_w = (n + kTileR - 1) / kTileR;
  const bool narrow = (m <= 128 && !(m > 32 && tiles_w > sm_count())) || (m <= 256 && tiles_w <= 12);
  const int kb = (k + kBlockK - 1) / kBlockK;

  GemmParams p;
  p.m = m;
  p.n = n;
  p.k = k;
  p.a_scale = a_scale;
  p.a_scale_ld = a_scale_ld;
  p.w_scale = w_scale;
  p.w_scale_ld = w_scale_ld;
  p.y = y;
  p.ldy = ldy;
  p.out_f16 = out_dtype == MIE_DTYPE_F16;
  p.status = status;
  static const int prefetch = [] {
    const char* v = getenv("MIE_GEMM_PREFETCH");
    return v != nullptr && v[0] == '0' ? 0 : 1;  // MIE_GEMM_PREFETCH=0 turns it off
  }();
  p.prefetch = prefetch && !(flags & MIE_GEMM_NO_WEIGHT_PREFETCH);
  p.tile_begin = p.tile_end = p.late_wait = 0;

  CUtensorMap mw, mx;
  if (narrow) {
    const int bn = swap_bn(m);
    const long long tiles = (long long)((n + kTileR - 1) / kTileR) * ((m + bn - 1) / bn);
    MIE_CHECK_ARG(tiles <= 0x7fffffff, "too many output tiles (%lld)", tiles);
    const int split = choose_split(tiles, kb, bn, bn <= 32 ? 2 : 1, max_split);
    if (int rc = operand_map(w8, n, k, ldw, kTileR, &mw)) return rc;
    if (int rc = operand_map(x8, m, k, ldx, bn, &mx)) return rc;
    switch (bn) {
      case 16: return launch_gemm<16>(mw, mx, p, tiles, split, stream);
      case 32: return launch_gemm<32>(mw, mx, p, tiles, split, stream);
      case 64: return launch_gemm<64>(mw, mx, p, tiles, split, stream);
      default: return launch_gemm<128>(mw, mx, p, tiles, split, stream);
    }
  }
  if (int rc = operand_map(x8, m, k, ldx, kTileR, &mx)) return rc;
  if (int rc = operand_map(w8, n, k, ldw, kWideBN, &mw)) return rc;
  return launch_wide(mx, mw, p, max_split, stream);
}
