// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA = one 128-row query tile: 128 / G consecutive query tokens of one request times the G query
// heads that share one KV head, so a K/V tile staged once serves the whole GQA group.  Per 128-token K/V
// tile:
//   S = Q K^T      UMMA 128x128x16 (bf16/fp16, fp32 accumulate) into one of two TMEM buffers;
//   softmax        256 threads, two per query row, read their half of the S row from TMEM, apply the causal /
//                  length mask and an exp2 softmax against a running reference maximum, and write
//                  P (16-bit, two per column) back into TMEM over the S buffer they just read;
//   O += P V       UMMA 128x128x16 with P as the TMEM A operand and V as the MN-major shared-memory B
//                  operand, accumulated in TMEM over all tiles.
// The reference maximum is only moved when a row's maximum grows by more than 2^8 (then that warp
// rescales its O rows in TMEM), so O is read from TMEM once, at the end.
// Warp roles: 8 softmax warps (two threads per query row), 1 TMA producer (K/V pages gathered through the block table, one 4 KiB
// box per 16-token page slab, 128-byte swizzle, no multicast), 1 MMA issuer that also owns
// the TMEM allocation.  Every wait is bounded and reports MIE_STATUS_WAIT_TIMEOUT.
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "umma.cuh"

namespace mie {


namespace {

constexpr int kDim = 128;
constexpr int kRows = 128;                       // query rows per CTA (tokens x group heads)
constexpr int kKv = 128;                         // K/V tokens per tile
constexpr int kSub = 16;                         // tokens per TMA box
constexpr int kBoxBytes = kSub * kDim * 2;       // 4 KiB: one box = 16 tokens x 128 dims
constexpr int kTile = kKv * kDim * 2;            // 32 KiB: one K or V tile
// Shared-memory layout of a K/V tile (what the 5-D box below writes, 128-byte swizzled):
//   [token / 8 (16 groups)][dim / 64 (2 halves)][token % 8][64 dims = 128 bytes]
// so for either operand role an 8-token group is 2048 bytes from the next and the two 64-dim halves of a
// group are 1024 bytes apart.
constexpr int kGroupStride = 2048;
constexpr int kHalfStride = 1024;
constexpr int kKvStages = 3;                     // K and V each have their own ring of this depth
constexpr int kSoftmaxWarps = 8;                 // two threads per query row: each owns 64 of the 128 keys / dims
constexpr int kHalf = 64;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr float kRescaleThreshold = 8.0f;        // log2 units

// Shared-memory map (1024-byte aligned): K[3] | V[3] | barriers.
constexpr int kOffK = 0;
constexpr int kOffV = kOffK + kKvStages * kTile;
constexpr int kOffBar = kOffV + kKvStages * kTile;
constexpr int kOffXchg = kOffBar + 256;          // [tile parity][key half][row] floats: the row pairs' exchange
constexpr int kOffIds = kOffXchg + 2 * 2 * kRows * 4;  // page id of every 16-token box of the request
constexpr int kMaxIds = 4096;                          // 64k tokens of context
constexpr int kSmemBytes = kOffIds + kMaxIds * 4 + 1024;

struct UmmaPrefillParams {
  const char* query;
  long long q_st, q_sh;
  char* out;
  long long o_st, o_sh;
  IndexView tables, cu_seqlens, kv_lens;
  int requests, q_heads, kv_heads, group, block_size, num_blocks, table_width;
  float scale_log2;
  int* status;
};

enum Bar { kQFull = 0, kKFull = 1, kKEmpty = 4, kVFull = 7, kVEmpty = 10, kSFull = 13, kPFull = 15, kPvDone = 17,
           kVClean = 19, kNumBars = 20 };

// 2^x on the special-function unit; -inf gives +0.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_umma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                        const UmmaPrefillParams p, const int q_tiles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int r = blockIdx.y, kvh = blockIdx.z;
  const int qt = q_tiles - 1 - (int)blockIdx.x;  // latest (heaviest) query tiles first
  const int tok_per_tile = kRows / p.group;
  const long long q_begin = p.cu_seqlens.at(r), q_end = p.cu_seqlens.at(r + 1);
  const int q_len = (int)(q_end - q_begin);
  const long long kv_len = p.kv_lens.at(r);
  const int i0 = qt * tok_per_tile;
  if (i0 >= q_len) return;
  if (kv_len < q_len || kv_len > (long long)p.table_width * p.block_size) {
    if (threadIdx.x == 0) raise_status(p.status, MIE_STATUS_BAD_LENGTH);
    return;
  }
  const long long offset = kv_len - q_len;  // position of query token 0
  const int toks = q_len - i0 < tok_per_tile ? q_len - i0 : tok_per_tile;
  const long long last_key = offset + i0 + toks - 1;
  const int n_tiles = (int)(last_key / kKv) + 1;

  if (threadIdx.x == 0) {
    mbar_init(&bars[kQFull], kSoftmaxWarps * 32);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&bars[kKFull + s], 1);
      mbar_init(&bars[kKEmpty + s], 1);
      mbar_init(&bars[kVFull + s], 1);
      mbar_init(&bars[kVEmpty + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars[kSFull + b], 1);
      mbar_init(&bars[kPFull + b], kSoftmaxWarps * 32);
      mbar_init(&bars[kPvDone + b], 1);
    }
    mbar_init(&bars[kVClean], 1);
    mbar_fence_init();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  if (warp == kSoftmaxWarps + 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  {
    // All threads fetch the block-table entries of the boxes this CTA will read (independent loads, all
    // in flight together), so the producer never waits on a dependent global load between TMA issues.
    int* ids = reinterpret_cast<int*>(smem + kOffIds);
    const int n_ids = n_tiles * (kKv / kSub) < kMaxIds ? n_tiles * (kKv / kSub) : kMaxIds;
    for (int i = threadIdx.x; i < n_ids; i += kThreads) {
      const long long tok = (long long)i * kSub;
      long long pid = 0;
      if (tok <= last_key) {
        pid = p.tables.at(r, tok / p.block_size);
        if (pid < 0 || pid >= p.num_blocks) {
          raise_status(p.status, MIE_STATUS_BAD_PAGE);
          pid = 0;
        }
      }
      ids[i] = (int)pid;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;            // two S buffers: columns [0,128) and [128,256); P(j) is
                                                // written over the first 64 columns of S(j)
  const uint32_t tmem_o = tmem_base + 256;      // O: columns [256,384)
  const uint32_t tmem_q = tmem_base + 384;      // Q (16-bit, two per column): columns [384,448)

  if (warp == kSoftmaxWarps) {
    // ---------------- TMA producer (+ V tail sanitiser) ----------------
    const uint64_t policy = l2_evict_first_policy();
    // One 128-token K or V tile = eight 16-token boxes per 64-dim half.  Lanes 0..7 each own one box row,
    // so the eight block-table lookups (dependent global loads) run in parallel.
    const int* page_ids = reinterpret_cast<const int*>(smem + kOffIds);
    auto load_tile = [&](const CUtensorMap* map, int off_base, int full0, int empty0, int j) -> bool {
      const int s = j % kKvStages;
      int pid = 0, tok_in_page = 0;
      if (lane < kKv / kSub) {
        const long long tok = (long long)j * kKv + lane * kSub;
        pid = page_ids[j * (kKv / kSub) + lane];
        if (tok <= last_key) tok_in_page = (int)(tok % p.block_size);
      }
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait_bounded(&bars[empty0 + s], ((j / kKvStages) & 1u) ^ 1u);
        if (ok)
          mbar_expect_tx(&bars[full0 + s], kTile);
        else
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && lane < kKv / kSub) {
        // One 4 KiB box per lane.  Boxes past the last needed key still land (page 0) so a stage always receives the same byte
        // count; their scores are masked and their V rows are zeroed below.
        uint8_t* dst = smem + off_base + s * kTile + lane * kBoxBytes;
        tma_load_5d_hint(dst, map, &bars[full0 + s], 0, 0, 0, kvh * (p.block_size / 8) + tok_in_page / 8, (int)pid,
                         policy);
      }
      __syncwarp();
      return ok;
    };
    // Issue order K(0), K(1), V(0), K(2), V(1), ... follows the order in which the MMA warp consumes and
    // frees the stages (S(j+1) is issued before P(j) V(j)).
    bool ok = load_tile(&kmap, kOffK, kKFull, kKEmpty, 0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) ok = load_tile(&kmap, kOffK, kKFull, kKEmpty, j + 1);
      if (ok) ok = load_tile(&vmap, kOffV, kVFull, kVEmpty, j);
    }
    if (ok) {
      // Slots past the request's length may hold anything (even NaN bits): zero those V rows of the last
      // tile so that a zero probability times V stays zero, then tell the MMA warp the stage is clean.
      const int j = n_tiles - 1, s = j % kKvStages;
      const bool landed = mbar_wait_bounded(&bars[kVFull + s], (j / kKvStages) & 1u);
      if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      } else {
        const long long first_bad = kv_len - (long long)j * kKv;  // rows >= first_bad are past the length
        uint8_t* vdst = smem + kOffV + s * kTile;
        for (int c = lane; c < kKv * 16; c += 32) {
          const int row = c >> 4, chunk = c & 15;
          if (row >= first_bad)
            *reinterpret_cast<uint4*>(vdst + (row >> 3) * kGroupStride + (chunk >> 3) * kHalfStride + (row & 7) * 128 +
                                      (chunk & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[kVClean]);
      }
    }
  } else if (warp == kSoftmaxWarps + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(kKv, kFmt, 0);   // S = Q K^T : A = Q in TMEM, B = K, K-major
      constexpr uint32_t idesc_o = instr_desc_f16(kDim, kFmt, 1);  // O += P V : A = P in TMEM, B = V, MN-major
      bool ok = mbar_wait_bounded(&bars[kQFull], 0);
      // S(j) overwrites the TMEM buffer that held S(j-2) / P(j-2); P(j-2) V(j-2) was issued earlier by this
      // thread and tcgen05.mma executes in issue order, so no barrier is needed for the reuse.
      auto issue_s = [&](int j) {
        const int s = j % kKvStages, b = j & 1;
        if (!mbar_wait_bounded(&bars[kKFull + s], (j / kKvStages) & 1u)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kOffK + s * kTile);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 8 x 16 dims
          const uint32_t off = (ks >> 2) * kHalfStride + (ks & 3) * 32;
          umma_f16_ts(tmem_s + b * kKv, tmem_q + ks * 8, smem_desc_k128(k_addr + off, kGroupStride), idesc_s,
                      ks > 0 ? 1u : 0u);
        }
        umma_commit(&bars[kKEmpty + s]);  // K stage free once these MMAs have read it
        umma_commit(&bars[kSFull + b]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kKvStages, b = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait_bounded(&bars[kPFull + b], (j >> 1) & 1u) ||
            !mbar_wait_bounded(&bars[kVFull + s], (j / kKvStages) & 1u) ||
            (j == n_tiles - 1 && !mbar_wait_bounded(&bars[kVClean], 0))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + kOffV + s * kTile);
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {  // 8 x 16 tokens = 8 TMEM columns of packed P each
          const uint64_t db = smem_desc_mn128(v_addr + kt * kBoxBytes, kHalfStride, kGroupStride);
          umma_f16_ts(tmem_o, tmem_s + b * kKv + kt * 8, db, idesc_o, (j > 0 || kt > 0) ? 1u : 0u);
        }
        umma_commit(&bars[kVEmpty + s]);  // V stage free once these MMAs have read it
        umma_commit(&bars[kPvDone + b]);  // O includes tile j
      }
      if (!ok) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
    }
  } else {
    // ---------------- Softmax warps: two threads per query row ----------------
    // Warps w and w + 4 share TMEM lane quadrant w % 4 (the same 32 rows); the first takes keys / output
    // dims [0, 64), the second [64, 128).  The pair meets on a named barrier once per tile to combine the
    // row maximum.  A failed wait only clears `ok` (later waits are skipped) so that both threads of a pair
    // always pass the same number of pair barriers.
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;                       // TMEM lane = row of the tile
    const int cbase = half * kHalf;
    const int tok_local = row / p.group, head_local = row % p.group;
    const bool row_live = tok_local < toks;
    const long long pos = row_live ? offset + i0 + tok_local : last_key;  // dead rows compute harmlessly
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float* xchg = reinterpret_cast<float*>(smem + kOffXchg);
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
    {
      // Stage this thread's half of the query row (64 16-bit values = 32 words) in TMEM, where it stays as
      // the A operand of every S = Q K^T; rows past the chunk are zero.
      const uint4* qrow = reinterpret_cast<const uint4*>(
          reinterpret_cast<const T*>(p.query) + (q_begin + i0 + (row_live ? tok_local : 0)) * p.q_st +
          (long long)(kvh * p.group + head_local) * p.q_sh + cbase);
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 v = row_live ? __ldg(qrow + i) : make_uint4(0, 0, 0, 0);
        w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
      }
      tmem_st32(tmem_q + lane_addr + half * 32, w);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[kQFull]);
    }
    // m_ref lives in the scaled log2 domain (score * scale * log2 e); scale > 0 is checked on the host, so
    // the row maximum can be taken over the raw scores.
    const float scale = p.scale_log2;
    const long long first_pos = offset + i0;  // smallest query position of the tile
    float m_ref = -INFINITY, l = 0.f;         // l: this thread's half of the row sum
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      if (ok && !mbar_wait_bounded(&bars[kSFull + b], (j >> 1) & 1u)) ok = false;
      tc_fence_after();
      float sv[kHalf];
#pragma unroll
      for (int c = 0; c < kHalf; c += 32)
        tmem_ld32(tmem_s + lane_addr + b * kKv + cbase + c, *reinterpret_cast<float(*)[32]>(&sv[c]));
      tmem_ld_wait();
      const long long key0 = (long long)j * kKv;
      if (key0 + kKv - 1 > first_pos) {
        // Only tiles that reach the causal diagonal (or the end of the request) carry masked keys.
        const long long d = pos - key0 - cbase;
        const int lim = d < kHalf - 1 ? (int)(d < -1 ? -1 : d) : kHalf - 1;  // keys [0, lim] of this half are visible
#pragma unroll
        for (int c = 0; c < kHalf; ++c)
          if (c > lim) sv[c] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kHalf; c += 8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], fmaxf(sv[c + 2 * q], sv[c + 2 * q + 1]));
      }
      const float mx_half = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Both halves have read their S columns before either writes P over them (the barrier below).
      xchg[(b * 2 + half) * kRows + row] = mx_half;
      pair_sync();
      const float mx = fmaxf(mx_half, xchg[(b * 2 + (half ^ 1)) * kRows + row]) * scale;
      // Move the reference maximum only on the first tile or when this row outgrew it by 2^8 (both threads
      // of the row see the same mx and decide alike).
      float alpha = 1.f;
      const bool grow = mx > m_ref + kRescaleThreshold || j == 0;
      if (grow) {
        const float m_new = fmaxf(m_ref, mx);
        alpha = ex2_approx(m_ref - m_new);  // 0 on the first tile
        m_ref = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // Rescale this warp's 32 rows x 64 dims of O in TMEM (rows that did not grow use alpha = 1); O must
        // first hold every tile before this one.
        if (ok && !mbar_wait_bounded(&bars[kPvDone + ((j - 1) & 1)], ((j - 1) >> 1) & 1u)) ok = false;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < kHalf; c += 32) {
          float ov[32];
          tmem_ld32(tmem_o + lane_addr + cbase + c, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] *= alpha;
          tmem_st32(tmem_o + lane_addr + cbase + c, ov);
        }
      }
      l *= alpha;
      const float2 scale2 = make_float2(scale, scale), neg_m2 = make_float2(-m_ref, -m_ref);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t w[32];  // 64 keys = 32 packed columns
#pragma unroll
      for (int q = 0; q < 32; ++q) {
        float2 e = __ffma2_rn(make_float2(sv[2 * q], sv[2 * q + 1]), scale2, neg_m2);
        e.x = ex2_approx(e.x);
        e.y = ex2_approx(e.y);
        sum2[q & 1] = __fadd2_rn(sum2[q & 1], e);
        w[q] = Mma16816<T>::pack(e.x, e.y);
      }
      tmem_st32(tmem_s + lane_addr + b * kKv + half * 32, w);
      l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[kPFull + b]);
    }
    // Row sum = this half + the partner's.
    xchg[((n_tiles & 1) * 2 + half) * kRows + row] = l;
    pair_sync();
    l += xchg[((n_tiles & 1) * 2 + (half ^ 1)) * kRows + row];
    if (ok && !mbar_wait_bounded(&bars[kPvDone + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1u)) ok = false;
    if (!ok) {
      raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
    } else {
      tc_fence_after();
      const float inv = 1.f / fmaxf(l, 1.17549435e-38f);
      T* orow = reinterpret_cast<T*>(p.out) + (q_begin + i0 + tok_local) * p.o_st +
                (long long)(kvh * p.group + head_local) * p.o_sh + cbase;
#pragma unroll
      for (int c = 0; c < kHalf; c += 32) {
        float ov[32];
        tmem_ld32(tmem_o + lane_addr + cbase + c, ov);
        tmem_ld_wait();
        if (row_live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = Mma16816<T>::pack(ov[i + 2 * q] * inv, ov[i + 2 * q + 1] * inv);
            *reinterpret_cast<uint4*>(orow + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kSoftmaxWarps + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

struct TileMapKey {
  void* ptr;
  long long s0, s2;
  int num_blocks, kv_heads, block_size, dtype;
  bool operator==(const TileMapKey& o) const {
    return ptr == o.ptr && s0 == o.s0 && s2 == o.s2 && num_blocks == o.num_blocks && kv_heads == o.kv_heads &&
           block_size == o.block_size && dtype == o.dtype;
  }
};
struct TileMapKeyHash {
  size_t operator()(const TileMapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.s0;
    h = h * 1000003u ^ (size_t)k.s2;
    h = h * 1000003u ^ (size_t)(k.num_blocks * 131 + k.kv_heads * 17 + k.block_size * 3 + k.dtype);
    return h;
  }
};

// 5-D map over pages [page, head, token, 128] whose box is one whole 16-token x 128-dim slab (4 KiB):
//   d0 = 64 dims, d1 = token % 8, d2 = 64-dim half, d3 = (head, token / 8) merged, d4 = page.
// Merging head and token / 8 needs head stride == block_size * token stride; the caller checks that.
int page_tile_map(const mie_view4_t& pages, int num_blocks, int kv_heads, int block_size, int dtype,
                  CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<TileMapKey, CUtensorMap, TileMapKeyHash> cache;
  TileMapKey key{pages.ptr, pages.stride[0], pages.stride[2], num_blocks, kv_heads, block_size, dtype};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t tok = (uint64_t)pages.stride[2] * 2;  // bytes between tokens
  const uint64_t dims[5] = {64, 8, 2, (uint64_t)kv_heads * (block_size / 8), (uint64_t)num_blocks};
  const uint64_t strides[4] = {tok, 128, 8 * tok, (uint64_t)pages.stride[0] * 2};
  const uint32_t box[5] = {64, 8, 2, kSub / 8, 1};
  const int rc = make_tensor_map(out, dtype == MIE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                 5, pages.ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

bool pages_fit_tile_map(const mie_view4_t& v, int block_size) {
  if (block_size % kSub != 0 || v.stride[3] != 1 || v.stride[2] != kDim) return false;
  if (v.stride[1] != (long long)block_size * v.stride[2]) return false;
  if (v.stride[0] <= 0 || (v.stride[0] * 2) % 16 != 0) return false;
  return (reinterpret_cast<uintptr_t>(v.ptr) & 15) == 0;
}

template <typename T>
int launch_umma(const CUtensorMap& kmap, const CUtensorMap& vmap,
                const UmmaPrefillParams& p, int q_tiles, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev] = true;
  }
  dim3 grid((unsigned)q_tiles, (unsigned)p.requests, (unsigned)p.kv_heads);
  prefill_umma_kernel<T><<<grid, kThreads, kSmemBytes, stream>>>(kmap, vmap, p, q_tiles);
  MIE_LAUNCH_CHECK("prefill_umma_kernel");
  return MIE_OK;
}

}  // namespace

// Returns MIE_ERR_UNSUPPORTED (without an error message) when the shape does not fit this kernel, so the
// caller can take the mma.sync kernel instead.
int prefill_attention_umma(const void* query, long long q_st, long long q_sh, long long total_tokens, void* out,
                           long long o_st, long long o_sh, const mie_view4_t& key_blocks,
                           const mie_view4_t& value_blocks, const mie_index_t& block_tables,
                           const mie_index_t& cu_seqlens, const mie_index_t& kv_lens, int requests, int max_query_len,
                           int q_heads, int kv_heads, int block_size, int num_blocks, int table_width, int dtype,
                           float scale, int* status, cudaStream_t stream) {
  const int group = q_heads / kv_heads;
  if (!(group == 1 || group == 2 || group == 4 || group == 8)) return MIE_ERR_UNSUPPORTED;
  if ((q_st * 2) % 16 || (q_sh * 2) % 16 || (reinterpret_cast<uintptr_t>(query) & 15)) return MIE_ERR_UNSUPPORTED;
  if ((o_st * 2) % 16 || (o_sh * 2) % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return MIE_ERR_UNSUPPORTED;
  if (total_tokens <= 0 || !(scale > 0.f)) return MIE_ERR_UNSUPPORTED;
  if (!pages_fit_tile_map(key_blocks, block_size) || !pages_fit_tile_map(value_blocks, block_size))
    return MIE_ERR_UNSUPPORTED;
  if ((long long)table_width * block_size / kSub + kKv / kSub > kMaxIds) return MIE_ERR_UNSUPPORTED;
  CUtensorMap kmap, vmap;
  if (int rc = page_tile_map(key_blocks, num_blocks, kv_heads, block_size, dtype, &kmap)) return rc;
  if (int rc = page_tile_map(value_blocks, num_blocks, kv_heads, block_size, dtype, &vmap)) return rc;
  UmmaPrefillParams p{(const char*)query, q_st, q_sh, (char*)out, o_st, o_sh, IndexView(block_tables), IndexView(cu_seqlens), IndexView(kv_lens),
                      requests, q_heads, kv_heads, group, block_size, num_blocks, table_width,
                      scale * 1.4426950408889634f, status};
  const int tok_per_tile = kRows / group;
  const int q_tiles = (max_query_len + tok_per_tile - 1) / tok_per_tile;
  if (dtype == MIE_DTYPE_BF16) return launch_umma<__nv_bfloat16>(kmap, vmap, p, q_tiles, stream);
  return launch_umma<__half>(kmap, vmap, p, q_tiles, stream);
}

}  // namespace mie
