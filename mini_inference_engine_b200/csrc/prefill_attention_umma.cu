// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA = one 128-row query tile: 128 / G consecutive query tokens of one request times the G query
// heads that share one KV head, so a K/V tile staged once serves the whole GQA group.  Per 128-token K/V
// tile:
//   S = Q K^T      UMMA 128x128x16 (bf16/fp16, fp32 accumulate) into one of two TMEM buffers;
//   softmax        128 threads, one query row each, read their S row from TMEM, apply the causal /
//                  length mask and an exp2 softmax against a running reference maximum, and write
//                  P (16-bit) into a 128-byte-swizzled shared-memory tile;
//   O += P V       UMMA 128x128x16 with V as the MN-major B operand, accumulated in TMEM over all tiles.
// The reference maximum is only moved when a row's maximum grows by more than 2^8 (then that warp
// rescales its O rows in TMEM), so O is read from TMEM once, at the end.
// Warp roles: 4 softmax warps, 1 TMA producer (K/V pages gathered through the block table with 16-token
// boxes, 128-byte swizzle, no multicast; Q with one 3-D box per 64-dim half), 1 MMA issuer that also owns
// the TMEM allocation.  Every wait is bounded and reports MIE_STATUS_WAIT_TIMEOUT.
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "umma.cuh"

namespace mie {

int page_tensor_map(const mie_view4_t& pages, int num_blocks, int kv_heads, int block_size, int dtype,
                    CUtensorMap* out);

namespace {

constexpr int kDim = 128;
constexpr int kRows = 128;                       // query rows per CTA (tokens x group heads)
constexpr int kKv = 128;                         // K/V tokens per tile
constexpr int kSub = 16;                         // tokens per TMA box
constexpr int kHalfTile = kKv * 64 * 2;          // [128 rows][64 elems] 16-bit = 16 KiB
constexpr int kTile = 2 * kHalfTile;             // 32 KiB: Q, K, V or P tile
constexpr int kKvStages = 2;
constexpr int kSoftmaxWarps = 4;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr float kRescaleThreshold = 8.0f;        // log2 units

// Shared-memory map (1024-byte aligned): Q | K[2] | V[2] | P | barriers.
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kTile;
constexpr int kOffV = kOffK + kKvStages * kTile;
constexpr int kOffP = kOffV + kKvStages * kTile;
constexpr int kOffBar = kOffP + kTile;
constexpr int kSmemBytes = kOffBar + 256 + 1024;

struct UmmaPrefillParams {
  char* out;
  long long o_st, o_sh;
  IndexView tables, cu_seqlens, kv_lens;
  int requests, q_heads, kv_heads, group, block_size, num_blocks, table_width;
  float scale_log2;
  int* status;
};

enum Bar { kQFull = 0, kKvFull = 1, kKvEmpty = 3, kSFull = 5, kSEmpty = 7, kPFull = 9, kPEmpty = 10, kVClean = 11,
           kNumBars = 12 };

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_umma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap, const UmmaPrefillParams p, const int q_tiles) {
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
    mbar_init(&bars[kQFull], 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&bars[kKvFull + s], 1);
      mbar_init(&bars[kKvEmpty + s], 1);
      mbar_init(&bars[kSFull + s], 1);
      mbar_init(&bars[kSEmpty + s], kSoftmaxWarps * 32);
    }
    mbar_init(&bars[kPFull], kSoftmaxWarps * 32);
    mbar_init(&bars[kPEmpty], 1);
    mbar_init(&bars[kVClean], 1);
    mbar_fence_init();
    tma_prefetch_desc(&qmap);
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  if (warp == kSoftmaxWarps + 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;            // two S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;      // O: columns [256,384)

  if (warp == kSoftmaxWarps) {
    // ---------------- TMA producer (+ V tail sanitiser) ----------------
    const uint64_t policy = l2_evict_first_policy();
    if (lane == 0) {
      mbar_expect_tx(&bars[kQFull], kTile);
      tma_load_3d(smem + kOffQ, &qmap, &bars[kQFull], 0, kvh * p.group, (int)(q_begin + i0));
      tma_load_3d(smem + kOffQ + kHalfTile, &qmap, &bars[kQFull], 64, kvh * p.group, (int)(q_begin + i0));
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % kKvStages;
      // Lanes 0..7 each own one 16-token box row of the tile: the eight block-table lookups (dependent
      // global loads) run in parallel instead of back to back.
      long long pid = 0;
      int tok_in_page = 0;
      if (lane < kKv / kSub) {
        const long long tok = (long long)j * kKv + lane * kSub;
        if (tok <= last_key) {
          pid = p.tables.at(r, tok / p.block_size);
          tok_in_page = (int)(tok % p.block_size);
          if (pid < 0 || pid >= p.num_blocks) {
            raise_status(p.status, MIE_STATUS_BAD_PAGE);
            pid = 0;
          }
        }
      }
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait_bounded(&bars[kKvEmpty + s], ((j / kKvStages) & 1u) ^ 1u);
        if (ok)
          mbar_expect_tx(&bars[kKvFull + s], 2 * kTile);
        else
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && lane < kKv / kSub) {
        // Boxes past the last needed key still land (page 0) so a stage always receives the same byte
        // count; their scores are masked and their V rows are zeroed below.
        uint8_t* kdst = smem + kOffK + s * kTile;
        uint8_t* vdst = smem + kOffV + s * kTile;
        const int off = lane * kSub * 128;  // 16 rows of 128 bytes
        tma_load_4d_hint(kdst + off, &kmap, &bars[kKvFull + s], 0, tok_in_page, kvh, (int)pid, policy);
        tma_load_4d_hint(kdst + kHalfTile + off, &kmap, &bars[kKvFull + s], 64, tok_in_page, kvh, (int)pid, policy);
        tma_load_4d_hint(vdst + off, &vmap, &bars[kKvFull + s], 0, tok_in_page, kvh, (int)pid, policy);
        tma_load_4d_hint(vdst + kHalfTile + off, &vmap, &bars[kKvFull + s], 64, tok_in_page, kvh, (int)pid, policy);
      }
      __syncwarp();
      if (!ok) break;
      if (j == n_tiles - 1) {
        // Slots past the request's length may hold anything (even NaN bits): zero those V rows so that a
        // zero probability times V stays zero, then tell the MMA warp the stage is clean.
        const bool landed = mbar_wait_bounded(&bars[kKvFull + s], (j / kKvStages) & 1u);
        if (!__all_sync(0xffffffffu, landed)) {
          if (lane == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        const long long first_bad = kv_len - (long long)j * kKv;  // rows >= first_bad are past the length
        uint8_t* vdst = smem + kOffV + s * kTile;
        for (int c = lane; c < kKv * 16; c += 32) {
          const int row = c >> 4, chunk = c & 15;
          if (row >= first_bad)
            *reinterpret_cast<uint4*>(vdst + (chunk >> 3) * kHalfTile + row * 128 + (chunk & 7) * 16) =
                make_uint4(0, 0, 0, 0);
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
      constexpr uint32_t idesc_s = instr_desc_f16(kKv, kFmt, 0);   // S = Q K^T : B = K, K-major
      constexpr uint32_t idesc_o = instr_desc_f16(kDim, kFmt, 1);  // O += P V : B = V, MN-major
      const uint32_t q_addr = smem_u32(smem + kOffQ), p_addr = smem_u32(smem + kOffP);
      bool ok = mbar_wait_bounded(&bars[kQFull], 0);
      auto issue_s = [&](int j) {
        const int s = j % kKvStages;
        if (!mbar_wait_bounded(&bars[kKvFull + s], (j / kKvStages) & 1u) ||
            !mbar_wait_bounded(&bars[kSEmpty + s], ((j / kKvStages) & 1u) ^ 1u))
          return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kOffK + s * kTile);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 8 x 16 dims
          const uint32_t off = (ks >> 2) * kHalfTile + (ks & 3) * 32;
          umma_f16(tmem_s + s * kKv, smem_desc_k128(q_addr + off), smem_desc_k128(k_addr + off), idesc_s,
                   ks > 0 ? 1u : 0u);
        }
        umma_commit(&bars[kSFull + s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kKvStages;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait_bounded(&bars[kPFull], j & 1u) ||
            (j == n_tiles - 1 && !mbar_wait_bounded(&bars[kVClean], 0))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + kOffV + s * kTile);
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {  // 8 x 16 tokens
          const uint64_t da = smem_desc_k128(p_addr + (kt >> 2) * kHalfTile + (kt & 3) * 32);
          const uint64_t db = smem_desc_mn128(v_addr + kt * kSub * 128, kHalfTile, 1024);
          umma_f16(tmem_o, da, db, idesc_o, (j > 0 || kt > 0) ? 1u : 0u);
        }
        umma_commit(&bars[kKvEmpty + s]);  // K/V stage free once these MMAs have read it
        umma_commit(&bars[kPEmpty]);       // P tile free, O includes tile j
      }
      if (!ok) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
    }
  } else {
    // ---------------- Softmax warps: one query row per thread ----------------
    const int row = warp * 32 + lane;                       // TMEM lane = row of the tile
    const int tok_local = row / p.group, head_local = row % p.group;
    const bool row_live = tok_local < toks;
    const long long pos = row_live ? offset + i0 + tok_local : last_key;  // dead rows compute harmlessly
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    uint8_t* p_tile = smem + kOffP;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kKvStages;
      if (!mbar_wait_bounded(&bars[kSFull + s], (j / kKvStages) & 1u)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sv[kKv];
#pragma unroll
      for (int c = 0; c < kKv; c += 32) tmem_ld32(tmem_s + lane_addr + s * kKv + c, *reinterpret_cast<float(*)[32]>(&sv[c]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars[kSEmpty + s]);  // the S buffer may be overwritten by tile j + 2
      const long long key0 = (long long)j * kKv;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < kKv; ++c) {
        sv[c] = key0 + c <= pos ? sv[c] * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, sv[c]);
      }
      // Move the reference maximum only on the first tile or when this row outgrew it by 2^8.
      float alpha = 1.f;
      const bool grow = mx > m_ref + kRescaleThreshold || j == 0;
      if (j > 0) {
        if (!mbar_wait_bounded(&bars[kPEmpty], (j - 1) & 1u)) {  // P tile free and O holds tiles < j
          ok = false;
          break;
        }
        tc_fence_after();
      }
      if (grow) {
        const float m_new = fmaxf(m_ref, mx);
        alpha = exp2f(m_ref - m_new);  // 0 on the first tile
        m_ref = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // Rescale this warp's 32 O rows in TMEM (rows that did not grow use alpha = 1).
#pragma unroll
        for (int c = 0; c < kDim; c += 32) {
          float ov[32];
          tmem_ld32(tmem_o + lane_addr + c, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] *= alpha;
          tmem_st32(tmem_o + lane_addr + c, ov);
        }
        tmem_st_wait();
      }
      l *= alpha;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < kKv; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float p0 = exp2f(sv[c + 2 * q] - m_ref), p1 = exp2f(sv[c + 2 * q + 1] - m_ref);
          sum += p0 + p1;
          w[q] = Mma16816<T>::pack(p0, p1);
        }
        const int chunk = c >> 3;  // 16-byte chunk = 8 tokens; 8 chunks per 64-token half
        *reinterpret_cast<uint4*>(p_tile + (chunk >> 3) * kHalfTile + row * 128 + (((chunk & 7) ^ (row & 7)) << 4)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
      l += sum;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars[kPFull]);
    }
    if (ok && !mbar_wait_bounded(&bars[kPEmpty], (n_tiles - 1) & 1u)) ok = false;
    if (!ok) {
      raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
    } else {
      tc_fence_after();
      const float inv = 1.f / fmaxf(l, 1.17549435e-38f);
      T* orow = reinterpret_cast<T*>(p.out) + (q_begin + i0 + tok_local) * p.o_st +
                (long long)(kvh * p.group + head_local) * p.o_sh;
#pragma unroll
      for (int c = 0; c < kDim; c += 32) {
        float ov[32];
        tmem_ld32(tmem_o + lane_addr + c, ov);
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

struct QMapKey {
  const void* ptr;
  long long tokens, heads, st, sh;
  int group, dtype;
  bool operator==(const QMapKey& o) const {
    return ptr == o.ptr && tokens == o.tokens && heads == o.heads && st == o.st && sh == o.sh && group == o.group &&
           dtype == o.dtype;
  }
};
struct QMapHash {
  size_t operator()(const QMapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.tokens;
    h = h * 1000003u ^ (size_t)k.st;
    h = h * 1000003u ^ (size_t)k.sh;
    h = h * 1000003u ^ (size_t)(k.heads * 64 + k.group * 4 + k.dtype);
    return h;
  }
};

// 3-D map over query [tokens, heads, 128]: box = 64 dims x `group` heads x (128 / group) tokens, which lands
// as 128 rows of 128 bytes ordered (token, head).
int query_tensor_map(const void* q, long long tokens, int heads, long long st, long long sh, int group, int dtype,
                     CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<QMapKey, CUtensorMap, QMapHash> cache;
  QMapKey key{q, tokens, heads, st, sh, group, dtype};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t dims[3] = {(uint64_t)kDim, (uint64_t)heads, (uint64_t)tokens};
  const uint64_t strides[2] = {(uint64_t)sh * 2, (uint64_t)st * 2};
  const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)(kRows / group)};
  const int rc = make_tensor_map(out, dtype == MIE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                 3, const_cast<void*>(q), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

template <typename T>
int launch_umma(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                const UmmaPrefillParams& p, int q_tiles, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev] = true;
  }
  dim3 grid((unsigned)q_tiles, (unsigned)p.requests, (unsigned)p.kv_heads);
  prefill_umma_kernel<T><<<grid, kThreads, kSmemBytes, stream>>>(qmap, kmap, vmap, p, q_tiles);
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
  if (total_tokens <= 0) return MIE_ERR_UNSUPPORTED;
  CUtensorMap qmap, kmap, vmap;
  if (int rc = query_tensor_map(query, total_tokens, q_heads, q_st, q_sh, group, dtype, &qmap)) return rc;
  if (int rc = page_tensor_map(key_blocks, num_blocks, kv_heads, block_size, dtype, &kmap)) return rc;
  if (int rc = page_tensor_map(value_blocks, num_blocks, kv_heads, block_size, dtype, &vmap)) return rc;
  UmmaPrefillParams p{(char*)out, o_st, o_sh, IndexView(block_tables), IndexView(cu_seqlens), IndexView(kv_lens),
                      requests, q_heads, kv_heads, group, block_size, num_blocks, table_width,
                      scale * 1.4426950408889634f, status};
  const int tok_per_tile = kRows / group;
  const int q_tiles = (max_query_len + tok_per_tile - 1) / tok_per_tile;
  if (dtype == MIE_DTYPE_BF16) return launch_umma<__nv_bfloat16>(qmap, kmap, vmap, p, q_tiles, stream);
  return launch_umma<__half>(qmap, kmap, vmap, p, q_tiles, stream);
}

}  // namespace mie
