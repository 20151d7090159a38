// Packed varlen causal attention over paged K/V (chunked prefill): query rows of
// request r sit at positions kv_len[r] - q_len[r] + i ("lower-right" causal), so a
// chunk sees its whole cached prefix plus the causal part of itself.
//
// One CTA = 16 query tokens x the G query heads that share one KV head (one warp per
// head, an m16 MMA tile each), so every K/V tile staged in shared memory serves the
// whole GQA group.  K/V pages are gathered through the block table with TMA (the same
// 16-token, 128-byte-swizzled boxes as the decode kernel; no multicast) into a 2-stage
// ring of 64-token tiles; Q.K^T and P.V run on mma.sync bf16/fp16 tensor-core tiles with
// an fp32 online softmax in registers.  Heaviest query tiles are scheduled first.
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace mie {

// Defined in decode_attention.cu: cached 4-D tensor map over [pages, kv_heads, page, 128].
int page_tensor_map(const mie_view4_t& pages, int num_blocks, int kv_heads, int block_size, int dtype,
                    CUtensorMap* out);
bool pages_fit_tma(const mie_view4_t& v, int head_dim, int block_size);
// Defined in prefill_attention_umma.cu: the tcgen05 kernel; MIE_ERR_UNSUPPORTED when the shape does not fit it.
int prefill_attention_umma(const void* query, long long q_st, long long q_sh, long long total_tokens, void* out,
                           long long o_st, long long o_sh, const mie_view4_t& key_blocks,
                           const mie_view4_t& value_blocks, const mie_index_t& block_tables,
                           const mie_index_t& cu_seqlens, const mie_index_t& kv_lens, int requests, int max_query_len,
                           int q_heads, int kv_heads, int block_size, int num_blocks, int table_width, int dtype,
                           float scale, int* status, cudaStream_t stream);

namespace {

constexpr int kHeadDim = 128;
constexpr int kQTile = 16;          // query tokens per CTA
constexpr int kSub = 16;            // tokens per TMA box
constexpr int kKvTile = 64;         // tokens per pipeline stage
constexpr int kSubBytes = kSub * kHeadDim * 2;       // 4 KiB
constexpr int kTileBytes = kKvTile * kHeadDim * 2;   // 16 KiB (K or V)
constexpr int kStageBytes = 2 * kTileBytes;          // K + V
constexpr int kStages = 2;
constexpr int kMaxGroup = 8;

struct PrefillParams {
  const char* q;
  long long q_st, q_sh;   // token / head strides (elements)
  char* out;
  long long o_st, o_sh;
  IndexView tables, cu_seqlens, kv_lens;
  int requests, q_heads, kv_heads, group, block_size, num_blocks, table_width;
  float scale_log2;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(kMaxGroup * 32, 1)
    prefill_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const PrefillParams p, const int q_tiles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int r = blockIdx.y, kvh = blockIdx.z;
  const int qt = q_tiles - 1 - (int)blockIdx.x;  // heaviest (latest) query tiles first
  const long long q_begin = p.cu_seqlens.at(r), q_end = p.cu_seqlens.at(r + 1);
  const int q_len = (int)(q_end - q_begin);
  const long long kv_len = p.kv_lens.at(r);
  const int i0 = qt * kQTile;
  if (i0 >= q_len) return;
  if (kv_len < q_len || kv_len > (long long)p.table_width * p.block_size) {
    if (threadIdx.x == 0) raise_status(p.status, MIE_STATUS_BAD_LENGTH);
    return;
  }
  const long long offset = kv_len - q_len;                       // position of query row 0
  const int rows = q_len - i0 < kQTile ? q_len - i0 : kQTile;
  const long long last_key = offset + i0 + rows - 1;             // largest key any row of this tile sees
  const int n_tiles = (int)(last_key / kKvTile) + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const uint64_t policy = l2_evict_first_policy();
  auto issue = [&](int tile) {
    const int s = tile % kStages;
    uint8_t* dst = smem + (size_t)s * kStageBytes;
    mbar_expect_tx(&bars[s], kStageBytes);
#pragma unroll
    for (int sub = 0; sub < kKvTile / kSub; ++sub) {
      const long long tok = (long long)tile * kKvTile + sub * kSub;
      long long pid = 0;
      int tok_in_page = 0;
      if (tok <= last_key) {
        pid = p.tables.at(r, tok / p.block_size);
        tok_in_page = (int)(tok % p.block_size);
        if (pid < 0 || pid >= p.num_blocks) {
          raise_status(p.status, MIE_STATUS_BAD_PAGE);
          pid = 0;
        }
      }
      // Sub-tiles past the last needed key still land (page 0) so the byte count of the stage is fixed;
      // their scores are masked.
      uint8_t* k_dst = dst + sub * kSubBytes;
      uint8_t* v_dst = dst + kTileBytes + sub * kSubBytes;
      tma_load_4d_hint(k_dst, &kmap, &bars[s], 0, tok_in_page, kvh, (int)pid, policy);
      tma_load_4d_hint(k_dst + kSubBytes / 2, &kmap, &bars[s], 64, tok_in_page, kvh, (int)pid, policy);
      tma_load_4d_hint(v_dst, &vmap, &bars[s], 0, tok_in_page, kvh, (int)pid, policy);
      tma_load_4d_hint(v_dst + kSubBytes / 2, &vmap, &bars[s], 64, tok_in_page, kvh, (int)pid, policy);
    }
  };
  if (threadIdx.x == 0) {
    for (int tile = 0; tile < kStages && tile < n_tiles; ++tile) issue(tile);
  }

  // Query fragments of this warp's head: rows g and g + 8 of the 16-token tile.
  const bool head_live = warp < p.group;
  const int head = kvh * p.group + (head_live ? warp : 0);
  uint32_t qa[8][4];
  {
    const T* q0 = reinterpret_cast<const T*>(p.q) + (q_begin + i0 + g) * p.q_st + (long long)head * p.q_sh;
    const T* q1 = q0 + 8 * p.q_st;
    const bool r0 = head_live && g < rows, r1 = head_live && g + 8 < rows;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
      qa[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
      qa[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
      qa[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  const long long pos0 = offset + i0 + g, pos1 = pos0 + 8;  // causal limits of this lane's two rows

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  const int k_tok = (lane & 7) + ((lane >> 4) & 1) * 8, k_sel = (lane >> 3) & 1;
  const int v_tok = (lane & 7) + ((lane >> 3) & 1) * 8, v_sel = (lane >> 4) & 1;
  const uint32_t k_row = k_tok * 128, k_key = k_tok & 7;
  const uint32_t v_row = v_tok * 128, v_key = v_tok & 7;

  uint32_t parity = 0;
  bool timed_out = false;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    const bool arrived = mbar_wait_bounded(&bars[s], (parity >> s) & 1u);
    if (!__all_sync(0xffffffffu, arrived)) {
      timed_out = true;
      break;
    }
    parity ^= 1u << s;
    const uint32_t kbase = smem_u32(smem + (size_t)s * kStageBytes);
    const uint32_t vbase = kbase + kTileBytes;
    const long long key0 = (long long)tile * kKvTile;
    if (key0 + kKvTile > kv_len) {
      // Slots past the request's length may hold anything (even NaN bits): zero those V rows so that
      // 0 * V stays 0.  K rows there only produce scores that the mask replaces.
      uint8_t* vt = smem + (size_t)s * kStageBytes + kTileBytes;
      for (int c = threadIdx.x; c < kKvTile * 16; c += blockDim.x) {
        const int row = c >> 4, chunk = c & 15;  // row = token in tile; 16 chunks of 16 bytes per row
        if (key0 + row >= kv_len) {
          *reinterpret_cast<uint4*>(vt + (row >> 4) * kSubBytes + (chunk >> 3) * (kSubBytes / 2) + (row & 15) * 128 +
                                    (chunk & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      fence_proxy_async_smem();
      __syncthreads();
    }

    // S = Q K^T : 16 x 64 per warp
    float sc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t addr = kbase + sub * kSubBytes + (ks >> 2) * (kSubBytes / 2) + k_row +
                              (((((ks & 3) * 2) | k_sel) ^ k_key) << 4);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(r0, r1, r2, r3, addr);
        Mma16816<T>::run(sc[2 * sub], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r0, r1);
        Mma16816<T>::run(sc[2 * sub + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r2, r3);
      }
    }
    // Mask (causal + length) and online softmax for rows g and g + 8.
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const long long key = key0 + n * 8 + 2 * t;
      sc[n][0] = key <= pos0 ? sc[n][0] * p.scale_log2 : -INFINITY;
      sc[n][1] = key + 1 <= pos0 ? sc[n][1] * p.scale_log2 : -INFINITY;
      sc[n][2] = key <= pos1 ? sc[n][2] * p.scale_log2 : -INFINITY;
      sc[n][3] = key + 1 <= pos1 ? sc[n][3] * p.scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // Key 0 is visible to every row, so after tile 0 the running maxima are finite.
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      sc[n][0] = exp2f(sc[n][0] - mn0);
      sc[n][1] = exp2f(sc[n][1] - mn0);
      sc[n][2] = exp2f(sc[n][2] - mn1);
      sc[n][3] = exp2f(sc[n][3] - mn1);
      s0 += sc[n][0] + sc[n][1];
      s1 += sc[n][2] + sc[n][3];
    }
    l0 = l0 * a0 + s0;
    l1 = l1 * a1 + s1;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      o[n][0] *= a0;
      o[n][1] *= a0;
      o[n][2] *= a1;
      o[n][3] *= a1;
    }
    // O += P V  (V rows past the request's length are multiplied by exact zeros; pages hold finite data
    // or the zero fill of the cache)
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) {
      const uint32_t pa0 = Mma16816<T>::pack(sc[2 * sub][0], sc[2 * sub][1]);
      const uint32_t pa1 = Mma16816<T>::pack(sc[2 * sub][2], sc[2 * sub][3]);
      const uint32_t pa2 = Mma16816<T>::pack(sc[2 * sub + 1][0], sc[2 * sub + 1][1]);
      const uint32_t pa3 = Mma16816<T>::pack(sc[2 * sub + 1][2], sc[2 * sub + 1][3]);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        const uint32_t addr = vbase + sub * kSubBytes + (np >> 2) * (kSubBytes / 2) + v_row +
                              (((((np & 3) * 2) | v_sel) ^ v_key) << 4);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(r0, r1, r2, r3, addr);
        Mma16816<T>::run(o[2 * np], pa0, pa1, pa2, pa3, r0, r1);
        Mma16816<T>::run(o[2 * np + 1], pa0, pa1, pa2, pa3, r2, r3);
      }
    }
    __syncthreads();  // every warp is done with stage s
    if (threadIdx.x == 0 && tile + kStages < n_tiles) issue(tile + kStages);
  }
  if (timed_out) {
    if (threadIdx.x == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
    return;
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (!head_live) return;
  const float inv0 = 1.f / fmaxf(l0, 1.17549435e-38f), inv1 = 1.f / fmaxf(l1, 1.17549435e-38f);
  T* out0 = reinterpret_cast<T*>(p.out) + (q_begin + i0 + g) * p.o_st + (long long)head * p.o_sh;
  T* out1 = out0 + 8 * p.o_st;
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    if (g < rows) *reinterpret_cast<uint32_t*>(out0 + n * 8 + 2 * t) = Mma16816<T>::pack(o[n][0] * inv0, o[n][1] * inv0);
    if (g + 8 < rows)
      *reinterpret_cast<uint32_t*>(out1 + n * 8 + 2 * t) = Mma16816<T>::pack(o[n][2] * inv1, o[n][3] * inv1);
  }
}

constexpr size_t kPrefillSmem = (size_t)kStages * kStageBytes + kStages * 8 + 1024;

template <typename T>
int launch_prefill(const CUtensorMap& kmap, const CUtensorMap& vmap, const PrefillParams& p, int q_tiles,
                   cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(prefill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrefillSmem));
    configured[dev] = true;
  }
  const int warps = p.group < 4 ? 4 : p.group;
  dim3 grid((unsigned)q_tiles, (unsigned)p.requests, (unsigned)p.kv_heads);
  prefill_kernel<T><<<grid, warps * 32, kPrefillSmem, stream>>>(kmap, vmap, p, q_tiles);
  MIE_LAUNCH_CHECK("prefill_kernel");
  return MIE_OK;
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_flash_prefill_attention(const void* query, int64_t q_token_stride, int64_t q_head_stride,
                                           int64_t total_tokens, void* out,
                                           int64_t o_token_stride, int64_t o_head_stride, mie_view4_t key_blocks,
                                           mie_view4_t value_blocks, mie_index_t block_tables, mie_index_t cu_seqlens,
                                           mie_index_t kv_lens, int32_t requests, int32_t max_query_len,
                                           int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t block_size,
                                           int32_t num_blocks, int32_t table_width, int32_t dtype, float scale,
                                           int32_t* status, void* stream) {
  MIE_CHECK_ARG(query && out && key_blocks.ptr && value_blocks.ptr && block_tables.ptr && cu_seqlens.ptr && kv_lens.ptr,
                "null tensor pointer");
  MIE_CHECK_ARG(requests >= 0 && max_query_len >= 0 && q_heads >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0,
                "invalid request / head counts");
  MIE_CHECK_ARG(dtype == MIE_DTYPE_BF16 || dtype == MIE_DTYPE_F16, "prefill attention supports bf16 and fp16");
  const int group = q_heads / kv_heads;
  MIE_CHECK_ARG(head_dim == kHeadDim && group <= kMaxGroup && block_size % kSub == 0,
                "prefill attention needs head_dim 128, at most 8 query heads per KV head and a page size that is a "
                "multiple of 16 (got head_dim %d, group %d, page %d)",
                head_dim, group, block_size);
  MIE_CHECK_ARG(pages_fit_tma(key_blocks, head_dim, block_size) && pages_fit_tma(value_blocks, head_dim, block_size),
                "K/V pages must be 16-byte aligned with a contiguous head_dim");
  MIE_CHECK_ARG(q_token_stride % 2 == 0 && q_head_stride % 2 == 0 && o_token_stride % 2 == 0 &&
                    o_head_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(query) & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(out) & 3) == 0,
                "query/out rows must be 4-byte aligned");
  if (requests == 0 || max_query_len == 0) return MIE_OK;
  // The tcgen05 kernel takes every shape it supports; MIE_PREFILL_KERNEL=mma forces the mma.sync kernel.
  static const bool force_mma = [] {
    const char* v = getenv("MIE_PREFILL_KERNEL");
    return v != nullptr && v[0] == 'm';
  }();
  if (!force_mma) {
    const int rc = prefill_attention_umma(query, q_token_stride, q_head_stride, total_tokens, out, o_token_stride,
                                          o_head_stride, key_blocks, value_blocks, block_tables, cu_seqlens, kv_lens,
                                          requests, max_query_len, q_heads, kv_heads, block_size, num_blocks,
                                          table_width, dtype, scale, status, (cudaStream_t)stream);
    if (rc != MIE_ERR_UNSUPPORTED) return rc;
  }
  CUtensorMap kmap, vmap;
  if (int rc = page_tensor_map(key_blocks, num_blocks, kv_heads, block_size, dtype, &kmap)) return rc;
  if (int rc = page_tensor_map(value_blocks, num_blocks, kv_heads, block_size, dtype, &vmap)) return rc;
  PrefillParams p{(const char*)query, q_token_stride, q_head_stride, (char*)out, o_token_stride, o_head_stride,
                  IndexView(block_tables), IndexView(cu_seqlens), IndexView(kv_lens), requests, q_heads, kv_heads,
                  group, block_size, num_blocks, table_width, scale * 1.4426950408889634f, status};
  const int q_tiles = (max_query_len + kQTile - 1) / kQTile;
  if (dtype == MIE_DTYPE_BF16) return launch_prefill<__nv_bfloat16>(kmap, vmap, p, q_tiles, (cudaStream_t)stream);
  return launch_prefill<__half>(kmap, vmap, p, q_tiles, (cudaStream_t)stream);
}
