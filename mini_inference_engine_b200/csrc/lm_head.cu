// Tied lm_head + greedy sampling in one pass over the vocabulary:
//
//   token[b] = argmax_v bf16( sum_k x[b, k] * W[v, k] )      (lowest v among equal bf16 logits)
//
// i.e. the bf16 matmul followed by argmax of the reference's decode step, without ever writing the
// [batch, vocab] logits.
//
// sm_100a design
//   * Persistent, one CTA per SM; CTA c scores vocabulary tiles c, c + P, ... of 128 rows each.
//   * tcgen05.mma kind::f16 (bf16, 128 x BN x 16): the 128 UMMA rows are vocabulary rows, the BN = 16..256
//     columns are tokens, so the kernel streams W from HBM exactly once; operands come in by TMA (2-D tiled
//     loads, 128-byte swizzle, no multicast), the whole K range accumulates in one TMEM buffer, and two
//     buffers ping-pong between the MMA issuer and the four scoring warps.
//   * Scoring: a thread holds one vocabulary row of the tile.  Every logit is rounded to bf16 (the matmul's
//     output type), turned into an order-preserving 16-bit key with the row's rank in the tile below it,
//     and the warp's maximum per token comes from one redux.sync; lane (token % 32) keeps the running best
//     (key, vocabulary index) of its tokens across the CTA's tiles.
//   * The CTA's winners go to a 64-bit key per token in global memory with atomicMax (value key above the
//     inverted vocabulary index, so ties resolve to the lowest index); a small second kernel turns the keys
//     into int64 token ids and clears them for the next call.
//   * Every mbarrier wait is bounded (MIE_STATUS_WAIT_TIMEOUT).
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "umma.cuh"

namespace mie {
namespace {

constexpr int kLmRows = 128;      // vocabulary rows per tile (UMMA M)
constexpr int kLmBlockK = 64;     // bf16 elements of K per pipeline stage (128 bytes)
constexpr int kLmThreads = 6 * 32;  // 4 scoring warps, TMA producer, MMA issuer

struct LmParams {
  int vocab, k, batch;
  long long vocab_offset;          // added to the row index (vocabulary-sharded heads)
  unsigned long long* keys;        // [batch], zero on entry
  int* status;
};

template <int BN>
struct LmSmem {
  static constexpr int kStageBytes = kLmRows * 128 + BN * 128;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 10 ? 10 : (200 * 1024 / kStageBytes);
  static constexpr int kTotal = kStages * kStageBytes + (2 * kStages + 4) * 8 + 64 + 1024;
};

// Order-preserving 16-bit key of a bf16 value (its upper 16 float bits): larger value <=> larger key.
__device__ __forceinline__ uint32_t bf16_order_key(float v) {
  const uint32_t u = __float_as_uint(__bfloat162float(__float2bfloat16_rn(v))) >> 16;
  return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

template <int BN>
__global__ void __launch_bounds__(kLmThreads, 1)
    lm_head_argmax_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const LmParams p) {
  using S = LmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  constexpr int kSlots = (BN + 31) / 32;  // tokens tracked per lane

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (p.k + kLmBlockK - 1) / kLmBlockK;
  const int tiles = (p.vocab + kLmRows - 1) / kLmRows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  chain_wait();
  chain_release();

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const uint64_t stream_policy = l2_evict_first_policy();
      uint32_t n = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < kb_total; ++kb, ++n) {
          const int s = n % kStages;
          if (!mbar_wait_bounded(&empty_bar[s], ((n / kStages) & 1u) ^ 1u)) {
            raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          uint8_t* dst = stage_base + (size_t)s * S::kStageBytes;
          mbar_expect_tx(&full_bar[s], S::kStageBytes);
          tma_load_2d_hint(dst, &map_w, &full_bar[s], kb * kLmBlockK, tile * kLmRows, stream_policy);
          tma_load_2d(dst + kLmRows * 128, &map_x, &full_bar[s], kb * kLmBlockK, 0);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(BN, 1, 0);
      uint32_t n = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
        const int b = t & 1;
        if (!mbar_wait_bounded(&tmem_empty[b], ((t >> 1) & 1u) ^ 1u)) {
          raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
          break;
        }
        for (int kb = 0; kb < kb_total; ++kb, ++n) {
          const int s = n % kStages;
          if (!mbar_wait_bounded(&full_bar[s], (n / kStages) & 1u)) {
            raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(stage_base + (size_t)s * S::kStageBytes);
          const uint64_t da = smem_desc_k128(a_addr), db = smem_desc_k128(a_addr + kLmRows * 128);
#pragma unroll
          for (int k = 0; k < kLmBlockK / 16; ++k) {
            umma_f16(tmem_base + b * BN, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                     (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tmem_full[b]);
      }
    }
  } else {
    // ---------------- Scoring warps ----------------
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    uint32_t best_key[kSlots];
    int best_row[kSlots];
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      best_key[i] = 0;
      best_row[i] = 0;
    }
    const uint32_t rank_bits = (uint32_t)(127 - (warp * 32 + lane));  // lower row wins among equal logits
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
      const int b = t & 1;
      if (!mbar_wait_bounded(&tmem_full[b], (t >> 1) & 1u)) {
        raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool live = tile * kLmRows + warp * 32 + lane < p.vocab;
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        float d[16];
        tmem_ld16(lane_addr + (uint32_t)(b * BN + c), d);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t mine = live ? ((bf16_order_key(d[j]) << 16) | rank_bits) : 0u;
          const uint32_t top = __reduce_max_sync(0xffffffffu, mine);
          // Tiles arrive in increasing vocabulary order, so a later tile only wins with a larger logit.
          if (((c + j) & 31) == lane && (top >> 16) > (best_key[(c + j) >> 5] >> 16)) {
            best_key[(c + j) >> 5] = top;
            best_row[(c + j) >> 5] = tile * kLmRows + 127 - (int)(top & 0xffffu);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[b]);
    }
    if (ok) {
#pragma unroll
      for (int i = 0; i < kSlots; ++i) {
        const int token = i * 32 + lane;
        if (token < p.batch && best_key[i] != 0u) {
          const unsigned long long row = (unsigned long long)(p.vocab_offset + best_row[i]);
          const unsigned long long key = ((unsigned long long)(best_key[i] >> 16) << 32) | (0xffffffffull - row);
          atomicMax(&p.keys[token], key);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// keys -> token ids; the keys are cleared for the next call.  `values` (optional) receives the winning
// bf16 logit's order key (what a vocabulary-sharded caller compares across ranks).  A row whose key was
// never raised (every CTA gave up on a bounded wait) or decodes to an id outside this call's vocabulary
// range gets the first id of the range and a status bit, so that whatever consumes the token next (an
// embedding gather, for one) stays inside its table.
__global__ void lm_head_finish_kernel(unsigned long long* keys, long long* tokens, int* values, int batch,
                                      long long vocab_offset, long long vocab, int* status) {
  chain_wait();
  chain_release();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const unsigned long long key = keys[b];
  long long token = (long long)(0xffffffffull - (key & 0xffffffffull));
  int value = (int)(key >> 32);
  if (key == 0ull || token < vocab_offset || token >= vocab_offset + vocab) {
    raise_status(status, MIE_STATUS_NO_TOKEN);
    token = vocab_offset;
    value = 0;  // below every real logit's key: a vocabulary-sharded caller prefers any other rank's row
  }
  tokens[b] = token;
  if (values != nullptr) values[b] = value;
  keys[b] = 0ull;
}

struct LmMapKey {
  const void* ptr;
  long long rows, k, ld;
  int box_rows;
  bool operator==(const LmMapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows;
  }
};
struct LmMapHash {
  size_t operator()(const LmMapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.k;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

// 2-D bf16 tensor map [rows, k] (row stride ld elements), box 64 x box_rows, 128-byte swizzle.
int lm_operand_map(const void* ptr, long long rows, long long k, long long ld, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<LmMapKey, CUtensorMap, LmMapHash> cache;
  LmMapKey key{ptr, rows, k, ld, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t dims[2] = {(uint64_t)k, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)ld * 2};
  const uint32_t box[2] = {(uint32_t)kLmBlockK, (uint32_t)box_rows};
  const int rc = make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

template <int BN>
int launch_lm_head(const CUtensorMap& mw, const CUtensorMap& mx, const LmParams& p, cudaStream_t stream) {
  using S = LmSmem<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(lm_head_argmax_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    configured[dev] = true;
  }
  const int tiles = (p.vocab + kLmRows - 1) / kLmRows;
  const int ctas = tiles < sm_count() ? tiles : sm_count();
  MIE_CUDA(launch_chained(lm_head_argmax_kernel<BN>, dim3(ctas), dim3(kLmThreads), (size_t)S::kTotal, stream, mw, mx, p));
  MIE_LAUNCH_CHECK("lm_head_argmax_kernel");
  return MIE_OK;
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_lm_head_argmax(const void* x, int64_t ldx, const void* w, int64_t ldw, int32_t batch,
                                  int32_t vocab, int32_t k, int64_t vocab_offset, uint64_t* keys, int64_t* tokens,
                                  int32_t* values, int32_t* status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MIE_CHECK_ARG(x && w && keys && tokens, "null pointer");
  MIE_CHECK_ARG(batch >= 0 && batch <= 256, "batch %d outside [0, 256]", batch);
  MIE_CHECK_ARG(vocab >= 1 && k >= 1 && vocab_offset >= 0 && vocab_offset + vocab <= 0xffffffffll,
                "invalid vocabulary range");
  MIE_CHECK_ARG(ldx >= k && ldw >= k && ldx % 8 == 0 && ldw % 8 == 0, "row strides must be multiples of 16 bytes");
  MIE_CHECK_ARG(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0,
                "operands must be 16-byte aligned");
  if (batch == 0) return MIE_OK;
  const int bn = batch <= 16 ? 16 : batch <= 32 ? 32 : batch <= 64 ? 64 : batch <= 128 ? 128 : 256;
  LmParams p;
  p.vocab = vocab;
  p.k = k;
  p.batch = batch;
  p.vocab_offset = vocab_offset;
  p.keys = reinterpret_cast<unsigned long long*>(keys);
  p.status = status;
  CUtensorMap mw, mx;
  if (int rc = lm_operand_map(w, vocab, k, ldw, kLmRows, &mw)) return rc;
  if (int rc = lm_operand_map(x, batch, k, ldx, bn, &mx)) return rc;
  int rc;
  switch (bn) {
    case 16: rc = launch_lm_head<16>(mw, mx, p, stream); break;
    case 32: rc = launch_lm_head<32>(mw, mx, p, stream); break;
    case 64: rc = launch_lm_head<64>(mw, mx, p, stream); break;
    case 128: rc = launch_lm_head<128>(mw, mx, p, stream); break;
    default: rc = launch_lm_head<256>(mw, mx, p, stream); break;
  }
  if (rc != MIE_OK) return rc;
  MIE_CUDA(launch_chained(lm_head_finish_kernel, dim3((batch + 127) / 128), dim3(128), (size_t)0, stream, p.keys,
                          reinterpret_cast<long long*>(tokens), values, (int)batch, (long long)vocab_offset,
                          (long long)vocab, status));
  MIE_LAUNCH_CHECK("lm_head_finish_kernel");
  return MIE_OK;
}
