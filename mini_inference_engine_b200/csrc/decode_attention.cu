// Ragged-batch paged decode attention for sm_100a.
//
// Fast path (bf16/fp16, head_dim 128, page size a multiple of 16, GQA group <= 8):
//   * a tiny plan kernel cuts every request's context into length-proportional
//     chunks (split-KV) and lists (request, chunk) work items;
//   * the main kernel is persistent: 8 autonomous warps per SM each pull
//     (request, chunk, KV head) items from a device counter, stream that item's
//     K/V pages HBM -> shared memory with TMA (16-token boxes, 128-byte
//     swizzle, a private 3-stage mbarrier ring per warp, no multicast), and
//     compute Q.K^T and P.V for all query heads that share the KV head with
//     mma.sync, so each K/V byte is read from HBM once per group; softmax is
//     online in fp32 with quad shuffles;
//   * a merge kernel (one block per request and KV head, exits at once for unsplit requests) combines
//     the chunks; both kernels can emit the e4m3 + per-head scale form the o_proj GEMM consumes.
// Everything else takes a generic one-warp-per-(request, head) kernel.
//
// The op is HBM-bound (4 FLOP per KV byte at GQA 4:1), so the MMA shape padding
// (4 real query rows of 16) costs nothing that matters.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace mie {
namespace {

constexpr int kWarps = 8;
constexpr int kStages = 3;
constexpr int kTileTokens = 16;
constexpr int kHeadDim = 128;
constexpr int kTileBytes = kTileTokens * kHeadDim * 2;  // one K or V tile
constexpr int kStageBytes = 2 * kTileBytes;             // K + V
constexpr int kPidBatch = 128;                          // tiles whose page ids are staged at once
constexpr int kMinChunk = 64;
constexpr int kMaxChunk = 2048;
constexpr int kPlanThreads = 1024;
constexpr int kHeaderInts = 128;  // [0]=chunk [1]=seq_chunks [2]=items; [16..79] work counters
constexpr int kCounterBase = 16;
constexpr int kCounters = 64;
constexpr int kMaxGroupMerge = 4;  // query heads per KV head the merge kernel handles in one block

struct View4 {
  char* ptr;
  long long s[4];
  __host__ View4(const mie_view4_t& v) : ptr(reinterpret_cast<char*>(v.ptr)) {
    for (int i = 0; i < 4; ++i) s[i] = v.stride[i];
  }
};

struct Scratch {
  int* header;
  int* offsets;     // [batch + 1]
  int* item_seq;    // [cap]
  int* item_chunk;  // [cap]
  float* part_m;    // [cap][q_heads]
  float* part_l;    // [cap][q_heads]
  float* part_o;    // [cap][q_heads][head_dim]
  int cap;
};

template <typename T>
__device__ __forceinline__ float round_act(float v) {
  return to_float<T>(from_float<T>(v));
}

__host__ __device__ inline long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

// Attention read length of request b, or 0 (with a status bit) when the
// metadata is unusable.
__device__ __forceinline__ long long read_length(const IndexView& lengths, const IndexView& positions, int b,
                                                 long long capacity, int* status) {
  const long long len = lengths.at(b);
  if (len < 1 || len > capacity) {
    raise_status(status, MIE_STATUS_BAD_LENGTH);
    return 0;
  }
  if (!positions.valid()) return len;
  const long long pos = positions.at(b);
  if (pos < 0) {
    raise_status(status, MIE_STATUS_BAD_POSITION);
    return 0;
  }
  return pos + 1 < len ? pos + 1 : len;
}

// ---------------------------------------------------------------------------
// Plan kernel: one CTA.
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long block_sum_ll(long long v, long long* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  long long t = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += smem[i];
  __syncthreads();
  return t;
}

// Split-KV planning.  The decode kernel is a dynamic queue of (request, chunk, KV head) items over
// `warps` persistent warps, so its time is close to
//     ceil(items / warps) x (time of one chunk + what a warp loses between two items),
// with items = kv_heads x sum_b ceil(length_b / chunk).  Policy 1 evaluates that with the batch's real
// lengths for a grid of chunk sizes and takes the cheapest: a chunk size that just misses a whole number of
// rounds costs a full extra round on a few warps (see the limit below for where this applies).
// `switch_tokens` is the between-items loss (queue pop,
// metadata, refilling the TMA ring, writing and later merging a partial) expressed in tokens of streaming;
// 128 tokens of one bf16 KV head (64 KB) reproduces the measured ranking of chunk sizes on an 8-way
// head shard (384 and 1024 tokens best, 512 and 192 worst).
constexpr int kPlanCands = 21;
// Candidate j (compile-time in the unrolled loops, so the divisions below are by constants).
__host__ __device__ constexpr int plan_chunk(int j) {
  constexpr int table[kPlanCands] = {64,  80,  96,  112, 128, 160, 192,  224,  256,  320, 384,
                                     448, 512, 640, 768, 896, 1024, 1280, 1536, 1792, 2048};
  return table[j];
}

__global__ void __launch_bounds__(kPlanThreads) plan_kernel(IndexView lengths, IndexView positions, int batch,
                                                            long long capacity_tokens, int kv_heads, int policy,
                                                            int warps, int switch_tokens, Scratch sc, int* status) {
  __shared__ long long red[32];
  __shared__ int warp_tot[32];
  __shared__ int cand_part[32][kPlanCands];
  __shared__ int cand_count[kPlanCands];
  __shared__ int running_s;
  __shared__ long long chunk_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  chain_wait();
  chain_release();

  // With one thread per request (the usual launch) a request's length is read once and kept.
  const bool one_each = batch <= (int)blockDim.x;
  long long own = 0, local = 0;
  if (one_each) {
    if (tid < batch) own = read_length(lengths, positions, tid, capacity_tokens, status);
    local = own;
  } else {
    for (int b = tid; b < batch; b += blockDim.x) local += read_length(lengths, positions, b, capacity_tokens, status);
  }
  const long long total = block_sum_ll(local, red);
  const long long room = sc.cap - batch;  // > 0, checked on the host

  long long chunk;
  if (policy == 0) {
    chunk = (1ll << 40);
  } else if (policy == 1) {
    int mine[kPlanCands];
#pragma unroll
    for (int j = 0; j < kPlanCands; ++j) mine[j] = 0;
    for (int b = tid; b < batch; b += blockDim.x) {
      const int rl = (int)(one_each ? own : read_length(lengths, positions, b, capacity_tokens, nullptr));
#pragma unroll
      for (int j = 0; j < kPlanCands; ++j) mine[j] += (rl + plan_chunk(j) - 1) / plan_chunk(j);
    }
#pragma unroll
    for (int j = 0; j < kPlanCands; ++j) {
      int v = mine[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) cand_part[warp][j] = v;
    }
    __syncthreads();
    if (tid < kPlanCands) {
      int t = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += cand_part[w][tid];
      cand_count[tid] = t;
    }
    __syncthreads();
    if (tid == 0) {
      // With several KV heads per rank and enough work for four items of at least 512 tokens per warp the kernel is bound by
      // HBM, not by the queue's rounds, and finer items measured better (C=256 at 1 / 2 ranks): there the
      // chunk stays at or below the four-items-per-warp size.  A single KV head per rank, or a batch too
      // small for that, is where whole rounds decide.
      long long limit = kMaxChunk;
      if (kv_heads >= 2) {
        const long long four = align_up((total * kv_heads + 4ll * warps - 1) / (4ll * warps), kTileTokens);
        if (four >= 512) limit = four;
      }
      long long best = plan_chunk(0);
      long long best_cost = -1;
#pragma unroll
      for (int j = kPlanCands - 1; j >= 0; --j) {  // larger chunks first: they win ties (fewer partials)
        if (plan_chunk(j) > limit && j > 0) continue;
        if (cand_count[j] > sc.cap) continue;      // more (request, chunk) pairs than the scratch holds
        const long long items = (long long)cand_count[j] * kv_heads;
        const long long rounds = (items + warps - 1) / warps;
        const long long cost = rounds * (plan_chunk(j) + switch_tokens);
        if (best_cost < 0 || cost < best_cost) {
          best_cost = cost;
          best = plan_chunk(j);
        }
      }
      chunk_s = best;
    }
    __syncthreads();
    chunk = chunk_s;
  } else {
    chunk = align_up(policy, kTileTokens);
  }
  // Never emit more (request, chunk) pairs than the caller's scratch holds.
  if (total / chunk + batch > sc.cap) {
    chunk = align_up((total + room - 1) / room, kTileTokens);  // still exact, only coarser
  }

  // Work list in request order, a request's chunks next to each other (queueing the full-sized chunks of
  // all requests first and the shorter last chunks at the end was measured 2 % slower at the same chunk size:
  // neighbouring items then no longer read neighbouring pages).
  if (tid == 0) running_s = 0;
  __syncthreads();
  for (int base = 0; base < batch; base += blockDim.x) {
    const int b = base + tid;
    int c = 0;
    if (b < batch) {
      const long long rl = one_each ? own : read_length(lengths, positions, b, capacity_tokens, nullptr);
      c = (int)((rl + chunk - 1) / chunk);
    }
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = running_s;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int excl = before + incl - c;
    if (b < batch) {
      sc.offsets[b] = excl;
      for (int j = 0; j < c; ++j) {
        sc.item_seq[excl + j] = b;
        sc.item_chunk[excl + j] = j;
      }
    }
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += warp_tot[w];
      running_s += t;
    }
    __syncthreads();
  }
  const int pairs = running_s;
  if (tid == 0) {
    sc.offsets[batch] = pairs;
    sc.header[0] = (int)(chunk > 0x7fffffffll ? 0x7fffffff : chunk);
    sc.header[1] = pairs;
    sc.header[2] = pairs * kv_heads;
  }
  if (tid < kCounters) sc.header[kCounterBase + tid] = 0;
}

// ---------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------
struct DecodeParams {
  View4 q, out;
  IndexView tables, lengths, positions;
  Scratch sc;
  int batch, q_heads, kv_heads, group, block_size, num_blocks, table_width;
  float scale_log2;
  int counter_slot;
  int* status;
  uint8_t* out_q8;     // optional e4m3 copy of the output for the next FP8 GEMM: [batch][ldq8 bytes]
  long long ldq8;
  float* out_scales;   // [q_heads][out_scale_ld]: one scale per (head, request) = per 128 columns
  int out_scale_ld;
  int merge_head0;     // first head of the group handled by this merge launch
};

template <typename T>
__global__ void __launch_bounds__(kWarps * 32, 1)
    decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(align_up((long long)reinterpret_cast<uintptr_t>(smem_raw), 1024));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* stages = smem + (size_t)warp * kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kWarps * kStages * kStageBytes) + warp * kStages;
  int* pids = reinterpret_cast<int*>(smem + (size_t)kWarps * kStages * kStageBytes + kWarps * kStages * 8) +
              warp * kPidBatch;

  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  __syncthreads();
  chain_wait();
  chain_release();

  const int g = lane >> 2, t = lane & 3;
  const int chunk = p.sc.header[0];
  const int total_items = p.sc.header[2];
  int* counter = p.sc.header + kCounterBase + p.counter_slot;
  const long long capacity_tokens = (long long)p.table_width * p.block_size;
  uint32_t parity = 0;
  const uint64_t stream_policy = l2_evict_first_policy();  // K/V pages are read once per step

  // ldmatrix lane geometry (constant per lane).
  const int k_tok = (lane & 7) + ((lane >> 4) & 1) * 8, k_sel = (lane >> 3) & 1;
  const int v_tok = (lane & 7) + ((lane >> 3) & 1) * 8, v_sel = (lane >> 4) & 1;
  const uint32_t k_row = k_tok * 128, k_key = k_tok & 7;
  const uint32_t v_row = v_tok * 128, v_key = v_tok & 7;

  while (true) {
    int item = 0;
    if (lane == 0) item = atomicAdd(counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= total_items) break;
    const int sci = item / p.kv_heads, h = item % p.kv_heads;
    const int b = p.sc.item_seq[sci], ck = p.sc.item_chunk[sci];
    const long long rl = read_length(p.lengths, p.positions, b, capacity_tokens, nullptr);
    const int nchunks = p.sc.offsets[b + 1] - p.sc.offsets[b];
    const long long t_begin = (long long)ck * chunk;
    const long long t_end = rl < t_begin + chunk ? rl : t_begin + chunk;
    const int ntiles = (int)((t_end - t_begin + kTileTokens - 1) / kTileTokens);

    // Query fragments: rows g < group are real heads, the rest of the 16 MMA rows are zero.
    uint32_t qa[8][2];
    {
      const bool real = g < p.group;
      const T* qrow = reinterpret_cast<const T*>(p.q.ptr) + (long long)b * p.q.s[0] +
                      (long long)(h * p.group + (real ? g : 0)) * p.q.s[1];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t);
        const uint32_t hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t);
        qa[ks][0] = real ? lo : 0u;
        qa[ks][1] = real ? hi : 0u;
      }
    }

    float m = -INFINITY, l = 0.f;
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    bool timed_out = false;
    for (int batch0 = 0; batch0 < ntiles && !timed_out; batch0 += kPidBatch) {
      const int nb = ntiles - batch0 < kPidBatch ? ntiles - batch0 : kPidBatch;
      __syncwarp();
      for (int i = lane; i < nb; i += 32) {
        const long long tok = t_begin + (long long)(batch0 + i) * kTileTokens;
        long long pid = p.tables.at(b, tok / p.block_size);
        if (pid < 0 || pid >= p.num_blocks) {
          raise_status(p.status, MIE_STATUS_BAD_PAGE);
          pid = 0;
        }
        pids[i] = (int)pid;
      }
      __syncwarp();
      auto issue = [&](int i) {
        const int s = i % kStages;
        const long long tok = t_begin + (long long)(batch0 + i) * kTileTokens;
        const int tok_in_page = (int)(tok % p.block_size);
        uint8_t* dst = stages + (size_t)s * kStageBytes;
        mbar_expect_tx(&bars[s], kStageBytes);
        tma_load_4d_hint(dst, &kmap, &bars[s], 0, tok_in_page, h, pids[i], stream_policy);
        tma_load_4d_hint(dst + kTileBytes / 2, &kmap, &bars[s], 64, tok_in_page, h, pids[i], stream_policy);
        tma_load_4d_hint(dst + kTileBytes, &vmap, &bars[s], 0, tok_in_page, h, pids[i], stream_policy);
        tma_load_4d_hint(dst + kTileBytes + kTileBytes / 2, &vmap, &bars[s], 64, tok_in_page, h, pids[i],
                         stream_policy);
      };
      if (lane == 0) {
        for (int i = 0; i < kStages && i < nb; ++i) issue(i);
      }
      for (int i = 0; i < nb; ++i) {
        const int s = i % kStages;
        const bool arrived = mbar_wait_bounded(&bars[s], (parity >> s) & 1u);
        if (!__all_sync(0xffffffffu, arrived)) {
          timed_out = true;
          break;
        }
        parity ^= 1u << s;
        const uint32_t kbase = smem_u32(stages + (size_t)s * kStageBytes);
        const uint32_t vbase = kbase + kTileBytes;
        const long long tok0 = t_begin + (long long)(batch0 + i) * kTileTokens;
        const int valid = (int)(t_end - tok0 < kTileTokens ? t_end - tok0 : kTileTokens);

        if (valid < kTileTokens) {
          // Rows past the read length may hold anything (even NaN bits): zero
          // them in V so that 0 * V stays 0.  K rows are masked by select below.
          uint8_t* vt = stages + (size_t)s * kStageBytes + kTileBytes;
          for (int c = lane; c < 2 * kTileTokens * 8; c += 32) {
            const int half = c / (kTileTokens * 8), rem = c % (kTileTokens * 8);
            const int row = rem / 8;
            if (row >= valid) {
              *reinterpret_cast<uint4*>(vt + half * (kTileBytes / 2) + row * 128 + (rem % 8) * 16) =
                  make_uint4(0, 0, 0, 0);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
        }

        // S = Q K^T for 16 tokens: two n-tiles, two accumulator sets to shorten the chain.
        float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float sb[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t addr =
              kbase + (ks >> 2) * (kTileBytes / 2) + k_row + (((((ks & 3) * 2) | k_sel) ^ k_key) << 4);
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4(r0, r1, r2, r3, addr);
          if (ks & 1) {
            Mma16816<T>::run(sb[0], qa[ks][0], 0u, qa[ks][1], 0u, r0, r1);
            Mma16816<T>::run(sb[1], qa[ks][0], 0u, qa[ks][1], 0u, r2, r3);
          } else {
            Mma16816<T>::run(sa[0], qa[ks][0], 0u, qa[ks][1], 0u, r0, r1);
            Mma16816<T>::run(sa[1], qa[ks][0], 0u, qa[ks][1], 0u, r2, r3);
          }
        }
        // This lane's four scores of head g: tokens 2t, 2t+1, 8+2t, 9+2t.  The reference keeps the
        // Q.K^T product in the activation dtype (a bf16/fp16 bmm per page) before the fp32 softmax;
        // rounding the fp32 dot product once reproduces that.
        float sv[4];
        sv[0] = round_act<T>(sa[0][0] + sb[0][0]) * p.scale_log2;
        sv[1] = round_act<T>(sa[0][1] + sb[0][1]) * p.scale_log2;
        sv[2] = round_act<T>(sa[1][0] + sb[1][0]) * p.scale_log2;
        sv[3] = round_act<T>(sa[1][1] + sb[1][1]) * p.scale_log2;
        const int tk = 2 * t;
        if (tk >= valid) sv[0] = -INFINITY;
        if (tk + 1 >= valid) sv[1] = -INFINITY;
        if (tk + 8 >= valid) sv[2] = -INFINITY;
        if (tk + 9 >= valid) sv[3] = -INFINITY;
        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);  // finite: token 0 of a tile is always valid
        const float alpha = exp2f(m - m_new);
        const float p0 = exp2f(sv[0] - m_new), p1 = exp2f(sv[1] - m_new);
        const float p2 = exp2f(sv[2] - m_new), p3 = exp2f(sv[3] - m_new);
        l = l * alpha + ((p0 + p1) + (p2 + p3));
        m = m_new;
        // P.V runs on the tensor cores in the activation dtype; the reference multiplies fp32 weights by
        // fp32 V, so P is split into a rounded part and its remainder (two MMAs) to keep ~16 more bits.
        const uint32_t pa0 = Mma16816<T>::pack(p0, p1), pa2 = Mma16816<T>::pack(p2, p3);
        const uint32_t pb0 = Mma16816<T>::pack(p0 - round_act<T>(p0), p1 - round_act<T>(p1));
        const uint32_t pb2 = Mma16816<T>::pack(p2 - round_act<T>(p2), p3 - round_act<T>(p3));
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          o[n][0] *= alpha;
          o[n][1] *= alpha;
        }
        // O += P V
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          const uint32_t addr =
              vbase + (np >> 2) * (kTileBytes / 2) + v_row + (((((np & 3) * 2) | v_sel) ^ v_key) << 4);
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4_trans(r0, r1, r2, r3, addr);
          Mma16816<T>::run(o[2 * np], pa0, 0u, pa2, 0u, r0, r1);
          Mma16816<T>::run(o[2 * np + 1], pa0, 0u, pa2, 0u, r2, r3);
          Mma16816<T>::run(o[2 * np], pb0, 0u, pb2, 0u, r0, r1);
          Mma16816<T>::run(o[2 * np + 1], pb0, 0u, pb2, 0u, r2, r3);
        }
        __syncwarp();
        if (lane == 0 && i + kStages < nb) issue(i + kStages);
      }
    }
    if (timed_out) {
      if (lane == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      break;
    }

    // Row sum over the quad, then write the result (final or partial).
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const bool head_live = g < p.group;
    const int head = h * p.group + (head_live ? g : 0);
    if (nchunks == 1) {
      const float inv = 1.f / fmaxf(l, 1.17549435e-38f);
      T* orow = reinterpret_cast<T*>(p.out.ptr) + (long long)b * p.out.s[0] + (long long)head * p.out.s[1];
      float amax = 0.f;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] = round_act<T>(o[n][0] * inv);  // the stored (and quantised) value is the rounded one
        o[n][1] = round_act<T>(o[n][1] * inv);
        amax = fmaxf(amax, fmaxf(fabsf(o[n][0]), fabsf(o[n][1])));
        if (head_live) *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * t) = Mma16816<T>::pack(o[n][0], o[n][1]);
      }
      if (p.out_q8 != nullptr) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float scale = __fdiv_rn(amax, 448.0f), denom = fmaxf(scale, 1e-12f);
        if (head_live) {
          uint8_t* qrow = p.out_q8 + (long long)b * p.ldq8 + head * kHeadDim;
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            *reinterpret_cast<__nv_fp8x2_storage_t*>(qrow + n * 8 + 2 * t) = __nv_cvt_float2_to_fp8x2(
                make_float2(__fdiv_rn(o[n][0], denom), __fdiv_rn(o[n][1], denom)), __NV_SATFINITE, __NV_E4M3);
          }
          if (t == 0) p.out_scales[(long long)head * p.out_scale_ld + b] = scale;
        }
      }
    } else {
      const long long first_row = (long long)p.sc.offsets[b] * p.q_heads;
      if (head_live) {
        const long long row = first_row + (long long)ck * p.q_heads + head;
        float* po = p.sc.part_o + row * kHeadDim;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          *reinterpret_cast<float2*>(po + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
        }
        if (t == 0) {
          p.sc.part_m[row] = m;
          p.sc.part_l[row] = l;
        }
      }
    }
  }

  // Requests with nothing to read (rejected metadata) get zeros.
  const int warps_total = gridDim.x * kWarps;
  for (int e = blockIdx.x * kWarps + warp; e < p.batch; e += warps_total) {
    if (p.sc.offsets[e + 1] != p.sc.offsets[e]) continue;
    for (int hq = 0; hq < p.q_heads; ++hq) {
      T* orow = reinterpret_cast<T*>(p.out.ptr) + (long long)e * p.out.s[0] + (long long)hq * p.out.s[1];
      *reinterpret_cast<uint2*>(orow + 4 * lane) = make_uint2(0u, 0u);
      if (p.out_q8 != nullptr) {
        *reinterpret_cast<uint32_t*>(p.out_q8 + (long long)e * p.ldq8 + hq * kHeadDim + 4 * lane) = 0u;
        if (lane == 0) p.out_scales[(long long)hq * p.out_scale_ld + e] = 0.f;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Main kernel over an e4m3 K/V pool (one fp32 scale per token and KV head)
// ---------------------------------------------------------------------------
// Pool layout [pages][kv_heads][2 = K, V][16 tokens][128 bytes] with scales [pages][kv_heads][2][16] fp32,
// so one page of one head is a single 4 KiB TMA box (K rows then V rows) plus one 128-byte bulk copy of
// its 32 scales: two copy instructions per 16 tokens instead of four.  Same work plan, same persistent
// warps and the same outputs (final rows, split-KV partials, e4m3 rows for o_proj) as decode_kernel.
//
// Arithmetic.  The e4m3 bytes are widened to fp16 in registers (exact) and both products run as fp16
// mma.sync with fp32 accumulation.  S = (q . k8) * k_scale[token]: the scale is applied to the fp32 dot
// product.  O += P . (v8 * v_scale): the scale of token j is folded into its probability, normalised by the
// largest V scale seen so far (a running maximum R, handled like the running maximum of the softmax: when
// it grows the accumulated output is rescaled) and lifted by 2^10 so that small probabilities stay normal
// fp16 numbers; the accumulators hold O * 1024 / R and the factor is taken out at the end.
// Fragment trick: ldmatrix hands a thread 4 consecutive bytes of a row; for Q.K^T they are taken as the
// k-slots (2t, 2t+1 | 2t+8, 2t+9) of the MMA, with the query fragment read in the same permuted order
// (a dot product does not care), and for P.V the transposed load yields two tokens x two adjacent
// dimensions, which a byte permute splits into the B fragments of an "even dimensions" and an "odd
// dimensions" n-tile.
constexpr int kWarps8 = 12;  // more warps than the bf16 kernel: a tile is half the bytes for the same latency chain
constexpr int kStages8 = 3;
constexpr int kTile8Bytes = kTileTokens * kHeadDim;    // 2 KiB of K or of V
constexpr int kStage8Bytes = 2 * kTile8Bytes + 1024;  // K + V + (128 bytes of scales, padded to the 1 KiB grid)

__device__ __forceinline__ void bulk_load_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      :
      : "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Two e4m3 values (low 16 bits of `pair`) -> two fp16 values, exact.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t pair) {
  uint32_t out;
  const unsigned short lo = (unsigned short)(pair & 0xffffu);
  asm volatile("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(out) : "h"(lo));
  return out;
}

template <typename T>
__device__ __forceinline__ uint32_t act_pair_to_f16x2(uint32_t raw);
template <>
__device__ __forceinline__ uint32_t act_pair_to_f16x2<__half>(uint32_t raw) {
  return raw;
}
template <>
__device__ __forceinline__ uint32_t act_pair_to_f16x2<__nv_bfloat16>(uint32_t raw) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 f = __bfloat1622float2(v);
  return Mma16816<__half>::pack(f.x, f.y);
}

struct Kv8Params {
  const float* kv_scales;  // [num_blocks][kv_heads][2][16]
};

template <typename T>
__global__ void __launch_bounds__(kWarps8 * 32, 1)
    decode_kv8_kernel(const __grid_constant__ CUtensorMap kvmap, const DecodeParams p, const Kv8Params kv) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(align_up((long long)reinterpret_cast<uintptr_t>(smem_raw), 1024));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* stages = smem + (size_t)warp * kStages8 * kStage8Bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kWarps8 * kStages8 * kStage8Bytes) + warp * kStages8;
  int* pids = reinterpret_cast<int*>(smem + (size_t)kWarps8 * kStages8 * kStage8Bytes + kWarps8 * kStages8 * 8) +
              warp * kPidBatch;

  if (lane == 0) {
    for (int s = 0; s < kStages8; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&kvmap);
  }
  __syncthreads();
  chain_wait();
  chain_release();

  const int g = lane >> 2, t = lane & 3;
  const int chunk = p.sc.header[0];
  const int total_items = p.sc.header[2];
  int* counter = p.sc.header + kCounterBase + p.counter_slot;
  const long long capacity_tokens = (long long)p.table_width * p.block_size;
  uint32_t parity = 0;
  const uint64_t stream_policy = l2_evict_first_policy();  // K/V pages are read once per step

  // ldmatrix lane geometry: lane i addresses row (i & 7) of matrix (i >> 3); matrices 0/1 are tokens
  // 0-7 / 8-15 of one 16-byte column chunk, matrices 2/3 the same tokens of the next chunk.
  const int m_tok = (lane & 7) + ((lane >> 3) & 1) * 8, m_sel = (lane >> 4) & 1;
  const uint32_t m_row = m_tok * 128, m_key = m_tok & 7;

  while (true) {
    int item = 0;
    if (lane == 0) item = atomicAdd(counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= total_items) break;
    const int sci = item / p.kv_heads, h = item % p.kv_heads;
    const int b = p.sc.item_seq[sci], ck = p.sc.item_chunk[sci];
    const long long rl = read_length(p.lengths, p.positions, b, capacity_tokens, nullptr);
    const int nchunks = p.sc.offsets[b + 1] - p.sc.offsets[b];
    const long long t_begin = (long long)ck * chunk;
    const long long t_end = rl < t_begin + chunk ? rl : t_begin + chunk;
    const int ntiles = (int)((t_end - t_begin + kTileTokens - 1) / kTileTokens);

    // Query fragments in the permuted k order: step c covers dims [16c, 16c + 16), this lane holds dims
    // 16c + 4t .. 16c + 4t + 3 of head g.  Rows g >= group are zero.
    uint32_t qa[8][2];
    {
      const bool real = g < p.group;
      const T* qrow = reinterpret_cast<const T*>(p.q.ptr) + (long long)b * p.q.s[0] +
                      (long long)(h * p.group + (real ? g : 0)) * p.q.s[1];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qrow + c * 16 + 4 * t);
        qa[c][0] = real ? act_pair_to_f16x2<T>(raw.x) : 0u;
        qa[c][1] = real ? act_pair_to_f16x2<T>(raw.y) : 0u;
      }
    }

    float m = -INFINITY, l = 0.f;
    float vref = 1e-30f;  // running maximum of the V scales: the accumulators hold O * 1024 / vref
    // MMA accumulators: oe[c] / oo[c] are the even- / odd-dimension n-tiles of chunk c; elements 0, 1 are
    // head g's dims 16c + 4t (+2) resp. 16c + 4t + 1 (+2), elements 2, 3 belong to the padding rows.
    float oe[8][4], oo[8][4];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      oe[c][0] = oe[c][1] = oe[c][2] = oe[c][3] = 0.f;
      oo[c][0] = oo[c][1] = oo[c][2] = oo[c][3] = 0.f;
    }

    bool timed_out = false;
    for (int batch0 = 0; batch0 < ntiles && !timed_out; batch0 += kPidBatch) {
      const int nb = ntiles - batch0 < kPidBatch ? ntiles - batch0 : kPidBatch;
      __syncwarp();
      for (int i = lane; i < nb; i += 32) {
        const long long tok = t_begin + (long long)(batch0 + i) * kTileTokens;
        long long pid = p.tables.at(b, tok / p.block_size);
        if (pid < 0 || pid >= p.num_blocks) {
          raise_status(p.status, MIE_STATUS_BAD_PAGE);
          pid = 0;
        }
        pids[i] = (int)pid;
      }
      __syncwarp();
      auto issue = [&](int i) {
        const int s = i % kStages8;
        uint8_t* dst = stages + (size_t)s * kStage8Bytes;
        mbar_expect_tx(&bars[s], 2 * kTile8Bytes + 128);
        tma_load_5d_hint(dst, &kvmap, &bars[s], 0, 0, 0, h, pids[i], stream_policy);
        bulk_load_hint(dst + 2 * kTile8Bytes, kv.kv_scales + ((long long)pids[i] * p.kv_heads + h) * 32, 128,
                       &bars[s], stream_policy);
      };
      if (lane == 0) {
        for (int i = 0; i < kStages8 && i < nb; ++i) issue(i);
      }
      for (int i = 0; i < nb; ++i) {
        const int s = i % kStages8;
        const bool arrived = mbar_wait_bounded(&bars[s], (parity >> s) & 1u);
        if (!__all_sync(0xffffffffu, arrived)) {
          timed_out = true;
          break;
        }
        parity ^= 1u << s;
        uint8_t* stage = stages + (size_t)s * kStage8Bytes;
        const uint32_t kbase = smem_u32(stage);
        const uint32_t vbase = kbase + kTile8Bytes;
        const float* scales = reinterpret_cast<const float*>(stage + 2 * kTile8Bytes);
        const long long tok0 = t_begin + (long long)(batch0 + i) * kTileTokens;
        const int valid = (int)(t_end - tok0 < kTileTokens ? t_end - tok0 : kTileTokens);

        if (valid < kTileTokens) {
          // Rows past the read length may hold anything (even NaN bytes): zero them in V so that
          // 0 * V stays 0.  K rows and all scales of such rows are masked by selects below.
          uint8_t* vt = stage + kTile8Bytes;
          for (int c = lane; c < kTileTokens * 8; c += 32) {
            if (c / 8 >= valid) *reinterpret_cast<uint4*>(vt + (c / 8) * 128 + (c % 8) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }

        // S = Q K^T for 16 tokens (two n-tiles), two accumulator sets to shorten the chain.
        float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float sb[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {  // chunks 2cp and 2cp + 1
          const uint32_t addr = kbase + m_row + ((((uint32_t)(2 * cp) | m_sel) ^ m_key) << 4);
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4(r0, r1, r2, r3, addr);
          Mma16816<__half>::run(sa[0], qa[2 * cp][0], 0u, qa[2 * cp][1], 0u, e4m3x2_to_f16x2(r0),
                                e4m3x2_to_f16x2(r0 >> 16));
          Mma16816<__half>::run(sa[1], qa[2 * cp][0], 0u, qa[2 * cp][1], 0u, e4m3x2_to_f16x2(r1),
                                e4m3x2_to_f16x2(r1 >> 16));
          Mma16816<__half>::run(sb[0], qa[2 * cp + 1][0], 0u, qa[2 * cp + 1][1], 0u, e4m3x2_to_f16x2(r2),
                                e4m3x2_to_f16x2(r2 >> 16));
          Mma16816<__half>::run(sb[1], qa[2 * cp + 1][0], 0u, qa[2 * cp + 1][1], 0u, e4m3x2_to_f16x2(r3),
                                e4m3x2_to_f16x2(r3 >> 16));
        }
        // This lane's four tokens of head g: 2t, 2t+1, 8+2t, 9+2t, and their K / V scales.
        const int tk = 2 * t;
        const float2 ks_lo = *reinterpret_cast<const float2*>(scales + tk);
        const float2 ks_hi = *reinterpret_cast<const float2*>(scales + 8 + tk);
        const float2 vs_lo = *reinterpret_cast<const float2*>(scales + 16 + tk);
        const float2 vs_hi = *reinterpret_cast<const float2*>(scales + 24 + tk);
        float sv[4], vs[4];
        sv[0] = round_act<T>((sa[0][0] + sb[0][0]) * ks_lo.x) * p.scale_log2;
        sv[1] = round_act<T>((sa[0][1] + sb[0][1]) * ks_lo.y) * p.scale_log2;
        sv[2] = round_act<T>((sa[1][0] + sb[1][0]) * ks_hi.x) * p.scale_log2;
        sv[3] = round_act<T>((sa[1][1] + sb[1][1]) * ks_hi.y) * p.scale_log2;
        vs[0] = vs_lo.x, vs[1] = vs_lo.y, vs[2] = vs_hi.x, vs[3] = vs_hi.y;
        if (tk >= valid) sv[0] = -INFINITY, vs[0] = 0.f;
        if (tk + 1 >= valid) sv[1] = -INFINITY, vs[1] = 0.f;
        if (tk + 8 >= valid) sv[2] = -INFINITY, vs[2] = 0.f;
        if (tk + 9 >= valid) sv[3] = -INFINITY, vs[3] = 0.f;
        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float vmax = fmaxf(fmaxf(vs[0], vs[1]), fmaxf(vs[2], vs[3]));  // scales are >= 0
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 1));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 2));
        const float vref_new = fmaxf(vref, vmax);
        const float m_new = fmaxf(m, mx);  // finite: token 0 of a tile is always valid
        const float alpha = exp2f(m - m_new);
        const float p0 = exp2f(sv[0] - m_new), p1 = exp2f(sv[1] - m_new);
        const float p2 = exp2f(sv[2] - m_new), p3 = exp2f(sv[3] - m_new);
        l = l * alpha + ((p0 + p1) + (p2 + p3));
        m = m_new;
        const float lift = __fdividef(1024.f, vref_new);
        const float rescale = alpha * __fdividef(vref, vref_new);  // softmax maximum and V-scale reference moved
        vref = vref_new;
        const uint32_t pa0 = Mma16816<__half>::pack(p0 * (vs[0] * lift), p1 * (vs[1] * lift));
        const uint32_t pa2 = Mma16816<__half>::pack(p2 * (vs[2] * lift), p3 * (vs[3] * lift));
        // Most tiles move neither the running maximum nor the V-scale reference of any head: then the
        // 32 multiplications by 1 are skipped (this kernel is bound by instruction issue, not by memory).
        if (__any_sync(0xffffffffu, rescale != 1.f)) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            oe[c][0] *= rescale;
            oe[c][1] *= rescale;
            oo[c][0] *= rescale;
            oo[c][1] *= rescale;
          }
        }
        // O += P' V8
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {
          const uint32_t addr = vbase + m_row + ((((uint32_t)(2 * cp) | m_sel) ^ m_key) << 4);
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4_trans(r0, r1, r2, r3, addr);
          // r0 / r1: tokens (2t, 2t+1) / (8+2t, 9+2t) x dims (2g, 2g+1) of chunk 2cp; r2 / r3: chunk 2cp + 1.
          // Bytes (tok a dim e, tok a dim o, tok b dim e, tok b dim o) -> (a e, b e | a o, b o).
          r0 = __byte_perm(r0, 0, 0x3120);
          r1 = __byte_perm(r1, 0, 0x3120);
          r2 = __byte_perm(r2, 0, 0x3120);
          r3 = __byte_perm(r3, 0, 0x3120);
          // Even-dimension tile: columns (2t, 2t+1) are dims 4t, 4t+2 of the chunk; odd tile: 4t+1, 4t+3.
          Mma16816<__half>::run(oe[2 * cp], pa0, 0u, pa2, 0u, e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r1));
          Mma16816<__half>::run(oo[2 * cp], pa0, 0u, pa2, 0u, e4m3x2_to_f16x2(r0 >> 16), e4m3x2_to_f16x2(r1 >> 16));
          Mma16816<__half>::run(oe[2 * cp + 1], pa0, 0u, pa2, 0u, e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r3));
          Mma16816<__half>::run(oo[2 * cp + 1], pa0, 0u, pa2, 0u, e4m3x2_to_f16x2(r2 >> 16),
                                e4m3x2_to_f16x2(r3 >> 16));
        }
        __syncwarp();
        if (lane == 0 && i + kStages8 < nb) issue(i + kStages8);
      }
    }
    if (timed_out) {
      if (lane == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
      break;
    }

    // Row sum over the quad, then write the result (final or partial).
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const bool head_live = g < p.group;
    const int head = h * p.group + (head_live ? g : 0);
    float o[8][4];  // o[c][j]: dim 16c + 4t + j of head g, with the V-scale reference taken out again
    {
      const float back = vref * (1.f / 1024.f);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        o[c][0] = oe[c][0] * back;
        o[c][1] = oo[c][0] * back;
        o[c][2] = oe[c][1] * back;
        o[c][3] = oo[c][1] * back;
      }
    }
    if (nchunks == 1) {
      const float inv = 1.f / fmaxf(l, 1.17549435e-38f);
      T* orow = reinterpret_cast<T*>(p.out.ptr) + (long long)b * p.out.s[0] + (long long)head * p.out.s[1];
      float amax = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[c][j] = round_act<T>(o[c][j] * inv);  // the stored (and quantised) value is the rounded one
          amax = fmaxf(amax, fabsf(o[c][j]));
        }
        if (head_live) {
          *reinterpret_cast<uint2*>(orow + c * 16 + 4 * t) =
              make_uint2(Mma16816<T>::pack(o[c][0], o[c][1]), Mma16816<T>::pack(o[c][2], o[c][3]));
        }
      }
      if (p.out_q8 != nullptr) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float scale = __fdiv_rn(amax, 448.0f), denom = fmaxf(scale, 1e-12f);
        if (head_live) {
          uint8_t* qrow = p.out_q8 + (long long)b * p.ldq8 + head * kHeadDim;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                make_float2(__fdiv_rn(o[c][0], denom), __fdiv_rn(o[c][1], denom)), __NV_SATFINITE, __NV_E4M3);
            const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
                make_float2(__fdiv_rn(o[c][2], denom), __fdiv_rn(o[c][3], denom)), __NV_SATFINITE, __NV_E4M3);
            *reinterpret_cast<uint32_t*>(qrow + c * 16 + 4 * t) = (uint32_t)lo | ((uint32_t)hi << 16);
          }
          if (t == 0) p.out_scales[(long long)head * p.out_scale_ld + b] = scale;
        }
      }
    } else {
      const long long first_row = (long long)p.sc.offsets[b] * p.q_heads;
      if (head_live) {
        const long long row = first_row + (long long)ck * p.q_heads + head;
        float* po = p.sc.part_o + row * kHeadDim;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<float4*>(po + c * 16 + 4 * t) = make_float4(o[c][0], o[c][1], o[c][2], o[c][3]);
        }
        if (t == 0) {
          p.sc.part_m[row] = m;
          p.sc.part_l[row] = l;
        }
      }
    }
  }

  // Requests with nothing to read (rejected metadata) get zeros.
  const int warps_total = gridDim.x * kWarps8;
  for (int e = blockIdx.x * kWarps8 + warp; e < p.batch; e += warps_total) {
    if (p.sc.offsets[e + 1] != p.sc.offsets[e]) continue;
    for (int hq = 0; hq < p.q_heads; ++hq) {
      T* orow = reinterpret_cast<T*>(p.out.ptr) + (long long)e * p.out.s[0] + (long long)hq * p.out.s[1];
      *reinterpret_cast<uint2*>(orow + 4 * lane) = make_uint2(0u, 0u);
      if (p.out_q8 != nullptr) {
        *reinterpret_cast<uint32_t*>(p.out_q8 + (long long)e * p.ldq8 + hq * kHeadDim + 4 * lane) = 0u;
        if (lane == 0) p.out_scales[(long long)hq * p.out_scale_ld + e] = 0.f;
      }
    }
  }
}

// Merge of split requests: one block per (request, KV head), exits at once when the request was not
// split.  Each query head of the group gets W warps that share the request's chunks (W = 2, 4 or 8, chosen
// by launch_merge from the number of blocks); their partial merges
// are combined through shared memory.  Also emits the e4m3 + per-head scale form for the o_proj GEMM.

template <typename T, int kMergeWarpsPerHead>
__global__ void __launch_bounds__(kMaxGroupMerge * kMergeWarpsPerHead * 32) merge_kernel(DecodeParams p) {
  __shared__ float part[kMaxGroupMerge][kMergeWarpsPerHead][2 + kHeadDim];
  chain_wait();
  chain_release();
  const int b = blockIdx.x / p.kv_heads, h = blockIdx.x % p.kv_heads;
  const int first = p.sc.offsets[b], n = p.sc.offsets[b + 1] - first;
  if (n <= 1) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gh = warp / kMergeWarpsPerHead, sub = warp % kMergeWarpsPerHead;
  const int head = h * p.group + p.merge_head0 + gh;
  const long long row0 = (long long)first * p.q_heads + head;
  const long long stride = p.q_heads;
  float big = -INFINITY, lsum = 0.f, a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
  for (int i = sub; i < n; i += kMergeWarpsPerHead) {
    const long long row = row0 + i * stride;
    const float mi = p.sc.part_m[row], li = p.sc.part_l[row];
    const float4 oi = reinterpret_cast<const float4*>(p.sc.part_o + row * kHeadDim)[lane];
    const float mn = fmaxf(big, mi);
    const float wo = exp2f(big - mn), wi = exp2f(mi - mn);
    lsum = lsum * wo + li * wi;
    a0 = a0 * wo + oi.x * wi;
    a1 = a1 * wo + oi.y * wi;
    a2 = a2 * wo + oi.z * wi;
    a3 = a3 * wo + oi.w * wi;
    big = mn;
  }
  float* mine = part[gh][sub];
  if (lane == 0) {
    mine[0] = big;
    mine[1] = lsum;
  }
  mine[2 + 4 * lane + 0] = a0;
  mine[2 + 4 * lane + 1] = a1;
  mine[2 + 4 * lane + 2] = a2;
  mine[2 + 4 * lane + 3] = a3;
  __syncthreads();
  if (sub != 0) return;
  big = -INFINITY;
  for (int w = 0; w < kMergeWarpsPerHead; ++w) big = fmaxf(big, part[gh][w][0]);
  lsum = a0 = a1 = a2 = a3 = 0.f;
  for (int w = 0; w < kMergeWarpsPerHead; ++w) {
    const float mw = part[gh][w][0];
    if (mw == -INFINITY) continue;  // this warp had no chunk
    const float wt = exp2f(mw - big);
    lsum += part[gh][w][1] * wt;
    a0 += part[gh][w][2 + 4 * lane + 0] * wt;
    a1 += part[gh][w][2 + 4 * lane + 1] * wt;
    a2 += part[gh][w][2 + 4 * lane + 2] * wt;
    a3 += part[gh][w][2 + 4 * lane + 3] * wt;
  }
  const float inv = 1.f / fmaxf(lsum, 1.17549435e-38f);
  a0 = round_act<T>(a0 * inv);
  a1 = round_act<T>(a1 * inv);
  a2 = round_act<T>(a2 * inv);
  a3 = round_act<T>(a3 * inv);
  T* orow = reinterpret_cast<T*>(p.out.ptr) + (long long)b * p.out.s[0] + (long long)head * p.out.s[1];
  *reinterpret_cast<uint2*>(orow + 4 * lane) = make_uint2(Mma16816<T>::pack(a0, a1), Mma16816<T>::pack(a2, a3));
  if (p.out_q8 != nullptr) {
    const float amax = warp_max(fmaxf(fmaxf(fabsf(a0), fabsf(a1)), fmaxf(fabsf(a2), fabsf(a3))));
    const float scale = __fdiv_rn(amax, 448.0f), denom = fmaxf(scale, 1e-12f);
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(a0, denom), __fdiv_rn(a1, denom)), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(a2, denom), __fdiv_rn(a3, denom)), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(p.out_q8 + (long long)b * p.ldq8 + head * kHeadDim + 4 * lane) =
        (uint32_t)lo | ((uint32_t)hi << 16);
    if (lane == 0) p.out_scales[(long long)head * p.out_scale_ld + b] = scale;
  }
}

// ---------------------------------------------------------------------------
// Generic kernel: any head_dim <= 1024, any page size, bf16/fp16/fp32.
// One warp per (request, query head); lanes split head_dim.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void generic_decode_kernel(View4 q, View4 out, View4 kb, View4 vb, IndexView tables, IndexView lengths,
                                      IndexView positions, int batch, int q_heads, int kv_heads, int head_dim,
                                      int block_size, int num_blocks, int table_width, float scale, int* status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= batch * q_heads) return;
  const int b = warp / q_heads, head = warp % q_heads;
  const int kvh = head / (q_heads / kv_heads);
  constexpr int kMaxPerLane = 32;
  const int per_lane = (head_dim + 31) / 32;
  float qv[kMaxPerLane], acc[kMaxPerLane];
  const T* qrow = reinterpret_cast<const T*>(q.ptr) + (long long)b * q.s[0] + (long long)head * q.s[1];
#pragma unroll 4
  for (int i = 0; i < per_lane; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < head_dim ? to_float<T>(qrow[(long long)d * q.s[3]]) : 0.f;
    acc[i] = 0.f;
  }
  const long long rl = read_length(lengths, positions, b, (long long)table_width * block_size,
                                   lane == 0 ? status : nullptr);
  float m = -INFINITY, l = 0.f;
  for (long long tok = 0; tok < rl; ++tok) {
    const long long page = tables.at(b, tok / block_size);
    if (page < 0 || page >= num_blocks) {
      if (lane == 0) raise_status(status, MIE_STATUS_BAD_PAGE);
      continue;
    }
    const long long slot = tok % block_size;
    const T* krow = reinterpret_cast<const T*>(kb.ptr) + page * kb.s[0] + (long long)kvh * kb.s[1] + slot * kb.s[2];
    const T* vrow = reinterpret_cast<const T*>(vb.ptr) + page * vb.s[0] + (long long)kvh * vb.s[1] + slot * vb.s[2];
    float dot = 0.f;
    for (int i = 0; i < per_lane; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) dot += qv[i] * to_float<T>(krow[(long long)d * kb.s[3]]);
    }
    dot = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, dot);
    const float alpha = __expf(m - m_new), pw = __expf(dot - m_new);
    l = l * alpha + pw;
    for (int i = 0; i < per_lane; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) acc[i] = acc[i] * alpha + pw * to_float<T>(vrow[(long long)d * vb.s[3]]);
    }
    m = m_new;
  }
  T* orow = reinterpret_cast<T*>(out.ptr) + (long long)b * out.s[0] + (long long)head * out.s[1];
  const float inv = rl > 0 ? 1.f / fmaxf(l, 1.17549435e-38f) : 0.f;
  for (int i = 0; i < per_lane; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) orow[(long long)d * out.s[3]] = from_float<T>(acc[i] * inv);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
}  // namespace

struct MapKey {
  void* ptr;
  long long s0, s1, s2;
  int num_blocks, kv_heads, block_size, dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && s0 == o.s0 && s1 == o.s1 && s2 == o.s2 && num_blocks == o.num_blocks &&
           kv_heads == o.kv_heads && block_size == o.block_size && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.s0;
    h = h * 1000003u ^ (size_t)k.s1;
    h = h * 1000003u ^ (size_t)k.s2;
    h = h * 1000003u ^ (size_t)(k.num_blocks * 131 + k.kv_heads * 17 + k.block_size * 3 + k.dtype);
    return h;
  }
};

int page_tensor_map(const mie_view4_t& pages, int num_blocks, int kv_heads, int block_size, int dtype,
                    CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{pages.ptr, pages.stride[0], pages.stride[1], pages.stride[2], num_blocks, kv_heads, block_size, dtype};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t dims[4] = {(uint64_t)kHeadDim, (uint64_t)block_size, (uint64_t)kv_heads, (uint64_t)num_blocks};
  const uint64_t strides[3] = {(uint64_t)pages.stride[2] * 2, (uint64_t)pages.stride[1] * 2,
                               (uint64_t)pages.stride[0] * 2};
  const uint32_t box[4] = {64, kTileTokens, 1, 1};
  const int rc = make_tensor_map(out, dtype == MIE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                 4, pages.ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

bool pages_fit_tma(const mie_view4_t& v, int head_dim, int block_size) {
  if (head_dim != kHeadDim || block_size % kTileTokens != 0 || v.stride[3] != 1) return false;
  if (reinterpret_cast<uintptr_t>(v.ptr) & 15) return false;
  for (int i = 0; i < 3; ++i) {
    if (v.stride[i] <= 0 || (v.stride[i] * 2) % 16 != 0) return false;
  }
  return true;
}

namespace {

constexpr size_t kDecodeSmem = (size_t)kWarps * kStages * kStageBytes + kWarps * kStages * 8 +
                               (size_t)kWarps * kPidBatch * 4 + 1024;

long long fixed_scratch_bytes(int batch, int kv_heads) {
  (void)kv_heads;
  return kHeaderInts * 4 + align_up((long long)(batch + 1) * 4, 256);
}
long long per_chunk_bytes(int q_heads, int head_dim) { return 8 + (long long)q_heads * (head_dim + 2) * 4; }

// (request, chunk) pairs `mie_decode_scratch_bytes` makes room for beyond one per request: four items per
// warp.  The plan kernel considers more items per warp only while they fit the scratch it was given.
// One thread per request, at least two warps, at most the kernel's bound: a small batch does not pay for
// block-wide reductions over 32 warps.
int plan_threads(int batch) {
  const int threads = (batch + 31) / 32 * 32;
  return threads < 64 ? 64 : threads > kPlanThreads ? kPlanThreads : threads;
}

int target_seq_chunks(int kv_heads) {
  const int items = sm_count() * kWarps * 4;
  return (items + kv_heads - 1) / kv_heads;
}

Scratch carve(void* scratch, long long bytes, int batch, int q_heads, int kv_heads, int head_dim) {
  Scratch s;
  char* base = reinterpret_cast<char*>(scratch);
  s.header = reinterpret_cast<int*>(base);
  s.offsets = reinterpret_cast<int*>(base + kHeaderInts * 4);
  long long off = fixed_scratch_bytes(batch, kv_heads);
  const long long avail = bytes - off - 1024;
  long long cap = avail / per_chunk_bytes(q_heads, head_dim);
  if (cap > 0x3fffffff) cap = 0x3fffffff;
  s.cap = (int)(cap > 0 ? cap : 0);
  s.item_seq = reinterpret_cast<int*>(base + off);
  off += align_up((long long)s.cap * 4, 256);
  s.item_chunk = reinterpret_cast<int*>(base + off);
  off += align_up((long long)s.cap * 4, 256);
  s.part_m = reinterpret_cast<float*>(base + off);
  off += align_up((long long)s.cap * q_heads * 4, 256);
  s.part_l = reinterpret_cast<float*>(base + off);
  off += align_up((long long)s.cap * q_heads * 4, 256);
  s.part_o = reinterpret_cast<float*>(base + off);
  return s;
}

// Warps per query head in the merge: the chunks of a request are shared by W warps, so the longest request
// (tens of chunks) sets the length of the kernel.  With many blocks (request x KV head) two warps per head
// keep more blocks resident; with fewer - smaller batches, or one to four KV heads per rank under tensor
// parallelism - four or eight warps per head shorten the longest chain (measured: 256 requests on a 4-way
// shard 148.4 -> 144.4 us for the whole attention call, 128 requests on one GPU 298 -> 294 us).
template <typename T>
int launch_merge(const DecodeParams& q, int heads, cudaStream_t stream) {
  const int blocks = q.batch * q.kv_heads;
  const int warps = blocks >= 2048 ? 2 : blocks >= 128 ? 4 : 8;
  if (warps == 2)
    MIE_CUDA(launch_chained(merge_kernel<T, 2>, dim3(blocks), dim3(heads * 2 * 32), 0, stream, q));
  else if (warps == 4)
    MIE_CUDA(launch_chained(merge_kernel<T, 4>, dim3(blocks), dim3(heads * 4 * 32), 0, stream, q));
  else
    MIE_CUDA(launch_chained(merge_kernel<T, 8>, dim3(blocks), dim3(heads * 8 * 32), 0, stream, q));
  MIE_LAUNCH_CHECK("merge_kernel");
  return MIE_OK;
}

template <typename T>
int launch_fast(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDecodeSmem));
    configured[dev] = true;
  }
  MIE_CUDA(launch_chained(decode_kernel<T>, dim3(sm_count()), dim3(kWarps * 32), kDecodeSmem, stream, kmap, vmap, p));
  MIE_LAUNCH_CHECK("decode_kernel");
  // Groups wider than kMaxGroupMerge take several passes of head sub-groups.
  for (int g0 = 0; g0 < p.group; g0 += kMaxGroupMerge) {
    DecodeParams q = p;
    q.merge_head0 = g0;
    const int heads = p.group - g0 < kMaxGroupMerge ? p.group - g0 : kMaxGroupMerge;
    if (int rc = launch_merge<T>(q, heads, stream)) return rc;
  }
  return MIE_OK;
}

template <typename T>
int launch_generic(mie_view4_t query, mie_view4_t out, mie_view4_t kb, mie_view4_t vb, mie_index_t tables,
                   mie_index_t lengths, mie_index_t positions, int batch, int q_heads, int kv_heads, int head_dim,
                   int block_size, int num_blocks, int table_width, float scale, int* status, cudaStream_t stream) {
  const int threads = 128;
  const long long warps = (long long)batch * q_heads;
  const int blocks = (int)((warps * 32 + threads - 1) / threads);
  generic_decode_kernel<T><<<blocks, threads, 0, stream>>>(View4(query), View4(out), View4(kb), View4(vb),
                                                          IndexView(tables), IndexView(lengths),
                                                          IndexView(positions), batch, q_heads, kv_heads, head_dim,
                                                          block_size, num_blocks, table_width, scale, status);
  MIE_LAUNCH_CHECK("generic_decode_kernel");
  return MIE_OK;
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int64_t mie_decode_scratch_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                            int64_t max_total_tokens) {
  if (batch < 0 || q_heads < 1 || kv_heads < 1 || head_dim < 1 || max_total_tokens < 0) return 0;
  // (request, chunk) pairs never exceed batch + min(target, total / min_chunk) + total / max_chunk.
  long long aimed = target_seq_chunks(kv_heads);
  if (max_total_tokens / kMinChunk + 1 < aimed) aimed = max_total_tokens / kMinChunk + 1;
  const long long cap = (long long)batch + aimed + max_total_tokens / kMaxChunk + 2;
  return fixed_scratch_bytes(batch, kv_heads) + cap * per_chunk_bytes(q_heads, head_dim) + 8 * 256 + 1024;
}

extern "C" int mie_paged_decode_attention(mie_view4_t query, mie_view4_t out, mie_view4_t key_blocks,
                                          mie_view4_t value_blocks, mie_index_t block_tables,
                                          mie_index_t sequence_lengths, mie_index_t query_positions, int32_t batch,
                                          int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t block_size,
                                          int32_t num_blocks, int32_t table_width, int32_t dtype, float scale,
                                          int32_t split_policy, int64_t max_total_tokens, void* scratch,
                                          int64_t scratch_bytes, int32_t plan_only, int32_t use_plan,
                                          int32_t plan_slot, void* out_q8, int64_t ldq8, float* out_scales,
                                          int32_t out_scale_ld, int32_t* status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MIE_CHECK_ARG(batch >= 0 && q_heads >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0,
                "query heads (%d) must be a positive multiple of KV heads (%d)", q_heads, kv_heads);
  MIE_CHECK_ARG(head_dim >= 1 && head_dim <= 1024, "head_dim must be in [1, 1024], got %d", head_dim);
  MIE_CHECK_ARG(block_size >= 1 && num_blocks >= 1 && table_width >= 1, "invalid page geometry");
  MIE_CHECK_ARG(dtype == MIE_DTYPE_BF16 || dtype == MIE_DTYPE_F16 || dtype == MIE_DTYPE_F32, "unknown dtype %d",
                dtype);
  MIE_CHECK_ARG(query.ptr && out.ptr && key_blocks.ptr && value_blocks.ptr && block_tables.ptr &&
                    sequence_lengths.ptr,
                "null tensor pointer");
  MIE_CHECK_ARG(split_policy >= 0, "split_policy must be >= 0");
  MIE_CHECK_ARG(plan_slot >= 0 && plan_slot < kCounters, "plan_slot must be in [0, %d)", kCounters);
  (void)max_total_tokens;
  if (batch == 0) return MIE_OK;

  const int group = q_heads / kv_heads;
  const bool fast = dtype != MIE_DTYPE_F32 && group <= 8 && kv_heads <= 64 && pages_fit_tma(key_blocks, head_dim, block_size) &&
                    pages_fit_tma(value_blocks, head_dim, block_size) && query.stride[3] == 1 &&
                    out.stride[3] == 1 && query.stride[0] % 2 == 0 && query.stride[1] % 2 == 0 &&
                    out.stride[0] % 2 == 0 && out.stride[1] % 2 == 0 &&
                    (reinterpret_cast<uintptr_t>(query.ptr) & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(out.ptr) & 3) == 0 && scratch != nullptr;
  MIE_CHECK_ARG(out_q8 == nullptr || (out_scales != nullptr && out_scale_ld >= batch &&
                                      ldq8 >= (long long)q_heads * head_dim && head_dim == kHeadDim),
                "the quantised output needs scale storage, a row stride >= q_heads * head_dim and head_dim 128");
  if (!fast) {
    MIE_CHECK_ARG(!plan_only && !use_plan, "work plans exist only for the TMA decode path");
    MIE_CHECK_ARG(out_q8 == nullptr, "the quantised output exists only on the TMA decode path");
    if (dtype == MIE_DTYPE_BF16)
      return launch_generic<__nv_bfloat16>(query, out, key_blocks, value_blocks, block_tables, sequence_lengths,
                                           query_positions, batch, q_heads, kv_heads, head_dim, block_size,
                                           num_blocks, table_width, scale, status, stream);
    if (dtype == MIE_DTYPE_F16)
      return launch_generic<__half>(query, out, key_blocks, value_blocks, block_tables, sequence_lengths,
                                    query_positions, batch, q_heads, kv_heads, head_dim, block_size, num_blocks,
                                    table_width, scale, status, stream);
    return launch_generic<float>(query, out, key_blocks, value_blocks, block_tables, sequence_lengths,
                                 query_positions, batch, q_heads, kv_heads, head_dim, block_size, num_blocks,
                                 table_width, scale, status, stream);
  }

  MIE_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, "scratch must be 256-byte aligned");
  Scratch sc = carve(scratch, scratch_bytes, batch, q_heads, kv_heads, head_dim);
  MIE_CHECK_ARG(sc.cap > batch, "scratch of %lld bytes is too small for batch %d", (long long)scratch_bytes, batch);

  DecodeParams p{View4(query), View4(out), IndexView(block_tables), IndexView(sequence_lengths),
                 IndexView(query_positions), sc, batch, q_heads, kv_heads, group, block_size, num_blocks,
                 table_width, scale * 1.4426950408889634f, plan_slot, status, reinterpret_cast<uint8_t*>(out_q8), ldq8,
                 out_scales, out_scale_ld, 0};
  if (!use_plan) {
    plan_kernel<<<1, plan_threads(batch), 0, stream>>>(p.lengths, p.positions, batch, (long long)table_width * block_size,
                                                kv_heads, split_policy, sm_count() * kWarps, 128, sc, status);
    MIE_LAUNCH_CHECK("plan_kernel");
  }
  if (plan_only) return MIE_OK;

  CUtensorMap kmap, vmap;
  if (int rc = page_tensor_map(key_blocks, num_blocks, kv_heads, block_size, dtype, &kmap)) return rc;
  if (int rc = page_tensor_map(value_blocks, num_blocks, kv_heads, block_size, dtype, &vmap)) return rc;
  if (dtype == MIE_DTYPE_BF16) return launch_fast<__nv_bfloat16>(p, kmap, vmap, stream);
  return launch_fast<__half>(p, kmap, vmap, stream);
}

// ---------------------------------------------------------------------------
// Decode attention over the e4m3 K/V pool
// ---------------------------------------------------------------------------
namespace mie {
namespace {

constexpr size_t kDecodeKv8Smem = (size_t)kWarps8 * kStages8 * kStage8Bytes + kWarps8 * kStages8 * 8 +
                                  (size_t)kWarps8 * kPidBatch * 4 + 1024;

struct Kv8MapKey {
  const void* ptr;
  long long page_stride;
  int num_blocks, kv_heads;
  bool operator==(const Kv8MapKey& o) const {
    return ptr == o.ptr && page_stride == o.page_stride && num_blocks == o.num_blocks && kv_heads == o.kv_heads;
  }
};
struct Kv8MapHash {
  size_t operator()(const Kv8MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ (size_t)k.page_stride;
    h = h * 1000003u ^ (size_t)(k.num_blocks * 131 + k.kv_heads);
    return h;
  }
};

// 5-D byte map over [pages][kv_heads][2][16][128]; one box = K and V rows of one (page, head) = 4 KiB.
int kv8_tensor_map(const void* pool, long long page_stride, int num_blocks, int kv_heads, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<Kv8MapKey, CUtensorMap, Kv8MapHash> cache;
  Kv8MapKey key{pool, page_stride, num_blocks, kv_heads};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MIE_OK;
    }
  }
  const uint64_t dims[5] = {(uint64_t)kHeadDim, (uint64_t)kTileTokens, 2, (uint64_t)kv_heads, (uint64_t)num_blocks};
  const uint64_t strides[4] = {(uint64_t)kHeadDim, (uint64_t)kTile8Bytes, (uint64_t)(2 * kTile8Bytes),
                               (uint64_t)page_stride};
  const uint32_t box[5] = {(uint32_t)kHeadDim, (uint32_t)kTileTokens, 2, 1, 1};
  const int rc = make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<void*>(pool), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MIE_OK) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return MIE_OK;
}

template <typename T>
int launch_kv8(const DecodeParams& p, const Kv8Params& kv, const CUtensorMap& kvmap, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MIE_CUDA(cudaFuncSetAttribute(decode_kv8_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kDecodeKv8Smem));
    configured[dev] = true;
  }
  MIE_CUDA(launch_chained(decode_kv8_kernel<T>, dim3(sm_count()), dim3(kWarps8 * 32), kDecodeKv8Smem, stream, kvmap, p,
                          kv));
  MIE_LAUNCH_CHECK("decode_kv8_kernel");
  for (int g0 = 0; g0 < p.group; g0 += kMaxGroupMerge) {
    DecodeParams q = p;
    q.merge_head0 = g0;
    const int heads = p.group - g0 < kMaxGroupMerge ? p.group - g0 : kMaxGroupMerge;
    if (int rc = launch_merge<T>(q, heads, stream)) return rc;
  }
  return MIE_OK;
}

}  // namespace
}  // namespace mie

extern "C" int mie_paged_decode_attention_kv8(mie_view4_t query, mie_view4_t out, const void* kv_pool,
                                              int64_t page_stride_bytes, const float* kv_scales,
                                              mie_index_t block_tables, mie_index_t sequence_lengths,
                                              mie_index_t query_positions, int32_t batch, int32_t q_heads,
                                              int32_t kv_heads, int32_t num_blocks, int32_t table_width,
                                              int32_t dtype, float scale, int32_t split_policy, void* scratch,
                                              int64_t scratch_bytes, int32_t plan_only, int32_t use_plan,
                                              int32_t plan_slot, void* out_q8, int64_t ldq8, float* out_scales,
                                              int32_t out_scale_ld, int32_t* status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MIE_CHECK_ARG(batch >= 0 && q_heads >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0 && kv_heads <= 64,
                "query heads (%d) must be a positive multiple of KV heads (%d)", q_heads, kv_heads);
  MIE_CHECK_ARG(q_heads / kv_heads <= 8, "at most 8 query heads per KV head");
  MIE_CHECK_ARG(num_blocks >= 1 && table_width >= 1, "invalid page geometry");
  MIE_CHECK_ARG(dtype == MIE_DTYPE_BF16 || dtype == MIE_DTYPE_F16, "query / output must be bf16 or fp16");
  MIE_CHECK_ARG(query.ptr && out.ptr && kv_pool && kv_scales && block_tables.ptr && sequence_lengths.ptr && scratch,
                "null pointer");
  MIE_CHECK_ARG(split_policy >= 0, "split_policy must be >= 0");
  MIE_CHECK_ARG(plan_slot >= 0 && plan_slot < kCounters, "plan_slot must be in [0, %d)", kCounters);
  MIE_CHECK_ARG(page_stride_bytes >= (long long)kv_heads * 2 * kTile8Bytes && page_stride_bytes % 16 == 0 &&
                    (reinterpret_cast<uintptr_t>(kv_pool) & 1023) == 0 &&
                    (reinterpret_cast<uintptr_t>(kv_scales) & 127) == 0,
                "the e4m3 pool must be 1 KiB aligned with a page stride of at least kv_heads * 4096 bytes, "
                "the scales 128-byte aligned");
  MIE_CHECK_ARG(query.stride[3] == 1 && out.stride[3] == 1 && query.stride[0] % 4 == 0 && query.stride[1] % 4 == 0 &&
                    out.stride[0] % 4 == 0 && out.stride[1] % 4 == 0 &&
                    (reinterpret_cast<uintptr_t>(query.ptr) & 7) == 0 && (reinterpret_cast<uintptr_t>(out.ptr) & 7) == 0,
                "query / output rows must be contiguous in head_dim and 8-byte aligned");
  MIE_CHECK_ARG(out_q8 == nullptr || (out_scales != nullptr && out_scale_ld >= batch &&
                                      ldq8 >= (long long)q_heads * kHeadDim),
                "the quantised output needs scale storage and a row stride >= q_heads * 128");
  MIE_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, "scratch must be 256-byte aligned");
  if (batch == 0) return MIE_OK;
  Scratch sc = carve(scratch, scratch_bytes, batch, q_heads, kv_heads, kHeadDim);
  MIE_CHECK_ARG(sc.cap > batch, "scratch of %lld bytes is too small for batch %d", (long long)scratch_bytes, batch);

  DecodeParams p{View4(query), View4(out), IndexView(block_tables), IndexView(sequence_lengths),
                 IndexView(query_positions), sc, batch, q_heads, kv_heads, q_heads / kv_heads, kTileTokens, num_blocks,
                 table_width, scale * 1.4426950408889634f, plan_slot, status, reinterpret_cast<uint8_t*>(out_q8), ldq8,
                 out_scales, out_scale_ld, 0};
  if (!use_plan) {
    plan_kernel<<<1, plan_threads(batch), 0, stream>>>(p.lengths, p.positions, batch, (long long)table_width * kTileTokens,
                                                kv_heads, split_policy, sm_count() * kWarps8, 256, sc, status);
    MIE_LAUNCH_CHECK("plan_kernel");
  }
  if (plan_only) return MIE_OK;
  CUtensorMap kvmap;
  if (int rc = kv8_tensor_map(kv_pool, page_stride_bytes, num_blocks, kv_heads, &kvmap)) return rc;
  Kv8Params kv{kv_scales};
  if (dtype == MIE_DTYPE_BF16) return launch_kv8<__nv_bfloat16>(p, kv, kvmap, stream);
  return launch_kv8<__half>(p, kv, kvmap, stream);
}

// ---------------------------------------------------------------------------
// Decode attention with built-in scratch (no allocation anywhere on the path)
// ---------------------------------------------------------------------------
namespace mie {
namespace {

// The work plan and split-KV partials of mie_paged_decode_attention_static live here instead of in a
// buffer from the caller.  16 MiB per GPU that loads this library, held until the process exits.
constexpr long long kBuiltinScratchBytes = 16ll << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// In host code `g_builtin_scratch` is only a handle for the runtime, not a device address: the address
// has to be asked for, once per device, while that device is current.
int builtin_scratch_address(void** out) {
  static void* cached[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  MIE_CUDA(cudaGetDevice(&dev));
  MIE_CHECK_ARG(dev >= 0 && dev < 64, "device index %d is outside the supported range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* address = nullptr;
    MIE_CUDA(cudaGetSymbolAddress(&address, g_builtin_scratch));
    MIE_CHECK_ARG(address != nullptr, "the built-in decode scratch has no address on device %d", dev);
    cached[dev] = address;
  }
  *out = cached[dev];
  return MIE_OK;
}

}  // namespace
}  // namespace mie

extern "C" int64_t mie_decode_builtin_scratch_bytes(void) { return mie::kBuiltinScratchBytes; }

extern "C" int mie_paged_decode_attention_static(mie_view4_t query, mie_view4_t out, mie_view4_t key_blocks,
                                                 mie_view4_t value_blocks, mie_index_t block_tables,
                                                 mie_index_t sequence_lengths, mie_index_t query_positions,
                                                 int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                                 int32_t block_size, int32_t num_blocks, int32_t table_width,
                                                 int32_t dtype, float scale, int32_t split_policy,
                                                 int64_t max_total_tokens, int32_t* status, void* stream) {
  MIE_CHECK_ARG(batch >= 0 && q_heads >= 1 && kv_heads >= 1 && head_dim >= 1 && max_total_tokens >= 0,
                "invalid decode shape");
  const long long needed = mie_decode_scratch_bytes(batch, q_heads, kv_heads, head_dim, max_total_tokens);
  MIE_CHECK_ARG(needed > 0 && needed <= mie::kBuiltinScratchBytes,
                "this batch needs %lld bytes of decode scratch but the built-in buffer holds %lld: lower batch / "
                "max_total_tokens or call mie_paged_decode_attention with a buffer of your own",
                needed, mie::kBuiltinScratchBytes);
  void* scratch = nullptr;
  if (int rc = mie::builtin_scratch_address(&scratch)) return rc;
  return mie_paged_decode_attention(query, out, key_blocks, value_blocks, block_tables, sequence_lengths,
                                    query_positions, batch, q_heads, kv_heads, head_dim, block_size, num_blocks,
                                    table_width, dtype, scale, split_policy, max_total_tokens, scratch,
                                    mie::kBuiltinScratchBytes, /*plan_only=*/0, /*use_plan=*/0, /*plan_slot=*/0,
                                    /*out_q8=*/nullptr, 0, /*out_scales=*/nullptr, 0, status, stream);
}

