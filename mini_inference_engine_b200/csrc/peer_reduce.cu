// Tensor-parallel exchange fused into the residual add + RMSNorm (+ e4m3 quantisation) that follows the
// row-parallel projections (o_proj, down_proj).
//
// Every rank holds its projection's partial sums [rows, cols] in a buffer the other ranks have mapped
// (CUDA IPC, peer access over NVLink).  Instead of an all-reduce followed by a norm kernel, ONE kernel per
// rank
//   1. tells the peers "my partial sums are complete" and waits for theirs (epoch flags in peer memory),
//   2. for the rows this rank owns (a contiguous slice of the batch) loads the partial rows of all ranks
//      with plain peer loads, sums them in fp32 in rank order, rounds once to bf16 (the all-reduced
//      value), adds the residual, normalises, and
//   3. stores the result the next column-parallel GEMM needs - e4m3 rows + per-128 scales, or bf16 rows -
//      straight into every rank's input buffer (peer stores), then
//   4. counts each finished row into the peers' "rows landed" counters (one remote atomic per CTA and peer,
//      after a system-scope fence) and waits until its own counter shows every peer's rows.
// The residual stream stays sharded by rows (a rank only ever updates the rows it owns), so the wire
// carries (tp-1)/tp of the partial sums once plus the 1-byte activations, about half of what a bf16
// all-reduce moves, and the separate norm/quantise launch disappears.
//
// No multimem / NVLS and no TMA: plain ld/st to peer addresses.  Both waits are bounded; a wait that runs
// out sets MIE_STATUS_WAIT_TIMEOUT and the kernel carries on to its normal exit (results are then
// undefined, the context stays usable).
#include <cstring>

#include "common.cuh"
#include "glue.cuh"

namespace mie {
namespace {

constexpr int kMaxRanks = MIE_TP_MAX_RANKS;

struct PeerReduceParams {
  const __nv_bfloat16* partial[kMaxRanks];
  uint8_t* q[kMaxRanks];
  float* scales[kMaxRanks];
  __nv_bfloat16* normed[kMaxRanks];
  unsigned* flags[kMaxRanks];  // rank r's flag block: [0..8) "partial ready" epochs, [8] count of rows landed
  unsigned* state;             // local: [0] last finished epoch, [1] CTA arrival counter, [2] rows landed so far
  const __nv_bfloat16* residual;
  __nv_bfloat16* summed;
  const __nv_bfloat16* weight;
  long long ld_partial, ldq;
  int scale_ld;
  int tp, rank, rows, cols, row_begin, row_count;
  float eps;
  int* status;
  unsigned max_polls;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Peer data written before the flag we acquired: read it past any stale L1 line.
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Epochs only grow; the signed difference keeps the comparison valid across the 2^32 wrap.
__device__ __forceinline__ bool wait_epoch(const unsigned* flag, unsigned epoch, unsigned max_polls) {
  for (unsigned i = 0; i < max_polls; ++i) {
    if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (i > 4096) __nanosleep(128);  // a late peer: stop hammering the memory system
  }
  return false;
}
__device__ __forceinline__ void red_add_sys(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(1024) peer_reduce_norm_kernel(PeerReduceParams p) {
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  chain_wait();  // the projection before this kernel has finished: its partial sums are complete
  chain_release();
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(p.state) + 1;

  // ---- 1. my partial sums are complete (this kernel follows the GEMM in stream order); wait for the peers' ----
  if (blockIdx.x == 0 && tid < p.tp && tid != p.rank) st_release_sys(p.flags[tid] + p.rank, epoch);
  bool ok = true;
  if (tid < p.tp && tid != p.rank) ok = wait_epoch(p.flags[p.rank] + tid, epoch, p.max_polls);
  if (!__syncthreads_and(ok ? 1 : 0) && tid == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);

  // ---- 2. + 3. reduce, add, normalise and scatter the rows this rank owns ----
  if ((int)blockIdx.x < p.row_count) {
    const long long row = p.row_begin + blockIdx.x;
    const int c0 = tid * 8;
    const bool active = c0 < p.cols;
    float v[8];
    float ss = 0.f;
    if (active) {
      // All ranks' loads are issued before the first one is used: one NVLink round trip, not tp of them.
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < p.tp) raw[r] = ld_volatile_v4(p.partial[r] + row * p.ld_partial + c0);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < p.tp) {
          float part[8];
          unpack8(raw[r], part);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += part[j];
        }
      }
      float res[8];
      unpack8(*reinterpret_cast<const uint4*>(p.residual + row * p.cols + c0), res);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = round_bf16(round_bf16(acc[j]) + res[j]);
      *reinterpret_cast<uint4*>(p.summed + row * p.cols + c0) = pack8(v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.f;
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 0; w < warps; ++w) total += red[w];
    const float inv = rsqrtf(total / (float)p.cols + p.eps);
    float w8[8];
    if (active) unpack8(*reinterpret_cast<const uint4*>(p.weight + c0), w8);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = active ? round_bf16(w8[j] * round_bf16(v[j] * inv)) : 0.f;
    if (p.normed[0] != nullptr) {
      if (active) {
        const uint4 raw = pack8(v);
        for (int r = 0; r < p.tp; ++r) *reinterpret_cast<uint4*>(p.normed[r] + row * p.cols + c0) = raw;
      }
    }
    if (p.q[0] != nullptr) {
      // Lanes past the row end (cols is a multiple of 128 here) hold zeros and write nothing.
      uint32_t packed[2];
      float scale;
      quantize_group(v, packed, scale);
      if (active) {
        const uint2 raw = make_uint2(packed[0], packed[1]);
        for (int r = 0; r < p.tp; ++r) {
          *reinterpret_cast<uint2*>(p.q[r] + row * p.ldq + c0) = raw;
          if ((tid & 15) == 0) p.scales[r][(long long)(c0 / 128) * p.scale_ld + row] = scale;
        }
      }
    }
  }

  // ---- 4. this CTA's row has been stored everywhere: count it into every peer's "rows landed" counter ----
  __syncthreads();
  if ((int)blockIdx.x < p.row_count && tid < p.tp && tid != p.rank) {
    __threadfence_system();  // the CTA's peer stores (ordered before the barrier) are performed first
    red_add_sys(p.flags[tid] + kMaxRanks, 1u);
  }
  // CTA 0 waits until the rows of all peers have landed here; the kernel (and with it the stream) only
  // moves on after that.
  if (blockIdx.x == 0) {
    const unsigned expected = *reinterpret_cast<volatile unsigned*>(p.state + 2) + (unsigned)(p.rows - p.row_count);
    ok = true;
    if (tid == 0) ok = wait_epoch(p.flags[p.rank] + kMaxRanks, expected, p.max_polls);
    if (!__syncthreads_and(ok ? 1 : 0) && tid == 0) raise_status(p.status, MIE_STATUS_WAIT_TIMEOUT);
  }
  // The last CTA to leave advances the local state for the next call (nobody reads it any more).
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.state + 1, 1u) == gridDim.x - 1) {
      p.state[1] = 0;
      p.state[0] = epoch;
      p.state[2] += (unsigned)(p.rows - p.row_count);
    }
  }
}

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetAddressRangeFn>(ptr);
    looked = true;
  }
  return fn;
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_ipc_export(const void* ptr, uint8_t* handle, int64_t* offset) {
  MIE_CHECK_ARG(ptr && handle && offset, "null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == MIE_IPC_HANDLE_BYTES, "IPC handle size");
  GetAddressRangeFn range = address_range_fn();
  if (range == nullptr) {
    set_error("cuMemGetAddressRange is not available from the CUDA driver");
    return MIE_ERR_CUDA;
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) {
    set_error("cuMemGetAddressRange failed with CUresult %d for %p", (int)r, ptr);
    return MIE_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  MIE_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle, &h, sizeof(h));
  *offset = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return MIE_OK;
}

extern "C" int mie_ipc_open(const uint8_t* handle, int64_t offset, void** mapped) {
  MIE_CHECK_ARG(handle && mapped && offset >= 0, "null pointer or negative offset");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  MIE_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *mapped = reinterpret_cast<char*>(base) + offset;
  return MIE_OK;
}

extern "C" int mie_ipc_close(void* mapped, int64_t offset) {
  MIE_CHECK_ARG(mapped && offset >= 0, "null pointer or negative offset");
  MIE_CUDA(cudaIpcCloseMemHandle(reinterpret_cast<char*>(mapped) - offset));
  return MIE_OK;
}

extern "C" int mie_tp_reduce_rms_norm(const mie_tp_peers_t* peers, int32_t tp, int32_t rank, int64_t ld_partial,
                                      const void* residual, void* summed, const void* weight, int64_t ldq,
                                      int32_t scale_ld, int32_t rows, int32_t cols, float eps, uint32_t* state,
                                      uint32_t max_polls, int32_t* status, void* stream) {
  MIE_CHECK_ARG(peers && residual && summed && weight && state, "null pointer");
  MIE_CHECK_ARG(tp >= 1 && tp <= kMaxRanks && rank >= 0 && rank < tp, "rank %d of %d is out of range", rank, tp);
  MIE_CHECK_ARG(rows >= 0 && cols >= 8 && cols % 8 == 0 && cols <= 8192 && ld_partial % 8 == 0 && ld_partial >= cols,
                "cols must be a multiple of 8 up to 8192 and partial rows 16-byte aligned");
  const bool want_q = peers->q[0] != nullptr, want_normed = peers->normed[0] != nullptr;
  MIE_CHECK_ARG(want_q || want_normed, "no output requested");
  MIE_CHECK_ARG(!want_q || (cols % 128 == 0 && scale_ld >= rows && ldq >= cols && ldq % 8 == 0),
                "quantised output needs cols %% 128 == 0 and scale storage");
  PeerReduceParams p;
  for (int r = 0; r < kMaxRanks; ++r) {
    const bool live = r < tp;
    MIE_CHECK_ARG(!live || (peers->partial[r] && peers->flags[r]), "rank %d: null partial or flag pointer", r);
    MIE_CHECK_ARG(!live || !want_q || (peers->q[r] && peers->scales[r]), "rank %d: null quantised output", r);
    MIE_CHECK_ARG(!live || !want_normed || peers->normed[r], "rank %d: null bf16 output", r);
    MIE_CHECK_ARG(!live || ((reinterpret_cast<uintptr_t>(peers->partial[r]) | reinterpret_cast<uintptr_t>(peers->q[r]) |
                             reinterpret_cast<uintptr_t>(peers->normed[r])) & 15) == 0,
                  "rank %d: buffers must be 16-byte aligned", r);
    p.partial[r] = live ? (const __nv_bfloat16*)peers->partial[r] : nullptr;
    p.q[r] = live && want_q ? (uint8_t*)peers->q[r] : nullptr;
    p.scales[r] = live && want_q ? peers->scales[r] : nullptr;
    p.normed[r] = live && want_normed ? (__nv_bfloat16*)peers->normed[r] : nullptr;
    p.flags[r] = live ? peers->flags[r] : nullptr;
  }
  MIE_CHECK_ARG(((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(summed) |
                  reinterpret_cast<uintptr_t>(weight)) & 15) == 0, "rows must be 16-byte aligned");
  const int per_rank = (rows + tp - 1) / tp;
  const int begin = per_rank * rank < rows ? per_rank * rank : rows;
  const int end = begin + per_rank < rows ? begin + per_rank : rows;
  p.state = state;
  p.residual = (const __nv_bfloat16*)residual;
  p.summed = (__nv_bfloat16*)summed;
  p.weight = (const __nv_bfloat16*)weight;
  p.ld_partial = ld_partial;
  p.ldq = ldq;
  p.scale_ld = scale_ld;
  p.tp = tp;
  p.rank = rank;
  p.rows = rows;
  p.cols = cols;
  p.row_begin = begin;
  p.row_count = end - begin;
  p.eps = eps;
  p.status = status;
  p.max_polls = max_polls == 0 ? (1u << 22) : max_polls;
  const int threads = ((cols / 8) + 31) / 32 * 32;
  const int blocks = p.row_count > 0 ? p.row_count : 1;  // a rank without rows still takes part in both waits
  MIE_CUDA(launch_chained(peer_reduce_norm_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, p));
  MIE_LAUNCH_CHECK("peer_reduce_norm_kernel");
  return MIE_OK;
}
