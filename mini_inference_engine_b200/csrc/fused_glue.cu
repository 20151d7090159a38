// Memory-bound glue between the projections: RMSNorm (plain, per-head strided,
// fused with the residual add), SiLU(gate) * up, rotate-half RoPE, and the
// decode-step fusion of q/k-norm + RoPE + KV-cache write.  Each kernel makes one
// pass over HBM with 16-byte accesses and keeps the bf16 rounding points where
// the unfused PyTorch ops round (fp32 math in between).  The norm and SiLU
// kernels can also emit the e4m3 activation + per-128 scales that the next FP8
// GEMM consumes, which removes the separate quantiser pass.
#include "common.cuh"
#include "glue.cuh"

namespace mie {
namespace {

// ---------------------------------------------------------------------------
// Row RMSNorm: one CTA per row, cols a multiple of 8 (<= 8 * 1024).
// ---------------------------------------------------------------------------
struct RowNormParams {
  const __nv_bfloat16* x;
  long long ldx;
  const __nv_bfloat16* residual;  // optional, contiguous rows of `cols`
  __nv_bfloat16* summed;          // optional: x + residual
  const __nv_bfloat16* weight;
  __nv_bfloat16* out;             // optional when only the quantised form is wanted
  uint8_t* q;                     // optional e4m3 output, row stride ldq
  long long ldq;
  float* scales;                  // [cols / 128][scale_ld]
  int scale_ld;
  int rows, cols;
  float eps;
};

__global__ void __launch_bounds__(1024) row_norm_kernel(RowNormParams p) {
  __shared__ float red[32];
  chain_wait();
  chain_release();
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c0 = tid * 8;
  const bool active = c0 < p.cols;
  float v[8];
  float ss = 0.f;
  if (active) {
    unpack8(*reinterpret_cast<const uint4*>(p.x + (long long)row * p.ldx + c0), v);
    if (p.residual != nullptr) {
      float r[8];
      unpack8(*reinterpret_cast<const uint4*>(p.residual + (long long)row * p.cols + c0), r);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] + r[j]);
      if (p.summed != nullptr) *reinterpret_cast<uint4*>(p.summed + (long long)row * p.cols + c0) = pack8(v);
    }
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
  if (active && p.out != nullptr) *reinterpret_cast<uint4*>(p.out + (long long)row * p.cols + c0) = pack8(v);
  if (p.q != nullptr) {
    // Lanes past the row end (cols is a multiple of 128 here) hold zeros and write nothing.
    quantize_group_store(v, active ? p.q + (long long)row * p.ldq + c0 : nullptr,
                         active ? p.scales + (long long)(c0 / 128) * p.scale_ld + row : nullptr, (tid & 15) == 0);
  }
}

// ---------------------------------------------------------------------------
// Head RMSNorm: width 128, 16 lanes per (row, head); rows addressed by strides.
// ---------------------------------------------------------------------------
__global__ void head_norm_kernel(const __nv_bfloat16* x, long long outer_stride, long long head_stride, int heads,
                                 const __nv_bfloat16* weight, __nv_bfloat16* out, long long rows_total, float eps) {
  const long long hw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const int l16 = threadIdx.x & 15;
  const bool live = hw < rows_total;
  const long long r = live ? hw : 0;
  const __nv_bfloat16* src = x + (r / heads) * outer_stride + (r % heads) * head_stride + l16 * 8;
  float v[8];
  unpack8(*reinterpret_cast<const uint4*>(src), v);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / 128.f + eps);
  float w8[8];
  unpack8(*reinterpret_cast<const uint4*>(weight + l16 * 8), w8);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = round_bf16(w8[j] * round_bf16(v[j] * inv));
  if (live) *reinterpret_cast<uint4*>(out + r * 128 + l16 * 8) = pack8(v);
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up, optional fused quantisation.  One thread per 8 columns.
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __nv_bfloat16* gate, const __nv_bfloat16* up, long long ld_in,
                                __nv_bfloat16* out, uint8_t* q, long long ldq, float* scales, int scale_ld,
                                int rows, int cols) {
  chain_wait();
  chain_release();
  const int per_row = cols / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < (long long)rows * per_row;
  const int row = live ? (int)(idx / per_row) : 0, c0 = live ? (int)(idx % per_row) * 8 : 0;
  float g[8], u[8], v[8];
  if (live) {
    unpack8(*reinterpret_cast<const uint4*>(gate + (long long)row * ld_in + c0), g);
    unpack8(*reinterpret_cast<const uint4*>(up + (long long)row * ld_in + c0), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = round_bf16(round_bf16(g[j] / (1.f + expf(-g[j]))) * u[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  if (live && out != nullptr) *reinterpret_cast<uint4*>(out + (long long)row * cols + c0) = pack8(v);
  if (q != nullptr) {
    quantize_group_store(v, live ? q + (long long)row * ldq + c0 : nullptr,
                         live ? scales + (long long)(c0 / 128) * scale_ld + row : nullptr,
                         (threadIdx.x & 15) == 0);
  }
}

// ---------------------------------------------------------------------------
// RoPE on [B, H, T, D] (D <= 256, even): one warp per (b, h, t) row.
// ---------------------------------------------------------------------------
__global__ void rope_kernel(const __nv_bfloat16* x, long long sb, long long sh, long long st,
                            const __nv_bfloat16* cos, const __nv_bfloat16* sin, long long cs_b, long long cs_t,
                            __nv_bfloat16* out, long long ob, long long oh, long long ot, int heads, int seq,
                            int dim, long long rows_total) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows_total) return;
  const int t = (int)(warp % seq), h = (int)((warp / seq) % heads);
  const long long b = warp / ((long long)seq * heads);
  const __nv_bfloat16* src = x + b * sb + h * sh + t * st;
  const __nv_bfloat16* c = cos + b * cs_b + t * cs_t;
  const __nv_bfloat16* s = sin + b * cs_b + t * cs_t;
  __nv_bfloat16* dst = out + b * ob + h * oh + t * ot;
  const int half = dim / 2;
  for (int i = lane; i < half; i += 32) {
    const float x1 = __bfloat162float(src[i]), x2 = __bfloat162float(src[i + half]);
    const float o1 = round_bf16(x1 * __bfloat162float(c[i])) + round_bf16(-x2 * __bfloat162float(s[i]));
    const float o2 =
        round_bf16(x2 * __bfloat162float(c[i + half])) + round_bf16(x1 * __bfloat162float(s[i + half]));
    dst[i] = __float2bfloat16_rn(o1);
    dst[i + half] = __float2bfloat16_rn(o2);
  }
}

// ---------------------------------------------------------------------------
// q/k RMSNorm + RoPE + KV-cache write over a merged qkv row (head_dim 128).
// One warp per (token, head); lanes hold 4 consecutive dims, partner dims
// (d +/- 64) sit 16 lanes away.
// ---------------------------------------------------------------------------
struct QkvParams {
  const __nv_bfloat16* qkv;  // [tokens][ld]: q heads | k heads | v heads
  long long ld;
  const __nv_bfloat16* q_weight;
  const __nv_bfloat16* k_weight;
  const __nv_bfloat16* cos_sin;  // [max_pos][2][128]: cos row then sin row
  int max_pos;
  IndexView positions;           // [tokens]
  IndexView token_to_sequence;   // [tokens] or null (token t belongs to sequence t)
  IndexView tables;              // [sequences][width]
  __nv_bfloat16* q_out;          // [tokens][q_heads][128]
  char* key_blocks;
  char* value_blocks;
  long long kb_s[3], vb_s[3];    // page, head, token strides (elements)
  int tokens, q_heads, kv_heads, block_size, num_blocks, table_rows, table_width;
  float eps;
  int* status;
  // e4m3 K/V pool [pages][kv_heads][2][16][128] with scales [pages][kv_heads][2][16] (block_size 16), or null.
  uint8_t* kv8_pool;
  long long kv8_page_stride;  // bytes
  float* kv8_scales;
};

__global__ void qkv_post_kernel(QkvParams p) {
  chain_wait();
  chain_release();
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads_total = p.q_heads + 2 * p.kv_heads;
  if (warp >= (long long)p.tokens * heads_total) return;
  const int t = (int)(warp / heads_total), h = (int)(warp % heads_total);
  const long long pos = p.positions.at(t);
  const long long seq = p.token_to_sequence.valid() ? p.token_to_sequence.at(t) : t;
  const bool is_q = h < p.q_heads, is_v = h >= p.q_heads + p.kv_heads;
  const __nv_bfloat16* src = p.qkv + (long long)t * p.ld + (long long)h * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  uint2 result = raw;
  if (!is_v) {
    const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(pr[0]), b2 = __bfloat1622float2(pr[1]);
    float v[4] = {a.x, a.y, b2.x, b2.y};
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 128.f + p.eps);
    const uint2 wraw = *reinterpret_cast<const uint2*>((is_q ? p.q_weight : p.k_weight) + lane * 4);
    const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wraw);
    const float2 w0 = __bfloat1622float2(pw[0]), w1 = __bfloat1622float2(pw[1]);
    const float w[4] = {w0.x, w0.y, w1.x, w1.y};
    const long long cpos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
    if (pos < 0 || pos >= p.max_pos) {
      if (lane == 0) raise_status(p.status, MIE_STATUS_BAD_POSITION);
    }
    const __nv_bfloat16* cs = p.cos_sin + cpos * 256 + lane * 4;
    const uint2 craw = *reinterpret_cast<const uint2*>(cs), sraw = *reinterpret_cast<const uint2*>(cs + 128);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&craw);
    const __nv_bfloat162* ps = reinterpret_cast<const __nv_bfloat162*>(&sraw);
    const float2 c0 = __bfloat1622float2(pc[0]), c1 = __bfloat1622float2(pc[1]);
    const float2 s0 = __bfloat1622float2(ps[0]), s1 = __bfloat1622float2(ps[1]);
    const float c[4] = {c0.x, c0.y, c1.x, c1.y}, s[4] = {s0.x, s0.y, s1.x, s1.y};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float n = round_bf16(w[j] * round_bf16(v[j] * inv));
      const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
      const float rot = lane < 16 ? -partner : partner;  // rotate_half: (-x2, x1)
      o[j] = round_bf16(n * c[j]) + round_bf16(rot * s[j]);
    }
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&result);
    po[0] = __floats2bfloat162_rn(o[0], o[1]);
    po[1] = __floats2bfloat162_rn(o[2], o[3]);
  }
  if (is_q) {
    *reinterpret_cast<uint2*>(p.q_out + ((long long)t * p.q_heads + h) * 128 + lane * 4) = result;
    return;
  }
  // K or V row -> its page slot.
  if (seq < 0 || seq >= p.table_rows) {
    if (lane == 0) raise_status(p.status, MIE_STATUS_BAD_SEQUENCE);
    return;
  }
  if (pos < 0 || pos >= (long long)p.table_width * p.block_size) {
    if (lane == 0) raise_status(p.status, MIE_STATUS_BAD_POSITION);
    return;
  }
  const long long page = p.tables.at(seq, pos / p.block_size);
  if (page < 0 || page >= p.num_blocks) {
    if (lane == 0) raise_status(p.status, MIE_STATUS_BAD_PAGE);
    return;
  }
  const int kvh = is_v ? h - p.q_heads - p.kv_heads : h - p.q_heads;
  if (p.kv8_pool != nullptr) {
    // One scale per (token, KV head): amax of the 128 bf16 values / 448, the row divided by it and rounded
    // to e4m3 (the activation quantiser's rule).
    const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&result);
    const float2 a = __bfloat1622float2(pv[0]), b2 = __bfloat1622float2(pv[1]);
    const float amax = warp_max(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b2.x), fabsf(b2.y))));
    const float scale = __fdiv_rn(amax, 448.0f), denom = fmaxf(scale, 1e-12f);
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(a.x, denom), __fdiv_rn(a.y, denom)), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(b2.x, denom), __fdiv_rn(b2.y, denom)), __NV_SATFINITE, __NV_E4M3);
    const int slot = (int)(pos % p.block_size);
    uint8_t* row = p.kv8_pool + page * p.kv8_page_stride + ((long long)kvh * 2 + (is_v ? 1 : 0)) * 2048 + slot * 128;
    *reinterpret_cast<uint32_t*>(row + lane * 4) = (uint32_t)lo | ((uint32_t)hi << 16);
    if (lane == 0) p.kv8_scales[((page * p.kv_heads + kvh) * 2 + (is_v ? 1 : 0)) * 16 + slot] = scale;
    return;
  }
  const long long* st = is_v ? p.vb_s : p.kb_s;
  char* base = is_v ? p.value_blocks : p.key_blocks;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(base) + page * st[0] + (long long)kvh * st[1] +
                       (pos % p.block_size) * st[2] + lane * 4;
  *reinterpret_cast<uint2*>(dst) = result;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_rms_norm(const void* x, int64_t ldx, const void* residual, void* summed, const void* weight,
                            void* out, void* q, int64_t ldq, float* scales, int32_t scale_ld, int32_t rows,
                            int32_t cols, float eps, void* stream) {
  MIE_CHECK_ARG(x && weight && (out || q), "null pointer");
  MIE_CHECK_ARG(rows >= 0 && cols >= 8 && cols % 8 == 0 && cols <= 8192, "cols must be a multiple of 8 in [8, 8192]");
  MIE_CHECK_ARG(ldx % 8 == 0 && aligned16(x) && aligned16(weight) && (!out || aligned16(out)) &&
                    (!residual || aligned16(residual)) && (!summed || aligned16(summed)),
                "rows must be 16-byte aligned");
  MIE_CHECK_ARG(!q || (scales && cols % 128 == 0 && scale_ld >= rows && ldq >= cols && ldq % 8 == 0),
                "fused quantisation needs cols %% 128 == 0 and scale storage");
  if (rows == 0) return MIE_OK;
  RowNormParams p{(const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)residual, (__nv_bfloat16*)summed,
                  (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, (uint8_t*)q, ldq, scales, scale_ld, rows, cols,
                  eps};
  const int threads = ((cols / 8) + 31) / 32 * 32;
  MIE_CUDA(launch_chained(row_norm_kernel, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, p));
  MIE_LAUNCH_CHECK("row_norm_kernel");
  return MIE_OK;
}

extern "C" int mie_head_rms_norm(const void* x, int64_t outer_stride, int64_t head_stride, int32_t heads,
                                 const void* weight, void* out, int64_t rows_total, float eps, void* stream) {
  MIE_CHECK_ARG(x && weight && out && heads >= 1 && rows_total >= 0, "invalid head-norm arguments");
  MIE_CHECK_ARG(outer_stride % 8 == 0 && head_stride % 8 == 0 && aligned16(x) && aligned16(weight) && aligned16(out),
                "head rows must be 16-byte aligned");
  if (rows_total == 0) return MIE_OK;
  const int threads = 256;
  const long long blocks = (rows_total * 16 + threads - 1) / threads;
  head_norm_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, outer_stride, head_stride, heads, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out,
      rows_total, eps);
  MIE_LAUNCH_CHECK("head_norm_kernel");
  return MIE_OK;
}

extern "C" int mie_silu_mul(const void* gate, const void* up, int64_t ld_in, void* out, void* q, int64_t ldq,
                            float* scales, int32_t scale_ld, int32_t rows, int32_t cols, void* stream) {
  MIE_CHECK_ARG(gate && up && (out || q), "null pointer");
  MIE_CHECK_ARG(rows >= 0 && cols >= 8 && cols % 8 == 0 && ld_in % 8 == 0, "cols and row stride must be multiples of 8");
  MIE_CHECK_ARG(aligned16(gate) && aligned16(up) && (!out || aligned16(out)), "rows must be 16-byte aligned");
  MIE_CHECK_ARG(!q || (scales && cols % 128 == 0 && scale_ld >= rows && ldq >= cols && ldq % 8 == 0),
                "fused quantisation needs cols %% 128 == 0 and scale storage");
  if (rows == 0) return MIE_OK;
  const long long work = (long long)rows * (cols / 8);
  const int threads = 256;
  MIE_CUDA(launch_chained(silu_mul_kernel, dim3((unsigned)((work + threads - 1) / threads)), dim3(threads), 0,
                          (cudaStream_t)stream,
      (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, ld_in, (__nv_bfloat16*)out, (uint8_t*)q, ldq, scales,
      scale_ld, rows, cols));
  MIE_LAUNCH_CHECK("silu_mul_kernel");
  return MIE_OK;
}

extern "C" int mie_rope(mie_view4_t x, const void* cos, const void* sin, int64_t cs_batch_stride,
                        int64_t cs_token_stride, mie_view4_t out, int32_t batch, int32_t heads, int32_t seq,
                        int32_t dim, void* stream) {
  MIE_CHECK_ARG(x.ptr && cos && sin && out.ptr, "null pointer");
  MIE_CHECK_ARG(dim >= 2 && dim % 2 == 0 && x.stride[3] == 1 && out.stride[3] == 1, "RoPE needs an even, contiguous head_dim");
  const long long rows = (long long)batch * heads * seq;
  if (rows == 0) return MIE_OK;
  const int threads = 256;
  rope_kernel<<<(unsigned)((rows * 32 + threads - 1) / threads), threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x.ptr, x.stride[0], x.stride[1], x.stride[2], (const __nv_bfloat16*)cos,
      (const __nv_bfloat16*)sin, cs_batch_stride, cs_token_stride, (__nv_bfloat16*)out.ptr, out.stride[0],
      out.stride[1], out.stride[2], heads, seq, dim, rows);
  MIE_LAUNCH_CHECK("rope_kernel");
  return MIE_OK;
}

namespace {

int launch_qkv_post(mie::QkvParams& p, const void* qkv, int64_t ld, const void* q_weight, const void* k_weight,
                    const void* cos_sin, int32_t max_pos, const mie_index_t& positions,
                    const mie_index_t& token_to_sequence, const mie_index_t& block_tables, void* q_out, int32_t tokens,
                    int32_t q_heads, int32_t kv_heads, int32_t block_size, int32_t num_blocks, int32_t table_rows,
                    int32_t table_width, float eps, int32_t* status, void* stream) {
  MIE_CHECK_ARG(qkv && q_weight && k_weight && cos_sin && positions.ptr && block_tables.ptr && q_out, "null pointer");
  MIE_CHECK_ARG(ld % 4 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 7) == 0, "qkv rows must be 8-byte aligned");
  MIE_CHECK_ARG(tokens >= 0 && q_heads >= 1 && kv_heads >= 1 && max_pos >= 1, "invalid shape");
  if (tokens == 0) return MIE_OK;
  p.qkv = (const __nv_bfloat16*)qkv;
  p.ld = ld;
  p.q_weight = (const __nv_bfloat16*)q_weight;
  p.k_weight = (const __nv_bfloat16*)k_weight;
  p.cos_sin = (const __nv_bfloat16*)cos_sin;
  p.max_pos = max_pos;
  p.positions = IndexView(positions);
  p.token_to_sequence = IndexView(token_to_sequence);
  p.tables = IndexView(block_tables);
  p.q_out = (__nv_bfloat16*)q_out;
  p.tokens = tokens;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.table_rows = table_rows;
  p.table_width = table_width;
  p.eps = eps;
  p.status = status;
  const long long warps = (long long)tokens * (q_heads + 2 * kv_heads);
  const int threads = 256;
  MIE_CUDA(launch_chained(qkv_post_kernel, dim3((unsigned)((warps * 32 + threads - 1) / threads)), dim3(threads), 0,
                          (cudaStream_t)stream, p));
  MIE_LAUNCH_CHECK("qkv_post_kernel");
  return MIE_OK;
}

}  // namespace

extern "C" int mie_qkv_norm_rope_write(const void* qkv, int64_t ld, const void* q_weight, const void* k_weight,
                                       const void* cos_sin, int32_t max_pos, mie_index_t positions,
                                       mie_index_t token_to_sequence, mie_index_t block_tables, void* q_out,
                                       mie_view4_t key_blocks, mie_view4_t value_blocks, int32_t tokens,
                                       int32_t q_heads, int32_t kv_heads, int32_t block_size, int32_t num_blocks,
                                       int32_t table_rows, int32_t table_width, float eps, int32_t* status,
                                       void* stream) {
  MIE_CHECK_ARG(key_blocks.ptr && value_blocks.ptr, "null pointer");
  MIE_CHECK_ARG(key_blocks.stride[3] == 1 && value_blocks.stride[3] == 1, "pages must be contiguous in head_dim");
  for (int i = 0; i < 3; ++i) {
    MIE_CHECK_ARG(key_blocks.stride[i] % 4 == 0 && value_blocks.stride[i] % 4 == 0, "page strides must be multiples of 4");
  }
  QkvParams p;
  p.key_blocks = (char*)key_blocks.ptr;
  p.value_blocks = (char*)value_blocks.ptr;
  for (int i = 0; i < 3; ++i) {
    p.kb_s[i] = key_blocks.stride[i];
    p.vb_s[i] = value_blocks.stride[i];
  }
  p.kv8_pool = nullptr;
  p.kv8_page_stride = 0;
  p.kv8_scales = nullptr;
  return launch_qkv_post(p, qkv, ld, q_weight, k_weight, cos_sin, max_pos, positions, token_to_sequence, block_tables,
                         q_out, tokens, q_heads, kv_heads, block_size, num_blocks, table_rows, table_width, eps,
                         status, stream);
}

extern "C" int mie_qkv_norm_rope_write_kv8(const void* qkv, int64_t ld, const void* q_weight, const void* k_weight,
                                           const void* cos_sin, int32_t max_pos, mie_index_t positions,
                                           mie_index_t token_to_sequence, mie_index_t block_tables, void* q_out,
                                           void* kv_pool, int64_t page_stride_bytes, float* kv_scales,
                                           int32_t tokens, int32_t q_heads, int32_t kv_heads, int32_t num_blocks,
                                           int32_t table_rows, int32_t table_width, float eps, int32_t* status,
                                           void* stream) {
  MIE_CHECK_ARG(kv_pool && kv_scales, "null pointer");
  MIE_CHECK_ARG(page_stride_bytes >= (long long)kv_heads * 4096 && page_stride_bytes % 4 == 0 &&
                    (reinterpret_cast<uintptr_t>(kv_pool) & 3) == 0,
                "the e4m3 pool needs a page stride of at least kv_heads * 4096 bytes");
  QkvParams p;
  p.key_blocks = p.value_blocks = nullptr;
  for (int i = 0; i < 3; ++i) p.kb_s[i] = p.vb_s[i] = 0;
  p.kv8_pool = (uint8_t*)kv_pool;
  p.kv8_page_stride = page_stride_bytes;
  p.kv8_scales = kv_scales;
  return launch_qkv_post(p, qkv, ld, q_weight, k_weight, cos_sin, max_pos, positions, token_to_sequence, block_tables,
                         q_out, tokens, q_heads, kv_heads, /*block_size=*/16, num_blocks, table_rows, table_width, eps,
                         status, stream);
}
