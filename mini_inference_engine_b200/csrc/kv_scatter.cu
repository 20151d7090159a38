// KV-cache scatter and block-table gather: pure byte copies addressed through
// the block table.  One warp moves one (token, KV head) row of K and of V with
// 16-byte vector accesses when the rows allow it.
#include "common.cuh"

namespace mie {
namespace {

struct View4 {
  char* ptr;
  long long s[4];
  __host__ View4(const mie_view4_t& v) : ptr(reinterpret_cast<char*>(v.ptr)) {
    for (int i = 0; i < 4; ++i) s[i] = v.stride[i];
  }
};

// Copy one head_dim row. `half` selects which 16 lanes take part (0 or 1) so a
// warp moves the K row and the V row at the same time.
__device__ __forceinline__ void copy_row(const char* src, long long src_last, char* dst, long long dst_last,
                                         int head_dim, int elem_bytes, int lane16) {
  const int row_bytes = head_dim * elem_bytes;
  const bool vec = src_last == 1 && dst_last == 1 && (row_bytes & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec) {
    for (int off = lane16 * 16; off < row_bytes; off += 256) {
      *reinterpret_cast<uint4*>(dst + off) = *reinterpret_cast<const uint4*>(src + off);
    }
  } else if (elem_bytes == 2) {
    for (int d = lane16; d < head_dim; d += 16) {
      reinterpret_cast<uint16_t*>(dst)[(long long)d * dst_last] =
          reinterpret_cast<const uint16_t*>(src)[(long long)d * src_last];
    }
  } else {
    for (int d = lane16; d < head_dim; d += 16) {
      reinterpret_cast<uint32_t*>(dst)[(long long)d * dst_last] =
          reinterpret_cast<const uint32_t*>(src)[(long long)d * src_last];
    }
  }
}

__global__ void write_decode_kv_kernel(View4 ks, View4 vs, IndexView tables, IndexView lengths, IndexView positions,
                                       View4 kb, View4 vb, int batch, int kv_heads, int head_dim, int block_size,
                                       int num_blocks, int table_width, int elem_bytes, int* status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= batch * kv_heads) return;
  const int b = warp / kv_heads;
  const int h = warp % kv_heads;
  const long long len = lengths.at(b);
  const long long pos = positions.valid() ? positions.at(b) : len - 1;
  if (len < 1 || len > (long long)table_width * block_size) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_LENGTH);
    return;
  }
  if (pos < 0 || pos >= len) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_POSITION);
    return;
  }
  const long long page = tables.at(b, pos / block_size);
  if (page < 0 || page >= num_blocks) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_PAGE);
    return;
  }
  const int slot = (int)(pos % block_size);
  const bool is_v = lane >= 16;
  const View4& src = is_v ? vs : ks;
  const View4& dst = is_v ? vb : kb;
  const char* s = src.ptr + ((long long)b * src.s[0] + (long long)h * src.s[1]) * elem_bytes;
  char* d = dst.ptr + (page * dst.s[0] + (long long)h * dst.s[1] + (long long)slot * dst.s[2]) * elem_bytes;
  copy_row(s, src.s[3], d, dst.s[3], head_dim, elem_bytes, lane & 15);
}

__global__ void write_packed_kv_kernel(View4 ks, View4 vs, IndexView tok2seq, IndexView tokpos, IndexView tables,
                                       View4 kb, View4 vb, int tokens, int kv_heads, int head_dim, int block_size,
                                       int num_blocks, int table_rows, int table_width, int elem_bytes,
                                       int* status) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)tokens * kv_heads) return;
  const int t = (int)(warp / kv_heads);
  const int h = (int)(warp % kv_heads);
  const long long seq = tok2seq.at(t);
  const long long pos = tokpos.at(t);
  if (seq < 0 || seq >= table_rows) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_SEQUENCE);
    return;
  }
  if (pos < 0 || pos >= (long long)table_width * block_size) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_POSITION);
    return;
  }
  const long long page = tables.at(seq, pos / block_size);
  if (page < 0 || page >= num_blocks) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_PAGE);
    return;
  }
  const int slot = (int)(pos % block_size);
  const bool is_v = lane >= 16;
  const View4& src = is_v ? vs : ks;
  const View4& dst = is_v ? vb : kb;
  const char* s = src.ptr + ((long long)h * src.s[1] + (long long)t * src.s[2]) * elem_bytes;
  char* d = dst.ptr + (page * dst.s[0] + (long long)h * dst.s[1] + (long long)slot * dst.s[2]) * elem_bytes;
  copy_row(s, src.s[3], d, dst.s[3], head_dim, elem_bytes, lane & 15);
}

__global__ void gather_kv_kernel(View4 kb, View4 vb, IndexView table, char* key_out, char* value_out, int length,
                                 int kv_heads, int head_dim, int block_size, int num_blocks, int elem_bytes,
                                 int* status) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)length * kv_heads) return;
  const int h = (int)(warp / length);
  const int t = (int)(warp % length);
  const long long page = table.at(t / block_size);
  const bool is_v = lane >= 16;
  char* out = (is_v ? value_out : key_out) + ((long long)h * length + t) * head_dim * elem_bytes;
  if (page < 0 || page >= num_blocks) {
    if (lane == 0) raise_status(status, MIE_STATUS_BAD_PAGE);
    return;
  }
  const View4& src = is_v ? vb : kb;
  const char* s =
      src.ptr + (page * src.s[0] + (long long)h * src.s[1] + (long long)(t % block_size) * src.s[2]) * elem_bytes;
  copy_row(s, src.s[3], out, 1, head_dim, elem_bytes, lane & 15);
}

int check_common(int head_dim, int block_size, int num_blocks, int elem_bytes) {
  MIE_CHECK_ARG(elem_bytes == 2 || elem_bytes == 4, "elem_bytes must be 2 or 4, got %d", elem_bytes);
  MIE_CHECK_ARG(head_dim >= 1 && block_size >= 1 && num_blocks >= 1,
                "head_dim, block_size and num_blocks must be positive");
  return MIE_OK;
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_write_decode_kv(mie_view4_t key_states, mie_view4_t value_states, mie_index_t block_tables,
                                   mie_index_t sequence_lengths, mie_index_t query_positions,
                                   mie_view4_t key_blocks, mie_view4_t value_blocks, int32_t batch,
                                   int32_t kv_heads, int32_t head_dim, int32_t block_size, int32_t num_blocks,
                                   int32_t table_width, int32_t elem_bytes, int32_t* status, void* stream) {
  if (int rc = check_common(head_dim, block_size, num_blocks, elem_bytes)) return rc;
  MIE_CHECK_ARG(batch >= 0 && kv_heads >= 1 && table_width >= 1, "invalid batch/kv_heads/table_width");
  MIE_CHECK_ARG(key_states.ptr && value_states.ptr && key_blocks.ptr && value_blocks.ptr && block_tables.ptr &&
                    sequence_lengths.ptr,
                "null tensor pointer");
  if (batch == 0) return MIE_OK;
  const long long warps = (long long)batch * kv_heads;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  write_decode_kv_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      View4(key_states), View4(value_states), IndexView(block_tables), IndexView(sequence_lengths),
      IndexView(query_positions), View4(key_blocks), View4(value_blocks), batch, kv_heads, head_dim, block_size,
      num_blocks, table_width, elem_bytes, status);
  MIE_LAUNCH_CHECK("write_decode_kv_kernel");
  return MIE_OK;
}

extern "C" int mie_write_packed_kv(mie_view4_t key_states, mie_view4_t value_states, mie_index_t token_to_sequence,
                                   mie_index_t token_positions, mie_index_t block_tables, mie_view4_t key_blocks,
                                   mie_view4_t value_blocks, int32_t tokens, int32_t kv_heads, int32_t head_dim,
                                   int32_t block_size, int32_t num_blocks, int32_t table_rows, int32_t table_width,
                                   int32_t elem_bytes, int32_t* status, void* stream) {
  if (int rc = check_common(head_dim, block_size, num_blocks, elem_bytes)) return rc;
  MIE_CHECK_ARG(tokens >= 0 && kv_heads >= 1 && table_rows >= 1 && table_width >= 1,
                "invalid tokens/kv_heads/table shape");
  MIE_CHECK_ARG(key_states.ptr && value_states.ptr && key_blocks.ptr && value_blocks.ptr && block_tables.ptr &&
                    token_to_sequence.ptr && token_positions.ptr,
                "null tensor pointer");
  if (tokens == 0) return MIE_OK;
  const long long warps = (long long)tokens * kv_heads;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  write_packed_kv_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      View4(key_states), View4(value_states), IndexView(token_to_sequence), IndexView(token_positions),
      IndexView(block_tables), View4(key_blocks), View4(value_blocks), tokens, kv_heads, head_dim, block_size,
      num_blocks, table_rows, table_width, elem_bytes, status);
  MIE_LAUNCH_CHECK("write_packed_kv_kernel");
  return MIE_OK;
}

extern "C" int mie_gather_kv(mie_view4_t key_blocks, mie_view4_t value_blocks, mie_index_t block_table_row,
                             void* key_out, void* value_out, int32_t length, int32_t kv_heads, int32_t head_dim,
                             int32_t block_size, int32_t num_blocks, int32_t elem_bytes, int32_t* status,
                             void* stream) {
  if (int rc = check_common(head_dim, block_size, num_blocks, elem_bytes)) return rc;
  MIE_CHECK_ARG(length >= 0 && kv_heads >= 1, "invalid length/kv_heads");
  MIE_CHECK_ARG(key_blocks.ptr && value_blocks.ptr && block_table_row.ptr && key_out && value_out,
                "null tensor pointer");
  if (length == 0) return MIE_OK;
  const long long warps = (long long)length * kv_heads;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  gather_kv_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      View4(key_blocks), View4(value_blocks), IndexView(block_table_row), (char*)key_out, (char*)value_out, length,
      kv_heads, head_dim, block_size, num_blocks, elem_bytes, status);
  MIE_LAUNCH_CHECK("gather_kv_kernel");
  return MIE_OK;
}
