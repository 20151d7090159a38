// Device-side decode-metadata validation that reports through a status word.
#include "common.cuh"

namespace mie {
namespace {

__global__ void validate_kernel(IndexView tables, IndexView lengths, IndexView positions, int batch,
                                int table_width, int block_size, int num_blocks, long long max_len, int* status) {
  // One warp per request; lanes sweep that request's live block-table entries.
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= batch) return;
  int bits = 0;
  const long long len = lengths.at(warp);
  long long live_tokens = len;
  if (len < 1 || len > (long long)table_width * block_size) {
    bits |= MIE_STATUS_BAD_LENGTH;
    live_tokens = 0;
  }
  long long read_len = len;
  if (positions.valid()) {
    const long long pos = positions.at(warp);
    if (pos < 0 || pos >= len) bits |= MIE_STATUS_BAD_POSITION;
    read_len = pos + 1;
  }
  if (max_len > 0 && read_len > max_len) bits |= MIE_STATUS_MAX_LENGTH;
  const long long live_pages = (live_tokens + block_size - 1) / block_size;
  for (long long p = lane; p < live_pages; p += 32) {
    const long long id = tables.at(warp, p);
    if (id < 0 || id >= num_blocks) bits |= MIE_STATUS_BAD_PAGE;
  }
  if (bits) raise_status(status, bits);
}

}  // namespace
}  // namespace mie

using namespace mie;

extern "C" int mie_validate_decode_metadata(mie_index_t block_tables, mie_index_t sequence_lengths,
                                            mie_index_t query_positions, int32_t batch, int32_t table_width,
                                            int32_t block_size, int32_t num_blocks, int64_t max_sequence_length,
                                            int32_t* status, void* stream) {
  MIE_CHECK_ARG(block_tables.ptr && sequence_lengths.ptr, "null metadata pointer");
  MIE_CHECK_ARG(status != nullptr, "status pointer is required");
  MIE_CHECK_ARG(batch >= 0 && table_width >= 1 && block_size >= 1 && num_blocks >= 1, "invalid metadata shape");
  if (batch == 0) return MIE_OK;
  const int threads = 128;
  const int blocks = (batch * 32 + threads - 1) / threads;
  validate_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(
      IndexView(block_tables), IndexView(sequence_lengths), IndexView(query_positions), batch, table_width,
      block_size, num_blocks, (long long)max_sequence_length, status);
  MIE_LAUNCH_CHECK("validate_kernel");
  return MIE_OK;
}
