// Self-describing container for one compressed 2:4 weight, so that a host can persist the packed
// values + metadata and skip pruning at load time.  Host-only code: these functions touch no GPU.
//
// Layout (little endian):  [256-byte header][payload]
//   payload = values [rows, K/2] 16-bit, zero padding to a 256-byte boundary, metadata tiles
// which is exactly the block `sparseflow_sparse_gemm` takes as `Bc`, so `blob + 256` can be handed
// to the GEMM without a copy once the blob is in device memory.
#include <cstring>

#include "../../include/sparseflow_b200.h"
#include "kernels.h"

namespace {

const char kMagic[8] = {'S', 'F', 'B', '2', '4', 'W', 0, 0};

struct RawHeader {  // 96 bytes used, the rest of the 256 is zero
  char magic[8];
  uint32_t layout_version;
  uint32_t header_bytes;
  int32_t dtype;
  int32_t rows;
  int32_t K;
  uint32_t flags;
  uint64_t values_bytes;
  uint64_t meta_offset;  // from the start of the payload
  uint64_t meta_bytes;
  uint64_t total_bytes;  // header + payload
  uint64_t checksum;     // FNV-1a 64 of the payload, 0 = not recorded
};
static_assert(sizeof(RawHeader) <= SFB200_BLOB_HEADER_BYTES, "header struct outgrew its slot");

bool shape_ok(int rows, int K) { return rows > 0 && K > 0 && K % 16 == 0; }

size_t meta_offset_of(int rows, int K) {
  const size_t v = sfb200::values_bytes(rows, K);
  return (v + 255) & ~static_cast<size_t>(255);
}

}  // namespace

extern "C" {

size_t sfb200_blob_bytes(int rows, int K) {
  if (!shape_ok(rows, K)) return 0;
  return SFB200_BLOB_HEADER_BYTES + meta_offset_of(rows, K) + sfb200::meta_bytes(rows, K);
}

uint64_t sfb200_blob_checksum(const void* payload_host, size_t bytes) {
  const unsigned char* p = static_cast<const unsigned char*>(payload_host);
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < bytes; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h == 0 ? 1 : h;  // 0 is reserved for "not recorded"
}

int sfb200_blob_write_header(void* header_host, int rows, int K, int dtype, unsigned flags,
                             uint64_t checksum) {
  if (!header_host || !shape_ok(rows, K)) return SFB200_ERROR_INVALID_ARGUMENT;
  if (dtype != SFB200_F16 && dtype != SFB200_BF16) return SFB200_ERROR_INVALID_ARGUMENT;
  if (flags & ~static_cast<unsigned>(SFB200_BLOB_GATE_UP | SFB200_BLOB_TIE_LOW))
    return SFB200_ERROR_INVALID_ARGUMENT;
  if ((flags & SFB200_BLOB_GATE_UP) && rows % 32 != 0) return SFB200_ERROR_INVALID_ARGUMENT;
  RawHeader h;
  std::memset(&h, 0, sizeof(h));
  std::memcpy(h.magic, kMagic, sizeof(kMagic));
  h.layout_version = SFB200_LAYOUT_VERSION;
  h.header_bytes = SFB200_BLOB_HEADER_BYTES;
  h.dtype = dtype;
  h.rows = rows;
  h.K = K;
  h.flags = flags;
  h.values_bytes = sfb200::values_bytes(rows, K);
  h.meta_offset = meta_offset_of(rows, K);
  h.meta_bytes = sfb200::meta_bytes(rows, K);
  h.total_bytes = sfb200_blob_bytes(rows, K);
  h.checksum = checksum;
  std::memset(header_host, 0, SFB200_BLOB_HEADER_BYTES);
  std::memcpy(header_host, &h, sizeof(h));
  return SFB200_SUCCESS;
}

int sfb200_blob_read_header(const void* header_host, size_t available_bytes, sfb200_blob_info* info) {
  if (!header_host || !info) return SFB200_ERROR_INVALID_ARGUMENT;
  if (available_bytes < SFB200_BLOB_HEADER_BYTES) return SFB200_ERROR_INVALID_ARGUMENT;
  RawHeader h;
  std::memcpy(&h, header_host, sizeof(h));
  if (std::memcmp(h.magic, kMagic, sizeof(kMagic)) != 0) return SFB200_ERROR_INVALID_ARGUMENT;
  if (h.layout_version != SFB200_LAYOUT_VERSION || h.header_bytes != SFB200_BLOB_HEADER_BYTES)
    return SFB200_ERROR_NOT_SUPPORTED;  // written by a build with another packed layout: re-prune
  if (!shape_ok(h.rows, h.K) || (h.dtype != SFB200_F16 && h.dtype != SFB200_BF16))
    return SFB200_ERROR_INVALID_ARGUMENT;
  // the sizes are functions of (rows, K): a header that disagrees is corrupt
  if (h.values_bytes != sfb200::values_bytes(h.rows, h.K) || h.meta_offset != meta_offset_of(h.rows, h.K) ||
      h.meta_bytes != sfb200::meta_bytes(h.rows, h.K) || h.total_bytes != sfb200_blob_bytes(h.rows, h.K))
    return SFB200_ERROR_INVALID_ARGUMENT;
  if (available_bytes < h.total_bytes) return SFB200_ERROR_INVALID_ARGUMENT;  // truncated
  info->layout_version = h.layout_version;
  info->dtype = h.dtype;
  info->rows = h.rows;
  info->K = h.K;
  info->flags = h.flags;
  info->values_offset = SFB200_BLOB_HEADER_BYTES;
  info->values_bytes = h.values_bytes;
  info->meta_offset = SFB200_BLOB_HEADER_BYTES + h.meta_offset;
  info->meta_bytes = h.meta_bytes;
  info->total_bytes = h.total_bytes;
  info->checksum = h.checksum;
  return SFB200_SUCCESS;
}

}  // extern "C"
