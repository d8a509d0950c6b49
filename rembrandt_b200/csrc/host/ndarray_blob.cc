// NdArray blob codec: byte-exact reader/writer for the reference's checkpoint and mean-file records.
#include "rembrandt_host.h"

#include <string.h>

static uint32_t rd_u32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static uint64_t rd_u64(const uint8_t* p) { return (uint64_t)rd_u32(p) | ((uint64_t)rd_u32(p + 4) << 32); }
static void wr_u32(uint8_t* p, uint32_t v) {
  for (int i = 0; i < 4; ++i) p[i] = (uint8_t)(v >> (8 * i));
}
static void wr_u64(uint8_t* p, uint64_t v) {
  for (int i = 0; i < 8; ++i) p[i] = (uint8_t)(v >> (8 * i));
}

extern "C" {

int rb_blob_parse(const uint8_t* buf, uint64_t len, uint64_t offset, uint32_t elem_size, rb_blob_record* out) {
  if (offset + 8 > len) return -1;
  const uint8_t* p = buf + offset;
  if (p[0] != 'N' || p[1] != 'D') return -2;
  out->tag[0] = p[2];
  out->tag[1] = p[3];
  out->ndim = rd_u32(p + 4);
  if (out->ndim > RB_BLOB_MAX_DIMS) return -3;
  const uint64_t hdr = 8 + 8ull * out->ndim;
  if (offset + hdr > len) return -1;
  uint64_t n = 1;
  for (uint32_t i = 0; i < out->ndim; ++i) {
    out->dims[i] = rd_u64(p + 8 + 8 * i);
    n *= out->dims[i];
  }
  for (uint32_t i = out->ndim; i < RB_BLOB_MAX_DIMS; ++i) out->dims[i] = 1;
  out->num_elems = n;
  out->data_offset = offset + hdr;
  out->next_offset = out->data_offset + n * elem_size;
  if (out->next_offset > len) return -4;
  return 0;
}

uint64_t rb_blob_record_size(uint32_t ndim, const uint64_t* dims, uint32_t elem_size) {
  uint64_t n = 1;
  for (uint32_t i = 0; i < ndim; ++i) n *= dims[i];
  return 8 + 8ull * ndim + n * elem_size;
}

uint64_t rb_blob_write(uint8_t* out, uint64_t cap, const uint8_t tag[2], uint32_t ndim, const uint64_t* dims,
                       const void* data, uint32_t elem_size) {
  const uint64_t total = rb_blob_record_size(ndim, dims, elem_size);
  if (total > cap || ndim > RB_BLOB_MAX_DIMS) return 0;
  out[0] = 'N';
  out[1] = 'D';
  out[2] = tag[0];
  out[3] = tag[1];
  wr_u32(out + 4, ndim);
  for (uint32_t i = 0; i < ndim; ++i) wr_u64(out + 8 + 8 * i, dims[i]);
  const uint64_t hdr = 8 + 8ull * ndim;
  memcpy(out + hdr, data, total - hdr);
  return total;
}

}  // extern "C"
