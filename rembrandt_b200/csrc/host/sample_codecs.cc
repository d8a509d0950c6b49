// Per-sample decoders that sit on the data-loading path: the Caffe `Datum` protobuf message of image databases
// (src/caffe_proto.proto:5-16 of the reference: channels, height, width, data, label, float_data, encoded) and the
// expansion of packed bit planes into bytes (Go positions). Both are bounds-checked parsers over untrusted bytes:
// they never read past `len` and report malformed input with a negative code.
#include "rembrandt_host.h"

#include <cstring>

namespace {

// Reads a base-128 varint at *pos. Returns false when the buffer ends inside it or it is longer than 10 bytes.
inline bool varint(const uint8_t* buf, uint64_t len, uint64_t* pos, uint64_t* out) {
  uint64_t v = 0;
  for (int shift = 0; shift < 70; shift += 7) {
    if (*pos >= len) return false;
    const uint8_t b = buf[(*pos)++];
    if (shift < 64) v |= (uint64_t)(b & 0x7F) << shift;
    if (!(b & 0x80)) {
      *out = v;
      return true;
    }
  }
  return false;
}

}  // namespace

extern "C" {

int rb_datum_parse(const uint8_t* buf, uint64_t len, rb_datum* out) {
  std::memset(out, 0, sizeof(*out));
  uint64_t pos = 0;
  while (pos < len) {
    uint64_t key;
    if (!varint(buf, len, &pos, &key)) return -1;
    const uint64_t field = key >> 3;
    const unsigned wire = (unsigned)(key & 7);
    if (wire == 0) {
      uint64_t v;
      if (!varint(buf, len, &pos, &v)) return -1;
      if (field == 1) out->channels = (int32_t)v;
      else if (field == 2) out->height = (int32_t)v;
      else if (field == 3) out->width = (int32_t)v;
      else if (field == 5) out->label = (int32_t)v;
      else if (field == 7) out->encoded = v ? 1 : 0;
    } else if (wire == 2) {
      uint64_t n;
      if (!varint(buf, len, &pos, &n)) return -1;
      if (n > len - pos) return -2;   // a length that runs past the message
      if (field == 4) {
        out->data_offset = pos;
        out->data_len = n;
      } else if (field == 6) {
        if (n % 4) return -3;
        out->float_count += n / 4;
      }
      pos += n;
    } else if (wire == 5) {
      if (len - pos < 4) return -2;
      if (field == 6) out->float_count += 1;
      pos += 4;
    } else if (wire == 1) {
      if (len - pos < 8) return -2;
      pos += 8;
    } else {
      return -4;   // groups and unknown wire types do not occur in this message
    }
  }
  return 0;
}

uint64_t rb_datum_floats(const uint8_t* buf, uint64_t len, float* out, uint64_t cap) {
  uint64_t pos = 0, count = 0;
  while (pos < len) {
    uint64_t key;
    if (!varint(buf, len, &pos, &key)) return count;
    const uint64_t field = key >> 3;
    const unsigned wire = (unsigned)(key & 7);
    if (wire == 0) {
      uint64_t v;
      if (!varint(buf, len, &pos, &v)) return count;
    } else if (wire == 2) {
      uint64_t n;
      if (!varint(buf, len, &pos, &n) || n > len - pos) return count;
      if (field == 6) {
        for (uint64_t i = 0; i + 4 <= n && count < cap; i += 4) std::memcpy(&out[count++], buf + pos + i, 4);
      }
      pos += n;
    } else if (wire == 5) {
      if (len - pos < 4) return count;
      if (field == 6 && count < cap) std::memcpy(&out[count++], buf + pos, 4);
      pos += 4;
    } else if (wire == 1) {
      if (len - pos < 8) return count;
      pos += 8;
    } else {
      return count;
    }
  }
  return count;
}

int rb_bits_unpack(const uint8_t* packed, uint64_t packed_len, uint64_t nbits, uint8_t scale, uint8_t* out) {
  if ((nbits + 7) / 8 > packed_len) return -1;
  const uint64_t full = nbits / 8;
  for (uint64_t i = 0; i < full; ++i) {
    const uint8_t b = packed[i];
    uint8_t* o = out + i * 8;
    for (int j = 0; j < 8; ++j) o[j] = ((b >> j) & 1) ? scale : 0;
  }
  for (uint64_t k = full * 8; k < nbits; ++k) out[k] = ((packed[k / 8] >> (k % 8)) & 1) ? scale : 0;
  return 0;
}

}  // extern "C"
