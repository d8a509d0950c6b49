// xorshift128+ generator (Vigna 2014) with the draws the framework needs, partition helper, readers.
#include "rembrandt_host.h"

#include <math.h>
#include <string.h>

extern "C" {

void rb_xs_seed(rb_xorshift* r, uint64_t s0, uint64_t s1) {
  r->s[0] = s0;
  r->s[1] = s1;
  if (r->s[0] == 0 && r->s[1] == 0) r->s[1] = 0x9E3779B97F4A7C15ull;  // the all-zero state is absorbing
}

uint64_t rb_xs_next(rb_xorshift* r) {
  uint64_t s1 = r->s[0];
  const uint64_t s0 = r->s[1];
  r->s[0] = s0;
  s1 ^= s1 << 23;
  r->s[1] = s1 ^ s0 ^ (s1 >> 17) ^ (s0 >> 26);
  return r->s[1] + s0;
}

double rb_xs_unit(rb_xorshift* r) { return (double)(rb_xs_next(r) >> 11) * (1.0 / 9007199254740992.0); }

uint32_t rb_xs_below(rb_xorshift* r, uint32_t n) {
  if (n <= 1) return 0;
  // rejection sampling on 32 high bits: unbiased
  const uint32_t limit = 0xFFFFFFFFu - (0xFFFFFFFFu % n + 1u) % n;
  while (true) {
    const uint32_t v = (uint32_t)(rb_xs_next(r) >> 32);
    if (v <= limit) return v % n;
  }
}

void rb_xs_fill_uniform(rb_xorshift* r, float* out, uint64_t n, float lo, float hi) {
  for (uint64_t i = 0; i < n; ++i) out[i] = lo + (hi - lo) * (float)rb_xs_unit(r);
}

void rb_xs_fill_normal(rb_xorshift* r, float* out, uint64_t n, float mean, float std) {
  for (uint64_t i = 0; i < n; i += 2) {
    double u0 = rb_xs_unit(r), u1 = rb_xs_unit(r);
    if (u0 < 1e-300) u0 = 1e-300;
    const double m = sqrt(-2.0 * log(u0));
    out[i] = mean + std * (float)(m * cos(6.283185307179586 * u1));
    if (i + 1 < n) out[i + 1] = mean + std * (float)(m * sin(6.283185307179586 * u1));
  }
}

void rb_xs_permutation(rb_xorshift* r, int32_t* out, int32_t n) {
  for (int32_t i = 0; i < n; ++i) out[i] = i;
  for (int32_t i = n - 1; i > 0; --i) {
    const int32_t j = (int32_t)rb_xs_below(r, (uint32_t)i + 1u);
    const int32_t t = out[i];
    out[i] = out[j];
    out[j] = t;
  }
}

void rb_partition_range(uint64_t n, uint32_t parts, uint32_t idx, uint64_t* lo, uint64_t* hi) {
  const uint64_t base = n / parts, extra = n % parts;
  *lo = base * idx + (idx < extra ? idx : extra);
  *hi = *lo + base + (idx < extra ? 1 : 0);
}

int rb_idx_header(const uint8_t* buf, uint64_t len, uint32_t* dtype, uint32_t* ndim, uint32_t dims[4],
                  uint64_t* data_offset) {
  if (len < 4 || buf[0] != 0 || buf[1] != 0) return -1;
  *dtype = buf[2];
  *ndim = buf[3];
  if (*ndim == 0 || *ndim > 4) return -2;
  if (len < 4 + 4ull * *ndim) return -3;
  uint64_t elems = 1;
  for (uint32_t i = 0; i < 4; ++i) dims[i] = 1;
  for (uint32_t i = 0; i < *ndim; ++i) {
    const uint8_t* p = buf + 4 + 4 * i;
    dims[i] = ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | (uint32_t)p[3];
    elems *= dims[i];
  }
  *data_offset = 4 + 4ull * *ndim;
  const uint64_t esize = (*dtype == 0x08 || *dtype == 0x09) ? 1 : (*dtype == 0x0B) ? 2 : (*dtype == 0x0E) ? 8 : 4;
  if (*data_offset + elems * esize > len) return -4;
  return 0;
}

int rb_cifar_split(const uint8_t* buf, uint64_t len, uint64_t first, uint64_t count, uint8_t* images,
                   int32_t* labels) {
  const uint64_t rec = 1 + 3072;
  if ((first + count) * rec > len) return -1;
  for (uint64_t i = 0; i < count; ++i) {
    const uint8_t* p = buf + (first + i) * rec;
    labels[i] = p[0];
    memcpy(images + i * 3072, p + 1, 3072);
  }
  return 0;
}

void rb_mean_u8(const uint8_t* images, uint64_t n, uint64_t elems, float* mean_out) {
  double* acc = new double[elems];
  for (uint64_t j = 0; j < elems; ++j) acc[j] = 0.0;
  for (uint64_t i = 0; i < n; ++i) {
    const uint8_t* p = images + i * elems;
    for (uint64_t j = 0; j < elems; ++j) acc[j] += p[j];
  }
  for (uint64_t j = 0; j < elems; ++j) mean_out[j] = n ? (float)(acc[j] / (double)n) : 0.f;
  delete[] acc;
}

}  // extern "C"
