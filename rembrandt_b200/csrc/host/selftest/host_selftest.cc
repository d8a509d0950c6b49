// Self-test of the CPU-side runtime library, meant to be built with -fsanitize=address,undefined and with
// -fsanitize=thread and run as a plain executable (the Python tests cannot load sanitizer runtimes into the
// interpreter). It drives every entry point of rembrandt_host.h, including malformed inputs and the threaded batch
// loader under contention. Usage: host_selftest [lmdb-environment-path expected-entries]
// Exit status 0 = every check passed; the sanitizers abort with their own report otherwise.
#include "../rembrandt_host.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

static int g_failures = 0;
#define CHECK(cond)                                                            \
  do {                                                                         \
    if (!(cond)) {                                                             \
      std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      ++g_failures;                                                            \
    }                                                                          \
  } while (0)

static void test_blob() {
  const uint64_t dims[3] = {3, 4, 5};
  std::vector<float> data(60);
  for (size_t i = 0; i < data.size(); ++i) data[i] = (float)i * 0.5f;
  const uint64_t size = rb_blob_record_size(3, dims, 4);
  CHECK(size == 4 + 4 + 3 * 8 + 60 * 4);
  std::vector<uint8_t> buf(size * 2);
  const uint8_t tag[2] = {0x00, 0x01};
  CHECK(rb_blob_write(buf.data(), size - 1, tag, 3, dims, data.data(), 4) == 0);   // does not fit
  CHECK(rb_blob_write(buf.data(), size, tag, 3, dims, data.data(), 4) == size);
  CHECK(rb_blob_write(buf.data() + size, size, tag, 3, dims, data.data(), 4) == size);
  rb_blob_record rec;
  CHECK(rb_blob_parse(buf.data(), buf.size(), 0, 4, &rec) == 0);
  CHECK(rec.ndim == 3 && rec.dims[2] == 5 && rec.num_elems == 60 && rec.next_offset == size);
  CHECK(std::memcmp(buf.data() + rec.data_offset, data.data(), 240) == 0);
  CHECK(rb_blob_parse(buf.data(), buf.size(), rec.next_offset, 4, &rec) == 0);
  CHECK(rec.next_offset == 2 * size);
  // every truncation of a valid record is rejected without reading past the end
  for (uint64_t len = 0; len < size; ++len) {
    std::vector<uint8_t> cut(buf.begin(), buf.begin() + len);   // exact-size allocation: overreads are caught
    CHECK(rb_blob_parse(cut.data(), len, 0, 4, &rec) < 0);
  }
  std::vector<uint8_t> bad(buf.begin(), buf.begin() + size);
  bad[0] = 'X';
  CHECK(rb_blob_parse(bad.data(), size, 0, 4, &rec) == -2);
  bad[0] = 'N';
  bad[4] = 200;   // ndim far beyond the limit
  CHECK(rb_blob_parse(bad.data(), size, 0, 4, &rec) == -3);
  // dimensions whose product overflows must not be accepted
  std::vector<uint8_t> huge(4 + 4 + 2 * 8, 0);
  huge[0] = 'N'; huge[1] = 'D'; huge[4] = 2;
  std::memset(huge.data() + 8, 0xFF, 16);
  CHECK(rb_blob_parse(huge.data(), huge.size(), 0, 4, &rec) < 0);
}

static void test_rng_and_partition() {
  rb_xorshift a, b;
  rb_xs_seed(&a, 17, 29);
  rb_xs_seed(&b, 17, 29);
  for (int i = 0; i < 100; ++i) CHECK(rb_xs_next(&a) == rb_xs_next(&b));
  for (int i = 0; i < 1000; ++i) {
    const double u = rb_xs_unit(&a);
    CHECK(u >= 0.0 && u < 1.0);
    CHECK(rb_xs_below(&a, 7) < 7);
  }
  std::vector<float> f(1001);
  rb_xs_fill_uniform(&a, f.data(), f.size(), -2.f, 3.f);
  for (float v : f) CHECK(v >= -2.f && v <= 3.f);
  rb_xs_fill_normal(&a, f.data(), f.size(), 1.f, 0.5f);   // odd length: the pairwise generator must not overrun
  double mean = 0;
  for (float v : f) mean += v;
  CHECK(std::abs(mean / f.size() - 1.0) < 0.1);
  std::vector<int32_t> perm(257);
  rb_xs_permutation(&a, perm.data(), (int32_t)perm.size());
  std::vector<int> seen(perm.size(), 0);
  for (int32_t p : perm) { CHECK(p >= 0 && p < (int32_t)perm.size()); if (p >= 0 && p < (int32_t)perm.size()) ++seen[p]; }
  for (int s : seen) CHECK(s == 1);
  rb_xs_permutation(&a, perm.data(), 0);
  for (uint64_t n : {0ull, 1ull, 10ull, 1000003ull})
    for (uint32_t parts : {1u, 3u, 8u}) {
      uint64_t expect = 0;
      for (uint32_t i = 0; i < parts; ++i) {
        uint64_t lo, hi;
        rb_partition_range(n, parts, i, &lo, &hi);
        CHECK(lo == expect && hi >= lo);
        expect = hi;
      }
      CHECK(expect == n);
    }
}

static void test_readers() {
  // IDX: 2 images of 3 x 2 bytes
  std::vector<uint8_t> idx = {0, 0, 8, 3, 0, 0, 0, 2, 0, 0, 0, 3, 0, 0, 0, 2, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12};
  uint32_t dtype, ndim, dims[4];
  uint64_t off;
  CHECK(rb_idx_header(idx.data(), idx.size(), &dtype, &ndim, dims, &off) == 0);
  CHECK(dtype == 8 && ndim == 3 && dims[0] == 2 && dims[1] == 3 && dims[2] == 2 && off == 16);
  for (uint64_t len = 0; len < 16; ++len) {
    std::vector<uint8_t> cut(idx.begin(), idx.begin() + len);
    CHECK(rb_idx_header(cut.data(), len, &dtype, &ndim, dims, &off) < 0);
  }
  // CIFAR: 3 records
  std::vector<uint8_t> cifar(3 * 3073);
  for (size_t i = 0; i < cifar.size(); ++i) cifar[i] = (uint8_t)(i * 7);
  std::vector<uint8_t> images(2 * 3072);
  int32_t labels[2];
  CHECK(rb_cifar_split(cifar.data(), cifar.size(), 1, 2, images.data(), labels) == 0);
  CHECK(labels[0] == cifar[3073] && images[0] == cifar[3074] && images[3072] == cifar[2 * 3073 + 1]);
  CHECK(rb_cifar_split(cifar.data(), cifar.size(), 2, 2, images.data(), labels) < 0);   // runs past the end
  std::vector<float> mean(3072);
  rb_mean_u8(images.data(), 2, 3072, mean.data());
  CHECK(std::abs(mean[5] - 0.5f * (images[5] + images[3072 + 5])) < 1e-4f);
}

static void test_sample_codecs() {
  // Datum: channels 3, height 2, width 2, data 12 bytes, label 7, two unpacked floats, one packed pair, encoded
  std::vector<uint8_t> msg = {0x08, 3, 0x10, 2, 0x18, 2, 0x22, 12};
  for (int i = 0; i < 12; ++i) msg.push_back((uint8_t)(i * 11));
  msg.insert(msg.end(), {0x28, 7});
  const float f[4] = {1.5f, -2.f, 0.25f, 8.f};
  for (int i = 0; i < 2; ++i) {
    msg.push_back(0x35);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&f[i]);
    msg.insert(msg.end(), b, b + 4);
  }
  msg.insert(msg.end(), {0x32, 8});
  const uint8_t* b2 = reinterpret_cast<const uint8_t*>(&f[2]);
  msg.insert(msg.end(), b2, b2 + 8);
  msg.insert(msg.end(), {0x38, 1});
  rb_datum d;
  CHECK(rb_datum_parse(msg.data(), msg.size(), &d) == 0);
  CHECK(d.channels == 3 && d.height == 2 && d.width == 2 && d.label == 7 && d.encoded == 1);
  CHECK(d.data_len == 12 && msg[d.data_offset + 1] == 11 && d.float_count == 4);
  float got[4] = {0, 0, 0, 0};
  CHECK(rb_datum_floats(msg.data(), msg.size(), got, 4) == 4);
  for (int i = 0; i < 4; ++i) CHECK(got[i] == f[i]);
  CHECK(rb_datum_floats(msg.data(), msg.size(), got, 3) == 3);   // a short output array is respected
  // every truncation either parses as a shorter message or is rejected; exact-size copies let ASan see overreads
  for (uint64_t len = 0; len < msg.size(); ++len) {
    std::vector<uint8_t> cut(msg.begin(), msg.begin() + len);
    const int rc = rb_datum_parse(cut.data(), len, &d);
    CHECK(rc <= 0);
    if (rc == 0) CHECK(d.data_offset + d.data_len <= len);
    rb_datum_floats(cut.data(), len, got, 4);
  }
  const uint8_t huge_len[] = {0x22, 0xFF, 0xFF, 0xFF, 0xFF, 0xFF, 0xFF, 0xFF, 0xFF, 0xFF, 0x01};
  CHECK(rb_datum_parse(huge_len, sizeof(huge_len), &d) == -2);
  const uint8_t endless[] = {0x08, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80, 0x80};
  CHECK(rb_datum_parse(endless, sizeof(endless), &d) == -1);
  const uint8_t group[] = {0x0B};
  CHECK(rb_datum_parse(group, sizeof(group), &d) == -4);
  // bit planes
  const uint8_t packed[2] = {0xA5, 0x03};
  std::vector<uint8_t> out(10);
  CHECK(rb_bits_unpack(packed, 2, 10, 255, out.data()) == 0);
  const uint8_t want[10] = {255, 0, 255, 0, 0, 255, 0, 255, 255, 255};
  CHECK(std::memcmp(out.data(), want, 10) == 0);
  CHECK(rb_bits_unpack(packed, 1, 10, 255, out.data()) == -1);
  CHECK(rb_bits_unpack(packed, 0, 0, 1, out.data()) == 0);
}

static void test_loader(uint32_t mode, uint32_t threads, uint32_t nslots) {
  const uint64_t n = 97, elems = 33;
  const uint32_t batch = 8;
  std::vector<uint8_t> images(n * elems);
  std::vector<int32_t> labels(n);
  for (uint64_t i = 0; i < n; ++i) {
    labels[i] = (int32_t)i;
    std::memset(images.data() + i * elems, (int)(i & 0xFF), elems);
  }
  std::vector<std::vector<uint8_t>> islots(nslots, std::vector<uint8_t>(batch * elems));
  std::vector<std::vector<int32_t>> lslots(nslots, std::vector<int32_t>(batch));
  std::vector<uint8_t*> ip;
  std::vector<int32_t*> lp;
  for (uint32_t s = 0; s < nslots; ++s) { ip.push_back(islots[s].data()); lp.push_back(lslots[s].data()); }
  CHECK(rb_loader_create(images.data(), labels.data(), elems, 5, 5, batch, mode, 1, threads, nslots, ip.data(),
                         lp.data()) == nullptr);   // empty shard
  void* L = rb_loader_create(images.data(), labels.data(), elems, 5, 90, batch, mode, 1234, threads, nslots, ip.data(),
                             lp.data());
  CHECK(L != nullptr);
  if (!L) return;
  for (uint64_t b = 0; b < 60; ++b) {
    uint64_t got = ~0ull;
    const int slot = rb_loader_acquire(L, &got);
    CHECK(slot >= 0 && got == b);
    if (slot < 0) break;
    for (uint32_t i = 0; i < batch; ++i) {
      const uint64_t want = rb_loader_sample_index(5, 90, mode, 1234, b * batch + i);
      CHECK(want >= 5 && want < 90);
      CHECK(lslots[slot][i] == (int32_t)want);
      CHECK(islots[slot][i * elems] == (uint8_t)(want & 0xFF) && islots[slot][i * elems + elems - 1] == (uint8_t)(want & 0xFF));
    }
    rb_loader_release(L, slot);
  }
  // destroy while the workers are blocked on full slots and one slot is still held by the consumer
  const int held = rb_loader_acquire(L, nullptr);
  CHECK(held >= 0);
  rb_loader_destroy(L);
  if (mode == 2) {   // shuffled epochs: every sample of the shard exactly once per epoch
    std::vector<int> seen(n, 0);
    for (uint64_t pos = 0; pos < 85; ++pos) ++seen[rb_loader_sample_index(5, 90, 2, 77, pos)];
    for (uint64_t i = 5; i < 90; ++i) CHECK(seen[i] == 1);
  }
}

static void test_lmdb(const char* path, uint64_t expected) {
  CHECK(rb_lmdb_open("/nonexistent/environment") == nullptr);
  if (!path) return;
  void* env = rb_lmdb_open(path);
  CHECK(env != nullptr);
  if (!env) return;
  CHECK(rb_lmdb_entries(env) == expected);
  CHECK(rb_lmdb_page_size(env) >= 512);
  uint64_t count = 0, bytes = 0;
  std::string prev;
  const uint8_t *k, *v;
  uint32_t kl;
  uint64_t vl;
  if (rb_lmdb_seek(env, nullptr, 0)) {
    while (rb_lmdb_next(env, &k, &kl, &v, &vl)) {
      std::string key((const char*)k, kl);
      CHECK(count == 0 || prev < key);   // strictly ascending
      prev = key;
      for (uint64_t i = 0; i < vl; ++i) bytes += v[i];   // touches every byte handed out
      ++count;
    }
  }
  CHECK(count == expected);
  // seek to the last key and beyond it
  CHECK(rb_lmdb_seek(env, (const uint8_t*)prev.data(), (uint32_t)prev.size()) == (expected ? 1 : 0));
  std::string beyond = prev + "\xff";
  CHECK(rb_lmdb_seek(env, (const uint8_t*)beyond.data(), (uint32_t)beyond.size()) == 0);
  CHECK(rb_lmdb_next(env, &k, &kl, &v, &vl) == 0);
  rb_lmdb_close(env);
  // the values of this environment are not image records: the database-backed loader must refuse it cleanly
  std::vector<uint8_t> slot_a(64), slot_b(64);
  std::vector<int32_t> lab_a(4), lab_b(4);
  uint8_t* ip[2] = {slot_a.data(), slot_b.data()};
  int32_t* lp[2] = {lab_a.data(), lab_b.data()};
  int32_t err = 0;
  CHECK(rb_loader_create_lmdb(path, 16, 0, expected, 4, 0, 1, 2, 2, ip, lp, &err) == nullptr);
  CHECK(err == 2 || err == 3);
  CHECK(rb_loader_create_lmdb("/nonexistent/environment", 16, 0, 8, 4, 0, 1, 2, 2, ip, lp, &err) == nullptr && err == 1);
  std::printf("lmdb: %llu entries, byte sum %llu\n", (unsigned long long)count, (unsigned long long)bytes);
}

int main(int argc, char** argv) {
  test_blob();
  test_rng_and_partition();
  test_readers();
  test_sample_codecs();
  for (uint32_t mode = 0; mode < 3; ++mode) {
    test_loader(mode, 1, 2);
    test_loader(mode, 4, 3);
    test_loader(mode, 8, 2);
  }
  test_lmdb(argc > 2 ? argv[1] : nullptr, argc > 2 ? std::strtoull(argv[2], nullptr, 10) : 0);
  if (g_failures) {
    std::fprintf(stderr, "%d check(s) failed\n", g_failures);
    return 1;
  }
  std::printf("host self-test: ok\n");
  return 0;
}
