// Read-only LMDB environment reader with a cursor (no dependency on liblmdb): the newer meta page, the main
// database's B+tree (branch / leaf / overflow pages), seek to the first key >= a given key, ordered iteration.
// The file is memory-mapped; keys and values handed out point into the mapping and stay valid until close.
// The reference reads its Caffe image databases through liblmdb cursors the same way
// (src/data/lmdb_data.rs:50-152: seek by zero-padded record number, then next, next, ...).
//
// On-disk layout (little endian, 64-bit, LMDB data format version 1):
//   page header   pgno u64 | pad u16 | flags u16 | lower u16, upper u16   (overflow pages: page count u32 instead)
//   meta page     header | magic 0xBEEFC0DE u32 | version u32 | address u64 | mapsize u64 | 2 x db record (48 bytes:
//                 pad u32 [page size in the first record], flags u16, depth u16, branch, leaf, overflow pages, entries,
//                 root, all u64) | last page u64 | txn id u64
//   node          lo u16 | hi u16 | flags u16 | key size u16 | key | data;  branch: child = lo | hi << 16 | flags << 32;
//                 leaf: data size = lo | hi << 16, flag 0x01 = data is the u64 number of an overflow page
#include "rembrandt_host.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr uint32_t kMagic = 0xBEEFC0DEu;
constexpr uint16_t kBranch = 0x01, kLeaf = 0x02;
constexpr uint16_t kBigData = 0x01;
constexpr uint64_t kHdr = 16;
constexpr uint64_t kInvalid = ~0ull;

template <class T>
inline T rd(const uint8_t* p) {
  T v;
  std::memcpy(&v, p, sizeof(T));
  return v;
}

struct Frame {
  uint64_t page_off;
  uint32_t nkeys;
  uint32_t idx;
};

struct Env {
  int fd = -1;
  const uint8_t* m = nullptr;
  uint64_t size = 0;
  uint32_t psize = 0, depth = 0;
  uint64_t entries = 0, root = kInvalid;
  std::vector<Frame> stack;   // cursor: path from the root to the current leaf
  bool at_end = true;

  bool page(uint64_t pgno, uint64_t* off, uint16_t* flags, uint32_t* nkeys) const {
    const uint64_t o = pgno * psize;
    if (o + kHdr > size) return false;
    *off = o;
    *flags = rd<uint16_t>(m + o + 10);
    const uint16_t lower = rd<uint16_t>(m + o + 12);
    *nkeys = lower >= kHdr ? (lower - kHdr) / 2 : 0;
    return true;
  }
  const uint8_t* node(uint64_t page_off, uint32_t i) const {
    return m + page_off + rd<uint16_t>(m + page_off + kHdr + 2 * i);
  }
  static uint64_t child(const uint8_t* nd) {
    return (uint64_t)rd<uint16_t>(nd) | ((uint64_t)rd<uint16_t>(nd + 2) << 16) | ((uint64_t)rd<uint16_t>(nd + 4) << 32);
  }
  static int cmp(const uint8_t* a, uint32_t al, const uint8_t* b, uint32_t bl) {
    const int c = std::memcmp(a, b, al < bl ? al : bl);
    return c ? c : (al < bl ? -1 : (al > bl ? 1 : 0));
  }

  // descend from `pgno` towards `key` (leftmost when key == nullptr), pushing frames
  bool descend(uint64_t pgno, const uint8_t* key, uint32_t klen) {
    for (;;) {
      uint64_t off;
      uint16_t flags;
      uint32_t n;
      if (!page(pgno, &off, &flags, &n) || n == 0) return false;
      if (flags & kLeaf) {
        stack.push_back({off, n, 0});
        return true;
      }
      if (!(flags & kBranch)) return false;
      uint32_t idx = 0;
      if (key) {   // last node whose key <= `key`; node 0 carries an empty key and covers everything smaller
        uint32_t lo = 1, hi = n;
        while (lo < hi) {
          const uint32_t mid = (lo + hi) / 2;
          const uint8_t* nd = node(off, mid);
          if (cmp(nd + 8, rd<uint16_t>(nd + 6), key, klen) <= 0) { idx = mid; lo = mid + 1; }
          else hi = mid;
        }
      }
      stack.push_back({off, n, idx});
      pgno = child(node(off, idx));
    }
  }

  // move to the first node of the next leaf; false at the end of the tree
  bool next_leaf() {
    stack.pop_back();
    while (!stack.empty()) {
      Frame& f = stack.back();
      if (f.idx + 1 < f.nkeys) {
        ++f.idx;
        return descend(child(node(f.page_off, f.idx)), nullptr, 0);
      }
      stack.pop_back();
    }
    return false;
  }
};

bool read_meta(const Env& e, uint64_t off, uint32_t* psize, uint16_t* depth, uint64_t* entries, uint64_t* root,
               uint64_t* txnid) {
  if (off + kHdr + 136 > e.size) return false;
  const uint8_t* p = e.m + off + kHdr;
  if (rd<uint32_t>(p) != kMagic || rd<uint32_t>(p + 4) != 1) return false;
  *psize = rd<uint32_t>(p + 24);
  const uint8_t* main_db = p + 24 + 48;
  *depth = rd<uint16_t>(main_db + 6);
  *entries = rd<uint64_t>(main_db + 32);
  *root = rd<uint64_t>(main_db + 40);
  *txnid = rd<uint64_t>(main_db + 48 + 8);
  return true;
}

}  // namespace

extern "C" {

void* rb_lmdb_open(const char* path) {
  std::string file(path);
  struct stat st;
  if (stat(path, &st) == 0 && S_ISDIR(st.st_mode)) file += "/data.mdb";
  Env* e = new Env();
  e->fd = open(file.c_str(), O_RDONLY);
  if (e->fd < 0 || fstat(e->fd, &st) != 0 || st.st_size < 2 * 512) { if (e->fd >= 0) close(e->fd); delete e; return nullptr; }
  e->size = (uint64_t)st.st_size;
  void* m = mmap(nullptr, e->size, PROT_READ, MAP_SHARED, e->fd, 0);
  if (m == MAP_FAILED) { close(e->fd); delete e; return nullptr; }
  e->m = static_cast<const uint8_t*>(m);
  uint32_t ps0 = 0;
  uint16_t d0 = 0;
  uint64_t en0 = 0, r0 = 0, t0 = 0;
  if (!read_meta(*e, 0, &ps0, &d0, &en0, &r0, &t0) || ps0 < 512 || (ps0 & (ps0 - 1))) {
    munmap(m, e->size); close(e->fd); delete e; return nullptr;
  }
  e->psize = ps0; e->depth = d0; e->entries = en0; e->root = r0;
  uint32_t ps1;
  uint16_t d1;
  uint64_t en1, r1, t1;
  if (read_meta(*e, ps0, &ps1, &d1, &en1, &r1, &t1) && t1 > t0) { e->depth = d1; e->entries = en1; e->root = r1; }
  return e;
}

uint64_t rb_lmdb_entries(void* h) { return static_cast<Env*>(h)->entries; }
uint32_t rb_lmdb_depth(void* h) { return static_cast<Env*>(h)->depth; }
uint32_t rb_lmdb_page_size(void* h) { return static_cast<Env*>(h)->psize; }

// Position the cursor on the first key >= `key` (on the first key when klen == 0). Returns 1 if such a key exists.
int rb_lmdb_seek(void* h, const uint8_t* key, uint32_t klen) {
  Env* e = static_cast<Env*>(h);
  e->stack.clear();
  e->at_end = true;
  if (e->root == kInvalid || e->entries == 0) return 0;
  if (!e->descend(e->root, klen ? key : nullptr, klen)) return 0;
  if (klen) {
    for (;;) {   // first node of this leaf (or a following one) that is not smaller than the key
      Frame& f = e->stack.back();
      while (f.idx < f.nkeys) {
        const uint8_t* nd = e->node(f.page_off, f.idx);
        if (Env::cmp(nd + 8, rd<uint16_t>(nd + 6), key, klen) >= 0) { e->at_end = false; return 1; }
        ++f.idx;
      }
      if (!e->next_leaf()) return 0;
    }
  }
  e->at_end = false;
  return 1;
}

// Hand out the item under the cursor and advance. Returns 1, or 0 at the end.
int rb_lmdb_next(void* h, const uint8_t** key, uint32_t* klen, const uint8_t** val, uint64_t* vlen) {
  Env* e = static_cast<Env*>(h);
  if (e->at_end || e->stack.empty()) return 0;
  Frame& f = e->stack.back();
  const uint8_t* nd = e->node(f.page_off, f.idx);
  const uint16_t flags = rd<uint16_t>(nd + 4), ks = rd<uint16_t>(nd + 6);
  const uint64_t dsize = (uint64_t)rd<uint16_t>(nd) | ((uint64_t)rd<uint16_t>(nd + 2) << 16);
  *key = nd + 8;
  *klen = ks;
  const uint8_t* data = nd + 8 + ks;
  if (flags & kBigData) {
    const uint64_t opg = rd<uint64_t>(data);
    if (opg * e->psize + kHdr + dsize > e->size) { e->at_end = true; return 0; }
    data = e->m + opg * e->psize + kHdr;
  }
  *val = data;
  *vlen = dsize;
  if (++f.idx >= f.nkeys && !e->next_leaf()) e->at_end = true;
  return 1;
}

void rb_lmdb_close(void* h) {
  Env* e = static_cast<Env*>(h);
  if (!e) return;
  munmap(const_cast<uint8_t*>(e->m), e->size);
  close(e->fd);
  delete e;
}

}  // extern "C"
