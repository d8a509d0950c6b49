// Prefetching batch loader for in-memory (memory-mapped) fixed-size datasets: worker threads assemble batches of
// u8 images + i32 labels straight into a ring of caller-owned (pinned) slots while the training loop consumes
// earlier ones. Counterpart of the reference's AsyncQueueDataIter / AsyncPoolDataIter (src/data/mod.rs:273-640:
// one prefetch thread with a bounded queue, or N transform threads with the order restored).
//
// Sample order is a pure function of (seed, batch number, position), never of thread timing:
//   mode 0  cyclic      sample = lo + (batch * B + i) mod (hi - lo)
//   mode 1  random      sample = lo + hash(seed, batch * B + i) mod (hi - lo)          (with replacement)
//   mode 2  shuffled    epoch e = (batch * B + i) / len walks a permutation of [lo, hi) seeded by (seed, e)
// Batches are delivered in order (batch k before k + 1) whatever the number of threads.
#include "rembrandt_host.h"

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <numeric>
#include <thread>
#include <vector>

namespace {

inline uint64_t mix64(uint64_t x) {   // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

struct Loader {
  const uint8_t* images = nullptr;
  const int32_t* labels = nullptr;
  // gather form: one pointer per sample instead of one contiguous array (records of a memory-mapped database)
  std::vector<const uint8_t*> sample_ptrs;
  std::vector<int32_t> sample_labels;
  void* owned_env = nullptr;   // LMDB environment kept open for the lifetime of the loader
  uint64_t elems, lo, hi, seed;
  uint32_t batch, nslots, mode;
  std::vector<uint8_t*> img_slots;
  std::vector<int32_t*> lbl_slots;

  std::mutex mu;
  std::condition_variable cv_ready, cv_free;
  uint64_t next_to_fill = 0;     // next batch number a worker will take
  uint64_t next_to_give = 0;     // next batch number the consumer receives
  std::vector<int> state;        // per slot: 0 free, 1 being filled, 2 ready, 3 held by the consumer
  std::vector<uint64_t> slot_batch;
  bool stop = false;
  std::vector<std::thread> workers;

  // permutation cache for mode 2 (one epoch at a time per worker call; small datasets only pay n * 8 bytes)
  std::mutex perm_mu;
  uint64_t perm_epoch = ~0ull;
  std::vector<uint64_t> perm;

  uint64_t sample_index(uint64_t pos) {
    const uint64_t len = hi - lo;
    if (mode == 0) return lo + pos % len;
    if (mode == 1) return lo + mix64(seed ^ mix64(pos)) % len;
    const uint64_t epoch = pos / len, k = pos % len;
    std::lock_guard<std::mutex> g(perm_mu);
    if (perm_epoch != epoch) {
      perm.resize(len);
      std::iota(perm.begin(), perm.end(), 0ull);
      uint64_t s = mix64(seed ^ mix64(epoch + 0x51ull));
      for (uint64_t i = len - 1; i > 0; --i) {   // Fisher-Yates with a counter-based generator
        s = mix64(s + i);
        std::swap(perm[i], perm[s % (i + 1)]);
      }
      perm_epoch = epoch;
    }
    return lo + perm[k];
  }

  void fill(uint32_t slot, uint64_t b) {
    for (uint32_t i = 0; i < batch; ++i) {
      const uint64_t idx = sample_index(b * batch + i);
      if (sample_ptrs.empty()) {
        std::memcpy(img_slots[slot] + (uint64_t)i * elems, images + idx * elems, elems);
        lbl_slots[slot][i] = labels ? labels[idx] : 0;
      } else {
        std::memcpy(img_slots[slot] + (uint64_t)i * elems, sample_ptrs[idx], elems);
        lbl_slots[slot][i] = sample_labels[idx];
      }
    }
  }

  void run() {
    for (;;) {
      uint32_t slot = 0;
      uint64_t b = 0;
      {
        std::unique_lock<std::mutex> lk(mu);
        // a batch may only go into the slot that the in-order consumer will look at for it: slot = b mod nslots
        cv_free.wait(lk, [&] { return stop || state[next_to_fill % nslots] == 0; });
        if (stop) return;
        b = next_to_fill++;
        slot = (uint32_t)(b % nslots);
        state[slot] = 1;
        slot_batch[slot] = b;
      }
      fill(slot, b);
      {
        std::lock_guard<std::mutex> lk(mu);
        state[slot] = 2;
      }
      cv_ready.notify_all();
      cv_free.notify_all();   // another worker may be waiting for the next slot to be taken
    }
  }
};

}  // namespace

extern "C" {

void* rb_loader_create(const uint8_t* images, const int32_t* labels, uint64_t elems, uint64_t lo, uint64_t hi,
                       uint32_t batch, uint32_t mode, uint64_t seed, uint32_t threads, uint32_t nslots,
                       uint8_t** image_slots, int32_t** label_slots) {
  if (!images || hi <= lo || batch == 0 || nslots < 2 || threads == 0 || mode > 2 || !image_slots || !label_slots)
    return nullptr;
  Loader* L = new Loader();
  L->images = images; L->labels = labels; L->elems = elems; L->lo = lo; L->hi = hi; L->seed = seed;
  L->batch = batch; L->nslots = nslots; L->mode = mode;
  L->img_slots.assign(image_slots, image_slots + nslots);
  L->lbl_slots.assign(label_slots, label_slots + nslots);
  L->state.assign(nslots, 0);
  L->slot_batch.assign(nslots, 0);
  for (uint32_t t = 0; t < threads; ++t) L->workers.emplace_back([L] { L->run(); });
  return L;
}

// A loader over the raw (not encoded) images of a Caffe database: the environment is walked once at creation, every
// `Datum` is parsed in place, and the workers copy pixel bytes straight from the memory mapping into the slots.
// Records [lo, hi) in key order form the shard. `elems` must equal channels * height * width of every record.
// On failure returns null and stores a reason in *error: 1 cannot open, 2 malformed record, 3 encoded or wrong size,
// 4 bad arguments.
void* rb_loader_create_lmdb(const char* path, uint64_t elems, uint64_t lo, uint64_t hi, uint32_t batch, uint32_t mode,
                            uint64_t seed, uint32_t threads, uint32_t nslots, uint8_t** image_slots,
                            int32_t** label_slots, int32_t* error) {
  int32_t dummy;
  if (!error) error = &dummy;
  *error = 4;
  if (!path || batch == 0 || nslots < 2 || threads == 0 || mode > 2 || !image_slots || !label_slots) return nullptr;
  void* env = rb_lmdb_open(path);
  if (!env) { *error = 1; return nullptr; }
  Loader* L = new Loader();
  L->owned_env = env;
  const uint64_t total = rb_lmdb_entries(env);
  if (hi > total) hi = total;
  const uint8_t *k, *v;
  uint32_t kl;
  uint64_t vl, n = 0;
  bool ok = hi > lo && rb_lmdb_seek(env, nullptr, 0) == 1;
  *error = ok ? 0 : 4;
  while (ok && n < hi && rb_lmdb_next(env, &k, &kl, &v, &vl)) {
    if (n++ < lo) continue;
    rb_datum d;
    if (rb_datum_parse(v, vl, &d) != 0) { *error = 2; ok = false; break; }
    if (d.encoded || d.data_len != elems) { *error = 3; ok = false; break; }
    L->sample_ptrs.push_back(v + d.data_offset);
    L->sample_labels.push_back(d.label);
  }
  if (ok && L->sample_ptrs.size() != hi - lo) { *error = 2; ok = false; }
  if (!ok) {
    rb_lmdb_close(env);
    delete L;
    return nullptr;
  }
  L->elems = elems; L->lo = 0; L->hi = L->sample_ptrs.size(); L->seed = seed;
  L->batch = batch; L->nslots = nslots; L->mode = mode;
  L->img_slots.assign(image_slots, image_slots + nslots);
  L->lbl_slots.assign(label_slots, label_slots + nslots);
  L->state.assign(nslots, 0);
  L->slot_batch.assign(nslots, 0);
  for (uint32_t t = 0; t < threads; ++t) L->workers.emplace_back([L] { L->run(); });
  return L;
}

// Blocks until the next batch (in order) is ready; returns its slot, which stays valid until it is released.
int rb_loader_acquire(void* handle, uint64_t* batch_number) {
  Loader* L = static_cast<Loader*>(handle);
  std::unique_lock<std::mutex> lk(L->mu);
  const uint32_t slot = (uint32_t)(L->next_to_give % L->nslots);
  L->cv_ready.wait(lk, [&] { return L->stop || (L->state[slot] == 2 && L->slot_batch[slot] == L->next_to_give); });
  if (L->stop) return -1;
  L->state[slot] = 3;
  if (batch_number) *batch_number = L->next_to_give;
  ++L->next_to_give;
  return (int)slot;
}

void rb_loader_release(void* handle, int slot) {
  Loader* L = static_cast<Loader*>(handle);
  {
    std::lock_guard<std::mutex> lk(L->mu);
    if (slot >= 0 && (uint32_t)slot < L->nslots && L->state[slot] == 3) L->state[slot] = 0;
  }
  L->cv_free.notify_all();
}

void rb_loader_destroy(void* handle) {
  Loader* L = static_cast<Loader*>(handle);
  if (!L) return;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv_free.notify_all();
  L->cv_ready.notify_all();
  for (auto& t : L->workers) t.join();
  if (L->owned_env) rb_lmdb_close(L->owned_env);
  delete L;
}

// The sample a loader with these settings reads at stream position `pos` (for tests and for resuming).
uint64_t rb_loader_sample_index(uint64_t lo, uint64_t hi, uint32_t mode, uint64_t seed, uint64_t pos) {
  Loader L;
  L.lo = lo; L.hi = hi; L.mode = mode; L.seed = seed;
  return L.sample_index(pos);
}

}  // extern "C"
