// C API of the CPU-side runtime library (no CUDA dependency).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- NdArray blob codec ------------------------------------------------------------------------------
// Record layout (evidence: tools/dump-array3d-header.rs:8-15 of the reference):
//   'N' 'D' tag0 tag1 | u32le ndim | u64le dim[ndim] | raw little-endian elements, first dimension fastest
// The element type is implied by context (f32 parameters and mean files, u8 images). The two tag bytes
// are opaque: they are returned on read and written back unchanged (default 0x00 0x01).
#define RB_BLOB_MAX_DIMS 8
typedef struct {
  uint8_t tag[2];
  uint32_t ndim;
  uint64_t dims[RB_BLOB_MAX_DIMS];
  uint64_t data_offset;   // offset of the first element inside the buffer
  uint64_t num_elems;
  uint64_t next_offset;   // offset of the record that follows
} rb_blob_record;

// Parse the record that starts at `offset`. Returns 0, or a negative code: -1 truncated header,
// -2 bad magic, -3 too many dimensions, -4 truncated data.
int rb_blob_parse(const uint8_t* buf, uint64_t len, uint64_t offset, uint32_t elem_size, rb_blob_record* out);
uint64_t rb_blob_record_size(uint32_t ndim, const uint64_t* dims, uint32_t elem_size);
// Serialise one record into `out` (capacity `cap`); returns bytes written or 0 if it does not fit.
uint64_t rb_blob_write(uint8_t* out, uint64_t cap, const uint8_t tag[2], uint32_t ndim, const uint64_t* dims,
                       const void* data, uint32_t elem_size);

// ---- xorshift128+ ---------------------------------------------------------------------------------
typedef struct { uint64_t s[2]; } rb_xorshift;
void rb_xs_seed(rb_xorshift* r, uint64_t s0, uint64_t s1);
uint64_t rb_xs_next(rb_xorshift* r);
double rb_xs_unit(rb_xorshift* r);                                 // [0,1)
void rb_xs_fill_uniform(rb_xorshift* r, float* out, uint64_t n, float lo, float hi);
void rb_xs_fill_normal(rb_xorshift* r, float* out, uint64_t n, float mean, float std);
void rb_xs_permutation(rb_xorshift* r, int32_t* out, int32_t n);   // Fisher-Yates
uint32_t rb_xs_below(rb_xorshift* r, uint32_t n);                  // uniform in [0,n)

// ---- partitioning (src/util.rs:3-41) -------------------------------------------------------------------
// Balanced contiguous split of [0,n) into `parts`; writes the bounds of part `idx`.
void rb_partition_range(uint64_t n, uint32_t parts, uint32_t idx, uint64_t* lo, uint64_t* hi);

// ---- dataset readers -----------------------------------------------------------------------------------
// IDX (MNIST): big-endian header {0,0,type,ndim} + ndim u32 dims. Returns 0 or negative on error.
int rb_idx_header(const uint8_t* buf, uint64_t len, uint32_t* dtype, uint32_t* ndim, uint32_t dims[4],
                  uint64_t* data_offset);
// CIFAR-10 binary: records of 1 label byte + 3072 planar RGB bytes. Splits `count` records starting at
// `first` into contiguous image and label arrays.
int rb_cifar_split(const uint8_t* buf, uint64_t len, uint64_t first, uint64_t count, uint8_t* images,
                   int32_t* labels);
// Per-pixel mean over u8 images laid out [n][elems]; accumulates in double.
void rb_mean_u8(const uint8_t* images, uint64_t n, uint64_t elems, float* mean_out);

// ---- prefetching batch loader (batch_loader.cc) -------------------------------------------------------
// Worker threads assemble batches of `batch` samples (u8 images of `elems` bytes + i32 labels) of the shard [lo, hi)
// into a ring of `nslots` caller-owned slots; the order of samples depends only on (mode, seed, position):
// mode 0 cyclic, 1 random with replacement, 2 shuffled epochs. Returns null on bad arguments.
void* rb_loader_create(const uint8_t* images, const int32_t* labels, uint64_t elems, uint64_t lo, uint64_t hi,
                       uint32_t batch, uint32_t mode, uint64_t seed, uint32_t threads, uint32_t nslots,
                       uint8_t** image_slots, int32_t** label_slots);
// The same loader over the raw images of a Caffe LMDB environment (records [lo, hi) in key order, pixel bytes copied
// straight from the memory mapping). *error: 1 cannot open, 2 malformed record, 3 encoded or wrong size, 4 arguments.
void* rb_loader_create_lmdb(const char* path, uint64_t elems, uint64_t lo, uint64_t hi, uint32_t batch, uint32_t mode,
                            uint64_t seed, uint32_t threads, uint32_t nslots, uint8_t** image_slots,
                            int32_t** label_slots, int32_t* error);
int rb_loader_acquire(void* handle, uint64_t* batch_number);   // blocks; slot index, or -1 after destroy
void rb_loader_release(void* handle, int slot);
void rb_loader_destroy(void* handle);
uint64_t rb_loader_sample_index(uint64_t lo, uint64_t hi, uint32_t mode, uint64_t seed, uint64_t pos);

// ---- read-only LMDB reader (lmdb_reader.cc) ------------------------------------------------------------
// `path` is the environment directory or its data file. Keys and values point into the memory mapping.
void* rb_lmdb_open(const char* path);                       // null on failure
uint64_t rb_lmdb_entries(void* env);
uint32_t rb_lmdb_depth(void* env);
uint32_t rb_lmdb_page_size(void* env);
int rb_lmdb_seek(void* env, const uint8_t* key, uint32_t klen);   // first key >= key (klen 0: first key); 1 if found
int rb_lmdb_next(void* env, const uint8_t** key, uint32_t* klen, const uint8_t** val, uint64_t* vlen);  // 1, or 0 at end
void rb_lmdb_close(void* env);

// ---- per-sample decoders (sample_codecs.cc) ------------------------------------------------------------
// Caffe `Datum` message (fields: 1 channels, 2 height, 3 width, 4 data, 5 label, 6 float_data, 7 encoded).
typedef struct {
  int32_t channels, height, width, label, encoded;
  uint64_t data_offset, data_len;   // the `data` bytes inside the message (not copied)
  uint64_t float_count;             // number of float_data values, packed or not
} rb_datum;
// 0, or negative: -1 truncated varint, -2 a field runs past the message, -3 packed floats of odd size, -4 wire type.
int rb_datum_parse(const uint8_t* buf, uint64_t len, rb_datum* out);
// Copies up to `cap` float_data values in message order; returns how many were written.
uint64_t rb_datum_floats(const uint8_t* buf, uint64_t len, float* out, uint64_t cap);
// Bit i of the packed stream (bit i % 8 of byte i / 8) -> out[i] = scale or 0. -1 if the stream is too short.
int rb_bits_unpack(const uint8_t* packed, uint64_t packed_len, uint64_t nbits, uint8_t scale, uint8_t* out);

#ifdef __cplusplus
}
#endif
