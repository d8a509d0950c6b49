// Input pipeline on the GPU: one pass from staged u8 images (planar, [N][C][H][W], the reference's
// "WHC bytes, first dimension fastest") to the bf16 NHWC tensor the first convolution reads:
//   u8 -> float (optionally /255) -> subtract element-wise mean -> random / centre crop (with zero
//   padding for negative offsets) -> horizontal flip -> PCA lighting noise -> optional space-to-depth.
// Covers the reference's cast_bytes[_normalized], cuDNN strided-transform crop, batch_blockmap256_flip,
// cuDNN add-tensor mean subtraction and batch_map_preproc_pca3_noise (src/operator/mod.rs:653-778,
// src/operator/input.rs:288-419) in a single kernel. Crop offsets and flip coins are per sample by
// default; `per_batch` reproduces the reference's one-draw-per-batch behaviour.
//
// Space-to-depth by f (used for strided first layers): output pixel (Y,X) holds the f*f*C values of
// source pixels (Y*f+dy, X*f+dx), channel = (dy*f+dx)*C + c, so an s-strided k x k convolution becomes
// a stride-1 ceil(k/f) x ceil(k/f) convolution on f*f*C channels.
#include "launch.cuh"
#include "common.cuh"

namespace rb {

struct InputArgs {
  const uint8_t* src;   // [N][C][H][W]
  const float* mean;    // optional [C][H][W]
  bf16* dst;            // [N][OH][OW][Cp]
  int N, C, H, W;
  int crop_h, crop_w;   // extent of the crop window
  int OH, OW, Cp, f;
  int lo_y, hi_y, lo_x, hi_x;  // inclusive range of the window's top-left corner (may be negative)
  int random_crop, random_flip, per_batch;
  float scale;          // 1/255 when normalising, else 1
  float mean_scale;     // multiplies the mean before subtraction
  float pca_sigma;      // 0 disables
  float pca_vals[3];
  float pca_vecs[9];    // row c, column j
  uint64_t seed;
  uint32_t step;
  const uint32_t* step_ptr;  // optional device counter added to `step` (keeps captured graphs fresh)
};

__device__ __forceinline__ void sample_draw(const InputArgs& a, int n, int& oy, int& ox, int& flip, float (&shift)[3]) {
  uint32_t r[4];
  const uint32_t step = a.step + (a.step_ptr ? *a.step_ptr : 0u);
  Philox::gen(a.seed, a.per_batch ? 0ull : (uint64_t)n, step, r);
  if (a.random_crop) {
    oy = a.lo_y + (int)(r[0] % (uint32_t)(a.hi_y - a.lo_y + 1));
    ox = a.lo_x + (int)(r[1] % (uint32_t)(a.hi_x - a.lo_x + 1));
  } else {
    oy = (a.lo_y + a.hi_y) / 2;
    ox = (a.lo_x + a.hi_x) / 2;
  }
  flip = a.random_flip ? (int)(r[2] & 1u) : 0;
  shift[0] = shift[1] = shift[2] = 0.f;
  if (a.pca_sigma > 0.f && a.C == 3) {
    uint32_t q[4];
    Philox::gen(a.seed ^ 0x5bd1e995ull, (uint64_t)n, step, q);
    // Box-Muller: three normals from four uniforms
    const float u0 = fmaxf(u32_to_unit(q[0]), 1e-7f), u1 = u32_to_unit(q[1]);
    const float u2 = fmaxf(u32_to_unit(q[2]), 1e-7f), u3 = u32_to_unit(q[3]);
    const float m0 = sqrtf(-2.f * __logf(u0)), m1 = sqrtf(-2.f * __logf(u2));
    const float al[3] = {a.pca_sigma * m0 * __cosf(6.2831853f * u1), a.pca_sigma * m0 * __sinf(6.2831853f * u1),
                         a.pca_sigma * m1 * __cosf(6.2831853f * u3)};
#pragma unroll
    for (int c = 0; c < 3; ++c)
      shift[c] = al[0] * a.pca_vals[0] * a.pca_vecs[c * 3 + 0] + al[1] * a.pca_vals[1] * a.pca_vecs[c * 3 + 1] +
                 al[2] * a.pca_vals[2] * a.pca_vecs[c * 3 + 2];
  }
}

__global__ void input_kernel(InputArgs a) {
  pdl_prolog();
  const int groups = a.Cp / 8;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int gidx = (int)(i % groups);
    long long t = i / groups;
    const int X = (int)(t % a.OW); t /= a.OW;
    const int Y = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    int oy, ox, flip;
    float shift[3];
    sample_draw(a, n, oy, ox, flip, shift);
    float out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ch = gidx * 8 + j;
      float v = 0.f;
      const int blk = ch / a.C, c = ch - blk * a.C;
      if (blk < a.f * a.f) {
        const int dy = blk / a.f, dx = blk - dy * a.f;
        const int y = Y * a.f + dy;
        int x = X * a.f + dx;
        if (y < a.crop_h && x < a.crop_w) {
          if (flip) x = a.crop_w - 1 - x;
          const int sy = oy + y, sx = ox + x;
          if (sy >= 0 && sy < a.H && sx >= 0 && sx < a.W) {
            const long long si = ((long long)c * a.H + sy) * a.W + sx;
            v = (float)a.src[(long long)n * a.C * a.H * a.W + si] * a.scale;
            if (a.mean) v -= a.mean_scale * a.mean[si];
            if (c < 3) v += shift[c];
          }
        }
      }
      out[j] = v;
    }
    store8(a.dst + i * 8, out);
  }
}

// Row-staged variant: one block per (sample, output row). The f source rows of every channel are read with
// coalesced byte loads, converted (scale, mean, lighting shift, crop / flip / zero padding) into shared memory
// as floats, then written out as 16-byte channel groups. The per-sample random draw is computed once per block.
__global__ void __launch_bounds__(256) input_rows_kernel(InputArgs a) {
  pdl_prolog();
  extern __shared__ float srow[];  // [f][C][seg_w]
  __shared__ int s_draw[3];
  __shared__ float s_shift[3];
  const int n = blockIdx.x / a.OH, Y = blockIdx.x % a.OH;
  if (threadIdx.x == 0) {
    int oy, ox, flip;
    float shift[3];
    sample_draw(a, n, oy, ox, flip, shift);
    s_draw[0] = oy; s_draw[1] = ox; s_draw[2] = flip;
    s_shift[0] = shift[0]; s_shift[1] = shift[1]; s_shift[2] = shift[2];
  }
  __syncthreads();
  const int oy = s_draw[0], ox = s_draw[1], flip = s_draw[2];
  const int seg_w = a.OW * a.f;
  const uint8_t* img = a.src + (long long)n * a.C * a.H * a.W;
  // phase 1: (source row dy, channel c) lines, threads stride along x. No per-element divisions; the loads of two
  // source rows (up to 8 lines) are issued before any of them is used, because a block moves only a few KB and
  // what it costs is load latency and instruction count, not bandwidth.
  const int Cn = a.C < 4 ? a.C : 4;
  if (a.C <= 4) {
    for (int dy0 = 0; dy0 < a.f; dy0 += 2) {
      for (int xc = threadIdx.x; xc < seg_w; xc += blockDim.x) {
        const int sx = ox + (flip ? a.crop_w - 1 - xc : xc);
        const bool col_in = xc < a.crop_w && sx >= 0 && sx < a.W;
        uint8_t px[8];
        float mu[8];
        bool ok[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int dy = dy0 + (u >> 2), c = u & 3;
          const int y = Y * a.f + dy;
          const int sy = oy + y;
          ok[u] = dy < a.f && c < Cn && col_in && y < a.crop_h && sy >= 0 && sy < a.H;
          px[u] = 0;
          mu[u] = 0.f;
          if (ok[u]) {
            const int idx = (c * a.H + sy) * a.W + sx;
            px[u] = img[idx];
            if (a.mean) mu[u] = a.mean[idx];
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int dy = dy0 + (u >> 2), c = u & 3;
          if (dy < a.f && c < Cn) {
            float v = 0.f;
            if (ok[u]) v = (float)px[u] * a.scale - a.mean_scale * mu[u] + (c < 3 ? s_shift[c] : 0.f);
            srow[(dy * a.C + c) * seg_w + xc] = v;
          }
        }
      }
    }
  } else {
    for (int line = 0; line < a.f * a.C; ++line) {
      const int dy = line / a.C, c = line - dy * a.C;
      const int y = Y * a.f + dy;
      const int sy = oy + y;
      const bool row_in = y < a.crop_h && sy >= 0 && sy < a.H;
      const long long rbase = ((long long)c * a.H + sy) * a.W;
      for (int xc = threadIdx.x; xc < seg_w; xc += blockDim.x) {
        float v = 0.f;
        const int sx = ox + (flip ? a.crop_w - 1 - xc : xc);
        if (row_in && xc < a.crop_w && sx >= 0 && sx < a.W) {
          v = (float)img[rbase + sx] * a.scale;
          if (a.mean) v -= a.mean_scale * a.mean[rbase + sx];
          if (c < 3) v += s_shift[c];
        }
        srow[line * seg_w + xc] = v;
      }
    }
  }
  // channel -> offset of its source line in shared memory (or -1 for padded channels), built once per block
  __shared__ int s_tab[512];
  const int ff = a.f * a.f;
  for (int ch = threadIdx.x; ch < a.Cp && ch < 512; ch += blockDim.x) {
    const int blk = ch / a.C, c = ch - blk * a.C;
    int off = -1;
    if (blk < ff) {
      const int dy = blk / a.f, dx = blk - dy * a.f;
      off = (dy * a.C + c) * seg_w + dx;
    }
    s_tab[ch] = off;
  }
  __syncthreads();
  const int groups = a.Cp / 8;
  bf16* drow = a.dst + ((long long)n * a.OH + Y) * a.OW * a.Cp;
  const int gshift = (groups & (groups - 1)) == 0 ? __ffs(groups) - 1 : -1;
  for (int i = threadIdx.x; i < a.OW * groups; i += blockDim.x) {
    const int X = gshift >= 0 ? (i >> gshift) : i / groups, g = i - X * groups;
    const int xoff = X * a.f;
    float out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int off = s_tab[g * 8 + j];
      out[j] = off >= 0 ? srow[off + xoff] : 0.f;
    }
    store8(drow + (long long)i * 8, out);
  }
}

// Synthetic N(0,1) activations (bf16, padded channels zero) and uniform labels, generated on the device.
__global__ void synth_normal_kernel(bf16* __restrict__ dst, long long pixels, int C, int Cp, uint64_t seed,
                                    uint32_t step) {
  pdl_prolog();
  const long long total = pixels * Cp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total / 4;
       i += (long long)gridDim.x * blockDim.x) {
    uint32_t r[4];
    Philox::gen(seed, (uint64_t)i, step, r);
    const float u0 = fmaxf(u32_to_unit(r[0]), 1e-7f), u1 = u32_to_unit(r[1]);
    const float u2 = fmaxf(u32_to_unit(r[2]), 1e-7f), u3 = u32_to_unit(r[3]);
    const float m0 = sqrtf(-2.f * __logf(u0)), m1 = sqrtf(-2.f * __logf(u2));
    float z[4] = {m0 * __cosf(6.2831853f * u1), m0 * __sinf(6.2831853f * u1), m1 * __cosf(6.2831853f * u3),
                  m1 * __sinf(6.2831853f * u3)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = i * 4 + j;
      const int c = (int)(e % Cp);
      dst[e] = f2bf(c < C ? z[j] : 0.f);
    }
  }
}

__global__ void synth_labels_kernel(int* __restrict__ labels, int n, int classes, uint64_t seed, uint32_t step) {
  pdl_prolog();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t r[4];
  Philox::gen(seed ^ 0x9e3779b97f4a7c15ull, (uint64_t)i, step, r);
  labels[i] = (int)(r[0] % (uint32_t)classes);
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_input_u8(const void* src, const float* mean, void* dst, int N, int C, int H, int W, int crop_h, int crop_w,
                int OH, int OW, int Cp, int f, int lo_y, int hi_y, int lo_x, int hi_x, int random_crop,
                int random_flip, int per_batch, float scale, float mean_scale, float pca_sigma, const float* pca_vals,
                const float* pca_vecs, unsigned long long seed, unsigned int step, const unsigned int* step_ptr,
                cudaStream_t st) {
  if (Cp % 8) return -10;
  InputArgs a;
  a.src = (const uint8_t*)src; a.mean = mean; a.dst = (bf16*)dst;
  a.N = N; a.C = C; a.H = H; a.W = W; a.crop_h = crop_h; a.crop_w = crop_w;
  a.OH = OH; a.OW = OW; a.Cp = Cp; a.f = f;
  a.lo_y = lo_y; a.hi_y = hi_y; a.lo_x = lo_x; a.hi_x = hi_x;
  a.random_crop = random_crop; a.random_flip = random_flip; a.per_batch = per_batch;
  a.scale = scale; a.mean_scale = mean_scale; a.pca_sigma = pca_sigma;
  for (int i = 0; i < 3; ++i) a.pca_vals[i] = pca_vals ? pca_vals[i] : 0.f;
  for (int i = 0; i < 9; ++i) a.pca_vecs[i] = pca_vecs ? pca_vecs[i] : 0.f;
  a.seed = seed; a.step = step; a.step_ptr = step_ptr;
  const long long total = (long long)N * OH * OW * (Cp / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  const size_t row_smem = (size_t)f * C * OW * f * sizeof(float);
  if (row_smem <= 40 * 1024 && Cp <= 512 && (long long)N * OH < 0x7FFFFFFF) {
    launch_pdl(input_rows_kernel, N * OH, 256, row_smem, st, a);
  } else {
    launch_pdl(input_kernel, (int)blocks, 256, 0, st, a);
  }
  return RB_LAUNCH_OK();
}

int rb_synth_normal(void* dst, long long pixels, int C, int Cp, unsigned long long seed, unsigned int step,
                    cudaStream_t st) {
  if ((pixels * Cp) % 4) return -10;
  long long blocks = (pixels * Cp / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  launch_pdl(synth_normal_kernel, (int)blocks, 256, 0, st, (bf16*)dst, pixels, C, Cp, seed, step);
  return RB_LAUNCH_OK();
}

int rb_synth_labels(int* labels, int n, int classes, unsigned long long seed, unsigned int step, cudaStream_t st) {
  launch_pdl(synth_labels_kernel, (n + 255) / 256, 256, 0, st, labels, n, classes, seed, step);
  return RB_LAUNCH_OK();
}

}  // extern "C"
