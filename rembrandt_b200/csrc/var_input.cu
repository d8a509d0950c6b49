// Variable-size input operator: every sample of the batch has its own source width and height. One kernel does
//   u8 -> float, Catmull-Rom (bicubic) rescale so that the shorter side becomes `scale_dim` (drawn per sample in
//   [scale_lower, scale_upper] when training, scale_lower at inference), crop of a crop_w x crop_h window (random
//   when training, centred at inference), horizontal flip, per-channel mean, PCA lighting noise, and the write into
//   the bf16 NHWC (or space-to-depth) tensor that the first convolution reads.
// Only the pixels of the crop window are ever interpolated: rescale and crop are fused, the rescaled image is never
// materialised. Covers VarData3dOperator's ScaleBicubic / Crop / FlipX / PCA-noise chain
// (src/operator/input.rs:288-464, kernels image3_catmullrom_scale, image3_crop, batch_blockmap256_flip).
//
// Source layout: sample n starts at src + n * in_stride and holds C planes of h x w bytes (x fastest), with
// (w, h) = shapes[n]. Taps outside the source image are clamped to its border; crop windows that reach outside the
// rescaled image (source too small) read zeros there.
#include "launch.cuh"
#include "common.cuh"

namespace rb {

struct VarInputArgs {
  const uint8_t* src;
  const int* shapes;   // [N][2] = (w, h)
  bf16* dst;           // nhwc: [N][crop_h][crop_w][Cp]; s2d: [N][OH][OW][Cp]
  int* draws;          // optional [N][4] = (scale_dim, offset_x, offset_y, flip), for inspection
  long long in_stride;
  int N, C, crop_h, crop_w, Cp;
  int f, ep, OH, OW;   // space-to-depth factor (1 = plain NHWC), absorbed convolution padding, output extent
  int scale_lower, scale_upper;  // 0 disables the rescale
  int train, random_flip, per_batch;
  float scale;         // multiplies the byte value
  float mean[4];       // per channel, subtracted after scaling
  float pca_sigma;
  float pca_vals[3];
  float pca_vecs[9];
  uint64_t seed;
  uint32_t step;
  const uint32_t* step_ptr;
};

__device__ __forceinline__ void catmull_rom(float t, float (&w)[4]) {
  const float t2 = t * t, t3 = t2 * t;
  w[0] = -0.5f * t3 + t2 - 0.5f * t;
  w[1] = 1.5f * t3 - 2.5f * t2 + 1.f;
  w[2] = -1.5f * t3 + 2.f * t2 + 0.5f * t;
  w[3] = 0.5f * t3 - 0.5f * t2;
}

__global__ void __launch_bounds__(256) var_input_kernel(const __grid_constant__ VarInputArgs a) {
  pdl_prolog();
  const long long total = (long long)a.N * a.crop_h * a.crop_w;
  const uint32_t step = a.step + (a.step_ptr ? *a.step_ptr : 0u);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % a.crop_w);
    const long long t0 = i / a.crop_w;
    const int y = (int)(t0 % a.crop_h);
    const int n = (int)(t0 / a.crop_h);
    const int w = a.shapes[n * 2 + 0], h = a.shapes[n * 2 + 1];
    uint32_t r[4];
    Philox::gen(a.seed, a.per_batch ? 0ull : (uint64_t)n, step, r);
    // rescaled extent (the reference's rounding: shorter side = scale_dim exactly)
    int rw = w, rh = h;
    int sdim = 0;
    if (a.scale_lower > 0) {
      sdim = a.train ? a.scale_lower + (int)(r[3] % (uint32_t)(a.scale_upper - a.scale_lower + 1)) : a.scale_lower;
      if (w <= h) {
        rw = sdim;
        rh = (int)rintf((float)sdim / (float)w * (float)h);
      } else {
        rw = (int)rintf((float)sdim / (float)h * (float)w);
        rh = sdim;
      }
    }
    int ox, oy;
    if (a.train && rw > a.crop_w) ox = (int)(r[0] % (uint32_t)(rw - a.crop_w + 1));
    else ox = (rw - a.crop_w) / 2;
    if (a.train && rh > a.crop_h) oy = (int)(r[1] % (uint32_t)(rh - a.crop_h + 1));
    else oy = (rh - a.crop_h) / 2;
    const int flip = (a.train && a.random_flip) ? (int)(r[2] & 1u) : 0;
    if (a.draws && x == 0 && y == 0) {
      a.draws[n * 4 + 0] = sdim; a.draws[n * 4 + 1] = ox; a.draws[n * 4 + 2] = oy; a.draws[n * 4 + 3] = flip;
    }
    float shift[3] = {0.f, 0.f, 0.f};
    if (a.train && a.pca_sigma > 0.f && a.C == 3) {
      uint32_t q[4];
      Philox::gen(a.seed ^ 0x5bd1e995ull, (uint64_t)n, step, q);
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
    // position in the rescaled image
    const int X = ox + (flip ? a.crop_w - 1 - x : x), Y = oy + y;
    const bool inside = X >= 0 && X < rw && Y >= 0 && Y < rh;
    float val[4] = {0.f, 0.f, 0.f, 0.f};
    if (inside) {
      const uint8_t* img = a.src + (long long)n * a.in_stride;
      if (rw == w && rh == h) {
        for (int c = 0; c < a.C; ++c) val[c] = (float)img[((long long)c * h + Y) * w + X];
      } else {
        const float fx = ((float)X + 0.5f) * ((float)w / (float)rw) - 0.5f;
        const float fy = ((float)Y + 0.5f) * ((float)h / (float)rh) - 0.5f;
        const float flx = floorf(fx), fly = floorf(fy);
        float wx[4], wy[4];
        catmull_rom(fx - flx, wx);
        catmull_rom(fy - fly, wy);
        int xi[4], yi[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          xi[k] = min(max((int)flx - 1 + k, 0), w - 1);
          yi[k] = min(max((int)fly - 1 + k, 0), h - 1);
        }
        for (int c = 0; c < a.C; ++c) {
          const uint8_t* pl = img + (long long)c * h * w;
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint8_t* row = pl + (long long)yi[j] * w;
            const float rsum = wx[0] * (float)row[xi[0]] + wx[1] * (float)row[xi[1]] + wx[2] * (float)row[xi[2]] +
                               wx[3] * (float)row[xi[3]];
            acc += wy[j] * rsum;
          }
          val[c] = fminf(fmaxf(acc, 0.f), 255.f);
        }
      }
      for (int c = 0; c < a.C; ++c) val[c] = val[c] * a.scale - a.mean[c] + (c < 3 ? shift[c] : 0.f);
    }
    // write: plain NHWC, or the space-to-depth position of (y + ep, x + ep)
    if (a.f == 1) {
      bf16* o = a.dst + (((long long)n * a.crop_h + y) * a.crop_w + x) * a.Cp;
      for (int c = 0; c < a.C; ++c) o[c] = __float2bfloat16(val[c]);
    } else {
      const int yy = y + a.ep, xx = x + a.ep;
      const int OY = yy / a.f, dy = yy - OY * a.f, OX = xx / a.f, dx = xx - OX * a.f;
      if (OY < a.OH && OX < a.OW) {
        bf16* o = a.dst + (((long long)n * a.OH + OY) * a.OW + OX) * a.Cp + (dy * a.f + dx) * a.C;
        for (int c = 0; c < a.C; ++c) o[c] = __float2bfloat16(val[c]);
      }
    }
  }
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_var_input_u8(const void* src, const int* shapes, void* dst, int* draws, long long in_stride, int N, int C,
                    int crop_h, int crop_w, int Cp, int f, int ep, int OH, int OW, int scale_lower, int scale_upper,
                    int train, int random_flip, int per_batch, float scale, const float* mean, float pca_sigma,
                    const float* pca_vals, const float* pca_vecs, unsigned long long seed, unsigned int step,
                    const unsigned int* step_ptr, cudaStream_t st) {
  if (C < 1 || C > 4 || Cp < C || f < 1 || (scale_lower > 0 && scale_upper < scale_lower)) return -10;
  if (f > 1 && f * f * C > Cp) return -10;
  VarInputArgs a;
  a.src = (const uint8_t*)src; a.shapes = shapes; a.dst = (bf16*)dst; a.draws = draws; a.in_stride = in_stride;
  a.N = N; a.C = C; a.crop_h = crop_h; a.crop_w = crop_w; a.Cp = Cp; a.f = f; a.ep = ep; a.OH = OH; a.OW = OW;
  a.scale_lower = scale_lower; a.scale_upper = scale_upper; a.train = train; a.random_flip = random_flip;
  a.per_batch = per_batch; a.scale = scale; a.pca_sigma = pca_sigma;
  for (int i = 0; i < 4; ++i) a.mean[i] = (mean && i < C) ? mean[i] : 0.f;
  for (int i = 0; i < 3; ++i) a.pca_vals[i] = pca_vals ? pca_vals[i] : 0.f;
  for (int i = 0; i < 9; ++i) a.pca_vecs[i] = pca_vecs ? pca_vecs[i] : 0.f;
  a.seed = seed; a.step = step; a.step_ptr = step_ptr;
  const long long total = (long long)N * crop_h * crop_w;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  launch_pdl(var_input_kernel, (int)blocks, 256, 0, st, a);
  return RB_LAUNCH_OK();
}

}  // extern "C"
