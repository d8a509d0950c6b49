// Cross-channel local response normalisation, NHWC bf16.
//   s_i = k + alpha_eff * sum_{j in window(i)} x_j^2 ,  y_i = x_i * s_i^(-beta)
//   dx_i = dy_i * s_i^(-beta) - 2 alpha_eff beta x_i * sum_{j : i in window(j)} dy_j y_j / s_j
// The reference names the layer (`local_res_norm`, cross_size/scale/power/min_div in
// examples/imagenet_alexnet.model:30-36) but leaves it a pass-through stub (src/layer.rs:1846-1899);
// this is the real operator. One thread owns one pixel's channel chunk; the channel vector sits in
// shared memory so window sums are cheap.
#include "launch.cuh"
#include "common.cuh"

namespace rb {

constexpr int LRN_PIX = 8;  // pixels per block

__global__ void lrn_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long pixels, int C, int size,
                               float alpha_eff, float beta, float kconst) {
  pdl_prolog();
  extern __shared__ float sm[];  // LRN_PIX * C squares
  const int half_lo = size / 2, half_hi = (size - 1) / 2;
  const long long pix0 = (long long)blockIdx.x * LRN_PIX;
  const int per = C * LRN_PIX;
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const long long pix = pix0 + i / C;
    float v = 0.f;
    if (pix < pixels) v = bf2f(x[pix * C + (i % C)]);
    sm[i] = v;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const int pl = i / C, c = i % C;
    const long long pix = pix0 + pl;
    if (pix >= pixels) continue;
    const float* row = sm + pl * C;
    float acc = 0.f;
    const int lo = max(0, c - half_lo), hi = min(C - 1, c + half_hi);
    for (int j = lo; j <= hi; ++j) acc += row[j] * row[j];
    const float s = kconst + alpha_eff * acc;
    y[pix * C + c] = f2bf(row[c] * __powf(s, -beta));
  }
}

__global__ void lrn_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                               const bf16* __restrict__ mask_src, long long pixels, int C, int size, float alpha_eff,
                               float beta, float kconst) {
  pdl_prolog();
  extern __shared__ float sm[];  // per pixel: x[C], s[C], t[C] = dy*y/s
  const int half_lo = size / 2, half_hi = (size - 1) / 2;
  const long long pix0 = (long long)blockIdx.x * LRN_PIX;
  const int per = C * LRN_PIX;
  float* sx = sm;
  float* ss = sm + per;
  float* stt = sm + 2 * per;
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const long long pix = pix0 + i / C;
    sx[i] = pix < pixels ? bf2f(x[pix * C + (i % C)]) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const int pl = i / C, c = i % C;
    const long long pix = pix0 + pl;
    const float* row = sx + pl * C;
    float acc = 0.f;
    const int lo = max(0, c - half_lo), hi = min(C - 1, c + half_hi);
    for (int j = lo; j <= hi; ++j) acc += row[j] * row[j];
    const float s = kconst + alpha_eff * acc;
    ss[i] = s;
    float g = 0.f;
    if (pix < pixels) g = bf2f(dy[pix * C + c]);
    // y/s = x * s^(-beta-1)
    stt[i] = g * row[c] * __powf(s, -beta - 1.f);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const int pl = i / C, c = i % C;
    const long long pix = pix0 + pl;
    if (pix >= pixels) continue;
    const float* trow = stt + pl * C;
    // channels j whose window contains c: j - half_lo <= c <= j + half_hi
    const int lo = max(0, c - half_hi), hi = min(C - 1, c + half_lo);
    float acc = 0.f;
    for (int j = lo; j <= hi; ++j) acc += trow[j];
    const float g = bf2f(dy[pix * C + c]);
    float r = g * __powf(ss[i], -beta) - 2.f * alpha_eff * beta * sx[i] * acc;
    if (mask_src && !(bf2f(mask_src[pix * C + c]) > 0.f)) r = 0.f;
    dx[pix * C + c] = f2bf(r);
  }
}

// ---- fast path (window <= 9): one thread owns 8 consecutive channels of a pixel and keeps the 24-channel
// neighbourhood (previous / own / next 16-byte chunk) in registers; all accesses are 16-byte and coalesced.
__device__ __forceinline__ void load24(const bf16* base, long long chunk, int cv, int c8, float (&v)[24]) {
  float t[8];
  if (c8 > 0) { load8(base + (chunk - 1) * 8, t); } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = 0.f;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = t[j];
  load8(base + chunk * 8, t);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[8 + j] = t[j];
  if (c8 + 1 < cv) { load8(base + (chunk + 1) * 8, t); } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = 0.f;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[16 + j] = t[j];
}

template <int SIZE>
__global__ void lrn_fwd_vec_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, unsigned int chunks, int cv,
                                   float alpha_eff, float beta, float kconst) {
  pdl_prolog();
  constexpr int LO = SIZE / 2, HI = (SIZE - 1) / 2;
  for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += gridDim.x * blockDim.x) {
    const int c8 = (int)(i % (unsigned)cv);
    float v[24];
    load24(x, i, cv, c8, v);
    float sq[24];
#pragma unroll
    for (int j = 0; j < 24; ++j) sq[j] = v[j] * v[j];
    float out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float acc = 0.f;
#pragma unroll
      for (int d = -LO; d <= HI; ++d) acc += sq[8 + j + d];
      out[j] = v[8 + j] * __powf(kconst + alpha_eff * acc, -beta);
    }
    store8(y + (size_t)i * 8, out);
  }
}

template <int SIZE>
__global__ void lrn_bwd_vec_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                   const bf16* __restrict__ mask_src, unsigned int chunks, int cv, float alpha_eff,
                                   float beta, float kconst) {
  pdl_prolog();
  constexpr int LO = SIZE / 2, HI = (SIZE - 1) / 2;
  static_assert(LO + HI <= 8, "window too wide for the register path");
  for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += gridDim.x * blockDim.x) {
    const int c8 = (int)(i % (unsigned)cv);
    float v[24], g[24];
    load24(x, i, cv, c8, v);
    load24(dy, i, cv, c8, g);
    float sq[24];
#pragma unroll
    for (int j = 0; j < 24; ++j) sq[j] = v[j] * v[j];
    // t_j = dy_j * x_j * s_j^(-beta-1) for the channels whose window can contain one of ours
    float t[8 + LO + HI];
    float s_own[8];
#pragma unroll
    for (int q = 0; q < 8 + LO + HI; ++q) {
      const int j = 8 - HI + q;  // position in the 24-vector
      float acc = 0.f;
#pragma unroll
      for (int d = -LO; d <= HI; ++d) acc += sq[j + d];
      const float s = kconst + alpha_eff * acc;
      t[q] = g[j] * v[j] * __powf(s, -beta - 1.f);
      if (q >= HI && q < HI + 8) s_own[q - HI] = s;
    }
    float out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // channels c with j in window(c): c - LO <= j <= c + HI  ->  c in [j - HI, j + LO]
      float acc = 0.f;
#pragma unroll
      for (int d = -HI; d <= LO; ++d) acc += t[HI + j + d];
      out[j] = g[8 + j] * __powf(s_own[j], -beta) - 2.f * alpha_eff * beta * v[8 + j] * acc;
    }
    if (mask_src) {
      float m[8];
      load8(mask_src + (size_t)i * 8, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) out[j] = 0.f;
    }
    store8(dx + (size_t)i * 8, out);
  }
}

template <int SIZE>
static int launch_lrn_vec(const void* x, const void* dy, void* out, const void* mask_src, long long pixels, int C,
                          float alpha_eff, float beta, float kconst, bool backward, cudaStream_t st) {
  const unsigned int chunks = (unsigned int)(pixels * (C / 8));
  int blocks = (int)((chunks + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  if (backward)
    launch_pdl(lrn_bwd_vec_kernel<SIZE>, blocks, 256, 0, st, (const bf16*)x, (const bf16*)dy, (bf16*)out,
               (const bf16*)mask_src, chunks, C / 8, alpha_eff, beta, kconst);
  else
    launch_pdl(lrn_fwd_vec_kernel<SIZE>, blocks, 256, 0, st, (const bf16*)x, (bf16*)out, chunks, C / 8, alpha_eff,
               beta, kconst);
  return RB_LAUNCH_OK();
}

static bool lrn_vec_ok(long long pixels, int C, int size) {
  return (C % 8 == 0) && (size == 3 || size == 5 || size == 7 || size == 9) && pixels * (C / 8) < 0xFFFFFFFFll;
}

static int dispatch_lrn_vec(int size, const void* x, const void* dy, void* out, const void* mask_src, long long pixels,
                            int C, float a, float b, float k, bool backward, cudaStream_t st) {
  switch (size) {
    case 3: return launch_lrn_vec<3>(x, dy, out, mask_src, pixels, C, a, b, k, backward, st);
    case 5: return launch_lrn_vec<5>(x, dy, out, mask_src, pixels, C, a, b, k, backward, st);
    case 7: return launch_lrn_vec<7>(x, dy, out, mask_src, pixels, C, a, b, k, backward, st);
    default: return launch_lrn_vec<9>(x, dy, out, mask_src, pixels, C, a, b, k, backward, st);
  }
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_lrn_fwd(const void* x, void* y, long long pixels, int C, int size, float alpha_eff, float beta, float kconst,
               cudaStream_t st) {
  if (lrn_vec_ok(pixels, C, size))
    return dispatch_lrn_vec(size, x, nullptr, y, nullptr, pixels, C, alpha_eff, beta, kconst, false, st);
  const int blocks = (int)((pixels + LRN_PIX - 1) / LRN_PIX);
  const size_t smem = (size_t)LRN_PIX * C * sizeof(float);
  if (smem > 48 * 1024) return -10;
  launch_pdl(lrn_fwd_kernel, blocks, 256, smem, st, (const bf16*)x, (bf16*)y, pixels, C, size, alpha_eff, beta,
             kconst);
  return RB_LAUNCH_OK();
}

int rb_lrn_bwd(const void* x, const void* dy, void* dx, const void* mask_src, long long pixels, int C, int size,
               float alpha_eff, float beta, float kconst, cudaStream_t st) {
  if (lrn_vec_ok(pixels, C, size))
    return dispatch_lrn_vec(size, x, dy, dx, mask_src, pixels, C, alpha_eff, beta, kconst, true, st);
  const int blocks = (int)((pixels + LRN_PIX - 1) / LRN_PIX);
  const size_t smem = (size_t)3 * LRN_PIX * C * sizeof(float);
  if (smem > 48 * 1024) return -10;
  launch_pdl(lrn_bwd_kernel, blocks, 256, smem, st, (const bf16*)x, (const bf16*)dy, (bf16*)dx, (const bf16*)mask_src,
             pixels, C, size, alpha_eff, beta, kconst);
  return RB_LAUNCH_OK();
}

}  // extern "C"
