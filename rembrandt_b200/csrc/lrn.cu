// Cross-channel local response normalisation, NHWC bf16.
//   s_i = k + alpha_eff * sum_{j in window(i)} x_j^2 ,  y_i = x_i * s_i^(-beta)
//   dx_i = dy_i * s_i^(-beta) - 2 alpha_eff beta x_i * sum_{j : i in window(j)} dy_j y_j / s_j
// The reference names the layer (`local_res_norm`, cross_size/scale/power/min_div in
// examples/imagenet_alexnet.model:30-36) but leaves it a pass-through stub (src/layer.rs:1846-1899);
// this is the real operator. One thread owns one pixel's channel chunk; the channel vector sits in
// shared memory so window sums are cheap.
#include "common.cuh"

namespace rb {

constexpr int LRN_PIX = 8;  // pixels per block

__global__ void lrn_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long pixels, int C, int size,
                               float alpha_eff, float beta, float kconst) {
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

}  // namespace rb

using namespace rb;

extern "C" {

int rb_lrn_fwd(const void* x, void* y, long long pixels, int C, int size, float alpha_eff, float beta, float kconst,
               cudaStream_t st) {
  const int blocks = (int)((pixels + LRN_PIX - 1) / LRN_PIX);
  const size_t smem = (size_t)LRN_PIX * C * sizeof(float);
  if (smem > 48 * 1024) return -10;
  lrn_fwd_kernel<<<blocks, 256, smem, st>>>((const bf16*)x, (bf16*)y, pixels, C, size, alpha_eff, beta, kconst);
  return RB_LAUNCH_OK();
}

int rb_lrn_bwd(const void* x, const void* dy, void* dx, const void* mask_src, long long pixels, int C, int size,
               float alpha_eff, float beta, float kconst, cudaStream_t st) {
  const int blocks = (int)((pixels + LRN_PIX - 1) / LRN_PIX);
  const size_t smem = (size_t)3 * LRN_PIX * C * sizeof(float);
  if (smem > 48 * 1024) return -10;
  lrn_bwd_kernel<<<blocks, 256, smem, st>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, (const bf16*)mask_src, pixels,
                                            C, size, alpha_eff, beta, kconst);
  return RB_LAUNCH_OK();
}

}  // extern "C"
