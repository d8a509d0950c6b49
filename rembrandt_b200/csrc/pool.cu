// Max / average pooling, forward and backward, NHWC bf16, 8 channels per thread (16-byte accesses).
// Output extent is given by the caller (floor or ceil rounding both occur in the reference:
// src/operator/mod.rs:2022-2027 floor, src/layer.rs:1741-1747 ceil). Average pooling divides by the
// full window size (padding counted), as cuDNN's AverageCountIncludingPadding does
// (src/operator/mod.rs:2053-2066). Max pooling records the window offset of the (first) maximum in
// one byte per output so that the backward pass is an exact gather with no atomics.
#include "common.cuh"

namespace rb {

template <typename IT>
__global__ void maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ idx, int N,
                                   int H, int W, int C, int P, int Q, int k, int stride, int pad, int relu) {
  const int cv = C / 8;
  const IT total = (IT)N * P * Q * cv;
  for (IT i = (IT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IT)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % cv);
    IT t = i / cv;
    const int q = (int)(t % Q); t /= Q;
    const int p = (int)(t % P);
    const int n = (int)(t / P);
    float best[8];
    int bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; bi[j] = 0; }
    const int h0 = p * stride - pad, w0 = q * stride - pad;
    for (int r = 0; r < k; ++r) {
      const int h = h0 + r;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < k; ++s) {
        const int w = w0 + s;
        if (w < 0 || w >= W) continue;
        float v[8];
        load8(x + (((long long)n * H + h) * W + w) * C + c8 * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v[j] > best[j]) { best[j] = v[j]; bi[j] = r * k + s; }
      }
    }
    const long long o = (((long long)n * P + p) * Q + q) * C + c8 * 8;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (best[j] == -INFINITY) best[j] = 0.f;
      if (relu && !(best[j] > 0.f)) { best[j] = 0.f; bi[j] = 255; }  // 255: no gradient flows
      if (j < 4) lo |= (uint32_t)(bi[j] & 255) << (8 * j); else hi |= (uint32_t)(bi[j] & 255) << (8 * (j - 4));
    }
    store8(y + o, best);
    *reinterpret_cast<uint2*>(idx + o) = make_uint2(lo, hi);
  }
}

// dx[n,h,w,c] = sum over windows covering (h,w) whose recorded argmax is (h,w) of dy.
template <typename IT>
__global__ void maxpool_bwd_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ idx, bf16* __restrict__ dx,
                                   const bf16* __restrict__ mask_src, int N, int H, int W, int C, int P, int Q,
                                   int k, int stride, int pad) {
  const int cv = C / 8;
  const IT total = (IT)N * H * W * cv;
  for (IT i = (IT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IT)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % cv);
    IT t = i / cv;
    const int w = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // windows p with p*stride - pad <= h <= p*stride - pad + k - 1
    const int p_lo = max(0, (h + pad - k + stride) / stride);  // ceil((h+pad-k+1)/stride)
    const int p_hi = min(P - 1, (h + pad) / stride);
    const int q_lo = max(0, (w + pad - k + stride) / stride);
    const int q_hi = min(Q - 1, (w + pad) / stride);
    for (int p = p_lo; p <= p_hi; ++p) {
      const int r = h - (p * stride - pad);
      for (int q = q_lo; q <= q_hi; ++q) {
        const int s = w - (q * stride - pad);
        const int code = r * k + s;
        const long long o = (((long long)n * P + p) * Q + q) * C + c8 * 8;
        const uint2 iv = *reinterpret_cast<const uint2*>(idx + o);
        float g[8];
        load8(dy + o, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t word = j < 4 ? iv.x : iv.y;
          const int b = (word >> (8 * (j & 3))) & 255;
          if (b == code) acc[j] += g[j];
        }
      }
    }
    const long long xi = (((long long)n * H + h) * W + w) * C + c8 * 8;
    if (mask_src) {
      float m[8];
      load8(mask_src + xi, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) acc[j] = 0.f;
    }
    store8(dx + xi, acc);
  }
}

template <typename IT>
__global__ void avgpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int N, int H, int W, int C, int P,
                                   int Q, int k, int stride, int pad, int relu) {
  const int cv = C / 8;
  const IT total = (IT)N * P * Q * cv;
  const float inv = 1.f / (float)(k * k);
  for (IT i = (IT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IT)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % cv);
    IT t = i / cv;
    const int q = (int)(t % Q); t /= Q;
    const int p = (int)(t % P);
    const int n = (int)(t / P);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const int h0 = p * stride - pad, w0 = q * stride - pad;
    for (int r = 0; r < k; ++r) {
      const int h = h0 + r;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < k; ++s) {
        const int w = w0 + s;
        if (w < 0 || w >= W) continue;
        float v[8];
        load8(x + (((long long)n * H + h) * W + w) * C + c8 * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] *= inv;
      if (relu) acc[j] = fmaxf(acc[j], 0.f);
    }
    store8(y + (((long long)n * P + p) * Q + q) * C + c8 * 8, acc);
  }
}

// y_relu: optional forward output; when given, dy is masked by (y > 0) first (pool with fused ReLU).
template <typename IT>
__global__ void avgpool_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y_relu,
                                   bf16* __restrict__ dx, const bf16* __restrict__ mask_src, int N, int H, int W,
                                   int C, int P, int Q, int k, int stride, int pad) {
  const int cv = C / 8;
  const IT total = (IT)N * H * W * cv;
  const float inv = 1.f / (float)(k * k);
  for (IT i = (IT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IT)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % cv);
    IT t = i / cv;
    const int w = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const int p_lo = max(0, (h + pad - k + stride) / stride);
    const int p_hi = min(P - 1, (h + pad) / stride);
    const int q_lo = max(0, (w + pad - k + stride) / stride);
    const int q_hi = min(Q - 1, (w + pad) / stride);
    for (int p = p_lo; p <= p_hi; ++p)
      for (int q = q_lo; q <= q_hi; ++q) {
        const long long o = (((long long)n * P + p) * Q + q) * C + c8 * 8;
        float g[8];
        load8(dy + o, g);
        if (y_relu) {
          float yv[8];
          load8(y_relu + o, yv);
#pragma unroll
          for (int j = 0; j < 8; ++j) if (!(yv[j] > 0.f)) g[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += g[j];
      }
    const long long xi = (((long long)n * H + h) * W + w) * C + c8 * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
    if (mask_src) {
      float m[8];
      load8(mask_src + xi, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) acc[j] = 0.f;
    }
    store8(dx + xi, acc);
  }
}

static inline int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  if (g > 148LL * 16) g = 148LL * 16;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_pool_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int P, int Q, int k, int stride,
                int pad, int is_max, int relu, cudaStream_t st) {
  if (C % 8) return -10;
  const long long total = (long long)N * P * Q * (C / 8);
  const bool small = (long long)N * (H > P ? H : P) * (W > Q ? W : Q) * C < 0x7FFFFFFFll;  // 32-bit index math
#define RB_POOL_FWD(IT)                                                                                              \
  if (is_max)                                                                                                        \
    maxpool_fwd_kernel<IT><<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, (uint8_t*)idx, N, H, W, C, \
                                                                P, Q, k, stride, pad, relu);                         \
  else                                                                                                               \
    avgpool_fwd_kernel<IT><<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, N, H, W, C, P, Q, k,       \
                                                                stride, pad, relu);
  if (small) { RB_POOL_FWD(unsigned int) } else { RB_POOL_FWD(long long) }
#undef RB_POOL_FWD
  return RB_LAUNCH_OK();
}

int rb_pool_bwd(const void* dy, const void* idx, const void* y_relu, void* dx, const void* mask_src, int N, int H,
                int W, int C, int P, int Q, int k, int stride, int pad, int is_max, cudaStream_t st) {
  if (C % 8) return -10;
  const long long total = (long long)N * H * W * (C / 8);
  const bool small = (long long)N * (H > P ? H : P) * (W > Q ? W : Q) * C < 0x7FFFFFFFll;
#define RB_POOL_BWD(IT)                                                                                               \
  if (is_max)                                                                                                         \
    maxpool_bwd_kernel<IT><<<grid_for(total, 256), 256, 0, st>>>((const bf16*)dy, (const uint8_t*)idx, (bf16*)dx,      \
                                                                (const bf16*)mask_src, N, H, W, C, P, Q, k, stride,   \
                                                                pad);                                                 \
  else                                                                                                                \
    avgpool_bwd_kernel<IT><<<grid_for(total, 256), 256, 0, st>>>((const bf16*)dy, (const bf16*)y_relu, (bf16*)dx,      \
                                                                (const bf16*)mask_src, N, H, W, C, P, Q, k, stride,   \
                                                                pad);
  if (small) { RB_POOL_BWD(unsigned int) } else { RB_POOL_BWD(long long) }
#undef RB_POOL_BWD
  return RB_LAUNCH_OK();
}

}  // extern "C"
