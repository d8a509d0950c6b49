// Max / average pooling, forward and backward, NHWC bf16, 8 channels per thread (16-byte accesses).
// Output extent is given by the caller (floor or ceil rounding both occur in the reference:
// src/operator/mod.rs:2022-2027 floor, src/layer.rs:1741-1747 ceil). Average pooling divides by the
// full window size (padding counted), as cuDNN's AverageCountIncludingPadding does
// (src/operator/mod.rs:2053-2066). Max pooling records the window offset of the (first) maximum in
// one byte per output so that the backward pass is an exact gather with no atomics.
#include "launch.cuh"
#include <cstdlib>

#include "common.cuh"

namespace rb {

template <typename IT>
__global__ void maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ idx, int N,
                                   int H, int W, int C, int P, int Q, int k, int stride, int pad, int relu) {
  pdl_prolog();
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
  pdl_prolog();
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
  pdl_prolog();
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
  pdl_prolog();
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

// Row-mapped variants of the two max-pooling kernels: one block per (sample, output row) [forward] or per
// (sample, input row) [backward], threads stride over (column, channel group of 8). The generic kernels above are
// bound by instruction issue (three div/mod pairs per element, bf16 -> fp32 conversions, per-channel selects);
// here the in-row index is split with one multiply-high, window size and stride are template constants for the
// common cases, and the 8 channels are handled as four packed bf16x2 values: compare / max / masked add are one
// instruction per pair, with no conversion (max and compare of bf16 values are exact; the backward sum of at
// most ceil(k/stride)^2 terms is rounded to bf16 per addition instead of once at the end).
__device__ __forceinline__ uint32_t div_magic(uint32_t x, uint32_t magic) { return __umulhi(x, magic); }
__device__ __forceinline__ __nv_bfloat162 as_bf2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

template <int KK, int SS>
__global__ void __launch_bounds__(256) maxpool_fwd_rows_kernel(const bf16* __restrict__ x, bf16* __restrict__ y,
                                                               uint8_t* __restrict__ idx, int H, int W, int C, int P,
                                                               int Q, int k_rt, int stride_rt, int pad, int relu,
                                                               uint32_t cv_magic) {
  pdl_prolog();
  const int k = KK ? KK : k_rt, stride = SS ? SS : stride_rt;
  const int cv = C / 8;
  const int n = blockIdx.x / P, p = blockIdx.x - n * P;
  const int h0 = p * stride - pad;
  const int r_lo = max(0, -h0), r_hi = min(k, H - h0);
  const bf16* xn = x + (long long)n * H * W * C;
  const long long orow = ((long long)n * P + p) * Q * C;
  const uint32_t ninf2 = 0xFF80FF80u;  // two bf16 -inf
  const __nv_bfloat162 zero2 = as_bf2(0u);
  for (int j = threadIdx.x; j < Q * cv; j += blockDim.x) {
    const int q = (int)div_magic((uint32_t)j, cv_magic), c8 = j - q * cv;
    const int w0 = q * stride - pad;
    const int s_lo = max(0, -w0), s_hi = min(k, W - w0);
    uint32_t best[4] = {ninf2, ninf2, ninf2, ninf2};
    uint32_t bi[4] = {0u, 0u, 0u, 0u};  // two 16-bit window codes per word
    const bf16* base = xn + (h0 * W + w0) * C + c8 * 8;
    auto visit = [&](int r, int s_) {
      const uint4 v = *reinterpret_cast<const uint4*>(base + (r * W + s_) * C);
      const uint32_t code2 = (uint32_t)(r * k + s_) * 0x00010001u;
      const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t gm = __hgt2_mask(as_bf2(vv[e]), as_bf2(best[e]));   // strictly greater: first maximum wins
        bi[e] = (bi[e] & ~gm) | (code2 & gm);
        best[e] = (best[e] & ~gm) | (vv[e] & gm);
      }
    };
    if (KK) {
#pragma unroll
      for (int r = 0; r < (KK ? KK : 1); ++r) {
        if (r < r_lo || r >= r_hi) continue;
#pragma unroll
        for (int s_ = 0; s_ < (KK ? KK : 1); ++s_) {
          if (s_ < s_lo || s_ >= s_hi) continue;
          visit(r, s_);
        }
      }
    } else {
      for (int r = r_lo; r < r_hi; ++r)
        for (int s_ = s_lo; s_ < s_hi; ++s_) visit(r, s_);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // an empty window leaves -inf: output 0; with a fused ReLU non-positive maxima become 0 with code 255
      uint32_t keep = ~__heq2_mask(as_bf2(best[e]), as_bf2(ninf2));
      if (relu) {
        const uint32_t pos = __hgt2_mask(as_bf2(best[e]), zero2);
        bi[e] = (bi[e] & pos) | (0x00FF00FFu & ~pos);
        keep &= pos;
      }
      best[e] &= keep;
    }
    const long long o = orow + (long long)j * 8;
    *reinterpret_cast<uint4*>(y + o) = make_uint4(best[0], best[1], best[2], best[3]);
    // low bytes of the four 16-bit code pairs -> 8 code bytes
    *reinterpret_cast<uint2*>(idx + o) = make_uint2(__byte_perm(bi[0], bi[1], 0x6420), __byte_perm(bi[2], bi[3], 0x6420));
  }
}

template <int KK, int SS>
__global__ void __launch_bounds__(256) maxpool_bwd_rows_kernel(const bf16* __restrict__ dy,
                                                               const uint8_t* __restrict__ idx, bf16* __restrict__ dx,
                                                               const bf16* __restrict__ mask_src, int H, int W, int C,
                                                               int P, int Q, int k_rt, int stride_rt, int pad,
                                                               uint32_t cv_magic) {
  pdl_prolog();
  const int k = KK ? KK : k_rt, stride = SS ? SS : stride_rt;
  const int cv = C / 8;
  const int n = blockIdx.x / H, h = blockIdx.x - n * H;
  // windows p with p*stride - pad <= h <= p*stride - pad + k - 1 (numerators are >= stride - k, so truncating
  // division agrees with the ceiling wherever max(0, .) does not already decide)
  const int p_lo = max(0, (h + pad - k + stride) / stride), p_hi = min(P - 1, (h + pad) / stride);
  const long long xrow = ((long long)n * H + h) * W * C;
  const bf16* dyn = dy + (long long)n * P * Q * C;
  const uint8_t* idn = idx + (long long)n * P * Q * C;
  const __nv_bfloat162 zero2 = as_bf2(0u);
  for (int j = threadIdx.x; j < W * cv; j += blockDim.x) {
    const int w = (int)div_magic((uint32_t)j, cv_magic), c8 = j - w * cv;
    const int q_lo = max(0, (w + pad - k + stride) / stride), q_hi = min(Q - 1, (w + pad) / stride);
    __nv_bfloat162 acc[4] = {zero2, zero2, zero2, zero2};
    for (int p = p_lo; p <= p_hi; ++p) {
      const int r = h - (p * stride - pad);
      for (int q = q_lo; q <= q_hi; ++q) {
        const int code = r * k + (w - (q * stride - pad));
        const int o = (p * Q + q) * C + c8 * 8;
        const uint2 iv = *reinterpret_cast<const uint2*>(idn + o);
        const uint32_t pat = (uint32_t)code * 0x01010101u;
        const uint32_t mlo = __vcmpeq4(iv.x, pat), mhi = __vcmpeq4(iv.y, pat);   // 0xff where the code matches
        if ((mlo | mhi) == 0u) continue;
        const uint4 g = *reinterpret_cast<const uint4*>(dyn + o);
        acc[0] = __hadd2(acc[0], as_bf2(g.x & __byte_perm(mlo, 0u, 0x1100)));
        acc[1] = __hadd2(acc[1], as_bf2(g.y & __byte_perm(mlo, 0u, 0x3322)));
        acc[2] = __hadd2(acc[2], as_bf2(g.z & __byte_perm(mhi, 0u, 0x1100)));
        acc[3] = __hadd2(acc[3], as_bf2(g.w & __byte_perm(mhi, 0u, 0x3322)));
      }
    }
    uint32_t out[4] = {as_u32(acc[0]), as_u32(acc[1]), as_u32(acc[2]), as_u32(acc[3])};
    const long long xi = xrow + (long long)j * 8;
    if (mask_src) {
      const uint4 m = *reinterpret_cast<const uint4*>(mask_src + xi);
      out[0] &= __hgt2_mask(as_bf2(m.x), zero2);
      out[1] &= __hgt2_mask(as_bf2(m.y), zero2);
      out[2] &= __hgt2_mask(as_bf2(m.z), zero2);
      out[3] &= __hgt2_mask(as_bf2(m.w), zero2);
    }
    *reinterpret_cast<uint4*>(dx + xi) = make_uint4(out[0], out[1], out[2], out[3]);
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
  // generic kernels with 32- or 64-bit index arithmetic
  auto generic = [&](auto maxk, auto avgk) {
    if (is_max)
      launch_pdl(maxk, grid_for(total, 256), 256, 0, st, (const bf16*)x, (bf16*)y, (uint8_t*)idx, N, H, W, C, P, Q, k,
                 stride, pad, relu);
    else
      launch_pdl(avgk, grid_for(total, 256), 256, 0, st, (const bf16*)x, (bf16*)y, N, H, W, C, P, Q, k, stride, pad,
                 relu);
  };
  const int cv = C / 8;
  if (is_max && small && !getenv("RB_POOL_GENERIC") && Q * cv >= 64 && Q * cv < 65536 && (long long)N * P < 0x7FFFFFFF) {
    const int threads = Q * cv >= 256 ? 256 : (Q * cv + 31) / 32 * 32;
    const uint32_t magic = (uint32_t)((0x100000000ull + cv - 1) / cv);
    auto rows = [&](auto kern) {
      launch_pdl(kern, N * P, threads, 0, st, (const bf16*)x, (bf16*)y, (uint8_t*)idx, H, W, C, P, Q, k, stride, pad,
                 relu, magic);
    };
    if (k == 3 && stride == 2) rows(maxpool_fwd_rows_kernel<3, 2>);
    else if (k == 2 && stride == 2) rows(maxpool_fwd_rows_kernel<2, 2>);
    else if (k == 3 && stride == 1) rows(maxpool_fwd_rows_kernel<3, 1>);
    else rows(maxpool_fwd_rows_kernel<0, 0>);
    return RB_LAUNCH_OK();
  }
  if (small) generic(maxpool_fwd_kernel<unsigned int>, avgpool_fwd_kernel<unsigned int>);
  else generic(maxpool_fwd_kernel<long long>, avgpool_fwd_kernel<long long>);
  return RB_LAUNCH_OK();
}

int rb_pool_bwd(const void* dy, const void* idx, const void* y_relu, void* dx, const void* mask_src, int N, int H,
                int W, int C, int P, int Q, int k, int stride, int pad, int is_max, cudaStream_t st) {
  if (C % 8) return -10;
  const long long total = (long long)N * H * W * (C / 8);
  const bool small = (long long)N * (H > P ? H : P) * (W > Q ? W : Q) * C < 0x7FFFFFFFll;
  auto generic = [&](auto maxk, auto avgk) {
    if (is_max)
      launch_pdl(maxk, grid_for(total, 256), 256, 0, st, (const bf16*)dy, (const uint8_t*)idx, (bf16*)dx,
                 (const bf16*)mask_src, N, H, W, C, P, Q, k, stride, pad);
    else
      launch_pdl(avgk, grid_for(total, 256), 256, 0, st, (const bf16*)dy, (const bf16*)y_relu, (bf16*)dx,
                 (const bf16*)mask_src, N, H, W, C, P, Q, k, stride, pad);
  };
  const int cv = C / 8;
  if (is_max && small && !getenv("RB_POOL_GENERIC") && W * cv >= 64 && W * cv < 65536 && (long long)N * H < 0x7FFFFFFF) {
    const int threads = W * cv >= 256 ? 256 : (W * cv + 31) / 32 * 32;
    const uint32_t magic = (uint32_t)((0x100000000ull + cv - 1) / cv);
    auto rows = [&](auto kern) {
      launch_pdl(kern, N * H, threads, 0, st, (const bf16*)dy, (const uint8_t*)idx, (bf16*)dx, (const bf16*)mask_src,
                 H, W, C, P, Q, k, stride, pad, magic);
    };
    if (k == 3 && stride == 2) rows(maxpool_bwd_rows_kernel<3, 2>);
    else if (k == 2 && stride == 2) rows(maxpool_bwd_rows_kernel<2, 2>);
    else if (k == 3 && stride == 1) rows(maxpool_bwd_rows_kernel<3, 1>);
    else rows(maxpool_bwd_rows_kernel<0, 0>);
    return RB_LAUNCH_OK();
  }
  if (small) generic(maxpool_bwd_kernel<unsigned int>, avgpool_bwd_kernel<unsigned int>);
  else generic(maxpool_bwd_kernel<long long>, avgpool_bwd_kernel<long long>);
  return RB_LAUNCH_OK();
}

}  // extern "C"
