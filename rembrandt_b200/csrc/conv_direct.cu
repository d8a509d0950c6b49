// Direct (CUDA-core) convolution kernels, NHWC bf16 with fp32 accumulation, any stride / padding.
// They are the fallback for shapes the tensor-core path does not take (strided data-gradient) and the
// on-device cross-check for it. Filters are [Kout][R*S][Cp] like the tensor-core path.
#include "common.cuh"

namespace rb {

__global__ void conv_direct_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                       const float* __restrict__ bias, bf16* __restrict__ y, int N, int H, int W,
                                       int Cp, int Kout, int Kp, int R, int S, int stride, int pad_h, int pad_w,
                                       int P, int Q, int relu) {
  const long long total = (long long)N * P * Q * Kp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kp);
    long long t = i / Kp;
    const int q = (int)(t % Q); t /= Q;
    const int p = (int)(t % P);
    const int n = (int)(t / P);
    float acc = 0.f;
    if (k < Kout) {
      for (int r = 0; r < R; ++r) {
        const int h = p * stride - pad_h + r;
        if (h < 0 || h >= H) continue;
        for (int s = 0; s < S; ++s) {
          const int ww = q * stride - pad_w + s;
          if (ww < 0 || ww >= W) continue;
          const bf16* xp = x + (((long long)n * H + h) * W + ww) * Cp;
          const bf16* wp = w + ((long long)k * R * S + r * S + s) * Cp;
          for (int c = 0; c < Cp; ++c) acc += bf2f(xp[c]) * bf2f(wp[c]);
        }
      }
      if (bias) acc += bias[k];
      if (relu) acc = fmaxf(acc, 0.f);
    }
    y[i] = f2bf(acc);
  }
}

// dx[n,h,w,c] = sum_{k,r,s : (h+pad-r) % stride == 0 ...} dy[n,p,q,k] * w[k][r,s][c]
__global__ void conv_direct_dgrad_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ w,
                                         bf16* __restrict__ dx, const bf16* __restrict__ mask_src, int N, int H, int W,
                                         int Cp, int Kout, int Kp, int R, int S, int stride, int pad_h, int pad_w,
                                         int P, int Q) {
  const long long total = (long long)N * H * W * Cp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    long long t = i / Cp;
    const int ww = (int)(t % W); t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    float acc = 0.f;
    for (int r = 0; r < R; ++r) {
      const int ph = h + pad_h - r;
      if (ph < 0 || ph % stride) continue;
      const int p = ph / stride;
      if (p >= P) continue;
      for (int s = 0; s < S; ++s) {
        const int qw = ww + pad_w - s;
        if (qw < 0 || qw % stride) continue;
        const int q = qw / stride;
        if (q >= Q) continue;
        const bf16* dp = dy + (((long long)n * P + p) * Q + q) * Kp;
        for (int k = 0; k < Kout; ++k) acc += bf2f(dp[k]) * bf2f(w[((long long)k * R * S + r * S + s) * Cp + c]);
      }
    }
    if (mask_src && !(bf2f(mask_src[i]) > 0.f)) acc = 0.f;
    dx[i] = f2bf(acc);
  }
}

// dw[k][r,s][c] += sum_{n,p,q} dy[n,p,q,k] * x[n, p*stride-pad+r, q*stride-pad+s, c]
__global__ void conv_direct_wgrad_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                         float* __restrict__ dw, int N, int H, int W, int Cp, int Kout, int Kp, int R,
                                         int S, int stride, int pad_h, int pad_w, int P, int Q) {
  const long long total = (long long)Kout * R * S * Cp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    long long t = i / Cp;
    const int s = (int)(t % S); t /= S;
    const int r = (int)(t % R);
    const int k = (int)(t / R);
    float acc = 0.f;
    for (int n = 0; n < N; ++n)
      for (int p = 0; p < P; ++p) {
        const int h = p * stride - pad_h + r;
        if (h < 0 || h >= H) continue;
        for (int q = 0; q < Q; ++q) {
          const int ww = q * stride - pad_w + s;
          if (ww < 0 || ww >= W) continue;
          acc += bf2f(dy[(((long long)n * P + p) * Q + q) * Kp + k]) *
                 bf2f(x[(((long long)n * H + h) * W + ww) * Cp + c]);
        }
      }
    dw[i] += acc;
  }
}

static inline int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  if (g > 148LL * 32) g = 148LL * 32;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_conv_direct_fwd(const void* x, const void* w, const float* bias, void* y, int N, int H, int W, int Cp, int Kout,
                       int Kp, int R, int S, int stride, int pad_h, int pad_w, int P, int Q, int relu,
                       cudaStream_t st) {
  conv_direct_fwd_kernel<<<grid_for((long long)N * P * Q * Kp, 128), 128, 0, st>>>(
      (const bf16*)x, (const bf16*)w, bias, (bf16*)y, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h, pad_w, P, Q, relu);
  return RB_LAUNCH_OK();
}

int rb_conv_direct_dgrad(const void* dy, const void* w, void* dx, const void* mask_src, int N, int H, int W, int Cp,
                         int Kout, int Kp, int R, int S, int stride, int pad_h, int pad_w, int P, int Q,
                         cudaStream_t st) {
  conv_direct_dgrad_kernel<<<grid_for((long long)N * H * W * Cp, 128), 128, 0, st>>>(
      (const bf16*)dy, (const bf16*)w, (bf16*)dx, (const bf16*)mask_src, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h,
      pad_w, P, Q);
  return RB_LAUNCH_OK();
}

int rb_conv_direct_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Cp, int Kout, int Kp,
                         int R, int S, int stride, int pad_h, int pad_w, int P, int Q, cudaStream_t st) {
  conv_direct_wgrad_kernel<<<grid_for((long long)Kout * R * S * Cp, 128), 128, 0, st>>>(
      (const bf16*)x, (const bf16*)dy, dw, N, H, W, Cp, Kout, Kp, R, S, stride, pad_h, pad_w, P, Q);
  return RB_LAUNCH_OK();
}

}  // extern "C"
