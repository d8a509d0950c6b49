// Spatial batch normalisation on NHWC bf16 tensors (rows = N*H*W, columns = channels):
//   forward (training): per-channel batch mean / inverse std, running-statistic update with a caller-given
//   factor, then y = act(gamma * xhat + beta [+ residual]);  inference uses the running statistics.
//   backward: dgamma = sum dy*xhat, dbeta = sum dy, dx = gamma*istd/M * (M*dy - dbeta - xhat*dgamma).
// Replaces cuDNN BatchNormalizationForwardTraining/Inference/Backward as used by the reference's
// BNormConv2d and residual operators, including its "add into a copy of x" residual trick
// (src/operator/conv.rs:494-535,595-608,1601-1644).
#include "launch.cuh"
#include "common.cuh"

namespace rb {

// Forward: sums[c] += sum (x - k_c), sums[C+c] += sum (x - k_c)^2 with the shift k_c = x[0][c] (the channel's value in
// the first row). Shifted sums keep the variance E[(x-k)^2] - E[x-k]^2 free of the cancellation that plain
// E[x^2] - E[x]^2 suffers when a channel's mean is large against its spread (the shift lies inside the data's range,
// so both terms are of the order of the variance). Backward: sums of dy and dy * xhat.
__global__ void bn_reduce_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                 const float* __restrict__ mean, const float* __restrict__ istd, long long rows, int C,
                                 float* __restrict__ sums, int backward) {
  pdl_prolog();
  __shared__ float red0[8][257];
  __shared__ float red1[8][257];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + tx) * 8;
  float a0[8], a1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { a0[j] = 0.f; a1[j] = 0.f; }
  if (c0 < C) {
    float mu[8], is[8];
    if (backward) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { mu[j] = mean[c0 + j]; is[j] = istd[c0 + j]; }
    } else {
      load8(x + c0, mu);   // the shift: row 0 of these channels
    }
    for (long long r = (long long)blockIdx.y * 8 + ty; r < rows; r += (long long)gridDim.y * 8) {
      float v[8];
      load8(x + r * C + c0, v);
      if (!backward) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[j] - mu[j];
          a0[j] += d;
          a1[j] += d * d;
        }
      } else {
        float g[8];
        load8(dy + r * C + c0, g);
        if (y) {  // ReLU after the normalisation: mask by the forward output
          float yy[8];
          load8(y + r * C + c0, yy);
#pragma unroll
          for (int j = 0; j < 8; ++j) if (!(yy[j] > 0.f)) g[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { a0[j] += g[j]; a1[j] += g[j] * (v[j] - mu[j]) * is[j]; }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { red0[ty][tx * 8 + j] = a0[j]; red1[ty][tx * 8 + j] = a1[j]; }
  __syncthreads();
  const int c = threadIdx.x;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) { s0 += red0[k][c]; s1 += red1[k][c]; }
  const int gc = blockIdx.x * 256 + c;
  if (gc < C) {
    atomicAdd(sums + gc, s0);
    atomicAdd(sums + C + gc, s1);
  }
}

// The same sums for channel counts of 64, 128 (every power of two up to 2048 that keeps C / 8 <= 256): the block's
// 256 threads cover (256 / (C / 8)) consecutive rows x all channel groups, so that every lane loads 16 bytes and a
// block reads whole contiguous rows. The kernel above gives each lane a fixed 8-channel group of a 256-channel slab,
// which leaves three lanes in four idle at 64 channels -- the widths of a ResNet's first stages, where this reduction
// was a seventh of the training step.
__global__ void __launch_bounds__(256) bn_reduce_flat_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                                             const bf16* __restrict__ y,
                                                             const float* __restrict__ mean,
                                                             const float* __restrict__ istd, long long rows, int C,
                                                             float* __restrict__ sums, int backward) {
  pdl_prolog();
  __shared__ float red0[2048];
  __shared__ float red1[2048];
  const int cg = C >> 3;                 // channel groups per row; divides 256
  const int rl = 256 / cg;               // rows per pass of the block
  const int g = threadIdx.x % cg, rr = threadIdx.x / cg;
  const int c0 = g * 8;
  float a0[8], a1[8], mu[8], is[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { a0[j] = 0.f; a1[j] = 0.f; is[j] = 1.f; }
  if (backward) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { mu[j] = mean[c0 + j]; is[j] = istd[c0 + j]; }
  } else {
    load8(x + c0, mu);   // the shift: row 0 of these channels
  }
  for (long long r = (long long)blockIdx.x * rl + rr; r < rows; r += (long long)gridDim.x * rl) {
    float v[8];
    load8(x + r * C + c0, v);
    if (!backward) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[j] - mu[j];
        a0[j] += d;
        a1[j] += d * d;
      }
    } else {
      float gr[8];
      load8(dy + r * C + c0, gr);
      if (y) {
        float yy[8];
        load8(y + r * C + c0, yy);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (!(yy[j] > 0.f)) gr[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { a0[j] += gr[j]; a1[j] += gr[j] * (v[j] - mu[j]) * is[j]; }
    }
  }
  // red[rr][channel]: rl x C = 2048 floats
#pragma unroll
  for (int j = 0; j < 8; ++j) { red0[rr * C + c0 + j] = a0[j]; red1[rr * C + c0 + j] = a1[j]; }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += 256) {
    float s0 = 0.f, s1 = 0.f;
    for (int k = 0; k < rl; ++k) { s0 += red0[k * C + c]; s1 += red1[k * C + c]; }
    atomicAdd(sums + c, s0);
    atomicAdd(sums + C + c, s1);
  }
}

// Launches the reduction that fits the channel count (see the two kernels above).
static void launch_bn_reduce(const bf16* x, const bf16* dy, const bf16* y, const float* mean, const float* istd,
                             long long rows, int C, float* sums, int backward, cudaStream_t st) {
  const int cg = C / 8;
  if (C % 8 == 0 && cg >= 1 && cg <= 256 && 256 % cg == 0) {
    const int rl = 256 / cg;
    long long blocks = rows / ((long long)rl * 8);     // about eight rows per thread
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 4) blocks = 148 * 4;
    launch_pdl(bn_reduce_flat_kernel, dim3((unsigned)blocks), dim3(256), 0, st, x, dy, y, mean, istd, rows, C, sums,
               backward);
    return;
  }
  dim3 grid((C + 255) / 256, 1);
  long long gy = rows / 64;
  if (gy < 1) gy = 1;
  if (gy > 256) gy = 256;
  grid.y = (unsigned)gy;
  launch_pdl(bn_reduce_kernel, grid, dim3(256), 0, st, x, dy, y, mean, istd, rows, C, sums, backward);
}

// mean/istd from the sums; running statistics: r = (1-f) r + f batch ; sums re-zeroed.
// With a step counter (`step_ptr`, the network's device-side count of training steps) the factor is derived on
// the device, so that a captured CUDA graph keeps averaging correctly: avg_kind 1 = cumulative 1 / (1 + t),
// avg_kind 2 = exponential `factor` with 1 at t = 0; avg_kind 0 (or no counter) uses `factor` as given.
__global__ void bn_finalize_kernel(float* __restrict__ sums, const bf16* __restrict__ x_row0, long long rows, int C,
                                   float eps, float factor,
                                   float* __restrict__ mean, float* __restrict__ istd, float* __restrict__ run_mean,
                                   float* __restrict__ run_var, int avg_kind = 0,
                                   const unsigned int* __restrict__ step_ptr = nullptr) {
  pdl_prolog();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (step_ptr && avg_kind) {
    const unsigned int t = *step_ptr;
    factor = avg_kind == 1 ? 1.f / (1.f + (float)t) : (t == 0u ? 1.f : factor);
  }
  const float ms = sums[c] / (float)rows;          // mean of the shifted values
  float var = sums[C + c] / (float)rows - ms * ms;
  var = fmaxf(var, 0.f);
  const float m = bf2f(x_row0[c]) + ms;
  mean[c] = m;
  istd[c] = rsqrtf(var + eps);
  if (run_mean) {
    const float unbiased = rows > 1 ? var * (float)rows / (float)(rows - 1) : var;
    run_mean[c] = (1.f - factor) * run_mean[c] + factor * m;
    run_var[c] = (1.f - factor) * run_var[c] + factor * unbiased;
  }
  sums[c] = 0.f;
  sums[C + c] = 0.f;
}

__global__ void bn_running_istd_kernel(const float* __restrict__ run_var, float eps, float* __restrict__ istd, int C) {
  pdl_prolog();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) istd[c] = rsqrtf(run_var[c] + eps);
}

__global__ void bn_apply_kernel(const bf16* __restrict__ x, const float* __restrict__ mean,
                                const float* __restrict__ istd, const float* __restrict__ gamma,
                                const float* __restrict__ beta, const bf16* __restrict__ residual,
                                bf16* __restrict__ y, long long rows, int C, int c_valid, int relu) {
  pdl_prolog();
  const int cv = C / 8;
  const long long total = rows * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % cv) * 8;
    float v[8], r[8];
    load8(x + i * 8, v);
    if (residual) load8(residual + i * 8, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      float o = 0.f;
      if (c < c_valid) {
        o = (v[j] - mean[c]) * istd[c] * gamma[c] + beta[c];
        if (residual) o += r[j];
        if (relu) o = fmaxf(o, 0.f);
      }
      v[j] = o;
    }
    store8(y + i * 8, v);
  }
}

// sums holds [dbeta | dgamma]; they are also accumulated into the gradient buffers.
__global__ void bn_bwd_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                                    const float* __restrict__ mean, const float* __restrict__ istd,
                                    const float* __restrict__ gamma, const float* __restrict__ sums,
                                    bf16* __restrict__ dx, long long rows, int C, int c_valid) {
  pdl_prolog();
  const int cv = C / 8;
  const long long total = rows * cv;
  const float invm = 1.f / (float)rows;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % cv) * 8;
    float v[8], g[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, g);
    if (y) {
      float yy[8];
      load8(y + i * 8, yy);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(yy[j] > 0.f)) g[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      float o = 0.f;
      if (c < c_valid) {
        const float xh = (v[j] - mean[c]) * istd[c];
        o = gamma[c] * istd[c] * (g[j] - invm * (sums[c] + xh * sums[C + c]));
      }
      v[j] = o;
    }
    store8(dx + i * 8, v);
  }
}

__global__ void bn_grad_accum_kernel(float* __restrict__ sums, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                     int C, int c_valid) {
  pdl_prolog();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (c < c_valid) {
    dbeta[c] += sums[c];
    dgamma[c] += sums[C + c];
  }
  sums[c] = 0.f;
  sums[C + c] = 0.f;
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

// sums: 2*C floats of scratch that must be zero on entry and is zero again on return.
int rb_bn_fwd_train(const void* x, long long rows, int C, int c_valid, float* sums, float eps, float factor,
                    float* mean, float* istd, float* run_mean, float* run_var, const float* gamma, const float* beta,
                    const void* residual, void* y, int relu, int avg_kind, const unsigned int* step_ptr,
                    cudaStream_t st) {
  if (C % 8) return -10;
  launch_bn_reduce((const bf16*)x, nullptr, nullptr, nullptr, nullptr, rows, C, sums, 0, st);
  launch_pdl(bn_finalize_kernel, dim3((C + 127) / 128), dim3(128), 0, st, sums, (const bf16*)x, rows, C, eps, factor,
             mean, istd, run_mean, run_var, avg_kind, step_ptr);
  launch_pdl(bn_apply_kernel, dim3(grid_for(rows * (C / 8), 256)), dim3(256), 0, st, (const bf16*)x, mean, istd, gamma,
             beta, (const bf16*)residual, (bf16*)y, rows, C, c_valid, relu);
  return RB_LAUNCH_OK();
}

int rb_bn_fwd_infer(const void* x, long long rows, int C, int c_valid, float eps, const float* run_mean,
                    const float* run_var, float* istd_tmp, const float* gamma, const float* beta, const void* residual,
                    void* y, int relu, cudaStream_t st) {
  if (C % 8) return -10;
  bn_running_istd_kernel<<<(C + 127) / 128, 128, 0, st>>>(run_var, eps, istd_tmp, C);
  bn_apply_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, st>>>((const bf16*)x, run_mean, istd_tmp, gamma, beta,
                                                                (const bf16*)residual, (bf16*)y, rows, C, c_valid, relu);
  return RB_LAUNCH_OK();
}

// y_relu: forward output when a ReLU followed the normalisation (masks dy), else null.
// dgamma/dbeta are accumulated (the optimizer zeroes them).
int rb_bn_bwd(const void* x, const void* dy, const void* y_relu, long long rows, int C, int c_valid, float* sums,
              const float* mean, const float* istd, const float* gamma, float* dgamma, float* dbeta, void* dx,
              cudaStream_t st) {
  if (C % 8) return -10;
  launch_bn_reduce((const bf16*)x, (const bf16*)dy, (const bf16*)y_relu, mean, istd, rows, C, sums, 1, st);
  launch_pdl(bn_bwd_apply_kernel, dim3(grid_for(rows * (C / 8), 256)), dim3(256), 0, st, (const bf16*)x,
             (const bf16*)dy, (const bf16*)y_relu, mean, istd, gamma, sums, (bf16*)dx, rows, C, c_valid);
  launch_pdl(bn_grad_accum_kernel, dim3((C + 127) / 128), dim3(128), 0, st, sums, dgamma, dbeta, C, c_valid);
  return RB_LAUNCH_OK();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in bn_noalloc.h).
#include "bn_noalloc.h"

namespace rb {
// Scratch for the per-channel sums: part of the library's device image, one copy per GPU.
static __device__ __align__(256) float g_bn_noalloc_scratch[2 * RB_BN_NOALLOC_MAX_CHANNELS];
constexpr int kMaxDevices = 64;
// Device address of the array above, per device. The array's name is only a host-side handle; kernels
// must be given the address that cudaGetSymbolAddress returns for the device they run on.
static float* g_bn_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace rb

extern "C" {

int rb_bn_fwd_train_noalloc(const void* x, long long rows, int C, int c_valid, float eps, float factor, float* mean,
                            float* istd, float* run_mean, float* run_var, const float* gamma, const float* beta,
                            const void* residual, void* y, int relu, cudaStream_t stream) {
  if (C % 8) return RB_BN_NOALLOC_E_CHANNEL_ALIGN;
  if (C > RB_BN_NOALLOC_MAX_CHANNELS) return RB_BN_NOALLOC_E_TOO_MANY_CHANNELS;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RB_BN_NOALLOC_E_DEVICE;
  if (g_bn_noalloc_ptr[dev] == nullptr) {
    // first call on this device: resolve the array's device address (the device is current here)
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_bn_noalloc_scratch) != cudaSuccess || p == nullptr)
      return RB_BN_NOALLOC_E_SYMBOL;
    g_bn_noalloc_ptr[dev] = p;
  }
  float* sums = g_bn_noalloc_ptr[dev];
  // the array keeps whatever the previous call left: clear the part this call accumulates into
  if (cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)C, stream) != cudaSuccess) return RB_BN_NOALLOC_E_LAUNCH;
  dim3 grid((C + 255) / 256, 1);
  long long gy = rows / 64;
  if (gy < 1) gy = 1;
  if (gy > 256) gy = 256;
  grid.y = (unsigned)gy;
  bn_reduce_kernel<<<grid, 256, 0, stream>>>((const bf16*)x, nullptr, nullptr, nullptr, nullptr, rows, C, sums, 0);
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, stream>>>(sums, (const bf16*)x, rows, C, eps, factor, mean, istd, run_mean,
                                                          run_var);
  bn_apply_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, stream>>>((const bf16*)x, mean, istd, gamma, beta,
                                                                    (const bf16*)residual, (bf16*)y, rows, C, c_valid,
                                                                    relu);
  return cudaGetLastError() == cudaSuccess ? RB_BN_NOALLOC_OK : RB_BN_NOALLOC_E_LAUNCH;
}

const char* rb_bn_noalloc_strerror(int code) {
  switch (code) {
    case RB_BN_NOALLOC_OK: return "ok";
    case RB_BN_NOALLOC_E_CHANNEL_ALIGN: return "channel count must be a multiple of 8";
    case RB_BN_NOALLOC_E_TOO_MANY_CHANNELS: return "channel count exceeds RB_BN_NOALLOC_MAX_CHANNELS (4096)";
    case RB_BN_NOALLOC_E_DEVICE: return "current CUDA device could not be determined or its index is >= 64";
    case RB_BN_NOALLOC_E_SYMBOL: return "cudaGetSymbolAddress failed for the built-in scratch array";
    case RB_BN_NOALLOC_E_LAUNCH: return "a kernel launch or the scratch-clearing memset failed";
    default: return "unknown code";
  }
}

}  // extern "C"
