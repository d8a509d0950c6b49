// Smooth and clipped activations of the older layer generations, plus the sparsity counters that go with them.
// ReLU never comes through here: it lives in the epilogues of the tensor-core and pooling kernels. The reference has
// logistic / tanh through cuDNN's activation call and a "bounded rect" (clipped ReLU) kernel in its first layer
// generation (src/layer.rs:55,1430-1446,1550-1567) and counts non-zero activations / non-sparse gradients for
// statistics (src/layer.rs:1457,1602).
//
// Activations are bf16 [rows][ld] with `n_valid` live columns; padded columns stay zero (a logistic would turn
// them into 0.5 and feed the next layer's padded input channels).
#include "launch.cuh"
#include "common.cuh"

namespace rb {

// `param` is the upper clip of the bounded rectifier and the input scale beta of the scaled logistic
// (sigmoid(beta x), src/layer_new.rs:164,1031-1038); the other kinds ignore it. ACT_RECT exists for the places where
// a ReLU cannot ride in a GEMM epilogue (after a residual sum that is not followed by batch normalisation).
enum { ACT_LOGISTIC = 1, ACT_TANH = 2, ACT_BOUNDED_RECT = 3, ACT_RECT = 4, ACT_SCALED_LOGISTIC = 5 };

__device__ __forceinline__ float act_apply(float x, int kind, float param) {
  if (kind == ACT_LOGISTIC) return 1.f / (1.f + __expf(-x));
  if (kind == ACT_TANH) return tanhf(x);
  if (kind == ACT_BOUNDED_RECT) return fminf(fmaxf(x, 0.f), param);
  if (kind == ACT_RECT) return fmaxf(x, 0.f);
  return 1.f / (1.f + __expf(-param * x));
}

// derivative written in terms of the OUTPUT y, so that backward needs no copy of the pre-activation
__device__ __forceinline__ float act_slope(float y, int kind, float param) {
  if (kind == ACT_LOGISTIC) return y * (1.f - y);
  if (kind == ACT_TANH) return 1.f - y * y;
  if (kind == ACT_BOUNDED_RECT) return (y > 0.f && y < param) ? 1.f : 0.f;
  if (kind == ACT_RECT) return y > 0.f ? 1.f : 0.f;
  return param * y * (1.f - y);
}

// y = f(y) in place on the live columns
__global__ void act_fwd_kernel(bf16* __restrict__ y, long long rows, int ld, int n_valid, int kind, float bound) {
  pdl_prolog();
  const int gpr = ld / 8;
  const long long groups = rows * gpr;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(g % gpr) * 8;
    float v[8];
    if (c0 >= n_valid) {  // a group that lies wholly in the padding: written as zeros, never left as it was
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      store8(y + g * 8, v);
      continue;
    }
    load8(y + g * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (c0 + j < n_valid) ? act_apply(v[j], kind, bound) : 0.f;
    store8(y + g * 8, v);
  }
}

// d *= f'(y) in place
__global__ void act_bwd_kernel(bf16* __restrict__ d, const bf16* __restrict__ y, long long rows, int ld, int n_valid,
                               int kind, float bound) {
  pdl_prolog();
  const int gpr = ld / 8;
  const long long groups = rows * gpr;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(g % gpr) * 8;
    float v[8], o[8];
    if (c0 >= n_valid) {  // padded columns of the delta must come out zero whatever came in
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      store8(d + g * 8, v);
      continue;
    }
    load8(d + g * 8, v);
    load8(y + g * 8, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (c0 + j < n_valid) ? v[j] * act_slope(o[j], kind, bound) : 0.f;
    store8(d + g * 8, v);
  }
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return bf2f(v); }

// out[0] += #{ i : |x[i]| > threshold }   (threshold 0 counts non-zeros)
template <typename T>
__global__ void count_above_kernel(const T* __restrict__ x, long long n, float threshold,
                                   unsigned long long* __restrict__ out) {
  pdl_prolog();
  unsigned int local = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    local += fabsf(to_float(x[i])) > threshold ? 1u : 0u;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  __shared__ unsigned int warp_sums[8];
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int total = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_sums[w];
    if (total) atomicAdd(out, (unsigned long long)total);
  }
}

static inline int act_grid(long long total, int block) {
  long long g = (total + block - 1) / block;
  if (g > 148LL * 16) g = 148LL * 16;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_act_fwd(void* y, long long rows, int ld, int n_valid, int kind, float bound, cudaStream_t st) {
  if (ld % 8 || kind < ACT_LOGISTIC || kind > ACT_SCALED_LOGISTIC) return -10;
  launch_pdl(act_fwd_kernel, act_grid(rows * (ld / 8), 256), 256, 0, st, (bf16*)y, rows, ld, n_valid, kind, bound);
  return RB_LAUNCH_OK();
}

int rb_act_bwd(void* d, const void* y, long long rows, int ld, int n_valid, int kind, float bound, cudaStream_t st) {
  if (ld % 8 || kind < ACT_LOGISTIC || kind > ACT_SCALED_LOGISTIC) return -10;
  launch_pdl(act_bwd_kernel, act_grid(rows * (ld / 8), 256), 256, 0, st, (bf16*)d, (const bf16*)y, rows, ld, n_valid,
             kind, bound);
  return RB_LAUNCH_OK();
}

int rb_count_above(const void* x, long long n, int is_f32, float threshold, unsigned long long* out, cudaStream_t st) {
  if (is_f32)
    launch_pdl(count_above_kernel<float>, act_grid(n, 256), 256, 0, st, (const float*)x, n, threshold, out);
  else
    launch_pdl(count_above_kernel<bf16>, act_grid(n, 256), 256, 0, st, (const bf16*)x, n, threshold, out);
  return RB_LAUNCH_OK();
}

}  // extern "C"
