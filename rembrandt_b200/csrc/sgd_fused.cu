// One-pass SGD over a flat fp32 parameter range: L2 regularisation, the momentum rule, the parameter
// update, the bf16 compute copy and the gradient reset, all in a single read-modify-write sweep.
// The reference does this as 6-8 saxpy/sscal launches per tensor (regularize / accumulate_grads /
// update_params / reset, src/operator/mod.rs:1178-1363 and src/opt/sgd/new.rs:358-495).
//
// The rules themselves are in sgd_rules.cuh.
#include "launch.cuh"
#include "common.cuh"
#include "sgd_rules.cuh"

namespace rb {

struct SgdArgs : SgdHyper {
  float* w;
  float* g;
  float* v;
  bf16* w16;   // optional
  long long n;
};

__global__ void sgd_fused_kernel(SgdArgs a) {
  pdl_prolog();
  const long long n4 = a.n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 w = reinterpret_cast<float4*>(a.w)[i];
    float4 g = reinterpret_cast<float4*>(a.g)[i];
    float4 v = a.v ? reinterpret_cast<float4*>(a.v)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sgd_elem(w.x, g.x, v.x, a);
    sgd_elem(w.y, g.y, v.y, a);
    sgd_elem(w.z, g.z, v.z, a);
    sgd_elem(w.w, g.w, v.w, a);
    if (a.phase & 3) reinterpret_cast<float4*>(a.w)[i] = w;
    if (a.v && (a.phase & 1)) reinterpret_cast<float4*>(a.v)[i] = v;
    if ((a.phase & 4) || a.mode == 5) reinterpret_cast<float4*>(a.g)[i] = g;
    if (a.w16 && (a.phase & 2)) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(a.w16)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    float w = a.w[i], g = a.g[i], v = a.v ? a.v[i] : 0.f;
    sgd_elem(w, g, v, a);
    if (a.phase & 3) a.w[i] = w;
    if (a.v && (a.phase & 1)) a.v[i] = v;
    if ((a.phase & 4) || a.mode == 5) a.g[i] = g;
    if (a.w16 && (a.phase & 2)) a.w16[i] = f2bf(w);
  }
}

// w += s * v (Nesterov look-ahead bookkeeping before the first step), refreshing the bf16 copy.
__global__ void axpy_shadow_kernel(float* __restrict__ w, const float* __restrict__ v, bf16* __restrict__ w16,
                                   long long n, float s) {
  pdl_prolog();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float x = w[i];
    if (v) x += s * v[i];
    w[i] = x;
    if (w16) w16[i] = f2bf(x);
  }
}

// y = a*x + b*y on fp32 ranges (exact averaging, elastic mixes on one device, snapshots)
__global__ void axpby_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, float a, float b) {
  pdl_prolog();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = a * x[i] + b * y[i];
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_sgd_fused(float* w, float* g, float* v, void* w16, long long n, float lr, float mu, float l2, float grad_scale,
                 int mode, int phase, cudaStream_t st) {
  if (n <= 0) return 0;
  SgdArgs a;
  a.lr = lr; a.mu = mu; a.l2 = l2; a.grad_scale = grad_scale; a.mode = mode; a.phase = phase;
  a.w = w; a.g = g; a.v = v; a.w16 = (bf16*)w16; a.n = n;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  launch_pdl(sgd_fused_kernel, (int)blocks, 256, 0, st, a);
  return RB_LAUNCH_OK();
}

// Same kernel with a caller-chosen grid: blocks of 128 threads fit on an SM next to a resident GEMM CTA, which lets
// the update of a finished gradient bucket run on a second stream while backward continues.
int rb_sgd_fused_grid(float* w, float* g, float* v, void* w16, long long n, float lr, float mu, float l2,
                      float grad_scale, int mode, int phase, int blocks, int threads, cudaStream_t st) {
  if (n <= 0) return 0;
  if (blocks < 1 || threads < 32 || threads > 1024 || (threads & 31)) return -10;
  SgdArgs a;
  a.lr = lr; a.mu = mu; a.l2 = l2; a.grad_scale = grad_scale; a.mode = mode; a.phase = phase;
  a.w = w; a.g = g; a.v = v; a.w16 = (bf16*)w16; a.n = n;
  const long long need = (n / 4 + threads - 1) / threads;
  if (need < blocks) blocks = need < 1 ? 1 : (int)need;
  launch_pdl(sgd_fused_kernel, blocks, threads, 0, st, a);
  return RB_LAUNCH_OK();
}

int rb_axpy_shadow(float* w, const float* v, void* w16, long long n, float s, cudaStream_t st) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  launch_pdl(axpy_shadow_kernel, (int)blocks, 256, 0, st, w, v, (bf16*)w16, n, s);
  return RB_LAUNCH_OK();
}

int rb_axpby(const float* x, float* y, long long n, float a, float b, cudaStream_t st) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  launch_pdl(axpby_kernel, (int)blocks, 256, 0, st, x, y, n, a, b);
  return RB_LAUNCH_OK();
}

}  // extern "C"
