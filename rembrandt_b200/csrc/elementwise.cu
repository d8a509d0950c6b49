// Small memory-bound helpers around the tensor-core kernels: bias-gradient column sums,
// the fp32 -> bf16 epilogue of split-K affine layers, dropout, ReLU masking, filter repacking.
#include "launch.cuh"
#include "common.cuh"

namespace rb {

// out[c] += sum_r x[r][c]   (bias gradient; replaces cuDNN ConvolutionBackwardBias and the ones-vector
// gemm of the reference, src/operator/mod.rs:1169,1775-1781)
__global__ void colsum_kernel(const bf16* __restrict__ x, long long rows, int ld, int cols, float* __restrict__ out,
                              int tpr) {
  pdl_prolog();
  // tpr threads (8 columns each) per row, 256 / tpr rows per pass: narrow matrices keep all lanes busy
  __shared__ float red[256 * 8];
  const int rpp = 256 / tpr;
  const int tx = threadIdx.x % tpr, ty = threadIdx.x / tpr;
  const int c0 = (blockIdx.x * tpr + tx) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (ty < rpp && c0 < ld) {
    for (long long r = (long long)blockIdx.y * rpp + ty; r < rows; r += (long long)gridDim.y * rpp) {
      float v[8];
      load8(x + r * ld + c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
  const int width = tpr * 8;
  if (ty < rpp) {
#pragma unroll
    for (int j = 0; j < 8; ++j) red[ty * width + tx * 8 + j] = acc[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < rpp; ++k) sum += red[k * width + c];
    const int gc = blockIdx.x * width + c;
    if (gc < cols) atomicAdd(out + gc, sum);
  }
}

// y[r][c] = act(acc[r][c] + bias[c]) for c < n_valid, 0 for padded columns; acc is re-zeroed so the
// split-K workspace is clean for its next use.
__global__ void bias_act_kernel(float* __restrict__ acc, long long rows, int ld, int n_valid,
                                const float* __restrict__ bias, int relu, bf16* __restrict__ y,
                                const bf16* __restrict__ mask_src, int rezero) {
  pdl_prolog();
  const long long total = rows * (ld / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % (ld / 8)) * 8;
    const long long r = i / (ld / 8);
    float4* ap = reinterpret_cast<float4*>(acc + r * ld + c0);
    const float4 a0 = ap[0], a1 = ap[1];
    float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      if (c < n_valid) {
        if (bias) v[j] += bias[c];
        if (relu) v[j] = fmaxf(v[j], 0.f);
      } else {
        v[j] = 0.f;
      }
    }
    if (mask_src) {
      float m[8];
      load8(mask_src + r * ld + c0, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) v[j] = 0.f;
    }
    store8(y + r * ld + c0, v);
    if (rezero) {
      ap[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      ap[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// Inverted dropout: y = x * keep / (1 - p), keep = (u >= p), u from Philox(seed, element/4).
// The mask is never stored; backward regenerates it from the same (seed, stream) pair.
// (reference: map_dropout / map_dropout_backprop call sites, src/operator/mod.rs:2210-2244)
__global__ void dropout_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const bf16* __restrict__ mask_src,
                               long long n, float p, uint64_t seed, uint32_t stream,
                               const uint32_t* __restrict__ step_ptr) {
  pdl_prolog();
  const float scale = 1.f / (1.f - p);
  if (step_ptr) seed += *step_ptr;  // device-side step counter: a captured graph draws a new mask per replay
  const long long groups = n / 8;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + g * 8, v);
    uint32_t r0[4], r1[4];
    Philox::gen(seed, (uint64_t)g * 2, stream, r0);
    Philox::gen(seed, (uint64_t)g * 2 + 1, stream, r1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = (u32_to_unit(r0[j]) >= p) ? v[j] * scale : 0.f;
      v[4 + j] = (u32_to_unit(r1[j]) >= p) ? v[4 + j] * scale : 0.f;
    }
    if (mask_src) {
      float m[8];
      load8(mask_src + g * 8, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) v[j] = 0.f;
    }
    store8(y + g * 8, v);
  }
}

// d *= (y > 0) in place
__global__ void relu_mask_kernel(bf16* __restrict__ d, const bf16* __restrict__ y, long long n) {
  pdl_prolog();
  const long long groups = n / 8;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    float v[8], m[8];
    load8(d + g * 8, v);
    load8(y + g * 8, m);
#pragma unroll
    for (int j = 0; j < 8; ++j) if (!(m[j] > 0.f)) v[j] = 0.f;
    store8(d + g * 8, v);
  }
}

// a += b (bf16), optional mask; used to sum branch deltas at fan-out points
__global__ void add_kernel(bf16* __restrict__ a, const bf16* __restrict__ b, long long n) {
  pdl_prolog();
  const long long groups = n / 8;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    float v[8], w[8];
    load8(a + g * 8, v);
    load8(b + g * 8, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += w[j];
    store8(a + g * 8, v);
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, bf16* __restrict__ y, long long n) {
  pdl_prolog();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = f2bf(x[i]);
}

// wt[c][(R-1-r)*S + (S-1-s)][k] = w[k][r*S+s][c]   (k < Kout, c < Cp; padded k are zero)
// Filters for the data-gradient, which runs as a forward convolution of dY with flipped taps.
__global__ void pack_dgrad_filters_kernel(const bf16* __restrict__ w, bf16* __restrict__ wt, int Kout, int Kp, int RS,
                                          int Cp) {
  pdl_prolog();
  const long long total = (long long)Cp * RS * Kp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kp);
    long long t = i / Kp;
    const int tap = (int)(t % RS);
    const int c = (int)(t / RS);
    bf16 v = f2bf(0.f);
    if (k < Kout) v = w[((long long)k * RS + (RS - 1 - tap)) * Cp + c];
    wt[i] = v;
  }
}

// Zero the entries of a space-to-depth'd first-layer filter gradient that have no counterpart in the
// original filter: taps (r,s) >= ksize and padded channels.  dw is [Kout][R2*S2][Cp], channel =
// (dy*f + dx)*cin + ci, original row = R2idx*f + dy.
__global__ void zero_s2d_structural_kernel(float* __restrict__ dw, int Kout, int R2, int Cp, int f, int cin,
                                           int ksize) {
  pdl_prolog();
  const long long total = (long long)Kout * R2 * R2 * Cp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % Cp);
    long long t = i / Cp;
    const int tap = (int)(t % (R2 * R2));
    const int r2 = tap / R2, s2 = tap % R2;
    bool dead = ch >= f * f * cin;
    if (!dead) {
      const int blk = ch / cin;
      const int dy = blk / f, dx = blk % f;
      dead = (r2 * f + dy >= ksize) || (s2 * f + dx >= ksize);
    }
    if (dead) dw[i] = 0.f;
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

// y[n] = beta * y[n] + alpha * sum_j val[j] * W(n, ind[j]) for a vector given by its `nnz` non-zero entries: the
// matrix x sparse-vector product that the reference's tools/bench-cublas.rs:98-115 times for board-game layers whose
// input is mostly zeros. `transposed` = W stored [k][n] (an entry's weights contiguous: coalesced), else [n][k] (a
// gather of one element per output and entry). One thread per output; the entries are split over blockIdx.y and the
// partial sums added with red.add; `y` is scaled by beta in a tiny launch of its own first, which keeps the two
// phases ordered.
__global__ void scale_vec_kernel(float* __restrict__ y, int n, float beta) {
  pdl_prolog();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = beta == 0.f ? 0.f : beta * y[i];
}
__global__ void gemv_sparse_kernel(const float* __restrict__ w, int n, int k, int transposed,
                                   const float* __restrict__ val, const int* __restrict__ ind, int nnz, float alpha,
                                   float* __restrict__ y) {
  pdl_prolog();
  __shared__ float s_val[256];
  __shared__ int s_ind[256];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int per = (nnz + gridDim.y - 1) / gridDim.y;
  const int j0 = blockIdx.y * per, j1 = min(nnz, j0 + per);
  float acc = 0.f;
  for (int base = j0; base < j1; base += 256) {
    const int m = min(256, j1 - base);
    __syncthreads();
    if (threadIdx.x < m) {
      s_val[threadIdx.x] = val[base + threadIdx.x];
      s_ind[threadIdx.x] = ind[base + threadIdx.x];
    }
    __syncthreads();
    if (i < n) {
      for (int j = 0; j < m; ++j) {
        const int c = s_ind[j];
        if (c >= 0 && c < k) acc += s_val[j] * (transposed ? w[(long long)c * n + i] : w[(long long)i * k + c]);
      }
    }
  }
  if (i < n && j0 < j1) atomicAdd(y + i, alpha * acc);
}

extern "C" {

int rb_gemv_sparse(const float* w, int n, int k, int transposed, const float* val, const int* ind, int nnz,
                   float alpha, float beta, float* y, cudaStream_t st) {
  if (n <= 0 || k <= 0 || nnz < 0) return -10;
  const int bx = (n + 255) / 256;
  launch_pdl(scale_vec_kernel, bx, 256, 0, st, y, n, beta);
  if (nnz > 0) {
    int gy = (148 * 4) / bx;                   // enough blocks for every SM when n is small (361 outputs = 2 blocks)
    const int max_gy = (nnz + 63) / 64;        // at least 64 entries per block
    if (gy > max_gy) gy = max_gy;
    if (gy < 1) gy = 1;
    launch_pdl(gemv_sparse_kernel, dim3(bx, gy), 256, 0, st, w, n, k, transposed, val, ind, nnz, alpha, y);
  }
  return RB_LAUNCH_OK();
}

int rb_colsum(const void* x, long long rows, int ld, int cols, float* out, cudaStream_t st) {
  if (ld % 8) return -10;
  const int groups = ld / 8;
  const int tpr = groups < 32 ? groups : 32;
  const int rpp = 256 / tpr;
  dim3 grid((groups + tpr - 1) / tpr, 1);
  long long gy = rows / (rpp * 4);
  if (gy < 1) gy = 1;
  const long long cap = (148LL * 8) / grid.x > 1 ? (148LL * 8) / grid.x : 1;
  if (gy > cap) gy = cap;
  grid.y = (unsigned)gy;
  launch_pdl(colsum_kernel, grid, 256, 0, st, (const bf16*)x, rows, ld, cols, out, tpr);
  return RB_LAUNCH_OK();
}

int rb_bias_act(float* acc, long long rows, int ld, int n_valid, const float* bias, int relu, void* y,
                const void* mask_src, int rezero, cudaStream_t st) {
  if (ld % 8) return -10;
  launch_pdl(bias_act_kernel, grid_for(rows * (ld / 8), 256), 256, 0, st, acc, rows, ld, n_valid, bias, relu, (bf16*)y,
             (const bf16*)mask_src, rezero);
  return RB_LAUNCH_OK();
}

int rb_dropout(const void* x, void* y, const void* mask_src, long long n, float p, unsigned long long seed,
               unsigned int stream_id, const unsigned int* step_ptr, cudaStream_t st) {
  if (n % 8) return -10;
  launch_pdl(dropout_kernel, grid_for(n / 8, 256), 256, 0, st, (const bf16*)x, (bf16*)y, (const bf16*)mask_src, n, p,
             seed, stream_id, step_ptr);
  return RB_LAUNCH_OK();
}

int rb_relu_mask(void* d, const void* y, long long n, cudaStream_t st) {
  if (n % 8) return -10;
  launch_pdl(relu_mask_kernel, grid_for(n / 8, 256), 256, 0, st, (bf16*)d, (const bf16*)y, n);
  return RB_LAUNCH_OK();
}

int rb_add_bf16(void* a, const void* b, long long n, cudaStream_t st) {
  if (n % 8) return -10;
  launch_pdl(add_kernel, grid_for(n / 8, 256), 256, 0, st, (bf16*)a, (const bf16*)b, n);
  return RB_LAUNCH_OK();
}

int rb_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t st) {
  launch_pdl(f32_to_bf16_kernel, grid_for(n, 256), 256, 0, st, x, (bf16*)y, n);
  return RB_LAUNCH_OK();
}

int rb_pack_dgrad_filters(const void* w, void* wt, int Kout, int Kp, int RS, int Cp, cudaStream_t st) {
  launch_pdl(pack_dgrad_filters_kernel, grid_for((long long)Cp * RS * Kp, 256), 256, 0, st, (const bf16*)w, (bf16*)wt,
             Kout, Kp, RS, Cp);
  return RB_LAUNCH_OK();
}

int rb_zero_s2d_structural(float* dw, int Kout, int R2, int Cp, int f, int cin, int ksize, cudaStream_t st) {
  launch_pdl(zero_s2d_structural_kernel, grid_for((long long)Kout * R2 * R2 * Cp, 256), 256, 0, st, dw, Kout, R2, Cp,
             f, cin, ksize);
  return RB_LAUNCH_OK();
}

}  // extern "C"
