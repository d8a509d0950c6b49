// Fill-only TMA probes: loads into a ring of shared-memory stages with no MMA behind them, to measure what the TMA
// path itself delivers. Two patterns:
//   rb_tma_probe_tiled       2-D tiled boxes of 64- or 128-byte rows at a chosen row pitch, issued by 1-4 threads
//                            (lanes of one warp, or one lane of each of several warps), any number of stages in flight;
//   rb_tma_probe_conv_stage  the loads of one pipeline stage of a 5 x 5 convolution forward pass on 27 x 27 images
//                            (two im2col boxes of 128 positions + one strided 3-D box of 256 filter rows).
// What they showed on B200 (one thread's loads do not overlap; im2col loads are bound by rows, not bytes) is what
// the producers of gemm_tc.cu are built around. Every wait is bounded and reports through the status word.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "ptx.cuh"

namespace rb {

struct ProbeArgs {
  CUtensorMap tm;
  int rows_total;   // rows of the source tensor (128-byte rows)
  int box_rows;
  int stages;
  int iters;        // tiles per CTA
  int shared_src;   // 1: all CTAs read the same tiles
  int inner_bytes;  // 64 or 128
  int issuers;      // warps that issue loads (each its own stages)
  int lane_mode;    // 1: the issuers are lanes 0.. of warp 0 instead of warps
  unsigned int* status;
};

__global__ void __launch_bounds__(128, 1) tma_probe_kernel(const __grid_constant__ ProbeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_all[4][16];
  const int tile_bytes = a.box_rows * a.inner_bytes;
  if (threadIdx.x == 0) {
    for (int w = 0; w < 4; ++w)
      for (int s = 0; s < a.stages; ++s) mbar_init(&full_all[w][s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  int warp = threadIdx.x >> 5;
  if (a.lane_mode) {
    if (threadIdx.x >= a.issuers) return;
    warp = threadIdx.x;
  } else if ((threadIdx.x & 31) != 0 || warp >= a.issuers) return;
  uint64_t* full = full_all[warp];
  uint8_t* mine = tiles + warp * a.stages * tile_bytes;
  const int tiles_total = a.rows_total / a.box_rows;
  int s = 0;
  uint32_t ph = 0;
  const int my_iters = a.iters / a.issuers;
  const int base = a.shared_src ? warp * my_iters : (blockIdx.x * a.issuers + warp) * my_iters;
  for (int i = 0; i < my_iters + a.stages; ++i) {
    if (i >= a.stages) {
      if (!mbar_wait_bounded(&full[s], ph, 2000000000ull)) { atomicOr(a.status, 1u); return; }
    }
    if (i < my_iters) {
      const int t = (base + i) % tiles_total;
      mbar_expect_tx(&full[s], (uint32_t)tile_bytes);
      tma_load_2d(mine + s * tile_bytes, &a.tm, &full[s], 0, t * a.box_rows);
    }
    if (++s == a.stages) { s = 0; if (i >= a.stages) ph ^= 1u; }
  }
}


struct StageArgs {
  CUtensorMap tm_a, tm_b;
  int stages, iters, do_a, do_b, a_lanes, a_bytes, b_bytes, cchunks, S, P, Q, bk;
  unsigned int* status;
};

__global__ void __launch_bounds__(64, 1) tma_stage_probe_kernel(const __grid_constant__ StageArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[2][8];
  if (threadIdx.x == 0) {
    for (int w = 0; w < 2; ++w) for (int s = 0; s < a.stages; ++s) mbar_init(&full[w][s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && !a.do_a) return;
  if (warp == 1 && !a.do_b) return;
  const int stage_bytes = 2 * a.a_bytes + a.b_bytes;
  int s = 0; uint32_t ph = 0;
  const int pq = a.P * a.Q;
  for (int i = 0; i < a.iters + a.stages; ++i) {
    int ok = 1;
    if (lane == 0) {
      if (i >= a.stages) ok = mbar_wait_bounded(&full[warp][s], ph, 2000000000ull) ? 1 : 0;
      if (ok && i < a.iters) mbar_expect_tx(&full[warp][s], warp == 0 ? (uint32_t)(a.a_lanes * a.a_bytes * 2 / a.a_lanes) : (uint32_t)a.b_bytes);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) { if (lane == 0) atomicOr(a.status, 1u); return; }
    if (i < a.iters) {
      const int kb = i % (25 * a.cchunks);
      const int tap = kb / a.cchunks, cc = kb - tap * a.cchunks;
      uint8_t* st = tiles + s * stage_bytes;
      if (warp == 0) {
        if (lane < a.a_lanes) {
          const int rows_per = 256 / a.a_lanes;
          const int pix = ((blockIdx.x * 7 + i / (25 * a.cchunks)) * 256 + lane * rows_per) % (128 * pq - 256);
          const int n = pix / pq, r2 = pix - n * pq, pp = r2 / a.Q, qq = r2 - pp * a.Q;
          tma_load_im2col_4d(st + lane * rows_per * a.bk * 2, &a.tm_a, &full[0][s], cc * a.bk, qq - 2, pp - 2, n,
                             (uint16_t)(tap % 5), (uint16_t)(tap / 5));
        }
      } else if (lane == 0) {
        tma_load_3d(st + 2 * a.a_bytes, &a.tm_b, &full[1][s], cc * a.bk, tap, 0);
      }
    }
    __syncwarp();
    if (++s == a.stages) { s = 0; if (i >= a.stages) ph ^= 1u; }
  }
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_enc_tiled = nullptr;
static EncodeIm2colFn g_enc_im2col = nullptr;

static int probe_init() {
  if (g_enc_tiled && g_enc_im2col) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -1;
  g_enc_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -1;
  g_enc_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  cudaFuncSetAttribute(tma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaFuncSetAttribute(tma_stage_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  return 0;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rb_tma_probe_tiled(const void* src, long long rows_total, int box_rows, int stages, int iters, int shared_src,
                         int blocks, int inner_bytes, long long pitch_bytes, int issuers, int lane_mode, unsigned int* status,
                         cudaStream_t st) {
  if (probe_init()) return -1;
  EncodeTiledFn enc = g_enc_tiled;
  if (stages < 1 || stages > 16 || issuers < 1 || issuers > 4 || issuers * stages * box_rows * inner_bytes > 190 * 1024 || box_rows > 256) return -10;
  ProbeArgs a;
  cuuint64_t dims[2] = {(cuuint64_t)inner_bytes / 2, (cuuint64_t)rows_total};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)inner_bytes / 2, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  if (enc(&a.tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(src), dims, strides, box, es,
          CU_TENSOR_MAP_INTERLEAVE_NONE, inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -2;
  a.rows_total = (int)rows_total; a.box_rows = box_rows; a.stages = stages; a.iters = iters; a.shared_src = shared_src;
  a.status = status; a.inner_bytes = inner_bytes; a.issuers = issuers; a.lane_mode = lane_mode;
  tma_probe_kernel<<<blocks, 128, issuers * stages * box_rows * inner_bytes + 1024, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int rb_tma_probe_conv_stage(const void* x, const void* w, int C, int bk, int stages, int iters, int do_a, int do_b,
                      int a_lanes, int blocks, unsigned int* status, cudaStream_t stm) {
  if (probe_init()) return -1;
  EncodeTiledFn enc = g_enc_tiled;
  EncodeIm2colFn enc2 = g_enc_im2col;
  if ((bk != 32 && bk != 64) || C % bk || stages < 1 || stages > 8 || a_lanes < 1 || a_lanes > 8 || 256 % a_lanes ||
      stages * (4 * 128 * bk + 2 * 256 * bk) > 190 * 1024)
    return -10;
  StageArgs a;
  const int N = 128, H = 27, W = 27, Kout = 256;
  const CUtensorMapSwizzle sw = bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  {
    cuuint64_t dims[4] = {(cuuint64_t)C, W, H, N};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)C * W * 2, (cuuint64_t)C * W * H * 2};
    int lower[2] = {-2, -2}, upper[2] = {-2, -2};
    cuuint32_t es[4] = {1, 1, 1, 1};
    if (enc2(&a.tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, lower, upper, bk,
             256 / a_lanes, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -2;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)C, 25, Kout};
    cuuint64_t strides[2] = {(cuuint64_t)C * 2, (cuuint64_t)25 * C * 2};
    cuuint32_t box[3] = {(cuuint32_t)bk, 1, 256};
    cuuint32_t es[3] = {1, 1, 1};
    if (enc(&a.tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -3;
  }
  a.stages = stages; a.iters = iters; a.do_a = do_a; a.do_b = do_b; a.a_lanes = a_lanes; a.bk = bk;
  a.a_bytes = 128 * bk * 2; a.b_bytes = 256 * bk * 2; a.cchunks = C / bk; a.S = 5; a.P = 27; a.Q = 27; a.status = status;
  tma_stage_probe_kernel<<<blocks, 64, stages * (2 * a.a_bytes + a.b_bytes) + 1024, stm>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
