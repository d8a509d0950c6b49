// Persistent, warp-specialised tcgen05 GEMM / implicit-GEMM convolution for sm_100a.
//
//   warp 0      TMA producer (one elected lane): tiled or im2col loads into a ring of smem stages
//   warp 1      MMA issuer (one elected lane): tcgen05.mma, fp32 accumulators in TMEM (2 x 256 columns,
//               so the epilogue of tile i overlaps the main loop of tile i+1); owns TMEM alloc/dealloc
//   warps 2..5  epilogue: tcgen05.ld -> bias / ReLU / mask -> bf16 stores, or fp32 store / red.add (split-K)
//
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, records
// RB_STATUS_MBAR_TIMEOUT in the status word, drains its outstanding TMA copies (bounded),
// frees TMEM and returns. No TMA load here uses cluster multicast.
#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "common.cuh"

namespace rb {

constexpr int BM = 128;
constexpr int GEMM_THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr int TILE_SMEM_BYTES = 192 * 1024;
constexpr int GEMM_SMEM_BYTES = TILE_SMEM_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct SharedCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ bool ctl_wait(SharedCtl* ctl, uint64_t* bar, uint32_t parity, unsigned int* status) {
  if (ctl->abort_flag) return false;
  if (mbar_wait_bounded(bar, parity, WAIT_LIMIT_NS)) return true;
  ctl->abort_flag = 1;
  if (status) atomicOr(status, RB_STATUS_MBAR_TIMEOUT);
  return false;
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  // tiles start on a 1024-byte boundary (swizzle atoms); control block follows the tiles
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(tiles + TILE_SMEM_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int a_bytes = BM * p.bk * 2;
  const int b_bytes = p.bn * p.bk * 2;
  const int stage_bytes = a_bytes + b_bytes;
  const int stages = p.stages;

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = p.n_tiles;
  const int num_work = m_tiles * n_tiles * p.split_k;
  const int kb_per_split = (p.num_kb + p.split_k - 1) / p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], 4);
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_a);
    tma_prefetch_desc(&p.tm_b);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        const int z = work / (m_tiles * n_tiles);
        const int rem = work - z * (m_tiles * n_tiles);
        const int tn = rem / m_tiles;
        const int tm = rem - tn * m_tiles;
        const int m0 = tm * BM;
        const int kb0 = z * kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + kb_per_split);

        // geometry that is fixed for the tile
        int a_w = 0, a_h = 0, a_n = 0;
        if (p.a_mode == A_IM2COL_K) {
          const int pq = p.cv_P * p.cv_Q;
          a_n = m0 / pq;
          const int r2 = m0 - a_n * pq;
          const int pp = r2 / p.cv_Q;
          const int qq = r2 - pp * p.cv_Q;
          a_w = qq * p.cv_stride + p.cv_lower_w;
          a_h = pp * p.cv_stride + p.cv_lower_h;
        }
        int b_tap = 0, b_c0 = 0, n0 = tn * p.bn;
        if (p.b_mode == B_IM2COL_MN) {
          b_tap = tn / p.wg_ctiles;
          b_c0 = (tn - b_tap * p.wg_ctiles) * p.bn;
        }

        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ctl_wait(ctl, &ctl->empty[s], ph ^ 1u, p.status)) { ok = false; break; }
          uint8_t* sa = tiles + s * stage_bytes;
          uint8_t* sb = sa + a_bytes;
          mbar_expect_tx(&ctl->full[s], (uint32_t)stage_bytes);
          // ---- A ----
          if (p.a_mode == A_TILED_K) {
            tma_load_2d(sa, &p.tm_a, &ctl->full[s], kb * p.bk, m0);
          } else if (p.a_mode == A_IM2COL_K) {
            const int tap = kb / p.cv_cchunks;
            const int cc = kb - tap * p.cv_cchunks;
            const int r = tap / p.cv_S;
            const int sx = tap - r * p.cv_S;
            tma_load_im2col_4d(sa, &p.tm_a, &ctl->full[s], cc * p.bk, a_w, a_h, a_n, (uint16_t)sx, (uint16_t)r);
          } else {  // A_TILED_MN: two boxes of 64 rows(M) x bk
            tma_load_2d(sa, &p.tm_a, &ctl->full[s], m0, kb * p.bk);
            tma_load_2d(sa + p.bk * 128, &p.tm_a, &ctl->full[s], m0 + 64, kb * p.bk);
          }
          // ---- B ----
          if (p.b_mode == B_TILED_K) {
            tma_load_2d(sb, &p.tm_b, &ctl->full[s], kb * p.bk, n0);
          } else if (p.b_mode == B_TILED_K3) {
            const int tap = kb / p.cv_cchunks;
            const int cc = kb - tap * p.cv_cchunks;
            tma_load_3d(sb, &p.tm_b, &ctl->full[s], cc * p.bk, tap, n0);
          } else if (p.b_mode == B_TILED_MN) {
            for (int j = 0; j < p.bn / 64; ++j)
              tma_load_2d(sb + j * p.bk * 128, &p.tm_b, &ctl->full[s], n0 + 64 * j, kb * p.bk);
          } else {  // B_IM2COL_MN
            const int pix = kb * p.bk;
            const int pq = p.cv_P * p.cv_Q;
            const int n_img = pix / pq;
            const int r2 = pix - n_img * pq;
            const int pp = r2 / p.cv_Q;
            const int qq = r2 - pp * p.cv_Q;
            const int w = qq * p.cv_stride + p.cv_lower_w;
            const int h = pp * p.cv_stride + p.cv_lower_h;
            const int r = b_tap / p.cv_S;
            const int sx = b_tap - r * p.cv_S;
            for (int j = 0; j < p.bn / 64; ++j)
              tma_load_im2col_4d(sb + j * p.bk * 128, &p.tm_b, &ctl->full[s], b_c0 + 64 * j, w, h, n_img,
                                 (uint16_t)sx, (uint16_t)r);
          }
          ++issued;
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        // drain: wait (bounded) until the copies already issued have landed
        const int back = min(issued, stages);
        int ds = s;
        uint32_t dph = ph;
        for (int i = 0; i < back; ++i) {
          if (ds == 0) { ds = stages; dph ^= 1u; }
          --ds;
          mbar_wait_bounded(&ctl->full[ds], dph, 100000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const bool a_mn = (p.a_mode == A_TILED_MN);
      const bool b_mn = (p.b_mode == B_TILED_MN || p.b_mode == B_IM2COL_MN);
      const uint32_t idesc = make_idesc_bf16(BM, (uint32_t)p.bn, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
      // K-major: rows of bk*2 bytes, 8-row atoms -> SBO = 8*bk*2; swizzle 128B (bk=64) or 64B (bk=32)
      // MN-major: 64-element (128 B) rows per k, atoms of 8 k -> SBO = 1024, LBO = bk*128 between 64-wide blocks
      const uint32_t k_layout = (p.bk == 64) ? 2u : 4u;
      const uint32_t a_lbo = a_mn ? (uint32_t)p.bk * 128u : 16u;
      const uint32_t a_sbo = a_mn ? 1024u : (uint32_t)p.bk * 16u;
      const uint32_t a_lay = a_mn ? 2u : k_layout;
      const uint32_t b_lbo = b_mn ? (uint32_t)p.bk * 128u : 16u;
      const uint32_t b_sbo = b_mn ? 1024u : (uint32_t)p.bk * 16u;
      const uint32_t b_lay = b_mn ? 2u : k_layout;
      const uint32_t a_adv = a_mn ? (2048u >> 4) : (32u >> 4);  // per 16-deep MMA, in 16-byte units
      const uint32_t b_adv = b_mn ? (2048u >> 4) : (32u >> 4);
      const int kk_steps = p.bk / 16;

      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        const int z = work / (m_tiles * n_tiles);
        const int kb0 = z * kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + kb_per_split);
        if (!ctl_wait(ctl, &ctl->acc_empty[acc], acc_ph ^ 1u, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * 256u;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ctl_wait(ctl, &ctl->full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + s * stage_bytes);
          const uint32_t sb = sa + (uint32_t)a_bytes;
          const uint64_t da = make_smem_desc(sa, a_lbo, a_sbo, a_lay);
          const uint64_t db = make_smem_desc(sb, b_lbo, b_sbo, b_lay);
          for (int kk = 0; kk < kk_steps; ++kk) {
            tc_mma_f16(d_tmem, da + (uint64_t)(a_adv * kk), db + (uint64_t)(b_adv * kk), idesc,
                       (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&ctl->empty[s]);  // stage is free once these MMAs have read it
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&ctl->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int lane_base = (warp & 3) * 32;  // TMEM lanes this warp may read
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      const int z = work / (m_tiles * n_tiles);
      const int rem = work - z * (m_tiles * n_tiles);
      const int tn = rem / m_tiles;
      const int tm = rem - tn * m_tiles;
      (void)z;
      if (!ctl_wait(ctl, &ctl->acc_full[acc], acc_ph, p.status)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + lane_base + lane;
      const bool row_ok = row < p.M;
      int col0;        // first column of D this tile writes
      int col_limit;   // tile-local bound on stored columns
      if (p.b_mode == B_IM2COL_MN) {
        const int tap = tn / p.wg_ctiles;
        const int c0 = (tn - tap * p.wg_ctiles) * p.bn;
        col0 = tap * p.wg_cpad + c0;
        col_limit = min(p.bn, p.wg_cpad - c0);
      } else {
        col0 = tn * p.bn;
        col_limit = min(p.bn, p.n_store - col0);
      }
      const uint32_t t_addr = tmem_base + (uint32_t)acc * 256u + ((uint32_t)lane_base << 16);
      for (int c = 0; c < p.bn; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_addr + (uint32_t)c, v);
        tmem_ld_wait();
        if (!row_ok || c >= col_limit) continue;
        const int gcol = col0 + c;
        if (p.epi == EPI_BF16) {
          __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + (size_t)row * p.ldd + gcol;
          const __nv_bfloat16* mrow = p.mask_src ? p.mask_src + (size_t)row * p.ldd + gcol : nullptr;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int n = gcol + q * 8 + j;
              float x = __uint_as_float(v[q * 8 + j]);
              if (n < p.n_valid) {
                if (p.bias) x += __ldg(p.bias + n);
                if (p.relu) x = fmaxf(x, 0.f);
              } else {
                x = 0.f;
              }
              f[j] = x;
            }
            if (mrow) {
              const uint4 mv = *reinterpret_cast<const uint4*>(mrow + q * 8);
              const __nv_bfloat162* m2 = reinterpret_cast<const __nv_bfloat162*>(&mv);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 mf = __bfloat1622float2(m2[j]);
                if (!(mf.x > 0.f)) f[2 * j] = 0.f;
                if (!(mf.y > 0.f)) f[2 * j + 1] = 0.f;
              }
            }
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            *reinterpret_cast<uint4*>(drow + q * 8) = o;
          }
        } else {
          float* drow = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + gcol;
          if (p.epi == EPI_F32_STORE) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                     __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
              *reinterpret_cast<float4*>(drow + 4 * q) = o;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(drow + 4 * q),
                           "f"(__uint_as_float(v[4 * q])), "f"(__uint_as_float(v[4 * q + 1])),
                           "f"(__uint_as_float(v[4 * q + 2])), "f"(__uint_as_float(v[4 * q + 3]))
                           : "memory");
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// =============================== host side ===============================

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;
static int g_num_sms = 0;
static int g_driver_version = 0;

static int ensure_driver_entry() {
  if (g_encode_tiled && g_encode_im2col) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
    return -1;
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
    return -1;
  g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDriverGetVersion(&g_driver_version);
  if (cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) !=
      cudaSuccess)
    return -2;
  return 0;
}

// 2-D bf16 map: dims {inner, outer}, outer pitch in elements, box {bi, bo}.
static int make_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
                       uint32_t bi, uint32_t bo, CUtensorMapSwizzle sw) {
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {bi, bo};
  cuuint32_t es[2] = {1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(100 + (int)r);
}
static int make_map_3d(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                       uint64_t pitch2, uint32_t b0, uint32_t b1, uint32_t b2, CUtensorMapSwizzle sw) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1 * 2, pitch2 * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(100 + (int)r);
}
// NHWC bf16 im2col map. The base pixel ranges over [lower, dim + upper) per spatial axis;
// a load fetches `pixels` base pixels (w fastest, then h, then n) x `channels` channels.
static int make_map_im2col(CUtensorMap* m, const void* ptr, int N, int H, int W, int C, int lower_h, int lower_w,
                           int upper_h, int upper_w, int stride, uint32_t channels, uint32_t pixels,
                           CUtensorMapSwizzle sw) {
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)C * W * 2, (cuuint64_t)C * W * H * 2};
  int lower[2] = {lower_w, lower_h};
  int upper[2] = {upper_w, upper_h};
  cuuint32_t es[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = g_encode_im2col(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, lower,
                               upper, channels, pixels, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(200 + (int)r);
  // Drivers up to 13.1 mis-handle im2col maps of tensors smaller than 128 KiB unless bit 21 of the
  // second descriptor word is cleared (same adjustment CUTLASS applies to its im2col descriptors).
  if (g_driver_version <= 13010 && (size_t)N * H * W * C * 2 < 131072) {
    reinterpret_cast<uint64_t*>(m)[1] &= ~(1ull << 21);
  }
  return 0;
}

static int pick_stages(int bn, int bk) {
  const int stage = (BM + bn) * bk * 2;
  int s = TILE_SMEM_BYTES / stage;
  if (s > MAX_STAGES) s = MAX_STAGES;
  return s;
}

static int launch(GemmTcParams& p, cudaStream_t stream, int max_ctas) {
  const int m_tiles = (p.M + BM - 1) / BM;
  const int work = m_tiles * p.n_tiles * p.split_k;
  if (work <= 0) return 0;
  p.stages = pick_stages(p.bn, p.bk);
  if (p.stages < 2) return -3;
  int grid = work < g_num_sms ? work : g_num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_tc_kernel<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// choose a reduction split so that about one wave of CTAs is busy
static int pick_split(int tiles, int num_kb, int min_kb_per_split) {
  if (tiles >= g_num_sms) return 1;
  int s = g_num_sms / tiles;
  int max_s = num_kb / min_kb_per_split;
  if (max_s < 1) max_s = 1;
  if (s > max_s) s = max_s;
  if (s < 1) s = 1;
  // every split must own at least one k-block
  while (s > 1 && (s - 1) * ((num_kb + s - 1) / s) >= num_kb) --s;
  return s;
}

static int round_bn(int n, int cap) {
  int bn = ((n + 31) / 32) * 32;
  if (bn > cap) bn = cap;
  return bn;
}

}  // namespace rb

using namespace rb;

extern "C" {

// Dense GEMM on bf16 operands:  D[M x N] = op(A) * op(B)^T-style contraction over K.
//   a_mn = 0: A is [M][K] (K contiguous, pitch lda)     a_mn = 1: A is [K][M] (M contiguous, pitch lda)
//   b_mn = 0: B is [N][K] (K contiguous, pitch ldb)     b_mn = 1: B is [K][N] (N contiguous, pitch ldb)
//   epi = 0: bf16 D (+bias, ReLU, mask);  epi = 1: fp32 D overwritten;  epi = 2: fp32 D accumulated (red.add)
// split_k <= 0 lets the library choose; epi 0/1 force split_k = 1.
int rb_gemm_tc(const void* A, int a_mn, long long lda, const void* B, int b_mn, long long ldb, int M, int N, int K,
               void* D, long long ldd, int epi, const float* bias, int relu, const void* mask_src, int n_valid,
               int n_store, int split_k, int bn_cap, unsigned int* status, cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  if ((n_store > 0 ? n_store : N) % 32 != 0 || ldd % 8 != 0) return -11;  // epilogue writes 32-column chunks
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  const bool any_mn = a_mn || b_mn;
  p.bk = (!any_mn && (K % 64 != 0) && (K % 32 == 0)) ? 32 : 64;
  if (bn_cap <= 0) bn_cap = 256;
  p.bn = round_bn(N, bn_cap);
  if (b_mn) p.bn = ((p.bn + 63) / 64) * 64;
  p.M = M;
  p.N = N;
  p.num_kb = (K + p.bk - 1) / p.bk;
  p.n_tiles = (N + p.bn - 1) / p.bn;
  const CUtensorMapSwizzle ksw = p.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  if (a_mn) {
    p.a_mode = A_TILED_MN;
    rc = make_map_2d(&p.tm_a, A, M, K, lda, 64, p.bk, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    p.a_mode = A_TILED_K;
    rc = make_map_2d(&p.tm_a, A, K, M, lda, p.bk, BM, ksw);
  }
  if (rc) return rc;
  if (b_mn) {
    p.b_mode = B_TILED_MN;
    rc = make_map_2d(&p.tm_b, B, N, K, ldb, 64, p.bk, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    p.b_mode = B_TILED_K;
    rc = make_map_2d(&p.tm_b, B, K, N, ldb, p.bk, p.bn, ksw);
  }
  if (rc) return rc;
  const int tiles = ((M + BM - 1) / BM) * p.n_tiles;
  if (epi != EPI_F32_ATOMIC) split_k = 1;
  else if (split_k <= 0) split_k = pick_split(tiles, p.num_kb, 4);
  if (split_k > p.num_kb) split_k = p.num_kb;
  while (split_k > 1 && (split_k - 1) * ((p.num_kb + split_k - 1) / split_k) >= p.num_kb) --split_k;
  p.split_k = split_k;
  p.epi = epi;
  p.relu = relu;
  p.n_valid = n_valid > 0 ? n_valid : N;
  p.n_store = n_store > 0 ? n_store : N;
  p.ldd = ldd;
  p.D = D;
  p.bias = bias;
  p.mask_src = reinterpret_cast<const __nv_bfloat16*>(mask_src);
  p.status = status;
  return launch(p, stream, 0);
}

// Convolution forward (also used for stride-1 data-grad with flipped filters).
//   x   NHWC bf16 [N][H][W][Cp]      w  bf16 [Kout][R*S][Cp]     y  bf16 [N*P*Q][ldy]
//   base pixel range: lower = -pad_lo, P/Q given by the caller.
int rb_conv_fprop_tc(const void* x, int N, int H, int W, int Cp, const void* w, int Kout, int R, int S, int stride,
                     int pad_h, int pad_w, int P, int Q, void* y, long long ldy, const float* bias, int relu,
                     const void* mask_src, int n_valid, int n_store, unsigned int* status, cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.bk = (Cp % 64 == 0) ? 64 : 32;
  if (Cp % 32 != 0) return -10;
  if ((n_store > 0 ? n_store : Kout) % 32 != 0 || ldy % 8 != 0) return -11;
  const CUtensorMapSwizzle ksw = p.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  p.bn = round_bn(n_store > 0 ? n_store : Kout, 256);
  p.M = N * P * Q;
  p.N = Kout;
  p.cv_cchunks = Cp / p.bk;
  p.num_kb = R * S * p.cv_cchunks;
  p.n_tiles = ((n_store > 0 ? n_store : Kout) + p.bn - 1) / p.bn;
  p.a_mode = A_IM2COL_K;
  p.b_mode = B_TILED_K3;
  p.cv_P = P;
  p.cv_Q = Q;
  p.cv_stride = stride;
  p.cv_lower_h = -pad_h;
  p.cv_lower_w = -pad_w;
  p.cv_S = S;
  // upper corner so that the base pixel takes exactly P x Q positions
  const int upper_h = (P - 1) * stride - pad_h - (H - 1);
  const int upper_w = (Q - 1) * stride - pad_w - (W - 1);
  rc = make_map_im2col(&p.tm_a, x, N, H, W, Cp, -pad_h, -pad_w, upper_h, upper_w, stride, p.bk, BM, ksw);
  if (rc) return rc;
  rc = make_map_3d(&p.tm_b, w, Cp, (uint64_t)R * S, Kout, Cp, (uint64_t)R * S * Cp, p.bk, 1, p.bn, ksw);
  if (rc) return rc;
  p.split_k = 1;
  p.epi = EPI_BF16;
  p.relu = relu;
  p.n_valid = n_valid > 0 ? n_valid : Kout;
  p.n_store = n_store > 0 ? n_store : Kout;
  p.ldd = ldy;
  p.D = y;
  p.bias = bias;
  p.mask_src = reinterpret_cast<const __nv_bfloat16*>(mask_src);
  p.status = status;
  return launch(p, stream, 0);
}

// Convolution weight-grad:  dw[Kout][R*S][Cp] (fp32) (+)= sum over pixels dy[pix][k] * x[pix shifted by tap][c].
//   accumulate = 0 requires dw to have been zeroed when the reduction is split (the library reports the
//   split it would use through rb_conv_wgrad_split so that callers can zero only when needed).
int rb_conv_wgrad_tc(const void* x, int N, int H, int W, int Cp, const void* dy, long long lddy, int Kout, int R,
                     int S, int stride, int pad_h, int pad_w, int P, int Q, float* dw, int split_k,
                     unsigned int* status, cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.bk = 64;
  int bn = ((Cp + 63) / 64) * 64;
  if (bn > 256) bn = 256;
  if (Cp > 256 && Cp % 256 != 0 && Cp % 128 == 0) bn = 128;
  p.bn = bn;
  p.M = Kout;
  p.N = R * S * Cp;
  const long long pixels = (long long)N * P * Q;
  p.num_kb = (int)((pixels + p.bk - 1) / p.bk);
  p.wg_ctiles = (Cp + p.bn - 1) / p.bn;
  p.wg_cpad = Cp;
  p.n_tiles = R * S * p.wg_ctiles;
  p.a_mode = A_TILED_MN;
  p.b_mode = B_IM2COL_MN;
  p.cv_P = P;
  p.cv_Q = Q;
  p.cv_stride = stride;
  p.cv_lower_h = -pad_h;
  p.cv_lower_w = -pad_w;
  p.cv_S = S;
  const int upper_h = (P - 1) * stride - pad_h - (H - 1);
  const int upper_w = (Q - 1) * stride - pad_w - (W - 1);
  rc = make_map_2d(&p.tm_a, dy, Kout, (uint64_t)pixels, lddy, 64, p.bk, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_map_im2col(&p.tm_b, x, N, H, W, Cp, -pad_h, -pad_w, upper_h, upper_w, stride, 64, p.bk,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const int tiles = ((Kout + BM - 1) / BM) * p.n_tiles;
  if (split_k <= 0) split_k = pick_split(tiles, p.num_kb, 8);
  if (split_k > p.num_kb) split_k = p.num_kb;
  while (split_k > 1 && (split_k - 1) * ((p.num_kb + split_k - 1) / split_k) >= p.num_kb) --split_k;
  p.split_k = split_k;
  p.epi = EPI_F32_ATOMIC;
  p.n_valid = p.N;
  p.n_store = p.N;
  p.ldd = (long long)R * S * Cp;
  p.D = dw;
  p.status = status;
  return launch(p, stream, 0);
}

int rb_num_sms() {
  ensure_driver_entry();
  return g_num_sms;
}

}  // extern "C"
