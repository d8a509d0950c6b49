// Persistent, warp-specialised tcgen05 GEMM / implicit-GEMM convolution for sm_100a.
//
//   warp 0      A producer: TMA loads (tiled, im2col, or halo tiles) of the A operand, one lane per box
//   warp 1      MMA issuer (one elected lane): tcgen05.mma, fp32 accumulators in TMEM; owns TMEM alloc/dealloc
//   warps 2..9  epilogue: tcgen05.ld -> bias / ReLU / mask -> swizzled smem -> TMA store (bf16), or fp32 TMA
//               store / reduce-add (split-K, gradient accumulation). Two warps share each TMEM lane quarter and
//               alternate column slabs: with one warp per scheduler the epilogue is bound by instruction latency.
//   warp 10     B producer: TMA loads of the B operand, one lane per box (or the resident panel, once)
//
// What was measured on this kernel and shaped it:
//   * one thread's TMA loads do not overlap (a box takes ~220 ns whatever its size) while loads issued by different
//     threads do, so the loads of a stage are spread over two producer warps and over lanes;
//   * im2col-mode loads cost ~2.8 ns per pixel row per SM and tiled loads 1-1.7 ns per row, independent of the
//     row's bytes: rows are kept 128 bytes wide (64 channels) even when that means a half-empty, zero-filled chunk;
//   * a tcgen05.mma (cta_group::1, M = 128, K = 16) costs ~200 cycles however narrow N is, so tiles are as wide as
//     the layer allows (N <= 256);
//   * a work item may cover two 128-row sub-tiles (mt = 2) that share one B stage and use two accumulators; when
//     the whole B panel fits in shared memory and the CTA only ever needs that one panel, it is loaded once per CTA
//     and stays resident (b_resident); split-K (fp32 reduce-add epilogue) spreads long reductions over all SMs;
//   * which of these a forward / data-grad launch uses is decided by timing the candidates the first time a shape
//     is seen (the launches are idempotent), see `launch`.
//   * stride-1 convolutions can load A as column-shifted halo tiles (A_HALO_K): a sub-tile is hl_rows output rows
//     of one image laid out at a row pitch of hl_pitch positions (128 rows of the MMA; positions past the image
//     width or height are computed and dropped by the clipping TMA store). For filter column s the producer
//     loads ONE tile of (mt * hl_rows + R - 1) input rows x hl_pitch columns starting at column s - pad (plain
//     tiled TMA, zero fill outside the image); the R filter rows of that column are then descriptor offsets of
//     r * hl_pitch rows into the same tile (multiples of the swizzle atom), so A is filled S times per item
//     instead of R * S times. B streams through its own ring, one (r, s, channel chunk) tile per stage. Taken
//     only when forced (RB_GEMM_FORCE_HALO=1): its padded tiles add MMA work, and MMA issue is what binds there.
// With two accumulator sets in TMEM the epilogue of work item i overlaps the main loop of item i+1; a
// 256 x 256 item needs all 512 columns and runs without that overlap.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, records
// RB_STATUS_MBAR_TIMEOUT in the status word, drains its outstanding TMA copies (bounded),
// frees TMEM and returns. No TMA load here uses cluster multicast.
#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "common.cuh"
#include "launch.cuh"
#include <ctype.h>
#include <stdlib.h>
#include <map>
#include <mutex>
#include <tuple>

namespace rb {

constexpr int BM = 128;
constexpr int GEMM_THREADS = 352;   // A-producer warp, MMA warp, 8 epilogue warps, B-producer warp
// Register budget: 352 threads x 144 registers leave 14.8 K of the SM's 64 K registers free, which is what one
// 128-thread block of the exchange kernels (80 registers per thread, 10 K) needs to run beside a resident CTA of this
// kernel. Above 155 registers those blocks no longer fit and the gradient exchange stops overlapping the backward
// pass (measured: 2.29 instead of 1.98 ms per AlexNet step on 2 GPUs); tests/test_register_budget.py keeps watch.
// Registers are handed out to whole warps, four warps at a time: the CTA's 11 warps take 12 x 32 x 144 = 55296, and
// the 10240 left are exactly the four warps x 80 registers of an exchange block. Hence the hard cap.
constexpr int GEMM_MAX_REGS = 144;
constexpr int PRODUCER_B_WARP = 10;
constexpr int EPI_WARPS = 8;
constexpr int MAX_STAGES = 8;
constexpr int TILE_SMEM_BYTES = 192 * 1024;   // B panel (if resident) + stage ring
constexpr int STAGING_BYTES = 32 * 1024;      // epilogue: 8 warps x one slab of 32 rows x 128 B
constexpr int GEMM_SMEM_BYTES = TILE_SMEM_BYTES + STAGING_BYTES + 1024 /*align*/ + 512 /*barriers*/;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct SharedCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t b_full;
  uint64_t a_full[2];    // halo mode: the A ring has its own barriers
  uint64_t a_empty[2];
  uint64_t mask_bar[EPI_WARPS];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ bool ctl_wait(SharedCtl* ctl, uint64_t* bar, uint32_t parity, unsigned int* status) {
  if (mbar_try_wait(bar, parity)) return true;    // the common case costs one instruction, no read of the abort flag
  if (ctl->abort_flag) return false;
  if (mbar_wait_bounded(bar, parity, WAIT_LIMIT_NS)) return true;
  ctl->abort_flag = 1;
  if (status) atomicOr(status, RB_STATUS_MBAR_TIMEOUT);
  return false;
}

// Role profile (built only with -DRB_GEMM_PROFILE, see `python -m rembrandt_b200._build --profile`): cycles that the
// roles of ONE CTA (block 3) spend waiting, summed over launches -- [0] A producer on a free stage, [1] B producer on
// a free stage, [2] MMA issuer on a filled stage, [3] MMA issuer on a drained accumulator, [4] the CTA's whole run,
// and for ONE epilogue warp (warp 2) in the bf16 epilogue: [5] waiting for a filled accumulator, [6] proxy fence +
// issue of the TMA store of a slab, [7] a slab's way from TMEM through registers into shared memory.
// A role that hardly waits is the one the others wait for. `rb_gemm_role_profile` reads and clears the counters.
#ifdef RB_GEMM_PROFILE
__device__ unsigned long long g_role_cycles[8];
__device__ __forceinline__ bool ctl_wait_role(SharedCtl* ctl, uint64_t* bar, uint32_t parity, unsigned int* status,
                                              int slot) {
  const long long t0 = clock64();
  const bool r = ctl_wait(ctl, bar, parity, status);
  if (blockIdx.x == 3) atomicAdd(&g_role_cycles[slot], (unsigned long long)(clock64() - t0));
  return r;
}
#else
__device__ __forceinline__ bool ctl_wait_role(SharedCtl* ctl, uint64_t* bar, uint32_t parity, unsigned int* status,
                                              int) {
  return ctl_wait(ctl, bar, parity, status);
}
#endif

#ifdef RB_GEMM_PROFILE
#define RB_PROF_T0(cond) const long long prof_t0_ = (cond) ? clock64() : 0
#define RB_PROF_ADD(cond, slot) \
  if ((cond) && blockIdx.x == 3 && (threadIdx.x & 31) == 0) \
    atomicAdd(&g_role_cycles[slot], (unsigned long long)(clock64() - prof_t0_))
#else
#define RB_PROF_T0(cond)
#define RB_PROF_ADD(cond, slot)
#endif

// base pixel (w, h, n) of output position `pix` for the im2col tensor maps
__device__ __forceinline__ void pixel_coords(const GemmTcParams& p, int pix, int& w, int& h, int& n) {
  const int pq = p.cv_P * p.cv_Q;
  n = pix / pq;
  const int r2 = pix - n * pq;
  const int pp = r2 / p.cv_Q;
  const int qq = r2 - pp * p.cv_Q;
  w = qq * p.cv_stride + p.cv_lower_w;
  h = pp * p.cv_stride + p.cv_lower_h;
}

// One unit of a CTA's work list: tile (tm, tn) over k-blocks [kb0, kb1). `tail` >= 0 marks a part of a cut item of
// the last wave (index among the cut items); its sums go to the fp32 workspace instead of D.
struct WorkItem {
  int tm, tn, kb0, kb1, tail;
};
__device__ __forceinline__ WorkItem decode_work(const GemmTcParams& p, int work, int m_items, int direct,
                                                int kb_per_split) {
  WorkItem w;
  int rem;
  if (p.tail_items > 0 && work >= direct) {
    const int w2 = work - direct;
    const int part = w2 / p.tail_items;
    w.tail = w2 - part * p.tail_items;
    rem = direct + w.tail;
    const int kbs = (p.num_kb + p.tail_split - 1) / p.tail_split;
    w.kb0 = part * kbs;
    w.kb1 = min(p.num_kb, w.kb0 + kbs);
  } else {
    const int per = m_items * p.n_tiles;
    const int z = work / per;
    rem = work - z * per;
    w.kb0 = z * kb_per_split;
    w.kb1 = min(p.num_kb, w.kb0 + kb_per_split);
    w.tail = -1;
  }
  w.tn = rem / m_items;
  w.tm = rem - w.tn * m_items;
  return w;
}

__device__ __forceinline__ void load_b(const GemmTcParams& p, uint8_t* sb, uint64_t* bar, int kb, int n0, int b_tap,
                                       int b_c0) {
  const int b_split = p.b_split > 0 ? p.b_split : 1;
  const int b_rows = p.bn_load / b_split;
  if (p.b_mode == B_TILED_K) {
    for (int q = 0; q < b_split; ++q)
      tma_load_2d(sb + q * b_rows * p.bk * 2, &p.tm_b, bar, kb * p.bk, n0 + q * b_rows);
  } else if (p.b_mode == B_TILED_K3) {
    const int tap = kb / p.cv_cchunks;
    const int cc = kb - tap * p.cv_cchunks;
    for (int q = 0; q < b_split; ++q)
      tma_load_3d(sb + q * b_rows * p.bk * 2, &p.tm_b, bar, cc * p.bk, tap, n0 + q * b_rows);
  } else if (p.b_mode == B_TILED_MN) {
    for (int j = 0; j < p.bn_load / 64; ++j) tma_load_2d(sb + j * p.bk * 128, &p.tm_b, bar, n0 + 64 * j, kb * p.bk);
  } else {  // B_IM2COL_MN
    int w, h, n_img;
    pixel_coords(p, kb * p.bk, w, h, n_img);
    if (p.wg_taps > 1) {
      // several filter taps side by side in one column tile: they share the A (dY) stage
      const int apt = p.wg_cw / 64;  // 64-column atoms per tap
      for (int t = 0; t < p.wg_taps; ++t) {
        const int tap = min(b_tap + t, p.wg_ntaps - 1);   // slots past the last tap reload it; the epilogue skips them
        const int r = tap / p.cv_S;
        const int sx = tap - r * p.cv_S;
        for (int j = 0; j < apt; ++j)
          tma_load_im2col_4d(sb + (t * apt + j) * p.bk * 128, &p.tm_b, bar, 64 * j, w, h, n_img, (uint16_t)sx,
                             (uint16_t)r);
      }
    } else {
      const int r = b_tap / p.cv_S;
      const int sx = b_tap - r * p.cv_S;
      for (int j = 0; j < p.bn_load / 64; ++j)
        tma_load_im2col_4d(sb + j * p.bk * 128, &p.tm_b, bar, b_c0 + 64 * j, w, h, n_img, (uint16_t)sx, (uint16_t)r);
    }
  }
}

// The MMAs of one k-block, fully unrolled: MT sub-tiles x KK 16-deep steps (x 2 for a tile wider than 256 columns).
// The one issuing thread's instruction stream is what bounds the kernel when operands arrive in time (a single extra
// branch per MMA in this loop cost 44 % on a weight-grad launch), so nothing here is computed per MMA that can be
// computed per k-block, and only the first MMA into an accumulator carries a predicate.
template <int KK, int MT, bool WIDE, bool PAIR>
__device__ __forceinline__ void issue_kblock(uint32_t d_tmem, uint32_t acc_stride, uint64_t da, uint64_t a_sub,
                                             uint64_t db, uint32_t a_adv, uint32_t b_adv, uint32_t idesc,
                                             uint32_t idesc2, uint64_t b_wide_off, bool fresh) {
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    const uint32_t dj = d_tmem + (uint32_t)j * acc_stride;
    const uint64_t daj = da + (uint64_t)j * a_sub;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const uint64_t ak = daj + (uint64_t)(a_adv * kk), bk_ = db + (uint64_t)(b_adv * kk);
      if (PAIR) {
        if (kk == 0) tc_mma2_f16(dj, ak, bk_, idesc, fresh ? 0u : 1u);
        else tc_mma2_f16_acc(dj, ak, bk_, idesc);
      } else if (kk == 0) {
        tc_mma_f16(dj, ak, bk_, idesc, fresh ? 0u : 1u);
        if (WIDE) tc_mma_f16(dj + 256u, ak, bk_ + b_wide_off, idesc2, fresh ? 0u : 1u);
      } else {
        tc_mma_f16_acc(dj, ak, bk_, idesc);
        if (WIDE) tc_mma_f16_acc(dj + 256u, ak, bk_ + b_wide_off, idesc2);
      }
    }
  }
}

// What the issuing thread needs for the k-blocks of one work item, fixed for the launch.
struct IssueCtx {
  uint32_t ring_u32, tiles_u32, stage_bytes, b_bytes, b_in_stage;   // b_in_stage: offset of B inside a stage
  uint32_t acc_stride, a_adv, b_adv, idesc, idesc2;
  uint64_t a_desc0, b_desc0, a_sub, b_wide_off;
  int stages, b_resident;
};

// k-blocks [kb0, kb1) of one work item; returns false after a wait that ran out.
template <int KK, int MT, bool WIDE, bool PAIR>
__device__ __forceinline__ bool issue_item(const IssueCtx& c, SharedCtl* ctl, unsigned int* status, uint32_t d_tmem,
                                           int kb0, int kb1, int& s, uint32_t& ph) {
  for (int kb = kb0; kb < kb1; ++kb) {
    if (!ctl_wait_role(ctl, &ctl->full[s], ph, status, 2)) return false;
    tc_fence_after();
    const uint32_t sa = c.ring_u32 + (uint32_t)s * c.stage_bytes;
    const uint32_t sb = c.b_resident ? c.tiles_u32 + (uint32_t)kb * c.b_bytes : sa + c.b_in_stage;
    // descriptors differ from the templates only in the 14-bit start address (no carry out of it: shared memory
    // ends below 256 KB)
    const uint64_t da = c.a_desc0 | (uint64_t)((sa >> 4) & 0x3FFFu);
    const uint64_t db = c.b_desc0 | (uint64_t)((sb >> 4) & 0x3FFFu);
    issue_kblock<KK, MT, WIDE, PAIR>(d_tmem, c.acc_stride, da, c.a_sub, db, c.a_adv, c.b_adv, c.idesc, c.idesc2,
                                     c.b_wide_off, kb == kb0);
    // stage is free once these MMAs have read it (in both CTAs of a pair)
    if (PAIR) tc_commit2_both(&ctl->empty[s]);
    else tc_commit(&ctl->empty[s]);
    if (++s == c.stages) { s = 0; ph ^= 1u; }
  }
  return true;
}

// PAIR: the instantiation that runs as clusters of two CTAs (p.pair != 0). It is a kernel of its own because a
// kernel that contains cta_group::2 instructions can only be launched with an even cluster size.
template <bool PAIR>
__global__ void __maxnreg__(GEMM_MAX_REGS) gemm_tc_kernel(const __grid_constant__ GemmTcParams p) {
#ifdef RB_GEMM_PROFILE
  const long long t_kernel0 = clock64();
#endif
  extern __shared__ uint8_t smem_raw[];
  // tiles start on a 1024-byte boundary (swizzle atoms); control block follows the tiles
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + TILE_SMEM_BYTES;
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(staging + STAGING_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // CTA pairs: rank of this CTA in its pair, and the persistent loop runs over pairs
  constexpr bool pair = PAIR;
  const uint32_t cta_rank = pair ? cluster_ctarank() : 0u;
  const int cta_id = pair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int cta_step = pair ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  const int mt = p.mt;
  const int a_bytes = BM * p.bk * 2;            // one 128-row sub-tile
  const int b_bytes = p.bn_load * p.bk * 2;
  const int panel_bytes = p.b_resident ? p.num_kb * b_bytes : 0;
  const int stage_bytes = mt * a_bytes + (p.b_resident ? 0 : b_bytes);
  uint8_t* ring = tiles + panel_bytes;
  const int stages = p.stages;

  const bool halo = p.a_mode == A_HALO_K;
  const bool box = p.a_mode == A_BOX_K;
  const int bx_groups = box ? (p.cv_P + mt * p.bx_rows - 1) / (mt * p.bx_rows) : 1;   // work items per image
  const int m_units = halo  ? (p.M / (p.cv_P * p.cv_Q)) * p.hl_groups
                      : box ? (p.M / (p.cv_P * p.cv_Q)) * bx_groups
                            : (p.M + BM * mt - 1) / (BM * mt);
  const int m_items = pair ? (m_units + 1) >> 1 : m_units;   // a pair's item is two CTA-sized units
  const int n_tiles = p.n_tiles;
  // whole items first, then the parts of the cut items of the last wave (tail cut; never in halo mode)
  const int direct = m_items * n_tiles - p.tail_items;
  const int num_work = p.tail_items > 0 ? direct + p.tail_items * p.tail_split : m_items * n_tiles * p.split_k;
  // halo mode: [A ring: hl_a_stages x hl_a_bytes][B ring: stages x b_bytes]
  uint8_t* a_ring = tiles;
  uint8_t* b_ring = tiles + p.hl_a_stages * p.hl_a_bytes;
  const int kb_per_split = (p.num_kb + p.split_k - 1) / p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      // one arrival per producer warp that fills it (a pair: both CTAs' producers arrive on the leader's barrier)
      mbar_init(&ctl->full[s], pair ? 4 : ((halo || p.b_resident) ? 1 : 2));
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], pair ? 2 * EPI_WARPS : EPI_WARPS);
    }
    mbar_init(&ctl->b_full, 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->a_full[a], 1);
      mbar_init(&ctl->a_empty[a], 1);
    }
    for (int w = 0; w < EPI_WARPS; ++w) mbar_init(&ctl->mask_bar[w], 1);
    ctl->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_a);
    tma_prefetch_desc(&p.tm_b);
    tma_prefetch_desc(&p.tm_d);
    if (p.epi == EPI_BF16 && p.mask_src) tma_prefetch_desc(&p.tm_mask);
    if (p.tail_items > 0) tma_prefetch_desc(&p.tm_ws);
  }
  if (warp == 1) {
    if (pair) {
      tmem_alloc2(&ctl->tmem_base, 512);   // both CTAs of the pair execute this; each gets the same address
      tmem_relinquish2();
    } else {
      tmem_alloc(&ctl->tmem_base, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (pair) cluster_sync_all();   // the peer's barriers are initialised before anything of ours signals them
  tc_fence_after();
  // Programmatic dependent launch (option `pdl`): everything above touched only this CTA's own shared memory, TMEM
  // and the launch parameters, so it may run while the kernels before this one on the stream are still finishing;
  // nothing below (operands, bias, mask, output, workspace) is touched before they have completed and flushed.
  // Without the launch attribute both instructions do nothing.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0 || warp == PRODUCER_B_WARP) {
    // ------------------------------ producers ------------------------------
    // A single thread gets one TMA instruction through every ~220 ns whatever the size of its box, and further
    // boxes it has in flight do not overlap with it (measured); boxes issued by other threads do. So the loads of
    // a stage are spread: warp 0 issues the A loads (one lane per box, all lanes of a mode execute the same
    // instruction), warp PRODUCER_B_WARP the B loads, and both arrive on the stage's `full` barrier with the
    // bytes they bring.
    const bool is_a = warp == 0;
    int s = 0, issued = 0;
    uint32_t ph = 0;
    bool ok = true;
    if (halo) {
      const uint32_t a_tx = (uint32_t)(p.hl_rtot * p.hl_pitch * p.bk * 2);
      const int nst = is_a ? p.hl_a_stages : stages;
      uint64_t* fullb = is_a ? ctl->a_full : ctl->full;
      uint64_t* emptyb = is_a ? ctl->a_empty : ctl->empty;
      if (lane == 0) {
        for (int work = cta_id; work < num_work && ok; work += cta_step) {
          const int tn = work / m_items;
          const int tm = work - tn * m_items;
          const int n_img = tm / p.hl_groups;
          const int p0 = (tm - n_img * p.hl_groups) * mt * p.hl_rows;
          const int n0 = tn * p.bn;
          for (int sx = 0; sx < p.cv_S && ok; ++sx) {
            for (int cc = 0; cc < p.cv_cchunks && ok; ++cc) {
              if (is_a) {
                if (!ctl_wait(ctl, &emptyb[s], ph ^ 1u, p.status)) { ok = false; break; }
                mbar_expect_tx(&fullb[s], a_tx);
                tma_load_4d(a_ring + s * p.hl_a_bytes, &p.tm_a, &fullb[s], cc * p.bk, sx - p.hl_pad_w,
                            p0 - p.hl_pad_h, n_img);
                ++issued;
                if (++s == nst) { s = 0; ph ^= 1u; }
              } else {
                for (int r = 0; r < p.hl_R; ++r) {
                  if (!ctl_wait(ctl, &emptyb[s], ph ^ 1u, p.status)) { ok = false; break; }
                  mbar_expect_tx(&fullb[s], (uint32_t)b_bytes);
                  tma_load_3d(b_ring + s * b_bytes, &p.tm_b, &fullb[s], cc * p.bk, r * p.cv_S + sx, n0);
                  ++issued;
                  if (++s == nst) { s = 0; ph ^= 1u; }
                }
              }
            }
          }
        }
        if (!ok) {
          // drain: wait (bounded) until the copies already issued have landed
          const int back = min(issued, nst);
          for (int i = 0; i < back; ++i) {
            if (s == 0) { s = nst; ph ^= 1u; }
            --s;
            mbar_wait_bounded(&fullb[s], ph, 100000000ull);
          }
        }
      }
    } else if (is_a || !p.b_resident) {
      // loads this warp issues per stage, one lane each
      int nload;
      const int a_split = p.a_split > 0 ? p.a_split : 1, b_split = p.b_split > 0 ? p.b_split : 1;
      if (is_a) nload = box ? mt : (p.a_mode == A_TILED_MN ? 2 : a_split) * mt;
      else if (p.b_mode == B_TILED_MN) nload = p.bn_load / 64;
      else if (p.b_mode == B_IM2COL_MN) nload = p.wg_taps > 1 ? p.wg_taps * (p.wg_cw / 64) : p.bn_load / 64;
      else nload = b_split;
      // a pair counts every load on the leader's `full` barriers
      const uint32_t full0_leader = pair ? mapa_shared(smem_u32(&ctl->full[0]), 0u) : 0u;
      const uint32_t my_tx = !is_a ? (uint32_t)b_bytes
                             : box ? (uint32_t)(mt * p.bx_rows * p.cv_Q * p.bk * 2)   // the boxes bring whole rows only
                                   : (uint32_t)(mt * a_bytes);
      for (int work = cta_id; work < num_work && ok; work += cta_step) {
        const WorkItem it = decode_work(p, work, m_items, direct, kb_per_split);
        const int tn = it.tn, kb0 = it.kb0, kb1 = it.kb1;
        const int tm = pair ? it.tm * 2 + (int)cta_rank : it.tm;
        const int m0 = tm * BM * mt;
        // geometry that is fixed for the work item (every lane keeps what its own load needs)
        // sub-tile of this lane's A load, and which of the sub-tile's boxes it is
        const int aj = (p.a_mode == A_TILED_MN) ? (lane >> 1) : lane / a_split;
        const int aq = (p.a_mode == A_TILED_MN) ? 0 : lane - aj * a_split;
        const int a_rows = BM / a_split;
        int a_w = 0, a_h = 0, a_n = 0;
        if (is_a && p.a_mode == A_IM2COL_K && lane < nload) pixel_coords(p, m0 + aj * BM + aq * a_rows, a_w, a_h, a_n);
        if (is_a && box) {   // lane j loads sub-tile j: image a_n, first output row a_h
          a_n = tm / bx_groups;
          a_h = ((tm - a_n * bx_groups) * mt + lane) * p.bx_rows;
        }
        int b_tap = 0, b_c0 = 0;
        const int n0 = tn * p.bn + (pair ? (int)cta_rank * p.bn_load : 0);   // a pair's CTA loads its half of the rows
        if (p.b_mode == B_IM2COL_MN) {
          if (p.wg_taps > 1) {
            b_tap = tn * p.wg_taps;
          } else {
            b_tap = tn / p.wg_ctiles;
            b_c0 = (tn - b_tap * p.wg_ctiles) * p.bn;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          int w_ok = 1;
          if (lane == 0) {
            w_ok = ctl_wait_role(ctl, &ctl->empty[s], ph ^ 1u, p.status, is_a ? 0 : 1) ? 1 : 0;
            if (w_ok) {
              if (pair) mbar_expect_tx_cluster(full0_leader + (uint32_t)s * 8u, my_tx);
              else mbar_expect_tx(&ctl->full[s], my_tx);
            }
          }
          w_ok = __shfl_sync(0xffffffffu, w_ok, 0);
          if (!w_ok) { ok = false; break; }
          uint8_t* sa = ring + s * stage_bytes;
          uint8_t* sb = sa + mt * a_bytes;
          uint64_t* bar = &ctl->full[s];
          if (pair) {
            // K-major operands only; the bytes are counted on the leader's barrier of this stage
            const uint32_t bar2 = full0_leader + (uint32_t)s * 8u;
            if (lane < nload) {
              const int tap = p.cv_cchunks > 0 ? kb / p.cv_cchunks : 0;   // filter tap (convolution operands)
              if (is_a) {
                uint8_t* saj = sa + aj * a_bytes + aq * a_rows * p.bk * 2;
                if (p.a_mode == A_TILED_K) {
                  tma2_load_2d(saj, &p.tm_a, bar2, kb * p.bk, m0 + aj * BM + aq * a_rows);
                } else {   // A_IM2COL_K
                  const int cc = kb - tap * p.cv_cchunks;
                  const int r = tap / p.cv_S;
                  const int sx = tap - r * p.cv_S;
                  tma2_load_im2col_4d(saj, &p.tm_a, bar2, cc * p.bk, a_w, a_h, a_n, (uint16_t)sx, (uint16_t)r);
                }
              } else {
                const int b_rows = p.bn_load / b_split;
                uint8_t* sbq = sb + lane * b_rows * p.bk * 2;
                if (p.b_mode == B_TILED_K) tma2_load_2d(sbq, &p.tm_b, bar2, kb * p.bk, n0 + lane * b_rows);
                else tma2_load_3d(sbq, &p.tm_b, bar2, (kb - tap * p.cv_cchunks) * p.bk, tap, n0 + lane * b_rows);
              }
            }
          } else if (lane < nload) {
            if (is_a) {
              uint8_t* saj = sa + aj * a_bytes + aq * a_rows * p.bk * 2;
              const int mj = m0 + aj * BM + aq * a_rows;
              if (p.a_mode == A_TILED_K) {
                tma_load_2d(saj, &p.tm_a, bar, kb * p.bk, mj);
              } else if (box) {
                const int tap = kb / p.cv_cchunks;
                const int cc = kb - tap * p.cv_cchunks;
                const int r = tap / p.cv_S;
                const int sx = tap - r * p.cv_S;
                tma_load_4d(sa + lane * a_bytes, &p.tm_a, bar, cc * p.bk, sx - p.bx_pad_w, a_h + r - p.bx_pad_h, a_n);
              } else if (p.a_mode == A_IM2COL_K) {
                const int tap = kb / p.cv_cchunks;
                const int cc = kb - tap * p.cv_cchunks;
                const int r = tap / p.cv_S;
                const int sx = tap - r * p.cv_S;
                tma_load_im2col_4d(saj, &p.tm_a, bar, cc * p.bk, a_w, a_h, a_n, (uint16_t)sx, (uint16_t)r);
              } else {  // A_TILED_MN: two boxes of 64 rows(M) x bk per sub-tile
                const int half = lane & 1;
                tma_load_2d(saj + half * p.bk * 128, &p.tm_a, bar, mj + 64 * half, kb * p.bk);
              }
            } else if (p.b_mode == B_TILED_K) {
              const int b_rows = p.bn_load / b_split;
              tma_load_2d(sb + lane * b_rows * p.bk * 2, &p.tm_b, bar, kb * p.bk, n0 + lane * b_rows);
            } else if (p.b_mode == B_TILED_K3) {
              const int tap = kb / p.cv_cchunks;
              const int cc = kb - tap * p.cv_cchunks;
              const int b_rows = p.bn_load / b_split;
              tma_load_3d(sb + lane * b_rows * p.bk * 2, &p.tm_b, bar, cc * p.bk, tap, n0 + lane * b_rows);
            } else if (p.b_mode == B_TILED_MN) {
              tma_load_2d(sb + lane * p.bk * 128, &p.tm_b, bar, n0 + 64 * lane, kb * p.bk);
            } else {  // B_IM2COL_MN
              int w, h, n_img;
              pixel_coords(p, kb * p.bk, w, h, n_img);
              if (p.wg_taps > 1) {
                // several filter taps side by side in one column tile: they share the A (dY) stage
                const int apt = p.wg_cw / 64;  // 64-column atoms per tap
                const int t = lane / apt, j = lane - t * apt;
                const int tap = min(b_tap + t, p.wg_ntaps - 1);   // slots past the last tap reload it; the epilogue skips them
                const int r = tap / p.cv_S;
                const int sx = tap - r * p.cv_S;
                tma_load_im2col_4d(sb + lane * p.bk * 128, &p.tm_b, bar, 64 * j, w, h, n_img, (uint16_t)sx, (uint16_t)r);
              } else {
                const int r = b_tap / p.cv_S;
                const int sx = b_tap - r * p.cv_S;
                tma_load_im2col_4d(sb + lane * p.bk * 128, &p.tm_b, bar, b_c0 + 64 * lane, w, h, n_img, (uint16_t)sx,
                                   (uint16_t)r);
              }
            }
          }
          __syncwarp();
          ++issued;
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok && lane == 0 && pair && cta_rank != 0) {
        // this CTA's copies complete on the leader's barriers, which cannot be waited on from here: give them time
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      } else if (!ok && lane == 0) {
        // drain: wait (bounded) until the copies already issued have landed
        const int back = min(issued, stages);
        for (int i = 0; i < back; ++i) {
          if (s == 0) { s = stages; ph ^= 1u; }
          --s;
          mbar_wait_bounded(&ctl->full[s], ph, 100000000ull);
        }
      }
    } else {
      // resident B: this warp loads the one panel the CTA will ever need, k-blocks spread over its lanes
      if (blockIdx.x < num_work) {
        if (lane == 0) mbar_expect_tx(&ctl->b_full, (uint32_t)panel_bytes);
        __syncwarp();
        for (int kb = lane; kb < p.num_kb; kb += 32) load_b(p, tiles + kb * b_bytes, &ctl->b_full, kb, 0, 0, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && cta_rank == 0) {   // of a pair, only the leader issues
      const bool a_mn = (p.a_mode == A_TILED_MN);
      const bool b_mn = (p.b_mode == B_TILED_MN || p.b_mode == B_IM2COL_MN);
      // a tile wider than 256 columns is two MMAs side by side (256 + the rest) that share the A descriptor
      const uint32_t idesc = make_idesc_bf16(pair ? 2 * BM : BM, (uint32_t)min(p.bn, 256), a_mn ? 1u : 0u, b_mn ? 1u : 0u);
      const uint32_t idesc2 = p.bn > 256 ? make_idesc_bf16(BM, (uint32_t)(p.bn - 256), a_mn ? 1u : 0u, b_mn ? 1u : 0u) : 0u;
      const uint64_t b_wide_off = (uint64_t)((256u * (uint32_t)p.bk * 2u) >> 4);   // K-major B: 256 rows further down
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
      const uint32_t set_cols = (uint32_t)(mt * p.acc_stride);

      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      if (p.b_resident && blockIdx.x < num_work) ok = ctl_wait(ctl, &ctl->b_full, 0u, p.status);
      if (halo) {
        int bs = 0, as = 0;
        uint32_t bph = 0, aph = 0;
        const uint32_t row_bytes = (uint32_t)p.bk * 2u;
        for (int work = cta_id; work < num_work && ok; work += cta_step) {
          if (!ctl_wait(ctl, &ctl->acc_empty[acc], acc_ph ^ 1u, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)acc * set_cols;
          bool fresh = true;   // the first MMA into each accumulator overwrites it
          for (int sx = 0; sx < p.cv_S && ok; ++sx) {
            for (int cc = 0; cc < p.cv_cchunks && ok; ++cc) {
              if (!ctl_wait(ctl, &ctl->a_full[as], aph, p.status)) { ok = false; break; }
              tc_fence_after();
              const uint32_t a_base = smem_u32(a_ring + as * p.hl_a_bytes);
              for (int r = 0; r < p.hl_R; ++r) {
                if (!ctl_wait(ctl, &ctl->full[bs], bph, p.status)) { ok = false; break; }
                tc_fence_after();
                const uint64_t db = make_smem_desc(smem_u32(b_ring + bs * b_bytes), b_lbo, b_sbo, b_lay);
                for (int j = 0; j < mt; ++j) {
                  // filter row r of sub-tile j: the same tile, (j * hl_rows + r) * hl_pitch rows further down
                  const uint32_t off = (uint32_t)((j * p.hl_rows + r) * p.hl_pitch) * row_bytes;
                  const uint64_t da = make_smem_desc(a_base + off, a_lbo, a_sbo, a_lay);
                  for (int kk = 0; kk < kk_steps; ++kk) {
                    tc_mma_f16(d_tmem + (uint32_t)(j * p.acc_stride), da + (uint64_t)(a_adv * kk),
                               db + (uint64_t)(b_adv * kk), idesc, (!fresh || kk > 0) ? 1u : 0u);
                  }
                }
                fresh = false;
                tc_commit(&ctl->empty[bs]);
                if (++bs == stages) { bs = 0; bph ^= 1u; }
              }
              if (!ok) break;
              tc_commit(&ctl->a_empty[as]);   // every MMA that reads this A tile has been issued before this point
              if (++as == p.hl_a_stages) { as = 0; aph ^= 1u; }
            }
          }
          if (!ok) break;
          tc_commit(&ctl->acc_full[acc]);
          if (++acc == p.acc_bufs) { acc = 0; acc_ph ^= 1u; }
        }
      }
      // what the unrolled issue code needs, fixed for the launch
      IssueCtx ic;
      ic.ring_u32 = smem_u32(ring);
      ic.tiles_u32 = smem_u32(tiles);
      ic.stage_bytes = (uint32_t)stage_bytes;
      ic.b_bytes = (uint32_t)b_bytes;
      ic.b_in_stage = (uint32_t)(mt * a_bytes);
      ic.acc_stride = (uint32_t)p.acc_stride;
      ic.a_adv = a_adv;
      ic.b_adv = b_adv;
      ic.idesc = idesc;
      ic.idesc2 = idesc2;
      ic.a_desc0 = make_smem_desc(0u, a_lbo, a_sbo, a_lay);
      ic.b_desc0 = make_smem_desc(0u, b_lbo, b_sbo, b_lay);
      ic.a_sub = (uint64_t)((uint32_t)a_bytes >> 4);     // next 128-row sub-tile of the stage
      ic.b_wide_off = b_wide_off;
      ic.stages = stages;
      ic.b_resident = p.b_resident;
      const int issue_kind = (kk_steps == 4 ? 0 : 3) + (idesc2 ? 2 : (mt == 2 ? 1 : 0));
      for (int work = cta_id; work < num_work && ok && !halo; work += cta_step) {
        const WorkItem it = decode_work(p, work, m_items, direct, kb_per_split);
        if (!ctl_wait_role(ctl, &ctl->acc_empty[acc], acc_ph ^ 1u, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * set_cols;
        switch (issue_kind) {
          case 0: ok = issue_item<4, 1, false, PAIR>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph); break;
          case 1: ok = issue_item<4, 2, false, PAIR>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph); break;
          case 3: ok = issue_item<2, 1, false, PAIR>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph); break;
          case 4: ok = issue_item<2, 2, false, PAIR>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph); break;
          default:   // one tile wider than 256 columns: never for pairs (refused on the host)
            if (PAIR) ok = false;
            else if (issue_kind == 2) ok = issue_item<4, 1, true, false>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph);
            else ok = issue_item<2, 1, true, false>(ic, ctl, p.status, d_tmem, it.kb0, it.kb1, s, ph);
            break;
        }
        if (!ok) break;
        if (pair) tc_commit2_both(&ctl->acc_full[acc]);
        else tc_commit(&ctl->acc_full[acc]);
        if (++acc == p.acc_bufs) { acc = 0; acc_ph ^= 1u; }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------ epilogue ------------------------------
    const int lane_base = (warp & 3) * 32;  // TMEM lanes this warp may read
    const uint32_t set_cols = (uint32_t)(mt * p.acc_stride);
    const int col_half = (warp - 2) >> 2;        // which of the two warps of this lane quarter
    uint8_t* stg = staging + (warp - 2) * 4096;  // one 32-row x 128-byte slab buffer per warp
    const bool has_bias = p.bias != nullptr;
    uint64_t* mbar_m = &ctl->mask_bar[warp - 2];
    uint32_t mask_ph = 0;
    const float act_lo = p.relu ? 0.f : -INFINITY;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int work = cta_id; work < num_work && ok; work += cta_step) {
      const WorkItem it = decode_work(p, work, m_items, direct, kb_per_split);
      const int tn = it.tn;
      const int tm = pair ? it.tm * 2 + (int)cta_rank : it.tm;
      const bool tail = it.tail >= 0;
      {
        RB_PROF_T0(warp == 2);
        if (!ctl_wait(ctl, &ctl->acc_full[acc], acc_ph, p.status)) { ok = false; break; }
        RB_PROF_ADD(warp == 2, 5);
      }
      tc_fence_after();
      int col0;        // first column of D this tile writes
      int col_limit;   // tile-local bound on stored columns
      if (p.b_mode == B_IM2COL_MN && p.wg_taps > 1) {
        col0 = 0;            // columns are mapped per 32-column chunk below
        col_limit = p.bn;
      } else if (p.b_mode == B_IM2COL_MN) {
        const int tap = tn / p.wg_ctiles;
        const int c0 = (tn - tap * p.wg_ctiles) * p.bn;
        col0 = tap * p.wg_cpad + c0;
        col_limit = min(p.bn, p.wg_cpad - c0);
      } else {
        col0 = tn * p.bn;
        col_limit = min(p.bn, p.n_store - col0);
      }
      for (int j = 0; j < mt; ++j) {
        // halo mode: this warp's 32-row band is (32 / pitch) output rows of one image, or a 32-wide piece of one
        int h_n = 0, h_p = 0, h_w = 0;
        if (halo) {
          h_n = tm / p.hl_groups;
          h_p = ((tm - h_n * p.hl_groups) * mt + j) * p.hl_rows + lane_base / p.hl_pitch;
          h_w = lane_base % p.hl_pitch;
          if (h_p >= p.cv_P || h_w >= p.cv_Q) continue;   // the whole band lies outside the image
        }
        int row0 = tm * BM * mt + j * BM + lane_base;   // first row of this warp's 32-row band
        int band_rows = 32;                             // rows of the band that belong to this tile
        if (box) {
          // the sub-tile is bx_rows whole output rows of one image: consecutive rows of D, fewer at the image's
          // lower edge; tile rows past them are computed from stale shared memory and dropped here
          const int b_n = tm / bx_groups;
          const int b_p = ((tm - b_n * bx_groups) * mt + j) * p.bx_rows;
          const int valid = max(0, min(p.bx_rows, p.cv_P - b_p)) * p.cv_Q;
          band_rows = max(0, min(32, valid - lane_base));
          row0 = (b_n * p.cv_P + b_p) * p.cv_Q + lane_base;
          if (band_rows == 0 && !tail) continue;
        }
        const uint32_t t_addr =
            tmem_base + (uint32_t)acc * set_cols + (uint32_t)(j * p.acc_stride) + ((uint32_t)lane_base << 16);
        if (p.epi == EPI_BF16 && !tail) {
          // 64-column slabs: TMEM -> registers -> bias / ReLU / mask -> swizzled shared memory -> TMA store.
          // Each warp owns a 4 KB slab buffer and issues its own stores, so no cross-warp sync is needed.
          // the two warps of a lane quarter alternate slabs, starting with the other warp on the second sub-tile, so
          // that a tile with an odd number of slabs (96 columns = a full and a half slab) splits evenly between them
          for (int c = ((col_half + j) & 1) * 64; c < p.bn && col0 + c < p.n_store; c += 128) {
            uint8_t* buf = stg;
            if (lane == 0) tma_store_wait_read<0>();   // the store that last used this buffer has read it
            __syncwarp();
            const int gcol = col0 + c;
            uint4 mreg[8];
            if (p.mask_src) {
              // the mask slab arrives through TMA into the slab buffer (same box and swizzle as the output),
              // is copied to registers, and the buffer is then reused for the output
              if (lane == 0) {
                mbar_expect_tx(mbar_m, 4096u);
                if (halo) tma_load_4d(buf, &p.tm_mask, mbar_m, gcol, h_w, h_p, h_n);
                else tma_load_2d(buf, &p.tm_mask, mbar_m, gcol, row0);
              }
              if (!mbar_wait_bounded(mbar_m, mask_ph, WAIT_LIMIT_NS)) {
                ctl->abort_flag = 1;
                if (p.status) atomicOr(p.status, RB_STATUS_MBAR_TIMEOUT);
              }
              mask_ph ^= 1u;
#pragma unroll
              for (int ch = 0; ch < 8; ++ch)
                mreg[ch] = *reinterpret_cast<const uint4*>(buf + lane * 128 + ((ch ^ (lane & 7)) * 16));
              __syncwarp();
            }
            RB_PROF_T0(warp == 2);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t v[32];
              const int nbase = gcol + half * 32;
              if (nbase >= p.n_store) continue;            // these columns do not exist in D: the store clips them
              const bool fast = nbase + 32 <= p.n_valid;   // no padded column in this 32-column group
              tmem_ld_32x32(t_addr + (uint32_t)(c + half * 32), v);
              tmem_ld_wait();
              const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
                const uint4 mv = p.mask_src ? mreg[half * 4 + q] : make_uint4(0u, 0u, 0u, 0u);
                const __nv_bfloat162* m2 = reinterpret_cast<const __nv_bfloat162*>(&mv);
                if (fast) {
                  // Two epilogue warps share a scheduler, so this is bound by instruction count and dependent-issue
                  // latency: packed fp32 adds for the bias, one conversion per pair, ReLU and the mask of the
                  // previous layer's ReLU on the packed bf16 pair (rounding is monotone, so clamping after it gives
                  // the same bits as clamping before).
                  // (the bias is fetched eight columns at a time: holding all 32 columns' worth in registers put the
                  // kernel over its register budget)
                  float4 bq[2];
                  if (has_bias) {
                    bq[0] = __ldg(reinterpret_cast<const float4*>(p.bias + nbase + q * 8));
                    bq[1] = __ldg(reinterpret_cast<const float4*>(p.bias + nbase + q * 8 + 4));
                  }
                  const float* bb = reinterpret_cast<const float*>(&bq[0]);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float x0 = __uint_as_float(v[q * 8 + 2 * e]), x1 = __uint_as_float(v[q * 8 + 2 * e + 1]);
                    if (has_bias) add2_f32(v[q * 8 + 2 * e], v[q * 8 + 2 * e + 1], bb[2 * e], bb[2 * e + 1], x0, x1);
                    __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
                    if (p.relu) h = __hmax2(h, zero2);
                    uint32_t w = *reinterpret_cast<uint32_t*>(&h);
                    if (p.mask_src) w &= __hgt2_mask(m2[e], zero2);
                    ow[e] = w;
                  }
                } else {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const int n = nbase + q * 8 + e;
                    float x = 0.f;
                    if (n < p.n_valid) x = fmaxf(__uint_as_float(v[q * 8 + e]) + (has_bias ? __ldg(p.bias + n) : 0.f), act_lo);
                    f[e] = x;
                  }
                  if (p.mask_src) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 mf = __bfloat1622float2(m2[e]);
                      if (!(mf.x > 0.f)) f[2 * e] = 0.f;
                      if (!(mf.y > 0.f)) f[2 * e + 1] = 0.f;
                    }
                  }
                  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                }
                // 128-byte swizzle: 16-byte chunk index XOR (row mod 8), the layout the store's tensor map expects
                const int chunk = (half * 4 + q) ^ (lane & 7);
                *reinterpret_cast<uint4*>(buf + lane * 128 + chunk * 16) = o;
              }
            }
            RB_PROF_ADD(warp == 2, 7);
#ifdef RB_GEMM_PROFILE
            const long long prof_t1_ = clock64();
#endif
            fence_proxy_async_smem();
            __syncwarp();
            if (band_rows < 32) {
              // ragged band (box mode): the rows after the tile's last belong to other tiles, so the valid rows are
              // copied out by hand, 16 bytes at a time, instead of a 32-row TMA store
              if (lane < band_rows) {
                bf16* drow = reinterpret_cast<bf16*>(p.D) + (long long)(row0 + lane) * p.ldd + gcol;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)
                  if (gcol + ch * 8 < p.n_store)
                    *reinterpret_cast<uint4*>(drow + ch * 8) =
                        *reinterpret_cast<const uint4*>(buf + lane * 128 + ((ch ^ (lane & 7)) * 16));
              }
              __syncwarp();
            } else if (lane == 0 && (halo || row0 < p.M)) {
              if (halo) tma_store_4d(&p.tm_d, buf, gcol, h_w, h_p, h_n);
              else tma_store_2d(&p.tm_d, buf, gcol, row0);
              tma_store_commit();
            }
#ifdef RB_GEMM_PROFILE
            if (warp == 2 && blockIdx.x == 3 && lane == 0)
              atomicAdd(&g_role_cycles[6], (unsigned long long)(clock64() - prof_t1_));
#endif
          }
          continue;
        }
        for (int c = ((col_half + j) & 1) * 32; c < p.bn; c += 64) {
          uint32_t v[32];
          tmem_ld_32x32(t_addr + (uint32_t)c, v);
          tmem_ld_wait();
          if (!tail && c >= col_limit) continue;
          int gcol = tail ? c : col0 + c;
          if (!tail && p.b_mode == B_IM2COL_MN && p.wg_taps > 1) {
            const int t = c / p.wg_cw, cc = c - t * p.wg_cw;
            const int tap = tn * p.wg_taps + t;
            if (tap >= p.wg_ntaps || cc >= p.wg_cpad) continue;
            gcol = tap * p.wg_cpad + cc;
          }
          // fp32 output: 32-column chunk -> swizzled slab buffer -> one TMA store (overwrite) or TMA reduce-add
          // (accumulate / split-K) per warp, instead of eight 16-byte red instructions per thread
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint4 o = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((q ^ (lane & 7)) * 16)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && (tail || row0 < p.M)) {
            // a part of a cut item adds into its rows of the workspace; everything else goes to D
            if (tail) tma_reduce_add_2d(&p.tm_ws, stg, gcol, (it.tail * mt + j) * BM + lane_base);
            else if (p.epi == EPI_F32_STORE) tma_store_2d(&p.tm_d, stg, gcol, row0);
            else tma_reduce_add_2d(&p.tm_d, stg, gcol, row0);
            tma_store_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        // the accumulators of both CTAs of a pair are refilled by the leader: it waits for both epilogues
        if (pair) mbar_arrive_cluster(mapa_shared(smem_u32(&ctl->acc_empty[acc]), 0u));
        else mbar_arrive(&ctl->acc_empty[acc]);
      }
      if (++acc == p.acc_bufs) { acc = 0; acc_ph ^= 1u; }
    }
    if (lane == 0) tma_store_wait_all<0>();   // every output store has completed before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
#ifdef RB_GEMM_PROFILE
  if (blockIdx.x == 3 && threadIdx.x == 0) atomicAdd(&g_role_cycles[4], (unsigned long long)(clock64() - t_kernel0));
#endif
  // a pair frees its TMEM together, after both epilogues have read it and nothing signals a peer's barrier any more
  if (pair) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if (pair) tmem_dealloc2(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
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
static int g_pair_clusters = 0;   // clusters of two CTAs of the kernel that the device runs at once (0 = none)

static void options_from_env();

static int ensure_driver_entry() {
  options_from_env();
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
  if (cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) !=
          cudaSuccess ||
      cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) !=
          cudaSuccess)
    return -2;
  {   // how many CTA pairs fit at once: the persistent loop of pair mode runs exactly that many clusters
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(g_num_sms / 2 * 2));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int nc = 0;
    if (cudaOccupancyMaxActiveClusters(&nc, gemm_tc_kernel<true>, &cfg) != cudaSuccess) nc = 0;
    cudaGetLastError();   // a refused query must not be taken for a failed launch later
    g_pair_clusters = nc > g_num_sms / 2 ? g_num_sms / 2 : nc;
  }
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

// Output map of the bf16 epilogue: columns [0, n_store) x rows [0, M), 64 x 32 boxes, 128-byte swizzle.
static int make_map_out(CUtensorMap* m, void* D, int n_store, int M, long long ldd) {
  return make_map_2d(m, D, (uint64_t)n_store, (uint64_t)M, (uint64_t)ldd, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
}

// fp32 output map: 32-column x 32-row boxes (128-byte rows), 128-byte swizzle; used by TMA store / reduce-add.
static int make_map_out_f32(CUtensorMap* m, void* D, long long n_cols, int M, long long ldd) {
  cuuint64_t dims[2] = {(cuuint64_t)n_cols, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)ldd * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t es[2] = {1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, D, dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(300 + (int)r);
}

// 4-D bf16 tiled map over an NHWC tensor: dims {C, W, H, N}, pixel pitch `ld` elements, box {bc, bw, bh, 1}.
static int make_map_nhwc(CUtensorMap* m, const void* ptr, uint64_t C, uint64_t W, uint64_t H, uint64_t N, uint64_t ld,
                         uint32_t bc, uint32_t bw, uint32_t bh, CUtensorMapSwizzle sw) {
  cuuint64_t dims[4] = {C, W, H, N};
  cuuint64_t strides[3] = {ld * 2, ld * W * 2, ld * W * H * 2};
  cuuint32_t box[4] = {bc, bw, bh, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(400 + (int)r);
}

// ---- options ----------------------------------------------------------------------------------------------------
// Switches of the planner. Their initial values come from the environment (RB_GEMM_*), read once when the library
// is first used; afterwards they change only through rb_gemm_set_option (tests, experiments).
struct GemmOptions {
  int force_mt = 0;          // RB_GEMM_FORCE_MT: 1 | 2 sub-tiles per item (0 = planner's choice)
  int force_resident = -1;   // RB_GEMM_FORCE_RESIDENT: 0 | 1
  int force_halo = -1;       // RB_GEMM_FORCE_HALO: 0 = never, 1 = whenever feasible
  int force_taps = 0;        // RB_GEMM_FORCE_TAPS: filter taps per weight-grad tile
  int force_tail = -1;       // RB_GEMM_FORCE_TAIL: 0 = never cut the last wave, 1 = whenever feasible
  int force_wide = -1;       // RB_GEMM_FORCE_WIDE: 0 = tiles of at most 256 columns, 1 = one wide tile when N <= 512
  int force_box = -1;        // RB_GEMM_FORCE_BOX: 0 = never load A as tap-shifted boxes, 1 = whenever feasible
  int force_pair = -1;       // RB_GEMM_FORCE_PAIR: 0 = never run as CTA pairs (cta_group::2), 1 = whenever feasible
  int pdl = 2;               // RB_GEMM_PDL: programmatic stream serialization (blocks become resident while the kernel
                             // before them finishes; see launch.cuh): 0 = off, 1 = this kernel only, 2 = every kernel
                             // of a step. Beside exchange kernels on other streams use at most 1: the waiting blocks
                             // of elementwise kernels fill the SMs' thread slots and the exchange kernels starve.
  int bk32 = 0;              // RB_GEMM_BK32: keep 32-channel chunks for channel counts such as 96
  int bn_cap = 256;          // RB_GEMM_BN_CAP: upper bound on the tile width chosen by the planner
  int a_split = 1;           // RB_GEMM_A_SPLIT / RB_GEMM_B_SPLIT: TMA boxes per K-major tile
  int b_split = 1;
  int autotune = 1;          // RB_GEMM_AUTOTUNE: 0 = cost model only, even in tuning mode
  int deterministic = 0;     // RB_GEMM_DETERMINISTIC: 1 = no launch lets several CTAs add into the same output element
                             // (no reduction split, no tail cut), so results are bit-identical from run to run
};
static GemmOptions g_opt;
static std::once_flag g_opt_once;
static int g_tune_mode = 0;   // set by rb_gemm_tune_mode: launches of unseen shapes time their candidates

static int* option_slot(const char* name) {
  struct { const char* name; int* slot; } table[] = {
      {"force_mt", &g_opt.force_mt}, {"force_resident", &g_opt.force_resident}, {"force_halo", &g_opt.force_halo},
      {"force_taps", &g_opt.force_taps}, {"force_tail", &g_opt.force_tail}, {"force_wide", &g_opt.force_wide},
      {"force_box", &g_opt.force_box}, {"force_pair", &g_opt.force_pair}, {"pdl", &g_opt.pdl},
      {"bk32", &g_opt.bk32}, {"bn_cap", &g_opt.bn_cap}, {"a_split", &g_opt.a_split}, {"b_split", &g_opt.b_split},
      {"autotune", &g_opt.autotune}, {"deterministic", &g_opt.deterministic}};
  for (auto& t : table)
    if (strcmp(t.name, name) == 0) return t.slot;
  return nullptr;
}
static void options_from_env() {
  std::call_once(g_opt_once, [] {
    const char* names[] = {"force_mt", "force_resident", "force_halo", "force_taps", "force_tail", "force_wide", "force_box",
                           "force_pair", "pdl", "bk32", "bn_cap", "a_split", "b_split", "autotune", "deterministic"};
    for (const char* n : names) {
      char env[64] = "RB_GEMM_";
      size_t k = strlen(env);
      for (const char* c = n; *c && k + 1 < sizeof(env); ++c) env[k++] = (char)toupper((unsigned char)*c);
      env[k] = 0;
      const char* e = getenv(env);
      if (e) *option_slot(n) = atoi(e);
    }
  });
}

int pdl_enabled() {
  options_from_env();
  return g_opt.pdl >= 2 ? 1 : 0;
}

// ---- tile-shape planning -----------------------------------------------------------------------------------
// Cost model in "rows": the kernel is bound by the 128-byte rows it fills into shared memory per k-block
// (see the header comment), so an item costs about k-blocks x (rows of A + rows of B) plus its epilogue, and a
// launch costs rounds x item (persistent CTAs, one per SM). The planner picks sub-tiles per item (mt),
// the reduction split, B residency and whether the last wave is cut along the reduction to minimise that.
struct Plan {
  int mt, split, resident, tail;   // tail: parts per cut item of the last wave (0 = no cut)
  double cost;
  int pair = 0;                    // run as CTA pairs (never with resident B or a tail cut)
};

// CTA pairs need K-major operands loaded by plain or im2col TMA, a tile of at most 256 columns whose halves are whole
// boxes of the B map (the map's box is bn / b_split rows, so b_split must be even), and more than one pair's rows.
static bool pair_ok(const GemmTcParams& p) {
  if (g_opt.force_pair == 0 || g_pair_clusters <= 0) return false;
  if (p.a_mode != A_TILED_K && p.a_mode != A_IM2COL_K) return false;
  if (p.b_mode != B_TILED_K && p.b_mode != B_TILED_K3) return false;
  if (p.bn > 256 || p.bn % 16 != 0 || p.b_split < 2 || p.b_split % 2 != 0) return false;
  return p.M > 2 * BM;
}
// Boxes per tile for K-major operands (each box is issued by its own lane). A box must keep whole 8-row swizzle
// atoms, start on a 1024-byte boundary in shared memory and have at most 256 rows.
static int pick_box_split(int sp, int rows, int bk) {
  if (sp < 1) sp = 1;
  while (rows / sp > 256) sp <<= 1;
  while (sp > 1 && (rows % sp != 0 || (rows / sp) % 8 != 0 || ((rows / sp) * bk * 2) % 1024 != 0)) sp >>= 1;
  return sp < 1 ? 1 : sp;
}

// Boxes per B tile such that half a tile is a whole number of boxes whenever the shape allows pairs.
static int pairable_b_split(int bn, int bk) {
  int sp = pick_box_split(g_opt.b_split, bn, bk);
  if (g_opt.force_pair != 0 && sp % 2 != 0 && bn <= 256) {
    const int sp2 = pick_box_split(sp * 2, bn, bk);
    if (sp2 % 2 == 0) sp = sp2;
  }
  return sp;
}

static bool split_ok(int s, int num_kb) { return s == 1 || (s - 1) * ((num_kb + s - 1) / s) < num_kb; }

static int acc_stride_for(int bn) { return bn > 256 ? 512 : (bn > 128 ? 256 : 128); }

// Work items along M for `mt` sub-tiles per item (box mode: whole output rows per sub-tile, per image).
static int m_items_of(const GemmTcParams& p, int mt) {
  if (p.a_mode == A_BOX_K) {
    const int groups = (p.cv_P + mt * p.bx_rows - 1) / (mt * p.bx_rows);
    return (p.M / (p.cv_P * p.cv_Q)) * groups;
  }
  const int units = (p.M + BM * mt - 1) / (BM * mt);
  return p.pair ? (units + 1) / 2 : units;
}

// Parts per cut item for `items` work items on `sms` SMs (0 = cutting does not pay or is not possible): the last
// wave must be at most half full, every SM gets at most one part, a part keeps at least four k-blocks. A launch with
// fewer items than half the SMs (small batches, 7 x 7 layers) is one such wave: all of its items are cut.
static int tail_parts(long long items, int sms, int num_kb) {
  const int rem = (int)(items % sms);
  if (rem == 0 || rem * 2 > sms) return 0;
  int s = sms / rem;
  if (s > num_kb / 4) s = num_kb / 4;
  if (s > 16) s = 16;
  while (s > 1 && !split_ok(s, num_kb)) --s;
  return s >= 2 ? s : 0;
}

static Plan plan_shape(const GemmTcParams& p, bool allow_split, int fixed_split, bool b_is_weights) {
  if (g_opt.deterministic) {   // one CTA per output tile, its k-blocks in order
    allow_split = false;
    fixed_split = 1;
  }
  const int a_bytes = BM * p.bk * 2, b_bytes = p.bn_load * p.bk * 2;
  const double epi_elem = (p.epi == EPI_BF16) ? 1.2 : 1.6;
  Plan best{1, 1, 0, 0, 1e300};
  // the force options restrict the search (ignored when infeasible)
  const int force_mt = g_opt.force_mt, force_res = g_opt.force_resident;
  for (int pass = 0; pass < 2 && best.cost >= 1e299; ++pass)
  for (int mt = 1; mt <= 2; ++mt) {
    if (pass == 0 && force_mt && mt != force_mt) continue;
    if (mt == 2 && (p.M <= BM || p.bn > 256)) continue;
    if (mt == 2 && p.a_mode == A_BOX_K && p.cv_P <= p.bx_rows) continue;
    const int acc_stride = acc_stride_for(p.bn);
    const int acc_bufs = (2 * mt * acc_stride <= 512) ? 2 : 1;
    const int m_items = m_items_of(p, mt);
    const long long tiles = (long long)m_items * p.n_tiles;
    // up to one part per SM (a layer with a single output tile, e.g. the weight-grad of a 1 x 1 convolution on 96
    // channels, would otherwise leave SMs idle), each part at least eight k-blocks long
    const int split_cap = g_num_sms > 0 ? g_num_sms : 148;
    const int max_split = allow_split ? (p.num_kb / 8 > split_cap ? split_cap : (p.num_kb / 8 < 1 ? 1 : p.num_kb / 8)) : 1;
    for (int s = (fixed_split > 0 ? fixed_split : 1); s <= (fixed_split > 0 ? fixed_split : max_split); ++s) {
      if (!split_ok(s, p.num_kb)) continue;
      for (int res = 0; res <= 1; ++res) {
        if (pass == 0 && force_res >= 0 && res != force_res) continue;
        const long long panel = (long long)p.num_kb * b_bytes;
        if (res) {
          if (!b_is_weights || p.n_tiles != 1 || s != 1 || panel > 112 * 1024) continue;
          if ((TILE_SMEM_BYTES - panel) / (mt * a_bytes) < 3) continue;
        } else if (TILE_SMEM_BYTES / (mt * a_bytes + b_bytes) < 2) {
          continue;
        }
        const int kbs = (p.num_kb + s - 1) / s;
        const double rows_kb = mt * BM + (res ? 0 : p.bn_load);
        const double mainloop = kbs * rows_kb * (p.bk / 64.0);
        const double epi = mt * p.bn * epi_elem;
        const double item = acc_bufs == 2 ? (mainloop > epi ? mainloop : epi) + 0.15 * epi : mainloop + epi;
        for (int tail = 0; tail <= 1; ++tail) {
          int parts = 0;
          if (tail) {
            if (p.epi != EPI_BF16 || s != 1 || !p.ws || g_opt.force_tail == 0 || g_opt.deterministic) continue;
            parts = tail_parts(tiles, g_num_sms, p.num_kb);
            if (parts == 0) continue;
            const long long need = (tiles % g_num_sms) * mt * BM * (long long)p.bn * 4;
            if (need > p.ws_bytes) continue;
          } else if (pass == 0 && g_opt.force_tail == 1 && p.epi == EPI_BF16 && s == 1 && p.ws &&
                     tail_parts(tiles, g_num_sms, p.num_kb) > 0) {
            continue;
          }
          double rounds = (double)((tiles * s + g_num_sms - 1) / g_num_sms);
          if (parts) rounds = (double)(tiles / g_num_sms) + 1.0 / parts + 0.1;   // + the fix-up pass
          const double cost = rounds * item + (res ? (double)p.num_kb * p.bn_load * (p.bk / 64.0) : 0.0);
          if (cost < best.cost * 0.97) best = Plan{mt, s, res, parts, cost};
        }
      }
    }
  }
  return best;
}

// Fill in what follows from a plan; returns the grid size, or 0 when the plan does not fit.
static int apply_plan(GemmTcParams& p, const Plan& pl) {
  p.mt = pl.mt;
  p.split_k = pl.split;
  p.b_resident = pl.resident;
  if (pl.pair) {
    if (!pair_ok(p) || pl.resident || pl.tail || p.M <= BM * pl.mt) return 0;
    p.pair = 1;
    p.bn_load = p.bn / 2;      // rows of B per CTA
    p.b_split = p.b_split / 2;
  }
  p.acc_stride = acc_stride_for(p.bn);
  p.acc_bufs = (2 * p.mt * p.acc_stride <= 512) ? 2 : 1;
  if (p.mt * p.acc_stride > 512) return 0;
  const int a_bytes = BM * p.bk * 2, b_bytes = p.bn_load * p.bk * 2;
  const int panel = p.b_resident ? p.num_kb * b_bytes : 0;
  const int stage = p.mt * a_bytes + (p.b_resident ? 0 : b_bytes);
  if (panel >= TILE_SMEM_BYTES) return 0;
  p.stages = (TILE_SMEM_BYTES - panel) / stage;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  if (p.stages < 2) return 0;
  if (p.mt == 2 && p.M <= BM) return 0;
  if (p.mt == 2 && p.a_mode == A_BOX_K && p.cv_P <= p.bx_rows) return 0;
  const int m_items = m_items_of(p, p.mt);
  const long long items = (long long)m_items * p.n_tiles;
  p.tail_items = 0;
  p.tail_split = 0;
  long long work = items * p.split_k;
  if (pl.tail > 0) {
    if (p.epi != EPI_BF16 || p.split_k != 1 || !p.ws) return 0;
    p.tail_items = (int)(items % g_num_sms);
    p.tail_split = pl.tail;
    const long long rows = (long long)p.tail_items * p.mt * BM;
    if (p.tail_items == 0 || rows * p.bn * 4 > p.ws_bytes || !split_ok(pl.tail, p.num_kb)) return 0;
    cuuint64_t dims[2] = {(cuuint64_t)p.bn, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)p.bn * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t es[2] = {1, 1};
    if (g_encode_tiled(&p.tm_ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.ws, dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return 0;
    work = items - p.tail_items + (long long)p.tail_items * p.tail_split;
  }
  if (p.pair) return 2 * (int)(work < g_pair_clusters ? work : g_pair_clusters);
  return work < g_num_sms ? (int)work : g_num_sms;
}

// Epilogue of the cut items: D = act(workspace + bias), masked, as bf16; the workspace rows are cleared again so
// that the next launch that uses the workspace finds zeros. One thread per 8 columns.
struct TailFixArgs {
  float* ws;
  __nv_bfloat16* D;
  const float* bias;
  const __nv_bfloat16* mask;
  long long ldd;
  int M, bn, rows_per_item, m_items, direct, tail_items, n_valid, n_store, relu;
  int box, P, Q, bx_rows, bx_groups, mt;   // box mode: rows of a sub-tile are whole output rows of one image
};
__global__ void tail_fix_kernel(const TailFixArgs a) {
  pdl_prolog();
  const int gpr = a.bn / 8;
  const long long groups = (long long)a.tail_items * a.rows_per_item * gpr;
  const float act_lo = a.relu ? 0.f : -INFINITY;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const int c8 = (int)(g % gpr);
    const long long wr = g / gpr;                    // row of the workspace
    const int ti = (int)(wr / a.rows_per_item);
    const int r = (int)(wr - (long long)ti * a.rows_per_item);
    const int rem = a.direct + ti;
    const int tn = rem / a.m_items, tm = rem - tn * a.m_items;
    long long row = (long long)tm * a.rows_per_item + r;
    bool live = true;
    if (a.box) {
      const int j = r / BM, i = r - j * BM;
      const int n_img = tm / a.bx_groups;
      const int p_sub = ((tm - n_img * a.bx_groups) * a.mt + j) * a.bx_rows;
      live = i < max(0, min(a.bx_rows, a.P - p_sub)) * a.Q;
      row = ((long long)n_img * a.P + p_sub) * a.Q + i;
    }
    const int col = tn * a.bn + c8 * 8;
    float4* src = reinterpret_cast<float4*>(a.ws + wr * a.bn + c8 * 8);
    const float4 v0 = src[0], v1 = src[1];
    src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!live || row >= a.M || col >= a.n_store) continue;
    float f[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int n = col + e;
      f[e] = n < a.n_valid ? fmaxf(f[e] + (a.bias ? __ldg(a.bias + n) : 0.f), act_lo) : 0.f;
    }
    if (a.mask) {
      float m[8];
      load8(a.mask + row * a.ldd + col, m);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (!(m[e] > 0.f)) f[e] = 0.f;
    }
    store8(a.D + row * a.ldd + col, f);
  }
}

// What the most recent launch of this process used (for benchmarks and tests; not synchronised between threads):
// {sub-tiles per item, reduction split, resident B, tail parts, CTA pairs, tile width, A load mode, stages, grid}.
static int g_last_launch[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
static int g_last_cuda_error = 0;   // what the runtime answered to the last launch that failed

static int run_plan(GemmTcParams p, const Plan& pl, cudaStream_t stream) {
  const int grid = apply_plan(p, pl);
  if (grid <= 0) return -3;
  const int last[9] = {p.mt, p.split_k, p.b_resident, pl.tail, p.pair, p.bn, p.a_mode, p.stages, grid};
  memcpy(g_last_launch, last, sizeof(last));
  {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    int n_at = 0;
    if (p.pair) {
      at[n_at].id = cudaLaunchAttributeClusterDimension;
      at[n_at].val.clusterDim.x = 2;
      at[n_at].val.clusterDim.y = 1;
      at[n_at].val.clusterDim.z = 1;
      ++n_at;
    }
    if (g_opt.pdl >= 1) {   // the kernel's prologue may overlap the end of the work before it on the stream
      at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[n_at].val.programmaticStreamSerializationAllowed = 1;
      ++n_at;
    }
    cfg.attrs = n_at ? at : nullptr;
    cfg.numAttrs = (unsigned)n_at;
    const cudaError_t e = p.pair ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true>, p)
                                 : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false>, p);
    if (e != cudaSuccess) {
      g_last_cuda_error = (int)e;
      cudaGetLastError();
      return -4;
    }
  }
  if (p.tail_items > 0) {
    TailFixArgs f;
    f.ws = p.ws;
    f.D = reinterpret_cast<__nv_bfloat16*>(p.D);
    f.bias = p.bias;
    f.mask = p.mask_src;
    f.ldd = p.ldd;
    f.M = p.M;
    f.bn = p.bn;
    f.rows_per_item = p.mt * BM;
    f.m_items = m_items_of(p, p.mt);
    f.box = p.a_mode == A_BOX_K ? 1 : 0;
    f.P = p.cv_P;
    f.Q = p.cv_Q;
    f.bx_rows = p.bx_rows;
    f.bx_groups = f.box ? (p.cv_P + p.mt * p.bx_rows - 1) / (p.mt * p.bx_rows) : 1;
    f.mt = p.mt;
    f.direct = f.m_items * p.n_tiles - p.tail_items;
    f.tail_items = p.tail_items;
    f.n_valid = p.n_valid;
    f.n_store = p.n_store;
    f.relu = p.relu;
    const long long groups = (long long)p.tail_items * f.rows_per_item * (p.bn / 8);
    long long blocks = (groups + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    launch_pdl(tail_fix_kernel, (int)blocks, 256, 0, stream, f);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) g_last_cuda_error = (int)e;
  return e == cudaSuccess ? 0 : -4;
}

// Shapes whose output is overwritten (bf16 epilogue: forward and data-grad passes) can be tuned by measurement:
// in tuning mode (rb_gemm_tune_mode(1), which a network switches on while it runs each of its convolution shapes
// once on scratch operands at build time) a launch of a shape that has no cached plan times every feasible
// (sub-tiles per item, resident B, tail cut) choice on the given stream and caches the fastest. The cost model
// alone mis-ranks them by up to 30 % (it knows rows filled, not how much of the epilogue is exposed). Outside
// tuning mode a launch never times anything: it takes the cached plan, or the cost model's.
typedef std::tuple<int, int, int, int, int, int, int, int, int, int> PlanKey;
static std::map<PlanKey, Plan> g_plan_cache;
static std::mutex g_plan_mutex;

static PlanKey plan_key(const GemmTcParams& p) {
  return PlanKey(p.a_mode, p.b_mode, p.M, p.N, p.num_kb, p.bn, p.bk, p.n_tiles, p.cv_stride, p.mask_src ? 1 : 0);
}

// Times the candidates of `p` (3 launches each, best of the last 2); returns the best time in ms, or a negative
// value when nothing could be run.
static float tune_plan(const GemmTcParams& p, bool b_is_weights, cudaStream_t stream, Plan* out) {
  // the candidates: plain plans first (sub-tiles x resident B x tail cut), then CTA pairs
  Plan cands[12];
  int n_cands = 0;
  for (int pr = 0; pr <= (pair_ok(p) ? 1 : 0); ++pr) {
    for (int mt = 1; mt <= 2; ++mt) {
      for (int res = 0; res <= (pr ? 0 : 1); ++res) {
        if (res && (!b_is_weights || p.n_tiles != 1)) continue;
        for (int tail = 0; tail <= (pr ? 0 : 1); ++tail) {
          Plan cand{mt, 1, res, 0, 0.0};
          cand.pair = pr;
          if (tail) {
            if (!p.ws || g_opt.force_tail == 0 || g_opt.deterministic) continue;
            cand.tail = tail_parts((long long)m_items_of(p, mt) * p.n_tiles, g_num_sms, p.num_kb);
            if (cand.tail == 0) continue;
          }
          GemmTcParams q = p;
          if (apply_plan(q, cand) <= 0 || (res && q.stages < 3)) continue;
          cands[n_cands++] = cand;
        }
      }
    }
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float best_ms = 1e30f;
  for (int c = 0; c < n_cands; ++c) {
    float ms = 1e30f;
    bool ok = true;
    for (int rep = 0; rep < 3 && ok; ++rep) {
      cudaEventRecord(e0, stream);
      ok = run_plan(p, cands[c], stream) == 0;
      cudaEventRecord(e1, stream);
      ok = ok && cudaEventSynchronize(e1) == cudaSuccess;
      float t = 0.f;
      if (ok) cudaEventElapsedTime(&t, e0, e1);
      if (ok && rep > 0 && t < ms) ms = t;   // the first run warms the caches
    }
    // pairs are timed after every plain plan and must win by 3 %: measured alone they tie to within 2 % on the
    // layers tried, and inside a training step (other kernels beside them) the plain plans did better
    if (ok && ms < best_ms * (cands[c].pair ? 0.97f : 1.0f)) {
      best_ms = ms;
      *out = cands[c];
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return best_ms < 1e29f ? best_ms : -1.f;
}

static bool tunable(const GemmTcParams& p, cudaStream_t stream) {
  if (!g_tune_mode || !g_opt.autotune || p.epi != EPI_BF16) return false;
  if (g_opt.force_mt || g_opt.force_resident >= 0 || g_opt.force_pair == 1) return false;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  return cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone;
}

static int launch(GemmTcParams& p, bool allow_split, int fixed_split, bool b_is_weights, cudaStream_t stream) {
  if (p.M <= 0 || p.n_tiles <= 0 || p.num_kb <= 0) return 0;
  Plan pl = plan_shape(p, allow_split, fixed_split, b_is_weights);
  if (pl.cost >= 1e299) return -3;
  bool forced = g_opt.force_mt || g_opt.force_resident >= 0 || g_opt.force_tail >= 0;
  if (g_opt.force_pair == 1 && pair_ok(p)) {   // pairs wherever they are feasible (tests, experiments)
    for (int mt = g_opt.force_mt ? g_opt.force_mt : 2; mt >= 1; --mt) {
      Plan pp{mt, pl.split, 0, 0, 0.0};
      pp.pair = 1;
      GemmTcParams q = p;
      if (apply_plan(q, pp) > 0) {
        pl = pp;
        forced = true;
        break;
      }
      if (g_opt.force_mt) break;
    }
  }
  if (p.epi == EPI_BF16 && !forced) {
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    auto it = g_plan_cache.find(plan_key(p));
    if (it != g_plan_cache.end()) {
      Plan cached = it->second;
      if (cached.tail && (!p.ws || g_opt.deterministic)) cached.tail = 0;   // tuned with a workspace, launched without
      if (cached.pair && !pair_ok(p)) cached = pl;
      pl = cached;
    } else if (tunable(p, stream)) {
      Plan best = pl;
      if (tune_plan(p, b_is_weights, stream, &best) > 0.f) pl = best;
      g_plan_cache[plan_key(p)] = pl;
    }
  }
  return run_plan(p, pl, stream);
}

static int round_bn(int n, int cap) {
  int bn = ((n + 31) / 32) * 32;
  if (bn > cap) bn = cap;
  return bn;
}

// Tile width for `n` output columns: among 1..4 column tiles (width a multiple of `gran`, at most 256), the one
// whose plan is cheapest. `setup(p, bn)` must fill the fields that depend on the width.
template <class Setup>
static int pick_bn(GemmTcParams& p, int n, int gran, bool allow_split, int fixed_split, bool b_is_weights,
                   Setup setup) {
  int best_bn = 0;
  double best_cost = 1e300;
  const int cap = g_opt.bn_cap > 0 ? g_opt.bn_cap : 256;
  for (int nt = 1; nt <= 4; ++nt) {
    int bn = (n + nt - 1) / nt;
    const int g = (nt > 1 && gran < 64) ? 64 : gran;   // the bf16 epilogue stores 64-column slabs
    bn = (bn + g - 1) / g * g;
    if (bn > 256 || bn > cap || bn == best_bn) continue;
    setup(p, bn);
    const Plan pl = plan_shape(p, allow_split, fixed_split, b_is_weights);
    if (pl.cost < best_cost * 0.97) { best_cost = pl.cost; best_bn = bn; }
  }
  if (best_bn == 0) best_bn = 256;
  setup(p, best_bn);
  return best_bn;
}

// Tile width chosen by measurement for a convolution shape (key: the plan key with the width left out).
static std::map<PlanKey, int> g_bn_cache;

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
               int n_store, int split_k, int bn_cap, float* ws, long long ws_bytes, unsigned int* status,
               cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  if ((n_store > 0 ? n_store : N) % 32 != 0 || ldd % 8 != 0) return -11;  // epilogue writes 32-column chunks
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.ws = ws;
  p.ws_bytes = ws ? ws_bytes : 0;
  const bool any_mn = a_mn || b_mn;
  p.bk = (!any_mn && (K % 64 != 0) && (K % 32 == 0)) ? 32 : 64;
  if (bn_cap <= 0) bn_cap = 256;
  p.bn = round_bn(N, bn_cap);
  if (b_mn || (epi == EPI_BF16 && N > p.bn)) p.bn = ((p.bn + 63) / 64) * 64;
  p.bn_load = p.bn;
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
    p.a_split = pick_box_split(g_opt.a_split, BM, p.bk);
    rc = make_map_2d(&p.tm_a, A, K, M, lda, p.bk, BM / p.a_split, ksw);
  }
  if (rc) return rc;
  if (b_mn) {
    p.b_mode = B_TILED_MN;
    rc = make_map_2d(&p.tm_b, B, N, K, ldb, 64, p.bk, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    p.b_mode = B_TILED_K;
    p.b_split = pairable_b_split(p.bn, p.bk);
    rc = make_map_2d(&p.tm_b, B, K, N, ldb, p.bk, p.bn / p.b_split, ksw);
  }
  if (rc) return rc;
  p.epi = epi;
  p.relu = relu;
  p.n_valid = n_valid > 0 ? n_valid : N;
  p.n_store = n_store > 0 ? n_store : N;
  p.ldd = ldd;
  p.D = D;
  p.bias = bias;
  p.mask_src = reinterpret_cast<const __nv_bfloat16*>(mask_src);
  p.status = status;
  if (epi == EPI_BF16) {
    rc = make_map_out(&p.tm_d, D, p.n_store, M, ldd);
    if (rc) return rc;
    if (mask_src) rc = make_map_out(&p.tm_mask, const_cast<void*>(mask_src), p.n_store, M, ldd);
    if (rc) return rc;
  } else {
    rc = make_map_out_f32(&p.tm_d, D, p.n_store, M, ldd);
    if (rc) return rc;
  }
  if (epi != EPI_F32_ATOMIC) split_k = 1;
  if (split_k > p.num_kb) split_k = p.num_kb;
  while (split_k > 1 && !split_ok(split_k, p.num_kb)) --split_k;
  return launch(p, epi == EPI_F32_ATOMIC && split_k <= 0, split_k > 0 ? split_k : 0, !b_mn, stream);
}

// Convolution forward (also used for stride-1 data-grad with flipped filters).
//   x   NHWC bf16 [N][H][W][Cp]      w  bf16 [Kout][R*S][Cp]     y  bf16 [N*P*Q][ldy]
//   base pixel range: lower = -pad_lo, P/Q given by the caller.
int rb_conv_fprop_tc(const void* x, int N, int H, int W, int Cp, const void* w, int Kout, int R, int S, int stride,
                     int pad_h, int pad_w, int P, int Q, void* y, long long ldy, const float* bias, int relu,
                     const void* mask_src, int n_valid, int n_store, float* ws, long long ws_bytes,
                     unsigned int* status, cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.ws = ws;
  p.ws_bytes = ws ? ws_bytes : 0;
  // The TMA unit is bound by rows (requests), not bytes: 64-channel (128-byte) rows halve the rows per MMA. A channel
  // count such as 96 therefore runs as two 64-channel chunks whose upper half lies outside the tensor and is
  // zero-filled by the TMA unit (both operands), rather than as three 32-channel chunks: a third more MMA work,
  // a third fewer loads, and the loads are what binds.
  p.bk = (Cp % 64 == 0 || (Cp > 64 && g_opt.bk32 != 1)) ? 64 : 32;   // option bk32: keep 32-channel chunks
  if (Cp % 32 != 0) return -10;
  if ((n_store > 0 ? n_store : Kout) % 32 != 0 || ldy % 8 != 0) return -11;
  const CUtensorMapSwizzle ksw = p.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const int n_cols = n_store > 0 ? n_store : Kout;
  p.M = N * P * Q;
  p.N = Kout;
  p.cv_cchunks = (Cp + p.bk - 1) / p.bk;
  p.num_kb = R * S * p.cv_cchunks;
  p.epi = EPI_BF16;
  pick_bn(p, n_cols, 32, false, 1, true, [n_cols](GemmTcParams& q, int bn) {
    q.bn = q.bn_load = bn;
    q.n_tiles = (n_cols + bn - 1) / bn;
  });
  p.a_mode = A_IM2COL_K;
  p.b_mode = B_TILED_K3;
  p.cv_P = P;
  p.cv_Q = Q;
  p.cv_stride = stride;
  p.cv_lower_h = -pad_h;
  p.cv_lower_w = -pad_w;
  p.cv_S = S;
  p.relu = relu;
  p.n_valid = n_valid > 0 ? n_valid : Kout;
  p.n_store = n_store > 0 ? n_store : Kout;
  p.ldd = ldy;
  p.D = y;
  p.bias = bias;
  p.mask_src = reinterpret_cast<const __nv_bfloat16*>(mask_src);
  p.status = status;
  // ---- halo mode (see the header comment): stride 1, more than one filter tap, image no wider than 128
  {
    const int force = g_opt.force_halo;   // 0 = never, 1 = whenever feasible
    if (stride == 1 && R * S > 1 && Q <= 128 && force != 0) {
      int pitch = 8;
      while (pitch < Q) pitch *= 2;
      const int rows = 128 / pitch;
      const int mt = P > rows ? 2 : 1;
      const int groups = (P + mt * rows - 1) / (mt * rows);
      const double util = ((double)Q / pitch) * ((double)P / (groups * mt * rows));
      // one column tile when it fits, else equal tiles of a multiple of 64 columns
      const int nt = (n_cols + 255) / 256;
      int bn = (n_cols + nt - 1) / nt;
      bn = nt > 1 ? (bn + 63) / 64 * 64 : (bn + 31) / 32 * 32;
      const int rtot = mt * rows + R - 1;
      const int a_bytes = (rtot * pitch * p.bk * 2 + 1023) / 1024 * 1024;
      const int b_bytes = bn * p.bk * 2;
      int stages = (TILE_SMEM_BYTES - 2 * a_bytes) / b_bytes;
      if (stages > MAX_STAGES) stages = MAX_STAGES;
      (void)util;
      // measured slower than the im2col path on every layer tried (0.239 vs 0.167 ms on AlexNet conv2), so the
      // mode is only taken when forced; it stays for the tests and for further work
      if (rtot <= 256 && bn <= 256 && stages >= 3 && force == 1) {
        p.a_mode = A_HALO_K;
        p.bn = p.bn_load = bn;
        p.n_tiles = (n_cols + bn - 1) / bn;
        p.hl_pitch = pitch;
        p.hl_rows = rows;
        p.hl_rtot = rtot;
        p.hl_groups = groups;
        p.hl_R = R;
        p.hl_pad_h = pad_h;
        p.hl_pad_w = pad_w;
        p.hl_a_stages = 2;
        p.hl_a_bytes = a_bytes;
        p.mt = mt;
        p.split_k = 1;
        p.b_resident = 0;
        p.acc_stride = bn > 128 ? 256 : 128;
        p.acc_bufs = (2 * mt * p.acc_stride <= 512) ? 2 : 1;
        p.stages = stages;
        rc = make_map_nhwc(&p.tm_a, x, Cp, W, H, N, Cp, p.bk, pitch, rtot, ksw);
        if (rc) return rc;
        rc = make_map_3d(&p.tm_b, w, Cp, (uint64_t)R * S, Kout, Cp, (uint64_t)R * S * Cp, p.bk, 1, p.bn, ksw);
        if (rc) return rc;
        const uint32_t bw = pitch < 32 ? pitch : 32, bh = 32 / bw;
        rc = make_map_nhwc(&p.tm_d, y, p.n_store, Q, P, N, ldy, 64, bw, bh, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (mask_src)
          rc = make_map_nhwc(&p.tm_mask, mask_src, p.n_store, Q, P, N, ldy, 64, bw, bh, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        const long long work = (long long)N * groups * p.n_tiles;
        const int grid = work < g_num_sms ? (int)work : g_num_sms;
        gemm_tc_kernel<false><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(p);
        return cudaGetLastError() == cudaSuccess ? 0 : -4;
      }
    }
  }
  // upper corner so that the base pixel takes exactly P x Q positions
  const int upper_h = (P - 1) * stride - pad_h - (H - 1);
  const int upper_w = (Q - 1) * stride - pad_w - (W - 1);
  p.a_split = pick_box_split(g_opt.a_split, BM, p.bk);
  const bool one_by_one = R == 1 && S == 1 && stride == 1 && pad_h == 0 && pad_w == 0 && P == H && Q == W;
  rc = make_map_out(&p.tm_d, y, p.n_store, p.M, ldy);
  if (rc) return rc;
  if (mask_src) rc = make_map_out(&p.tm_mask, const_cast<void*>(mask_src), p.n_store, p.M, ldy);
  if (rc) return rc;
  // How the A operand is loaded (`box` = tap-shifted tiled boxes of whole output rows, else the im2col map, or plain
  // tiled rows for a 1 x 1 convolution) and what depends on the tile width: column tiling, the filter map's box.
  auto configure = [&](GemmTcParams& q, int box, int bn) -> int {
    int e;
    if (box) {
      q.a_mode = A_BOX_K;
      q.a_split = 1;
      q.bx_rows = BM / Q;
      q.bx_pad_h = pad_h;
      q.bx_pad_w = pad_w;
      e = make_map_nhwc(&q.tm_a, x, Cp, W, H, N, Cp, q.bk, Q, q.bx_rows, ksw);
    } else if (one_by_one) {
      // a 1 x 1 convolution is a plain GEMM over the pixel rows: tiled loads, which the TMA unit serves 2-3x
      // faster per row than im2col-mode loads
      q.a_mode = A_TILED_K;
      e = make_map_2d(&q.tm_a, x, Cp, (uint64_t)q.M, Cp, q.bk, BM / q.a_split, ksw);
    } else {
      q.a_mode = A_IM2COL_K;
      e = make_map_im2col(&q.tm_a, x, N, H, W, Cp, -pad_h, -pad_w, upper_h, upper_w, stride, q.bk, BM / q.a_split, ksw);
    }
    if (e) return e;
    q.bn = q.bn_load = bn;
    q.n_tiles = (n_cols + bn - 1) / bn;
    q.b_split = pairable_b_split(bn, q.bk);
    return make_map_3d(&q.tm_b, w, Cp, (uint64_t)R * S, Kout, Cp, (uint64_t)R * S * Cp, q.bk, 1, bn / q.b_split, ksw);
  };
  // Candidates beside the default (im2col loads, tiles of at most 256 columns):
  //  * between 257 and 512 output columns, ONE tile as wide as the layer (two MMAs side by side, one accumulator
  //    set, no overlap of epilogue and main loop) instead of narrower tiles that each load the A operand again;
  //  * for stride-1 convolutions with more than one tap and output rows of at most 128 positions, box loads:
  //    cheaper per row for the TMA unit, at the price of tile rows that are computed and dropped when Q does not
  //    divide 128 (and when bx_rows does not divide P).
  // Which is fastest is decided by measurement in tuning mode and remembered per shape; without a measurement the
  // default is taken.
  const int bn_default = p.bn;
  const int bn_wide = (n_cols > 256 && n_cols <= 512 && g_opt.force_wide != 0 && g_opt.bn_cap >= 256) ? n_cols : 0;
  const bool box_ok = stride == 1 && R * S > 1 && Q <= BM && g_opt.force_box != 0 && g_opt.force_halo != 1;
  int use = bn_default;   // low 16 bits: tile width; bit 16: box loads
  if (bn_wide || box_ok) {
    p.bn = p.n_tiles = 0;
    p.a_mode = A_IM2COL_K;
    const PlanKey ckey = plan_key(p);
    std::lock_guard<std::mutex> lock(g_plan_mutex);   // released at the end of this block, before `launch` takes it
    auto it = g_bn_cache.find(ckey);
    if (g_opt.force_wide == 1 || g_opt.force_box == 1) {
      use = ((bn_wide && g_opt.force_wide == 1) ? bn_wide : bn_default) | ((box_ok && g_opt.force_box == 1) ? 1 << 16 : 0);
    } else if (it != g_bn_cache.end()) {
      use = it->second;
    } else if (tunable(p, stream)) {
      float best_ms = 1e30f;
      for (int box = 0; box <= (box_ok ? 1 : 0); ++box) {
        for (int bn : {bn_default, bn_wide}) {
          if (bn == 0) continue;
          GemmTcParams q = p;
          if (configure(q, box, bn)) continue;
          Plan pl{1, 1, 0, 0, 0.0};
          const float ms = tune_plan(q, true, stream, &pl);
          if (ms > 0.f) {
            g_plan_cache[plan_key(q)] = pl;
            if (ms < best_ms) { best_ms = ms; use = bn | (box << 16); }
          }
        }
      }
      g_bn_cache[ckey] = use;
    }
  }
  rc = configure(p, (use >> 16) & 1, use & 0xFFFF);
  if (rc) return rc;
  return launch(p, false, 1, true, stream);
}

// Convolution weight-grad:  dw[Kout][R*S][Cp] (fp32) (+)= sum over pixels dy[pix][k] * x[pix shifted by tap][c].
//   The result is always accumulated into dw (red.add), so dw holds zeros or the running gradient on entry.
int rb_conv_wgrad_tc(const void* x, int N, int H, int W, int Cp, const void* dy, long long lddy, int Kout, int R,
                     int S, int stride, int pad_h, int pad_w, int P, int Q, float* dw, int split_k,
                     unsigned int* status, cudaStream_t stream) {
  int rc = ensure_driver_entry();
  if (rc) return rc;
  GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.bk = 64;
  p.M = Kout;
  p.N = R * S * Cp;
  const long long pixels = (long long)N * P * Q;
  p.num_kb = (int)((pixels + p.bk - 1) / p.bk);
  p.wg_cpad = Cp;
  p.epi = EPI_F32_ATOMIC;
  if (split_k > p.num_kb) split_k = p.num_kb;
  while (split_k > 1 && !split_ok(split_k, p.num_kb)) --split_k;
  const int taps = R * S;
  p.wg_ntaps = taps;
  const bool auto_split = split_k <= 0;
  const int fixed = split_k > 0 ? split_k : 0;
  // candidates: (a) one tap per tile, 1..4 channel tiles; (b) several taps side by side when a tap is narrow
  double best_cost = 1e300;
  int best_bn = 0, best_taps = 1;
  auto setup = [Cp, taps](GemmTcParams& q, int bn, int T) {
    q.bn = q.bn_load = bn;
    q.wg_taps = T;
    if (T > 1) {
      q.wg_cw = bn / T;
      q.wg_ctiles = 1;
      q.n_tiles = (taps + T - 1) / T;
    } else {
      q.wg_cw = bn;
      q.wg_ctiles = (Cp + bn - 1) / bn;
      q.n_tiles = taps * q.wg_ctiles;
    }
  };
  for (int nt = 1; nt <= 4; ++nt) {
    int bn = (Cp + nt - 1) / nt;
    bn = (bn + 63) / 64 * 64;
    if (bn > 256) continue;
    setup(p, bn, 1);
    const Plan pl = plan_shape(p, auto_split, fixed, false);
    if (pl.cost < best_cost * 0.97) { best_cost = pl.cost; best_bn = bn; best_taps = 1; }
  }
  const int cw = (Cp + 63) / 64 * 64;
  for (int T = 2; T * cw <= 256 && T <= taps; ++T) {
    setup(p, T * cw, T);
    const Plan pl = plan_shape(p, auto_split, fixed, false);
    // a tile with idle tap slots still pays for them: scale by the slots actually computed
    const double waste = (double)(p.n_tiles * T) / taps;
    if (pl.cost * waste < best_cost * 0.97) { best_cost = pl.cost * waste; best_bn = T * cw; best_taps = T; }
  }
  {  // option force_taps = T takes the T-taps-per-tile candidate when it is feasible
    const int T = g_opt.force_taps;
    if (T == 1 && best_taps != 1) { best_taps = 1; best_bn = cw > 256 ? 256 : cw; }
    if (T > 1 && T * cw <= 256 && T <= taps) { best_taps = T; best_bn = T * cw; }
  }
  if (best_bn == 0) return -3;
  setup(p, best_bn, best_taps);
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
  p.epi = EPI_F32_ATOMIC;
  p.n_valid = p.N;
  p.n_store = p.N;
  p.ldd = (long long)R * S * Cp;
  p.D = dw;
  rc = make_map_out_f32(&p.tm_d, dw, p.ldd, Kout, p.ldd);
  if (rc) return rc;
  p.status = status;
  if (split_k > p.num_kb) split_k = p.num_kb;
  while (split_k > 1 && !split_ok(split_k, p.num_kb)) --split_k;
  return launch(p, split_k <= 0, split_k > 0 ? split_k : 0, false, stream);
}

// Planner options by name (see GemmOptions); returns 0, or -1 for an unknown name.
int rb_gemm_set_option(const char* name, int value) {
  options_from_env();
  int* slot = option_slot(name);
  if (!slot) return -1;
  *slot = value;
  return 0;
}

int rb_gemm_get_option(const char* name, int* value) {
  options_from_env();
  int* slot = option_slot(name);
  if (!slot) return -1;
  *value = *slot;
  return 0;
}

// Tuning mode: while on, a bf16-epilogue launch of a shape without a cached plan times its candidates (it
// synchronises the stream, so it must not run inside a stream capture) and caches the winner.
int rb_gemm_tune_mode(int on) {
  g_tune_mode = on ? 1 : 0;
  return 0;
}

int rb_gemm_clear_plans() {
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  g_plan_cache.clear();
  g_bn_cache.clear();
  return 0;
}

// out[0..7]: the role-profile counters (all zero in a build without -DRB_GEMM_PROFILE, returns 1 then); cleared on read.
int rb_gemm_role_profile(unsigned long long* out) {
  for (int i = 0; i < 8; ++i) out[i] = 0ull;
#ifdef RB_GEMM_PROFILE
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, g_role_cycles, sizeof(unsigned long long) * 8) != cudaSuccess) return -1;
  const unsigned long long zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cudaMemcpyToSymbol(g_role_cycles, zeros, sizeof(zeros)) != cudaSuccess) return -1;
  return 0;
#else
  return 1;
#endif
}

// Runtime error code of the last launch that failed (a launcher's return value of -4), 0 if none did.
int rb_gemm_last_cuda_error() { return g_last_cuda_error; }

// out[0..8]: the tile plan of the most recent launch, see g_last_launch.
int rb_gemm_last_launch(int* out) {
  memcpy(out, g_last_launch, sizeof(g_last_launch));
  return 0;
}

int rb_num_sms() {
  ensure_driver_entry();
  return g_num_sms;
}

}  // extern "C"
