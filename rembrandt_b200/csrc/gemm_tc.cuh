// Parameter block of the persistent tcgen05 GEMM / implicit-GEMM convolution
// kernel (gemm_tc.cu). One kernel, configured at run time, serves:
//   conv fprop   A = im2col(X) K-major (TMA im2col)   B = filters K-major
//                or, stride 1: A = column-shifted halo tiles of X (plain tiled TMA, A_HALO_K), see gemm_tc.cu
//   conv dgrad   A = im2col(dY) K-major               B = flipped/transposed filters K-major
//   conv wgrad   A = dY^T MN-major (tiled)            B = im2col(X) MN-major (TMA im2col)
//   affine fwd   A = X K-major                        B = W K-major
//   affine dgrad A = dY K-major                       B = W MN-major
//   affine wgrad A = dY^T MN-major                    B = X^T MN-major
// Reference parity: these replace the cuDNN convolution forward / backward-data /
// backward-filter calls and the cuBLAS sgemm calls of the reference operators
// (src/operator/mod.rs:1075-1176 affine, :1663-1795 conv).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace rb {

enum : int { A_TILED_K = 0, A_IM2COL_K = 1, A_TILED_MN = 2, A_HALO_K = 3, A_BOX_K = 4 };
enum : int { B_TILED_K = 0, B_TILED_MN = 1, B_IM2COL_MN = 2, B_TILED_K3 = 3 };
enum : int { EPI_BF16 = 0, EPI_F32_STORE = 1, EPI_F32_ATOMIC = 2 };

struct alignas(64) GemmTcParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  CUtensorMap tm_mask; // EPI_BF16 with mask_src: same geometry as tm_d over the mask tensor (epilogue TMA loads)
  CUtensorMap tm_d;    // EPI_BF16: output map for the TMA stores of the epilogue (box 64 columns x 32 rows)
  int a_mode, b_mode;
  int M, N;            // extent of D in rows / columns (tiles are clipped against these)
  int bn;              // tile width (multiple of 32); above 256 the tile is two MMAs wide (256 + the rest), mt = 1
  int bn_load;         // rows of B brought in per k-block (= bn; kept separate from the MMA width)
  int bk;              // k-block depth (64 or 32)
  int num_kb;          // k-blocks over the whole reduction
  int split_k;         // reduction split; > 1 requires EPI_F32_ATOMIC
  int stages;
  int mt;              // 128-row sub-tiles per work item (1 or 2): they share one B stage
  int b_resident;      // 1: the whole B panel (all k-blocks) is loaded once per CTA and stays in shared memory
  int acc_stride;      // TMEM columns between the accumulators of the sub-tiles (128, 256 or 512)
  int acc_bufs;        // accumulator sets in TMEM (2 = epilogue overlaps the next main loop, 1 = no overlap)
  // convolution geometry (im2col operands)
  int cv_P, cv_Q;      // output height / width per image
  int cv_stride;       // traversal stride
  int cv_lower_h, cv_lower_w;  // lower corner of the base pixel (= -pad)
  int cv_S;            // filter width (taps are enumerated r*S+s)
  int cv_cchunks;      // channel chunks of bk per tap (A_IM2COL_K / B_TILED_K3)
  int wg_taps;         // filter taps per column tile (B_IM2COL_MN; > 1 only when one tap's channels fit 128 columns)
  int wg_cw;           // columns reserved per tap inside a tile (multiple of 64)
  int wg_ntaps;        // R*S
  int wg_ctiles;       // channel tiles of bn per tap (B_IM2COL_MN)
  int wg_cpad;         // padded input channels: column of D = tap*wg_cpad + channel
  int a_split, b_split; // K-major operands: TMA boxes (one issuing lane each) per 128-row A sub-tile / per B tile
  int n_tiles;         // tiles along N (taps*wg_ctiles for wgrad)
  // halo mode (A_HALO_K): a sub-tile is hl_rows output rows of one image at a row pitch of hl_pitch positions
  int hl_pitch;        // 8..128, a power of two >= Q; hl_rows * hl_pitch = 128
  int hl_rows;
  int hl_rtot;         // input rows per A stage = mt * hl_rows + R - 1
  int hl_groups;       // work items per image = ceil(P / (mt * hl_rows))
  int hl_R;            // filter height
  int hl_pad_h, hl_pad_w;
  int hl_a_stages;     // A stages in shared memory (each hl_a_bytes apart)
  int hl_a_bytes;
  // box mode (A_BOX_K, stride-1 convolutions): a sub-tile is bx_rows whole output rows of one image (bx_rows * Q <=
  // 128 positions, contiguous in the NHWC output); the A operand of filter tap (r, s) is ONE tiled 4-D box of
  // bx_rows x Q pixels x bk channels whose corner is shifted by the tap (zero fill outside the image), which the TMA
  // unit serves at the rate of tiled loads instead of the 2-3 times slower im2col mode
  int bx_rows;
  int bx_pad_h, bx_pad_w;
  // epilogue
  int epi;
  int relu;            // EPI_BF16: clamp at zero after the bias
  int n_valid;         // columns >= n_valid are written as zero (channel padding)
  int n_store;         // columns >= n_store are not written at all
  long long ldd;       // row pitch of D in elements
  void* D;
  const float* bias;               // optional, indexed by column
  const __nv_bfloat16* mask_src;   // optional, same layout as D: D is zeroed where mask_src <= 0
  unsigned int* status;            // error bits (see ptx.cuh)
  // Tail cut (EPI_BF16, split_k = 1): the work items of the last, partly filled wave are cut along the reduction
  // into `tail_split` parts each, so that every SM gets a share of them instead of a few SMs a whole item. The
  // parts add their fp32 partial sums into a workspace (TMA reduce-add); `tail_fix_kernel` then applies the
  // epilogue (bias, activation, mask, bf16) to those items and clears the workspace again.
  CUtensorMap tm_ws;   // fp32 workspace: [tail_items * mt * 128 rows][bn columns], 32 x 32 boxes
  float* ws;           // zero on entry, zero again after the fix-up; null = no tail cut possible
  long long ws_bytes;
  int tail_items;      // 0 = no tail cut
  int tail_split;
  // CTA pairs (tcgen05 cta_group::2; K-major operands only): the kernel runs as clusters of two CTAs. A work item
  // is 2 * mt sub-tiles of 128 rows, CTA r of the pair owns sub-tiles (2 * tm + r) * mt .. + mt: it loads their A
  // rows, rows [r * bn_load, (r + 1) * bn_load) of the B tile (bn_load = bn / 2), and runs their epilogue from its
  // own TMEM. The even CTA issues one 256 x bn x 16 MMA where two CTAs alone would issue two 128 x bn x 16 ones,
  // and each SM reads only half of B from its shared memory.
  int pair;
};

}  // namespace rb
