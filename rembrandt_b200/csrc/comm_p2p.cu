// Communication kernels that move data between GPUs themselves: peer-to-peer loads / stores / reductions
// over NVLink (and NVSwitch multimem instructions where a multicast mapping exists), fused with the maths
// that follows the exchange.
//
//   allreduce_sgd   gradient all-reduce + 1/N + SGD momentum / weight decay + bf16 weight refresh in one
//                   kernel. Two-shot: rank r reduces shard r of the bucket from every peer's gradient
//                   buffer, applies the optimizer to its shard of the fp32 master weights (master and
//                   momentum are therefore sharded), and stores the new bf16 weights into every peer's
//                   compute copy. One-shot (small buckets): every rank reduces the whole bucket itself.
//                   op = 1 turns it into a plain in-place fp32 average (exact parameter sync, benchmarks).
//   publish / gossip_mix   a rank publishes a snapshot of its parameters; a peer pulls it through NVLink and
//                   applies x <- x - alpha (x - x_peer) in one pass (pair / pull gossip).
//   push_add / push_finalize   push gossip: vectors are red.add'ed into the target's accumulator.
//   elastic_pull / elastic_apply   elastic averaging against a centre held by rank 0.
//
// Replaces the reference's ring all-reduce (src/arch_new.rs:554-573), its MPI all-reduce through host memory
// (src/worker/allreduce_dist.rs:211-241) and its gossip / elastic-averaging workers (src/operator/comm.rs:125-296,
// src/worker/gossip_*.rs, src/worker/elasticserver_dist.rs).
//
// Cross-GPU ordering uses per-bucket flag words in peer-visible memory carrying an epoch number; every wait
// on a flag is bounded (globaltimer deadline) and a wait that runs out sets RB_STATUS_PEER_TIMEOUT in the
// status word, skips the data movement that depended on it and lets the kernel finish normally.
// No TMA is used here at all.
#include "common.cuh"
#include "ptx.cuh"
#include "sgd_rules.cuh"

namespace rb {

constexpr int MAX_RANKS = 8;
constexpr uint64_t PEER_WAIT_NS = 3000000000ull;  // default limit of a wait on a peer: 3 s

// Every argument block carries `wait_ns`, the limit of each wait on a peer in this launch; 0 takes the default.
__device__ __forceinline__ uint64_t wait_limit(long long wait_ns) {
  return wait_ns > 0 ? (uint64_t)wait_ns : PEER_WAIT_NS;
}

struct ArSgdArgs {
  float* grads[MAX_RANKS];     // peer-visible buffers, identical layout on every rank
  bf16* w16[MAX_RANKS];        // peer-visible bf16 compute weights (op 0)
  float* w32[MAX_RANKS];       // optional: peer-visible fp32 masters to keep replicated (op 0)
  uint32_t* flags[MAX_RANKS];  // peer-visible flag pads: [slot][phase 0/1][source rank]
  float* stage[MAX_RANKS];     // peer-visible staging: per bucket, `world` slots (one per source rank) of shard length
  float* w;                    // local master weights
  float* v;                    // local momentum
  const float* mc_grads;       // multimem (NVSwitch multicast) address of the gradient buffer, or null
  bf16* mc_w16;                // multimem address of the bf16 weights, or null
  uint32_t* epoch_ptr;         // local: last completed epoch of this slot
  unsigned int* block_counter; // local, zero between launches
  unsigned int* status;
  uint32_t* wait_ok;           // local: outcome of ar_wait_kernel for this slot (null: the reducing kernel waits itself)
  long long off, n, decay_len, stage_off;
  int rank, world, slot, one_shot, op, zero_grads;
  float avg_scale;             // op 1: result = sum * avg_scale
  SgdHyper h;
  long long wait_ns;           // limit of each wait on a peer, ns (0: the 3 s default)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// true once *p has reached `epoch` (wrap-around safe); false after the deadline
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t epoch, uint64_t limit_ns) {
  if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) return false;
  }
}
__device__ __forceinline__ float4 ld_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 mm_ld_reduce_f4(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_f4(void* p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ uint32_t* flag_at(uint32_t* pad, int slot, int phase, int src) {
  return pad + ((slot * 2 + phase) * MAX_RANKS + src);
}

// All threads of the block return the same answer.
__device__ __forceinline__ bool start_barrier(uint32_t* const* flags, int rank, int world, int slot, uint32_t epoch,
                                              unsigned int* status, uint64_t limit_ns) {
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flag_at(flags[threadIdx.x], slot, 0, rank), epoch);
  }
  int ok = 1;
  if (threadIdx.x < world) ok = wait_epoch(flag_at(flags[rank], slot, 0, threadIdx.x), epoch, limit_ns) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (!ok && threadIdx.x == 0) atomicOr(status, RB_STATUS_PEER_TIMEOUT);
  return ok != 0;
}

// Called by every thread after its data movement. The last block to arrive tells every peer that this rank
// is done with the epoch and waits until every peer has said the same, so that when the kernel ends nobody
// still reads this rank's buffers and every store of a peer into this rank's memory has landed.
__device__ __forceinline__ void end_barrier(uint32_t* const* flags, int rank, int world, int slot, uint32_t epoch,
                                            unsigned int* block_counter, uint32_t* epoch_ptr, unsigned int* status,
                                            uint64_t limit_ns) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < world) st_release_sys(flag_at(flags[threadIdx.x], slot, 1, rank), epoch);
  int ok = 1;
  if (threadIdx.x < world) ok = wait_epoch(flag_at(flags[rank], slot, 1, threadIdx.x), epoch, limit_ns) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0) {
    if (!ok) atomicOr(status, RB_STATUS_PEER_TIMEOUT);
    *block_counter = 0u;
    *epoch_ptr = epoch;
    __threadfence();
  }
}

// Thread blocks are small (128 threads, <= 85 registers) on purpose: the kernels run on their own stream while the
// backward pass's GEMM CTAs (one per SM, most of the register file and all of the shared memory) are resident,
// and only a block this size fits beside them. With so few threads a design that PULLS gradients from peers is
// latency bound (a remote load takes ~2 us; 148 x 128 threads x 64 B in flight is ~0.5 TB/s at best and far less
// once the loads compete with local ones for registers), whereas remote STORES are posted and saturate the link
// from any grid. So the exchange is push based:
//   ar_push_kernel        rank r copies shard p of its gradients into slot r of peer p's staging buffer
//                         (local loads, remote stores), zeroes what it read, and raises phase-0 flags;
//   allreduce_sgd_kernel  waits for every peer's phase-0 flag, sums its own shard with the N-1 staged copies
//                         (all local loads), applies 1/N + SGD to its shard of master/momentum and stores the
//                         new bf16 weights into every peer (remote stores, or one multimem.st).
// With a multimem mapping of the gradient buffer the push is skipped and the second kernel fetches the sum with
// multimem.ld_reduce (the switch does the N-way read).
constexpr int AR_THREADS = 128;
constexpr int AR_SLOTS = 8;

__device__ __forceinline__ long long shard_len(long long n, int world) {
  long long per = (n + world - 1) / world;
  return (per + 7) / 8 * 8;
}

__global__ void __launch_bounds__(AR_THREADS, 6) ar_push_kernel(const __grid_constant__ ArSgdArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  // one-shot buckets: every rank reduces the whole bucket, and all of them must arrive at the same bits, so the
  // reducer sums the staged copies of ALL ranks in rank order -- the own copy is staged too (a local store)
  const int peers = a.one_shot ? a.world : a.world - 1;
  const long long per = a.one_shot ? a.n : shard_len(a.n, a.world);
  const uint32_t per4 = (uint32_t)(per / 4);
  const uint32_t total4 = per4 * (uint32_t)peers;
  const uint32_t gthreads = gridDim.x * blockDim.x;
  float* g = a.grads[a.rank] + a.off;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t base = blockIdx.x * blockDim.x + threadIdx.x; base < total4; base += gthreads * 4u) {
    float4 t[4];
    float* dstp[4];
    float* srcp[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t j = base + (uint32_t)u * gthreads;
      dstp[u] = nullptr;
      if (j < total4) {
        const uint32_t po = j / per4, k = j - po * per4;
        int peer = a.rank + 1 + (int)po;
        if (peer >= a.world) peer -= a.world;
        const long long si = (a.one_shot ? 0 : (long long)peer * per) + (long long)k * 4;
        if (si < a.n) {
          srcp[u] = g + si;
          t[u] = ld_f4(srcp[u]);
          dstp[u] = a.stage[peer] + a.stage_off + (long long)a.rank * per + (long long)k * 4;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (dstp[u]) {
        *reinterpret_cast<float4*>(dstp[u]) = t[u];
        // in one-shot mode the own copy is still needed by the reducing kernel, which zeroes it itself
        if (a.zero_grads && !a.one_shot) *reinterpret_cast<float4*>(srcp[u]) = zero;
      }
    }
  }
  // last block: every store of this rank into the peers' staging has been fenced; tell them
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < a.world) st_release_sys(flag_at(a.flags[threadIdx.x], a.slot, 0, a.rank), epoch);
    if (threadIdx.x == 0) {
      *a.block_counter = 0u;
      __threadfence();
    }
  }
}

__global__ void __launch_bounds__(AR_THREADS, 6) allreduce_sgd_kernel(const __grid_constant__ ArSgdArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  bool ready;
  if (a.wait_ok) {
    ready = *reinterpret_cast<volatile uint32_t*>(a.wait_ok) == epoch;
  } else if (a.mc_grads) {
    ready = start_barrier(a.flags, a.rank, a.world, a.slot, epoch, a.status, wait_limit(a.wait_ns));
  } else {
    int ok = 1;
    if (threadIdx.x < a.world)
      ok = wait_epoch(flag_at(a.flags[a.rank], a.slot, 0, threadIdx.x), epoch, wait_limit(a.wait_ns)) ? 1 : 0;
    ok = __syncthreads_and(ok);
    if (!ok && threadIdx.x == 0) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
    ready = ok != 0;
  }
  if (ready) {
    long long s0 = 0, s1 = a.n, per = a.n;
    if (!a.one_shot) {
      per = shard_len(a.n, a.world);
      s0 = min(a.n, (long long)a.rank * per);
      s1 = min(a.n, s0 + per);
    }
    const int peers = a.world - 1;
    const int U = (peers <= 3) ? 2 : 1;   // groups of 4 elements per thread and sweep: U * (3 + peers) loads in flight
    const long long gthreads = (long long)gridDim.x * blockDim.x;
    const long long sweep = gthreads * 4 * U;
    const long long tid4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const float* stage = a.stage[a.rank] + a.stage_off;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long base = s0; base < s1; base += sweep) {
      float4 ga[2], wa[2], va[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const long long i = base + (long long)u * gthreads * 4 + tid4;
        if (u < U && i < s1) {
          ga[u] = a.mc_grads ? mm_ld_reduce_f4(a.mc_grads + a.off + i) : ld_f4(a.grads[a.rank] + a.off + i);
          if (a.op == 0) {
            wa[u] = ld_f4(a.w + a.off + i);
            va[u] = ld_f4(a.v + a.off + i);
          }
        }
      }
      if (!a.mc_grads && peers > 0) {
        // staged copies of the peers, summed in a fixed order (run-to-run deterministic)
        float4 t[AR_SLOTS];
#pragma unroll
        for (int sl = 0; sl < AR_SLOTS; ++sl) {
          const int u = (peers <= 3) ? sl / 4 : 0, po = (peers <= 3) ? (sl & 3) : sl;
          const long long i = base + (long long)u * gthreads * 4 + tid4;
          t[sl] = zero;
          if (a.one_shot) {
            // slot = absolute rank (the own staged copy among them): the same operands in the same tree everywhere
            if (po < a.world && i < s1) t[sl] = ld_f4(stage + (long long)po * per + (i - s0));
          } else if (po < peers && i < s1) {
            int peer = a.rank + 1 + po;
            if (peer >= a.world) peer -= a.world;
            t[sl] = ld_f4(stage + (long long)peer * per + (i - s0));
          }
        }
        if (a.one_shot) {
          if (peers <= 3) {
            ga[0] = add4(add4(t[0], t[1]), add4(t[2], t[3]));
            ga[1] = add4(add4(t[4], t[5]), add4(t[6], t[7]));
          } else {
            ga[0] = add4(add4(add4(t[0], t[1]), add4(t[2], t[3])), add4(add4(t[4], t[5]), add4(t[6], t[7])));
          }
        } else if (peers <= 3) {
          ga[0] = add4(ga[0], add4(add4(t[0], t[1]), t[2]));
          ga[1] = add4(ga[1], add4(add4(t[4], t[5]), t[6]));
        } else {
          ga[0] = add4(ga[0], add4(add4(add4(t[0], t[1]), add4(t[2], t[3])), add4(add4(t[4], t[5]), t[6])));
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const long long i = base + (long long)u * gthreads * 4 + tid4;
        if (u >= U || i >= s1) continue;
        const long long e = a.off + i;
        float4 g = ga[u];
        if (a.op == 1) {
          // plain average, written back to every rank's buffer in place
          const float s = a.avg_scale;
          g = make_float4(g.x * s, g.y * s, g.z * s, g.w * s);
          if (a.mc_grads) {
            mm_st_f4(const_cast<float*>(a.mc_grads) + e, g);
          } else {
#pragma unroll
            for (int p = 0; p < MAX_RANKS; ++p)
              if (p < a.world) *reinterpret_cast<float4*>(a.grads[p] + e) = g;
          }
          continue;
        }
        if (a.zero_grads) *reinterpret_cast<float4*>(a.grads[a.rank] + e) = zero;
        SgdHyper h = a.h;
        if (e >= a.decay_len) h.l2 = 0.f;
        float4 w = wa[u], v = va[u];
        sgd_elem(w.x, g.x, v.x, h);
        sgd_elem(w.y, g.y, v.y, h);
        sgd_elem(w.z, g.z, v.z, h);
        sgd_elem(w.w, g.w, v.w, h);
        *reinterpret_cast<float4*>(a.w + e) = w;
        *reinterpret_cast<float4*>(a.v + e) = v;
        uint2 packed;
        {
          __nv_bfloat162 b0 = __floats2bfloat162_rn(w.x, w.y), b1 = __floats2bfloat162_rn(w.z, w.w);
          packed.x = *reinterpret_cast<uint32_t*>(&b0);
          packed.y = *reinterpret_cast<uint32_t*>(&b1);
        }
        if (a.one_shot) {
          *reinterpret_cast<uint2*>(a.w16[a.rank] + e) = packed;
        } else if (a.mc_w16) {
          asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(a.mc_w16 + e),
                       "f"(__uint_as_float(packed.x)), "f"(__uint_as_float(packed.y)) : "memory");
        } else {
#pragma unroll
          for (int p = 0; p < MAX_RANKS; ++p)
            if (p < a.world) *reinterpret_cast<uint2*>(a.w16[p] + e) = packed;
        }
        if (!a.one_shot && a.w32[0]) {
#pragma unroll
          for (int p = 0; p < MAX_RANKS; ++p)
            if (p < a.world && p != a.rank) *reinterpret_cast<float4*>(a.w32[p] + e) = w;
        }
      }
    }
  }
  end_barrier(a.flags, a.rank, a.world, a.slot, epoch, a.block_counter, a.epoch_ptr, a.status, wait_limit(a.wait_ns));
}

// The wait for the peers' phase-0 flags as a kernel of its own (one warp): the reducing kernel that follows in
// stream order then never spins, so its blocks do not sit on SMs that the backward pass's GEMM CTAs need.
// With a multimem gradient mapping there is no push kernel, so this kernel also announces the rank.
__global__ void ar_wait_kernel(const __grid_constant__ ArSgdArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  if (a.mc_grads && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(flag_at(a.flags[threadIdx.x], a.slot, 0, a.rank), epoch);
  }
  int ok = 1;
  if (threadIdx.x < a.world)
    ok = wait_epoch(flag_at(a.flags[a.rank], a.slot, 0, threadIdx.x), epoch, wait_limit(a.wait_ns)) ? 1 : 0;
  ok = __all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0) {
    if (!ok) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
    *a.wait_ok = ok ? epoch : 0u;
    __threadfence();
  }
}

// ------------------------------------------------------------------------------------------ gossip
struct MixArgs {
  uint32_t* flags[MAX_RANKS];
  float* w;               // local parameters (updated in place)
  bf16* w16;              // local bf16 copy (refreshed), may be null
  float* pub_local;       // local published snapshots: two buffers of `n` back to back
  const float* pub_peer;  // the peer's published snapshots (same layout), P2P address
  float* acc_target;      // push gossip: the target's accumulator (P2P) / own accumulator in finalize
  float* count_target;    // push gossip: the target's receive counter
  uint32_t* epoch_ptr;
  unsigned int* block_counter;
  unsigned int* status;
  long long n;
  int rank, world, slot, peer;
  int wait_peer;          // 1: wait until the peer has published this epoch (synchronous gossip)
  float alpha;            // mixing weight: x <- (1-alpha) x + alpha x_peer
  float w_self;           // push gossip: weight of the own vector
  int not_last;           // gossip mix: 1 = another pull of the same round follows (keep the epoch, do not report done)
  int mix_self;           // gossip mix: 1 = a pull that lands on this rank mixes with its own published snapshot
  long long wait_ns;      // limit of each wait on a peer, ns (0: the 3 s default)
  unsigned long long* gate;   // asynchronous push gossip: the target's (push) or the own (fold) gate word;
                              // asynchronous elastic averaging: the centre's lock word
  int* ticket;            // local: what the `begin` kernel of an asynchronous exchange decided for the kernel that follows
  unsigned int* skipped;  // local counter of exchanges given up because the centre stayed busy (may be null)
};

// pub[epoch & 1] <- w, then tell every peer that epoch is published. Before overwriting the buffer last used
// two epochs ago, wait until every peer has reported being done with that epoch.
__global__ void __launch_bounds__(512) publish_kernel(const __grid_constant__ MixArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  int ok = 1;
  // (only the lock-step form waits: an asynchronous publisher never waits for a peer; a puller that is two whole
  // exchanges late may then read a snapshot while it is being replaced, and mixes values of two consecutive ones)
  if (a.wait_peer && epoch > 2u && threadIdx.x < a.world && threadIdx.x != a.rank)
    ok = wait_epoch(flag_at(a.flags[a.rank], a.slot, 1, threadIdx.x), epoch - 2u, wait_limit(a.wait_ns)) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (!ok && threadIdx.x == 0) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
  float* dst = a.pub_local + (size_t)(epoch & 1u) * a.n;
  const long long n4 = a.n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(a.w)[i];
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < a.world) st_release_sys(flag_at(a.flags[threadIdx.x], a.slot, 0, a.rank), epoch);
    if (threadIdx.x == 0) *a.block_counter = 0u;  // epoch_ptr advances in the mix kernel that follows
  }
}

// x <- (1 - alpha) x + alpha x_peer, reading the peer's published snapshot of this epoch over NVLink.
__global__ void __launch_bounds__(512) gossip_mix_kernel(const __grid_constant__ MixArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  int ok = 1;
  if (a.wait_peer && a.peer != a.rank && threadIdx.x == 0)
    ok = wait_epoch(flag_at(a.flags[a.rank], a.slot, 0, a.peer), epoch, wait_limit(a.wait_ns)) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (!ok && threadIdx.x == 0) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
  // An asynchronous puller takes whichever snapshot the peer published last (nothing yet: no mixing). Blocks
  // sample the peer's epoch independently, so an asynchronous pull may combine two consecutive snapshots.
  __shared__ uint32_t s_pe;
  if (threadIdx.x == 0)
    s_pe = a.wait_peer ? epoch : ld_acquire_sys(flag_at(a.flags[a.rank], a.slot, 0, a.peer));
  __syncthreads();
  const uint32_t pe = s_pe;
  if (ok && (a.peer != a.rank || a.mix_self) && pe != 0u) {
    const float* src = a.pub_peer + (size_t)(pe & 1u) * a.n;
    const long long n4 = a.n / 4;
    const float al = a.alpha, be = 1.f - a.alpha;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
      const float4 p = ld_f4(src + i * 4);
      float4 x = reinterpret_cast<float4*>(a.w)[i];
      x = make_float4(be * x.x + al * p.x, be * x.y + al * p.y, be * x.z + al * p.z, be * x.w + al * p.w);
      reinterpret_cast<float4*>(a.w)[i] = x;
      if (a.w16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(a.w16)[i] = o;
      }
    }
  }
  // last block: report "done with this epoch" to every peer and advance the local epoch
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    if (!a.not_last && threadIdx.x < a.world) st_release_sys(flag_at(a.flags[threadIdx.x], a.slot, 1, a.rank), epoch);
    if (threadIdx.x == 0) {
      *a.block_counter = 0u;
      if (!a.not_last) *a.epoch_ptr = epoch;
    }
  }
}

// Push gossip, step 1: add this rank's published snapshot into the target's accumulator and count it.
__global__ void __launch_bounds__(512) push_add_kernel(const __grid_constant__ MixArgs a) {
  const long long n4 = a.n / 4;
  if (a.peer != a.rank) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
      const float4 x = reinterpret_cast<const float4*>(a.w)[i];
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.acc_target + i * 4), "f"(x.x), "f"(x.y),
                   "f"(x.z), "f"(x.w) : "memory");
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(a.count_target, 1.f);
  }
}

// Push gossip, step 2 (after a barrier): x <- (w_self x + acc) / (w_self + count); accumulator cleared.
__global__ void __launch_bounds__(512) push_finalize_kernel(const __grid_constant__ MixArgs a) {
  const float cnt = *reinterpret_cast<volatile float*>(a.count_target);
  const float inv = 1.f / (a.w_self + cnt);
  const long long n4 = a.n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 x = reinterpret_cast<float4*>(a.w)[i];
    const float4 s = reinterpret_cast<float4*>(a.acc_target)[i];
    if (cnt > 0.f) {
      x = make_float4((a.w_self * x.x + s.x) * inv, (a.w_self * x.y + s.y) * inv, (a.w_self * x.z + s.z) * inv,
                      (a.w_self * x.w + s.w) * inv);
      reinterpret_cast<float4*>(a.w)[i] = x;
      reinterpret_cast<float4*>(a.acc_target)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.w16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(a.w16)[i] = o;
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    *a.count_target = 0.f;
    *a.block_counter = 0u;
  }
}

// Elastic averaging, client side: read the centre (rank 0's memory), move toward it, and add the opposite
// pull into the centre's delta accumulator:  x <- x - beta (x - c) ;  delta_centre += beta (x - c).
__global__ void __launch_bounds__(512) elastic_pull_kernel(const __grid_constant__ MixArgs a) {
  const long long n4 = a.n / 4;
  const float be = a.alpha;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 c = ld_f4(a.pub_peer + i * 4);
    float4 x = reinterpret_cast<float4*>(a.w)[i];
    const float4 d = make_float4(be * (x.x - c.x), be * (x.y - c.y), be * (x.z - c.z), be * (x.w - c.w));
    x = make_float4(x.x - d.x, x.y - d.y, x.z - d.z, x.w - d.w);
    reinterpret_cast<float4*>(a.w)[i] = x;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.acc_target + i * 4), "f"(d.x), "f"(d.y),
                 "f"(d.z), "f"(d.w) : "memory");
    if (a.w16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(a.w16)[i] = o;
    }
  }
}

// Elastic averaging, centre side (rank 0): centre += delta ; delta = 0.
__global__ void elastic_apply_kernel(float* __restrict__ center, float* __restrict__ delta, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    center[i] += delta[i];
    delta[i] = 0.f;
  }
}


// --------------------------------------------------------------------------- asynchronous push gossip
// The reference's asynchronous push gossip (src/worker/gossip_dist.rs:474-593 passive receiver, :883-976 active
// side) has no barrier anywhere: a rank sends its vector to a random target whenever it gets there; a receiver
// thread on the target accumulates whole vectors as they arrive and counts them; at its own exchange a rank pauses
// its receiver, keeps (w_self x + received) / (w_self + count) -- or its own x when nothing arrived -- and
// resumes. Ranks may be any number of iterations apart.
//
// Here the receiver thread is the target's memory: every rank owns two accumulators acc[0], acc[1] with a count
// each, and a 64-bit gate word  [ epoch : 32 | pushes in flight into acc[1] : 16 | into acc[0] : 16 ].
//   push_begin (one thread)   registers at the TARGET's gate with a compare-and-swap: reads the epoch, adds one to
//                             the in-flight field of acc[epoch & 1]; the buffer index goes to the local ticket
//   push_add   (grid)         red.add of the own vector into the target's acc[ticket] over NVLink; the last block
//                             fences, adds 1 to that accumulator's count and takes the registration off the gate
//   fold_begin (one thread)   adds 1 to the OWN gate's epoch (later pushes go to the other accumulator), then waits
//                             -- bounded -- until the pushes still in flight into the closed accumulator are done:
//                             a wait for transfers already under way, never for another rank to reach a round
//   fold       (grid)         x <- (w_self x + acc[closed]) / (w_self + count[closed]) if count > 0; clears both
// A push that registers after the epoch moved lands in the other accumulator and is folded one exchange later,
// which is what a late message does in the reference.
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long atom_cas_sys_u64(unsigned long long* p, unsigned long long cmp,
                                                               unsigned long long val) {
  unsigned long long old;
  asm volatile("atom.acq_rel.sys.global.cas.b64 %0, [%1], %2, %3;" : "=l"(old) : "l"(p), "l"(cmp), "l"(val) : "memory");
  return old;
}
__device__ __forceinline__ unsigned long long atom_add_sys_u64(unsigned long long* p, unsigned long long val) {
  unsigned long long old;
  asm volatile("atom.acq_rel.sys.global.add.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(val) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_sys_f4(float* p, float4 x) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x.x), "f"(x.y), "f"(x.z),
               "f"(x.w) : "memory");
}
constexpr int GATE_CAS_TRIES = 4096;

// ticket: 0 / 1 = accumulator to push into, -1 = nothing to push (target is this rank, or registration failed)
__global__ void push_begin_kernel(const __grid_constant__ MixArgs a) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int buf = -1;
  if (a.peer != a.rank) {
    unsigned long long seen = ld_acquire_sys_u64(a.gate);
    for (int t = 0; t < GATE_CAS_TRIES; ++t) {
      const int b = (int)((seen >> 32) & 1ull);
      const unsigned long long want = seen + (1ull << (16 * b));
      const unsigned long long old = atom_cas_sys_u64(a.gate, seen, want);
      if (old == seen) { buf = b; break; }
      seen = old;
    }
    if (buf < 0) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);   // the gate changed under every one of the tries
  }
  *a.ticket = buf;
  __threadfence();
}

__global__ void __launch_bounds__(512) push_add_async_kernel(const __grid_constant__ MixArgs a) {
  const int buf = *reinterpret_cast<volatile int*>(a.ticket);
  if (buf < 0) return;
  float* acc = a.acc_target + (size_t)buf * a.n;
  const long long n4 = a.n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x)
    red_add_sys_f4(acc + i * 4, reinterpret_cast<const float4*>(a.w)[i]);
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.f32 [%0], %1;" ::"l"(a.count_target + buf), "f"(1.f) : "memory");
    atom_add_sys_u64(a.gate, 0ull - (1ull << (16 * buf)));   // the registration comes off after the count is in
    *a.block_counter = 0u;
    __threadfence();
  }
}

// ticket: 0 / 1 = accumulator that was closed and is safe to fold, -1 = a push into it never finished (not folded)
__global__ void fold_begin_kernel(const __grid_constant__ MixArgs a) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const unsigned long long old = atom_add_sys_u64(a.gate, 1ull << 32);
  const int closed = (int)((old >> 32) & 1ull);
  const uint64_t limit = wait_limit(a.wait_ns), t0 = globaltimer_ns();
  bool ok = true;
  uint32_t spins = 0;
  while (((ld_acquire_sys_u64(a.gate) >> (16 * closed)) & 0xffffull) != 0ull) {
    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > limit) { ok = false; break; }
  }
  if (!ok) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
  *a.ticket = ok ? closed : -1;
  __threadfence();
}

__global__ void __launch_bounds__(512) fold_kernel(const __grid_constant__ MixArgs a) {
  const int buf = *reinterpret_cast<volatile int*>(a.ticket);
  const float cnt = buf >= 0 ? *reinterpret_cast<volatile float*>(a.count_target + buf) : 0.f;
  if (cnt > 0.f) {
    float* acc = a.acc_target + (size_t)buf * a.n;
    const float inv = 1.f / (a.w_self + cnt), ws = a.w_self;
    const long long n4 = a.n / 4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
      float4 x = reinterpret_cast<float4*>(a.w)[i];
      const float4 s = reinterpret_cast<float4*>(acc)[i];
      x = make_float4((ws * x.x + s.x) * inv, (ws * x.y + s.y) * inv, (ws * x.z + s.z) * inv, (ws * x.w + s.w) * inv);
      reinterpret_cast<float4*>(a.w)[i] = x;
      reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a.w16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(a.w16)[i] = o;
      }
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    if (buf >= 0) a.count_target[buf] = 0.f;
    *a.block_counter = 0u;
    __threadfence();
  }
}

// ------------------------------------------------------------------- asynchronous elastic averaging
// The reference's parameter server serves one client at a time, each with the centre as it is at that moment, and
// clients may be any number of iterations apart (src/worker/elasticserver_dist.rs:249-255,667-715); its one-sided
// form guards the centre with a compare-and-swap state word (src/worker/elasticserver_dist_rdma.rs:74-104,565-649).
// Here the centre lives in rank 0's memory with a lock word beside it:
//   elastic_begin (one thread)  compare-and-swap 0 -> rank + 1 on the centre's lock, retried for at most `wait_ns`;
//                               a client that does not get the lock in time gives this exchange up (counted in
//                               `skipped`, no error: the centre was busy) -- ticket 1 = locked, 0 = skipped
//   elastic_mix   (grid)        with the lock: c = centre (peer loads); d = beta (x - c); x <- x - d;
//                               centre <- c + d (peer stores); the last block fences and releases the lock
__global__ void elastic_begin_kernel(const __grid_constant__ MixArgs a) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const unsigned long long mine = (unsigned long long)(a.rank + 1);
  const uint64_t limit = wait_limit(a.wait_ns), t0 = globaltimer_ns();
  int got = 0;
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_sys_u64(a.gate) == 0ull && atom_cas_sys_u64(a.gate, 0ull, mine) == 0ull) { got = 1; break; }
    if ((++spins & 15u) == 0u && globaltimer_ns() - t0 > limit) break;
  }
  if (!got && a.skipped) atomicAdd(a.skipped, 1u);
  *a.ticket = got;
  __threadfence();
}

__global__ void __launch_bounds__(512) elastic_mix_kernel(const __grid_constant__ MixArgs a) {
  if (*reinterpret_cast<volatile int*>(a.ticket) != 1) return;
  const long long n4 = a.n / 4;
  const float be = a.alpha;
  float* center = const_cast<float*>(a.pub_peer);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 c = ld_f4(center + i * 4);
    float4 x = reinterpret_cast<float4*>(a.w)[i];
    const float4 d = make_float4(be * (x.x - c.x), be * (x.y - c.y), be * (x.z - c.z), be * (x.w - c.w));
    x = make_float4(x.x - d.x, x.y - d.y, x.z - d.z, x.w - d.w);
    reinterpret_cast<float4*>(a.w)[i] = x;
    *reinterpret_cast<float4*>(center + i * 4) = make_float4(c.x + d.x, c.y + d.y, c.z + d.z, c.w + d.w);
    if (a.w16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(a.w16)[i] = o;
    }
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.gate), "l"(0ull) : "memory");   // unlock
    *a.block_counter = 0u;
    __threadfence();
  }
}

// Cross-GPU barrier as a kernel of one block (orders the kernels before it on every rank's stream against
// the kernels after it on every other rank's stream).
struct BarrierArgs {
  uint32_t* flags[MAX_RANKS];
  uint32_t* epoch_ptr;
  unsigned int* status;
  int rank, world, slot;
  long long wait_ns;     // limit of the wait for the peers, ns (0: the 3 s default)
};
__global__ void barrier_kernel(const __grid_constant__ BarrierArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  __threadfence_system();
  if (threadIdx.x < a.world) st_release_sys(flag_at(a.flags[threadIdx.x], a.slot, 0, a.rank), epoch);
  int ok = 1;
  if (threadIdx.x < a.world)
    ok = wait_epoch(flag_at(a.flags[a.rank], a.slot, 0, threadIdx.x), epoch, wait_limit(a.wait_ns)) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0) {
    if (!ok) atomicOr(a.status, RB_STATUS_PEER_TIMEOUT);
    *a.epoch_ptr = epoch;
  }
}


// Link probe: what one direction of the NVLink fabric gives to SM-issued traffic, as a function of how many
// 16-byte accesses each thread keeps in flight. mode 0 = load from `src` (sum kept in a register), 1 = store a
// constant to `dst`, 2 = copy src -> dst. Which of the two pointers is a peer's memory is the caller's choice.
template <int UNROLL>
__global__ void __launch_bounds__(512) link_probe_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                         float* __restrict__ sink, long long n4, int mode) {
  const long long gthreads = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long base = tid; base < n4; base += gthreads * UNROLL) {
    float4 t[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = base + (long long)u * gthreads;
      if (mode != 1 && i < n4) t[u] = ld_f4(src + i * 4);
      else t[u] = make_float4(1.f, 2.f, 3.f, 4.f);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = base + (long long)u * gthreads;
      if (i >= n4) continue;
      if (mode == 0) acc = add4(acc, t[u]);
      else *reinterpret_cast<float4*>(dst + i * 4) = t[u];
    }
  }
  if (mode == 0 && acc.x + acc.y + acc.z + acc.w == 1.2345e-30f) sink[0] = acc.x;
}

}  // namespace rb

using namespace rb;

extern "C" {

// Host-side mirror of ArSgdArgs with plain pointers (filled through ctypes).
int rb_allreduce_sgd_p2p(const void* args, int blocks, cudaStream_t st) {
  const ArSgdArgs* a = reinterpret_cast<const ArSgdArgs*>(args);
  if (a->world < 1 || a->world > MAX_RANKS || (a->n % 8) || (a->off % 8)) return -10;
  if (blocks < 1) blocks = 1;
  if (!a->mc_grads && a->world > 1 && !a->stage[a->rank]) return -11;
  allreduce_sgd_kernel<<<blocks, AR_THREADS, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_allreduce_wait_p2p(const void* args, cudaStream_t st) {
  const ArSgdArgs* a = reinterpret_cast<const ArSgdArgs*>(args);
  if (a->world < 1 || a->world > MAX_RANKS || !a->wait_ok) return -10;
  ar_wait_kernel<<<1, 32, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

// First half of the push-based exchange (not needed with a multimem gradient mapping or on one rank).
int rb_allreduce_push_p2p(const void* args, int blocks, cudaStream_t st) {
  const ArSgdArgs* a = reinterpret_cast<const ArSgdArgs*>(args);
  if (a->world < 2 || a->world > MAX_RANKS || (a->n % 8) || (a->off % 8) || (a->stage_off % 4)) return -10;
  if (!a->stage[a->rank] || a->n / 4 * (a->world - 1) >= (1ll << 31)) return -11;
  if (blocks < 1) blocks = 1;
  ar_push_kernel<<<blocks, AR_THREADS, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_publish_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4) return -10;
  publish_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_gossip_mix_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4) return -10;
  gossip_mix_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_push_add_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4) return -10;
  push_add_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_push_finalize(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4) return -10;
  push_finalize_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_elastic_pull_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4) return -10;
  elastic_pull_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_elastic_apply(float* center, float* delta, long long n, cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  elastic_apply_kernel<<<(int)blocks, 256, 0, st>>>(center, delta, n);
  return RB_LAUNCH_OK();
}

int rb_push_begin_p2p(const void* args, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (!a->ticket || (a->peer != a->rank && !a->gate)) return -10;
  push_begin_kernel<<<1, 32, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_push_add_async_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4 || !a->ticket) return -10;
  push_add_async_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_fold_begin_p2p(const void* args, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (!a->ticket || !a->gate) return -10;
  fold_begin_kernel<<<1, 32, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_fold_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4 || !a->ticket) return -10;
  fold_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_elastic_begin_p2p(const void* args, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (!a->ticket || !a->gate) return -10;
  elastic_begin_kernel<<<1, 32, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_elastic_mix_p2p(const void* args, int blocks, cudaStream_t st) {
  const MixArgs* a = reinterpret_cast<const MixArgs*>(args);
  if (a->n % 4 || !a->ticket || !a->gate) return -10;
  elastic_mix_kernel<<<blocks < 1 ? 1 : blocks, 512, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_barrier_p2p(const void* args, cudaStream_t st) {
  const BarrierArgs* a = reinterpret_cast<const BarrierArgs*>(args);
  barrier_kernel<<<1, 32, 0, st>>>(*a);
  return RB_LAUNCH_OK();
}

int rb_link_probe(const float* src, float* dst, float* sink, long long n, int mode, int unroll, int blocks,
                  int threads, cudaStream_t st) {
  if (n % 4 || threads < 32 || threads > 512 || blocks < 1 || mode < 0 || mode > 2) return -10;
  const long long n4 = n / 4;
  switch (unroll) {
    case 1: link_probe_kernel<1><<<blocks, threads, 0, st>>>(src, dst, sink, n4, mode); break;
    case 2: link_probe_kernel<2><<<blocks, threads, 0, st>>>(src, dst, sink, n4, mode); break;
    case 4: link_probe_kernel<4><<<blocks, threads, 0, st>>>(src, dst, sink, n4, mode); break;
    case 8: link_probe_kernel<8><<<blocks, threads, 0, st>>>(src, dst, sink, n4, mode); break;
    case 16: link_probe_kernel<16><<<blocks, threads, 0, st>>>(src, dst, sink, n4, mode); break;
    default: return -10;
  }
  return RB_LAUNCH_OK();
}

}  // extern "C"
