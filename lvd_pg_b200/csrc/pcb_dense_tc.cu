// pcb_dense_tc.cu — dense sum blocks on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// The three contractions of a dense block (see pcb_dense.cu for the algebra)
//   FWD        D[b][r] = sum_t A[b][t] * W[r][t]          A = exp(M - mx),  W = exp(theta)
//   BWD_CHILD  D[b][t] = sum_r G[b][r] * W[r][t]          G = flows * exp(mx - mars)
//   BWD_EDGE   D[r][t] = sum_b G[b][r] * A[b][t]
// run as 128 x N x K tiles (N <= 256) with fp32 accumulators in tensor memory.  Operands are
// produced in the kernel: eight producer warps read the fp32 work matrices, apply the exp /
// rescale, split every value into a TF32 "hi" part (top 19 bits) and the exact fp32 remainder
// "lo", and write both into shared memory in the K-major 128-byte-swizzled layout the tensor
// core reads.  One elected thread issues three tcgen05.mma per 8-deep K step
// (hi*hi + lo*hi + hi*lo; the lo*lo term is below 2^-20 relative), so results carry fp32-class
// accuracy (about 2^-20 relative per product) while the multiply-accumulates run on the tensor
// pipe.  The epilogue warps read the accumulators with tcgen05.ld and apply log / rescale /
// the statistics update, writing rows that are contiguous in the example index.
//
// Synchronisation: a two-stage ring of shared-memory tiles guarded by mbarriers
// (full: 256 producer arrivals, empty: one tcgen05.commit), one more mbarrier for "accumulator
// complete".  Every wait is bounded; on expiry the thread raises the circuit's status word,
// leaves its loop and still reaches the common exit where tensor memory is released.
#include <algorithm>

#include "pcb_internal.h"

namespace {

enum { MODE_FWD = 0, MODE_BWD_CHILD = 1, MODE_BWD_EDGE = 2 };

constexpr uint32_t TM = 128;         // tile rows (TMEM lanes)
constexpr uint32_t TN_MAX = 256;     // tile columns
constexpr uint32_t KCH = 32;         // K elements per stage (one 128-byte swizzle row of tf32)
constexpr uint32_t STAGES = 2;
constexpr uint32_t NPROD = 256;      // producer threads (warps 0..7)
constexpr uint32_t NTHREADS = NPROD + 32;
constexpr uint32_t A_BYTES = TM * 128;        // one A sub-tile (hi or lo)
constexpr uint32_t B_BYTES = TN_MAX * 128;    // one B sub-tile (hi or lo)
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 2048 /*barriers, mx*/;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait: false (and status raised) when the phase did not complete in time
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(100);
  }
  atomicExch(status, 1);
  return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);          // start address
  d |= (uint64_t)0 << 16;                                // leading byte offset (unused, swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;                     // stride byte offset
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
  return d;
}
// instruction descriptor: D fp32, A/B tf32, both K-major, M x N
__device__ __forceinline__ uint32_t make_idesc(uint32_t m, uint32_t n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// byte offset of element (row, kk) inside a K-major SWIZZLE_128B tile of tf32
__device__ __forceinline__ uint32_t sw_off(uint32_t row, uint32_t kk) {
  return row * 128u + ((((kk >> 2) ^ (row & 7u)) << 4) | ((kk & 3u) << 2));
}
__device__ __forceinline__ void put_split(uint8_t* hi, uint8_t* lo, uint32_t off, float v) {
  float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
  *reinterpret_cast<float*>(hi + off) = h;
  *reinterpret_cast<float*>(lo + off) = v - h;
}

struct TcArgs {
  float* mars;
  float* flows;
  float* blk_mx;
  float* aggr;
  const float* theta;
  const PcbDenseBlock* blocks;
  int* status;
  uint32_t ld, B, b_per_cta;
};

__device__ __forceinline__ float child_val(const float* __restrict__ mars, uint32_t ld, const PcbDenseBlock& k,
                                           uint32_t t, uint32_t b) {
  float v = mars[(size_t)(k.c0 + t) * ld + b];
  if (k.d0 != PCB_NONE) v += mars[(size_t)(k.d0 + t) * ld + b];
  return v;
}

// grid: FWD / BWD_CHILD (example tiles of 128, column tiles of 256, blocks)
//       BWD_EDGE        (example slices, row tiles x column tiles, blocks)
template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 1) dense_tc_kernel(TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctl = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);          // [STAGES]
  uint64_t* empty = full + STAGES;                            // [STAGES]
  uint64_t* accfull = empty + STAGES;                         // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);
  float* mxs = reinterpret_cast<float*>(ctl + 128);           // [128] (+ [128] scratch)

  const PcbDenseBlock k = a.blocks[blockIdx.z];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ld = a.ld;

  // ---- tile coordinates ---------------------------------------------------------------------
  uint32_t m0, n0, n_count, k_begin, k_end;  // rows [m0, m0+128), columns [n0, n0+n_count), K range
  if (MODE == MODE_FWD) {
    m0 = blockIdx.x * TM; n0 = blockIdx.y * TN_MAX;
    if (n0 >= k.R) return;
    n_count = min(TN_MAX, k.R - n0); k_begin = 0; k_end = k.K;
  } else if (MODE == MODE_BWD_CHILD) {
    m0 = blockIdx.x * TM; n0 = blockIdx.y * TN_MAX;
    if (n0 >= k.K) return;
    n_count = min(TN_MAX, k.K - n0); k_begin = 0; k_end = k.R;
  } else {
    const uint32_t tiles_n = (k.K + TN_MAX - 1) / TN_MAX;
    m0 = (blockIdx.y / tiles_n) * TM; n0 = (blockIdx.y % tiles_n) * TN_MAX;
    if (m0 >= k.R) return;
    n_count = min(TN_MAX, k.K - n0);
    k_begin = blockIdx.x * a.b_per_cta; k_end = min(a.B, k_begin + a.b_per_cta);
    if (k_begin >= k_end) return;
  }
  const uint32_t n_tile = (n_count + 15u) & ~15u;           // UMMA N: multiple of 16
  const uint32_t nchunks = (k_end - k_begin + KCH - 1) / KCH;
  const float* mxrow = a.blk_mx + (size_t)k.mx_row * ld;

  // ---- set-up: barriers, tensor memory, per-example max --------------------------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) { mbar_init(&full[s], NPROD); mbar_init(&empty[s], 1); }
    mbar_init(accfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (MODE == MODE_FWD) {
    if (tid < NPROD) {  // max over the K children of the tile's 128 examples, two threads per example
      uint32_t bl = tid & 127, half = tid >> 7, b = m0 + bl;
      float mx = -INFINITY;
      if (b < ld) {
        uint32_t t = half;
        for (; t + 14 < k.K; t += 16) {  // eight independent loads per round
          float v[8];
#pragma unroll
          for (uint32_t u = 0; u < 8; ++u) v[u] = child_val(a.mars, ld, k, t + 2 * u, b);
#pragma unroll
          for (uint32_t u = 0; u < 8; ++u) mx = fmaxf(mx, v[u]);
        }
        for (; t < k.K; t += 2) mx = fmaxf(mx, child_val(a.mars, ld, k, t, b));
      }
      mxs[half * 128 + bl] = mx;
    }
  } else if (MODE == MODE_BWD_CHILD) {
    if (tid < 128) mxs[tid] = (m0 + tid < ld) ? mxrow[m0 + tid] : -INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (MODE == MODE_FWD) {
    if (tid < 128) {
      float mx = fmaxf(mxs[tid], mxs[128 + tid]);
      mxs[tid] = mx;
      if (blockIdx.y == 0 && m0 + tid < ld) a.blk_mx[(size_t)k.mx_row * ld + m0 + tid] = mx;
    }
    __syncthreads();
  }
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp < 8) {
    // =========================== producers ===================================================
    // Each chunk is produced in two phases so that the global loads of a whole chunk are in
    // flight together (and overlap the wait for the stage to drain): (1) raw loads into
    // registers, (2) exp / rescale / split and the swizzled shared-memory stores.
    const uint32_t nq = n_tile / 8;  // B rows per thread in the K-contiguous pattern
    for (uint32_t i = 0; i < nchunks && ok; ++i) {
      const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
      const uint32_t kc = k_begin + i * KCH;  // first K index of the chunk
      float ra[16], rm[16], rb[32];
      float mx = 0.0f;
      bool vok = false;
      // ---- phase 1: loads ----
      if (MODE == MODE_FWD) {
        const uint32_t row = tid & 127, b = m0 + row;
        mx = mxs[row];
        vok = b < ld && mx != -INFINITY;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q) {  // A[m = example][kk = child]: rows contiguous in the source
          uint32_t t = kc + (tid >> 7) * 16 + q;
          ra[q] = (vok && t < k_end) ? child_val(a.mars, ld, k, t, b) : -INFINITY;
        }
        const uint32_t t = kc + (tid & 31);
#pragma unroll
        for (uint32_t q = 0; q < 32; ++q) {  // B[n = parent][kk = child]: K contiguous in the source
          uint32_t r = n0 + (tid >> 5) + 8 * q;
          rb[q] = (q < nq && r < k.R && t < k_end) ? __ldg(a.theta + k.pid0 + (size_t)r * k.K + t) : -INFINITY;
        }
      } else if (MODE == MODE_BWD_CHILD) {
        const uint32_t row = tid & 127, b = m0 + row;
        mx = mxs[row];
        vok = b < ld && mx != -INFINITY;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q) {  // A[m = example][kk = parent] = G
          uint32_t r = kc + (tid >> 7) * 16 + q;
          bool e = vok && r < k_end;
          size_t o = (size_t)(k.p0 + (e ? r : 0)) * ld + (e ? b : 0);
          ra[q] = e ? a.flows[o] : 0.0f;
          rm[q] = e ? a.mars[o] : 0.0f;
        }
        const uint32_t t = n0 + tid;
#pragma unroll
        for (uint32_t kk = 0; kk < 32; ++kk) {  // B[n = child][kk = parent] = W[r][t]: rows contiguous
          uint32_t r = kc + kk;
          rb[kk] = (tid < n_tile && t < k.K && r < k_end) ? __ldg(a.theta + k.pid0 + (size_t)r * k.K + t) : -INFINITY;
        }
      } else {
        const uint32_t b = kc + (tid & 31);
        mx = b < k_end ? mxrow[b] : -INFINITY;
        vok = b < k_end && mx != -INFINITY;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q) {  // A[m = parent][kk = example] = G: K contiguous
          uint32_t r = m0 + (tid >> 5) + 8 * q;
          bool e = vok && r < k.R;
          size_t o = (size_t)(k.p0 + (e ? r : 0)) * ld + (e ? b : 0);
          ra[q] = e ? a.flows[o] : 0.0f;
          rm[q] = e ? a.mars[o] : 0.0f;
        }
#pragma unroll
        for (uint32_t q = 0; q < 32; ++q) {  // B[n = child][kk = example] = exp(M - mx)
          uint32_t t = n0 + (tid >> 5) + 8 * q;
          rb[q] = (q < nq && vok && t < k.K) ? child_val(a.mars, ld, k, t, b) : -INFINITY;
        }
      }
      // ---- wait for the stage, then phase 2: transform + store ----
      ok = mbar_wait(&empty[s], ph ^ 1u, a.status);
      if (!ok) break;
      uint8_t* a_hi = smem + s * STAGE_BYTES;
      uint8_t* a_lo = a_hi + A_BYTES;
      uint8_t* b_hi = a_lo + A_BYTES;
      uint8_t* b_lo = b_hi + B_BYTES;
      if (MODE == MODE_FWD) {
        const uint32_t row = tid & 127;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q)
          put_split(a_hi, a_lo, sw_off(row, (tid >> 7) * 16 + q), vok ? __expf(ra[q] - mx) : 0.0f);
#pragma unroll
        for (uint32_t q = 0; q < 32; ++q)
          if (q < nq) put_split(b_hi, b_lo, sw_off((tid >> 5) + 8 * q, tid & 31), __expf(rb[q]));
      } else if (MODE == MODE_BWD_CHILD) {
        const uint32_t row = tid & 127;
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q)
          put_split(a_hi, a_lo, sw_off(row, (tid >> 7) * 16 + q), vok ? ra[q] * __expf(mx - rm[q]) : 0.0f);
        if (tid < n_tile) {
#pragma unroll
          for (uint32_t kk = 0; kk < 32; ++kk) put_split(b_hi, b_lo, sw_off(tid, kk), __expf(rb[kk]));
        }
      } else {
#pragma unroll
        for (uint32_t q = 0; q < 16; ++q)
          put_split(a_hi, a_lo, sw_off((tid >> 5) + 8 * q, tid & 31), vok ? ra[q] * __expf(mx - rm[q]) : 0.0f);
#pragma unroll
        for (uint32_t q = 0; q < 32; ++q)
          if (q < nq) put_split(b_hi, b_lo, sw_off((tid >> 5) + 8 * q, tid & 31), vok ? __expf(rb[q] - mx) : 0.0f);
      }
      fence_proxy_async();   // make the generic-proxy writes visible to the tensor core
      mbar_arrive(&full[s]);
    }

    // =========================== epilogue ====================================================
    if (ok) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t q4 = warp & 3, half = warp >> 2;
      const uint32_t row = q4 * 32 + lane;
      const uint32_t c_begin = half * (TN_MAX / 2), c_end = min(n_tile, c_begin + TN_MAX / 2);
      float acc[32];
      for (uint32_t c0 = c_begin; c0 < c_end; c0 += 32) {
        tmem_ld32(tmem_base + ((q4 * 32u) << 16) + c0, acc);
        if (MODE == MODE_FWD) {
          uint32_t b = m0 + row;
          float mx = mxs[row];
          if (b < ld) {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              uint32_t r = n0 + c0 + j;
              if (r < k.R) a.mars[(size_t)(k.p0 + r) * ld + b] = mx == -INFINITY ? -INFINITY : __logf(acc[j]) + mx;
            }
          }
        } else if (MODE == MODE_BWD_CHILD) {
          uint32_t b = m0 + row;
          float mx = mxs[row];
          if (b < ld) {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              uint32_t t = n0 + c0 + j;
              if (t < k.K) {
                float av = mx == -INFINITY ? 0.0f : __expf(child_val(a.mars, ld, k, t, b) - mx);
                float f = acc[j] * av;
                a.flows[(size_t)(k.c0 + t) * ld + b] = f;
                if (k.d0 != PCB_NONE) a.flows[(size_t)(k.d0 + t) * ld + b] = f;
              }
            }
          }
        } else {
          uint32_t r = m0 + row;
          if (r < k.R) {
            const bool whole = gridDim.x == 1;
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              uint32_t t = n0 + c0 + j;
              if (t < k.K) {
                size_t p = k.pid0 + (size_t)r * k.K + t;
                float v = __expf(__ldg(a.theta + p)) * acc[j];
                if (whole) a.aggr[p] += v; else atomicAdd(a.aggr + p, v);
              }
            }
          }
        }
      }
    }
  } else {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc(TM, n_tile);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
        ok = mbar_wait(&full[s], ph, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t d_ahi = make_desc(sa), d_alo = make_desc(sa + A_BYTES);
        const uint64_t d_bhi = make_desc(sa + 2 * A_BYTES), d_blo = make_desc(sa + 2 * A_BYTES + B_BYTES);
#pragma unroll
        for (uint32_t ks = 0; ks < KCH / 8; ++ks) {
          const uint64_t adv = (uint64_t)((ks * 32u) >> 4);  // 8 tf32 = 32 bytes along K
          umma_tf32(tmem_base, d_ahi + adv, d_bhi + adv, idesc, (i | ks) ? 1u : 0u);
          umma_tf32(tmem_base, d_alo + adv, d_bhi + adv, idesc, 1u);
          umma_tf32(tmem_base, d_ahi + adv, d_blo + adv, idesc, 1u);
        }
        umma_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
      }
      if (ok) umma_commit(accfull);
    }
    __syncwarp();
  }

  // ---- common exit: release tensor memory ---------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int MODE>
int32_t launch(dim3 grid, const TcArgs& args, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    PCB_CUDA(cudaFuncSetAttribute(dense_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured = true;
  }
  dense_tc_kernel<MODE><<<grid, NTHREADS, SMEM_BYTES, st>>>(args);
  return PCB_OK;
}

}  // namespace

#define PCB_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != PCB_OK) return _s;   \
  } while (0)

int32_t pcb_dense_tc_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  TcArgs args{ws->mars, ws->flows, ws->blk_mx, c->aggr, c->theta, c->dense + o0, c->status, ws->ld, ws->B, 0};
  dim3 grid((pcb_round_up(ws->B, 32) + TM - 1) / TM, (c->max_dense_R + TN_MAX - 1) / TN_MAX, o1 - o0);
  PcbProfScope ps(c, st, PCB_K_DENSE_FWD);
  return launch<MODE_FWD>(grid, args, st);
}

int32_t pcb_dense_tc_backward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  TcArgs args{ws->mars, ws->flows, ws->blk_mx, c->aggr, c->theta, c->dense + o0, c->status, ws->ld, ws->B, 0};
  {
    dim3 grid((pcb_round_up(ws->B, 32) + TM - 1) / TM, (c->max_dense_K + TN_MAX - 1) / TN_MAX, o1 - o0);
    PcbProfScope ps(c, st, PCB_K_DENSE_BWD_CHILD);
    PCB_TRY(launch<MODE_BWD_CHILD>(grid, args, st));
  }
  {
    uint32_t tiles = ((c->max_dense_R + TM - 1) / TM) * ((c->max_dense_K + TN_MAX - 1) / TN_MAX);
    // slice the examples so that small layers still fill the GPU
    uint32_t want = std::max(1u, 148u / std::max(1u, tiles * (o1 - o0)));
    uint32_t slices = std::min(want, (ws->B + 255) / 256);
    uint32_t b_per = pcb_round_up((ws->B + slices - 1) / slices, KCH);
    slices = (ws->B + b_per - 1) / b_per;
    args.b_per_cta = b_per;
    dim3 grid(slices, tiles, o1 - o0);
    PcbProfScope ps(c, st, PCB_K_DENSE_BWD_EDGE);
    PCB_TRY(launch<MODE_BWD_EDGE>(grid, args, st));
  }
  return PCB_OK;
}
