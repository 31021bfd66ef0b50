// pcb_dense_tc.cu — dense sum blocks on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// The three contractions of a dense block (see pcb_dense.cu for the algebra)
//   FWD        D[b][r] = sum_t A[b][t] * W[r][t]          A = exp(M - mx),  W = exp(theta)
//   BWD_CHILD  D[b][t] = sum_r G[b][r] * W[r][t]          G = flows * exp(mx - mars)
//   BWD_EDGE   D[r][t] = sum_b G[b][r] * A[b][t]
// run as 128 x N x K tiles (N <= 256) with fp32 accumulators in tensor memory.
//
// Precision: every operand value v is split into a TF32 "hi" part (top 19 bits of the fp32
// pattern) and the exact fp32 remainder "lo"; three tcgen05.mma per 8-deep K step compute
// hi*hi + lo*hi + hi*lo (the dropped lo*lo term is below 2^-20 relative), so results carry
// fp32-class accuracy while the multiply-accumulates run on the tensor pipe.
//
// Operands:
//   * data-dependent operands (A, G) are produced in the kernel: sixteen producer warps read the
//     fp32 work matrices, apply exp / rescale, split, and store into shared memory in the K-major
//     128-byte-swizzled layout the tensor core reads;
//   * the weight operand W is the same for every example tile, so once per parameter update
//     w_image_kernel writes exp(theta), already split and already in the swizzled tile layout,
//     to two images (W for FWD, W^T for BWD_CHILD); the GEMM kernels fetch a tile of an image
//     with two cp.async.bulk copies that complete on the stage's mbarrier.
//   * the per-example maximum mx is computed by the FWD kernel's producers in a first pass over
//     the child rows (which the K loop then re-reads from L2) and kept in blk_mx for the backward
//     kernels.
//
// Synchronisation: a two-stage ring of shared-memory tiles guarded by mbarriers
// (full: one arrival per producer warp + the bulk copies' byte count, empty: one tcgen05.commit), one
// more mbarrier for "accumulator complete".  Every wait is bounded; on expiry the thread raises
// the circuit's status word, leaves its loop and still reaches the common exit where tensor
// memory is released.
#include <algorithm>
#include <cstdlib>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {
using namespace pcbtc;

enum { MODE_FWD = 0, MODE_BWD_CHILD = 1, MODE_BWD_EDGE = 2 };

constexpr uint32_t TM = 128;         // tile rows (TMEM lanes)
constexpr uint32_t TN_MAX = 256;     // tile columns
constexpr uint32_t KCH = 32;         // K elements per stage (one 128-byte swizzle row of tf32)
#ifndef PCB_TC_STAGES
#define PCB_TC_STAGES 2
#define PCB_TC_NPROD 512
#define PCB_TC_CTAS 1
#endif
constexpr uint32_t STAGES = PCB_TC_STAGES;
constexpr uint32_t NPROD = PCB_TC_NPROD;      // producer threads
constexpr uint32_t PW = NPROD / 32;  // producer warps
constexpr uint32_t RG = 16 / PW;     // row groups per thread in the row-contiguous map
constexpr uint32_t QA = 128 / PW;    // A rows per thread in the K-contiguous map
constexpr uint32_t QB = 256 / PW;    // B rows per thread in the K-contiguous map
constexpr uint32_t MMA_WARP = NPROD / 32;
constexpr uint32_t NTHREADS = NPROD + 32;
constexpr uint32_t A_BYTES = TM * 128;        // one A sub-tile (hi or lo)
constexpr uint32_t B_BYTES = TN_MAX * 128;    // one B sub-tile (hi or lo)
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 1024 /*barriers, mx*/ + 2048 /*partial maxima*/;
constexpr uint32_t TMEM_COLS = 256;


// Timing experiments (skipping parts of a kernel, %globaltimer stamps of CTA 0) exist only in a
// build with -DPCB_DIAG; the default build compiles them out.
#ifdef PCB_DIAG
#define PCB_DBG(a, bit) ((a).dbg & (bit))
#define PCB_TRACE_ON(a) ((a).trace != nullptr)
#else
#define PCB_DBG(a, bit) 0u
#define PCB_TRACE_ON(a) false
#endif

struct TcArgs {
  float* mars;
  float* flows;
  float* blk_mx;
  float* aggr;
  const float* theta;
  const float* w_img;
  const PcbDenseBlock* blocks;
  const PcbDenseImg* imgs;
  int* status;
  uint32_t ld, B, b_per_cta;
  uint32_t nsplit;   // FWD / BWD_CHILD: CTAs sharing one 256-column tile (1, 2 or 4), each taking 256 / nsplit columns
  unsigned long long* trace;   // timing trace of CTA (0,0,0), or null
  uint32_t dbg;   // timing experiments only: 1 skip MMAs, 2 skip global loads, 4 skip epilogue, 8 skip smem stores,
                  // 16 skip the child-flow stores, 32 skip the child-value loads of the child-flow epilogue
};

// ---- exp(theta), split and laid out as operand tiles ------------------------------------------------
// One block converts a 32 x 32 patch (rows r, columns t) of a dense block's weights and writes it
// to the FWD image (rows r, K = t) and, transposed through shared memory, to the BWD_CHILD image
// (rows t, K = r).  Image of a dense block: [column tile][K chunk][hi | lo][rows x 128 bytes].
__global__ void __launch_bounds__(256) w_image_kernel(const float* __restrict__ theta, float* __restrict__ img,
                                                      const PcbDenseBlock* __restrict__ blocks,
                                                      const PcbDenseImg* __restrict__ imgs) {
  __shared__ float tile[32][33];
  const PcbDenseBlock k = blocks[blockIdx.z];
  const PcbDenseImg im = imgs[blockIdx.z];
  const uint32_t t0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  if (t0 >= k.K || r0 >= k.R) return;
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (uint32_t i = ty; i < 32; i += 8) {
    uint32_t r = r0 + i, t = t0 + tx;
    tile[i][tx] = (r < k.R && t < k.K) ? __expf(__ldg(theta + k.pid0 + (size_t)r * k.K + t)) : 0.0f;
  }
  __syncthreads();
  {  // FWD image: row = r, kk = t
    const uint32_t c = t0 / KCH;
    for (uint32_t i = ty; i < 32; i += 8) {
      uint32_t r = r0 + i;
      if (r >= k.R) continue;
      uint32_t j = r / TN_MAX, row = r % TN_MAX;
      float* base = img + im.off_f + ((size_t)(j * im.nch_f + c) * 2) * im.rows_f * 32;
      float v = tile[i][tx], h = tf32_hi(v);
      uint32_t o = sw_off(row, tx) / 4;
      base[o] = h;
      base[(size_t)im.rows_f * 32 + o] = v - h;
    }
  }
  {  // BWD_CHILD image: row = t, kk = r
    const uint32_t c = r0 / KCH;
    for (uint32_t i = ty; i < 32; i += 8) {
      uint32_t t = t0 + i;
      if (t >= k.K) continue;
      uint32_t j = t / TN_MAX, row = t % TN_MAX;
      float* base = img + im.off_t + ((size_t)(j * im.nch_t + c) * 2) * im.rows_t * 32;
      float v = tile[tx][i], h = tf32_hi(v);
      uint32_t o = sw_off(row, tx) / 4;
      base[o] = h;
      base[(size_t)im.rows_t * 32 + o] = v - h;
    }
  }
}

// ---- producer side: one K chunk of the data-dependent operands -----------------------------------
struct ProdCtx {
  const float* mars;
  const float* flows;
  const float* mxrow;   // per-example max of this dense block
  const float* mxs;     // the same for the tile's 128 examples, in shared memory (FWD, BWD_CHILD)
  PcbDenseBlock k;
  uint32_t tid, ld, m0, n0, k_begin, k_end, nq;
};
struct ChunkRegs {
  float ra[QA > 8 * RG ? QA : 8 * RG], rm[QA > 8 * RG ? QA : 8 * RG], rb[QB];
  float mx;
  bool vok;
};

// Thread -> element maps of the producers.
//  * "row-contiguous" operands (source contiguous along the tile's row index: A of FWD and
//    BWD_CHILD): a warp covers 8 rows x 4 K positions per step, so its 32 shared-memory stores
//    fall into 32 different banks of the swizzled tile and its global loads are four full
//    32-byte sectors; thread: row = 8*(warp + PW*g) + (lane & 7), kk = (lane >> 3) + 4*q, q = 0..7,
//    g = 0..RG-1.
//  * "K-contiguous" operands (BWD_EDGE): a warp covers one whole 128-byte row per step;
//    thread: kk = lane, row = warp + PW*q.
__device__ __forceinline__ uint32_t rc_row(uint32_t tid, uint32_t g = 0) { return (((tid >> 5) + PW * g) << 3) + (tid & 7u); }
__device__ __forceinline__ uint32_t rc_kk(uint32_t tid, uint32_t q) { return ((tid & 31u) >> 3) + 4u * q; }
//  * 16-byte variant of the row-contiguous map (sixteen producer warps): a thread loads four
//    consecutive examples of one K position; warp w covers examples 8w .. 8w+7 (lane & 1 picks the
//    half) and sixteen K positions (lane >> 1), two passes per chunk.  A quarter of the load
//    instructions of the 4-byte map for the same sectors; the four stores of a load go to rows
//    r .. r+3, and over a warp (two row halves x sixteen K positions) they still fall into 32 banks.
//    Used by BWD_CHILD (two source matrices per element: K loop 15 -> 13 us per tile); FWD measured
//    slower with it and keeps the 4-byte map.
constexpr bool VEC_MAP = PW == 16;
__device__ __forceinline__ uint32_t v4_row(uint32_t tid) { return ((tid >> 5) << 3) + ((tid & 1u) << 2); }
__device__ __forceinline__ uint32_t v4_kk(uint32_t tid, uint32_t q) { return ((tid & 31u) >> 1) + 16u * q; }

// child value M[t][b] with unconditional loads: invalid positions read a safe address and are
// replaced afterwards, so a chunk's loads carry no control dependence and issue back to back
__device__ __forceinline__ float child_val_nb(const float* __restrict__ mars, uint32_t ld, const PcbDenseBlock& k,
                                              uint32_t t, uint32_t b, bool valid) {
  const uint32_t tt = valid ? t : 0u, bb = valid ? b : 0u;
  const bool has_sub = k.d0 != PCB_NONE;
  float v = __ldcg(mars + (size_t)(k.c0 + tt) * ld + bb);
  float w = __ldcg(mars + (size_t)((has_sub ? k.d0 : k.c0) + tt) * ld + bb);
  v += has_sub ? w : 0.0f;
  return valid ? v : -INFINITY;
}

// Per-thread quantities that do not change from chunk to chunk.  Rows and examples outside the
// tile are clamped to a valid address once, here; what they load is masked at store time, so the
// chunk loop itself is straight-line: affine addresses, unconditional loads.
struct ProdInv {
  const float* pc[RG];  // prime-child rows (or the parents' mars rows for G), per row group
  const float* pd[RG];  // sub-child rows (or the parents' flows rows for G)
  const float* pb;      // BWD_EDGE: prime-child rows of the B operand
  const float* pbd;     // BWD_EDGE: sub-child rows of the B operand
  float mx[RG];         // FWD / BWD_CHILD: the example's max (an infinity masks the whole row)
  float mx4[4];         // the same for the four examples of the 16-byte map
  uint32_t rmask;       // BWD_EDGE: bit q set when A row q of this thread is inside the block
  uint32_t bmask;       // BWD_EDGE: bit q set when B row q of this thread is inside the block
  bool has_sub;
  bool full;            // BWD_EDGE: all 128 A rows and all 256 B rows of the tile are inside the block
};

template <int MODE>
__device__ __forceinline__ ProdInv make_inv(const ProdCtx& c) {
  ProdInv v{};
  const uint32_t tid = c.tid, ld = c.ld;
  v.has_sub = c.k.d0 != PCB_NONE;
  if (MODE == MODE_BWD_CHILD && VEC_MAP) {
    // 16-byte map: four consecutive examples (rows v4_row .. +3) of one K position per load
    const uint32_t row = v4_row(tid), b = c.m0 + row, kk0 = v4_kk(tid, 0);
    const bool bok = b < ld;                  // the pitch is a multiple of 4: a group is inside or outside as a whole
    const uint32_t bb = bok ? b : 0u;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const float mx = c.mxs[row + j];
      if (MODE == MODE_FWD) v.mx4[j] = (bok && mx != -INFINITY) ? mx : INFINITY;     // exp(x - inf) = 0
      else                  v.mx4[j] = (bok && mx != -INFINITY) ? mx : -INFINITY;    // exp(-inf - m) = 0
    }
    if (MODE == MODE_FWD) {
      v.pc[0] = c.mars + (size_t)(c.k.c0 + kk0) * ld + bb;
      v.pd[0] = c.mars + (size_t)((v.has_sub ? c.k.d0 : c.k.c0) + kk0) * ld + bb;
    } else {
      v.pc[0] = c.mars + (size_t)(c.k.p0 + kk0) * ld + bb;
      v.pd[0] = c.flows + (size_t)(c.k.p0 + kk0) * ld + bb;
    }
  } else if (MODE == MODE_FWD || MODE == MODE_BWD_CHILD) {
    const uint32_t kk0 = rc_kk(tid, 0);
#pragma unroll
    for (uint32_t g = 0; g < RG; ++g) {
      const uint32_t row = rc_row(tid, g), b = c.m0 + row;
      const bool bok = b < ld;
      const float mx = c.mxs[row];
      const uint32_t bb = bok ? b : 0u;
      if (MODE == MODE_FWD) {
        v.mx[g] = (bok && mx != -INFINITY) ? mx : INFINITY;   // exp(x - inf) = 0
        v.pc[g] = c.mars + (size_t)(c.k.c0 + kk0) * ld + bb;
        v.pd[g] = c.mars + (size_t)((v.has_sub ? c.k.d0 : c.k.c0) + kk0) * ld + bb;
      } else {
        v.mx[g] = (bok && mx != -INFINITY) ? mx : -INFINITY;  // exp(-inf - m) = 0
        v.pc[g] = c.mars + (size_t)(c.k.p0 + kk0) * ld + bb;
        v.pd[g] = c.flows + (size_t)(c.k.p0 + kk0) * ld + bb;
      }
    }
  } else {
    const uint32_t r0 = c.m0 + (tid >> 5), t0 = c.n0 + (tid >> 5), bl = tid & 31;
    v.pc[0] = c.mars + (size_t)c.k.p0 * ld + bl;
    v.pd[0] = c.flows + (size_t)c.k.p0 * ld + bl;
    v.pb = c.mars + (size_t)c.k.c0 * ld + bl;
    v.pbd = c.mars + (size_t)(v.has_sub ? c.k.d0 : c.k.c0) * ld + bl;
#pragma unroll
    for (uint32_t q = 0; q < QA; ++q) v.rmask |= (r0 + PW * q < c.k.R ? 1u : 0u) << q;
#pragma unroll
    for (uint32_t q = 0; q < QB; ++q) v.bmask |= ((q < c.nq && t0 + PW * q < c.k.K) ? 1u : 0u) << q;
    v.full = c.m0 + TM <= c.k.R && c.n0 + TN_MAX <= c.k.K;
  }
  return v;
}

// raw global loads of chunk i (nothing depends on shared memory, so they can run chunks ahead)
template <int MODE>
__device__ __forceinline__ void load_chunk(const ProdCtx& c, const ProdInv& v, uint32_t i, ChunkRegs& r) {
  const uint32_t kc = c.k_begin + i * KCH, tid = c.tid, ld = c.ld;
  if (MODE == MODE_BWD_CHILD && VEC_MAP) {
    const uint32_t kk0 = v4_kk(tid, 0);
    const uint32_t klast = (c.k_end - 1 - kk0) & ~15u;   // a valid row of this thread's K phase (K >= 16)
#pragma unroll
    for (uint32_t q = 0; q < 2; ++q) {
      const uint32_t kq = kc + 16 * q;
      const bool ok = kq + kk0 < c.k_end;
      const size_t o = (size_t)(ok ? kq : klast) * ld;
      const float4 x = *reinterpret_cast<const float4*>(v.pc[0] + o);
      const float4 y = *reinterpret_cast<const float4*>(v.pd[0] + o);
      if (MODE == MODE_FWD) {
        r.ra[q * 4 + 0] = ok ? x.x + (v.has_sub ? y.x : 0.0f) : -INFINITY;
        r.ra[q * 4 + 1] = ok ? x.y + (v.has_sub ? y.y : 0.0f) : -INFINITY;
        r.ra[q * 4 + 2] = ok ? x.z + (v.has_sub ? y.z : 0.0f) : -INFINITY;
        r.ra[q * 4 + 3] = ok ? x.w + (v.has_sub ? y.w : 0.0f) : -INFINITY;
      } else {
        r.rm[q * 4 + 0] = x.x; r.rm[q * 4 + 1] = x.y; r.rm[q * 4 + 2] = x.z; r.rm[q * 4 + 3] = x.w;   // mars of the parent
        r.ra[q * 4 + 0] = ok ? y.x : 0.0f; r.ra[q * 4 + 1] = ok ? y.y : 0.0f;                       // flows of the parent
        r.ra[q * 4 + 2] = ok ? y.z : 0.0f; r.ra[q * 4 + 3] = ok ? y.w : 0.0f;
      }
    }
  } else if (MODE == MODE_FWD || MODE == MODE_BWD_CHILD) {
    // K index of element q: kc + kk0 + 4q; rows past the end of K are clamped and masked
    const uint32_t kk0 = rc_kk(tid, 0);
    const uint32_t klast = (c.k_end - 1 - kk0) & ~3u;   // largest valid multiple of 4 for this thread
#pragma unroll
    for (uint32_t q = 0; q < 8; ++q) {
      const uint32_t kq = kc + 4 * q;
      const bool ok = kq + kk0 < c.k_end;
      const size_t o = (size_t)(ok ? kq : klast) * ld;
#pragma unroll
      for (uint32_t g = 0; g < RG; ++g) {
        float x = v.pc[g][o], y = v.pd[g][o];
        if (MODE == MODE_FWD) {
          x += v.has_sub ? y : 0.0f;
          r.ra[g * 8 + q] = ok ? x : -INFINITY;
        } else {
          r.rm[g * 8 + q] = x;                 // mars of the parent
          r.ra[g * 8 + q] = ok ? y : 0.0f;     // flows of the parent
        }
      }
    }
  } else {
    const uint32_t b = kc + (tid & 31);
    const bool bok = b < c.k_end;
    const uint32_t bo = bok ? kc : c.k_end - 1 - (tid & 31);   // clamped example offset (pointers carry the lane)
    const float mx = c.mxrow[bok ? b : c.k_end - 1];
    r.vok = bok && mx != -INFINITY;
    r.mx = mx;
    const uint32_t r0 = c.m0 + (tid >> 5), t0 = c.n0 + (tid >> 5);
    // A chunk takes one 128-byte line from each of several hundred rows that lie a whole matrix
    // row apart, which DRAM serves as that many page misses.  Every fourth chunk, four lanes of
    // each warp ask L2 for the next 512 bytes of every row (the lines of chunks i+4 .. i+7) in one
    // go, so DRAM sees four adjacent lines per open page and the later chunk loads hit L2.
    if ((i & 3u) == 0 && (tid & 31) < 4) {
      const uint32_t pb0 = kc + 128 + 32 * (tid & 31);   // first example of the line to prefetch
      if (pb0 < c.k_end) {
        const size_t po = (size_t)pb0 - (tid & 31);      // the row pointers already carry the lane
#pragma unroll
        for (uint32_t q = 0; q < QA; ++q) {
          const size_t o = (size_t)((v.rmask >> q & 1u) ? r0 + PW * q : 0u) * ld + po;
          prefetch_l2(v.pc[0] + o);
          prefetch_l2(v.pd[0] + o);
        }
#pragma unroll
        for (uint32_t q = 0; q < QB; ++q) {
          const size_t o = (size_t)((v.bmask >> q & 1u) ? t0 + PW * q : 0u) * ld + po;
          prefetch_l2(v.pb + o);
          if (v.has_sub) prefetch_l2(v.pbd + o);
        }
      }
    }
    if (v.full) {
      // every row of the tile lies inside the block: affine addresses, no masks
      const size_t sa = (size_t)PW * ld;
      const float* pm = v.pc[0] + (size_t)r0 * ld + bo;
      const float* pf = v.pd[0] + (size_t)r0 * ld + bo;
#pragma unroll
      for (uint32_t q = 0; q < QA; ++q) {
        r.rm[q] = pm[q * sa];
        r.ra[q] = pf[q * sa];
      }
      const float* pc = v.pb + (size_t)t0 * ld + bo;
      const float* pd = v.pbd + (size_t)t0 * ld + bo;
      if (v.has_sub) {
#pragma unroll
        for (uint32_t q = 0; q < QB; ++q) r.rb[q] = pc[q * sa] + pd[q * sa];
      } else {
#pragma unroll
        for (uint32_t q = 0; q < QB; ++q) r.rb[q] = pc[q * sa];
      }
      return;
    }
#pragma unroll
    for (uint32_t q = 0; q < QA; ++q) {  // A[m = parent][kk = example] = G: K contiguous
      const uint32_t rr = (v.rmask >> q & 1u) ? r0 + PW * q : 0u;
      const size_t o = (size_t)rr * ld + bo;
      r.rm[q] = v.pc[0][o];
      r.ra[q] = v.pd[0][o];
    }
#pragma unroll
    for (uint32_t q = 0; q < QB; ++q) {  // B[n = child][kk = example] = exp(M - mx)
      const uint32_t tt = (v.bmask >> q & 1u) ? t0 + PW * q : 0u;
      const size_t o = (size_t)tt * ld + bo;
      float x = v.pb[o], y = v.pbd[o];
      r.rb[q] = x + (v.has_sub ? y : 0.0f);
    }
  }
}

// exp / rescale / split and the swizzled shared-memory stores of a loaded chunk
template <int MODE>
__device__ __forceinline__ void store_chunk(const ProdCtx& c, const ProdInv& v, const ChunkRegs& r, uint8_t* a_hi,
                                            uint8_t* a_lo, uint8_t* b_hi, uint8_t* b_lo,
                                            unsigned long long* tmark = nullptr) {
  const uint32_t tid = c.tid;
  if (MODE == MODE_BWD_CHILD && VEC_MAP) {
    const uint32_t row0 = v4_row(tid);
#pragma unroll
    for (uint32_t q = 0; q < 2; ++q) {
      const uint32_t kk = v4_kk(tid, q);
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        const float val = MODE == MODE_FWD ? __expf(r.ra[q * 4 + j] - v.mx4[j])
                                           : r.ra[q * 4 + j] * __expf(v.mx4[j] - r.rm[q * 4 + j]);
        put_split(a_hi, a_lo, sw_off(row0 + j, kk), val);
      }
    }
  } else if (MODE == MODE_FWD || MODE == MODE_BWD_CHILD) {
    // element q sits in 16-byte chunk q of the row (kk >> 2 == q), swizzled with the row index
#pragma unroll
    for (uint32_t g = 0; g < RG; ++g) {
      const uint32_t row = rc_row(tid, g);
      const uint32_t base = row * 128u + (((tid & 31u) >> 3) << 2);
      const uint32_t r7 = row & 7u;
#pragma unroll
      for (uint32_t q = 0; q < 8; ++q) {
        const float val = MODE == MODE_FWD ? __expf(r.ra[g * 8 + q] - v.mx[g])
                                           : r.ra[g * 8 + q] * __expf(v.mx[g] - r.rm[g * 8 + q]);
        put_split(a_hi, a_lo, base + ((q ^ r7) << 4), val);
      }
    }
  } else {
    const uint32_t kk = tid & 31, w = tid >> 5;
    const uint32_t cpos = (kk >> 2), csub = (kk & 3u) << 2;
    if (v.full) {
      // PW is a multiple of 8, so the swizzle term (row & 7) == (w & 7) for all of a thread's rows:
      // one base offset, then a fixed 128 * PW bytes per step; an example outside the batch is
      // masked through the max (exp(-inf) = 0) instead of per element
      static_assert(PW % 8 == 0, "row & 7 must not depend on q");
      const uint32_t base = w * 128u + (((cpos ^ (w & 7u)) << 4) | csub);
      const float mxa = r.vok ? r.mx : -INFINITY, mxb = r.vok ? r.mx : INFINITY;
#pragma unroll
      for (uint32_t q = 0; q < QA; ++q) put_split(a_hi, a_lo, base + q * (PW * 128u), r.ra[q] * __expf(mxa - r.rm[q]));
      if (tmark) *tmark = gtime();
#pragma unroll
      for (uint32_t q = 0; q < QB; ++q) put_split(b_hi, b_lo, base + q * (PW * 128u), __expf(r.rb[q] - mxb));
      return;
    }
#pragma unroll
    for (uint32_t q = 0; q < QA; ++q) {
      const uint32_t row = w + PW * q;
      const bool ok = r.vok && (v.rmask >> q & 1u);
      put_split(a_hi, a_lo, row * 128u + (((cpos ^ (row & 7u)) << 4) | csub), ok ? r.ra[q] * __expf(r.mx - r.rm[q]) : 0.0f);
    }
    if (tmark) *tmark = gtime();
#pragma unroll
    for (uint32_t q = 0; q < QB; ++q) {
      if (q < c.nq) {
        const uint32_t row = w + PW * q;
        const bool ok = r.vok && (v.bmask >> q & 1u);
        put_split(b_hi, b_lo, row * 128u + (((cpos ^ (row & 7u)) << 4) | csub), ok ? __expf(r.rb[q] - r.mx) : 0.0f);
      }
    }
  }
}

// grid: FWD / BWD_CHILD (example tiles of 128, column tiles of 256, blocks)
//       BWD_EDGE        (example slices, row tiles x column tiles, blocks)
template <int MODE>
__global__ void __launch_bounds__(NTHREADS, PCB_TC_CTAS) dense_tc_kernel(TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctl = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);          // [STAGES]
  uint64_t* empty = full + STAGES;                            // [STAGES]
  uint64_t* accfull = empty + STAGES;                         // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);
  uint64_t* ebar = reinterpret_cast<uint64_t*>(ctl + 64);     // [3] child-value copies of the BWD_CHILD epilogue
  uint32_t* epi_fail = reinterpret_cast<uint32_t*>(ctl + 96); // a producer warp lost a wait
  float* mxs = reinterpret_cast<float*>(ctl + 128);           // [128]

  if (PCB_TRACE_ON(a) && threadIdx.x == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[504] = gtime();
  pcb_grid_dep_launch();
  const PcbDenseBlock k = a.blocks[blockIdx.z];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ld = a.ld;

  // ---- tile coordinates ---------------------------------------------------------------------
  uint32_t m0, n0, n_count, k_begin, k_end, jn;  // rows [m0, m0+128), columns [n0, n0+n_count), K range
  uint32_t part0 = 0;                            // first column of this CTA inside its 256-column tile
  if (MODE == MODE_FWD || MODE == MODE_BWD_CHILD) {
    const uint32_t ncols = MODE == MODE_FWD ? k.R : k.K, sw = TN_MAX / a.nsplit;
    m0 = blockIdx.x * TM; jn = blockIdx.y / a.nsplit; part0 = (blockIdx.y % a.nsplit) * sw;
    n0 = jn * TN_MAX + part0;
    if (n0 >= ncols) return;
    n_count = min(sw, ncols - n0); k_begin = 0; k_end = MODE == MODE_FWD ? k.K : k.R;
  } else {
    const uint32_t tiles_n = (k.K + TN_MAX - 1) / TN_MAX;
    m0 = (blockIdx.y / tiles_n) * TM; jn = blockIdx.y % tiles_n; n0 = jn * TN_MAX;
    if (m0 >= k.R) return;
    n_count = min(TN_MAX, k.K - n0);
    k_begin = blockIdx.x * a.b_per_cta; k_end = min(a.B, k_begin + a.b_per_cta);
    if (k_begin >= k_end) return;
  }
  const uint32_t nchunks = (k_end - k_begin + KCH - 1) / KCH;
  const float* mxrow = a.blk_mx + (size_t)k.mx_row * ld;
  // B tile rows: the image's row count for the bulk-copied operand, else N rounded up to 16
  uint32_t n_tile = (n_count + 15u) & ~15u;
  const float* img_tile = nullptr;   // first K chunk of this column tile in the weight image
  uint32_t img_rows = 0;
  if (MODE != MODE_BWD_EDGE) {
    const PcbDenseImg im = a.imgs[blockIdx.z];
    img_rows = MODE == MODE_FWD ? im.rows_f : im.rows_t;
    const uint32_t nch = MODE == MODE_FWD ? im.nch_f : im.nch_t;
    img_tile = a.w_img + (MODE == MODE_FWD ? im.off_f : im.off_t) + (size_t)jn * nch * 2 * img_rows * 32 + part0 * 32;
    n_tile = min(TN_MAX / a.nsplit, img_rows - part0);   // rows beyond n_count are zero in the image
  }

  // ---- set-up: barriers, tensor memory, per-example max --------------------------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) { mbar_init(&full[s], NPROD / 32); mbar_init(&empty[s], 1); }
    mbar_init(accfull, 1);
    for (uint32_t j = 0; j < 3; ++j) mbar_init(&ebar[j], 1);
    *epi_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Up to here only static circuit data was read: a launch with programmatic stream serialization
  // may have come this far while the previous kernel of the stream was still running.
  pcb_grid_dep_wait();
  if (MODE == MODE_BWD_CHILD && tid < 128) mxs[tid] = (m0 + tid < ld) ? mxrow[m0 + tid] : -INFINITY;
  if (MODE == MODE_FWD && warp < MMA_WARP) {
    // Per-example maximum of the block's child values over all K children.  The child rows for
    // the tile's examples (512 bytes each, prime and sub) come in by bulk copies, 96 children per
    // batch, into two buffers carved from the operand stages (idle before the K loop): slot c of
    // 1 KB = [prime row | sub row].  Thread (example e, part q) scans its share of a batch's slots;
    // batch j + 2 is requested as soon as batch j has been read.  The K loop reads the rows again,
    // from L2.  The maxima also go to blk_mx for the backward kernels (one CTA per example tile).
    constexpr uint32_t NQ = NPROD / 128, BATCH = 96, PER_Q = BATCH / NQ;
    const bool has_sub = k.d0 != PCB_NONE;
    const uint32_t ex = min(TM, ld - m0), rowb = ex * 4u, per = has_sub ? 2u : 1u;
    const uint32_t nbatch = (k.K + BATCH - 1) / BATCH;
    const uint32_t e = tid & 127u, q = tid >> 7;
    float* part = reinterpret_cast<float*>(ctl + 1024);   // [NQ][128]
    auto rows_of = [&](uint32_t j) { return min(BATCH, k.K - j * BATCH); };
    auto issue_batch = [&](uint32_t j) {
      if (tid < 2 * BATCH) {
        const uint32_t c = tid % BATCH, which = tid / BATCH;
        if (c < rows_of(j) && (which == 0u || has_sub))
          bulk_g2s(smem + ((j & 1u) * BATCH + c) * 1024u + which * 512u,
                   a.mars + (size_t)((which ? k.d0 : k.c0) + j * BATCH + c) * ld + m0, rowb, &ebar[j & 1u]);
      }
    };
    if (tid == 0) {
      mbar_arrive_expect_tx(&ebar[0], rows_of(0) * rowb * per);
      if (nbatch > 1) mbar_arrive_expect_tx(&ebar[1], rows_of(1) * rowb * per);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // byte counts posted before the first copy
    issue_batch(0);
    if (nbatch > 1) issue_batch(1);
    float mx = -INFINITY;
    bool got = true;
    for (uint32_t j = 0; j < nbatch; ++j) {
      bool g1 = lane != 0 || mbar_wait(&ebar[j & 1u], (j >> 1) & 1u, a.status);
      got = __all_sync(0xffffffffu, g1) && got;
      const uint32_t nr = rows_of(j);
      const float* base = reinterpret_cast<const float*>(smem + (j & 1u) * BATCH * 1024u) + e;
      if (got && e < ex) {
#pragma unroll 8
        for (uint32_t c = q * PER_Q; c < min(nr, (q + 1) * PER_Q); ++c) {
          float v = base[c * 256u];
          if (has_sub) v += base[c * 256u + 128u];
          mx = fmaxf(mx, v);
        }
      }
      if (j + 2 < nbatch) {   // CTA-uniform
        asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // the buffer has been read by everyone
        if (tid == 0) mbar_arrive_expect_tx(&ebar[j & 1u], rows_of(j + 2) * rowb * per);
        asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
        fence_proxy_async();
        issue_batch(j + 2);
      }
    }
    if (!got) *reinterpret_cast<volatile uint32_t*>(epi_fail) = 1u;
    part[q * 128u + e] = mx;
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
    if (tid < 128u) {
#pragma unroll
      for (uint32_t u = 1; u < NQ; ++u) mx = fmaxf(mx, part[u * 128u + tid]);
      const bool bok = tid < ex;
      mxs[tid] = bok ? mx : -INFINITY;
      if (bok && blockIdx.y == 0) a.blk_mx[(size_t)k.mx_row * ld + m0 + tid] = mx;
    }
    fence_proxy_async();   // the K loop's copies and MMAs touch the same memory next
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  if (PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[503] = gtime();

  if (warp < MMA_WARP) {
    // =========================== producers ===================================================
    // The global loads of chunk i+1 are issued before chunk i is transformed and stored, so
    // their latency overlaps the exp / split / store work and the wait for the stage.
    ProdCtx ctx{a.mars, a.flows, mxrow, mxs, k, tid, ld, m0, n0, k_begin, k_end, n_tile / PW};
    const ProdInv inv = make_inv<MODE>(ctx);
    ChunkRegs ra0, ra1;   // two register sets, used alternately: no copies on the loop edge
    auto process = [&](uint32_t i, const ChunkRegs& cr) -> bool {
      const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
      const bool tr = PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && i < 60;
      if (tr) a.trace[i * 8 + 0] = gtime();
      // one lane per warp polls; __syncwarp orders the other lanes' stores behind the observed phase
      bool got = lane != 0 || mbar_wait(&empty[s], ph ^ 1u, a.status);
      got = __all_sync(0xffffffffu, got);
      if (!got) return false;
      uint8_t* a_hi = smem + s * STAGE_BYTES;
      uint8_t* a_lo = a_hi + A_BYTES;
      uint8_t* b_hi = a_lo + A_BYTES;
      uint8_t* b_lo = b_hi + B_BYTES;
      if (tr) a.trace[i * 8 + 1] = gtime();
      if (MODE != MODE_BWD_EDGE && tid == 0) {  // weight tile: hi and lo parts straight from the image
        const uint32_t bytes = n_tile * 128u;
        const float* src = img_tile + (size_t)i * 2 * img_rows * 32;
        mbar_expect_tx(&full[s], 2 * bytes);
        bulk_g2s(b_hi, src, bytes, &full[s]);
        bulk_g2s(b_lo, src + (size_t)img_rows * 32, bytes, &full[s]);
      }
      if (!(PCB_DBG(a, 8u))) store_chunk<MODE>(ctx, inv, cr, a_hi, a_lo, b_hi, b_lo, tr ? a.trace + i * 8 + 7 : nullptr);
      if (tr) a.trace[i * 8 + 2] = gtime();
      fence_proxy_async();   // make the generic-proxy writes visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);   // one arrival per warp: 512 arrivals on one word serialise
      if (tr) a.trace[i * 8 + 3] = gtime();
      return true;
    };
    load_chunk<MODE>(ctx, inv, 0, ra0);
    for (uint32_t i = 0; i < nchunks && ok; i += 2) {
      if (i + 1 < nchunks) load_chunk<MODE>(ctx, inv, i + 1, ra1);
      ok = process(i, ra0);
      if (!ok || i + 1 >= nchunks) break;
      if (i + 2 < nchunks) load_chunk<MODE>(ctx, inv, i + 2, ra0);
      ok = process(i + 1, ra1);
    }

    // =========================== epilogue ====================================================
    if (PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[500] = gtime();
    if (ok && lane == 0) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[501] = gtime();
    constexpr bool COPY_EPI = MODE == MODE_BWD_CHILD && PW == 16;
    if (COPY_EPI) {
      // Child flows  f[t][b] = acc[b][t] * exp(M[t][b] - mx[b])  need the children's value rows for
      // the tile's examples: up to 2 x 256 rows of 512 bytes.  Plain loads of that shape (every
      // request a line of another row) run at a fraction of what the copy engine delivers, so the
      // rows are fetched with one bulk copy each into the operand stages, idle by now: slot c of
      // 1 KB holds column c's prime row and sub row.  192 slots fit; columns 192..255 reuse slots
      // 0..63 once the first round has read them.  Round r, warp group g: columns 128 r + 32 g ...
      if (!ok) *reinterpret_cast<volatile uint32_t*>(epi_fail) = 1u;
      const uint32_t ex = min(TM, ld - m0);              // examples of this tile (ld is a multiple of 32)
      const uint32_t rowb = ex * 4u;
      const bool has_sub = k.d0 != PCB_NONE;
      const uint32_t per = has_sub ? 2u : 1u;
      const uint32_t cnt0 = min(n_count, 128u), cnt1 = n_count > 128u ? min(n_count - 128u, 64u) : 0u,
                     cnt2 = n_count > 192u ? n_count - 192u : 0u;
      if (tid == 0) {
        mbar_arrive_expect_tx(&ebar[0], cnt0 * rowb * per);
        mbar_arrive_expect_tx(&ebar[1], cnt1 * rowb * per);
        mbar_arrive_expect_tx(&ebar[2], cnt2 * rowb * per);
      }
      // every producer warp is past the accumulator wait (the stages are idle) and the byte counts
      // are posted before the first copy is issued
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
      const bool go = *reinterpret_cast<volatile uint32_t*>(epi_fail) == 0u && !(PCB_DBG(a, 4u));
      if (go) {
        tc_fence_after();
        auto issue = [&](uint32_t c, uint32_t which, uint64_t* bar) {
          const uint32_t slot = c < 192u ? c : c - 192u;
          const float* src = a.mars + (size_t)((which ? k.d0 : k.c0) + n0 + c) * ld + m0;
          bulk_g2s(smem + slot * 1024u + which * 512u, src, rowb, bar);
        };
        if (tid < 384u) {
          const uint32_t c = tid % 192u, which = tid / 192u;
          if (c < n_count && (which == 0u || has_sub)) issue(c, which, c < 128u ? &ebar[0] : &ebar[1]);
        }
        const uint32_t q4 = warp & 3, grp = warp >> 2, row = q4 * 32 + lane, b = m0 + row;
        const float mx = mxs[row];
        auto round = [&](uint32_t c0, uint64_t* bar) {   // 32 columns from c0, warp-uniform
          if (c0 >= n_tile) return;
          bool got = lane != 0 || mbar_wait(bar, 0, a.status);
          got = __all_sync(0xffffffffu, got);
          float acc[32];
          tmem_ld32(tmem_base + ((q4 * 32u) << 16) + c0, acc);
          if (got && b < ld) {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              const uint32_t c = c0 + j, t = n0 + c;
              if (t < k.K) {
                const float* sp = reinterpret_cast<const float*>(smem + (c < 192u ? c : c - 192u) * 1024u) + row;
                float cv = sp[0];
                if (has_sub) cv += sp[128];
                const float f = mx == -INFINITY ? 0.0f : acc[j] * __expf(cv - mx);
                a.flows[(size_t)(k.c0 + t) * ld + b] = f;
                if (has_sub) a.flows[(size_t)(k.d0 + t) * ld + b] = f;
              }
            }
          }
        };
        round(32u * grp, &ebar[0]);
        if (n_tile > 128u) {
          asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // slots 0..63 have been read
          if (tid < 128u) {
            const uint32_t c = 192u + (tid & 63u), which = tid >> 6;
            if (c < n_count && (which == 0u || has_sub)) {
              fence_proxy_async();
              issue(c, which, &ebar[2]);
            }
          }
          round(128u + 32u * grp, grp < 2u ? &ebar[1] : &ebar[2]);
        }
      }
    } else if (ok && !(PCB_DBG(a, 4u))) {
      tc_fence_after();
      constexpr uint32_t NG = PW / 4;                                             // epilogue warp groups
      const uint32_t CG = max(32u, ((n_tile + 32u * NG - 1u) / (32u * NG)) * 32u);   // columns per group
      const uint32_t q4 = warp & 3, grp = warp >> 2;   // lane quarter, column group
      const uint32_t row = q4 * 32 + lane;
      const uint32_t c_begin = grp * CG, c_end = min(n_tile, c_begin + CG);
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
            // all child values first (independent loads), then the products and the stores:
            // the stores to flows would otherwise order every later load behind them
            float cv[32];
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              uint32_t t = n0 + c0 + j;
              cv[j] = (PCB_DBG(a, 32u)) ? mx : child_val_nb(a.mars, ld, k, t, b, t < k.K && mx != -INFINITY);
            }
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j) {
              uint32_t t = n0 + c0 + j;
              if (t < k.K) {
                float f = acc[j] * __expf(cv[j] - mx);   // exp(-inf) = 0 for masked entries
                if ((PCB_DBG(a, 16u)) && f != 12345.0f) continue;
                a.flows[(size_t)(k.c0 + t) * ld + b] = f;
                if (k.d0 != PCB_NONE) a.flows[(size_t)(k.d0 + t) * ld + b] = f;
              }
            }
          }
        } else {
          // The accumulator arrives with one tile row per lane; the statistics rows are
          // contiguous along the column index.  Transpose the 32 x 32 patch through shared memory
          // (the operand stages are idle once the accumulator is complete) so that a warp reads
          // theta and issues its reductions as whole 128-byte lines.
          float* patch = reinterpret_cast<float*>(smem) + warp * (32 * 33);
#pragma unroll
          for (uint32_t j = 0; j < 32; ++j) patch[lane * 33 + j] = acc[j];
          __syncwarp();
          const uint32_t t = n0 + c0 + lane;
          if (t < k.K) {
#pragma unroll 8
            for (uint32_t rr = 0; rr < 32; ++rr) {
              const uint32_t r = m0 + q4 * 32 + rr;
              if (r < k.R) {
                const size_t p = k.pid0 + (size_t)r * k.K + t;
                // reduction without a return value: fire-and-forget; one writer per element unless
                // the examples are sliced over several CTAs
                atomicAdd(a.aggr + p, __expf(__ldg(a.theta + p)) * patch[rr * 33 + lane]);
              }
            }
          }
          __syncwarp();
        }
      }
    }
  } else {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc(TM, n_tile);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
        const bool tr = PCB_TRACE_ON(a) && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && i < 60;
        if (tr) a.trace[i * 8 + 4] = gtime();
        ok = mbar_wait(&full[s], ph, a.status);
        if (!ok) break;
        if (tr) a.trace[i * 8 + 5] = gtime();
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t d_ahi = make_desc(sa), d_alo = make_desc(sa + A_BYTES);
        const uint64_t d_bhi = make_desc(sa + 2 * A_BYTES), d_blo = make_desc(sa + 2 * A_BYTES + B_BYTES);
        if (!(PCB_DBG(a, 1u)))
#pragma unroll
        for (uint32_t ks = 0; ks < KCH / 8; ++ks) {
          const uint64_t adv = (uint64_t)((ks * 32u) >> 4);  // 8 tf32 = 32 bytes along K
          umma_tf32(tmem_base, d_ahi + adv, d_bhi + adv, idesc, (i | ks) ? 1u : 0u);
          umma_tf32(tmem_base, d_alo + adv, d_bhi + adv, idesc, 1u);
          umma_tf32(tmem_base, d_ahi + adv, d_blo + adv, idesc, 1u);
        }
        umma_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
        if (tr) a.trace[i * 8 + 6] = gtime();
      }
      if (ok) umma_commit(accfull);
    }
    __syncwarp();
  }

  if (PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[502] = gtime();
  // ---- common exit: release tensor memory ---------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (PCB_TRACE_ON(a) && tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[505] = gtime();
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int MODE>
int32_t launch(dim3 grid, const TcArgs& args, cudaStream_t st, bool pdl = false) {
  static PcbPerDeviceOnce once;
  PCB_CUDA(once.run([] {
    return cudaFuncSetAttribute(dense_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  }));
  PCB_CUDA(pcb_launch_pdl(dense_tc_kernel<MODE>, grid, dim3(NTHREADS), SMEM_BYTES, st, pdl, args));
  return PCB_OK;
}

unsigned long long* g_trace = nullptr;   // diagnostic buffer, allocated when PCB_TC_TRACE is set

TcArgs make_args(pcb_circuit* c, pcb_workspace* ws, uint32_t o0) {
  uint32_t dbg = 0;
#ifdef PCB_DIAG
  if (!g_trace && getenv("PCB_TC_TRACE")) {
    cudaMalloc((void**)&g_trace, 512 * sizeof(unsigned long long));
    cudaMemset(g_trace, 0, 512 * sizeof(unsigned long long));
  }
  if (const char* e = getenv("PCB_TC_DEBUG")) dbg = (uint32_t)atoi(e);
#endif
  return TcArgs{ws->mars, ws->flows, ws->blk_mx, c->aggr, c->theta, c->w_img, c->dense + o0, c->dense_img + o0,
                c->status, ws->ld, ws->B, 0, 1, g_trace, dbg};
}

// A layer that would not fill the GPU with 256-column tiles is cut into narrower tiles: the CTAs
// of one tile then repeat the production of the data-dependent operand, but each has half (a
// quarter) of the weight tile to fetch, of the MMAs to wait for and of the epilogue, and a layer's
// latency is what a chain of small layers pays.
uint32_t pick_nsplit(uint32_t ctas, uint32_t max_cols, int forced) {
  if (forced == 1 || forced == 2 || forced == 4) return (uint32_t)forced;
  uint32_t n = 1;
  while (n < 4 && ctas * n * 2 <= 160 && max_cols > TN_MAX / (2 * n)) n *= 2;
  return n;
}

}  // namespace

#define PCB_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != PCB_OK) return _s;   \
  } while (0)

// Lays out the weight images of every dense block (host side) and allocates them.
int32_t pcb_dense_tc_prepare(pcb_circuit* c, uint64_t* bytes) {
  if (const char* e = getenv("PCB_TC_IMPL")) c->tc_mn = std::string(e) != "km";   // km: the K-major staging kernels of this file
  if (c->tc_mn) PCB_TRY(pcb_dense_mn_prepare(c, bytes));
  std::vector<PcbDenseImg> imgs(c->tc_mn ? 0 : c->h_dense.size());
  uint64_t off = 0;
  for (size_t i = 0; i < imgs.size(); ++i) {
    const PcbDenseBlock& k = c->h_dense[i];
    PcbDenseImg& im = imgs[i];
    im.rows_f = std::min<uint32_t>(TN_MAX, pcb_round_up(k.R, 16));
    im.rows_t = std::min<uint32_t>(TN_MAX, pcb_round_up(k.K, 16));
    im.nch_f = (k.K + KCH - 1) / KCH;
    im.nch_t = (k.R + KCH - 1) / KCH;
    uint64_t tiles_f = (k.R + TN_MAX - 1) / TN_MAX, tiles_t = (k.K + TN_MAX - 1) / TN_MAX;
    im.off_f = off; off += tiles_f * im.nch_f * 2 * im.rows_f * 32;
    im.off_t = off; off += tiles_t * im.nch_t * 2 * im.rows_t * 32;
  }
  c->w_img_len = off;
  PCB_CUDA(cudaMalloc((void**)&c->w_img, std::max<uint64_t>(off, 1) * sizeof(float)));
  PCB_CUDA(cudaMemset(c->w_img, 0, std::max<uint64_t>(off, 1) * sizeof(float)));  // padding rows / columns stay zero
  PCB_CUDA(cudaMalloc((void**)&c->dense_img, std::max<size_t>(imgs.size(), 1) * sizeof(PcbDenseImg)));
  if (!imgs.empty())
    PCB_CUDA(cudaMemcpy(c->dense_img, imgs.data(), imgs.size() * sizeof(PcbDenseImg), cudaMemcpyHostToDevice));
  *bytes += off * sizeof(float) + imgs.size() * sizeof(PcbDenseImg);
  c->w_img_valid = false;
  if (!(getenv("PCB_NO_SIDE_STREAM") && atoi(getenv("PCB_NO_SIDE_STREAM")))) {
    PCB_CUDA(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
    PCB_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    PCB_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
    PCB_CUDA(cudaStreamCreateWithFlags(&c->side2, cudaStreamNonBlocking));
    PCB_CUDA(cudaEventCreateWithFlags(&c->ev_fork2, cudaEventDisableTiming));
    PCB_CUDA(cudaEventCreateWithFlags(&c->ev_join2, cudaEventDisableTiming));
  }
  if (const char* e = getenv("PCB_EDGE_BATCH_TILES")) c->edge_batch_tiles = (uint32_t)std::max(1, atoi(e));
  return PCB_OK;
}

// Regenerates the weight images if the parameters changed since they were last written.
int32_t pcb_dense_tc_refresh(pcb_circuit* c, cudaStream_t st) {
  if (c->w_img_valid || c->n_dense == 0) return PCB_OK;
  if (c->tc_mn) {
    PCB_TRY(pcb_dense_mn_refresh(c, st));
    c->w_img_valid = true;
    return PCB_OK;
  }
  for (uint32_t z0 = 0; z0 < c->n_dense; z0 += 65535) {
    uint32_t nz = std::min<uint32_t>(65535, c->n_dense - z0);
    dim3 grid((c->max_dense_K + 31) / 32, (c->max_dense_R + 31) / 32, nz);
    PcbProfScope ps(c, st, PCB_K_W_IMAGE);
    w_image_kernel<<<grid, 256, 0, st>>>(c->theta, c->w_img, c->dense + z0, c->dense_img + z0);
  }
  c->w_img_valid = true;
  return PCB_OK;
}

int32_t pcb_dense_tc_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  if (c->tc_mn) return pcb_dense_mn_forward(c, ws, layer, st);
  const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM;
  TcArgs args = make_args(c, ws, o0);
  const uint32_t ct = (c->max_dense_R + TN_MAX - 1) / TN_MAX;
  args.nsplit = pick_nsplit(bt * ct * (o1 - o0), c->max_dense_R, c->tc_nsplit);
  dim3 grid(bt, ct * args.nsplit, o1 - o0);
  PcbProfScope ps(c, st, PCB_K_DENSE_FWD);
  return launch<MODE_FWD>(grid, args, st, c->pdl);
}

// Launches the edge-statistics kernel over the pending block range [edge_lo, edge_hi).
// The parents' flows of every pending block are final on `st` and nothing later in the backward
// pass reads the statistics, so the kernel goes to the side stream (when there is one) and overlaps
// the child-flow kernels that follow on `st`.
int32_t pcb_dense_tc_flush_edges(pcb_circuit* c, pcb_workspace* ws, cudaStream_t st) {
  if (c->edge_hi <= c->edge_lo) return PCB_OK;
  const uint32_t o0 = c->edge_lo, n = c->edge_hi - c->edge_lo;
  c->edge_lo = c->edge_hi = 0;
  TcArgs args = make_args(c, ws, o0);
  uint32_t tiles = ((c->max_dense_R + TM - 1) / TM) * ((c->max_dense_K + TN_MAX - 1) / TN_MAX);
  // slice the examples so that a short range still fills the GPU
  uint32_t want = std::max(1u, 148u / std::max(1u, tiles * n));
  uint32_t slices = std::min(want, (ws->B + 255) / 256);
  uint32_t b_per = pcb_round_up((ws->B + slices - 1) / slices, KCH);
  slices = (ws->B + b_per - 1) / b_per;
  args.b_per_cta = b_per;
  cudaStream_t es = st;
  if (c->side && !c->prof.on) {   // per-class timing wants every class alone on the GPU
    PCB_CUDA(cudaEventRecord(c->ev_fork, st));
    PCB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    es = c->side;
    c->side_busy = true;
  }
  if (ws->have_tm) return pcb_dense_edge_launch(c, ws, o0, n, slices, b_per, es);
  for (uint32_t z0 = 0; z0 < n; z0 += 65535) {
    TcArgs a2 = args;
    a2.blocks = args.blocks + z0;
    a2.imgs = args.imgs + z0;
    dim3 grid(slices, tiles, std::min<uint32_t>(65535, n - z0));
    PcbProfScope ps(c, es, PCB_K_DENSE_BWD_EDGE);
    PCB_TRY(launch<MODE_BWD_EDGE>(grid, a2, es));
  }
  return PCB_OK;
}

int32_t pcb_dense_tc_backward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  // Edge statistics: layers are visited top down and their blocks are stored layer after layer, so
  // consecutive layers extend one block range downwards.  The range is launched once it holds
  // enough tiles for a few waves of CTAs; most layers alone would fill only a few SMs.
  if (!c->skip_stats) {
    if (c->edge_hi > c->edge_lo && c->edge_lo != o1) PCB_TRY(pcb_dense_tc_flush_edges(c, ws, st));
    if (c->edge_hi <= c->edge_lo) c->edge_hi = o1;
    c->edge_lo = o0;
    uint32_t tiles = ((c->max_dense_R + TM - 1) / TM) * ((c->max_dense_K + TN_MAX - 1) / TN_MAX);
    if (!c->side || (c->edge_hi - c->edge_lo) * tiles >= c->edge_batch_tiles) PCB_TRY(pcb_dense_tc_flush_edges(c, ws, st));
  }
  if (c->tc_mn) return pcb_dense_mn_backward_child(c, ws, layer, st);
  TcArgs args = make_args(c, ws, o0);
  {
    const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM, ct = (c->max_dense_K + TN_MAX - 1) / TN_MAX;
    args.nsplit = pick_nsplit(bt * ct * (o1 - o0), c->max_dense_K, c->tc_nsplit);
    dim3 grid(bt, ct * args.nsplit, o1 - o0);
    PcbProfScope ps(c, st, PCB_K_DENSE_BWD_CHILD);
    PCB_TRY(launch<MODE_BWD_CHILD>(grid, args, st, c->pdl));
  }
  return PCB_OK;
}

// Makes `st` wait for everything queued on the side stream.
int32_t pcb_side_join(pcb_circuit* c, cudaStream_t st) {
  if (!c->side || !c->side_busy) return PCB_OK;
  PCB_CUDA(cudaEventRecord(c->ev_join, c->side));
  PCB_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
  c->side_busy = false;
  return PCB_OK;
}

// Diagnostic: copies the timing trace of the last traced kernel (PCB_TC_TRACE set) to the host.
unsigned long long* pcb_dense_mn_trace();
extern "C" int32_t pcb_debug_read_trace(unsigned long long* out) {
  if (unsigned long long* t = pcb_dense_mn_trace()) {   // the example-major kernels are the ones in use
    cudaDeviceSynchronize();
    return cudaMemcpy(out, t, 512 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? PCB_OK : PCB_ERR_CUDA;
  }
  if (!g_trace) return PCB_ERR_STATE;
  cudaDeviceSynchronize();
  return cudaMemcpy(out, g_trace, 512 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? PCB_OK : PCB_ERR_CUDA;
}
