// pcb_dense_mn.cu — values (forward) and child flows (backward) of dense sum blocks on tcgen05, with
// the data-dependent operand read the way it lies in memory.
//
//   FWD        D[b][r] = sum_t A[b][t] * W[r][t]     A = exp(M[t][b] - mx[b]),  W = exp(theta)
//              mars[r][b] = log D[b][r] + mx[b]      M[t][b] = mars[prime t][b] + mars[sub t][b]
//   BWD_CHILD  D[b][t] = sum_r G[b][r] * W[r][t]     G = flows[r][b] * exp(mx[b] - mars[r][b])
//              flows[child t][b] = D[b][t] * exp(M[t][b] - mx[b])
//
// Replaces layer_up_kernel (VariationalJuice.jl/src/queries/likelihood.jl:4-68) and layer_down_kernel /
// reg_layer_down_kernel (queries/flow.jl:8-106, regularization/reg_flow.jl:120-222) on k x k blocks.
//
// The work matrices are node-major with the example index contiguous, so the rows a tile needs are
// [K rows][128 examples] slabs: 512 contiguous bytes per row.  That is an M-major ("MN-major") A
// operand for a 128 (examples) x N x K tile, and tcgen05 reads such an operand from shared memory
// directly: 128-byte rows of 32 examples, four K rows per 512-byte swizzle atom.  A producer warp
// therefore loads one K row of the tile with a single fully coalesced 16-byte-per-lane request,
// applies exp / rescale, splits into TF32 hi / lo and stores 16 bytes per lane — no transposition
// through registers, a quarter of the instructions of a K-major staging.
//
// The weight operand comes from pre-split, pre-swizzled images of exp(theta) (K-major, 16 K values
// = 64 bytes per row, 64-byte swizzle), one bulk copy per part and chunk.
//
// Precision: v = hi + lo with hi = top 19 bits; three MMAs per K step (hi*hi + lo*hi + hi*lo).
//
// A CTA is 8 producer warps (which also run the max pass of FWD and the epilogue) + 1 MMA warp and
// keeps two 48 KB stages, so two CTAs share an SM: while one is in its K loop (shared-memory and
// tensor-pipe bound) the other runs its max pass or its epilogue (memory bound).
// Every mbarrier wait is bounded; on expiry the status word is raised and all roles drain to the
// common exit where tensor memory is released.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {
using namespace pcbtc;

enum { MN_FWD = 0, MN_BWD_CHILD = 1 };

constexpr uint32_t TM = 128;            // examples per tile (TMEM lanes)
constexpr uint32_t TN = 256;            // columns per tile (TMEM columns)
constexpr uint32_t KC = 16;             // K values per chunk
constexpr uint32_t PW = 8;              // producer warps: warp w owns K rows w and w + 8 of every chunk
constexpr uint32_t NPROD = PW * 32;
constexpr uint32_t MMA_WARP = PW, COPY_WARP = PW + 1;
constexpr uint32_t NTHREADS = NPROD + 64;
constexpr uint32_t ROW_BYTES = TM * 4;          // one row of a tile: 128 examples
constexpr uint32_t A_BYTES = KC * ROW_BYTES;    // one A part (hi or lo): 16 swizzle atoms of 512 bytes
constexpr uint32_t A_STAGE = 2 * A_BYTES;       // hi | lo
constexpr uint32_t A_STAGES = 2;                // A stages of a launch that fills the GPU (two CTAs per SM)
constexpr uint32_t A_MAX_STAGES = 8;            // ... of a launch of at most one CTA per SM (the small layers of the chain)
constexpr uint32_t W_RING = 64 * 1024;          // weight chunks [hi | lo] of n_tile rows x 64 bytes: 2 chunks of a 256-column
constexpr uint32_t W_MAX_STAGES = 16;           // tile, 8 of a 64-column tile
constexpr uint32_t BUF_BYTES = A_STAGES * A_STAGE + W_RING;   // 96 KB: also the staging area of the row copies
constexpr uint32_t CTL_BYTES = 4096;            // barriers, per-example maxima, partial maxima
constexpr uint32_t SMEM_BYTES = BUF_BYTES + 1024 /*alignment*/ + CTL_BYTES;
constexpr uint32_t SMEM_BYTES_MAX = A_MAX_STAGES * A_STAGE + W_RING + 1024 + CTL_BYTES;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t MAXP_CHUNKS = 3;             // FWD maximum pass: chunks of rows per copy round, two rounds in flight
constexpr uint32_t EPI_COLS = 32;               // BWD epilogue: child rows of 32 columns per round, three rounds in flight

struct MnArgs {
  float* mars;
  float* flows;
  float* blk_mx;
  const float* w_img;
  const PcbDenseBlock* blocks;
  const PcbDenseImg* imgs;
  int* status;
  uint32_t ld;
  uint32_t nsplit;   // CTAs sharing one 256-column tile (1, 2 or 4), each taking 256 / nsplit columns
  uint32_t a_stages; // stages of the A ring (a power of two up to A_MAX_STAGES); the launch sizes shared memory to it
  uint32_t ksplit;   // CTAs sharing the K range of one tile (1, 2 or 4): each accumulates chunks / ksplit chunks
  float* part;       // ksplit > 1: per CTA a slot of 128 x (256 / nsplit + 1) floats for its partial tile
  uint32_t* tickets; // ksplit > 1: arrival counter per tile (zero between launches)
  unsigned long long* trace;   // -DPCB_DIAG builds: %globaltimer stamps of CTA (0,0,0), else null
};

// Timing stamps exist only in a build with -DPCB_DIAG; the default build compiles them out.
#ifdef PCB_DIAG
// running log of every launch (CTA (0,0,0)): [mode << 48 | blocks << 16 | ksplit, entered, dependencies done, exit]
__device__ unsigned long long g_mn_log[4 * 2048];
__device__ unsigned int g_mn_logn;
__device__ int g_mn_halfw;   // timing experiments (results are wrong): 1 half of every weight chunk, 2 no row loads in the K loop, 4 no maximum pass, 8 one MMA pass instead of three
#define MN_TRACE(slot)                                                                                   \
  do {                                                                                                   \
    if (a.trace && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[(MODE == MN_FWD ? 0 : 256) + (slot)] = gtime(); \
  } while (0)
// stamps of the CTA that completes K-split tile 0 (whichever part it is)
#define MN_TRACE_F(slot)                                                                                 \
  do {                                                                                                   \
    if (a.trace && tile_id == 0 && tid == 0) a.trace[(MODE == MN_FWD ? 0 : 256) + (slot)] = gtime();     \
  } while (0)
#else
#define MN_TRACE(slot) do { } while (0)
#define MN_TRACE_F(slot) do { } while (0)
#endif

// byte offset of element (row, kk) inside a K-major tile with 64-byte rows and 64-byte swizzle
__host__ __device__ __forceinline__ uint32_t sw64_off(uint32_t row, uint32_t kk) {
  return row * 64u + ((((kk >> 2) ^ ((row >> 1) & 3u)) << 4) | ((kk & 3u) << 2));
}
// K-major operand descriptor, 64-byte rows: 8-row groups 512 bytes apart, 64-byte swizzle
__device__ __forceinline__ uint64_t desc_k64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(512u >> 4) << 32;     // stride byte offset: next group of 8 rows
  d |= (uint64_t)1 << 46;               // descriptor version (sm_100)
  d |= (uint64_t)4 << 61;               // SWIZZLE_64B
  return d;
}
// M-major operand descriptor for a 128 x 8 slice of the A tile.  For 32-bit operands the M-major
// layout tcgen05 reads is the 128-byte swizzle with 32-byte atoms: rows of 128 bytes (32 examples)
// per K value, atoms of [4 K rows][32 examples] = 512 bytes, inside an atom the four 32-byte units
// of a row are XORed with the row index (address bits [5,7) ^= bits [7,9)).  The four atoms along
// the examples lie 512 bytes apart (leading byte offset), the next group of 4 K rows 2 KB further
// (stride byte offset); a K step of 8 takes two such groups.
__device__ __forceinline__ uint64_t desc_mn128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(512u >> 4) << 16;     // leading byte offset: next 32 examples
  d |= (uint64_t)(2048u >> 4) << 32;    // stride byte offset: next 4 K rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;               // SWIZZLE_128B with 32-byte atoms
  return d;
}
// instruction descriptor: D fp32, A/B tf32, A M-major (bit 15), B K-major, M x N
__device__ __forceinline__ uint32_t idesc_mn(uint32_t m, uint32_t n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 f4max(float4 a, float4 b) {
  return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
}

// ---- exp(theta), split and laid out as 16-deep operand tiles ---------------------------------------
// One block converts a 32 x 32 patch (rows r, columns t) of a dense block's weights and writes it to
// the FWD image (rows r, K = t) and, transposed through shared memory, to the BWD_CHILD image
// (rows t, K = r).  Image of a dense block: [column tile][K chunk of 16][hi | lo][rows x 64 bytes].
__global__ void __launch_bounds__(256) w_image16_kernel(const float* __restrict__ theta, float* __restrict__ img,
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
    const uint32_t t = t0 + tx, c = t / KC, kk = t % KC;
    for (uint32_t i = ty; i < 32; i += 8) {
      uint32_t r = r0 + i;
      if (r >= k.R || t >= k.K) continue;
      uint32_t j = r / TN, row = r % TN;
      float* base = img + im.off_f + ((size_t)(j * im.nch_f + c) * 2) * im.rows_f * KC;
      float v = tile[i][tx], h = tf32_hi(v);
      uint32_t o = sw64_off(row, kk) / 4;
      base[o] = h;
      base[(size_t)im.rows_f * KC + o] = v - h;
    }
  }
  {  // BWD_CHILD image: row = t, kk = r
    const uint32_t r = r0 + tx, c = r / KC, kk = r % KC;
    for (uint32_t i = ty; i < 32; i += 8) {
      uint32_t t = t0 + i;
      if (t >= k.K || r >= k.R) continue;
      uint32_t j = t / TN, row = t % TN;
      float* base = img + im.off_t + ((size_t)(j * im.nch_t + c) * 2) * im.rows_t * KC;
      float v = tile[tx][i], h = tf32_hi(v);
      uint32_t o = sw64_off(row, kk) / 4;
      base[o] = h;
      base[(size_t)im.rows_t * KC + o] = v - h;
    }
  }
}

// grid: (example tiles of 128, column tiles x nsplit, blocks)
//
// Roles: 8 producer warps (they also compute the per-example maximum of FWD and run the epilogue),
// one MMA thread, one weight-copy thread.  Shared memory (96 KB, two CTAs per SM): two 16 KB A
// stages and a 64 KB ring of weight chunks that the copy thread fills as far ahead as it reaches
// (2 chunks of a 256-column tile, 8 of a 64-column tile: the small layers of the chain do not wait
// for weights).  Whatever comes from global memory in bulk outside the K loop comes by cp.async.bulk
// into the same 96 KB while they are idle: the child rows of the maximum pass (FWD, before the
// weights start to arrive) and the children's value rows of the child-flow epilogue (BWD) — plain
// loads of row-strided 512-byte pieces reach a third of what the copy engine delivers.
template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 2) dense_mn_kernel(const __grid_constant__ CUtensorMap tm_rows, MnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* aring = smem;
  const uint32_t a_stages = a.a_stages, a_mask = a_stages - 1u, a_shift = 31u - __clz(a_stages);
  uint8_t* wring = smem + a_stages * A_STAGE;
  uint8_t* ctl = wring + W_RING;
  uint64_t* wfull = reinterpret_cast<uint64_t*>(ctl);         // [W_MAX_STAGES]
  uint64_t* wempty = wfull + W_MAX_STAGES;                    // [W_MAX_STAGES]
  uint64_t* afull = wempty + W_MAX_STAGES;                    // [A_MAX_STAGES]
  uint64_t* aempty = afull + A_MAX_STAGES;                    // [A_MAX_STAGES]
  uint64_t* accfull = aempty + A_MAX_STAGES;                  // [1]
  uint64_t* wgo = accfull + 1;                                // [1] FWD: the staging area is free for weights
  uint64_t* xbar = wgo + 1;                                   // [3] row-copy rounds
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 3);
  uint32_t* last_flag = tmem_slot + 1;                        // K split: this CTA completes the tile
  float* mxs = reinterpret_cast<float*>(ctl + 512);           // [128] per-example max of the tile
  float* part = reinterpret_cast<float*>(ctl + 1024);         // [PW/2][128] partial maxima (FWD)

  pcb_grid_dep_launch();
  const PcbDenseBlock k = a.blocks[blockIdx.z];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ld = a.ld;

  // ---- tile coordinates ---------------------------------------------------------------------
  const uint32_t ncols = MODE == MN_FWD ? k.R : k.K, kdim = MODE == MN_FWD ? k.K : k.R;
  const uint32_t sw = TN / a.nsplit;
  // blockIdx.y = (column tile, column part, K part)
  const uint32_t ks = a.ksplit, yk = blockIdx.y / ks, kp = blockIdx.y - yk * ks;
  const uint32_t m0 = blockIdx.x * TM, jn = yk / a.nsplit, part0 = (yk % a.nsplit) * sw;
  const uint32_t n0 = jn * TN + part0;
  if (n0 >= ncols) return;   // the same for every K part of the tile
  // this CTA's chunks cb .. cb + nchunks - 1 of the block's K range (the launch splits K only when
  // every block of the layer has a multiple of ksplit chunks)
  const uint32_t nchunks = ((kdim + KC - 1) / KC) / ks, cb = kp * nchunks;
  const uint32_t tile_id = (blockIdx.z * (gridDim.y / ks) + yk) * gridDim.x + blockIdx.x;
  const size_t slot_floats = (size_t)TM * (sw + 1u);
  const PcbDenseImg im = a.imgs[blockIdx.z];
  const uint32_t img_rows = MODE == MN_FWD ? im.rows_f : im.rows_t;
  const uint32_t nch = MODE == MN_FWD ? im.nch_f : im.nch_t;
  // first K chunk of this CTA's rows in the weight image; rows beyond the block are zero in the image
  const float* img_tile = a.w_img + (MODE == MN_FWD ? im.off_f : im.off_t) + (size_t)jn * nch * 2 * img_rows * KC + part0 * KC;
  const uint32_t n_tile = min(sw, img_rows - part0);
  const uint32_t w_part = n_tile * KC * 4u;                    // bytes of one part (hi or lo) of a weight chunk
  const uint32_t w_stages = min(W_MAX_STAGES, W_RING / (2u * w_part));
  const bool w_reuse = w_stages < nchunks;                     // else every chunk has a slot of its own
  const bool has_sub = k.d0 != PCB_NONE;
  const uint32_t ex = min(TM, ld - m0), rowb = ex * 4u;        // examples of this tile (the pitch is a multiple of 32)

  // ---- set-up: barriers, tensor memory ---------------------------------------------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < W_MAX_STAGES; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], 1); }
    for (uint32_t s = 0; s < a_stages; ++s) { mbar_init(&afull[s], PW); mbar_init(&aempty[s], 1); }
    mbar_init(accfull, 1);
    mbar_init(wgo, 1);
    for (uint32_t s = 0; s < 3; ++s) mbar_init(&xbar[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Up to here only static circuit data was read: a launch with programmatic stream serialization
  // may have come this far while the previous kernel of the stream was still running.
  if (tid == 0) MN_TRACE(0);
#ifdef PCB_DIAG
  unsigned long long log_t0 = 0, log_t1 = 0;
  if (tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) log_t0 = gtime();
#endif
  pcb_grid_dep_wait();
#ifdef PCB_DIAG
  if (tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) log_t1 = gtime();
#endif
  if (tid == 0) MN_TRACE(1);
  bool ok = true;

  if (warp < PW) {
    // =========================== producers ===================================================
    // A thread's four examples m0 + 4*lane .. +3 are the same in every chunk: lane -> (32-example
    // group, 16-byte slot); warp -> K rows warp and warp + 8 of the chunk.
    const uint32_t bq = m0 + 4u * lane;
    const bool bok = bq < ld;                  // the row pitch is a multiple of 32: a group of four is in or out as a whole
    const uint32_t bb = bok ? bq : 0u;
    const float* rowsA = MODE == MN_FWD ? a.mars + (size_t)k.c0 * ld + bb : a.mars + (size_t)k.p0 * ld + bb;
    const float* rowsB = MODE == MN_FWD ? a.mars + (size_t)(has_sub ? k.d0 : k.c0) * ld + bb : a.flows + (size_t)k.p0 * ld + bb;
    const float4 ninf4 = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    auto lds4 = [](const uint8_t* p) { return *reinterpret_cast<const float4*>(p); };
    auto wait_warp = [&](uint64_t* bar, uint32_t parity) {   // one lane polls, the warp follows
      bool got = lane != 0 || mbar_wait(bar, parity, a.status);
      return __all_sync(0xffffffffu, got);
    };

    if (MODE == MN_FWD) {
      // ---- per-example maximum of the child values over all K children ------------------------------
      // The child rows come by bulk copies, three chunks per round (slot of 16 KB per chunk: [16 prime
      // rows | 16 sub rows]), two rounds in flight through the still idle 96 KB; warp w reads rows w
      // and w + 8 of every chunk.  The K loop reads the rows again, from L2.
      uint32_t nrounds = (nchunks + MAXP_CHUNKS - 1) / MAXP_CHUNKS;
#ifdef PCB_DIAG
      if (g_mn_halfw & 4) nrounds = 1;
#endif
      auto issue_round = [&](uint32_t R) {   // called by every producer thread (one barrier inside)
        asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // the slots' readers are done
        if (tid == 0) {
          // one tensor-map copy per chunk and operand: a [16 rows][128 examples] slab as it lies in memory
          // (rows past the block belong to other nodes or are zero-filled; their values are never used)
          const uint32_t c_first = R * MAXP_CHUNKS, nc = min(MAXP_CHUNKS, nchunks - c_first);
          mbar_arrive_expect_tx(&xbar[R & 1u], nc * (has_sub ? 2u : 1u) * A_BYTES);
          for (uint32_t c = 0; c < nc; ++c) {
            uint8_t* slot = smem + ((R & 1u) * MAXP_CHUNKS + c) * A_STAGE;
            tma_load_2d(slot, &tm_rows, (int32_t)m0, (int32_t)(k.c0 + (cb + c_first + c) * KC), &xbar[R & 1u]);
            if (has_sub) tma_load_2d(slot + A_BYTES, &tm_rows, (int32_t)m0, (int32_t)(k.d0 + (cb + c_first + c) * KC), &xbar[R & 1u]);
          }
        }
      };
      float4 mx = ninf4;
      issue_round(0);
      if (nrounds > 1) issue_round(1);
      for (uint32_t R = 0; R < nrounds; ++R) {
        const bool got = wait_warp(&xbar[R & 1u], (R >> 1) & 1u);
        ok = ok && got;
#pragma unroll
        for (uint32_t c = 0; c < MAXP_CHUNKS; ++c) {
          const uint8_t* slot = smem + ((R & 1u) * MAXP_CHUNKS + c) * A_STAGE + lane * 16u;
#pragma unroll
          for (uint32_t ps = 0; ps < 2; ++ps) {
            const uint32_t row = ps * 8u + warp;
            if (got && R * MAXP_CHUNKS + c < nchunks && (cb + R * MAXP_CHUNKS + c) * KC + row < kdim) {
              float4 v = lds4(slot + row * ROW_BYTES);
              if (has_sub) { const float4 q = lds4(slot + A_BYTES + row * ROW_BYTES); v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w; }
              mx = f4max(mx, v);
            }
          }
        }
        if (R + 2 < nrounds) {   // CTA-uniform
          fence_proxy_async();   // these generic reads precede the next copies into the same slots
          issue_round(R + 2);
        }
      }
      // combine the eight warps: two rounds through shared memory
      if (warp >= PW / 2) *reinterpret_cast<float4*>(part + (warp - PW / 2) * 128u + 4u * lane) = mx;
      fence_proxy_async();
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // also: every read of the staging area is done
      if (tid == 0) mbar_arrive(wgo);                              // the weight copies may start
      if (warp < PW / 2) mx = f4max(mx, *reinterpret_cast<const float4*>(part + warp * 128u + 4u * lane));
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
      if (warp < PW / 2) *reinterpret_cast<float4*>(part + warp * 128u + 4u * lane) = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
#pragma unroll
      for (uint32_t u = 0; u < PW / 2; ++u) mx = f4max(mx, *reinterpret_cast<const float4*>(part + u * 128u + 4u * lane));
      if (!bok) mx = ninf4;
      if (warp == 0) {
        *reinterpret_cast<float4*>(mxs + 4u * lane) = mx;   // for the epilogue (read after the barrier behind the K loop)
        // kept for the backward kernels (one CTA per example tile writes; with a K split the CTA that
        // completes the tile writes the maximum over all parts)
        if (bok && blockIdx.y == 0 && ks == 1) *reinterpret_cast<float4*>(a.blk_mx + (size_t)k.mx_row * ld + bq) = mx;
      }
      if (tid == 0) MN_TRACE(2);   // per-example maximum known
      // a masked example (outside the batch, or no child possible): exp(x - inf) = 0
      if (mx.x == -INFINITY) mx.x = INFINITY;
      if (mx.y == -INFINITY) mx.y = INFINITY;
      if (mx.z == -INFINITY) mx.z = INFINITY;
      if (mx.w == -INFINITY) mx.w = INFINITY;
      {
        const float4 mx4 = mx;
        // byte offset of this thread's 16 bytes inside an A part: K row kr = 8 * pass + warp lies in row
        // kr % 4 of the atom (kr / 4, lane / 8); the lane's 32-byte unit (lane % 8) / 2 is XORed with the row
        const uint32_t r4 = warp & 3u;
        const uint32_t aoff = ((warp >> 2) * 4u + (lane >> 3)) * 512u + r4 * 128u + (((((lane & 7u) >> 1) ^ r4)) << 5) +
                              ((lane & 1u) << 4);
        struct Regs { float4 x[2], y[2]; };
        auto load = [&](uint32_t i, Regs& r) {
#ifdef PCB_DIAG
          if ((g_mn_halfw & 2) && i > 0) return;
#endif
#pragma unroll
          for (uint32_t ps = 0; ps < 2; ++ps) {
            const uint32_t t = (cb + i) * KC + ps * 8u + warp;
            const size_t o = (size_t)(t < kdim ? t : 0u) * ld;
            r.x[ps] = ldg4(rowsA + o);
            if (has_sub) r.y[ps] = ldg4(rowsB + o);
          }
        };
        auto process = [&](uint32_t i, const Regs& r) -> bool {
          const uint32_t s = i & a_mask, ph = (i >> a_shift) & 1u;
          if (!wait_warp(&aempty[s], ph ^ 1u)) return false;
          uint8_t* a_hi = aring + s * A_STAGE;
#pragma unroll
          for (uint32_t ps = 0; ps < 2; ++ps) {
            float4 v = r.x[ps];
            if (has_sub) { v.x += r.y[ps].x; v.y += r.y[ps].y; v.z += r.y[ps].z; v.w += r.y[ps].w; }
            v.x = __expf(v.x - mx4.x); v.y = __expf(v.y - mx4.y); v.z = __expf(v.z - mx4.z); v.w = __expf(v.w - mx4.w);
            if ((cb + i) * KC + ps * 8u + warp >= kdim) v = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
            const uint32_t o = aoff + ps * 4096u;
            *reinterpret_cast<float4*>(a_hi + o) = h;
            *reinterpret_cast<float4*>(a_hi + A_BYTES + o) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
          }
          fence_proxy_async();   // make the generic-proxy writes visible to the tensor core
          __syncwarp();
          if (lane == 0) mbar_arrive(&afull[s]);
          if (tid == 0 && i < 32) MN_TRACE(16 + i);   // chunk i stored
          return true;
        };
        Regs r0, r1;
        load(0, r0);
        for (uint32_t i = 0; i < nchunks && ok; i += 2) {
          if (i + 1 < nchunks) load(i + 1, r1);
          ok = process(i, r0);
          if (!ok || i + 1 >= nchunks) break;
          if (i + 2 < nchunks) load(i + 2, r0);
          ok = process(i + 1, r1);
        }
      }
    } else {
      // ---- G = flows * exp(mx - mars) of the parents; the loads of chunk i + 1 are in flight while chunk i is stored
      const float* mxrow = a.blk_mx + (size_t)k.mx_row * ld;
      float4 mx4 = bok ? *reinterpret_cast<const float4*>(mxrow + bq) : ninf4;   // -inf: exp(-inf - m) = 0
      if (tid < 128) mxs[tid] = (m0 + tid < ld) ? mxrow[m0 + tid] : -INFINITY;
      const uint32_t r4 = warp & 3u;
      const uint32_t aoff = ((warp >> 2) * 4u + (lane >> 3)) * 512u + r4 * 128u + (((((lane & 7u) >> 1) ^ r4)) << 5) +
                            ((lane & 1u) << 4);
      struct Regs { float4 x[2], y[2]; };
      auto load = [&](uint32_t i, Regs& r) {
#pragma unroll
        for (uint32_t ps = 0; ps < 2; ++ps) {
          const uint32_t t = (cb + i) * KC + ps * 8u + warp;
          const size_t o = (size_t)(t < kdim ? t : 0u) * ld;
          r.x[ps] = ldg4(rowsA + o);
          r.y[ps] = ldg4(rowsB + o);
        }
      };
      auto process = [&](uint32_t i, const Regs& r) -> bool {
        const uint32_t s = i & a_mask, ph = (i >> a_shift) & 1u;
        if (!wait_warp(&aempty[s], ph ^ 1u)) return false;
        uint8_t* a_hi = aring + s * A_STAGE;
#pragma unroll
        for (uint32_t ps = 0; ps < 2; ++ps) {
          float4 v;   // x: mars of the parent, y: flows of the parent
          v.x = r.y[ps].x * __expf(mx4.x - r.x[ps].x); v.y = r.y[ps].y * __expf(mx4.y - r.x[ps].y);
          v.z = r.y[ps].z * __expf(mx4.z - r.x[ps].z); v.w = r.y[ps].w * __expf(mx4.w - r.x[ps].w);
          if ((cb + i) * KC + ps * 8u + warp >= kdim) v = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
          const uint32_t o = aoff + ps * 4096u;
          *reinterpret_cast<float4*>(a_hi + o) = h;
          *reinterpret_cast<float4*>(a_hi + A_BYTES + o) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&afull[s]);
        if (tid == 0 && i < 32) MN_TRACE(16 + i);
        return true;
      };
      Regs r0, r1;
      load(0, r0);
      for (uint32_t i = 0; i < nchunks && ok; i += 2) {
        if (i + 1 < nchunks) load(i + 1, r1);
        ok = process(i, r0);
        if (!ok || i + 1 >= nchunks) break;
        if (i + 2 < nchunks) load(i + 2, r0);
        ok = process(i + 1, r1);
      }
    }
    if (tid == 0) MN_TRACE(3);   // last chunk stored
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // mxs is complete for every epilogue warp

    // =========================== epilogue ====================================================
    if (ok && lane == 0) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (tid == 0) MN_TRACE(4);   // accumulator complete
    const uint32_t q4 = warp & 3, half = warp >> 2;   // warp -> (TMEM lane quarter, column half)
    const uint32_t row = q4 * 32 + lane, b = m0 + row;
    const float mx = mxs[row];
    float acc[16];
    // K split: every CTA of the tile leaves its partial accumulators (and, FWD, the maximum they are
    // relative to) in its slot and takes a ticket; the CTA that draws the last ticket completes the
    // tile from its own tensor memory and the other slots.  Nobody waits for anybody.
    float* my_slot = ks > 1 ? a.part + ((size_t)tile_id * ks + kp) * slot_floats : nullptr;
    auto take_ticket = [&]() -> bool {   // called by every producer thread
      __threadfence();                   // this thread's slot writes are visible before the ticket is
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
      if (tid == 0) {
        const uint32_t t = atomicAdd(a.tickets + tile_id, 1u);
        const bool last = t == ks - 1u;
        if (last) a.tickets[tile_id] = 0u;   // ready for the next launch
        __threadfence();
        *last_flag = last ? 1u : 0u;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
      return *last_flag != 0u;
    };
    if (MODE == MN_FWD) {
      // a thread owns one example and walks 16 columns at a time
      const uint32_t CG = max(16u, ((n_tile + 31u) / 32u) * 16u);   // columns per half, a multiple of 16
      const uint32_t c_begin = half * CG, c_end = min(n_tile, c_begin + CG);
      bool finish = true;
      float gm = mx, own_scale = 1.0f, sc[3] = {0.f, 0.f, 0.f};
      const float* oslot[3] = {nullptr, nullptr, nullptr};   // the other parts' slots: parts kp + 1 + q (mod ksplit)
      if (ks > 1) {
        if (ok) {
          tc_fence_after();
          if (half == 0) my_slot[row] = mx;
          for (uint32_t c0 = c_begin; c0 < c_end; c0 += 16) {
            tmem_ld16(tmem_base + ((q4 * 32u) << 16) + c0, acc);
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j) my_slot[TM + (size_t)(c0 + j) * TM + row] = acc[j];
          }
        }
        finish = take_ticket();
        if (finish) MN_TRACE_F(7);
        if (finish) {
          // the sums of a part are relative to its own maximum: rescale to the maximum over the parts
          float pm[3];
#pragma unroll
          for (uint32_t q = 0; q < 3; ++q) {
            oslot[q] = a.part + ((size_t)tile_id * ks + ((kp + 1u + q) & (ks - 1u))) * slot_floats;
            pm[q] = q + 1u < ks ? __ldcg(oslot[q] + row) : -INFINITY;
            gm = fmaxf(gm, pm[q]);
          }
#pragma unroll
          for (uint32_t q = 0; q < 3; ++q) sc[q] = pm[q] != -INFINITY ? __expf(pm[q] - gm) : 0.0f;
          own_scale = mx == -INFINITY ? 0.0f : __expf(mx - gm);
          if (yk == 0 && half == 0 && b < ld) a.blk_mx[(size_t)k.mx_row * ld + b] = gm;
        }
      }
      if (ok && finish) {
        tc_fence_after();
        for (uint32_t c0 = c_begin; c0 < c_end; c0 += 16) {
          float pv[3][16];
          if (ks > 1 && b < ld) {   // all loads of the round first: one latency, not one per part
#pragma unroll
            for (uint32_t q = 0; q < 3; ++q) {
              if (q + 1u < ks) {
                const float* ps = oslot[q] + TM + (size_t)c0 * TM + row;
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) pv[q][j] = __ldcg(ps + (size_t)j * TM);
              }
            }
          }
          tmem_ld16(tmem_base + ((q4 * 32u) << 16) + c0, acc);
          if (b >= ld) continue;
          if (ks > 1) {
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j) acc[j] *= own_scale;
#pragma unroll
            for (uint32_t q = 0; q < 3; ++q) {
              if (q + 1u < ks) {
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) acc[j] = fmaf(pv[q][j], sc[q], acc[j]);
              }
            }
          }
#pragma unroll
          for (uint32_t j = 0; j < 16; ++j) {
            const uint32_t r = n0 + c0 + j;
            if (r < k.R) a.mars[(size_t)(k.p0 + r) * ld + b] = gm == -INFINITY ? -INFINITY : __logf(acc[j]) + gm;
          }
        }
      }
      if (ks > 1 && finish) MN_TRACE_F(8);
    } else {
      // Child flows f[t][b] = acc[b][t] * exp(M[t][b] - mx[b]) need the children's value rows: copied 32
      // columns per round into the idle 96 KB (32 KB per round: [32 prime rows | 32 sub rows]), three
      // rounds in flight; warp (q4, half) takes columns 16 half .. 16 half + 15 of every round.
      const uint32_t nrounds = (n_tile + EPI_COLS - 1) / EPI_COLS;
      const uint32_t per = has_sub ? 2u : 1u;
      auto issue_round = [&](uint32_t R) {   // called by every producer thread (one barrier inside)
        asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");   // the buffer's readers are done
        if (tid == 0) {
          // buffer: [32 prime rows | 32 sub rows] of 512 bytes, fetched as slabs of 16 rows
          const uint32_t c_first = R * EPI_COLS;
          const uint32_t groups = c_first + 16u < ncols - n0 ? 2u : 1u;
          uint8_t* buf = smem + (R % 3u) * (EPI_COLS * 1024u);
          mbar_arrive_expect_tx(&xbar[R % 3u], groups * per * A_BYTES);
          for (uint32_t g = 0; g < groups; ++g) {
            tma_load_2d(buf + g * A_BYTES, &tm_rows, (int32_t)m0, (int32_t)(k.c0 + n0 + c_first + g * 16u), &xbar[R % 3u]);
            if (has_sub)
              tma_load_2d(buf + EPI_COLS * ROW_BYTES + g * A_BYTES, &tm_rows, (int32_t)m0, (int32_t)(k.d0 + n0 + c_first + g * 16u), &xbar[R % 3u]);
          }
        }
      };
      // The first rounds of child rows are requested before the hand-over of a K split: every CTA of
      // the tile fetches them although only the completing one uses them, whose epilogue then starts
      // with the rows already there (these layers leave the memory system idle).
      fence_proxy_async();
      const uint32_t first_rounds = min(3u, nrounds);
      for (uint32_t R = 0; R < first_rounds; ++R) issue_round(R);
      bool finish = true;
      if (ks > 1) {   // the partial sums are linear in the K range: the completing CTA adds the other slots
        if (ok) {
          tc_fence_after();
          for (uint32_t c0 = half * 16u; c0 < n_tile; c0 += EPI_COLS) {
            tmem_ld16(tmem_base + ((q4 * 32u) << 16) + c0, acc);
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j) my_slot[TM + (size_t)(c0 + j) * TM + row] = acc[j];
          }
        }
        finish = take_ticket();
        if (finish) MN_TRACE_F(7);
        if (!finish)   // the copies in flight land before the CTA gives its memory back
          for (uint32_t R = 0; R < first_rounds; ++R) wait_warp(&xbar[R], 0u);
      }
      for (uint32_t R = 0; R < nrounds && finish; ++R) {
        const bool got = wait_warp(&xbar[R % 3u], (R / 3u) & 1u);
        const uint32_t c0 = R * EPI_COLS + half * 16u;   // first column of this warp in the round (within the CTA's tile)
        if (c0 < n_tile) {
          float pv[3][16];
          if (ok && ks > 1) {   // all loads of the round first: one latency, not one per part
#pragma unroll
            for (uint32_t q = 0; q < 3; ++q) {
              if (q + 1u < ks) {
                const float* ps = a.part + ((size_t)tile_id * ks + ((kp + 1u + q) & (ks - 1u))) * slot_floats + TM + (size_t)c0 * TM + row;
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) pv[q][j] = __ldcg(ps + (size_t)j * TM);
              }
            }
          }
          if (ok) { tc_fence_after(); tmem_ld16(tmem_base + ((q4 * 32u) << 16) + c0, acc); }
          if (ok && ks > 1) {
#pragma unroll
            for (uint32_t q = 0; q < 3; ++q) {
              if (q + 1u < ks) {
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) acc[j] += pv[q][j];
              }
            }
          }
          if (ok && got && b < ld) {
            const uint8_t* sp = smem + (R % 3u) * (EPI_COLS * 1024u) + (half * 16u) * ROW_BYTES + row * 4u;
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j) {
              const uint32_t t = n0 + c0 + j;
              if (t < k.K) {
                float cv = *reinterpret_cast<const float*>(sp + j * ROW_BYTES);
                if (has_sub) cv += *reinterpret_cast<const float*>(sp + EPI_COLS * ROW_BYTES + j * ROW_BYTES);
                const float f = mx == -INFINITY ? 0.0f : acc[j] * __expf(cv - mx);
                a.flows[(size_t)(k.c0 + t) * ld + b] = f;
                if (has_sub) a.flows[(size_t)(k.d0 + t) * ld + b] = f;
              }
            }
          }
        }
        if (R + 3 < nrounds) {   // CTA-uniform
          fence_proxy_async();   // these generic reads precede the next copies into the same buffer
          issue_round(R + 3);
        }
      }
    }
    if (MODE != MN_FWD && ks > 1) MN_TRACE_F(8);   // (only the completing CTA gets here with work done; others stamp earlier)
    if (tid == 0) MN_TRACE(5);   // epilogue of warp 0 done
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      const uint32_t idesc = idesc_mn(TM, n_tile);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t sa = i & a_mask, pa = (i >> a_shift) & 1u;
        const uint32_t sb = i % w_stages, pb = (i / w_stages) & 1u;
        ok = mbar_wait(&wfull[sb], pb, a.status) && mbar_wait(&afull[sa], pa, a.status);
        if (i < 32) MN_TRACE(96 + i);    // operands of chunk i ready
        if (!ok) break;
        tc_fence_after();
        const uint32_t aa = smem_u32(aring + sa * A_STAGE), wa = smem_u32(wring + sb * 2u * w_part);
#pragma unroll
        for (uint32_t ks = 0; ks < KC / 8; ++ks) {
          // A: the next 8 K rows are the next eight atoms (4 KB); W: 8 tf32 = 32 bytes along the row
          const uint64_t d_ahi = desc_mn128(aa + ks * 4096u), d_alo = desc_mn128(aa + A_BYTES + ks * 4096u);
          const uint64_t d_bhi = desc_k64(wa) + (uint64_t)((ks * 32u) >> 4);
          const uint64_t d_blo = desc_k64(wa + w_part) + (uint64_t)((ks * 32u) >> 4);
          umma_tf32(tmem_base, d_ahi, d_bhi, idesc, (i | ks) ? 1u : 0u);
#ifdef PCB_DIAG
          if (g_mn_halfw & 8) continue;   // timing experiment: one pass instead of three
#endif
          umma_tf32(tmem_base, d_alo, d_bhi, idesc, 1u);
          umma_tf32(tmem_base, d_ahi, d_blo, idesc, 1u);
        }
        umma_commit(&aempty[sa]);              // the A stage may be refilled once these MMAs have read it
        if (w_reuse) umma_commit(&wempty[sb]);
      }
      if (ok) umma_commit(accfull);
    }
    __syncwarp();
  } else {
    // =========================== weight copies ===============================================
    if (lane == 0) {
      // FWD: the ring doubles as the staging area of the maximum pass; wait until it has been read
      bool go = MODE != MN_FWD || mbar_wait(wgo, 0, a.status);
      uint32_t issued = 0;
      for (uint32_t i = 0; i < nchunks && go; ++i) {
        const uint32_t sb = i % w_stages, pb = (i / w_stages) & 1u;
        if (w_reuse && !mbar_wait(&wempty[sb], pb ^ 1u, a.status)) break;
        uint8_t* dst = wring + sb * 2u * w_part;
        const float* src = img_tile + (size_t)(cb + i) * 2 * img_rows * KC;   // hi part, then lo part img_rows x 16 floats later
        if (i < 32) MN_TRACE(128 + i);   // copies of chunk i issued
#ifdef PCB_DIAG
        const uint32_t wb = (g_mn_halfw & 1) ? w_part / 2 : w_part;
#else
        const uint32_t wb = w_part;
#endif
        mbar_arrive_expect_tx(&wfull[sb], 2u * wb);
        bulk_g2s(dst, src, wb, &wfull[sb]);
        bulk_g2s(dst + w_part, src + (size_t)img_rows * KC, wb, &wfull[sb]);
        issued = i + 1;
      }
      if (issued < nchunks) {
        // a wait was lost: let the copies already issued land before the CTA gives its memory back
        for (uint32_t j = issued > w_stages ? issued - w_stages : 0; j < issued; ++j)
          mbar_wait(&wfull[j % w_stages], (j / w_stages) & 1u, a.status);
      }
    }
    __syncwarp();
  }

  // ---- common exit: release tensor memory ---------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0) MN_TRACE(6);
#ifdef PCB_DIAG
  if (tid == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) {
    const unsigned int i = atomicAdd(&g_mn_logn, 1u) % 2048u;
    g_mn_log[4 * i] = ((unsigned long long)MODE << 48) | ((unsigned long long)gridDim.z << 16) | a.ksplit;
    g_mn_log[4 * i + 1] = log_t0; g_mn_log[4 * i + 2] = log_t1; g_mn_log[4 * i + 3] = gtime();
  }
#endif
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int MODE>
int32_t launch(dim3 grid, const pcb_workspace* ws, const MnArgs& args, cudaStream_t st, bool pdl) {
  if (!ws->have_tm_rows)
    return pcb_fail(PCB_ERR_CUDA, "cuTensorMapEncodeTiled is not available: the dense-block kernels cannot fetch their row slabs");
  static PcbPerDeviceOnce once;
  PCB_CUDA(once.run([] {
    return cudaFuncSetAttribute(dense_mn_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES_MAX);
  }));
  alignas(64) CUtensorMap tm;
  memcpy(&tm, ws->tm_rows, sizeof(tm));
  const uint32_t smem = args.a_stages * A_STAGE + W_RING + 1024 + CTL_BYTES;
  PCB_CUDA(pcb_launch_pdl(dense_mn_kernel<MODE>, grid, dim3(NTHREADS), smem, st, pdl, tm, args));
  return PCB_OK;
}

#ifdef PCB_DIAG
unsigned long long* g_mn_trace = nullptr;
uint32_t g_mn_minz = 0, g_mn_maxz = 0xffffffffu;   // only launches with that many blocks are traced
void mn_diag_switches() {
  static bool done = false;
  if (done) return;
  done = true;
  int v = getenv("PCB_MN_HALFW") ? atoi(getenv("PCB_MN_HALFW")) : 0;
  cudaMemcpyToSymbol(g_mn_halfw, &v, sizeof(v));
}
unsigned long long* mn_trace() {
  mn_diag_switches();
  if (!g_mn_trace && getenv("PCB_TC_TRACE")) {
    if (const char* e = getenv("PCB_TC_TRACE_MINZ")) g_mn_minz = (uint32_t)atoi(e);
    if (const char* e = getenv("PCB_TC_TRACE_MAXZ")) g_mn_maxz = (uint32_t)atoi(e);
    cudaMalloc((void**)&g_mn_trace, 512 * sizeof(unsigned long long));
    cudaMemset(g_mn_trace, 0, 512 * sizeof(unsigned long long));
  }
  return g_mn_trace;
}
unsigned long long* mn_trace_for(uint32_t blocks) {
  unsigned long long* t = mn_trace();
  return (t && blocks >= g_mn_minz && blocks <= g_mn_maxz) ? t : nullptr;
}
#else
unsigned long long* mn_trace() { return nullptr; }
unsigned long long* mn_trace_for(uint32_t) { return nullptr; }
#endif

// A layer that would not fill the GPU (two CTAs per SM) with 256-column tiles is cut into narrower
// tiles: the CTAs of one tile repeat the production of the data-dependent operand, but each has
// half (a quarter) of the weight tile to fetch, of the MMAs to wait for and of the epilogue.
// A launch of at most one CTA per SM has the shared memory of a whole SM to itself: the A ring then
// holds eight chunks, so the producers of a small layer never wait for the tensor core to hand a
// stage back (with two stages that round trip, not the loads, paces the K loop of such a launch).
uint32_t pick_a_stages(dim3 grid, const pcb_circuit* c) {
  if (c->tc_a_stages) return (uint32_t)c->tc_a_stages;
  return (uint64_t)grid.x * grid.y * grid.z <= 148 ? A_MAX_STAGES : A_STAGES;
}

// A layer that still leaves most of the GPU idle after the column split also splits the K range:
// four CTAs accumulate a quarter of the chunks each, leave their partial tiles in a scratch slot and
// the one that finishes last completes the tile.  The K loop, which the single issuing thread paces
// (about 0.75 us per chunk), is the longest piece of such a layer's kernel, and these layers form
// the dependent chain of the circuit.  Measured per layer of one 256 x 256 block at 2048 examples:
// forward 22.2 -> 15.6 us, child flows 24.0 -> 19.5 us; a two-way split (layers of two blocks) gains
// nothing over the cost of the hand-over and is only taken when forced (PCB_TC_KSPLIT=2).  Only
// when every block of the layer has a multiple of ksplit chunks with at least two chunks per part,
// and while the launch stays within two CTAs per SM.
template <class Blocks>
uint32_t pick_ksplit(uint32_t ctas, const Blocks& blocks, uint32_t o0, uint32_t o1, bool fwd, int forced) {
  if (forced == 1) return 1;
  for (uint32_t ks = 4; ks >= 2; ks >>= 1) {
    if (forced && (uint32_t)forced != ks) continue;
    if ((uint64_t)ctas * ks > 296) continue;
    bool fits = true;
    for (uint32_t i = o0; i < o1 && fits; ++i) {
      const uint32_t nch = ((fwd ? blocks[i].K : blocks[i].R) + KC - 1) / KC;
      fits = nch % ks == 0 && nch / ks >= 2;
    }
    if (fits) return ks;
  }
  return 1;
}

uint32_t pick_nsplit(uint32_t ctas, uint32_t max_cols, int forced) {
  if (forced == 1 || forced == 2 || forced == 4) return (uint32_t)forced;
  uint32_t n = 1;
  while (n < 4 && ctas * n * 2 <= 296 && max_cols > TN / (2 * n)) n *= 2;
  return n;
}

}  // namespace

#define PCB_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != PCB_OK) return _s;   \
  } while (0)

// Lays out the 16-deep weight images of every dense block and allocates them.
int32_t pcb_dense_mn_prepare(pcb_circuit* c, uint64_t* bytes) {
  std::vector<PcbDenseImg> imgs(c->h_dense.size());
  uint64_t off = 0;
  for (size_t i = 0; i < c->h_dense.size(); ++i) {
    const PcbDenseBlock& k = c->h_dense[i];
    PcbDenseImg& im = imgs[i];
    im.rows_f = std::min<uint32_t>(TN, pcb_round_up(k.R, 16));
    im.rows_t = std::min<uint32_t>(TN, pcb_round_up(k.K, 16));
    im.nch_f = (k.K + KC - 1) / KC;
    im.nch_t = (k.R + KC - 1) / KC;
    uint64_t tiles_f = (k.R + TN - 1) / TN, tiles_t = (k.K + TN - 1) / TN;
    im.off_f = off; off += tiles_f * im.nch_f * 2 * im.rows_f * KC;
    im.off_t = off; off += tiles_t * im.nch_t * 2 * im.rows_t * KC;
  }
  c->w_img16_len = off;
  PCB_CUDA(cudaMalloc((void**)&c->w_img16, std::max<uint64_t>(off, 1) * sizeof(float)));
  PCB_CUDA(cudaMemset(c->w_img16, 0, std::max<uint64_t>(off, 1) * sizeof(float)));  // padding rows / columns stay zero
  PCB_CUDA(cudaMalloc((void**)&c->dense_img16, std::max<size_t>(imgs.size(), 1) * sizeof(PcbDenseImg)));
  if (!imgs.empty())
    PCB_CUDA(cudaMemcpy(c->dense_img16, imgs.data(), imgs.size() * sizeof(PcbDenseImg), cudaMemcpyHostToDevice));
  *bytes += off * sizeof(float) + imgs.size() * sizeof(PcbDenseImg);
  return PCB_OK;
}

// Regenerates the 16-deep weight images (the caller tracks whether the parameters changed).
int32_t pcb_dense_mn_refresh(pcb_circuit* c, cudaStream_t st) {
  for (uint32_t z0 = 0; z0 < c->n_dense; z0 += 65535) {
    uint32_t nz = std::min<uint32_t>(65535, c->n_dense - z0);
    dim3 grid((c->max_dense_K + 31) / 32, (c->max_dense_R + 31) / 32, nz);
    PcbProfScope ps(c, st, PCB_K_W_IMAGE);
    w_image16_kernel<<<grid, 256, 0, st>>>(c->theta, c->w_img16, c->dense + z0, c->dense_img16 + z0);
  }
  return PCB_OK;
}

// Diagnostic (-DPCB_DIAG builds with PCB_TC_TRACE set): the stamps of the last traced launches,
// forward in words [0, 256), child flows in [256, 512); null otherwise.
unsigned long long* pcb_dense_mn_trace() { return mn_trace(); }
#ifdef PCB_DIAG
// Diagnostic builds only: the running launch log (4 words per launch, the last 2048 launches) and its count.
extern "C" int32_t pcb_debug_mn_log(unsigned long long* out, unsigned int* n, int reset) {
  cudaDeviceSynchronize();
  if (out && cudaMemcpyFromSymbol(out, g_mn_log, sizeof(g_mn_log)) != cudaSuccess) return PCB_ERR_CUDA;
  if (n && cudaMemcpyFromSymbol(n, g_mn_logn, sizeof(unsigned int)) != cudaSuccess) return PCB_ERR_CUDA;
  if (reset) { unsigned int z = 0; cudaMemcpyToSymbol(g_mn_logn, &z, sizeof(z)); }
  return PCB_OK;
}
#endif

int32_t pcb_dense_mn_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM, ct = (c->max_dense_R + TN - 1) / TN;
  MnArgs args{ws->mars, ws->flows, ws->blk_mx, c->w_img16, c->dense + o0, c->dense_img16 + o0, c->status, ws->ld,
              pick_nsplit(bt * ct * (o1 - o0), c->max_dense_R, c->tc_nsplit), A_STAGES, 1, ws->mn_part, ws->mn_tickets,
              mn_trace_for(o1 - o0)};
  args.ksplit = ws->mn_part ? pick_ksplit(bt * ct * args.nsplit * (o1 - o0), c->h_dense, o0, o1, true, c->tc_ksplit) : 1;
  dim3 grid(bt, ct * args.nsplit * args.ksplit, o1 - o0);
  args.a_stages = pick_a_stages(grid, c);
  PcbProfScope ps(c, st, PCB_K_DENSE_FWD);
  return launch<MN_FWD>(grid, ws, args, st, c->pdl);
}

int32_t pcb_dense_mn_backward_child(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM, ct = (c->max_dense_K + TN - 1) / TN;
  MnArgs args{ws->mars, ws->flows, ws->blk_mx, c->w_img16, c->dense + o0, c->dense_img16 + o0, c->status, ws->ld,
              pick_nsplit(bt * ct * (o1 - o0), c->max_dense_K, c->tc_nsplit), A_STAGES, 1, ws->mn_part, ws->mn_tickets,
              mn_trace_for(o1 - o0)};
  args.ksplit = ws->mn_part ? pick_ksplit(bt * ct * args.nsplit * (o1 - o0), c->h_dense, o0, o1, false, c->tc_ksplit) : 1;
  dim3 grid(bt, ct * args.nsplit * args.ksplit, o1 - o0);
  args.a_stages = pick_a_stages(grid, c);
  PcbProfScope ps(c, st, PCB_K_DENSE_BWD_CHILD);
  return launch<MN_BWD_CHILD>(grid, ws, args, st, c->pdl);
}
