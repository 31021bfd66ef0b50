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
#include <algorithm>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {
using namespace pcbtc;

enum { MN_FWD = 0, MN_BWD_CHILD = 1 };

constexpr uint32_t TM = 128;            // examples per tile (TMEM lanes)
constexpr uint32_t TN = 256;            // columns per tile (TMEM columns)
constexpr uint32_t KC = 16;             // K values per stage
constexpr uint32_t STAGES = 2;
constexpr uint32_t PW = 8;              // producer warps
constexpr uint32_t NPROD = PW * 32;
constexpr uint32_t NTHREADS = NPROD + 32;
constexpr uint32_t A_BYTES = TM * KC * 4;       // one A part (hi or lo): 16 swizzle atoms of 512 bytes
constexpr uint32_t B_BYTES = TN * KC * 4;       // one W part (hi or lo): 256 rows x 64 bytes
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;   // 48 KB
constexpr uint32_t CTL_BYTES = 4096;            // barriers, per-example maxima, partial maxima
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + CTL_BYTES;
constexpr uint32_t TMEM_COLS = 256;

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
};

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
template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 2) dense_mn_kernel(MnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctl = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);          // [STAGES]
  uint64_t* empty = full + STAGES;                            // [STAGES]
  uint64_t* accfull = empty + STAGES;                         // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);
  float* mxs = reinterpret_cast<float*>(ctl + 128);           // [128] per-example max of the tile
  float* part = reinterpret_cast<float*>(ctl + 1024);         // [PW/2][128] partial maxima (FWD)

  pcb_grid_dep_launch();
  const PcbDenseBlock k = a.blocks[blockIdx.z];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ld = a.ld;

  // ---- tile coordinates ---------------------------------------------------------------------
  const uint32_t ncols = MODE == MN_FWD ? k.R : k.K, kdim = MODE == MN_FWD ? k.K : k.R;
  const uint32_t sw = TN / a.nsplit;
  const uint32_t m0 = blockIdx.x * TM, jn = blockIdx.y / a.nsplit, part0 = (blockIdx.y % a.nsplit) * sw;
  const uint32_t n0 = jn * TN + part0;
  if (n0 >= ncols) return;
  const uint32_t n_count = min(sw, ncols - n0);
  const uint32_t nchunks = (kdim + KC - 1) / KC;
  const PcbDenseImg im = a.imgs[blockIdx.z];
  const uint32_t img_rows = MODE == MN_FWD ? im.rows_f : im.rows_t;
  const uint32_t nch = MODE == MN_FWD ? im.nch_f : im.nch_t;
  // first K chunk of this CTA's rows in the weight image; rows beyond n_count are zero in the image
  const float* img_tile = a.w_img + (MODE == MN_FWD ? im.off_f : im.off_t) + (size_t)jn * nch * 2 * img_rows * KC + part0 * KC;
  const uint32_t n_tile = min(sw, img_rows - part0);
  const bool has_sub = k.d0 != PCB_NONE;

  // ---- set-up: barriers, tensor memory ---------------------------------------------------------
  if (tid == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) { mbar_init(&full[s], PW); mbar_init(&empty[s], 1); }
    mbar_init(accfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == PW) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Up to here only static circuit data was read: a launch with programmatic stream serialization
  // may have come this far while the previous kernel of the stream was still running.
  pcb_grid_dep_wait();

  // A thread's four examples m0 + 4*lane .. +3 are the same in every pass: lane -> (32-example group,
  // 16-byte slot), warp -> K row of the chunk
  const uint32_t bq = m0 + 4u * lane;
  const bool bok = bq < ld;                  // the row pitch is a multiple of 32: a group of four is in or out as a whole
  const uint32_t bb = bok ? bq : 0u;
  const float* rowsA = MODE == MN_FWD ? a.mars + (size_t)k.c0 * ld + bb : a.mars + (size_t)k.p0 * ld + bb;
  const float* rowsB = MODE == MN_FWD ? a.mars + (size_t)(has_sub ? k.d0 : k.c0) * ld + bb : a.flows + (size_t)k.p0 * ld + bb;

  if (MODE == MN_FWD && warp < PW) {
    // ---- per-example maximum of the child values over all K children ------------------------------
    // Warp w scans K rows w, w + 8, ...: one coalesced 512-byte request per row (and per sub row);
    // eight rows are requested before the first is used.  The K loop reads the rows again from L2.
    float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    for (uint32_t t0 = 0; t0 < kdim; t0 += 8 * PW) {
      float4 p[8], q[8];
#pragma unroll
      for (uint32_t u = 0; u < 8; ++u) {
        const uint32_t t = t0 + u * PW + warp;
        const size_t o = (size_t)(t < kdim ? t : 0u) * ld;
        p[u] = ldg4(rowsA + o);
        if (has_sub) q[u] = ldg4(rowsB + o);
      }
#pragma unroll
      for (uint32_t u = 0; u < 8; ++u) {
        const uint32_t t = t0 + u * PW + warp;
        if (t < kdim) {
          float4 v = p[u];
          if (has_sub) { v.x += q[u].x; v.y += q[u].y; v.z += q[u].z; v.w += q[u].w; }
          mx = f4max(mx, v);
        }
      }
    }
    // combine the eight warps: two rounds through shared memory
    if (warp >= PW / 2) *reinterpret_cast<float4*>(part + (warp - PW / 2) * 128u + 4u * lane) = mx;
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
    if (warp < PW / 2) {
      mx = f4max(mx, *reinterpret_cast<const float4*>(part + warp * 128u + 4u * lane));
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
    if (warp < PW / 2) *reinterpret_cast<float4*>(part + warp * 128u + 4u * lane) = mx;
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
    if (warp == 0) {
#pragma unroll
      for (uint32_t u = 1; u < PW / 2; ++u) mx = f4max(mx, *reinterpret_cast<const float4*>(part + u * 128u + 4u * lane));
      if (!bok) mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      *reinterpret_cast<float4*>(mxs + 4u * lane) = mx;
      // kept for the backward kernels (one CTA per example tile writes)
      if (bok && blockIdx.y == 0) *reinterpret_cast<float4*>(a.blk_mx + (size_t)k.mx_row * ld + bq) = mx;
    }
  }
  if (MODE == MN_BWD_CHILD && tid < 128) {
    const float* mxrow = a.blk_mx + (size_t)k.mx_row * ld;
    mxs[tid] = (m0 + tid < ld) ? mxrow[m0 + tid] : -INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp < PW) {
    // =========================== producers ===================================================
    // Chunk i = K rows 16 i .. 16 i + 15; warp w takes rows w and w + 8 of the chunk.  The loads of
    // chunk i + 1 are in flight while chunk i is transformed and stored.
    float4 mx4 = *reinterpret_cast<const float4*>(mxs + 4u * lane);
    // a masked example (outside the batch, or no child possible): FWD exp(x - inf) = 0; BWD exp(-inf - m) = 0
    const float dead = MODE == MN_FWD ? INFINITY : -INFINITY;
    if (!bok || mx4.x == -INFINITY) mx4.x = dead;
    if (!bok || mx4.y == -INFINITY) mx4.y = dead;
    if (!bok || mx4.z == -INFINITY) mx4.z = dead;
    if (!bok || mx4.w == -INFINITY) mx4.w = dead;
    // byte offset of this thread's 16 bytes inside an A part: K row kr = 8 * pass + warp lies in row
    // kr % 4 of the atom (kr / 4, lane / 8); the lane's 32-byte unit (lane % 8) / 2 is XORed with the row
    const uint32_t r4 = warp & 3u;
    const uint32_t aoff = ((warp >> 2) * 4u + (lane >> 3)) * 512u + r4 * 128u + (((((lane & 7u) >> 1) ^ r4)) << 5) +
                          ((lane & 1u) << 4);
    struct Regs { float4 x[2], y[2]; };
    auto load = [&](uint32_t i, Regs& r) {
#pragma unroll
      for (uint32_t ps = 0; ps < 2; ++ps) {
        const uint32_t t = i * KC + ps * 8u + warp;
        const size_t o = (size_t)(t < kdim ? t : 0u) * ld;
        r.x[ps] = ldg4(rowsA + o);
        if (MODE == MN_BWD_CHILD || has_sub) r.y[ps] = ldg4(rowsB + o);
      }
    };
    auto process = [&](uint32_t i, const Regs& r) -> bool {
      const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
      // one lane per warp polls; __all_sync orders the other lanes' stores behind the observed phase
      bool got = lane != 0 || mbar_wait(&empty[s], ph ^ 1u, a.status);
      got = __all_sync(0xffffffffu, got);
      if (!got) return false;
      uint8_t* a_hi = smem + s * STAGE_BYTES;
      uint8_t* a_lo = a_hi + A_BYTES;
      if (tid == 0) {   // weight tile of the chunk: hi and lo parts straight from the image
        const uint32_t bytes = n_tile * KC * 4u;
        const float* src = img_tile + (size_t)i * 2 * img_rows * KC;
        mbar_expect_tx(&full[s], 2 * bytes);
        bulk_g2s(a_hi + 2 * A_BYTES, src, bytes, &full[s]);
        bulk_g2s(a_hi + 2 * A_BYTES + B_BYTES, src + (size_t)img_rows * KC, bytes, &full[s]);
      }
#pragma unroll
      for (uint32_t ps = 0; ps < 2; ++ps) {
        const bool tok = i * KC + ps * 8u + warp < kdim;
        float4 v;
        if (MODE == MN_FWD) {
          v = r.x[ps];
          if (has_sub) { v.x += r.y[ps].x; v.y += r.y[ps].y; v.z += r.y[ps].z; v.w += r.y[ps].w; }
          v.x = __expf(v.x - mx4.x); v.y = __expf(v.y - mx4.y); v.z = __expf(v.z - mx4.z); v.w = __expf(v.w - mx4.w);
        } else {   // x: mars of the parent, y: flows of the parent
          v.x = r.y[ps].x * __expf(mx4.x - r.x[ps].x); v.y = r.y[ps].y * __expf(mx4.y - r.x[ps].y);
          v.z = r.y[ps].z * __expf(mx4.z - r.x[ps].z); v.w = r.y[ps].w * __expf(mx4.w - r.x[ps].w);
        }
        if (!tok) v = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        const uint32_t o = aoff + ps * 4096u;
        *reinterpret_cast<float4*>(a_hi + o) = h;
        *reinterpret_cast<float4*>(a_lo + o) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
      }
      fence_proxy_async();   // make the generic-proxy writes visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
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

    // =========================== epilogue ====================================================
    if (ok && lane == 0) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      // warp -> (TMEM lane quarter, column half); a thread owns one example and walks 16 columns at a time
      const uint32_t q4 = warp & 3, half = warp >> 2;
      const uint32_t CG = max(16u, ((n_tile + 31u) / 32u) * 16u);   // columns per half, a multiple of 16
      const uint32_t row = q4 * 32 + lane, b = m0 + row;
      const uint32_t c_begin = half * CG, c_end = min(n_tile, c_begin + CG);
      const float mx = mxs[row];
      float acc[16];
      for (uint32_t c0 = c_begin; c0 < c_end; c0 += 16) {
        tmem_ld16(tmem_base + ((q4 * 32u) << 16) + c0, acc);
        if (b >= ld) continue;
        if (MODE == MN_FWD) {
#pragma unroll
          for (uint32_t j = 0; j < 16; ++j) {
            const uint32_t r = n0 + c0 + j;
            if (r < k.R) a.mars[(size_t)(k.p0 + r) * ld + b] = mx == -INFINITY ? -INFINITY : __logf(acc[j]) + mx;
          }
        } else {
          // all child values first (independent loads), then the products and the stores
          float cv[16], dv[16];
#pragma unroll
          for (uint32_t j = 0; j < 16; ++j) {
            const uint32_t t = n0 + c0 + j;
            const uint32_t tt = t < k.K ? t : 0u;
            cv[j] = __ldcg(a.mars + (size_t)(k.c0 + tt) * ld + b);
            dv[j] = has_sub ? __ldcg(a.mars + (size_t)(k.d0 + tt) * ld + b) : 0.0f;
          }
#pragma unroll
          for (uint32_t j = 0; j < 16; ++j) {
            const uint32_t t = n0 + c0 + j;
            if (t < k.K) {
              const float f = mx == -INFINITY ? 0.0f : acc[j] * __expf((cv[j] + dv[j]) - mx);
              a.flows[(size_t)(k.c0 + t) * ld + b] = f;
              if (has_sub) a.flows[(size_t)(k.d0 + t) * ld + b] = f;
            }
          }
        }
      }
    }
  } else {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      const uint32_t idesc = idesc_mn(TM, n_tile);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
        ok = mbar_wait(&full[s], ph, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
#pragma unroll
        for (uint32_t ks = 0; ks < KC / 8; ++ks) {
          // A: the next 8 K rows are the next eight atoms (4 KB); W: 8 tf32 = 32 bytes along the row
          const uint64_t d_ahi = desc_mn128(sa + ks * 4096u), d_alo = desc_mn128(sa + A_BYTES + ks * 4096u);
          const uint64_t d_bhi = desc_k64(sa + 2 * A_BYTES) + (uint64_t)((ks * 32u) >> 4);
          const uint64_t d_blo = desc_k64(sa + 2 * A_BYTES + B_BYTES) + (uint64_t)((ks * 32u) >> 4);
          umma_tf32(tmem_base, d_ahi, d_bhi, idesc, (i | ks) ? 1u : 0u);
          umma_tf32(tmem_base, d_alo, d_bhi, idesc, 1u);
          umma_tf32(tmem_base, d_ahi, d_blo, idesc, 1u);
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
  if (warp == PW) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int MODE>
int32_t launch(dim3 grid, const MnArgs& args, cudaStream_t st, bool pdl) {
  static PcbPerDeviceOnce once;
  PCB_CUDA(once.run([] {
    return cudaFuncSetAttribute(dense_mn_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  }));
  PCB_CUDA(pcb_launch_pdl(dense_mn_kernel<MODE>, grid, dim3(NTHREADS), SMEM_BYTES, st, pdl, args));
  return PCB_OK;
}

// A layer that would not fill the GPU (two CTAs per SM) with 256-column tiles is cut into narrower
// tiles: the CTAs of one tile repeat the production of the data-dependent operand, but each has
// half (a quarter) of the weight tile to fetch, of the MMAs to wait for and of the epilogue.
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

int32_t pcb_dense_mn_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM, ct = (c->max_dense_R + TN - 1) / TN;
  MnArgs args{ws->mars, ws->flows, ws->blk_mx, c->w_img16, c->dense + o0, c->dense_img16 + o0, c->status, ws->ld,
              pick_nsplit(bt * ct * (o1 - o0), c->max_dense_R, c->tc_nsplit)};
  dim3 grid(bt, ct * args.nsplit, o1 - o0);
  PcbProfScope ps(c, st, PCB_K_DENSE_FWD);
  return launch<MN_FWD>(grid, args, st, c->pdl);
}

int32_t pcb_dense_mn_backward_child(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  const uint32_t bt = (pcb_round_up(ws->B, 32) + TM - 1) / TM, ct = (c->max_dense_K + TN - 1) / TN;
  MnArgs args{ws->mars, ws->flows, ws->blk_mx, c->w_img16, c->dense + o0, c->dense_img16 + o0, c->status, ws->ld,
              pick_nsplit(bt * ct * (o1 - o0), c->max_dense_K, c->tc_nsplit)};
  dim3 grid(bt, ct * args.nsplit, o1 - o0);
  PcbProfScope ps(c, st, PCB_K_DENSE_BWD_CHILD);
  return launch<MN_BWD_CHILD>(grid, args, st, c->pdl);
}
