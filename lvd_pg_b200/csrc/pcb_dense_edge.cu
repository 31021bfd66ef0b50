// pcb_dense_edge.cu — edge statistics of dense sum blocks with operands fetched by tensor-map copies.
//
//   D[r][t] = sum_b G[r][b] * E[t][b],   G = flows_r * exp(mx - mars_r),   E = exp(mars_t - mx)
//   aggr[edge(r, t)] += exp(theta[edge(r, t)]) * D[r][t]
//
// Both operands are K-major in the work matrices as they lie in memory (K = the example index, which is
// contiguous), so a 2-D tensor-map copy with a swizzle as wide as its rows drops a
// [rows][KCH examples] box into shared memory in exactly the layout tcgen05.mma reads.  Per chunk of
// KCH examples one elected thread issues the copies (parents' mars, parents' flows, prime
// children's mars and, where edges carry a sub child, the sub children's mars), sixteen converter
// warps turn the raw boxes into the TF32 hi / lo operand tiles IN PLACE with 16-byte shared-memory
// accesses (hi(G) over the mars box, lo(G) over the flows box, hi(E) over the prime children's
// box, lo(E) over the sub children's box), and one thread issues the MMAs (hi*hi + lo*hi + hi*lo) into a
// 128 x 256 fp32 accumulator in tensor memory.  A stage cycles through
//   empty -> (copies) -> raw_full -> (convert) -> conv_full -> (MMA, commit) -> empty.
// Every wait is bounded; on expiry the thread raises the circuit's status word and all roles
// drain to the common exit where tensor memory is released.
//
// The load-based kernel in pcb_dense_tc.cu stays as the fallback when tensor maps cannot be encoded.
#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {
using namespace pcbtc;

constexpr uint32_t TM = 128;          // parents per tile (TMEM lanes)
constexpr uint32_t TN = 256;          // children per tile (TMEM columns)
// Examples per stage (32: 128-byte rows and swizzle, two stages; 16: 64-byte rows and swizzle, four
// stages).  Both run at the same speed: per 32 examples the stage memory sees 96 KB written by the
// copies, 96 KB read and 96 KB written by the conversion and 144 KB read by the MMAs, which is the
// shared-memory bandwidth of an SM over the ~1.9 us a chunk takes; 32 keeps whole 128-byte lines
// per row in each copy.
constexpr uint32_t KCH = 32;
constexpr uint32_t STAGES = 2;
constexpr uint32_t ROWB = KCH * 4;    // bytes per operand row in a stage
constexpr uint32_t SLOTS = ROWB / 16; // 16-byte slots per row
static_assert(KCH == 16 || KCH == 32, "one swizzle row per stage row");
constexpr uint32_t CW = 16;           // converter warps
constexpr uint32_t MMA_WARP = CW;   // warp CW + 1 issues the copies
constexpr uint32_t NTHREADS = (CW + 2) * 32;
constexpr uint32_t A_BYTES = TM * ROWB, B_BYTES = TN * ROWB;
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr uint32_t RAW_BYTES = 2 * A_BYTES + B_BYTES;   // what the copies of one chunk deliver
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 1024 /*barriers*/;
constexpr uint32_t TMEM_COLS = 256;
constexpr float L2E = 1.4426950408889634f;

struct EdgeArgs {
  const float* blk_mx;
  float* aggr;
  const float* theta;
  const PcbDenseBlock* blocks;
  int* status;
  uint32_t ld, B, b_per_cta;
  unsigned long long* trace;   // timing trace of CTA (0,0,0), or null
  uint32_t dbg;                // timing experiments only: 1 skip MMAs, 2 copies re-read the first chunk, 4 skip conversion
};

__device__ __forceinline__ float4 split_hi(float4 v) {
  return make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
}
__device__ __forceinline__ float4 sub4(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }

// Timing experiments exist only in a build with -DPCB_DIAG; the default build compiles them out.
#ifdef PCB_DIAG
#define PCB_DBG(a, bit) ((a).dbg & (bit))
#define EDGE_TRACE(slot)                                                            \
  do {                                                                              \
    if (a.trace && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) a.trace[slot] = gtime(); \
  } while (0)
#else
#define PCB_DBG(a, bit) 0u
#define EDGE_TRACE(slot) do { } while (0)
#endif

// K-major operand descriptor for this kernel's row width: 8-row groups ROWB * 8 bytes apart, swizzle
// span = row width (layout code 2: 128-byte swizzle, 4: 64-byte swizzle)
__device__ __forceinline__ uint64_t edge_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((ROWB * 8u) >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(KCH == 32 ? 2 : 4) << 61;
  return d;
}
// swizzle term of a row: the 16-byte slot index is XORed with it
__device__ __forceinline__ uint32_t row_swz(uint32_t row) { return KCH == 32 ? (row & 7u) : ((row >> 1) & 3u); }

// grid: (example slices, row tiles x column tiles, blocks)
__global__ void __launch_bounds__(NTHREADS, 1)
dense_edge_tma_kernel(const __grid_constant__ CUtensorMap tm_mars_a, const __grid_constant__ CUtensorMap tm_flows_a,
                      const __grid_constant__ CUtensorMap tm_mars_b, EdgeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctl = smem + STAGES * STAGE_BYTES;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(ctl);   // [STAGES] copies landed
  uint64_t* conv_full = raw_full + STAGES;                 // [STAGES] operand tiles written
  uint64_t* empty = conv_full + STAGES;                    // [STAGES] MMAs have read the stage
  uint64_t* accfull = empty + STAGES;                      // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);

  const PcbDenseBlock k = a.blocks[blockIdx.z];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ld = a.ld;
  const uint32_t tiles_n = (k.K + TN - 1) / TN;
  const uint32_t m0 = (blockIdx.y / tiles_n) * TM, n0 = (blockIdx.y % tiles_n) * TN;
  if (m0 >= k.R) return;
  const uint32_t n_count = min(TN, k.K - n0);
  const uint32_t k_begin = blockIdx.x * a.b_per_cta, k_end = min(a.B, k_begin + a.b_per_cta);
  if (k_begin >= k_end) return;
  const uint32_t nchunks = (k_end - k_begin + KCH - 1) / KCH;
  const uint32_t n_tile = (n_count + 15u) & ~15u;
  const float* mxrow = a.blk_mx + (size_t)k.mx_row * ld;
  const bool has_sub = k.d0 != PCB_NONE;

  if (tid == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&conv_full[s], CW);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accfull, 1);
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
  bool ok = true;
  if (tid == 0) EDGE_TRACE(503);

  if (warp < CW) {
    // =========================== converters ==================================================
    // thread -> (row, 16-byte slot): logical slot kk4 (examples 4*kk4 .. 4*kk4+3) is fixed per
    // thread, rows advance by 64, so the swizzled byte offset is one base plus a constant step and
    // the thread's four per-example maxima are the same for all of its rows.  The eight lanes of a
    // quarter warp cover the eight slots of one row: every 16-byte access is conflict-free.
    constexpr uint32_t RP = CW * 32 / SLOTS;          // rows per pass of the 512 threads
    const uint32_t kk4 = tid % SLOTS, rbase = tid / SLOTS;
    const uint32_t off0 = rbase * ROWB + ((kk4 ^ row_swz(rbase)) << 4);
    static_assert(RP % 8 == 0, "the swizzle term must not change from pass to pass");
    auto load_mx = [&](uint32_t i) { return *reinterpret_cast<const float4*>(mxrow + k_begin + i * KCH + 4u * kk4); };
    float4 mxn = load_mx(0);
    for (uint32_t i = 0; i < nchunks; ++i) {
      const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
      const float4 mx = mxn;
      if (i + 1 < nchunks) mxn = load_mx(i + 1);
      if (i + 8 == nchunks || (nchunks < 8 && i == 0)) {
        // the epilogue reads theta and reduces into aggr over this tile's 128 rows x 1 KB: ask L2
        // for those lines a few chunks ahead (earlier, the operand stream would evict them again)
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j) {
          const uint32_t lid = tid + CW * 32u * j;          // 1024 lines per array
          const uint32_t r = m0 + (lid >> 3), t = n0 + ((lid & 7u) << 5);
          if (r < k.R && t < k.K) {
            const size_t p = k.pid0 + (size_t)r * k.K + t;
            prefetch_l2(a.theta + p);
            prefetch_l2(a.aggr + p);
          }
        }
      }
      const uint32_t b0 = k_begin + i * KCH + 4u * kk4;
      const bool v0 = b0 < k_end && mx.x != -INFINITY, v1 = b0 + 1 < k_end && mx.y != -INFINITY,
                 v2 = b0 + 2 < k_end && mx.z != -INFINITY, v3 = b0 + 3 < k_end && mx.w != -INFINITY;
      const bool allv = v0 && v1 && v2 && v3;
      const float4 sx = make_float4(mx.x * L2E, mx.y * L2E, mx.z * L2E, mx.w * L2E);
      bool got = lane != 0 || mbar_wait(&raw_full[s], ph, a.status);
      got = __all_sync(0xffffffffu, got);
      if (!got) { ok = false; break; }
      if (tid == 0 && i < 60) EDGE_TRACE(i * 8 + 2);
      uint8_t* st = smem + s * STAGE_BYTES + off0;
      if (!(PCB_DBG(a, 4u))) {
#pragma unroll
      for (uint32_t q = 0; q < TM / RP; ++q) {   // G = flows * exp(mx - mars), exponent clamped: inf * 0 stays out
        uint8_t* p = st + q * (RP * ROWB);
        const float4 m = *reinterpret_cast<const float4*>(p);
        const float4 f = *reinterpret_cast<const float4*>(p + A_BYTES);
        float4 g;
        g.x = f.x * ex2_ftz(fminf(fmaf(m.x, -L2E, sx.x), 126.0f));
        g.y = f.y * ex2_ftz(fminf(fmaf(m.y, -L2E, sx.y), 126.0f));
        g.z = f.z * ex2_ftz(fminf(fmaf(m.z, -L2E, sx.z), 126.0f));
        g.w = f.w * ex2_ftz(fminf(fmaf(m.w, -L2E, sx.w), 126.0f));
        if (!allv) { g.x = v0 ? g.x : 0.0f; g.y = v1 ? g.y : 0.0f; g.z = v2 ? g.z : 0.0f; g.w = v3 ? g.w : 0.0f; }
        const float4 h = split_hi(g);
        *reinterpret_cast<float4*>(p) = h;
        *reinterpret_cast<float4*>(p + A_BYTES) = sub4(g, h);
      }
#pragma unroll
      for (uint32_t q = 0; q < TN / RP; ++q) {   // E = exp(mars_child - mx) <= 1
        if (rbase + RP * q < n_tile) {
          uint8_t* p = st + 2 * A_BYTES + q * (RP * ROWB);
          float4 c = *reinterpret_cast<const float4*>(p);
          if (has_sub) {   // child value = prime row + sub row (the sub box lies where lo(E) goes)
            const float4 d = *reinterpret_cast<const float4*>(p + B_BYTES);
            c.x += d.x; c.y += d.y; c.z += d.z; c.w += d.w;
          }
          float4 e;
          e.x = ex2_ftz(fmaf(c.x, L2E, -sx.x));
          e.y = ex2_ftz(fmaf(c.y, L2E, -sx.y));
          e.z = ex2_ftz(fmaf(c.z, L2E, -sx.z));
          e.w = ex2_ftz(fmaf(c.w, L2E, -sx.w));
          if (!allv) { e.x = v0 ? e.x : 0.0f; e.y = v1 ? e.y : 0.0f; e.z = v2 ? e.z : 0.0f; e.w = v3 ? e.w : 0.0f; }
          const float4 h = split_hi(e);
          *reinterpret_cast<float4*>(p) = h;
          *reinterpret_cast<float4*>(p + B_BYTES) = sub4(e, h);
        }
      }
      }
      fence_proxy_async();   // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&conv_full[s]);
      if (tid == 0 && i < 60) EDGE_TRACE(i * 8 + 3);
    }
    if (tid == 0) EDGE_TRACE(500);

    // =========================== epilogue ====================================================
    if (ok && lane == 0) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (tid == 0) EDGE_TRACE(501);
    if (ok) {
      tc_fence_after();
      constexpr uint32_t CG = TN / (CW / 4);           // columns per epilogue warp group
      const uint32_t q4 = warp & 3, grp = warp >> 2;   // lane quarter, column group
      const uint32_t c_begin = grp * CG, c_end = min(n_tile, c_begin + CG);
      // The accumulator arrives with one tile row per lane; the statistics rows are contiguous
      // along the column index.  Each warp transposes its 32 x 32 patches through shared memory
      // (the stages are idle once the accumulator is complete) and issues whole-line reductions.
      float* patch = reinterpret_cast<float*>(smem) + warp * (32 * 33);
      float acc[32];
      for (uint32_t c0 = c_begin; c0 < c_end; c0 += 32) {
        tmem_ld32(tmem_base + ((q4 * 32u) << 16) + c0, acc);
#pragma unroll
        for (uint32_t j = 0; j < 32; ++j) patch[lane * 33 + j] = acc[j];
        __syncwarp();
        const uint32_t t = n0 + c0 + lane;
        if (t < k.K) {
#pragma unroll 16
          for (uint32_t rr = 0; rr < 32; ++rr) {
            const uint32_t r = m0 + q4 * 32 + rr;
            if (r < k.R) {
              const size_t p = k.pid0 + (size_t)r * k.K + t;
              atomicAdd(a.aggr + p, __expf(__ldg(a.theta + p)) * patch[rr * 33 + lane]);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc(TM, n_tile);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
        ok = mbar_wait(&conv_full[s], ph, a.status);
        if (!ok) break;
        if (i < 60) EDGE_TRACE(i * 8 + 4);
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t d_ahi = edge_desc(sa), d_alo = edge_desc(sa + A_BYTES);
        const uint64_t d_bhi = edge_desc(sa + 2 * A_BYTES), d_blo = edge_desc(sa + 2 * A_BYTES + B_BYTES);
        if (!(PCB_DBG(a, 1u)))
#pragma unroll
        for (uint32_t ks = 0; ks < KCH / 8; ++ks) {
          const uint64_t adv = (uint64_t)((ks * 32u) >> 4);  // 8 tf32 = 32 bytes along K
          umma_tf32(tmem_base, d_ahi + adv, d_bhi + adv, idesc, (i | ks) ? 1u : 0u);
          umma_tf32(tmem_base, d_alo + adv, d_bhi + adv, idesc, 1u);
          umma_tf32(tmem_base, d_ahi + adv, d_blo + adv, idesc, 1u);
        }
        umma_commit(&empty[s]);
        if (i < 60) EDGE_TRACE(i * 8 + 5);
      }
      if (ok) umma_commit(accfull);
    }
    __syncwarp();
  } else {
    // =========================== copy issuer =================================================
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t i = 0; i < nchunks; ++i) {
        const uint32_t s = i & (STAGES - 1), ph = (i / STAGES) & 1u;
        if (i < 60) EDGE_TRACE(i * 8 + 0);
        if (!mbar_wait(&empty[s], ph ^ 1u, a.status)) break;
        if (i < 60) EDGE_TRACE(i * 8 + 1);
        uint8_t* st = smem + s * STAGE_BYTES;
        const int32_t x = (int32_t)(k_begin + ((PCB_DBG(a, 2u)) ? 0u : i * KCH));
        mbar_arrive_expect_tx(&raw_full[s], has_sub ? RAW_BYTES + B_BYTES : RAW_BYTES);
        tma_load_2d(st, &tm_mars_a, x, (int32_t)(k.p0 + m0), &raw_full[s]);
        tma_load_2d(st + A_BYTES, &tm_flows_a, x, (int32_t)(k.p0 + m0), &raw_full[s]);
        tma_load_2d(st + 2 * A_BYTES, &tm_mars_b, x, (int32_t)(k.c0 + n0), &raw_full[s]);
        if (has_sub) tma_load_2d(st + 2 * A_BYTES + B_BYTES, &tm_mars_b, x, (int32_t)(k.d0 + n0), &raw_full[s]);
        issued = i + 1;
      }
      if (issued < nchunks) {
        // a wait was lost: let the copies already issued land before the CTA gives its memory back
        for (uint32_t j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j)
          mbar_wait(&raw_full[j & (STAGES - 1)], (j / STAGES) & 1u, a.status);
      }
    }
    __syncwarp();
  }

  if (tid == 0) EDGE_TRACE(502);
  // ---- common exit: release tensor memory -------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

unsigned long long* g_edge_trace = nullptr;   // diagnostic buffer, allocated when PCB_TC_TRACE is set

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [box_rows][box_cols examples] boxes of an [n_rows][ld] fp32 matrix, zero fill outside; swizzled
// as wide as the box's rows (box_cols = KCH) or not at all (row slabs)
bool encode_map(void* out, float* base, uint32_t ld, uint64_t n_rows, uint32_t box_cols, uint32_t box_rows, bool swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  alignas(64) CUtensorMap m;
  cuuint64_t gdim[2] = {ld, n_rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = !swizzle ? CU_TENSOR_MAP_SWIZZLE_NONE : (KCH == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  memcpy(out, &m, sizeof(m));
  return true;
}

bool encode_rows_map(void* out, float* base, uint32_t ld, uint64_t n_rows, uint32_t box_rows) {
  return encode_map(out, base, ld, n_rows, KCH, box_rows, true);
}

}  // namespace

// Encodes the workspace's tensor maps (parents' boxes of 128 rows over mars and flows, children's
// boxes of 256 rows over mars).  Leaves have_tm false when the driver entry point is missing.
int32_t pcb_dense_edge_prepare_ws(pcb_workspace* ws) {
  ws->have_tm = false;
  ws->have_tm_rows = false;
  pcb_circuit* c = ws->c;
  if (!c->use_tc || c->n_dense == 0) return PCB_OK;
  // row slabs [16 rows][128 examples] of mars, as they lie in memory (pcb_dense_mn.cu)
  ws->have_tm_rows = encode_map(ws->tm_rows, ws->mars, ws->ld, c->N, 128, 16, false);
  if (c->edge_ld) return PCB_OK;
  bool good = encode_rows_map(ws->tm[0], ws->mars, ws->ld, c->N, TM) &&
              encode_rows_map(ws->tm[1], ws->flows, ws->ld, c->N, TM) &&
              encode_rows_map(ws->tm[2], ws->mars, ws->ld, c->N, TN);
  ws->have_tm = good;
  return PCB_OK;
}

// Edge statistics of dense blocks [o0, o0 + n) with the examples cut into `slices` ranges of b_per.
int32_t pcb_dense_edge_launch(pcb_circuit* c, pcb_workspace* ws, uint32_t o0, uint32_t n, uint32_t slices,
                              uint32_t b_per, cudaStream_t st) {
  static PcbPerDeviceOnce once;
  PCB_CUDA(once.run([] {
    return cudaFuncSetAttribute(dense_edge_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  }));
  uint32_t dbg = 0;
#ifdef PCB_DIAG
  if (!g_edge_trace && getenv("PCB_TC_TRACE")) {
    cudaMalloc((void**)&g_edge_trace, 512 * sizeof(unsigned long long));
    cudaMemset(g_edge_trace, 0, 512 * sizeof(unsigned long long));
  }
  if (const char* e = getenv("PCB_TC_DEBUG")) dbg = (uint32_t)atoi(e);
#endif
  alignas(64) CUtensorMap ma, fa, mb;
  memcpy(&ma, ws->tm[0], sizeof(ma));
  memcpy(&fa, ws->tm[1], sizeof(fa));
  memcpy(&mb, ws->tm[2], sizeof(mb));
  const uint32_t tiles = ((c->max_dense_R + TM - 1) / TM) * ((c->max_dense_K + TN - 1) / TN);
  for (uint32_t z0 = 0; z0 < n; z0 += 65535) {
    EdgeArgs args{ws->blk_mx, c->aggr, c->theta, c->dense + o0 + z0, c->status, ws->ld, ws->B, b_per, g_edge_trace, dbg};
    dim3 grid(slices, tiles, std::min<uint32_t>(65535, n - z0));
    PcbProfScope ps(c, st, PCB_K_DENSE_BWD_EDGE);
    dense_edge_tma_kernel<<<grid, NTHREADS, SMEM_BYTES, st>>>(ma, fa, mb, args);
  }
  return PCB_OK;
}

// Diagnostic: copies the timing trace of the last traced edge-statistics kernel (PCB_TC_TRACE set) to the host.
extern "C" int32_t pcb_debug_read_edge_trace(unsigned long long* out) {
  if (!g_edge_trace) return PCB_ERR_STATE;
  cudaDeviceSynchronize();
  return cudaMemcpy(out, g_edge_trace, 512 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? PCB_OK : PCB_ERR_CUDA;
}
