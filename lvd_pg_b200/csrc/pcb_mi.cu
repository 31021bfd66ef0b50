// pcb_mi.cu — pairwise mutual information of categorical columns (the input of Chow-Liu structure
// learning, the step before the circuit exists).
//
// Reference (paths relative to VariationalJuice.jl/src): pairwise_marginal_kernel, single_marginal_kernel,
// single_and_pairwise_marginal, pairwise_MI_chunked — utils/information.jl:3-157.  The reference
// counts co-occurrences with one global atomic per (example, variable pair), copies the [V, V, C, C]
// table to the host in chunks and forms MI there.
//
// Here the co-occurrence table is what it is algebraically: onehot(X)^T * onehot(X), a
// (V*C) x (V*C) x rows contraction of 0/1 values — exact in bf16 with fp32 accumulation up to 2^24
// rows — and it never leaves the SM: a CTA builds the two one-hot operand tiles (128 (variable,
// category) rows x 64 examples, K-major, 128-byte swizzle) in shared memory straight from the uint8
// columns, one thread issues tcgen05.mma.kind::f16 into a 128 x 128 fp32 accumulator in tensor
// memory, and the epilogue turns the counts of the tile into sum p log(p / (p_a p_b)) per variable
// pair (the pseudocount spread over the table as in the reference) and adds it to MI[v1, v2].
// Only tiles on or above the diagonal are computed; an off-diagonal tile also feeds MI[v2, v1].
#include <algorithm>
#include <string>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {

using namespace pcbtc;

constexpr uint32_t TILE = 128;                 // (variable, category) rows per operand tile = TMEM lanes / columns
constexpr uint32_t KCH = 64;                   // examples per stage: one 128-byte swizzled row of bf16
constexpr uint32_t OP_BYTES = TILE * 128;      // one operand tile of a stage
constexpr uint32_t STAGES = 3;
constexpr uint32_t NPROD = 128;                // producer / epilogue threads: one per tile row
constexpr uint32_t NTHREADS = NPROD + 32;      // + the MMA warp
constexpr uint32_t SMEM = STAGES * 2 * OP_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t idesc_bf16(uint32_t m, uint32_t n) {
  // D fp32, A and B bf16, both K-major
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// counts of every (variable, category), then log of the smoothed marginal
__global__ void mi_hist_kernel(const uint8_t* __restrict__ data, uint64_t rows, uint32_t V, uint32_t C,
                               unsigned int* __restrict__ counts) {
  const uint32_t v = blockIdx.x;
  for (uint64_t n = blockIdx.y * blockDim.x + threadIdx.x; n < rows; n += (uint64_t)gridDim.y * blockDim.x) {
    const uint32_t x = data[(size_t)v * rows + n];
    if (x < C) atomicAdd(counts + (size_t)v * C + x, 1u);
  }
}
__global__ void mi_logp_kernel(const unsigned int* __restrict__ counts, uint32_t n, float smooth, float z,
                               float* __restrict__ logp) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) logp[i] = logf(((float)counts[i] + smooth) / z);
}

struct MiArgs {
  const uint8_t* data;    // [rows, V] column-major
  uint64_t rows;
  uint32_t V, C, tiles;
  const float* logp;      // [V * C] log marginals
  float pair_smooth, z;   // pseudocount / C^2, rows + pseudocount
  float* mi;              // [V, V]
  int* status;
};

__global__ void __launch_bounds__(NTHREADS) mi_tile_kernel(MiArgs a) {
  // upper-triangular tile pair from the linear block index
  uint32_t ti = 0, rest = blockIdx.x;
  while (rest >= a.tiles - ti) { rest -= a.tiles - ti; ++ti; }
  const uint32_t tj = ti + rest;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctl = smem + STAGES * 2 * OP_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);   // [STAGES] operands of a stage written
  uint64_t* empty = full + STAGES;                     // [STAGES] the MMAs that read a stage are done
  uint64_t* accfull = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) { mbar_init(&full[s], NPROD / 32); mbar_init(&empty[s], 1); }
    mbar_init(accfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == NPROD / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TILE)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t nchunks = (uint32_t)((a.rows + KCH - 1) / KCH);
  const uint32_t total_rows = a.V * a.C;
  bool ok = true;

  if (warp < NPROD / 32) {
    // =========================== producers: one tile row each, for both operands ================
    const uint32_t ra = ti * TILE + tid, rb = tj * TILE + tid;
    const bool va = ra < total_rows, vb = rb < total_rows;
    const uint32_t ca = va ? ra % a.C : 0, cb = vb ? rb % a.C : 0;
    const uint8_t* cola = a.data + (size_t)(va ? ra / a.C : 0) * a.rows;
    const uint8_t* colb = a.data + (size_t)(vb ? rb / a.C : 0) * a.rows;
    const bool same = ti == tj;   // then the B tile is the A tile
    auto onehot8 = [&](const uint8_t* col, uint64_t n0, uint32_t cat, bool valid) {
      // eight examples n0 .. n0 + 7 of one (variable, category) row as bf16 0 / 1
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      if (valid && n0 < a.rows) {
        uint8_t x[8];
        if (n0 + 8 <= a.rows && ((reinterpret_cast<uintptr_t>(col) + n0) & 7) == 0) {
          const uint2 q = *reinterpret_cast<const uint2*>(col + n0);
          memcpy(x, &q, 8);
        } else {
#pragma unroll
          for (uint32_t k = 0; k < 8; ++k) x[k] = n0 + k < a.rows ? col[n0 + k] : 0u;   // examples past the end are masked below
        }
#pragma unroll
        for (uint32_t k = 0; k < 8; ++k)
          if (x[k] == cat && n0 + k < a.rows) w[k >> 1] |= 0x3f80u << ((k & 1u) * 16u);   // bf16 1.0
      }
      return make_uint4(w[0], w[1], w[2], w[3]);
    };
    for (uint32_t i = 0; i < nchunks && ok; ++i) {
      const uint32_t s = i % STAGES, ph = (i / STAGES) & 1u;
      bool got = lane != 0 || mbar_wait(&empty[s], ph ^ 1u, a.status);
      ok = __all_sync(0xffffffffu, got);
      if (!ok) break;
      uint8_t* ta = smem + s * 2 * OP_BYTES;
      uint8_t* tb = ta + OP_BYTES;
      const uint64_t n0 = (uint64_t)i * KCH;
#pragma unroll
      for (uint32_t k8 = 0; k8 < 8; ++k8) {
        const uint32_t off = tid * 128u + ((k8 ^ (tid & 7u)) << 4);   // K-major, 128-byte swizzle
        *reinterpret_cast<uint4*>(ta + off) = onehot8(cola, n0 + 8u * k8, ca, va);
        if (!same) *reinterpret_cast<uint4*>(tb + off) = onehot8(colb, n0 + 8u * k8, cb, vb);
      }
      fence_proxy_async();   // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
    }

    // =========================== epilogue =====================================================
    if (ok && lane == 0) ok = mbar_wait(accfull, 0, a.status);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t C = a.C;
      const float lpa = va ? a.logp[ra] : 0.0f;
      const uint32_t v1 = va ? ra / C : 0;
      const uint32_t seg = C < 32 ? C : 32;   // lanes of this warp that share v1
#pragma unroll 1
      for (uint32_t c0 = 0; c0 < TILE; c0 += 32) {
        float acc[32];
        tmem_ld32(tmem_base + ((warp * 32u) << 16) + c0, acc);
        // columns c0 .. c0 + 31: groups of min(C, 32) columns share v2
        for (uint32_t g0 = 0; g0 < 32; g0 += seg) {
          const uint32_t col = tj * TILE + c0 + g0;
          const bool vcol = col < total_rows;
          const uint32_t v2 = vcol ? col / C : 0;
          float part = 0.0f;
          if (va && vcol) {
#pragma unroll
            for (uint32_t k = 0; k < 32; ++k) {
              if (k < g0 || k >= g0 + seg) continue;
              const float pxy = (acc[k] + a.pair_smooth) / a.z;
              if (pxy > 0.0f) part += pxy * (logf(pxy) - lpa - a.logp[col + (k - g0)]);
            }
          }
          // sum over the lanes that hold the categories of v1
          for (uint32_t o = seg >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
          if ((lane & (seg - 1)) == 0 && va && vcol) {
            atomicAdd(a.mi + (size_t)v1 * a.V + v2, part);
            if (ti != tj) atomicAdd(a.mi + (size_t)v2 * a.V + v1, part);
          }
        }
      }
    }
  } else {
    // =========================== MMA issuer ====================================================
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(TILE, TILE);
      for (uint32_t i = 0; i < nchunks && ok; ++i) {
        const uint32_t s = i % STAGES, ph = (i / STAGES) & 1u;
        ok = mbar_wait(&full[s], ph, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aa = smem_u32(smem + s * 2 * OP_BYTES), bb = ti == tj ? aa : aa + OP_BYTES;
#pragma unroll
        for (uint32_t ks = 0; ks < KCH / 16; ++ks) {   // 16 bf16 = 32 bytes along the swizzled row
          const uint64_t da = make_desc(aa) + (uint64_t)((ks * 32u) >> 4), db = make_desc(bb) + (uint64_t)((ks * 32u) >> 4);
          umma_bf16(tmem_base, da, db, idesc, (i | ks) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(accfull);
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == NPROD / 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TILE) : "memory");
  }
}

}  // namespace

extern "C" int32_t pcb_pairwise_mi(const uint8_t* data_dev, uint64_t num_rows, uint32_t num_vars, uint32_t num_cats,
                                   float pseudocount, float* mi_dev, pcb_stream s) {
  PCB_REQUIRE(data_dev && mi_dev, "null argument");
  PCB_REQUIRE(num_rows >= 1 && num_rows < (1ull << 24), "row count must be below 2^24 (counts are exact in fp32 up to there)");
  PCB_REQUIRE(num_vars >= 1 && num_cats >= 2 && num_cats <= 256 && (num_cats & (num_cats - 1)) == 0,
              "the number of categories must be a power of two between 2 and 256");
  PCB_REQUIRE(pseudocount >= 0.0f, "negative pseudocount");
  cudaDeviceProp prop;
  int dev = 0;
  PCB_CUDA(cudaGetDevice(&dev));
  PCB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    return pcb_fail(PCB_ERR_INVALID, "pairwise MI needs an sm_100 device (tcgen05)");
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t VC = num_vars * num_cats;
  unsigned int* counts = nullptr;
  float* logp = nullptr;
  int* status = nullptr;
  PCB_CUDA(cudaMalloc((void**)&counts, (size_t)VC * sizeof(unsigned int)));
  auto release = [&]() { cudaFree(counts); if (logp) cudaFree(logp); if (status) cudaFree(status); };
  if (cudaMalloc((void**)&logp, (size_t)VC * sizeof(float)) != cudaSuccess || cudaMalloc((void**)&status, sizeof(int)) != cudaSuccess) {
    release();
    return pcb_fail(PCB_ERR_CUDA, "pairwise MI: scratch allocation failed");
  }
  cudaMemsetAsync(counts, 0, (size_t)VC * sizeof(unsigned int), st);
  cudaMemsetAsync(status, 0, sizeof(int), st);
  cudaMemsetAsync(mi_dev, 0, (size_t)num_vars * num_vars * sizeof(float), st);
  const float z = (float)num_rows + pseudocount;
  mi_hist_kernel<<<dim3(num_vars, (uint32_t)std::min<uint64_t>(64, (num_rows + 255) / 256)), 256, 0, st>>>(data_dev, num_rows, num_vars,
                                                                                                         num_cats, counts);
  mi_logp_kernel<<<(VC + 255) / 256, 256, 0, st>>>(counts, VC, pseudocount / (float)num_cats, z, logp);
  static PcbPerDeviceOnce once;
  cudaError_t ce = once.run([] {
    return cudaFuncSetAttribute(mi_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
  });
  if (ce != cudaSuccess) { release(); return pcb_fail(PCB_ERR_CUDA, std::string("pairwise MI: ") + cudaGetErrorString(ce)); }
  MiArgs a{data_dev, num_rows, num_vars, num_cats, (VC + TILE - 1) / TILE, logp,
           pseudocount / ((float)num_cats * (float)num_cats), z, mi_dev, status};
  const uint64_t blocks = (uint64_t)a.tiles * (a.tiles + 1) / 2;
  if (blocks > 0x7fffffffull) { release(); return pcb_fail(PCB_ERR_INVALID, "pairwise MI: too many tiles for one launch"); }
  mi_tile_kernel<<<(uint32_t)blocks, NTHREADS, SMEM, st>>>(a);
  int h = 0;
  ce = cudaMemcpyAsync(&h, status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
  release();
  if (ce != cudaSuccess) return pcb_fail(PCB_ERR_CUDA, std::string("pairwise MI: ") + cudaGetErrorString(ce));
  if (h != 0) return pcb_fail(PCB_ERR_CUDA, "pairwise MI: a kernel gave up a bounded wait");
  return PCB_OK;
}
