// pcb_sample.cu — top-down sampling.
//
//  * pcb_sample_hard: Gumbel-max walk.  At a sum node the lanes of a warp split the edges, the
//    arg-max of key = logp + g(u) (lowest index on ties) picks the edge; a product node passes all
//    its children on; a leaf does the same arg-max over its categories.  The keys that decide are
//    fp64 values of the shared host/device routine of include/pcb200_gumbel.h; an fp32 evaluation
//    with an error bound first removes the entries that cannot win (warp_select64).  One CTA per
//    sample takes the pending nodes of a round in parallel (sample_hard_cta_kernel); one warp per
//    sample with a stack (sample_hard_kernel) serves very wide circuits and the entry point that
//    allocates nothing.
//    This is the temperature -> 0 limit of the reference's relaxed sampler
//    (VariationalJuice.jl/src/queries/sample.jl:8-148,233-296), fed with caller-supplied
//    uniforms instead of the in-kernel rand(Float32) of sample.jl:45.
//  * pcb_sample_soft: the relaxed sampler itself — gumbel_params_down_kernel (sample.jl:8-58),
//    gumbel_sample_down_kernel (:60-148), gumbel_input_sample_down_kernel (:233-296).
#include <algorithm>
#include <mutex>

#include "../../include/pcb200_gumbel.h"
#include "pcb_internal.h"

namespace {

struct Shape2 {
  dim3 block, grid;
};
Shape2 shape_for(uint32_t S, uint32_t items) {
  uint32_t bx = 1;
  while (bx < S && bx < 32) bx <<= 1;
  uint32_t by = 128 / bx;
  Shape2 s;
  s.block = dim3(bx, by, 1);
  s.grid = dim3((items + by - 1) / by, (S + bx - 1) / bx, 1);
  return s;
}

__device__ __forceinline__ void warp_argmax(double& key, uint32_t& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    double ok = __shfl_xor_sync(0xffffffffu, key, o);
    uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oi != 0xffffffffu && (idx == 0xffffffffu || ok > key || (ok == key && oi < idx))) {
      key = ok;
      idx = oi;
    }
  }
}

// Arg-max of up to 64 Gumbel keys by one warp (entries `lane` and `lane + 32`), with the same result
// as the fp64 arg-max above, bit for bit, at a fraction of its cost: every key is first evaluated in
// fp32 together with a bound eps on its distance from the fp64 key; an entry whose upper bound lies
// below the best lower bound cannot win and drops out.  Almost always a single candidate is left and
// is the answer; otherwise the fp64 keys of the candidates alone decide (lowest index on ties, as
// before: an entry that dropped out is strictly below the winner, so it takes no part in a tie).
// Bound: x = u (1 - 1e-6) + 1e-6 carries a relative error <= 2.4e-7 in fp32, so inner = -log x is off
// by <= 2.4e-7 (1 + inner) + 1 ulp, g = -log inner by that over inner plus 1 ulp, the sum by 1 ulp more;
// eps takes four times the total.  Entries whose inner is below 1e-4 (u within 1e-4 of one, where the
// relative error of inner is no longer small) always stay candidates.
__device__ __forceinline__ void key32(float lp, float u, float& key, float& eps) {
  const float x = fmaf(u, 0.999999f, 1e-6f);
  const float inner = -logf(x);
  const float g = -logf(inner);
  key = lp + g;
  eps = inner < 1e-4f ? INFINITY : 1e-6f * (1.0f / inner + 2.0f + fabsf(g) + fabsf(lp));
  if (lp == -INFINITY) { key = -INFINITY; eps = 0.0f; }
}
__device__ __forceinline__ uint32_t warp_select64(float lp0, float u0, bool v0, float lp1, float u1, bool v1, uint32_t lane,
                                                  bool exact) {
  float k0 = -INFINITY, e0 = 0.0f, k1 = -INFINITY, e1 = 0.0f;
  if (v0) key32(lp0, u0, k0, e0);
  if (v1) key32(lp1, u1, k1, e1);
  if (exact) { e0 = INFINITY; e1 = INFINITY; }   // cross-check switch: every entry stays a candidate, fp64 decides
  // best lower bound over the warp
  float lo = fmaxf(v0 ? k0 - e0 : -INFINITY, v1 ? k1 - e1 : -INFINITY);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lo = fmaxf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
  const bool all_impossible = lo == -INFINITY;            // every key is -inf (or unbounded): decide in fp64
  const bool c0 = v0 && (all_impossible || k0 + e0 >= lo);
  const bool c1 = v1 && (all_impossible || k1 + e1 >= lo);
  const uint32_t b0 = __ballot_sync(0xffffffffu, c0), b1 = __ballot_sync(0xffffffffu, c1);
  if (__popc(b0) + __popc(b1) == 1) return b0 ? (uint32_t)__ffs(b0) - 1u : 32u + (uint32_t)__ffs(b1) - 1u;
  double best = 0.0;
  uint32_t bi = 0xffffffffu;
  if (c0) { best = pcb_gumbel_key(lp0, u0); bi = lane; }
  if (c1) {
    const double key = pcb_gumbel_key(lp1, u1);
    if (bi == 0xffffffffu || key > best) { best = key; bi = lane + 32; }
  }
  warp_argmax(best, bi);
  return bi;
}

// status word: 0 ok, 1 stack overflow, 2 iteration limit (malformed circuit)
__global__ void sample_hard_kernel(uint32_t S, const float* __restrict__ params, uint32_t Sp,
                                   const float* __restrict__ u_sum, const float* __restrict__ u_leaf, uint32_t R,
                                   uint32_t kmax, uint32_t cmax, uint32_t V, uint32_t N,
                                   const uint8_t* __restrict__ kind, const uint32_t* __restrict__ n_estart,
                                   const uint32_t* __restrict__ n_ecount, const uint32_t* __restrict__ n_pid0,
                                   const uint32_t* __restrict__ n_region, const uint32_t* __restrict__ e_prime,
                                   const uint32_t* __restrict__ e_sub, const uint32_t* __restrict__ node2input,
                                   const uint32_t* __restrict__ in_var, const uint32_t* __restrict__ in_cats,
                                   const uint64_t* __restrict__ in_poff, uint64_t P,
                                   const float* __restrict__ theta, uint32_t* __restrict__ stack_all,
                                   uint32_t stack_cap, int32_t* __restrict__ x_out, int32_t* __restrict__ status,
                                   uint32_t smem_stack, const uint4* __restrict__ s_node,
                                   const uint4* __restrict__ s_leaf, bool exact) {
  extern __shared__ uint32_t sstack[];   // [warps per block][stack_cap] when smem_stack is set
  const uint32_t s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (s >= S) return;
  const size_t ps = Sp == 1 ? 0 : s, pld = Sp;
  // the walk pops and pushes once per visited node: with the stack in shared memory those are not
  // global round trips on the walk's dependent chain
  uint32_t* stack = smem_stack ? sstack + (size_t)(threadIdx.x >> 5) * stack_cap : stack_all + (size_t)s * stack_cap;
  for (uint32_t v = lane; v < V; v += 32) x_out[s + (size_t)S * v] = -1;
  uint32_t sp = 1;
  if (lane == 0) stack[0] = N - 1;
  __syncwarp();
  const uint32_t max_iter = 4u * N + 8u;
  for (uint32_t it = 0; sp > 0; ++it) {
    if (it >= max_iter) {
      if (lane == 0) atomicMax(status, 2);
      break;
    }
    uint32_t n = stack[--sp];
    __syncwarp();
    const uint4 nm = s_node[n];             // one load instead of kind / edge range / parameter id / region
    const uint8_t kd = (uint8_t)(nm.w & 3u);
    if (kd == PCB_INPUT) {
      uint32_t C = nm.y & 0xffffu, var = nm.y >> 16;
      uint64_t off = nm.x;
      if (nm.x == 0xffffffffu) {   // a leaf whose record did not fit the node's own
        const uint4 lm = s_leaf[nm.z];
        C = lm.z; var = lm.w;
        off = (uint64_t)lm.x | ((uint64_t)lm.y << 32);
      }
      const float* us = u_leaf + ((size_t)s * V + var) * cmax;
      double best = 0.0;
      uint32_t bi = 0xffffffffu;
      // fixed leaves keep their log-probs in the circuit, not in the caller's parameter matrix
      if (C <= 64) {
        const bool v0 = lane < C, v1 = lane + 32 < C;
        auto lpa = [&](uint32_t c) { return off < P ? params[ps + pld * (off + c)] : theta[off + c]; };
        bi = warp_select64(v0 ? lpa(lane) : 0.0f, v0 ? us[lane] : 0.0f, v0, v1 ? lpa(lane + 32) : 0.0f,
                           v1 ? us[lane + 32] : 0.0f, v1, lane, exact);
      } else {
        for (uint32_t c = lane; c < C; c += 32) {
          float lp = off < P ? params[ps + pld * (off + c)] : theta[off + c];
          double key = pcb_gumbel_key(lp, us[c]);
          if (bi == 0xffffffffu || key > best) { best = key; bi = c; }
        }
        warp_argmax(best, bi);
      }
      if (lane == 0) x_out[s + (size_t)S * var] = (int32_t)bi;
    } else if (kd == PCB_PRODUCT) {
      uint32_t e0 = nm.x, cnt = nm.y;
      // count pushes first so that every lane keeps the same stack pointer
      uint32_t pushes = 0;
      for (uint32_t j = lane; j < cnt; j += 32) pushes += e_sub[e0 + j] != PCB_NONE ? 2 : 1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) pushes += __shfl_xor_sync(0xffffffffu, pushes, o);
      if (sp + pushes > stack_cap) {
        if (lane == 0) atomicMax(status, 1);
        break;
      }
      if (lane == 0) {
        uint32_t q = sp;
        for (uint32_t j = 0; j < cnt; ++j) {
          stack[q++] = e_prime[e0 + j];
          uint32_t sb = e_sub[e0 + j];
          if (sb != PCB_NONE) stack[q++] = sb;
        }
      }
      sp += pushes;
      __syncwarp();
    } else {
      uint32_t e0 = nm.x, cnt = nm.y, pid0 = nm.z;
      const float* us = u_sum + ((size_t)s * R + (nm.w >> 2)) * kmax;
      double best = 0.0;
      uint32_t bi = 0xffffffffu;
      // the children of this lane's first two edges are fetched with the parameters, not after the
      // arg-max: one dependent load less on the walk's chain
      uint32_t pr0 = PCB_NONE, sb0 = PCB_NONE, pr1 = PCB_NONE, sb1 = PCB_NONE;
      if (lane < cnt) { pr0 = e_prime[e0 + lane]; sb0 = e_sub[e0 + lane]; }
      if (lane + 32 < cnt) { pr1 = e_prime[e0 + lane + 32]; sb1 = e_sub[e0 + lane + 32]; }
      if (cnt <= 64) {
        const bool v0 = lane < cnt, v1 = lane + 32 < cnt;
        bi = warp_select64(v0 ? params[ps + pld * (size_t)(pid0 + lane)] : 0.0f, v0 ? us[lane] : 0.0f, v0,
                           v1 ? params[ps + pld * (size_t)(pid0 + lane + 32)] : 0.0f, v1 ? us[lane + 32] : 0.0f, v1, lane, exact);
      } else {
        for (uint32_t j = lane; j < cnt; j += 32) {
          double key = pcb_gumbel_key(params[ps + pld * (size_t)(pid0 + j)], us[j]);
          if (bi == 0xffffffffu || key > best) { best = key; bi = j; }
        }
        warp_argmax(best, bi);
      }
      uint32_t pr, sb;
      if (bi < 64) {
        const uint32_t src = bi & 31u;
        const uint32_t a = __shfl_sync(0xffffffffu, bi < 32 ? pr0 : pr1, src);
        const uint32_t b = __shfl_sync(0xffffffffu, bi < 32 ? sb0 : sb1, src);
        pr = a; sb = b;
      } else {
        pr = e_prime[e0 + bi]; sb = e_sub[e0 + bi];
      }
      uint32_t pushes = sb != PCB_NONE ? 2 : 1;
      if (sp + pushes > stack_cap) {
        if (lane == 0) atomicMax(status, 1);
        break;
      }
      if (lane == 0) {
        stack[sp] = pr;
        if (sb != PCB_NONE) stack[sp + 1] = sb;
      }
      sp += pushes;
      __syncwarp();
    }
  }
}

// The same walk with one CTA per sample: the pending nodes of a sample are roots of sub-circuits over
// disjoint scopes, so they are independent, and a single warp that visits them one after another
// spends its time in the dependent loads of each visit (node record -> parameters and noise ->
// children: ~1.8 us per visit, 1600 visits per sample at 784 variables).  Here the warps of the CTA
// take the pending nodes of a round in parallel and push what they select to the next round's list
// (two lists in shared memory, at most one pending node per variable, so V + 2 entries each); the
// arg-max at a node is the same computation, so the samples are the same bit for bit.
#ifndef PCB_SAMPLE_CTA_WARPS
#define PCB_SAMPLE_CTA_WARPS 4
#endif
constexpr uint32_t CW = PCB_SAMPLE_CTA_WARPS;   // warps per sample
__global__ void __launch_bounds__(CW * 32) sample_hard_cta_kernel(
    uint32_t S, const float* __restrict__ params, uint32_t Sp, const float* __restrict__ u_sum,
    const float* __restrict__ u_leaf, uint32_t R, uint32_t kmax, uint32_t cmax, uint32_t V, uint32_t N,
    const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub, uint64_t P, const float* __restrict__ theta,
    uint32_t cap, int32_t* __restrict__ x_out, int32_t* __restrict__ status, const uint4* __restrict__ s_node,
    const uint4* __restrict__ s_leaf, bool exact) {
  extern __shared__ uint32_t lists[];   // [2][cap]
  __shared__ uint32_t count[2];
  const uint32_t s = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t ps = Sp == 1 ? 0 : s, pld = Sp;
  for (uint32_t v = threadIdx.x; v < V; v += blockDim.x) x_out[s + (size_t)S * v] = -1;
  if (threadIdx.x == 0) { lists[0] = N - 1; count[0] = 1; count[1] = 0; }
  __syncthreads();
  uint32_t cur = 0;
  for (uint32_t round = 0;; ++round) {
    const uint32_t n_cur = count[cur];
    if (n_cur == 0) break;
    if (round > N + 8u) {   // a circuit is at most N levels deep
      if (threadIdx.x == 0) atomicMax(status, 2);
      break;
    }
    __syncthreads();                       // every thread has read the count
    if (threadIdx.x == 0) count[cur] = 0;  // this list is the next round's target after the one being filled
    uint32_t* out = lists + (cur ^ 1u) * cap;
    uint32_t* out_n = &count[cur ^ 1u];
    for (uint32_t idx = warp; idx < n_cur; idx += CW) {
      const uint32_t n = lists[cur * cap + idx];
      const uint4 nm = s_node[n];
      const uint8_t kd = (uint8_t)(nm.w & 3u);
      if (kd == PCB_INPUT) {
        uint32_t C = nm.y & 0xffffu, var = nm.y >> 16;
        uint64_t off = nm.x;
        if (nm.x == 0xffffffffu) {
          const uint4 lm = s_leaf[nm.z];
          C = lm.z; var = lm.w;
          off = (uint64_t)lm.x | ((uint64_t)lm.y << 32);
        }
        const float* us = u_leaf + ((size_t)s * V + var) * cmax;
        double best = 0.0;
        uint32_t bi = 0xffffffffu;
        if (C <= 64) {
          const bool v0 = lane < C, v1 = lane + 32 < C;
          auto lpa = [&](uint32_t c) { return off < P ? params[ps + pld * (off + c)] : theta[off + c]; };
          bi = warp_select64(v0 ? lpa(lane) : 0.0f, v0 ? us[lane] : 0.0f, v0, v1 ? lpa(lane + 32) : 0.0f,
                             v1 ? us[lane + 32] : 0.0f, v1, lane, exact);
        } else {
          for (uint32_t c = lane; c < C; c += 32) {
            float lp = off < P ? params[ps + pld * (off + c)] : theta[off + c];
            double key = pcb_gumbel_key(lp, us[c]);
            if (bi == 0xffffffffu || key > best) { best = key; bi = c; }
          }
          warp_argmax(best, bi);
        }
        if (lane == 0) x_out[s + (size_t)S * var] = (int32_t)bi;
      } else if (kd == PCB_PRODUCT) {
        const uint32_t e0 = nm.x, cnt = nm.y;
        for (uint32_t j = lane; j < cnt; j += 32) {
          const uint32_t pr = e_prime[e0 + j], sb = e_sub[e0 + j];
          const uint32_t np = sb != PCB_NONE ? 2u : 1u;
          const uint32_t pos = atomicAdd(out_n, np);
          if (pos + np > cap) { atomicMax(status, 1); continue; }
          out[pos] = pr;
          if (sb != PCB_NONE) out[pos + 1] = sb;
        }
      } else {
        const uint32_t e0 = nm.x, cnt = nm.y, pid0 = nm.z;
        const float* us = u_sum + ((size_t)s * R + (nm.w >> 2)) * kmax;
        double best = 0.0;
        uint32_t bi = 0xffffffffu;
        uint32_t pr0 = PCB_NONE, sb0 = PCB_NONE, pr1 = PCB_NONE, sb1 = PCB_NONE;
        if (lane < cnt) { pr0 = e_prime[e0 + lane]; sb0 = e_sub[e0 + lane]; }
        if (lane + 32 < cnt) { pr1 = e_prime[e0 + lane + 32]; sb1 = e_sub[e0 + lane + 32]; }
        if (cnt <= 64) {
          const bool v0 = lane < cnt, v1 = lane + 32 < cnt;
          bi = warp_select64(v0 ? params[ps + pld * (size_t)(pid0 + lane)] : 0.0f, v0 ? us[lane] : 0.0f, v0,
                             v1 ? params[ps + pld * (size_t)(pid0 + lane + 32)] : 0.0f, v1 ? us[lane + 32] : 0.0f, v1, lane, exact);
        } else {
          for (uint32_t j = lane; j < cnt; j += 32) {
            double key = pcb_gumbel_key(params[ps + pld * (size_t)(pid0 + j)], us[j]);
            if (bi == 0xffffffffu || key > best) { best = key; bi = j; }
          }
          warp_argmax(best, bi);
        }
        uint32_t pr, sb;
        if (bi < 64) {
          const uint32_t src = bi & 31u;
          pr = __shfl_sync(0xffffffffu, bi < 32 ? pr0 : pr1, src);
          sb = __shfl_sync(0xffffffffu, bi < 32 ? sb0 : sb1, src);
        } else {
          pr = e_prime[e0 + bi]; sb = e_sub[e0 + bi];
        }
        if (lane == 0) {
          const uint32_t np = sb != PCB_NONE ? 2u : 1u;
          const uint32_t pos = atomicAdd(out_n, np);
          if (pos + np > cap) {
            atomicMax(status, 1);
          } else {
            out[pos] = pr;
            if (sb != PCB_NONE) out[pos + 1] = sb;
          }
        }
      }
    }
    __syncthreads();   // the next list is complete
    cur ^= 1u;
  }
}

// ---- soft sampling ------------------------------------------------------------------------------
// unnormalised relaxed edge probabilities and their per-node sums; cum is stored per sum NODE
__global__ void soft_params_kernel(float* __restrict__ eprob, float* __restrict__ cum, uint32_t ld, uint32_t S,
                                   const float* __restrict__ params, uint32_t Sp, const float* __restrict__ u,
                                   float temperature, const uint32_t* __restrict__ grp_node, uint32_t n_groups,
                                   const uint32_t* __restrict__ n_pid0, const uint32_t* __restrict__ n_ecount) {
  uint32_t g = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (g >= n_groups || s >= S) return;
  uint32_t n = grp_node[g];
  uint32_t pid0 = n_pid0[n], cnt = n_ecount[n];
  const size_t ps = Sp == 1 ? 0 : s, pld = Sp;
  float sum = 0.0f;
  for (uint32_t j = 0; j < cnt; ++j) {
    float logp = params[ps + pld * (size_t)(pid0 + j)];
    double gv = 0.0;
    if (u) gv = -log(-log((double)u[s + (size_t)S * (pid0 + j)] * (1.0 - 1e-6) + 1e-6));
    float unnorm = (float)exp(((double)logp + gv) / (double)temperature);
    eprob[(size_t)(pid0 + j) * ld + s] = unnorm;
    sum += unnorm;
  }
  cum[(size_t)n * ld + s] = sum;
}

__global__ void soft_down_kernel(float* __restrict__ td, uint32_t ld, uint32_t S, const float* __restrict__ eprob,
                                 const float* __restrict__ cum, const uint32_t* __restrict__ nodes, uint32_t count,
                                 uint32_t root, const uint32_t* __restrict__ in_off,
                                 const PcbInEntry* __restrict__ in_ent) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= count || s >= S) return;
  uint32_t n = nodes[i];
  uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  float acc = (i0 == i1 && n == root) ? 1.0f : 0.0f;
  for (uint32_t x = i0; x < i1; ++x) {
    PcbInEntry en = in_ent[x];
    float tp = td[(size_t)en.parent * ld + s];
    if (en.pid != PCB_NONE) tp *= eprob[(size_t)en.pid * ld + s] / cum[(size_t)en.parent * ld + s];
    acc += tp;
  }
  td[(size_t)n * ld + s] = acc;
}

__global__ void soft_leaf_kernel(const float* __restrict__ td, uint32_t ld, uint32_t S,
                                 const float* __restrict__ params, uint32_t Sp, uint32_t n_inputs, uint32_t V,
                                 const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_var,
                                 const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                 uint64_t P, const float* __restrict__ theta, float* __restrict__ out) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n_inputs || s >= S) return;
  const size_t ps = Sp == 1 ? 0 : s, pld = Sp;
  float tp = td[(size_t)in_node[i] * ld + s];
  uint32_t C = in_cats[i], var = in_var[i];
  uint64_t off = in_poff[i];
  for (uint32_t k = 0; k < C; ++k) {
    // fixed leaves keep their log-probs in the circuit, not in the caller's parameter matrix
    float lp = off < P ? params[ps + pld * (off + k)] : theta[off + k];
    atomicAdd(out + s + (size_t)S * (var + (size_t)V * k), tp * expf(lp));
  }
}

}  // namespace

extern "C" int32_t pcb_sample_hard(pcb_circuit* c, pcb_workspace* ws, const float* params_dev, uint32_t Sp,
                                   const float* u_sum_dev, const float* u_leaf_dev, uint32_t S, int32_t* x_out_dev,
                                   pcb_stream s) {
  PCB_REQUIRE(c && ws && params_dev && u_leaf_dev && x_out_dev, "null argument");
  PCB_REQUIRE(u_sum_dev || c->n_regions == 0, "u_sum missing");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(S >= 1 && (Sp == 1 || Sp == S), "params must hold 1 or S parameter sets");
  PCB_CUDA(cudaSetDevice(c->device));
  // one CTA per sample keeps its lists in shared memory; only the one-warp walk of a very wide circuit
  // (or on request) needs stacks in global memory
  const bool cta_walk = (size_t)2 * (c->V + 2) * 4 <= 40 * 1024 && !c->sample_walk_warp;
  int32_t st0 = pcb_ws_ensure_sets(ws, S, cta_walk ? 0 : PCB_WS_STACK);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  int32_t* status = ws->sample_status;
  PCB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  if (cta_walk) {
    // one CTA per sample, its warps sharing the rounds of pending nodes
    ++c->prof.launches[PCB_K_SAMPLE];
    sample_hard_cta_kernel<<<S, CW * 32, (size_t)2 * ws->stack_cap * 4, st>>>(
        S, params_dev, Sp, u_sum_dev, u_leaf_dev, c->n_regions, c->max_group, c->max_cats, c->V, c->N, c->e_prime, c->e_sub,
        c->P, c->theta, ws->stack_cap, x_out_dev, status, c->s_node, c->s_leaf, c->sample_exact_keys);
    PCB_CUDA(cudaGetLastError());
    int32_t h0 = 0;
    PCB_CUDA(cudaMemcpyAsync(&h0, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    PCB_CUDA(cudaStreamSynchronize(st));
    if (h0 == 1) return pcb_fail(PCB_ERR_TOO_LARGE, "sampling walk overflowed its lists (circuit not decomposable?)");
    if (h0 == 2) return pcb_fail(PCB_ERR_INVALID, "sampling walk exceeded its round limit (malformed circuit)");
    return PCB_OK;
  }
  uint32_t warps_per_block = 4;
  while (warps_per_block > 1 && (size_t)warps_per_block * ws->stack_cap * 4 > 48 * 1024) warps_per_block /= 2;
  const size_t sm = (size_t)warps_per_block * ws->stack_cap * 4;
  const uint32_t smem_stack = sm <= 48 * 1024 ? 1u : 0u;
  ++c->prof.launches[PCB_K_SAMPLE];
  sample_hard_kernel<<<(S + warps_per_block - 1) / warps_per_block, warps_per_block * 32, smem_stack ? sm : 0, st>>>(
      S, params_dev, Sp, u_sum_dev, u_leaf_dev, c->n_regions, c->max_group, c->max_cats, c->V, c->N, c->kind,
      c->n_estart, c->n_ecount, c->n_pid0, c->n_region, c->e_prime, c->e_sub, c->node2input, c->in_var, c->in_cats,
      c->in_poff, c->P, c->theta, ws->stack, ws->stack_cap, x_out_dev, status, smem_stack, c->s_node, c->s_leaf,
      c->sample_exact_keys);
  PCB_CUDA(cudaGetLastError());
  int32_t h = 0;
  PCB_CUDA(cudaMemcpyAsync(&h, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  PCB_CUDA(cudaStreamSynchronize(st));
  if (h == 1) return pcb_fail(PCB_ERR_TOO_LARGE, "sampling walk overflowed its stack (circuit not decomposable?)");
  if (h == 2) return pcb_fail(PCB_ERR_INVALID, "sampling walk exceeded its iteration limit (malformed circuit)");
  return PCB_OK;
}

extern "C" int32_t pcb_sample_soft(pcb_circuit* c, pcb_workspace* ws, const float* params_dev, uint32_t Sp,
                                   const float* u_dev, float temperature, uint32_t S, float* out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && params_dev && out_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(S >= 1 && (Sp == 1 || Sp == S), "params must hold 1 or S parameter sets");
  PCB_REQUIRE(temperature > 0.0f, "temperature must be positive");
  PCB_CUDA(cudaSetDevice(c->device));
  int32_t st0 = pcb_ws_ensure_sets(ws, S, PCB_WS_NODES | PCB_WS_EDGES);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t ld = ws->ldS;
  ws->have_kld = false;  // klds rows are reused for the per-node normalisers
  float* cum = ws->klds;
  float* td = ws->grads;
  PCB_CUDA(cudaMemsetAsync(out_dev, 0, (size_t)S * c->V * c->max_cats * sizeof(float), st));
  if (c->n_groups) {
    Shape2 sh = shape_for(S, c->n_groups);
    ++c->prof.launches[PCB_K_SAMPLE];
    soft_params_kernel<<<sh.grid, sh.block, 0, st>>>(ws->eprob, cum, ld, S, params_dev, Sp, u_dev, temperature,
                                                     c->grp_node, c->n_groups, c->n_pid0, c->n_ecount);
  }
  for (int64_t lay = c->L; lay >= 0; --lay) {
    uint32_t o0 = c->h_down_all_off[lay], o1 = c->h_down_all_off[lay + 1];
    if (o1 == o0) continue;
    Shape2 sh = shape_for(S, o1 - o0);
    ++c->prof.launches[PCB_K_SAMPLE];
    soft_down_kernel<<<sh.grid, sh.block, 0, st>>>(td, ld, S, ws->eprob, cum, c->down_all + o0, o1 - o0, c->N - 1,
                                                   c->in_off, c->in_ent);
  }
  if (c->n_inputs) {
    Shape2 sh = shape_for(S, c->n_inputs);
    ++c->prof.launches[PCB_K_SAMPLE];
    soft_leaf_kernel<<<sh.grid, sh.block, 0, st>>>(td, ld, S, params_dev, Sp, c->n_inputs, c->V, c->in_node, c->in_var,
                                                   c->in_cats, c->in_poff, c->P, c->theta, out_dev);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

// ---- conditioned top-down probabilities ------------------------------------------------------------------
// conditioned_td_prob (queries/td_prob.jl:161-291): the top-down pass with the circuit's own weights in
// which a marked inner node does not take what its parents send but node_probs[s, z_var, z_cat]; the
// leaves then spread their probability over their categories (gumbel_input_sample_down with the
// circuit's leaf parameters, queries/sample.jl:233-336).  As in the reference nothing starts at the
// root: an unmarked node without parents has probability 0.
namespace {
__global__ void cond_td_down_kernel(float* __restrict__ td, uint32_t ld, uint32_t S, const float* __restrict__ theta,
                                    const uint32_t* __restrict__ nodes, uint32_t count, const uint8_t* __restrict__ kind,
                                    const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                                    const int32_t* __restrict__ marked_var, const int32_t* __restrict__ marked_cat,
                                    const float* __restrict__ node_probs, uint32_t Z1) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= count || s >= S) return;
  const uint32_t n = nodes[i];
  float acc = 0.0f;
  if (kind[n] != PCB_INPUT && marked_var[n] > 0) {
    acc = node_probs[s + (size_t)S * ((uint32_t)(marked_var[n] - 1) + (size_t)Z1 * (uint32_t)(marked_cat[n] - 1))];
  } else {
    for (uint32_t x = in_off[n]; x < in_off[n + 1]; ++x) {
      const PcbInEntry en = in_ent[x];
      float tp = td[(size_t)en.parent * ld + s];
      if (en.pid != PCB_NONE) tp *= expf(__ldg(theta + en.pid));
      acc += tp;
    }
  }
  td[(size_t)n * ld + s] = acc;
}
}  // namespace

extern "C" int32_t pcb_cond_td_prob(pcb_circuit* c, pcb_workspace* ws, const int32_t* marked_var_dev,
                                    const int32_t* marked_cat_dev, const float* node_probs_dev, uint32_t S, uint32_t Z1,
                                    float* out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && marked_var_dev && marked_cat_dev && node_probs_dev && out_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(S >= 1 && Z1 >= 1, "empty input");
  PCB_CUDA(cudaSetDevice(c->device));
  int32_t st0 = pcb_ws_ensure_sets(ws, S, PCB_WS_NODES);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t ld = ws->ldS;
  ws->have_kld = false;   // the gradient rows are reused for the top-down probabilities
  float* td = ws->grads;
  PCB_CUDA(cudaMemsetAsync(out_dev, 0, (size_t)S * c->V * c->max_cats * sizeof(float), st));
  for (int64_t lay = c->L; lay >= 0; --lay) {
    uint32_t o0 = c->h_down_all_off[lay], o1 = c->h_down_all_off[lay + 1];
    if (o1 == o0) continue;
    Shape2 sh = shape_for(S, o1 - o0);
    ++c->prof.launches[PCB_K_SAMPLE];
    cond_td_down_kernel<<<sh.grid, sh.block, 0, st>>>(td, ld, S, c->theta, c->down_all + o0, o1 - o0, c->kind, c->in_off,
                                                      c->in_ent, marked_var_dev, marked_cat_dev, node_probs_dev, Z1);
  }
  if (c->n_inputs) {
    Shape2 sh = shape_for(S, c->n_inputs);
    ++c->prof.launches[PCB_K_SAMPLE];
    soft_leaf_kernel<<<sh.grid, sh.block, 0, st>>>(td, ld, S, c->theta, 1, c->n_inputs, c->V, c->in_node, c->in_var,
                                                   c->in_cats, c->in_poff, c->P, c->theta, out_dev);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

// ---- hard sampling without any allocation --------------------------------------------------------------
// Some hosts of this library must not see it allocate device memory.  Julia's CUDA.jl, which is
// where the reference lives, keeps nearly all free device memory in its own pool, so a
// cudaMalloc issued behind its back can fail with memory "free" from Julia's point of view, and
// it synchronises the whole device under the caller's running streams; a serving loop that has
// already handed every byte to its own arena is in the same position.  pcb_sample_hard needs a
// workspace and grows it on demand; this variant keeps the per-sample walk stacks (and the
// status word the bounded walk reports to) in a fixed array that is part of the library image
// instead, so every GPU that loads the library holds PCB_STATIC_SAMPLE_WORDS * 4 bytes (4 MiB)
// of it until the process exits.
//
// The array is shared by all calls on a device and keeps whatever the last call left in it:
// stacks are written before they are read and the status word is cleared on the stream at the
// start of every call, but two calls whose kernels overlap on the GPU (different streams) race.
// A circuit with at most 12 286 variables keeps one warp's stack within 48 KB of shared memory and
// then only the status word of the array is used; larger circuits walk on the array itself.
// Like pcb_sample_hard the call ends by reading the status word back and waiting for the stream,
// so it cannot be made while that stream is being captured.
#define PCB_STATIC_SAMPLE_WORDS (1u << 20)
static __device__ __align__(256) uint32_t g_static_sample_scratch[PCB_STATIC_SAMPLE_WORDS + 64];

namespace {
constexpr int kMaxDevices = 64;
uint32_t* g_scratch_addr[kMaxDevices] = {nullptr};  // device address of the array, per device
std::mutex g_scratch_mutex;                          // host threads may make their first calls together

// In host code the array's name is only a handle for the runtime, not a device pointer: the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device while that
// device is current.
int32_t static_scratch(int device, uint32_t** out) {
  PCB_REQUIRE(device >= 0 && device < kMaxDevices, "device index beyond the static scratch table");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[device]) {
    uint32_t* p = nullptr;
    PCB_CUDA(cudaGetSymbolAddress((void**)&p, g_static_sample_scratch));
    g_scratch_addr[device] = p;
  }
  *out = g_scratch_addr[device];
  return PCB_OK;
}
}  // namespace

extern "C" int32_t pcb_sample_hard_static(pcb_circuit* c, const float* params_dev, uint32_t Sp,
                                          const float* u_sum_dev, const float* u_leaf_dev, uint32_t S,
                                          int32_t* x_out_dev, pcb_stream s) {
  PCB_REQUIRE(c && params_dev && u_leaf_dev && x_out_dev, "null argument");
  PCB_REQUIRE(u_sum_dev || c->n_regions == 0, "u_sum missing");
  PCB_REQUIRE(S >= 1 && (Sp == 1 || Sp == S), "params must hold 1 or S parameter sets");
  const uint64_t stack_cap = (uint64_t)c->V + 2;
  if ((uint64_t)S * stack_cap > PCB_STATIC_SAMPLE_WORDS)
    return pcb_fail(PCB_ERR_TOO_LARGE,
                    "pcb_sample_hard_static: S * (num_vars + 2) = " + std::to_string((uint64_t)S * stack_cap) +
                        " exceeds the static scratch of " + std::to_string(PCB_STATIC_SAMPLE_WORDS) +
                        " words; sample in smaller groups or use pcb_sample_hard");
  PCB_CUDA(cudaSetDevice(c->device));
  uint32_t* scratch = nullptr;
  int32_t st0 = static_scratch(c->device, &scratch);   // first call on a device resolves the symbol
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  int32_t* status = reinterpret_cast<int32_t*>(scratch + PCB_STATIC_SAMPLE_WORDS);
  PCB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  uint32_t warps_per_block = 4;
  while (warps_per_block > 1 && (size_t)warps_per_block * stack_cap * 4 > 48 * 1024) warps_per_block /= 2;
  const size_t sm = (size_t)warps_per_block * stack_cap * 4;
  const uint32_t smem_stack = sm <= 48 * 1024 ? 1u : 0u;   // else the walk stacks stay in the static scratch
  ++c->prof.launches[PCB_K_SAMPLE];
  sample_hard_kernel<<<(S + warps_per_block - 1) / warps_per_block, warps_per_block * 32, smem_stack ? sm : 0, st>>>(
      S, params_dev, Sp, u_sum_dev, u_leaf_dev, c->n_regions, c->max_group, c->max_cats, c->V, c->N, c->kind,
      c->n_estart, c->n_ecount, c->n_pid0, c->n_region, c->e_prime, c->e_sub, c->node2input, c->in_var, c->in_cats,
      c->in_poff, c->P, c->theta, scratch, (uint32_t)stack_cap, x_out_dev, status, smem_stack, c->s_node, c->s_leaf,
      c->sample_exact_keys);
  PCB_CUDA(cudaGetLastError());
  int32_t h = 0;
  PCB_CUDA(cudaMemcpyAsync(&h, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  PCB_CUDA(cudaStreamSynchronize(st));
  if (h == 1) return pcb_fail(PCB_ERR_TOO_LARGE, "sampling walk overflowed its stack (circuit not decomposable?)");
  if (h == 2) return pcb_fail(PCB_ERR_INVALID, "sampling walk exceeded its iteration limit (malformed circuit)");
  return PCB_OK;
}
