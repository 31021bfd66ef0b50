// pcb_em.cu — forward pass, backward flow pass, leaf statistics and the fused EM update.
//
// Reference kernels replaced (paths relative to VariationalJuice.jl/src):
//   leaf_forward_kernel    init_mar!_with_reg_kernel       regularization/reg_likelihood.jl:16-49
//   sparse_up_kernel       layer_up_kernel                 queries/likelihood.jl:4-68
//   sparse_down_kernel     layer_down_kernel / reg_layer_down_kernel
//                                                          queries/flow.jl:8-106, regularization/reg_flow.jl:120-222
//   leaf_flow_kernel       input_flows_circuit_with_reg_kernel   regularization/reg_flow.jl:24-48
//   em_update_*_kernel     add_pseudocount + aggr_node_flows + update_params + update_input_node_params
//                                                          regularization/reg_em.jl:292-299 (arithmetic:
//                                                          pretrain/mini_batch_warmup.jl:4-76, sgd/adam.jl:27-37,
//                                                          nodes/fixable_categorical_dist.jl:223-248)
//
// All kernels put the example index on threadIdx.x, so every access to a work matrix is a
// 128-byte coalesced row segment and edge metadata is a warp-wide broadcast.  The top-down pass
// is pull-based (CSR by child): a node sums the flows of its incoming edges itself, so node flows
// need no atomics and no zero-fill; only the per-edge statistics are reduced (warp shuffle, then
// one atomic per warp and edge).
#include <algorithm>

#include <cstring>

#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {

constexpr int TPB = 128;  // threads per block along the example axis

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int64_t data_row(const int32_t* row_ids, uint32_t row_start, uint32_t b) {
  return row_ids ? (int64_t)row_ids[b] - 1 : (int64_t)row_start - 1 + b;
}

// One thread per (node, four consecutive examples): every row access is a 16-byte load, so a warp
// keeps 512 bytes per request in flight (the chain node -> edge list -> child row is four dependent
// loads deep; with one example per thread it ran at a third of the memory roof).  Sum nodes: two
// passes over the children (max, then sum of exp), one exp per edge instead of the exp + log of a
// binary fold.  The last thread of a row may cover padding examples: the row pitch is a multiple
// of 32, and whatever lands in the padding is never read as a result.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 adds4(float4 a, float s) { return make_float4(a.x + s, a.y + s, a.z + s, a.w + s); }
__device__ __forceinline__ float4 max4(float4 a, float4 b) {
  return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
}

__global__ void sparse_up_kernel(float* __restrict__ mars, uint32_t ld, uint32_t B,
                                 const uint32_t* __restrict__ nodes, const uint8_t* __restrict__ kind,
                                 const uint32_t* __restrict__ n_estart, const uint32_t* __restrict__ n_ecount,
                                 const uint32_t* __restrict__ n_pid0, const uint32_t* __restrict__ e_prime,
                                 const uint32_t* __restrict__ e_sub, const float* __restrict__ theta) {
  pcb_grid_dep_launch();
  uint32_t n = nodes[blockIdx.x];
  uint32_t b = (blockIdx.y * blockDim.x + threadIdx.x) * 4u;
  if (b >= B) return;
  uint32_t e0 = n_estart[n], cnt = n_ecount[n];
  pcb_grid_dep_wait();   // everything above is static circuit data
  auto child = [&](uint32_t j) {
    float4 v = ld4(mars + (size_t)e_prime[e0 + j] * ld + b);
    uint32_t sb = e_sub[e0 + j];
    if (sb != PCB_NONE) v = add4(v, ld4(mars + (size_t)sb * ld + b));
    return v;
  };
  float4 out;
  if (kind[n] == PCB_SUM) {
    const float* w = theta + n_pid0[n];
    float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    for (uint32_t j = 0; j < cnt; ++j) mx = max4(mx, adds4(child(j), __ldg(w + j)));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t j = 0; j < cnt; ++j) {
      const float4 v = adds4(child(j), __ldg(w + j));
      // a maximum of -inf (every child impossible) gives exp(nan): masked below
      acc.x += __expf(v.x - mx.x); acc.y += __expf(v.y - mx.y); acc.z += __expf(v.z - mx.z); acc.w += __expf(v.w - mx.w);
    }
    out.x = mx.x == -INFINITY ? -INFINITY : mx.x + __logf(acc.x);
    out.y = mx.y == -INFINITY ? -INFINITY : mx.y + __logf(acc.y);
    out.z = mx.z == -INFINITY ? -INFINITY : mx.z + __logf(acc.z);
    out.w = mx.w == -INFINITY ? -INFINITY : mx.w + __logf(acc.w);
  } else {
    out = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t j = 0; j < cnt; ++j) out = add4(out, child(j));
  }
  *reinterpret_cast<float4*>(mars + (size_t)n * ld + b) = out;
}

// Pull-based top-down pass: flows[n][b] = sum over incoming edges of the edge flow
//   product parent: flows[parent]; sum parent: flows[parent] * exp(child value + logp - mars[parent]).
// The root (no incoming edge, last node) gets 1, any other parentless node 0.
// Multi-head circuits (head_mask != null): the flow of head h starts at head_mask[row, h], every
// other parentless node at 0 (src-jl/multi_head_pc/flow.jl:141-176).
struct HeadInit {
  const uint32_t* n_head;
  const float* head_mask;
  uint64_t mask_rows;
  const int32_t* row_ids;
  uint32_t row_start;
};
__global__ void sparse_down_kernel(float* __restrict__ flows, const float* __restrict__ mars, uint32_t ld,
                                   uint32_t B, const uint32_t* __restrict__ nodes, uint32_t root,
                                   const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                                   const float* __restrict__ theta, float* __restrict__ aggr, HeadInit hi) {
  pcb_grid_dep_launch();
  uint32_t n = nodes[blockIdx.x];
  uint32_t b = (blockIdx.y * blockDim.x + threadIdx.x) * 4u;
  const bool any = b < B;                      // examples b .. b+3, those below B count
  const uint32_t bb = any ? b : 0;
  const bool a0 = b < B, a1 = b + 1 < B, a2 = b + 2 < B, a3 = b + 3 < B;
  uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  pcb_grid_dep_wait();   // everything above is static circuit data
  float4 acc;
  if (hi.head_mask) {
    const uint32_t h = hi.n_head[n];
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (h != PCB_NONE) {
      const float* mk = hi.head_mask + (size_t)hi.mask_rows * h;
      if (a0) acc.x = mk[data_row(hi.row_ids, hi.row_start, b)];
      if (a1) acc.y = mk[data_row(hi.row_ids, hi.row_start, b + 1)];
      if (a2) acc.z = mk[data_row(hi.row_ids, hi.row_start, b + 2)];
      if (a3) acc.w = mk[data_row(hi.row_ids, hi.row_start, b + 3)];
    }
  } else {
    const float init = (i0 == i1 && n == root) ? 1.0f : 0.0f;
    acc = make_float4(init, init, init, init);
  }
  const float4 my = ld4(mars + (size_t)n * ld + bb);
  for (uint32_t i = i0; i < i1; ++i) {
    PcbInEntry en = in_ent[i];
    float4 f = ld4(flows + (size_t)en.parent * ld + bb);
    if (en.pid != PCB_NONE) {
      const float4 pm = ld4(mars + (size_t)en.parent * ld + bb);
      const float lp = __ldg(theta + en.pid);
      // order of additions as in flow.jl:55-58: prime + logp, then + sub
      float4 child;
      if (en.sib == PCB_NONE) {
        child = adds4(my, lp);
      } else {
        const float4 sv = ld4(mars + (size_t)en.sib * ld + bb);
        child = (en.flags & 1u) ? add4(adds4(my, lp), sv) : add4(adds4(sv, lp), my);
      }
      f.x *= __expf(child.x - pm.x); f.y *= __expf(child.y - pm.y);
      f.z *= __expf(child.z - pm.z); f.w *= __expf(child.w - pm.w);
      if (aggr && (en.flags & 1u)) {   // aggr == null: flows only (uniform over the grid)
        float s = warp_sum((a0 ? f.x : 0.0f) + (a1 ? f.y : 0.0f) + (a2 ? f.z : 0.0f) + (a3 ? f.w : 0.0f));
        if ((threadIdx.x & 31) == 0) atomicAdd(aggr + en.pid, s);
      }
    }
    acc = add4(acc, f);
  }
  if (any) *reinterpret_cast<float4*>(flows + (size_t)n * ld + b) = acc;
}

// leaf statistics: aggr[foff + x_b] += flows[leaf][b] * w_b ; missing -> slot C
__global__ void leaf_flow_kernel(const float* __restrict__ flows, uint32_t ld, uint32_t B,
                                 float* __restrict__ aggr, const uint32_t* __restrict__ in_node,
                                 const uint32_t* __restrict__ in_var, const uint32_t* __restrict__ in_cats,
                                 const uint64_t* __restrict__ in_foff, const uint8_t* __restrict__ data,
                                 const uint8_t* __restrict__ miss, uint64_t num_rows,
                                 const int32_t* __restrict__ row_ids, uint32_t row_start,
                                 const float* __restrict__ weights) {
  uint32_t i = blockIdx.x;
  uint64_t fo = in_foff[i];
  if (fo == ~0ull) return;  // fixed leaf
  uint32_t b = blockIdx.y * blockDim.x + threadIdx.x;
  bool active = b < B;
  uint32_t slot = 0xffffffffu;
  float f = 0.0f;
  if (active) {
    int64_t row = data_row(row_ids, row_start, b);
    size_t di = (size_t)row + (size_t)num_rows * in_var[i];
    f = flows[(size_t)in_node[i] * ld + b];
    if (weights) f *= weights[row];
    slot = (miss && miss[di]) ? in_cats[i] : (uint32_t)data[di];
  }
  // combine the lanes of a warp that hit the same category before touching memory
  uint32_t peers = __match_any_sync(0xffffffffu, slot);
  uint32_t lane = threadIdx.x & 31;
  uint32_t leader = __ffs(peers) - 1;
  float total = 0.0f;
  for (uint32_t m = peers; m; m &= m - 1) {
    uint32_t src = __ffs(m) - 1;
    total += __shfl_sync(peers, f, src);
  }
  if (active && lane == leader) atomicAdd(aggr + fo + slot, total);
}

// ---- chunked leaf kernels -------------------------------------------------------------------------
// One block serves up to PCB_LEAF_CHUNK leaves of one variable for a tile of LBT examples: the
// variable's observed values are gathered once into shared memory (0xffff = missing) and reused
// by every leaf of the chunk, so the per-leaf work is a coalesced row read or write plus a
// table lookup that stays in L1.
constexpr int LBT = 2048;
constexpr int LTH = 256;

__device__ __forceinline__ void stage_values(uint16_t* xs, uint32_t b0, uint32_t nb, uint32_t var,
                                             const uint8_t* __restrict__ data, const uint8_t* __restrict__ miss,
                                             uint64_t num_rows, const int32_t* __restrict__ row_ids,
                                             uint32_t row_start) {
  for (uint32_t b = threadIdx.x; b < nb; b += blockDim.x) {
    int64_t row = data_row(row_ids, row_start, b0 + b);
    size_t di = (size_t)row + (size_t)num_rows * var;
    xs[b] = (miss && miss[di]) ? (uint16_t)0xffff : (uint16_t)data[di];
  }
}

__global__ void __launch_bounds__(LTH) leaf_forward_chunk_kernel(
    float* __restrict__ mars, uint32_t ld, uint32_t B, const float* __restrict__ theta,
    const uint32_t* __restrict__ in_node, const uint64_t* __restrict__ in_poff,
    const uint32_t* __restrict__ lchunk_var, const uint32_t* __restrict__ lchunk_off,
    const uint32_t* __restrict__ lchunk_inputs, const uint8_t* __restrict__ data,
    const uint8_t* __restrict__ miss, uint64_t num_rows, const int32_t* __restrict__ row_ids, uint32_t row_start) {
  __shared__ __align__(8) uint16_t xs[LBT];
  const uint32_t chunk = blockIdx.x, b0 = blockIdx.y * LBT;
  const uint32_t nb = min((uint32_t)LBT, B - b0);
  stage_values(xs, b0, nb, lchunk_var[chunk], data, miss, num_rows, row_ids, row_start);
  __syncthreads();
  // A thread takes four consecutive examples per pass (one 16-byte store per leaf and pass); its
  // examples are the same for every leaf of the group, so their values are fetched once.  The last
  // store of a row may reach into the padding of the row pitch (a multiple of 32).
  // A slice of at most 512 examples (the shard of a many-GPU step) leaves most threads without
  // examples: the block then walks several leaves at once, `tb` threads (whole warps) per leaf.
  constexpr uint32_t U = LBT / (4 * LTH);
  uint32_t tb = LTH;
  if (nb <= 2 * LTH) { tb = 32; while (4 * tb < nb) tb <<= 1; }
  const uint32_t te = threadIdx.x % tb, leaf_lane = threadIdx.x / tb, leaf_lanes = LTH / tb;
  uint16_t xv[U][4];
#pragma unroll
  for (uint32_t u = 0; u < U; ++u) {
    const uint32_t b = 4 * te + 4 * LTH * u;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) xv[u][j] = b + j < nb ? xs[b + j] : (uint16_t)0xffff;
  }
  for (uint32_t li = lchunk_off[chunk] + leaf_lane; li < lchunk_off[chunk + 1]; li += leaf_lanes) {
    uint32_t i = lchunk_inputs[li];
    const float* tab = theta + in_poff[i];
    float* out = mars + (size_t)in_node[i] * ld + b0;
    float v[U][4];
#pragma unroll
    for (uint32_t u = 0; u < U; ++u)
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) v[u][j] = xv[u][j] == 0xffff ? 0.0f : __ldg(tab + xv[u][j]);
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t b = 4 * te + 4 * LTH * u;
      if (b < nb) *reinterpret_cast<float4*>(out + b) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
    }
  }
}

// Leaf statistics through a shared-memory histogram per leaf; a block that covers the whole
// batch owns its leaves' slots and adds without atomics.
__global__ void __launch_bounds__(LTH) leaf_flow_chunk_kernel(
    const float* __restrict__ flows, uint32_t ld, uint32_t B, float* __restrict__ aggr, uint32_t hstride,
    const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_cats,
    const uint64_t* __restrict__ in_foff, const uint32_t* __restrict__ lchunk_var,
    const uint32_t* __restrict__ lchunk_off, const uint32_t* __restrict__ lchunk_inputs,
    const uint8_t* __restrict__ data, const uint8_t* __restrict__ miss, uint64_t num_rows,
    const int32_t* __restrict__ row_ids, uint32_t row_start, const float* __restrict__ weights) {
  extern __shared__ float hist[];  // [PCB_LEAF_CHUNK][hstride]
  __shared__ uint16_t xs[LBT];
  const uint32_t chunk = blockIdx.x, b0 = blockIdx.y * LBT;
  const uint32_t nb = min((uint32_t)LBT, B - b0);
  const uint32_t l0 = lchunk_off[chunk], nl = lchunk_off[chunk + 1] - l0;
  for (uint32_t x = threadIdx.x; x < nl * hstride; x += LTH) hist[x] = 0.0f;
  stage_values(xs, b0, nb, lchunk_var[chunk], data, miss, num_rows, row_ids, row_start);
  __syncthreads();
  // a thread's examples (and their values and weights) are the same for every leaf of the chunk;
  // per leaf all of the thread's flow loads are issued before the first histogram update
  constexpr uint32_t U = LBT / LTH;
  uint16_t xv[U];
  float wv[U];
#pragma unroll
  for (uint32_t u = 0; u < U; ++u) {
    const uint32_t b = threadIdx.x + LTH * u;
    xv[u] = b < nb ? xs[b] : (uint16_t)0xfffe;   // 0xfffe: no example
    wv[u] = (weights && b < nb) ? weights[data_row(row_ids, row_start, b0 + b)] : 1.0f;
  }
  for (uint32_t l = 0; l < nl; ++l) {
    uint32_t i = lchunk_inputs[l0 + l];
    if (in_foff[i] == ~0ull) continue;  // fixed leaf
    const uint32_t C = in_cats[i];
    const float* f = flows + (size_t)in_node[i] * ld + b0;
    float* h = hist + l * hstride;
    float v[U];
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t b = threadIdx.x + LTH * u;
      v[u] = f[b < nb ? b : 0u];
    }
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t slot = xv[u] == 0xffff ? C : (uint32_t)xv[u];   // missing value -> the extra slot
      if (xv[u] != 0xfffe && slot <= C) atomicAdd(h + slot, v[u] * wv[u]);
    }
  }
  __syncthreads();
  const bool whole = gridDim.y == 1;
  for (uint32_t x = threadIdx.x; x < nl * hstride; x += LTH) {
    uint32_t l = x / hstride, sl = x - l * hstride;
    uint32_t i = lchunk_inputs[l0 + l];
    uint64_t fo = in_foff[i];
    if (fo == ~0ull || sl > in_cats[i]) continue;
    float v = hist[x];
    if (v == 0.0f) continue;
    if (whole) aggr[fo + sl] += v; else atomicAdd(aggr + fo + sl, v);
  }
}

// Leaf statistics by sorted examples: the examples of the block's slice are sorted by the
// variable's value once (counting sort in shared memory), and every thread keeps up to LSE consecutive
// positions of the sorted order in registers for the whole group: the example behind each position,
// its value segment and (if given) its weight.  Then every leaf row of the group streams through a
// three-deep ring of shared-memory buffers (one bulk copy per row); a thread gathers its LSE values
// (independent loads, the same work for every thread whatever the histogram of the values looks
// like), sums runs of equal segment in registers and adds one partial sum per run to the row's
// shared-memory histogram; after the barrier the histogram leaves with one RED per slot while the
// next row is already being gathered into the other histogram.  A missing value sorts into the
// extra segment C.  The group's leaves share one variable, so one sort serves up to 64 rows.
constexpr int LSB = 2048;   // examples per block slice
constexpr int LST = 256;    // threads
constexpr int LSE = LSB / LST;   // sorted positions per thread
constexpr int LSR = 4;      // row buffers; the last one holds the sort's arrays until the sort is done
constexpr int LSC = 508;    // most categories of a variable (static + dynamic shared memory stay under 48 KB)
template <bool WEIGHTED>
__global__ void __launch_bounds__(LST) leaf_flow_sorted_kernel(
    const float* __restrict__ flows, uint32_t ld, uint32_t B, float* __restrict__ aggr,
    const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_foff,
    const uint32_t* __restrict__ lgrp_var, const uint32_t* __restrict__ lgrp_off,
    const uint32_t* __restrict__ linputs, uint32_t max_cats, const uint8_t* __restrict__ data,
    const uint8_t* __restrict__ miss, uint64_t num_rows, const int32_t* __restrict__ row_ids, uint32_t row_start,
    const float* __restrict__ weights, int* __restrict__ status) {
  __shared__ __align__(128) float rowbuf[LSR][LSB];
  __shared__ uint32_t binoff[LSC + 4];   // segment starts and the end; afterwards histogram 0
  __shared__ uint32_t cursor[LSC + 4];   // scatter cursors; afterwards histogram 1
  __shared__ uint64_t s_fo[PCB_LEAF_GROUP];   // the group's leaves: first statistics slot, categories
  __shared__ uint32_t s_cats[PCB_LEAF_GROUP];
  __shared__ __align__(8) uint64_t bar[LSR];
  static_assert(sizeof(float) * LSB == 2 * sizeof(uint16_t) * LSB, "the sort's two arrays fill one row buffer");
  uint16_t* xs = reinterpret_cast<uint16_t*>(rowbuf[LSR - 1]);   // values of the examples
  uint16_t* perm = xs + LSB;                                      // examples in sorted order
  const uint32_t grp = blockIdx.x, b0 = blockIdx.y * LSB, tid = threadIdx.x;
  const uint32_t nb = min((uint32_t)LSB, B - b0);
  const uint32_t l0 = lgrp_off[grp], nl = lgrp_off[grp + 1] - l0;
  // segments: values 0 .. max_cats (a value equal to a leaf's category count lands in that leaf's
  // extra slot, larger ones are dropped, as in the atomic kernel), then the missing-value segment
  const uint32_t miss_bin = max_cats + 1, nbins = max_cats + 2;
  if (tid == 0) {
    for (int r = 0; r < LSR; ++r) pcbtc::mbar_init(&bar[r], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (uint32_t x = tid; x <= nbins; x += LST) { binoff[x] = 0; }
  if (tid < nl) {
    const uint32_t i = linputs[l0 + tid];
    s_fo[tid] = in_foff[i];
    s_cats[tid] = in_cats[i];
  }
  stage_values(xs, b0, nb, lgrp_var[grp], data, miss, num_rows, row_ids, row_start);
  __syncthreads();
  // rows are requested as early as possible: the sort below hides their latency
  const uint32_t rowbytes = ((nb + 3u) & ~3u) * 4u;   // the pitch is a multiple of 32 floats: stays inside the row
  auto request = [&](uint32_t l) {
    const uint32_t i = linputs[l0 + l];
    pcbtc::mbar_arrive_expect_tx(&bar[l % LSR], rowbytes);
    pcbtc::bulk_g2s(rowbuf[l % LSR], flows + (size_t)in_node[i] * ld + b0, rowbytes, &bar[l % LSR]);
  };
  if (tid == 0) for (uint32_t l = 0; l < min(nl, (uint32_t)LSR - 1u); ++l) request(l);
  // counting sort of the examples by value
  for (uint32_t b = tid; b < nb; b += LST) {
    const uint32_t x = xs[b] == 0xffff ? miss_bin : (uint32_t)xs[b];
    if (x <= miss_bin) atomicAdd(&binoff[x + 1], 1u);
  }
  __syncthreads();
  if (tid < 32) {   // inclusive scan of the counts, one warp
    uint32_t carry = 0;
    for (uint32_t base = 0; base <= nbins; base += 32) {
      const uint32_t idx = base + tid;
      uint32_t v = idx <= nbins ? binoff[idx] : 0u;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, v, d);
        if ((int)tid >= d) v += u;
      }
      v += carry;
      if (idx <= nbins) binoff[idx] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  for (uint32_t x = tid; x < nbins; x += LST) cursor[x] = binoff[x];
  __syncthreads();
  for (uint32_t b = tid; b < nb; b += LST) {
    const uint32_t x = xs[b] == 0xffff ? miss_bin : (uint32_t)xs[b];
    if (x <= miss_bin) perm[atomicAdd(&cursor[x], 1u)] = (uint16_t)b;
  }
  __syncthreads();
  // this thread's sorted positions LSE * tid .. + LSE - 1: example, segment, weight
  constexpr uint32_t NOSEG = 0xffffffffu;
  uint32_t pos[LSE], seg[LSE];
  float wv[LSE];
  {
    // the sorted examples are dealt out evenly: a slice of fewer than 2048 examples still keeps every
    // thread busy, with fewer positions each
    const uint32_t total = binoff[nbins], per = (total + LST - 1u) / LST, j0 = per * tid;
    // segment of position j0: the last x with binoff[x] <= j0
    uint32_t lo = 0, hi = nbins;   // invariant: binoff[lo] <= j0 (binoff[0] = 0), answer in [lo, hi)
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (binoff[mid] <= j0) lo = mid; else hi = mid;
    }
    uint32_t x = lo;
#pragma unroll
    for (uint32_t e = 0; e < (uint32_t)LSE; ++e) {
      const uint32_t j = j0 + e;
      const bool in = e < per && j < total;
      while (in && binoff[x + 1] <= j) ++x;   // empty segments are stepped over
      pos[e] = in ? (uint32_t)perm[j] : 0u;
      seg[e] = in ? x : NOSEG;
      wv[e] = (WEIGHTED && in) ? weights[data_row(row_ids, row_start, b0 + pos[e])] : 1.0f;
    }
  }
  __syncthreads();   // binoff, cursor and the sort's arrays have been read by everyone
  if (tid == 0 && nl >= (uint32_t)LSR) {   // the last row buffer is free now
    pcbtc::fence_proxy_async();
    request(LSR - 1);
  }
  float* hist0 = reinterpret_cast<float*>(binoff);
  float* hist1 = reinterpret_cast<float*>(cursor);
  for (uint32_t x = tid; x < nbins; x += LST) { hist0[x] = 0.0f; hist1[x] = 0.0f; }
  __syncthreads();
  bool ok = true;
  for (uint32_t l = 0; l < nl; ++l) {
    const uint64_t fo = s_fo[l];
    const uint32_t C = s_cats[l];
    ok = ok && pcbtc::mbar_wait(&bar[l % LSR], (l / LSR) & 1u, status);
    const float* row = rowbuf[l % LSR];
    float* h = (l & 1u) ? hist1 : hist0;
    const bool live = ok && fo != ~0ull;
    if (live) {
      float v[LSE];
#pragma unroll
      for (uint32_t e = 0; e < (uint32_t)LSE; ++e) v[e] = row[pos[e]];
      float acc = 0.0f;
#pragma unroll
      for (uint32_t e = 0; e < (uint32_t)LSE; ++e) {
        if (e > 0 && seg[e] != seg[e - 1]) {   // positions past the end come last and carry NOSEG
          atomicAdd(h + seg[e - 1], acc);
          acc = 0.0f;
        }
        acc += WEIGHTED ? v[e] * wv[e] : v[e];
      }
      if (seg[LSE - 1] != NOSEG) atomicAdd(h + seg[LSE - 1], acc);
    }
    __syncthreads();   // the row has been read and its histogram is complete
    if (tid == 0 && ok && l + LSR < nl) {
      pcbtc::fence_proxy_async();
      request(l + LSR);
    }
    if (live) {
      // one fire-and-forget RED per slot; the histogram is cleared for the row after the next
      for (uint32_t x = tid; x < nbins; x += LST) {
        const float a = h[x];
        if (a == 0.0f) continue;
        h[x] = 0.0f;
        // leaf slot: value x <= C -> x, missing -> C; values beyond the leaf's categories are dropped
        const uint32_t slot = x == miss_bin ? C : x;
        if (slot <= C) atomicAdd(aggr + fo + slot, a);
      }
    }
  }
  if (!ok && tid == 0) {   // a wait was lost: let the copies in flight land before the block ends
    for (int r = 0; r < LSR; ++r) pcbtc::mbar_wait(&bar[r], 0, status);
  }
}

// ---- leaves under soft evidence / soft regularisation ----------------------------------------------
// One block per leaf, threads over the examples.  soft != null: per-category log-weights
// soft[row, var, c] ([rows, V, C] column-major) stand where the observed category stands
// (init_mar!_with_reg_cat_kernel, regularization/reg_likelihood.jl:51-91); else hard evidence with
// soft_reg > 0 (soft_loglikelihood, reg_likelihood.jl:4-14).
__global__ void leaf_forward_gen_kernel(float* __restrict__ mars, uint32_t ld, uint32_t B, const float* __restrict__ theta,
                                        const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_var,
                                        const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                        uint32_t num_vars, const uint8_t* __restrict__ data, const uint8_t* __restrict__ miss,
                                        const float* __restrict__ soft, uint64_t num_rows,
                                        const int32_t* __restrict__ row_ids, uint32_t row_start, float soft_reg, int32_t width) {
  const uint32_t i = blockIdx.x, b = blockIdx.y * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int64_t row = data_row(row_ids, row_start, b);
  const uint32_t C = in_cats[i], var = in_var[i];
  const float* tab = theta + in_poff[i];
  float v;
  if (soft) {
    const float* sp = soft + (size_t)row + (size_t)num_rows * var;
    const size_t cs = (size_t)num_rows * num_vars;
    float mx = -INFINITY;
    for (uint32_t c = 0; c < C; ++c) mx = fmaxf(mx, sp[c * cs] + __ldg(tab + c));
    float acc = 0.0f;
    for (uint32_t c = 0; c < C; ++c) acc += expf(sp[c * cs] + __ldg(tab + c) - mx);
    v = mx == -INFINITY ? -INFINITY : mx + logf(acc);
  } else {
    const size_t di = (size_t)row + (size_t)num_rows * var;
    if (miss && miss[di]) {
      v = 0.0f;
    } else {
      const int32_t x = data[di];
      const int32_t c_start = max(0, x - width / 2), c_end = min(c_start + width - 1, (int32_t)C - 1);
      float sp = 0.0f;
      for (int32_t c = c_start; c <= c_end; ++c) sp += expf(__ldg(tab + c));
      sp /= (float)(c_end - c_start + 1);
      const float u = __ldg(tab + x) + logf(1.0f - soft_reg), w = logf(sp) + logf(soft_reg);
      const float m = fmaxf(u, w);
      v = (isfinite(u) && isfinite(w)) ? m + log1pf(expf(-fabsf(u - w))) : m;
    }
  }
  mars[(size_t)in_node[i] * ld + b] = v;
}

// Leaf statistics of the same two forms (input_flows_circuit_with_reg_cat_kernel reg_flow.jl:50-82;
// soft_flow reg_flow.jl:3-22, which uses the stored LOG-probabilities where it says heap[...]: kept
// as written).  A warp reduces its 32 examples per category before touching memory.
__global__ void leaf_flow_gen_kernel(const float* __restrict__ flows, const float* __restrict__ mars, uint32_t ld, uint32_t B,
                                     float* __restrict__ aggr, const float* __restrict__ theta,
                                     const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_var,
                                     const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                     const uint64_t* __restrict__ in_foff, uint32_t num_vars,
                                     const uint8_t* __restrict__ data, const uint8_t* __restrict__ miss,
                                     const float* __restrict__ soft, uint64_t num_rows, const int32_t* __restrict__ row_ids,
                                     uint32_t row_start, const float* __restrict__ weights, float soft_reg, int32_t width) {
  const uint32_t i = blockIdx.x, b = blockIdx.y * blockDim.x + threadIdx.x, lane = threadIdx.x & 31;
  const uint64_t fo = in_foff[i];
  if (fo == ~0ull) return;   // fixed leaf
  const bool active = b < B;
  const int64_t row = active ? data_row(row_ids, row_start, b) : 0;
  const uint32_t C = in_cats[i], var = in_var[i];
  const float* tab = theta + in_poff[i];
  float f = active ? flows[(size_t)in_node[i] * ld + b] : 0.0f;
  if (active && weights) f *= weights[row];
  if (soft) {
    const float logp = active ? mars[(size_t)in_node[i] * ld + b] : 0.0f;
    const float* sp = soft + (size_t)row + (size_t)num_rows * var;
    const size_t cs = (size_t)num_rows * num_vars;
    for (uint32_t c = 0; c < C; ++c) {
      float v = active ? expf(sp[c * cs] + __ldg(tab + c) - logp) * f : 0.0f;
      v = warp_sum(v);
      if (lane == 0 && v != 0.0f) atomicAdd(aggr + fo + c, v);
    }
    return;
  }
  if (!active) return;
  const size_t di = (size_t)row + (size_t)num_rows * var;
  if (miss && miss[di]) { atomicAdd(aggr + fo + C, f); return; }
  const int32_t x = data[di];
  const int32_t c_start = max(0, x - width / 2), c_end = min(c_start + width - 1, (int32_t)C - 1);
  float sp = 0.0f;
  for (int32_t c = c_start; c <= c_end; ++c) sp += expf(__ldg(tab + c));
  sp /= (float)(c_end - c_start + 1);
  const float base = (1.0f - soft_reg) * __ldg(tab + x) + soft_reg * sp;
  atomicAdd(aggr + fo + x, (1.0f - soft_reg) * __ldg(tab + x) * f / base);
  for (int32_t c = c_start; c <= c_end; ++c)
    atomicAdd(aggr + fo + c, soft_reg / (float)(c_end - c_start + 1) * __ldg(tab + c) * f / base);
}

// Log-likelihoods of a multi-head circuit (extract_lls_from_root_nodes,
// src-jl/multi_head_pc/bit_circuit.jl:95-109): with a mask out[b] = logsumexp_h(mars[root_h][b] +
// log mask[row, h]) - log sum_h mask[row, h]; without one out is [B, H] with the roots' values.
__global__ void head_ll_kernel(const float* __restrict__ mars, uint32_t ld, uint32_t B, const uint32_t* __restrict__ roots,
                               uint32_t H, const float* __restrict__ head_mask, uint64_t mask_rows,
                               const int32_t* __restrict__ row_ids, uint32_t row_start, float* __restrict__ out) {
  const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (!head_mask) {
    for (uint32_t h = 0; h < H; ++h) out[(size_t)h * B + b] = mars[(size_t)roots[h] * ld + b];
    return;
  }
  const int64_t row = data_row(row_ids, row_start, b);
  float mx = -INFINITY, tot = 0.0f;
  for (uint32_t h = 0; h < H; ++h) {
    const float m = head_mask[(size_t)row + mask_rows * h];
    mx = fmaxf(mx, mars[(size_t)roots[h] * ld + b] + logf(m));
    tot += m;
  }
  float acc = 0.0f;
  for (uint32_t h = 0; h < H; ++h) {
    const float m = head_mask[(size_t)row + mask_rows * h];
    const float v = mars[(size_t)roots[h] * ld + b] + logf(m);
    if (v != -INFINITY) acc += expf(v - mx);
  }
  out[b] = (mx == -INFINITY ? -INFINITY : mx + logf(acc)) - logf(tot);
}

__global__ void scale_kernel(float* __restrict__ x, uint64_t n, float rate) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = rate == 0.0f ? 0.0f : x[i] * rate;
}

// One warp per sum node: pseudocount, node normaliser, inertia blend, all in one pass.
__global__ void em_update_sum_kernel(float* __restrict__ theta, float* __restrict__ aggr,
                                     const uint32_t* __restrict__ grp_node, uint32_t n_groups,
                                     const uint32_t* __restrict__ n_pid0, const uint32_t* __restrict__ n_ecount,
                                     float pseudocount, float inertia) {
  uint32_t g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint32_t lane = threadIdx.x & 31;
  if (g >= n_groups) return;
  uint32_t n = grp_node[g];
  uint32_t p0 = n_pid0[n], cnt = n_ecount[n];
  float pc = pseudocount / (float)cnt;
  float tot = 0.0f;
  if ((cnt & 3u) == 0 && (p0 & 3u) == 0 && cnt <= 1024 && cnt > 1) {
    // aligned group of up to 1024 edges (every dense block): 16-byte accesses, statistics and
    // parameters loaded together and kept in registers between the two passes
    float4 a[8], th[8];
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t j = 4u * lane + 128u * u;
      if (j < cnt) {
        a[u] = *reinterpret_cast<const float4*>(aggr + p0 + j);
        th[u] = *reinterpret_cast<const float4*>(theta + p0 + j);
      }
    }
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t j = 4u * lane + 128u * u;
      if (j < cnt) {
        a[u].x += pc; a[u].y += pc; a[u].z += pc; a[u].w += pc;
        *reinterpret_cast<float4*>(aggr + p0 + j) = a[u];   // the reference keeps the pseudocount in edge_aggr
        tot += (a[u].x + a[u].y) + (a[u].z + a[u].w);
      }
    }
    tot = warp_sum(tot);
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t j = 4u * lane + 128u * u;
      if (j < cnt) {
        float4 o;
        o.x = logf(inertia * expf(th[u].x) + (1.0f - inertia) * a[u].x / tot);
        o.y = logf(inertia * expf(th[u].y) + (1.0f - inertia) * a[u].y / tot);
        o.z = logf(inertia * expf(th[u].z) + (1.0f - inertia) * a[u].z / tot);
        o.w = logf(inertia * expf(th[u].w) + (1.0f - inertia) * a[u].w / tot);
        *reinterpret_cast<float4*>(theta + p0 + j) = o;
      }
    }
    return;
  }
  for (uint32_t j = lane; j < cnt; j += 32) {
    float a = aggr[p0 + j] + pc;
    aggr[p0 + j] = a;  // the reference keeps the pseudocount in edge_aggr
    tot += a;
  }
  tot = warp_sum(tot);
  if (cnt == 1) return;  // single-edge sum nodes keep their parameter (reg_em.jl:150)
  for (uint32_t j = lane; j < cnt; j += 32) {
    float oldv = inertia * expf(theta[p0 + j]);
    float newv = (1.0f - inertia) * aggr[p0 + j] / tot;
    theta[p0 + j] = logf(oldv + newv);
  }
}

// One warp per learnable leaf (fixable_categorical_dist.jl:223-248).
__global__ void em_update_leaf_kernel(float* __restrict__ theta, const float* __restrict__ aggr,
                                      uint32_t n_inputs, const uint32_t* __restrict__ in_cats,
                                      const uint64_t* __restrict__ in_poff, const uint64_t* __restrict__ in_foff,
                                      float pseudocount, float inertia) {
  uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint32_t lane = threadIdx.x & 31;
  if (i >= n_inputs) return;
  uint64_t fo = in_foff[i];
  if (fo == ~0ull) return;
  uint32_t C = in_cats[i];
  uint64_t po = in_poff[i];
  if (C <= 256) {
    // statistics and parameters of the leaf loaded together and kept in registers between the passes
    float a[8], th[8];
    float s = 0.0f;
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t k = lane + 32u * u;
      if (k < C) { a[u] = aggr[fo + k]; th[u] = theta[po + k]; }
    }
    const float missing_flow = aggr[fo + C];
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) if (lane + 32u * u < C) s += a[u];
    s = warp_sum(s);
    const float node_flow = s + (missing_flow + pseudocount);
    const float cat_pc = pseudocount / (float)C;
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t k = lane + 32u * u;
      if (k < C) {
        const float oldp = expf(th[u]);
        const float newv = (1.0f - inertia) * (a[u] + cat_pc + missing_flow * oldp) / node_flow;
        theta[po + k] = logf(inertia * oldp + newv);
      }
    }
    return;
  }
  float s = 0.0f;
  for (uint32_t k = lane; k < C; k += 32) s += aggr[fo + k];
  s = warp_sum(s);
  float missing_flow = aggr[fo + C];
  float node_flow = s + (missing_flow + pseudocount);
  float cat_pc = pseudocount / (float)C;
  for (uint32_t k = lane; k < C; k += 32) {
    float oldp = expf(theta[po + k]);
    float oldv = inertia * oldp;
    float newv = (1.0f - inertia) * (aggr[fo + k] + cat_pc + missing_flow * oldp) / node_flow;
    theta[po + k] = logf(oldv + newv);
  }
}

__global__ void iota_ids_kernel(int32_t* __restrict__ ids, int32_t first, uint32_t n) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ids[i] = first + (int32_t)i;
}

__global__ void ll_sum_kernel(const float* __restrict__ root_mars, uint32_t B, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.0f;
  for (uint32_t b = threadIdx.x; b < B; b += blockDim.x) s += root_mars[b];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) *out = v;
  }
}

dim3 grid2(uint32_t items, uint32_t B) { return dim3(items, (B + TPB - 1) / TPB, 1); }
// grid of the kernels that take four examples per thread
dim3 grid2v(uint32_t items, uint32_t B) { return dim3(items, (B + 4 * TPB - 1) / (4 * TPB), 1); }

}  // namespace

#define PCB_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != PCB_OK) return _s;   \
  } while (0)

// ---- checked mode (PCB_CHECKED=1) ------------------------------------------------------------------
// The circuit's own index arrays are validated on the host when it is compiled; what arrives on the
// device at run time and is used as an index is the batch: row ids and observed categories.  The
// reference reads both under @inbounds.  In checked mode every pass first runs this kernel, which
// touches only what it has found in range, waits for it and refuses the pass with the first finding
// (no kernel of the pass is launched on a bad index).  word: [code, example, variable, value],
// code 1 = row id outside [1, num_rows], 2 = category not below the variable's category count.
__global__ void check_batch_kernel(const int32_t* __restrict__ row_ids, uint32_t row_start, uint32_t B, uint64_t num_rows,
                                   const uint8_t* __restrict__ data, const uint8_t* __restrict__ miss, uint32_t V,
                                   const uint32_t* __restrict__ var_cats, int32_t* __restrict__ word) {
  const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int64_t row = row_ids ? (int64_t)row_ids[b] - 1 : (int64_t)row_start - 1 + b;
  if (row < 0 || (uint64_t)row >= num_rows) {
    if (atomicCAS(word, 0, 1) == 0) { word[1] = (int32_t)b; word[2] = 0; word[3] = (int32_t)(row + 1); }
    return;
  }
  if (!data) return;
  for (uint32_t v = blockIdx.y; v < V; v += gridDim.y) {
    const size_t di = (size_t)row + (size_t)num_rows * v;
    if (miss && miss[di]) continue;
    const uint32_t x = data[di];
    if (x >= var_cats[v] && atomicCAS(word, 0, 2) == 0) { word[1] = (int32_t)b; word[2] = (int32_t)v; word[3] = (int32_t)x; }
  }
}

int32_t pcb_check_batch(pcb_circuit* c, const pcb_evidence& ev, cudaStream_t st) {
  PCB_CUDA(cudaMemsetAsync(c->check_word, 0, 4 * sizeof(int32_t), st));
  dim3 grid((ev.B + 127) / 128, std::min<uint32_t>(std::max<uint32_t>(c->V, 1u), 64u));
  check_batch_kernel<<<grid, 128, 0, st>>>(ev.row_ids_dev, ev.row_start, ev.B, ev.num_rows, ev.data_dev, ev.miss_dev, c->V,
                                           c->var_cats, c->check_word);
  int32_t w[4] = {0, 0, 0, 0};
  PCB_CUDA(cudaMemcpyAsync(w, c->check_word, sizeof(w), cudaMemcpyDeviceToHost, st));
  PCB_CUDA(cudaStreamSynchronize(st));
  if (w[0] == 1)
    return pcb_fail(PCB_ERR_INVALID, "checked mode: example " + std::to_string(w[1]) + " of the batch names row " +
                                         std::to_string(w[3]) + ", outside 1 .. " + std::to_string(ev.num_rows));
  if (w[0] == 2)
    return pcb_fail(PCB_ERR_INVALID, "checked mode: example " + std::to_string(w[1]) + " of the batch has value " +
                                         std::to_string(w[3]) + " for variable " + std::to_string(w[2] + 1) +
                                         ", which has fewer categories");
  return PCB_OK;
}

static int32_t forward_impl(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence& ev, float* ll_out_dev,
                            cudaStream_t st) {
  const uint32_t B = ev.B;
  PCB_REQUIRE(ev.data_dev || ev.soft_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(B >= 1 && B <= ws->max_batch, "batch size exceeds the workspace");
  PCB_REQUIRE(ev.row_ids_dev || (ev.row_start >= 1 && (uint64_t)ev.row_start - 1 + B <= ev.num_rows),
              "row range out of bounds");
  PCB_REQUIRE(ev.soft_reg >= 0.0f && ev.soft_reg < 1.0f, "soft_reg must lie in [0, 1)");
  PCB_REQUIRE(ev.soft_reg == 0.0f || ev.soft_dev || ev.soft_reg_width >= 1, "soft_reg_width must be at least 1");
  PCB_REQUIRE(!ev.head_mask_dev || c->n_heads, "a head mask needs a multi-head circuit");
  PCB_CUDA(cudaSetDevice(c->device));
  if (c->checked) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cap);
    if (cap == cudaStreamCaptureStatusNone) PCB_TRY(pcb_check_batch(c, ev, st));
  }
  ws->B = B; ws->data = ev.data_dev; ws->miss = ev.miss_dev; ws->num_rows = ev.num_rows;
  ws->row_ids = ev.row_ids_dev; ws->row_start = ev.row_start; ws->have_forward = false;
  ws->soft = ev.soft_dev; ws->head_mask = ev.head_mask_dev;
  ws->soft_reg = ev.soft_dev ? 0.0f : ev.soft_reg; ws->soft_width = ev.soft_reg_width;
  if (c->use_tc) PCB_TRY(pcb_dense_tc_refresh(c, st));
  // the arrival counters of the K-split dense tiles return to zero by themselves; a pass that a lost
  // wait cut short must not leave a stale count to the next one
  if (ws->mn_tickets) PCB_CUDA(cudaMemsetAsync(ws->mn_tickets, 0, 296 * sizeof(uint32_t), st));
  if (c->n_inputs) {
    PcbProfScope ps(c, st, PCB_K_LEAF_FWD);
    if (ws->soft || ws->soft_reg > 0.0f) {
      leaf_forward_gen_kernel<<<grid2(c->n_inputs, B), TPB, 0, st>>>(
          ws->mars, ws->ld, B, c->theta, c->in_node, c->in_var, c->in_cats, c->in_poff, c->V, ev.data_dev, ev.miss_dev,
          ws->soft, ev.num_rows, ev.row_ids_dev, ev.row_start, ws->soft_reg, (int32_t)ws->soft_width);
    } else {
      dim3 grid(c->n_lgrps, (B + LBT - 1) / LBT);   // groups of up to 64 leaves of one variable share the staged values
      leaf_forward_chunk_kernel<<<grid, LTH, 0, st>>>(ws->mars, ws->ld, B, c->theta, c->in_node, c->in_poff,
                                                      c->lgrp_var, c->lgrp_off, c->lchunk_inputs, ev.data_dev,
                                                      ev.miss_dev, ev.num_rows, ev.row_ids_dev, ev.row_start);
    }
  }
  const bool fwd_split = c->fwd_split;
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    uint32_t o0 = c->h_up_sparse_off[lay - 1], o1 = c->h_up_sparse_off[lay];
    // The sparse nodes and the dense blocks of one layer do not depend on each other (both read
    // lower layers only): with a side stream the two kernels of a layer run side by side.
    const bool has_dense = c->h_dense_off[lay + 1] > c->h_dense_off[lay];
    const bool split = c->side && !c->prof.on && fwd_split && o1 > o0 && has_dense;
    cudaStream_t ss = st;
    if (split) {
      PCB_CUDA(cudaEventRecord(c->ev_fork, st));
      PCB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
      ss = c->side;
    }
    if (o1 > o0)
      { PcbProfScope ps(c, ss, PCB_K_SPARSE_UP); pcb_launch_pdl(sparse_up_kernel, grid2v(o1 - o0, B), dim3(TPB), 0, ss, c->pdl && !split, ws->mars, ws->ld, B, c->up_sparse + o0, c->kind,
                                                          c->n_estart, c->n_ecount, c->n_pid0, c->e_prime,
                                                          c->e_sub, c->theta); }
    PCB_TRY(pcb_dense_forward(c, ws, lay, st));
    if (split) {
      PCB_CUDA(cudaEventRecord(c->ev_join, c->side));
      PCB_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
    }
  }
  if (ll_out_dev) {
    if (c->n_heads) {
      PcbProfScope ps(c, st, PCB_K_MISC);
      head_ll_kernel<<<(B + 255) / 256, 256, 0, st>>>(ws->mars, ws->ld, B, c->head_roots, c->n_heads, ws->head_mask,
                                                      ev.num_rows, ev.row_ids_dev, ev.row_start, ll_out_dev);
    } else {
      PCB_CUDA(cudaMemcpyAsync(ll_out_dev, ws->mars + (size_t)(c->N - 1) * ws->ld, B * sizeof(float),
                               cudaMemcpyDeviceToDevice, st));
    }
  }
  PCB_CUDA(cudaGetLastError());
  ws->have_forward = true;
  return PCB_OK;
}

static pcb_evidence hard_evidence(const uint8_t* data_dev, const uint8_t* miss_dev, uint64_t num_rows,
                                  const int32_t* row_ids_dev, uint32_t row_start, uint32_t B) {
  pcb_evidence ev;
  memset(&ev, 0, sizeof(ev));
  ev.data_dev = data_dev; ev.miss_dev = miss_dev; ev.num_rows = num_rows; ev.row_ids_dev = row_ids_dev;
  ev.row_start = row_start; ev.B = B; ev.soft_reg_width = 1;
  return ev;
}

extern "C" int32_t pcb_forward(pcb_circuit* c, pcb_workspace* ws, const uint8_t* data_dev,
                               const uint8_t* miss_dev, uint64_t num_rows, const int32_t* row_ids_dev,
                               uint32_t row_start, uint32_t B, float* ll_out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && data_dev, "null argument");
  return forward_impl(c, ws, hard_evidence(data_dev, miss_dev, num_rows, row_ids_dev, row_start, B), ll_out_dev,
                      (cudaStream_t)s);
}

extern "C" int32_t pcb_forward_ex(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, float* ll_out_dev,
                                  pcb_stream s) {
  PCB_REQUIRE(c && ws && ev, "null argument");
  return forward_impl(c, ws, *ev, ll_out_dev, (cudaStream_t)s);
}

// Multi-GPU step: once every edge statistic of the batch is final (the sparse nodes' in stream order,
// the dense blocks' on the side stream) their slice of the statistics vector is summed over the ranks
// on the communication stream, while this stream goes on to the leaf statistics.
static int32_t comm_edges_begin(pcb_circuit* c, cudaStream_t st) {
  PCB_CUDA(cudaEventRecord(c->ev_c0, st));
  PCB_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_c0, 0));
  if (c->side && c->side_busy) {
    PCB_CUDA(cudaEventRecord(c->ev_c1, c->side));
    PCB_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_c1, 0));
  }
  PcbProfScope ps(c, c->comm_stream, PCB_K_ALLREDUCE);
  return pcb_allreduce_range(c, 0, c->n_inner, c->comm_stream);
}
// ... and the rest (leaf slots, batch log-likelihood) after them; the caller's stream waits for both.
static int32_t comm_rest_and_join(pcb_circuit* c, cudaStream_t st) {
  PCB_CUDA(cudaEventRecord(c->ev_c2, st));
  PCB_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_c2, 0));
  { PcbProfScope ps(c, c->comm_stream, PCB_K_ALLREDUCE);
    PCB_TRY(pcb_allreduce_range(c, c->n_inner, c->aggr_len - c->n_inner, c->comm_stream)); }
  PCB_CUDA(cudaEventRecord(c->ev_c3, c->comm_stream));
  PCB_CUDA(cudaStreamWaitEvent(st, c->ev_c3, 0));
  return PCB_OK;
}

// early: a single-GPU step updates the sum parameters (and refreshes the weight images) on the side
// stream as soon as the last edge statistics are in, beside the leaf statistics of this stream.
struct EarlyUpdate { float pseudocount, inertia; bool done; };
static int32_t em_update_sums(pcb_circuit* c, float pseudocount, float inertia, cudaStream_t st);
static int32_t backward_impl(pcb_circuit* c, pcb_workspace* ws, const float* weights_dev, cudaStream_t st, bool split_comm,
                             EarlyUpdate* early = nullptr);

extern "C" int32_t pcb_backward(pcb_circuit* c, pcb_workspace* ws, const float* weights_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws, "null argument");
  return backward_impl(c, ws, weights_dev, (cudaStream_t)s, false);
}

static int32_t backward_impl(pcb_circuit* c, pcb_workspace* ws, const float* weights_dev, cudaStream_t st, bool split_comm,
                             EarlyUpdate* early) {
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  if (!ws->have_forward) return pcb_fail(PCB_ERR_STATE, "pcb_backward needs a preceding pcb_forward on this workspace");
  PCB_CUDA(cudaSetDevice(c->device));
  const uint32_t B = ws->B;
  PCB_REQUIRE(!c->n_heads || ws->head_mask, "the flows of a multi-head circuit need a head mask");
  const HeadInit hi{c->n_head, ws->head_mask, ws->num_rows, ws->row_ids, ws->row_start};
  c->edge_lo = c->edge_hi = 0;
  auto sparse_down = [&](int64_t lay, cudaStream_t ss, bool pdl) -> int32_t {
    uint32_t o0 = c->h_down_sparse_off[lay], o1 = c->h_down_sparse_off[lay + 1];
    if (o1 > o0) {
      PcbProfScope ps(c, ss, PCB_K_SPARSE_DOWN);
      PCB_CUDA(pcb_launch_pdl(sparse_down_kernel, grid2v(o1 - o0, B), dim3(TPB), 0, ss, pdl, ws->flows, ws->mars, ws->ld,
                              B, c->down_sparse + o0, c->N - 1, c->in_off, c->in_ent, c->theta, c->skip_stats ? nullptr : c->aggr, hi));
    }
    return PCB_OK;
  };
  // Layer l: its sparse nodes pull their flows, then its dense blocks push flows to their children.
  // The sparse nodes of layer l-1 read parents of layers >= l that are never children of a layer-l
  // block, so they do not wait for the layer-l blocks: with a second side stream they run beside them.
  const bool split = c->side2 && !c->prof.on && c->bwd_split;
  PCB_TRY(sparse_down(c->L, st, c->pdl));
  for (int64_t lay = c->L; lay >= 1; --lay) {
    const bool has_dense = c->h_dense_off[lay + 1] > c->h_dense_off[lay];
    const bool has_sparse = c->h_down_sparse_off[lay] > c->h_down_sparse_off[lay - 1];
    if (split && has_dense && has_sparse) {
      PCB_CUDA(cudaEventRecord(c->ev_fork2, st));
      PCB_CUDA(cudaStreamWaitEvent(c->side2, c->ev_fork2, 0));
      PCB_TRY(sparse_down(lay - 1, c->side2, false));
      PCB_TRY(pcb_dense_backward(c, ws, (uint32_t)lay, st));
      PCB_CUDA(cudaEventRecord(c->ev_join2, c->side2));
      PCB_CUDA(cudaStreamWaitEvent(st, c->ev_join2, 0));
    } else {
      PCB_TRY(pcb_dense_backward(c, ws, (uint32_t)lay, st));
      PCB_TRY(sparse_down(lay - 1, st, c->pdl));
    }
  }
  if (c->use_tc && !c->skip_stats) PCB_TRY(pcb_dense_tc_flush_edges(c, ws, st));
  if (split_comm) PCB_TRY(comm_edges_begin(c, st));
  if (early && c->side && c->use_tc && !c->prof.on) {
    // every edge statistic is final once this stream's kernels so far and the side stream's are done
    PCB_CUDA(cudaEventRecord(c->ev_fork, st));
    PCB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    PCB_TRY(em_update_sums(c, early->pseudocount, early->inertia, c->side));
    PCB_TRY(pcb_dense_tc_refresh(c, c->side));
    c->side_busy = true;
    early->done = true;
  }
  if (c->n_inputs && !c->skip_stats) {
    PcbProfScope ps(c, st, PCB_K_LEAF_FLOW);
    // sorted segments pay off once a variable has enough values to keep a block's threads busy;
    // PCB_LEAF_FLOW_IMPL=atomic / sorted (read when the circuit is created) forces one of the two kernels
    const bool want_sorted = c->leaf_flow_impl ? c->leaf_flow_impl == 2 : c->max_cats >= 16;
    if (ws->soft || ws->soft_reg > 0.0f) {
      leaf_flow_gen_kernel<<<grid2(c->n_inputs, B), TPB, 0, st>>>(
          ws->flows, ws->mars, ws->ld, B, c->aggr, c->theta, c->in_node, c->in_var, c->in_cats, c->in_poff, c->in_foff,
          c->V, ws->data, ws->miss, ws->soft, ws->num_rows, ws->row_ids, ws->row_start, weights_dev, ws->soft_reg,
          (int32_t)ws->soft_width);
    } else if (c->max_cats <= LSC && want_sorted) {
      dim3 grid(c->n_lgrps, (B + LSB - 1) / LSB);
      auto* kern = weights_dev ? leaf_flow_sorted_kernel<true> : leaf_flow_sorted_kernel<false>;
      kern<<<grid, LST, 0, st>>>(
          ws->flows, ws->ld, B, c->aggr, c->in_node, c->in_cats, c->in_foff, c->lgrp_var, c->lgrp_off,
          c->lchunk_inputs, c->max_cats, ws->data, ws->miss, ws->num_rows, ws->row_ids, ws->row_start, weights_dev,
          c->status);
    } else if (c->max_cats <= 1024) {
      uint32_t hstride = c->max_cats + 1;
      dim3 grid(c->n_lchunks, (B + LBT - 1) / LBT);
      leaf_flow_chunk_kernel<<<grid, LTH, PCB_LEAF_CHUNK * hstride * sizeof(float), st>>>(
          ws->flows, ws->ld, B, c->aggr, hstride, c->in_node, c->in_cats, c->in_foff, c->lchunk_var, c->lchunk_off,
          c->lchunk_inputs, ws->data, ws->miss, ws->num_rows, ws->row_ids, ws->row_start, weights_dev);
    } else {
      leaf_flow_kernel<<<grid2(c->n_inputs, B), TPB, 0, st>>>(ws->flows, ws->ld, B, c->aggr, c->in_node, c->in_var,
                                                              c->in_cats, c->in_foff, ws->data, ws->miss,
                                                              ws->num_rows, ws->row_ids, ws->row_start, weights_dev);
    }
  }
  PCB_TRY(pcb_side_join(c, st));  // the leaf statistics above overlap the last edge-statistics kernels
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

extern "C" int32_t pcb_clear_flows(pcb_circuit* c, float rate, pcb_stream s) {
  PCB_REQUIRE(c, "null argument");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  if (rate == 0.0f) {
    PCB_CUDA(cudaMemsetAsync(c->aggr, 0, c->aggr_len * sizeof(float), st));
  } else {
    uint64_t n = c->aggr_len - 1;
    uint32_t blocks = (uint32_t)std::min<uint64_t>((n + 255) / 256, 148 * 16);
    if (n) { PcbProfScope ps(c, st, PCB_K_MISC); scale_kernel<<<blocks, 256, 0, st>>>(c->aggr, n, rate); }
    PCB_CUDA(cudaMemsetAsync(c->aggr + n, 0, sizeof(float), st));
    PCB_CUDA(cudaGetLastError());
  }
  return PCB_OK;
}

static int32_t em_update_sums(pcb_circuit* c, float pseudocount, float inertia, cudaStream_t st) {
  if (c->n_groups)
    { PcbProfScope ps(c, st, PCB_K_UPDATE); em_update_sum_kernel<<<(c->n_groups + 7) / 8, 256, 0, st>>>(c->theta, c->aggr, c->grp_node, c->n_groups,
                                                                c->n_pid0, c->n_ecount, pseudocount, inertia); }
  c->w_img_valid = false;  // the weights changed
  return PCB_OK;
}
static int32_t em_update_leaves(pcb_circuit* c, float pseudocount, float inertia, cudaStream_t st) {
  if (c->n_inputs)
    { PcbProfScope ps(c, st, PCB_K_UPDATE); em_update_leaf_kernel<<<(c->n_inputs + 7) / 8, 256, 0, st>>>(c->theta, c->aggr, c->n_inputs, c->in_cats,
                                                                 c->in_poff, c->in_foff, pseudocount, inertia); }
  return PCB_OK;
}

extern "C" int32_t pcb_em_update(pcb_circuit* c, float pseudocount, float inertia, pcb_stream s) {
  PCB_REQUIRE(c, "null argument");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  PCB_TRY(em_update_sums(c, pseudocount, inertia, st));
  PCB_TRY(em_update_leaves(c, pseudocount, inertia, st));
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

// clear, forward, backward, (all-reduce,) update: the launches of one EM step on stream st.  The
// batch log-likelihood stays in the last slot of the statistics vector; pcb_em_step copies it out.
static int32_t em_step_body(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence& ev, const float* weights_dev,
                            float clear_rate, float pseudocount, float inertia, cudaStream_t st) {
  pcb_stream s = (pcb_stream)st;
  const uint32_t B = ev.B;
  // With a communicator every rank enters the step holding the same summed statistics of the last
  // step (pseudocount included, as the reference keeps it in edge_aggr); the all-reduce below adds
  // the ranks' vectors, so each rank carries rate / nranks of them and the sum is rate * previous
  // + this step's flows, as reg_em.jl:276-284 computes it on one device.
  const float carried = (c->comm && c->nranks > 1) ? clear_rate / (float)c->nranks : clear_rate;
  PCB_TRY(pcb_clear_flows(c, carried, s));
  // multi-head circuits: the per-example log-likelihoods mix the heads (em.jl:71 of multi_head_pc)
  { PcbNvtxRange r("pcb forward"); PCB_TRY(forward_impl(c, ws, ev, c->n_heads ? ws->ll_tmp : nullptr, st)); }
  const bool multi = c->comm && c->nranks > 1 && c->comm_enabled;
  const bool split = multi && c->comm_split && !c->prof.on;   // per-class timing wants every class alone on the GPU
  EarlyUpdate early{pseudocount, inertia, false};
  { PcbNvtxRange r("pcb backward"); PCB_TRY(backward_impl(c, ws, weights_dev, st, split, (!multi && c->early_update) ? &early : nullptr)); }
  PcbNvtxRange r_update("pcb reduce + update");
  // batch log-likelihood into the last slot of the statistics vector, so it is reduced with them
  { PcbProfScope ps(c, st, PCB_K_MISC);
    ll_sum_kernel<<<1, 256, 0, st>>>(c->n_heads ? ws->ll_tmp : ws->mars + (size_t)(c->N - 1) * ws->ld, B,
                                     c->aggr + c->aggr_len - 1); }
  const bool pipe = multi && !split && c->comm_pipe && !c->prof.on && c->n_inner && c->comm_stream;
  if (pipe) {
    // Two collectives on the communication stream, edge statistics first; this stream updates the sum
    // parameters and rebuilds the weight images while the leaf slots are still being summed.
    PCB_CUDA(cudaEventRecord(c->ev_c0, st));
    PCB_CUDA(cudaStreamWaitEvent(c->comm_stream, c->ev_c0, 0));
    PCB_TRY(pcb_allreduce_range(c, 0, c->n_inner, c->comm_stream));
    PCB_CUDA(cudaEventRecord(c->ev_c1, c->comm_stream));
    PCB_TRY(pcb_allreduce_range(c, c->n_inner, c->aggr_len - c->n_inner, c->comm_stream));
    PCB_CUDA(cudaEventRecord(c->ev_c3, c->comm_stream));
    PCB_CUDA(cudaStreamWaitEvent(st, c->ev_c1, 0));
    PCB_TRY(em_update_sums(c, pseudocount, inertia, st));
    if (c->use_tc) PCB_TRY(pcb_dense_tc_refresh(c, st));
    PCB_CUDA(cudaStreamWaitEvent(st, c->ev_c3, 0));
    PCB_TRY(em_update_leaves(c, pseudocount, inertia, st));
    PCB_CUDA(cudaGetLastError());
    return PCB_OK;
  }
  if (split) PCB_TRY(comm_rest_and_join(c, st));
  else if (multi) { PcbProfScope ps(c, st, PCB_K_ALLREDUCE); PCB_TRY(pcb_allreduce_aggr(c, st)); }
  if (early.done) PCB_TRY(em_update_leaves(c, pseudocount, inertia, st));
  else PCB_TRY(pcb_em_update(c, pseudocount, inertia, s));
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

static int32_t em_step_impl(pcb_circuit* c, pcb_workspace* ws, pcb_evidence ev, const float* weights_dev,
                            float clear_rate, float pseudocount, float inertia, float* ll_sum_dev, pcb_stream s) {
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  const uint32_t B = ev.B;
  PCB_REQUIRE(B >= 1 && B <= ws->max_batch, "batch size exceeds the workspace");
  PCB_REQUIRE(!c->n_heads || ev.head_mask_dev, "the flows of a multi-head circuit need a head mask");
  if (c->comm_lost)
    return pcb_fail(PCB_ERR_STATE, "the communicator was aborted: pcb_comm_destroy, then attach a new one or train alone");
  PCB_CUDA(cudaSetDevice(c->device));
  if (c->n_heads && !ws->ll_tmp) PCB_CUDA(cudaMalloc(&ws->ll_tmp, (size_t)ws->max_batch * sizeof(float)));
  const uint8_t* data_dev = ev.data_dev;
  const uint8_t* miss_dev = ev.miss_dev;
  const uint64_t num_rows = ev.num_rows;
  const int32_t* row_ids_dev = ev.row_ids_dev;
  uint32_t row_start = ev.row_start;
  cudaStream_t st = (cudaStream_t)s;
  // the step reads the row ids from the workspace's own buffer, so a replayed graph sees the ids
  // of the current call
  if (row_ids_dev) {
    PCB_CUDA(cudaMemcpyAsync(ws->ids_stage, row_ids_dev, (size_t)B * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  } else {
    // a row range becomes staged ids too, so that consecutive batches of an epoch replay one graph
    PCB_REQUIRE(row_start >= 1 && (uint64_t)row_start - 1 + B <= num_rows, "row range out of bounds");
    iota_ids_kernel<<<(B + 255) / 256, 256, 0, st>>>(ws->ids_stage, (int32_t)row_start, B);
    row_start = 1;
  }
  row_ids_dev = ws->ids_stage;
  ev.row_ids_dev = row_ids_dev; ev.row_start = row_start;
  if (c->checked) PCB_TRY(pcb_check_batch(c, ev, st));   // before the statistics are cleared
  // The log-likelihood leaves through a copy issued after the step (the update does not touch its
  // slot), outside any captured graph: a training loop hands in a different slot for every batch.
  auto ll_out = [&](cudaStream_t on) -> int32_t {
    if (ll_sum_dev)
      PCB_CUDA(cudaMemcpyAsync(ll_sum_dev, c->aggr + c->aggr_len - 1, sizeof(float), cudaMemcpyDeviceToDevice, on));
    return PCB_OK;
  };
  auto plain = [&]() -> int32_t {
    PCB_TRY(em_step_body(c, ws, ev, weights_dev, clear_rate, pseudocount, inertia, st));
    return ll_out(st);
  };
  if (!c->graph_enabled || c->prof.on || c->checked) return plain();   // checked mode synchronises inside the pass

  pcb_workspace::StepKey key;
  memset(&key, 0, sizeof(key));
  key.data = data_dev; key.miss = miss_dev; key.weights = weights_dev; key.comm = c->comm;
  key.stream = (void*)st; key.num_rows = num_rows; key.row_start = row_start; key.B = B;
  key.clear_rate = clear_rate; key.pseudocount = pseudocount; key.inertia = inertia;
  key.has_ids = row_ids_dev != nullptr; key.w_valid = c->w_img_valid; key.comm_on = c->comm_enabled;
  key.soft = ev.soft_dev; key.head_mask = ev.head_mask_dev; key.soft_reg = ev.soft_reg; key.soft_width = ev.soft_reg_width;

  // the legacy default stream cannot be captured: graphs run on a stream of the circuit's own,
  // ordered after and before the caller's stream with two events
  cudaStream_t gs = st;
  const bool legacy = st == nullptr || st == cudaStreamLegacy;
  if (legacy) {
    if (!c->gstream) {
      PCB_CUDA(cudaStreamCreateWithFlags(&c->gstream, cudaStreamNonBlocking));
      PCB_CUDA(cudaEventCreateWithFlags(&c->ev_g0, cudaEventDisableTiming));
      PCB_CUDA(cudaEventCreateWithFlags(&c->ev_g1, cudaEventDisableTiming));
    }
    gs = c->gstream;
  }
  auto enter = [&]() -> int32_t {
    if (legacy) { PCB_CUDA(cudaEventRecord(c->ev_g0, st)); PCB_CUDA(cudaStreamWaitEvent(gs, c->ev_g0, 0)); }
    return PCB_OK;
  };
  auto leave = [&]() -> int32_t {
    if (legacy) { PCB_CUDA(cudaEventRecord(c->ev_g1, gs)); PCB_CUDA(cudaStreamWaitEvent(st, c->ev_g1, 0)); }
    return PCB_OK;
  };

  if (ws->step_exec && !memcmp(&key, &ws->exec_key, sizeof(key))) {
    // replay; the host-side state is what the captured run left behind
    PCB_TRY(enter());
    PCB_CUDA(cudaGraphLaunch(ws->step_exec, gs));
    PCB_TRY(ll_out(gs));
    PCB_TRY(leave());
    for (int k = 0; k < PCB_K_COUNT; ++k) c->prof.launches[k] += ws->step_launches[k];
    ws->B = B; ws->data = data_dev; ws->miss = miss_dev; ws->num_rows = num_rows;
    ws->row_ids = row_ids_dev; ws->row_start = row_start; ws->have_forward = true;
    ws->soft = ev.soft_dev; ws->head_mask = ev.head_mask_dev;
    ws->soft_reg = ev.soft_dev ? 0.0f : ev.soft_reg; ws->soft_width = ev.soft_reg_width;
    c->w_img_valid = ws->exec_end_w_valid;
    return PCB_OK;
  }
  const bool capture = ws->have_key && !memcmp(&key, &ws->last_key, sizeof(key));
  ws->last_key = key;
  ws->have_key = true;
  if (!capture) return plain();

  if (ws->step_exec) { cudaGraphExecDestroy(ws->step_exec); ws->step_exec = nullptr; }
  uint64_t before[PCB_K_COUNT];
  for (int k = 0; k < PCB_K_COUNT; ++k) before[k] = c->prof.launches[k];
  PCB_TRY(enter());
  PCB_CUDA(cudaStreamBeginCapture(gs, cudaStreamCaptureModeRelaxed));
  int32_t body = em_step_body(c, ws, ev, weights_dev, clear_rate, pseudocount, inertia, gs);
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(gs, &graph);
  if (body != PCB_OK || ce != cudaSuccess || !graph) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    c->graph_enabled = false;   // this circuit's step does not capture: stay with plain launches
    if (body != PCB_OK) return body;
    for (int k = 0; k < PCB_K_COUNT; ++k) c->prof.launches[k] = before[k];
    c->w_img_valid = key.w_valid != 0;
    return plain();
  }
  ce = cudaGraphInstantiate(&ws->step_exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ce != cudaSuccess) {
    ws->step_exec = nullptr;
    c->graph_enabled = false;
    for (int k = 0; k < PCB_K_COUNT; ++k) c->prof.launches[k] = before[k];
    c->w_img_valid = key.w_valid != 0;
    cudaGetLastError();
    return plain();
  }
  for (int k = 0; k < PCB_K_COUNT; ++k) ws->step_launches[k] = c->prof.launches[k] - before[k];
  ws->exec_key = key;
  ws->exec_end_w_valid = c->w_img_valid;   // host-side state the captured step ends in
  PCB_CUDA(cudaGraphLaunch(ws->step_exec, gs));
  PCB_TRY(ll_out(gs));
  PCB_TRY(leave());
  return PCB_OK;
}

extern "C" int32_t pcb_em_step(pcb_circuit* c, pcb_workspace* ws, const uint8_t* data_dev,
                               const uint8_t* miss_dev, uint64_t num_rows, const int32_t* row_ids_dev,
                               uint32_t row_start, uint32_t B, const float* weights_dev, float clear_rate,
                               float pseudocount, float inertia, float* ll_sum_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && data_dev, "null argument");
  return em_step_impl(c, ws, hard_evidence(data_dev, miss_dev, num_rows, row_ids_dev, row_start, B), weights_dev,
                      clear_rate, pseudocount, inertia, ll_sum_dev, s);
}

extern "C" int32_t pcb_em_step_ex(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, const float* weights_dev,
                                  float clear_rate, float pseudocount, float inertia, float* ll_sum_dev,
                                  pcb_stream s) {
  PCB_REQUIRE(c && ws && ev, "null argument");
  PCB_REQUIRE(ev->data_dev || ev->soft_dev, "null argument");
  return em_step_impl(c, ws, *ev, weights_dev, clear_rate, pseudocount, inertia, ll_sum_dev, s);
}

static int32_t get_matrix(pcb_circuit* c, pcb_workspace* ws, const float* src, float* host, uint64_t n) {
  PCB_REQUIRE(c && ws && host, "null argument");
  PCB_REQUIRE(ws->have_forward, "no batch has been evaluated on this workspace");
  PCB_REQUIRE(n == (uint64_t)ws->B * c->N, "matrix has the wrong size");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_TRY(pcb_check_status(c));
  PCB_CUDA(cudaMemcpy2D(host, ws->B * sizeof(float), src, ws->ld * sizeof(float), ws->B * sizeof(float), c->N,
                        cudaMemcpyDeviceToHost));
  return PCB_OK;
}
extern "C" int32_t pcb_get_mars(pcb_circuit* c, pcb_workspace* ws, float* mars_host, uint64_t n) {
  return get_matrix(c, ws, ws ? ws->mars : nullptr, mars_host, n);
}
extern "C" int32_t pcb_get_flows(pcb_circuit* c, pcb_workspace* ws, float* flows_host, uint64_t n) {
  return get_matrix(c, ws, ws ? ws->flows : nullptr, flows_host, n);
}
