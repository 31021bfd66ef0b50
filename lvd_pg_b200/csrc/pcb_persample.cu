// pcb_persample.cu — per-sample normalised flows, with the circuit's own parameters or with one
// parameter vector per data row.
//
// Reference kernels replaced (paths relative to VariationalJuice.jl/src):
//   ps_leaf_kernel    init_mar!_kernel with params          queries/likelihood.jl:214-283
//   ps_up_kernel      layer_up_kernel with params           queries/likelihood.jl:119-210
//   ps_down_kernel    layer_down_kernel with params         queries/flow.jl:240-403
//   norm_sum_kernel   map_flows_kernel                      queries/flow.jl:496-547
//   norm_leaf_kernel  input_flows_circuit_kernel +          queries/flow.jl:165-226,
//                     map_input_flows_kernel                queries/flow.jl:549-612
//   pcb_normalized_flows   per_sample_normalized_flows      queries/flow.jl:417-494
//
// The reference materialises edge_mars and edge_flows ([B, E] each) and normalises them in a third
// pass.  Here an edge flow is formed where it is consumed: the normalising kernel recomputes
// flow(parent) * exp(child + log theta - parent) from the node matrices, sums a parameter group in
// registers and writes log(flow / (sum + 1e-8) + 1e-8) straight to the [rows, P] output, whose row
// index is the fastest one, so a warp writes 128 contiguous bytes per parameter.  With the
// circuit's own parameters the node matrices come from the ordinary forward / backward passes
// (tensor-core blocks included); with per-row parameters every sum edge has one weight per example
// and the passes are the gather kernels of this file.
#include <algorithm>

#include "pcb_internal.h"

namespace {

constexpr uint32_t TPB = 128;

__device__ __forceinline__ int64_t data_row(const int32_t* row_ids, uint32_t row_start, uint32_t b) {
  return row_ids ? (int64_t)row_ids[b] - 1 : (int64_t)row_start - 1 + b;
}

// log-parameter of parameter `pid` for example b: the row's own vector, or the circuit's
struct Params {
  const float* per_row;   // [rows, P] column-major, or null
  const float* theta;     // [P]
  uint64_t rows;
  __device__ __forceinline__ float at(int64_t row, uint64_t pid) const {
    return per_row ? per_row[(size_t)row + (size_t)rows * pid] : __ldg(theta + pid);
  }
};

__global__ void ps_leaf_kernel(float* __restrict__ mars, uint32_t ld, uint32_t B, Params p, uint64_t P,
                               const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_var,
                               const uint64_t* __restrict__ in_poff, const uint8_t* __restrict__ data,
                               const uint8_t* __restrict__ miss, uint64_t num_rows, const int32_t* __restrict__ row_ids,
                               uint32_t row_start) {
  const uint32_t i = blockIdx.x, b = blockIdx.y * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int64_t row = data_row(row_ids, row_start, b);
  const size_t di = (size_t)row + (size_t)num_rows * in_var[i];
  float v = 0.0f;   // a missing value marginalises the leaf
  if (!(miss && miss[di])) {
    const uint64_t po = in_poff[i] + data[di];
    v = in_poff[i] < P ? p.at(row, po) : __ldg(p.theta + po);   // fixed leaves live behind P in the circuit's vector
  }
  mars[(size_t)in_node[i] * ld + b] = v;
}

__global__ void ps_up_kernel(float* __restrict__ mars, uint32_t ld, uint32_t B, Params p,
                             const uint32_t* __restrict__ nodes, const uint4* __restrict__ s_node,
                             const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub,
                             const int32_t* __restrict__ row_ids, uint32_t row_start) {
  const uint32_t n = nodes[blockIdx.x], b = blockIdx.y * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint4 sn = s_node[n];   // edge start, edge count, first parameter, kind | region << 2
  const int64_t row = data_row(row_ids, row_start, b);
  const bool issum = (sn.w & 3u) == PCB_SUM;
  float m = -INFINITY, acc = 0.0f;   // running maximum and sum of exp(v - m)
  for (uint32_t j = 0; j < sn.y; ++j) {
    float v = mars[(size_t)e_prime[sn.x + j] * ld + b];
    const uint32_t sb = e_sub[sn.x + j];
    if (sb != PCB_NONE) v += mars[(size_t)sb * ld + b];
    if (!issum) { acc += v; continue; }
    v += p.at(row, sn.z + j);
    if (v > m) { acc = acc * __expf(m - v) + 1.0f; m = v; }
    else if (v != -INFINITY) acc += __expf(v - m);
  }
  mars[(size_t)n * ld + b] = issum ? (m == -INFINITY ? -INFINITY : m + __logf(acc)) : acc;
}

__global__ void ps_down_kernel(float* __restrict__ flows, const float* __restrict__ mars, uint32_t ld, uint32_t B,
                               Params p, const uint32_t* __restrict__ nodes, uint32_t root,
                               const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                               const int32_t* __restrict__ row_ids, uint32_t row_start) {
  const uint32_t n = nodes[blockIdx.x], b = blockIdx.y * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  const int64_t row = data_row(row_ids, row_start, b);
  const float mine = mars[(size_t)n * ld + b];
  float acc = (i0 == i1 && n == root) ? 1.0f : 0.0f;
  for (uint32_t x = i0; x < i1; ++x) {
    const PcbInEntry en = in_ent[x];
    float ef = flows[(size_t)en.parent * ld + b];
    if (en.pid != PCB_NONE && ef != 0.0f) {
      float child = mine + p.at(row, en.pid);
      if (en.sib != PCB_NONE) child += mars[(size_t)en.sib * ld + b];
      ef *= __expf(child - mars[(size_t)en.parent * ld + b]);
    }
    acc += ef;
  }
  flows[(size_t)n * ld + b] = acc;
}

// One block per (sum node, 128 examples), one thread per example: the node's edge list (and, with the
// circuit's own parameters, its weights) is staged in shared memory once, a thread keeps up to 32
// edge flows in registers between the sum and the normalised write; wider nodes recompute them.
constexpr uint32_t NS_REG = 32, NS_STAGE = 256;
__global__ void __launch_bounds__(TPB) norm_sum_kernel(const float* __restrict__ flows, const float* __restrict__ mars,
                                                       uint32_t ld, uint32_t B, Params p,
                                                       const uint32_t* __restrict__ grp_node, const uint4* __restrict__ s_node,
                                                       const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub,
                                                       const int32_t* __restrict__ row_ids, uint32_t row_start,
                                                       float* __restrict__ out, uint64_t out_rows) {
  __shared__ uint32_t s_pr[NS_STAGE], s_sb[NS_STAGE];
  __shared__ float s_w[NS_STAGE];
  const uint32_t n = grp_node[blockIdx.x], b = blockIdx.y * blockDim.x + threadIdx.x;
  const uint4 sn = s_node[n];
  const uint32_t cnt = sn.y, staged = min(cnt, NS_STAGE);
  for (uint32_t j = threadIdx.x; j < staged; j += blockDim.x) {
    s_pr[j] = e_prime[sn.x + j];
    s_sb[j] = e_sub[sn.x + j];
    s_w[j] = p.per_row ? 0.0f : __ldg(p.theta + sn.z + j);
  }
  __syncthreads();
  if (b >= B) return;
  const int64_t row = data_row(row_ids, row_start, b);
  const float pf = flows[(size_t)n * ld + b], pm = mars[(size_t)n * ld + b];
  auto edge_flow = [&](uint32_t j) {
    if (pf == 0.0f) return 0.0f;
    const uint32_t pr = j < NS_STAGE ? s_pr[j] : e_prime[sn.x + j], sb = j < NS_STAGE ? s_sb[j] : e_sub[sn.x + j];
    float child = mars[(size_t)pr * ld + b];
    child += p.per_row ? p.per_row[(size_t)row + (size_t)p.rows * (sn.z + j)] : (j < NS_STAGE ? s_w[j] : __ldg(p.theta + sn.z + j));
    if (sb != PCB_NONE) child += mars[(size_t)sb * ld + b];
    return pf * __expf(child - pm);
  };
  float ef[NS_REG];
  float total = 1e-8f;   // par_groups .= 1e-8 (flow.jl:535)
#pragma unroll
  for (uint32_t j = 0; j < NS_REG; ++j) {
    ef[j] = j < cnt ? edge_flow(j) : 0.0f;
    total += ef[j];
  }
  for (uint32_t j = NS_REG; j < cnt; ++j) total += edge_flow(j);
  float* o = out + (size_t)row + (size_t)out_rows * sn.z;
  const float inv = 1.0f / total;
#pragma unroll
  for (uint32_t j = 0; j < NS_REG; ++j)
    if (j < cnt) o[(size_t)out_rows * j] = __logf(ef[j] * inv + 1e-8f);
  for (uint32_t j = NS_REG; j < cnt; ++j) o[(size_t)out_rows * j] = __logf(edge_flow(j) * inv + 1e-8f);
}

// The same with four consecutive examples per thread (16-byte loads of the node rows, 16-byte stores):
// a block of 128 threads then writes 2 KB of every output column in one piece.  Columns are a whole
// matrix row apart, and with 512-byte pieces per column the writes of the resident blocks land on as
// many DRAM pages as there are pieces (measured 0.6 TB/s); used when the batch is a row range whose
// start and the output's row count are multiples of four.
constexpr uint32_t NS_REG4 = 16;
__global__ void __launch_bounds__(TPB) norm_sum4_kernel(const float* __restrict__ flows, const float* __restrict__ mars,
                                                        uint32_t ld, uint32_t B, Params p,
                                                        const uint32_t* __restrict__ grp_node, const uint4* __restrict__ s_node,
                                                        const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub,
                                                        uint32_t row_start, float* __restrict__ out, uint64_t out_rows) {
  __shared__ uint32_t s_pr[NS_STAGE], s_sb[NS_STAGE];
  __shared__ float s_w[NS_STAGE];
  const uint32_t n = grp_node[blockIdx.x], b = (blockIdx.y * blockDim.x + threadIdx.x) * 4u;
  const uint4 sn = s_node[n];
  const uint32_t cnt = sn.y, staged = min(cnt, NS_STAGE);
  for (uint32_t j = threadIdx.x; j < staged; j += blockDim.x) {
    s_pr[j] = e_prime[sn.x + j];
    s_sb[j] = e_sub[sn.x + j];
    s_w[j] = p.per_row ? 0.0f : __ldg(p.theta + sn.z + j);
  }
  __syncthreads();
  if (b >= B) return;
  const size_t row = (size_t)row_start - 1 + b;
  auto ld4 = [](const float* q) { return *reinterpret_cast<const float4*>(q); };
  const float4 pf = ld4(flows + (size_t)n * ld + b), pm = ld4(mars + (size_t)n * ld + b);
  auto edge_flow = [&](uint32_t j) {
    const uint32_t pr = j < NS_STAGE ? s_pr[j] : e_prime[sn.x + j], sb = j < NS_STAGE ? s_sb[j] : e_sub[sn.x + j];
    float4 c = ld4(mars + (size_t)pr * ld + b);
    if (sb != PCB_NONE) { const float4 d = ld4(mars + (size_t)sb * ld + b); c.x += d.x; c.y += d.y; c.z += d.z; c.w += d.w; }
    if (p.per_row) {
      const float4 w = ld4(p.per_row + row + (size_t)p.rows * (sn.z + j));
      c.x += w.x; c.y += w.y; c.z += w.z; c.w += w.w;
    } else {
      const float w = j < NS_STAGE ? s_w[j] : __ldg(p.theta + sn.z + j);
      c.x += w; c.y += w; c.z += w; c.w += w;
    }
    float4 e;
    e.x = pf.x == 0.0f ? 0.0f : pf.x * __expf(c.x - pm.x);
    e.y = pf.y == 0.0f ? 0.0f : pf.y * __expf(c.y - pm.y);
    e.z = pf.z == 0.0f ? 0.0f : pf.z * __expf(c.z - pm.z);
    e.w = pf.w == 0.0f ? 0.0f : pf.w * __expf(c.w - pm.w);
    return e;
  };
  float4 ef[NS_REG4];
  float4 total = make_float4(1e-8f, 1e-8f, 1e-8f, 1e-8f);
#pragma unroll
  for (uint32_t j = 0; j < NS_REG4; ++j) {
    ef[j] = j < cnt ? edge_flow(j) : make_float4(0.f, 0.f, 0.f, 0.f);
    total.x += ef[j].x; total.y += ef[j].y; total.z += ef[j].z; total.w += ef[j].w;
  }
  for (uint32_t j = NS_REG4; j < cnt; ++j) {
    const float4 e = edge_flow(j);
    total.x += e.x; total.y += e.y; total.z += e.z; total.w += e.w;
  }
  const float4 inv = make_float4(1.0f / total.x, 1.0f / total.y, 1.0f / total.z, 1.0f / total.w);
  float* o = out + row + (size_t)out_rows * sn.z;
  const bool whole = b + 4 <= B;
  auto put = [&](uint32_t j, const float4& e) {
    const float4 v = make_float4(__logf(e.x * inv.x + 1e-8f), __logf(e.y * inv.y + 1e-8f), __logf(e.z * inv.z + 1e-8f),
                                 __logf(e.w * inv.w + 1e-8f));
    float* q = o + (size_t)out_rows * j;
    if (whole) { *reinterpret_cast<float4*>(q) = v; return; }
    q[0] = v.x;
    if (b + 1 < B) q[1] = v.y;
    if (b + 2 < B) q[2] = v.z;
  };
#pragma unroll
  for (uint32_t j = 0; j < NS_REG4; ++j)
    if (j < cnt) put(j, ef[j]);
  for (uint32_t j = NS_REG4; j < cnt; ++j) put(j, edge_flow(j));
}

// A learnable leaf hands its whole flow to the observed category (get_edge_flow,
// nodes/fixable_categorical_dist.jl:162-176): log(flow / flow) = 0 there and log(0) = -inf elsewhere;
// a leaf without flow gives 0 / 0 as in the reference.
__global__ void norm_leaf_kernel(const float* __restrict__ flows, uint32_t ld, uint32_t B, uint64_t P,
                                 const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_var,
                                 const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                 const uint8_t* __restrict__ data, uint64_t num_rows,
                                 const int32_t* __restrict__ row_ids, uint32_t row_start, float* __restrict__ out,
                                 uint64_t out_rows) {
  const uint32_t i = blockIdx.x, b = blockIdx.y * blockDim.x + threadIdx.x;
  if (b >= B || in_poff[i] >= P) return;
  const int64_t row = data_row(row_ids, row_start, b);
  const size_t di = (size_t)row + (size_t)num_rows * in_var[i];
  const float f = flows[(size_t)in_node[i] * ld + b];
  const uint32_t x = data[di], C = in_cats[i];
  for (uint32_t c = 0; c < C; ++c)
    out[(size_t)row + (size_t)out_rows * (in_poff[i] + c)] = logf((c == x ? f : 0.0f) / f);
}

// normalize_params (misc.jl:363-392, 405-447): on a [S, P] matrix of parameter sets, in place.
// Leaves: exp and division by the leaf's sum, i.e. PROBABILITIES (undo: log(p + 1e-6) of positive
// entries, the others kept); sum groups: log-parameters minus the log of the group's summed exp
// (in both directions: the reference's inner kernel has no undo form).
__global__ void normalize_leaf_kernel(float* __restrict__ params, uint32_t S, uint32_t n_inputs, uint64_t P,
                                      const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff, int undo) {
  const uint32_t i = blockIdx.x, s = blockIdx.y * blockDim.x + threadIdx.x;
  if (s >= S || in_poff[i] >= P) return;
  float* q = params + s + (size_t)S * in_poff[i];
  const uint32_t C = in_cats[i];
  if (undo) {
    for (uint32_t k = 0; k < C; ++k) {
      const float v = q[(size_t)S * k];
      if (v > 0.0f) q[(size_t)S * k] = logf(v + 1e-6f);
    }
    return;
  }
  float total = 0.0f;
  for (uint32_t k = 0; k < C; ++k) {
    const float v = expf(q[(size_t)S * k]);
    q[(size_t)S * k] = v;
    total += v;
  }
  for (uint32_t k = 0; k < C; ++k) q[(size_t)S * k] /= total;
}

__global__ void normalize_sum_kernel(float* __restrict__ params, uint32_t S, const uint32_t* __restrict__ grp_node,
                                     const uint4* __restrict__ s_node) {
  const uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const uint4 sn = s_node[grp_node[blockIdx.x]];
  float* q = params + s + (size_t)S * sn.z;
  float total = 0.0f;
  for (uint32_t j = 0; j < sn.y; ++j) total += expf(q[(size_t)S * j]);
  const float lt = logf(total);
  for (uint32_t j = 0; j < sn.y; ++j) q[(size_t)S * j] -= lt;
}

// map_pc_parameters_kernel (utils/map_params.jl:128-146): dst[s, ids_dst[i]] = src[s, ids_src[i]], ids 1-based
__global__ void map_columns_kernel(float* __restrict__ dst, const float* __restrict__ src, uint32_t S,
                                   const uint32_t* __restrict__ ids_dst, const uint32_t* __restrict__ ids_src) {
  const uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (s >= S) return;
  dst[s + (size_t)S * (ids_dst[blockIdx.x] - 1)] = src[s + (size_t)S * (ids_src[blockIdx.x] - 1)];
}

dim3 grid2(uint32_t items, uint32_t B) { return dim3(items, (B + TPB - 1) / TPB, 1); }

}  // namespace

#define PCB_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != PCB_OK) return _s;   \
  } while (0)

extern "C" int32_t pcb_normalized_flows(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, const float* params_dev,
                                        float* out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && ev && out_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(ev->data_dev && !ev->miss_dev && !ev->soft_dev && ev->soft_reg == 0.0f && !ev->head_mask_dev,
              "normalised flows take hard evidence without missing values");
  PCB_REQUIRE(!c->n_heads, "normalised flows take a single-head circuit");
  const uint32_t B = ev->B;
  PCB_REQUIRE(B >= 1 && B <= ws->max_batch, "batch size exceeds the workspace");
  PCB_REQUIRE(ev->row_ids_dev || (ev->row_start >= 1 && (uint64_t)ev->row_start - 1 + B <= ev->num_rows),
              "row range out of bounds");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  const Params p{params_dev, c->theta, ev->num_rows};
  if (!params_dev) {
    // the circuit's own parameters: the ordinary passes, flows only (the reference hands edge_aggr = nothing)
    PCB_TRY(pcb_forward_ex(c, ws, ev, nullptr, s));
    c->skip_stats = true;
    const int32_t rb = pcb_backward(c, ws, nullptr, s);
    c->skip_stats = false;
    PCB_TRY(rb);
  } else {
    if (c->checked) PCB_TRY(pcb_check_batch(c, *ev, st));
    ws->have_forward = false;
    ws->B = B; ws->data = ev->data_dev; ws->miss = ev->miss_dev; ws->num_rows = ev->num_rows;
    ws->row_ids = ev->row_ids_dev; ws->row_start = ev->row_start;
    ws->soft = nullptr; ws->head_mask = nullptr; ws->soft_reg = 0.0f;
    if (c->n_inputs) {
      ++c->prof.launches[PCB_K_MISC];
      ps_leaf_kernel<<<grid2(c->n_inputs, B), TPB, 0, st>>>(ws->mars, ws->ld, B, p, c->P, c->in_node, c->in_var, c->in_poff,
                                                           ev->data_dev, ev->miss_dev, ev->num_rows, ev->row_ids_dev,
                                                           ev->row_start);
    }
    for (uint32_t lay = 1; lay <= c->L; ++lay) {
      const uint32_t o0 = c->h_up_all_off[lay - 1], o1 = c->h_up_all_off[lay];
      if (o1 == o0) continue;
      ++c->prof.launches[PCB_K_MISC];
      ps_up_kernel<<<grid2(o1 - o0, B), TPB, 0, st>>>(ws->mars, ws->ld, B, p, c->up_all + o0, c->s_node, c->e_prime,
                                                     c->e_sub, ev->row_ids_dev, ev->row_start);
    }
    for (int64_t lay = c->L; lay >= 0; --lay) {
      const uint32_t o0 = c->h_down_all_off[lay], o1 = c->h_down_all_off[lay + 1];
      if (o1 == o0) continue;
      ++c->prof.launches[PCB_K_MISC];
      ps_down_kernel<<<grid2(o1 - o0, B), TPB, 0, st>>>(ws->flows, ws->mars, ws->ld, B, p, c->down_all + o0, c->N - 1,
                                                       c->in_off, c->in_ent, ev->row_ids_dev, ev->row_start);
    }
    ws->have_forward = true;
  }
  const bool quads = !ev->row_ids_dev && (ev->row_start - 1) % 4 == 0 && ev->num_rows % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(out_dev) & 15) == 0 && (!params_dev || (reinterpret_cast<uintptr_t>(params_dev) & 15) == 0);
  if (c->n_groups && quads) {
    ++c->prof.launches[PCB_K_MISC];
    norm_sum4_kernel<<<dim3(c->n_groups, (B + 4 * TPB - 1) / (4 * TPB)), TPB, 0, st>>>(
        ws->flows, ws->mars, ws->ld, B, p, c->grp_node, c->s_node, c->e_prime, c->e_sub, ev->row_start, out_dev, ev->num_rows);
  } else if (c->n_groups) {
    ++c->prof.launches[PCB_K_MISC];
    norm_sum_kernel<<<grid2(c->n_groups, B), TPB, 0, st>>>(ws->flows, ws->mars, ws->ld, B, p, c->grp_node, c->s_node,
                                                          c->e_prime, c->e_sub, ev->row_ids_dev, ev->row_start, out_dev,
                                                          ev->num_rows);
  }
  if (c->n_inputs) {
    ++c->prof.launches[PCB_K_MISC];
    norm_leaf_kernel<<<grid2(c->n_inputs, B), TPB, 0, st>>>(ws->flows, ws->ld, B, c->P, c->in_node, c->in_var, c->in_cats,
                                                           c->in_poff, ev->data_dev, ev->num_rows, ev->row_ids_dev,
                                                           ev->row_start, out_dev, ev->num_rows);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

extern "C" int32_t pcb_normalize_params(pcb_circuit* c, float* params_dev, uint32_t S, int32_t undo, pcb_stream s) {
  PCB_REQUIRE(c && params_dev, "null argument");
  PCB_REQUIRE(S >= 1, "no parameter sets");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t tpb = S >= TPB ? TPB : 32;
  const uint32_t gy = (S + tpb - 1) / tpb;
  if (c->n_inputs) {
    ++c->prof.launches[PCB_K_MISC];
    normalize_leaf_kernel<<<dim3(c->n_inputs, gy), tpb, 0, st>>>(params_dev, S, c->n_inputs, c->P, c->in_cats, c->in_poff, undo);
  }
  if (c->n_groups) {
    ++c->prof.launches[PCB_K_MISC];
    normalize_sum_kernel<<<dim3(c->n_groups, gy), tpb, 0, st>>>(params_dev, S, c->grp_node, c->s_node);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

extern "C" int32_t pcb_map_param_columns(float* dst_dev, const float* src_dev, uint32_t S, const uint32_t* ids_dst_dev,
                                         const uint32_t* ids_src_dev, uint32_t n, pcb_stream s) {
  PCB_REQUIRE(dst_dev && src_dev && (n == 0 || (ids_dst_dev && ids_src_dev)), "null argument");
  PCB_REQUIRE(S >= 1, "no parameter sets");
  if (n == 0) return PCB_OK;
  const uint32_t tpb = S >= TPB ? TPB : 32;
  map_columns_kernel<<<dim3(n, (S + tpb - 1) / tpb), tpb, 0, (cudaStream_t)s>>>(dst_dev, src_dev, S, ids_dst_dev, ids_src_dev);
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}
