// pcb_kld.cu — KLD between two parameterisations of one circuit, its gradient, and Adam.
//
// Reference kernels replaced (paths relative to VariationalJuice.jl/src):
//   kld_leaf_kernel      init_kld!_kernel + kl_div      queries/kld.jl:6-37, nodes/fixable_categorical_dist.jl:178-196
//   kld_up_kernel        kld_layer_up_kernel            queries/kld.jl:71-133
//   kld_down_kernel      kld_layer_down_logparam_kernel queries/kld.jl:212-320 (+ merge_params, misc.jl:710-754)
//   kld_leaf_grad_kernel input_kld_down_kernel          queries/kld.jl:502-547, fixable_categorical_dist.jl:215-221
//   adam_kernel + renorm apply_gradients / hard_update_params / update_params_adam
//                                                       sgd/adam.jl:63-127,218-242,314-315
//
// "Examples" here are parameter sets: params are [S, P] column-major, work matrices are
// [N][ldS].  Threads are laid out (set, node): blockDim.x covers sets, blockDim.y nodes, so a
// single parameter set still fills the block.
#include <algorithm>
#include <cstring>

#include "pcb_internal.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

#ifdef PCB_DIAG
// Diagnostic builds only: block 0 of every kernel of the chain stamps the global timer on entry,
// after the wait on the preceding launch and on exit.
__device__ unsigned long long g_kld_trace[3 * 256];
__device__ unsigned int g_kld_slot;
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define KLD_T_ENTER() unsigned int _slot = 0xffffffffu; \
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0) { _slot = atomicAdd(&g_kld_slot, 1u) & 255u; g_kld_trace[3 * _slot] = gtime(); }
#define KLD_T_WAITED() if (_slot != 0xffffffffu) g_kld_trace[3 * _slot + 1] = gtime();
#define KLD_T_EXIT() if (_slot != 0xffffffffu) g_kld_trace[3 * _slot + 2] = gtime();
#else
#define KLD_T_ENTER()
#define KLD_T_WAITED()
#define KLD_T_EXIT()
#endif

// Pins a value fetched ahead of griddepcontrol.wait: without a use in front of the wait the compiler
// is free to sink the load of read-only data below it, which puts the fetch back on the critical path.
__device__ __forceinline__ void keep(float& x) { asm volatile("" : "+f"(x)); }
__device__ __forceinline__ void keep(uint32_t& x) { asm volatile("" : "+r"(x)); }

struct Shape2 {
  dim3 block, grid;
};
// x = sets (power of two up to 32), y = items
Shape2 shape_for(uint32_t S, uint32_t items) {
  uint32_t bx = 1;
  while (bx < S && bx < 32) bx <<= 1;
  uint32_t by = 128 / bx;
  Shape2 s;
  s.block = dim3(bx, by, 1);
  s.grid = dim3((items + by - 1) / by, (S + bx - 1) / bx, 1);
  return s;
}

__global__ void kld_leaf_kernel(float* __restrict__ klds, uint32_t ld, uint32_t S, const float* __restrict__ p1,
                                const float* __restrict__ p2, uint32_t n_inputs, uint64_t P,
                                const uint32_t* __restrict__ in_node, const uint32_t* __restrict__ in_cats,
                                const uint64_t* __restrict__ in_poff, int* __restrict__ bump,
                                float* __restrict__ zero_grads, uint32_t N) {
  pcb_grid_dep_launch();   // the first layer above may fetch its static operands meanwhile
  KLD_T_ENTER();
  KLD_T_WAITED();
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (bump && i == 0 && s == 0) *bump += 1;   // the fused step counts its calls in a device word
  if (zero_grads && blockIdx.y == 0 && threadIdx.x == 0)   // the push pass of the fused step (one set) adds into these
    for (uint32_t k = i; k < N; k += gridDim.x * blockDim.y) zero_grads[(size_t)k * ld] = k == N - 1 ? 1.0f : 0.0f;
  if (i >= n_inputs || s >= S) return;
  float v = 0.0f;
  uint64_t po = in_poff[i];
  if (po < P) {  // learnable leaf; fixed leaves contribute 0
    uint32_t C = in_cats[i];
    for (uint32_t k = 0; k < C; ++k) {
      float a = p1[s + (size_t)S * (po + k)], b = p2[s + (size_t)S * (po + k)];
      v += expf(a) * (a - b);
    }
  }
  klds[(size_t)in_node[i] * ld + s] = v;
  KLD_T_EXIT();
}

__global__ void kld_up_kernel(float* __restrict__ klds, uint32_t ld, uint32_t S, const float* __restrict__ p1,
                              const float* __restrict__ p2, const uint32_t* __restrict__ nodes, uint32_t count,
                              const uint8_t* __restrict__ kind, const uint32_t* __restrict__ n_estart,
                              const uint32_t* __restrict__ n_ecount, const uint32_t* __restrict__ n_pid0,
                              const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= count || s >= S) return;
  uint32_t n = nodes[i];
  uint32_t e0 = n_estart[n], cnt = n_ecount[n];
  bool issum = kind[n] == PCB_SUM;
  uint32_t pid0 = n_pid0[n];
  float acc = 0.0f;
  for (uint32_t j = 0; j < cnt; ++j) {
    float k = klds[(size_t)e_prime[e0 + j] * ld + s];
    uint32_t sb = e_sub[e0 + j];
    if (sb != PCB_NONE) k += klds[(size_t)sb * ld + s];
    if (issum) {
      float a = p1[s + (size_t)S * (pid0 + j)], b = p2[s + (size_t)S * (pid0 + j)];
      k = expf(a) * (k + a - b);
    }
    acc += k;
  }
  klds[(size_t)n * ld + s] = acc;
}

// The same with one warp per (node, set): lanes over the node's edges.  With a handful of parameter
// sets the (set, node) layout above leaves every thread a serial loop over up to k edges; a layer
// of a single-set call then takes tens of microseconds instead of a few.  Such a call is a chain of
// short dependent launches, so everything that does not depend on the layer below (the edge lists,
// both parameters of the first 64 edges and exp of one) is fetched BEFORE the wait on the preceding
// launch; after it only the children's values are gathered.
constexpr int KLD_PRE = 2;   // edges per lane held across the wait
__global__ void kld_up_warp_kernel(float* __restrict__ klds, uint32_t ld, uint32_t S, const float* __restrict__ p1,
                                   const float* __restrict__ p2, const uint32_t* __restrict__ nodes, uint32_t count,
                                   const uint8_t* __restrict__ kind, const uint32_t* __restrict__ n_estart,
                                   const uint32_t* __restrict__ n_ecount, const uint32_t* __restrict__ n_pid0,
                                   const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub,
                                   uint32_t root, float* __restrict__ root_out) {
  pcb_grid_dep_launch();
  KLD_T_ENTER();
  const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= count * S) return;
  const uint32_t i = w / S, s = w % S;
  const uint32_t n = nodes[i];
  const uint32_t e0 = n_estart[n], cnt = n_ecount[n];
  const bool issum = kind[n] == PCB_SUM;
  const uint32_t pid0 = n_pid0[n];
  uint32_t pr[KLD_PRE], sb[KLD_PRE];
  float wgt[KLD_PRE], dif[KLD_PRE];
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const uint32_t j = lane + 32 * r;
    pr[r] = sb[r] = PCB_NONE; wgt[r] = 1.0f; dif[r] = 0.0f;
    if (j < cnt) {
      pr[r] = e_prime[e0 + j];
      sb[r] = e_sub[e0 + j];
      if (issum) {
        const float a = p1[s + (size_t)S * (pid0 + j)], b = p2[s + (size_t)S * (pid0 + j)];
        wgt[r] = expf(a);
        dif[r] = a - b;
      }
    }
    keep(pr[r]); keep(sb[r]); keep(wgt[r]); keep(dif[r]);
  }
  pcb_grid_dep_wait();   // everything above is static circuit data or this call's parameters
  KLD_T_WAITED();
  // all gathers of the held edges are issued back to back (an edge without a second child reads
  // the first one again), so the layer costs one round trip to L2, not one per operand
  float k0[KLD_PRE], k1[KLD_PRE];
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const uint32_t a0 = pr[r] != PCB_NONE ? pr[r] : n, a1 = sb[r] != PCB_NONE ? sb[r] : a0;
    k0[r] = klds[(size_t)a0 * ld + s];
    k1[r] = klds[(size_t)a1 * ld + s];
  }
  float acc = 0.0f;
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const float k = k0[r] + (sb[r] != PCB_NONE ? k1[r] : 0.0f);
    const float term = issum ? wgt[r] * (k + dif[r]) : k;
    acc += pr[r] != PCB_NONE ? term : 0.0f;
  }
  for (uint32_t j = lane + 32 * KLD_PRE; j < cnt; j += 32) {
    float k = klds[(size_t)e_prime[e0 + j] * ld + s];
    uint32_t sb2 = e_sub[e0 + j];
    if (sb2 != PCB_NONE) k += klds[(size_t)sb2 * ld + s];
    if (issum) {
      float a = p1[s + (size_t)S * (pid0 + j)], b = p2[s + (size_t)S * (pid0 + j)];
      k = expf(a) * (k + a - b);
    }
    acc += k;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    klds[(size_t)n * ld + s] = acc;
    if (root_out && n == root) root_out[s] = acc;
  }
  KLD_T_EXIT();
}

// edge_klds of sum and product edges in up-edge order, [E][ldS]-free: written straight to a
// [S, E] column-major buffer (parity accessor only)
__global__ void kld_edge_kernel(const float* __restrict__ klds, uint32_t ld, uint32_t S, const float* __restrict__ p1,
                                const float* __restrict__ p2, const uint32_t* __restrict__ nodes, uint32_t count,
                                const uint8_t* __restrict__ kind, const uint32_t* __restrict__ n_estart,
                                const uint32_t* __restrict__ n_ecount, const uint32_t* __restrict__ n_pid0,
                                const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub,
                                float* __restrict__ out) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= count || s >= S) return;
  uint32_t n = nodes[i];
  uint32_t e0 = n_estart[n], cnt = n_ecount[n];
  bool issum = kind[n] == PCB_SUM;
  uint32_t pid0 = n_pid0[n];
  for (uint32_t j = 0; j < cnt; ++j) {
    float k = klds[(size_t)e_prime[e0 + j] * ld + s];
    uint32_t sb = e_sub[e0 + j];
    if (sb != PCB_NONE) k += klds[(size_t)sb * ld + s];
    if (issum) {
      float a = p1[s + (size_t)S * (pid0 + j)], b = p2[s + (size_t)S * (pid0 + j)];
      k = expf(a) * (k + a - b);
    }
    out[s + (size_t)S * (e0 + j)] = k;
  }
}

// node gradients top-down (pull) + the two parameter gradients of every sum edge
__global__ void kld_down_kernel(float* __restrict__ grads, const float* __restrict__ klds, uint32_t ld, uint32_t S,
                                const float* __restrict__ p1, const float* __restrict__ p2,
                                const uint32_t* __restrict__ nodes, uint32_t count, uint32_t root,
                                const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                                float* __restrict__ g1, float* __restrict__ g2) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= count || s >= S) return;
  uint32_t n = nodes[i];
  uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  float acc = (i0 == i1 && n == root) ? 1.0f : 0.0f;
  float myk = klds[(size_t)n * ld + s];
  for (uint32_t x = i0; x < i1; ++x) {
    PcbInEntry en = in_ent[x];
    float pg = grads[(size_t)en.parent * ld + s];
    float eg = pg;
    if (en.pid != PCB_NONE) {
      float a = p1[s + (size_t)S * en.pid];
      float ea = expf(a);
      eg = pg * ea;
      if (en.flags & 1u) {
        float b = p2[s + (size_t)S * en.pid];
        float ck = myk + (en.sib != PCB_NONE ? klds[(size_t)en.sib * ld + s] : 0.0f);
        float edge_kld = ea * (ck + a - b);
        g1[s + (size_t)S * en.pid] = pg * (edge_kld + ea);
        g2[s + (size_t)S * en.pid] = -pg * ea;
      }
    }
    acc += eg;
  }
  grads[(size_t)n * ld + s] = acc;
}

// one warp per (node, set): lanes over the node's incoming edges; the entries and the parameters of
// the first 64 of them are fetched before the wait on the preceding launch.  g2 may be null (the
// fused step needs the gradient with respect to the first parameter set only).
__global__ void kld_down_warp_kernel(float* __restrict__ grads, const float* __restrict__ klds, uint32_t ld,
                                     uint32_t S, const float* __restrict__ p1, const float* __restrict__ p2,
                                     const uint32_t* __restrict__ nodes, uint32_t count, uint32_t root,
                                     const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                                     float* __restrict__ g1, float* __restrict__ g2) {
  pcb_grid_dep_launch();
  KLD_T_ENTER();
  const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= count * S) return;
  const uint32_t i = w / S, s = w % S;
  const uint32_t n = nodes[i];
  const uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  PcbInEntry en[KLD_PRE];
  float pa[KLD_PRE], pea[KLD_PRE], pb[KLD_PRE];
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const uint32_t x = i0 + lane + 32 * r;
    en[r].parent = en[r].sib = en[r].pid = PCB_NONE; en[r].flags = 0; pa[r] = pb[r] = 0.0f; pea[r] = 1.0f;
    if (x < i1) {
      en[r] = in_ent[x];
      if (en[r].pid != PCB_NONE) {
        pa[r] = p1[s + (size_t)S * en[r].pid];
        pea[r] = expf(pa[r]);
        if (en[r].flags & 1u) pb[r] = p2[s + (size_t)S * en[r].pid];
      }
    }
    keep(en[r].parent); keep(en[r].sib); keep(en[r].pid); keep(en[r].flags); keep(pa[r]); keep(pea[r]); keep(pb[r]);
  }
  pcb_grid_dep_wait();   // everything above is static circuit data or this call's parameters
  KLD_T_WAITED();
  // every gather of the held entries is issued before the first use: one round trip to L2
  const float myk = klds[(size_t)n * ld + s];
  float pg[KLD_PRE], sk[KLD_PRE];
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const uint32_t ap = en[r].parent != PCB_NONE ? en[r].parent : n;
    const uint32_t as = (g1 && en[r].sib != PCB_NONE) ? en[r].sib : n;
    pg[r] = grads[(size_t)ap * ld + s];
    sk[r] = klds[(size_t)as * ld + s];
  }
  float acc = 0.0f;
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    if (en[r].parent == PCB_NONE) continue;
    float eg = pg[r];
    if (en[r].pid != PCB_NONE) {
      eg = pg[r] * pea[r];
      if (g1 && (en[r].flags & 1u)) {
        const float ck = myk + (en[r].sib != PCB_NONE ? sk[r] : 0.0f);
        const float edge_kld = pea[r] * (ck + pa[r] - pb[r]);
        g1[s + (size_t)S * en[r].pid] = pg[r] * (edge_kld + pea[r]);
        if (g2) g2[s + (size_t)S * en[r].pid] = -pg[r] * pea[r];
      }
    }
    acc += eg;
  }
  for (uint32_t x = i0 + lane + 32 * KLD_PRE; x < i1; x += 32) {
    PcbInEntry e2 = in_ent[x];
    float pgx = grads[(size_t)e2.parent * ld + s];
    float eg = pgx;
    if (e2.pid != PCB_NONE) {
      float a = p1[s + (size_t)S * e2.pid];
      float ea = expf(a);
      eg = pgx * ea;
      if (g1 && (e2.flags & 1u)) {
        float b = p2[s + (size_t)S * e2.pid];
        float ck = myk + (e2.sib != PCB_NONE ? klds[(size_t)e2.sib * ld + s] : 0.0f);
        float edge_kld = ea * (ck + a - b);
        g1[s + (size_t)S * e2.pid] = pgx * (edge_kld + ea);
        if (g2) g2[s + (size_t)S * e2.pid] = -pgx * ea;
      }
    }
    acc += eg;
  }
  acc = warp_sum(acc);
  if (lane == 0) grads[(size_t)n * ld + s] = acc + ((i0 == i1 && n == root) ? 1.0f : 0.0f);
  KLD_T_EXIT();
}

__global__ void kld_leaf_grad_kernel(const float* __restrict__ grads, uint32_t ld, uint32_t S,
                                     const float* __restrict__ p1, const float* __restrict__ p2, uint32_t n_inputs,
                                     uint64_t P, const uint32_t* __restrict__ in_node,
                                     const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                     float* __restrict__ g1, float* __restrict__ g2) {
  pcb_grid_dep_launch();
  KLD_T_ENTER();
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n_inputs || s >= S) return;
  uint64_t po = in_poff[i];
  if (po >= P) return;
  const uint32_t node = in_node[i];
  uint32_t C = in_cats[i];
  uint32_t node_k = node;
  keep(node_k); keep(C);
  pcb_grid_dep_wait();
  KLD_T_WAITED();
  float g = grads[(size_t)node * ld + s];
  for (uint32_t k = 0; k < C; ++k) {
    float a = p1[s + (size_t)S * (po + k)], b = p2[s + (size_t)S * (po + k)];
    g1[s + (size_t)S * (po + k)] = g * (a - b + 1.0f);
    if (g2) g2[s + (size_t)S * (po + k)] = g * expf(a - b);  // plus sign, as the reference returns it for leaves
  }
  KLD_T_EXIT();
}

__global__ void copy_root_kernel(const float* __restrict__ klds_root, uint32_t S, float* __restrict__ out) {
  uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < S) out[s] = klds_root[s];
}

// t_dev != null: the step count comes from a device word (a replayed CUDA graph cannot take it as an
// argument) and the bias corrections 1 - beta^t are computed here
__global__ void adam_kernel(float* __restrict__ theta, const float* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, uint64_t n, float lr, float b1, float b2, float eps, float c1,
                            float c2, float sign, const int* __restrict__ t_dev) {
  if (t_dev) {
    const float t = (float)*t_dev;
    c1 = 1.0f - powf(b1, t);
    c2 = 1.0f - powf(b2, t);
  }
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float gi = g[i];
    float mi = b1 * m[i] + (1.0f - b1) * gi;
    float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    float m_hat = mi / c1, v_hat = vi / c2;
    theta[i] += sign * lr * (m_hat / (sqrtf(v_hat) + eps));
  }
}

// one warp per normalised group: sum groups first, then learnable leaves
__global__ void renorm_kernel(float* __restrict__ theta, uint32_t n_groups, const uint32_t* __restrict__ grp_node,
                              const uint32_t* __restrict__ n_pid0, const uint32_t* __restrict__ n_ecount,
                              uint32_t n_inputs, uint64_t P, const uint32_t* __restrict__ in_cats,
                              const uint64_t* __restrict__ in_poff) {
  uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint32_t lane = threadIdx.x & 31;
  uint64_t off;
  uint32_t cnt;
  if (w < n_groups) {
    uint32_t n = grp_node[w];
    off = n_pid0[n];
    cnt = n_ecount[n];
    if (cnt == 1) return;  // single-edge sum nodes are left alone (adam.jl:113)
  } else if (w < n_groups + n_inputs) {
    uint32_t i = w - n_groups;
    off = in_poff[i];
    cnt = in_cats[i];
    if (off >= P) return;
  } else {
    return;
  }
  float s = 0.0f;
  for (uint32_t j = lane; j < cnt; j += 32) s += expf(theta[off + j]);
  s = warp_sum(s);
  float ls = logf(s);
  for (uint32_t j = lane; j < cnt; j += 32) theta[off + j] -= ls;
}

}  // namespace

extern "C" int32_t pcb_kld(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev, const float* params2_dev,
                           uint32_t S, float* kld_out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && params1_dev && params2_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(S >= 1, "no parameter sets");
  PCB_CUDA(cudaSetDevice(c->device));
  int32_t st0 = pcb_ws_ensure_sets(ws, S, PCB_WS_NODES);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t ld = ws->ldS;
  if (c->n_inputs) {
    Shape2 sh = shape_for(S, c->n_inputs);
    ++c->prof.launches[PCB_K_KLD];
    kld_leaf_kernel<<<sh.grid, sh.block, 0, st>>>(ws->klds, ld, S, params1_dev, params2_dev, c->n_inputs, c->P,
                                                  c->in_node, c->in_cats, c->in_poff, ws->kld_bump,
                                                  ws->kld_bump ? ws->grads : nullptr, c->N);
  }
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    uint32_t o0 = c->h_up_all_off[lay - 1], o1 = c->h_up_all_off[lay];
    if (o1 == o0) continue;
    Shape2 sh = shape_for(S, o1 - o0);
    ++c->prof.launches[PCB_K_KLD];
    if (S <= 8) {
      PCB_CUDA(pcb_launch_pdl(kld_up_warp_kernel, dim3((uint32_t)(((uint64_t)(o1 - o0) * S + 7) / 8)), dim3(256), 0, st, c->pdl,
                              ws->klds, ld, S, params1_dev, params2_dev, c->up_all + o0, o1 - o0, c->kind, c->n_estart,
                              c->n_ecount, c->n_pid0, c->e_prime, c->e_sub, c->N - 1, kld_out_dev));
      continue;
    }
    kld_up_kernel<<<sh.grid, sh.block, 0, st>>>(ws->klds, ld, S, params1_dev, params2_dev, c->up_all + o0, o1 - o0,
                                                c->kind, c->n_estart, c->n_ecount, c->n_pid0, c->e_prime, c->e_sub);
  }
  if (kld_out_dev && (S > 8 || c->L == 0))   // the warp kernels write the root's value themselves
    ++c->prof.launches[PCB_K_KLD], copy_root_kernel<<<(S + 127) / 128, 128, 0, st>>>(ws->klds + (size_t)(c->N - 1) * ld, S, kld_out_dev);
  PCB_CUDA(cudaGetLastError());
  ws->have_kld = true;
  ws->kld_S = S;
  return PCB_OK;
}

extern "C" int32_t pcb_kld_backward(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev,
                                    const float* params2_dev, uint32_t S, float* grads1_dev, float* grads2_dev,
                                    pcb_stream s) {
  PCB_REQUIRE(c && ws && params1_dev && params2_dev && grads1_dev && grads2_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  if (!ws->have_kld || ws->kld_S != S)
    return pcb_fail(PCB_ERR_STATE, "pcb_kld_backward needs a preceding pcb_kld with the same number of sets");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t ld = ws->ldS;
  for (int64_t lay = c->L; lay >= 0; --lay) {
    uint32_t o0 = c->h_down_all_off[lay], o1 = c->h_down_all_off[lay + 1];
    if (o1 == o0) continue;
    Shape2 sh = shape_for(S, o1 - o0);
    ++c->prof.launches[PCB_K_KLD];
    if (S <= 8) {
      PCB_CUDA(pcb_launch_pdl(kld_down_warp_kernel, dim3((uint32_t)(((uint64_t)(o1 - o0) * S + 7) / 8)), dim3(256), 0, st, c->pdl,
                              ws->grads, (const float*)ws->klds, ld, S, params1_dev, params2_dev, c->down_all + o0, o1 - o0,
                              c->N - 1, c->in_off, c->in_ent, grads1_dev, grads2_dev));
      continue;
    }
    kld_down_kernel<<<sh.grid, sh.block, 0, st>>>(ws->grads, ws->klds, ld, S, params1_dev, params2_dev,
                                                  c->down_all + o0, o1 - o0, c->N - 1, c->in_off, c->in_ent,
                                                  grads1_dev, grads2_dev);
  }
  if (c->n_inputs) {
    Shape2 sh = shape_for(S, c->n_inputs);
    ++c->prof.launches[PCB_K_KLD];
    PCB_CUDA(pcb_launch_pdl(kld_leaf_grad_kernel, sh.grid, sh.block, 0, st, c->pdl && S <= 8, (const float*)ws->grads, ld, S,
                            params1_dev, params2_dev, c->n_inputs, c->P, c->in_node, c->in_cats, c->in_poff, grads1_dev,
                            grads2_dev));
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

// klds [S, N] of the last pcb_kld call, column-major.
extern "C" int32_t pcb_get_klds(pcb_circuit* c, pcb_workspace* ws, uint32_t S, float* klds_host) {
  PCB_REQUIRE(c && ws && klds_host, "null argument");
  PCB_REQUIRE(ws->have_kld && ws->kld_S == S, "no matching pcb_kld call");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_CUDA(cudaMemcpy2D(klds_host, S * sizeof(float), ws->klds, ws->ldS * sizeof(float), S * sizeof(float), c->N,
                        cudaMemcpyDeviceToHost));
  return PCB_OK;
}

extern "C" int32_t pcb_kld_edge_klds(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev,
                                     const float* params2_dev, uint32_t S, float* edge_klds_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && params1_dev && params2_dev && edge_klds_dev, "null argument");
  PCB_REQUIRE(ws->have_kld && ws->kld_S == S, "no matching pcb_kld call");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  uint32_t total = c->h_up_all_off[c->L];
  if (total) {
    Shape2 sh = shape_for(S, total);
    ++c->prof.launches[PCB_K_KLD];
    kld_edge_kernel<<<sh.grid, sh.block, 0, st>>>(ws->klds, ws->ldS, S, params1_dev, params2_dev, c->up_all, total,
                                                  c->kind, c->n_estart, c->n_ecount, c->n_pid0, c->e_prime, c->e_sub,
                                                  edge_klds_dev);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

extern "C" int32_t pcb_adam_step(pcb_circuit* c, float* theta_dev, const float* grad_dev, float* m_dev, float* v_dev,
                                 int32_t t, float lr, float beta1, float beta2, float eps, float sign, pcb_stream s) {
  PCB_REQUIRE(c && theta_dev && grad_dev && m_dev && v_dev, "null argument");
  PCB_REQUIRE(t >= 1, "Adam step count starts at 1");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  float c1 = 1.0f - powf(beta1, (float)t), c2 = 1.0f - powf(beta2, (float)t);
  if (c->P) {
    uint32_t blocks = (uint32_t)std::min<uint64_t>((c->P + 255) / 256, 148 * 16);
    ++c->prof.launches[PCB_K_KLD];
    adam_kernel<<<blocks, 256, 0, st>>>(theta_dev, grad_dev, m_dev, v_dev, c->P, lr, beta1, beta2, eps, c1, c2, sign, nullptr);
    uint32_t warps = c->n_groups + c->n_inputs;
    ++c->prof.launches[PCB_K_KLD];
    renorm_kernel<<<(warps + 7) / 8, 256, 0, st>>>(theta_dev, c->n_groups, c->grp_node, c->n_pid0, c->n_ecount,
                                                   c->n_inputs, c->P, c->in_cats, c->in_poff);
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

// ---- KLD + gradient + Adam as one unit --------------------------------------------------------------
// One step of the variational loop on a single parameter set q against p: kld (queries/kld.jl:164-206),
// kld_backward with respect to q (:593-649), Adam descent on q's log-parameters and the
// re-normalisation of every sum group and leaf (sgd/adam.jl:63-127,218-242).  A single parameter set
// has no batch dimension, so the step is a chain of ~2 L small launches: the second call with the same
// arguments captures the chain as a CUDA graph (the step count lives in a device word that the graph
// increments itself) and later calls replay it.
namespace {
__global__ void set_step_kernel(int* __restrict__ t, int value) { *t = value; }

// ---- the fused single-set step: node gradients pushed down by the parents -------------------------
// One warp per node of an up layer, layers from the root down: every parent of the node lies in a
// higher layer, so its gradient is complete.  A sum edge hands pg * exp(theta) to both children, a
// product edge hands pg.  Lanes run over the edges of the node, so the parameters are read
// contiguously (the pull form reads them with the stride of the fan-in).  The eight nodes of a block
// usually have the same children (up_same): their contributions are added in shared memory and reach
// memory as one atomic per child; otherwise every edge adds its own.  The sums are floating-point
// atomics, like the reference's CUDA.@atomic on partially owned nodes (queries/kld.jl:258-300): the
// order of the additions, and with it the last bits, can differ from run to run.
__global__ void __launch_bounds__(256) kld1_push_kernel(float* __restrict__ grads, const float* __restrict__ p1,
                                                        const uint32_t* __restrict__ nodes, uint32_t count,
                                                        const uint4* __restrict__ s_node,
                                                        const uint32_t* __restrict__ e_prime,
                                                        const uint32_t* __restrict__ e_sub,
                                                        const uint8_t* __restrict__ same_flags, uint32_t ld) {
  __shared__ float red[8][256];
  pcb_grid_dep_launch();
  KLD_T_ENTER();
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t i = blockIdx.x * 8 + warp;
  const bool valid = i < count;
  const uint32_t n = nodes[valid ? i : blockIdx.x * 8];
  const uint4 sn = s_node[n];                     // edge start, edge count, first parameter, kind | region << 2
  const uint32_t e0 = sn.x, cnt = sn.y, pid0 = sn.z;
  const bool issum = (sn.w & 3u) == PCB_SUM;
  const bool same = same_flags[blockIdx.x] != 0;   // then every warp of the block sees the same e0-relative children
  float wgt[KLD_PRE];
  uint32_t pr[KLD_PRE], sb[KLD_PRE];
#pragma unroll
  for (int r = 0; r < KLD_PRE; ++r) {
    const uint32_t j = lane + 32 * r;
    wgt[r] = 0.0f; pr[r] = sb[r] = PCB_NONE;
    if (j < cnt) {
      wgt[r] = issum ? expf(p1[pid0 + j]) : 1.0f;
      if (!same) { pr[r] = e_prime[e0 + j]; sb[r] = e_sub[e0 + j]; }
    }
    keep(wgt[r]); keep(pr[r]); keep(sb[r]);
  }
  // the threads that will add a column of the block: its two children
  uint32_t cpr = PCB_NONE, csb = PCB_NONE;
  if (same && threadIdx.x < cnt) { cpr = e_prime[e0 + threadIdx.x]; csb = e_sub[e0 + threadIdx.x]; }
  keep(cpr); keep(csb);
  pcb_grid_dep_wait();   // everything above is static circuit data or this call's parameters
  KLD_T_WAITED();
  const float pg = valid ? grads[(size_t)n * ld] : 0.0f;
  if (same) {
#pragma unroll
    for (int r = 0; r < KLD_PRE; ++r)
      if (lane + 32 * r < cnt) red[warp][lane + 32 * r] = pg * wgt[r];
    for (uint32_t j = lane + 32 * KLD_PRE; j < cnt; j += 32) red[warp][j] = pg * expf(p1[pid0 + j]);
    __syncthreads();
    if (threadIdx.x < cnt) {
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += red[w][threadIdx.x];
      atomicAdd(grads + (size_t)cpr * ld, v);
      if (csb != PCB_NONE) atomicAdd(grads + (size_t)csb * ld, v);
    }
  } else if (valid) {
#pragma unroll
    for (int r = 0; r < KLD_PRE; ++r)
      if (pr[r] != PCB_NONE) {
        atomicAdd(grads + (size_t)pr[r] * ld, pg * wgt[r]);
        if (sb[r] != PCB_NONE) atomicAdd(grads + (size_t)sb[r] * ld, pg * wgt[r]);
      }
    for (uint32_t j = lane + 32 * KLD_PRE; j < cnt; j += 32) {
      const float eg = issum ? pg * expf(p1[pid0 + j]) : pg;
      atomicAdd(grads + (size_t)e_prime[e0 + j] * ld, eg);
      if (e_sub[e0 + j] != PCB_NONE) atomicAdd(grads + (size_t)e_sub[e0 + j] * ld, eg);
    }
  }
  KLD_T_EXIT();
}

// Gradient with respect to q's log-parameters, Adam descent and the re-normalisation in one pass for
// the fused step.  The normalised groups partition the parameters: blocks [0, sum_blocks) take one
// warp per sum node, the blocks after them the leaves (one thread per leaf with up to four
// categories, else one warp per leaf).  A sum edge's gradient is pg * (exp(a) * (kld(children) + a - b)
// + exp(a)) (queries/kld.jl:258-300 with merge_params, misc.jl:710-754), a leaf parameter's is
// g * (a - b + 1) (kld.jl:502-547); neither is stored.  Both parameter sets, both moments and the edge
// lists are fetched before the wait on the push kernels; groups of up to 128 stay in registers
// between the update and the scaling.
struct AdamArgs {
  float* theta; const float* theta_p; const float* klds; const float* grads; float* m; float* v;
  float lr, b1, b2, eps;
  const int* t_dev;
  uint32_t n_groups, sum_blocks, n_inputs, leaf_thread_mode, ld;
  uint64_t P;
  const uint32_t* grp_node; const uint4* s_node; const uint32_t* e_prime; const uint32_t* e_sub;
  const uint32_t* in_node; const uint32_t* in_cats; const uint64_t* in_poff;
};

__device__ __forceinline__ void adam_update(float& thv, float& mv, float& vv, float gi, float lr, float b1, float b2,
                                            float eps, float c1, float c2) {
  mv = b1 * mv + (1.0f - b1) * gi;
  vv = b2 * vv + (1.0f - b2) * gi * gi;
  const float m_hat = mv / c1, v_hat = vv / c2;
  thv += -lr * (m_hat / (sqrtf(v_hat) + eps));
}

template <bool SUM>
__device__ __forceinline__ void adam_group_warp(const AdamArgs& a, uint32_t node, uint32_t e0, uint32_t cnt, uint64_t off,
                                                uint32_t lane) {
  constexpr int R = 4;
  const bool renorm = !(SUM && cnt == 1);   // single-edge sum nodes are left alone (adam.jl:113)
  float th[R], mi[R], vi[R], dif[R];
  uint32_t pr[R], sb[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t j = lane + 32 * r;
    th[r] = mi[r] = vi[r] = dif[r] = 0.0f; pr[r] = sb[r] = PCB_NONE;
    if (j < cnt) {
      th[r] = a.theta[off + j]; mi[r] = a.m[off + j]; vi[r] = a.v[off + j];
      dif[r] = th[r] - a.theta_p[off + j];
      if (SUM) { pr[r] = a.e_prime[e0 + j]; sb[r] = a.e_sub[e0 + j]; }
    }
    keep(th[r]); keep(mi[r]); keep(vi[r]); keep(dif[r]);
    if (SUM) { keep(pr[r]); keep(sb[r]); }
  }
  pcb_grid_dep_wait();
  const float t = (float)*a.t_dev;
  const float pg = a.grads[(size_t)node * a.ld];
  float ck[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {   // the children's values of a sum group, all gathers in flight at once
    ck[r] = 0.0f;
    if (SUM) {
      const uint32_t a0 = pr[r] != PCB_NONE ? pr[r] : node, a1 = sb[r] != PCB_NONE ? sb[r] : a0;
      const float k0 = a.klds[(size_t)a0 * a.ld], k1 = a.klds[(size_t)a1 * a.ld];
      ck[r] = k0 + (sb[r] != PCB_NONE ? k1 : 0.0f);
    }
  }
  const float c1 = 1.0f - powf(a.b1, t), c2 = 1.0f - powf(a.b2, t);
  auto grad_of = [&](float av, float d, float kids) {
    if (!SUM) return pg * (d + 1.0f);
    const float ea = expf(av);
    return pg * (ea * (kids + d) + ea);
  };
  float total = 0.0f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t j = lane + 32 * r;
    if (j < cnt) {
      adam_update(th[r], mi[r], vi[r], grad_of(th[r], dif[r], ck[r]), a.lr, a.b1, a.b2, a.eps, c1, c2);
      a.m[off + j] = mi[r];
      a.v[off + j] = vi[r];
      total += expf(th[r]);
    }
  }
  for (uint32_t j = lane + 32 * R; j < cnt; j += 32) {   // the rare wide group goes through memory
    float tv = a.theta[off + j], mv = a.m[off + j], vv = a.v[off + j];
    float kids = 0.0f;
    if (SUM) {
      kids = a.klds[(size_t)a.e_prime[e0 + j] * a.ld];
      if (a.e_sub[e0 + j] != PCB_NONE) kids += a.klds[(size_t)a.e_sub[e0 + j] * a.ld];
    }
    adam_update(tv, mv, vv, grad_of(tv, tv - a.theta_p[off + j], kids), a.lr, a.b1, a.b2, a.eps, c1, c2);
    a.m[off + j] = mv; a.v[off + j] = vv; a.theta[off + j] = tv;
    total += expf(tv);
  }
  total = warp_sum(total);
  const float ls = renorm ? logf(total) : 0.0f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t j = lane + 32 * r;
    if (j < cnt) a.theta[off + j] = th[r] - ls;
  }
  if (renorm)
    for (uint32_t j = lane + 32 * R; j < cnt; j += 32) a.theta[off + j] -= ls;
}

__global__ void __launch_bounds__(256) adam_renorm_kernel(AdamArgs a) {
  KLD_T_ENTER();
  const uint32_t lane = threadIdx.x & 31;
  if (blockIdx.x < a.sum_blocks) {
    const uint32_t w = (blockIdx.x * 256 + threadIdx.x) >> 5;
    if (w >= a.n_groups) return;
    const uint32_t node = a.grp_node[w];
    const uint4 sn = a.s_node[node];
    adam_group_warp<true>(a, node, sn.x, sn.y, sn.z, lane);
  } else if (!a.leaf_thread_mode) {
    const uint32_t i = ((blockIdx.x - a.sum_blocks) * 256 + threadIdx.x) >> 5;
    if (i >= a.n_inputs) return;
    const uint64_t off = a.in_poff[i];
    if (off >= a.P) return;
    adam_group_warp<false>(a, a.in_node[i], 0, a.in_cats[i], off, lane);
  } else {
    // leaves with up to four categories: one thread each
    const uint32_t i = (blockIdx.x - a.sum_blocks) * 256 + threadIdx.x;
    if (i >= a.n_inputs) return;
    const uint64_t off = a.in_poff[i];
    if (off >= a.P) return;
    const uint32_t C = a.in_cats[i], node = a.in_node[i];
    float th[4], mi[4], vi[4], dif[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      th[k] = mi[k] = vi[k] = dif[k] = 0.0f;
      if (k < C) {
        th[k] = a.theta[off + k]; mi[k] = a.m[off + k]; vi[k] = a.v[off + k];
        dif[k] = th[k] - a.theta_p[off + k];
      }
      keep(th[k]); keep(mi[k]); keep(vi[k]); keep(dif[k]);
    }
    pcb_grid_dep_wait();
    const float t = (float)*a.t_dev;
    const float g = a.grads[(size_t)node * a.ld];
    const float c1 = 1.0f - powf(a.b1, t), c2 = 1.0f - powf(a.b2, t);
    float total = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < C) {
        adam_update(th[k], mi[k], vi[k], g * (dif[k] + 1.0f), a.lr, a.b1, a.b2, a.eps, c1, c2);
        a.m[off + k] = mi[k];
        a.v[off + k] = vi[k];
        total += expf(th[k]);
      }
    const float ls = logf(total);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < C) a.theta[off + k] = th[k] - ls;
  }
  KLD_T_EXIT();
}
}

#ifdef PCB_DIAG
// diagnostic builds only: the stamps of the last 256 kernels of the chain and the slot counter
extern "C" int32_t pcb_debug_kld_trace(unsigned long long* out, unsigned int* slot, int reset) {
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_CUDA(cudaMemcpyFromSymbol(out, g_kld_trace, sizeof(unsigned long long) * 3 * 256));
  PCB_CUDA(cudaMemcpyFromSymbol(slot, g_kld_slot, sizeof(unsigned int)));
  if (reset) { unsigned int z = 0; PCB_CUDA(cudaMemcpyToSymbol(g_kld_slot, &z, sizeof(z))); }
  return PCB_OK;
}
#endif

static int32_t kld_adam_body(pcb_circuit* c, pcb_workspace* ws, float* theta_q, const float* theta_p, float* m_dev,
                             float* v_dev, float lr, float beta1, float beta2, float eps, float* kld_out, cudaStream_t st) {
  pcb_stream s = (pcb_stream)st;
  // the leaf kernel, first of the chain, counts the step and clears the node gradients
  ws->kld_bump = ws->kld_t_dev;
  int32_t r = pcb_kld(c, ws, theta_q, theta_p, 1, kld_out, s);
  ws->kld_bump = nullptr;
  if (r != PCB_OK) return r;
  for (int64_t lay = c->L; lay >= 1; --lay) {
    const uint32_t o0 = c->h_up_all_off[lay - 1], o1 = c->h_up_all_off[lay];
    if (o1 == o0) continue;
    ++c->prof.launches[PCB_K_KLD];
    PCB_CUDA(pcb_launch_pdl(kld1_push_kernel, dim3((o1 - o0 + 7) / 8), dim3(256), 0, st, c->pdl, ws->grads,
                            (const float*)theta_q, (const uint32_t*)(c->up_all + o0), o1 - o0, (const uint4*)c->s_node,
                            (const uint32_t*)c->e_prime, (const uint32_t*)c->e_sub,
                            (const uint8_t*)(c->up_same + c->h_up_chunk_off[lay - 1]), ws->ldS));
  }
  if (c->P) {
    AdamArgs a;
    a.theta = theta_q; a.theta_p = theta_p; a.klds = ws->klds; a.grads = ws->grads; a.m = m_dev; a.v = v_dev;
    a.lr = lr; a.b1 = beta1; a.b2 = beta2; a.eps = eps; a.t_dev = ws->kld_t_dev;
    a.n_groups = c->n_groups; a.sum_blocks = (c->n_groups + 7) / 8; a.n_inputs = c->n_inputs;
    a.leaf_thread_mode = c->max_cats <= 4; a.ld = ws->ldS; a.P = c->P;
    a.grp_node = c->grp_node; a.s_node = c->s_node; a.e_prime = c->e_prime; a.e_sub = c->e_sub;
    a.in_node = c->in_node; a.in_cats = c->in_cats; a.in_poff = c->in_poff;
    const uint32_t leaf_blocks = a.leaf_thread_mode ? (c->n_inputs + 255) / 256 : (c->n_inputs + 7) / 8;
    ++c->prof.launches[PCB_K_KLD];
    PCB_CUDA(pcb_launch_pdl(adam_renorm_kernel, dim3(a.sum_blocks + leaf_blocks), dim3(256), 0, st, c->pdl, a));
  }
  PCB_CUDA(cudaGetLastError());
  return PCB_OK;
}

extern "C" int32_t pcb_kld_adam_step(pcb_circuit* c, pcb_workspace* ws, float* theta_q_dev, const float* theta_p_dev,
                                     float* m_dev, float* v_dev, int32_t t, float lr, float beta1, float beta2,
                                     float eps, float* kld_out_dev, pcb_stream s) {
  PCB_REQUIRE(c && ws && theta_q_dev && theta_p_dev && m_dev && v_dev, "null argument");
  PCB_REQUIRE(ws->c == c, "workspace belongs to another circuit");
  PCB_REQUIRE(t >= 1, "Adam step count starts at 1");
  PCB_CUDA(cudaSetDevice(c->device));
  int32_t st0 = pcb_ws_ensure_sets(ws, 1, PCB_WS_NODES);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  if (!ws->kld_t_dev) {
    PCB_CUDA(cudaMalloc((void**)&ws->kld_t_dev, sizeof(int)));
    ws->kld_t_host = -1;
  }
  // the graph increments the device word itself; it is set from the host only when the caller's
  // count does not continue the last call's
  cudaStream_t gs = st;
  const bool legacy = st == nullptr || st == cudaStreamLegacy;
  if (legacy) {
    if (!c->gstream) {
      PCB_CUDA(cudaStreamCreateWithFlags(&c->gstream, cudaStreamNonBlocking));
      PCB_CUDA(cudaEventCreateWithFlags(&c->ev_g0, cudaEventDisableTiming));
      PCB_CUDA(cudaEventCreateWithFlags(&c->ev_g1, cudaEventDisableTiming));
    }
    gs = c->gstream;
    PCB_CUDA(cudaEventRecord(c->ev_g0, st));
    PCB_CUDA(cudaStreamWaitEvent(gs, c->ev_g0, 0));
  }
  auto leave = [&]() -> int32_t {
    if (legacy) { PCB_CUDA(cudaEventRecord(c->ev_g1, gs)); PCB_CUDA(cudaStreamWaitEvent(st, c->ev_g1, 0)); }
    return PCB_OK;
  };
  if (ws->kld_t_host != t - 1) set_step_kernel<<<1, 1, 0, gs>>>(ws->kld_t_dev, t - 1);
  ws->kld_t_host = t;

  pcb_workspace::KldKey key;
  memset(&key, 0, sizeof(key));
  key.q = theta_q_dev; key.p = theta_p_dev; key.m = m_dev; key.v = v_dev; key.out = kld_out_dev; key.stream = (void*)st;
  key.lr = lr; key.b1 = beta1; key.b2 = beta2; key.eps = eps;
  auto plain = [&]() -> int32_t {
    int32_t r = kld_adam_body(c, ws, theta_q_dev, theta_p_dev, m_dev, v_dev, lr, beta1, beta2, eps, kld_out_dev, gs);
    if (r != PCB_OK) return r;
    return leave();
  };
  if (!c->graph_enabled || c->prof.on) return plain();
  if (ws->kld_exec && !memcmp(&key, &ws->kld_exec_key, sizeof(key))) {
    PCB_CUDA(cudaGraphLaunch(ws->kld_exec, gs));
    for (int k = 0; k < PCB_K_COUNT; ++k) c->prof.launches[k] += ws->kld_launches[k];
    ws->have_kld = true; ws->kld_S = 1;
    return leave();
  }
  const bool capture = ws->have_kld_key && !memcmp(&key, &ws->kld_last_key, sizeof(key));
  ws->kld_last_key = key;
  ws->have_kld_key = true;
  if (!capture) return plain();
  if (ws->kld_exec) { cudaGraphExecDestroy(ws->kld_exec); ws->kld_exec = nullptr; }
  uint64_t before[PCB_K_COUNT];
  for (int k = 0; k < PCB_K_COUNT; ++k) before[k] = c->prof.launches[k];
  PCB_CUDA(cudaStreamBeginCapture(gs, cudaStreamCaptureModeRelaxed));
  int32_t body = kld_adam_body(c, ws, theta_q_dev, theta_p_dev, m_dev, v_dev, lr, beta1, beta2, eps, kld_out_dev, gs);
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(gs, &graph);
  if (body == PCB_OK && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&ws->kld_exec, graph, 0);
  if (graph) cudaGraphDestroy(graph);
  if (body != PCB_OK || ce != cudaSuccess || !ws->kld_exec) {
    ws->kld_exec = nullptr;
    cudaGetLastError();
    c->graph_enabled = false;   // this chain does not capture: stay with plain launches
    for (int k = 0; k < PCB_K_COUNT; ++k) c->prof.launches[k] = before[k];
    if (body != PCB_OK) return body;
    return plain();
  }
  for (int k = 0; k < PCB_K_COUNT; ++k) ws->kld_launches[k] = c->prof.launches[k] - before[k];
  ws->kld_exec_key = key;
  PCB_CUDA(cudaGraphLaunch(ws->kld_exec, gs));
  return leave();
}
