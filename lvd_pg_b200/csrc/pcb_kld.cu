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
                                const uint64_t* __restrict__ in_poff) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
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
// of a single-set call then takes tens of microseconds instead of a few.
__global__ void kld_up_warp_kernel(float* __restrict__ klds, uint32_t ld, uint32_t S, const float* __restrict__ p1,
                                   const float* __restrict__ p2, const uint32_t* __restrict__ nodes, uint32_t count,
                                   const uint8_t* __restrict__ kind, const uint32_t* __restrict__ n_estart,
                                   const uint32_t* __restrict__ n_ecount, const uint32_t* __restrict__ n_pid0,
                                   const uint32_t* __restrict__ e_prime, const uint32_t* __restrict__ e_sub) {
  pcb_grid_dep_launch();
  const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= count * S) return;
  const uint32_t i = w / S, s = w % S;
  const uint32_t n = nodes[i];
  const uint32_t e0 = n_estart[n], cnt = n_ecount[n];
  const bool issum = kind[n] == PCB_SUM;
  const uint32_t pid0 = n_pid0[n];
  pcb_grid_dep_wait();   // everything above is static circuit data
  float acc = 0.0f;
  for (uint32_t j = lane; j < cnt; j += 32) {
    float k = klds[(size_t)e_prime[e0 + j] * ld + s];
    uint32_t sb = e_sub[e0 + j];
    if (sb != PCB_NONE) k += klds[(size_t)sb * ld + s];
    if (issum) {
      float a = p1[s + (size_t)S * (pid0 + j)], b = p2[s + (size_t)S * (pid0 + j)];
      k = expf(a) * (k + a - b);
    }
    acc += k;
  }
  acc = warp_sum(acc);
  if (lane == 0) klds[(size_t)n * ld + s] = acc;
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

// one warp per (node, set): lanes over the node's incoming edges
__global__ void kld_down_warp_kernel(float* __restrict__ grads, const float* __restrict__ klds, uint32_t ld,
                                     uint32_t S, const float* __restrict__ p1, const float* __restrict__ p2,
                                     const uint32_t* __restrict__ nodes, uint32_t count, uint32_t root,
                                     const uint32_t* __restrict__ in_off, const PcbInEntry* __restrict__ in_ent,
                                     float* __restrict__ g1, float* __restrict__ g2) {
  pcb_grid_dep_launch();
  const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= count * S) return;
  const uint32_t i = w / S, s = w % S;
  const uint32_t n = nodes[i];
  const uint32_t i0 = in_off[n], i1 = in_off[n + 1];
  pcb_grid_dep_wait();   // everything above is static circuit data
  const float myk = klds[(size_t)n * ld + s];
  float acc = 0.0f;
  for (uint32_t x = i0 + lane; x < i1; x += 32) {
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
  acc = warp_sum(acc);
  if (lane == 0) grads[(size_t)n * ld + s] = acc + ((i0 == i1 && n == root) ? 1.0f : 0.0f);
}

__global__ void kld_leaf_grad_kernel(const float* __restrict__ grads, uint32_t ld, uint32_t S,
                                     const float* __restrict__ p1, const float* __restrict__ p2, uint32_t n_inputs,
                                     uint64_t P, const uint32_t* __restrict__ in_node,
                                     const uint32_t* __restrict__ in_cats, const uint64_t* __restrict__ in_poff,
                                     float* __restrict__ g1, float* __restrict__ g2) {
  uint32_t i = blockIdx.x * blockDim.y + threadIdx.y;
  uint32_t s = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n_inputs || s >= S) return;
  uint64_t po = in_poff[i];
  if (po >= P) return;
  float g = grads[(size_t)in_node[i] * ld + s];
  uint32_t C = in_cats[i];
  for (uint32_t k = 0; k < C; ++k) {
    float a = p1[s + (size_t)S * (po + k)], b = p2[s + (size_t)S * (po + k)];
    g1[s + (size_t)S * (po + k)] = g * (a - b + 1.0f);
    g2[s + (size_t)S * (po + k)] = g * expf(a - b);  // plus sign, as the reference returns it for leaves
  }
}

__global__ void copy_root_kernel(const float* __restrict__ klds_root, uint32_t S, float* __restrict__ out) {
  uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < S) out[s] = klds_root[s];
}

__global__ void bump_step_kernel(int* __restrict__ t) { *t += 1; }

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
  int32_t st0 = pcb_ws_ensure_sets(ws, S, false);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  const uint32_t ld = ws->ldS;
  if (c->n_inputs) {
    Shape2 sh = shape_for(S, c->n_inputs);
    ++c->prof.launches[PCB_K_KLD];
    kld_leaf_kernel<<<sh.grid, sh.block, 0, st>>>(ws->klds, ld, S, params1_dev, params2_dev, c->n_inputs, c->P,
                                                  c->in_node, c->in_cats, c->in_poff);
  }
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    uint32_t o0 = c->h_up_all_off[lay - 1], o1 = c->h_up_all_off[lay];
    if (o1 == o0) continue;
    Shape2 sh = shape_for(S, o1 - o0);
    ++c->prof.launches[PCB_K_KLD];
    if (S <= 8) {
      PCB_CUDA(pcb_launch_pdl(kld_up_warp_kernel, dim3((uint32_t)(((uint64_t)(o1 - o0) * S + 7) / 8)), dim3(256), 0, st, c->pdl,
                              ws->klds, ld, S, params1_dev, params2_dev, c->up_all + o0, o1 - o0, c->kind, c->n_estart,
                              c->n_ecount, c->n_pid0, c->e_prime, c->e_sub));
      continue;
    }
    kld_up_kernel<<<sh.grid, sh.block, 0, st>>>(ws->klds, ld, S, params1_dev, params2_dev, c->up_all + o0, o1 - o0,
                                                c->kind, c->n_estart, c->n_ecount, c->n_pid0, c->e_prime, c->e_sub);
  }
  if (kld_out_dev)
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
    kld_leaf_grad_kernel<<<sh.grid, sh.block, 0, st>>>(ws->grads, ld, S, params1_dev, params2_dev, c->n_inputs, c->P,
                                                       c->in_node, c->in_cats, c->in_poff, grads1_dev, grads2_dev);
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
}

static int32_t kld_adam_body(pcb_circuit* c, pcb_workspace* ws, float* theta_q, const float* theta_p, float* m_dev,
                             float* v_dev, float lr, float beta1, float beta2, float eps, float* kld_out, cudaStream_t st) {
  pcb_stream s = (pcb_stream)st;
  ++c->prof.launches[PCB_K_KLD];
  bump_step_kernel<<<1, 1, 0, st>>>(ws->kld_t_dev);
  int32_t r = pcb_kld(c, ws, theta_q, theta_p, 1, kld_out, s);
  if (r != PCB_OK) return r;
  r = pcb_kld_backward(c, ws, theta_q, theta_p, 1, ws->kld_g1, ws->kld_g2, s);
  if (r != PCB_OK) return r;
  if (c->P) {
    uint32_t blocks = (uint32_t)std::min<uint64_t>((c->P + 255) / 256, 148 * 16);
    ++c->prof.launches[PCB_K_KLD];
    adam_kernel<<<blocks, 256, 0, st>>>(theta_q, ws->kld_g1, m_dev, v_dev, c->P, lr, beta1, beta2, eps, 1.0f, 1.0f, -1.0f,
                                        ws->kld_t_dev);
    uint32_t warps = c->n_groups + c->n_inputs;
    ++c->prof.launches[PCB_K_KLD];
    renorm_kernel<<<(warps + 7) / 8, 256, 0, st>>>(theta_q, c->n_groups, c->grp_node, c->n_pid0, c->n_ecount, c->n_inputs,
                                                   c->P, c->in_cats, c->in_poff);
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
  int32_t st0 = pcb_ws_ensure_sets(ws, 1, false);
  if (st0 != PCB_OK) return st0;
  cudaStream_t st = (cudaStream_t)s;
  if (!ws->kld_g1) {
    PCB_CUDA(cudaMalloc((void**)&ws->kld_g1, std::max<uint64_t>(c->P, 1) * sizeof(float)));
    PCB_CUDA(cudaMalloc((void**)&ws->kld_g2, std::max<uint64_t>(c->P, 1) * sizeof(float)));
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
