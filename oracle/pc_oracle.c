/* pc_oracle.c — CPU restatement of the reference's probabilistic-circuit algorithms.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared
 * against and the timed CPU baseline of the benchmark; nothing in the product path
 * links, imports or calls it.
 *
 * It follows, function by function, the CUDA.jl kernels of VariationalJuice.jl
 * (paths relative to VariationalJuice.jl/src):
 *   forward      queries/likelihood.jl:4-68, regularization/reg_likelihood.jl:16-49
 *   backward     queries/flow.jl:8-106, regularization/reg_flow.jl:120-222
 *   leaf flows   regularization/reg_flow.jl:3-48, nodes/fixable_categorical_dist.jl:121-130
 *   EM update    pretrain/mini_batch_warmup.jl:4-17 (without its >1e-8 gate),
 *                sgd/adam.jl:27-37, regularization/reg_em.jl:136-168,
 *                nodes/fixable_categorical_dist.jl:223-260
 *   KLD          queries/kld.jl:6-133, nodes/fixable_categorical_dist.jl:178-196
 *   KLD backward queries/kld.jl:212-320,502-547, misc.jl:710-754
 *   Adam         sgd/adam.jl:63-127,218-242
 *   sampling     queries/sample.jl:8-148,233-296 (soft); its temperature->0 limit (hard)
 *   flat params  bits_circuit.jl:39-113, misc.jl:5-135
 *
 * Parity status: the part of the EM arithmetic that lives in the un-vendored,
 * un-pinned ProbabilisticCircuits.jl (add_pseudocount, aggr_node_flows, update_params,
 * logsumexp) is restated from the in-tree twins cited above -> that part is
 * "parity unpinned"; everything else is pinned by the identities and closed forms of
 * the reference's own unit tests (see tests/).
 *
 * The work is a loop over examples (OpenMP) with, per example, the reference's
 * per-edge loop in edge order.  Sums over examples (edge_aggr, leaf flows) are
 * accumulated in double and rounded once.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include "../include/pcb200.h"
#include "../include/pcb200_gumbel.h"

#define IDX(b, n, ld) ((size_t)(b) + (size_t)(ld) * (size_t)(n))

/* The EM path (forward, backward, leaf statistics, clear, M-step) is written over `real`.  The
 * default build has real = float and follows the reference's Float32 arithmetic; a second build
 * with -DORC_F64 has real = double and takes every matrix, the statistics and the parameter
 * arrays as double (the caller converts the same fp32 parameters), which gives the exact answer
 * that two fp32 implementations with different summation orders are both compared with. */
#ifdef ORC_F64
typedef double real;
#define REXP exp
#define RLOG log
#define RLOG1P log1p
#define RMAX fmax
#define RABS fabs
#else
typedef float real;
#define REXP expf
#define RLOG logf
#define RLOG1P log1pf
#define RMAX fmaxf
#define RABS fabsf
#endif
int orc_real_bytes(void) { return (int)sizeof(real); }

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

double orc_gumbel_key(float logp, float u) { return pcb_gumbel_key(logp, u); }
double orc_log(double x) { return pcb_log(x); }

/* ProbabilisticCircuits.logsumexp(x::Float32, y::Float32), the sum_agg_func of
 * queries/likelihood.jl:101-102. */
static inline real lse2(real x, real y) {
  if (isfinite(x) && isfinite(y)) return RMAX(x, y) + RLOG1P(REXP(-RABS(x - y)));
  return RMAX(x, y);
}

/* ------------------------------------------------------------------------------------ */
/* flat parameter maps, bits_circuit.jl:44-84 (all 1-based, 0 = none)                     */
/* ------------------------------------------------------------------------------------ */
static int edge_is_sum(const pcb_circuit_desc* d, uint32_t e0) {
  return d->node_kind[d->up_parent[e0] - 1] == PCB_SUM;
}
static int edge_first(const pcb_circuit_desc* d, uint32_t e0) {
  return e0 == 0 || d->up_parent[e0 - 1] != d->up_parent[e0];
}
static int edge_last(const pcb_circuit_desc* d, uint32_t e0) {
  return e0 + 1 == d->num_edges || d->up_parent[e0 + 1] != d->up_parent[e0];
}
static uint32_t leaf_nparams(const pcb_circuit_desc* d, uint32_t node0) {
  return d->node_fixed[node0] ? 0u : d->node_num_cats[node0];
}

void orc_counts(const pcb_circuit_desc* d, uint32_t* n_inner, uint32_t* n_input, uint32_t* n_groups) {
  uint32_t ni = 0, ng = 0, nl = 0;
  for (uint32_t e = 0; e < d->num_edges; ++e)
    if (edge_is_sum(d, e)) { ++ni; if (edge_last(d, e)) ++ng; }
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) nl += leaf_nparams(d, d->input_node_ids[i] - 1);
  *n_inner = ni; *n_input = nl; *n_groups = ng;
}

/* edge2param[E], param2edge[n_inner], param2group[n_inner], innode2ncumparam[n_in] */
void orc_meta(const pcb_circuit_desc* d, uint32_t* edge2param, uint32_t* param2edge,
              uint32_t* param2group, uint32_t* innode2ncumparam) {
  uint32_t pid = 1, grp = 1;
  for (uint32_t e = 0; e < d->num_edges; ++e) {
    if (edge_is_sum(d, e)) {
      if (edge2param) edge2param[e] = pid;
      if (param2edge) param2edge[pid - 1] = e + 1;
      if (param2group) param2group[pid - 1] = grp;
      ++pid;
      if (edge_last(d, e)) ++grp;
    } else if (edge2param) edge2param[e] = 0;
  }
  if (innode2ncumparam) {
    uint32_t cum = 0;
    for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
      cum += leaf_nparams(d, d->input_node_ids[i] - 1);
      innode2ncumparam[i] = cum;
    }
  }
}

/* vectorize_parameters, misc.jl:5-68 */
void orc_vectorize(const pcb_circuit_desc* d, const float* up_logp, const float* heap, float* params) {
  uint32_t pid = 0;
  for (uint32_t e = 0; e < d->num_edges; ++e)
    if (edge_is_sum(d, e)) params[pid++] = up_logp[e];
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1, np = leaf_nparams(d, n);
    for (uint32_t c = 0; c < np; ++c) params[pid++] = heap[d->node_heap_start[n] - 1 + c];
  }
}
/* update_parameters, misc.jl:73-135 */
void orc_update_parameters(const pcb_circuit_desc* d, float* up_logp, float* heap, const float* params) {
  uint32_t pid = 0;
  for (uint32_t e = 0; e < d->num_edges; ++e)
    if (edge_is_sum(d, e)) up_logp[e] = params[pid++];
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1, np = leaf_nparams(d, n);
    for (uint32_t c = 0; c < np; ++c) heap[d->node_heap_start[n] - 1 + c] = params[pid++];
  }
}

/* ------------------------------------------------------------------------------------ */
/* forward: init_mar! + layer_up over all layers                                          */
/* ------------------------------------------------------------------------------------ */
static inline int64_t data_row(const int32_t* row_ids, uint32_t row_start, uint32_t b) {
  return row_ids ? (int64_t)row_ids[b] - 1 : (int64_t)row_start - 1 + b;
}

/* mars [B, N] column-major (ld = B); edge_mars [B, E] or NULL */
/* Examples are processed in blocks of ORC_RB consecutive rows: the loop over the rows of a block is
 * the innermost one, so an edge's indices are read once per block and the rows of a node are
 * contiguous in memory.  Per example the sequence of operations is exactly the reference's
 * per-edge loop in edge order. */
#define ORC_RB 16
static uint32_t g_row_block = ORC_RB;
/* rows per block, 1 .. ORC_RB: a short batch timed on many threads takes smaller blocks */
void orc_set_row_block(int n) { g_row_block = n < 1 ? 1u : (n > ORC_RB ? (uint32_t)ORC_RB : (uint32_t)n); }

/* Leaf value of one example.
 *  - hard evidence, soft_reg = 0: the plain lookup (reg_likelihood.jl:4-14 reduces to it);
 *  - hard evidence, soft_reg > 0: soft_loglikelihood, reg_likelihood.jl:4-14 (window of `width`
 *    categories starting at max(0, x - width / 2), clipped at the last category);
 *  - soft evidence: per-category log-weights soft[row, var, c] ([rows, V, C] column-major), binary
 *    logsumexp fold in category order, init_mar!_with_reg_cat_kernel reg_likelihood.jl:51-91. */
static real leaf_value(const pcb_circuit_desc* d, const real* heap, uint32_t n, int64_t row, const uint8_t* data,
                       const uint8_t* miss, const float* soft, uint64_t num_rows, real soft_reg, int32_t width) {
  const uint32_t var0 = d->node_var[n] - 1, C = d->node_num_cats[n];
  const real* tab = heap + d->node_heap_start[n] - 1;
  if (soft) {
    real logp = -(real)INFINITY;
    for (uint32_t c = 0; c < C; ++c)
      logp = lse2(logp, (real)soft[(size_t)row + (size_t)num_rows * (var0 + (size_t)d->num_vars * c)] + tab[c]);
    return logp;
  }
  size_t di = (size_t)row + (size_t)num_rows * var0;
  if (miss && miss[di]) return (real)0;
  int32_t x = data[di];
  if (soft_reg == (real)0) return tab[x];
  int32_t c_start = x - width / 2 > 0 ? x - width / 2 : 0;
  int32_t c_end = c_start + width - 1 < (int32_t)C - 1 ? c_start + width - 1 : (int32_t)C - 1;
  real sp = (real)0;
  for (int32_t c = c_start; c <= c_end; ++c) sp += REXP(tab[c]);
  sp /= (real)(c_end - c_start + 1);
  return lse2(tab[x] + RLOG((real)1 - soft_reg), RLOG(sp) + RLOG(soft_reg));
}

void orc_forward_ex(const pcb_circuit_desc* d, const real* up_logp, const real* heap,
                    const uint8_t* data, const uint8_t* miss, const float* soft, uint64_t num_rows,
                    const int32_t* row_ids, uint32_t row_start, uint32_t B, real soft_reg, int32_t soft_reg_width,
                    real* mars, real* edge_mars);

void orc_forward(const pcb_circuit_desc* d, const real* up_logp, const real* heap,
                 const uint8_t* data, const uint8_t* miss, uint64_t num_rows,
                 const int32_t* row_ids, uint32_t row_start, uint32_t B, real* mars,
                 real* edge_mars) {
  orc_forward_ex(d, up_logp, heap, data, miss, NULL, num_rows, row_ids, row_start, B, (real)0, 1, mars, edge_mars);
}

void orc_forward_ex(const pcb_circuit_desc* d, const real* up_logp, const real* heap,
                    const uint8_t* data, const uint8_t* miss, const float* soft, uint64_t num_rows,
                    const int32_t* row_ids, uint32_t row_start, uint32_t B, real soft_reg, int32_t soft_reg_width,
                    real* mars, real* edge_mars) {
  const uint32_t N = d->num_nodes, E = d->num_edges, RB = g_row_block;
  const int64_t nblk = ((int64_t)B + RB - 1) / RB;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t blk = 0; blk < nblk; ++blk) {
    const uint32_t b0 = (uint32_t)(blk * RB);
    const uint32_t nb = B - b0 < RB ? B - b0 : RB;
    int64_t rows[ORC_RB];
    for (uint32_t j = 0; j < nb; ++j) rows[j] = data_row(row_ids, row_start, b0 + j);
    /* reg_likelihood.jl:26-46 (soft_reg = 0: the plain lookup) */
    for (uint32_t n = 0; n < N; ++n) {
      real* out = mars + IDX(b0, n, B);
      if (d->node_kind[n] == PCB_SUM) { for (uint32_t j = 0; j < nb; ++j) out[j] = -(real)INFINITY; }
      else if (d->node_kind[n] == PCB_PRODUCT) { for (uint32_t j = 0; j < nb; ++j) out[j] = (real)0; }
      else {
        for (uint32_t j = 0; j < nb; ++j)
          out[j] = leaf_value(d, heap, n, rows[j], data, miss, soft, num_rows, soft_reg, soft_reg_width);
      }
    }
    /* likelihood.jl:18-64, one thread owning every edge of the node */
    real acc[ORC_RB];
    for (uint32_t j = 0; j < ORC_RB; ++j) acc[j] = (real)0;
    for (uint32_t e = 0; e < E; ++e) {
      const int issum = edge_is_sum(d, e), first = edge_first(d, e);
      const real* pv = mars + IDX(b0, d->up_prime[e] - 1, B);
      const real* sv = d->up_sub[e] != 0 ? mars + IDX(b0, d->up_sub[e] - 1, B) : NULL;
      const real lp = issum ? up_logp[e] : (real)0;
      for (uint32_t j = 0; j < nb; ++j) {
        real child = pv[j];
        if (sv) child += sv[j];
        if (issum) child += lp;
        if (edge_mars) edge_mars[IDX(b0 + j, e, B)] = child;
        if (first) acc[j] = child;
        else if (issum) acc[j] = lse2(acc[j], child);
        else acc[j] += child;
      }
      if (edge_last(d, e)) {
        real* out = mars + IDX(b0, d->up_parent[e] - 1, B);
        for (uint32_t j = 0; j < nb; ++j) out[j] = acc[j];
      }
    }
  }
}

/* ------------------------------------------------------------------------------------ */
/* backward: flows_circuit / reg_flows_circuit                                            */
/* ------------------------------------------------------------------------------------ */
/* flows [B, N]; edge_flows [B, E] in up-edge order or NULL (flow.jl:70-71);
 * edge_aggr [E] in down-edge order, accumulated into (flow.jl:75-81), may be NULL.  The sum over
 * the examples of an edge is collected in one double per edge shared by all threads (one atomic
 * add per edge and block of rows) and rounded once at the end. */
void orc_backward_ex(const pcb_circuit_desc* d, const real* up_logp, const real* mars, uint32_t B,
                     real* flows, real* edge_flows, real* edge_aggr, const uint32_t* head_roots, uint32_t H,
                     const float* head_mask, uint64_t mask_rows, const int32_t* row_ids, uint32_t row_start);

void orc_backward(const pcb_circuit_desc* d, const real* up_logp, const real* mars, uint32_t B,
                  real* flows, real* edge_flows, real* edge_aggr) {
  orc_backward_ex(d, up_logp, mars, B, flows, edge_flows, edge_aggr, NULL, 0, NULL, 0, NULL, 1);
}

/* With head_roots / head_mask the circuit has several roots under a fake root sum (the last node):
 * the flow of root h starts at head_mask[row, h] ([rows, H] column-major), every other node at 0
 * (src-jl/multi_head_pc/flow.jl:141-176), and the fake root's edges — tagged with the user bit by
 * the builder, bit_circuit.jl:22-34 — are skipped (flow.jl:45). */
void orc_backward_ex(const pcb_circuit_desc* d, const real* up_logp, const real* mars, uint32_t B,
                     real* flows, real* edge_flows, real* edge_aggr, const uint32_t* head_roots, uint32_t H,
                     const float* head_mask, uint64_t mask_rows, const int32_t* row_ids, uint32_t row_start) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  double* part = edge_aggr ? (double*)calloc((size_t)E, sizeof(double)) : NULL;
  const uint32_t RB = g_row_block;
  const int64_t nblk = ((int64_t)B + RB - 1) / RB;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t blk = 0; blk < nblk; ++blk) {
    const uint32_t b0 = (uint32_t)(blk * RB);
    const uint32_t nb = B - b0 < RB ? B - b0 : RB;
    for (uint32_t n = 0; n < N; ++n) { /* flow.jl:140-143 */
      real* f = flows + IDX(b0, n, B);
      const real init = (n == N - 1 && !head_mask) ? (real)1 : (real)0;
      for (uint32_t j = 0; j < nb; ++j) f[j] = init;
    }
    if (head_mask)
      for (uint32_t h = 0; h < H; ++h) {
        real* f = flows + IDX(b0, head_roots[h] - 1, B);
        for (uint32_t j = 0; j < nb; ++j)
          f[j] = (real)head_mask[(size_t)data_row(row_ids, row_start, b0 + j) + (size_t)mask_rows * h];
      }
    for (uint32_t de = 0; de < E; ++de) {
      const uint32_t e = d->down2up[de] - 1;
      const uint32_t parent = d->up_parent[e] - 1, prime = d->up_prime[e] - 1, sub = d->up_sub[e];
      const int issum = edge_is_sum(d, e);
      if (H > 0 && d->up_tag && (d->up_tag[e] & PCB_TAG_USER)) {   /* skipped edge: contributes nothing */
        if (edge_flows) for (uint32_t j = 0; j < nb; ++j) edge_flows[IDX(b0 + j, e, B)] = (real)0;
        continue;
      }
      const real* fp = flows + IDX(b0, parent, B);
      const real* mp = mars + IDX(b0, parent, B);
      const real* mc = mars + IDX(b0, prime, B);
      const real* ms = sub != 0 ? mars + IDX(b0, sub - 1, B) : NULL;
      real* fc = flows + IDX(b0, prime, B);
      real* fs = sub != 0 ? flows + IDX(b0, sub - 1, B) : NULL;
      double tot = 0.0;
      for (uint32_t j = 0; j < nb; ++j) {
        real ef = fp[j];
        if (issum) { /* flow.jl:53-60 */
          real child = mc[j] + up_logp[e];
          if (ms) child += ms[j];
          ef = ef * REXP(child - mp[j]);
        }
        if (fs) fs[j] += ef;
        if (edge_flows) edge_flows[IDX(b0 + j, e, B)] = ef;
        tot += (double)ef;
        fc[j] += ef;
      }
      if (part) {
#pragma omp atomic
        part[de] += tot;
      }
    }
  }
  if (edge_aggr) {
    for (uint32_t de = 0; de < E; ++de) edge_aggr[de] = (real)((double)edge_aggr[de] + part[de]);
    free(part);
  }
}

/* input_flows_circuit_with_reg_kernel (reg_flow.jl:24-48) with soft_reg = 0, i.e. the plain
 * flow() of fixable_categorical_dist.jl:121-130.  weights is per data row or NULL. */
void orc_input_flows(const pcb_circuit_desc* d, real* heap, const real* flows,
                     const uint8_t* data, const uint8_t* miss, uint64_t num_rows,
                     const int32_t* row_ids, uint32_t row_start, uint32_t B, const real* weights) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t i = 0; i < (int64_t)d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1;
    if (d->node_fixed[n]) continue;
    uint32_t C = d->node_num_cats[n];
    size_t hs = d->node_heap_start[n] - 1;
    double* acc = (double*)calloc(C + 1, sizeof(double));
    for (uint32_t b = 0; b < B; ++b) {
      int64_t row = data_row(row_ids, row_start, b);
      real f = flows[IDX(b, n, B)];
      if (weights) f *= weights[row];
      size_t di = (size_t)row + (size_t)num_rows * (d->node_var[n] - 1);
      if (miss && miss[di]) acc[C] += (double)f;
      else acc[data[di]] += (double)f;
    }
    for (uint32_t c = 0; c <= C; ++c) heap[hs + C + c] = (real)((double)heap[hs + C + c] + acc[c]);
    free(acc);
  }
}

/* extract_lls_from_root_nodes (src-jl/multi_head_pc/bit_circuit.jl:95-109): with a head mask
 * lls[b] = logsumexp_h(mars[b, root_h] + log mask[row, h]) - log sum_h mask[row, h]; without one
 * lls is [B, H] with the roots' values. */
void orc_multihead_lls(const pcb_circuit_desc* d, const real* mars, uint32_t B, const uint32_t* head_roots,
                       uint32_t H, const float* head_mask, uint64_t mask_rows, const int32_t* row_ids,
                       uint32_t row_start, real* lls) {
  (void)d;
  for (uint32_t b = 0; b < B; ++b) {
    if (!head_mask) {
      for (uint32_t h = 0; h < H; ++h) lls[IDX(b, h, B)] = mars[IDX(b, head_roots[h] - 1, B)];
      continue;
    }
    int64_t row = data_row(row_ids, row_start, b);
    real acc = -(real)INFINITY, tot = (real)0;
    for (uint32_t h = 0; h < H; ++h) {
      real m = (real)head_mask[(size_t)row + (size_t)mask_rows * h];
      acc = lse2(acc, mars[IDX(b, head_roots[h] - 1, B)] + RLOG(m));
      tot += m;
    }
    lls[b] = acc - RLOG(tot);
  }
}

/* Leaf statistics for soft evidence (input_flows_circuit_with_reg_cat_kernel, reg_flow.jl:50-82:
 * slot c += exp(soft[row, var, c] + logp_c - logp) * flow) and for hard evidence with soft_reg > 0
 * (soft_flow, reg_flow.jl:3-22 — which mixes the heap's LOG-probabilities where probabilities would
 * be expected; restated as written). */
void orc_input_flows_ex(const pcb_circuit_desc* d, real* heap, const real* flows,
                        const uint8_t* data, const uint8_t* miss, const float* soft, uint64_t num_rows,
                        const int32_t* row_ids, uint32_t row_start, uint32_t B, const real* weights,
                        real soft_reg, int32_t width) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t i = 0; i < (int64_t)d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1;
    if (d->node_fixed[n]) continue;
    const uint32_t C = d->node_num_cats[n], var0 = d->node_var[n] - 1;
    size_t hs = d->node_heap_start[n] - 1;
    double* acc = (double*)calloc(C + 1, sizeof(double));
    for (uint32_t b = 0; b < B; ++b) {
      int64_t row = data_row(row_ids, row_start, b);
      real f = flows[IDX(b, n, B)];
      if (weights) f *= weights[row];
      if (soft) {
        real logp = -(real)INFINITY;
        for (uint32_t c = 0; c < C; ++c)
          logp = lse2(logp, (real)soft[(size_t)row + (size_t)num_rows * (var0 + (size_t)d->num_vars * c)] + heap[hs + c]);
        for (uint32_t c = 0; c < C; ++c)
          acc[c] += (double)(REXP((real)soft[(size_t)row + (size_t)num_rows * (var0 + (size_t)d->num_vars * c)] + heap[hs + c] - logp) * f);
        continue;
      }
      size_t di = (size_t)row + (size_t)num_rows * var0;
      if (miss && miss[di]) { acc[C] += (double)f; continue; }
      int32_t x = data[di];
      if (soft_reg == (real)0) { acc[x] += (double)f; continue; }
      int32_t c_start = x - width / 2 > 0 ? x - width / 2 : 0;
      int32_t c_end = c_start + width - 1 < (int32_t)C - 1 ? c_start + width - 1 : (int32_t)C - 1;
      real sp = (real)0;
      for (int32_t c = c_start; c <= c_end; ++c) sp += REXP(heap[hs + c]);
      sp /= (real)(c_end - c_start + 1);
      real base = ((real)1 - soft_reg) * heap[hs + x] + soft_reg * sp;
      acc[x] += (double)(((real)1 - soft_reg) * heap[hs + x] * f / base);
      for (int32_t c = c_start; c <= c_end; ++c)
        acc[c] += (double)(soft_reg / (real)(c_end - c_start + 1) * heap[hs + c] * f / base);
    }
    for (uint32_t c = 0; c <= C; ++c) heap[hs + C + c] = (real)((double)heap[hs + C + c] + acc[c]);
    free(acc);
  }
}

/* edge_aggr .*= rate ; clear_memory(d, heap, rate) (fixable_categorical_dist.jl:250-260) */
void orc_clear_flows(const pcb_circuit_desc* d, real* edge_aggr, real* heap, real rate) {
  if (edge_aggr) for (uint32_t e = 0; e < d->num_edges; ++e) edge_aggr[e] = (rate == (real)0) ? (real)0 : edge_aggr[e] * rate;
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1;
    if (d->node_fixed[n]) continue;
    uint32_t C = d->node_num_cats[n];
    size_t hs = d->node_heap_start[n] - 1;
    for (uint32_t c = 0; c <= C; ++c) heap[hs + C + c] = (rate == (real)0) ? (real)0 : heap[hs + C + c] * rate;
  }
}

/* M-step.  edge_aggr is in down-edge order and is modified (pseudocount added), as the
 * reference does.  up_logp is updated in place (the reference writes both edge copies). */
void orc_em_update(const pcb_circuit_desc* d, real* up_logp, real* edge_aggr, real* heap,
                   real pseudocount, real inertia) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  real* node_aggr = (real*)calloc(N, sizeof(real));
  /* count_siblings + add_pseudocount (mini_batch_warmup.jl:4-23, gate removed) */
  for (uint32_t e = 0; e < E; ++e)
    if (edge_is_sum(d, e)) node_aggr[d->up_parent[e] - 1] += (real)1;
#pragma omp parallel for schedule(static)
  for (int64_t de = 0; de < (int64_t)E; ++de) {
    uint32_t e = d->down2up[de] - 1;
    if (edge_is_sum(d, e)) edge_aggr[de] += pseudocount / node_aggr[d->up_parent[e] - 1];
  }
  /* aggr_node_flows (adam.jl:30-36) */
  memset(node_aggr, 0, N * sizeof(real));
  {
    double* na = (double*)calloc(N, sizeof(double));
#pragma omp parallel for schedule(static)
    for (int64_t de = 0; de < (int64_t)E; ++de) {
      uint32_t e = d->down2up[de] - 1;
      if (edge_is_sum(d, e)) {
#pragma omp atomic
        na[d->up_parent[e] - 1] += (double)edge_aggr[de];
      }
    }
    for (uint32_t n = 0; n < N; ++n) node_aggr[n] = (real)na[n];
    free(na);
  }
  /* update_params (reg_em.jl:136-168 / mini_batch_warmup.jl:39-76 without the gate) */
#pragma omp parallel for schedule(static)
  for (int64_t de = 0; de < (int64_t)E; ++de) {
    uint32_t e = d->down2up[de] - 1;
    if (!edge_is_sum(d, e)) continue;
    if (edge_first(d, e) && edge_last(d, e)) continue;
    real oldv = inertia * REXP(up_logp[e]);
    real newv = ((real)1 - inertia) * edge_aggr[de] / node_aggr[d->up_parent[e] - 1];
    up_logp[e] = RLOG(oldv + newv);
  }
  free(node_aggr);
  /* update_input_node_params (fixable_categorical_dist.jl:223-248) */
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t i = 0; i < (int64_t)d->num_input_nodes; ++i) {
    uint32_t n = d->input_node_ids[i] - 1;
    if (d->node_fixed[n]) continue;
    uint32_t C = d->node_num_cats[n];
    size_t hs = d->node_heap_start[n] - 1;
    real node_flow = (real)0, cat_pc = pseudocount / (real)C;
    for (uint32_t c = 0; c < C; ++c) node_flow += heap[hs + C + c];
    real missing_flow = heap[hs + 2 * C];
    node_flow += missing_flow + pseudocount;
    for (uint32_t c = 0; c < C; ++c) {
      real oldp = REXP(heap[hs + c]);
      real oldv = inertia * oldp;
      real newv = ((real)1 - inertia) * (heap[hs + C + c] + cat_pc + missing_flow * oldp) / node_flow;
      heap[hs + c] = RLOG(oldv + newv);
    }
  }
}

/* ------------------------------------------------------------------------------------ */
/* KLD                                                                                    */
/* ------------------------------------------------------------------------------------ */
/* params1/2 [S, P] column-major; klds [S, N]; edge_klds [S, E] (up-edge order) */
void orc_kld(const pcb_circuit_desc* d, const float* params1, const float* params2, uint32_t S,
             float* klds, float* edge_klds) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  uint32_t n_inner, n_input, n_groups;
  orc_counts(d, &n_inner, &n_input, &n_groups);
  uint32_t* edge2param = (uint32_t*)malloc(sizeof(uint32_t) * (E ? E : 1));
  uint32_t* cum = (uint32_t*)malloc(sizeof(uint32_t) * (d->num_input_nodes ? d->num_input_nodes : 1));
  uint32_t* node2input = (uint32_t*)calloc(N, sizeof(uint32_t));
  orc_meta(d, edge2param, NULL, NULL, cum);
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) node2input[d->input_node_ids[i] - 1] = i + 1;
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < (int64_t)S; ++s) {
    /* init_kld! (kld.jl:17-35) + kl_div (fixable_categorical_dist.jl:178-196, norm_params=false) */
    for (uint32_t n = 0; n < N; ++n) {
      float v = 0.0f;
      if (d->node_kind[n] == PCB_INPUT && !d->node_fixed[n]) {
        uint32_t i = node2input[n] - 1, np = d->node_num_cats[n];
        size_t start = (size_t)n_inner + cum[i] - np; /* 0-based first param */
        for (uint32_t c = 0; c < np; ++c) {
          float p1 = params1[IDX(s, start + c, S)], p2 = params2[IDX(s, start + c, S)];
          v += expf(p1) * (p1 - p2);
        }
      }
      klds[IDX(s, n, S)] = v;
    }
    /* kld_layer_up_kernel (kld.jl:86-130) */
    float acc = 0.0f;
    for (uint32_t e = 0; e < E; ++e) {
      float k = klds[IDX(s, d->up_prime[e] - 1, S)];
      if (d->up_sub[e] != 0) k += klds[IDX(s, d->up_sub[e] - 1, S)];
      if (edge_is_sum(d, e)) {
        float p1 = params1[IDX(s, edge2param[e] - 1, S)], p2 = params2[IDX(s, edge2param[e] - 1, S)];
        k = expf(p1) * (k + p1 - p2);
      }
      if (edge_klds) edge_klds[IDX(s, e, S)] = k;
      if (edge_first(d, e)) acc = k; else acc += k;
      if (edge_last(d, e)) klds[IDX(s, d->up_parent[e] - 1, S)] = acc;
    }
  }
  free(edge2param); free(cum); free(node2input);
}

/* kld_backward_inner + input_kld_down + merge_params.  grads [S, N] node gradients;
 * edge_grads1/2 [S, E] up-edge order (may be NULL); param_grads1/2 [S, P].
 * The leaf gradient pair is (g*(p1-p2+1), +g*exp(p1-p2)) — the reference returns the second
 * element with a plus sign for leaves and a minus sign for inner edges; mirrored here. */
void orc_kld_backward(const pcb_circuit_desc* d, const float* params1, const float* params2,
                      uint32_t S, const float* klds, const float* edge_klds, float* grads,
                      float* edge_grads1, float* edge_grads2, float* param_grads1,
                      float* param_grads2) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  (void)klds;
  uint32_t n_inner, n_input, n_groups;
  orc_counts(d, &n_inner, &n_input, &n_groups);
  uint32_t* edge2param = (uint32_t*)malloc(sizeof(uint32_t) * (E ? E : 1));
  uint32_t* cum = (uint32_t*)malloc(sizeof(uint32_t) * (d->num_input_nodes ? d->num_input_nodes : 1));
  orc_meta(d, edge2param, NULL, NULL, cum);
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < (int64_t)S; ++s) {
    for (uint32_t n = 0; n < N; ++n) grads[IDX(s, n, S)] = 0.0f; /* kld.jl:476-479 */
    grads[IDX(s, N - 1, S)] = 1.0f;
    for (uint32_t de = 0; de < E; ++de) { /* kld.jl:236-316 */
      uint32_t e = d->down2up[de] - 1;
      uint32_t parent = d->up_parent[e] - 1, prime = d->up_prime[e] - 1, sub = d->up_sub[e];
      float par_grad = grads[IDX(s, parent, S)], edge_grad = par_grad, g1 = 0.0f, g2 = 0.0f;
      if (edge_is_sum(d, e)) {
        float logp1 = params1[IDX(s, edge2param[e] - 1, S)];
        float p1 = expf(logp1);
        float edge_kld = edge_klds[IDX(s, e, S)];
        edge_grad = edge_grad * p1;
        g1 = par_grad * (edge_kld + p1);
        g2 = -par_grad * p1;
        param_grads1[IDX(s, edge2param[e] - 1, S)] = g1; /* merge_params, misc.jl:710-730 */
        param_grads2[IDX(s, edge2param[e] - 1, S)] = g2;
      }
      if (edge_grads1) edge_grads1[IDX(s, e, S)] = g1;
      if (edge_grads2) edge_grads2[IDX(s, e, S)] = g2;
      if (sub != 0) grads[IDX(s, sub - 1, S)] += edge_grad;
      grads[IDX(s, prime, S)] += edge_grad;
    }
    for (uint32_t i = 0; i < d->num_input_nodes; ++i) { /* kld.jl:515-543 */
      uint32_t n = d->input_node_ids[i] - 1, np = leaf_nparams(d, n);
      float g = grads[IDX(s, n, S)];
      size_t start = (size_t)n_inner + cum[i] - np;
      for (uint32_t c = 0; c < np; ++c) {
        float p1 = params1[IDX(s, start + c, S)], p2 = params2[IDX(s, start + c, S)];
        param_grads1[IDX(s, start + c, S)] = g * (p1 - p2 + 1.0f);
        param_grads2[IDX(s, start + c, S)] = g * expf(p1 - p2);
      }
    }
  }
  free(edge2param); free(cum);
}

/* ------------------------------------------------------------------------------------ */
/* Adam + renormalise (sgd/adam.jl:63-75, 88-127, 218-242, 314-315)                       */
/* ------------------------------------------------------------------------------------ */
void orc_adam_step(const pcb_circuit_desc* d, float* theta, const float* grad, float* m, float* v,
                   int32_t t, float lr, float beta1, float beta2, float eps, float sign) {
  uint32_t n_inner, n_input, n_groups;
  orc_counts(d, &n_inner, &n_input, &n_groups);
  size_t P = (size_t)n_inner + n_input;
  float c1 = 1.0f - powf(beta1, (float)t), c2 = 1.0f - powf(beta2, (float)t);
  for (size_t i = 0; i < P; ++i) {
    m[i] = beta1 * m[i] + (1.0f - beta1) * grad[i];
    v[i] = beta2 * v[i] + (1.0f - beta2) * grad[i] * grad[i];
    float m_hat = m[i] / c1, v_hat = v[i] / c2;
    theta[i] += sign * lr * (m_hat / (sqrtf(v_hat) + eps));
  }
  /* hard_update_params: logp <- theta - log sum exp(theta) per sum node, and per leaf */
  size_t pid = 0;
  uint32_t e = 0;
  while (e < d->num_edges) {
    if (!edge_is_sum(d, e)) { ++e; continue; }
    uint32_t e1 = e;
    while (!edge_last(d, e1)) ++e1;
    uint32_t deg = e1 - e + 1;
    float sum = 0.0f;
    for (uint32_t j = 0; j < deg; ++j) sum += expf(theta[pid + j]);
    if (deg > 1) { float ls = logf(sum); for (uint32_t j = 0; j < deg; ++j) theta[pid + j] -= ls; }
    pid += deg; e = e1 + 1;
  }
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
    uint32_t np = leaf_nparams(d, d->input_node_ids[i] - 1);
    if (!np) continue;
    float sum = 0.0f;
    for (uint32_t c = 0; c < np; ++c) sum += expf(theta[pid + c]);
    float ls = logf(sum);
    for (uint32_t c = 0; c < np; ++c) theta[pid + c] -= ls;
    pid += np;
  }
}

/* ------------------------------------------------------------------------------------ */
/* sum regions: sum nodes with identical scope share one region id (1-based, numbered by  */
/* first appearance in node order).  Scope signatures add up over products.               */
/* ------------------------------------------------------------------------------------ */
void orc_sum_regions(const pcb_circuit_desc* d, uint32_t* node_region, uint32_t* num_regions) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  uint64_t* sig = (uint64_t*)calloc(N, sizeof(uint64_t));
  uint8_t* seen = (uint8_t*)calloc(N, 1);
  for (uint32_t n = 0; n < N; ++n)
    if (d->node_kind[n] == PCB_INPUT) { sig[n] = pcb_scope_mix(d->node_var[n]); seen[n] = 1; }
  for (uint32_t e = 0; e < E; ++e) {
    uint32_t p = d->up_parent[e] - 1;
    uint64_t cs = sig[d->up_prime[e] - 1] + (d->up_sub[e] ? sig[d->up_sub[e] - 1] : 0);
    if (d->node_kind[p] == PCB_PRODUCT) sig[p] += cs;
    else if (!seen[p]) { sig[p] = cs; seen[p] = 1; }
  }
  /* rank unique signatures of sum nodes by first appearance */
  uint32_t R = 0;
  uint64_t* rs = (uint64_t*)malloc(sizeof(uint64_t) * (N ? N : 1));
  /* open-addressing hash: key -> region */
  size_t cap = 16; while (cap < (size_t)N * 2 + 16) cap <<= 1;
  uint64_t* hk = (uint64_t*)calloc(cap, sizeof(uint64_t));
  uint32_t* hv = (uint32_t*)calloc(cap, sizeof(uint32_t));
  for (uint32_t n = 0; n < N; ++n) {
    node_region[n] = 0;
    if (d->node_kind[n] != PCB_SUM) continue;
    uint64_t k = sig[n] | 1ull; /* never 0 */
    size_t h = (size_t)(pcb_scope_mix(k) & (cap - 1));
    while (hv[h] != 0 && hk[h] != k) h = (h + 1) & (cap - 1);
    if (hv[h] == 0) { hk[h] = k; hv[h] = ++R; }
    node_region[n] = hv[h];
  }
  *num_regions = R;
  free(sig); free(seen); free(rs); free(hk); free(hv);
}

/* first up-edge (0-based) and number of up-edges of every node */
static void node_edge_ranges(const pcb_circuit_desc* d, uint32_t* estart, uint32_t* ecount) {
  memset(ecount, 0, sizeof(uint32_t) * d->num_nodes);
  for (uint32_t e = 0; e < d->num_edges; ++e) {
    uint32_t p = d->up_parent[e] - 1;
    if (ecount[p] == 0) estart[p] = e;
    ++ecount[p];
  }
}

/* Hard Gumbel-max sampling.  params [Sp, P] (Sp == 1 or S).  u_sum [S][R][kmax],
 * u_leaf [S][V][cmax] (last index fastest).  x_out [S, V] column-major, -1 if unreached. */
void orc_sample_hard(const pcb_circuit_desc* d, const float* heap, const float* params, uint32_t Sp,
                     const float* u_sum, const float* u_leaf, uint32_t S, uint32_t kmax,
                     uint32_t cmax, int32_t* x_out) {
  const uint32_t N = d->num_nodes, E = d->num_edges, V = d->num_vars;
  uint32_t n_inner, n_input, n_groups, R;
  orc_counts(d, &n_inner, &n_input, &n_groups);
  uint32_t* edge2param = (uint32_t*)malloc(sizeof(uint32_t) * (E ? E : 1));
  uint32_t* cum = (uint32_t*)malloc(sizeof(uint32_t) * (d->num_input_nodes ? d->num_input_nodes : 1));
  uint32_t* node2input = (uint32_t*)calloc(N, sizeof(uint32_t));
  uint32_t* region = (uint32_t*)malloc(sizeof(uint32_t) * N);
  uint32_t* estart = (uint32_t*)malloc(sizeof(uint32_t) * N);
  uint32_t* ecount = (uint32_t*)malloc(sizeof(uint32_t) * N);
  orc_meta(d, edge2param, NULL, NULL, cum);
  orc_sum_regions(d, region, &R);
  node_edge_ranges(d, estart, ecount);
  for (uint32_t i = 0; i < d->num_input_nodes; ++i) node2input[d->input_node_ids[i] - 1] = i + 1;
#pragma omp parallel
  {
    uint32_t* stack = (uint32_t*)malloc(sizeof(uint32_t) * ((size_t)N + 2));
#pragma omp for schedule(static)
    for (int64_t s = 0; s < (int64_t)S; ++s) {
      size_t ps = (Sp == 1) ? 0 : (size_t)s, pld = Sp;
      for (uint32_t v = 0; v < V; ++v) x_out[IDX(s, v, S)] = -1;
      size_t sp = 0;
      stack[sp++] = N - 1;
      while (sp) {
        uint32_t n = stack[--sp];
        if (d->node_kind[n] == PCB_INPUT) {
          uint32_t C = d->node_num_cats[n], var = d->node_var[n] - 1;
          const float* us = u_leaf + ((size_t)s * V + var) * cmax;
          double best = 0.0; int32_t bi = -1;
          for (uint32_t c = 0; c < C; ++c) {
            float lp;
            if (d->node_fixed[n]) lp = heap[d->node_heap_start[n] - 1 + c];
            else lp = params[ps + pld * ((size_t)n_inner + cum[node2input[n] - 1] - C + c)];
            double key = pcb_gumbel_key(lp, us[c]);
            if (bi < 0 || key > best) { best = key; bi = (int32_t)c; }
          }
          x_out[IDX(s, var, S)] = bi;
        } else if (d->node_kind[n] == PCB_PRODUCT) {
          for (uint32_t j = 0; j < ecount[n]; ++j) {
            uint32_t e = estart[n] + j;
            stack[sp++] = d->up_prime[e] - 1;
            if (d->up_sub[e]) stack[sp++] = d->up_sub[e] - 1;
          }
        } else {
          const float* us = u_sum + ((size_t)s * R + (region[n] - 1)) * kmax;
          double best = 0.0; int32_t bi = -1;
          for (uint32_t j = 0; j < ecount[n]; ++j) {
            float lp = params[ps + pld * (size_t)(edge2param[estart[n] + j] - 1)];
            double key = pcb_gumbel_key(lp, us[j]);
            if (bi < 0 || key > best) { best = key; bi = (int32_t)j; }
          }
          uint32_t e = estart[n] + (uint32_t)bi;
          stack[sp++] = d->up_prime[e] - 1;
          if (d->up_sub[e]) stack[sp++] = d->up_sub[e] - 1;
        }
      }
    }
    free(stack);
  }
  free(edge2param); free(cum); free(node2input); free(region); free(estart); free(ecount);
}

/* Soft Gumbel-softmax sampling (sample.jl:8-148,233-296).  u [S, n_inner] column-major or
 * NULL (no_gumbel).  Outputs: edge_probs [S, n_inner], cum_probs [S, n_groups],
 * td_probs [S, N], out = input_aggr_params [S, V, cmax] column-major. */
void orc_sample_soft(const pcb_circuit_desc* d, const float* heap, const float* params, uint32_t Sp,
                     const float* u, float temperature, uint32_t S, uint32_t cmax,
                     float* edge_probs, float* cum_probs, float* td_probs, float* out) {
  const uint32_t N = d->num_nodes, E = d->num_edges, V = d->num_vars;
  uint32_t n_inner, n_input, n_groups;
  orc_counts(d, &n_inner, &n_input, &n_groups);
  uint32_t* edge2param = (uint32_t*)malloc(sizeof(uint32_t) * (E ? E : 1));
  uint32_t* param2group = (uint32_t*)malloc(sizeof(uint32_t) * (n_inner ? n_inner : 1));
  uint32_t* cum = (uint32_t*)malloc(sizeof(uint32_t) * (d->num_input_nodes ? d->num_input_nodes : 1));
  orc_meta(d, edge2param, NULL, param2group, cum);
  memset(out, 0, sizeof(float) * (size_t)S * V * cmax);
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < (int64_t)S; ++s) {
    size_t ps = (Sp == 1) ? 0 : (size_t)s, pld = Sp;
    for (uint32_t n = 0; n < N; ++n) td_probs[IDX(s, n, S)] = 0.0f;
    td_probs[IDX(s, N - 1, S)] = 1.0f;
    for (uint32_t g = 0; g < n_groups; ++g) cum_probs[IDX(s, g, S)] = 0.0f;
    /* gumbel_params_down_kernel (sample.jl:24-54): Float64 promotion through the 1e-6 literals */
    for (uint32_t p = 0; p < n_inner; ++p) {
      float logp = params[ps + pld * (size_t)p];
      double gv = 0.0;
      if (u) gv = -log(-log((double)u[IDX(s, p, S)] * (1.0 - 1e-6) + 1e-6));
      float unnorm = (float)exp(((double)logp + gv) / (double)temperature);
      edge_probs[IDX(s, p, S)] = unnorm;
      cum_probs[IDX(s, param2group[p] - 1, S)] += unnorm;
    }
    /* gumbel_sample_down_kernel (sample.jl:79-144) */
    for (uint32_t de = 0; de < E; ++de) {
      uint32_t e = d->down2up[de] - 1;
      uint32_t parent = d->up_parent[e] - 1, prime = d->up_prime[e] - 1, sub = d->up_sub[e];
      float tp = td_probs[IDX(s, parent, S)];
      if (edge_is_sum(d, e)) {
        uint32_t p = edge2param[e] - 1;
        tp *= edge_probs[IDX(s, p, S)] / cum_probs[IDX(s, param2group[p] - 1, S)];
      }
      if (sub != 0) td_probs[IDX(s, sub - 1, S)] += tp;
      td_probs[IDX(s, prime, S)] += tp;
    }
    /* gumbel_input_sample_down_kernel + gumbel_input_step (sample.jl:233-296) */
    for (uint32_t i = 0; i < d->num_input_nodes; ++i) {
      uint32_t n = d->input_node_ids[i] - 1, C = d->node_num_cats[n], var = d->node_var[n] - 1;
      float tp = td_probs[IDX(s, n, S)];
      for (uint32_t c = 0; c < C; ++c) {
        float lp;
        if (d->node_fixed[n]) lp = heap[d->node_heap_start[n] - 1 + c];
        else lp = params[ps + pld * ((size_t)n_inner + cum[i] - C + c)];
        out[(size_t)s + (size_t)S * (var + (size_t)V * c)] += tp * expf(lp);
      }
    }
  }
  free(edge2param); free(param2group); free(cum);
}
